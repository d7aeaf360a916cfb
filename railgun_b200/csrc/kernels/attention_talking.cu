// Attention whose heads' scores are mixed before the softmax ("talking heads": Shazeer et al.,
// "Talking-Heads Attention"), with grouped key/value heads, a norm on q and k, partial rotation and
// values of another size than the keys.
//
//   q_h, k_g   <- rotate(w ∘ unit(q_h)), rotate(w ∘ unit(k_g))      unit = divided by its root mean square
//   s_g[i, j]  = scale * q_g[i] . k_kv(g)[j]                        kv(g) = g / (H / G)
//   s'_h[i, j] = sum_g M[h, g] s_g[i, j]                            M [H, H]
//   p_h        = softmax of s'_h over the keys the query sees (j <= i, and i - j < window if there is one)
//   out_h[i]   = sum_j p_h[i, j] v_kv(h)[j]
// All of it 32-bit; the cache and the outputs are in the storage type.
//
// Cache layout: one row per token, [pages * page_size, G * dv + G * d] = all value heads, then all key heads.
//
// Kernels here:
//   talking_prepare             per token: norm and rotation of q (into q_out [T, H, d]) and k, cache row write
//   talking_attention_general   one block per token, all heads together, any sizes with H * dv <= 4096
//
// On the tensor cores the mixing moves into the queries, where it is linear: with the keys of all G key/value
// heads side by side, K_j = [k_0[j] | ... | k_(G-1)[j]], and
//   Q'_h = [ scale sum_{g in group 0} M[h, g] q_g | ... | scale sum_{g in group G-1} M[h, g] q_g ]   (G d numbers)
// the mixed score is s'_h[i, j] = Q'_h[i] . K_j: every head attends to the same rows, as in attention over a
// latent cache, and that kernel (attention_latent_mma.cu) runs it: its queries are [0 (G dv) | Q'_h], its
// scores run over the whole cache row [V | K], its values are the row's first G dv numbers, of which head h
// keeps the dv of its own key/value head.  talking_prepare writes those queries when asked (qa).  Prompts can
// also run on the flash kernel of ordinary paged attention (talking_pack_kv, talking_select below).
#include "common.cuh"

#define TK_THREADS 128
#define TK_TILE 128              // keys per tile: one per thread in the score phase
#define TK_MAX_ACC 32            // output numbers per thread: H * dv <= 32 * 128

// qkv row: [H * d | G * d | G * dv].  freq: dims / 2 frequencies (64-bit); pairs (i, i + dims / 2).
template <typename A>
__global__ void talking_prepare_kernel(const A* __restrict__ qkv, int ld, A* __restrict__ q_out, A* __restrict__ cache,
                                       const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                       const double* __restrict__ freq, int dims, const int* __restrict__ positions,
                                       const int* __restrict__ slots, int H, int G, int d, int dv,
                                       A* __restrict__ qa, const float* __restrict__ talk, float scale,
                                       A* __restrict__ qc) {
    extern __shared__ float sm[];                    // cos | sin of the token's dims / 2 angles, then one head's numbers per warp
    float* cs = sm;                                  // (and, for qa, all heads' rotated queries behind them)
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = dims >> 1;
    const double pos = (double)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) rotary_cos_sin(pos, freq[i], &cs[i], &cs[half + i]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    float* buf = sm + dims + warp * d;
    float* qall = sm + dims + nwarp * d;             // [H * d], only with qa
    float* tk = qall + H * d;                        // [H * H], only with qa and talk
    const bool mixes = qa || qc;
    if (mixes && talk) for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = talk[i];
    const A* row = qkv + (size_t)t * ld;
    const int slot = slots ? slots[t] : -1;
    const int rowlen = G * (d + dv);
    // one warp per head: q heads 0..H-1, then k heads
    for (int hh = warp; hh < H + G; hh += nwarp) {
        const bool is_q = hh < H;
        if (!is_q && slot < 0) continue;
        const A* src = row + (size_t)hh * d;
        const float* w = is_q ? q_norm : k_norm;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) { const float v = to_f32(src[i]); buf[i] = v; ss += v * v; }
        ss = warp_sum(ss);
        const float inv = w ? rsqrtf(ss / (float)d + eps) : 1.f;
        __syncwarp();
        A* dst = is_q ? (q_out ? q_out + ((size_t)t * H + hh) * d : nullptr)
                      : cache + (size_t)slot * rowlen + (size_t)G * dv + (size_t)(hh - H) * d;
        for (int i = lane; i < d; i += 32) {
            const float wi = w ? w[i] : 1.f;
            float v = buf[i] * inv * wi;
            if (i < half) v = v * cs[i] - buf[i + half] * inv * (w ? w[i + half] : 1.f) * cs[half + i];
            else if (i < dims) v = v * cs[i - half] + buf[i - half] * inv * (w ? w[i - half] : 1.f) * cs[i];
            if (dst) dst[i] = from_f32<A>(v);
            if (is_q && mixes) qall[hh * d + i] = v;
        }
        __syncwarp();
    }
    if (slot >= 0) {
        const A* vsrc = row + (size_t)(H + G) * d;
        A* vdst = cache + (size_t)slot * rowlen;
        for (int i = threadIdx.x; i < G * dv; i += blockDim.x) vdst[i] = vsrc[i];
    }
    if (!mixes) return;
    // the queries of the tensor-core forms: for every key/value head c the numbers scale sum_{g in c} M[h, g] q_g,
    // behind G dv zeros in qa [T, H, G dv + G d] and on their own in qc [T, H, G d]
    __syncthreads();
    const int hpg = H / G, Gd = G * d, Gdv = G * dv, Dq = Gd + Gdv;
    if (qa) {
        A* qrow = qa + (size_t)t * H * Dq;
        for (int e = threadIdx.x; e < H * Gdv; e += blockDim.x) {
            const int h = e / Gdv;
            qrow[(size_t)h * Dq + (e - h * Gdv)] = from_f32<A>(0.f);
        }
    }
    for (int e = threadIdx.x; e < H * Gd; e += blockDim.x) {
        const int h = e / Gd, j = e - h * Gd, c = j / d, i = j - c * d;
        const float* trow = tk + h * H;                      // M[h, :] in shared memory
        float v = 0.f;
        if (talk) { for (int g = c * hpg; g < (c + 1) * hpg; ++g) v += trow[g] * qall[g * d + i]; }
        else if (h / hpg == c) v = qall[h * d + i];
        if (qa) qa[((size_t)t * H + h) * Dq + Gdv + j] = from_f32<A>(v * scale);
        if (qc) qc[((size_t)t * H + h) * Gd + j] = from_f32<A>(v * scale);
    }
}

// Prompts on the flash kernel of ordinary paged attention.  With the queries mixed (qc above) a head's score is
// Q'_h . [k_0 | ... | k_(G-1)]: the contexts of the step's requests that bring several tokens are laid out as
// temporary key/value pages [requests * max_blocks, 2, G, page_size, G d] in which every key/value head c has the
// same keys, all G key heads side by side, and its own values v_c, zero-padded from dv to G d; page j of the
// step's request r is page r * max_blocks + j.  talking_select then keeps the first dv numbers of every head's
// output row, times a constant, for the rows of those requests.
template <typename A>
__global__ void talking_pack_kv_kernel(const A* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
                                       const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                                       A* __restrict__ kv, int page_size, int G, int d, int dv) {
    pdl_wait();
    pdl_trigger();
    const int j = blockIdx.x, r = blockIdx.y;
    if (cu_seqlens[r + 1] - cu_seqlens[r] < 2) return;
    const int ctx = context_lens[r];
    if (j * page_size >= ctx) return;
    const int page = block_table[(size_t)r * max_blocks + j];
    if (page < 0) return;
    const int n = min(page_size, ctx - j * page_size);
    const int Gd = G * d, Gdv = G * dv, rowlen = Gd + Gdv;
    const A* src = cache + (size_t)page * page_size * rowlen;
    A* kdst = kv + ((size_t)r * max_blocks + j) * 2 * G * page_size * Gd;
    A* vdst = kdst + (size_t)G * page_size * Gd;
    for (int i = threadIdx.x; i < G * n * Gd; i += blockDim.x) {
        const int c = i / (n * Gd), rem = i - c * n * Gd, o = rem / Gd, col = rem - o * Gd;
        kdst[((size_t)c * page_size + o) * Gd + col] = src[(size_t)o * rowlen + Gdv + col];
        vdst[((size_t)c * page_size + o) * Gd + col] = col < dv ? src[(size_t)o * rowlen + c * dv + col] : from_f32<A>(0.f);
    }
}

extern "C" int rg_talking_pack_kv(const void* cache, const int* block_table, int max_blocks, const int* cu_seqlens,
                                  const int* context_lens, void* kv, int dtype, int requests, int page_size, int G, int d,
                                  int dv, void* stream) {
    if (requests <= 0 || max_blocks <= 0) return 0;
    if (dv > G * d || requests > 65535) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(max_blocks, requests);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(talking_pack_kv_kernel<bf16>, grid, dim3(256), 0, s, 1, (const bf16*)cache, block_table, max_blocks,
                         cu_seqlens, context_lens, (bf16*)kv, page_size, G, d, dv);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(talking_pack_kv_kernel<float>, grid, dim3(256), 0, s, 1, (const float*)cache, block_table,
                         max_blocks, cu_seqlens, context_lens, (float*)kv, page_size, G, d, dv);
    return RG_ERR_UNSUPPORTED;
}

// wide [T, H * Gd] -> out[t, h * dv + c] = wide[t, h * Gd + c] * out_scale, for the rows of requests with several tokens
template <typename A>
__global__ void talking_select_kernel(const A* __restrict__ wide, A* __restrict__ out, int out_ld, float out_scale,
                                      const int* __restrict__ cu_seqlens, const int* __restrict__ req_of_token, int H,
                                      int Gd, int dv) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int r = req_of_token[t];
    if (cu_seqlens[r + 1] - cu_seqlens[r] < 2) return;
    for (int e = threadIdx.x; e < H * dv; e += blockDim.x) {
        const int h = e / dv, c = e - h * dv;
        out[(size_t)t * out_ld + e] = from_f32<A>(to_f32(wide[((size_t)t * H + h) * Gd + c]) * out_scale);
    }
}

extern "C" int rg_talking_select(const void* wide, void* out, int out_ld, float out_scale, int dtype,
                                 const int* cu_seqlens, const int* req_of_token, int T, int H, int Gd, int dv,
                                 void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(talking_select_kernel<bf16>, dim3(T), dim3(256), 0, s, 1, (const bf16*)wide, (bf16*)out, out_ld,
                         out_scale, cu_seqlens, req_of_token, H, Gd, dv);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(talking_select_kernel<float>, dim3(T), dim3(256), 0, s, 1, (const float*)wide, (float*)out, out_ld,
                         out_scale, cu_seqlens, req_of_token, H, Gd, dv);
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_talking_prepare(const void* qkv, int dtype, int ld, void* q_out, void* cache, const float* q_norm,
                                  const float* k_norm, float eps, const double* freq, int dims, const int* positions,
                                  const int* slots, int T, int H, int G, int d, int dv, void* qa, const float* talk,
                                  float scale, void* qc, void* stream) {
    if (T <= 0) return 0;
    if (dims < 0 || dims > d || (dims & 1) || H < 1 || G < 1 || H % G || d < 1 || dv < 1 || (!q_out && !qa && !qc))
        return RG_ERR_UNSUPPORTED;
    // a warp per head: as many warps as heads (up to 16), so that the heads' dependent loads overlap
    int nwarp = H + G < 16 ? H + G : 16;
    if (nwarp < 4) nwarp = 4;
    while (nwarp > 4 && (size_t)(dims + nwarp * d + ((qa || qc) ? H * d + H * H : 0)) * sizeof(float) > 48 * 1024) --nwarp;
    const size_t smem = (size_t)(dims + nwarp * d + ((qa || qc) ? H * d + H * H : 0)) * sizeof(float);
    if (smem > 48 * 1024) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int prep_threads = 32 * nwarp;
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(talking_prepare_kernel<bf16>, dim3(T), dim3(prep_threads), smem, s, 1, (const bf16*)qkv, ld,
                         (bf16*)q_out, (bf16*)cache, q_norm, k_norm, eps, freq, dims, positions, slots, H, G, d, dv,
                         (bf16*)qa, talk, scale, (bf16*)qc);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(talking_prepare_kernel<float>, dim3(T), dim3(prep_threads), smem, s, 1, (const float*)qkv, ld,
                         (float*)q_out, (float*)cache, q_norm, k_norm, eps, freq, dims, positions, slots, H, G, d, dv,
                         (float*)qa, talk, scale, (float*)qc);
    return RG_ERR_UNSUPPORTED;
}

// q [T, H, d]; out [T, H * dv] rows out_ld apart, times out_scale; talk [H, H] or null (no mixing).
template <typename A>
__global__ void talking_attention_general_kernel(
        const A* __restrict__ q, A* __restrict__ out, int out_ld, float out_scale, const A* __restrict__ cache,
        const float* __restrict__ talk, const int* __restrict__ block_table, int max_blocks,
        const int* __restrict__ req_of_token, const int* __restrict__ positions, int H, int G, int d, int dv,
        int page_size, int window, float scale) {
    extern __shared__ float sm[];
    float* qs = sm;                                  // [H * d] queries times scale
    float* tk = qs + H * d;                          // [H * H]
    float* raw = tk + H * H;                         // [H][TILE] unmixed scores
    float* sc = raw + H * TK_TILE;                   // [H][TILE] mixed scores, then weights
    float* sm_m = sc + H * TK_TILE;                  // [H] running maximum
    float* sm_l = sm_m + H;                          // [H] running sum
    float* sm_a = sm_l + H;                          // [H] this tile's rescaling of what was accumulated
    int* srow = reinterpret_cast<int*>(sm_a + H);    // [TILE] cache row of each key of the tile
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = talk ? talk[i] : ((i / H) == (i % H) ? 1.f : 0.f);
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int r = req_of_token[t];
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)r * max_blocks;
    const int hpg = H / G, rowlen = G * (d + dv);
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) qs[i] = to_f32(q[(size_t)t * H * d + i]) * scale;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { sm_m[i] = -INFINITY; sm_l[i] = 0.f; }
    float acc[TK_MAX_ACC];
    int acc_h[TK_MAX_ACC], acc_off[TK_MAX_ACC];
#pragma unroll
    for (int k = 0; k < TK_MAX_ACC; ++k) {
        acc[k] = 0.f;
        const int e = threadIdx.x + k * TK_THREADS;
        const int h = e < H * dv ? e / dv : 0;
        acc_h[k] = e < H * dv ? h : -1;
        acc_off[k] = (h / hpg) * dv + (e - h * dv);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = lo; base <= pos; base += TK_TILE) {
        const int j = base + threadIdx.x;
        const bool valid = j <= pos;
        if (valid) {
            const int row = bt[j / page_size] * page_size + j % page_size;
            srow[threadIdx.x] = row;
            const A* krow = cache + (size_t)row * rowlen;
            for (int g = 0; g < H; ++g) {
                const A* kh = krow + G * dv + (g / hpg) * d;
                const float* qh = qs + g * d;
                float dot = 0.f;
                for (int i = 0; i < d; ++i) dot += qh[i] * to_f32(kh[i]);
                raw[g * TK_TILE + threadIdx.x] = dot;
            }
            for (int h = 0; h < H; ++h) {
                float s = 0.f;
                for (int g = 0; g < H; ++g) s += tk[h * H + g] * raw[g * TK_TILE + threadIdx.x];
                sc[h * TK_TILE + threadIdx.x] = s;
            }
        } else {
            for (int h = 0; h < H; ++h) sc[h * TK_TILE + threadIdx.x] = -INFINITY;
        }
        __syncthreads();
        for (int h = warp; h < H; h += TK_THREADS / 32) {
            float s[TK_TILE / 32], mx = -INFINITY;
#pragma unroll
            for (int k = 0; k < TK_TILE / 32; ++k) { s[k] = sc[h * TK_TILE + lane + 32 * k]; mx = fmaxf(mx, s[k]); }
            const float m_old = sm_m[h];
            const float m_new = fmaxf(m_old, warp_max(mx));
            float sum = 0.f;
#pragma unroll
            for (int k = 0; k < TK_TILE / 32; ++k) {
                const float p = expf(s[k] - m_new);                    // a key outside the tile's range has -inf: 0
                sc[h * TK_TILE + lane + 32 * k] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = expf(m_old - m_new);              // 0 for the first tile
                sm_a[h] = alpha;
                sm_l[h] = sm_l[h] * alpha + sum;
                sm_m[h] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK_MAX_ACC; ++k) if (acc_h[k] >= 0) acc[k] *= sm_a[acc_h[k]];
        const int n = min(TK_TILE, pos - base + 1);
        for (int kk = 0; kk < n; ++kk) {
            const A* vrow = cache + (size_t)srow[kk] * rowlen;
#pragma unroll
            for (int k = 0; k < TK_MAX_ACC; ++k)
                if (acc_h[k] >= 0) acc[k] += sc[acc_h[k] * TK_TILE + kk] * to_f32(vrow[acc_off[k]]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < TK_MAX_ACC; ++k) {
        if (acc_h[k] >= 0) {
            const float l = sm_l[acc_h[k]];
            out[(size_t)t * out_ld + threadIdx.x + k * TK_THREADS] = from_f32<A>(l > 0.f ? acc[k] / l * out_scale : 0.f);
        }
    }
}

static size_t talking_general_smem(int H, int d) {
    return (size_t)(H * d + H * H + 2 * H * TK_TILE + 3 * H) * sizeof(float) + TK_TILE * sizeof(int);
}

extern "C" int rg_talking_attention_general(
        const void* q, void* out, int out_ld, float out_scale, const void* cache, int dtype, const float* talk,
        const int* block_table, int max_blocks, const int* req_of_token, const int* positions, int T, int H, int G,
        int d, int dv, int page_size, int window, float scale, void* stream) {
    if (T <= 0) return 0;
    if (H < 1 || G < 1 || H % G || d < 1 || dv < 1 || H * dv > TK_MAX_ACC * TK_THREADS || page_size < 1)
        return RG_ERR_UNSUPPORTED;
    const size_t smem = talking_general_smem(H, d);
    if (smem > 200 * 1024) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define TK_GO(A) { \
        if (smem > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(talking_attention_general_kernel<A>, \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
        } \
        return rg_launch(talking_attention_general_kernel<A>, dim3(T), dim3(TK_THREADS), smem, s, 1, (const A*)q, (A*)out, \
                         out_ld, out_scale, (const A*)cache, talk, block_table, max_blocks, req_of_token, positions, H, G, \
                         d, dv, page_size, window, scale); }
    if (dtype == RG_DTYPE_BF16) TK_GO(bf16)
    if (dtype == RG_DTYPE_F32) TK_GO(float)
#undef TK_GO
    return RG_ERR_UNSUPPORTED;
}
