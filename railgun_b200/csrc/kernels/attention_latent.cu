// Attention over a compressed ("latent") key/value cache.
//
// Every token keeps ONE vector for all heads: c (R numbers, RMS-normed) followed by a rotated key part
// k_r (dr numbers).  A head's keys and values are linear in c (k = U_k c, v = U_v c), so the head never
// expands them: with the query taken through U_k^T once (qa = [U_k^T q_plain | q_rot], D = R + dr numbers),
//   score_j  = scale * qa . [c_j | k_r,j]
//   out      = U_v (sum_j p_j c_j),   p = softmax over the visible keys
// which makes all heads read the same cache rows: attention with one shared key/value "head" of size D whose
// values are the first R numbers of the keys.  The products with U_k^T and U_v are batched matrix products
// outside these kernels.
//
// Cache layout: [pages, page_size, D] rows, token slot = page * page_size + offset.
//
// Kernels here:
//   latent_rope_cache    per token: RMS norm of the latent part and rotation of the shared key part into the
//                        cache row; rotation of every head's rotated query part into qa[:, :, R:]; pairs
//                        (i, i + dims/2) or (2i, 2i + 1)
//   latent_attention_general  one block per (token, head), all arithmetic in 32-bit, any sizes: the true
//                        32-bit path and every shape the tensor-core kernels refuse; optionally a sink per
//                        head in the softmax's denominator
#include "common.cuh"

#define LAT_THREADS 128
#define LAT_MAX_ACC 8            // output numbers per thread of the general kernel: R <= 8 * 128

// One number of a rotated vector.  Pair p < dims/2 is (p, p + dims/2), or (2p, 2p + 1) when `interleaved`; it
// turns by the angle pos * freq[p]: (u, v) -> (u cos - v sin, v cos + u sin).  cs holds cos | sin of the dims/2
// angles (computed once per token); numbers from `dims` on pass unchanged.
template <typename A>
__device__ __forceinline__ float rotated_number(const A* __restrict__ src, int j, int dims, bool interleaved,
                                                const float* __restrict__ cs) {
    const int half = dims >> 1;
    if (j >= dims) return to_f32(src[j]);
    if (interleaved) {
        const int p = j >> 1;
        return (j & 1) ? to_f32(src[j]) * cs[p] + to_f32(src[j - 1]) * cs[half + p]
                       : to_f32(src[j]) * cs[p] - to_f32(src[j + 1]) * cs[half + p];
    }
    if (j < half) return to_f32(src[j]) * cs[j] - to_f32(src[j + half]) * cs[half + j];
    return to_f32(src[j]) * cs[j - half] + to_f32(src[j - half]) * cs[j];
}

template <typename A, typename B>
__device__ __forceinline__ void rotate_pairs(const A* __restrict__ src, B* __restrict__ dst, int n, int dims,
                                             bool interleaved, const float* __restrict__ cs) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = from_f32<B>(rotated_number(src, i, dims, interleaved, cs));
}

// proj: [T, ld] = per head [dn plain | dr rotated] query numbers, then at offset kv_off the down-projection
// [R latent | dr key part].  qa: [T, H, R + dr]; only its last dr numbers per head are written here.
template <typename A>
__global__ void latent_rope_cache_kernel(const A* __restrict__ proj, int ld, int kv_off, A* __restrict__ qa,
                                         A* __restrict__ cache, const float* __restrict__ norm_w, float eps,
                                         const double* __restrict__ freq, int rot_dims, int interleaved,
                                         const int* __restrict__ positions, const int* __restrict__ slots,
                                         int H, int dn, int dr, int R, A* __restrict__ q_back) {
    __shared__ float scratch[33];
    extern __shared__ float cs[];                    // cos | sin of the token's rot_dims / 2 angles; then H * dr rotated numbers
    float* rot_q = cs + rot_dims;
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const double pos = (double)positions[t];
    const A* row = proj + (size_t)t * ld;
    const int D = R + dr;
    for (int i = threadIdx.x; i < (rot_dims >> 1); i += blockDim.x)        // angles in 64-bit: a handful per token
        rotary_cos_sin(pos, freq[i], &cs[i], &cs[(rot_dims >> 1) + i]);
    __syncthreads();
    for (int i = threadIdx.x; i < H * dr; i += blockDim.x) {     // all heads' rotated parts at once
        const int h = i / dr, j = i - h * dr;
        const A* src = row + (size_t)h * (dn + dr) + dn;
        const float v = rotated_number(src, j, rot_dims, interleaved != 0, cs);
        if (qa) qa[((size_t)t * H + h) * D + R + j] = from_f32<A>(v);
        if (q_back) rot_q[i] = v;
    }
    if (q_back) {                                    // in place: every partner has been read before anything is written
        __syncthreads();
        for (int i = threadIdx.x; i < H * dr; i += blockDim.x) {
            const int h = i / dr, j = i - h * dr;
            q_back[(size_t)t * ld + (size_t)h * (dn + dr) + dn + j] = from_f32<A>(rot_q[i]);
        }
    }
    const int slot = slots ? slots[t] : -1;
    if (slot < 0) return;
    const A* lat = row + kv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = to_f32(lat[i]); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)R + eps);
    A* dst = cache + (size_t)slot * D;
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f32<A>(to_f32(lat[i]) * inv * norm_w[i]);
    rotate_pairs(lat + R, dst + R, dr, rot_dims, interleaved != 0, cs);
}

// q_in_place: the rotated query parts also replace the unrotated ones in proj (qa may then be null).
extern "C" int rg_latent_rope_cache(const void* proj, int ld, int kv_off, void* qa, void* cache, int dtype,
                                    const float* norm_w, float eps, const double* freq, int rot_dims,
                                    int interleaved, const int* positions, const int* slots, int T, int H, int dn, int dr, int R,
                                    int q_in_place, void* stream) {
    if (T <= 0) return 0;
    if (rot_dims < 0 || rot_dims > dr || (rot_dims & 1) || R < 1 || H < 1 || rot_dims > 8192) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t cs_bytes = (size_t)((rot_dims > 0 ? rot_dims : 1) + (q_in_place ? H * dr : 0)) * sizeof(float);
    if (cs_bytes > 48 * 1024) return RG_ERR_UNSUPPORTED;
    // few tokens: more threads per token, so that each phase's dependent loads are one round
    const int rope_threads = T <= 256 ? 512 : LAT_THREADS;
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(latent_rope_cache_kernel<bf16>, dim3(T), dim3(rope_threads), cs_bytes, s, 1, (const bf16*)proj, ld,
                         kv_off, (bf16*)qa, (bf16*)cache, norm_w, eps, freq, rot_dims, interleaved, positions, slots, H, dn, dr, R,
                         q_in_place ? (bf16*)proj : (bf16*)nullptr);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(latent_rope_cache_kernel<float>, dim3(T), dim3(rope_threads), cs_bytes, s, 1, (const float*)proj, ld,
                         kv_off, (float*)qa, (float*)cache, norm_w, eps, freq, rot_dims, interleaved, positions, slots, H, dn, dr, R,
                         q_in_place ? (float*)proj : (float*)nullptr);
    return RG_ERR_UNSUPPORTED;
}

// qa: [T, H, D]; out: [T, H, R]; cache: [pages * page_size, D]; block_table: [requests, max_blocks].
// A query at position p of request r sees the keys of r at positions [max(0, p - window + 1), p].
template <typename A>
__global__ void latent_attention_general_kernel(
        const A* __restrict__ qa, A* __restrict__ out, const A* __restrict__ cache,
        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ req_of_token,
        const int* __restrict__ positions, int H, int R, int D, int page_size, int window, float scale,
        const float* __restrict__ sink) {
    extern __shared__ float smem[];
    float* qs = smem;                    // [D]
    float* ps = qs + D;                  // [LAT_THREADS]
    float* scratch = ps + LAT_THREADS;   // [33]
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y;
    const int r = req_of_token[t];
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* bt = block_table + (size_t)r * max_blocks;
    const A* qrow = qa + ((size_t)t * H + h) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) qs[i] = to_f32(qrow[i]) * scale;
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[LAT_MAX_ACC];
#pragma unroll
    for (int k = 0; k < LAT_MAX_ACC; ++k) acc[k] = 0.f;
    for (int base = lo; base <= pos; base += LAT_THREADS) {
        const int j = base + threadIdx.x;
        float s = -INFINITY;
        if (j <= pos) {
            const A* krow = cache + ((size_t)bt[j / page_size] * page_size + j % page_size) * D;
            float dot = 0.f;
            for (int i = 0; i < D; ++i) dot += qs[i] * to_f32(krow[i]);
            s = dot;
        }
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float p = (j <= pos) ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);           // 0 when m = -inf
        l = l * alpha + block_sum(p, scratch);
        m = m_new;
        ps[threadIdx.x] = p;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < LAT_MAX_ACC; ++k) acc[k] *= alpha;
        const int n = min(LAT_THREADS, pos - base + 1);
        for (int kk = 0; kk < n; ++kk) {
            const int jj = base + kk;
            const A* vrow = cache + ((size_t)bt[jj / page_size] * page_size + jj % page_size) * D;
            const float pk = ps[kk];
#pragma unroll
            for (int k = 0; k < LAT_MAX_ACC; ++k) {
                const int i = threadIdx.x + k * LAT_THREADS;
                if (i < R) acc[k] += pk * to_f32(vrow[i]);
            }
        }
        __syncthreads();
    }
    if (sink) {                          // a term of the denominator without key or value: exp(sink[h]), unscaled, once
        const float m_new = fmaxf(m, sink[h]);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sink[h] - m_new);
#pragma unroll
        for (int k = 0; k < LAT_MAX_ACC; ++k) acc[k] *= alpha;
    }
    A* orow = out + ((size_t)t * H + h) * R;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int k = 0; k < LAT_MAX_ACC; ++k) {
        const int i = threadIdx.x + k * LAT_THREADS;
        if (i < R) orow[i] = from_f32<A>(acc[k] * inv);
    }
}

extern "C" int rg_latent_attention_general(
        const void* qa, void* out, const void* cache, int dtype, const int* block_table, int max_blocks,
        const int* req_of_token, const int* positions, int T, int H, int R, int D, int page_size, int window,
        float scale, const float* sink, void* stream) {
    if (T <= 0) return 0;
    if (R < 1 || R > LAT_MAX_ACC * LAT_THREADS || D < R || H < 1 || page_size < 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, H);
    const size_t smem = (size_t)(D + LAT_THREADS + 33) * sizeof(float);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(latent_attention_general_kernel<bf16>, grid, dim3(LAT_THREADS), smem, s, 1,
                         (const bf16*)qa, (bf16*)out, (const bf16*)cache, block_table, max_blocks, req_of_token,
                         positions, H, R, D, page_size, window, scale, sink);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(latent_attention_general_kernel<float>, grid, dim3(LAT_THREADS), smem, s, 1,
                         (const float*)qa, (float*)out, (const float*)cache, block_table, max_blocks, req_of_token,
                         positions, H, R, D, page_size, window, scale, sink);
    return RG_ERR_UNSUPPORTED;
}


// ---------------------------------------------------------------------------------------------------
// Prompts in the expanded form.  For a request that brings several tokens, a head's keys [U_k c | k_r] and
// values U_v c are cheaper to attend to than the compressed rows (dn + dr + dv numbers per key and head instead
// of 2 R + dr), so the step expands the request's context once: latent_gather copies the context's latent
// vectors into a dense matrix (a library product then applies U_k and U_v to all of them), and latent_pack_kv
// lays the result out as ordinary key/value pages [pages, 2, H, page, d], d = dn + dr (values zero-padded from
// dv to d), which the dense model's flash kernel reads.  The temporary pages are numbered request by request:
// page j of the step's request r is page r * max_blocks + j.  Requests that bring one token are skipped.

// lat [requests * max_blocks * page_size, R]: row (r * max_blocks + j) * page_size + o = latent of r's token j * page_size + o
template <typename A>
__global__ void latent_gather_kernel(const A* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
                                     const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                                     A* __restrict__ lat, int page_size, int R, int D) {
    pdl_wait();
    pdl_trigger();
    const int j = blockIdx.x, r = blockIdx.y;
    if (cu_seqlens[r + 1] - cu_seqlens[r] < 2) return;
    const int ctx = context_lens[r];
    if (j * page_size >= ctx) return;
    const int page = block_table[(size_t)r * max_blocks + j];
    if (page < 0) return;
    const int n = min(page_size, ctx - j * page_size);
    const A* src = cache + (size_t)page * page_size * D;
    A* dst = lat + ((size_t)r * max_blocks + j) * page_size * R;
    for (int i = threadIdx.x; i < n * R; i += blockDim.x) {
        const int o = i / R, c = i - o * R;
        dst[(size_t)o * R + c] = src[(size_t)o * D + c];
    }
}

extern "C" int rg_latent_gather(const void* cache, const int* block_table, int max_blocks, const int* cu_seqlens,
                                const int* context_lens, void* lat, int dtype, int requests, int page_size, int R, int D,
                                void* stream) {
    if (requests <= 0 || max_blocks <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(max_blocks, requests);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(latent_gather_kernel<bf16>, grid, dim3(256), 0, s, 1, (const bf16*)cache, block_table, max_blocks,
                         cu_seqlens, context_lens, (bf16*)lat, page_size, R, D);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(latent_gather_kernel<float>, grid, dim3(256), 0, s, 1, (const float*)cache, block_table,
                         max_blocks, cu_seqlens, context_lens, (float*)lat, page_size, R, D);
    return RG_ERR_UNSUPPORTED;
}

// kn [N, H * dn], vv [N, H * dv] (rows as in lat), the rotated key parts from the cache rows' last dr numbers
// -> kv [requests * max_blocks, 2, H, page_size, d]
template <typename A>
__global__ void latent_pack_kv_kernel(const A* __restrict__ kn, const A* __restrict__ vv, const A* __restrict__ cache,
                                      const int* __restrict__ block_table, int max_blocks,
                                      const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                                      A* __restrict__ kv, int page_size, int H, int dn, int dr, int dv, int R) {
    pdl_wait();
    pdl_trigger();
    const int j = blockIdx.x, r = blockIdx.y;
    if (cu_seqlens[r + 1] - cu_seqlens[r] < 2) return;
    const int ctx = context_lens[r];
    if (j * page_size >= ctx) return;
    const int page = block_table[(size_t)r * max_blocks + j];
    if (page < 0) return;
    const int n = min(page_size, ctx - j * page_size);
    const int d = dn + dr, D = R + dr;
    const size_t tp = (size_t)r * max_blocks + j;                  // the temporary page
    A* kdst = kv + tp * 2 * H * page_size * d;
    A* vdst = kdst + (size_t)H * page_size * d;
    const size_t row0 = tp * page_size;
    const A* krot = cache + (size_t)page * page_size * D + R;
    for (int i = threadIdx.x; i < H * n * d; i += blockDim.x) {
        const int h = i / (n * d), rem = i - h * n * d, o = rem / d, c = rem - o * d;
        kdst[((size_t)h * page_size + o) * d + c] = c < dn ? kn[(row0 + o) * H * dn + (size_t)h * dn + c]
                                                           : krot[(size_t)o * D + c - dn];
        vdst[((size_t)h * page_size + o) * d + c] = c < dv ? vv[(row0 + o) * H * dv + (size_t)h * dv + c] : from_f32<A>(0.f);
    }
}

extern "C" int rg_latent_pack_kv(const void* kn, const void* vv, const void* cache, const int* block_table,
                                 int max_blocks, const int* cu_seqlens, const int* context_lens, void* kv, int dtype,
                                 int requests, int page_size, int H, int dn, int dr, int dv, int R, void* stream) {
    if (requests <= 0 || max_blocks <= 0) return 0;
    if (dv > dn + dr) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(max_blocks, requests);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(latent_pack_kv_kernel<bf16>, grid, dim3(256), 0, s, 1, (const bf16*)kn, (const bf16*)vv,
                         (const bf16*)cache, block_table, max_blocks, cu_seqlens, context_lens, (bf16*)kv, page_size, H, dn,
                         dr, dv, R);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(latent_pack_kv_kernel<float>, grid, dim3(256), 0, s, 1, (const float*)kn, (const float*)vv,
                         (const float*)cache, block_table, max_blocks, cu_seqlens, context_lens, (float*)kv, page_size, H,
                         dn, dr, dv, R);
    return RG_ERR_UNSUPPORTED;
}
