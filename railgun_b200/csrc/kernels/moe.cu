// Routed experts: the router, the grouping of (token, choice) pairs by expert, the experts' products over
// those groups, and the weighted sum.
//
//   z = W_r h (32-bit), s = softmax(z) over all N router outputs
//   the `top` outputs with the largest s + correction are chosen; their weights are s / (sum of the chosen s
//   + 1e-20).  Outputs E..N-1 stand for identity experts (the expert's result is h itself); outputs 0..E-1
//   for gated experts  down(silu(gate h) * (up h)).
//   out = sum_k weight_k * expert_k(h)  (+ an always-on shared expert's result, computed elsewhere)
//
// Nothing here is planned on the host: the number of rows every expert gets is only known on the device, so
// the products run over a list of row tiles that `moe_align` writes (at most pairs / tile + E of them; the
// launch covers that bound and unused tiles return at once), which keeps a step capturable in a CUDA graph.
//
//   moe_route          one warp per token
//   moe_align          one block: counts per expert, segment starts, the pairs in expert order, the tile list
//   moe_grouped_gemm   32-bit arithmetic on CUDA cores, any sizes and both storage types (the true 32-bit path)
//   moe_combine        one block per token, 32-bit sum in the order of the choices
#include "common.cuh"

#define ROUTE_WARPS 4

template <typename A>
__global__ void moe_route_kernel(const A* __restrict__ x, const float* __restrict__ router,
                                 const float* __restrict__ correction, int* __restrict__ ids,
                                 float* __restrict__ weights, int T, int W, int N, int top) {
    extern __shared__ float sm[];                 // per warp: N scores, N choice scores
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;
    float* s = sm + (size_t)warp * 2 * N;
    float* c = s + N;
    const A* h = x + (size_t)t * W;
    for (int n = 0; n < N; ++n) {
        const float* wr = router + (size_t)n * W;
        float dot = 0.f;
        for (int i = lane; i < W; i += 32) dot += wr[i] * to_f32(h[i]);
        dot = warp_sum(dot);
        if (lane == 0) s[n] = dot;
    }
    __syncwarp();
    float mx = -INFINITY;
    for (int n = lane; n < N; n += 32) mx = fmaxf(mx, s[n]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int n = lane; n < N; n += 32) { const float e = expf(s[n] - mx); s[n] = e; sum += e; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int n = lane; n < N; n += 32) { const float p = s[n] * inv; s[n] = p; c[n] = p + correction[n]; }
    __syncwarp();
    float chosen_sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = N;
        for (int n = lane; n < N; n += 32)
            if (c[n] > best) { best = c[n]; arg = n; }         // the lowest index among a lane's equals
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= N) arg = 0;                                  // only if every score is NaN or -inf
        const float p = s[arg];
        chosen_sum += p;
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            weights[(size_t)t * top + k] = p;
            c[arg] = -INFINITY;
        }
        __syncwarp();
    }
    const float norm = 1.f / (chosen_sum + 1e-20f);
    if (lane < top) weights[(size_t)t * top + lane] *= norm;
    for (int k = 32 + lane; k < top; k += 32) weights[(size_t)t * top + k] *= norm;
}

extern "C" int rg_moe_route(const void* x, int dtype, const float* router, const float* correction, int* ids,
                            float* weights, int T, int W, int N, int top, void* stream) {
    if (T <= 0) return 0;
    if (top < 1 || top > N) return RG_ERR_UNSUPPORTED;
    const size_t smem = (size_t)ROUTE_WARPS * 2 * N * sizeof(float);
    if (smem > 48 * 1024) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((T + ROUTE_WARPS - 1) / ROUTE_WARPS), block(ROUTE_WARPS * 32);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(moe_route_kernel<bf16>, grid, block, smem, s, 1, (const bf16*)x, router, correction, ids,
                         weights, T, W, N, top);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(moe_route_kernel<float>, grid, block, smem, s, 1, (const float*)x, router, correction, ids,
                         weights, T, W, N, top);
    return RG_ERR_UNSUPPORTED;
}

// ids: [P] chosen router outputs of the P = T * top pairs.  Pairs whose output is >= E (identity experts) get
// no place.  sorted_pair[pos] = pair at place pos; pair_pos[pair] = its place or -1; tiles[i] = (expert, first
// place, places) in tiles of `tile_rows`, expert -1 for the unused tail of the list (max_tiles entries).
__global__ void moe_align_kernel(const int* __restrict__ ids, int P, int E, int tile_rows, int* __restrict__ sorted_pair,
                                 int* __restrict__ pair_pos, int* __restrict__ tiles, int max_tiles) {
    extern __shared__ int ism[];                  // count[E], start[E + 1], fill[E], tile_start[E + 1]
    int* count = ism;
    int* start = count + E;
    int* fill = start + E + 1;
    int* tstart = fill + E;
    pdl_wait();
    pdl_trigger();
    for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0, b = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = a;
            tstart[e] = b;
            a += count[e];
            b += (count[e] + tile_rows - 1) / tile_rows;
        }
        start[E] = a;
        tstart[E] = b;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        int pos = -1;
        if (e >= 0 && e < E) {
            pos = start[e] + atomicAdd(&fill[e], 1);
            sorted_pair[pos] = p;
        }
        pair_pos[p] = pos;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = tstart[e + 1] - tstart[e];
        for (int i = 0; i < n; ++i) {
            int* tl = tiles + 3 * (size_t)(tstart[e] + i);
            tl[0] = e;
            tl[1] = start[e] + i * tile_rows;
            tl[2] = min(tile_rows, count[e] - i * tile_rows);
        }
    }
    for (int i = tstart[E] + threadIdx.x; i < max_tiles; i += blockDim.x) {
        tiles[3 * (size_t)i] = -1;
        tiles[3 * (size_t)i + 1] = 0;
        tiles[3 * (size_t)i + 2] = 0;
    }
}

extern "C" int rg_moe_align(const int* ids, int P, int E, int tile_rows, int* sorted_pair, int* pair_pos, int* tiles,
                            int max_tiles, void* stream) {
    if (P <= 0) return 0;
    const size_t smem = (size_t)(4 * E + 2) * sizeof(int);
    if (E < 1 || smem > 48 * 1024 || tile_rows < 1 || max_tiles < (P + tile_rows - 1) / tile_rows + E)
        return RG_ERR_UNSUPPORTED;
    return rg_launch(moe_align_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, 1, ids, P, E, tile_rows,
                     sorted_pair, pair_pos, tiles, max_tiles);
}

// One tile of the list: rows [first, first + n) of expert e.  Row `pos` of A is a[src[pos] / src_div] when
// src is given (the token of the pair at that place), else a[pos].  w: [E, (GATED ? 2 N : N), K], the gated
// form holding N gate rows and then N up rows per expert; out[pos, n] = sum_k a_k w_nk, or with GATED
// silu(gate) * up.  32-bit accumulation in the order of k.
#define GG_BM 32
#define GG_BN 64
#define GG_BK 32
template <typename A, bool GATED>
__global__ void __launch_bounds__(256) moe_grouped_gemm_kernel(
        const A* __restrict__ a, int lda, const int* __restrict__ src, int src_div, const A* __restrict__ w,
        A* __restrict__ out, int ldo, const int* __restrict__ tiles, int N, int K) {
    __shared__ float As[GG_BK][GG_BM + 1];
    __shared__ float Ws[GATED ? 2 : 1][GG_BK][GG_BN + 1];
    __shared__ int rowsrc[GG_BM];
    pdl_wait();
    pdl_trigger();
    const int* tl = tiles + 3 * (size_t)blockIdx.x;
    const int e = tl[0], first = tl[1], nrows = tl[2];
    if (e < 0) return;
    const int n0 = blockIdx.y * GG_BN;
    const int tid = threadIdx.x;
    if (tid < GG_BM) rowsrc[tid] = tid < nrows ? (src ? src[first + tid] / src_div : first + tid) : -1;
    __syncthreads();
    const A* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    const int tr = tid / 16, tc = tid % 16;          // rows tr, tr + 16; columns tc + 16 j, j < 4
    float acc[2][4] = {}, acc2[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        for (int i = tid; i < GG_BM * GG_BK; i += 256) {
            const int r = i / GG_BK, k = i % GG_BK;
            const int row = rowsrc[r];
            As[k][r] = (row >= 0 && k0 + k < K) ? to_f32(a[(size_t)row * lda + k0 + k]) : 0.f;
        }
        for (int i = tid; i < GG_BN * GG_BK; i += 256) {
            const int n = i / GG_BK, k = i % GG_BK;
            const bool ok = n0 + n < N && k0 + k < K;
            Ws[0][k][n] = ok ? to_f32(we[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
            if (GATED) Ws[1][k][n] = ok ? to_f32(we[(size_t)(N + n0 + n) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < GG_BK; ++k) {
            const float a0 = As[k][tr], a1 = As[k][tr + 16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Ws[0][k][tc + 16 * j];
                acc[0][j] += a0 * b;
                acc[1][j] += a1 * b;
                if (GATED) {
                    const float b2 = Ws[1][k][tc + 16 * j];
                    acc2[0][j] += a0 * b2;
                    acc2[1][j] += a1 * b2;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = tr + 16 * i;
        if (r >= nrows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tc + 16 * j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (GATED) v = v / (1.f + expf(-v)) * acc2[i][j];
            out[(size_t)(first + r) * ldo + n] = from_f32<A>(v);
        }
    }
}

extern "C" int rg_moe_grouped_gemm(const void* a, int lda, const int* src, int src_div, const void* w, void* out,
                                   int ldo, int dtype, const int* tiles, int max_tiles, int tile_rows, int N, int K,
                                   int gated, void* stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (tile_rows != GG_BM || K < 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(max_tiles, (N + GG_BN - 1) / GG_BN), block(256);
#define RG_GG(A, G) return rg_launch(moe_grouped_gemm_kernel<A, G>, grid, block, 0, s, 1, (const A*)a, lda, src, \
        src_div, (const A*)w, (A*)out, ldo, tiles, N, K)
    if (dtype == RG_DTYPE_BF16 && gated) RG_GG(bf16, true);
    if (dtype == RG_DTYPE_BF16 && !gated) RG_GG(bf16, false);
    if (dtype == RG_DTYPE_F32 && gated) RG_GG(float, true);
    if (dtype == RG_DTYPE_F32 && !gated) RG_GG(float, false);
#undef RG_GG
    return RG_ERR_UNSUPPORTED;
}

// out[t] (32-bit) = sum_k weights[t, k] * (ids[t, k] < E ? y[pair_pos[t, k]] : x[t])  (+ shared[t])
template <typename A>
__global__ void moe_combine_kernel(const A* __restrict__ x, const A* __restrict__ y, const A* __restrict__ shared,
                                   const int* __restrict__ ids, const float* __restrict__ weights,
                                   const int* __restrict__ pair_pos, float* __restrict__ out, int W, int E, int top) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) {
            const size_t p = (size_t)t * top + k;
            const int e = ids[p];
            const float g = weights[p];
            v += g * (e < E ? to_f32(y[(size_t)pair_pos[p] * W + i]) : to_f32(x[(size_t)t * W + i]));
        }
        if (shared) v += to_f32(shared[(size_t)t * W + i]);
        out[(size_t)t * W + i] = v;
    }
}

extern "C" int rg_moe_combine(const void* x, const void* y, const void* shared, int dtype, const int* ids,
                              const float* weights, const int* pair_pos, float* out, int T, int W, int E, int top,
                              void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = W >= 1024 ? 256 : 128;
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, (const bf16*)x, (const bf16*)y,
                         (const bf16*)shared, ids, weights, pair_pos, out, W, E, top);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, s, 1, (const float*)x, (const float*)y,
                         (const float*)shared, ids, weights, pair_pos, out, W, E, top);
    return RG_ERR_UNSUPPORTED;
}
