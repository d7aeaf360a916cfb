// Hyper-connections: S copies of the residual stream instead of one.
//
// For a part behind a norm, with coefficients a [S] ("in"), M [S, S] ("mix", indexed [from, to]) and b [S] ("out"):
//   u    = sum_s a[s] x_s                  what the part's norm reads
//   y    = part(norm(u))
//   x_t <- sum_s M[s, t] x_s + b[t] y      all copies at once, from the old ones
// The update of one part and the read of the next are one pass over the copies here: the kernel takes the
// y, M and b of the part that just ran (or nothing, right after the embedding) and the a and norm weight of
// the part that runs next (or no norm weight: the plain sum, 32-bit, which is how the copies are folded into
// one stream at the end).  Everything is 32-bit; only the normed rows are rounded to the activation type.
//
// Layout: copies [T, S, W], one token's copies side by side.
#include "common.cuh"

#define HC_MAX_STREAMS 8
#define HC_THREADS 256

// y: [T, W] of type Y (may be null: no update).  first: the copies do not exist yet; x0 [T, W] is the
// embedding's output and every copy starts as x0 (written here).
template <int S, typename Y, typename O>
__global__ void hyper_step_kernel(float* __restrict__ xs, const float* __restrict__ x0, const Y* __restrict__ y,
                                  const float* __restrict__ mix, const float* __restrict__ outc,
                                  const float* __restrict__ inc, const float* __restrict__ norm_w, float eps,
                                  O* __restrict__ out, int out_ld, int W) {
    extern __shared__ float us[];            // [W] the weighted sum of this row's copies
    __shared__ float scratch[33];
    __shared__ float cm[S * S], cb[S], ca[S];
    if (threadIdx.x < S * S) cm[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) { cb[threadIdx.x] = outc ? outc[threadIdx.x] : 0.f; ca[threadIdx.x] = inc ? inc[threadIdx.x] : 1.f; }
    pdl_wait();
    pdl_trigger();
    __syncthreads();
    const size_t t = blockIdx.x;
    float* row = xs + t * S * (size_t)W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[S];
        if (x0) {
            const float v = x0[t * W + c];
#pragma unroll
            for (int s = 0; s < S; ++s) { x[s] = v; row[(size_t)s * W + c] = v; }
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) x[s] = row[(size_t)s * W + c];
            if (y) {
                const float yv = to_f32(y[t * W + c]);
                float n[S];
#pragma unroll
                for (int k = 0; k < S; ++k) {
                    float v = cb[k] * yv;
#pragma unroll
                    for (int s = 0; s < S; ++s) v += cm[s * S + k] * x[s];
                    n[k] = v;
                }
#pragma unroll
                for (int s = 0; s < S; ++s) { x[s] = n[s]; row[(size_t)s * W + c] = n[s]; }
            }
        }
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) u += ca[s] * x[s];
        us[c] = u;
        ss += u * u;
    }
    if (!out) return;
    if (!norm_w) {
        for (int c = threadIdx.x; c < W; c += blockDim.x) out[t * out_ld + c] = from_f32<O>(us[c]);
        return;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) out[t * out_ld + c] = from_f32<O>(us[c] * inv * norm_w[c]);
}


__device__ __forceinline__ float4 hc_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 hc_load4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void hc_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void hc_store4(bf16* p, float4 v) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = o;
}

// The same with four columns per thread and 16-byte loads and stores (W % 4 == 0, rows 16-byte aligned).
template <int S, typename Y, typename O>
__global__ void hyper_step_vec4_kernel(float* __restrict__ xs, const float* __restrict__ x0, const Y* __restrict__ y,
                                       const float* __restrict__ mix, const float* __restrict__ outc,
                                       const float* __restrict__ inc, const float* __restrict__ norm_w, float eps,
                                       O* __restrict__ out, int out_ld, int W) {
    extern __shared__ float us[];
    __shared__ float scratch[33];
    __shared__ float cm[S * S], cb[S], ca[S];
    if (threadIdx.x < S * S) cm[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) { cb[threadIdx.x] = outc ? outc[threadIdx.x] : 0.f; ca[threadIdx.x] = inc ? inc[threadIdx.x] : 1.f; }
    pdl_wait();
    pdl_trigger();
    __syncthreads();
    const size_t t = blockIdx.x;
    float* row = xs + t * S * (size_t)W;
    float ss = 0.f;
    for (int c = 4 * threadIdx.x; c < W; c += 4 * blockDim.x) {
        float4 x[S];
        if (x0) {
            const float4 v = hc_load4(x0 + t * W + c);
#pragma unroll
            for (int s = 0; s < S; ++s) { x[s] = v; hc_store4(row + (size_t)s * W + c, v); }
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) x[s] = hc_load4(row + (size_t)s * W + c);
            if (y) {
                const float4 yv = hc_load4(y + t * W + c);
                float4 n[S];
#pragma unroll
                for (int k = 0; k < S; ++k) {
                    float4 v = make_float4(cb[k] * yv.x, cb[k] * yv.y, cb[k] * yv.z, cb[k] * yv.w);
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        const float m = cm[s * S + k];
                        v.x += m * x[s].x; v.y += m * x[s].y; v.z += m * x[s].z; v.w += m * x[s].w;
                    }
                    n[k] = v;
                }
#pragma unroll
                for (int s = 0; s < S; ++s) { x[s] = n[s]; hc_store4(row + (size_t)s * W + c, n[s]); }
            }
        }
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < S; ++s) { u.x += ca[s] * x[s].x; u.y += ca[s] * x[s].y; u.z += ca[s] * x[s].z; u.w += ca[s] * x[s].w; }
        hc_store4(us + c, u);
        ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    if (!out) return;
    float inv = 1.f;
    if (norm_w) {
        ss = block_sum(ss, scratch);
        inv = rsqrtf(ss / (float)W + eps);
    }
    for (int c = 4 * threadIdx.x; c < W; c += 4 * blockDim.x) {          // every thread reads back what it wrote itself
        float4 u = hc_load4(us + c);
        if (norm_w) {
            const float4 w = hc_load4(norm_w + c);
            u = make_float4(u.x * inv * w.x, u.y * inv * w.y, u.z * inv * w.z, u.w * inv * w.w);
        }
        hc_store4(out + t * out_ld + c, u);
    }
}

template <int S, typename Y, typename O>
static int hyper_launch(float* xs, const float* x0, const void* y, const float* mix, const float* outc, const float* inc,
                        const float* norm_w, float eps, void* out, int out_ld, int T, int W, cudaStream_t s) {
    // few rows: more threads per row, so that a thread's loads are few and all in flight at once
    const int threads = T >= 512 ? HC_THREADS : min(1024, max(HC_THREADS, (W + 63) / 64 * 32));
    const bool aligned = W % 4 == 0 && out_ld % 4 == 0 && ((uintptr_t)xs | (uintptr_t)x0 | (uintptr_t)y | (uintptr_t)norm_w |
                                                             (uintptr_t)out) % 16 == 0;
    if (aligned && T >= 512)
        return rg_launch(hyper_step_vec4_kernel<S, Y, O>, dim3(T), dim3(HC_THREADS), (size_t)W * sizeof(float), s, 1, xs, x0,
                         (const Y*)y, mix, outc, inc, norm_w, eps, (O*)out, out_ld, W);
    return rg_launch(hyper_step_kernel<S, Y, O>, dim3(T), dim3(threads), (size_t)W * sizeof(float), s, 1, xs, x0,
                     (const Y*)y, mix, outc, inc, norm_w, eps, (O*)out, out_ld, W);
}

template <int S>
static int hyper_dispatch(float* xs, const float* x0, const void* y, int y_dtype, const float* mix, const float* outc,
                          const float* inc, const float* norm_w, float eps, void* out, int out_dtype, int out_ld, int T,
                          int W, cudaStream_t s) {
#define HC_GO(Y, O) return hyper_launch<S, Y, O>(xs, x0, y, mix, outc, inc, norm_w, eps, out, out_ld, T, W, s)
    const bool yb = y && y_dtype == RG_DTYPE_BF16;
    if (out_dtype == RG_DTYPE_BF16) { if (yb) HC_GO(bf16, bf16); HC_GO(float, bf16); }
    if (yb) HC_GO(bf16, float);
    HC_GO(float, float);
#undef HC_GO
}

// xs [T, S, W] float (updated in place when y is given, created from x0 when x0 is given); out: [T, W]
// rows out_ld apart, bfloat16 or float, or null.  norm_w null: out receives the plain weighted sum.
extern "C" int rg_hyper_step(float* xs, const float* x0, const void* y, int y_dtype, const float* mix, const float* outc,
                             const float* inc, const float* norm_w, float eps, void* out, int out_dtype, int out_ld,
                             int T, int S, int W, void* stream) {
    if (T <= 0) return 0;
    if (S < 1 || S > HC_MAX_STREAMS || W < 1 || (size_t)W * sizeof(float) > 200 * 1024) return RG_ERR_UNSUPPORTED;
    if (y && y_dtype != RG_DTYPE_BF16 && y_dtype != RG_DTYPE_F32) return RG_ERR_UNSUPPORTED;
    if (out && out_dtype != RG_DTYPE_BF16 && out_dtype != RG_DTYPE_F32) return RG_ERR_UNSUPPORTED;
    if (y && (!mix || !outc)) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if ((size_t)W * sizeof(float) > 48 * 1024) return RG_ERR_UNSUPPORTED;
    switch (S) {
#define HC_CASE(N) case N: return hyper_dispatch<N>(xs, x0, y, y_dtype, mix, outc, inc, norm_w, eps, out, out_dtype, out_ld, T, W, s)
        HC_CASE(1); HC_CASE(2); HC_CASE(3); HC_CASE(4); HC_CASE(5); HC_CASE(6); HC_CASE(7); HC_CASE(8);
#undef HC_CASE
    }
    return RG_ERR_UNSUPPORTED;
}
