// A gated linear recurrence behind a short causal convolution (the recurrent block of Griffin: De et al.,
// "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models").
//
// Per token, from one product proj = [W_y h | W_x h] (C numbers each):
//   g     = gelu_tanh(proj_y + b_y)                                 the gate branch
//   xin   = proj_x + b_x
//   u_t   = b_c + sum_k taps[:, K-1-k] xin_(t-k)                    causal, per channel, zeros before the start
//   r, i  = sigmoid(R_b u_b + b_r), sigmoid(I_b u_b + b_i)          per block b of C / blocks channels (a batched
//                                                                   product outside these kernels gives R_b u_b | I_b u_b)
//   a     = exp(-c r softplus(lam))
//   S_t   = a S_(t-1) + sqrt(1 - a^2) i u_t                         S = 0 before the first token
//   out_t = S_t g
// Everything after the product is 32-bit.  Between steps a request keeps, in its state slot, the last K - 1
// values of xin (rows 0..K-2 of the slot, oldest first) and S (row K-1): state [slots, K, C] float.
//
// The step's tokens are packed request by request (cu_seqlens); a request whose start position is 0 begins
// from zeros whatever its slot holds; a row whose request has slot -1 (padding of a static batch) reads zeros
// and writes no state.
#include "common.cuh"

#define REC_THREADS 128
#define REC_MAX_TAPS 16

__device__ __forceinline__ float rec_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rec_softplus(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }
__device__ __forceinline__ float rec_gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// u [T, C] float
template <typename A>
__global__ void recurrent_conv_kernel(const A* __restrict__ proj, int ld, int x_off, const float* __restrict__ xb,
                                      const float* __restrict__ taps, const float* __restrict__ cb,
                                      const float* __restrict__ state, const int* __restrict__ cu_seqlens,
                                      const int* __restrict__ req_of_token, const int* __restrict__ start_pos,
                                      const int* __restrict__ slots, float* __restrict__ u, int C, int K,
                                      bf16* __restrict__ halves, int bs) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r = req_of_token[t];
    const int i = t - cu_seqlens[r];
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    const float b = xb[c];
    float acc = cb[c];
    for (int k = 0; k < K; ++k) {
        const int idx = i - k;
        float xin;
        if (idx >= 0) xin = to_f32(proj[(size_t)(t - k) * ld + x_off + c]) + b;
        else xin = has_past ? state[((size_t)slot * K + (K - 1 + idx)) * C + c] : 0.f;
        acc += taps[(size_t)c * K + (K - 1 - k)] * xin;
    }
    u[(size_t)t * C + c] = acc;
    if (halves) {
        // u as two bfloat16 numbers, u = hi + lo to 2^-17: [T, blocks, 2, bs], for a tensor-core product with
        // 32-bit accumulation that is as good as a 32-bit one
        const int blk = c / bs, i = c - blk * bs;
        const bf16 hi = __float2bfloat16_rn(acc);
        bf16* dst = halves + ((size_t)t * (C / bs) + blk) * 2 * bs + i;
        dst[0] = hi;
        dst[bs] = __float2bfloat16_rn(acc - __bfloat162float(hi));
    }
}

// gates [blocks, T, 2 bs] float: R_b u_b | I_b u_b.  out [T, C] rows out_ld apart, times out_scale.
template <typename A>
__global__ void recurrent_scan_kernel(const A* __restrict__ proj, int ld, int y_off, int x_off,
                                      const float* __restrict__ yb, const float* __restrict__ xb,
                                      const float* __restrict__ u, const float* __restrict__ gates,
                                      const float* __restrict__ rb, const float* __restrict__ ib,
                                      const float* __restrict__ lam, float decay, float* __restrict__ state,
                                      const int* __restrict__ cu_seqlens, const int* __restrict__ start_pos,
                                      const int* __restrict__ slots, A* __restrict__ out, int out_ld, float out_scale,
                                      int T, int C, int K, int bs) {
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float sp = decay * rec_softplus(lam[c]);
    const float byc = yb[c], bxc = xb[c], brc = rb[c], bic = ib[c];
    const int blk = c / bs, o = c - blk * bs;
    pdl_wait();
    pdl_trigger();
    const int lo = cu_seqlens[r], hi = cu_seqlens[r + 1];
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    float* st = slot >= 0 ? state + (size_t)slot * K * C : nullptr;
    float S = has_past ? st[(size_t)(K - 1) * C + c] : 0.f;
    const float* grow = gates + ((size_t)blk * T) * 2 * bs + o;
    for (int t = lo; t < hi; ++t) {
        const float gr = grow[(size_t)t * 2 * bs] + brc;
        const float gi = grow[(size_t)t * 2 * bs + bs] + bic;
        const float log_a = -sp * rec_sigmoid(gr);
        const float a = expf(log_a);
        const float m = sqrtf(-expm1f(2.f * log_a));                  // sqrt(1 - a^2) without cancellation near a = 1
        S = a * S + m * rec_sigmoid(gi) * u[(size_t)t * C + c];
        const float g = rec_gelu_tanh(to_f32(proj[(size_t)t * ld + y_off + c]) + byc);
        out[(size_t)t * out_ld + c] = from_f32<A>(S * g * out_scale);
    }
    if (!st) return;
    st[(size_t)(K - 1) * C + c] = S;
    // the last K - 1 inputs of the convolution: from this step's tokens, and before them from the old tail
    const int n = hi - lo;
    float tail[REC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < REC_MAX_TAPS; ++j) {
        if (j < K - 1) {
            const int src = n - (K - 1) + j;
            if (src >= 0) tail[j] = to_f32(proj[(size_t)(lo + src) * ld + x_off + c]) + bxc;
            else tail[j] = has_past ? st[(size_t)(n + j) * C + c] : 0.f;
        }
    }
#pragma unroll
    for (int j = 0; j < REC_MAX_TAPS; ++j)
        if (j < K - 1) st[(size_t)j * C + c] = tail[j];
}

// For portions of several tokens the transcendental work leaves the sequential loop: recurrent_gate computes,
// for every token and channel at once, a = exp(-c r softplus(lam)) and b = sqrt(1 - a^2) i u (the same
// expressions as above); what is left is S = a S + b along the tokens.
__global__ void recurrent_gate_kernel(const float* __restrict__ u, const float* __restrict__ gates,
                                      const float* __restrict__ rb, const float* __restrict__ ib,
                                      const float* __restrict__ lam, float decay, float* __restrict__ a_out,
                                      float* __restrict__ b_out, int T, int C, int bs) {
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float sp = decay * rec_softplus(lam[c]);
    const float brc = rb[c], bic = ib[c];
    pdl_wait();
    pdl_trigger();
    const int blk = c / bs, o = c - blk * bs;
    const float* g = gates + ((size_t)blk * T + t) * 2 * bs + o;
    const float log_a = -sp * rec_sigmoid(g[0] + brc);
    a_out[(size_t)t * C + c] = expf(log_a);
    b_out[(size_t)t * C + c] = sqrtf(-expm1f(2.f * log_a)) * rec_sigmoid(g[bs] + bic) * u[(size_t)t * C + c];
}


// Four channels per thread with 16-byte accesses (C, bs, x_off and ld multiples of 4, 16-byte aligned bases): the
// same arithmetic as recurrent_conv_kernel and recurrent_gate_kernel, for steps of many tokens.
__device__ __forceinline__ float4 rec_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 rec_load4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void rec_store4(bf16* p, float4 v) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = o;
}

template <typename A>
__global__ void recurrent_conv_vec4_kernel(const A* __restrict__ proj, int ld, int x_off, const float* __restrict__ xb,
                                           const float* __restrict__ taps, const float* __restrict__ cb,
                                           const float* __restrict__ state, const int* __restrict__ cu_seqlens,
                                           const int* __restrict__ req_of_token, const int* __restrict__ start_pos,
                                           const int* __restrict__ slots, float* __restrict__ u, int C, int K,
                                           bf16* __restrict__ halves, int bs) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (c >= C) return;
    const int r = req_of_token[t];
    const int i = t - cu_seqlens[r];
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    const float4 b = rec_load4(xb + c);
    float4 acc = rec_load4(cb + c);
    const float* tp = taps + (size_t)c * K;                    // four channels' taps, K each
    for (int k = 0; k < K; ++k) {
        const int idx = i - k;
        float4 xin;
        if (idx >= 0) {
            xin = rec_load4(proj + (size_t)(t - k) * ld + x_off + c);
            xin.x += b.x; xin.y += b.y; xin.z += b.z; xin.w += b.w;
        } else if (has_past) {
            xin = rec_load4(state + ((size_t)slot * K + (K - 1 + idx)) * C + c);
        } else {
            xin = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const int j = K - 1 - k;
        acc.x += tp[j] * xin.x; acc.y += tp[K + j] * xin.y; acc.z += tp[2 * K + j] * xin.z; acc.w += tp[3 * K + j] * xin.w;
    }
    *reinterpret_cast<float4*>(u + (size_t)t * C + c) = acc;
    if (halves) {
        const int blk = c / bs, o = c - blk * bs;
        bf16* dst = halves + ((size_t)t * (C / bs) + blk) * 2 * bs + o;
        const float4 hi = make_float4(__bfloat162float(__float2bfloat16_rn(acc.x)), __bfloat162float(__float2bfloat16_rn(acc.y)),
                                      __bfloat162float(__float2bfloat16_rn(acc.z)), __bfloat162float(__float2bfloat16_rn(acc.w)));
        rec_store4(dst, hi);
        rec_store4(dst + bs, make_float4(acc.x - hi.x, acc.y - hi.y, acc.z - hi.z, acc.w - hi.w));
    }
}

__global__ void recurrent_gate_vec4_kernel(const float* __restrict__ u, const float* __restrict__ gates,
                                           const float* __restrict__ rb, const float* __restrict__ ib,
                                           const float* __restrict__ lam, float decay, float* __restrict__ a_out,
                                           float* __restrict__ b_out, int T, int C, int bs) {
    const int t = blockIdx.x;
    const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (c >= C) return;
    const float4 l4 = rec_load4(lam + c), br = rec_load4(rb + c), bi = rec_load4(ib + c);
    pdl_wait();
    pdl_trigger();
    const int blk = c / bs, o = c - blk * bs;
    const float* g = gates + ((size_t)blk * T + t) * 2 * bs + o;
    const float4 gr = rec_load4(g), gi = rec_load4(g + bs), uu = rec_load4(u + (size_t)t * C + c);
    float4 a, b;
#define REC_ONE(f) { const float log_a = -decay * rec_softplus(l4.f) * rec_sigmoid(gr.f + br.f); a.f = expf(log_a); \
                     b.f = sqrtf(-expm1f(2.f * log_a)) * rec_sigmoid(gi.f + bi.f) * uu.f; }
    REC_ONE(x) REC_ONE(y) REC_ONE(z) REC_ONE(w)
#undef REC_ONE
    *reinterpret_cast<float4*>(a_out + (size_t)t * C + c) = a;
    *reinterpret_cast<float4*>(b_out + (size_t)t * C + c) = b;
}

#define REC_AHEAD 8
#define REC_CHUNK 64
// The recurrence is associative, so a request's tokens are cut into chunks of REC_CHUNK that run side by side.
// recurrent_chunk: within each chunk, from S = 0: a[t] <- the product of the chunk's a up to t, b[t] <- the
// chunk's own S_t (both in place).  recurrent_finish: the state that enters chunk k is folded from the ends of
// the chunks before it (S <- b_end + a_end S, starting from the request's stored state), then
// S_t = b[t] + a[t] S_in, times the gate branch; the request's last chunk leaves S and the convolution's tail
// in the state slot.  Grid of both: (chunks of the longest request, requests, channels / threads).
__global__ void recurrent_chunk_kernel(float* __restrict__ a, float* __restrict__ b, const int* __restrict__ cu_seqlens,
                                       int C) {
    const int r = blockIdx.y;
    const int c = blockIdx.z * blockDim.x + threadIdx.x;
    pdl_wait();
    pdl_trigger();
    if (c >= C) return;
    const int end = cu_seqlens[r + 1];
    const int lo = cu_seqlens[r] + (int)blockIdx.x * REC_CHUNK, hi = min(end, lo + REC_CHUNK);
    float P = 1.f, S = 0.f;
    for (int t0 = lo; t0 < hi; t0 += REC_AHEAD) {
        float av[REC_AHEAD], bv[REC_AHEAD];
#pragma unroll
        for (int k = 0; k < REC_AHEAD; ++k) {
            const int t = min(t0 + k, hi - 1);
            av[k] = a[(size_t)t * C + c];
            bv[k] = b[(size_t)t * C + c];
        }
#pragma unroll
        for (int k = 0; k < REC_AHEAD; ++k) {
            if (t0 + k < hi) {
                P *= av[k];
                S = av[k] * S + bv[k];
                a[(size_t)(t0 + k) * C + c] = P;
                b[(size_t)(t0 + k) * C + c] = S;
            }
        }
    }
}

template <typename A>
__global__ void recurrent_finish_kernel(const A* __restrict__ proj, int ld, int y_off, int x_off,
                                        const float* __restrict__ yb, const float* __restrict__ xb,
                                        const float* __restrict__ a_in, const float* __restrict__ b_in,
                                        float* __restrict__ state, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ start_pos, const int* __restrict__ slots,
                                        A* __restrict__ out, int out_ld, float out_scale, int C, int K) {
    const int r = blockIdx.y;
    const int c = blockIdx.z * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float byc = yb[c], bxc = xb[c];
    pdl_wait();
    pdl_trigger();
    const int first = cu_seqlens[r], end = cu_seqlens[r + 1];
    const int lo = first + (int)blockIdx.x * REC_CHUNK, hi = min(end, lo + REC_CHUNK);
    if (lo >= end) return;
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    float* st = slot >= 0 ? state + (size_t)slot * K * C : nullptr;
    float S_in = has_past ? st[(size_t)(K - 1) * C + c] : 0.f;
    for (int j0 = 0; j0 < (int)blockIdx.x; j0 += REC_AHEAD) {        // the ends of the chunks before this one
        float av[REC_AHEAD], bv[REC_AHEAD];
#pragma unroll
        for (int k = 0; k < REC_AHEAD; ++k) {
            const int j = min(j0 + k, (int)blockIdx.x - 1);
            const size_t e = (size_t)(first + (j + 1) * REC_CHUNK - 1) * C + c;
            av[k] = a_in[e];
            bv[k] = b_in[e];
        }
#pragma unroll
        for (int k = 0; k < REC_AHEAD; ++k)
            if (j0 + k < (int)blockIdx.x) S_in = bv[k] + av[k] * S_in;
    }
    float S = S_in;
    for (int t0 = lo; t0 < hi; t0 += REC_AHEAD) {
        float av[REC_AHEAD], bv[REC_AHEAD], gv[REC_AHEAD];
#pragma unroll
        for (int k = 0; k < REC_AHEAD; ++k) {
            const int t = min(t0 + k, hi - 1);
            av[k] = a_in[(size_t)t * C + c];
            bv[k] = b_in[(size_t)t * C + c];
            gv[k] = to_f32(proj[(size_t)t * ld + y_off + c]);
        }
#pragma unroll
        for (int k = 0; k < REC_AHEAD; ++k) {
            if (t0 + k < hi) {
                S = bv[k] + av[k] * S_in;
                out[(size_t)(t0 + k) * out_ld + c] = from_f32<A>(S * rec_gelu_tanh(gv[k] + byc) * out_scale);
            }
        }
    }
    if (!st || hi != end) return;
    st[(size_t)(K - 1) * C + c] = S;
    const int n = end - first;
    float tail[REC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < REC_MAX_TAPS; ++j) {
        if (j < K - 1) {
            const int src = n - (K - 1) + j;
            if (src >= 0) tail[j] = to_f32(proj[(size_t)(first + src) * ld + x_off + c]) + bxc;
            else tail[j] = has_past ? st[(size_t)(n + j) * C + c] : 0.f;
        }
    }
#pragma unroll
    for (int j = 0; j < REC_MAX_TAPS; ++j)
        if (j < K - 1) st[(size_t)j * C + c] = tail[j];
}

extern "C" int rg_recurrent_conv(const void* proj, int dtype, int ld, int x_off, const float* xb, const float* taps,
                                 const float* cb, const float* state, const int* cu_seqlens, const int* req_of_token,
                                 const int* start_pos, const int* slots, float* u, int T, int C, int K, void* halves,
                                 int bs, void* stream) {
    if (T <= 0) return 0;
    if (C < 1 || K < 1 || K > REC_MAX_TAPS || (halves && (bs < 1 || C % bs))) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, (C + REC_THREADS - 1) / REC_THREADS);
    const bool vec4 = T >= 64 && C % 4 == 0 && ld % 4 == 0 && x_off % 4 == 0 && (!halves || bs % 4 == 0) &&
                      ((uintptr_t)proj | (uintptr_t)xb | (uintptr_t)taps | (uintptr_t)cb | (uintptr_t)state | (uintptr_t)u |
                       (uintptr_t)halves) % 16 == 0;
    if (vec4) {
        dim3 g4(T, (C / 4 + REC_THREADS - 1) / REC_THREADS);
        if (dtype == RG_DTYPE_BF16)
            return rg_launch(recurrent_conv_vec4_kernel<bf16>, g4, dim3(REC_THREADS), 0, s, 1, (const bf16*)proj, ld, x_off,
                             xb, taps, cb, state, cu_seqlens, req_of_token, start_pos, slots, u, C, K, (bf16*)halves, bs);
        if (dtype == RG_DTYPE_F32)
            return rg_launch(recurrent_conv_vec4_kernel<float>, g4, dim3(REC_THREADS), 0, s, 1, (const float*)proj, ld,
                             x_off, xb, taps, cb, state, cu_seqlens, req_of_token, start_pos, slots, u, C, K, (bf16*)halves, bs);
    }
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(recurrent_conv_kernel<bf16>, grid, dim3(REC_THREADS), 0, s, 1, (const bf16*)proj, ld, x_off, xb,
                         taps, cb, state, cu_seqlens, req_of_token, start_pos, slots, u, C, K, (bf16*)halves, bs);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(recurrent_conv_kernel<float>, grid, dim3(REC_THREADS), 0, s, 1, (const float*)proj, ld, x_off, xb,
                         taps, cb, state, cu_seqlens, req_of_token, start_pos, slots, u, C, K, (bf16*)halves, bs);
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_recurrent_scan(const void* proj, int dtype, int ld, int y_off, int x_off, const float* yb,
                                 const float* xb, const float* u, const float* gates, const float* rb, const float* ib,
                                 const float* lam, float decay, float* state, const int* cu_seqlens,
                                 const int* start_pos, const int* slots, void* out, int out_ld, float out_scale, int T,
                                 int R, int C, int K, int bs, float* ab, int max_tokens, void* stream) {
    if (T <= 0 || R <= 0) return 0;
    if (C < 1 || K < 1 || K > REC_MAX_TAPS || bs < 1 || C % bs) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(R, (C + REC_THREADS - 1) / REC_THREADS);
    if (ab) {
        // portions of several tokens: the gates of all tokens at once (ab: room for 2 T C floats), then the
        // recurrence in chunks side by side
        float* a_buf = ab;
        float* b_buf = ab + (size_t)T * C;
        if (max_tokens < 1 || R > 65535 || grid.y > 65535) return RG_ERR_UNSUPPORTED;
        int e;
        if (bs % 4 == 0 && ((uintptr_t)u | (uintptr_t)gates | (uintptr_t)rb | (uintptr_t)ib | (uintptr_t)lam | (uintptr_t)ab) % 16 == 0 &&
            ((size_t)T * C) % 4 == 0)
            e = rg_launch(recurrent_gate_vec4_kernel, dim3(T, (C / 4 + REC_THREADS - 1) / REC_THREADS), dim3(REC_THREADS), 0, s, 1,
                          u, gates, rb, ib, lam, decay, a_buf, b_buf, T, C, bs);
        else
            e = rg_launch(recurrent_gate_kernel, dim3(T, grid.y), dim3(REC_THREADS), 0, s, 1, u, gates, rb, ib, lam, decay,
                          a_buf, b_buf, T, C, bs);
        if (e) return e;
        dim3 cgrid((max_tokens + REC_CHUNK - 1) / REC_CHUNK, R, grid.y);
        e = rg_launch(recurrent_chunk_kernel, cgrid, dim3(REC_THREADS), 0, s, 1, a_buf, b_buf, cu_seqlens, C);
        if (e) return e;
        if (dtype == RG_DTYPE_BF16)
            return rg_launch(recurrent_finish_kernel<bf16>, cgrid, dim3(REC_THREADS), 0, s, 1, (const bf16*)proj, ld, y_off,
                             x_off, yb, xb, (const float*)a_buf, (const float*)b_buf, state, cu_seqlens, start_pos, slots,
                             (bf16*)out, out_ld, out_scale, C, K);
        if (dtype == RG_DTYPE_F32)
            return rg_launch(recurrent_finish_kernel<float>, cgrid, dim3(REC_THREADS), 0, s, 1, (const float*)proj, ld,
                             y_off, x_off, yb, xb, (const float*)a_buf, (const float*)b_buf, state, cu_seqlens, start_pos,
                             slots, (float*)out, out_ld, out_scale, C, K);
        return RG_ERR_UNSUPPORTED;
    }
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(recurrent_scan_kernel<bf16>, grid, dim3(REC_THREADS), 0, s, 1, (const bf16*)proj, ld, y_off,
                         x_off, yb, xb, u, gates, rb, ib, lam, decay, state, cu_seqlens, start_pos, slots, (bf16*)out,
                         out_ld, out_scale, T, C, K, bs);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(recurrent_scan_kernel<float>, grid, dim3(REC_THREADS), 0, s, 1, (const float*)proj, ld, y_off,
                         x_off, yb, xb, u, gates, rb, ib, lam, decay, state, cu_seqlens, start_pos, slots, (float*)out,
                         out_ld, out_scale, T, C, K, bs);
    return RG_ERR_UNSUPPORTED;
}
