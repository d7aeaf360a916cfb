// Attention over the compressed key/value cache on the tensor cores (bfloat16, mma.sync m16n8k16).
//
// One cache row per token, shared by all heads: [c (R numbers) | k_r (dr numbers)], D = R + dr.  Queries
// arrive with their plain part already taken through U_k^T: qa [T, H, D].
//   score[row, j] = scale * qa[row] . cache[j]      row = (token, head), j <= the token's position
//   out[row]      = sum_j softmax(score)[row, j] * cache[j][:R]
// so K and V are the SAME shared-memory tile (V is its first R columns): one load feeds both products, and
// the heads of a token are rows of one tile: a decode step's H heads make one 16-row tile that reads every
// cache row once.
//
// A block works on up to 64 rows: `tt` consecutive tokens of one request x `nh` heads, in row groups of 16.
// Each row group has CW warps (2 for prompts, 4 for single tokens with up to 32 heads).  For a tile of 32
// keys, warp c of the group computes the scores of 32 / CW keys (the long product over D, on two or four
// accumulator sets so that consecutive products do not wait for each other), the warps exchange their row
// maxima and the bfloat16 weights P through shared memory (two barriers of the group's threads), and then
// warp c accumulates O[:, its share of the R columns] += P V over all 32 keys.  Neither product is done
// twice, and a thread holds R / (2 CW) accumulators instead of R/2.  Softmax in 32-bit in the log2 domain,
// running maximum and sum per row; key tiles arrive through a two-stage cp.async ring, rows gathered through
// the block table.
//
// With `nsplit` > 1 (single tokens with long contexts) block z takes a contiguous share of the key tiles and
// writes an unnormalised partial result with its maximum and sum; latent_merge adds the shares.
#include "mma.cuh"
using namespace rgmma;

#define LM_BN 32                     // keys per tile
#define LM_PAD 8                     // bf16 of padding per shared-memory row (conflict-free ldmatrix)
#define LM_PSTRIDE (LM_BN + 8)       // row stride of the exchanged weights

// NDH: 8-column tiles of the output per warp at most (R <= 8 NDH CW); CW: warps per row group
template <int NDH, int CW>
__global__ void __launch_bounds__(256, 1) latent_attention_mma_kernel(
        const bf16* __restrict__ qa, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
        const bf16* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
        const int* __restrict__ tiles, int sub, int tt, const int* __restrict__ rows_list,
        const int* __restrict__ req_of_token, const int* __restrict__ positions, int H, int hc, int R, int D,
        int page_size, int window, float scale_log2, int nsplit, const float* __restrict__ sink, int sel_dv, int sel_hpg,
        int out_ld, float out_scale, int kd0) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int GT = 32 * CW;                                    // threads of a row group
    constexpr int KW = LM_BN / CW;                                 // keys a warp scores per tile: 16 or 8
    constexpr int NJ = KW / 8;
    const int RW = blockDim.x / GT;                                // row groups of 16
    const int stride = D + LM_PAD;
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);                  // [16 RW][stride]
    bf16* sK = sQ + 16 * RW * stride;                              // 2 stages x [LM_BN][stride]
    bf16* sP = sK + 2 * LM_BN * stride;                            // [RW][16][LM_PSTRIDE]
    float* sM = reinterpret_cast<float*>(sP + RW * 16 * LM_PSTRIDE);   // [RW][CW][16] row maxima of a warp's keys
    float* sL = sM + RW * CW * 16;                                 // [RW][CW][16] row sums, at the end
    pdl_wait();
    pdl_trigger();

    int row0, nt, req;
    if (tiles) {
        const int e = blockIdx.x / sub, s = blockIdx.x - e * sub;
        row0 = tiles[3 * e] + s * tt;
        nt = min(tt, tiles[3 * e + 1] - s * tt);
        if (nt <= 0) return;
        req = tiles[3 * e + 2];
    } else {
        row0 = rows_list ? rows_list[blockIdx.x] : blockIdx.x;
        nt = 1;
        req = req_of_token[row0];
    }
    const int h0 = blockIdx.y * hc, nh = min(hc, H - h0), nrows = nt * nh;
    const int p0 = positions[row0], hi = p0 + nt - 1;
    const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int kt_first = lo / LM_BN, kt_last = hi / LM_BN;
    const int per = (kt_last - kt_first + nsplit) / nsplit;
    const int kt0 = kt_first + (int)blockIdx.z * per, kt1 = min(kt_last, kt0 + per - 1);
    const int* bt = block_table + (size_t)req * max_blocks;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rw = warp / CW, cw = warp % CW;
    const int g = lane >> 2, tq = lane & 3;
    const int lr0 = rw * 16 + g, lr1 = lr0 + 8;
    const bool ok0 = lr0 < nrows, ok1 = lr1 < nrows;
    const int tok0 = row0 + lr0 / nh, tok1 = row0 + lr1 / nh, hd0 = h0 + lr0 % nh, hd1 = h0 + lr1 % nh;

    if (kt0 > kt1) {                                               // a share without keys
        if (cw == 0 && tq == 0) {
            if (ok0) { float* ml = part_ml + (((size_t)tok0 * H + hd0) * nsplit + blockIdx.z) * 2; ml[0] = -INFINITY; ml[1] = 0.f; }
            if (ok1) { float* ml = part_ml + (((size_t)tok1 * H + hd1) * nsplit + blockIdx.z) * 2; ml[0] = -INFINITY; ml[1] = 0.f; }
        }
        return;
    }

    const int chunks = D >> 3;                                     // 16-byte pieces of a row
    for (int idx = tid; idx < 16 * RW * chunks; idx += blockDim.x) {
        const int lr = idx / chunks, c = idx - lr * chunks;
        const bool valid = lr < nrows;
        const bf16* src = valid ? qa + ((size_t)(row0 + lr / nh) * H + h0 + lr % nh) * D + c * 8 : qa;
        cp_async16(sQ + lr * stride + c * 8, src, valid);
    }
    // a key row is copied by blockDim.x / 32 threads, 16 bytes at a time; keys beyond `hi` are zeros
    const int tpk = blockDim.x >> 5, my_key = tid / tpk, my_c0 = tid - my_key * tpk;
    // the page of this thread's key row is looked up one tile ahead, so that the table read is off the
    // critical path when the copies are issued
    auto page_of = [&](int kt) {
        const int key = kt * LM_BN + my_key;
        return key <= hi ? bt[key / page_size] : -1;
    };
    int page_next = page_of(kt0);
    auto load_keys = [&](int kt, bf16* dst) {
        const int key = kt * LM_BN + my_key;
        const bool valid = page_next >= 0;
        const bf16* src = valid ? cache + ((size_t)page_next * page_size + key % page_size) * D : cache;
        bf16* d = dst + my_key * stride;
        for (int c = my_c0; c < chunks; c += tpk) cp_async16(d + c * 8, src + c * 8, valid);
        page_next = page_of(kt + 1);
    };
    load_keys(kt0, sK);
    cp_async_commit();

    // positions of this thread's two rows (-1: a padding row sees nothing), and of the warp's first and last row
    const int pos0 = ok0 ? p0 + lr0 / nh : -1, pos1 = ok1 ? p0 + lr1 / nh : -1;
    const bool warp_has_rows = rw * 16 < nrows;
    const int wfirst = p0 + (rw * 16) / nh, wlast = p0 + min(rw * 16 + 15, nrows - 1) / nh;
    const int per16 = ((R >> 4) + CW - 1) / CW;                    // groups of 16 output columns per warp
    const int c0 = cw * per16 * 16, nd2 = max(0, min(per16, (R >> 4) - cw * per16));
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_key = (lane & 7) + (lane >> 4) * 8, b_dim = ((lane >> 3) & 1) * 8;
    const int v_key = (lane & 7) + ((lane >> 3) & 1) * 8, v_dim = (lane >> 4) * 8;
    bf16* sPw = sP + rw * 16 * LM_PSTRIDE;
    float* sMw = sM + rw * CW * 16;
    const int d16 = D >> 4;

    float o[NDH][4];
#pragma unroll
    for (int i = 0; i < NDH; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int kt = kt0; kt <= kt1; ++kt) {
        const int stage = (kt - kt0) & 1;
        const bf16* sKs = sK + stage * LM_BN * stride;
        if (kt + 1 <= kt1) {
            load_keys(kt + 1, sK + (stage ^ 1) * LM_BN * stride);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key_base = kt * LM_BN;
        const bool skip = !warp_has_rows || key_base > wlast || (window > 0 && key_base + LM_BN - 1 < wfirst - window + 1);
        if (!skip) {                                               // the same for both warps of a row group
            // NCH accumulator sets take the steps over D in turn, so that consecutive products do not wait for
            // each other and the fragment loads of several steps are in flight together
            constexpr int NCH = CW == 4 ? 4 : 2;
            float sc[NCH][NJ][4];
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
                for (int j = 0; j < NJ; ++j) { sc[c][j][0] = sc[c][j][1] = sc[c][j][2] = sc[c][j][3] = 0.f; }
            const bf16* qrow = sQ + (rw * 16 + a_row) * stride + a_col;
            const bf16* krow = CW == 2 ? sKs + (cw * KW + b_key) * stride + b_dim
                                       : sKs + (cw * KW + (lane & 7)) * stride + ((lane >> 3) & 1) * 8;
#pragma unroll 1
            for (int kd = kd0; kd < d16; kd += NCH) {           // kd0 > 0: the queries' first 16 kd0 numbers are zeros
                uint32_t a[NCH][4], b[NCH][4];
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    if (kd + c < d16) {
                        ldmatrix_x4(a[c], qrow + (kd + c) * 16);
                        if (CW == 2) ldmatrix_x4(b[c], krow + (kd + c) * 16);
                        else ldmatrix_x2(b[c], krow + (kd + c) * 16);
                    }
                }
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    if (kd + c < d16) {
                        mma_bf16(sc[c][0], a[c], b[c][0], b[c][1]);
                        if (CW == 2) mma_bf16(sc[c][NJ - 1], a[c], b[c][2], b[c][3]);
                    }
                }
            }
            float s[NJ][4];
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = sc[0][j][e];
#pragma unroll
                    for (int c = 1; c < NCH; ++c) v += sc[c][j][e];
                    s[j][e] = v;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key_base + cw * KW + j * 8 + tq * 2 + (e & 1);
                    const int prow = e < 2 ? pos0 : pos1;
                    float v = s[j][e] * scale_log2;
                    if (!(key <= prow && (window <= 0 || key > prow - window))) v = -INFINITY;
                    s[j][e] = v;
                    if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            if (tq == 0) { sMw[cw * 16 + g] = mx0; sMw[cw * 16 + g + 8] = mx1; }
            group_barrier<GT>(1 + rw);
#pragma unroll
            for (int c = 0; c < CW; ++c) {
                mx0 = fmaxf(mx0, sMw[c * 16 + g]);
                mx1 = fmaxf(mx1, sMw[c * 16 + g + 8]);
            }
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float al0 = ex2(m0 - ms0), al1 = ex2(m1 - ms1);
            m0 = mn0; m1 = mn1;
            float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                s[j][0] = ex2(s[j][0] - ms0); s[j][1] = ex2(s[j][1] - ms0);
                s[j][2] = ex2(s[j][2] - ms1); s[j][3] = ex2(s[j][3] - ms1);
                rs0 += s[j][0] + s[j][1];
                rs1 += s[j][2] + s[j][3];
                *reinterpret_cast<uint32_t*>(sPw + g * LM_PSTRIDE + cw * KW + j * 8 + tq * 2) = pack_bf16(s[j][0], s[j][1]);
                *reinterpret_cast<uint32_t*>(sPw + (g + 8) * LM_PSTRIDE + cw * KW + j * 8 + tq * 2) = pack_bf16(s[j][2], s[j][3]);
            }
            l0 = l0 * al0 + rs0;                                   // this thread's keys only; added up at the end
            l1 = l1 * al1 + rs1;
            if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                for (int i = 0; i < NDH; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
            }
            group_barrier<GT>(1 + rw);
#pragma unroll
            for (int kk = 0; kk < LM_BN / 16; ++kk) {
                uint32_t a[4];
                ldmatrix_x4(a, sPw + a_row * LM_PSTRIDE + kk * 16 + a_col);
#pragma unroll
                for (int n2 = 0; n2 < NDH / 2; ++n2) {
                    if (n2 < nd2) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, sKs + (kk * 16 + v_key) * stride + c0 + n2 * 16 + v_dim);
                        mma_bf16(o[2 * n2], a, b[0], b[1]);
                        mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                           // the stage is overwritten by the next iteration's copies
    }
    if (!warp_has_rows) return;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* sLw = sL + rw * CW * 16;
    if (tq == 0) { sLw[cw * 16 + g] = l0; sLw[cw * 16 + g + 8] = l1; }
    group_barrier<GT>(1 + rw);
    l0 = l1 = 0.f;
#pragma unroll
    for (int c = 0; c < CW; ++c) { l0 += sLw[c * 16 + g]; l1 += sLw[c * 16 + g + 8]; }
    if (nsplit == 1) {
        if (sink) {                                                // exp(sink[head]) joins the denominator, once
            if (ok0 && m0 > -INFINITY) l0 += ex2(sink[hd0] * 1.4426950408889634f - m0);
            if (ok1 && m1 > -INFINITY) l1 += ex2(sink[hd1] * 1.4426950408889634f - m1);
        }
        const float inv0 = l0 > 0.f ? out_scale / l0 : 0.f, inv1 = l1 > 0.f ? out_scale / l1 : 0.f;
        if (sel_dv > 0) {
            // head h keeps columns [(h / sel_hpg) sel_dv, + sel_dv) of the R, as out[token, h sel_dv + c]
            const int lo0 = (hd0 / sel_hpg) * sel_dv, lo1 = (hd1 / sel_hpg) * sel_dv;
            bf16* o0 = out + (size_t)tok0 * out_ld + (size_t)hd0 * sel_dv - lo0;
            bf16* o1 = out + (size_t)tok1 * out_ld + (size_t)hd1 * sel_dv - lo1;
#pragma unroll
            for (int i = 0; i < NDH; ++i) {
                if (i < 2 * nd2) {
                    const int col = c0 + i * 8 + tq * 2;
                    if (ok0 && col >= lo0 && col < lo0 + sel_dv) {
                        o0[col] = __float2bfloat16_rn(o[i][0] * inv0); o0[col + 1] = __float2bfloat16_rn(o[i][1] * inv0);
                    }
                    if (ok1 && col >= lo1 && col < lo1 + sel_dv) {
                        o1[col] = __float2bfloat16_rn(o[i][2] * inv1); o1[col + 1] = __float2bfloat16_rn(o[i][3] * inv1);
                    }
                }
            }
            return;
        }
        bf16* o0 = out + ((size_t)tok0 * H + hd0) * R + c0;
        bf16* o1 = out + ((size_t)tok1 * H + hd1) * R + c0;
#pragma unroll
        for (int i = 0; i < NDH; ++i) {
            if (i < 2 * nd2) {
                const int col = i * 8 + tq * 2;
                if (ok0) *reinterpret_cast<uint32_t*>(o0 + col) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
                if (ok1) *reinterpret_cast<uint32_t*>(o1 + col) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
            }
        }
    } else {
        const size_t r0 = ((size_t)tok0 * H + hd0) * nsplit + blockIdx.z, r1 = ((size_t)tok1 * H + hd1) * nsplit + blockIdx.z;
        if (cw == 0 && tq == 0) {
            if (ok0) { part_ml[r0 * 2] = m0; part_ml[r0 * 2 + 1] = l0; }
            if (ok1) { part_ml[r1 * 2] = m1; part_ml[r1 * 2 + 1] = l1; }
        }
#pragma unroll
        for (int i = 0; i < NDH; ++i) {
            if (i < 2 * nd2) {
                const int col = c0 + i * 8 + tq * 2;
                if (ok0) *reinterpret_cast<float2*>(part_o + r0 * R + col) = make_float2(o[i][0], o[i][1]);
                if (ok1) *reinterpret_cast<float2*>(part_o + r1 * R + col) = make_float2(o[i][2], o[i][3]);
            }
        }
    }
}

// out[token, head] = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z over the shares that saw keys, in share order
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, const int* __restrict__ rows_list, int H, int R, int nsplit,
                                    const float* __restrict__ sink, int sel_dv, int sel_hpg, int out_ld, float out_scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float wz[];                  // a share's factor 2^(m_z - M) / L, 0 for a share without keys
    const int t = rows_list ? rows_list[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    const size_t base = ((size_t)t * H + h) * nsplit;
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int z = threadIdx.x; z < nsplit; z += 32)
            if (part_ml[(base + z) * 2 + 1] > 0.f) M = fmaxf(M, part_ml[(base + z) * 2]);
        M = warp_max(M);
        float L = 0.f;
        for (int z = threadIdx.x; z < nsplit; z += 32) {
            const float l = part_ml[(base + z) * 2 + 1];
            const float f = l > 0.f ? ex2(part_ml[(base + z) * 2] - M) : 0.f;
            wz[z] = f;
            L += l * f;
        }
        L = warp_sum(L);
        if (sink && M > -INFINITY) L += ex2(sink[h] * 1.4426950408889634f - M);
        const float inv = L > 0.f ? out_scale / L : 0.f;
        for (int z = threadIdx.x; z < nsplit; z += 32) wz[z] *= inv;
    }
    __syncthreads();
    const int first = sel_dv > 0 ? (h / sel_hpg) * sel_dv : 0, count = sel_dv > 0 ? sel_dv : R;
    bf16* orow = sel_dv > 0 ? out + (size_t)t * out_ld + (size_t)h * sel_dv : out + ((size_t)t * H + h) * R;
    for (int c = threadIdx.x; c < count; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int z = 0; z < nsplit; ++z) {
            const float f = wz[z];
            if (f > 0.f) acc += part_o[(base + z) * R + first + c] * f;
        }
        orow[c] = __float2bfloat16_rn(acc);
    }
}

// Options of both kernels: `sink` [H] (exp(sink[h]) joins head h's denominator once: in the kernel without
// shares, in the merge with them); `sel_dv` > 0: head h keeps only columns [(h / sel_hpg) sel_dv, + sel_dv) of
// its R output numbers and writes them to out[token * out_ld + h * sel_dv + c] (a cache row that holds several
// value heads side by side, of which a head wants its own); `out_scale` multiplies the result; `score_from`
// (a multiple of 16): the scores run over the row's numbers from there on only (the queries are zero before).
template <typename K> static int lm_allow_smem(K kernel, size_t bytes) {
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

static size_t lm_smem_bytes(int RW, int D) {
    return (size_t)(16 * RW + 2 * LM_BN) * (D + LM_PAD) * 2 + (size_t)RW * 16 * LM_PSTRIDE * 2 + (size_t)RW * 128 * 4;
}

// Whether the sizes fit these kernels (0: yes).
extern "C" int rg_latent_attention_mma_ok(int H, int R, int D) {
    if (R < 16 || (R & 15) || (D & 15) || D < R || H < 1) return RG_ERR_UNSUPPORTED;
    if (((R >> 4) + 1) / 2 * 2 > 32) return RG_ERR_UNSUPPORTED;                // more than 32 column tiles per warp
    if (lm_smem_bytes(4, D) > 227 * 1024) return RG_ERR_UNSUPPORTED;
    return 0;
}

// tiles != nullptr: requests with several tokens, [n_items][3] = first row, rows (<= 64), request; every entry
// is cut into work items of 64 / heads tokens.  tiles == nullptr: n_items single tokens (rows_list or rows
// 0..n_items-1), each context cut into nsplit shares (part_o [T, H, nsplit, R], part_ml [T, H, nsplit, 2]).
extern "C" int rg_latent_attention_mma(
        const void* qa, void* out, float* part_o, float* part_ml, const void* cache, const int* block_table,
        int max_blocks, const int* tiles, const int* rows_list, int n_items, const int* req_of_token,
        const int* positions, int H, int R, int D, int page_size, int window, float scale, int nsplit,
        const float* sink, int sel_dv, int sel_hpg, int out_ld, float out_scale, int score_from, void* stream) {
    if (n_items <= 0) return 0;
    if (score_from < 0 || score_from % 16 || score_from >= D) return RG_ERR_UNSUPPORTED;
    if (sel_dv < 0 || (sel_dv > 0 && (sel_hpg < 1 || (sel_dv & 1) || ((H + sel_hpg - 1) / sel_hpg) * sel_dv > R)))
        return RG_ERR_UNSUPPORTED;
    if (rg_latent_attention_mma_ok(H, R, D) || page_size < 1 || nsplit < 1 || nsplit > 65535) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int hc = H < 64 ? H : 64, chunks = (H + hc - 1) / hc;
    int tt = 1, sub = 1, RW;
    if (tiles) {
        tt = 64 / hc;
        sub = (64 + tt - 1) / tt;
        RW = 4;
        nsplit = 1;
    } else {
        RW = (hc + 15) / 16;
        if (nsplit > 1 && (!part_o || !part_ml)) return RG_ERR_UNSUPPORTED;
    }
    const size_t smem = lm_smem_bytes(RW, D);
    const int CW = (!tiles && RW <= 2) ? 4 : 2;                    // single tokens of up to 32 heads: four warps per row group
    const int ndh = ((R >> 4) + CW - 1) / CW * 2;
    dim3 grid(n_items * sub, chunks, nsplit), block(32 * CW * RW);
    const float scale_log2 = scale * 1.4426950408889634f;
    int e;
#define RG_LM(N, C) { e = lm_allow_smem(latent_attention_mma_kernel<N, C>, smem); if (e) return e; \
        e = rg_launch(latent_attention_mma_kernel<N, C>, grid, block, smem, s, 1, (const bf16*)qa, (bf16*)out, part_o, part_ml, \
                      (const bf16*)cache, block_table, max_blocks, tiles, sub, tt, rows_list, req_of_token, positions, H, hc, \
                      R, D, page_size, window, scale_log2, nsplit, sink, sel_dv, sel_hpg, out_ld, out_scale, score_from >> 4); }
    if (CW == 2) { if (ndh <= 8) RG_LM(8, 2) else if (ndh <= 16) RG_LM(16, 2) else RG_LM(32, 2) }
    else { if (ndh <= 4) RG_LM(4, 4) else if (ndh <= 8) RG_LM(8, 4) else RG_LM(16, 4) }
#undef RG_LM
    if (e || nsplit == 1) return e;
    return rg_launch(latent_merge_kernel, dim3(n_items, H), dim3(R >= 256 ? 128 : 64), (size_t)nsplit * sizeof(float), s, 1, (const float*)part_o,
                     (const float*)part_ml, (bf16*)out, rows_list, H, R, nsplit, sink, sel_dv, sel_hpg, out_ld, out_scale);
}
