// The fasterquant stage: weight/gradient permutation, GPTQ+ first-order terms, the per-block
// column loop (round/clamp quantize, error feedback, first-order term) and the lazy trailing
// update, plus the un-permuting epilogue.  All row sub-groups of a linear run in the same launches.
//
// Rows are independent in this algorithm (every formula combines one row of W with the shared
// Hinv of its group), so the column loop gives each weight row to one warp: the 128-column panel
// of the row lives in registers (4 columns per lane), the 128x128 Hinv block in shared memory, and
// the per-column scalars travel by warp shuffle.
#include "rq_common.cuh"
#include "rq_gemm.cuh"
#include "rq_umma_gemm.cuh"

namespace rq {
namespace fq {

constexpr int BS = 128;                      // column block (the reference's blocksize)
constexpr int kRowsPerCta = 16;              // one warp per row
constexpr int kBlockThreads = kRowsPerCta * 32;

// ------------------------------------------------------------------------------------------
// Wp[r][j] = dead(g(r), perm[j]) ? 0 : W[r][perm[j]];   Gp[r][j] = Grad[r][perm[j]]
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prep_kernel(const float* __restrict__ W, const float* __restrict__ Grad,
                                                   const float* __restrict__ H, const int64_t* __restrict__ perm,
                                                   int R, int C, int G, float* __restrict__ Wp,
                                                   float* __restrict__ Gp) {
    for (int r = blockIdx.y; r < R; r += gridDim.y) {
        const int g = r / (R / G);
        const float* Hg = H + (int64_t)g * C * C;
        for (int j = blockIdx.x * 256 + threadIdx.x; j < C; j += gridDim.x * 256) {
            const int64_t pj = perm ? perm[j] : j;
            const bool dead = Hg[pj * C + pj] == 0.f;
            Wp[(int64_t)r * C + j] = dead ? 0.f : W[(int64_t)r * C + pj];
            if (Gp) Gp[(int64_t)r * C + j] = Grad[(int64_t)r * C + pj];
        }
    }
}

// ------------------------------------------------------------------------------------------
// GPTQ+ first-order terms
// ------------------------------------------------------------------------------------------
// T = Gp . U^T  (step 1, U upper: k starts at the column tile)   GHI = T . U  (step 2: k ends with it)
// grid (tiles_m, tiles_n, G)
__global__ void __launch_bounds__(gemm::kThreads, 2) terms_gemm_kernel(const float* __restrict__ In,
                                                                    const float* __restrict__ U,
                                                                    float* __restrict__ Out, int Rg, int C, int Cp,
                                                                    int step) {
    extern __shared__ float smem[];
    const int g = blockIdx.z;
    gemm::Args a;
    a.A = In + (int64_t)g * Rg * C; a.lda = C;
    a.B = U + (int64_t)g * Cp * Cp; a.ldb = Cp;
    a.C = Out + (int64_t)g * Rg * C; a.ldc = C;
    a.Aux = nullptr; a.ldaux = 0;
    a.M = Rg; a.N = C; a.K = C;
    a.alpha = 1.f; a.beta = 0.f; a.gamma = 0.f;
    const int j0 = blockIdx.y * gemm::TN;
    if (step == 1) {
        a.k_begin = j0; a.k_end = C;
        gemm::tile<true>(a, blockIdx.x * gemm::TM, j0, smem);
    } else {
        a.k_begin = 0; a.k_end = (j0 + gemm::TN < C) ? j0 + gemm::TN : C;
        gemm::tile<false>(a, blockIdx.x * gemm::TM, j0, smem);
    }
}

// hdiag[g][j] = diag(H^-1)_j = sum_i U[i][j]^2
__global__ void __launch_bounds__(256) hinv_diag_kernel(const float* __restrict__ U, int C, int Cp,
                                                        float* __restrict__ hdiag) {
    const int g = blockIdx.y;
    const int j = blockIdx.x * 256 + threadIdx.x;
    if (j >= C) return;
    const float* Ug = U + (int64_t)g * Cp * Cp;
    float s = 0.f;
    for (int i = 0; i <= j; ++i) {
        const float v = Ug[(int64_t)i * Cp + j];
        s = fmaf(v, v, s);
    }
    hdiag[(int64_t)g * C + j] = s;
}

// beta[r] from c = sum_j G*GHI - mean_j(GHI^2 / diag(H^-1)); then Z = beta*T, GH = beta*GHI in place.
// One block per row.
__global__ void __launch_bounds__(256) beta_kernel(const float* __restrict__ Gp, float* __restrict__ T,
                                                   float* __restrict__ GHI, const float* __restrict__ hdiag, int R,
                                                   int C, int G, float alpha_eff, float ref_loss,
                                                   float* __restrict__ beta) {
    __shared__ float red[16];
    __shared__ float bsh;
    const int r = blockIdx.x;
    const int g = r / (R / G);
    const float* gp = Gp + (int64_t)r * C;
    float* t = T + (int64_t)r * C;
    float* gh = GHI + (int64_t)r * C;
    const float* hd = hdiag + (int64_t)g * C;
    float s1 = 0.f, s2 = 0.f;
    for (int j = threadIdx.x; j < C; j += 256) {
        const float v = gh[j];
        s1 += gp[j] * v;
        s2 += __fdiv_rn(v * v, hd[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = s1; red[8 + (threadIdx.x >> 5)] = s2; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.f, b = 0.f;
        for (int w = 0; w < 8; ++w) { a += red[w]; b += red[8 + w]; }
        float bv = 0.f;
        if (ref_loss > 0.f) {
            float c = a - b / (float)C;
            const float target = 2.f * alpha_eff * ref_loss;
            if (c < target) c = target;                            // clamp(min=target); a NaN stays NaN
            float ratio = (c > 0.f) ? __fdiv_rn(target, c) : 0.f;  // NaN compares false -> 0
            ratio = fminf(fmaxf(ratio, 0.f), 1.f);
            bv = 1.f - sqrtf(fmaxf(1.f - ratio, 0.f));
            if (isnan(bv)) bv = 0.f;
            else if (isinf(bv)) bv = bv > 0.f ? 1.f : 0.f;
        }
        bsh = bv;
        beta[r] = bv;
    }
    __syncthreads();
    const float bv = bsh;
    for (int j = threadIdx.x; j < C; j += 256) {
        t[j] *= bv;
        gh[j] *= bv;
    }
}

// ------------------------------------------------------------------------------------------
// the column loop of one block [i1, i1+count)
// ------------------------------------------------------------------------------------------
struct BlockArgs {
    float* Wp;               // [R, C] working weights (permuted order), updated in place for the block
    float* GH;               // [R, C] first-order term GHinv (PLUS)
    const float* Z;          // [R, C] (PLUS)
    const float* Hinv;       // [G, Cp, Cp] upper factor
    float* Q;                // [R, C] dequantized result (permuted order)
    int16_t* codes;           // [R, C] integer codes (permuted order)
    float* Eeff;             // [R, BS]: Err (- D*Z1 when PLUS), A operand of the lazy update
    __nv_bfloat16* Ehi;      // optional: the same operand split into bf16 planes [R][BS] for the tensor-core update
    __nv_bfloat16* Elo;
    // optional second operand for a deferred update of the columns beyond the current group of blocks:
    // Err - (D + far_after) * Z split into planes [R][far_ld] at column offset far_k0 (far_after = number of
    // columns between this block's end and the end of its group)
    __nv_bfloat16* Fhi;
    __nv_bfloat16* Flo;
    int far_ld, far_k0;
    float far_after;
    const float* scale_row;  // mode 0: [R]
    const float* scale_tab;  // mode 1: [ngroups, R] static groups
    const int* colgrp;       // mode 1: [C] group of (permuted) column j
    float* scale_blk;        // mode 2: [C/gs_dyn blocks..., R] scales found on the fly (output)
    int R, C, Cp, G, i1, count;
    const float* anchor;     // [R, C] weights as they were before the first block (surrogate modes)
    const float* beta;       // [R] (surrogate modes)
    int inner_mode;          // 0 frozen, 1 surrogate_block, 2 surrogate_online: GHinv_eff = GHinv + beta*(W - anchor)
    int atomic;              // quantize the whole block from its start values, then solve for the errors
    float so_scale;          // factor on the in-block weight update (block_gd's second_order_scale); 1 elsewhere
    int mode;                // 0 per-row scale, 1 static groups, 2 dynamic groups
    int dyn_gs;              // mode 2: group width (divides BS)
    int sym;                 // mode 2: range rule
    float qlo, qhi;          // clamp bounds -(maxq+1), maxq
    float maxq;
};

template <bool PLUS>
__global__ void __launch_bounds__(kBlockThreads) block_kernel(const BlockArgs p) {
    extern __shared__ float Hs[];                          // [BS][BS] Hinv1, row-major
    const int Rg = p.R / p.G;
    const int ctas_per_group = (Rg + kRowsPerCta - 1) / kRowsPerCta;
    const int g = blockIdx.x / ctas_per_group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_in_group = (blockIdx.x % ctas_per_group) * kRowsPerCta + warp;
    const float* Hb = p.Hinv + (int64_t)g * p.Cp * p.Cp + (int64_t)p.i1 * p.Cp + p.i1;
    for (int e = threadIdx.x; e < BS * BS; e += kBlockThreads) {
        const int i = e >> 7, j = e & 127;
        Hs[e] = (i < p.count && j < p.count) ? Hb[(int64_t)i * p.Cp + j] : 0.f;
    }
    __syncthreads();
    if (row_in_group >= Rg) return;
    const int r = g * Rg + row_in_group;
    const int64_t base = (int64_t)r * p.C + p.i1;

    float w[4], gh[4], z[4], sc[4], qv[4], cv[4], ev[4], dref[4];
    const bool surrogate = PLUS && p.inner_mode != 0;
    const float bt = surrogate ? p.beta[r] : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int col = lane + 32 * k;
        const bool in = col < p.count;
        w[k] = in ? p.Wp[base + col] : 0.f;
        gh[k] = (PLUS && in) ? p.GH[base + col] : 0.f;
        z[k] = (PLUS && in) ? p.Z[base + col] : 0.f;
        qv[k] = 0.f; cv[k] = 0.f; ev[k] = 0.f;
        sc[k] = 1.f;
        // surrogate_block keeps (W_block_start - W_anchor); surrogate_online needs the anchor itself
        dref[k] = (surrogate && in) ? p.anchor[base + col] : 0.f;
        if (surrogate && p.inner_mode == 1) dref[k] = __fsub_rn(w[k], dref[k]);
    }
    if (p.mode == 0) {
        const float s = p.scale_row[r];
#pragma unroll
        for (int k = 0; k < 4; ++k) sc[k] = s;
    } else if (p.mode == 1) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int col = lane + 32 * k;
            if (col < p.count) sc[k] = p.scale_tab[(int64_t)p.colgrp[p.i1 + col] * p.R + r];
        }
    } else {
        // dynamic groups: ranges of the block-start values, one per dyn_gs-wide group inside the block
        const int ngrp = (p.count + p.dyn_gs - 1) / p.dyn_gs;
        for (int gi = 0; gi < ngrp; ++gi) {
            float lo = 0.f, hi = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int col = lane + 32 * k;
                if (col < p.count && col / p.dyn_gs == gi) { lo = fminf(lo, w[k]); hi = fmaxf(hi, w[k]); }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
                hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
            }
            float s;
            if (p.sym) {
                s = __fdiv_rn(fmaxf(fmaxf(fabsf(lo), hi), 1e-5f), p.maxq);
            } else {
                if (lo == 0.f && hi == 0.f) { lo = -1.f; hi = 1.f; }
                s = __fdiv_rn(fmaxf(hi - lo, 1e-5f), p.maxq);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int col = lane + 32 * k;
                if (col / p.dyn_gs == gi) sc[k] = s;
            }
            if (lane == 0) p.scale_blk[(int64_t)((p.i1 + gi * p.dyn_gs) / p.dyn_gs) * p.R + r] = s;
        }
    }

    // effective first-order term of column k right now (the reference's _current_ghinv)
    auto effective = [&](int k) -> float {
        if (!surrogate) return gh[k];
        const float diff = (p.inner_mode == 1) ? dref[k] : __fsub_rn(w[k], dref[k]);
        return __fadd_rn(gh[k], __fmul_rn(bt, diff));
    };
    if (p.atomic) {
        // whole block quantized from its start values; Err solves  Err . Hinv1 = W_start - Q - GHinv_eff
        float res[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float qi = quant_code(w[k], sc[k], p.qlo, p.qhi);
            cv[k] = qi;
            qv[k] = __fmul_rn(sc[k], qi);
            res[k] = __fsub_rn(w[k], qv[k]);
            if (PLUS) res[k] = __fsub_rn(res[k], effective(k));
        }
#pragma unroll
        for (int slot = 0; slot < 4; ++slot) {
            const int ibase = slot * 32;
            if (ibase >= p.count) break;
            const int iend = (p.count - ibase < 32) ? p.count - ibase : 32;
            for (int o = 0; o < iend; ++o) {
                const int i = ibase + o;
                const float x = __fdiv_rn(__shfl_sync(0xffffffffu, res[slot], o), Hs[i * BS + i]);
                if (lane == o) ev[slot] = x;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int col = lane + 32 * k;
                    if (col > i && col < p.count) res[k] = __fsub_rn(res[k], __fmul_rn(x, Hs[i * BS + col]));
                }
            }
        }
    } else {
#pragma unroll
    for (int slot = 0; slot < 4; ++slot) {
        const int ibase = slot * 32;
        if (ibase >= p.count) break;
        const int iend = (p.count - ibase < 32) ? p.count - ibase : 32;
        for (int o = 0; o < iend; ++o) {
            const int i = ibase + o;
            const float wi = __shfl_sync(0xffffffffu, w[slot], o);
            const float si = __shfl_sync(0xffffffffu, sc[slot], o);
            const float qi = quant_code(wi, si, p.qlo, p.qhi);
            const float q = __fmul_rn(si, qi);
            const float d = Hs[i * BS + i];
            float err;
            float zi = 0.f;
            float eff[4] = {0.f, 0.f, 0.f, 0.f};
            if (PLUS) {
#pragma unroll
                for (int k = 0; k < 4; ++k) eff[k] = effective(k);
                const float ghi = __shfl_sync(0xffffffffu, eff[slot], o);
                zi = __shfl_sync(0xffffffffu, z[slot], o);
                err = __fdiv_rn(__fsub_rn(__fsub_rn(wi, q), ghi), d);
            } else {
                err = __fdiv_rn(__fsub_rn(wi, q), d);
            }
            if (lane == o) { qv[slot] = q; cv[slot] = qi; ev[slot] = err; }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (32 * k + 31 < i) continue;             // every column of this slot is already quantized (warp-uniform)
                const int col = lane + 32 * k;
                if (col >= i && col < p.count) {
                    const float h = Hs[i * BS + col];
                    float upd = __fmul_rn(err, h);
                    if (PLUS) {
                        upd = __fadd_rn(upd, eff[k]);
                        gh[k] = __fsub_rn(gh[k], __fmul_rn(zi, h));
                    }
                    if (p.so_scale != 1.f) upd = __fmul_rn(p.so_scale, upd);
                    w[k] = __fsub_rn(w[k], upd);
                }
            }
        }
    }
    }

#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int col = lane + 32 * k;
        if (col < p.count) {
            p.Q[base + col] = qv[k];
            p.codes[base + col] = (int16_t)cv[k];
            float e = ev[k];
            if (PLUS) e = e - (float)(p.count - 1 - col) * z[k];
            p.Eeff[(int64_t)r * BS + col] = e;
            if (p.Ehi) {
                const __nv_bfloat16 h = __float2bfloat16_rn(e);
                p.Ehi[(int64_t)r * BS + col] = h;
                p.Elo[(int64_t)r * BS + col] = __float2bfloat16_rn(e - __bfloat162float(h));
            }
            if (p.Fhi) {
                float f = ev[k];
                if (PLUS) f = f - ((float)(p.count - 1 - col) + p.far_after) * z[k];
                const __nv_bfloat16 h = __float2bfloat16_rn(f);
                p.Fhi[(int64_t)r * p.far_ld + p.far_k0 + col] = h;
                p.Flo[(int64_t)r * p.far_ld + p.far_k0 + col] = __float2bfloat16_rn(f - __bfloat162float(h));
            }
        } else {
            p.Eeff[(int64_t)r * BS + col] = 0.f;
            if (p.Ehi) {
                p.Ehi[(int64_t)r * BS + col] = __float2bfloat16_rn(0.f);
                p.Elo[(int64_t)r * BS + col] = __float2bfloat16_rn(0.f);
            }
            if (p.Fhi) {
                p.Fhi[(int64_t)r * p.far_ld + p.far_k0 + col] = __float2bfloat16_rn(0.f);
                p.Flo[(int64_t)r * p.far_ld + p.far_k0 + col] = __float2bfloat16_rn(0.f);
            }
        }
    }
}

// outer surrogate term: the lazy update subtracts count * beta * (W - anchor) as well, taken at the weights
// before the update (gptq_plus_utils.py:1502-1513 with outer mode surrogate_block); applied as a pre-pass.
__global__ void __launch_bounds__(256) surrogate_outer_kernel(float* __restrict__ Wp, const float* __restrict__ anchor,
                                                              const float* __restrict__ beta, int R, int C, int i2,
                                                              float count) {
    for (int r = blockIdx.y; r < R; r += gridDim.y) {
        const float cb = count * beta[r];
        for (int j = i2 + blockIdx.x * 256 + threadIdx.x; j < C; j += gridDim.x * 256) {
            const int64_t e = (int64_t)r * C + j;
            Wp[e] = __fsub_rn(Wp[e], __fmul_rn(cb, __fsub_rn(Wp[e], anchor[e])));
        }
    }
}

// lazy update for the columns right of the block:  grid (tiles_m, tiles_n, G)
//   step 1:  W[:, i2:]  -= Eeff . Hinv[i1:i2, i2:]  +  count * GH[:, i2:]     (the latter when PLUS)
//   step 2:  GH[:, i2:] -= Z[:, i1:i2] . Hinv[i1:i2, i2:]                      (PLUS only)
__global__ void __launch_bounds__(gemm::kThreads, 2) lazy_kernel(float* __restrict__ Wp, float* __restrict__ GH,
                                                              const float* __restrict__ Z,
                                                              const float* __restrict__ Eeff,
                                                              const float* __restrict__ Hinv, int R, int C, int Cp,
                                                              int G, int i1, int count, int step, int plus,
                                                              float so_scale) {
    extern __shared__ float smem[];
    const int g = blockIdx.z;
    const int Rg = R / G;
    const int i2 = i1 + count;
    const int64_t rofs = (int64_t)g * Rg;
    gemm::Args a;
    a.B = Hinv + (int64_t)g * Cp * Cp + (int64_t)i1 * Cp + i2; a.ldb = Cp;
    a.M = Rg; a.N = C - i2; a.K = count;
    a.alpha = -1.f; a.beta = 1.f;
    a.k_begin = 0; a.k_end = count;
    a.Aux = nullptr; a.ldaux = 0; a.gamma = 0.f;
    if (step == 1) {
        a.A = Eeff + rofs * BS; a.lda = BS;
        a.C = Wp + rofs * C + i2; a.ldc = C;
        a.alpha = -so_scale;                                    // block_gd scales the whole weight update
        if (plus) { a.Aux = GH + rofs * C + i2; a.ldaux = C; a.gamma = -so_scale * (float)count; }
    } else {
        a.A = Z + rofs * C + i1; a.lda = C;
        a.C = GH + rofs * C + i2; a.ldc = C;
    }
    gemm::tile<false>(a, blockIdx.x * gemm::TM, blockIdx.y * gemm::TN, smem);
}

// ------------------------------------------------------------------------------------------
// epilogue: un-permute and cast.  out[r][perm[j]] = Q[r][j]  (also codes / scale when exported)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) unpermute_kernel(const float* __restrict__ Q, const int16_t* __restrict__ codes,
                                                        const int64_t* __restrict__ perm, int R, int C,
                                                        T* __restrict__ out, float* __restrict__ out_codes,
                                                        float* __restrict__ out_scale,
                                                        const float* __restrict__ scale_row,
                                                        const float* __restrict__ scale_tab,
                                                        const int* __restrict__ colgrp, int permute_export) {
    for (int r = blockIdx.y; r < R; r += gridDim.y) {
        for (int j = blockIdx.x * 256 + threadIdx.x; j < C; j += gridDim.x * 256) {
            const int64_t dst = perm ? perm[j] : j;
            store_from_float<T>(out, (int64_t)r * C + dst, Q[(int64_t)r * C + j]);
            if (out_codes) {
                const int64_t edst = permute_export ? dst : j;
                out_codes[(int64_t)r * C + edst] = (float)codes[(int64_t)r * C + j];
                out_scale[(int64_t)r * C + edst] = scale_tab ? scale_tab[(int64_t)colgrp[j] * R + r] : scale_row[r];
            }
        }
    }
}

}  // namespace fq
}  // namespace rq

using namespace rq;

extern "C" int rq_fq_prepare(const float* W, const float* Grad, const float* H, const int64_t* perm, int R, int C,
                             int G, float* Wp, float* Gp, void* stream) {
    if (!W || !H || !Wp || R <= 0 || C <= 0 || G <= 0 || R % G != 0 || (Gp && !Grad)) return RQ_ERR_INVALID;
    dim3 grid((unsigned)((C + 1023) / 1024), (unsigned)(R < 65535 ? R : 65535));
    fq::prep_kernel<<<grid, 256, 0, as_stream(stream)>>>(W, Grad, H, perm, R, C, G, Wp, Gp);
    return check_launch();
}

extern "C" int rq_gptqplus_terms(const float* Gp, const float* Hinv, int R, int C, int G, float alpha_eff,
                                 float ref_loss, float* Z, float* GHinv, float* beta, float* hdiag, void* stream) {
    if (!Gp || !Hinv || !Z || !GHinv || !beta || !hdiag || R <= 0 || C <= 0 || G <= 0 || R % G != 0)
        return RQ_ERR_INVALID;
    cudaStream_t st = as_stream(stream);
    const int Cp = (C + 127) / 128 * 128;
    const int Rg = R / G;
    dim3 grid((unsigned)((Rg + gemm::TM - 1) / gemm::TM), (unsigned)((C + gemm::TN - 1) / gemm::TN), (unsigned)G);
    fq::terms_gemm_kernel<<<grid, gemm::kThreads, gemm::kSmemBytes, st>>>(Gp, Hinv, Z, Rg, C, Cp, 1);
    fq::terms_gemm_kernel<<<grid, gemm::kThreads, gemm::kSmemBytes, st>>>(Z, Hinv, GHinv, Rg, C, Cp, 2);
    fq::hinv_diag_kernel<<<dim3((unsigned)((C + 255) / 256), (unsigned)G), 256, 0, st>>>(Hinv, C, Cp, hdiag);
    fq::beta_kernel<<<R, 256, 0, st>>>(Gp, Z, GHinv, hdiag, R, C, G, alpha_eff, ref_loss, beta);
    return check_launch();
}

static int fq_block_launch(float* Wp, float* GH, const float* Z, const float* Hinv, float* Q, int16_t* codes,
                           float* Eeff, __nv_bfloat16* Ehi, __nv_bfloat16* Elo, const float* scale_row,
                           const float* scale_tab, const int* colgrp, float* scale_blk, int R, int C, int G, int i1,
                           int count, int mode, int dyn_gs, int sym, int maxq, int plus, const float* anchor,
                           const float* beta, int inner_mode, int atomic, void* stream,
                           __nv_bfloat16* Fhi = nullptr, __nv_bfloat16* Flo = nullptr, int far_ld = 0, int far_k0 = 0,
                           int far_after = 0, float so_scale = 1.f) {
    using namespace rq::fq;
    if (!Wp || !Hinv || !Q || !codes || !Eeff || R <= 0 || C <= 0 || G <= 0 || R % G != 0) return RQ_ERR_INVALID;
    if (i1 < 0 || count <= 0 || count > BS || i1 + count > C) return RQ_ERR_INVALID;
    if (plus && (!GH || !Z)) return RQ_ERR_INVALID;
    if (mode == 0 && !scale_row) return RQ_ERR_INVALID;
    if (mode == 1 && (!scale_tab || !colgrp)) return RQ_ERR_INVALID;
    if (mode == 2 && (!scale_blk || dyn_gs <= 0 || BS % dyn_gs != 0 || i1 % dyn_gs != 0)) return RQ_ERR_INVALID;
    if (mode < 0 || mode > 2 || maxq <= 0 || maxq > 32767) return RQ_ERR_INVALID;
    if (inner_mode < 0 || inner_mode > 2 || (inner_mode != 0 && (!plus || !anchor || !beta))) return RQ_ERR_INVALID;
    cudaStream_t st = as_stream(stream);
    BlockArgs p;
    p.anchor = anchor; p.beta = beta; p.inner_mode = inner_mode; p.atomic = atomic ? 1 : 0;
    p.so_scale = so_scale;
    p.Wp = Wp; p.GH = GH; p.Z = Z; p.Hinv = Hinv; p.Q = Q; p.codes = codes; p.Eeff = Eeff;
    p.Ehi = Ehi; p.Elo = Elo;
    p.Fhi = Fhi; p.Flo = Flo; p.far_ld = far_ld; p.far_k0 = far_k0; p.far_after = (float)far_after;
    p.scale_row = scale_row; p.scale_tab = scale_tab; p.colgrp = colgrp; p.scale_blk = scale_blk;
    p.R = R; p.C = C; p.Cp = (C + 127) / 128 * 128; p.G = G; p.i1 = i1; p.count = count;
    p.mode = mode; p.dyn_gs = dyn_gs; p.sym = sym;
    p.qlo = -(float)(maxq + 1); p.qhi = (float)maxq; p.maxq = (float)maxq;
    const int Rg = R / G;
    const int ctas = G * ((Rg + kRowsPerCta - 1) / kRowsPerCta);
    const size_t smem = (size_t)BS * BS * sizeof(float);
    prof::Scope timed(RQ_PROF_BLOCK, st);
    if (plus) {
        if (cudaFuncSetAttribute(block_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return RQ_ERR_CUDA;
        block_kernel<true><<<ctas, kBlockThreads, smem, st>>>(p);
    } else {
        if (cudaFuncSetAttribute(block_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return RQ_ERR_CUDA;
        block_kernel<false><<<ctas, kBlockThreads, smem, st>>>(p);
    }
    return check_launch();
}

extern "C" int rq_fq_block(float* Wp, float* GH, const float* Z, const float* Hinv, float* Q, int16_t* codes,
                           float* Eeff, const float* scale_row, const float* scale_tab, const int* colgrp,
                           float* scale_blk, int R, int C, int G, int i1, int count, int mode, int dyn_gs, int sym,
                           int maxq, int plus, const float* anchor, const float* beta, int inner_mode, int atomic,
                           float second_order_scale, void* stream) {
    return fq_block_launch(Wp, GH, Z, Hinv, Q, codes, Eeff, nullptr, nullptr, scale_row, scale_tab, colgrp, scale_blk, R,
                           C, G, i1, count, mode, dyn_gs, sym, maxq, plus, anchor, beta, inner_mode, atomic, stream,
                           nullptr, nullptr, 0, 0, 0, second_order_scale);
}

static int surrogate_outer(float* Wp, const float* anchor, const float* beta, int R, int C, int i2, int count,
                           cudaStream_t st) {
    dim3 grid((unsigned)((C - i2 + 1023) / 1024), (unsigned)(R < 65535 ? R : 65535));
    fq::surrogate_outer_kernel<<<grid, 256, 0, st>>>(Wp, anchor, beta, R, C, i2, (float)count);
    return check_launch();
}

extern "C" int rq_fq_lazy_update(float* Wp, float* GH, const float* Z, const float* Eeff, const float* Hinv, int R,
                                 int C, int G, int i1, int count, int plus, const float* anchor, const float* beta,
                                 int outer_surrogate, float second_order_scale, void* stream) {
    if (!Wp || !Eeff || !Hinv || R <= 0 || C <= 0 || G <= 0 || R % G != 0 || count <= 0 || count > fq::BS)
        return RQ_ERR_INVALID;
    if (plus && (!GH || !Z)) return RQ_ERR_INVALID;
    const int i2 = i1 + count;
    if (i2 >= C) return RQ_OK;                       // nothing to the right of the last block
    cudaStream_t st = as_stream(stream);
    const int Cp = (C + 127) / 128 * 128;
    const int Rg = R / G;
    dim3 grid((unsigned)((Rg + gemm::TM - 1) / gemm::TM), (unsigned)((C - i2 + gemm::TN - 1) / gemm::TN), (unsigned)G);
    prof::Scope timed(RQ_PROF_LAZY, st);
    if (outer_surrogate) {
        if (!plus || !anchor || !beta) return RQ_ERR_INVALID;
        const int rc0 = surrogate_outer(Wp, anchor, beta, R, C, i2, count, st);
        if (rc0 != RQ_OK) return rc0;
    }
    fq::lazy_kernel<<<grid, gemm::kThreads, gemm::kSmemBytes, st>>>(Wp, GH, Z, Eeff, Hinv, R, C, Cp, G, i1, count, 1, plus,
                                                                    second_order_scale);
    if (plus)
        fq::lazy_kernel<<<grid, gemm::kThreads, gemm::kSmemBytes, st>>>(Wp, GH, Z, Eeff, Hinv, R, C, Cp, G, i1, count, 2, plus,
                                                                        1.f);
    return check_launch();
}

extern "C" int rq_fq_finish(const float* Q, const int16_t* codes, const int64_t* perm, int R, int C, void* out,
                            int out_dtype, float* out_codes, float* out_scale, const float* scale_row,
                            const float* scale_tab, const int* colgrp, int permute_export, void* stream) {
    using namespace rq::fq;
    if (!Q || !out || R <= 0 || C <= 0) return RQ_ERR_INVALID;
    if (out_codes && (!codes || !out_scale || (!scale_row && !(scale_tab && colgrp)))) return RQ_ERR_INVALID;
    dim3 grid((unsigned)((C + 1023) / 1024), (unsigned)(R < 65535 ? R : 65535));
    cudaStream_t st = as_stream(stream);
    if (out_dtype == RQ_F32)
        unpermute_kernel<float><<<grid, 256, 0, st>>>(Q, codes, perm, R, C, reinterpret_cast<float*>(out), out_codes,
                                                      out_scale, scale_row, scale_tab, colgrp, permute_export);
    else if (out_dtype == RQ_BF16)
        unpermute_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(Q, codes, perm, R, C, reinterpret_cast<__nv_bfloat16*>(out),
                                                              out_codes, out_scale, scale_row, scale_tab, colgrp,
                                                              permute_export);
    else if (out_dtype == RQ_F16)
        unpermute_kernel<__half><<<grid, 256, 0, st>>>(Q, codes, perm, R, C, reinterpret_cast<__half*>(out), out_codes,
                                                       out_scale, scale_row, scale_tab, colgrp, permute_export);
    else
        return RQ_ERR_INVALID;
    return check_launch();
}

// Every block of a linear in one call (the callback-free modes need no host work between blocks).
extern "C" int rq_fq_run(float* Wp, float* GH, const float* Z, const float* Hinv, float* Q, int16_t* codes,
                         float* Eeff, const float* scale_row, const float* scale_tab, const int* colgrp,
                         float* scale_blk, int R, int C, int G, int mode, int dyn_gs, int sym, int maxq, int plus,
                         const float* anchor, const float* beta, int inner_mode, int atomic, void* stream) {
    for (int i1 = 0; i1 < C; i1 += fq::BS) {
        const int count = (C - i1 < fq::BS) ? C - i1 : fq::BS;
        const int last = i1 + count >= C;
        int rc = rq_fq_block(Wp, GH, Z, Hinv, Q, codes, Eeff, scale_row, scale_tab, colgrp, scale_blk, R, C, G, i1,
                             count, mode, dyn_gs, sym, maxq, plus, anchor, beta, inner_mode, (atomic && !last) ? 1 : 0,
                             1.f, stream);
        if (rc != RQ_OK) return rc;
        rc = rq_fq_lazy_update(Wp, GH, Z, Eeff, Hinv, R, C, G, i1, count, plus, anchor, beta, inner_mode != 0, 1.f,
                               stream);
        if (rc != RQ_OK) return rc;
    }
    return RQ_OK;
}

// ------------------------------------------------------------------------------------------
// tensor-core variants: the GEMM-shaped parts run on tcgen05 from bf16-split operand planes
// ------------------------------------------------------------------------------------------
namespace {
constexpr int kFarBlocks = 4;        // blocks per group of the two-level lazy update
struct TcLayout {
    size_t put, pu, pa, pe, pf, status, total;
    int Cp;
};

TcLayout tc_layout(int R, int C, int G, int plus) {
    TcLayout L;
    L.Cp = (C + 127) / 128 * 128;
    auto up = [](size_t v) { return (v + 1023) / 1024 * 1024; };
    size_t off = 0;
    L.put = off; off = up(off + (size_t)G * 2 * L.Cp * L.Cp * 2);
    L.pu = off;  if (plus) off = up(off + (size_t)G * 2 * L.Cp * L.Cp * 2);
    L.pa = off;  if (plus) off = up(off + (size_t)2 * R * L.Cp * 2);
    L.pe = off;  off = up(off + (size_t)2 * R * rq::fq::BS * 2);
    L.pf = off;  off = up(off + (size_t)2 * R * rq::fq::BS * kFarBlocks * 2);
    L.status = off; off += 1024;
    L.total = off;
    return L;
}

int split_full_rows(const float* src, int R, int C, int Cp, __nv_bfloat16* dst, cudaStream_t st) {
    rq::tcgemm::SplitArgs a;
    a.src = src; a.ld = C; a.src_z = 0; a.rows = R; a.cols = C;
    a.dst = dst; a.Kp = Cp; a.plane_stride = (long long)R * Cp;
    a.plane = 0; a.plane_z = 0; a.dst_row0 = 0; a.dst_row_z = 0; a.dst_k0 = 0; a.pad_k_to = Cp;
    return rq::tcgemm::split_rows(a, 1, st);
}
}  // namespace

extern "C" size_t rq_fq_tc_workspace_bytes(int R, int C, int G, int plus) {
    if (R <= 0 || C <= 0 || G <= 0) return 0;
    return tc_layout(R, C, G, plus).total + 1024;
}

// Split Hinv into the operand planes used below: U^T (rows = columns of U) always, U itself when plus.
extern "C" int rq_fq_tc_prepare(const float* Hinv, int R, int C, int G, int plus, void* workspace, size_t workspace_bytes,
                                void* stream) {
    if (!Hinv || !workspace || R <= 0 || C <= 0 || G <= 0) return RQ_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(workspace) % 1024 != 0) return RQ_ERR_INVALID;
    const TcLayout L = tc_layout(R, C, G, plus);
    if (workspace_bytes < L.total) return RQ_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    if (cudaMemsetAsync(ws + L.status, 0, sizeof(int), st) != cudaSuccess) return RQ_ERR_CUDA;
    rq::tcgemm::SplitArgs a;
    a.src = Hinv; a.ld = L.Cp; a.src_z = (long long)L.Cp * L.Cp; a.rows = L.Cp; a.cols = L.Cp;
    a.Kp = L.Cp; a.plane_stride = (long long)L.Cp * L.Cp; a.plane = 0; a.plane_z = 2;
    a.dst_row0 = 0; a.dst_row_z = 0; a.dst_k0 = 0; a.pad_k_to = 0;
    a.dst = reinterpret_cast<__nv_bfloat16*>(ws + L.put);
    int rc = rq::tcgemm::split_transpose(a, G, st);
    if (rc != RQ_OK) return rc;
    if (plus) {
        a.dst = reinterpret_cast<__nv_bfloat16*>(ws + L.pu);
        rc = rq::tcgemm::split_rows(a, G, st);
    }
    return rc;
}

extern "C" int rq_gptqplus_terms_tc(const float* Gp, const float* Hinv, int R, int C, int G, float alpha_eff,
                                    float ref_loss, float* Z, float* GHinv, float* beta, float* hdiag, void* workspace,
                                    size_t workspace_bytes, int* status, void* stream) {
    using namespace rq::tcgemm;
    if (!Gp || !Hinv || !Z || !GHinv || !beta || !hdiag || !workspace || R <= 0 || C <= 0 || G <= 0 || R % G != 0)
        return RQ_ERR_INVALID;
    const TcLayout L = tc_layout(R, C, G, 1);
    if (workspace_bytes < L.total) return RQ_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    __nv_bfloat16* PA = reinterpret_cast<__nv_bfloat16*>(ws + L.pa);
    int* tc_status = status ? status : reinterpret_cast<int*>(ws + L.status);
    const int Rg = R / G, Cp = L.Cp;
    prof::Scope timed(RQ_PROF_TERMS, st);
    PlaneTensor tA{PA, Cp, R, 2};
    PlaneTensor tU{ws + L.pu, Cp, Cp, 2LL * G};
    PlaneTensor tUt{ws + L.put, Cp, Cp, 2LL * G};
    Params p;
    p.a_row0 = 0; p.b_row0 = 0; p.a_k0 = 0; p.b_k0 = 0; p.a_plane = 0; p.b_plane = 0;
    p.a_plane_z = 0; p.b_plane_z = 2; p.a_row_z = Rg; p.b_row_z = 0;
    p.M = Rg; p.N = C; p.k_len = Cp; p.tri = 0; p.batch = G;
    p.ldc = C; p.c_z = (long long)Rg * C; p.Aux = nullptr; p.ldaux = 0; p.aux_z = 0;
    p.alpha = 1.f; p.beta = 0.f; p.gamma = 0.f;
    int rc = split_full_rows(Gp, R, C, Cp, PA, st);                 // T = Gp . U^T
    if (rc != RQ_OK) return rc;
    p.kmode = 3; p.C = Z;
    rc = launch(tA, tU, p, tc_status, st);
    if (rc != RQ_OK) return rc;
    rc = split_full_rows(Z, R, C, Cp, PA, st);                      // G.H^-1 = T . U
    if (rc != RQ_OK) return rc;
    p.kmode = 2; p.C = GHinv;
    rc = launch(tA, tUt, p, tc_status, st);
    if (rc != RQ_OK) return rc;
    fq::hinv_diag_kernel<<<dim3((unsigned)((C + 255) / 256), (unsigned)G), 256, 0, st>>>(Hinv, C, Cp, hdiag);
    fq::beta_kernel<<<R, 256, 0, st>>>(Gp, Z, GHinv, hdiag, R, C, G, alpha_eff, ref_loss, beta);
    rc = check_launch();
    if (rc != RQ_OK) return rc;
    return split_full_rows(Z, R, C, Cp, PA, st);                     // planes of Z = beta * T for the lazy updates
}

extern "C" int rq_fq_run_tc(float* Wp, float* GH, const float* Z, const float* Hinv, float* Q, int16_t* codes,
                            float* Eeff, const float* scale_row, const float* scale_tab, const int* colgrp,
                            float* scale_blk, int R, int C, int G, int mode, int dyn_gs, int sym, int maxq, int plus,
                            const float* anchor, const float* beta, int inner_mode, int atomic, void* workspace,
                            size_t workspace_bytes, int* status, void* stream) {
    using namespace rq::tcgemm;
    if (!workspace || R <= 0 || C <= 0 || G <= 0 || R % G != 0) return RQ_ERR_INVALID;
    const TcLayout L = tc_layout(R, C, G, plus);
    if (workspace_bytes < L.total) return RQ_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    __nv_bfloat16* PE = reinterpret_cast<__nv_bfloat16*>(ws + L.pe);
    int* tc_status = status ? status : reinterpret_cast<int*>(ws + L.status);
    const int Rg = R / G, Cp = L.Cp;
    PlaneTensor tE{PE, fq::BS, R, 2};
    PlaneTensor tZ{ws + L.pa, Cp, R, 2};
    PlaneTensor tUt{ws + L.put, Cp, Cp, 2LL * G};
    // Two-level lazy update (frozen mode): blocks are grouped four to a group of 512 columns.  After a block only
    // the rest of its own group is brought up to date (k-extent 128); the columns beyond the group receive one
    // update per group with k-extent 512, a quarter of the read-modify-write traffic.  For those columns the
    // first-order term seen by block b is GH_start - sum_{b' < b} Z_b'.H_b', so the group's total is
    //   W_far -= sum_b (Err_b - (D + after_b) o Z_b) . H_b,far + n_group * GH_far,   GH_far -= sum_b Z_b . H_b,far
    // with after_b the number of group columns behind block b: the block kernel writes that operand directly.
    // The surrogate modes read the trailing weights after every block and keep the one-level schedule.
    const bool two_level = inner_mode == 0;
    const int W = fq::BS * kFarBlocks;
    __nv_bfloat16* PF = reinterpret_cast<__nv_bfloat16*>(ws + L.pf);
    PlaneTensor tF{PF, W, R, 2};
    for (int i1 = 0; i1 < C; i1 += fq::BS) {
        const int count = (C - i1 < fq::BS) ? C - i1 : fq::BS;
        const int i2 = i1 + count;
        const int o0 = i1 / W * W;                                   // current group [o0, o1)
        const int o1 = two_level ? ((o0 + W < C) ? o0 + W : C) : C;
        const bool far = two_level && o1 < C;
        int rc = fq_block_launch(Wp, GH, Z, Hinv, Q, codes, Eeff, PE, PE + (size_t)R * fq::BS, scale_row, scale_tab,
                                 colgrp, scale_blk, R, C, G, i1, count, mode, dyn_gs, sym, maxq, plus, anchor, beta,
                                 inner_mode, (atomic && i2 < C) ? 1 : 0, stream, far ? PF : nullptr,
                                 far ? PF + (size_t)R * W : nullptr, W, i1 - o0, o1 - i2);
        if (rc != RQ_OK) return rc;
        if (i2 >= C) break;
        prof::Scope timed(RQ_PROF_LAZY, st);
        if (inner_mode != 0) {
            rc = surrogate_outer(Wp, anchor, beta, R, C, i2, count, st);
            if (rc != RQ_OK) return rc;
        }
        Params p;
        p.a_row0 = 0; p.a_plane = 0; p.a_plane_z = 0; p.a_row_z = Rg;
        p.b_plane = 0; p.b_plane_z = 2; p.b_row_z = 0;
        p.M = Rg; p.tri = 0; p.kmode = 0; p.batch = G;
        p.ldc = C; p.c_z = (long long)Rg * C; p.ldaux = C; p.aux_z = (long long)Rg * C;
        p.alpha = -1.f; p.beta = 1.f;
        if (i2 < o1) {                                               // rest of the group (or of the matrix)
            p.a_k0 = 0; p.b_row0 = i2; p.b_k0 = i1; p.N = o1 - i2; p.k_len = fq::BS;
            p.C = Wp + i2; p.Aux = plus ? GH + i2 : nullptr; p.gamma = plus ? -(float)count : 0.f;
            rc = launch(tE, tUt, p, tc_status, st);                  // W[:, i2:o1] -= Eeff . Hinv[i1:i2, i2:o1] + count * GH
            if (rc != RQ_OK) return rc;
            if (plus) {
                p.a_k0 = i1; p.C = GH + i2; p.Aux = nullptr; p.gamma = 0.f;
                rc = launch(tZ, tUt, p, tc_status, st);              // GH[:, i2:o1] -= Z[:, i1:i2] . Hinv[i1:i2, i2:o1]
                if (rc != RQ_OK) return rc;
            }
        } else if (far) {                                            // the group is complete: everything beyond it
            p.a_k0 = 0; p.b_row0 = o1; p.b_k0 = o0; p.N = C - o1; p.k_len = o1 - o0;
            p.C = Wp + o1; p.Aux = plus ? GH + o1 : nullptr; p.gamma = plus ? -(float)(o1 - o0) : 0.f;
            rc = launch(tF, tUt, p, tc_status, st);
            if (rc != RQ_OK) return rc;
            if (plus) {
                p.a_k0 = o0; p.C = GH + o1; p.Aux = nullptr; p.gamma = 0.f;
                rc = launch(tZ, tUt, p, tc_status, st);
                if (rc != RQ_OK) return rc;
            }
        }
    }
    return RQ_OK;
}

// ==========================================================================================
// GPTAQ (asymmetric calibration): gptq_utils/gptaq_utils.py.  Besides H it accumulates
//   dXXT = mean-normalised sum over tokens of (x_fp - x) x^T          (:36-39, not symmetric)
// and fasterquant adds, per quantized column i, the term  + w_i (x) P[i, i:]  with
//   P = alpha * triu(dXXT . Hinv^T, 1) . Hinv                         (:105)
// to the error feedback (:140), and  + Q1 . P[i1:i2, i2:]  to the lazy update (:146).
// ==========================================================================================
namespace rq {
namespace aq {

using fq::BS;
using fq::kBlockThreads;
using fq::kRowsPerCta;

// planes of d' = fl(x_fp * s) - fl(x * s) and x' = fl(x * s), transposed: dst[c][t].  grid (ceil(C/32), ceil(Np/64)).
// x: [N, C] (row stride ldx); x_fp: [N, C] (row stride ldf) or, with FT, channel-major [C, N] as the reference's
// input cache stores it (gptaq_utils.py:185-189).
template <typename TX, typename TF, bool FT>
__global__ void __launch_bounds__(256) diff_pack_kernel(const TX* __restrict__ x, int64_t ldx, const TF* __restrict__ xf,
                                                        int64_t ldf, int64_t N, int C, float s,
                                                        __nv_bfloat16* __restrict__ PD, __nv_bfloat16* __restrict__ PX,
                                                        int64_t Kp) {
    __shared__ float td[64][33], tx[64][33];
    const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 32;
    const int64_t t0 = (int64_t)blockIdx.y * 64;
    if (FT) {                                              // stage x_fp with the lanes running along the tokens
#pragma unroll
        for (int cc = ly; cc < 32; cc += 8)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t t = t0 + 32 * h + lx;
                const int c = c0 + cc;
                td[32 * h + lx][cc] = (t < N && c < C) ? load_as_float<TF>(xf, (int64_t)c * ldf + t) : 0.f;
            }
        __syncthreads();
    }
#pragma unroll
    for (int rr = ly; rr < 64; rr += 8) {
        const int64_t t = t0 + rr;
        const int c = c0 + lx;
        float xv = 0.f, dv = 0.f;
        if (t < N && c < C) {
            xv = __fmul_rn(load_as_float<TX>(x, t * ldx + c), s);
            const float fv = FT ? td[rr][lx] : load_as_float<TF>(xf, t * ldf + c);
            dv = __fsub_rn(__fmul_rn(fv, s), xv);
        }
        tx[rr][lx] = xv;
        td[rr][lx] = dv;
    }
    __syncthreads();
    const int64_t plane = (int64_t)C * Kp;
#pragma unroll
    for (int cc = ly; cc < 32; cc += 8) {
        const int c = c0 + cc;
        const int64_t t = t0 + 2 * lx;
        if (c >= C || t >= Kp) continue;
        const int64_t d = (int64_t)c * Kp + t;
        __nv_bfloat16 h0, l0, h1, l1;
        tcgemm::split2(td[2 * lx][cc], h0, l0);
        tcgemm::split2(td[2 * lx + 1][cc], h1, l1);
        *reinterpret_cast<__nv_bfloat162*>(PD + d) = __halves2bfloat162(h0, h1);
        *reinterpret_cast<__nv_bfloat162*>(PD + plane + d) = __halves2bfloat162(l0, l1);
        tcgemm::split2(tx[2 * lx][cc], h0, l0);
        tcgemm::split2(tx[2 * lx + 1][cc], h1, l1);
        *reinterpret_cast<__nv_bfloat162*>(PX + d) = __halves2bfloat162(h0, h1);
        *reinterpret_cast<__nv_bfloat162*>(PX + plane + d) = __halves2bfloat162(l0, l1);
    }
}

// D[i][j] = dXXT[perm[i]][perm[j]], zero where column perm[j] is dead (H[pj][pj] == 0)  (:72, :84)
__global__ void __launch_bounds__(256) gather_dxxt_kernel(const float* __restrict__ dXXT, const float* __restrict__ H,
                                                          const int64_t* __restrict__ perm, int C, float* __restrict__ D) {
    const int i = blockIdx.y;
    const int64_t pi = perm ? perm[i] : i;
    for (int j = blockIdx.x * 256 + threadIdx.x; j < C; j += gridDim.x * 256) {
        const int64_t pj = perm ? perm[j] : j;
        const bool dead = H[pj * C + pj] == 0.f;
        D[(int64_t)i * C + j] = dead ? 0.f : dXXT[pi * C + pj];
    }
}

// T[i][k] = k > i ? alpha * T[i][k] : 0
__global__ void __launch_bounds__(256) triu_scale_kernel(float* __restrict__ T, int C, float alpha) {
    const int i = blockIdx.y;
    for (int k = blockIdx.x * 256 + threadIdx.x; k < C; k += gridDim.x * 256)
        T[(int64_t)i * C + k] = (k > i) ? __fmul_rn(alpha, T[(int64_t)i * C + k]) : 0.f;
}

struct AqArgs {
    float* Wp;               // [R, C] working weights, permuted order
    const float* Hinv;       // [Cp, Cp]
    const float* P;          // [C, C]
    float* Q;                // [R, C]
    __nv_bfloat16 *Ehi, *Elo, *Qhi, *Qlo;   // [R][BS] operand planes of the lazy update
    const float* scale_row; const float* zero_row;      // mode 0: [R]
    const float* scale_tab; const float* zero_tab;      // mode 1: [ngroups, R]
    const int* colgrp;
    int R, C, Cp, i1, count, mode, asym;
    int dyn_gs;              // mode 2: width of the groups ranged from the block-start values (divides BS)
    float maxq;
};

// One warp per weight row; Hinv and P blocks of the current 128 columns in shared memory.
__global__ void __launch_bounds__(kBlockThreads) aq_block_kernel(const AqArgs p) {
    extern __shared__ float smem[];
    float* Hs = smem;                                      // [BS][BS]
    float* Ps = smem + BS * BS;                            // [BS][BS]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* Hb = p.Hinv + (int64_t)p.i1 * p.Cp + p.i1;
    const float* Pb = p.P + (int64_t)p.i1 * p.C + p.i1;
    for (int e = threadIdx.x; e < BS * BS; e += kBlockThreads) {
        const int i = e >> 7, j = e & 127;
        const bool in = i < p.count && j < p.count;
        Hs[e] = in ? Hb[(int64_t)i * p.Cp + j] : 0.f;
        Ps[e] = in ? Pb[(int64_t)i * p.C + j] : 0.f;
    }
    __syncthreads();
    const int r = blockIdx.x * kRowsPerCta + warp;
    if (r >= p.R) return;
    const int64_t base = (int64_t)r * p.C + p.i1;
    float w[4], sc[4], zr[4], qv[4], ev[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int col = lane + 32 * k;
        const bool in = col < p.count;
        w[k] = in ? p.Wp[base + col] : 0.f;
        qv[k] = 0.f; ev[k] = 0.f; sc[k] = 1.f; zr[k] = 0.f;
        if (p.mode == 0) {
            sc[k] = p.scale_row[r];
            if (p.asym) zr[k] = p.zero_row[r];
        } else if (p.mode == 1 && in) {
            const int64_t gi = (int64_t)p.colgrp[p.i1 + col] * p.R + r;
            sc[k] = p.scale_tab[gi];
            if (p.asym) zr[k] = p.zero_tab[gi];
        }
    }
    if (p.mode == 2) {
        // dynamic groups (gptaq_utils.py:126-131): find_params on the working columns of the group as they are when
        // the block starts (the range contains 0; an all-zero group takes (-1, +1) in the asymmetric rule)
        const int ngrp = (p.count + p.dyn_gs - 1) / p.dyn_gs;
        for (int gi = 0; gi < ngrp; ++gi) {
            float lo = 0.f, hi = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int col = lane + 32 * k;
                if (col < p.count && col / p.dyn_gs == gi) { lo = fminf(lo, w[k]); hi = fmaxf(hi, w[k]); }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
                hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
            }
            float s, z = 0.f;
            if (!p.asym) {
                s = __fdiv_rn(fmaxf(fmaxf(fabsf(lo), hi), 1e-5f), p.maxq);
            } else {
                if (lo == 0.f && hi == 0.f) { lo = -1.f; hi = 1.f; }
                s = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-5f), p.maxq);
                z = rintf(__fdiv_rn(-lo, s));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int col = lane + 32 * k;
                if (col / p.dyn_gs == gi) { sc[k] = s; zr[k] = z; }
            }
        }
    }
#pragma unroll
    for (int slot = 0; slot < 4; ++slot) {
        const int ibase = slot * 32;
        if (ibase >= p.count) break;
        const int iend = (p.count - ibase < 32) ? p.count - ibase : 32;
        for (int o = 0; o < iend; ++o) {
            const int i = ibase + o;
            const float wi = __shfl_sync(0xffffffffu, w[slot], o);
            const float si = __shfl_sync(0xffffffffu, sc[slot], o);
            const float zi = __shfl_sync(0xffffffffu, zr[slot], o);
            float q;                                       // WeightQuantizer.quantize: the zero point is honoured
            if (p.asym) {
                float c = __fadd_rn(rintf(__fdiv_rn(wi, si)), zi);
                c = c < 0.f ? 0.f : (c > p.maxq ? p.maxq : c);
                q = __fmul_rn(si, __fsub_rn(c, zi));
            } else {
                q = __fmul_rn(si, quant_code(wi, si, -(p.maxq + 1.f), p.maxq));
            }
            const float err = __fdiv_rn(__fsub_rn(wi, q), Hs[i * BS + i]);
            if (lane == o) { qv[slot] = q; ev[slot] = err; }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (32 * k + 31 < i) continue;             // slot already quantized (warp-uniform)
                const int col = lane + 32 * k;
                if (col >= i && col < p.count) {
                    const float upd = __fsub_rn(__fmul_rn(err, Hs[i * BS + col]), __fmul_rn(wi, Ps[i * BS + col]));
                    w[k] = __fsub_rn(w[k], upd);
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int col = lane + 32 * k;
        const bool in = col < p.count;
        if (in) p.Q[base + col] = qv[k];
        // the lazy update multiplies the block's working weights after the loop (W1, :146); column i of it is
        // w_i - err_i * d_i, the quantized value up to one rounding
        const float e = in ? ev[k] : 0.f, qq = in ? w[k] : 0.f;
        __nv_bfloat16 h, l;
        tcgemm::split2(e, h, l);
        p.Ehi[(int64_t)r * BS + col] = h; p.Elo[(int64_t)r * BS + col] = l;
        tcgemm::split2(qq, h, l);
        p.Qhi[(int64_t)r * BS + col] = h; p.Qlo[(int64_t)r * BS + col] = l;
    }
}

struct Layout {
    size_t put, ppt, pe, pq, tmp1, tmp2, status, total;
    int Cp;
};
static Layout layout(int R, int C) {
    Layout L;
    L.Cp = (C + 127) / 128 * 128;
    auto up = [](size_t v) { return (v + 1023) / 1024 * 1024; };
    size_t off = 0;
    L.put = off; off = up(off + (size_t)2 * L.Cp * L.Cp * 2);          // planes of U^T
    L.ppt = off; off = up(off + (size_t)2 * L.Cp * L.Cp * 2);          // planes of P^T
    L.pe = off; off = up(off + (size_t)2 * R * BS * 2);
    L.pq = off; off = up(off + (size_t)2 * R * BS * 2);
    L.tmp1 = off; off = up(off + (size_t)C * C * 4);                   // gathered dXXT, then T
    L.tmp2 = off; off = up(off + (size_t)C * C * 4);
    L.status = off; off += 1024;
    L.total = off;
    return L;
}

}  // namespace aq
}  // namespace rq

extern "C" size_t rq_gptaq_accum_workspace_bytes(int64_t tokens, int C) {
    if (tokens <= 0 || C <= 0) return 0;
    const int64_t Kp = (tokens + 63) / 64 * 64;
    return (size_t)2 * 2 * C * Kp * 2 + 2048;
}

// dXXT = beta * dXXT + (fl(x_fp * s) - fl(x * s))^T . fl(x * s) over the N tokens  (gptaq_utils.py:33-39)
extern "C" int rq_gptaq_accum(const void* x, int x_dtype, int64_t ldx, const void* x_fp, int fp_dtype, int64_t ldf,
                              int fp_channel_major, int64_t N, int C, float s, float beta, float* dXXT, void* workspace,
                              size_t workspace_bytes, int* status, void* stream) {
    using namespace rq::tcgemm;
    if (!x || !x_fp || !dXXT || !workspace || N <= 0 || C <= 0) return RQ_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(workspace) % 1024 != 0) return RQ_ERR_INVALID;
    if (workspace_bytes < rq_gptaq_accum_workspace_bytes(N, C)) return RQ_ERR_WORKSPACE;
    if ((x_dtype != RQ_F32 && x_dtype != RQ_BF16 && x_dtype != RQ_F16) ||
        (fp_dtype != RQ_F32 && fp_dtype != RQ_BF16 && fp_dtype != RQ_F16)) return RQ_ERR_INVALID;
    cudaStream_t st = as_stream(stream);
    const int64_t Kp = (N + 63) / 64 * 64;
    __nv_bfloat16* PD = reinterpret_cast<__nv_bfloat16*>(workspace);
    __nv_bfloat16* PX = PD + (size_t)2 * C * Kp;
    dim3 grid((unsigned)((C + 31) / 32), (unsigned)(Kp / 64));
#define RQ_AQ_PACK(TX, TF)                                                                                          \
    do {                                                                                                            \
        if (fp_channel_major)                                                                                       \
            rq::aq::diff_pack_kernel<TX, TF, true><<<grid, 256, 0, st>>>(                                           \
                reinterpret_cast<const TX*>(x), ldx, reinterpret_cast<const TF*>(x_fp), ldf, N, C, s, PD, PX, Kp);  \
        else                                                                                                        \
            rq::aq::diff_pack_kernel<TX, TF, false><<<grid, 256, 0, st>>>(                                          \
                reinterpret_cast<const TX*>(x), ldx, reinterpret_cast<const TF*>(x_fp), ldf, N, C, s, PD, PX, Kp);  \
    } while (0)
#define RQ_AQ_PACK_F(TX)                                                                 \
    do {                                                                                 \
        if (fp_dtype == RQ_F32) RQ_AQ_PACK(TX, float);                                   \
        else if (fp_dtype == RQ_BF16) RQ_AQ_PACK(TX, __nv_bfloat16);                     \
        else RQ_AQ_PACK(TX, __half);                                                     \
    } while (0)
    if (x_dtype == RQ_F32) RQ_AQ_PACK_F(float);
    else if (x_dtype == RQ_BF16) RQ_AQ_PACK_F(__nv_bfloat16);
    else RQ_AQ_PACK_F(__half);
#undef RQ_AQ_PACK_F
#undef RQ_AQ_PACK
    int rc = check_launch();
    if (rc != RQ_OK) return rc;
    PlaneTensor tD{PD, Kp, C, 2}, tX{PX, Kp, C, 2};
    Params p;
    p.a_row0 = p.b_row0 = 0; p.a_k0 = p.b_k0 = 0; p.a_plane = p.b_plane = 0; p.a_plane_z = p.b_plane_z = 0;
    p.a_row_z = p.b_row_z = 0;
    p.M = C; p.N = C; p.k_len = (int)Kp; p.tri = 0; p.kmode = 0; p.batch = 1;
    p.C = dXXT; p.ldc = C; p.c_z = 0; p.Aux = nullptr; p.ldaux = 0; p.aux_z = 0;
    p.alpha = 1.f; p.beta = beta; p.gamma = 0.f;
    return launch(tD, tX, p, status, st);
}

extern "C" size_t rq_gptaq_workspace_bytes(int R, int C) {
    if (R <= 0 || C <= 0) return 0;
    return rq::aq::layout(R, C).total + 1024;
}

// P = alpha * triu(D . Hinv^T, 1) . Hinv with D the permuted dXXT, dead columns zeroed (gptaq_utils.py:72, 84, 105).
// H: the un-damped Hessian [C, C] (only its diagonal is read, for the dead-column test).  P: [C, C] output.
extern "C" int rq_gptaq_terms(const float* dXXT, const float* H, const int64_t* perm, const float* Hinv, int C,
                              float alpha, float* P, void* workspace, size_t workspace_bytes, int* status,
                              void* stream) {
    using namespace rq;
    using namespace rq::tcgemm;
    if (!dXXT || !H || !Hinv || !P || !workspace || C <= 0) return RQ_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(workspace) % 1024 != 0) return RQ_ERR_INVALID;
    const aq::Layout L = aq::layout(1, C);
    if (workspace_bytes < L.total) return RQ_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    const int Cp = L.Cp;
    float* D = reinterpret_cast<float*>(ws + L.tmp1);
    float* T = reinterpret_cast<float*>(ws + L.tmp2);
    // both products on the tensor cores from bf16-split planes, as the GPTQ+ first-order terms: the operand planes of
    // D (then T) take the region that later holds the planes of U^T, those of U (then U^T) the region of P^T's -
    // rq_gptaq_run rebuilds both for itself
    __nv_bfloat16* PA = reinterpret_cast<__nv_bfloat16*>(ws + L.put);
    __nv_bfloat16* PU = reinterpret_cast<__nv_bfloat16*>(ws + L.ppt);
    int* tc_status = status ? status : reinterpret_cast<int*>(ws + L.status);
    if (!status && cudaMemsetAsync(ws + L.status, 0, sizeof(int), st) != cudaSuccess) return RQ_ERR_CUDA;
    dim3 eg((unsigned)((C + 1023) / 1024), (unsigned)C);
    aq::gather_dxxt_kernel<<<eg, 256, 0, st>>>(dXXT, H, perm, C, D);
    SplitArgs a;
    a.src = Hinv; a.ld = Cp; a.src_z = 0; a.rows = Cp; a.cols = Cp;
    a.Kp = Cp; a.plane_stride = (long long)Cp * Cp; a.plane = 0; a.plane_z = 0;
    a.dst_row0 = 0; a.dst_row_z = 0; a.dst_k0 = 0; a.pad_k_to = 0;
    a.dst = PU;
    int rc = split_rows(a, 1, st);                                   // planes of U
    if (rc != RQ_OK) return rc;
    PlaneTensor tA{PA, Cp, C, 2};
    PlaneTensor tU{PU, Cp, Cp, 2};
    Params p;
    p.a_row0 = 0; p.b_row0 = 0; p.a_k0 = 0; p.b_k0 = 0; p.a_plane = 0; p.b_plane = 0;
    p.a_plane_z = 0; p.b_plane_z = 2; p.a_row_z = C; p.b_row_z = 0;
    p.M = C; p.N = C; p.k_len = Cp; p.tri = 0; p.batch = 1;
    p.ldc = C; p.c_z = (long long)C * C; p.Aux = nullptr; p.ldaux = 0; p.aux_z = 0;
    p.alpha = 1.f; p.beta = 0.f; p.gamma = 0.f;
    rc = split_full_rows(D, C, C, Cp, PA, st);                       // T = D . U^T
    if (rc != RQ_OK) return rc;
    p.kmode = 3; p.C = T;
    rc = launch(tA, tU, p, tc_status, st);
    if (rc != RQ_OK) return rc;
    aq::triu_scale_kernel<<<eg, 256, 0, st>>>(T, C, alpha);
    a.dst = PU;
    rc = split_transpose(a, 1, st);                                  // planes of U^T over those of U
    if (rc != RQ_OK) return rc;
    rc = split_full_rows(T, C, C, Cp, PA, st);                       // P = alpha * triu(T, 1) . U
    if (rc != RQ_OK) return rc;
    p.kmode = 2; p.C = P;
    rc = launch(tA, tU, p, tc_status, st);
    if (rc != RQ_OK) return rc;
    return check_launch();
}

// The block loop of GPTAQ.fasterquant (gptaq_utils.py:107-146) for every block of the linear.  mode 0: per-row
// scale_row / zero_row [R]; mode 1: static groups scale_tab / zero_tab [ngroups, R] indexed by colgrp [C].
// asym != 0 honours the zero point (WeightQuantizer.quantize).  Wp is consumed; Q receives the quantized weights.
extern "C" int rq_gptaq_run(float* Wp, const float* Hinv, const float* P, float* Q, const float* scale_row,
                            const float* zero_row, const float* scale_tab, const float* zero_tab, const int* colgrp,
                            int R, int C, int mode, int dyn_gs, int asym, int maxq, void* workspace,
                            size_t workspace_bytes, int* status, void* stream) {
    using namespace rq;
    using namespace rq::tcgemm;
    if (!Wp || !Hinv || !P || !Q || !workspace || R <= 0 || C <= 0 || maxq <= 0) return RQ_ERR_INVALID;
    if (mode < 0 || mode > 2) return RQ_ERR_INVALID;
    if (mode == 0 && (!scale_row || (asym && !zero_row))) return RQ_ERR_INVALID;
    if (mode == 1 && (!scale_tab || !colgrp || (asym && !zero_tab))) return RQ_ERR_INVALID;
    if (mode == 2 && (dyn_gs <= 0 || fq::BS % dyn_gs != 0)) return RQ_ERR_INVALID;
    const aq::Layout L = aq::layout(R, C);
    if (workspace_bytes < L.total) return RQ_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    __nv_bfloat16* PUt = reinterpret_cast<__nv_bfloat16*>(ws + L.put);
    __nv_bfloat16* PPt = reinterpret_cast<__nv_bfloat16*>(ws + L.ppt);
    __nv_bfloat16* PE = reinterpret_cast<__nv_bfloat16*>(ws + L.pe);
    __nv_bfloat16* PQ = reinterpret_cast<__nv_bfloat16*>(ws + L.pq);
    int* tc_status = status ? status : reinterpret_cast<int*>(ws + L.status);
    const int Cp = L.Cp;
    {   // operand planes of U^T and P^T (rows = output columns, k = rows of the block)
        SplitArgs a;
        a.src = Hinv; a.ld = Cp; a.src_z = 0; a.rows = Cp; a.cols = Cp;
        a.dst = PUt; a.Kp = Cp; a.plane_stride = (long long)Cp * Cp; a.plane = 0; a.plane_z = 0;
        a.dst_row0 = 0; a.dst_row_z = 0; a.dst_k0 = 0; a.pad_k_to = 0;
        int rc = split_transpose(a, 1, st);
        if (rc != RQ_OK) return rc;
        a.src = P; a.ld = C; a.rows = C; a.cols = C; a.dst = PPt; a.pad_k_to = Cp;
        if (cudaMemsetAsync(PPt, 0, (size_t)2 * Cp * Cp * 2, st) != cudaSuccess) return RQ_ERR_CUDA;
        rc = split_transpose(a, 1, st);
        if (rc != RQ_OK) return rc;
    }
    const size_t smem = (size_t)2 * fq::BS * fq::BS * sizeof(float);
    if (cudaFuncSetAttribute(aq::aq_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return RQ_ERR_CUDA;
    PlaneTensor tE{PE, fq::BS, R, 2}, tQ{PQ, fq::BS, R, 2}, tUt{PUt, Cp, Cp, 2}, tPt{PPt, Cp, Cp, 2};
    for (int i1 = 0; i1 < C; i1 += fq::BS) {
        const int count = (C - i1 < fq::BS) ? C - i1 : fq::BS;
        const int i2 = i1 + count;
        aq::AqArgs p;
        p.Wp = Wp; p.Hinv = Hinv; p.P = P; p.Q = Q;
        p.Ehi = PE; p.Elo = PE + (size_t)R * fq::BS; p.Qhi = PQ; p.Qlo = PQ + (size_t)R * fq::BS;
        p.scale_row = scale_row; p.zero_row = zero_row; p.scale_tab = scale_tab; p.zero_tab = zero_tab;
        p.colgrp = colgrp; p.R = R; p.C = C; p.Cp = Cp; p.i1 = i1; p.count = count; p.mode = mode; p.asym = asym;
        p.dyn_gs = dyn_gs > 0 ? dyn_gs : fq::BS;
        p.maxq = (float)maxq;
        {
            prof::Scope timed(RQ_PROF_BLOCK, st);
            aq::aq_block_kernel<<<(R + fq::kRowsPerCta - 1) / fq::kRowsPerCta, fq::kBlockThreads, smem, st>>>(p);
        }
        int rc = check_launch();
        if (rc != RQ_OK) return rc;
        if (i2 >= C) break;
        prof::Scope timed(RQ_PROF_LAZY, st);
        Params g;
        g.a_row0 = 0; g.a_k0 = 0; g.a_plane = 0; g.a_plane_z = 0; g.a_row_z = 0;
        g.b_row0 = i2; g.b_k0 = i1; g.b_plane = 0; g.b_plane_z = 0; g.b_row_z = 0;
        g.M = R; g.N = C - i2; g.k_len = fq::BS; g.tri = 0; g.kmode = 0; g.batch = 1;
        g.C = Wp + i2; g.ldc = C; g.c_z = 0; g.Aux = nullptr; g.ldaux = 0; g.aux_z = 0;
        g.alpha = -1.f; g.beta = 1.f; g.gamma = 0.f;
        rc = launch(tE, tUt, g, tc_status, st);                     // W[:, i2:] -= Err1 . Hinv[i1:i2, i2:]
        if (rc != RQ_OK) return rc;
        g.alpha = 1.f;
        rc = launch(tQ, tPt, g, tc_status, st);                     // W[:, i2:] += Q1 . P[i1:i2, i2:]
        if (rc != RQ_OK) return rc;
    }
    return RQ_OK;
}
