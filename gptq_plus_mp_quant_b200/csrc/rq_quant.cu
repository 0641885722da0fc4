// Weight-quantizer kernels: per-row / per-group range search (optionally with the shrink-grid
// error search) and round/clamp quantize-dequantize.  All HBM-bound except the grid search.
#include "rq_common.cuh"

namespace rq {
namespace quant {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// scale / zero from a range that already contains 0.
__device__ __forceinline__ void range_to_params(float lo, float hi, int maxq, int sym, float& scale, float& zero) {
    if (sym) {
        scale = __fdiv_rn(fmaxf(fmaxf(fabsf(lo), hi), 1e-5f), (float)maxq);
        zero = 0.f;
    } else {
        if (lo == 0.f && hi == 0.f) { lo = -1.f; hi = 1.f; }
        scale = __fdiv_rn(fmaxf(hi - lo, 1e-5f), (float)maxq);
        zero = rintf(__fdiv_rn(-lo, scale));
    }
}

// block-wide min/max of (lo, hi); result valid in every thread
__device__ __forceinline__ void block_minmax(float& lo, float& hi, float* red) {
    lo = warp_min(lo);
    hi = warp_max(hi);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { red[warp] = lo; red[8 + warp] = hi; }
    __syncthreads();
    lo = red[0];
    hi = red[8];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) { lo = fminf(lo, red[w]); hi = fmaxf(hi, red[8 + w]); }
}

__device__ __forceinline__ double block_sum(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double s = 0.0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) s += red[w];
    return s;
}

// One block per (row, group).  groups == 1 covers the per-channel case.  With mse the block
// re-reads its span once per lattice point (it stays in L1/L2).
__global__ void __launch_bounds__(kThreads) find_params_kernel(const float* __restrict__ W, int64_t R, int64_t C,
                                                               int64_t ldw, int groupsize, int maxq, int sym, int mse,
                                                               float norm, int grid, float maxshrink,
                                                               float* __restrict__ scale, float* __restrict__ zero) {
    __shared__ float red[16];
    __shared__ double dred[8];
    const int64_t r = blockIdx.x;
    const int g = blockIdx.y;
    const int64_t c0 = groupsize > 0 ? (int64_t)g * groupsize : 0;
    const int64_t c1 = groupsize > 0 ? (c0 + groupsize < C ? c0 + groupsize : C) : C;
    const float* row = W + r * ldw;
    float lo = 0.f, hi = 0.f;                                // the range always contains 0
    for (int64_t c = c0 + threadIdx.x; c < c1; c += kThreads) {
        const float v = row[c];
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    block_minmax(lo, hi, red);
    float s, z;
    range_to_params(lo, hi, maxq, sym, s, z);
    if (!sym && lo == 0.f && hi == 0.f) { lo = -1.f; hi = 1.f; }
    if (mse) {
        float best = __int_as_float(0x7f800000);
        const int steps = (int)(maxshrink * (float)grid);
        const float fmaxq = (float)maxq;
        for (int i = 0; i < steps; ++i) {
            for (int j = 0; j < steps; ++j) {
                // (1 - i/grid) is evaluated in double like the reference's Python scalar, then rounded to fp32
                const float lo1 = (float)(1.0 - (double)i / (double)grid) * lo;
                const float hi1 = (float)(1.0 - (double)j / (double)grid) * hi;
                float s1, z1;
                if (sym) {
                    s1 = __fdiv_rn(fmaxf(fmaxf(fabsf(lo1), hi1), 1e-5f), fmaxq);
                    z1 = 0.f;
                } else {
                    s1 = __fdiv_rn(hi1 - lo1, fmaxq);
                    z1 = rintf(__fdiv_rn(-lo1, s1));
                }
                double acc = 0.0;
                for (int64_t c = c0 + threadIdx.x; c < c1; c += kThreads) {
                    const float v = row[c];
                    float q;
                    if (sym) {
                        q = rintf(__fdiv_rn(v, s1));
                        q = q < -(fmaxq + 1.f) ? -(fmaxq + 1.f) : (q > fmaxq ? fmaxq : q);
                        q = s1 * q;
                    } else {
                        q = rintf(__fdiv_rn(v, s1)) + z1;
                        q = q < 0.f ? 0.f : (q > fmaxq ? fmaxq : q);
                        q = s1 * (q - z1);
                    }
                    acc += (double)powf(fabsf(q - v), norm);
                }
                const float err = (float)block_sum(acc, dred);
                if (err < best) { best = err; s = s1; z = z1; }
            }
        }
    }
    if (threadIdx.x == 0) {
        scale[(int64_t)g * R + r] = s;
        zero[(int64_t)g * R + r] = z;
    }
}


// Shrink-grid search with the unit (a row, or one column group of a row) held in registers: TPU threads per unit
// (a warp for spans up to 1024 columns, the whole block beyond), EPT values per thread.  The 625 candidates then cost
// arithmetic only - no reloads, and for a warp-sized unit no block barrier per candidate.  Same arithmetic, candidate
// order and strictly-smaller rule as find_params_kernel.
// |d|^norm.  The default norm 2.4 is evaluated as d^2 * 2^(0.4 * log2 d): the squaring is exact to one rounding and the
// transcendental part carries a sixth of the exponent, which keeps the result within a few ulp (the accuracy class of
// powf itself) at about a third of its instructions.  Equal inputs still give equal outputs, so candidates that
// quantize identically still tie exactly, as the first-strictly-smaller rule needs.
template <bool FAST24>
__device__ __forceinline__ float abs_pow(float d, float norm) {
    if (FAST24) return (d * d) * exp2f(0.4f * log2f(d));
    return powf(d, norm);
}

template <int TPU, int EPT, bool FAST24>
__global__ void __launch_bounds__(kThreads) mse_search_kernel(const float* __restrict__ W, int64_t R, int64_t C,
                                                              int64_t ldw, int groupsize, int64_t groups, int maxq,
                                                              int sym, float norm, int grid, float maxshrink,
                                                              float* __restrict__ scale, float* __restrict__ zero) {
    __shared__ float red[16];
    __shared__ double dred[8];
    constexpr int UPB = kThreads / TPU;
    const int sub = threadIdx.x / TPU, t = threadIdx.x % TPU;
    const int64_t u = (int64_t)blockIdx.x * UPB + sub;
    const bool live = u < R * groups;                       // a dead unit idles through the same shuffles
    const int64_t r = live ? u / groups : 0;
    const int g = live ? (int)(u - r * groups) : 0;
    const int64_t c0 = groupsize > 0 ? (int64_t)g * groupsize : 0;
    const int64_t c1 = groupsize > 0 ? (c0 + groupsize < C ? c0 + groupsize : C) : C;
    const int len = (int)(c1 - c0);
    const float* row = W + r * ldw + c0;
    float v[EPT];
    float lo = 0.f, hi = 0.f;                               // the range always contains 0
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int c = t + j * TPU;
        v[j] = (live && c < len) ? row[c] : 0.f;            // padding zeros quantize to 0: no error contribution
        lo = fminf(lo, v[j]);
        hi = fmaxf(hi, v[j]);
    }
    if (TPU == kThreads) {
        block_minmax(lo, hi, red);
    } else {
        lo = warp_min(lo);
        hi = warp_max(hi);
    }
    float s, z;
    range_to_params(lo, hi, maxq, sym, s, z);
    if (!sym && lo == 0.f && hi == 0.f) { lo = -1.f; hi = 1.f; }
    float best = __int_as_float(0x7f800000);
    const int steps = (int)(maxshrink * (float)grid);
    const float fmaxq = (float)maxq;
    // Symmetric rule: the candidate's scale is max(|lo1|, hi1) / maxq, so the 25 x 25 lattice holds at most 25 + 25
    // different scales.  A candidate whose scale was evaluated before has the same error sum and can never be strictly
    // smaller than the best so far: skipping it leaves the result unchanged.  seen_hi marks the j whose hi1 was the
    // maximum once; within one i, |lo1| is the maximum for every j after the first such j.
    unsigned seen_hi = 0u;
    for (int i = 0; i < steps; ++i) {
        const float lo1 = (float)(1.0 - (double)i / (double)grid) * lo;
        bool lo_done = false;
        for (int j = 0; j < steps; ++j) {
            const float hi1 = (float)(1.0 - (double)j / (double)grid) * hi;
            float s1, z1;
            if (sym) {
                if (fabsf(lo1) >= hi1) {
                    if (lo_done) continue;
                    lo_done = true;
                } else if (j < 32) {
                    if ((seen_hi >> j) & 1u) continue;
                    seen_hi |= 1u << j;
                }
                s1 = __fdiv_rn(fmaxf(fmaxf(fabsf(lo1), hi1), 1e-5f), fmaxq);
                z1 = 0.f;
            } else {
                s1 = __fdiv_rn(hi1 - lo1, fmaxq);
                z1 = rintf(__fdiv_rn(-lo1, s1));
            }
            double acc = 0.0;
#pragma unroll
            for (int e = 0; e < EPT; ++e) {
                if (t + e * TPU < len) {
                    const float x = v[e];
                    float q;
                    if (sym) {
                        q = rintf(__fdiv_rn(x, s1));
                        q = q < -(fmaxq + 1.f) ? -(fmaxq + 1.f) : (q > fmaxq ? fmaxq : q);
                        q = s1 * q;
                    } else {
                        q = rintf(__fdiv_rn(x, s1)) + z1;
                        q = q < 0.f ? 0.f : (q > fmaxq ? fmaxq : q);
                        q = s1 * (q - z1);
                    }
                    acc += (double)abs_pow<FAST24>(fabsf(q - x), norm);
                }
            }
            float err;
            if (TPU == kThreads) {
                err = (float)block_sum(acc, dred);
            } else {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                err = (float)acc;
            }
            if (err < best) { best = err; s = s1; z = z1; }
        }
    }
    if (live && t == 0) {
        scale[(int64_t)g * R + r] = s;
        zero[(int64_t)g * R + r] = z;
    }
}

// whole-tensor range (perchannel == 0): single block, result replicated to all R entries
__global__ void __launch_bounds__(kThreads) find_params_tensor_kernel(const float* __restrict__ W, int64_t R, int64_t C,
                                                                      int64_t ldw, int maxq, int sym,
                                                                      float* __restrict__ scale,
                                                                      float* __restrict__ zero) {
    __shared__ float red[16];
    float lo = 0.f, hi = 0.f;
    for (int64_t e = threadIdx.x; e < R * C; e += kThreads) {
        const float v = W[(e / C) * ldw + (e % C)];
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    block_minmax(lo, hi, red);
    float s, z;
    range_to_params(lo, hi, maxq, sym, s, z);
    for (int64_t r = threadIdx.x; r < R; r += kThreads) { scale[r] = s; zero[r] = z; }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_kernel(const T* __restrict__ x, T* __restrict__ deq,
                                                            float* __restrict__ codes, int64_t R, int64_t C,
                                                            const float* __restrict__ scale,
                                                            const float* __restrict__ zero, int pertensor, int maxq,
                                                            int honour_zero) {
    const int64_t total = R * C;
    const float fmaxq = (float)maxq;
    for (int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x; e < total; e += (int64_t)gridDim.x * kThreads) {
        const int64_t r = pertensor ? 0 : e / C;
        const float s = scale[r];
        const float v = load_as_float<T>(x, e);
        float q = rintf(__fdiv_rn(v, s));
        float d;
        if (honour_zero) {
            const float z = zero[r];
            q = q + z;
            q = q < 0.f ? 0.f : (q > fmaxq ? fmaxq : q);
            d = s * (q - z);
        } else {
            q = q < -(fmaxq + 1.f) ? -(fmaxq + 1.f) : (q > fmaxq ? fmaxq : q);
            d = s * q;
        }
        if (deq) store_from_float<T>(deq, e, d);
        if (codes) codes[e] = q;
    }
}

}  // namespace quant
}  // namespace rq

using namespace rq;

extern "C" int rq_find_params(const float* W, int64_t R, int64_t C, int64_t ldw, int groupsize, int perchannel,
                              int maxq, int sym, int mse, float norm, int grid, float maxshrink, float* scale,
                              float* zero, void* stream) {
    using namespace rq::quant;
    if (!W || !scale || !zero || R <= 0 || C <= 0 || ldw < C || maxq <= 0) return RQ_ERR_INVALID;
    cudaStream_t st = as_stream(stream);
    if (!perchannel) {
        if (groupsize > 0 || mse) return RQ_ERR_UNSUPPORTED;
        find_params_tensor_kernel<<<1, kThreads, 0, st>>>(W, R, C, ldw, maxq, sym, scale, zero);
        return check_launch();
    }
    const int64_t groups = groupsize > 0 ? (C + groupsize - 1) / groupsize : 1;
    if (R > 2147483647LL || groups > 65535) return RQ_ERR_INVALID;
    {   // the register-resident kernel also serves the plain range search (no lattice steps): a warp per short unit
        if (!mse) maxshrink = 0.f;
        const int64_t span = groupsize > 0 ? (groupsize < C ? groupsize : C) : C;
        const int64_t units = R * groups;
#define RQ_MSE_LAUNCH(TPU, EPT)                                                                                     \
    if (norm == 2.4f)                                                                                               \
        mse_search_kernel<TPU, EPT, true><<<(unsigned)((units + kThreads / TPU - 1) / (kThreads / TPU)), kThreads,  \
                                            0, st>>>(W, R, C, ldw, groupsize, groups, maxq, sym, norm, grid,        \
                                                     maxshrink, scale, zero);                                       \
    else                                                                                                            \
        mse_search_kernel<TPU, EPT, false><<<(unsigned)((units + kThreads / TPU - 1) / (kThreads / TPU)), kThreads, \
                                             0, st>>>(W, R, C, ldw, groupsize, groups, maxq, sym, norm, grid,       \
                                                      maxshrink, scale, zero)
        if (units <= 2147483647LL) {
            if (span <= 128) { RQ_MSE_LAUNCH(32, 4); return check_launch(); }
            if (span <= 256) { RQ_MSE_LAUNCH(32, 8); return check_launch(); }
            if (span <= 1024) { RQ_MSE_LAUNCH(32, 32); return check_launch(); }
            if (span <= 4096) { RQ_MSE_LAUNCH(256, 16); return check_launch(); }
            if (span <= 8192) { RQ_MSE_LAUNCH(256, 32); return check_launch(); }
            if (span <= 16384) { RQ_MSE_LAUNCH(256, 64); return check_launch(); }
        }
#undef RQ_MSE_LAUNCH
    }
    dim3 gridDim3((unsigned)R, (unsigned)groups);
    find_params_kernel<<<gridDim3, kThreads, 0, st>>>(W, R, C, ldw, groupsize, maxq, sym, mse, norm, grid, maxshrink,
                                                      scale, zero);
    return check_launch();
}

extern "C" int rq_quantize(const void* x, void* deq, float* codes, int dtype, int64_t R, int64_t C, const float* scale,
                           const float* zero, int pertensor, int maxq, int honour_zero, void* stream) {
    using namespace rq::quant;
    if (!x || !scale || (!deq && !codes) || R < 0 || C < 0 || (honour_zero && !zero)) return RQ_ERR_INVALID;
    if (R * C == 0) return RQ_OK;
    int64_t blocks = (R * C + kThreads - 1) / kThreads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t st = as_stream(stream);
    if (dtype == RQ_F32)
        quantize_kernel<float><<<(unsigned)blocks, kThreads, 0, st>>>(reinterpret_cast<const float*>(x),
                                                                      reinterpret_cast<float*>(deq), codes, R, C, scale,
                                                                      zero, pertensor, maxq, honour_zero);
    else if (dtype == RQ_BF16)
        quantize_kernel<__nv_bfloat16><<<(unsigned)blocks, kThreads, 0, st>>>(
            reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(deq), codes, R, C, scale, zero,
            pertensor, maxq, honour_zero);
    else if (dtype == RQ_F16)
        quantize_kernel<__half><<<(unsigned)blocks, kThreads, 0, st>>>(reinterpret_cast<const __half*>(x),
                                                                       reinterpret_cast<__half*>(deq), codes, R, C,
                                                                       scale, zero, pertensor, maxq, honour_zero);
    else
        return RQ_ERR_INVALID;
    return check_launch();
}


// ------------------------------------------------------------------------------------------
// Pre-clip of a weight matrix to the range its quantizer can represent
// (gptq_utils/gptq_plus_utils.py:197-225): per row r, with s = max(scale[r], 1e-8),
//   symmetric:  [s * -(maxq+1), s * maxq];   asymmetric:  [s * (-zero[r]), s * (maxq - zero[r])],
// w = min(max(w, lo), hi) evaluated in fp32, stored in the matrix's own dtype.
// ------------------------------------------------------------------------------------------
namespace rq {
namespace quant {
template <typename T>
__global__ void __launch_bounds__(kThreads) clip_bounds_kernel(T* __restrict__ w, int64_t R, int64_t C, int64_t ldw,
                                                              const float* __restrict__ scale,
                                                              const float* __restrict__ zero, float maxq, int sym) {
    for (int64_t r = blockIdx.y; r < R; r += gridDim.y) {
        const float s = fmaxf(scale[r], 1e-8f);
        float lo, hi;
        if (sym) {
            lo = __fmul_rn(s, -(maxq + 1.f));
            hi = __fmul_rn(s, maxq);
        } else {
            const float z = zero[r];
            lo = __fmul_rn(s, -z);
            hi = __fmul_rn(s, __fsub_rn(maxq, z));
        }
        for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < C; c += (int64_t)gridDim.x * kThreads) {
            const float v = load_as_float<T>(w, r * ldw + c);
            if (v == v) store_from_float<T>(w, r * ldw + c, fminf(fmaxf(v, lo), hi));   // NaN stays, as torch.maximum keeps it
        }
    }
}
}  // namespace quant
}  // namespace rq

extern "C" int rq_clip_to_quant_bounds(void* W, int dtype, int64_t R, int64_t C, int64_t ldw, const float* scale,
                                       const float* zero, int maxq, int sym, void* stream) {
    using namespace rq::quant;
    if (!W || !scale || (!sym && !zero) || R < 0 || C < 0 || ldw < C || maxq <= 0) return RQ_ERR_INVALID;
    if (R * C == 0) return RQ_OK;
    dim3 grid((unsigned)((C + kThreads - 1) / kThreads > 64 ? 64 : (C + kThreads - 1) / kThreads),
              (unsigned)(R < 32768 ? R : 32768));
    cudaStream_t st = as_stream(stream);
    if (dtype == RQ_F32)
        clip_bounds_kernel<float><<<grid, kThreads, 0, st>>>(reinterpret_cast<float*>(W), R, C, ldw, scale, zero, (float)maxq, sym);
    else if (dtype == RQ_BF16)
        clip_bounds_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(W), R, C, ldw, scale,
                                                                      zero, (float)maxq, sym);
    else if (dtype == RQ_F16)
        clip_bounds_kernel<__half><<<grid, kThreads, 0, st>>>(reinterpret_cast<__half*>(W), R, C, ldw, scale, zero,
                                                               (float)maxq, sym);
    else
        return RQ_ERR_INVALID;
    return check_launch();
}

// ------------------------------------------------------------------------------------------
// Packed export of integer codes: the fp32 code matrix that fasterquant registers as `int_weight`
// (gptq_utils/gptq_plus_utils.py:1866-1871 keeps it as fp32 [R, C]) as a little-endian bit stream per row,
// `bits` bits per code in two's complement: 8 consecutive codes fill `bits` bytes.  One thread per 8 codes.
// ------------------------------------------------------------------------------------------
namespace rq {
namespace quant {
__global__ void __launch_bounds__(kThreads) pack_codes_kernel(const float* __restrict__ codes, int64_t R, int64_t C,
                                                             int64_t ldc, int bits, uint8_t* __restrict__ out,
                                                             int64_t row_bytes) {
    const int64_t groups = (C + 7) / 8;
    const uint64_t mask = (1ull << bits) - 1ull;
    for (int64_t u = (int64_t)blockIdx.x * kThreads + threadIdx.x; u < R * groups; u += (int64_t)gridDim.x * kThreads) {
        const int64_t r = u / groups, gidx = u - r * groups;
        uint64_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t c = gidx * 8 + i;
            const long long v = c < C ? (long long)codes[r * ldc + c] : 0;
            word |= ((uint64_t)v & mask) << (i * bits);
        }
        uint8_t* dst = out + r * row_bytes + gidx * bits;
        for (int b = 0; b < bits; ++b)
            if (gidx * bits + b < row_bytes) dst[b] = (uint8_t)(word >> (8 * b));
    }
}
}  // namespace quant
}  // namespace rq

extern "C" int64_t rq_packed_row_bytes(int64_t C, int bits) {
    if (C <= 0 || bits < 2 || bits > 8) return 0;
    return (C + 7) / 8 * bits;
}

extern "C" int rq_pack_codes(const float* codes, int64_t R, int64_t C, int64_t ldc, int bits, uint8_t* out,
                             void* stream) {
    using namespace rq::quant;
    if (!codes || !out || R < 0 || C <= 0 || ldc < C || bits < 2 || bits > 8) return RQ_ERR_INVALID;
    if (R == 0) return RQ_OK;
    const int64_t groups = (C + 7) / 8;
    int64_t blocks = (R * groups + kThreads - 1) / kThreads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    pack_codes_kernel<<<(unsigned)blocks, kThreads, 0, rq::as_stream(stream)>>>(codes, R, C, ldc, bits, out,
                                                                               rq_packed_row_bytes(C, bits));
    return rq::check_launch();
}
