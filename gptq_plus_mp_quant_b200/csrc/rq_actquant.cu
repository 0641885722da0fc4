// Dynamic per-token (or per-token-group) fake quantization of activations: ActQuantizer.find_params followed by
// STEQuantize / AsymSTEQuantize.forward (utils/quant_utils.py:60-84, 133-206) in one pass over the tensor.
// The reference's group-wise path evaluates every step in the tensor's own dtype (bf16 / fp16 inputs: each torch op
// computes in fp32 and rounds its result to the dtype); its per-token path mixes in an fp32 zero vector when it
// forms the range (:180-182), which promotes everything after it to fp32 with one cast at the end.  Both are
// followed here (dtype_math selects which), so the result is the reference's bit for bit.  T(.) below is that
// rounding (the identity with fp32 math):
//   range     per-token rows include 0 in the range, group-wise ranges do not (amax / amin of the group)
//             xmin = T(min * clip), xmax = T(max * clip)
//   symmetric xmax = max(|xmin|, xmax); scale = T(xmax / maxq) (1 where xmax == 0); q = clamp(rint(T(x / scale)),
//             -(maxq+1), maxq); out = T(scale * q)
//             (weight_rule, WeightQuantizer's group-wise ranges :333-352: scale = T(T(max(xmax, 1e-5)) / maxq), and
//             T(max(T(xmax - xmin), 1e-5)) in the asymmetric span)
//   otherwise (xmin, xmax) = (-1, +1) where both are 0; scale = T(T(xmax - xmin) / maxq); zero = rint(T(-xmin / scale));
//             q = clamp(T(rint(T(x / scale)) + zero), 0, maxq); out = T(scale * T(q - zero))
// HBM-bound: the unit is read from DRAM once (the second read hits L1 / L2) and written once.
#include "rq_common.cuh"

namespace rq {
namespace actq {

template <typename T>
__device__ __forceinline__ float rnd(float v);
template <>
__device__ __forceinline__ float rnd<float>(float v) { return v; }
template <>
__device__ __forceinline__ float rnd<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ float rnd<__half>(float v) { return __half2float(__float2half_rn(v)); }

// 16-byte vectors: 4 floats or 8 half-precision values
template <typename T>
struct Vec {
    static constexpr int N = 16 / sizeof(T);
    uint4 raw;
    __device__ __forceinline__ float get(int i) const { return load_as_float<T>(reinterpret_cast<const T*>(&raw), i); }
    __device__ __forceinline__ void set(int i, float v) { store_from_float<T>(reinterpret_cast<T*>(&raw), i, v); }
};

// TPU threads cooperate on one unit (a token row or one group of a token); blockDim.x = 256.
template <typename T, int TPU>
__global__ void __launch_bounds__(256) act_quant_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t units,
                                                        int len, int with_zero, float clip, float maxq, int sym,
                                                        float* __restrict__ scale_out, float* __restrict__ zero_out,
                                                        const float* __restrict__ scale_in,
                                                        const float* __restrict__ zero_in, int codes, int dtype_math,
                                                        int vec_ok, int weight_rule) {
    constexpr int UPB = 256 / TPU;                       // units per block
    constexpr int VN = Vec<T>::N;
    auto R = [dtype_math](float v) { return dtype_math ? rnd<T>(v) : v; };
    __shared__ float red_lo[8], red_hi[8];
    const int sub = threadIdx.x / TPU, t = threadIdx.x % TPU;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t u0 = (int64_t)blockIdx.x * UPB; u0 < units; u0 += (int64_t)gridDim.x * UPB) {
        const int64_t u = u0 + sub;
        const bool live = u < units;
        const T* xr = x + (live ? u : 0) * (int64_t)len;
        float scale, zero = 0.f;
        if (scale_in != nullptr) {
            scale = live ? scale_in[u] : 1.f;
            zero = (live && zero_in != nullptr) ? zero_in[u] : 0.f;
        } else {
            float lo = with_zero ? 0.f : INFINITY, hi = with_zero ? 0.f : -INFINITY;
            if (live && vec_ok) {
                for (int c = t * VN; c < len; c += TPU * VN) {
                    Vec<T> v;
                    v.raw = *reinterpret_cast<const uint4*>(xr + c);
#pragma unroll
                    for (int i = 0; i < VN; ++i) {
                        lo = fminf(lo, v.get(i));
                        hi = fmaxf(hi, v.get(i));
                    }
                }
            } else if (live) {
                for (int c = t; c < len; c += TPU) {
                    const float v = load_as_float<T>(xr, c);
                    lo = fminf(lo, v);
                    hi = fmaxf(hi, v);
                }
            }
#pragma unroll
            for (int o = (TPU < 32 ? TPU : 32) / 2; o > 0; o >>= 1) {
                lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
                hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
            }
            if (TPU > 32) {                              // one unit per block: combine the 8 warps
                __syncthreads();
                if (lane == 0) { red_lo[warp] = lo; red_hi[warp] = hi; }
                __syncthreads();
                lo = red_lo[0]; hi = red_hi[0];
#pragma unroll
                for (int w = 1; w < 8; ++w) { lo = fminf(lo, red_lo[w]); hi = fmaxf(hi, red_hi[w]); }
            }
            float xmin = R(lo * clip), xmax = R(hi * clip);
            if (sym) {
                xmax = fmaxf(fabsf(xmin), xmax);
                if (weight_rule) scale = R(__fdiv_rn(R(fmaxf(xmax, 1e-5f)), maxq));      // .clamp(min=1e-5) / maxq
                else scale = (xmax == 0.f) ? 1.f : R(__fdiv_rn(xmax, maxq));
            } else {
                if (xmin == 0.f && xmax == 0.f) { xmin = -1.f; xmax = 1.f; }
                const float span = R(xmax - xmin);
                scale = R(__fdiv_rn(weight_rule ? R(fmaxf(span, 1e-5f)) : span, maxq));
                zero = rintf(R(__fdiv_rn(-xmin, scale)));
            }
            if (live && t == 0) {
                if (scale_out) scale_out[u] = scale;
                if (zero_out) zero_out[u] = zero;
            }
        }
        if (live && out != nullptr) {
            T* orow = out + u * (int64_t)len;
            auto one = [&](float v) -> float {
                float q = rintf(R(__fdiv_rn(v, scale)));
                float r;
                if (sym) {
                    q = fminf(fmaxf(q, -(maxq + 1.f)), maxq);
                    r = codes ? q : R(scale * q);
                } else {
                    q = fminf(fmaxf(R(q + zero), 0.f), maxq);
                    r = codes ? q : R(scale * R(q - zero));
                }
                return (v != v) ? v : r;                 // NaN propagates as in the reference
            };
            if (vec_ok) {
                for (int c = t * VN; c < len; c += TPU * VN) {
                    Vec<T> v, w;
                    v.raw = *reinterpret_cast<const uint4*>(xr + c);
#pragma unroll
                    for (int i = 0; i < VN; ++i) w.set(i, one(v.get(i)));
                    *reinterpret_cast<uint4*>(orow + c) = w.raw;
                }
            } else {
                for (int c = t; c < len; c += TPU) store_from_float<T>(orow, c, one(load_as_float<T>(xr, c)));
            }
        }
    }
}


// Shrink-lattice search over grouped weight ranges (WeightQuantizer.find_params_weight_groupwise with mse,
// utils/quant_utils.py:355-385): for every group the 25 x 25 candidates (1 - i/grid) * xmin, (1 - j/grid) * xmax,
// error sum |q - x|^norm over the group, the first strictly smaller sum wins.  Every step is rounded to the weight's
// dtype as the reference's chain of torch ops rounds it (T(.)); the sum is accumulated wide and rounded once, as
// torch.sum does for half-precision inputs.  One warp per group; the group is re-read from L1 per candidate.
template <typename T>
__global__ void __launch_bounds__(256) group_mse_kernel(const T* __restrict__ x, int64_t units, int len, float maxq,
                                                        int sym, float norm, int grid, int steps,
                                                        float* __restrict__ scale_out, float* __restrict__ zero_out) {
    const int lane = threadIdx.x & 31;
    const int64_t u = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (u >= units) return;                                   // whole warps leave together
    const T* xr = x + u * (int64_t)len;
    float lo = INFINITY, hi = -INFINITY;
    for (int c = lane; c < len; c += 32) {
        const float v = load_as_float<T>(xr, c);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    float scale, zero = 0.f;
    if (sym) {
        scale = rnd<T>(__fdiv_rn(rnd<T>(fmaxf(fmaxf(fabsf(lo), hi), 1e-5f)), maxq));
    } else {
        if (lo == 0.f && hi == 0.f) { lo = -1.f; hi = 1.f; }
        scale = rnd<T>(__fdiv_rn(rnd<T>(fmaxf(rnd<T>(hi - lo), 1e-5f)), maxq));
        zero = rnd<T>(rintf(rnd<T>(__fdiv_rn(-lo, scale))));
    }
    float best = INFINITY;
    const float expo = rnd<T>(norm);                          // torch casts a scalar exponent to the tensor's dtype
    // symmetric rule: the scale is a function of max(|lo1|, hi1) alone, so a candidate whose maximum was evaluated
    // before repeats that error sum and cannot be strictly smaller than the best so far: skipped, same result
    unsigned seen_hi = 0u;
    for (int i = 0; i < steps; ++i) {
        const float lo1 = rnd<T>((float)(1.0 - (double)i / (double)grid) * lo);
        bool lo_done = false;
        for (int j = 0; j < steps; ++j) {
            const float hi1 = rnd<T>((float)(1.0 - (double)j / (double)grid) * hi);
            float s1, z1 = 0.f;
            if (sym) {
                if (fabsf(lo1) >= hi1) {
                    if (lo_done) continue;
                    lo_done = true;
                } else if (j < 32) {
                    if ((seen_hi >> j) & 1u) continue;
                    seen_hi |= 1u << j;
                }
                s1 = rnd<T>(__fdiv_rn(rnd<T>(fmaxf(fmaxf(fabsf(lo1), hi1), 1e-5f)), maxq));
            } else {
                s1 = rnd<T>(__fdiv_rn(rnd<T>(hi1 - lo1), maxq));
                z1 = rnd<T>(rintf(rnd<T>(__fdiv_rn(-lo1, s1))));
            }
            double acc = 0.0;
            for (int c = lane; c < len; c += 32) {
                const float v = load_as_float<T>(xr, c);
                float q = rnd<T>(rintf(rnd<T>(__fdiv_rn(v, s1))));
                if (sym) {
                    q = fminf(fmaxf(q, -(maxq + 1.f)), maxq);
                    q = rnd<T>(s1 * q);
                } else {
                    q = fminf(fmaxf(rnd<T>(q + z1), 0.f), maxq);
                    q = rnd<T>(s1 * rnd<T>(q - z1));
                }
                acc += (double)rnd<T>(powf(fabsf(rnd<T>(q - v)), expo));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            const float err = rnd<T>((float)acc);
            if (err < best) { best = err; scale = s1; zero = z1; }       // NaN sums never win
        }
    }
    if (lane == 0) {
        scale_out[u] = scale;
        zero_out[u] = zero;
    }
}

}  // namespace actq
}  // namespace rq

extern "C" int rq_act_quant(const void* x, void* out, int dtype, int64_t units, int unit_len, int with_zero,
                            float clip_ratio, int maxq, int sym, float* scale_out, float* zero_out,
                            const float* scale_in, const float* zero_in, int codes, int dtype_math, int weight_rule,
                            void* stream) {
    using namespace rq::actq;
    if (!x || units < 0 || unit_len <= 0 || maxq <= 0 || !(clip_ratio > 0.f) || clip_ratio > 1.f) return RQ_ERR_INVALID;
    if (!out && !scale_out) return RQ_ERR_INVALID;
    if (!sym && scale_in && !zero_in) return RQ_ERR_INVALID;
    if (units == 0) return RQ_OK;
    cudaStream_t st = rq::as_stream(stream);
    const int vn = dtype == RQ_F32 ? 4 : 8;
    const int vec_ok = (unit_len % vn == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                        (!out || reinterpret_cast<uintptr_t>(out) % 16 == 0)) ? 1 : 0;
    const bool wide = unit_len > 1024;                    // a block per unit, else a warp (or half a warp) per unit
    // short units (a group of 128 half-precision values is 16 words of 16 bytes): 16 threads per unit, so that every
    // lane has a word (65536 x 4096 bf16 in groups of 128: 1.12 -> 0.57 ms against a warp per unit)
    const bool narrow = vec_ok && unit_len / vn <= 16;
    int64_t blocks = wide ? units : narrow ? (units + 15) / 16 : (units + 7) / 8;
    if (blocks > 148 * 64) blocks = 148 * 64;
#define RQ_ACTQ_ARGS(T)                                                                                            \
    reinterpret_cast<const T*>(x), reinterpret_cast<T*>(out), units, unit_len, with_zero, clip_ratio, (float)maxq, \
        sym, scale_out, zero_out, scale_in, zero_in, codes, dtype_math, vec_ok, weight_rule
#define RQ_ACTQ_LAUNCH(T)                                                                                          \
    do {                                                                                                           \
        if (wide) act_quant_kernel<T, 256><<<(unsigned)blocks, 256, 0, st>>>(RQ_ACTQ_ARGS(T));                     \
        else if (narrow) act_quant_kernel<T, 16><<<(unsigned)blocks, 256, 0, st>>>(RQ_ACTQ_ARGS(T));               \
        else act_quant_kernel<T, 32><<<(unsigned)blocks, 256, 0, st>>>(RQ_ACTQ_ARGS(T));                           \
    } while (0)
    if (dtype == RQ_F32) RQ_ACTQ_LAUNCH(float);
    else if (dtype == RQ_BF16) RQ_ACTQ_LAUNCH(__nv_bfloat16);
    else if (dtype == RQ_F16) RQ_ACTQ_LAUNCH(__half);
    else return RQ_ERR_INVALID;
#undef RQ_ACTQ_ARGS
#undef RQ_ACTQ_LAUNCH
    return rq::check_launch();
}

extern "C" int rq_group_mse_search(const void* x, int dtype, int64_t units, int unit_len, int maxq, int sym, float norm,
                                   int grid, float maxshrink, float* scale_out, float* zero_out, void* stream) {
    using namespace rq::actq;
    if (!x || !scale_out || !zero_out || units < 0 || unit_len <= 0 || maxq <= 0 || grid <= 0) return RQ_ERR_INVALID;
    if (units == 0) return RQ_OK;
    cudaStream_t st = rq::as_stream(stream);
    const int steps = (int)(maxshrink * (float)grid);
    const unsigned blocks = (unsigned)((units + 7) / 8);
    if (dtype == RQ_F32)
        group_mse_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(x), units, unit_len, (float)maxq,
                                                        sym, norm, grid, steps, scale_out, zero_out);
    else if (dtype == RQ_BF16)
        group_mse_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), units,
                                                                unit_len, (float)maxq, sym, norm, grid, steps,
                                                                scale_out, zero_out);
    else if (dtype == RQ_F16)
        group_mse_kernel<__half><<<blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(x), units, unit_len,
                                                         (float)maxq, sym, norm, grid, steps, scale_out, zero_out);
    else
        return RQ_ERR_INVALID;
    return rq::check_launch();
}
