// Saliency statistics of the calibration backward pass (gptq_utils/gptq_plus_utils.py:2388-2404): the
// per-token mean of the squared output gradient over each channel group,
//     s[b, t, g] = mean_{c in group g} grad[b, t, c]^2,
// the per-token weights of the grouped Hessians.  HBM-bound: every gradient element is read once
// (2 or 4 bytes), G floats are written per token.
#include "rq_common.cuh"

namespace rq {
namespace sal {

constexpr int kWarps = 8;

template <typename T>
__device__ __forceinline__ float sum_sq_vec(const T* p);
template <>
__device__ __forceinline__ float sum_sq_vec<float>(const float* p) {          // 4 floats
    const float4 v = *reinterpret_cast<const float4*>(p);
    return fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
}
template <>
__device__ __forceinline__ float sum_sq_vec<__nv_bfloat16>(const __nv_bfloat16* p) {   // 8 bf16
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        s = fmaf(f.x, f.x, fmaf(f.y, f.y, s));
    }
    return s;
}
template <>
__device__ __forceinline__ float sum_sq_vec<__half>(const __half* p) {         // 8 fp16
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        s = fmaf(f.x, f.x, fmaf(f.y, f.y, s));
    }
    return s;
}

// one warp per (token, group); tokens are addressed as (batch b, position t) with their own strides so that a
// slice along the sequence (dropped sink positions) needs no copy.  VEC: elements per 16-byte load, or 1.
template <typename T, int VEC>
__global__ void __launch_bounds__(32 * kWarps) group_mean_square_kernel(const T* __restrict__ g, int64_t stride_b,
                                                                       int64_t stride_t, int64_t seq, int64_t tokens,
                                                                       int hidden, int G, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int gs = hidden / G;
    const float inv = 1.f / (float)gs;
    for (int64_t u = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); u < tokens * G; u += (int64_t)gridDim.x * kWarps) {
        const int64_t tok = u / G;
        const int grp = (int)(u - tok * G);
        const int64_t b = tok / seq, t = tok - b * seq;
        const T* p = g + b * stride_b + t * stride_t + (int64_t)grp * gs;
        float s0 = 0.f, s1 = 0.f;
        if (VEC > 1) {
            int c = lane * VEC;
            for (; c + 32 * VEC < gs; c += 64 * VEC) {          // two independent chains
                s0 += sum_sq_vec<T>(p + c);
                s1 += sum_sq_vec<T>(p + c + 32 * VEC);
            }
            if (c < gs) s0 += sum_sq_vec<T>(p + c);
        } else {
            for (int c = lane; c < gs; c += 32) {
                const float v = load_as_float<T>(p, c);
                s0 = fmaf(v, v, s0);
            }
        }
        float s = s0 + s1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) out[u] = s * inv;
    }
}

}  // namespace sal
}  // namespace rq

extern "C" int rq_group_mean_square(const void* grad, int dtype, int64_t batch, int64_t seq, int64_t stride_b,
                                    int64_t stride_t, int hidden, int G, float* out, void* stream) {
    using namespace rq::sal;
    if (!grad || !out || batch < 0 || seq < 0 || hidden <= 0 || G <= 0 || hidden % G != 0) return RQ_ERR_INVALID;
    const int64_t tokens = batch * seq;
    if (tokens == 0) return RQ_OK;
    const int gs = hidden / G;
    const int esz = dtype == RQ_F32 ? 4 : 2;
    const int vec = 16 / esz;
    const bool aligned = (reinterpret_cast<uintptr_t>(grad) % 16 == 0) && gs % vec == 0 && stride_b % vec == 0 &&
                         stride_t % vec == 0;
    int64_t blocks = (tokens * G + kWarps - 1) / kWarps;
    if (blocks > 148 * 32) blocks = 148 * 32;
    cudaStream_t st = rq::as_stream(stream);
#define RQ_SAL_LAUNCH(T, V)                                                                                        \
    group_mean_square_kernel<T, V><<<(unsigned)blocks, 32 * kWarps, 0, st>>>(reinterpret_cast<const T*>(grad), stride_b, \
                                                                            stride_t, seq, tokens, hidden, G, out)
    if (dtype == RQ_F32) { if (aligned) RQ_SAL_LAUNCH(float, 4); else RQ_SAL_LAUNCH(float, 1); }
    else if (dtype == RQ_BF16) { if (aligned) RQ_SAL_LAUNCH(__nv_bfloat16, 8); else RQ_SAL_LAUNCH(__nv_bfloat16, 1); }
    else if (dtype == RQ_F16) { if (aligned) RQ_SAL_LAUNCH(__half, 8); else RQ_SAL_LAUNCH(__half, 1); }
    else return RQ_ERR_INVALID;
#undef RQ_SAL_LAUNCH
    return rq::check_launch();
}
