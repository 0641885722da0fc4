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

// ------------------------------------------------------------------------------------------
// Percentile clip of the saliencies (gptq_utils/gptq_plus_utils.py:2834-2839):
//     cap = torch.quantile(s.flatten(), q);  s = clamp(s, max=cap)
// torch.quantile sorts; only two order statistics are needed.  With rank = fl32(q) * fl32(n - 1), the values at
// floor(rank) and ceil(rank) are found exactly by a most-significant-digit-first radix selection over the
// order-preserving integer image of the floats: four passes of a 256-bin histogram per statistic (a pass only
// counts the elements whose higher digits match the digits chosen so far), then
//     cap = lerp(lo, hi, rank - floor(rank))        (torch's two-sided lerp)
// and one clamp pass.  NaN anywhere makes the quantile, and with it every clamped value, NaN as in torch.
// HBM-bound, five reads and one write of the tensor (which is small: tokens x G floats).
// ------------------------------------------------------------------------------------------
namespace rq {
namespace sal {

struct SelectState {
    unsigned int prefix[2];      // digits chosen so far (higher bytes), order-preserving image
    unsigned int remaining[2];   // rank of the wanted element among those that match the prefix
    unsigned int nan_count;
    unsigned int pad[3];
    unsigned int hist[2][256];
};

__device__ __forceinline__ unsigned int ordered_bits(float v) {
    const unsigned int b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(unsigned int u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

__global__ void select_init_kernel(SelectState* st, unsigned int k0, unsigned int k1) {
    for (int i = threadIdx.x; i < 512; i += blockDim.x) (&st->hist[0][0])[i] = 0u;
    if (threadIdx.x == 0) {
        st->prefix[0] = st->prefix[1] = 0u;
        st->remaining[0] = k0;
        st->remaining[1] = k1;
        st->nan_count = 0u;
    }
}

__global__ void __launch_bounds__(256) select_hist_kernel(const float* __restrict__ x, int64_t n, SelectState* st,
                                                          int shift) {
    __shared__ unsigned int h[2][256];
    h[0][threadIdx.x] = 0u;
    h[1][threadIdx.x] = 0u;
    __syncthreads();
    const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    const unsigned int p0 = st->prefix[0] & mask, p1 = st->prefix[1] & mask;
    unsigned int nans = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        if (shift == 24 && v != v) ++nans;
        const unsigned int u = ordered_bits(v);
        const unsigned int d = (u >> shift) & 255u;
        if ((u & mask) == p0) atomicAdd(&h[0][d], 1u);
        if ((u & mask) == p1) atomicAdd(&h[1][d], 1u);
    }
    __syncthreads();
    if (h[0][threadIdx.x]) atomicAdd(&st->hist[0][threadIdx.x], h[0][threadIdx.x]);
    if (h[1][threadIdx.x]) atomicAdd(&st->hist[1][threadIdx.x], h[1][threadIdx.x]);
    if (nans) atomicAdd(&st->nan_count, nans);
}

// one warp per statistic: pick the digit whose bin holds the wanted rank, descend into it
__global__ void select_scan_kernel(SelectState* st, int shift) {
    const int sel = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (sel < 2) {
        unsigned int c[8], sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) { c[j] = st->hist[sel][lane * 8 + j]; sum += c[j]; }
        unsigned int incl = sum;                                   // inclusive scan over lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        unsigned int below = incl - sum;
        const unsigned int want = st->remaining[sel];
        int digit = -1;
        unsigned int rem = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (digit < 0 && want >= below && want < below + c[j]) { digit = lane * 8 + j; rem = want - below; }
            below += c[j];
        }
        __syncwarp();
        if (digit >= 0) {
            st->prefix[sel] |= (unsigned int)digit << shift;
            st->remaining[sel] = rem;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 512; i += blockDim.x) (&st->hist[0][0])[i] = 0u;
}

__global__ void __launch_bounds__(256) clamp_to_quantile_kernel(float* __restrict__ x, int64_t n,
                                                                const SelectState* __restrict__ st, float weight,
                                                                float* __restrict__ cap_out) {
    const float lo = from_ordered_bits(st->prefix[0]), hi = from_ordered_bits(st->prefix[1]);
    float cap = (fabsf(weight) < 0.5f) ? lo + weight * (hi - lo) : hi - (hi - lo) * (1.f - weight);
    if (st->nan_count) cap = __uint_as_float(0x7fc00000u);
    if (blockIdx.x == 0 && threadIdx.x == 0 && cap_out) *cap_out = cap;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        x[i] = (cap != cap) ? cap : ((v != v) ? v : fminf(v, cap));
    }
}

}  // namespace sal
}  // namespace rq

extern "C" size_t rq_quantile_workspace_bytes(void) { return sizeof(rq::sal::SelectState); }

extern "C" int rq_clamp_to_quantile(float* x, int64_t n, float q, float* cap_out, void* workspace,
                                    size_t workspace_bytes, void* stream) {
    using namespace rq::sal;
    if (!x || n < 0 || !(q >= 0.f) || q > 1.f || n >= (int64_t)1 << 31) return RQ_ERR_INVALID;
    if (!workspace || workspace_bytes < sizeof(SelectState) || reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
        return RQ_ERR_WORKSPACE;
    if (n == 0) return RQ_OK;
    cudaStream_t st = rq::as_stream(stream);
    SelectState* state = static_cast<SelectState*>(workspace);
    const float rank = q * (float)(n - 1);                         // fp32, as torch forms it
    const float below = floorf(rank), above = ceilf(rank);
    int64_t grid = (n + 255) / 256;
    if (grid > 148 * 8) grid = 148 * 8;
    select_init_kernel<<<1, 256, 0, st>>>(state, (unsigned int)below, (unsigned int)above);
    for (int shift = 24; shift >= 0; shift -= 8) {
        select_hist_kernel<<<(unsigned)grid, 256, 0, st>>>(x, n, state, shift);
        select_scan_kernel<<<1, 64, 0, st>>>(state, shift);
    }
    clamp_to_quantile_kernel<<<(unsigned)grid, 256, 0, st>>>(x, n, state, rank - below, cap_out);
    return rq::check_launch();
}
