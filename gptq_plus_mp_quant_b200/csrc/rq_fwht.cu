// Walsh-Hadamard rotation  y = x . H_n * scale  for n = K * 2^m  (HBM-bound).
//
// A work item is one row (or, for short rows, a batch of rows) held in shared memory as fp32.
// The power-of-two part runs as radix-16 register butterflies over shared memory (at most
// ceil(m/4) passes); the optional K x K mix (K = 12, 20, 28, ...: the non-power-of-two factor)
// is a small +-1 matrix product per position.  Input is read once and output written once with
// 16-byte accesses where alignment allows; all arithmetic is fp32 whatever the I/O type.
#include "rq_common.cuh"
#include "rq_fwht_warp.cuh"

namespace rq {
namespace fwht {

constexpr int kThreads = 256;
constexpr int kMaxK = 64;       // register-resident mix, matrix in shared memory
constexpr int kMaxWideK = 256;  // beyond kMaxK: the mix reads the matrix from global memory (L1-resident) and
                                // writes its sums straight to the output

// one padding word per 16 keeps the strided radix-16 accesses of every pass on distinct banks
__device__ __forceinline__ int pad(int i) { return i + (i >> 4); }

template <int R>
__device__ __forceinline__ void butterflies(float (&v)[1 << R]) {
#pragma unroll
    for (int h = 1; h < (1 << R); h <<= 1) {
#pragma unroll
        for (int b = 0; b < (1 << R); ++b) {
            if ((b & h) == 0) {
                const float a = v[b], c = v[b | h];
                v[b] = a + c;
                v[b | h] = a - c;
            }
        }
    }
}

// One pass over index bits [lo, lo+R) of `total` shared-memory elements.
template <int R>
__device__ __forceinline__ void smem_pass(float* buf, int total, int lo) {
    const int groups = total >> R;
    const int lomask = (1 << lo) - 1;
    for (int gi = threadIdx.x; gi < groups; gi += kThreads) {
        const int base = ((gi >> lo) << (lo + R)) | (gi & lomask);
        float v[1 << R];
#pragma unroll
        for (int b = 0; b < (1 << R); ++b) v[b] = buf[pad(base + (b << lo))];
        butterflies<R>(v);
#pragma unroll
        for (int b = 0; b < (1 << R); ++b) buf[pad(base + (b << lo))] = v[b];
    }
}

// chunk k' = sum_k hadK[k'][k] * chunk k at one position; hadK entries are +-1 so the products are exact.
template <int KK>
__device__ __forceinline__ void mix(float* buf, const float* hk, int base, int P) {
    float v[KK];
#pragma unroll
    for (int k = 0; k < KK; ++k) v[k] = buf[pad(base + k * P)];
#pragma unroll 4
    for (int ko = 0; ko < KK; ++ko) {
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < KK; ++k) acc = fmaf(hk[ko * KK + k], v[k], acc);
        buf[pad(base + ko * P)] = acc;
    }
}

__device__ __noinline__ void mix_any(float* buf, const float* hk, int base, int P, int K) {
    float v[kMaxK];
    for (int k = 0; k < K; ++k) v[k] = buf[pad(base + k * P)];
    for (int ko = 0; ko < K; ++ko) {
        float acc = 0.f;
        for (int k = 0; k < K; ++k) acc = fmaf(hk[ko * K + k], v[k], acc);
        buf[pad(base + ko * P)] = acc;
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) fwht_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows,
                                                        int n, int K, int m, int rows_per_item,
                                                        const float* __restrict__ hadK, float scale) {
    extern __shared__ float buf[];                       // pad(rows_per_item * n) floats, then K*K mix matrix
    const int item_elems = rows_per_item * n;
    float* hk = buf + pad(item_elems) + 1;
    if (K > 1 && K <= kMaxK)
        for (int e = threadIdx.x; e < K * K; e += kThreads) hk[e] = hadK[e];
    const int64_t items = (rows + rows_per_item - 1) / rows_per_item;
    const int P = n / K;

    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const int64_t row0 = item * rows_per_item;
        const int64_t valid = (rows - row0 < rows_per_item ? rows - row0 : rows_per_item) * (int64_t)n;
        const T* src = x + row0 * n;
        T* dst = y + row0 * n;
        __syncthreads();                                  // previous item fully written out
        // ---- load (16-byte vectors when the item start is aligned)
        constexpr int V = 16 / sizeof(T);
        const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0 &&
                             (valid % V) == 0;
        if (aligned) {
            for (int64_t e = (int64_t)threadIdx.x * V; e < valid; e += (int64_t)kThreads * V) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src + e);
                const T* t = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int k = 0; k < V; ++k) buf[pad((int)e + k)] = load_as_float<T>(t, k);
            }
        } else {
            for (int e = threadIdx.x; e < valid; e += kThreads) buf[pad(e)] = load_as_float<T>(src, e);
        }
        for (int e = (int)valid + threadIdx.x; e < item_elems; e += kThreads) buf[pad(e)] = 0.f;   // ragged last item
        __syncthreads();
        // ---- butterflies over bits [0, m)
        int lo = 0;
        while (lo < m) {
            const int r = (m - lo) >= 4 ? 4 : (m - lo);
            if (r == 4) smem_pass<4>(buf, item_elems, lo);
            else if (r == 3) smem_pass<3>(buf, item_elems, lo);
            else if (r == 2) smem_pass<2>(buf, item_elems, lo);
            else smem_pass<1>(buf, item_elems, lo);
            lo += r;
            __syncthreads();
        }
        if (K > kMaxK) {
            // ---- wide mix, straight from shared memory to the output: a thread owns 4 output chunks x 2
            // neighbouring positions, so that a term costs 2 shared-memory words and 4 matrix entries (the same
            // address in every lane of a warp: a broadcast from L1) for 8 multiply-adds
            const int kt = (K + 3) >> 2, half = P >> 1;                // P is a power of two >= 2 on this path
            const int live_rows = (int)(valid / n);
            const int tiles = live_rows * kt * half;
            if (P == 1) {                                              // n == K: a plain matrix-vector product per row
                for (int e = threadIdx.x; e < (int)valid; e += kThreads) {
                    const int r = e / n, ko = e - r * n;
                    float acc = 0.f;
                    for (int k = 0; k < K; ++k) acc = fmaf(__ldg(hadK + (size_t)ko * K + k), buf[pad(r * n + k)], acc);
                    store_from_float<T>(dst, e, acc * scale);
                }
            }
            for (int t = threadIdx.x; t < tiles; t += kThreads) {
                const int pp = t % half, rest = t / half;
                const int k4 = rest % kt, r = rest / kt;
                const int ko = 4 * k4, p = 2 * pp;
                const float* h0 = hadK + (size_t)ko * K;
                const float* h1 = h0 + (ko + 1 < K ? K : 0);
                const float* h2 = h0 + (ko + 2 < K ? 2 * K : 0);
                const float* h3 = h0 + (ko + 3 < K ? 3 * K : 0);
                const int base = r * n + p;
                float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f, a20 = 0.f, a21 = 0.f, a30 = 0.f, a31 = 0.f;
                for (int k = 0; k < K; ++k) {
                    const float v0 = buf[pad(base + k * P)], v1 = buf[pad(base + k * P + 1)];
                    const float c0 = __ldg(h0 + k), c1 = __ldg(h1 + k), c2 = __ldg(h2 + k), c3 = __ldg(h3 + k);
                    a00 = fmaf(c0, v0, a00); a01 = fmaf(c0, v1, a01);
                    a10 = fmaf(c1, v0, a10); a11 = fmaf(c1, v1, a11);
                    a20 = fmaf(c2, v0, a20); a21 = fmaf(c2, v1, a21);
                    a30 = fmaf(c3, v0, a30); a31 = fmaf(c3, v1, a31);
                }
                T* o = dst + (size_t)r * n + (size_t)ko * P + p;
                store_from_float<T>(o, 0, a00 * scale); store_from_float<T>(o, 1, a01 * scale);
                if (ko + 1 < K) { store_from_float<T>(o, P, a10 * scale); store_from_float<T>(o, P + 1, a11 * scale); }
                if (ko + 2 < K) { store_from_float<T>(o, 2 * P, a20 * scale); store_from_float<T>(o, 2 * P + 1, a21 * scale); }
                if (ko + 3 < K) { store_from_float<T>(o, 3 * P, a30 * scale); store_from_float<T>(o, 3 * P + 1, a31 * scale); }
            }
            continue;
        }
        // ---- K x K mix across the K chunks of each row (in place: a thread owns one position of one row)
        if (K > 1) {
            const int positions = rows_per_item * P;
            for (int pi = threadIdx.x; pi < positions; pi += kThreads) {
                const int r = pi / P, p = pi - r * P;
                const int base = r * n + p;
                if (K == 12) mix<12>(buf, hk, base, P);
                else if (K == 20) mix<20>(buf, hk, base, P);
                else if (K == 28) mix<28>(buf, hk, base, P);
                else mix_any(buf, hk, base, P, K);
            }
            __syncthreads();
        }
        // ---- store
        if (aligned) {
            for (int64_t e = (int64_t)threadIdx.x * V; e < valid; e += (int64_t)kThreads * V) {
                uint4 raw;
                T* t = reinterpret_cast<T*>(&raw);
#pragma unroll
                for (int k = 0; k < V; ++k) store_from_float<T>(t, k, buf[pad((int)e + k)] * scale);
                *reinterpret_cast<uint4*>(dst + e) = raw;
            }
        } else {
            for (int e = threadIdx.x; e < valid; e += kThreads) store_from_float<T>(dst, e, buf[pad(e)] * scale);
        }
    }
}

}  // namespace fwht
}  // namespace rq

using namespace rq;

// rqp != nullptr: the fused rotation + per-token quantization, which only the register-resident paths offer
static int fwht_impl(const void* x, void* y, int dtype, int64_t rows, int n, int K, const float* hadK, float scale,
                     const rq::fwht::RowQuant* rqp, void* stream) {
    using namespace rq::fwht;
    if (!x || !y || rows < 0 || n <= 0 || K <= 0 || n % K != 0) return RQ_ERR_INVALID;
    if (K > 1 && !hadK) return RQ_ERR_INVALID;
    if (K > kMaxWideK) return RQ_ERR_UNSUPPORTED;
    const int P = n / K;
    if ((P & (P - 1)) != 0) return RQ_ERR_INVALID;
    if (rows == 0) return RQ_OK;
    int m = 0;
    while ((1 << m) < P) ++m;
    int dev0 = 0, sms0 = 148;
    cudaGetDevice(&dev0);
    cudaDeviceGetAttribute(&sms0, cudaDevAttrMultiProcessorCount, dev0);
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    // ---- fast path: register-resident warp transform
    if (aligned16 && K == 1 && (P == 2048 || P == 4096 || P == 8192)) {
        // one chunk per CTA of P/1024 warps
        cudaStream_t st = as_stream(stream);
        prof::Scope timed(RQ_PROF_FWHT, st);
        const int W = P / 1024;
        const int64_t nchunks = rows;
        const size_t smem = (size_t)W * warp_slice_floats(1024) * sizeof(float);
        int per_sm = (int)((200 * 1024) / (smem + 1024));
        if (per_sm > 16 / W * 2) per_sm = 16 / W * 2;
        if (per_sm < 1) per_sm = 1;
        int64_t grid = nchunks < (int64_t)sms0 * per_sm ? nchunks : (int64_t)sms0 * per_sm;
        cudaError_t e = cudaSuccess;
#define RQ_SPLIT_LAUNCH(T, WW)                                                                                    \
    if (rqp) {                                                                                                     \
        e = cudaFuncSetAttribute(fwht_split_kernel<T, WW, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                 (int)smem);                                                                       \
        if (e != cudaSuccess) return RQ_ERR_CUDA;                                                                  \
        fwht_split_kernel<T, WW, true><<<(unsigned)grid, 32 * WW, smem, st>>>(                                     \
            reinterpret_cast<const T*>(x), reinterpret_cast<T*>(y), nchunks, scale, *rqp);                         \
    } else {                                                                                                       \
        e = cudaFuncSetAttribute(fwht_split_kernel<T, WW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return RQ_ERR_CUDA;                                                                  \
        /* a grid-stride loop: no more CTAs than are resident at once, or the surplus would run as a tail */      \
        int occ = 0;                                                                                               \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fwht_split_kernel<T, WW>, 32 * WW, smem) ==        \
                cudaSuccess && occ > 0 && grid > (int64_t)sms0 * occ)                                              \
            grid = (int64_t)sms0 * occ;                                                                            \
        fwht_split_kernel<T, WW><<<(unsigned)grid, 32 * WW, smem, st>>>(reinterpret_cast<const T*>(x),             \
                                                                        reinterpret_cast<T*>(y), nchunks, scale);  \
    }
#define RQ_SPLIT_DISPATCH(T)                                \
    if (W == 2) { RQ_SPLIT_LAUNCH(T, 2); }                  \
    else if (W == 4) { RQ_SPLIT_LAUNCH(T, 4); }             \
    else { RQ_SPLIT_LAUNCH(T, 8); }
        if (dtype == RQ_F32) { RQ_SPLIT_DISPATCH(float) }
        else if (dtype == RQ_BF16) { RQ_SPLIT_DISPATCH(__nv_bfloat16) }
        else if (dtype == RQ_F16) { RQ_SPLIT_DISPATCH(__half) }
        else return RQ_ERR_INVALID;
#undef RQ_SPLIT_DISPATCH
#undef RQ_SPLIT_LAUNCH
        return check_launch();
    }
    if (aligned16 && P <= 4096 && (K == 1 || (P >= 1024 && K <= 28))) {
        cudaStream_t st = as_stream(stream);
        prof::Scope timed(RQ_PROF_FWHT, st);
        const int logs = m < 10 ? 10 : m;
        const int S = 1 << logs;
        cudaError_t e = cudaSuccess;
        if (K == 1 && rqp) return RQ_ERR_UNSUPPORTED;
        if (K == 1) {
            const int64_t total = rows * (int64_t)n;
            const int64_t nsc = (total + S - 1) / S;
            const size_t smem = (size_t)kWarpsPerCta * warp_slice_floats(S) * sizeof(float);
            int per_sm = (int)((200 * 1024) / (smem + 1024));
            if (per_sm > 8) per_sm = 8;
            int64_t grid = (nsc + kWarpsPerCta - 1) / kWarpsPerCta;
            if (grid > (int64_t)sms0 * per_sm) grid = (int64_t)sms0 * per_sm;
#define RQ_WARP_LAUNCH(T, L)                                                                                      \
    e = cudaFuncSetAttribute(fwht_warp_kernel<T, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    if (e != cudaSuccess) return RQ_ERR_CUDA;                                                                      \
    fwht_warp_kernel<T, L><<<(unsigned)grid, 32 * kWarpsPerCta, smem, st>>>(reinterpret_cast<const T*>(x),         \
                                                                            reinterpret_cast<T*>(y), total, m, scale)
#define RQ_WARP_DISPATCH(T)                                  \
    if (logs == 10) { RQ_WARP_LAUNCH(T, 10); }               \
    else if (logs == 11) { RQ_WARP_LAUNCH(T, 11); }          \
    else { RQ_WARP_LAUNCH(T, 12); }
            if (dtype == RQ_F32) { RQ_WARP_DISPATCH(float) }
            else if (dtype == RQ_BF16) { RQ_WARP_DISPATCH(__nv_bfloat16) }
            else if (dtype == RQ_F16) { RQ_WARP_DISPATCH(__half) }
            else return RQ_ERR_INVALID;
#undef RQ_WARP_DISPATCH
#undef RQ_WARP_LAUNCH
            return check_launch();
        }
        const bool swz = mix_swizzled(logs, K <= 12 ? 12 : 28, rqp != nullptr);     // as the kernel chosen below
        const size_t smem = ((size_t)K * warp_slice_floats(S, swz) + (mix_matrix_shared(K, swz) ? (size_t)K * K : 0)) *
                            sizeof(float);
        if (smem <= 220 * 1024) {
            int64_t grid = rows;
            // one row per CTA and a grid-stride loop: as many CTAs as are resident at once (two per SM up to K = 28 at
            // S = 1024, which needs the whole shared-memory carve-out)
#define RQ_MIX_GO(KERNEL, THREADS, ...)                                                                           \
    {                                                                                                              \
        auto kfn = KERNEL;                                                                                         \
        e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                     \
        if (e != cudaSuccess) return RQ_ERR_CUDA;                                                                  \
        cudaFuncSetAttribute(kfn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared); \
        int occ = 0;                                                                                               \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kfn, THREADS, smem) != cudaSuccess || occ < 1)     \
            occ = 1;                                                                                               \
        if (grid > (int64_t)sms0 * occ) grid = (int64_t)sms0 * occ;                                                \
        kfn<<<(unsigned)grid, THREADS, smem, st>>>(__VA_ARGS__);                                                   \
    }
#define RQ_MIX_LAUNCH(T, L)                                                                                       \
    if (rqp) {                                                                                                     \
        RQ_MIX_GO((fwht_mix_kernel<T, L, true>), 32 * kMixWarps, reinterpret_cast<const T*>(x),                    \
                  reinterpret_cast<T*>(y), rows, K, hadK, scale, *rqp)                                             \
    } else if (K <= 12) {                                                                                          \
        RQ_MIX_GO((fwht_mix_kernel<T, L, false, 12, RQ_MIX12_WARPS>), 32 * RQ_MIX12_WARPS,                         \
                  reinterpret_cast<const T*>(x), reinterpret_cast<T*>(y), rows, K, hadK, scale, RowQuant())        \
    } else {                                                                                                       \
        RQ_MIX_GO((fwht_mix_kernel<T, L, false, 28, (L == 10 ? RQ_MIX28_WARPS : kMixWarps)>),                      \
                  32 * (L == 10 ? RQ_MIX28_WARPS : kMixWarps), reinterpret_cast<const T*>(x),                      \
                  reinterpret_cast<T*>(y), rows, K, hadK, scale, RowQuant())                                       \
    }
#define RQ_MIX_DISPATCH(T)                                  \
    if (logs == 10) { RQ_MIX_LAUNCH(T, 10); }               \
    else if (logs == 11) { RQ_MIX_LAUNCH(T, 11); }          \
    else { RQ_MIX_LAUNCH(T, 12); }
            if (dtype == RQ_F32) { RQ_MIX_DISPATCH(float) }
            else if (dtype == RQ_BF16) { RQ_MIX_DISPATCH(__nv_bfloat16) }
            else if (dtype == RQ_F16) { RQ_MIX_DISPATCH(__half) }
            else return RQ_ERR_INVALID;
#undef RQ_MIX_DISPATCH
#undef RQ_MIX_LAUNCH
#undef RQ_MIX_GO
            return check_launch();
        }
    }
    if (rqp) return RQ_ERR_UNSUPPORTED;
    // ---- general path: shared-memory radix passes (any K, chunks longer than 4096, unaligned buffers)
    // short rows are batched so that an item has about 4096 elements; whole chunks only
    int rows_per_item = 1;
    if (n < 4096) {
        rows_per_item = 4096 / n;
        if (rows_per_item > rows) rows_per_item = (int)rows;
        if (rows_per_item < 1) rows_per_item = 1;
    }
    const int64_t item_elems = (int64_t)rows_per_item * n;
    const size_t smem = ((size_t)(item_elems + (item_elems >> 4)) + 2 + (K <= kMaxK ? (size_t)K * K : 0)) * sizeof(float);
    if (smem > 220 * 1024) return RQ_ERR_UNSUPPORTED;
    const int64_t items = (rows + rows_per_item - 1) / rows_per_item;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int per_sm = (int)((200 * 1024) / (smem + 1024));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 8) per_sm = 8;
    int64_t grid = (int64_t)sms * per_sm;
    if (grid > items) grid = items;
    cudaStream_t st = as_stream(stream);
    cudaError_t e = cudaSuccess;
    prof::Scope timed2(RQ_PROF_FWHT, st);
#define RQ_FWHT_LAUNCH(T)                                                                                       \
    e = cudaFuncSetAttribute(fwht_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
    if (e != cudaSuccess) return RQ_ERR_CUDA;                                                                   \
    fwht_kernel<T><<<(unsigned)grid, kThreads, smem, st>>>(reinterpret_cast<const T*>(x), reinterpret_cast<T*>(y), \
                                                           rows, n, K, m, rows_per_item, hadK, scale)
    if (dtype == RQ_F32) { RQ_FWHT_LAUNCH(float); }
    else if (dtype == RQ_BF16) { RQ_FWHT_LAUNCH(__nv_bfloat16); }
    else if (dtype == RQ_F16) { RQ_FWHT_LAUNCH(__half); }
    else return RQ_ERR_INVALID;
#undef RQ_FWHT_LAUNCH
    return check_launch();
}

extern "C" int rq_fwht(const void* x, void* y, int dtype, int64_t rows, int n, int K, const float* hadK, float scale,
                       void* stream) {
    return fwht_impl(x, y, dtype, rows, n, K, hadK, scale, nullptr, stream);
}

extern "C" int rq_fwht_act_quant(const void* x, void* y, int dtype, int64_t rows, int n, int K, const float* hadK,
                                 float scale, float clip_ratio, int maxq, int sym, float* scale_out, float* zero_out,
                                 void* stream) {
    if (maxq <= 0 || !(clip_ratio > 0.f) || clip_ratio > 1.f) return RQ_ERR_INVALID;
    rq::fwht::RowQuant q;
    q.clip = clip_ratio;
    q.maxq = (float)maxq;
    q.sym = sym ? 1 : 0;
    q.scale_out = scale_out;
    q.zero_out = zero_out;
    return fwht_impl(x, y, dtype, rows, n, K, hadK, scale, &q, stream);
}

// ------------------------------------------------------------------------------------------
// Hadamard transform ACROSS the heads of an attention output (the online partial rotation in front of o_proj,
// utils/quant_utils.py:258-281): x viewed [tokens, H, D]; for every token and every position d inside a head
//     y[t][h'][d] = scale * sum_h Had_H[h'][h] * x[t][h][d].
// One thread owns a (token, d) pair and holds the H values in registers: the loads and stores of a warp are
// contiguous along d, the transform needs no shared memory.  H = K * 2^m, K * 2^m <= 64; hadK as in rq_fwht.
// ------------------------------------------------------------------------------------------
namespace rq {
namespace fwht {

template <typename T, int HMAX>
__global__ void __launch_bounds__(256) heads_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t tokens, int H,
                                                    int D, int K, const float* __restrict__ hadK, float scale) {
    __shared__ float hk[kMaxK * kMaxK];
    if (K > 1)
        for (int e = threadIdx.x; e < K * K; e += blockDim.x) hk[e] = hadK[e];
    __syncthreads();
    const int P = H / K;                                   // power-of-two part, contiguous inside each of the K chunks
    const int64_t total = tokens * D;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = u / D;
        const int d = (int)(u - t * D);
        const T* px = x + t * (int64_t)H * D + d;
        float v[HMAX];
#pragma unroll
        for (int h = 0; h < HMAX; ++h) v[h] = (h < H) ? load_as_float<T>(px, (int64_t)h * D) : 0.f;
#pragma unroll
        for (int len = 1; len < HMAX; len <<= 1) {
            if (len < P) {
#pragma unroll
                for (int h = 0; h < HMAX; ++h) {
                    if ((h & len) == 0 && h + len < HMAX) {
                        const float a = v[h], b = v[h + len];
                        v[h] = a + b;
                        v[h + len] = a - b;
                    }
                }
            }
        }
        T* py = y + t * (int64_t)H * D + d;
        if (K == 1) {
#pragma unroll
            for (int h = 0; h < HMAX; ++h)
                if (h < H) store_from_float<T>(py, (int64_t)h * D, v[h] * scale);
        } else {
            // chunk k' = sum_k hadK[k'][k] * chunk k, position by position
            for (int ko = 0; ko < K; ++ko) {
                for (int pp = 0; pp < P; ++pp) {
                    float s = 0.f;
                    for (int k = 0; k < K; ++k) {
                        float val = 0.f;
#pragma unroll
                        for (int h = 0; h < HMAX; ++h)
                            if (h == k * P + pp) val = v[h];
                        s = fmaf(hk[ko * K + k], val, s);
                    }
                    store_from_float<T>(py, (int64_t)(ko * P + pp) * D, s * scale);
                }
            }
        }
    }
}

}  // namespace fwht
}  // namespace rq

extern "C" int rq_fwht_heads(const void* x, void* y, int dtype, int64_t tokens, int H, int D, int K, const float* hadK,
                             float scale, void* stream) {
    using namespace rq::fwht;
    if (!x || !y || tokens < 0 || H <= 0 || D <= 0 || K <= 0 || H % K != 0 || H > 64) return RQ_ERR_INVALID;
    if (K > 1 && !hadK) return RQ_ERR_INVALID;
    if (K > kMaxK) return RQ_ERR_UNSUPPORTED;
    const int P = H / K;
    if ((P & (P - 1)) != 0) return RQ_ERR_INVALID;
    if (K > 1 && x == y) return RQ_ERR_INVALID;            // the K x K mix is not done in place
    if (tokens == 0) return RQ_OK;
    cudaStream_t st = as_stream(stream);
    prof::Scope timed(RQ_PROF_FWHT, st);
    int64_t blocks = (tokens * D + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
#define RQ_HEADS(T)                                                                                              \
    do {                                                                                                         \
        if (H <= 32)                                                                                             \
            heads_kernel<T, 32><<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const T*>(x),                 \
                                                                  reinterpret_cast<T*>(y), tokens, H, D, K, hadK, scale); \
        else                                                                                                     \
            heads_kernel<T, 64><<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const T*>(x),                 \
                                                                  reinterpret_cast<T*>(y), tokens, H, D, K, hadK, scale); \
    } while (0)
    if (dtype == RQ_F32) RQ_HEADS(float);
    else if (dtype == RQ_BF16) RQ_HEADS(__nv_bfloat16);
    else if (dtype == RQ_F16) RQ_HEADS(__half);
    else return RQ_ERR_INVALID;
#undef RQ_HEADS
    return check_launch();
}
