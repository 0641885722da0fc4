// Warp-level Walsh-Hadamard transform: the fast path of rq_fwht for power-of-two chunks up to 4096.
//
// One warp owns a "super-chunk" of S = 1024 / 2048 / 4096 consecutive elements (one chunk, or several
// short ones) and keeps it in registers, E = S/32 per lane:
//   load   lane l reads 8 consecutive elements (16 B for bf16/fp16) at j*256 + l*8, j < E/8;
//   phase A  butterflies over the index bits that are thread-local in this mapping (0-2 and 8+);
//   transposition through the warp's private shared-memory slice (128-bit accesses, an XOR swizzle of the
//            256-element blocks keeps every access conflict free) so that index bits 3-7 become thread-local;
//   phase B  butterflies over bits 3-7; the result goes back to the same shared-memory slots.
// About 16 instructions per element instead of the ~50 of a shared-memory radix pass design, which is
// what an HBM-bound kernel can afford at 6.5 TB/s.  The K x K mix (n = K * 2^m) runs per row from shared memory.
#pragma once

#include "rq_common.cuh"
#include "rq_had_tables.cuh"

namespace rq {
namespace fwht {

constexpr int kWarpsPerCta = 4;
constexpr int kMixSharedMatrixMaxK = 24;
// which mix kernels use the unpadded, swizzled slices, and whether the caller's K x K matrix is copied behind them
__host__ __device__ constexpr bool mix_swizzled(int logs, int kmax, bool quant) { return logs == 10 && kmax > 12 && !quant; }
__host__ __device__ constexpr bool mix_matrix_shared(int K, bool swz) { return !swz || K <= kMixSharedMatrixMaxK; }
constexpr int kMixWarps = 8;          // warps of a CTA that transforms and mixes one row (n = K * 2^m, K > 1)

// Position of natural index idx inside a slice.  Two layouts keep the four (or more) 256-element blocks a warp
// touches in the second mapping on different banks: 8 padding words per 256 elements (addresses stay base + constant,
// which costs the fewest registers), or, SWZ, bits 3-4 XORed with bits 8-9 (no padding: 28 slices of 1024 floats are
// 112 KB, so that two rows fit an SM's shared memory).  Both keep aligned groups of 8 elements together.
template <bool SWZ = false>
__device__ __forceinline__ int wphys(int idx) {
    return SWZ ? (idx ^ (((idx >> 8) & 3) << 3)) : (idx + ((idx >> 8) << 3));
}
__host__ __device__ constexpr int warp_slice_floats(int S, bool swz = false) { return swz ? S : S + (S >> 8) * 8; }

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

// eight 16-bit values held in a 16-byte register quadruple -> fp32
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& r, float (&v)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& r, float (&v)[8]) {
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
    v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
    v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
}
__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t w) {
    __half2 h;
    *reinterpret_cast<uint32_t*>(&h) = w;
    return __half22float2(h);
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& r, float (&v)[8]) {
    const float2 a = half2_bits_to_float2(r.x), b = half2_bits_to_float2(r.y);
    const float2 c = half2_bits_to_float2(r.z), d = half2_bits_to_float2(r.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}

// sm_100 issues fp32 additions two at a time on aligned register pairs (add.f32x2 / fma.f32x2).  Where a kernel is
// short of issue slots the butterflies run on pairs (PACK), wherever both partners of two neighbouring registers
// are themselves neighbours.  Each half is the same IEEE round-to-nearest operation as the scalar form: u - w is
// computed as fma(w, -1, u), one rounding of the exact difference, so PACK changes no bit of the result.  It is
// chosen per kernel by measurement (bf16, GB/s of read + write, scalar -> paired): chunks of 4096 in four warps
// 4336 -> 4521, the 12-chunk mix 3795 -> 3992; the register pairs cost occupancy elsewhere (one warp per 1024-long
// chunk 3702 -> 2597, the 28-chunk mix 3085 -> 2858), and those stay scalar.
__device__ __forceinline__ float2 add2(float2 u, float2 w) { return __fadd2_rn(u, w); }
__device__ __forceinline__ float2 sub2(float2 u, float2 w) { return __ffma2_rn(w, make_float2(-1.f, -1.f), u); }
__device__ __forceinline__ void bfly2(float& u0, float& u1, float& w0, float& w1) {
    const float2 u = make_float2(u0, u1), w = make_float2(w0, w1);
    const float2 s = add2(u, w), d = sub2(u, w);
    u0 = s.x; u1 = s.y; w0 = d.x; w1 = d.y;
}

// butterfly over register-index bit RB of a[E]
template <int E, int RB, bool PACK>
__device__ __forceinline__ void reg_butterfly(float (&a)[E]) {
    if (!PACK) {
#pragma unroll
        for (int r = 0; r < E; ++r) {
            if ((r & (1 << RB)) == 0) {
                const float u = a[r], w = a[r | (1 << RB)];
                a[r] = u + w;
                a[r | (1 << RB)] = u - w;
            }
        }
    } else if (RB == 0) {
#pragma unroll
        for (int r = 0; r < E; r += 2) {
            const float u = a[r], w = a[r + 1];
            a[r] = u + w;
            a[r + 1] = u - w;
        }
    } else {
#pragma unroll
        for (int r = 0; r < E; r += 2)
            if ((r & (1 << RB)) == 0) bfly2(a[r], a[r + 1], a[r | (1 << RB)], a[(r | (1 << RB)) + 1]);
    }
}

template <int E, int RB, int LOG2E, bool PACK>
struct PhaseA {   // register bit rb <-> index bit rb (rb < 3) or rb + 5 (rb >= 3)
    static __device__ __forceinline__ void run(float (&a)[E], int m) {
        if ((RB < 3 ? RB : RB + 5) < m) reg_butterfly<E, RB, PACK>(a);
        PhaseA<E, RB + 1, LOG2E, PACK>::run(a, m);
    }
};
template <int E, int LOG2E, bool PACK>
struct PhaseA<E, LOG2E, LOG2E, PACK> {
    static __device__ __forceinline__ void run(float (&)[E], int) {}
};

template <int E, int CB, int LOG2V, bool PACK>
struct PhaseB {   // register bit LOG2V + cb <-> index bit 3 + cb, cb < 5
    static __device__ __forceinline__ void run(float (&a)[E], int m) {
        if (3 + CB < m) reg_butterfly<E, LOG2V + CB, PACK>(a);
        PhaseB<E, CB + 1, LOG2V, PACK>::run(a, m);
    }
};
template <int E, int LOG2V, bool PACK>
struct PhaseB<E, 5, LOG2V, PACK> {
    static __device__ __forceinline__ void run(float (&)[E], int) {}
};

// The J pieces of 8 consecutive elements a lane loads of a super-chunk, still in the I/O type: loading them into
// registers ahead of the transform that will use them keeps more global loads in flight per warp.
template <typename T, int J>
struct RawChunk {
    uint4 v[J];
    __device__ __forceinline__ void load(const T* __restrict__ src, int lane) {
#pragma unroll
        for (int j = 0; j < J; ++j) v[j] = *reinterpret_cast<const uint4*>(src + j * 256 + lane * 8);
    }
    template <int E>
    __device__ __forceinline__ void unpack(float (&a)[E]) const {
#pragma unroll
        for (int j = 0; j < J; ++j) {
            float t[8];
            unpack8<T>(v[j], t);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[j * 8 + e] = t[e];
        }
    }
};
template <int J>
struct RawChunk<float, J> {
    float4 v[2 * J];
    __device__ __forceinline__ void load(const float* __restrict__ src, int lane) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
            v[2 * j] = *reinterpret_cast<const float4*>(src + j * 256 + lane * 8);
            v[2 * j + 1] = *reinterpret_cast<const float4*>(src + j * 256 + lane * 8 + 4);
        }
    }
    template <int E>
    __device__ __forceinline__ void unpack(float (&a)[E]) const {
#pragma unroll
        for (int j = 0; j < 2 * J; ++j) {
            a[j * 4] = v[j].x; a[j * 4 + 1] = v[j].y; a[j * 4 + 2] = v[j].z; a[j * 4 + 3] = v[j].w;
        }
    }
};

// Transform the super-chunk held in a[] (lane l: elements j*256 + l*8 .. +7 in a[8j .. 8j+7]); the result is left
// in `wbuf` (this warp's slice) at wphys<>(natural index).
template <int LOGS, bool PACK = false, bool SWZ = false>
__device__ __forceinline__ void warp_transform_loaded(float (&a)[(1 << LOGS) / 32], int m, float* wbuf, int lane) {
    constexpr int S = 1 << LOGS, E = S / 32, LOG2E = LOGS - 5, J = E / 8, V = E / 32, LOG2V = LOG2E - 5;
    PhaseA<E, 0, LOG2E, PACK>::run(a, m);
    // swizzled layout: the XOR only ever takes four values per thread, so four base addresses serve every access
    // (wphys<true>(j * 256 + lane * 8) = j * 256 + ((lane ^ (j & 3)) << 3))
    float* abase[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) abase[k] = wbuf + (SWZ ? ((lane ^ k) << 3) : lane * 8);
#pragma unroll
    for (int j = 0; j < J; ++j) {
        float* p = SWZ ? abase[j & 3] + j * 256 : wbuf + wphys<false>(j * 256 + lane * 8);
        *reinterpret_cast<float4*>(p) = make_float4(a[j * 8], a[j * 8 + 1], a[j * 8 + 2], a[j * 8 + 3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(a[j * 8 + 4], a[j * 8 + 5], a[j * 8 + 6], a[j * 8 + 7]);
    }
    __syncwarp();
    // second mapping: thread-local = bits 3-7 (c) and the lowest LOG2V bits (u); lane = remaining low bits + bits 8+
    constexpr int LOWN = 8 / V;                               // lanes that share a 256-element block differ in the low part
    const int lowpart = lane % LOWN, highpart = lane / LOWN;
    const int off = highpart * 256 + lowpart * V;
    // wphys<true>(off + c * 8) = off + (c >> 2) * 32 + (((c & 3) ^ (highpart & 3)) << 3)
    float* bbase[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) bbase[k] = wbuf + off + ((k ^ (highpart & 3)) << 3);
    float b[E];
#pragma unroll
    for (int c = 0; c < 32; ++c) {
        const float* p = SWZ ? bbase[c & 3] + (c >> 2) * 32 : wbuf + wphys<false>(off + c * 8);
        if (V == 4) {
            const float4 t = *reinterpret_cast<const float4*>(p);
            b[c * 4] = t.x; b[c * 4 + 1] = t.y; b[c * 4 + 2] = t.z; b[c * 4 + 3] = t.w;
        } else if (V == 2) {
            const float2 t = *reinterpret_cast<const float2*>(p);
            b[c * 2] = t.x; b[c * 2 + 1] = t.y;
        } else {
            b[c] = *p;
        }
    }
    PhaseB<E, 0, LOG2V, PACK>::run(b, m);
#pragma unroll
    for (int c = 0; c < 32; ++c) {
        float* p = SWZ ? bbase[c & 3] + (c >> 2) * 32 : wbuf + wphys<false>(off + c * 8);
        if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(b[c * 4], b[c * 4 + 1], b[c * 4 + 2], b[c * 4 + 3]);
        else if (V == 2) *reinterpret_cast<float2*>(p) = make_float2(b[c * 2], b[c * 2 + 1]);
        else *p = b[c];
    }
    __syncwarp();
}

// Transform the super-chunk that starts at element `base` of src (elements at or beyond `total` read as 0).
template <typename T, int LOGS, bool PACK = false, bool SWZ = false>
__device__ __forceinline__ void warp_transform(const T* __restrict__ src, int64_t base, int64_t total, int m,
                                               float* wbuf, int lane) {
    constexpr int S = 1 << LOGS, E = S / 32, J = E / 8;
    float a[E];
#pragma unroll
    for (int j = 0; j < J; ++j) {
        const int idx = j * 256 + lane * 8;
        float v[8];
        if (base + idx + 8 <= total) {
            load8<T>(src + base + idx, v);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = (base + idx + e < total) ? load_as_float<T>(src, base + idx + e) : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) a[j * 8 + e] = v[e];
    }
    warp_transform_loaded<LOGS, PACK, SWZ>(a, m, wbuf, lane);
}

// K == 1: every warp transforms super-chunks independently and writes them back with 16-byte stores.
template <typename T, int LOGS>
__global__ void __launch_bounds__(32 * kWarpsPerCta) fwht_warp_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                      int64_t total, int m, float scale) {
    constexpr int S = 1 << LOGS, E = S / 32, J = E / 8;
    extern __shared__ float wsm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* wbuf = wsm + warp * warp_slice_floats(S);
    const int64_t nsc = (total + S - 1) / S;
    for (int64_t sc = (int64_t)blockIdx.x * kWarpsPerCta + warp; sc < nsc; sc += (int64_t)gridDim.x * kWarpsPerCta) {
        const int64_t base = sc * S;
        warp_transform<T, LOGS>(x, base, total, m, wbuf, lane);
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int idx = j * 256 + lane * 8;
            const float* p = wbuf + wphys<>(idx);
            const float4 t0 = *reinterpret_cast<const float4*>(p);
            const float4 t1 = *reinterpret_cast<const float4*>(p + 4);
            const float v[8] = {t0.x * scale, t0.y * scale, t0.z * scale, t0.w * scale,
                                t1.x * scale, t1.y * scale, t1.z * scale, t1.w * scale};
            if (base + idx + 8 <= total) {
                store8<T>(y + base + idx, v);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (base + idx + e < total) store_from_float<T>(y, base + idx + e, v[e]);
            }
        }
        __syncwarp();
    }
}

// ---- optional fused epilogue: dynamic per-token fake quantization of the rotated row (the activation quantizer
// that follows the online rotation in front of a linear).  The rotated values are first rounded to the I/O type,
// exactly what a separate rotation kernel would have stored, and kept in shared memory; the range (which includes
// 0), scale and zero point then follow the per-token rule in fp32, and the row is written once.
struct RowQuant {
    float clip, maxq;
    int sym;
    float* scale_out;     // [rows] or nullptr
    float* zero_out;      // [rows] or nullptr
};

template <typename T>
__device__ __forceinline__ float round_io(float v);
template <>
__device__ __forceinline__ float round_io<float>(float v) { return v; }
template <>
__device__ __forceinline__ float round_io<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ float round_io<__half>(float v) { return __half2float(__float2half_rn(v)); }

// CTA-wide min / max (every thread calls; red: 64 floats of shared memory), then the row's scale and zero point.
__device__ __forceinline__ void row_quant_params(float lo, float hi, float* red, const RowQuant& q, float& scale,
                                                 float& zero) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane == 0) { red[warp] = lo; red[32 + warp] = hi; }
    __syncthreads();
    lo = red[0]; hi = red[32];
    for (int w = 1; w < nwarps; ++w) { lo = fminf(lo, red[w]); hi = fmaxf(hi, red[32 + w]); }
    float xmin = lo * q.clip, xmax = hi * q.clip;
    zero = 0.f;
    if (q.sym) {
        xmax = fmaxf(fabsf(xmin), xmax);
        scale = (xmax == 0.f) ? 1.f : __fdiv_rn(xmax, q.maxq);
    } else {
        if (xmin == 0.f && xmax == 0.f) { xmin = -1.f; xmax = 1.f; }
        scale = __fdiv_rn(xmax - xmin, q.maxq);
        zero = rintf(__fdiv_rn(-xmin, scale));
    }
}

__device__ __forceinline__ float row_quant_one(float v, float scale, float zero, const RowQuant& q) {
    float c = rintf(__fdiv_rn(v, scale)), r;
    if (q.sym) {
        c = fminf(fmaxf(c, -(q.maxq + 1.f)), q.maxq);
        r = scale * c;
    } else {
        c = fminf(fmaxf(c + zero, 0.f), q.maxq);
        r = scale * (c - zero);
    }
    return (v != v) ? v : r;
}

// Quantize the row held in shared memory as `chunks` slices of S floats (wphys layout) and write it out.
template <typename T, bool SWZ = false>
__device__ __forceinline__ void row_quant_store(const float* wsm, int slice, int S, int chunks, T* yrow, float scale,
                                                float zero, const RowQuant& q) {
    const int n = chunks * S;
    for (int idx = 8 * threadIdx.x; idx < n; idx += 8 * blockDim.x) {
        const int c = idx / S, p = idx - c * S;
        const float* src = wsm + (size_t)c * slice + wphys<SWZ>(p);
        const float4 t0 = *reinterpret_cast<const float4*>(src);
        const float4 t1 = *reinterpret_cast<const float4*>(src + 4);
        const float o[8] = {row_quant_one(t0.x, scale, zero, q), row_quant_one(t0.y, scale, zero, q),
                            row_quant_one(t0.z, scale, zero, q), row_quant_one(t0.w, scale, zero, q),
                            row_quant_one(t1.x, scale, zero, q), row_quant_one(t1.y, scale, zero, q),
                            row_quant_one(t1.z, scale, zero, q), row_quant_one(t1.w, scale, zero, q)};
        store8<T>(yrow + idx, o);
    }
}

// K == 1, chunk length P = W * 1024 with W = 2, 4 or 8: a CTA of W warps owns one chunk.  Every warp transforms
// its 1024-element quarter over index bits 0-9 (32 registers per lane, so many warps stay resident and hide
// the load latency); after a CTA barrier a last radix-W pass over bits 10+ combines the W slices position by
// position and writes the result with 16-byte stores.
template <typename T, int W, bool QUANT = false>
__global__ void __launch_bounds__(32 * W) fwht_split_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                            int64_t nchunks, float scale, RowQuant rq = RowQuant()) {
    constexpr int S = 1024;
    constexpr int slice = warp_slice_floats(S);
    constexpr bool PACK = W <= 4;                               // paired additions (see add2)
    extern __shared__ float wsm[];
    __shared__ float red[64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // every chunk is complete (total = nchunks * W * S), so a warp's quarter is loaded without bounds checks, one
    // grid stride ahead of the transform that consumes it
    RawChunk<T, 4> ahead;
    if ((int64_t)blockIdx.x < nchunks) ahead.load(x + (int64_t)blockIdx.x * (W * S) + (int64_t)warp * S, lane);
    for (int64_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
        const int64_t base = ch * (int64_t)(W * S);
        float a[32];
        ahead.unpack(a);
        if (ch + gridDim.x < nchunks) ahead.load(x + (ch + gridDim.x) * (int64_t)(W * S) + (int64_t)warp * S, lane);
        __syncthreads();                                        // previous chunk fully written out
        warp_transform_loaded<10, PACK>(a, 10, wsm + warp * slice, lane);
        __syncthreads();
        // thread t handles positions 8t .. 8t+7 of every slice (W * 32 threads cover 1024 positions when W = 4;
        // other W loop)
        float lo = 0.f, hi = 0.f;
        for (int p = 8 * threadIdx.x; p < S; p += 8 * 32 * W) {
            float v[W][8];
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const float* q = wsm + w * slice + wphys<>(p);
                const float4 t0 = *reinterpret_cast<const float4*>(q);
                const float4 t1 = *reinterpret_cast<const float4*>(q + 4);
                v[w][0] = t0.x; v[w][1] = t0.y; v[w][2] = t0.z; v[w][3] = t0.w;
                v[w][4] = t1.x; v[w][5] = t1.y; v[w][6] = t1.z; v[w][7] = t1.w;
            }
#pragma unroll
            for (int h = 1; h < W; h <<= 1)
#pragma unroll
                for (int w = 0; w < W; ++w)
                    if ((w & h) == 0) {
                        if (PACK) {
#pragma unroll
                            for (int e = 0; e < 8; e += 2) bfly2(v[w][e], v[w][e + 1], v[w | h][e], v[w | h][e + 1]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const float a = v[w][e], b = v[w | h][e];
                                v[w][e] = a + b;
                                v[w | h][e] = a - b;
                            }
                        }
                    }
#pragma unroll
            for (int w = 0; w < W; ++w) {
                float o[8];
                if (PACK) {
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const float2 t = __fmul2_rn(make_float2(v[w][e], v[w][e + 1]), make_float2(scale, scale));
                        o[e] = t.x;
                        o[e + 1] = t.y;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[e] = v[w][e] * scale;
                }
                if (QUANT) {                                    // back into place, rounded as a store would round
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        o[e] = round_io<T>(o[e]);
                        lo = fminf(lo, o[e]);
                        hi = fmaxf(hi, o[e]);
                    }
                    float* q = wsm + w * slice + wphys<>(p);
                    *reinterpret_cast<float4*>(q) = make_float4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<float4*>(q + 4) = make_float4(o[4], o[5], o[6], o[7]);
                } else {
                    store8<T>(y + base + (int64_t)w * S + p, o);
                }
            }
        }
        if (QUANT) {
            float qs, qz;
            row_quant_params(lo, hi, red, rq, qs, qz);          // its barrier also publishes the rounded row
            if (threadIdx.x == 0) {
                if (rq.scale_out) rq.scale_out[ch] = qs;
                if (rq.zero_out) rq.zero_out[ch] = qz;
            }
            row_quant_store<T>(wsm, slice, S, W, y + base, qs, qz, rq);
        }
    }
}

template <typename T>
__device__ __forceinline__ void store2(T* p, float a, float b);
template <>
__device__ __forceinline__ void store2<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
template <>
__device__ __forceinline__ void store2<__half>(__half* p, float a, float b) {
    *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
}

// two neighbouring positions of every chunk -> K outputs each; hadK entries are +-1, so the products are exact
template <typename T, int KK, bool QUANT = false, bool SWZ = false>
__device__ __forceinline__ void mix_pair(float* buf, int slice, const float* hk, int p, int P, T* yrow,
                                         float scale, int K, float* lo = nullptr, float* hi = nullptr,
                                         bool hk_vec = true) {
    float v0[KK], v1[KK];
#pragma unroll
    for (int k = 0; k < KK; ++k) {
        if (k < K) {
            const float2 t = *reinterpret_cast<const float2*>(buf + k * slice + wphys<SWZ>(p));
            v0[k] = t.x;
            v1[k] = t.y;
        }
    }
    for (int ko = 0; ko < K; ++ko) {
        float s0 = 0.f, s1 = 0.f;
        if ((K & 3) == 0 && hk_vec) {                // rows of hadK as 16-byte words (same address in every lane)
            const float4* hrow = reinterpret_cast<const float4*>(hk + ko * K);
#pragma unroll
            for (int k4 = 0; k4 < KK / 4; ++k4) {
                if (4 * k4 < K) {
                    const float4 h = hrow[k4];
                    s0 = fmaf(h.x, v0[4 * k4 + 0], s0); s1 = fmaf(h.x, v1[4 * k4 + 0], s1);
                    s0 = fmaf(h.y, v0[4 * k4 + 1], s0); s1 = fmaf(h.y, v1[4 * k4 + 1], s1);
                    s0 = fmaf(h.z, v0[4 * k4 + 2], s0); s1 = fmaf(h.z, v1[4 * k4 + 2], s1);
                    s0 = fmaf(h.w, v0[4 * k4 + 3], s0); s1 = fmaf(h.w, v1[4 * k4 + 3], s1);
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < KK; ++k) {
                if (k < K) {
                    const float h = hk[ko * K + k];
                    s0 = fmaf(h, v0[k], s0);
                    s1 = fmaf(h, v1[k], s1);
                }
            }
        }
        if (QUANT) {                                 // every input of this position pair is already in registers
            const float r0 = round_io<T>(s0 * scale), r1 = round_io<T>(s1 * scale);
            *lo = fminf(*lo, fminf(r0, r1));
            *hi = fmaxf(*hi, fmaxf(r0, r1));
            *reinterpret_cast<float2*>(buf + ko * slice + wphys<SWZ>(p)) = make_float2(r0, r1);
        } else {
            store2<T>(yrow + (int64_t)ko * P + p, s0 * scale, s1 * scale);
        }
    }
}

// The mix for the tabulated matrices of order 12, 20 and 28, with the signs known at compile time.  A generic
// +-1 matrix costs K multiply-adds per output.  Here the K inputs are taken four at a time: the eight values
// (a +- b) +- (c +- d) a quad can contribute (up to an overall sign) cost 12 additions, after which every output is
// one signed term per quad: 12 * K/4 + K * (K/4 - 1) additions per position instead of K * K multiply-adds
// (60 instead of 144 at K = 12, 252 instead of 784 at K = 28).  The sums are the same fp32 additions of the same
// exact +-v terms, associated quad by quad.  Combinations no row uses are never computed (their indices are
// constants after unrolling).
template <int K>
__device__ __forceinline__ void mix_fixed(const float (&v)[K], float (&y)[K]) {
    constexpr int NQ = K / 4;
#pragma unroll
    for (int q = 0; q < NQ; ++q) {              // quad by quad, so that a quad's inputs and combinations die early
        const float ab0 = v[4 * q] + v[4 * q + 1], ab1 = v[4 * q] - v[4 * q + 1];
        const float cd0 = v[4 * q + 2] + v[4 * q + 3], cd1 = v[4 * q + 2] - v[4 * q + 3];
        const float c[8] = {ab0 + cd0, ab1 + cd0, ab0 - cd0, ab1 - cd0, ab0 + cd1, ab1 + cd1, ab0 - cd1, ab1 - cd1};
#pragma unroll
        for (int r = 0; r < K; ++r) {
            const uint32_t bits = (had_row<K>(r) >> (4 * q)) & 15u;
            const bool s0 = bits & 1u, s1 = bits & 2u, s2 = bits & 4u, s3 = bits & 8u;
            const int idx = (s1 != s0 ? 1 : 0) | (s2 != s0 ? 2 : 0) | (s3 != s2 ? 4 : 0);
            const float t = c[idx];
            y[r] = (q == 0) ? (s0 ? t : -t) : (s0 ? y[r] + t : y[r] - t);
        }
    }
}

// the same mix on two neighbouring positions at once (.x and .y), every addition as one paired instruction; the
// inputs are chunk k of this position pair at src + k * slice
template <int K>
__device__ __forceinline__ void mix_fixed2(const float* __restrict__ src, int slice, float2 (&y)[K]) {
    constexpr int NQ = K / 4;
    float2 v[K];
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = *reinterpret_cast<const float2*>(src + k * slice);
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        const int b = 4 * q;
        const float2 ab0 = add2(v[b], v[b + 1]), ab1 = sub2(v[b], v[b + 1]);
        const float2 cd0 = add2(v[b + 2], v[b + 3]), cd1 = sub2(v[b + 2], v[b + 3]);
        const float2 c[8] = {add2(ab0, cd0), add2(ab1, cd0), sub2(ab0, cd0), sub2(ab1, cd0),
                             add2(ab0, cd1), add2(ab1, cd1), sub2(ab0, cd1), sub2(ab1, cd1)};
#pragma unroll
        for (int r = 0; r < K; ++r) {
            const uint32_t bits = (had_row<K>(r) >> (4 * q)) & 15u;
            const bool s0 = bits & 1u, s1 = bits & 2u, s2 = bits & 4u, s3 = bits & 8u;
            const int idx = (s1 != s0 ? 1 : 0) | (s2 != s0 ? 2 : 0) | (s3 != s2 ? 4 : 0);
            const float2 t = c[idx];
            y[r] = (q == 0) ? (s0 ? t : make_float2(-t.x, -t.y)) : (s0 ? add2(y[r], t) : sub2(y[r], t));
        }
    }
}

// true in every thread when the K x K matrix at hk is the tabulated one of that order
template <int K>
__device__ __forceinline__ bool matches_table(const float* hk) {
    uint32_t tab[K];
#pragma unroll
    for (int r = 0; r < K; ++r) tab[r] = had_row<K>(r);
    bool ok = true;
    for (int e = threadIdx.x; e < K * K; e += blockDim.x) {
        const int r = e / K, col = e - r * K;
        ok = ok && hk[e] == (((tab[r] >> col) & 1u) ? 1.f : -1.f);
    }
    return __syncthreads_and(ok) != 0;
}

// two neighbouring positions of every chunk through mix_fixed, stored as pairs (QUANT: rounded to the I/O type and
// put back into shared memory, min / max tracked, as mix_pair does)
template <typename T, int K, bool QUANT, bool SWZ = false>
__device__ __forceinline__ void mix_pair_fixed(float* buf, int slice, int p, int P, T* yrow, float scale, float* lo,
                                               float* hi) {
    float2 y[K];
    const float* src = buf + wphys<SWZ>(p);
    mix_fixed2<K>(src, slice, y);
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const float2 o = __fmul2_rn(y[k], make_float2(scale, scale));
        if (QUANT) {
            const float r0 = round_io<T>(o.x), r1 = round_io<T>(o.y);
            *lo = fminf(*lo, fminf(r0, r1));
            *hi = fmaxf(*hi, fmaxf(r0, r1));
            *reinterpret_cast<float2*>(buf + k * slice + wphys<SWZ>(p)) = make_float2(r0, r1);
        } else {
            store2<T>(yrow + (int64_t)k * P + p, o.x, o.y);
        }
    }
}

// one position of every chunk through mix_fixed (scalar additions; lanes take consecutive positions, so a warp
// still writes 64 contiguous bytes per output chunk); used at K = 28, where the paired form does not fit the registers.
template <typename T, int K, bool QUANT, bool SWZ = false>
__device__ __forceinline__ void mix_one_fixed(float* buf, int slice, int p, int P, T* yrow, float scale, float* lo,
                                              float* hi) {
    float v[K], y[K];
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = buf[k * slice + wphys<SWZ>(p)];
    mix_fixed<K>(v, y);
#pragma unroll
    for (int k = 0; k < K; ++k) {
        if (QUANT) {
            const float r = round_io<T>(y[k] * scale);
            *lo = fminf(*lo, r);
            *hi = fmaxf(*hi, r);
            buf[k * slice + wphys<SWZ>(p)] = r;
        } else {
            store_from_float<T>(yrow, (int64_t)k * P + p, y[k] * scale);
        }
    }
}

// K > 1 with chunk length P = S: one CTA per row; warps transform the K chunks into shared memory, then
// all threads mix the chunks position by position.
// KMAX bounds K at compile time: the kernel for K <= 12 holds 24 instead of 56 chunk values per thread during the mix,
// so that four CTAs instead of two share an SM's registers; it runs with 6 warps, which take the 12 chunks of a
// 12288-long row in two full rounds (measured on 65536 x 12288 bf16: 8 warps and two CTAs per SM 1.98 TB/s, 8 warps
// and four CTAs 2.36, 4 warps 2.43, 6 warps 2.68).
#ifndef RQ_MIX12_WARPS
#define RQ_MIX12_WARPS 6
#endif
// Larger K: 8 warps and two CTAs per SM (28 unpadded slices of 4 KB are 112 KB, so two rows fit an SM's shared
// memory; 128 registers per thread), so that one CTA's load-bound transform phase overlaps the other's issue-bound
// mix.  Measured (bf16, 16384 rows, GB/s of read + write): n = 28672 one CTA of 16 warps 2779, two of 8 warps 3031,
// with paired additions in the transform 3093; n = 20480 2695 -> 3010.  At K = 28 the mix itself stays scalar, one
// position per thread: the paired form needs 56 two-wide sums (spills at 128 registers: 2655), and in two halves
// of 14 outputs with the inputs read twice it reaches 2991.
#ifndef RQ_MIX28_WARPS
#define RQ_MIX28_WARPS 8
#endif
#ifndef RQ_MIX28_PACK
#define RQ_MIX28_PACK 1
#endif
template <typename T, int LOGS, bool QUANT = false, int KMAX = 28, int WARPS = kMixWarps>
__global__ void __launch_bounds__(32 * WARPS, (LOGS != 10 || QUANT) ? 1 : (KMAX <= 12 ? 4 : (WARPS <= 8 ? 2 : 1))) fwht_mix_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                     int64_t rows, int K,
                                                                     const float* __restrict__ hadK, float scale,
                                                                     RowQuant rq = RowQuant()) {
    constexpr int S = 1 << LOGS;
    constexpr bool SWZ = mix_swizzled(LOGS, KMAX, QUANT);
    constexpr int slice = warp_slice_floats(S, SWZ);
    constexpr bool PACK = LOGS == 10 && (KMAX <= 12 || RQ_MIX28_PACK);   // paired additions (see add2)
    extern __shared__ float wsm[];
    __shared__ float red[64];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the caller's matrix sits behind the slices in shared memory, except where that would cost the second CTA of an
    // SM (K > kMixSharedMatrixMaxK at S = 1024): there the tabulated matrices need no copy and any other matrix is
    // read in place, entry by entry
    const bool hk_shared = mix_matrix_shared(K, SWZ);
    const float* hk = hadK;
    if (hk_shared) {
        float* hs = wsm + (size_t)K * slice;
        for (int e = threadIdx.x; e < K * K; e += blockDim.x) hs[e] = hadK[e];
        hk = hs;
        __syncthreads();
    }
    // 0: the caller's matrix, entry by entry; 12 / 20 / 28: the tabulated matrix of that order (uniform over the CTA)
    int fixed = 0;
    if (K == 12) fixed = matches_table<12>(hk) ? 12 : 0;
    else if (KMAX > 12 && K == 20) fixed = matches_table<20>(hk) ? 20 : 0;
    else if (KMAX > 12 && K == 28) fixed = matches_table<28>(hk) ? 28 : 0;
    const int64_t n = (int64_t)K * S;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        __syncthreads();                                        // previous row's mix has finished reading
        if (LOGS == 10 && sizeof(T) == 2 && KMAX > 12) {
            // rows are complete: a warp issues the loads of its next two chunks before it transforms the first
            // (bf16, n = 28672: 2.53 -> 2.77 TB/s; the 12-chunk kernel, short of registers, lost with it: 3.99 -> 3.69)
            for (int c = warp; c < K; c += 2 * WARPS) {
                RawChunk<T, (1 << LOGS) / 256> r0, r1;
                const bool two = c + WARPS < K;
                r0.load(x + row * n + (int64_t)c * S, lane);
                if (two) r1.load(x + row * n + (int64_t)(c + WARPS) * S, lane);
                float a[(1 << LOGS) / 32];
                r0.unpack(a);
                warp_transform_loaded<LOGS, PACK, SWZ>(a, LOGS, wsm + (size_t)c * slice, lane);
                if (two) {
                    r1.unpack(a);
                    warp_transform_loaded<LOGS, PACK, SWZ>(a, LOGS, wsm + (size_t)(c + WARPS) * slice, lane);
                }
            }
        } else {
            for (int c = warp; c < K; c += WARPS)
                warp_transform<T, LOGS, PACK, SWZ>(x, row * n + (int64_t)c * S, (rows * n), LOGS, wsm + (size_t)c * slice,
                                              lane);
        }
        __syncthreads();
        T* yrow = y + row * n;
        float lo = 0.f, hi = 0.f;
        if (KMAX > 12 && fixed == 28) {
            for (int p = threadIdx.x; p < S; p += blockDim.x)
                mix_one_fixed<T, 28, QUANT, SWZ>(wsm, slice, p, S, yrow, scale, &lo, &hi);
        } else
        for (int p = 2 * threadIdx.x; p < S; p += 2 * blockDim.x) {
            if (fixed == 12) {
                mix_pair_fixed<T, 12, QUANT, SWZ>(wsm, slice, p, S, yrow, scale, &lo, &hi);
            } else if (KMAX > 12 && fixed == 20) {
                mix_pair_fixed<T, 20, QUANT, SWZ>(wsm, slice, p, S, yrow, scale, &lo, &hi);
            } else if (KMAX <= 12 || K <= 12) {
                mix_pair<T, 12, QUANT, SWZ>(wsm, slice, hk, p, S, yrow, scale, K, &lo, &hi, hk_shared);
            } else if (KMAX > 12) {
                if (K <= 20) mix_pair<T, 20, QUANT, SWZ>(wsm, slice, hk, p, S, yrow, scale, K, &lo, &hi, hk_shared);
                else mix_pair<T, 28, QUANT, SWZ>(wsm, slice, hk, p, S, yrow, scale, K, &lo, &hi, hk_shared);
            }
        }
        if (QUANT) {
            float qs, qz;
            row_quant_params(lo, hi, red, rq, qs, qz);          // its barrier also publishes the rounded row
            if (threadIdx.x == 0) {
                if (rq.scale_out) rq.scale_out[row] = qs;
                if (rq.zero_out) rq.zero_out[row] = qz;
            }
            row_quant_store<T, SWZ>(wsm, slice, S, K, yrow, qs, qz, rq);
        }
    }
}

}  // namespace fwht
}  // namespace rq
