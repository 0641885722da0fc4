// Saliency-weighted Hessian accumulation  H[g] = beta*H[g] + alpha * X^T diag(s_g) X  on the
// 5th-generation tensor cores (tcgen05 + tensor memory), fed by TMA.
//
// The contraction runs on fp16 operand planes.  fp16 carries 11 significant bits per plane (bf16: 8), so a value
// split into hi + lo keeps 22 bits, within two bits of fp32, where two bf16 planes keep 16; what fp16 lacks is
// exponent range, and that is supplied by exact power-of-two scalings chosen per chunk of tokens:
//   * per saliency group g:  s' = s * 2^-c_g  brings the chunk's largest saliency of the group into [1, 2);
//   * per token t:           X' = x * 2^a_t,  Y'_g = (s'_g * x) * 2^(E - a_t):  every product x'_i * y'_j equals
//     s' x_i x_j * 2^E whatever a_t is, so a_t is free to balance the two operands of the token, and the global E
//     puts the chunk's largest token just under the top of fp16's range.  With P_t = max_g s'_tg * (max_c |x_tc|)^2:
//     E = 28 - floor(log2 max_t P_t),  a_t = floor((floor(log2 max_g s'_tg) + E) / 2), which gives
//     max |x'_t| < 2^14.5 and max |y'_t| < 2^15.5 for every token.
//   The epilogue multiplies the sums by 2^(c_g - E).  Tokens that weigh little in H (small P_t) sit lower in the
//   format and lose relative precision in proportion to how little they contribute.
//
// Per chunk:
//   1. group_scale (one block) and token_stats (a warp per token, one extra read of X): c_g, then per token
//      max_c |x| and max_g s', and the chunk's largest P_t.
//   2. pack:  reads X (fp32 / bf16 / fp16) and the saliency once, and writes token-contiguous ("K-major") fp16
//             planes  X' (one plane for bf16 / fp16 input, whose 8 / 11 significant bits fit; hi and lo for fp32
//             input)  and  Y'_g hi, lo  per group; also the per-channel sum of squares.
//   3. umma:  persistent, warp-specialised GEMM over the upper-triangular 128x256 tiles of every H[g]:
//             D = X'.Y'_lo^T + X'.Y'_hi^T  (bf16 / fp16 input)  or  X'_lo.Y'_hi^T + X'_hi.Y'_lo^T + X'_hi.Y'_hi^T
//             (fp32 input; the lo.lo term, 2^-22, is dropped), every product exact in fp32, accumulated in
//             tensor memory over windows of 128 tokens; the epilogue warps sum the windows in registers with
//             round-to-nearest adds (the tensor core's own accumulation truncates toward zero and would drift
//             by ~4e-8 per MMA; measured: 5e-5 over 8192 tokens, and the same with the operand sign flipped)
//             and add the tile into H at the end.
#include <cuda.h>

#include "rq_common.cuh"
#include "rq_sm100.cuh"

namespace rq {
namespace hess {

using namespace rq::sm100;

constexpr int BM = 128;          // tile rows   (channels i)   = UMMA M
constexpr int BN = 256;          // tile cols   (channels j)   = UMMA N
constexpr int UK = 16;           // 16-bit UMMA K
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;   // warp 0: TMA producer, warp 1: MMA issuer, warps 2-9: epilogue
constexpr int kTmemCols = 512;   // two 128x256 fp32 accumulators
constexpr int kWindowTokens = 128;   // tokens accumulated on the tensor core before a round-to-nearest add (default)
constexpr int kTopExp = 28;      // 2^E * (largest P_t of the chunk) lands in [2^28, 2^29)

// NX = number of fp16 planes of X' (1 for bf16 / fp16 input, 2 for fp32 input); Y' always has two.
template <int BK, int NX, bool WIDE_Y = false>
struct Cfg {
    static constexpr int kLayout = BK == 64 ? 2 : 4;              // UMMA swizzle mode: 128 B / 64 B
    static constexpr int kSBO = 8 * BK * 2;                        // bytes between 8-row groups
    static constexpr int kATile = BM * BK * 2;
    static constexpr int kBTile = BN * BK * 2;
    // NX == 2:  A side (128 rows) = X' hi, lo;  B side (256 rows) = Y' hi, lo.
    // NX == 1:  the two-plane operand Y' goes on the narrow A side and the single plane X' on the wide B side,
    // 64 KB per stage instead of 80 KB: less L2->SM traffic per MMA and room for a third stage.
    // WIDE_Y keeps Y' on the wide side also for NX == 1 (80 KB per stage), for comparison.
    static constexpr bool kSwap = NX == 1 && !WIDE_Y;
    static constexpr int kAPlanes = kSwap ? 2 : NX;
    static constexpr int kBPlanes = kSwap ? 1 : 2;
    static constexpr int kStageBytes = kAPlanes * kATile + kBPlanes * kBTile;
    static constexpr int kStages = (200 * 1024) / kStageBytes;
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;   // +1024: alignment slack
    static_assert(kStages >= 2, "the ring needs two stages");
    // products of a k-step as (X' plane, Y' plane), smallest terms first
    static constexpr int kProducts = NX == 1 ? 2 : 3;
};
__device__ constexpr int kProdX[2][3] = {{0, 0, 0}, {1, 0, 0}};
__device__ constexpr int kProdY[2][3] = {{1, 0, 0}, {0, 1, 0}};

// ------------------------------------------------------------------------------------------
// scales.  `aux` (16 floats per chunk slot): [0..7] 2^-c_g, [8..15] 2^c_g; `pmax`: bit pattern of max_t P_t.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ bool finite_pos(float v) { return v > 0.f && v <= 3.0e38f; }

// c_g = floor(log2(max_t |s[t, g]|)) over the chunk (0 when the group has no positive finite saliency, or when
// there is no saliency at all).  One block; also clears pmax.
__global__ void __launch_bounds__(1024) group_scale_kernel(const float* __restrict__ sal, int nvalid, int G,
                                                           float* __restrict__ aux, unsigned int* __restrict__ pmax) {
    __shared__ float red[32][8];
    float m[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) m[g] = 0.f;
    if (sal != nullptr) {
        for (int t = threadIdx.x; t < nvalid; t += 1024) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if (g < G) {
                    const float v = fabsf(sal[(int64_t)t * G + g]);
                    if (v > m[g] && v <= 3.0e38f) m[g] = v;             // skips NaN and Inf
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m[g] = fmaxf(m[g], __shfl_xor_sync(0xffffffffu, m[g], o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5][g] = m[g];
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        float v = 0.f;
        for (int w = 0; w < 32; ++w) v = fmaxf(v, red[w][threadIdx.x]);
        int c = (sal != nullptr && v > 0.f) ? ilogbf(v) : 0;
        c = c < -100 ? -100 : (c > 100 ? 100 : c);
        aux[threadIdx.x] = exp2f((float)-c);
        aux[8 + threadIdx.x] = exp2f((float)c);
    }
    if (threadIdx.x == 0) *pmax = 0u;
}

// tok[t] = (max_g s'_tg, max_c |x_tc|), both 0 for padding tokens and for tokens that carry a non-finite value;
// pmax = bit pattern of the largest P_t = tok.x * tok.y^2 (positive floats order like their bit patterns).
// One warp per token.
template <typename T>
__global__ void __launch_bounds__(256) token_stats_kernel(const T* __restrict__ x, int64_t ldx,
                                                          const float* __restrict__ sal, const float* __restrict__ aux,
                                                          int nvalid, int Kc, int C, int G, float2* __restrict__ tok,
                                                          unsigned int* __restrict__ pmax) {
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= Kc) return;
    float m = 0.f;
    bool finite = true;
    if (t < nvalid) {
        const T* row = x + (int64_t)t * ldx;
        const bool vec = (ldx * (int64_t)sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
        constexpr int PER = 16 / (int)sizeof(T);
        const int nvec = vec ? C / PER : 0;
        const uint4* r4 = reinterpret_cast<const uint4*>(row);
        for (int i = lane; i < nvec; i += 32) {
            const uint4 w = r4[i];
            const T* h = reinterpret_cast<const T*>(&w);
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const float a = fabsf(load_as_float<T>(h, e));
                finite = finite && a <= 3.0e38f;
                m = fmaxf(m, a);
            }
        }
        for (int c = nvec * PER + lane; c < C; c += 32) {
            const float a = fabsf(load_as_float<T>(row, c));
            finite = finite && a <= 3.0e38f;
            m = fmaxf(m, a);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    finite = __all_sync(0xffffffffu, finite);
    if (lane == 0) {
        float smax = t < nvalid ? 1.f : 0.f;
        if (sal != nullptr && t < nvalid) {
            smax = 0.f;
            for (int g = 0; g < G; ++g) {
                const float v = fabsf(sal[(int64_t)t * G + g]) * aux[g];
                if (!(v <= 3.0e38f)) finite = false;
                smax = fmaxf(smax, v);
            }
        }
        const float p = smax * m * m;
        if (finite && finite_pos(p)) {
            tok[t] = make_float2(smax, m);
            atomicMax(pmax, __float_as_uint(p));
        } else {
            tok[t] = make_float2(0.f, 0.f);
        }
    }
}

// E of the chunk and the factor 2^-E the epilogue needs (clamped so that both stay ordinary floats).
__device__ __forceinline__ int chunk_exponent(unsigned int pmax_bits) {
    const float pm = __uint_as_float(pmax_bits);
    int e = finite_pos(pm) ? kTopExp - ilogbf(pm) : 0;
    return e < -60 ? -60 : (e > 60 ? 60 : e);
}

// (2^a_t, 2^(E - a_t)) of a token; (1, 2^E) for a token without a usable magnitude.
__device__ __forceinline__ float2 token_scales(float2 tk, int E) {
    int a = 0;
    if (finite_pos(tk.x)) {
        const int u = ilogbf(tk.x) + E;
        a = (u >= 0) ? (u >> 1) : -((1 - u) >> 1);            // floor(u / 2)
    }
    a = a < -100 ? -100 : (a > 100 ? 100 : a);
    return make_float2(exp2f((float)a), exp2f((float)(E - a)));
}

// ------------------------------------------------------------------------------------------
// pack
// ------------------------------------------------------------------------------------------
// (a, b) -> packed fp16 pair (one conversion instruction), a in the low half
__device__ __forceinline__ uint32_t pair_f16(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// hi = fp16(a, b) packed, (la, lb) = what the rounding left over (exact in fp32)
__device__ __forceinline__ uint32_t split_pair_f16(float a, float b, float& la, float& lb) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 f = __half22float2(h);
    la = a - f.x;
    lb = b - f.y;
    return *reinterpret_cast<const uint32_t*>(&h);
}

// grid (ceil(Kc/128), ceil(C/32)), 256 threads: a block packs 128 tokens x 32 channels; token tiles vary fastest,
// so that concurrently running blocks extend the same plane rows.  A lane owns four consecutive tokens: it reads
// them from the channel-major shared tile as one 16-byte word and writes four fp16 values per plane as one 8-byte
// word, 256 contiguous bytes per (plane, channel) and warp.
// planes: [NX + 2G][C][Kc] fp16: X' (hi[, lo]) then per group Y' (hi, lo).
// partial: [ceil(Kc/128)][C] per-tile sums of x^2 (may be NULL).
constexpr int kPackTokens = 128, kPackChannels = 32;

template <typename T, int NX>
__global__ void __launch_bounds__(256) pack_kernel(const T* __restrict__ x, int64_t ldx,
                                                   const float* __restrict__ sal, const float* __restrict__ aux,
                                                   const float2* __restrict__ tok, const unsigned int* __restrict__ pmax,
                                                   int nvalid, int C, int G, int Kc, uint16_t* __restrict__ planes,
                                                   float* __restrict__ partial) {
    __shared__ __align__(16) float xs[kPackChannels][kPackTokens + 4];
    __shared__ __align__(16) float ss[8][kPackTokens];         // saliencies, group-major
    __shared__ __align__(16) float sx[kPackTokens];            // 2^a_t
    __shared__ __align__(16) float sy[kPackTokens];            // 2^(E - a_t)
    const int t0 = blockIdx.x * kPackTokens;
    const int c0 = blockIdx.y * kPackChannels;
    const int tid = threadIdx.x;
    {   // load: 32 consecutive channels of one token per warp, eight tokens per pass; all sixteen loads of a thread
        // are issued before the first is consumed
        const int cc = tid & 31, tr = tid >> 5;
        float v[16];
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            const int t = p * 8 + tr;
            v[p] = (t0 + t < nvalid && c0 + cc < C) ? load_as_float<T>(x, (int64_t)(t0 + t) * ldx + c0 + cc) : 0.f;
        }
#pragma unroll
        for (int p = 0; p < 16; ++p) xs[cc][p * 8 + tr] = v[p];
        for (int e = tid; e < 8 * kPackTokens; e += 256) {
            const int g = e >> 7, t = e & (kPackTokens - 1);
            float sv = 0.f;
            if (g < G && t0 + t < nvalid) sv = (sal != nullptr) ? sal[(int64_t)(t0 + t) * G + g] : 1.f;
            ss[g][t] = sv;
        }
        if (tid < kPackTokens) {
            const int E = chunk_exponent(*pmax);
            const float2 tk = (t0 + tid < Kc) ? tok[t0 + tid] : make_float2(0.f, 0.f);
            const float2 sc = token_scales(tk, E);
            sx[tid] = sc.x;
            sy[tid] = sc.y;
        }
    }
    __syncthreads();

    const int warp = tid >> 5, lane = tid & 31;
    const int64_t plane_stride = (int64_t)C * Kc;
    const int ta = 4 * lane;
    const bool in_range = t0 + ta < Kc;                        // Kc is a multiple of 64: a group of four never straddles
    const float4 ax = *reinterpret_cast<const float4*>(&sx[ta]);
    const float4 ay = *reinterpret_cast<const float4*>(&sy[ta]);
    float gn[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) gn[g] = g < G ? aux[g] : 0.f;
    for (int cc = warp; cc < kPackChannels; cc += 8) {
        const int c = c0 + cc;
        if (c >= C) break;                                     // warp-uniform
        const float4 xv = *reinterpret_cast<const float4*>(&xs[cc][ta]);
        const int64_t off = (int64_t)c * Kc + t0 + ta;          // multiple of 4 elements: 8-byte aligned
        if (in_range) {
            float l0, l1, l2, l3;
            uint2 hi;
            hi.x = split_pair_f16(xv.x * ax.x, xv.y * ax.y, l0, l1);        // exact scalings: powers of two
            hi.y = split_pair_f16(xv.z * ax.z, xv.w * ax.w, l2, l3);
            *reinterpret_cast<uint2*>(planes + off) = hi;
            if (NX == 2) *reinterpret_cast<uint2*>(planes + plane_stride + off) = make_uint2(pair_f16(l0, l1), pair_f16(l2, l3));
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if (g >= G) break;
                const float4 sg = *reinterpret_cast<const float4*>(&ss[g][ta]);
                // the reference's fp32 product x * s, then the exact scaling
                const float y0 = __fmul_rn(xv.x, sg.x) * (ay.x * gn[g]);
                const float y1 = __fmul_rn(xv.y, sg.y) * (ay.y * gn[g]);
                const float y2 = __fmul_rn(xv.z, sg.z) * (ay.z * gn[g]);
                const float y3 = __fmul_rn(xv.w, sg.w) * (ay.w * gn[g]);
                uint2 yh;
                yh.x = split_pair_f16(y0, y1, l0, l1);
                yh.y = split_pair_f16(y2, y3, l2, l3);
                *reinterpret_cast<uint2*>(planes + (NX + 2 * g) * plane_stride + off) = yh;
                *reinterpret_cast<uint2*>(planes + (NX + 2 * g + 1) * plane_stride + off) =
                    make_uint2(pair_f16(l0, l1), pair_f16(l2, l3));
            }
        }
        if (partial != nullptr) {
            float sq = (xv.x * xv.x + xv.y * xv.y) + (xv.z * xv.z + xv.w * xv.w);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) partial[(int64_t)blockIdx.x * C + c] = sq;
        }
    }
}

// act_sq[c] += sum over token tiles, in tile order (deterministic).
__global__ void act_reduce_kernel(const float* __restrict__ partial, int ntiles, int C, float* __restrict__ act_sq) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float s = 0.f;
    for (int t = 0; t < ntiles; ++t) s += partial[(int64_t)t * C + c];
    act_sq[c] += s;
}

// ------------------------------------------------------------------------------------------
// tile schedule: upper-triangular 128x256 tiles.  Column block j (256 wide) needs row blocks
// i = 0 .. min(MT-1, 2j+1).  Linear index u -> (i, j) with cum(j) = j*(j+1).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void decode_tile(int u, int& i, int& j) {
    int jj = static_cast<int>((sqrtf(4.f * static_cast<float>(u) + 1.f) - 1.f) * 0.5f);
    while ((jj + 1) * (jj + 2) <= u) ++jj;
    while (jj * (jj + 1) > u) --jj;
    j = jj;
    i = u - jj * (jj + 1);
}

// Tile order of one launch.  Concurrently running CTAs take consecutive indices, so the order decides what
// they share in L2.  The operand that depends on the group (Y_g) is the expensive one: no two groups share it.
//   Y on the 256-wide side: group fastest, then row block i inside column block j (CTAs share X_hi[i] across
//     groups and Y_g[j] across the i of a column block);
//   Y on the 128-row side (bf16 X): row-major, all column blocks j of one (i, g) consecutively, so the CTAs of
//     a wave share a handful of Y_g[i] row blocks and stream the X_hi plane once.
template <bool ROW_MAJOR>
__device__ __forceinline__ void decode_work(int t, int G, int NT, int& g, int& i, int& j) {
    if (ROW_MAJOR) {
        int rem = t;
        i = 0;
        for (;;) {
            const int cnt = G * (NT - (i >> 1));
            if (rem < cnt) break;
            rem -= cnt;
            ++i;
        }
        const int per = NT - (i >> 1);
        g = rem / per;
        j = (i >> 1) + (rem - g * per);
    } else {
        g = t % G;
        decode_tile(t / G, i, j);
    }
}

struct Bars {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t tfull[2];
    uint64_t tempty[2];
    uint32_t tmem_slot;
    int abort_flag;
};
static_assert(sizeof(Bars) <= 256, "barrier block");

// x_plane0 / y_plane0: index of the first X' plane and of group 0's first Y' plane in the plane tensor.
// aux / pmax: the chunk's group scales and largest P_t (see the scales section); the sums leave as
// alpha * 2^(c_g - E) * D.
template <int BK, int NX, bool WIDE_Y>
__global__ void __launch_bounds__(kThreads, 1)
umma_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
            float* __restrict__ H, int C, int G, int MT, int NT, int kblocks, int x_plane0, int y_plane0,
            float alpha, float beta, const float* __restrict__ aux, const unsigned int* __restrict__ pmax,
            int win_blocks, int* __restrict__ status) {
    using K = Cfg<BK, NX, WIDE_Y>;
    const int WIN = win_blocks;                                          // k-blocks per accumulation window
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;                       // shared-space address of stage 0
    Bars* bars = reinterpret_cast<Bars*>(smem_raw + (tiles - raw) + K::kStages * K::kStageBytes);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_per_group = (NT - 1) * NT + MT;
    const int total_tiles = tiles_per_group * G;

    if (threadIdx.x == 0) {
        for (int s = 0; s < K::kStages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->tfull[a]), 1);
            mbar_init(smem_u32(&bars->tempty[a]), kEpilogueWarps);
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&mapA);
        tma_prefetch_desc(&mapB);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&bars->tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                int g, i, j;
                decode_work<K::kSwap>(t, G, NT, g, i, j);
                // A side: 128 rows of block i; B side: 256 rows of block j
                const int a_first = K::kSwap ? y_plane0 + 2 * g : x_plane0;
                const int b_first = K::kSwap ? x_plane0 : y_plane0 + 2 * g;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const uint32_t s = it % K::kStages;
                    const uint32_t ph = (it / K::kStages) & 1u;
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t fb = smem_u32(&bars->full[s]);
                    const uint32_t dst = tiles + s * K::kStageBytes;
                    mbar_expect_tx(fb, K::kStageBytes);
#pragma unroll
                    for (int pl = 0; pl < K::kAPlanes; ++pl)
                        tma_load_3d(dst + pl * K::kATile, &mapA, fb, kb * BK, i * BM, a_first + pl);
#pragma unroll
                    for (int pl = 0; pl < K::kBPlanes; ++pl)
                        tma_load_3d(dst + K::kAPlanes * K::kATile + pl * K::kBTile, &mapB, fb, kb * BK, j * BN, b_first + pl);
                }
            }
            if (!ok) {
                // Another role gave up: let the copies already issued land before the CTA exits.
                const uint32_t inflight = it < (uint32_t)K::kStages ? it : (uint32_t)K::kStages;
                for (uint32_t b = 0; b < inflight; ++b) {
                    const uint32_t q = it - 1 - b;
                    const uint32_t fb = smem_u32(&bars->full[q % K::kStages]);
                    const long long t0 = clock64();
                    while (!mbar_try_wait(fb, (q / K::kStages) & 1u) && clock64() - t0 < kWaitCycles) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16_f32(BM, BN);      // fp16 x fp16 -> fp32
            uint32_t it = 0, win_iter = 0;
            bool ok = true;
            const int nwin = (kblocks + WIN - 1) / WIN;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                for (int w = 0; w < nwin && ok; ++w, ++win_iter) {
                    const uint32_t acc = win_iter & 1u;
                    const uint32_t acc_ph = (win_iter >> 1) & 1u;
                    if (!mbar_wait(smem_u32(&bars->tempty[acc]), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    const int kb_begin = w * WIN;
                    const int kb_end = (kb_begin + WIN < kblocks) ? kb_begin + WIN : kblocks;
                    for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                        const uint32_t s = it % K::kStages;
                        const uint32_t ph = (it / K::kStages) & 1u;
                        if (!mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_base = tiles + s * K::kStageBytes;
                        const uint32_t b_base = a_base + K::kAPlanes * K::kATile;
#pragma unroll
                        for (int k = 0; k < BK / UK; ++k) {
                            const uint32_t koff = k * UK * 2;           // bytes along K inside the swizzle row
#pragma unroll
                            for (int pr = 0; pr < K::kProducts; ++pr) {
                                const int px = kProdX[NX - 1][pr], py = kProdY[NX - 1][pr];
                                const int pa = K::kSwap ? py : px, pb = K::kSwap ? px : py;
                                const uint64_t da = umma_smem_desc(a_base + pa * K::kATile + koff, K::kSBO, K::kLayout);
                                const uint64_t db = umma_smem_desc(b_base + pb * K::kBTile + koff, K::kSBO, K::kLayout);
                                // the first MMA of a window overwrites the accumulator; small terms go first
                                umma_bf16(d_tmem, da, db, idesc, (kb != kb_begin || k != 0 || pr != 0) ? 1u : 0u);
                            }
                        }
                        umma_commit(smem_u32(&bars->empty[s]));        // frees the stage when these MMAs retire
                    }
                    if (ok) umma_commit(smem_u32(&bars->tfull[acc]));  // window complete
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: 8 warps.  Warp (2+e) reads
        // tensor-memory lanes 32*(warp%4).. and the column half e/4 of the tile.  The tensor core's fp32
        // accumulation truncates, which drifts over thousands of MMAs; so an accumulator only ever
        // collects one window (kWindowTokens tokens) and the windows are summed here, in registers,
        // with round-to-nearest adds.
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        uint32_t win_iter = 0;
        const bool vec_ok = (C & 3) == 0;
        bool alive = true;
        const int nwin = (kblocks + WIN - 1) / WIN;
        for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
            int g, i, j;
            decode_work<K::kSwap>(t, G, NT, g, i, j);
            const float alpha_g = (alpha * aux[8 + g]) * exp2f((float)-chunk_exponent(*pmax));
            const int row0 = i * BM + q * 32;
            const int row = row0 + lane;
            const int colbase = j * BN + half * 128;
            // warp-uniform activity of the four 32-column chunks: inside the matrix and not wholly below the diagonal
            bool use[4];
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                const int col0 = colbase + cb * 32;
                use[cb] = !(col0 >= C || col0 + 31 < row0 || row0 >= C);
            }
            float run[128];
#pragma unroll
            for (int e = 0; e < 128; ++e) run[e] = 0.f;
            for (int w = 0; w < nwin; ++w, ++win_iter) {
                const uint32_t acc = win_iter & 1u;
                const uint32_t acc_ph = (win_iter >> 1) & 1u;
                int ok = 1;
                if (lane == 0) ok = mbar_wait(smem_u32(&bars->tfull[acc]), acc_ph, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
                tc_fence_after();
#pragma unroll
                for (int cb = 0; cb < 4; ++cb) {
                    if (use[cb]) {
                        float v[32];
                        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + half * 128 + cb * 32, v);
#pragma unroll
                        for (int e = 0; e < 32; ++e) run[cb * 32 + e] += v[e];
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->tempty[acc]));
            }
            if (!alive) break;
            if (row < C) {
                float* hrow = H + ((int64_t)g * C + row) * (int64_t)C;
#pragma unroll
                for (int cb = 0; cb < 4; ++cb) {
                    const int col0 = colbase + cb * 32;
                    if (!use[cb]) continue;
                    if (vec_ok && col0 + 32 <= C && beta == 1.f) {
                        // accumulate in place with fire-and-forget vector reductions: this launch updates every
                        // element of H from exactly one thread, so the result is the same add as a
                        // load-add-store, without the read round trip that would keep this warp away from
                        // the next tile's accumulation windows
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(hrow + col0 + 4 * e),
                                         "f"(alpha_g * run[cb * 32 + 4 * e + 0]), "f"(alpha_g * run[cb * 32 + 4 * e + 1]),
                                         "f"(alpha_g * run[cb * 32 + 4 * e + 2]), "f"(alpha_g * run[cb * 32 + 4 * e + 3])
                                         : "memory");
                    } else if (vec_ok && col0 + 32 <= C) {
                        float4* p4 = reinterpret_cast<float4*>(hrow + col0);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            float4 o = (beta != 0.f) ? p4[e] : make_float4(0.f, 0.f, 0.f, 0.f);
                            if (beta != 1.f) { o.x *= beta; o.y *= beta; o.z *= beta; o.w *= beta; }
                            o.x += alpha_g * run[cb * 32 + 4 * e + 0];
                            o.y += alpha_g * run[cb * 32 + 4 * e + 1];
                            o.z += alpha_g * run[cb * 32 + 4 * e + 2];
                            o.w += alpha_g * run[cb * 32 + 4 * e + 3];
                            p4[e] = o;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            if (col0 + e < C) {
                                float o = (beta != 0.f) ? hrow[col0 + e] : 0.f;
                                if (beta != 1.f) o *= beta;
                                hrow[col0 + e] = o + alpha_g * run[cb * 32 + e];
                            }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
    if (threadIdx.x == 0 && *abort_flag && status != nullptr) atomicExch(status, RQ_ERR_TIMEOUT);
}

// ------------------------------------------------------------------------------------------
// finalize / mirror: one block per 32x32 tile pair (bi <= bj) of one group
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) finalize_kernel(float* __restrict__ H, float* __restrict__ act_sq, int C,
                                                       float div_tokens, float div_scale, float div_seq,
                                                       int sanitize, unsigned long long* __restrict__ counts) {
    __shared__ float tile[32][33];
    const int g = blockIdx.y;
    int bi, bj;
    {   // pairs ordered by bj: cum(bj) = bj*(bj+1)/2, bi in [0, bj]
        const int u = blockIdx.x;
        int jj = static_cast<int>((sqrtf(8.f * static_cast<float>(u) + 1.f) - 1.f) * 0.5f);
        while ((jj + 1) * (jj + 2) / 2 <= u) ++jj;
        while (jj * (jj + 1) / 2 > u) --jj;
        bj = jj;
        bi = u - jj * (jj + 1) / 2;
    }
    float* Hg = H + (int64_t)g * C * C;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    unsigned int n_nan = 0, n_inf = 0;
    const unsigned int weight = (bi == bj) ? 1u : 2u;
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int row = bi * 32 + r, col = bj * 32 + tx;
        float v = 0.f;
        if (row < C && col < C) {
            v = Hg[(int64_t)row * C + col];
            if (div_tokens != 1.f) v = __fdiv_rn(v, div_tokens);
            if (div_scale != 1.f) v = __fdiv_rn(v, div_scale);
            if (sanitize && (bi != bj || row <= col)) {
                if (isnan(v)) { n_nan += (bi == bj && row != col) ? 2u : weight; v = 0.f; }
                else if (isinf(v)) { n_inf += (bi == bj && row != col) ? 2u : weight; v = 0.f; }
            }
        }
        tile[r][tx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
        if (bi == bj) {
            const int row = bi * 32 + r, col = bi * 32 + tx;
            if (row < C && col < C) Hg[(int64_t)row * C + col] = (r <= tx) ? tile[r][tx] : tile[tx][r];
        } else {
            int row = bi * 32 + r, col = bj * 32 + tx;
            if (row < C && col < C) Hg[(int64_t)row * C + col] = tile[r][tx];
            row = bj * 32 + r;
            col = bi * 32 + tx;
            if (row < C && col < C) Hg[(int64_t)row * C + col] = tile[tx][r];
        }
    }
    if (sanitize && counts != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            n_nan += __shfl_xor_sync(0xffffffffu, n_nan, o);
            n_inf += __shfl_xor_sync(0xffffffffu, n_inf, o);
        }
        if (tx == 0) {
            if (n_nan) atomicAdd(&counts[0], (unsigned long long)n_nan);
            if (n_inf) atomicAdd(&counts[1], (unsigned long long)n_inf);
        }
    }
    if (act_sq != nullptr && div_seq != 1.f && g == 0) {
        for (int c = blockIdx.x * 256 + threadIdx.x; c < C; c += gridDim.x * 256) act_sq[c] = __fdiv_rn(act_sq[c], div_seq);
    }
}

// ------------------------------------------------------------------------------------------
// packed upper storage for the cross-rank exchange.  Only entries on or above the diagonal of H[g] carry
// information before finalize; row r keeps its columns from the start of its 128-row block, c0 = (r / 128) * 128,
// to C - 1, rows back to back:  offset(r) = 128 * b * C - 128 * 128 * b * (b - 1) / 2 + (r - 128 * b) * (C - 128 * b),
// b = r / 128.  Row starts stay 16-byte aligned when C is a multiple of 4.
// ------------------------------------------------------------------------------------------
__host__ __device__ inline long long packed_row_offset(int r, int C) {
    const long long b = r / 128;
    return 128ll * b * C - 8192ll * b * (b - 1) + (r - 128 * b) * (C - 128 * b);
}

// grid (C, G), 256 threads: one row of one group per block.  to_packed != 0: H -> packed, else packed -> H.
__global__ void __launch_bounds__(256) upper_copy_kernel(float* __restrict__ H, float* __restrict__ packed, int C,
                                                         long long group_stride, int to_packed) {
    const int r = blockIdx.x, g = blockIdx.y;
    const int c0 = (r / 128) * 128;
    const int n = C - c0;
    float* hrow = H + ((long long)g * C + r) * C + c0;
    float* prow = packed + (long long)g * group_stride + packed_row_offset(r, C);
    float* dst = to_packed ? prow : hrow;
    const float* src = to_packed ? hrow : prow;
    if ((C & 3) == 0) {
        for (int i = threadIdx.x; i < n / 4; i += 256)
            reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < n; i += 256) dst[i] = src[i];
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int encode_map(CUtensorMap* map, void* base, int64_t Kc, int C, int planes, int box_k, int box_rows, int bk) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return RQ_ERR_CUDA;
    cuuint64_t dims[3] = {(cuuint64_t)Kc, (cuuint64_t)C, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)Kc * 2, (cuuint64_t)Kc * 2 * (cuuint64_t)C};
    cuuint32_t box[3] = {(cuuint32_t)box_k, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RQ_OK : RQ_ERR_CUDA;
}

static int num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BK, int NX, bool WIDE_Y = false>
static int launch_umma(void* planes, int64_t Kc, int C, int G, int nplanes, float* H, float alpha, float beta,
                       const float* aux, const unsigned int* pmax, int window_tokens, int* status, cudaStream_t st) {
    using K = Cfg<BK, NX, WIDE_Y>;
    const int win_blocks = window_tokens / BK > 0 ? window_tokens / BK : 1;
    CUtensorMap mapA, mapB;
    int rc = encode_map(&mapA, planes, Kc, C, nplanes, BK, BM, BK);
    if (rc != RQ_OK) return rc;
    rc = encode_map(&mapB, planes, Kc, C, nplanes, BK, BN, BK);
    if (rc != RQ_OK) return rc;
    if (cudaFuncSetAttribute(umma_kernel<BK, NX, WIDE_Y>, cudaFuncAttributeMaxDynamicSharedMemorySize, K::kSmemBytes) !=
        cudaSuccess)
        return RQ_ERR_CUDA;
    const int MT = (C + BM - 1) / BM, NT = (C + BN - 1) / BN;
    const int total = ((NT - 1) * NT + MT) * G;
    const int kblocks = (int)(Kc / BK);
    // One work unit per tile and launch: every element of H receives exactly one add per launch, so the
    // accumulated Hessian is the same bit pattern from run to run (splitting a tile's tokens over several
    // CTAs would even out the last round of small problems, but H + a + b is not H + b + a in fp32).
    const int grid = total < num_sms() ? total : num_sms();
    prof::Scope timed(RQ_PROF_HESSIAN_UMMA, st);
    umma_kernel<BK, NX, WIDE_Y><<<grid, kThreads, K::kSmemBytes, st>>>(mapA, mapB, H, C, G, MT, NT, kblocks, 0, NX, alpha,
                                                                      beta, aux, pmax, win_blocks, status);
    return check_launch();
}

template <typename T, int NX>
static void launch_pack(const void* xp, int64_t ldx, const float* sp, float* aux, float2* tok, unsigned int* pmax,
                        int nvalid, int C, int G, int64_t Kc, uint16_t* planes, float* partial, cudaStream_t st) {
    const T* x = reinterpret_cast<const T*>(xp);
    group_scale_kernel<<<1, 1024, 0, st>>>(sp, nvalid, G, aux, pmax);
    token_stats_kernel<T><<<(unsigned)((Kc + 7) / 8), 256, 0, st>>>(x, ldx, sp, aux, nvalid, (int)Kc, C, G, tok, pmax);
    dim3 pgrid((unsigned)((Kc + kPackTokens - 1) / kPackTokens), (unsigned)((C + kPackChannels - 1) / kPackChannels));
    pack_kernel<T, NX><<<pgrid, 256, 0, st>>>(x, ldx, sp, aux, tok, pmax, nvalid, C, G, (int)Kc, planes, partial);
}

}  // namespace hess
}  // namespace rq

using namespace rq;

// Layout of one chunk slot: planes [nx + 2G][C][Kc] fp16 | per-tile sums of squares [Kc/64][C] fp32 |
// token statistics [Kc] float2 | group scales [16] fp32, largest P_t.  Sized for two X' planes (fp32 input),
// whatever the dtype.
static size_t slot_plane_bytes(int64_t Kc, int C, int nplanes) {
    const size_t bytes = (size_t)nplanes * (size_t)C * (size_t)Kc * 2;
    return (bytes + 1023) / 1024 * 1024;
}

extern "C" size_t rq_hessian_workspace_bytes(int64_t chunk_tokens, int C, int G, int has_saliency) {
    (void)has_saliency;
    if (chunk_tokens <= 0 || C <= 0 || G <= 0) return 0;
    const int64_t Kc = (chunk_tokens + 63) / 64 * 64;
    size_t bytes = slot_plane_bytes(Kc, C, 2 + 2 * G);
    bytes += ((size_t)(Kc / 64) * (size_t)C * 4 + 1023) / 1024 * 1024;   // per-tile sums of squares
    bytes += (size_t)Kc * 8 + 1024;                                        // token statistics, group scales
    return bytes + 1024;
}

// Shared body of rq_hessian_accum and rq_hessian_accum_pipelined.  With gemm_stream == pack stream the
// launches are simply ordered; otherwise the workspace is cut into chunk slots, the packing of chunk c runs on
// `st` while the tensor-core kernel of an earlier chunk runs on `gst`, and events order the two per slot.
static int hessian_accum_impl(const void* x, int x_dtype, int64_t ldx, const float* sal, float* H, float* act_sq,
                              int64_t N, int C, int G, float alpha, float beta, void* workspace,
                              size_t workspace_bytes, int* status, int variant, int64_t chunk_tokens, cudaStream_t st,
                              cudaStream_t gst) {
    using namespace rq::hess;
    if (!x || !H || !workspace || C <= 0 || G <= 0 || G > 8 || N < 0 || ldx < C) return RQ_ERR_INVALID;
    if (!sal && G != 1) return RQ_ERR_INVALID;
    if (x_dtype != RQ_F32 && x_dtype != RQ_BF16 && x_dtype != RQ_F16) return RQ_ERR_INVALID;
    // bits 0-3: operand layout; bits 4-5: accumulation window of 128 >> n tokens (32 needs the 32-token stages)
    const int wincode = (variant >> 4) & 3;
    if (variant < 0 || (variant & 15) > 2 || (variant >> 6) != 0 || wincode == 3) return RQ_ERR_UNSUPPORTED;
    const int window = kWindowTokens >> wincode;
    variant = (wincode == 2 && (variant & 15) == 0) ? 1 : (variant & 15);
    if (reinterpret_cast<uintptr_t>(workspace) % 1024 != 0) return RQ_ERR_INVALID;
    if (N == 0) return RQ_OK;
    const bool piped = gst != st;

    // largest chunk (multiple of 64 tokens) the workspace can hold; pipelined: the requested chunk, as many slots as fit
    const int has_sal = sal != nullptr;
    int64_t chunk = (N + 63) / 64 * 64;
    if (piped && chunk_tokens > 0 && chunk_tokens < chunk) chunk = (chunk_tokens + 63) / 64 * 64;
    while (chunk > 64 && rq_hessian_workspace_bytes(chunk, C, G, has_sal) > workspace_bytes) chunk -= 64;
    const size_t slot_bytes = rq_hessian_workspace_bytes(chunk, C, G, has_sal);
    if (slot_bytes > workspace_bytes) return RQ_ERR_WORKSPACE;
    int nslots = 1;
    if (piped) {
        nslots = (int)(workspace_bytes / slot_bytes);
        if (nslots > 4) nslots = 4;
    }
    cudaEvent_t slot_free[4] = {nullptr, nullptr, nullptr, nullptr};

    const int nx = x_dtype == RQ_F32 ? 2 : 1;
    const int nplanes = nx + 2 * G;
    const size_t esz = x_dtype == RQ_F32 ? 4 : 2;
    int rc = RQ_OK;
    int64_t ci = 0;
    for (int64_t n0 = 0; n0 < N && rc == RQ_OK; n0 += chunk, ++ci) {
        const int slot = (int)(ci % nslots);
        uint8_t* slot_base = reinterpret_cast<uint8_t*>(workspace) + (size_t)slot * slot_bytes;
        uint16_t* planes = reinterpret_cast<uint16_t*>(slot_base);
        if (piped && slot_free[slot]) {                       // the kernel that last read this slot must be done
            if (cudaStreamWaitEvent(st, slot_free[slot], 0) != cudaSuccess) { rc = RQ_ERR_CUDA; break; }
            cudaEventDestroy(slot_free[slot]);
            slot_free[slot] = nullptr;
        }
        const int nvalid = (int)((N - n0) < chunk ? (N - n0) : chunk);
        const int64_t Kc = ((int64_t)nvalid + 63) / 64 * 64;
        const size_t plane_bytes = slot_plane_bytes(Kc, C, nplanes);
        const size_t partial_bytes = ((size_t)(Kc / 64) * (size_t)C * 4 + 1023) / 1024 * 1024;
        float* partial = act_sq ? reinterpret_cast<float*>(slot_base + plane_bytes) : nullptr;
        float2* tok = reinterpret_cast<float2*>(slot_base + plane_bytes + partial_bytes);
        float* aux = reinterpret_cast<float*>(slot_base + plane_bytes + partial_bytes + (size_t)Kc * 8);
        unsigned int* pmax = reinterpret_cast<unsigned int*>(aux + 16);
        const uint8_t* xp = reinterpret_cast<const uint8_t*>(x) + (size_t)n0 * (size_t)ldx * esz;
        const float* sp = has_sal ? sal + n0 * G : nullptr;
        {
        prof::Scope timed(RQ_PROF_HESSIAN_PACK, st);
        if (x_dtype == RQ_F32)
            launch_pack<float, 2>(xp, ldx, sp, aux, tok, pmax, nvalid, C, G, Kc, planes, partial, st);
        else if (x_dtype == RQ_BF16)
            launch_pack<__nv_bfloat16, 1>(xp, ldx, sp, aux, tok, pmax, nvalid, C, G, Kc, planes, partial, st);
        else
            launch_pack<__half, 1>(xp, ldx, sp, aux, tok, pmax, nvalid, C, G, Kc, planes, partial, st);
        }
        rc = check_launch();
        if (rc != RQ_OK) break;
        if (act_sq) {
            act_reduce_kernel<<<(C + 255) / 256, 256, 0, st>>>(partial, (int)((Kc + kPackTokens - 1) / kPackTokens), C, act_sq);
            rc = check_launch();
            if (rc != RQ_OK) break;
        }
        if (piped) {
            cudaEvent_t packed;
            if (cudaEventCreateWithFlags(&packed, cudaEventDisableTiming) != cudaSuccess) { rc = RQ_ERR_CUDA; break; }
            const bool ok = cudaEventRecord(packed, st) == cudaSuccess && cudaStreamWaitEvent(gst, packed, 0) == cudaSuccess;
            cudaEventDestroy(packed);                          // released once the recorded work has completed
            if (!ok) { rc = RQ_ERR_CUDA; break; }
        }
        const float b = (n0 == 0) ? beta : 1.f;
        if (nx == 2)
            rc = variant == 1 ? launch_umma<32, 2>(planes, Kc, C, G, nplanes, H, alpha, b, aux, pmax, window, status, gst)
                              : launch_umma<64, 2>(planes, Kc, C, G, nplanes, H, alpha, b, aux, pmax, window, status, gst);
        else if (variant == 2)
            rc = launch_umma<64, 1, true>(planes, Kc, C, G, nplanes, H, alpha, b, aux, pmax, window, status, gst);
        else if (variant == 1)
            rc = launch_umma<32, 1>(planes, Kc, C, G, nplanes, H, alpha, b, aux, pmax, window, status, gst);
        else
            rc = launch_umma<64, 1>(planes, Kc, C, G, nplanes, H, alpha, b, aux, pmax, window, status, gst);
        if (rc != RQ_OK) break;
        if (piped && n0 + chunk < N) {
            if (cudaEventCreateWithFlags(&slot_free[slot], cudaEventDisableTiming) != cudaSuccess ||
                cudaEventRecord(slot_free[slot], gst) != cudaSuccess) { rc = RQ_ERR_CUDA; break; }
        }
    }
    for (int i = 0; i < 4; ++i)
        if (slot_free[i]) cudaEventDestroy(slot_free[i]);
    return rc;
}

extern "C" int rq_hessian_accum(const void* x, int x_dtype, int64_t ldx, const float* sal, float* H, float* act_sq,
                                int64_t N, int C, int G, float alpha, float beta, void* workspace,
                                size_t workspace_bytes, int* status, int variant, void* stream) {
    return hessian_accum_impl(x, x_dtype, ldx, sal, H, act_sq, N, C, G, alpha, beta, workspace, workspace_bytes, status,
                              variant, 0, as_stream(stream), as_stream(stream));
}

extern "C" int rq_hessian_accum_pipelined(const void* x, int x_dtype, int64_t ldx, const float* sal, float* H,
                                          float* act_sq, int64_t N, int C, int G, float alpha, float beta,
                                          void* workspace, size_t workspace_bytes, int* status, int variant,
                                          int64_t chunk_tokens, void* stream, void* gemm_stream) {
    if (!gemm_stream || gemm_stream == stream) return RQ_ERR_INVALID;
    return hessian_accum_impl(x, x_dtype, ldx, sal, H, act_sq, N, C, G, alpha, beta, workspace, workspace_bytes, status,
                              variant, chunk_tokens, as_stream(stream), as_stream(gemm_stream));
}

extern "C" int rq_hessian_finalize(float* H, float* act_sq, int C, int G, float div_tokens, float div_scale,
                                   float div_seq, int sanitize, unsigned long long* counts, void* stream) {
    if (!H || C <= 0 || G <= 0) return RQ_ERR_INVALID;
    if (div_tokens == 0.f || div_scale == 0.f || div_seq == 0.f) return RQ_ERR_INVALID;
    const int T = (C + 31) / 32;
    dim3 grid((unsigned)(T * (T + 1) / 2), (unsigned)G);
    rq::hess::finalize_kernel<<<grid, 256, 0, as_stream(stream)>>>(H, act_sq, C, div_tokens, div_scale, div_seq,
                                                                  sanitize, counts);
    return check_launch();
}

extern "C" int64_t rq_hessian_packed_elems(int C) {
    return C <= 0 ? 0 : (int64_t)rq::hess::packed_row_offset(C, C);
}

extern "C" int rq_hessian_pack_upper(const float* H, int C, int G, float* packed, int64_t group_stride, void* stream) {
    if (!H || !packed || C <= 0 || G <= 0 || group_stride < rq_hessian_packed_elems(C)) return RQ_ERR_INVALID;
    if ((C & 3) == 0 && ((group_stride & 3) != 0 || (reinterpret_cast<uintptr_t>(packed) & 15) != 0 ||
                         (reinterpret_cast<uintptr_t>(H) & 15) != 0))
        return RQ_ERR_INVALID;
    rq::hess::upper_copy_kernel<<<dim3((unsigned)C, (unsigned)G), 256, 0, as_stream(stream)>>>(
        const_cast<float*>(H), packed, C, (long long)group_stride, 1);
    return check_launch();
}

extern "C" int rq_hessian_unpack_upper(const float* packed, int64_t group_stride, int C, int G, float* H, void* stream) {
    if (!H || !packed || C <= 0 || G <= 0 || group_stride < rq_hessian_packed_elems(C)) return RQ_ERR_INVALID;
    if ((C & 3) == 0 && ((group_stride & 3) != 0 || (reinterpret_cast<uintptr_t>(packed) & 15) != 0 ||
                         (reinterpret_cast<uintptr_t>(H) & 15) != 0))
        return RQ_ERR_INVALID;
    rq::hess::upper_copy_kernel<<<dim3((unsigned)C, (unsigned)G), 256, 0, as_stream(stream)>>>(
        H, const_cast<float*>(packed), C, (long long)group_stride, 0);
    return check_launch();
}
