// Saliency-weighted Hessian accumulation  H[g] = beta*H[g] + alpha * X^T diag(s_g) X  on the
// 5th-generation tensor cores (tcgen05 + tensor memory), fed by TMA.
//
// Two kernels per chunk of tokens:
//   1. pack:  reads X (fp32 / bf16 / fp16) and the saliency once, and writes token-contiguous
//             ("K-major") bf16 planes  X_hi, X_lo, Y_hi[g], Y_lo[g]  with  Y_g = s_g * X,
//             v_hi = bf16(v), v_lo = bf16(v - v_hi); also the per-channel sum of squares.
//   2. umma:  persistent, warp-specialised GEMM over the upper-triangular 128x256 tiles of
//             every H[g]:  D = X_hi.Y_lo^T + X_lo.Y_hi^T + X_hi.Y_hi^T  accumulated in fp32 in
//             tensor memory over windows of 128 tokens; the epilogue warps sum the windows in
//             registers with round-to-nearest adds (the tensor core's own accumulation truncates
//             toward zero and would drift by ~4e-8 per MMA; measured: 5e-5 over 8192 tokens, and the
//             same with the operand sign flipped) and read-modify-write the tile into H at the end.
// The three-product split keeps the result within ~1e-6 relative Frobenius of an fp32 GEMM.
#include <cuda.h>

#include "rq_common.cuh"
#include "rq_sm100.cuh"

namespace rq {
namespace hess {

using namespace rq::sm100;

constexpr int BM = 128;          // tile rows   (channels i)   = UMMA M
constexpr int BN = 256;          // tile cols   (channels j)   = UMMA N
constexpr int UK = 16;           // bf16 UMMA K
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;   // warp 0: TMA producer, warp 1: MMA issuer, warps 2-9: epilogue
constexpr int kTmemCols = 512;   // two 128x256 fp32 accumulators
constexpr int kWindowTokens = 128;   // tokens accumulated on the tensor core before a round-to-nearest add
constexpr int kPackTile = 64;    // pack kernel tile edge (tokens and channels)

template <int BK, int NPROD, bool WIDE_Y = false>
struct Cfg {
    static constexpr int kLayout = BK == 64 ? 2 : 4;              // UMMA swizzle mode: 128 B / 64 B
    static constexpr int kSBO = 8 * BK * 2;                        // bytes between 8-row groups
    static constexpr int kATile = BM * BK * 2;
    static constexpr int kBTile = BN * BK * 2;
    // NPROD == 3 (fp32 / fp16 X):  A side (128 rows) = X_hi, X_lo;  B side (256 rows) = Y_hi, Y_lo.
    // NPROD == 2 (bf16 X, X_lo = 0): the two-plane operand Y goes on the narrow A side and the single
    // plane X_hi on the wide B side, 64 KB per stage instead of 80 KB: less L2->SM traffic per MMA
    // and room for a third stage.
    // WIDE_Y keeps Y on the wide side also for NPROD == 2 (80 KB per stage), for comparison.
    static constexpr bool kSwap = NPROD == 2 && !WIDE_Y;
    static constexpr int kAPlanes = (NPROD == 3 || kSwap) ? 2 : 1;
    static constexpr int kBPlanes = (NPROD == 3 || !kSwap) ? 2 : 1;
    static constexpr int kStageBytes = kAPlanes * kATile + kBPlanes * kBTile;
    static constexpr int kStages = (200 * 1024) / kStageBytes;
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;   // +1024: alignment slack
};

// ------------------------------------------------------------------------------------------
// pack
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// grid (Kc/64, ceil(C/64)), 256 threads: token tiles vary fastest, so that concurrently running blocks
// extend the same plane rows (contiguous DRAM pages on the write side).  planes: [P][C][Kc] bf16, P = 2 (no saliency) or 2+2G.
// partial: [Kc/64][C] per-tile sums of x^2 (may be NULL).
template <typename T>
__global__ void __launch_bounds__(256) pack_kernel(const T* __restrict__ x, int64_t ldx,
                                                   const float* __restrict__ sal, int nvalid, int C, int G, int Kc,
                                                   __nv_bfloat16* __restrict__ planes, float* __restrict__ partial,
                                                   int write_xlo) {
    // channel-major tile: the write side (64 consecutive channels of one token per 64 threads) strides by the
    // row length, the read side takes two adjacent tokens of one channel as one 8-byte word
    __shared__ __align__(8) float xs[kPackTile][kPackTile + 2];
    __shared__ float ss[kPackTile][8];
    const int t0 = blockIdx.x * kPackTile;
    const int c0 = blockIdx.y * kPackTile;
    const int tid = threadIdx.x;

    {   // load: 64 consecutive channels of one token per pass of 64 threads
        const int cc = tid & 63;
        const int tr = tid >> 6;
#pragma unroll 4
        for (int p = 0; p < 16; ++p) {
            const int t = p * 4 + tr;
            float v = 0.f;
            if (t0 + t < nvalid && c0 + cc < C) v = load_as_float<T>(x, (int64_t)(t0 + t) * ldx + c0 + cc);
            xs[cc][t] = v;
        }
        if (sal != nullptr) {
            for (int e = tid; e < kPackTile * G; e += 256) {
                const int t = e / G, g = e - t * G;
                ss[t][g] = (t0 + t < nvalid) ? sal[(int64_t)(t0 + t) * G + g] : 0.f;
            }
        }
    }
    __syncthreads();

    const int warp = tid >> 5, lane = tid & 31;
    const int64_t plane_stride = (int64_t)C * Kc;
    const int ta = 2 * lane, tb = 2 * lane + 1;
    float sa[8], sb[8];                                        // this lane's two tokens' saliencies, read once
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        sa[g] = (sal != nullptr && g < G) ? ss[ta][g] : 0.f;
        sb[g] = (sal != nullptr && g < G) ? ss[tb][g] : 0.f;
    }
    for (int cc = warp; cc < kPackTile; cc += 8) {
        const int c = c0 + cc;
        if (c >= C) break;                                     // warp-uniform
        const float2 xab = *reinterpret_cast<const float2*>(&xs[cc][ta]);
        const float xa = xab.x, xb = xab.y;
        const int64_t off = (int64_t)c * Kc + t0 + ta;          // even -> 4-byte aligned pair
        __nv_bfloat16 ha, la, hb, lb;
        split_bf16(xa, ha, la);
        split_bf16(xb, hb, lb);
        *reinterpret_cast<__nv_bfloat162*>(planes + off) = __halves2bfloat162(ha, hb);
        if (write_xlo) *reinterpret_cast<__nv_bfloat162*>(planes + plane_stride + off) = __halves2bfloat162(la, lb);
        if (sal != nullptr) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if (g >= G) break;
                const float ya = __fmul_rn(xa, sa[g]);
                const float yb = __fmul_rn(xb, sb[g]);
                split_bf16(ya, ha, la);
                split_bf16(yb, hb, lb);
                *reinterpret_cast<__nv_bfloat162*>(planes + (2 + 2 * g) * plane_stride + off) = __halves2bfloat162(ha, hb);
                *reinterpret_cast<__nv_bfloat162*>(planes + (3 + 2 * g) * plane_stride + off) = __halves2bfloat162(la, lb);
            }
        }
        if (partial != nullptr) {
            float sq = xa * xa + xb * xb;
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

template <int BK, int NPROD, bool WIDE_Y>
__global__ void __launch_bounds__(kThreads, 1)
umma_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
            float* __restrict__ H, int C, int G, int MT, int NT, int kblocks, int a_plane, int b_plane0,
            float alpha, float beta, int ksplit, int* __restrict__ status) {
    using K = Cfg<BK, NPROD, WIDE_Y>;
    constexpr int WIN = kWindowTokens / BK;                              // k-blocks per accumulation window
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;                       // shared-space address of stage 0
    Bars* bars = reinterpret_cast<Bars*>(smem_raw + (tiles - raw) + K::kStages * K::kStageBytes);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_per_group = (NT - 1) * NT + MT;
    const int total_tiles = tiles_per_group * G;
    // A work unit is (tile, part of the chunk's tokens): with ksplit > 1 every tile is visited ksplit times, each
    // visit adding the sum over its share of the k-blocks into H (only with the reduction epilogue, beta == 1),
    // which evens out the last round when the tile count is a poor multiple of the grid.  Units are ordered
    // part-major so that concurrently running CTAs stream the same token range.
    const int total_units = total_tiles * ksplit;
    const int kb_per_part = ((kblocks + ksplit - 1) / ksplit + WIN - 1) / WIN * WIN;

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
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                const int part = u / total_tiles, t = u - part * total_tiles;
                const int kb0 = part * kb_per_part;
                const int kb1 = (kb0 + kb_per_part < kblocks) ? kb0 + kb_per_part : kblocks;
                int g, i, j;
                decode_work<K::kSwap>(t, G, NT, g, i, j);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % K::kStages;
                    const uint32_t ph = (it / K::kStages) & 1u;
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t fb = smem_u32(&bars->full[s]);
                    uint32_t dst = tiles + s * K::kStageBytes;
                    mbar_expect_tx(fb, K::kStageBytes);
                    if (NPROD == 3) {
                        tma_load_3d(dst, &mapA, fb, kb * BK, i * BM, a_plane);
                        tma_load_3d(dst + K::kATile, &mapA, fb, kb * BK, i * BM, a_plane + 1);
                        dst += 2 * K::kATile;
                        tma_load_3d(dst, &mapB, fb, kb * BK, j * BN, b_plane0 + 2 * g);
                        tma_load_3d(dst + K::kBTile, &mapB, fb, kb * BK, j * BN, b_plane0 + 2 * g + 1);
                    } else if (K::kSwap) {
                        tma_load_3d(dst, &mapA, fb, kb * BK, i * BM, b_plane0 + 2 * g);
                        tma_load_3d(dst + K::kATile, &mapA, fb, kb * BK, i * BM, b_plane0 + 2 * g + 1);
                        tma_load_3d(dst + 2 * K::kATile, &mapB, fb, kb * BK, j * BN, a_plane);
                    } else {
                        tma_load_3d(dst, &mapA, fb, kb * BK, i * BM, a_plane);
                        tma_load_3d(dst + K::kATile, &mapB, fb, kb * BK, j * BN, b_plane0 + 2 * g);
                        tma_load_3d(dst + K::kATile + K::kBTile, &mapB, fb, kb * BK, j * BN, b_plane0 + 2 * g + 1);
                    }
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
            constexpr uint32_t idesc = umma_idesc_bf16_f32(BM, BN);
            uint32_t it = 0, win_iter = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                const int part = u / total_tiles;
                const int kb0 = part * kb_per_part;
                const int kb1 = (kb0 + kb_per_part < kblocks) ? kb0 + kb_per_part : kblocks;
                const int nwin = (kb1 - kb0 + WIN - 1) / WIN;
                for (int w = 0; w < nwin && ok; ++w, ++win_iter) {
                    const uint32_t acc = win_iter & 1u;
                    const uint32_t acc_ph = (win_iter >> 1) & 1u;
                    if (!mbar_wait(smem_u32(&bars->tempty[acc]), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    const int kb_begin = kb0 + w * WIN;
                    const int kb_end = (kb_begin + WIN < kb1) ? kb_begin + WIN : kb1;
                    for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                        const uint32_t s = it % K::kStages;
                        const uint32_t ph = (it / K::kStages) & 1u;
                        if (!mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_hi = tiles + s * K::kStageBytes;
                        const uint32_t a_lo = a_hi + K::kATile;
                        const uint32_t b_hi = a_hi + K::kAPlanes * K::kATile;
                        const uint32_t b_lo = b_hi + K::kBTile;
#pragma unroll
                        for (int k = 0; k < BK / UK; ++k) {
                            const uint32_t koff = k * UK * 2;           // bytes along K inside the swizzle row
                            const uint64_t dah = umma_smem_desc(a_hi + koff, K::kSBO, K::kLayout);
                            const uint64_t dal = umma_smem_desc(a_lo + koff, K::kSBO, K::kLayout);
                            const uint64_t dbh = umma_smem_desc(b_hi + koff, K::kSBO, K::kLayout);
                            // the first MMA of a window overwrites the accumulator; small terms go first
                            const uint32_t keep = (kb != kb_begin || k != 0) ? 1u : 0u;
                            if (NPROD == 3) {
                                const uint64_t dbl = umma_smem_desc(b_lo + koff, K::kSBO, K::kLayout);
                                umma_bf16(d_tmem, dah, dbl, idesc, keep);
                                umma_bf16(d_tmem, dal, dbh, idesc, 1u);
                            } else if (K::kSwap) {
                                umma_bf16(d_tmem, dal, dbh, idesc, keep);
                            } else {
                                const uint64_t dbl = umma_smem_desc(b_lo + koff, K::kSBO, K::kLayout);
                                umma_bf16(d_tmem, dah, dbl, idesc, keep);
                            }
                            umma_bf16(d_tmem, dah, dbh, idesc, 1u);
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
        for (int u = blockIdx.x; u < total_units && alive; u += gridDim.x) {
            const int part = u / total_tiles, t = u - part * total_tiles;
            const int kb0 = part * kb_per_part;
            const int kb1 = (kb0 + kb_per_part < kblocks) ? kb0 + kb_per_part : kblocks;
            const int nwin = (kb1 - kb0 + WIN - 1) / WIN;
            if (nwin <= 0) continue;
            int g, i, j;
            decode_work<K::kSwap>(t, G, NT, g, i, j);
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
                                         "f"(alpha * run[cb * 32 + 4 * e + 0]), "f"(alpha * run[cb * 32 + 4 * e + 1]),
                                         "f"(alpha * run[cb * 32 + 4 * e + 2]), "f"(alpha * run[cb * 32 + 4 * e + 3])
                                         : "memory");
                    } else if (vec_ok && col0 + 32 <= C) {
                        float4* p4 = reinterpret_cast<float4*>(hrow + col0);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            float4 o = (beta != 0.f) ? p4[e] : make_float4(0.f, 0.f, 0.f, 0.f);
                            if (beta != 1.f) { o.x *= beta; o.y *= beta; o.z *= beta; o.w *= beta; }
                            o.x += alpha * run[cb * 32 + 4 * e + 0];
                            o.y += alpha * run[cb * 32 + 4 * e + 1];
                            o.z += alpha * run[cb * 32 + 4 * e + 2];
                            o.w += alpha * run[cb * 32 + 4 * e + 3];
                            p4[e] = o;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            if (col0 + e < C) {
                                float o = (beta != 0.f) ? hrow[col0 + e] : 0.f;
                                if (beta != 1.f) o *= beta;
                                hrow[col0 + e] = o + alpha * run[cb * 32 + e];
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

template <int BK, int NPROD, bool WIDE_Y = false>
static int launch_umma(void* planes, int64_t Kc, int C, int G, int nplanes, int b_plane0, float* H, float alpha,
                       float beta, int* status, cudaStream_t st) {
    using K = Cfg<BK, NPROD, WIDE_Y>;
    CUtensorMap mapA, mapB;
    int rc = encode_map(&mapA, planes, Kc, C, nplanes, BK, BM, BK);
    if (rc != RQ_OK) return rc;
    rc = encode_map(&mapB, planes, Kc, C, nplanes, BK, BN, BK);
    if (rc != RQ_OK) return rc;
    if (cudaFuncSetAttribute(umma_kernel<BK, NPROD, WIDE_Y>, cudaFuncAttributeMaxDynamicSharedMemorySize, K::kSmemBytes) !=
        cudaSuccess)
        return RQ_ERR_CUDA;
    const int MT = (C + BM - 1) / BM, NT = (C + BN - 1) / BN;
    const int total = ((NT - 1) * NT + MT) * G;
    const int kblocks = (int)(Kc / BK);
    // The kernel can visit every tile ksplit times, each visit adding the sum over a share of the k-blocks with
    // the reduction epilogue (units are (tile, part), part-major); that evens out the last round when the tile
    // count is a poor multiple of the grid (+11 % at C = 1024, nothing at C = 4096).  It is left at 1: the order
    // in which two parts reach an element of H is not fixed, and H + a + b is not H + b + a in fp32, so the
    // split would make the accumulated Hessian differ from run to run in the last bit.
    const int ksplit = 1;
    const long long units = (long long)total * ksplit;
    const int grid = units < num_sms() ? (int)units : num_sms();
    prof::Scope timed(RQ_PROF_HESSIAN_UMMA, st);
    umma_kernel<BK, NPROD, WIDE_Y><<<grid, kThreads, K::kSmemBytes, st>>>(mapA, mapB, H, C, G, MT, NT, kblocks, 0,
                                                                  b_plane0, alpha, beta, ksplit, status);
    return check_launch();
}

}  // namespace hess
}  // namespace rq

using namespace rq;

extern "C" size_t rq_hessian_workspace_bytes(int64_t chunk_tokens, int C, int G, int has_saliency) {
    if (chunk_tokens <= 0 || C <= 0 || G <= 0) return 0;
    const int64_t Kc = (chunk_tokens + 63) / 64 * 64;
    const int64_t planes = has_saliency ? 2 + 2 * (int64_t)G : 2;
    size_t bytes = (size_t)planes * (size_t)C * (size_t)Kc * 2;
    bytes = (bytes + 1023) / 1024 * 1024;
    bytes += (size_t)(Kc / 64) * (size_t)C * 4;            // per-tile sums of squares
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
    if (variant < 0 || variant > 2) return RQ_ERR_UNSUPPORTED;
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

    const int nplanes = has_sal ? 2 + 2 * G : 2;
    const int b_plane0 = has_sal ? 2 : 0;
    const int nprod = (x_dtype == RQ_BF16) ? 2 : 3;
    const size_t esz = x_dtype == RQ_F32 ? 4 : 2;
    int rc = RQ_OK;
    int64_t ci = 0;
    for (int64_t n0 = 0; n0 < N && rc == RQ_OK; n0 += chunk, ++ci) {
        const int slot = (int)(ci % nslots);
        uint8_t* slot_base = reinterpret_cast<uint8_t*>(workspace) + (size_t)slot * slot_bytes;
        __nv_bfloat16* planes = reinterpret_cast<__nv_bfloat16*>(slot_base);
        if (piped && slot_free[slot]) {                       // the kernel that last read this slot must be done
            if (cudaStreamWaitEvent(st, slot_free[slot], 0) != cudaSuccess) { rc = RQ_ERR_CUDA; break; }
            cudaEventDestroy(slot_free[slot]);
            slot_free[slot] = nullptr;
        }
        const int nvalid = (int)((N - n0) < chunk ? (N - n0) : chunk);
        const int64_t Kc = ((int64_t)nvalid + 63) / 64 * 64;
        size_t plane_bytes = (size_t)nplanes * (size_t)C * (size_t)Kc * 2;
        plane_bytes = (plane_bytes + 1023) / 1024 * 1024;
        float* partial = act_sq ? reinterpret_cast<float*>(slot_base + plane_bytes) : nullptr;
        const uint8_t* xp = reinterpret_cast<const uint8_t*>(x) + (size_t)n0 * (size_t)ldx * esz;
        const float* sp = has_sal ? sal + n0 * G : nullptr;
        dim3 pgrid((unsigned)(Kc / kPackTile), (unsigned)((C + kPackTile - 1) / kPackTile));
        const int write_xlo = (nprod == 3 || !has_sal) ? 1 : 0;     // without saliency X_lo doubles as Y_lo
        {
        prof::Scope timed(RQ_PROF_HESSIAN_PACK, st);
        if (x_dtype == RQ_F32)
            pack_kernel<float><<<pgrid, 256, 0, st>>>(reinterpret_cast<const float*>(xp), ldx, sp, nvalid, C, G, (int)Kc,
                                                       planes, partial, write_xlo);
        else if (x_dtype == RQ_BF16)
            pack_kernel<__nv_bfloat16><<<pgrid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(xp), ldx, sp, nvalid,
                                                               C, G, (int)Kc, planes, partial, write_xlo);
        else
            pack_kernel<__half><<<pgrid, 256, 0, st>>>(reinterpret_cast<const __half*>(xp), ldx, sp, nvalid, C, G,
                                                        (int)Kc, planes, partial, write_xlo);
        }
        rc = check_launch();
        if (rc != RQ_OK) break;
        if (act_sq) {
            act_reduce_kernel<<<(C + 255) / 256, 256, 0, st>>>(partial, (int)(Kc / kPackTile), C, act_sq);
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
        if (variant == 2)
            rc = nprod == 3 ? launch_umma<64, 3>(planes, Kc, C, G, nplanes, b_plane0, H, alpha, b, status, gst)
                            : launch_umma<64, 2, true>(planes, Kc, C, G, nplanes, b_plane0, H, alpha, b, status, gst);
        else if (variant == 0)
            rc = nprod == 3 ? launch_umma<64, 3>(planes, Kc, C, G, nplanes, b_plane0, H, alpha, b, status, gst)
                            : launch_umma<64, 2>(planes, Kc, C, G, nplanes, b_plane0, H, alpha, b, status, gst);
        else
            rc = nprod == 3 ? launch_umma<32, 3>(planes, Kc, C, G, nplanes, b_plane0, H, alpha, b, status, gst)
                            : launch_umma<32, 2>(planes, Kc, C, G, nplanes, b_plane0, H, alpha, b, status, gst);
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
