// fp32-faithful GEMM on the 5th-generation tensor cores for the Cholesky trailing updates, the
// triangular inverse, the GPTQ+ first-order terms and the lazy block update:
//
//     C[z][m, n] = beta * C + alpha * sum_k A[z][m, k] * B[z][n, k] + gamma * Aux[z][m, n]
//
// Operands are fp32 matrices split beforehand into bf16 planes  v = hi + lo  (hi = bf16(v),
// lo = bf16(v - hi)), stored K-contiguous as [plane][row][K].  Every k-step issues the four products
// lo.lo + hi.lo + lo.hi + hi.hi into an fp32 accumulator in tensor memory; as in the Hessian kernel an
// accumulator only collects 128 values of k and the epilogue warps add the windows in registers with
// round-to-nearest adds, because the tensor core's own accumulation truncates.  What is lost is the
// third bf16 term of each operand (2^-17 relative, random sign), the same order as fp32 rounding over
// the k loop.  TMA feeds 128x64 / 256x64 operand tiles (128-byte swizzle, no multicast) through a
// two-stage ring; persistent CTAs walk the tiles of all batches.
#pragma once

#include <cuda.h>

#include "rq_common.cuh"
#include "rq_sm100.cuh"

namespace rq {
namespace tcgemm {

using namespace rq::sm100;

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
constexpr int kStages = 2;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kTmemCols = 512;
constexpr int kWindowBlocks = 2;                       // k-blocks (of 64) per accumulation window
constexpr int kATile = BM * BK * 2, kBTile = BN * BK * 2;
constexpr int kStageBytes = 2 * kATile + 2 * kBTile;
constexpr int kSmemBytes = kStages * kStageBytes + 256 + 1024;
constexpr int kLayoutSW128 = 2, kSBO = 1024;

struct Params {
    int a_row0, b_row0;            // first row of the operand inside its plane tensor
    int a_k0, b_k0;                // first k (elements) inside the plane tensors
    int a_plane, b_plane;          // hi plane index; lo plane = +1
    int a_plane_z, b_plane_z;      // plane increment per batch
    int a_row_z, b_row_z;          // row increment per batch
    int M, N, k_len;               // output extent and k extent (k_len is covered in 64-blocks; padding must be zero)
    int tri;                       // 1: skip tiles that lie wholly below the diagonal (i0 >= tri_col0 + j0 + BN)
    int tri_col0 = 0;              // global column index of C's column 0 (row 0 is global row 0)
    int kmode;                     // 0: all k;  1: k >= i0 (A[m,k] = 0 for k < m);  2: k < j0 + BN (B[n,k] = 0 for k > n);
                                   // 3: k >= j0 (B[n,k] = 0 for k < n)
    int batch;                     // total batch count = nz1 * (number of outer batches)
    float* C; long long ldc, c_z;
    const float* Aux; long long ldaux, aux_z;
    float alpha, beta, gamma;
    // optional inner batch (z = z1 + nz1 * z2; the *_z fields above step with z2): used for the block pairs
    // of one level of the triangular inverse.  n_limit > 0 clips N per inner batch to n_limit - z1 * n_limit_z1.
    int nz1 = 1;
    int a_row_z1 = 0, b_row_z1 = 0, a_k_z1 = 0, b_k_z1 = 0;
    long long c_z1 = 0;
    int n_limit = 0, n_limit_z1 = 0;
    // 1: the planes hold fp16 (11 significant bits each, the caller having scaled the operands into fp16's range by
    // powers of two that alpha undoes); the lo.lo product, 2^-22 relative, is then left out (three products)
    int fp16 = 0;
};

struct TileCtx {
    int i, j, z1, z2, n_eff;
    bool skip;
};

__device__ __forceinline__ TileCtx decode(const Params& p, int t, int MT, int NT) {
    TileCtx c;
    c.i = t % MT;
    c.j = (t / MT) % NT;
    const int z = t / (MT * NT);
    c.z1 = z % p.nz1;
    c.z2 = z / p.nz1;
    c.n_eff = p.N;
    if (p.n_limit > 0) {
        const int lim = p.n_limit - c.z1 * p.n_limit_z1;
        if (lim < c.n_eff) c.n_eff = lim;
    }
    c.skip = (p.tri && c.i * BM >= p.tri_col0 + (c.j + 1) * BN) || c.j * BN >= c.n_eff;
    return c;
}

struct Bars {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tfull[2];
    uint64_t tempty[2];
    uint32_t tmem_slot;
    int abort_flag;
};

// C[0..3] += v without reading C back: the add is performed by the L2 atomic unit (one fp32 round-to-nearest
// add per element, like a load-add-store) and the thread does not wait for it, so the epilogue is not
// limited by the latency of a read round trip per row segment.
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void tile_k_range(const Params& p, int i0, int j0, int& kb0, int& kb1) {
    int k_begin = 0, k_end = p.k_len;
    if (p.kmode == 1) k_begin = i0;
    else if (p.kmode == 3) k_begin = j0;
    else if (p.kmode == 2) k_end = (j0 + BN < p.k_len) ? j0 + BN : p.k_len;
    kb0 = k_begin / BK;
    kb1 = (k_end + BK - 1) / BK;
    if (kb1 < kb0) kb1 = kb0;
}

static __global__ void __launch_bounds__(kThreads, 1)
split_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const Params p,
                  int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    Bars* bars = reinterpret_cast<Bars*>(smem_raw + (tiles - raw) + kStages * kStageBytes);
    volatile int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int MT = (p.M + BM - 1) / BM, NT = (p.N + BN - 1) / BN;
    const int total_tiles = MT * NT * p.batch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
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
                const TileCtx c = decode(p, t, MT, NT);
                if (c.skip) continue;
                const int i = c.i, j = c.j;
                int kb0, kb1;
                tile_k_range(p, i * BM, j * BN, kb0, kb1);
                const int arow = p.a_row0 + c.z2 * p.a_row_z + c.z1 * p.a_row_z1 + i * BM;
                const int brow = p.b_row0 + c.z2 * p.b_row_z + c.z1 * p.b_row_z1 + j * BN;
                const int apl = p.a_plane + c.z2 * p.a_plane_z, bpl = p.b_plane + c.z2 * p.b_plane_z;
                const int ak0 = p.a_k0 + c.z1 * p.a_k_z1, bk0 = p.b_k0 + c.z1 * p.b_k_z1;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t fb = smem_u32(&bars->full[s]);
                    const uint32_t dst = tiles + s * kStageBytes;
                    mbar_expect_tx(fb, kStageBytes);
                    tma_load_3d(dst, &mapA, fb, ak0 + kb * BK, arow, apl);
                    tma_load_3d(dst + kATile, &mapA, fb, ak0 + kb * BK, arow, apl + 1);
                    tma_load_3d(dst + 2 * kATile, &mapB, fb, bk0 + kb * BK, brow, bpl);
                    tma_load_3d(dst + 2 * kATile + kBTile, &mapB, fb, bk0 + kb * BK, brow, bpl + 1);
                }
            }
            if (!ok) {
                const uint32_t inflight = it < (uint32_t)kStages ? it : (uint32_t)kStages;
                for (uint32_t b = 0; b < inflight; ++b) {
                    const uint32_t q = it - 1 - b;
                    const uint32_t fb = smem_u32(&bars->full[q % kStages]);
                    const long long t0 = clock64();
                    while (!mbar_try_wait(fb, (q / kStages) & 1u) && clock64() - t0 < kWaitCycles) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = p.fp16 ? umma_idesc_f16_f32(BM, BN) : umma_idesc_bf16_f32(BM, BN);
            const bool four = p.fp16 == 0;
            uint32_t it = 0, win_iter = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const TileCtx c = decode(p, t, MT, NT);
                if (c.skip) continue;
                int kb0, kb1;
                tile_k_range(p, c.i * BM, c.j * BN, kb0, kb1);
                for (int w0 = kb0; w0 < kb1 && ok; w0 += kWindowBlocks, ++win_iter) {
                    const uint32_t acc = win_iter & 1u, acc_ph = (win_iter >> 1) & 1u;
                    if (!mbar_wait(smem_u32(&bars->tempty[acc]), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    const int w1 = (w0 + kWindowBlocks < kb1) ? w0 + kWindowBlocks : kb1;
                    for (int kb = w0; kb < w1; ++kb, ++it) {
                        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                        if (!mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_hi = tiles + s * kStageBytes, a_lo = a_hi + kATile;
                        const uint32_t b_hi = a_hi + 2 * kATile, b_lo = b_hi + kBTile;
#pragma unroll
                        for (int k = 0; k < BK / UK; ++k) {
                            const uint32_t koff = k * UK * 2;
                            const uint64_t dah = umma_smem_desc(a_hi + koff, kSBO, kLayoutSW128);
                            const uint64_t dal = umma_smem_desc(a_lo + koff, kSBO, kLayoutSW128);
                            const uint64_t dbh = umma_smem_desc(b_hi + koff, kSBO, kLayoutSW128);
                            const uint64_t dbl = umma_smem_desc(b_lo + koff, kSBO, kLayoutSW128);
                            const uint32_t keep = (kb != w0 || k != 0) ? 1u : 0u;    // a window's first MMA overwrites
                            if (four) umma_bf16(d_tmem, dal, dbl, idesc, keep);
                            umma_bf16(d_tmem, dah, dbl, idesc, four ? 1u : keep);
                            umma_bf16(d_tmem, dal, dbh, idesc, 1u);
                            umma_bf16(d_tmem, dah, dbh, idesc, 1u);
                        }
                        umma_commit(smem_u32(&bars->empty[s]));
                    }
                    if (ok) umma_commit(smem_u32(&bars->tfull[acc]));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: 8 warps, warp (2+e) owns
        // tensor-memory lanes 32*(warp%4).. and the column half e/4; 128 running sums per thread
        const int q = warp & 3, half = (warp - 2) >> 2;
        uint32_t win_iter = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
            const TileCtx c = decode(p, t, MT, NT);
            if (c.skip) continue;
            const int i = c.i, j = c.j, n_eff = c.n_eff;
            int kb0, kb1;
            tile_k_range(p, i * BM, j * BN, kb0, kb1);
            const int row0 = i * BM + q * 32, row = row0 + lane;
            const int colbase = j * BN + half * 128;
            bool use[4];
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                const int col0 = colbase + cb * 32;
                use[cb] = !(col0 >= n_eff || row0 >= p.M || (p.tri && p.tri_col0 + col0 + 31 < row0));
            }
            float run[128];
#pragma unroll
            for (int e = 0; e < 128; ++e) run[e] = 0.f;
            for (int w0 = kb0; w0 < kb1; w0 += kWindowBlocks, ++win_iter) {
                const uint32_t acc = win_iter & 1u, acc_ph = (win_iter >> 1) & 1u;
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
            if (row < p.M) {
                float* crow = p.C + (long long)c.z2 * p.c_z + (long long)c.z1 * p.c_z1 + (long long)row * p.ldc;
                const float* xrow = p.Aux ? p.Aux + (long long)c.z2 * p.aux_z + (long long)row * p.ldaux : nullptr;
                const bool vec_ok = ((reinterpret_cast<uintptr_t>(crow) | (xrow ? reinterpret_cast<uintptr_t>(xrow) : 0)) & 15) == 0;
#pragma unroll
                for (int cb = 0; cb < 4; ++cb) {
                    const int col0 = colbase + cb * 32;
                    if (!use[cb]) continue;
                    if (vec_ok && col0 + 32 <= n_eff && p.beta == 1.f) {
                        const float4* x4 = xrow ? reinterpret_cast<const float4*>(xrow + col0) : nullptr;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            float4 o = make_float4(p.alpha * run[cb * 32 + 4 * e + 0], p.alpha * run[cb * 32 + 4 * e + 1],
                                                   p.alpha * run[cb * 32 + 4 * e + 2], p.alpha * run[cb * 32 + 4 * e + 3]);
                            if (x4) {
                                const float4 x = x4[e];
                                o.x += p.gamma * x.x; o.y += p.gamma * x.y; o.z += p.gamma * x.z; o.w += p.gamma * x.w;
                            }
                            red_add_v4(crow + col0 + 4 * e, o.x, o.y, o.z, o.w);
                        }
                    } else if (vec_ok && col0 + 32 <= n_eff) {
                        float4* c4 = reinterpret_cast<float4*>(crow + col0);
                        const float4* x4 = xrow ? reinterpret_cast<const float4*>(xrow + col0) : nullptr;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            float4 o = (p.beta != 0.f) ? c4[e] : make_float4(0.f, 0.f, 0.f, 0.f);
                            if (p.beta != 1.f) { o.x *= p.beta; o.y *= p.beta; o.z *= p.beta; o.w *= p.beta; }
                            o.x += p.alpha * run[cb * 32 + 4 * e + 0];
                            o.y += p.alpha * run[cb * 32 + 4 * e + 1];
                            o.z += p.alpha * run[cb * 32 + 4 * e + 2];
                            o.w += p.alpha * run[cb * 32 + 4 * e + 3];
                            if (x4) {
                                const float4 x = x4[e];
                                o.x += p.gamma * x.x; o.y += p.gamma * x.y; o.z += p.gamma * x.z; o.w += p.gamma * x.w;
                            }
                            c4[e] = o;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            if (col0 + e < n_eff) {
                                float o = (p.beta != 0.f) ? p.beta * crow[col0 + e] : 0.f;
                                o += p.alpha * run[cb * 32 + e];
                                if (xrow) o += p.gamma * xrow[col0 + e];
                                crow[col0 + e] = o;
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
// operand splitting.  Destination planes: [plane][rows_total][Kp] bf16, hi in `plane`, lo in plane+1.
// ------------------------------------------------------------------------------------------
struct SplitArgs {
    const float* src; long long ld, src_z;      // source matrix, row stride, batch stride (elements)
    int rows, cols;                             // source extent
    __nv_bfloat16* dst; long long Kp, plane_stride;   // plane row stride and plane size (elements)
    int plane, plane_z;                         // hi plane index and its per-batch increment
    int dst_row0, dst_row_z, dst_k0;            // where the block lands inside the plane
    int pad_k_to;                               // zero-fill k in [cols_k, pad_k_to) (relative to dst_k0); 0 = no fill
    // second batch dimension (blockIdx.z = z * nz1 + z1): a series of equally shaped blocks of one matrix
    int nz1 = 1;
    long long src_z1 = 0;                       // source offset per z1 (elements)
    int dst_row_z1 = 0, dst_k_z1 = 0;           // destination offsets per z1
    // when src_cols_total > 0 the block's columns are clipped to src_cols_total - (src_col0 + z1 * src_col_z1)
    int src_col0 = 0, src_col_z1 = 0, src_cols_total = 0;
    // likewise for rows: src_rows_total - (src_row0 + z1 * src_row_z1)
    int src_row0 = 0, src_row_z1 = 0, src_rows_total = 0;
    int upper_only = 0;                         // transpose: skip source tiles that lie strictly below the diagonal
    int vec4 = 0;                               // set by the launcher when every offset is a multiple of 4 elements
    // fp16 planes: v * scale (a power of two chosen by the caller so that the products stay inside fp16's range)
    // split into two fp16 values; otherwise two bf16 values of v itself
    int fp16 = 0;
    float scale = 1.f;
};

__device__ __forceinline__ void split2(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// 16-bit patterns of hi and lo: bf16 (v = hi + lo to 16 bits) or fp16 of the scaled value (22 bits)
__device__ __forceinline__ void split2(float v, const SplitArgs& a, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    if (a.fp16) {
        const float w = v * a.scale;
        const __half h = __float2half_rn(w);
        const __half l = __float2half_rn(w - __half2float(h));
        hi = __ushort_as_bfloat16(__half_as_ushort(h));
        lo = __ushort_as_bfloat16(__half_as_ushort(l));
    } else {
        hi = __float2bfloat16_rn(v);
        lo = __float2bfloat16_rn(v - __bfloat162float(hi));
    }
}

__device__ __forceinline__ int split_clipped_rows(const SplitArgs& a, int z1) {
    int rows = a.rows;
    if (a.src_rows_total > 0) {
        const int lim = a.src_rows_total - (a.src_row0 + z1 * a.src_row_z1);
        if (lim < rows) rows = lim;
    }
    return rows;
}

__device__ __forceinline__ int split_clipped_cols(const SplitArgs& a, int z1) {
    int cols = a.cols;
    if (a.src_cols_total > 0) {
        const int lim = a.src_cols_total - (a.src_col0 + z1 * a.src_col_z1);
        if (lim < cols) cols = lim;
    }
    return cols;
}

// rows stay rows: dst[row0 + r][k0 + c] = src[r][c].  grid (ceil(kspan/1024), rows (capped), batch)
static __global__ void __launch_bounds__(256) split_rows_kernel(const SplitArgs a) {
    const int z = blockIdx.z / a.nz1, z1 = blockIdx.z - z * a.nz1;
    const float* src = a.src + (long long)z * a.src_z + (long long)z1 * a.src_z1;
    __nv_bfloat16* hi = a.dst + (long long)(a.plane + z * a.plane_z) * a.plane_stride;
    __nv_bfloat16* lo = hi + a.plane_stride;
    const int cols = split_clipped_cols(a, z1);
    if (cols <= 0 && a.pad_k_to <= 0) return;
    const int kspan = a.pad_k_to > cols ? a.pad_k_to : cols;
    const int rows = split_clipped_rows(a, z1);
    for (int r = blockIdx.y; r < rows; r += gridDim.y) {
        const long long drow =
            (long long)(a.dst_row0 + z * a.dst_row_z + z1 * a.dst_row_z1 + r) * a.Kp + a.dst_k0 + z1 * a.dst_k_z1;
        const float* srow = src + (long long)r * a.ld;
        if (a.vec4) {
            for (int c = (blockIdx.x * 256 + threadIdx.x) * 4; c < kspan; c += gridDim.x * 1024) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c + 3 < cols) {
                    v = *reinterpret_cast<const float4*>(srow + c);
                } else {
                    if (c + 0 < cols) v.x = srow[c + 0];
                    if (c + 1 < cols) v.y = srow[c + 1];
                    if (c + 2 < cols) v.z = srow[c + 2];
                }
                __nv_bfloat16 h0, h1, h2, h3, l0, l1, l2, l3;
                split2(v.x, a, h0, l0); split2(v.y, a, h1, l1); split2(v.z, a, h2, l2); split2(v.w, a, h3, l3);
                if (c + 3 < kspan) {
                    __nv_bfloat162 hp[2] = {__halves2bfloat162(h0, h1), __halves2bfloat162(h2, h3)};
                    __nv_bfloat162 lp[2] = {__halves2bfloat162(l0, l1), __halves2bfloat162(l2, l3)};
                    *reinterpret_cast<uint2*>(hi + drow + c) = *reinterpret_cast<const uint2*>(hp);
                    *reinterpret_cast<uint2*>(lo + drow + c) = *reinterpret_cast<const uint2*>(lp);
                } else {
                    const __nv_bfloat16 hs[4] = {h0, h1, h2, h3}, ls[4] = {l0, l1, l2, l3};
                    for (int e = 0; e < 4 && c + e < kspan; ++e) { hi[drow + c + e] = hs[e]; lo[drow + c + e] = ls[e]; }
                }
            }
        } else {
            for (int c = blockIdx.x * 256 + threadIdx.x; c < kspan; c += gridDim.x * 256) {
                const float v = c < cols ? srow[c] : 0.f;
                __nv_bfloat16 h, l;
                split2(v, a, h, l);
                hi[drow + c] = h;
                lo[drow + c] = l;
            }
        }
    }
}

// transpose: dst[row0 + c][k0 + r] = src[r][c]   (source rows become k).  One CTA moves 64 source rows x 32 columns;
// a thread stores two consecutive k.  grid (ceil(cols/32), ceil(kspan/64), batch)
static __global__ void __launch_bounds__(256) split_transpose_kernel(const SplitArgs a) {
    __shared__ float tile[64][33];
    const int z = blockIdx.z / a.nz1, z1 = blockIdx.z - z * a.nz1;
    const float* src = a.src + (long long)z * a.src_z + (long long)z1 * a.src_z1;
    __nv_bfloat16* hi = a.dst + (long long)(a.plane + z * a.plane_z) * a.plane_stride;
    __nv_bfloat16* lo = hi + a.plane_stride;
    const int cols = split_clipped_cols(a, z1);
    const int rows = split_clipped_rows(a, z1);
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 64;
    if (c0 >= cols || (r0 >= rows && a.pad_k_to <= rows)) return;
    if (a.upper_only && r0 > c0 + 31) return;            // every element of the tile has row > column
#pragma unroll
    for (int rr = ty; rr < 64; rr += 8) {
        const int r = r0 + rr, c = c0 + tx;
        tile[rr][tx] = (r < rows && c < cols) ? src[(long long)r * a.ld + c] : 0.f;
    }
    __syncthreads();
    const int kspan = a.pad_k_to > rows ? a.pad_k_to : rows;
    const bool pair_ok = ((a.Kp | a.dst_k0 | a.dst_k_z1 | a.plane_stride) & 1) == 0;
#pragma unroll
    for (int cc = ty; cc < 32; cc += 8) {
        const int c = c0 + cc, r = r0 + 2 * tx;           // r runs along k of the destination
        if (c >= cols || r >= kspan) continue;
        const long long d =
            (long long)(a.dst_row0 + z * a.dst_row_z + z1 * a.dst_row_z1 + c) * a.Kp + a.dst_k0 + z1 * a.dst_k_z1 + r;
        __nv_bfloat16 h0, l0, h1, l1;
        split2(tile[2 * tx][cc], a, h0, l0);
        split2(tile[2 * tx + 1][cc], a, h1, l1);
        if (pair_ok && r + 1 < kspan) {
            *reinterpret_cast<__nv_bfloat162*>(hi + d) = __halves2bfloat162(h0, h1);
            *reinterpret_cast<__nv_bfloat162*>(lo + d) = __halves2bfloat162(l0, l1);
        } else {
            hi[d] = h0; lo[d] = l0;
            if (r + 1 < kspan) { hi[d + 1] = h1; lo[d + 1] = l1; }
        }
    }
}

// ------------------------------------------------------------------------------------------
// host helpers
// ------------------------------------------------------------------------------------------
struct PlaneTensor {
    void* base;            // bf16 [planes][rows][Kp]
    long long Kp, rows, planes;
};

inline int encode_planes(CUtensorMap* map, const PlaneTensor& t, int box_rows) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return RQ_ERR_CUDA;
    cuuint64_t dims[3] = {(cuuint64_t)t.Kp, (cuuint64_t)t.rows, (cuuint64_t)t.planes};
    cuuint64_t strides[2] = {(cuuint64_t)t.Kp * 2, (cuuint64_t)t.Kp * 2 * (cuuint64_t)t.rows};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, t.base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RQ_OK : RQ_ERR_CUDA;
}

inline int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

inline int launch(const PlaneTensor& A, const PlaneTensor& B, const Params& p, int* status, cudaStream_t st) {
    if (p.M <= 0 || p.N <= 0 || p.batch <= 0) return RQ_OK;
    CUtensorMap mapA, mapB;
    int rc = encode_planes(&mapA, A, BM);
    if (rc != RQ_OK) return rc;
    rc = encode_planes(&mapB, B, BN);
    if (rc != RQ_OK) return rc;
    if (cudaFuncSetAttribute(split_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
        return RQ_ERR_CUDA;
    const long long MT = (p.M + BM - 1) / BM, NT = (p.N + BN - 1) / BN;
    long long total = MT * NT * p.batch;
    const int grid = (int)(total < sm_count() ? total : sm_count());
    split_gemm_kernel<<<grid, kThreads, kSmemBytes, st>>>(mapA, mapB, p, status);
    return check_launch();
}

inline int split_rows(const SplitArgs& a_in, int batch, cudaStream_t st) {
    SplitArgs a = a_in;
    if (a.rows <= 0 || batch <= 0 || a.nz1 <= 0) return RQ_OK;
    const int kspan = a.pad_k_to > a.cols ? a.pad_k_to : a.cols;
    if (kspan <= 0) return RQ_OK;
    a.vec4 = ((reinterpret_cast<uintptr_t>(a.src) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.dst) & 7) == 0 &&
              ((a.ld | a.src_z | a.src_z1 | a.Kp | a.plane_stride) & 3) == 0 && ((a.dst_k0 | a.dst_k_z1) & 3) == 0)
                 ? 1 : 0;
    dim3 grid((unsigned)((kspan + 1023) / 1024), (unsigned)(a.rows < 16384 ? a.rows : 16384), (unsigned)(batch * a.nz1));
    split_rows_kernel<<<grid, 256, 0, st>>>(a);
    return check_launch();
}

inline int split_transpose(const SplitArgs& a, int batch, cudaStream_t st) {
    if (a.rows <= 0 || a.cols <= 0 || batch <= 0 || a.nz1 <= 0) return RQ_OK;
    const int kspan = a.pad_k_to > a.rows ? a.pad_k_to : a.rows;
    dim3 grid((unsigned)((a.cols + 31) / 32), (unsigned)((kspan + 63) / 64), (unsigned)(batch * a.nz1));
    split_transpose_kernel<<<grid, 256, 0, st>>>(a);
    return check_launch();
}

}  // namespace tcgemm
}  // namespace rq
