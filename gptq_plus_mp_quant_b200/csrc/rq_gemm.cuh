// fp32 GEMM tile engine (CUDA cores, FMA accumulation) for the parts of the path whose
// results feed the integer rounding decisions and therefore stay in full fp32: trailing updates
// of the blocked Cholesky, triangular inverse, GPTQ+ first-order terms, lazy block update.
//
//   C[i,j] = beta*C[i,j] + alpha * sum_k A[i,k] * B'(k,j) + gamma * Aux[i,j]
//
// A is row-major [M,K]; B is row-major [K,N] (kBT = false) or row-major [N,K] (kBT = true,
// i.e. C = A.B^T).  128x128 tiles, 256 threads, 8x8 outputs per thread, 16-deep k slabs with
// register prefetch.  Triangular operands are handled by restricting each tile's k range
// (tile-granular: operands hold explicit zeros in their unused triangle).
#pragma once

#include "rq_common.cuh"

namespace rq {
namespace gemm {

constexpr int TM = 128, TN = 128, TK = 16, kThreads = 256;

struct Args {
    const float* A; int64_t lda;
    const float* B; int64_t ldb;
    float* C; int64_t ldc;
    const float* Aux; int64_t ldaux;      // optional, added as gamma*Aux
    int M, N, K;
    float alpha, beta, gamma;
    int k_begin, k_end;                   // k range of this tile (already clipped to [0, K))
};

// Computes one 128x128 tile at (i0, j0).  smem: As[2][TK][TM+4], Bs[2][TK][TN+4] floats.
template <bool kBT>
__device__ __forceinline__ void tile(const Args& g, int i0, int j0, float* smem) {
    float (*As)[TK][TM + 4] = reinterpret_cast<float (*)[TK][TM + 4]>(smem);
    float (*Bs)[TK][TN + 4] = reinterpret_cast<float (*)[TK][TN + 4]>(smem + 2 * TK * (TM + 4));
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;

    // global -> register staging: A slab is [TM rows][TK k] = 2048 floats -> 8 per thread
    // thread t loads row (t >> 1), k offset (t & 1) * 8 .. +8
    const int a_row = tid >> 1, a_k = (tid & 1) * 8;
    // B (kBT: [TN rows][TK k], same pattern; else [TK k][TN cols]: row t>>4, cols (t&15)*8 .. +8)
    const int b_row = kBT ? (tid >> 1) : (tid >> 4);
    const int b_col = kBT ? ((tid & 1) * 8) : ((tid & 15) * 8);
    const bool a_vec = (g.lda & 3) == 0 && (reinterpret_cast<uintptr_t>(g.A) & 15) == 0;
    const bool b_vec = (g.ldb & 3) == 0 && (reinterpret_cast<uintptr_t>(g.B) & 15) == 0;

    float ra[8], rb[8];
    auto load_slab = [&](int k0) {
        {   // A[i0 + a_row][k0 + a_k .. +8]
            const int r = i0 + a_row;
            const int kk = k0 + a_k;
            const float* p = g.A + (int64_t)r * g.lda + kk;
            if (r < g.M && kk + 8 <= g.k_end && a_vec) {
                const float4 v0 = *reinterpret_cast<const float4*>(p);
                const float4 v1 = *reinterpret_cast<const float4*>(p + 4);
                ra[0] = v0.x; ra[1] = v0.y; ra[2] = v0.z; ra[3] = v0.w;
                ra[4] = v1.x; ra[5] = v1.y; ra[6] = v1.z; ra[7] = v1.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) ra[e] = (r < g.M && kk + e < g.k_end) ? p[e] : 0.f;
            }
        }
        if (kBT) {   // B[j0 + b_row][k0 + b_col .. +8]
            const int r = j0 + b_row;
            const int kk = k0 + b_col;
            const float* p = g.B + (int64_t)r * g.ldb + kk;
            if (r < g.N && kk + 8 <= g.k_end && b_vec) {
                const float4 v0 = *reinterpret_cast<const float4*>(p);
                const float4 v1 = *reinterpret_cast<const float4*>(p + 4);
                rb[0] = v0.x; rb[1] = v0.y; rb[2] = v0.z; rb[3] = v0.w;
                rb[4] = v1.x; rb[5] = v1.y; rb[6] = v1.z; rb[7] = v1.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) rb[e] = (r < g.N && kk + e < g.k_end) ? p[e] : 0.f;
            }
        } else {     // B[k0 + b_row][j0 + b_col .. +8]
            const int kk = k0 + b_row;
            const int c = j0 + b_col;
            const float* p = g.B + (int64_t)kk * g.ldb + c;
            if (kk < g.k_end && c + 8 <= g.N && b_vec) {
                const float4 v0 = *reinterpret_cast<const float4*>(p);
                const float4 v1 = *reinterpret_cast<const float4*>(p + 4);
                rb[0] = v0.x; rb[1] = v0.y; rb[2] = v0.z; rb[3] = v0.w;
                rb[4] = v1.x; rb[5] = v1.y; rb[6] = v1.z; rb[7] = v1.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) rb[e] = (kk < g.k_end && c + e < g.N) ? p[e] : 0.f;
            }
        }
    };
    auto store_slab = [&](int buf) {
#pragma unroll
        for (int e = 0; e < 8; ++e) As[buf][a_k + e][a_row] = ra[e];
        if (kBT) {
#pragma unroll
            for (int e = 0; e < 8; ++e) Bs[buf][b_col + e][b_row] = rb[e];
        } else {
            *reinterpret_cast<float4*>(&Bs[buf][b_row][b_col]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
            *reinterpret_cast<float4*>(&Bs[buf][b_row][b_col + 4]) = make_float4(rb[4], rb[5], rb[6], rb[7]);
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    const int kb = g.k_begin - (g.k_begin % TK);            // slab-aligned start (extra k read real data or masked 0)
    int buf = 0;
    if (kb < g.k_end) {
        // the first slab may start before k_begin only when k_begin is not slab aligned; callers pass aligned values
        load_slab(kb);
        store_slab(0);
    }
    __syncthreads();
    for (int k0 = kb; k0 < g.k_end; k0 += TK) {
        const bool more = k0 + TK < g.k_end;
        if (more) load_slab(k0 + TK);
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) store_slab(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }

    // epilogue: rows ty*4+{0..3}, 64+ty*4+{0..3}; cols tx*4+{0..3}, 64+tx*4+{0..3}
    const bool c_vec = (g.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(g.C) & 15) == 0 &&
                       (g.Aux == nullptr || ((g.ldaux & 3) == 0 && (reinterpret_cast<uintptr_t>(g.Aux) & 15) == 0));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = i0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (r >= g.M) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = j0 + (h == 0 ? tx * 4 : 64 + tx * 4);
            float* cp = g.C + (int64_t)r * g.ldc + c;
            const float* xp = g.Aux ? g.Aux + (int64_t)r * g.ldaux + c : nullptr;
            if (c + 4 <= g.N && c_vec) {
                float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
                if (g.beta != 0.f) {
                    o = *reinterpret_cast<const float4*>(cp);
                    if (g.beta != 1.f) { o.x *= g.beta; o.y *= g.beta; o.z *= g.beta; o.w *= g.beta; }
                }
                o.x += g.alpha * acc[i][h * 4 + 0];
                o.y += g.alpha * acc[i][h * 4 + 1];
                o.z += g.alpha * acc[i][h * 4 + 2];
                o.w += g.alpha * acc[i][h * 4 + 3];
                if (xp) {
                    const float4 x = *reinterpret_cast<const float4*>(xp);
                    o.x += g.gamma * x.x; o.y += g.gamma * x.y; o.z += g.gamma * x.z; o.w += g.gamma * x.w;
                }
                *reinterpret_cast<float4*>(cp) = o;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (c + e < g.N) {
                        float o = g.beta != 0.f ? g.beta * cp[e] : 0.f;
                        o += g.alpha * acc[i][h * 4 + e];
                        if (xp) o += g.gamma * xp[e];
                        cp[e] = o;
                    }
                }
            }
        }
    }
}

constexpr size_t kSmemBytes = (size_t)(2 * TK * (TM + 4) + 2 * TK * (TN + 4)) * sizeof(float);

}  // namespace gemm
}  // namespace rq
