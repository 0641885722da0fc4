// Damped inverse-Hessian factor: Hinv = upper Cholesky factor U of (H + lambda I)^-1, i.e.
// H^-1 = U^T U, which is what the reference obtains from potrf -> potri -> potrf(upper).
//
// B200 route (2/3 C^3 flops instead of 4/3 C^3):  write P = H + lambda I = R R^T with R UPPER
// triangular (a Cholesky factorisation that runs from the last column to the first); then
// P^-1 = R^-T R^-1, so U = R^-1, an upper-triangular inverse.
//   phase 1  blocked right-looking "reverse" Cholesky, 128-wide block columns, last to first:
//            diagonal block factored and inverted inside one CTA (fp32, register-distributed); panel R_ik = A_ik.inv(R_kk)^T
//            and trailing update A_ij -= R_ik.R_jk^T as fp32 GEMM tiles;
//   phase 2  recursive-doubling triangular inverse: inv([[A,B],[0,D]]) = [[A^-1, -A^-1.B.D^-1],[0, D^-1]],
//            two batched GEMM launches per level.
// All G groups of a linear are processed in the same launches (grid.z).
#include "rq_common.cuh"
#include "rq_gemm.cuh"
#include "rq_umma_gemm.cuh"

namespace rq {
namespace chol {

constexpr int NB = 128;                       // block-column width = GEMM tile edge
constexpr int kDiagThreads = 512;

// ------------------------------------------------------------------------------------------
// mean of the dead-fixed diagonal per group (one block per group)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) diag_mean_kernel(const float* __restrict__ H, int C, float* __restrict__ mean) {
    __shared__ double red[8];
    const float* Hg = H + (int64_t)blockIdx.x * C * C;
    double s = 0.0;
    for (int c = threadIdx.x; c < C; c += 256) {
        const float d = Hg[(int64_t)c * C + c];
        s += (d == 0.f) ? 1.0 : (double)d;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += red[w];
        mean[blockIdx.x] = (float)(t / (double)C);
    }
}

// ------------------------------------------------------------------------------------------
// Equilibration by powers of two.  dsc[g][i] = 2^-h_i with h_i chosen so that the damped diagonal entry
// a_ii * dsc_i^2 lies in [0.5, 2).  The factorisation then runs on A' = D A D (D = diag(dsc)): scaling by powers
// of two is exact and commutes with every fp32 operation of the factorisation, so R' = D R and
// U' = R'^-1 = U D^-1 are the same numbers as without it, differently scaled; the result is scaled back at the
// end, Hinv[i][j] = U'[i][j] * dsc[j].  What it buys: every entry of R' is below sqrt(2), which lets the operand
// planes of the trailing updates be fp16 (22 bits in two planes) with ONE fixed scale, whatever the spread of the
// channels' energies.  Padding rows and bad diagonals (non-positive, non-finite) keep dsc = 1.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) equil_kernel(const float* __restrict__ H, const int64_t* __restrict__ perm,
                                                    const float* __restrict__ mean, const float* __restrict__ factor,
                                                    int C, int Cp, float* __restrict__ dsc) {
    const int g = blockIdx.y;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= Cp) return;
    float d = 1.f;
    if (i < C) {
        const int64_t pi = perm ? perm[i] : i;
        float a = H[(int64_t)g * C * C + pi * C + pi];
        if (a == 0.f) a = 1.f;
        a += factor[g] * mean[g];
        if (a > 0.f && a <= 3.0e38f) {
            const int e = ilogbf(a);
            const int h = (e >= 0) ? (e + 1) / 2 : -((-e) / 2);
            d = exp2f((float)-(h < -60 ? -60 : (h > 60 ? 60 : h)));
        }
    }
    dsc[(int64_t)g * Cp + i] = d;
}

// ------------------------------------------------------------------------------------------
// A[g][i][j] = dsc_i * H[g][perm[i]][perm[j]] * dsc_j (+ dead fix, + damping on the diagonal), padded to Cp with
// an identity block.  Only the upper triangle is consumed afterwards.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_kernel(const float* __restrict__ H, const int64_t* __restrict__ perm,
                                                     const float* __restrict__ mean, const float* __restrict__ factor,
                                                     const float* __restrict__ dsc, int C, int Cp,
                                                     float* __restrict__ A) {
    const int g = blockIdx.z;
    const int i = blockIdx.y;
    const float* Hg = H + (int64_t)g * C * C;
    float* Arow = A + ((int64_t)g * Cp + i) * Cp;
    const float* dg = dsc + (int64_t)g * Cp;
    const float lambda = factor[g] * mean[g];
    const float di = dg[i];
    const int64_t pi = (i < C) ? (perm ? perm[i] : i) : 0;
    for (int j = blockIdx.x * 256 + threadIdx.x; j < Cp; j += gridDim.x * 256) {
        float v;
        if (i < C && j < C) {
            const int64_t pj = perm ? perm[j] : j;
            v = Hg[pi * C + pj];
            if (i == j) {
                if (v == 0.f) v = 1.f;               // dead input channel
                v += lambda;
            }
            v = (v * di) * dg[j];
        } else {
            v = (i == j) ? 1.f : 0.f;
        }
        Arow[j] = v;
    }
}

// ------------------------------------------------------------------------------------------
// Diagonal block k: A_kk = R_kk R_kk^T (R upper) and U_kk = R_kk^-1.  One CTA of 512 threads per group, the
// block and its inverse in shared memory, fp32 throughout with correctly rounded division and square root: the
// accuracy class of an fp32 LAPACK potrf / trtri on the block, which is what the reference runs.  (fp64
// arithmetic runs at 1/64 of the fp32 rate on this part; an unblocked column-by-column formulation with CTA-wide
// barriers per column was latency-bound at ~1300 cycles per column.)
// The 128-wide block is itself blocked 4 x 32, last sub-block first:
//   sub-block factor + inverse  one warp, row i (factor) / column j (inverse) in the registers of lane i / j,
//                               the pivot column travels through a 32-float shared buffer, no CTA barrier;
//   panel                       R_ib = A_ib . W_bb^T           (W_bb = R_bb^-1), 32x32x32 jobs of 64 threads;
//   trailing                    A_ij -= R_ib . R_jb^T          for i <= j < b;
// then the inverse of the block-triangular R by recursive doubling (sub-block pairs, then the 64-wide pair):
//   U_ab = -(U_aa . R_ab) . U_bb, the inner product parked in the unused lower blocks of the inverse.
// ------------------------------------------------------------------------------------------
constexpr int kDiagLd = NB + 4;               // fp32 row stride: rows 4 banks apart, rows 16-byte aligned
constexpr int SB = 32;                        // sub-block width

// acc[x][y] += sum_k A[4*tr+x][k] * B[tc+8*y][k], k < 32 (both operands k-contiguous).  Output columns are
// interleaved over the 8 threads of a row group so that their B rows are consecutive: conflict-free 16-byte loads.
__device__ __forceinline__ void diag_job_nt(float (&acc)[4][4], const float* __restrict__ Ab, const float* __restrict__ Bb,
                                            int tr, int tc) {
#pragma unroll
    for (int k = 0; k < SB; k += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) a[x] = *reinterpret_cast<const float4*>(Ab + (4 * tr + x) * kDiagLd + k);
#pragma unroll
        for (int y = 0; y < 4; ++y) b[y] = *reinterpret_cast<const float4*>(Bb + (tc + 8 * y) * kDiagLd + k);
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) {
                acc[x][y] = fmaf(a[x].x, b[y].x, acc[x][y]);
                acc[x][y] = fmaf(a[x].y, b[y].y, acc[x][y]);
                acc[x][y] = fmaf(a[x].z, b[y].z, acc[x][y]);
                acc[x][y] = fmaf(a[x].w, b[y].w, acc[x][y]);
            }
    }
}

// acc[x][y] += sum_k A[4*tr+x][k] * B[k][4*tc+y], k < 32 (A k-contiguous, B column-contiguous)
__device__ __forceinline__ void diag_job_nn(float (&acc)[4][4], const float* __restrict__ Ab, const float* __restrict__ Bb,
                                            int tr, int tc) {
#pragma unroll
    for (int k = 0; k < SB; k += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) a[x] = *reinterpret_cast<const float4*>(Ab + (4 * tr + x) * kDiagLd + k);
#pragma unroll
        for (int l = 0; l < 4; ++l) b[l] = *reinterpret_cast<const float4*>(Bb + (k + l) * kDiagLd + 4 * tc);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const float av[4] = {a[x].x, a[x].y, a[x].z, a[x].w};
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                acc[x][0] = fmaf(av[l], b[l].x, acc[x][0]);
                acc[x][1] = fmaf(av[l], b[l].y, acc[x][1]);
                acc[x][2] = fmaf(av[l], b[l].z, acc[x][2]);
                acc[x][3] = fmaf(av[l], b[l].w, acc[x][3]);
            }
        }
    }
}

__device__ __forceinline__ void diag_store(float* __restrict__ Cb, const float (&acc)[4][4], int tr, int tc, float sign) {
#pragma unroll
    for (int x = 0; x < 4; ++x)
        *reinterpret_cast<float4*>(Cb + (4 * tr + x) * kDiagLd + 4 * tc) =
            make_float4(sign * acc[x][0], sign * acc[x][1], sign * acc[x][2], sign * acc[x][3]);
}

// One warp: the 32x32 block at Sb (upper part valid) becomes R (upper, zero below), Vb receives R^-1 (upper;
// the part below the diagonal is left as it is, i.e. zero).  Returns non-zero when a pivot was not positive.
// 1/sqrt(pivot) comes from the hardware approximation plus one Newton step (about one ulp); the column is scaled by
// it instead of being divided by the square root, which takes two long-latency operations out of the chain between
// consecutive pivots.  That chain is: scale -> update of the next pivot row's entry -> broadcast by shuffle; the
// rest of the rank-1 update travels through shared memory off the critical path.
__device__ __forceinline__ int diag_factor_sub(float* __restrict__ Sb, float* __restrict__ Vb, float* __restrict__ colbuf,
                                               float* __restrict__ rdiag, int lane) {
    float m[SB];
#pragma unroll
    for (int j = 0; j < SB; ++j) m[j] = Sb[lane * kDiagLd + j];        // entries left of the diagonal are never used
    int bad = 0;
    float d = __shfl_sync(0xffffffffu, m[SB - 1], SB - 1);
    float4 pend[SB / 4] = {};                                          // column c+1 as read back from shared memory
    float rprev = 0.f;
#pragma unroll
    for (int c = SB - 1; c >= 0; --c) {
        if (!(d > 0.f)) bad = 1;                                       // catches <= 0 and NaN
        float rinv = rsqrtf(d);
        rinv = fmaf(0.5f * rinv, fmaf(-d * rinv, rinv, 1.f), rinv);
        const float r = (lane == c) ? d * rinv : ((lane < c) ? m[c] * rinv : 0.f);
        // the two entries the next two pivots depend on go by shuffle ...
        if (c > 0) {
            const float dn = fmaf(-r, r, m[c - 1]);                    // meaningful in lane c-1: the next pivot
            const float rho = __shfl_sync(0xffffffffu, r, c - 1);
            d = __shfl_sync(0xffffffffu, dn, c - 1);
            m[c - 1] = fmaf(-r, rho, m[c - 1]);
        }
        if (c > 1) m[c - 2] = fmaf(-r, __shfl_sync(0xffffffffu, r, c - 2), m[c - 2]);
        Sb[lane * kDiagLd + c] = r;
        if (lane == c) rdiag[c] = rinv;
        float* cb = colbuf + (c & 1) * SB;                             // two buffers: one warp barrier per column
        cb[lane] = r;
        // ... the rest of the rank-1 update m[i][j] -= R[i][c] R[j][c] (j < c-2) through shared memory, applied one
        // column late so that its round trip stays off the pivot chain: here column c+1, j < c-1
        if (c < SB - 1) {
#pragma unroll
            for (int j4 = SB / 4 - 1; j4 >= 0; --j4) {
                if (4 * j4 + 3 < c - 1) m[4 * j4 + 3] = fmaf(-rprev, pend[j4].w, m[4 * j4 + 3]);
                if (4 * j4 + 2 < c - 1) m[4 * j4 + 2] = fmaf(-rprev, pend[j4].z, m[4 * j4 + 2]);
                if (4 * j4 + 1 < c - 1) m[4 * j4 + 1] = fmaf(-rprev, pend[j4].y, m[4 * j4 + 1]);
                if (4 * j4 + 0 < c - 1) m[4 * j4 + 0] = fmaf(-rprev, pend[j4].x, m[4 * j4 + 0]);
            }
        }
        __syncwarp();
#pragma unroll
        for (int j4 = 0; j4 < SB / 4; ++j4)
            if (4 * j4 < c - 2) pend[j4] = *reinterpret_cast<const float4*>(cb + 4 * j4);
        rprev = r;
    }
    __syncwarp();
    // inverse: lane j owns column j; W[c][j] = -(sum_{c<l<=j} R[c][l] W[l][j]) / R[c][c], W[j][j] = 1 / R[j][j];
    // terms are added from the far end so that the newest entry closes the chain
    float w[SB];
#pragma unroll
    for (int c = 0; c < SB; ++c) w[c] = 0.f;
#pragma unroll
    for (int c = SB - 1; c >= 0; --c) {
        float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int l4 = SB / 4 - 1; l4 >= (c >> 2); --l4) {
            const float4 v = *reinterpret_cast<const float4*>(Sb + c * kDiagLd + 4 * l4);   // same address in every lane
            if (4 * l4 + 3 > c) p[3] = fmaf(v.w, w[4 * l4 + 3], p[3]);  // w[l] is zero for l > lane
            if (4 * l4 + 2 > c) p[2] = fmaf(v.z, w[4 * l4 + 2], p[2]);
            if (4 * l4 + 1 > c) p[1] = fmaf(v.y, w[4 * l4 + 1], p[1]);
            if (4 * l4 + 0 > c) p[0] = fmaf(v.x, w[4 * l4 + 0], p[0]);
        }
        const float num = (c == lane) ? 1.f : -((p[0] + p[1]) + (p[2] + p[3]));
        w[c] = (c <= lane) ? num * rdiag[c] : 0.f;
        if (c <= lane) Vb[c * kDiagLd + lane] = w[c];
    }
    return bad;
}

__global__ void __launch_bounds__(kDiagThreads) diag_block_kernel(float* __restrict__ A, float* __restrict__ U, int Cp,
                                                                  int kblk, int* __restrict__ info) {
    extern __shared__ __align__(16) float dsm[];
    float* S = dsm;                               // [NB][kDiagLd]  A, then R (upper)
    float* V = dsm + NB * kDiagLd;                // [NB][kDiagLd]  R^-1 (upper); lower blocks are scratch
    __shared__ __align__(16) float colbuf[2 * SB];
    __shared__ float rdiag[SB];
    __shared__ int bad;
    const int g = blockIdx.x;
    const int64_t origin = ((int64_t)g * Cp + (int64_t)kblk * NB) * Cp + (int64_t)kblk * NB;
    float* Ab = A + origin;
    float* Ub = U + origin;
    const int tid = threadIdx.x;
    const int job = tid >> 6, t = tid & 63, tr = t >> 3, tc = t & 7;     // 8 job slots of 64 threads, 4x4 outputs each
    if (tid == 0) bad = 0;
    {   // 16-byte loads, all of a thread's requests in flight at once; entries below the diagonal are never read
        float4 in[NB * NB / 4 / kDiagThreads];
#pragma unroll
        for (int it = 0; it < NB * NB / 4 / kDiagThreads; ++it) {
            const int e = tid + it * kDiagThreads, i = e >> 5, j = (e & 31) * 4;
            in[it] = (j + 3 >= i) ? *reinterpret_cast<const float4*>(Ab + (int64_t)i * Cp + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int it = 0; it < NB * NB / 4 / kDiagThreads; ++it) {
            const int e = tid + it * kDiagThreads, i = e >> 5, j = (e & 31) * 4;
            *reinterpret_cast<float4*>(S + i * kDiagLd + j) = in[it];
            *reinterpret_cast<float4*>(V + i * kDiagLd + j) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    __syncthreads();
    auto blk = [&](float* M, int bi, int bj) -> float* { return M + (bi * SB) * kDiagLd + bj * SB; };

    // ---- factorisation, sub-block columns from the last to the first
    for (int b = NB / SB - 1; b >= 0; --b) {
        if (tid < 32) {
            if (diag_factor_sub(blk(S, b, b), blk(V, b, b), colbuf, rdiag, tid) && tid == 0) bad = 1;
        }
        __syncthreads();
        if (b == 0) break;
        float acc[4][4] = {};
        if (job < b) diag_job_nt(acc, blk(S, job, b), blk(V, b, b), tr, tc);          // R_ib = A_ib . W_bb^T
        __syncthreads();
        if (job < b) {
            float* Cb = blk(S, job, b);
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) Cb[(4 * tr + x) * kDiagLd + tc + 8 * y] = acc[x][y];
        }
        __syncthreads();
        if (job < b * (b + 1) / 2) {                                                  // A_ij -= R_ib . R_jb^T
            int i = 0, rest = job;
            while (rest >= b - i) { rest -= b - i; ++i; }
            const int jj = i + rest;
            float a2[4][4] = {};
            diag_job_nt(a2, blk(S, i, b), blk(S, jj, b), tr, tc);
            float* Cb = blk(S, i, jj);
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) Cb[(4 * tr + x) * kDiagLd + tc + 8 * y] -= a2[x][y];
        }
        __syncthreads();
    }

    // ---- inverse of the block-triangular factor
    {   // sub-block pairs (0,1) and (2,3):  T = W_aa . R_ab (parked at V(b,a)),  U_ab = -T . W_bb
        const int a = 2 * job, b = 2 * job + 1;
        float acc[4][4] = {};
        if (job < 2) {
            diag_job_nn(acc, blk(V, a, a), blk(S, a, b), tr, tc);
            diag_store(blk(V, b, a), acc, tr, tc, 1.f);
        }
        __syncthreads();
        float ac2[4][4] = {};
        if (job < 2) {
            diag_job_nn(ac2, blk(V, b, a), blk(V, b, b), tr, tc);
            diag_store(blk(V, a, b), ac2, tr, tc, -1.f);
        }
        __syncthreads();
    }
    {   // the 64-wide pair: p in {0,1}, q in {2,3}:  T_pq = sum_{l=p..1} U_pl . R_lq (parked at V(q,p)),
        //                                            U_pq = -sum_{l=2..q} T_pl . U_lq
        const int p = job >> 1, q = 2 + (job & 1);
        float acc[4][4] = {};
        if (job < 4) {
            for (int l = p; l < 2; ++l) diag_job_nn(acc, blk(V, p, l), blk(S, l, q), tr, tc);
            diag_store(blk(V, q, p), acc, tr, tc, 1.f);
        }
        __syncthreads();
        float ac2[4][4] = {};
        if (job < 4) {
            for (int l = 2; l <= q; ++l) diag_job_nn(ac2, blk(V, l, p), blk(V, l, q), tr, tc);
            diag_store(blk(V, p, q), ac2, tr, tc, -1.f);
        }
        __syncthreads();
    }
#pragma unroll
    for (int it = 0; it < NB * NB / 4 / kDiagThreads; ++it) {
        const int e = tid + it * kDiagThreads, i = e >> 5, j = (e & 31) * 4;
        float4 r = *reinterpret_cast<const float4*>(S + i * kDiagLd + j);
        float4 u = *reinterpret_cast<const float4*>(V + i * kDiagLd + j);
        if (j + 0 < i) { r.x = 0.f; u.x = 0.f; }
        if (j + 1 < i) { r.y = 0.f; u.y = 0.f; }
        if (j + 2 < i) { r.z = 0.f; u.z = 0.f; }
        if (j + 3 < i) { r.w = 0.f; u.w = 0.f; }
        *reinterpret_cast<float4*>(Ab + (int64_t)i * Cp + j) = r;
        *reinterpret_cast<float4*>(Ub + (int64_t)i * Cp + j) = u;
    }
    if (tid == 0 && bad) atomicCAS(&info[g], 0, kblk + 1);
}

// ------------------------------------------------------------------------------------------
// GEMM-shaped steps (one 128x128 tile per CTA, grid.z = group)
// ------------------------------------------------------------------------------------------
// panel: A[i-block][k] <- A[i-block][k] . U_kk^T   for i < k      grid (k, 1, G)
__global__ void __launch_bounds__(gemm::kThreads, 2) panel_kernel(float* __restrict__ A, const float* __restrict__ U,
                                                               int Cp, int kblk) {
    extern __shared__ float smem[];
    const int64_t gofs = (int64_t)blockIdx.z * Cp * Cp;
    gemm::Args a;
    a.A = A + gofs + (int64_t)kblk * NB; a.lda = Cp;                                 // columns of block k
    a.B = U + gofs + ((int64_t)kblk * NB) * Cp + (int64_t)kblk * NB; a.ldb = Cp;      // U_kk as [N, K]
    a.C = A + gofs + (int64_t)kblk * NB; a.ldc = Cp;
    a.Aux = nullptr; a.ldaux = 0;
    a.M = kblk * NB; a.N = NB; a.K = NB;
    a.alpha = 1.f; a.beta = 0.f; a.gamma = 0.f;
    a.k_begin = 0; a.k_end = NB;
    gemm::tile<true>(a, blockIdx.x * NB, 0, smem);
}

// trailing: A[i][j] -= R[i][k] . R[j][k]^T   for i <= j < k      grid (k(k+1)/2, 1, G)
__global__ void __launch_bounds__(gemm::kThreads, 2) trailing_kernel(float* __restrict__ A, int Cp, int kblk) {
    extern __shared__ float smem[];
    int bi, bj;
    {
        const int u = blockIdx.x;
        int jj = static_cast<int>((sqrtf(8.f * static_cast<float>(u) + 1.f) - 1.f) * 0.5f);
        while ((jj + 1) * (jj + 2) / 2 <= u) ++jj;
        while (jj * (jj + 1) / 2 > u) --jj;
        bj = jj;
        bi = u - jj * (jj + 1) / 2;
    }
    const int64_t gofs = (int64_t)blockIdx.z * Cp * Cp;
    gemm::Args a;
    a.A = A + gofs + (int64_t)kblk * NB; a.lda = Cp;
    a.B = A + gofs + (int64_t)kblk * NB; a.ldb = Cp;
    a.C = A + gofs; a.ldc = Cp;
    a.Aux = nullptr; a.ldaux = 0;
    a.M = kblk * NB; a.N = kblk * NB; a.K = NB;
    a.alpha = -1.f; a.beta = 1.f; a.gamma = 0.f;
    a.k_begin = 0; a.k_end = NB;
    gemm::tile<true>(a, bi * NB, bj * NB, smem);
}

// inverse, level with block size s: for pair m: a = [2ms, (2m+1)s), b = [(2m+1)s, min((2m+2)s, Cp))
//   step 1: T[a, b] = U[a, a] . R[a, b]          (U[a,a] upper: k starts at the row block)
//   step 2: U[a, b] = - T[a, b] . U[b, b]        (U[b,b] upper: k ends with the column block)
// grid (tiles_m * tiles_n, pairs, G)
__global__ void __launch_bounds__(gemm::kThreads, 2) inv_level_kernel(const float* __restrict__ R, float* __restrict__ U,
                                                                   float* __restrict__ T, int Cp, int s, int step) {
    extern __shared__ float smem[];
    const int m = blockIdx.y;
    const int a0 = 2 * m * s, b0 = a0 + s;
    if (b0 >= Cp) return;
    const int b1 = (b0 + s < Cp) ? b0 + s : Cp;
    const int nb_cols = b1 - b0;
    const int tiles_n = (nb_cols + NB - 1) / NB;
    const int tiles_m = s / NB;
    const int ti = blockIdx.x % tiles_m, tj = blockIdx.x / tiles_m;
    if (tj >= tiles_n) return;
    const int64_t gofs = (int64_t)blockIdx.z * Cp * Cp;
    gemm::Args a;
    a.Aux = nullptr; a.ldaux = 0; a.gamma = 0.f; a.beta = 0.f;
    a.M = s; a.N = nb_cols;
    if (step == 1) {
        a.A = U + gofs + (int64_t)a0 * Cp + a0; a.lda = Cp;
        a.B = R + gofs + (int64_t)a0 * Cp + b0; a.ldb = Cp;
        a.C = T + gofs + (int64_t)a0 * Cp + b0; a.ldc = Cp;
        a.K = s; a.alpha = 1.f;
        a.k_begin = ti * NB; a.k_end = s;
    } else {
        a.A = T + gofs + (int64_t)a0 * Cp + b0; a.lda = Cp;
        a.B = U + gofs + (int64_t)b0 * Cp + b0; a.ldb = Cp;
        a.C = U + gofs + (int64_t)a0 * Cp + b0; a.ldc = Cp;
        a.K = nb_cols; a.alpha = -1.f;
        a.k_begin = 0; a.k_end = ((tj + 1) * NB < nb_cols) ? (tj + 1) * NB : nb_cols;
    }
    gemm::tile<false>(a, ti * NB, tj * NB, smem);
}

// Last pass over the result: undo the equilibration, Hinv[i][j] = U'[i][j] * dsc[j] (exact), and scan for
// non-finite entries; marks info[g] = -1 when info[g] == 0.  grid (row blocks, G): a block walks whole rows.
__global__ void __launch_bounds__(256) unscale_check_kernel(float* __restrict__ U, const float* __restrict__ dsc, int Cp,
                                                            int* __restrict__ info) {
    const int g = blockIdx.y;
    float* Ug = U + (int64_t)g * Cp * Cp;
    const float* dg = dsc + (int64_t)g * Cp;
    int badv = 0;
    for (int i = blockIdx.x; i < Cp; i += gridDim.x) {
        float* row = Ug + (int64_t)i * Cp;
        for (int j = (i & ~3) + 4 * threadIdx.x; j < Cp; j += 1024) {          // nothing but zeros left of the diagonal
            float4 v = *reinterpret_cast<float4*>(row + j);
            const float4 d = *reinterpret_cast<const float4*>(dg + j);
            v.x *= d.x; v.y *= d.y; v.z *= d.z; v.w *= d.w;
            if (!(fabsf(v.x) <= 3.4e38f) || !(fabsf(v.y) <= 3.4e38f) || !(fabsf(v.z) <= 3.4e38f) || !(fabsf(v.w) <= 3.4e38f))
                badv = 1;
            *reinterpret_cast<float4*>(row + j) = v;
        }
    }
    if (__syncthreads_or(badv) && threadIdx.x == 0) atomicCAS(&info[g], 0, -1);
}

// a device-side wait of a tensor-core launch ran out: report it through every group's info word
__global__ void merge_status_kernel(const int* __restrict__ status, int* __restrict__ info, int G) {
    if (*status != 0)
        for (int g = threadIdx.x; g < G; g += blockDim.x) info[g] = -2;
}

// use the tensor-core trailing update from this many block columns on (below that the launch is all prologue)
constexpr int kTensorTrailingMinBlocks = 4;
// block columns per outer block of the two-level trailing update (must equal kTensorTrailingMinBlocks: block
// columns below it form the outer block that is updated on the CUDA cores)
constexpr int kOuterBlocks = 4;
// levels of the triangular inverse with blocks at least this wide run on the tensor cores
constexpr int kTensorInverseMinBlock = 512;
// fp16 planes of the panels: entries of the equilibrated factor are below sqrt(2); 2^13 puts them below 11586
constexpr float kPanelScale = 8192.f;

}  // namespace chol
}  // namespace rq

using namespace rq;

static size_t chol_panel_plane_bytes(size_t Cp, int G) {
    return (size_t)G * 2 * Cp * chol::NB * chol::kOuterBlocks * 2;
}
static size_t chol_full_plane_bytes(size_t Cp, int G) {       // hi + lo planes of one Cp x Cp matrix per group
    return Cp >= (size_t)chol::kTensorInverseMinBlock * 2 ? (size_t)G * 2 * Cp * Cp * 2 + 1024 : 0;
}

extern "C" size_t rq_chol_workspace_bytes(int C, int G) {
    if (C <= 0 || G <= 0) return 0;
    const size_t Cp = (size_t)(C + chol::NB - 1) / chol::NB * chol::NB;
    // A, T, per-group means / factors / status, bf16 planes of one block column
    return 2 * (size_t)G * Cp * Cp * sizeof(float) + 256 * sizeof(float) + chol_panel_plane_bytes(Cp, G) + 4096 +
           4 * chol_full_plane_bytes(Cp, G) +                 // R^T, U, U^T, T planes for the inverse
           (size_t)G * Cp * sizeof(float) + 1024;             // equilibration factors
}

static int chol_hinv_impl(const float* H, const int64_t* perm, const float* damp_factor, float* Hinv, int C, int G,
                          int* info, void* workspace, size_t workspace_bytes, int flags, void* stream) {
    using namespace rq::chol;
    const bool bf16_only = (flags & 1) != 0;
    if (!H || !damp_factor || !Hinv || !info || !workspace || C <= 0 || G <= 0 || G > 64) return RQ_ERR_INVALID;
    if (workspace_bytes < rq_chol_workspace_bytes(C, G)) return RQ_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || reinterpret_cast<uintptr_t>(Hinv) % 16 != 0)
        return RQ_ERR_INVALID;
    cudaStream_t st = as_stream(stream);
    const int Cp = (C + NB - 1) / NB * NB;
    const int nblk = Cp / NB;
    const size_t mat = (size_t)G * Cp * Cp;
    float* A = reinterpret_cast<float*>(workspace);
    float* T = A + mat;
    float* mean = T + mat;              // [G] means, then [G] damping factors, then the tensor-core status word
    float* factor = mean + 64;
    int* tc_status = reinterpret_cast<int*>(mean + 128);
    __nv_bfloat16* panel_planes = reinterpret_cast<__nv_bfloat16*>(
        (reinterpret_cast<uintptr_t>(mean + 256) + 1023) / 1024 * 1024);
    float* dsc = reinterpret_cast<float*>(
        (reinterpret_cast<uintptr_t>(panel_planes) + chol_panel_plane_bytes(Cp, G) + 4 * chol_full_plane_bytes(Cp, G) + 2048 +
         1023) / 1024 * 1024);
    prof::Scope timed(RQ_PROF_CHOL, st);
    if (cudaMemsetAsync(tc_status, 0, sizeof(int), st) != cudaSuccess) return RQ_ERR_CUDA;

    if (cudaMemcpyAsync(factor, damp_factor, (size_t)G * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess)
        return RQ_ERR_CUDA;
    if (cudaMemsetAsync(info, 0, (size_t)G * sizeof(int), st) != cudaSuccess) return RQ_ERR_CUDA;
    if (cudaMemsetAsync(Hinv, 0, mat * sizeof(float), st) != cudaSuccess) return RQ_ERR_CUDA;
    diag_mean_kernel<<<G, 256, 0, st>>>(H, C, mean);
    equil_kernel<<<dim3((unsigned)((Cp + 255) / 256), (unsigned)G), 256, 0, st>>>(H, perm, mean, factor, C, Cp, dsc);
    {
        dim3 grid((unsigned)((Cp + 1023) / 1024), (unsigned)Cp, (unsigned)G);
        gather_kernel<<<grid, 256, 0, st>>>(H, perm, mean, factor, dsc, C, Cp, A);
    }
    int rc = check_launch();
    if (rc != RQ_OK) return rc;

    const size_t diag_smem = (size_t)2 * NB * kDiagLd * sizeof(float);
    if (cudaFuncSetAttribute(diag_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)diag_smem) != cudaSuccess)
        return RQ_ERR_CUDA;
    // phase 1: block columns from the last to the first
    for (int k = nblk - 1; k >= 0; --k) {
        {
            prof::Scope t1(RQ_PROF_CHOL_DIAG, st);
            diag_block_kernel<<<G, kDiagThreads, diag_smem, st>>>(A, Hinv, Cp, k, info);
        }
        if (k > 0) {
            {
                prof::Scope t2(RQ_PROF_CHOL_PANEL, st);
                panel_kernel<<<dim3((unsigned)k, 1, (unsigned)G), gemm::kThreads, gemm::kSmemBytes, st>>>(A, Hinv, Cp, k);
            }
            prof::Scope t3(RQ_PROF_CHOL_TRAILING, st);
            if (k >= kTensorTrailingMinBlocks) {
                // Two-level update on the tensor cores.  Block columns are grouped four to an outer block; the
                // panel R[0:k*128, block k] is split into bf16 planes at its place inside the outer block's
                // 512-wide panel.  Inside an outer block only its own columns are brought up to date after
                // each step (k-extent 128); everything to the left receives ONE update per outer block with
                // k-extent 512, which divides the read-modify-write traffic of the trailing matrix by four.
                const int c0 = k / kOuterBlocks * kOuterBlocks, p = k - c0;
                const int W = NB * kOuterBlocks;
                tcgemm::SplitArgs sa;
                sa.src = A + (size_t)k * NB; sa.ld = Cp; sa.src_z = (long long)Cp * Cp;
                sa.rows = k * NB; sa.cols = NB;
                sa.dst = panel_planes; sa.Kp = W; sa.plane_stride = (long long)Cp * W;
                sa.plane = 0; sa.plane_z = 2; sa.dst_row0 = 0; sa.dst_row_z = 0; sa.dst_k0 = p * NB; sa.pad_k_to = 0;
                sa.fp16 = bf16_only ? 0 : 1;                   // |R'| < sqrt(2) after the equilibration
                sa.scale = bf16_only ? 1.f : kPanelScale;
                rc = tcgemm::split_rows(sa, G, st);
                if (rc != RQ_OK) return rc;
                tcgemm::PlaneTensor pt{panel_planes, W, Cp, 2LL * G};
                tcgemm::Params gp;
                gp.a_plane = gp.b_plane = 0; gp.a_plane_z = gp.b_plane_z = 2; gp.a_row_z = gp.b_row_z = 0;
                gp.tri = 1; gp.kmode = 0; gp.batch = G;
                gp.ldc = Cp; gp.c_z = (long long)Cp * Cp;
                gp.Aux = nullptr; gp.ldaux = 0; gp.aux_z = 0;
                gp.alpha = bf16_only ? -1.f : -1.f / (kPanelScale * kPanelScale); gp.beta = 1.f; gp.gamma = 0.f;
                gp.fp16 = bf16_only ? 0 : 1;
                gp.a_row0 = 0;
                if (p > 0) {            // columns [c0*128, k*128) of the outer block: A_ij -= R_ik . R_jk^T
                    gp.b_row0 = c0 * NB; gp.a_k0 = gp.b_k0 = p * NB; gp.k_len = NB;
                    gp.M = k * NB; gp.N = p * NB; gp.tri_col0 = c0 * NB; gp.C = A + (size_t)c0 * NB;
                } else {                // everything left of the outer block, all of its block columns at once
                    const int blocks = (nblk - c0 < kOuterBlocks) ? nblk - c0 : kOuterBlocks;
                    gp.b_row0 = 0; gp.a_k0 = gp.b_k0 = 0; gp.k_len = blocks * NB;
                    gp.M = gp.N = k * NB; gp.tri_col0 = 0; gp.C = A;
                }
                rc = tcgemm::launch(pt, pt, gp, tc_status, st);
                if (rc != RQ_OK) return rc;
            } else {
                trailing_kernel<<<dim3((unsigned)(k * (k + 1) / 2), 1, (unsigned)G), gemm::kThreads, gemm::kSmemBytes, st>>>(
                    A, Cp, k);
            }
        }
    }
    rc = check_launch();
    if (rc != RQ_OK) return rc;
    // phase 2: merge inverses of neighbouring diagonal blocks, doubling the block size each level
    prof::Scope t4(RQ_PROF_CHOL_INVERSE, st);
    const size_t fpb = chol_full_plane_bytes(Cp, G);
    uint8_t* plane_base = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(panel_planes) + chol_panel_plane_bytes(Cp, G) + 1023) / 1024 * 1024);
    __nv_bfloat16* PRt = reinterpret_cast<__nv_bfloat16*>(plane_base);
    __nv_bfloat16* PU = reinterpret_cast<__nv_bfloat16*>(plane_base + fpb);
    __nv_bfloat16* PUt = reinterpret_cast<__nv_bfloat16*>(plane_base + 2 * fpb);
    __nv_bfloat16* PT = reinterpret_cast<__nv_bfloat16*>(plane_base + 3 * fpb);
    // Operand planes are filled only where a level reads them.  Entries of U are final once written, so its
    // planes (U and U^T) start as the band of diagonal blocks the CUDA-core levels produced and then receive,
    // level by level, just the off-diagonal blocks that level created; T is split block by block as well;
    // R^T once, above the diagonal.
    // fp16 planes for the inverse as well.  The equilibrated damped matrix satisfies A' >= lambda D^2 with
    // D^2 >= 1 / (2 max_i a_ii), so every entry of U' = R'^-1 is at most B = sqrt(2 max_i a_ii / lambda)
    // <= sqrt(2 (1 + C / p)), p the smallest damping fraction of the groups: the scale of the U planes follows from
    // that bound and cannot overflow.  The intermediate T = U'_aa.R'_ab has no comparably tight bound (its entries
    // are at most B times a column norm of R'); its planes get a quarter of the head room of U's, 4.4 B, which
    // real Hessians stay far below.  Should a matrix exceed it, the planes hold infinities, the result fails the
    // finiteness scan (info = -1), and the caller repeats the factorisation with flag 1 (bf16 planes, four products)
    // before treating it as a failed attempt.  Where B leaves less than one binary digit of head room the levels use
    // bf16 planes from the start.
    float pmin = damp_factor[0];
    for (int g = 1; g < G; ++g) pmin = damp_factor[g] < pmin ? damp_factor[g] : pmin;
    const double ubound = pmin > 0.f ? sqrt(2.0 * (1.0 + (double)C / (double)pmin)) : 1e30;
    const float sU = (float)exp2(floor(log2(30000.0 / ubound)));
    const int inv_fp16 = (sU >= 2.f && !bf16_only) ? 1 : 0;
    const float sT = inv_fp16 ? sU * 0.5f : 1.f, sUu = inv_fp16 ? sU : 1.f, sR = inv_fp16 ? kPanelScale : 1.f;
    auto plane_args = [&](const float* src, __nv_bfloat16* dst, float scale) {
        tcgemm::SplitArgs sa;
        sa.src = src; sa.ld = Cp; sa.src_z = (long long)Cp * Cp; sa.rows = Cp; sa.cols = Cp;
        sa.dst = dst; sa.Kp = Cp; sa.plane_stride = (long long)Cp * Cp; sa.plane = 0; sa.plane_z = 2;
        sa.dst_row0 = 0; sa.dst_row_z = 0; sa.dst_k0 = 0; sa.pad_k_to = 0;
        sa.fp16 = inv_fp16; sa.scale = scale;
        return sa;
    };
    // blocks (a, b) of level s: rows [2ms, 2ms+s), columns [2ms+s, min(2ms+2s, Cp)), m = 0 .. pairs-1
    auto split_pair_blocks = [&](const float* src, __nv_bfloat16* dst, int s, int pairs, bool transpose, float scale) {
        tcgemm::SplitArgs sa = plane_args(src + s, dst, scale);
        sa.rows = s; sa.cols = s; sa.nz1 = pairs; sa.src_z1 = (long long)2 * s * Cp + 2 * s;
        sa.src_col0 = s; sa.src_col_z1 = 2 * s; sa.src_cols_total = Cp;
        sa.src_row0 = 0; sa.src_row_z1 = 2 * s; sa.src_rows_total = Cp;
        if (transpose) { sa.dst_row0 = s; sa.dst_k0 = 0; } else { sa.dst_row0 = 0; sa.dst_k0 = s; }
        sa.dst_row_z1 = 2 * s; sa.dst_k_z1 = 2 * s;
        return transpose ? tcgemm::split_transpose(sa, G, st) : tcgemm::split_rows(sa, G, st);
    };
    bool planes_ready = false;
    for (int s = NB; s < Cp; s *= 2) {
        const int pairs = (Cp + 2 * s - 1) / (2 * s);
        if (s < kTensorInverseMinBlock || fpb == 0) {
            const int tiles = (s / NB) * (s / NB);
            for (int step = 1; step <= 2; ++step)
                inv_level_kernel<<<dim3((unsigned)tiles, (unsigned)pairs, (unsigned)G), gemm::kThreads, gemm::kSmemBytes, st>>>(
                    A, Hinv, T, Cp, s, step);
            continue;
        }
        // tensor-core level: pair m merges a = [2ms, 2ms+s) and b = [2ms+s, min(2ms+2s, Cp))
        if (!planes_ready) {
            tcgemm::SplitArgs sa = plane_args(A, PRt, sR);         // planes of R^T: [n][k] = R[k][n], k <= n
            sa.upper_only = 1;
            rc = tcgemm::split_transpose(sa, G, st);
            if (rc != RQ_OK) return rc;
            for (int tr = 0; tr < 2; ++tr) {                       // diagonal blocks of width s of U and U^T
                tcgemm::SplitArgs sd = plane_args(Hinv, tr ? PUt : PU, sUu);
                sd.rows = s; sd.cols = s; sd.nz1 = (Cp + s - 1) / s; sd.src_z1 = (long long)s * Cp + s;
                sd.src_col0 = 0; sd.src_col_z1 = s; sd.src_cols_total = Cp;
                sd.src_row0 = 0; sd.src_row_z1 = s; sd.src_rows_total = Cp;
                sd.dst_row_z1 = s; sd.dst_k_z1 = s;
                rc = tr ? tcgemm::split_transpose(sd, G, st) : tcgemm::split_rows(sd, G, st);
                if (rc != RQ_OK) return rc;
            }
            planes_ready = true;
        }
        tcgemm::PlaneTensor tRt{PRt, Cp, Cp, 2LL * G}, tU{PU, Cp, Cp, 2LL * G}, tUt{PUt, Cp, Cp, 2LL * G},
            tT{PT, Cp, Cp, 2LL * G};
        tcgemm::Params gp;
        gp.a_plane = gp.b_plane = 0; gp.a_plane_z = gp.b_plane_z = 2; gp.a_row_z = gp.b_row_z = 0;
        gp.M = s; gp.N = s; gp.k_len = s; gp.tri = 0; gp.batch = pairs * G; gp.nz1 = pairs;
        gp.ldc = Cp; gp.c_z = (long long)Cp * Cp; gp.c_z1 = (long long)2 * s * Cp + 2 * s;
        gp.Aux = nullptr; gp.ldaux = 0; gp.aux_z = 0; gp.gamma = 0.f; gp.beta = 0.f;
        gp.n_limit = Cp - s; gp.n_limit_z1 = 2 * s;
        gp.a_row_z1 = 2 * s; gp.b_row_z1 = 2 * s; gp.a_k_z1 = 2 * s; gp.b_k_z1 = 2 * s;
        // step 1: T[a, b] = U[a, a] . R[a, b]
        gp.fp16 = inv_fp16;
        gp.a_row0 = 0; gp.a_k0 = 0; gp.b_row0 = s; gp.b_k0 = 0; gp.kmode = 1;
        gp.C = T + s; gp.alpha = 1.f / (sUu * sR);
        rc = tcgemm::launch(tU, tRt, gp, tc_status, st);
        if (rc != RQ_OK) return rc;
        rc = split_pair_blocks(T, PT, s, pairs, false, sT);
        if (rc != RQ_OK) return rc;
        // step 2: U[a, b] = -T[a, b] . U[b, b]
        gp.a_row0 = 0; gp.a_k0 = s; gp.b_row0 = s; gp.b_k0 = s; gp.kmode = 2;
        gp.C = Hinv + s; gp.alpha = -1.f / (sT * sUu);
        rc = tcgemm::launch(tT, tUt, gp, tc_status, st);
        if (rc != RQ_OK) return rc;
        if (2 * s < Cp) {                                          // the next level reads the blocks just created
            rc = split_pair_blocks(Hinv, PU, s, pairs, false, sUu);
            if (rc != RQ_OK) return rc;
            rc = split_pair_blocks(Hinv, PUt, s, pairs, true, sUu);
            if (rc != RQ_OK) return rc;
        }
    }
    unscale_check_kernel<<<dim3(592, (unsigned)G), 256, 0, st>>>(Hinv, dsc, Cp, info);
    merge_status_kernel<<<1, 64, 0, st>>>(tc_status, info, G);
    return check_launch();
}

extern "C" int rq_chol_hinv(const float* H, const int64_t* perm, const float* damp_factor, float* Hinv, int C, int G,
                            int* info, void* workspace, size_t workspace_bytes, void* stream) {
    return chol_hinv_impl(H, perm, damp_factor, Hinv, C, G, info, workspace, workspace_bytes, 0, stream);
}

extern "C" int rq_chol_hinv_flags(const float* H, const int64_t* perm, const float* damp_factor, float* Hinv, int C,
                                  int G, int* info, void* workspace, size_t workspace_bytes, int flags, void* stream) {
    return chol_hinv_impl(H, perm, damp_factor, Hinv, C, G, info, workspace, workspace_bytes, flags, stream);
}
