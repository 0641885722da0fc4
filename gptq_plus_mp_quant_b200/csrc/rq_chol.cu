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
// A[g][i][j] = H[g][perm[i]][perm[j]] (+ dead fix, + damping on the diagonal), padded to Cp with
// an identity block.  Only the upper triangle is consumed afterwards.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_kernel(const float* __restrict__ H, const int64_t* __restrict__ perm,
                                                     const float* __restrict__ mean, const float* __restrict__ factor,
                                                     int C, int Cp, float* __restrict__ A) {
    const int g = blockIdx.z;
    const int i = blockIdx.y;
    const float* Hg = H + (int64_t)g * C * C;
    float* Arow = A + ((int64_t)g * Cp + i) * Cp;
    const float lambda = factor[g] * mean[g];
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
// arithmetic runs at 1/64 of the fp32 rate on this part; formulations with fp64 or compensated dot products,
// with the block spread over registers, and with shared-memory rank-1 updates were all measured slower.)
// Four lanes share a row (factorisation, left-looking: column c needs t_i = A[i][c] - sum_{l>c} R[i][l] R[c][l])
// or a column (inverse: U[c][j] = -(sum_{c<l<=j} R[c][l] U[l][j]) / R[c][c]).
// ------------------------------------------------------------------------------------------
constexpr int kDiagLd = NB + 4;               // fp32 row stride: rows 4 banks apart

__global__ void __launch_bounds__(kDiagThreads) diag_block_kernel(float* __restrict__ A, float* __restrict__ U, int Cp,
                                                                  int kblk, int* __restrict__ info) {
    extern __shared__ float dsm[];
    float* S = dsm;                               // [NB][kDiagLd]  R (upper)
    float* V = dsm + NB * kDiagLd;                // [NB][kDiagLd]  R^-1 (upper)
    __shared__ float piv;
    __shared__ int bad;
    const int g = blockIdx.x;
    const int64_t origin = ((int64_t)g * Cp + (int64_t)kblk * NB) * Cp + (int64_t)kblk * NB;
    float* Ab = A + origin;
    float* Ub = U + origin;
    const int tid = threadIdx.x;
    const int own = tid >> 2, q = tid & 3;        // row (phase 1) / column (phase 2) and quarter of the dot product
    if (tid == 0) bad = 0;
    for (int e = tid; e < NB * NB; e += kDiagThreads) {
        const int i = e >> 7, j = e & (NB - 1);
        S[i * kDiagLd + j] = (j >= i) ? Ab[(int64_t)i * Cp + j] : 0.f;
        V[i * kDiagLd + j] = 0.f;
    }
    __syncthreads();

    // ---- phase 1: columns from the last to the first
    for (int c = NB - 1; c >= 0; --c) {
        const float* ri = S + own * kDiagLd;
        const float* rc = S + c * kDiagLd;
        if ((tid & ~31) >> 2 > c) {                   // none of this warp's 8 rows takes part any more
            __syncthreads();
            __syncthreads();
            continue;
        }
        float acc = 0.f;
        if (own <= c) {
            float p0 = 0.f, p1 = 0.f;                 // two chains
#pragma unroll 4
            for (int l = c + 1 + q; l < NB; l += 8) {
                p0 = fmaf(ri[l], rc[l], p0);
                if (l + 4 < NB) p1 = fmaf(ri[l + 4], rc[l + 4], p1);
            }
            acc = p0 + p1;
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);  // executed by every lane of the warp
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        const float t = __fsub_rn(ri[c], acc);
        if (own == c && q == 0) {
            if (!(t > 0.f)) bad = 1;                  // catches <= 0 and NaN
            piv = __fsqrt_rn(t);
        }
        __syncthreads();
        if (own <= c && q == 0) S[own * kDiagLd + c] = (own == c) ? piv : __fdiv_rn(t, piv);
        __syncthreads();
    }

    // ---- phase 2: inverse, one column per lane quad, no CTA-wide dependency
    {
        const int j = own;
        if (q == 0) V[j * kDiagLd + j] = __fdiv_rn(1.f, S[j * kDiagLd + j]);
        __syncwarp();
        const int jmax = (tid | 31) >> 2;             // last column handled by this warp: uniform trip count
        for (int c = jmax - 1; c >= 0; --c) {
            const float* rc = S + c * kDiagLd;
            float acc = 0.f;
            if (c < j) {
                float p0 = 0.f, p1 = 0.f;
#pragma unroll 4
                for (int l = c + 1 + q; l <= j; l += 8) {
                    p0 = fmaf(rc[l], V[l * kDiagLd + j], p0);
                    if (l + 4 <= j) p1 = fmaf(rc[l + 4], V[(l + 4) * kDiagLd + j], p1);
                }
                acc = p0 + p1;
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (q == 0 && c < j) V[c * kDiagLd + j] = __fdiv_rn(-acc, rc[c]);
            __syncwarp();
        }
    }
    __syncthreads();
    for (int e = tid; e < NB * NB; e += kDiagThreads) {
        const int i = e >> 7, j = e & (NB - 1);
        Ab[(int64_t)i * Cp + j] = (j >= i) ? S[i * kDiagLd + j] : 0.f;
        Ub[(int64_t)i * Cp + j] = (j >= i) ? V[i * kDiagLd + j] : 0.f;
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

// non-finite scan of the result (upper triangle incl. diagonal); marks info[g] = -1 when info[g] == 0
__global__ void __launch_bounds__(256) finite_check_kernel(const float* __restrict__ U, int Cp, int* __restrict__ info) {
    const int g = blockIdx.y;
    const float* Ug = U + (int64_t)g * Cp * Cp;
    int badv = 0;
    for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < (int64_t)Cp * Cp; e += (int64_t)gridDim.x * 256) {
        const float v = Ug[e];
        if (isnan(v) || isinf(v)) badv = 1;
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
// levels of the triangular inverse with blocks at least this wide run on the tensor cores
constexpr int kTensorInverseMinBlock = 512;

}  // namespace chol
}  // namespace rq

using namespace rq;

static size_t chol_panel_plane_bytes(size_t Cp, int G) { return (size_t)G * 2 * Cp * chol::NB * 2; }
static size_t chol_full_plane_bytes(size_t Cp, int G) {       // hi + lo planes of one Cp x Cp matrix per group
    return Cp >= (size_t)chol::kTensorInverseMinBlock * 2 ? (size_t)G * 2 * Cp * Cp * 2 + 1024 : 0;
}

extern "C" size_t rq_chol_workspace_bytes(int C, int G) {
    if (C <= 0 || G <= 0) return 0;
    const size_t Cp = (size_t)(C + chol::NB - 1) / chol::NB * chol::NB;
    // A, T, per-group means / factors / status, bf16 planes of one block column
    return 2 * (size_t)G * Cp * Cp * sizeof(float) + 256 * sizeof(float) + chol_panel_plane_bytes(Cp, G) + 4096 +
           4 * chol_full_plane_bytes(Cp, G);                  // R^T, U, U^T, T planes for the inverse
}

extern "C" int rq_chol_hinv(const float* H, const int64_t* perm, const float* damp_factor, float* Hinv, int C, int G,
                            int* info, void* workspace, size_t workspace_bytes, void* stream) {
    using namespace rq::chol;
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
    prof::Scope timed(RQ_PROF_CHOL, st);
    if (cudaMemsetAsync(tc_status, 0, sizeof(int), st) != cudaSuccess) return RQ_ERR_CUDA;

    if (cudaMemcpyAsync(factor, damp_factor, (size_t)G * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess)
        return RQ_ERR_CUDA;
    if (cudaMemsetAsync(info, 0, (size_t)G * sizeof(int), st) != cudaSuccess) return RQ_ERR_CUDA;
    if (cudaMemsetAsync(Hinv, 0, mat * sizeof(float), st) != cudaSuccess) return RQ_ERR_CUDA;
    diag_mean_kernel<<<G, 256, 0, st>>>(H, C, mean);
    {
        dim3 grid((unsigned)((Cp + 1023) / 1024), (unsigned)Cp, (unsigned)G);
        gather_kernel<<<grid, 256, 0, st>>>(H, perm, mean, factor, C, Cp, A);
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
                // split the panel R[0:k*128, block k] into bf16 planes and run A_ij -= R_ik . R_jk^T on the tensor cores
                tcgemm::SplitArgs sa;
                sa.src = A + (size_t)k * NB; sa.ld = Cp; sa.src_z = (long long)Cp * Cp;
                sa.rows = k * NB; sa.cols = NB;
                sa.dst = panel_planes; sa.Kp = NB; sa.plane_stride = (long long)Cp * NB;
                sa.plane = 0; sa.plane_z = 2; sa.dst_row0 = 0; sa.dst_row_z = 0; sa.dst_k0 = 0; sa.pad_k_to = 0;
                rc = tcgemm::split_rows(sa, G, st);
                if (rc != RQ_OK) return rc;
                tcgemm::PlaneTensor pt{panel_planes, NB, Cp, 2LL * G};
                tcgemm::Params gp;
                gp.a_row0 = gp.b_row0 = 0; gp.a_k0 = gp.b_k0 = 0; gp.a_plane = gp.b_plane = 0;
                gp.a_plane_z = gp.b_plane_z = 2; gp.a_row_z = gp.b_row_z = 0;
                gp.M = gp.N = k * NB; gp.k_len = NB; gp.tri = 1; gp.kmode = 0; gp.batch = G;
                gp.C = A; gp.ldc = Cp; gp.c_z = (long long)Cp * Cp;
                gp.Aux = nullptr; gp.ldaux = 0; gp.aux_z = 0;
                gp.alpha = -1.f; gp.beta = 1.f; gp.gamma = 0.f;
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
    auto split_full = [&](const float* src, __nv_bfloat16* dst, bool transpose) {
        tcgemm::SplitArgs sa;
        sa.src = src; sa.ld = Cp; sa.src_z = (long long)Cp * Cp; sa.rows = Cp; sa.cols = Cp;
        sa.dst = dst; sa.Kp = Cp; sa.plane_stride = (long long)Cp * Cp; sa.plane = 0; sa.plane_z = 2;
        sa.dst_row0 = 0; sa.dst_row_z = 0; sa.dst_k0 = 0; sa.pad_k_to = 0;
        return transpose ? tcgemm::split_transpose(sa, G, st) : tcgemm::split_rows(sa, G, st);
    };
    bool rt_ready = false;
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
        if (!rt_ready) {
            rc = split_full(A, PRt, true);                       // planes of R^T: [n][k] = R[k][n]
            if (rc != RQ_OK) return rc;
            rt_ready = true;
        }
        rc = split_full(Hinv, PU, false);
        if (rc != RQ_OK) return rc;
        rc = split_full(Hinv, PUt, true);
        if (rc != RQ_OK) return rc;
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
        gp.a_row0 = 0; gp.a_k0 = 0; gp.b_row0 = s; gp.b_k0 = 0; gp.kmode = 1;
        gp.C = T + s; gp.alpha = 1.f;
        rc = tcgemm::launch(tU, tRt, gp, tc_status, st);
        if (rc != RQ_OK) return rc;
        rc = split_full(T, PT, false);
        if (rc != RQ_OK) return rc;
        // step 2: U[a, b] = -T[a, b] . U[b, b]
        gp.a_row0 = 0; gp.a_k0 = s; gp.b_row0 = s; gp.b_k0 = s; gp.kmode = 2;
        gp.C = Hinv + s; gp.alpha = -1.f;
        rc = tcgemm::launch(tT, tUt, gp, tc_status, st);
        if (rc != RQ_OK) return rc;
    }
    finite_check_kernel<<<dim3(64, (unsigned)G), 256, 0, st>>>(Hinv, Cp, info);
    merge_status_kernel<<<1, 64, 0, st>>>(tc_status, info, G);
    return check_launch();
}
