/*
 * realq_b200 — C ABI of the B200 (sm_100a) kernels behind the per-layer GPTQ / GPTQ+
 * quantization path of REAL-Q (Mrluxianseng/gptq_plus_mp_quant).
 *
 * The reference is pure PyTorch and has no FFI layer of its own; each entry point below names
 * the reference statements (file:line inside the reference project) that it replaces.  All
 * pointers are DEVICE pointers unless stated otherwise, all matrices are row-major, `stream`
 * is a cudaStream_t passed as void*, and every function returns an RQ_* status code.  Nothing
 * here allocates device memory: scratch is passed in by the caller.  No function synchronises
 * the stream.
 */
#ifndef REALQ_B200_H_
#define REALQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define RQ_OK 0
#define RQ_ERR_INVALID 1     /* bad argument (null pointer, unsupported size, misaligned) */
#define RQ_ERR_CUDA 2        /* a CUDA runtime / driver call failed                       */
#define RQ_ERR_TIMEOUT 3     /* a bounded device-side wait ran out (written to `status`)   */
#define RQ_ERR_WORKSPACE 4   /* caller-provided scratch too small                          */
#define RQ_ERR_UNSUPPORTED 5 /* configuration not implemented by this build                */
#define RQ_ERR_TOO_LARGE 6   /* problem exceeds the fixed scratch of an allocation-free entry point */

/* element types of activations / weights crossing the boundary */
#define RQ_F32 0
#define RQ_BF16 1
#define RQ_F16 2

int rq_version(void);
const char* rq_error_string(int code);

/* Per-kernel device timing for benchmarks (no counterpart in the reference, which wraps its
 * stages in CUDA-event pairs from Python, gptq_utils/gptq_plus_utils.py:228-289).  While enabled,
 * every launch of a tagged kernel is bracketed by two CUDA events on its stream;
 * rq_profile_read waits for them and returns the summed duration and launch count of one tag.
 * rq_profile_enable (either value) drops the spans recorded so far. */
#define RQ_PROF_HESSIAN_UMMA 1
#define RQ_PROF_HESSIAN_PACK 2
#define RQ_PROF_FWHT 3
#define RQ_PROF_CHOL 4
#define RQ_PROF_BLOCK 5
#define RQ_PROF_LAZY 6
#define RQ_PROF_CHOL_DIAG 7
#define RQ_PROF_CHOL_PANEL 8
#define RQ_PROF_CHOL_TRAILING 9
#define RQ_PROF_CHOL_INVERSE 10
#define RQ_PROF_TERMS 11
int rq_profile_enable(int on);
int rq_profile_read(int tag, double* total_ms, long long* launches);

/* ------------------------------------------------------------------------------------------
 * Hessian accumulation.
 * Replaces GPTQPlus.add_batch (gptq_utils/gptq_plus_utils.py:839-856:
 *   weighted = inp[None] * sal^T[:, :, None]; H += bmm(inp^T, weighted); act_square += (inp**2).sum(0))
 * and GPTQ.add_batch (gptq_utils/gptq_utils.py:39-43: H *= n/(n+b); H += (2/n) X^T X).
 *
 *   H[g] = beta * H[g] + alpha * X^T diag(sal[:, g]) X        g < G   (sal == NULL: weights 1, G must be 1)
 *   act_sq += sum_tokens x^2                                   (skipped when act_sq == NULL)
 *
 * x: [N, C] with row stride ldx elements, dtype x_dtype; sal: [N, G] fp32; H: [G, C, C] fp32.
 * Only tiles on or above the diagonal of every H[g] are written; rq_hessian_finalize (or its
 * mirror-only mode) fills the lower triangle.  The contraction runs on the tensor cores as a split
 * product of fp16 planes with fp32 accumulation: x and s*x are scaled per token and per group by
 * powers of two (exact) so that they fit fp16's range, s*x is carried as hi + lo (22 significant
 * bits), x as one plane when it is bf16 / fp16 and as hi + lo when it is fp32: two products per
 * k-step for 16-bit input, three for fp32 input.
 * workspace: rq_hessian_workspace_bytes(chunk_tokens, C, G, sal != NULL) bytes for the chunk
 * size the caller wants (a multiple of 64; tokens are processed chunk by chunk), 1024-byte aligned.
 * status: optional device int; set to RQ_ERR_TIMEOUT if a device-side wait ran out.
 * variant: bits 0-3: 0 = 64-token pipeline stages (128-byte swizzle), 1 = 32-token stages (64-byte
 *          swizzle), 2 = as 0 but with the two-plane operand on the 256-row side also for 16-bit input;
 *          bits 4-5: tokens summed inside the tensor core before a round-to-nearest add, 128 >> n
 *          (the tensor core's own accumulation truncates; shorter windows cost epilogue work).
 */
size_t rq_hessian_workspace_bytes(int64_t chunk_tokens, int C, int G, int has_saliency);
int rq_hessian_accum(const void* x, int x_dtype, int64_t ldx, const float* sal, float* H, float* act_sq,
                     int64_t N, int C, int G, float alpha, float beta, void* workspace, size_t workspace_bytes,
                     int* status, int variant, void* stream);

/* Same accumulation, with the packing launches on `stream` and the tensor-core launches on `gemm_stream` (two
 * different streams of the caller): the workspace is cut into up to four slots of `chunk_tokens` tokens, chunk c
 * is packed while an earlier chunk is being contracted, events order the two per slot.  act_sq is complete in
 * `stream` order; H is complete in `gemm_stream` order: make the stream that reads H wait for `gemm_stream`
 * (cudaStreamWaitEvent) first, and do not reuse `workspace` on `stream` before the kernels of this call have left
 * `gemm_stream`.  Feeding the linears of a layer through one gemm_stream lets the packing of one linear overlap
 * the contraction of another. */
int rq_hessian_accum_pipelined(const void* x, int x_dtype, int64_t ldx, const float* sal, float* H, float* act_sq,
                               int64_t N, int C, int G, float alpha, float beta, void* workspace,
                               size_t workspace_bytes, int* status, int variant, int64_t chunk_tokens, void* stream,
                               void* gemm_stream);

/* Allocation-free variant of rq_hessian_accum.  It has no counterpart in the reference; it exists
 * for hosts that must not allocate device memory where they feed calibration batches (a hook that
 * runs while the framework's memory pool is frozen, a process whose device-memory budget belongs to
 * another component, a caller with no allocator to borrow scratch from).  Same arguments and result
 * as rq_hessian_accum minus workspace and variant: the bf16 operand planes are packed into a fixed
 * rq_hessian_noalloc_scratch_bytes() = 64 MiB array inside the library's device image (every GPU that
 * loads the library holds it until the process exits), tokens being processed in as many chunks as
 * that takes.  Limit: one 64-token chunk must fit, i.e. roughly C * (2 + 2G) <= 520 000 (C = 28672
 * with G = 4 fits); wider problems return RQ_ERR_TOO_LARGE.  The function calls no cudaMalloc /
 * cudaFree or other allocating routine.  Its first call on a device looks up the array's address
 * on that device (with that device current); make that first call outside any stream capture.
 * All calls share the one array: calls that overlap on the same GPU (two streams, two threads)
 * race and must be serialised by the caller.  Nothing needs clearing between calls. */
size_t rq_hessian_noalloc_scratch_bytes(void);
int rq_hessian_accum_noalloc(const void* x, int x_dtype, int64_t ldx, const float* sal, float* H, float* act_sq,
                             int64_t N, int C, int G, float alpha, float beta, int* status, void* stream);

/* Packed upper storage of the un-finalised sums, for the cross-rank exchange that stands in for the all-reduce of
 * GPTQPlus.finalize_hessian (gptq_utils/gptq_plus_utils.py:875-878: dist_utils.allreduce_sum_(self.H)).  Before
 * finalize only the entries on or above the diagonal carry information (the finalize step mirrors them), so only
 * those cross the wire: row r of a group keeps its columns from (r / 128) * 128 to C - 1, rows back to back,
 * rq_hessian_packed_elems(C) = C (C + 128) / 2 floats per group when 128 divides C, a little over half of C * C.
 * packed: [G][group_stride] fp32 with group_stride >= rq_hessian_packed_elems(C) (a multiple of 4 and 16-byte
 * aligned buffers when C is a multiple of 4).  rq_hessian_unpack_upper writes the same entries back into H[g]
 * (the strictly lower part of each 128-row block's first columns is left as it is; rq_hessian_finalize
 * overwrites it). */
int64_t rq_hessian_packed_elems(int C);
int rq_hessian_pack_upper(const float* H, int C, int G, float* packed, int64_t group_stride, void* stream);
int rq_hessian_unpack_upper(const float* packed, int64_t group_stride, int C, int G, float* H, void* stream);

/* Replaces GPTQPlus.finalize_hessian after its all-reduce (gptq_utils/gptq_plus_utils.py:881-907):
 *   H /= div_tokens; H /= div_scale (skipped when 1); act_sq /= div_seq;
 *   H = (H + H^T)/2  — realised by mirroring the computed upper triangle —; non-finite -> 0.
 * counts: optional device uint64[2] receiving the number of NaN and Inf entries found (in the
 * full symmetric matrix), which the host turns into the reference's warning.
 * With div_tokens = div_scale = div_seq = 1, act_sq = NULL and sanitize = 0 this is a pure mirror. */
int rq_hessian_finalize(float* H, float* act_sq, int C, int G, float div_tokens, float div_scale, float div_seq,
                        int sanitize, unsigned long long* counts, void* stream);

/* ------------------------------------------------------------------------------------------
 * Walsh-Hadamard rotation y = x . H_n * scale, n = K * 2^m.
 * Replaces hadamard_utils.matmul_hadU_cuda / HadamardTransform (utils/hadamard_utils.py:89-98,121-130)
 * and the third-party fast_hadamard_transform call (utils/hadamard_utils.py:31-34).
 * x, y: [rows, n] contiguous, same dtype (in place allowed); hadK: device fp32 [K, K] (+-1), NULL when K == 1.
 * The FWHT runs over each contiguous n/K chunk, then chunk k' = sum_k hadK[k'][k] * chunk k.
 * K <= 256 (every order of the reference's table); RQ_ERR_UNSUPPORTED when a row does not fit shared memory
 * (about 50 000 elements). */
int rq_fwht(const void* x, void* y, int dtype, int64_t rows, int n, int K, const float* hadK, float scale,
            void* stream);

/* The online rotation in front of a linear fused with the dynamic per-token fake quantization that follows it
 * (ActQuantWrapper.forward, utils/quant_utils.py:258-289: matmul_hadU_cuda, then ActQuantizer.find_params and the
 * quantizer call): y = fake_quant(rq_fwht(x)), bit for bit what rq_fwht followed by rq_act_quant (per-token,
 * with_zero = 1, dtype_math = 0) writes, with one read and one write of the activations instead of two each.
 * scale_out / zero_out: optional [rows] fp32.  Only the shapes of the register-resident rotation paths (16-byte
 * aligned buffers and n = 2048, 4096, 8192, or K <= 28 with 1024 <= n/K <= 4096); RQ_ERR_UNSUPPORTED otherwise -
 * call the two entry points in turn then. */
int rq_fwht_act_quant(const void* x, void* y, int dtype, int64_t rows, int n, int K, const float* hadK, float scale,
                      float clip_ratio, int maxq, int sym, float* scale_out, float* zero_out, void* stream);

/* rq_fwht_heads replaces the online partial rotation in front of o_proj (utils/quant_utils.py:258-281): x viewed
 * [tokens, H, D] (H heads of width D); y[t][h'][d] = scale * sum_h Had[h'][h] * x[t][h][d], i.e. the transform runs
 * ACROSS the heads for every position inside a head.  K == 1: H a power of two, Sylvester order (the reference's
 * HadamardTransform on the transposed view); K > 1: H = K * 2^m with the K x K matrix hadK mixing the 2^m-chunks
 * (K = H, m = 0 is the reference's dense had_K @ x).  H <= 64; in place allowed when K == 1. */
int rq_fwht_heads(const void* x, void* y, int dtype, int64_t tokens, int H, int D, int K, const float* hadK,
                  float scale, void* stream);

/* ------------------------------------------------------------------------------------------
 * Weight quantizer.
 * rq_find_params replaces WeightQuantizer.find_params (utils/quant_utils.py:390-457), and, with
 * groupsize > 0, the static-group loop `deepcopy(quantizer).find_params(W[:, g*gs:(g+1)*gs])`
 * (gptq_utils/gptq_plus_utils.py:995-1002, gptq_utils/gptq_utils.py:72-77).
 * W: [R, C] fp32 row stride ldw.  groupsize <= 0: one range per row (or one for the whole tensor
 * when perchannel == 0) -> scale/zero [R].  groupsize > 0: ngroups = ceil(C/groupsize) ranges
 * per row -> scale/zero [ngroups, R].  mse != 0 runs the shrink-grid search (norm, grid, maxshrink). */
int rq_find_params(const float* W, int64_t R, int64_t C, int64_t ldw, int groupsize, int perchannel, int maxq,
                   int sym, int mse, float norm, int grid, float maxshrink, float* scale, float* zero,
                   void* stream);

/* rq_quantize replaces STEQuantize / AsymSTEQuantize forward and WeightQuantizer.fake_quantize
 * (utils/quant_utils.py:60-84, 471-480).  x, deq: [R, C] of dtype; scale/zero: [R] fp32 (row r uses
 * entry r; pertensor != 0: entry 0).  honour_zero != 0: clamp(round(x/s)+z, 0, maxq), deq = s*(q-z);
 * otherwise the symmetric clamp [-(maxq+1), maxq] and deq = s*q.  codes (optional, fp32 [R, C])
 * receives the integer codes. */
int rq_quantize(const void* x, void* deq, float* codes, int dtype, int64_t R, int64_t C, const float* scale,
                const float* zero, int pertensor, int maxq, int honour_zero, void* stream);

/* rq_group_mean_square replaces the arithmetic of SaliencyCache's gradient hook
 * (gptq_utils/gptq_plus_utils.py:2388-2404): out[b, t, g] = mean over the hidden/G channels of group g of
 * grad[b, t, c]^2, in fp32.  grad: [batch, seq, hidden] of dtype with element strides stride_b / stride_t (channels
 * contiguous), so a slice along the sequence (dropped sink positions, :2395-2396) needs no copy; out: [batch, seq, G]
 * fp32 contiguous.  The layer-output Fisher sum grad^T grad (:2908-2921) is rq_hessian_accum with sal = NULL. */
int rq_group_mean_square(const void* grad, int dtype, int64_t batch, int64_t seq, int64_t stride_b, int64_t stride_t,
                         int hidden, int G, float* out, void* stream);

/* Percentile clip of the saliencies (gptq_utils/gptq_plus_utils.py:2834-2839): cap = torch.quantile(x.flatten(), q)
 * (linear interpolation between the two neighbouring order statistics, rank = fl32(q) * fl32(n - 1)), then
 * x = clamp(x, max = cap) in place; cap_out (optional, device fp32) receives the cap.  The order statistics are exact
 * (radix selection, no sort); a NaN anywhere makes the cap and every output NaN, as in torch.  n < 2^31.
 * workspace: rq_quantile_workspace_bytes() bytes of device memory, 16-byte aligned. */
size_t rq_quantile_workspace_bytes(void);
int rq_clamp_to_quantile(float* x, int64_t n, float q, float* cap_out, void* workspace, size_t workspace_bytes,
                         void* stream);

/* rq_act_quant replaces ActQuantizer.find_params followed by STEQuantize / AsymSTEQuantize.forward
 * (utils/quant_utils.py:60-84, 133-206; call site ActQuantWrapper.forward :283-295): dynamic fake quantization of
 * activations per unit, a unit being one token row (with_zero = 1: the range includes 0, :180-183) or one group of a
 * token (with_zero = 0: amax / amin of the group, :139-140).  x, out: [units, unit_len] of dtype.  dtype_math != 0:
 * every intermediate is rounded to dtype, as the reference's group-wise chain of torch ops does; dtype_math == 0: fp32
 * throughout with one final cast, as its per-token path does (the fp32 zero vector of :180 promotes it); with the
 * matching setting results agree bit for bit.  scale_out / zero_out
 * (optional, fp32 [units]) receive the ranges; scale_in / zero_in (optional) replace the range search (forward with
 * stored ranges); out may be NULL when only the ranges are wanted; codes != 0 writes the integer codes
 * (ActQuantizer.quantize, :112-117) instead of the dequantized values.  weight_rule != 0 selects the range rule of
 * WeightQuantizer.find_params_weight_groupwise (:333-352: the magnitude / span is clamped at 1e-5 instead of a zero
 * range mapping to scale 1), which makes the same kernel serve grouped weight quantization (units = row groups). */
int rq_act_quant(const void* x, void* out, int dtype, int64_t units, int unit_len, int with_zero, float clip_ratio,
                 int maxq, int sym, float* scale_out, float* zero_out, const float* scale_in, const float* zero_in,
                 int codes, int dtype_math, int weight_rule, void* stream);

/* Shrink-lattice search over grouped weight ranges: WeightQuantizer.find_params_weight_groupwise with mse
 * (utils/quant_utils.py:333-388).  x: [units, unit_len] of dtype (a weight [R, C] viewed as R * C / groupsize groups);
 * scale_out / zero_out: [units] fp32.  Starts from the group's amin / amax range (an all-zero group: (-1, +1) in the
 * asymmetric rule) and keeps, among the int(maxshrink * grid)^2 candidates (1 - i/grid) * xmin, (1 - j/grid) * xmax,
 * the first with a strictly smaller sum |q - x|^norm, every step rounded to dtype as the reference's torch ops
 * round it. */
int rq_group_mse_search(const void* x, int dtype, int64_t units, int unit_len, int maxq, int sym, float norm,
                        int grid, float maxshrink, float* scale_out, float* zero_out, void* stream);

/* Packed export (an addition: the reference registers its integer codes as an fp32 [R, C] buffer `int_weight`,
 * gptq_utils/gptq_plus_utils.py:1866-1871, and has no packed format).  rq_pack_codes turns that matrix (row stride
 * ldc) into a little-endian bit stream per row, `bits` in 2..8 bits per code in two's complement, 8 consecutive codes
 * filling `bits` bytes; out: uint8 [R, rq_packed_row_bytes(C, bits)]. */
int64_t rq_packed_row_bytes(int64_t C, int bits);
int rq_pack_codes(const float* codes, int64_t R, int64_t C, int64_t ldc, int bits, uint8_t* out, void* stream);

/* rq_clip_to_quant_bounds replaces clip_module_weight_to_quant_bounds_'s arithmetic
 * (gptq_utils/gptq_plus_utils.py:197-225: compute_quant_clip_bounds + clip_tensor_to_quant_bounds) once
 * rq_find_params has produced scale / zero: W [R, C] of dtype (row stride ldw) is clamped in place, per row, to
 * [s * -(maxq+1), s * maxq] (sym) or [s * (-zero), s * (maxq - zero)] with s = max(scale, 1e-8); the comparison
 * runs in fp32 on the widened value, the result is stored in W's dtype. */
int rq_clip_to_quant_bounds(void* W, int dtype, int64_t R, int64_t C, int64_t ldw, const float* scale,
                            const float* zero, int maxq, int sym, void* stream);

/* ------------------------------------------------------------------------------------------
 * Damped inverse-Hessian factor.
 * Replaces _compute_hessian_inverse_with_fallback's numerical body (gptq_utils/gptq_plus_utils.py:525-531)
 * and its twin in GPTQ.fasterquant (gptq_utils/gptq_utils.py:91-98), together with the act_order
 * gather H[perm][:, perm] (gptq_utils/gptq_plus_utils.py:1048) and the dead-channel fix H[dead,dead] = 1
 * (:1036-1037):  for every group g
 *     P = H[g][perm][:, perm];  P[d,d] = 1 where P[d,d] == 0;  P += damp_factor[g] * mean(diag P) * I;
 *     Hinv[g] = upper-triangular U with U^T U = P^-1          (the reference's potrf -> potri -> potrf(upper)).
 * H: [G, C, C] symmetric fp32 (only read); perm: device int64 [C] or NULL; damp_factor: HOST float [G]
 * (percdamp for the first attempt; prod(1 + p_i) - 1 over the attempts so far when damping is added
 * cumulatively on retries, as the reference does); Hinv: [G, Cp, Cp] fp32 with Cp = C rounded up to 128,
 * row stride Cp, zero below the diagonal, 16-byte aligned.
 * info: device int [G]: 0 = ok, k > 0 = non-positive pivot met in block column k-1 (not positive
 * definite: the host retries with more damping), -1 = non-finite entries in the result,
 * -2 = a bounded device-side wait of a tensor-core launch ran out (treat as RQ_ERR_TIMEOUT).
 * workspace: rq_chol_workspace_bytes(C, G) bytes, 256-byte aligned. */
size_t rq_chol_workspace_bytes(int C, int G);
int rq_chol_hinv(const float* H, const int64_t* perm, const float* damp_factor, float* Hinv, int C, int G,
                 int* info, void* workspace, size_t workspace_bytes, void* stream);
/* rq_chol_hinv with options.  flags bit 0: keep every tensor-core operand plane in bf16 (four split products, 16
 * significant bits per operand).  By default the matrix is equilibrated by powers of two (exact) and the planes are
 * fp16 (22 bits, three products): the entries of the factor are then bounded by sqrt(2) and those of its inverse by
 * sqrt(2 (1 + C / p)), which fixes the scales; only an intermediate of the inverse has no tight bound, and a matrix
 * that overflows it shows up as info = -1 (non-finite result): repeat the call with flag 1 before counting the
 * attempt as failed. */
int rq_chol_hinv_flags(const float* H, const int64_t* perm, const float* damp_factor, float* Hinv, int C, int G,
                       int* info, void* workspace, size_t workspace_bytes, int flags, void* stream);

/* ------------------------------------------------------------------------------------------
 * fasterquant.  R = out_features, C = in_features, G row sub-groups of R/G rows (group g uses Hinv[g]);
 * Hinv is the [G, Cp, Cp] factor of rq_chol_hinv.  All [R, C] work matrices are fp32 in the
 * act_order-permuted column order.
 *
 * rq_fq_prepare replaces W_sub = W[rows][:, perm] with W_sub[:, dead] = 0 and gradients_sub[:, perm]
 * (gptq_utils/gptq_plus_utils.py:1033-1049; gptq_utils/gptq_utils.py:68-82); dead = diag(H[g]) == 0.
 * Gp/Grad may be NULL. */
int rq_fq_prepare(const float* W, const float* Grad, const float* H, const int64_t* perm, int R, int C, int G,
                  float* Wp, float* Gp, void* stream);

/* rq_gptqplus_terms replaces compute_safe_beta_from_reference_loss and _compute_gradient_terms
 * (gptq_utils/gptq_plus_utils.py:174-194, 563-578) for alpha > 0:
 *   T = Gp . Hinv^T;  GHI = T . Hinv (= G . H^-1);  c = sum_j Gp*GHI - mean_j(GHI^2 / diag(H^-1));
 *   beta = 1 - sqrt(1 - clamp(2*alpha_eff*ref_loss / max(c, 2*alpha_eff*ref_loss), 0, 1));
 *   Z = beta * T;  GHinv = beta * GHI.       alpha_eff = alpha / (R*C).
 * Z, GHinv: [R, C] outputs; beta: [R]; hdiag: [G, C] scratch receiving diag(H^-1). */
int rq_gptqplus_terms(const float* Gp, const float* Hinv, int R, int C, int G, float alpha_eff, float ref_loss,
                      float* Z, float* GHinv, float* beta, float* hdiag, void* stream);

/* rq_fq_block replaces the inner column loop over one block [i1, i1+count), count <= 128
 * (gptq_utils/gptq_plus_utils.py:1296-1372; gptq_utils/gptq_utils.py:120-151):
 *   q_int = clamp(round(w/scale), -(maxq+1), maxq); q = scale*q_int; err = (w - q - GHinv[:, i]) / Hinv[i,i];
 *   W[:, i:i2] -= err (x) Hinv[i, i:i2] + GHinv[:, i:i2];  GHinv[:, i:i2] -= Z[:, i] (x) Hinv[i, i:i2].
 * Q receives q, codes q_int (int16: maxq up to 32767, e.g. 255 for asymmetric 8-bit), Eeff [R, 128] the A operand of the lazy update:
 * Err (minus (count-1-i) * Z[:, i] when plus).  Scale source: mode 0 scale_row [R]; mode 1 static
 * groups scale_tab [ngroups, R] indexed by colgrp [C]; mode 2 dynamic groups of width dyn_gs (divides
 * 128) ranged from the block-start values (sym selects the range rule), written to scale_blk
 * [C/dyn_gs, R].  plus == 0 ignores GH and Z (plain GPTQ, or GPTQ+ with beta = 0).
 *
 * rq_fq_lazy_update replaces the outer update (gptq_utils/gptq_plus_utils.py:1500-1570;
 * gptq_utils/gptq_utils.py:153):  W[:, i2:] -= Eeff . Hinv[i1:i2, i2:] + count * GHinv[:, i2:];
 * GHinv[:, i2:] -= Z[:, i1:i2] . Hinv[i1:i2, i2:].
 *
 * rq_fq_run performs both for every block of the linear.
 *
 * Modes without a host callback: inner_mode 0 = frozen, 1 = surrogate_block, 2 = surrogate_online add
 * beta * (W - anchor) to the first-order term (gptq_utils/gptq_plus_utils.py:580-584, 1190-1200, 1360-1367, 1500-1509;
 * anchor = Wp as it was before the first block, beta [R] from rq_gptqplus_terms); atomic != 0 quantizes the whole
 * block from its start values and obtains Err from the triangular solve Err . Hinv[i1:i2, i1:i2] = W - Q - GHinv
 * (:1238-1288; rq_fq_run never applies it to the last block, :1174).
 * second_order_scale (rq_fq_block, rq_fq_lazy_update): factor on the weight update of W, 1 everywhere except in
 * g_update_mode="block_gd" (:1344-1349, 1546-1550), whose optimizer steps between the blocks stay on the host. */
int rq_fq_block(float* Wp, float* GH, const float* Z, const float* Hinv, float* Q, int16_t* codes, float* Eeff,
                const float* scale_row, const float* scale_tab, const int* colgrp, float* scale_blk, int R, int C,
                int G, int i1, int count, int mode, int dyn_gs, int sym, int maxq, int plus, const float* anchor,
                const float* beta, int inner_mode, int atomic, float second_order_scale, void* stream);
int rq_fq_lazy_update(float* Wp, float* GH, const float* Z, const float* Eeff, const float* Hinv, int R, int C, int G,
                      int i1, int count, int plus, const float* anchor, const float* beta, int outer_surrogate,
                      float second_order_scale, void* stream);
int rq_fq_run(float* Wp, float* GH, const float* Z, const float* Hinv, float* Q, int16_t* codes, float* Eeff,
              const float* scale_row, const float* scale_tab, const int* colgrp, float* scale_blk, int R, int C, int G,
              int mode, int dyn_gs, int sym, int maxq, int plus, const float* anchor, const float* beta,
              int inner_mode, int atomic, void* stream);

/* Tensor-core variants of the GEMM-shaped parts of fasterquant (same reference lines as above): operands
 * are split into bf16 hi/lo planes and multiplied with four tcgen05 products per k-step, which keeps
 * fp32-level accuracy.  rq_fq_tc_prepare splits Hinv once per linear (U^T always, U too when plus) into
 * `workspace` (rq_fq_tc_workspace_bytes bytes, 1024-byte aligned); rq_gptqplus_terms_tc and rq_fq_run_tc then
 * take the same workspace (terms first: it leaves the planes of Z there for the lazy updates).
 * status: optional device int receiving RQ_ERR_TIMEOUT if a bounded device wait ran out. */
size_t rq_fq_tc_workspace_bytes(int R, int C, int G, int plus);
int rq_fq_tc_prepare(const float* Hinv, int R, int C, int G, int plus, void* workspace, size_t workspace_bytes,
                     void* stream);
int rq_gptqplus_terms_tc(const float* Gp, const float* Hinv, int R, int C, int G, float alpha_eff, float ref_loss,
                         float* Z, float* GHinv, float* beta, float* hdiag, void* workspace, size_t workspace_bytes,
                         int* status, void* stream);
int rq_fq_run_tc(float* Wp, float* GH, const float* Z, const float* Hinv, float* Q, int16_t* codes, float* Eeff,
                 const float* scale_row, const float* scale_tab, const int* colgrp, float* scale_blk, int R, int C,
                 int G, int mode, int dyn_gs, int sym, int maxq, int plus, const float* anchor, const float* beta,
                 int inner_mode, int atomic, void* workspace, size_t workspace_bytes, int* status, void* stream);

/* rq_fq_finish replaces the epilogue (gptq_utils/gptq_plus_utils.py:1850-1875; gptq_utils/gptq_utils.py:157-166):
 * out[r][perm[j]] = Q[r][j] cast to out_dtype; when out_codes != NULL also the fp32 int_weight / scale
 * buffers, un-permuted (permute_export != 0, GPTQ+) or left in permuted order (plain GPTQ). */
int rq_fq_finish(const float* Q, const int16_t* codes, const int64_t* perm, int R, int C, void* out, int out_dtype,
                 float* out_codes, float* out_scale, const float* scale_row, const float* scale_tab,
                 const int* colgrp, int permute_export, void* stream);

/* ------------------------------------------------------------------------------------------
 * GPTAQ (gptq_utils/gptaq_utils.py), the asymmetric-calibration sibling of GPTQ, on the same kernels.
 * rq_gptaq_accum replaces the dXXT update of GPTAQ.add_batch (:33-39):
 *     dXXT = beta * dXXT + (fl(x_fp * s) - fl(x * s))^T . fl(x * s)        (s = sqrt(2 / nsamples), beta = n_old / n_new)
 * x: [N, C] of its dtype (row stride ldx); x_fp: [N, C] (row stride ldf) or, with fp_channel_major != 0, [C, N] with
 * row stride ldf as the reference's input cache stores it (:185-189); dXXT [C, C] fp32, not symmetric; the product
 * runs as a split-bf16 tcgen05 GEMM over the tokens.  rq_gptaq_terms replaces :72, :84 and :105:
 *     P = alpha * triu(D . Hinv^T, 1) . Hinv,  D = dXXT[perm][:, perm] with the dead columns (H[j][j] == 0) zeroed.
 * rq_gptaq_run replaces the block loop (:107-146): per column  q = quantize(w) (zero point honoured when asym),
 * err = (w - q) / Hinv[i,i],  W1[:, i:] -= err (x) Hinv[i, i:] - w (x) P[i, i:];  per block
 * W[:, i2:] -= Err1 . Hinv[i1:i2, i2:] - W1 . P[i1:i2, i2:].  mode 0: scale_row / zero_row [R]; mode 1: static groups
 * scale_tab / zero_tab [ngroups, R] indexed by colgrp [C]; mode 2: dynamic groups of width dyn_gs (divides 128), ranged
 * from the working columns as they are when their block starts (:126-131).  Wp (permuted working weights) is consumed, Q receives the
 * quantized weights in permuted order (rq_fq_finish un-permutes).  Workspaces: 1024-byte aligned device memory. */
size_t rq_gptaq_accum_workspace_bytes(int64_t tokens, int C);
int rq_gptaq_accum(const void* x, int x_dtype, int64_t ldx, const void* x_fp, int fp_dtype, int64_t ldf,
                   int fp_channel_major, int64_t N, int C, float s, float beta, float* dXXT, void* workspace,
                   size_t workspace_bytes, int* status, void* stream);
size_t rq_gptaq_workspace_bytes(int R, int C);
int rq_gptaq_terms(const float* dXXT, const float* H, const int64_t* perm, const float* Hinv, int C, float alpha,
                   float* P, void* workspace, size_t workspace_bytes, int* status, void* stream);
int rq_gptaq_run(float* Wp, const float* Hinv, const float* P, float* Q, const float* scale_row, const float* zero_row,
                 const float* scale_tab, const float* zero_tab, const int* colgrp, int R, int C, int mode, int dyn_gs, int asym,
                 int maxq, void* workspace, size_t workspace_bytes, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* REALQ_B200_H_ */
