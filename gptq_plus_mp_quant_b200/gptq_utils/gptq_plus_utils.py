"""GPTQ+ on B200: the ``GPTQPlus`` object of the reference's ``gptq_utils/gptq_plus_utils.py``
(:430-2361) with the same constructor, methods, keyword arguments and attributes.  The
saliency-grouped Hessian accumulation, its finalisation, the damped inverse factor, the
first-order terms and the block loop run in the sm_100a kernels of this package; the
cross-rank sum stays a ``torch.distributed`` all-reduce."""
from __future__ import annotations

import functools
import logging
from contextlib import nullcontext

import torch

from .. import ops
from ..utils import dist_utils
from . import fasterquant_impl, ghinv_analysis

_NULL_CONTEXT = nullcontext()


def compute_quant_clip_bounds(scale, zero, maxq, sym):
    """Representable range of a quantizer per row (gptq_plus_utils.py:197-203)."""
    scale = scale.clamp(min=1e-8)
    maxq_value = int(maxq.item()) if isinstance(maxq, torch.Tensor) else int(maxq)
    if sym:
        return scale * (-(maxq_value + 1)), scale * maxq_value
    return scale * (-zero), scale * (maxq_value - zero)


def clip_tensor_to_quant_bounds(weight, clip_min, clip_max):
    """gptq_plus_utils.py:206-209, for callers that bring their own bounds."""
    clip_min = clip_min.to(weight.device, dtype=weight.dtype)
    clip_max = clip_max.to(weight.device, dtype=weight.dtype)
    return torch.minimum(torch.maximum(weight, clip_min), clip_max)


def clip_module_weight_to_quant_bounds_(module, bits, sym, mse):
    """Clamp a linear's weight, in place, to the range its (shrink-grid searched) quantizer represents
    (gptq_plus_utils.py:212-225): native range search on the fp32 view, then one clamp kernel on the weight in its
    own dtype."""
    from .. import _lib
    from ..utils import quant_utils
    if bits >= 16 or not mse:
        return
    quantizer = quant_utils.WeightQuantizer()
    quantizer.configure(bits, perchannel=True, sym=sym, mse=mse)
    w = module.weight.data
    _lib.require_cuda(w)
    quantizer.find_params(w.float())
    if not w.is_contiguous():
        raise ValueError("clip_module_weight_to_quant_bounds_ needs a contiguous weight")
    R, Cc = w.shape
    scale = quantizer.scale.to(w.device, torch.float32).reshape(-1).contiguous()
    zero = quantizer.zero.to(w.device, torch.float32).reshape(-1).contiguous()
    with torch.cuda.device(w.device):
        rc = _lib.lib.rq_clip_to_quant_bounds(_lib.ptr(w), _lib.dtype_code(w), R, Cc, w.stride(0), _lib.ptr(scale),
                                              _lib.ptr(zero), int(quantizer.maxq), 1 if sym else 0, _lib.stream_of(w))
    _lib.check("rq_clip_to_quant_bounds", rc)


class GPTQPlus:
    def __init__(self, layer, saliency: torch.Tensor, gradient: torch.Tensor, num_groups: int, alpha: float,
                 reference_loss: float, hessian_saliency_scale: float = 1.0):
        self.layer = layer
        self.dev = self.layer.weight.device
        self.rows = layer.weight.shape[0]
        self.columns = layer.weight.shape[1]
        self.num_groups = num_groups
        assert self.num_groups == saliency.shape[2], "Number of groups for GuidedQuant must match saliency shape!"
        self.alpha = alpha
        self.reference_loss = max(reference_loss, 0)
        self.hessian_saliency_scale = float(hessian_saliency_scale)
        self.saliencies = saliency.float()
        self.gradients = gradient.float()
        # [G, C, C]; an un-normalised SUM until finalize_hessian.  The accumulation kernel
        # maintains the tiles on or above the diagonal; reads through ``H`` see the full matrix.
        self._H = torch.zeros((self.num_groups, self.columns, self.columns), device=self.dev)
        self._H_upper_only = False
        self.act_square = torch.zeros((self.columns), device=self.dev)
        self.nsamples = saliency.shape[0]
        self.index = 0
        self.token_count = 0
        self._finalized = False
        self.profile_recorder = None
        # Rank that runs fasterquant for this linear when the linears of a layer are spread over the
        # ranks; None keeps the reference behaviour (every rank receives the summed Hessian).
        self.hessian_owner = None
        # Finer spreading: one owning rank per saliency group (list of num_groups ranks).  The groups of a
        # linear are independent problems (own Hessian, own rows), so finalize_hessian sums group g on
        # group_owners[g] only and fasterquant quantizes just the rows of the groups this rank owns; the
        # other rows of layer.weight keep their values until the caller gathers them from their owners.
        self.group_owners = None
        # Row-parallel mode (new, default off): with W ranks, rank r quantizes rows [r*R/W, (r+1)*R/W) of this
        # linear.  finalize_hessian then delivers to every rank the summed Hessian of the saliency group(s) that
        # cover its rows (only the upper triangles cross the wire: one reduce-scatter, plus an all-gather among the
        # ranks that share a group), fasterquant quantizes the rank's rows only, and gather_rows_() completes
        # layer.weight on every rank.  W must divide num_groups or be a multiple of it.
        self.row_parallel = False
        self._owned_groups = None       # (first, count) of the Hessian groups this rank holds after finalize
        self._exchange = None           # (stream, totals) while begin_exchange's collectives are in flight
        assert self.rows % self.num_groups == 0, (
            f"Number of rows ({self.rows}) must be divisible by num_groups ({self.num_groups})")

    @property
    def H(self):
        if self._H is not None and self._H_upper_only:
            ops.hessian_finalize(self._H, None)
            self._H_upper_only = False
        return self._H

    @H.setter
    def H(self, value):
        self._H = value
        self._H_upper_only = False

    @torch.no_grad()
    def add_batch(self, inp: torch.Tensor, out):
        """``H[g] += X^T diag(s_g) X``; ``act_square += sum x^2`` (gptq_plus_utils.py:798-857)."""
        if self._finalized:
            raise RuntimeError("add_batch called after finalize_hessian. Re-init GPTQPlus to reuse.")
        if self._exchange is not None:
            raise RuntimeError("add_batch called after begin_exchange: the partial sums are already being reduced.")
        rec = self.profile_recorder
        with rec.section("add_batch.total") if rec else _NULL_CONTEXT:
            if inp.dim() == 2:
                inp = inp.unsqueeze(0)
            else:
                assert inp.dim() == 3, "Input must be 2D or 3D. Got %dD." % inp.dim()
            with rec.section("add_batch.slice_saliency") if rec else _NULL_CONTEXT:
                bsz = inp.shape[0]
                sal_batch = self.saliencies[self.index: self.index + bsz].to(self.dev, non_blocking=True)
                self.index += bsz
            if sal_batch.dim() == 3 and inp.shape[1] > sal_batch.shape[1]:
                inp = inp[:, inp.shape[1] - sal_batch.shape[1]:]          # leading sink tokens carry no saliency
            with rec.section("add_batch.prepare_inputs") if rec else _NULL_CONTEXT:
                inp = inp.reshape(-1, inp.shape[-1])
                sal_batch = sal_batch.reshape(-1, sal_batch.shape[-1])
                n_tokens = inp.shape[0]
            with rec.section("add_batch.hessian_block") if rec else _NULL_CONTEXT:
                ops.hessian_accum(inp, sal_batch, self._H, self.act_square, alpha=1.0, beta=1.0,
                                  pipeline=ops.HESSIAN_PIPELINE)
                self._H_upper_only = True
            self.token_count += n_tokens

    def _reduce_sums_(self):
        """The cross-rank sums of the accumulators, to the owners that hessian_owner / group_owners / row_parallel
        name.  Returns the summed (sample count, token count) as a device tensor when it travelled with
        act_square, else None."""
        if self.row_parallel and dist_utils.get_world_size() > 1:
            _, _, _, pieces = dist_utils.row_parallel_layout(self.num_groups)
            packed = ops.pack_upper(self._H, pieces)
            first, count = dist_utils.exchange_group_sums_(packed)
            ops.unpack_upper(packed[first:first + count], self._H[first:first + count])
            self._owned_groups = (first, count)
            # the two counters ride along with act_square (both are integers below 2^24: exact in fp32)
            small = torch.cat([self.act_square, torch.tensor([float(self.index), float(self.token_count)],
                                                             device=self.act_square.device)])
            dist_utils.allreduce_sum_(small)
            self.act_square.copy_(small[:-2])
            return small[-2:].double()
        if self.group_owners is not None:
            assert len(self.group_owners) == self.num_groups
            dist_utils.reduce_groups_to_owners_(self._H, self.group_owners)
        elif self.hessian_owner is None:
            dist_utils.allreduce_sum_(self._H)
        else:
            dist_utils.reduce_sum_(self._H, self.hessian_owner)
        dist_utils.allreduce_sum_(self.act_square)
        return None

    @torch.no_grad()
    def begin_exchange(self, stream=None):
        """Starts finalize_hessian's cross-rank sums without waiting for them.  Call it after this linear's last
        add_batch, on every rank and in the same order over linears; the collectives are enqueued on ``stream``
        (which first waits for the work already queued on the current stream), so that they overlap whatever the
        current stream runs next, e.g. the Hessian GEMMs of the other linears.  The host does not block.
        finalize_hessian then waits for them instead of issuing its own.  No-op for a single process."""
        if self._finalized or self._exchange is not None or dist_utils.get_world_size() <= 1:
            return
        ops.hessian_join(self.dev)
        on_gpu = self._H.is_cuda
        side = None
        if on_gpu:
            cur = torch.cuda.current_stream(self.dev)
            side = stream if stream is not None else cur
            if side is not cur:
                side.wait_stream(cur)
        with (torch.cuda.stream(side) if on_gpu else _NULL_CONTEXT):
            totals = self._reduce_sums_()
            if totals is None:
                totals = torch.tensor([float(self.index), float(self.token_count)], dtype=torch.float64,
                                      device=self._H.device)
                dist_utils.allreduce_sum_(totals)
        self._exchange = (side, totals)

    @torch.no_grad()
    def finalize_hessian(self):
        """All-reduce the sums over ranks, normalise, symmetrise, zero non-finite entries
        (gptq_plus_utils.py:859-908)."""
        if self._finalized:
            return
        if self._exchange is not None:
            side, totals = self._exchange
            self._exchange = None
            if side is not None:
                torch.cuda.current_stream(self.dev).wait_stream(side)
            total_samples, total_tokens = (float(v) for v in totals.tolist())
        else:
            ops.hessian_join(self.dev)
            totals = self._reduce_sums_()
            if totals is not None:
                total_samples, total_tokens = (float(v) for v in totals.tolist())
            else:
                total_samples = dist_utils.allreduce_sum_scalar(self.index)
                total_tokens = dist_utils.allreduce_sum_scalar(self.token_count)
        if total_samples <= 0 or total_tokens <= 0:
            raise RuntimeError("finalize_hessian called before any add_batch ran.")
        seq_len = total_tokens / total_samples
        held = self._H
        if self._owned_groups is not None:             # row-parallel: only the groups this rank will factorise
            first, count = self._owned_groups
            held = self._H[first:first + count]
        counts = ops.hessian_finalize(held, self.act_square, div_tokens=total_samples * seq_len,
                                      div_scale=self.hessian_saliency_scale, div_seq=seq_len, sanitize=True)
        self._H_upper_only = False
        ops.check_status(self.dev)
        n_nan, n_inf = (int(v) for v in counts.tolist())
        if n_nan or n_inf:
            logging.warning(
                "finalize_hessian: non-finite in H (nan=%d, inf=%d, total=%d, module=%s); "
                "sanitising to 0 — fasterquant's dead-channel check will take over.",
                n_nan, n_inf, self._H.numel(), self.layer.__class__.__name__)
        self._finalized = True

    def fasterquant(self, blocksize=128, percdamp=0.01, groupsize=-1, actorder=False, static_groups=False,
                    enable_gradient_update=True, g_update_mode="frozen", export_to_et=False, profile_recorder=None,
                    gradient_refresh_fn=None, grad_lr=1e-3, grad_optimizer="sgd", curvature_damping=0.1,
                    grad_reg_strategy="none", grad_reg_lambda=0.0, grad_gate_floor=0.1, grad_gate_sharpness=1.0,
                    grad_gate_sine_amp=0.0, second_order_scale=1.0, block_atomic_quant=False, block_observer=None,
                    grad_clip=1.0, diagnostic_recorder=None, slide_refresh_start=0, slide_refresh_block_total=None,
                    refresh_full_metrics=False):
        """gptq_plus_utils.py:910-1896."""
        profile_recorder = profile_recorder or self.profile_recorder
        with profile_recorder.section("fasterquant.total") if profile_recorder else _NULL_CONTEXT:
            fasterquant_impl.plus_fasterquant(
                self, blocksize=blocksize, percdamp=percdamp, groupsize=groupsize, actorder=actorder,
                static_groups=static_groups, enable_gradient_update=enable_gradient_update,
                g_update_mode=g_update_mode, export_to_et=export_to_et, profile_recorder=profile_recorder,
                gradient_refresh_fn=gradient_refresh_fn, grad_reg_strategy=grad_reg_strategy,
                second_order_scale=second_order_scale, block_atomic_quant=block_atomic_quant,
                block_observer=block_observer, diagnostic_recorder=diagnostic_recorder, grad_clip=grad_clip,
                refresh_full_metrics=refresh_full_metrics,
                gd=dict(grad_lr=grad_lr, grad_optimizer=grad_optimizer, curvature_damping=curvature_damping,
                        grad_reg_strategy=grad_reg_strategy, grad_reg_lambda=grad_reg_lambda,
                        grad_gate_floor=grad_gate_floor, grad_gate_sharpness=grad_gate_sharpness,
                        grad_gate_sine_amp=grad_gate_sine_amp, second_order_scale=second_order_scale,
                        grad_clip=grad_clip, slide_refresh_start=slide_refresh_start,
                        slide_refresh_block_total=slide_refresh_block_total))
        if torch.any(torch.isnan(self.layer.weight.data)):
            logging.warning("NaN in weights")
            raise ValueError("NaN in weights")

    @torch.no_grad()
    # ---- diagnostics (gptq_plus_utils.py:489-492, 1898-2347): summaries of G.H^-1 and of the weight drift
    def _selected_column_count(self, blocksize, max_blocks):
        return ghinv_analysis.selected_column_count(self, blocksize, max_blocks)

    def analyze_ghinv_dynamics(self, blocksize=128, percdamp=0.01, groupsize=-1, actorder=False, static_groups=False,
                               enable_gradient_update=True, g_update_mode="frozen", max_subgroups=None,
                               max_blocks=None, return_tensors=False):
        return ghinv_analysis.analyze_ghinv_dynamics(
            self, blocksize=blocksize, percdamp=percdamp, groupsize=groupsize, actorder=actorder,
            static_groups=static_groups, enable_gradient_update=enable_gradient_update, g_update_mode=g_update_mode,
            max_subgroups=max_subgroups, max_blocks=max_blocks, return_tensors=return_tensors)

    def summarize_ghinv(self, percdamp=0.01, blocksize=128, actorder=False, enable_gradient_update=True,
                        gradient_override=None, reference_loss_override=None, max_subgroups=None, max_blocks=None,
                        return_tensors=False):
        return ghinv_analysis.summarize_ghinv(
            self, percdamp=percdamp, blocksize=blocksize, actorder=actorder,
            enable_gradient_update=enable_gradient_update, gradient_override=gradient_override,
            reference_loss_override=reference_loss_override, max_subgroups=max_subgroups, max_blocks=max_blocks,
            return_tensors=return_tensors)

    def summarize_weight_delta(self, blocksize=128, actorder=False, max_subgroups=None, max_blocks=None,
                               ref_weight_override=None, weight_override=None, return_tensors=False):
        return ghinv_analysis.summarize_weight_delta(
            self, blocksize=blocksize, actorder=actorder, max_subgroups=max_subgroups, max_blocks=max_blocks,
            ref_weight_override=ref_weight_override, weight_override=weight_override, return_tensors=return_tensors)

    def gather_rows_(self):
        """Row-parallel mode: after fasterquant every rank holds its own rows of the quantized weight; this
        all-gathers them (and the export buffers, if present) so that layer.weight is complete on every rank."""
        if not self.row_parallel or dist_utils.get_world_size() <= 1:
            return
        w = self.layer.weight.data
        if not w.is_contiguous():
            w = self.layer.weight.data = w.contiguous()
        dist_utils.allgather_rows_(w)
        for name in ("int_weight", "scale"):
            buf = getattr(self.layer, name, None)
            if isinstance(buf, torch.Tensor) and buf.shape[0] == self.rows:
                dist_utils.allgather_rows_(buf)

    def free(self):
        # Drops the Hessian; unlike the reference this does not return cached blocks to the driver
        # (torch.cuda.empty_cache / cleanup_memory): the next linear re-uses them without a cudaMalloc.
        ops.hessian_join(self.dev)          # no contraction may still be writing the buffer that is released
        self.H = None
        self.Losses = None


# loss scale of the static saliency / Fisher precompute and its square (gptq_plus_utils.py:34-37)
_E2E_PRECOMPUTE_LOSS_GRAD_SCALE = 1000.0
_E2E_PRECOMPUTE_QUADRATIC_SCALE = _E2E_PRECOMPUTE_LOSS_GRAD_SCALE * _E2E_PRECOMPUTE_LOSS_GRAD_SCALE


class SaliencyCache:
    """Per-token saliencies of the named linears: mean squared output gradient per channel group, collected by a
    gradient hook during the calibration backward pass (gptq_plus_utils.py:2363-2431).  The hook's arithmetic runs in
    one kernel that reads the gradient once, sink positions sliced off without a copy."""

    def __init__(self, names, num_groups, sink_size=0, clip_percentile=None):
        self.num_groups = num_groups
        # cap every hook call's saliencies at this quantile of theirs (the saliency_clip_percentile of the
        # calibration backward pass, gptq_plus_utils.py:2834-2839); None or outside (0, 1): no clip
        self.clip_percentile = clip_percentile
        self.saliency_cache = {name: [] for name in names}
        self.names = names
        self.handles = []
        self.hooks_enabled = False
        self.sink_size = max(0, int(sink_size))

    def cache_saliency(self, module, inp, out, name):
        out.retain_grad()

        def grad_hook(grad):
            if not self.hooks_enabled:
                return
            g = grad
            if self.sink_size > 0 and g.dim() >= 2 and g.shape[1] > self.sink_size:
                g = g[:, self.sink_size:]
            sal = ops.group_mean_square(g, self.num_groups)
            if self.clip_percentile is not None and 0 < self.clip_percentile < 1:
                ops.clamp_to_quantile_(sal, self.clip_percentile)
            self.saliency_cache[name].append(sal)

        out.register_hook(grad_hook)

    def add_hook(self, full, enable=True):
        for name in self.names:
            self.handles.append(
                full.get(name, full.get(name + ".module", None)).register_forward_hook(
                    functools.partial(self.cache_saliency, name=name)))
        self.hooks_enabled = enable

    def enable_hooks(self):
        self.hooks_enabled = True

    def disable_hooks(self):
        self.hooks_enabled = False

    def clear_hook(self):
        for h in self.handles:
            h.remove()
        self.handles = []
        self.hooks_enabled = False

    def clear_cache(self):
        for name in self.names:
            self.saliency_cache[name] = []


def fisher_accumulate_(fisher: torch.Tensor, grad: torch.Tensor, sink_size: int = 0,
                       scale: float = _E2E_PRECOMPUTE_QUADRATIC_SCALE) -> torch.Tensor:
    """``fisher += grad_flat^T grad_flat / scale`` for a layer-output gradient ``[batch, seq, hidden]``, the body of the
    Fisher hook (gptq_plus_utils.py:2908-2921) on the tensor-core Gram kernel.  Only the tiles on or above the
    diagonal are maintained; fisher_finalize_ mirrors them once after the last batch."""
    if sink_size > 0 and grad.dim() >= 2 and grad.shape[1] > sink_size:
        grad = grad[:, sink_size:]
    flat = grad.detach().reshape(-1, grad.shape[-1])
    ops.hessian_accum(flat, None, fisher, None, alpha=1.0 / float(scale), beta=1.0)
    return fisher


def fisher_finalize_(fisher: torch.Tensor) -> torch.Tensor:
    """Fill the lower triangle of a matrix accumulated by fisher_accumulate_."""
    ops.hessian_finalize(fisher, None)
    return fisher
