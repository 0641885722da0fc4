"""The per-layer driver around ``GPTQPlus``: what the body of the reference's ``gptq_plus_fwrd`` layer loop does
for one decoder layer (gptq_utils/gptq_plus_utils.py:6930-7530), re-laid for one process per GPU.

For every sequential module group ``[q, k, v] -> [o] -> [up, gate] -> [down]`` (utils/model_utils.py:406-418):
build one ``GPTQPlus`` per linear (:6956-6998), hang ``add_batch`` on the linears as forward hooks and run the
layer over the rank's calibration shard in batches (:7000-7031), ``finalize_hessian`` (:7037-7039), ``fasterquant``
every linear of the group (:7467-7502) and free it.  Afterwards the quantized layer is replayed over the shard to
produce the next layer's inputs (:7517-7524).

The layer's forward stays stock PyTorch and is the caller's; saliencies, weight gradients and the reference loss of
each linear come from the caller too (the reference obtains them from an autograd pass,
``collect_layer_grad_hessian_stats``, :7187-7227, which this package does not replace).

Differences from the reference that a caller can see:
* the linears of a group are quantized concurrently, one CUDA stream and host thread each (they are independent);
* with more than one rank ``row_parallel`` shards every linear's rows over the ranks instead of repeating the
  whole ``fasterquant`` on every rank, and the weights are all-gathered before the next group's forward pass;
* a group's calibration pass leaves the layer's forward as soon as the last linear of the group has seen its input
  (the rest of the layer would compute values that nobody reads; the reference runs the layer to the end);
* ``hessian_once=True`` is the reference's ``layer_hessian_once`` path (:6951, :7041-7100): the Hessians of all
  linears are accumulated in ONE forward pass of the still unquantized layer, then the groups are quantized;
* ``stage_fns`` (optional) lets a caller who knows the layer's structure avoid recomputing what earlier passes
  already produced: the layer's forward cut at the inputs of every module group.  ``stage_fns[k](layer, carry)``
  takes what stage k-1 left for one batch (the batch itself for k = 0), applies the linears of group k-1, which are
  quantized by then, and everything up to the inputs of group k, and returns ``({linear name: input}, carry)``;
  the last entry, one past the groups, returns the layer's output.  The inputs the linears see are the tensors a
  pass from the top of the partly quantized layer would compute, bit for bit, so the result is the same; the work
  is ONE forward of the layer instead of one per group plus the replay.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor

import torch

from ..utils import dist_utils
from ..utils.quant_utils import WeightQuantizer
from .gptq_plus_utils import GPTQPlus

# utils/model_utils.py:406-418
SEQUENTIAL_GROUPS = [["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], ["self_attn.o_proj"],
                     ["mlp.up_proj", "mlp.gate_proj"], ["mlp.down_proj"]]


def find_linears(layer, names=None):
    """name -> nn.Linear for the quantizable projections of a decoder layer (utils/model_utils.py:398-402)."""
    found = {n: m for n, m in layer.named_modules() if isinstance(m, torch.nn.Linear) and n.endswith("_proj")}
    return found if names is None else {n: found[n] for n in names if n in found}


class _GroupDone(Exception):
    """Raised by the hook of the last linear of a group to leave the layer's forward early."""


class _FqPool:
    """One worker thread and one CUDA stream per concurrently quantized linear."""

    def __init__(self, device, width):
        self.device = device
        self.pool = ThreadPoolExecutor(max_workers=width)
        # slot 0 runs the longest job, a serial chain of short launches: higher priority keeps its next launch from
        # queueing behind the other linears' kernels
        self.streams = [torch.cuda.Stream(device=device, priority=-1 if i == 0 else 0) for i in range(width)]

    def run(self, jobs):
        """jobs: callables in priority order (longest first); returns when they are all enqueued, the current stream
        waiting for their completion."""
        main = torch.cuda.current_stream(self.device)
        if len(jobs) <= 1 or len(self.streams) <= 1:
            for job in jobs:
                job()
            return
        ready = torch.cuda.Event()
        ready.record(main)
        index = self.device.index

        def work(slot, mine):
            torch.cuda.set_device(index)
            st = self.streams[slot]
            st.wait_event(ready)
            with torch.cuda.stream(st):
                for job in mine:
                    job()
            done = torch.cuda.Event()
            done.record(st)
            return done

        width = len(self.streams)
        futures = [self.pool.submit(work, i, jobs[i::width]) for i in range(min(width, len(jobs)))]
        for f in futures:
            main.wait_event(f.result())


class LayerQuantizer:
    """Quantizes decoder layers one after the other with GPTQ+.

    ``stats_fn(layer_index, name, module) -> (saliency [n_local, T, G], gradient [R, C], reference_loss)`` supplies
    what the reference's gradient pass computes; ``forward_fn(layer, x) -> y`` runs the layer on a batch
    ``[b, T, hidden]``.  ``fasterquant_kwargs`` go to ``GPTQPlus.fasterquant`` unchanged."""

    def __init__(self, stats_fn, forward_fn, num_groups=4, alpha=0.25, w_bits=4, w_sym=True, w_clip=False,
                 hessian_accum_bsz=8, row_parallel=None, hessian_once=False, groups=None, streams=3,
                 fasterquant_kwargs=None, stage_fns=None):
        self.stats_fn, self.forward_fn = stats_fn, forward_fn
        self.stage_fns = stage_fns
        self.num_groups, self.alpha = num_groups, alpha
        self.w_bits, self.w_sym, self.w_clip = w_bits, w_sym, w_clip
        self.bsz = hessian_accum_bsz
        self.row_parallel = dist_utils.get_world_size() > 1 if row_parallel is None else bool(row_parallel)
        self.hessian_once = hessian_once
        self.groups = groups or SEQUENTIAL_GROUPS
        self.streams = streams
        self.fq_kwargs = dict(blocksize=128, percdamp=0.01, groupsize=-1, actorder=True, static_groups=True)
        self.fq_kwargs.update(fasterquant_kwargs or {})
        self._pool = None
        self.events = None              # set to a list to collect (stage, start event, end event)

    # ------------------------------------------------------------------ pieces
    def _build(self, index, subset):
        objs = {}
        for name, module in subset.items():
            saliency, gradient, ref_loss = self.stats_fn(index, name, module)
            o = GPTQPlus(module, saliency, gradient, self.num_groups, self.alpha, ref_loss)
            o.quantizer = WeightQuantizer()
            o.quantizer.configure(self.w_bits, perchannel=True, sym=self.w_sym, mse=self.w_clip)
            o.row_parallel = self.row_parallel
            objs[name] = o
        return objs

    def _accumulate(self, layer, objs, subset, inps, leave_early=True):
        seen = set()

        def hook(name):
            def tmp(_, inp, out):
                objs[name].add_batch(inp[0].data, out.data)
                seen.add(name)
                if leave_early and len(seen) == len(objs):
                    raise _GroupDone()
            return tmp

        handles = [subset[name].register_forward_hook(hook(name)) for name in objs]
        try:
            for j in range(0, inps.shape[0], self.bsz):
                seen.clear()
                try:
                    self.forward_fn(layer, inps[j:j + self.bsz])
                except _GroupDone:
                    pass
        finally:
            for h in handles:
                h.remove()
        for name in objs:
            objs[name].finalize_hessian()

    def _quantize(self, objs, subset):
        if self._pool is None:
            dev = next(iter(subset.values())).weight.device
            self._pool = _FqPool(dev, self.streams)
        order = sorted(objs, key=lambda n: -(objs[n].columns ** 3 + objs[n].rows * objs[n].columns ** 2))
        self._pool.run([(lambda n=n: objs[n].fasterquant(**self.fq_kwargs)) for n in order])
        for name in objs:
            objs[name].gather_rows_()
            objs[name].free()

    def _span(self, name, start):
        if self.events is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.events.append((name, start, e))

    def _now(self):
        if self.events is None:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    # ------------------------------------------------------------------ one layer, forward cut into stages
    def _quantize_layer_staged(self, index, layer, inps, outs):
        full = find_linears(layer)
        present = [[n for n in grp if n in full] for grp in self.groups]
        if len(self.stage_fns) != len(self.groups) + 1:
            raise ValueError(f"stage_fns needs {len(self.groups) + 1} entries (one per module group and the tail), "
                             f"got {len(self.stage_fns)}")
        carries = [inps[j:j + self.bsz] for j in range(0, inps.shape[0], self.bsz)]
        for k, names in enumerate(present):
            t = self._now()
            subset = {n: full[n] for n in names}
            objs = self._build(index, subset) if subset else {}
            for b in range(len(carries)):
                fed, carries[b] = self.stage_fns[k](layer, carries[b])
                for name, obj in objs.items():
                    obj.add_batch(fed[name].data, None)
            for obj in objs.values():
                obj.finalize_hessian()
            self._span("hessian_pass", t)
            if subset:
                t = self._now()
                self._quantize(objs, subset)
                self._span("fasterquant", t)
        t = self._now()
        if outs is None:
            outs = torch.empty_like(inps)
        for b, j in enumerate(range(0, inps.shape[0], self.bsz)):
            outs[j:j + self.bsz] = self.stage_fns[-1](layer, carries[b])
            carries[b] = None
        self._span("replay", t)
        return outs

    # ------------------------------------------------------------------ one layer
    @torch.no_grad()
    def quantize_layer(self, index, layer, inps, outs=None):
        """Quantizes ``layer`` in place from the rank's calibration inputs ``inps`` [n_local, T, hidden] and returns
        the quantized layer's outputs on them (written into ``outs`` when given)."""
        if self.stage_fns is not None and not self.hessian_once:
            return self._quantize_layer_staged(index, layer, inps, outs)
        full = find_linears(layer)
        if self.hessian_once:
            t = self._now()
            objs_all = self._build(index, {n: full[n] for grp in self.groups for n in grp if n in full})
            self._accumulate(layer, objs_all, full, inps, leave_early=False)
            self._span("hessian_pass", t)
        for grp in self.groups:
            subset = {n: full[n] for n in grp if n in full}
            if not subset:
                continue
            if self.hessian_once:
                objs = {n: objs_all[n] for n in subset}
            else:
                t = self._now()
                objs = self._build(index, subset)
                self._accumulate(layer, objs, subset, inps)
                self._span("hessian_pass", t)
            t = self._now()
            self._quantize(objs, subset)
            self._span("fasterquant", t)
        t = self._now()
        if outs is None:
            outs = torch.empty_like(inps)
        for j in range(0, inps.shape[0], self.bsz):
            outs[j:j + self.bsz] = self.forward_fn(layer, inps[j:j + self.bsz])
        self._span("replay", t)
        return outs
