#!/usr/bin/env python
"""Benchmark of the per-layer GPTQ+ quantization path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--schedule sequential|all_at_once]
                    [--workload c2|c3|c4_down] [--layers L] [--c3-forward staged|passes] [--c4-seqs S]
                    [--profile-steps P] [--no-parity] [--no-cpu]

Prints ONE JSON line.  The default workload (c2) is one Qwen3-8B-shape decoder layer (hidden 4096,
intermediate 12288, 32 query / 8 KV heads of 128): a step quantizes the layer's four module groups
[q, k, v] -> [o] -> [gate, up] -> [down] one after the other, as the reference's caller must (each group's
calibration inputs depend on the groups quantized before it); for every group it rotates the group's
calibration activations online (Hadamard on [N, 4096] and [N, 12288]), accumulates the saliency-weighted
Hessians of the group's linears over 128 x 2048 tokens, finalises them and runs fasterquant (W4, groupsize
128, act_order, GPTQ+ first-order term), the linears of a group concurrently.  `--schedule all_at_once`
feeds all seven linears in one pass and runs all seven fasterquant calls concurrently, which no caller of
the drop-in API can do for a real model; it is kept for comparison.  Inputs are seeded synthetic tensors
with the shapes and value distributions of the reference's calibration run; no dataset or checkpoint is
used.  With N > 1 (torchrun, one rank per GPU) the calibration sequences are sharded over the ranks as the
reference shards them (sequence s is the same tensor for every N), the upper triangles of the partial
Hessian sums go through one NCCL reduce-scatter per linear (plus an all-gather among the ranks that share
a saliency group), every rank quantizes its R/N rows of every linear, and one all-gather per linear
completes the weights; timing is on the device, max over ranks, and after the timed region the result is
compared with a one-rank run of the same data (`parity_vs_n1`).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

METRIC = "seconds per decoder layer quantized (Qwen3-8B shape)"


# ----------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


class EventRecorder:
    """Stand-in for the reference's QuantProfileRecorder: `section(name)` brackets a stage with CUDA events
    on the current stream; `summary()` returns milliseconds per section name."""

    def __init__(self):
        self.spans = []

    class _Span:
        def __init__(self, owner, name):
            self.owner, self.name = owner, name

        def __enter__(self):
            self.a = torch.cuda.Event(enable_timing=True)
            self.b = torch.cuda.Event(enable_timing=True)
            self.a.record()

        def __exit__(self, *exc):
            self.b.record()
            self.owner.spans.append((self.name, self.a, self.b))

    def section(self, name):
        return EventRecorder._Span(self, name)

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.spans:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out


def dist_setup():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        # plain peer-to-peer rings, no NVLink multicast objects: the exchanges here are two large reduce-scatter /
        # all-gather calls per linear, which gain nothing from in-switch reduction, and ranks that leave at slightly
        # different moments then never unmap memory that another rank's multicast object still refers to
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def dist_teardown(world):
    """All ranks leave together: nothing in flight, then the communicator goes."""
    if world > 1:
        torch.cuda.synchronize()
        torch.distributed.barrier()
        torch.cuda.synchronize()
        torch.distributed.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the Hessian kernel at C = 4096, G = 4, 8192 tokens
# (one ncu capture of that launch)
UMMA_TRAFFIC_BYTES = 1.203e9


KERNEL_TRACE = {}


def count_library_launches(step):
    """Runs `step` once under torch's kernel activity trace and returns how many of the launched kernels are this
    library's (namespace rq::); 0 when no trace can be taken.  Leaves the ten kernels with the most device time of
    that step in KERNEL_TRACE (name -> launches, milliseconds, share of all kernel time)."""
    try:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        rows = [(e.key, int(e.count), float(getattr(e, "device_time_total", 0.0) or getattr(e, "cuda_time_total", 0.0)))
                for e in prof.key_averages() if "cuda" in str(getattr(e, "device_type", "cuda")).lower()]
        total = sum(r[2] for r in rows) or 1.0
        KERNEL_TRACE.clear()
        for name, n, us in sorted(rows, key=lambda r: -r[2])[:10]:
            short = name.split("(")[0].replace("void ", "")[:70]
            KERNEL_TRACE[short] = {"launches": n, "ms": round(us / 1e3, 2), "share": round(us / total, 3)}
        return sum(n for name, n, _ in rows if "rq::" in name)
    except Exception:
        step()
        return 0


# ----------------------------------------------------------------------------------------------
# workload: one Qwen3-8B-shape decoder layer (configs[2])
# ----------------------------------------------------------------------------------------------
class LayerWorkload:
    name = ("c2: one Qwen3-8B-shape decoder layer, 7 linears W4 g128 act_order GPTQ+ (G=4), "
            "128x2048 calibration tokens bf16, online Hadamard on [N,4096] and [N,12288]")
    HID, INTER, KV = 4096, 12288, 1024
    NSEQ, T, G, BSZ = 128, 2048, 4, 8
    LINEARS = [  # name, out_features, in_features, input stream
        ("q_proj", 4096, 4096, "hid"), ("k_proj", 1024, 4096, "hid"), ("v_proj", 1024, 4096, "hid"),
        ("o_proj", 4096, 4096, "attn"), ("gate_proj", 12288, 4096, "hid"), ("up_proj", 12288, 4096, "hid"),
        ("down_proj", 4096, 12288, "mlp"),
    ]
    # the reference's caller quantizes these groups strictly one after the other, because each group's calibration
    # inputs are produced by a forward pass through the groups quantized before it (utils/model_utils.py:406-418,
    # gptq_utils/gptq_plus_utils.py:7096-7229)
    MODULE_GROUPS = [["q_proj", "k_proj", "v_proj"], ["o_proj"], ["gate_proj", "up_proj"], ["down_proj"]]
    STREAM_SEED = {"hid": 11, "attn": 12, "mlp": 13}

    def __init__(self, rank, world, nseq=None, schedule="sequential", full_data=False):
        from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
        self.rank, self.world = rank, world
        self.schedule = schedule
        total = nseq or self.NSEQ
        self.nseq_total = total
        # every rank materialises its shard of ONE dataset: sequence s is the same tensor whatever the world size
        # (full_data: all of it, for the one-rank run a data-parallel result is compared with)
        self.seqs = list(range(total)) if (full_data or world == 1) else \
            list(range(rank * (total // world), (rank + 1) * (total // world)))
        self.nseq_local = len(self.seqs)
        self.parallel = world > 1 and not full_data
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        n, T = self.nseq_local, self.T

        def acts(key, width):
            g = torch.Generator(device=dev)
            g.manual_seed(4321 + self.STREAM_SEED[key])
            ch = torch.exp(torch.randn(width, generator=g, device=dev))          # shared channel scales
            out = torch.empty(n, T, width, dtype=torch.bfloat16, device=dev)
            for i, sq in enumerate(self.seqs):
                g.manual_seed(1_000_003 * self.STREAM_SEED[key] + sq)            # by GLOBAL sequence index
                out[i] = (torch.randn(T, width, generator=g, device=dev) * ch).bfloat16()
            return out

        self.dev_in = {"hid": acts("hid", self.HID), "attn": acts("attn", self.HID), "mlp": acts("mlp", self.INTER)}
        self.host_in = None
        self.had12, _ = hu.get_hadK(self.INTER)
        gw = torch.Generator(device=dev)
        gw.manual_seed(99)                                       # weights, gradients, saliencies: same on every rank
        self.layers, self.master, self.sal, self.grad = {}, {}, {}, {}
        for name, R, C, _ in self.LINEARS:
            w = (torch.randn(R, C, generator=gw, device=dev) * 0.02).bfloat16()
            lin = torch.nn.Linear(C, R, bias=False, device=dev, dtype=torch.bfloat16)
            lin.weight.requires_grad_(False)
            self.layers[name], self.master[name] = lin, w
            s = torch.exp(3.0 * torch.randn(total, T, self.G, generator=gw, device=dev))
            cap = torch.quantile(s.flatten()[:1_000_000], 0.99)
            self.sal[name] = torch.clamp(s, max=cap)[self.seqs[0]:self.seqs[-1] + 1].contiguous()
            self.grad[name] = torch.randn(R, C, generator=gw, device=dev) * 1e-4
        self.recorder = None
        self.copy_stream = None
        self.comm_stream = None
        # "1": start each linear's exchange of partial Hessians right after its last add_batch, on a side stream
        # (GPTQPlus.begin_exchange), so that it runs under the Hessian GEMMs of the group's other linears
        self.overlap_exchange = os.environ.get("REALQ_BENCH_OVERLAP_EXCHANGE", "0") != "0"
        self.fq_streams = int(os.environ.get("REALQ_BENCH_FQ_STREAMS", str(len(self.LINEARS))))
        self.fq_pool = None
        self.stage_events = None                                 # list of (stage name, start event, end event)
        self.keep = None                                         # dict: per-linear H / codes of the last step
        self.force_act_square = None                             # dict: per-linear act_square to order the columns by

    def groups(self):
        if self.schedule == "sequential":
            return self.MODULE_GROUPS
        return [[name for name, _, _, _ in self.LINEARS]]        # all seven at once

    # ---- algorithmic work figures
    def hessian_flops(self, local=False):
        n = (self.nseq_local if local else self.nseq_total) * self.T
        return sum(2.0 * n * C * C * self.G for _, _, C, _ in self.LINEARS)

    def rotations_per_step(self):
        """(stream, width) of every online rotation a step performs: each group's pass rotates its own inputs."""
        out = []
        for grp in self.groups():
            keys = {key for name, _, _, key in self.LINEARS if name in grp}
            out += [(k, self.HID if k == "hid" else self.INTER) for k in sorted(keys) if k != "attn"]
        return out

    def fwht_bytes_local(self):
        n = self.nseq_local * self.T
        return sum(2 * n * width * 2 for _, width in self.rotations_per_step())

    def _mark(self, name, start):
        if self.stage_events is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.stage_events.append((name, start, e))

    def _quantize(self, from_host, export=False):
        from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
        from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
        from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
        if from_host and self.host_in is None:
            self.host_in = {k: v.cpu().pin_memory() for k, v in self.dev_in.items()}
        inputs = self.host_in if from_host else self.dev_in
        main = torch.cuda.current_stream()
        spec = {name: (R, C, key) for name, R, C, key in self.LINEARS}
        checksum = torch.zeros((), device=self.dev)
        # from the host every activation stream crosses PCIe once per step: a stream that a later module group
        # consumes again (the hidden states feed [q, k, v] and [gate, up]) stays on the device in between
        groups = self.groups()
        uses = {k: sum(any(spec[nm][2] == k for nm in g) for g in groups) for k in ("hid", "attn", "mlp")}
        kept = {}
        for grp in groups:
            keys = [k for k in ("hid", "attn", "mlp") if any(spec[nm][2] == k for nm in grp)]
            objs = {}
            for name in grp:
                self.layers[name].weight.data.copy_(self.master[name])
                o = GPTQPlus(self.layers[name], self.sal[name], self.grad[name], self.G, 0.25, 0.7)
                o.quantizer = WeightQuantizer()
                o.quantizer.configure(4, perchannel=True, sym=True, mse=False)
                o.profile_recorder = self.recorder
                o.row_parallel = self.parallel
                objs[name] = o
            t_pass = torch.cuda.Event(enable_timing=True) if self.stage_events is not None else None
            if t_pass is not None:
                t_pass.record()

            def fetch(s):
                """Batch s of this group's activation streams.  From the host: copied on a side stream, one batch
                ahead of the kernels that consume it, so that the transfer overlaps the Hessian GEMMs before it."""
                if s >= self.nseq_local:
                    return None
                if not from_host:
                    return {key: inputs[key][s:s + self.BSZ] for key in keys}, None
                if self.copy_stream is None:
                    self.copy_stream = torch.cuda.Stream()
                got, evs = {}, {}
                with torch.cuda.stream(self.copy_stream):
                    for key in keys:
                        if (key, s) in kept:
                            got[key], evs[key] = kept[(key, s)]
                            continue
                        got[key] = inputs[key][s:s + self.BSZ].cuda(non_blocking=True)
                        evs[key] = torch.cuda.Event()
                        evs[key].record(self.copy_stream)
                        if uses[key] > 1:
                            kept[(key, s)] = (got[key], evs[key])
                return got, evs

            nxt = fetch(0)
            for s in range(0, self.nseq_local, self.BSZ):
                batch, ready = nxt
                nxt = fetch(s + self.BSZ)
                rot = {}

                def rotated(key):
                    if key not in rot:
                        if ready is not None:
                            main.wait_event(ready[key])
                            batch[key].record_stream(main)
                        rot[key] = (hu.matmul_hadU_cuda(batch[key], None, 1) if key == "hid" else
                                    batch[key] if key == "attn" else hu.matmul_hadU_cuda(batch[key], self.had12, 12))
                    return rot[key]

                last = self.parallel and self.overlap_exchange and s + self.BSZ >= self.nseq_local
                if last and self.comm_stream is None:
                    self.comm_stream = torch.cuda.Stream()
                # in the last batch the widest linear goes first: its exchange is the longest, and it then runs under
                # the GEMMs of the others (every rank uses the same order, as the collectives require)
                for name in (sorted(grp, key=lambda nm: -spec[nm][1] * spec[nm][1]) if last else grp):
                    objs[name].add_batch(rotated(spec[name][2]), None)
                    if last:
                        objs[name].begin_exchange(self.comm_stream)
            if t_pass is not None:
                self._mark("hessian_pass", t_pass)
                t_x = torch.cuda.Event(enable_timing=True)
                t_x.record()
            for name in grp:
                objs[name].finalize_hessian()
                if self.keep is not None:
                    self.keep[name] = {"act_square": objs[name].act_square.clone()}
                if self.force_act_square is not None:
                    objs[name].act_square.copy_(self.force_act_square[name])
            if t_pass is not None:
                self._mark("exchange_finalize", t_x)
                t_f = torch.cuda.Event(enable_timing=True)
                t_f.record()

            def quantize(name):
                objs[name].fasterquant(blocksize=128, percdamp=0.01, groupsize=128, actorder=True, static_groups=True,
                                       export_to_et=export)

            if self.fq_streams <= 1 or len(grp) <= 1:
                for name in grp:
                    quantize(name)
            else:
                # The linears of a group are independent, and much of fasterquant is a chain of short dependent
                # launches (the diagonal blocks of the factorisation, the 128-column block loop): one host thread
                # and one stream per linear lets those chains overlap each other and the other linears' GEMMs.
                if self.fq_pool is None:
                    from concurrent.futures import ThreadPoolExecutor
                    self.fq_pool = ThreadPoolExecutor(max_workers=self.fq_streams)
                    # the first slot gets the longest job (a serial chain of short launches): its stream has the
                    # higher priority, so that its next launch is never queued behind the other linears' kernels
                    self.fq_stream_list = [torch.cuda.Stream(priority=-1 if i == 0 else 0)
                                           for i in range(self.fq_streams)]
                ready_ev = torch.cuda.Event()
                ready_ev.record(main)
                dev_index = self.dev.index

                def work(slot, names):
                    torch.cuda.set_device(dev_index)
                    st = self.fq_stream_list[slot]
                    st.wait_event(ready_ev)
                    with torch.cuda.stream(st):
                        for name in names:
                            quantize(name)
                    done = torch.cuda.Event()
                    done.record(st)
                    return done

                order = sorted(grp, key=lambda nm: -(spec[nm][1] ** 3 + spec[nm][0] * spec[nm][1] ** 2))
                slots = [order[i::self.fq_streams] for i in range(self.fq_streams)]
                futures = [self.fq_pool.submit(work, i, names) for i, names in enumerate(slots) if names]
                for f in futures:
                    main.wait_event(f.result())
            if t_pass is not None:
                self._mark("fasterquant", t_f)
                t_g = torch.cuda.Event(enable_timing=True)
                t_g.record()
            for name in grp:
                objs[name].gather_rows_()
                checksum += self.layers[name].weight.data.float().abs().mean()
            if t_pass is not None:
                self._mark("gather_rows", t_g)
            for name in grp:
                if self.keep is not None:
                    o = objs[name]
                    first, count = o._owned_groups if o._owned_groups is not None else (0, self.G)
                    self.keep[name].update({"H": o._H[first:first + count].clone(), "groups": (first, count),
                                            "codes": self.layers[name].int_weight.clone() if export else None,
                                            "weight": self.layers[name].weight.data.clone()})
                objs[name].free()
        return checksum

    def step_device(self):
        return self._quantize(False)

    def step_e2e(self):
        """Public API with HOST activations: each batch is copied from pinned host memory inside the timed
        region and a checksum of the quantized weights is read back."""
        return float(self._quantize(True).item())

    def h2d_bytes(self):
        """Bytes copied from the host per step: every activation stream once."""
        n = self.nseq_local * self.T
        return sum(n * (self.INTER if k == "mlp" else self.HID) * 2 for k in ("hid", "attn", "mlp"))

    def launches_per_step(self):
        """Kernel launches of this library in one step on this rank, counted from the host loops (used where no
        activity trace is taken; agrees with the traced count of the 1-GPU step to a few per cent)."""
        batches = self.nseq_local // self.BSZ
        chunks = max(1, (self.BSZ * self.T) // 8192)
        n = batches * len(self.rotations_per_step())
        n += batches * len(self.LINEARS) * chunks * 5           # scales (2) + pack + sum-of-squares reduce + GEMM
        for name, R, C, _ in self.LINEARS:
            n += 1 + (2 if self.parallel else 0)                      # finalize (+ pack / unpack of the exchange)
            blocks = C // 128
            levels = max(0, math.ceil(math.log2(max(C / 512, 1))))    # tensor-core levels of the triangular inverse
            chol = 4 * blocks + 5 * levels + 3                        # diag, panel, (split +) trailing, inverse, checks
            loop = 3 * blocks + 9                                     # prepare, splits, terms, block + 2 updates, epilogue
            n += chol + loop + 3                                      # + range searches
        return n


def parity_vs_one_rank(wl, rank, world):
    """Outside the timed region: the data-parallel result against a one-rank run of the same data.  Every rank runs
    the one-rank computation itself on the full data set (no communication), then compares: the Hessian groups it
    holds (relative Frobenius), act_square, the integer codes and the written weights of every linear.  Also
    asserts that all ranks hold the same gathered weights, bit for bit (the reference's own check,
    utils/dist_utils.py:179-199).

    act_order sorts the input channels by act_square.  Sums over the same tokens taken in another order (per rank,
    then over ranks) differ by fp32 rounding, ~1e-7 relative, and among thousands of channels a few neighbours in
    the sorted order are closer than that; where two such channels swap, every row is quantized in a different
    column order and its codes change for real, not by rounding.  That is a property of the ordering rule, not of
    the sums, so the one-rank run is given the data-parallel run's act_square to order by, and the number of
    positions at which its own order would have differed is reported beside the comparison."""
    import torch.distributed as dist
    from gptq_plus_mp_quant_b200.utils import dist_utils as du
    wl.keep = {}
    wl._quantize(False, export=True)
    got = wl.keep
    for name in got:
        du.assert_bit_exact(got[name]["weight"], tag=f"{name}.weight")
    torch.cuda.synchronize()
    solo = LayerWorkload(rank, world, nseq=wl.nseq_total, schedule=wl.schedule, full_data=True)
    solo.keep = {}
    solo.force_act_square = {name: got[name]["act_square"] for name in got}
    with du.local_only():
        solo._quantize(False, export=True)
    ref = solo.keep
    out = {}
    for name in got:
        first, count = got[name]["groups"]
        h_ref = ref[name]["H"][first:first + count].double()
        h_err = float(((got[name]["H"].double() - h_ref).norm() / h_ref.norm()).item())
        a_ref = ref[name]["act_square"]
        a_err = float(((got[name]["act_square"] - a_ref).abs() / a_ref.abs().clamp_min(1e-30)).max().item())
        moved = int((torch.argsort(got[name]["act_square"], descending=True)
                     != torch.argsort(a_ref, descending=True)).sum().item())
        diff = got[name]["codes"] != ref[name]["codes"]
        w_ok = torch.allclose(got[name]["weight"].float(), ref[name]["weight"].float(), rtol=1e-4, atol=1e-3)
        stats = torch.tensor([h_err, a_err, float(diff.float().mean().item()),
                              float(diff.any(dim=1).float().mean().item()), 0.0 if w_ok else 1.0],
                             device=wl.dev, dtype=torch.float64)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        out[name] = {"H_rel_fro": float(f"{stats[0].item():.3e}"), "act_square_rel_max": float(f"{stats[1].item():.3e}"),
                     "act_order_positions_moved": moved, "codes_differ": float(f"{stats[2].item():.3e}"),
                     "rows_touched": float(f"{stats[3].item():.3e}"),
                     "weights_allclose_atol1e-3_rtol1e-4": bool(stats[4].item() == 0.0)}
    wl.keep = None
    del solo
    return out


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's own classes (oracle/_ref, when that copy was built), else the oracle port, on the host cores
# ----------------------------------------------------------------------------------------------
CPU_SAMPLE_SEQS, CPU_SAMPLE_ROWS = 16, 1024   # bounded sample of the CPU arm: a few seconds on 16 host cores


def _cpu_arm():
    """('reference', modules) when oracle/_ref holds the reference's modules, else ('port', None)."""
    try:
        from oracle import ref_loader
        mods = ref_loader.load()
    except Exception:
        mods = None
    return ("reference", mods) if mods else ("port", None)


def cpu_layer_seconds(hess_seqs: int, fq_rows: int, arm=None):
    """Times the CPU path on a bounded sample and extrapolates to the whole layer:
    Hessian stage by its flop count, fasterquant by rows (the sample quantizes `fq_rows` rows of a
    4096-input linear with G = 4; Cholesky cost is per linear, the block loop per row).
    Returns (layer seconds extrapolated, Hessian TFLOP/s, seconds of CPU work, kind)."""
    import cases
    kind, mods = arm or _cpu_arm()
    W = LayerWorkload
    C, G, T = W.HID, W.G, W.T
    X = cases.make_acts(hess_seqs, T, C, seed=77)
    S = cases.make_saliency(hess_seqs, T, G, seed=77)
    Wt = cases.make_weight(fq_rows, C, seed=78)
    Gr = cases.make_grad(fq_rows, C, seed=78)
    if kind == "reference":
        gp, qu = mods["gptq_plus_utils"], mods["quant_utils"]
        layer = torch.nn.Linear(C, fq_rows, bias=False)
        layer.weight.data.copy_(Wt)
        obj = gp.GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
        obj.quantizer = qu.WeightQuantizer()
        obj.quantizer.configure(4, perchannel=True, sym=True, mse=False)
        t0 = time.perf_counter()
        for s in range(0, hess_seqs, W.BSZ):
            obj.add_batch(X[s:s + W.BSZ], None)
        t_h = time.perf_counter() - t0
        obj.finalize_hessian()
        t0 = time.perf_counter()
        obj._compute_hessian_inverse_with_fallback(obj.H[0].clone(), 0.01)      # one group's damped inverse factor
        t_chol = (time.perf_counter() - t0) * G                                 # per 4096-input linear
        t0 = time.perf_counter()
        obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=128, actorder=True, static_groups=True)
        t_fq = time.perf_counter() - t0
    else:
        from oracle import gptq as ogptq
        from oracle import hessian as ohess
        from oracle import quantizer as oq
        acc = ohess.GroupedHessian(C, S)
        t0 = time.perf_counter()
        for s in range(0, hess_seqs, W.BSZ):
            acc.add_batch(X[s:s + W.BSZ])
        t_h = time.perf_counter() - t0
        acc.finalize()
        q = oq.OracleWeightQuantizer()
        q.configure(4, perchannel=True, sym=True)
        t0 = time.perf_counter()
        ogptq.hinv_with_fallback(acc.H[0], 0.01)
        t_chol = (time.perf_counter() - t0) * G                            # per 4096-input linear
        t0 = time.perf_counter()
        ogptq.plus_fasterquant(Wt, acc.H, acc.act_square, Gr, q, G, 0.25, 0.7, groupsize=128, actorder=True,
                               static_groups=True)
        t_fq = time.perf_counter() - t0
    hess_tflops = 2.0 * hess_seqs * T * C * C * G / t_h / 1e12
    per_row = max(t_fq - t_chol, 0.0) / fq_rows                        # block loop + lazy update per row at C = 4096
    total_h = sum(2.0 * W.NSEQ * T * c * c * G for _, _, c, _ in W.LINEARS) / (hess_tflops * 1e12)
    total_fq = 0.0
    for _, R, Cc, _ in W.LINEARS:
        scale_c = (Cc / C)
        total_fq += t_chol * scale_c ** 3 + per_row * R * scale_c ** 2
    return total_h + total_fq, hess_tflops, t_h + t_fq, kind


def cpu_c0_full_seconds(arm=None):
    """configs[0] in full on the host cores, nothing extrapolated: plain GPTQ, 4096 x 4096, 32 x 2048 fp32 tokens fed
    one sequence per add_batch, 4-bit asymmetric per-channel, act_order, block 128."""
    kind, mods = arm or _cpu_arm()
    g = torch.Generator().manual_seed(0)
    C = 4096
    Wt = torch.randn(C, C, generator=g) * 0.02
    Wt[:, torch.randperm(C, generator=g)[:20]] *= 10.0
    ch = torch.exp(torch.randn(C, generator=g))
    X = torch.stack([torch.randn(2048, C, generator=g) * ch for _ in range(32)])
    t0 = time.perf_counter()
    if kind == "reference":
        layer = torch.nn.Linear(C, C, bias=False)
        layer.weight.data.copy_(Wt)
        obj = mods["gptq_utils"].GPTQ(layer)
        obj.quantizer = mods["quant_utils"].WeightQuantizer()
        obj.quantizer.configure(4, perchannel=True, sym=False, mse=False)
        for s in range(32):
            obj.add_batch(X[s:s + 1], None)
        obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=-1, actorder=True, static_groups=True)
    else:
        from oracle import gptq as ogptq
        from oracle import hessian as ohess
        from oracle import quantizer as oq
        acc = ohess.PlainHessian(C)
        for s in range(32):
            acc.add_batch(X[s:s + 1])
        q = oq.OracleWeightQuantizer()
        q.configure(4, perchannel=True, sym=False)
        ogptq.plain_fasterquant(Wt, acc.H, q, blocksize=128, percdamp=0.01, groupsize=-1, actorder=True,
                                static_groups=True)
    return time.perf_counter() - t0


def _cpu_sample_text(kind):
    who = "the reference's own GPTQPlus class (oracle/_ref)" if kind == "reference" else "the oracle port of the reference"
    return (f"per step: {who} on all host cores: add_batch of {CPU_SAMPLE_SEQS} of 128 sequences at C=4096 G=4 (batches of "
            f"8) plus fasterquant of a {CPU_SAMPLE_ROWS} x 4096 linear (G=4, g128 static groups, act_order, alpha=0.25); "
            "extrapolated to the layer's seven linears by flops (Hessian), C^3 (factorisation) and rows*C^2 (block loop)")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    arm = _cpu_arm()
    vals, busy = [], []
    for i in range(max(args.warmup, 0) + args.steps):
        v, tf, b, kind = cpu_layer_seconds(hess_seqs=CPU_SAMPLE_SEQS, fq_rows=CPU_SAMPLE_ROWS, arm=arm)
        if i >= args.warmup:
            vals.append(v)
            busy.append(b)
    v = sum(vals) / len(vals)
    c0 = cpu_c0_full_seconds(arm)
    sample = _cpu_sample_text(kind)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(v, 2), "unit": "s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * sum(busy) / len(busy), 1),
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": LayerWorkload.name, "sample": sample},
        "cpu_baseline": {"value": round(v, 2), "unit": "s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample, "c0_full_seconds": round(c0, 2),
                         "c0_note": "configs[0] (plain GPTQ, 4096 x 4096, 32 x 2048 fp32 tokens) run in full, "
                                    "nothing extrapolated"},
        "e2e": {"value": round(v, 2), "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def fwht_alone_gbs(dev, lengths=(4096, 12288), rows=16384, reps=10):
    """Achieved GB/s (bytes read + written) of the online rotation on its own, per row length of this workload, bf16,
    one batch of 8 x 2048 tokens per call: outside the timed region, at whatever clock the idle GPU boosts to (inside
    a step the same kernels run under the power cap of the Hessian contraction, see fwht_gbs)."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    out = {}
    for n in lengths:
        x = torch.randn(rows, n, device=dev).to(torch.bfloat16)
        hadK, K = hu.get_hadK(n)
        for _ in range(3):
            hu.matmul_hadU_cuda(x, hadK, K)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            hu.matmul_hadU_cuda(x, hadK, K)
        e1.record()
        torch.cuda.synchronize(dev)
        out[str(n)] = round(2.0 * x.numel() * 2 * reps / (e0.elapsed_time(e1) * 1e-3) / 1e9, 1)
    return out


def reference_torch_path_on_gpu(dev):
    """Informative only: the reference's arithmetic as stock torch calls on this GPU (the oracle port with CUDA
    tensors: fp32 bmm with TF32 off, torch.linalg.cholesky / cholesky_inverse, the per-column Python loop) for ONE
    4096 x 4096 linear with G = 4 and 16 sequences.  This is the library-call bar the kernels replace; it is not
    part of any timed figure of this benchmark."""
    import cases
    from oracle import gptq as ogptq
    from oracle import hessian as ohess
    from oracle import quantizer as oq
    C, G, T, nseq, R = 4096, 4, 2048, 16, 1024
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        X = cases.make_acts(nseq, T, C, seed=77).to(dev)
        S = cases.make_saliency(nseq, T, G, seed=77).to(dev)
        Wt = cases.make_weight(R, C, seed=78).to(dev)
        Gr = cases.make_grad(R, C, seed=78).to(dev)
        with torch.device(dev):                                          # the port's own tensors are created here too
            acc = ohess.GroupedHessian(C, S)
            for rep in range(2):                                         # second pass is the warm one
                acc.H.zero_()
                acc.act_square.zero_()
                acc.index = acc.token_count = 0
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for s in range(0, nseq, 8):
                    acc.add_batch(X[s:s + 8])
                torch.cuda.synchronize()
                t_h = time.perf_counter() - t0
            acc.finalize()
            q = oq.OracleWeightQuantizer()
            q.configure(4, perchannel=True, sym=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ogptq.plus_fasterquant(Wt, acc.H, acc.act_square, Gr, q, G, 0.25, 0.7, groupsize=128, actorder=True,
                                   static_groups=True)
            torch.cuda.synchronize()
            t_fq = time.perf_counter() - t0
        return {"hessian_tflops": round(2.0 * nseq * T * C * C * G / t_h / 1e12, 1),
                "hessian_ms_16seq_C4096_G4": round(t_h * 1e3, 1), "fasterquant_ms_1024x4096_G4": round(t_fq * 1e3, 1),
                "what": "stock torch on this GPU with the reference's arithmetic (fp32 bmm, TF32 off; "
                        "torch.linalg.cholesky / cholesky_inverse; per-column Python loop); informative"}
    except Exception as e:                                               # never let the extra break the line
        return {"error": repr(e)[:200]}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


# ----------------------------------------------------------------------------------------------
def run_ours(args):
    from gptq_plus_mp_quant_b200 import _lib
    rank, world, local = dist_setup()
    peaks = load_peaks()
    wl = LayerWorkload(rank, world, schedule=args.schedule)
    dev = wl.dev

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, device=dev, dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t.tolist()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks([e0.elapsed_time(e1)])[0]

    if args.profile_steps > 0:
        # for profilers: exactly this many steps of the workload, nothing else (no timing, no CPU arm)
        for _ in range(args.profile_steps):
            wl.step_device()
        torch.cuda.synchronize()
        if rank == 0:
            print(json.dumps({"profile_steps": args.profile_steps, "workload": wl.name, "schedule": wl.schedule}))
        dist_teardown(world)
        return
    warm = max(args.warmup, 3)
    for _ in range(warm):
        wl.step_device()
    sampler = ClockSampler(local)
    sampler.start()
    _lib.profile_enable(True)
    total_ms = timed(wl.step_device, args.steps)
    prof = {name: _lib.profile_read(tag) for name, tag in
            (("umma", _lib.PROF_HESSIAN_UMMA), ("pack", _lib.PROF_HESSIAN_PACK), ("fwht", _lib.PROF_FWHT),
             ("chol", _lib.PROF_CHOL), ("chol_diag", _lib.PROF_CHOL_DIAG), ("chol_panel", _lib.PROF_CHOL_PANEL),
             ("chol_trailing", _lib.PROF_CHOL_TRAILING), ("chol_inverse", _lib.PROF_CHOL_INVERSE),
             ("terms", _lib.PROF_TERMS), ("block", _lib.PROF_BLOCK), ("lazy", _lib.PROF_LAZY))}
    _lib.profile_enable(False)
    clocks = sampler.stop()
    # one extra, untimed step for the wall-clock stages of the schedule (events on the main stream between the
    # phases of every module group, summed over the groups, max over ranks) and the host-level sections
    wl.recorder = EventRecorder()
    wl.stage_events = []
    barrier()
    if world == 1:
        counted = count_library_launches(wl.step_device)   # ... and for the launch count (activity trace of that step)
    else:
        counted = 0                                  # ranks must not diverge inside a step with collectives
        wl.step_device()
    torch.cuda.synchronize()
    stage_names = ["hessian_pass", "exchange_finalize", "fasterquant", "gather_rows"]
    wall = {k: 0.0 for k in stage_names}
    for name, a, b in wl.stage_events:
        wall[name] += a.elapsed_time(b)
    wall = dict(zip(stage_names, (round(v, 2) for v in max_over_ranks([wall[k] for k in stage_names]))))
    wl.stage_events = None
    sections = {k: round(v, 2) for k, v in sorted(wl.recorder.summary().items(), key=lambda kv: -kv[1])}
    wl.recorder = None
    checksum = wl.step_e2e()
    e2e_ms = timed(wl.step_e2e, args.steps)
    parity = parity_vs_one_rank(wl, rank, world) if (world > 1 and not args.no_parity) else None

    sec_per_layer = total_ms / args.steps / 1e3
    umma_ms, umma_n = prof["umma"]
    # roofline of the dominant kernel: algorithmic flops 2*N*C^2*G of the launches / their summed duration
    achieved = wl.hessian_flops(local=True) * args.steps / (umma_ms * 1e-3) / 1e12 if umma_ms else 0.0
    peak = peaks["bf16_tflops_sustained"]
    fwht_ms, fwht_n = prof["fwht"]
    if world > 1:
        par = (f"dp{world}: calibration sequences sharded (sequence s is the same tensor for every world size); per "
               "linear one NCCL reduce-scatter of the packed upper triangles of the partial Hessians"
               + (" and an all-gather among the ranks that share a saliency group" if world > wl.G else "")
               + f"; every rank runs fasterquant on its R/{world} rows of every linear; one all-gather per linear "
               "completes the weights")
    else:
        par = "single GPU"
    out = {
        "metric": METRIC, "value": round(sec_per_layer, 4), "unit": "s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": round(total_ms / args.steps, 2), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 split products, f32 accumulate; f32 elsewhere",
        "data": "synthetic",
        "config": {"workload": wl.name, "tokens": wl.nseq_total * wl.T, "hessian_accum_bsz": wl.BSZ,
                   "schedule": (wl.schedule + (": module groups [q,k,v] -> [o] -> [gate,up] -> [down] one after the "
                                               "other, concurrency only inside a group"
                                               if wl.schedule == "sequential" else
                                               ": all seven linears fed in one pass and quantized concurrently")),
                   "l2": "per-step inputs (10.7 GB of activations, 4 GB of Hessians) exceed the 126 MB L2",
                   "parallelism": par},
        "hessian_accum_tflops": round(wl.hessian_flops() * args.steps / (umma_ms * 1e-3 + prof["pack"][0] * 1e-3)
                                      / 1e12, 1) if umma_ms else None,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(achieved / peak, 4), "traffic": UMMA_TRAFFIC_BYTES,
                     "traffic_note": "dram__bytes_read+write of one C=4096 G=4 8192-token launch (6 of the 7 launches "
                                     "per chunk), ncu; algorithmic 0.89e9",
                     "peak_source": peaks["source"] + " sustained",
                     "kernel": "rq::hess::umma_kernel<64,1> (<64,2> for fp32 inputs)", "launches": umma_n,
                     "note": "algorithmic 2*N*C^2*G; the kernel issues 2 fp16 products on the ~53% of tiles that "
                             "touch the upper triangle"},
        # device time of the tagged kernels, summed over their launches (the linears of a group run on concurrent
        # streams, so the fasterquant-side figures add up to more than the wall time of that phase)
        "kernel_ms_per_step": {k: round(v[0] / args.steps, 2) for k, v in prof.items()},
        # wall time of the phases of the schedule, from events on the main stream, summed over the module groups
        "stage_ms_per_step": wall,
        "section_ms": sections,
        "fwht_gbs": round(wl.fwht_bytes_local() * args.steps / (fwht_ms * 1e-3) / 1e9, 1) if fwht_ms else None,
        "e2e": {"value": round(e2e_ms / args.steps / 1e3, 4), "unit": "s", "h2d_bytes_per_step": wl.h2d_bytes(),
                "d2h_bytes_per_step": 4},
        "gpu_launches": (counted if counted else wl.launches_per_step()) * args.steps,
        "gpu_launches_source": ("kernels named rq::* in a CUPTI activity trace of one untimed step of the same workload"
                                if counted else "counted from the host loops (no activity trace available)"),
        "top_kernels_one_step": dict(KERNEL_TRACE) or None,   # CUPTI activity trace of the untimed extra step
        "clocks": clocks,
        "checksum": checksum,                          # sum over linears of mean |quantized weight| (rank 0's copy)
        "parity_vs_n1": parity,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        torch.set_num_threads(os.cpu_count() or 1)
        arm = _cpu_arm()
        v, tf, busy, kind = cpu_layer_seconds(hess_seqs=CPU_SAMPLE_SEQS, fq_rows=CPU_SAMPLE_ROWS, arm=arm)
        out["cpu_baseline"] = {"value": round(v, 1), "unit": "s", "cores": torch.get_num_threads(), "kind": kind,
                               "sample": _cpu_sample_text(kind) + f" ({busy:.1f} s of CPU work, Hessian stage at "
                                         f"{tf:.2f} TFLOP/s)",
                               "c0_full_seconds": round(cpu_c0_full_seconds(arm), 2),
                               "c0_note": "configs[0] (plain GPTQ, 4096 x 4096, 32 x 2048 fp32 tokens) run in full on "
                                          "the host cores, nothing extrapolated"}
        out["reference_torch_path_on_this_gpu"] = reference_torch_path_on_gpu(dev)
    if rank == 0 and world == 1:
        out["fwht_alone_gbs_bf16"] = fwht_alone_gbs(dev)
    if rank == 0:
        print(json.dumps(out))
    dist_teardown(world)


# ----------------------------------------------------------------------------------------------
# workload c3: the whole 36-layer Qwen3-8B-shape model, layer by layer (configs[3])
# ----------------------------------------------------------------------------------------------
def _common_line(args, world, value_s, steps, warm, total_ms, prof, peaks, flops_local, clocks, config, extra):
    umma_ms, umma_n = prof["umma"]
    achieved = flops_local / (umma_ms * 1e-3) / 1e12 if umma_ms else 0.0
    peak = peaks["bf16_tflops_sustained"]
    out = {"metric": METRIC, "value": round(value_s, 4), "unit": "s", "n_gpus": world, "steps": steps, "warmup": warm,
           "ms_per_step": round(total_ms / steps, 2), "higher_is_better": False, "scaling": "strong",
           "vs_baseline": None, "dtype": "f16 split products, f32 accumulate; f32 elsewhere", "data": "synthetic",
           "config": config,
           "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
                        "frac": round(achieved / peak, 4), "traffic": None, "peak_source": peaks["source"] + " sustained",
                        "kernel": "rq::hess::umma_kernel<64,1>", "launches": umma_n,
                        "note": "algorithmic 2*N*C^2*G of this rank's launches / their summed device time"},
           "kernel_ms_per_step": {k: round(v[0] / steps, 2) for k, v in prof.items()},
           "clocks": clocks}
    out.update(extra)
    return out


def _read_prof(_lib):
    return {name: _lib.profile_read(tag) for name, tag in
            (("umma", _lib.PROF_HESSIAN_UMMA), ("pack", _lib.PROF_HESSIAN_PACK), ("fwht", _lib.PROF_FWHT),
             ("chol", _lib.PROF_CHOL), ("terms", _lib.PROF_TERMS), ("block", _lib.PROF_BLOCK),
             ("lazy", _lib.PROF_LAZY))}


def run_c3(args):
    """36 random-init Qwen3-8B-shape layers: stock-PyTorch forward feeds the add_batch hooks group by group, every
    group is quantized (GPTQ+ W4 per-channel, act_order, G = 4) before the next group's forward pass, and the
    quantized layer is replayed to produce the next layer's inputs.  A step is one decoder layer."""
    from gptq_plus_mp_quant_b200 import _lib
    from gptq_plus_mp_quant_b200.gptq_utils.layer_loop import LayerQuantizer
    from gptq_plus_mp_quant_b200.utils import dist_utils as du
    import bench_model as bm
    rank, world, local = dist_setup()
    peaks = load_peaks()
    dev = torch.device("cuda", torch.cuda.current_device())
    NL, NSEQ, T, HID, VOCAB, G = args.layers, 128, 2048, 4096, 151936, 4
    sl = du.shard_slice(NSEQ, rank, world)
    n_local = sl.stop - sl.start
    gen = torch.Generator(device=dev)
    gen.manual_seed(2024)
    embed = (torch.randn(VOCAB, HID, generator=gen, device=dev) * 0.02).bfloat16()
    ids_host = torch.randint(0, VOCAB, (NSEQ, T), generator=torch.Generator().manual_seed(7)).pin_memory()
    cos, sin = bm.rotary_tables(T, 128, dev, torch.bfloat16)
    warm = max(args.warmup, 3)
    layers = [bm.DecoderLayer(device=dev, seed=i) for i in range(NL + warm)]   # the last `warm` ones are throwaways

    def stats_fn(index, name, module):
        # stand-ins for what the reference's gradient pass produces: seeded by (layer, linear), the same on every
        # rank, saliencies indexed by GLOBAL sequence
        g = torch.Generator(device=dev)
        g.manual_seed(100_003 * index + sum(name.encode()))
        s = torch.exp(3.0 * torch.randn(NSEQ, T, G, generator=g, device=dev))
        s = torch.clamp(s, max=torch.quantile(s.flatten()[:1_000_000], 0.99))[sl].contiguous()
        grad = torch.randn(module.weight.shape, generator=g, device=dev) * 1e-4
        return s, grad, 0.7

    lq = LayerQuantizer(stats_fn, lambda layer, x: layer(x, cos, sin), num_groups=G, alpha=0.25, w_bits=4,
                        hessian_accum_bsz=8, hessian_once=(args.schedule == "all_at_once"),
                        stage_fns=bm.decoder_layer_stages(cos, sin) if args.c3_forward == "staged" else None,
                        fasterquant_kwargs=dict(groupsize=-1, actorder=True, static_groups=True))

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def run_model(first, count, inps):
        outs = torch.empty_like(inps)
        for i in range(first, first + count):
            lq.quantize_layer(i, layers[i], inps, outs)
            inps, outs = outs, inps
        return inps

    def embed_ids():
        ids = ids_host[sl].to(dev, non_blocking=True)
        return embed[ids]

    x0 = embed_ids()
    run_model(NL, warm, x0.clone())                                   # warm-up on the throwaway layers
    sampler = ClockSampler(local)
    sampler.start()
    _lib.profile_enable(True)
    lq.events = []
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    e0.record()
    x = embed_ids()                                                   # host token ids -> device -> embedding
    y = run_model(0, NL, x)
    checksum = float(y.float().abs().mean().item())                   # read back
    e1.record()
    barrier()
    t_wall = time.perf_counter() - t_wall
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    total_ms = float(ms.item())
    prof = _read_prof(_lib)
    _lib.profile_enable(False)
    clocks = sampler.stop()
    walls = {}
    for name, a, b in lq.events:
        walls[name] = walls.get(name, 0.0) + a.elapsed_time(b)
    if world > 1:
        for i, layer in enumerate(layers[:NL]):
            if i in (0, NL - 1):
                du.assert_bit_exact(layer.mlp.down_proj.weight.data, tag=f"layers.{i}.mlp.down_proj")
    shapes = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (12288, 4096), (12288, 4096), (4096, 12288)]
    flops_local = NL * sum(2.0 * n_local * T * c * c * G for _, c in shapes)
    config = {"workload": f"c3: {NL}-layer Qwen3-8B-shape random-init model (vocab 151936), layer-by-layer GPTQ+ W4 "
                          "per-channel, act_order, num_groups=4, online Hadamard on the down_proj input; calibration = "
                          "128 x 2048 uniform-random token ids; stock-PyTorch layer forward feeds the hooks and replays "
                          "the quantized layer; a step is one decoder layer",
              "tokens": NSEQ * T, "hessian_accum_bsz": 8,
              "schedule": (("sequential module groups; the layer's forward is cut at the groups and run once per "
                            "layer (every stage applies the linears quantized before it), its tail is the replay"
                            if args.c3_forward == "staged" else
                            "sequential module groups, one forward pass over the shard per group plus the replay")
                           if args.schedule == "sequential" else
                           "one forward pass accumulates all seven Hessians (the reference's layer_hessian_once path), "
                           "then the groups are quantized, then the replay"),
              "parallelism": (f"dp{world}: sequences sharded, row-parallel fasterquant" if world > 1 else "single GPU"),
              "l2": "per-layer inputs (2.1 GB of hidden states per pass, 4 GB of Hessians) exceed the 126 MB L2"}
    extra = {"model_seconds": round(total_ms / 1e3, 2), "host_wall_seconds": round(t_wall, 2),
             "stage_ms_per_step": {k: round(v / NL, 2) for k, v in walls.items()},
             "e2e": {"value": round(total_ms / 1e3 / NL, 4), "unit": "s", "h2d_bytes_per_step": n_local * T * 8 // NL,
                     "d2h_bytes_per_step": 4,
                     "note": "the timed region starts from token ids in pinned host memory and ends with a checksum "
                             "read back; value and e2e are the same measurement for this workload"},
             "gpu_launches": sum(v[1] for v in prof.values()), "gpu_launches_source": "launches of the tagged kernels",
             "checksum": checksum}
    out = _common_line(args, world, total_ms / 1e3 / NL, NL, warm, total_ms, prof, peaks, flops_local, clocks, config, extra)
    if rank == 0:
        print(json.dumps(out))
    dist_teardown(world)


# ----------------------------------------------------------------------------------------------
# workload c4_down: the 28672-wide down_proj of a Llama-70B-shape layer (configs[4])
# ----------------------------------------------------------------------------------------------
def run_c4_down(args):
    from gptq_plus_mp_quant_b200 import _lib
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils import dist_utils as du
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rank, world, local = dist_setup()
    peaks = load_peaks()
    dev = torch.device("cuda", torch.cuda.current_device())
    R, C, G, NSEQ, T, BSZ = 8192, 28672, 4, args.c4_seqs, 2048, 8
    sl = du.shard_slice(NSEQ, rank, world)
    n_local = sl.stop - sl.start
    g = torch.Generator(device=dev)
    g.manual_seed(777)
    ch = torch.exp(torch.randn(C, generator=g, device=dev))
    X = torch.empty(n_local, T, C, dtype=torch.bfloat16, device=dev)
    for i, sq in enumerate(range(sl.start, sl.stop)):
        g.manual_seed(5_000_011 + sq)
        X[i] = (torch.randn(T, C, generator=g, device=dev) * ch).bfloat16()
    g.manual_seed(778)
    W = (torch.randn(R, C, generator=g, device=dev) * 0.02).bfloat16()
    S = torch.exp(3.0 * torch.randn(NSEQ, T, G, generator=g, device=dev))
    S = torch.clamp(S, max=torch.quantile(S.flatten()[:1_000_000], 0.99))[sl].contiguous()
    grad = torch.randn(R, C, generator=g, device=dev) * 1e-4
    lin = torch.nn.Linear(C, R, bias=False, device=dev, dtype=torch.bfloat16)
    lin.weight.requires_grad_(False)
    hadK, K = hu.get_hadK(C)
    walls = {"hessian_pass": 0.0, "exchange_finalize": 0.0, "fasterquant": 0.0, "gather_rows": 0.0}
    probe = {}

    def step(measure=False):
        lin.weight.data = W.clone()
        o = GPTQPlus(lin, S, grad, G, 0.25, 0.7)
        o.quantizer = WeightQuantizer()
        o.quantizer.configure(3, perchannel=True, sym=True, mse=False)
        o.row_parallel = world > 1
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        for s in range(0, n_local, BSZ):
            o.add_batch(hu.matmul_hadU_cuda(X[s:s + BSZ], hadK, K), None)
        ev[1].record()
        o.finalize_hessian()
        ev[2].record()
        if measure:
            first, count = o._owned_groups if o._owned_groups is not None else (0, G)
            probe["H"] = o._H[first]
            probe["diag_mean"] = float(o._H[first].diagonal().mean().item())
        o.fasterquant(blocksize=128, percdamp=0.01, groupsize=128, actorder=True, static_groups=True)
        ev[3].record()
        o.gather_rows_()
        ev[4].record()
        if measure:
            torch.cuda.synchronize()
            for k, name in enumerate(walls):
                walls[name] += ev[k].elapsed_time(ev[k + 1])
            probe["damp"] = o._last_fasterquant["damp_percent"]
            probe["identity"] = o._last_fasterquant["identity_fallback"]
        chk = lin.weight.data.float().abs().mean()
        o.free()
        return chk

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    sampler = ClockSampler(local)
    sampler.start()
    _lib.profile_enable(True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        chk = step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    total_ms = float(ms.item())
    prof = _read_prof(_lib)
    _lib.profile_enable(False)
    clocks = sampler.stop()
    step(measure=True)
    if world > 1:
        du.assert_bit_exact(lin.weight.data, tag="c4.down_proj.weight")
    wl = torch.tensor([walls[k] for k in walls], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(wl, op=torch.distributed.ReduceOp.MAX)
    flops_local = args.steps * 2.0 * n_local * T * C * C * G
    config = {"workload": f"c4_down: down_proj of a Llama-70B-shape layer, 8192 x 28672, Hessian [4, 28672, 28672] fp32, W3 "
                          f"groupsize 128 static groups, act_order, GPTQ+ (G=4), {NSEQ} x 2048 bf16 tokens, online Hadamard "
                          "(K = 28) on the input; a step is this one linear, not a decoder layer",
              "tokens": NSEQ * T, "hessian_accum_bsz": BSZ,
              "parallelism": (f"dp{world}: sequences sharded, packed upper-triangle reduce-scatter, row-parallel "
                              "fasterquant" if world > 1 else "single GPU"),
              "l2": "30 GB of activations and 13 GB of Hessians per step exceed the 126 MB L2"}
    extra = {"stage_ms_per_step": dict(zip(walls, (round(v, 2) for v in wl.tolist()))),
             "damp_percent": probe.get("damp"), "identity_fallback": probe.get("identity"),
             "gpu_launches": sum(v[1] for v in prof.values()), "gpu_launches_source": "launches of the tagged kernels",
             "e2e": None, "checksum": float(chk.item())}
    out = _common_line(args, world, total_ms / args.steps / 1e3, args.steps, warm, total_ms, prof, peaks, flops_local,
                       clocks, config, extra)
    out["metric"] = "seconds per 28672-wide down_proj quantized (Llama-70B shape)"
    if rank == 0:
        print(json.dumps(out))
    dist_teardown(world)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", dest="no_cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-parity", dest="no_parity", action="store_true",
                    help="N > 1: skip the comparison with a one-rank run of the same data")
    ap.add_argument("--schedule", default="sequential", choices=["sequential", "all_at_once"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4_down"])
    ap.add_argument("--profile-steps", dest="profile_steps", type=int, default=0,
                    help="c2: run exactly this many steps and exit (for a profiler's launch list)")
    ap.add_argument("--layers", type=int, default=36, help="c3: number of decoder layers")
    ap.add_argument("--c3-forward", dest="c3_forward", default="staged", choices=["staged", "passes"],
                    help="c3: 'staged' cuts the layer's forward at the module groups and keeps what earlier stages "
                         "produced (one forward per layer in all); 'passes' runs the layer from the top for every "
                         "group, as a caller without knowledge of the layer must, plus the replay")
    ap.add_argument("--c4-seqs", dest="c4_seqs", type=int, default=256, help="c4_down: calibration sequences in total")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c3":
        run_c3(args)
    elif args.workload == "c4_down":
        run_c4_down(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
