"""Generate the golden fixtures of this directory from the UNMODIFIED reference.

Run where the reference checkout is mounted (it cannot travel to the GPU box):

    python tests/golden/make_golden.py --ref /path/to/gptq_plus_mp_quant      (or REALQ_REFERENCE_ROOT=...)

The script imports the reference's own classes (``GPTQ``, ``GPTQPlus``, ``GPTQGuided``, ``GPTAQ``,
``WeightQuantizer``, ``ActQuantizer``, ``SaliencyCache``, ``QKRotationWrapper``, ``hadamard_utils``) on CPU, feeds them the seeded inputs of
``cases.py`` and stores their outputs in ``*.npz`` files next to this script.  The
only accommodations, none of which edits the reference: ``transformers`` is imported
first, the absent ``accelerate`` package is stubbed, and the CUDA-only calls
``torch.cuda.synchronize`` / ``memory_utils.cleanup_memory`` are turned into no-ops.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def import_reference(ref_root: str):
    import transformers  # noqa: F401  (must precede the reference's own imports)
    for name, attrs in (("accelerate", ("dispatch_model", "infer_auto_device_map")),
                        ("accelerate.utils", ("get_balanced_memory",)),
                        ("accelerate.hooks", ("remove_hook_from_module",))):
        if name not in sys.modules:
            mod = types.ModuleType(name)
            for a in attrs:
                setattr(mod, a, lambda *args, **kw: None)
            sys.modules[name] = mod
    sys.path.insert(0, ref_root)
    from utils import quant_utils, hadamard_utils, memory_utils, rotation_utils
    from gptq_utils import gptq_utils, gptq_plus_utils, gptq_guided_utils, gptaq_utils
    torch.cuda.synchronize = lambda *a, **k: None
    memory_utils.cleanup_memory = lambda *a, **k: None
    import_reference.rotation_utils = rotation_utils
    return quant_utils, hadamard_utils, gptq_utils, gptq_plus_utils, gptq_guided_utils, gptaq_utils


# cases whose full Hessian / inverse factor is stored (the rest keep only the small outputs)
HEAVY = {"plain_pc_act", "plain_ragged_block", "plus_frozen_pc", "plus_ragged"}


def np32(t):
    return t.detach().float().cpu().clone().numpy()       # clone: later in-place edits must not leak in


def gen_quantizer(qu, out):
    for name, rows, cols, bits, pc, sym, mse in cases.QUANTIZER_CASES:
        W = cases.make_weight(rows, cols, seed=11)
        q = qu.WeightQuantizer()
        q.configure(bits, perchannel=pc, sym=sym, mse=mse)
        q.find_params(W)
        deq, codes, scale = q.fake_quantize(W)
        ste = q.quantize(W)
        out[f"{name}.digest"] = np.array(cases.digest(W))
        out[f"{name}.scale"] = np32(q.scale)
        out[f"{name}.zero"] = np32(q.zero)
        out[f"{name}.maxq"] = np.array(int(q.maxq))
        out[f"{name}.fake_deq"] = np32(deq)
        out[f"{name}.fake_codes"] = np32(codes)
        out[f"{name}.ste"] = np32(ste)


def gen_wgroup(qu, out):
    """WeightQuantizer with weight_groupsize > 0 (the round-to-nearest path of rtn_fwrd), in the weight's dtype."""
    for name, rows, cols, bits, gs, sym, dtype in cases.WGROUP_CASES:
        W = cases.make_weight(rows, cols, seed=19).to(getattr(torch, dtype))
        W[0, :gs] = 0                                                # one all-zero group
        q = qu.WeightQuantizer()
        q.configure(bits, perchannel=True, sym=sym, mse=False, weight_groupsize=gs)
        q.find_params(W)
        deq, codes, scale = q.fake_quantize(W)
        out[f"{name}.digest"] = np.array(cases.digest(W.float()))
        out[f"{name}.scale"] = np32(q.scale.float())
        out[f"{name}.zero"] = np32(q.zero.float())
        out[f"{name}.fake"] = np32(deq.float())
        out[f"{name}.codes"] = np32(codes.float())
        out[f"{name}.ste"] = np32(q.quantize(W).float())


def gen_wgroup_mse(qu, out):
    """WeightQuantizer with weight_groupsize > 0 and the shrink-grid search (mse=True), in the weight's dtype."""
    for name, rows, cols, bits, gs, sym, dtype in cases.WGROUP_MSE_CASES:
        W = cases.make_weight(rows, cols, seed=23).to(getattr(torch, dtype))
        W[0, :gs] = 0                                                # one all-zero group
        W[1, :gs] = 0.5                                              # one constant group
        q = qu.WeightQuantizer()
        q.configure(bits, perchannel=True, sym=sym, mse=True, weight_groupsize=gs)
        q.find_params(W)
        out[f"{name}.digest"] = np.array(cases.digest(W.float()))
        out[f"{name}.scale"] = np32(q.scale.float())
        out[f"{name}.zero"] = np32(q.zero.float())
        out[f"{name}.ste"] = np32(q.quantize(W).float())


def gen_clip(qu, gpu, out):
    """Pre-clip of a linear's weight to its quantizer's range (clip_module_weight_to_quant_bounds_)."""
    for name, rows, cols, bits, sym, dtype in cases.CLIP_CASES:
        W = cases.make_weight(rows, cols, seed=13).to(getattr(torch, dtype))
        layer = _Lin(W.clone())
        gpu.clip_module_weight_to_quant_bounds_(layer, bits, sym, True)
        out[f"{name}.digest"] = np.array(cases.digest(W.float()))
        out[f"{name}.clipped"] = np32(layer.weight.data.float())
        out[f"{name}.changed"] = np.array(int((layer.weight.data.float() != W.float()).sum()))


def gen_saliency(gpu, out):
    """SaliencyCache's gradient hook on a linear whose output gradient is known exactly: the loss is
    sum(out * coef), so d loss / d out = coef (in the layer's dtype)."""
    for name, batch, seq, hidden, G, sink, dtype in cases.SALIENCY_CASES:
        dt = getattr(torch, dtype)
        lin = torch.nn.Linear(hidden, hidden, bias=False).to(dt)
        x = cases.make_acts(batch, seq, hidden, seed=17).to(dt)
        coef = cases.make_out_grad(batch, seq, hidden, seed=17).to(dt)
        cache = gpu.SaliencyCache(["lin"], G, sink_size=sink)
        cache.add_hook({"lin": lin})
        with torch.enable_grad():
            (lin(x) * coef).sum().backward()
        (sal,) = cache.saliency_cache["lin"]
        cache.clear_hook()
        out[f"{name}.digest"] = np.array(cases.digest(coef.float()))
        out[f"{name}.saliency"] = np32(sal)


def gen_guided(qu, gg, out):
    for (name, rows, cols, nseq, seqlen, G, bits, gs, act, static) in cases.GUIDED_CASES:
        W = cases.make_weight(rows, cols, seed=61)
        X = cases.make_acts(nseq, seqlen, cols, seed=61)
        S = cases.make_saliency(nseq, seqlen, G, seed=61)
        layer = _Lin(W)
        g = gg.GPTQGuided(layer, S, G)
        g.quantizer = qu.WeightQuantizer()
        g.quantizer.configure(bits, perchannel=True, sym=True, mse=False)
        g.add_batch(X[:1], None)
        g.add_batch(X[1:], None)
        out[f"{name}.digest"] = np.array(cases.digest(W, X, S))
        out[f"{name}.act_square"] = np32(g.act_square)
        out[f"{name}.H_trace"] = np32(torch.einsum("iig->g", g.H))
        g.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static, export_to_et=True)
        out[f"{name}.Q"] = np32(layer.weight.data)
        out[f"{name}.W_int"] = np32(layer.int_weight).astype(np.int8)
        out[f"{name}.Scale"] = np32(layer.scale)


def gen_gptaq(qu, ga, out):
    for (name, rows, cols, nseq, seqlen, bits, sym, gs, act, static, alpha) in cases.GPTAQ_CASES:
        W = cases.make_weight(rows, cols, seed=71)
        X = cases.make_acts(nseq, seqlen, cols, seed=71)
        Xfp = cases.make_fp_acts(X, seed=72)
        layer = _Lin(W)
        g = ga.GPTAQ(layer)
        g.quantizer = qu.WeightQuantizer()
        g.quantizer.configure(bits, perchannel=True, sym=sym, mse=False)
        for s_ in range(nseq):
            g.fp_inp.append(Xfp[s_].t().contiguous())              # [C, tokens], as FPInputsCache stores it
            g.add_batch(X[s_:s_ + 1], None)
        out[f"{name}.digest"] = np.array(cases.digest(W, X, Xfp))
        out[f"{name}.dXXT"] = np32(g.dXXT)
        out[f"{name}.H_diag"] = np32(torch.diag(g.H))
        g.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static, alpha=alpha)
        out[f"{name}.Q"] = np32(layer.weight.data)


def gen_qk(ru, out):
    """QKRotationWrapper behind an identity (q, k) function."""
    for name, (b, h, kvh, t_, d), bits, gs, sym, clip, dtype in cases.QK_CASES:
        dt = getattr(torch, dtype)
        q = cases.make_act_tensor((b * h, t_, d), seed=41).reshape(b, h, t_, d).to(dt)
        k = cases.make_act_tensor((b * kvh, t_, d), seed=42).reshape(b, kvh, t_, d).to(dt)
        wrap = ru.QKRotationWrapper(lambda a, c: (a, c), d, k_bits=bits, k_groupsize=gs, k_sym=sym, k_clip_ratio=clip)
        qo, ko = wrap(q, k)
        out[f"{name}.digest"] = np.array(cases.digest(q.float(), k.float()))
        out[f"{name}.q"] = np32(qo.float())
        out[f"{name}.k"] = np32(ko.float())


def gen_act_quant(qu, out):
    """ActQuantizer: find_params then forward (what ActQuantWrapper.forward does), and the integer codes."""
    for name, shape, bits, gs, sym, clip, dtype in cases.ACT_QUANT_CASES:
        x = cases.make_act_tensor(shape, seed=23).to(getattr(torch, dtype))
        q = qu.ActQuantizer()
        q.configure(bits, groupsize=gs, sym=sym, clip_ratio=clip)
        q.find_params(x)
        y = q(x)
        codes = q.quantize(x)[0]
        out[f"{name}.digest"] = np.array(cases.digest(x.float()))
        out[f"{name}.deq"] = np32(y.float())
        out[f"{name}.codes"] = np32(codes.float())
        out[f"{name}.scale"] = np32(q.scale.float())
        out[f"{name}.zero"] = np32(q.zero.float())


def gen_hadamard(hu, out):
    had_tab = torch.load(os.path.join(os.path.dirname(hu.__file__), "had_mat.pt"))
    for k in (12, 20, 28):
        out[f"had{k}"] = np32(had_tab[k]).astype(np.int8)
    out["table_keys"] = np.array(sorted(had_tab.keys()))
    import hashlib
    for k in sorted(had_tab.keys()):
        raw = np.ascontiguousarray(np32(had_tab[k]).astype(np.int8)).tobytes()
        out[f"had_sha.{k}"] = np.array(hashlib.sha256(raw).hexdigest()[:16])
    for name, rows, n, dtype in cases.HADAMARD_CASES:
        dt = getattr(torch, dtype)
        x = cases.make_acts(1, rows, n, seed=5).reshape(rows, n).to(dt)
        hadK, K = hu.get_hadK(n)
        y_cuda_form = hu.matmul_hadU_cuda(x.clone(), hadK, K)      # FWHT chunks + hadK mix
        y_strided = hu.matmul_hadU(x.clone())                      # strided radix-2 form
        out[f"{name}.digest"] = np.array(cases.digest(x))
        out[f"{name}.K"] = np.array(K)
        out[f"{name}.y"] = np32(y_cuda_form)
        out[f"{name}.y_strided"] = np32(y_strided)


class _Lin(torch.nn.Module):
    def __init__(self, W):
        super().__init__()
        self.weight = torch.nn.Parameter(W.clone(), requires_grad=False)


def gen_plain(qu, gu, out):
    for (name, rows, cols, nseq, seqlen, bits, sym, gs, act, static, bs) in cases.PLAIN_CASES:
        W = cases.make_weight(rows, cols, seed=21)
        X = cases.make_acts(nseq, seqlen, cols, seed=21)
        if "ragged" in name:
            X[..., 7] = 0.0                                         # a dead input channel
        layer = _Lin(W)
        g = gu.GPTQ(layer)
        g.quantizer = qu.WeightQuantizer()
        g.quantizer.configure(bits, perchannel=True, sym=sym, mse="mse" in name)
        for s in range(nseq):
            g.add_batch(X[s:s + 1], None)
        out[f"{name}.digest"] = np.array(cases.digest(W, X))
        if name in HEAVY:
            out[f"{name}.H"] = np32(g.H)
        g.fasterquant(blocksize=bs, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static,
                      export_to_et=True)
        out[f"{name}.Q"] = np32(layer.weight.data)
        out[f"{name}.W_int"] = np32(layer.int_weight).astype(np.int8)
        out[f"{name}.Scale"] = np32(layer.scale)


def gen_plus(qu, gpu, out):
    for (name, rows, cols, nseq, seqlen, G, bits, gs, act, static, alpha, ref_loss, mode, atomic) in cases.PLUS_CASES:
        W = cases.make_weight(rows, cols, seed=31)
        X = cases.make_acts(nseq, seqlen, cols, seed=31)
        if "ragged" in name:
            X[..., 5] = 0.0
        S = cases.make_saliency(nseq, seqlen, G, seed=31)
        Gr = cases.make_grad(rows, cols, seed=31)
        layer = _Lin(W)
        g = gpu.GPTQPlus(layer, S, Gr, G, alpha, ref_loss)
        g.quantizer = qu.WeightQuantizer()
        g.quantizer.configure(bits, perchannel=True, sym=True, mse=False)
        g.add_batch(X[:1], None)
        g.add_batch(X[1:], None)
        act_sum = g.act_square.clone()
        g.finalize_hessian()
        out[f"{name}.digest"] = np.array(cases.digest(W, X, S, Gr))
        out[f"{name}.act_sum"] = np32(act_sum)
        if name in HEAVY:
            out[f"{name}.H"] = np32(g.H)
        out[f"{name}.act_square"] = np32(g.act_square)
        # inverse factor and first-order terms of sub-group 0, as fasterquant derives them
        H0 = g.H[0].clone()
        dead = torch.diag(H0) == 0
        H0[dead, dead] = 1
        G0 = Gr[: rows // G].clone()
        if act:
            perm = torch.argsort(g.act_square, descending=True)
            H0 = H0[perm][:, perm]
            G0 = G0[:, perm]
            out[f"{name}.perm"] = perm.numpy()
        hinv_init, hinv, damp, ident = g._compute_hessian_inverse_with_fallback(H0, percdamp=0.01)
        beta, bview, Z, GH = g._compute_gradient_terms(G0, hinv_init, hinv, True)
        if name in HEAVY:
            out[f"{name}.Hinv0"] = np32(hinv)
        out[f"{name}.Hinv_init0_diag"] = np32(torch.diagonal(hinv_init))
        out[f"{name}.beta0"] = np32(beta)
        out[f"{name}.Z0"] = np32(Z)
        out[f"{name}.GHinv0"] = np32(GH)
        g.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static,
                      enable_gradient_update=True, g_update_mode=mode, export_to_et=True,
                      block_atomic_quant=atomic,
                      gradient_refresh_fn=cases.make_refresh_fn(W, Gr) if mode == "block_backward" else None)
        out[f"{name}.Q"] = np32(layer.weight.data)
        out[f"{name}.W_int"] = np32(layer.int_weight).astype(np.int8)
        out[f"{name}.Scale"] = np32(layer.scale)


def gen_plus_dynamic(qu, gpu, out):
    for (name, rows, cols, nseq, seqlen, G, bs, mse, act) in cases.PLUS_DYNAMIC_CASES:
        W = cases.make_weight(rows, cols, seed=43)
        X = cases.make_acts(nseq, seqlen, cols, seed=43)
        S = cases.make_saliency(nseq, seqlen, G, seed=43)
        Gr = cases.make_grad(rows, cols, seed=43)
        layer = _Lin(W)
        g = gpu.GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
        g.quantizer = qu.WeightQuantizer()
        g.quantizer.configure(4, perchannel=True, sym=True, mse=mse)
        g.add_batch(X, None)
        g.finalize_hessian()
        out[f"{name}.digest"] = np.array(cases.digest(W, X, S, Gr))
        g.fasterquant(blocksize=bs, percdamp=0.01, groupsize=bs, actorder=act, static_groups=False,
                      enable_gradient_update=True, g_update_mode="frozen", export_to_et=True)
        out[f"{name}.Q"] = np32(layer.weight.data)
        out[f"{name}.W_int"] = np32(layer.int_weight).astype(np.int8)
        out[f"{name}.Scale"] = np32(layer.scale)


def gen_block_gd(qu, gpu, out):
    """g_update_mode="block_gd": optimizer steps on the trailing weights between blocks, driven by the deterministic
    refresh function of cases.make_refresh_fn."""
    for (name, rows, cols, nseq, seqlen, G, gs, act, static, alpha, ref_loss, atomic, gd) in cases.GD_CASES:
        W = cases.make_weight(rows, cols, seed=37)
        X = cases.make_acts(nseq, seqlen, cols, seed=37)
        S = cases.make_saliency(nseq, seqlen, G, seed=37)
        Gr = cases.make_grad(rows, cols, seed=37)
        layer = _Lin(W)
        g = gpu.GPTQPlus(layer, S, Gr, G, alpha, ref_loss)
        g.quantizer = qu.WeightQuantizer()
        g.quantizer.configure(4, perchannel=True, sym=True, mse=False)
        g.add_batch(X, None)
        g.finalize_hessian()
        out[f"{name}.digest"] = np.array(cases.digest(W, X, S, Gr))
        reports = []
        g.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static,
                      enable_gradient_update=True, g_update_mode="block_gd", export_to_et=True,
                      block_atomic_quant=atomic, gradient_refresh_fn=cases.make_refresh_fn(W, Gr),
                      block_observer=reports.append, **gd)
        out[f"{name}.Q"] = np32(layer.weight.data)
        out[f"{name}.W_int"] = np32(layer.int_weight).astype(np.int8)
        out[f"{name}.Scale"] = np32(layer.scale)
        out[f"{name}.n_reports"] = np.array(len(reports))
        out[f"{name}.refresh_loss"] = np.array([r["mean_refresh_loss"] for r in reports], dtype=np.float64)


def gen_faults(qu, gpu, out):
    """Numeric guards: a non-SPD Hessian that needs damping retries, and non-finite entries."""
    torch.manual_seed(7)
    C = 64
    A = torch.randn(C, 8)
    H = A @ A.t()                                   # rank 8: Cholesky needs damping to succeed
    H[3, 5] += 5.0
    H[5, 3] += 5.0                                  # and an indefinite perturbation
    layer = _Lin(torch.zeros(4, C))
    g = gpu.GPTQPlus(layer, torch.ones(1, 1, 1), torch.zeros(4, C), 1, 0.0, 0.0)
    import logging
    logging.disable(logging.WARNING)
    hinv_init, hinv, damp, ident = g._compute_hessian_inverse_with_fallback(H, percdamp=0.01)
    logging.disable(logging.NOTSET)
    out["nonspd.H"] = np32(H)
    out["nonspd.Hinv"] = np32(hinv)
    out["nonspd.damp"] = np.array(damp)
    out["nonspd.identity"] = np.array(ident)


ANALYSIS_CASES = [
    # name, groupsize, actorder, static_groups, g_update_mode
    ("frozen_pc_act", -1, True, True, "frozen"),
    ("online_g128_static_act", 128, True, True, "surrogate_online"),
    ("block_g128_dynamic", 128, False, False, "surrogate_block"),
]


def gen_analysis(qu, gpu):
    """The three diagnostic summaries of GPTQPlus (nested dicts of floats), written as JSON."""
    rows, cols, nseq, seqlen, G = 64, 256, 4, 96, 4
    W = cases.make_weight(rows, cols, seed=31)
    X = cases.make_acts(nseq, seqlen, cols, seed=31)
    X[..., 5] = 0.0                                                  # a dead input channel
    S = cases.make_saliency(nseq, seqlen, G, seed=31)
    Gr = cases.make_grad(rows, cols, seed=31)
    other = cases.make_weight(rows, cols, seed=32)
    out = {}
    for name, gs, act, static, mode in ANALYSIS_CASES:
        layer = _Lin(W)
        g = gpu.GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
        g.quantizer = qu.WeightQuantizer()
        g.quantizer.configure(4, perchannel=True, sym=True, mse=False)
        g.add_batch(X, None)
        g.finalize_hessian()
        out[name] = {
            "summarize_ghinv": g.summarize_ghinv(actorder=act, max_blocks=1),
            "summarize_ghinv_off": g.summarize_ghinv(actorder=act, enable_gradient_update=False,
                                                     reference_loss_override=0.3),
            "summarize_weight_delta": g.summarize_weight_delta(actorder=act, ref_weight_override=other, max_subgroups=3),
            "analyze_ghinv_dynamics": g.analyze_ghinv_dynamics(blocksize=128, percdamp=0.01, groupsize=gs,
                                                               actorder=act, static_groups=static,
                                                               g_update_mode=mode),
        }
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("REALQ_REFERENCE_ROOT"), required="REALQ_REFERENCE_ROOT" not in os.environ,
                    help="checkout of the unmodified reference repository")
    ap.add_argument("--only", nargs="*", default=None, help="regenerate just these files, e.g. plain_gptq.npz")
    args = ap.parse_args()
    torch.set_num_threads(1)                        # fixed reduction order on any host
    qu, hu, gu, gpu, gg, ga = import_reference(args.ref)
    if args.only is None or "analysis.json" in args.only:
        import json
        with torch.no_grad():
            res = gen_analysis(qu, gpu)
        with open(os.path.join(HERE, "analysis.json"), "w") as f:
            json.dump(res, f, indent=1, sort_keys=True)
        print(f"analysis.json: {len(res)} cases")
    for fname, fn, mods in (("quantizer.npz", gen_quantizer, (qu,)),
                            ("hadamard.npz", gen_hadamard, (hu,)),
                            ("plain_gptq.npz", gen_plain, (qu, gu)),
                            ("gptq_plus.npz", gen_plus, (qu, gpu)),
                            ("gptq_plus_dynamic.npz", gen_plus_dynamic, (qu, gpu)),
                            ("block_gd.npz", gen_block_gd, (qu, gpu)),
                            ("faults.npz", gen_faults, (qu, gpu)),
                            ("clip.npz", gen_clip, (qu, gpu)),
                            ("wgroup.npz", gen_wgroup, (qu,)),
                            ("wgroup_mse.npz", gen_wgroup_mse, (qu,)),
                            ("saliency.npz", gen_saliency, (gpu,)),
                            ("act_quant.npz", gen_act_quant, (qu,)),
                            ("guided.npz", gen_guided, (qu, gg)),
                            ("gptaq.npz", gen_gptaq, (qu, ga)),
                            ("qk.npz", gen_qk, (import_reference.rotation_utils,))):
        if args.only is not None and fname not in args.only:
            continue
        out = {}
        with torch.no_grad():
            fn(*mods, out)
        path = os.path.join(HERE, fname)
        np.savez_compressed(path, **out)
        print(f"{fname}: {len(out)} arrays, {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
