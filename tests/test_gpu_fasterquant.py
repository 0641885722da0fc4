"""Parity of the Cholesky / first-order-term / fasterquant kernels with the CPU oracle and the
golden outputs of the unmodified reference.

Tolerances: Hinv <= 2e-5 relative Frobenius when both sides factor the same H (fp32 factorisations
of matrices with condition number ~1e3-1e4 differ by that much between LAPACK builds as well) and
<= 5e-4 when the H comes from a few hundred tokens through the split-bf16 kernel (its ~3e-6 error is
amplified by the conditioning); beta, Z, GHinv <= 1e-3 relative there; per-row and static-group
scales <= 1e-6 relative, dynamic-group scales (ranged from the updated working weights) <= 1e-4; integer codes: >= 99.9 % identical on the pooled cases, every
mismatch off by exactly one code (a rounding tie that fell the other way) or downstream of one in
the same row.
"""
import numpy as np
import pytest
import torch

import cases
from oracle import gptq as ogptq
from oracle import hessian as ohess
from oracle import quantizer as oq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_fro(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm())


def _layer(W, dtype=torch.float32):
    layer = torch.nn.Linear(W.shape[1], W.shape[0], bias=False, device=DEV, dtype=dtype)
    layer.weight.data.copy_(W)
    return layer


# ---------------------------------------------------------------------------- Cholesky route
@pytest.mark.parametrize("C,G,actorder", [(256, 2, True), (200, 1, False), (384, 4, True), (1024, 2, True)])
def test_hinv_factor_vs_oracle(C, G, actorder):
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    X = cases.make_acts(4, max(128, C // 2), C, seed=17)
    S = cases.make_saliency(4, max(128, C // 2), G, seed=17)
    acc = ohess.GroupedHessian(C, S)
    acc.add_batch(X)
    acc.finalize()
    perm = torch.argsort(acc.act_square, descending=True) if actorder else None
    Hinv, damp, ident = fi.hinv_with_fallback(acc.H.to(DEV), None if perm is None else perm.to(DEV), 0.01, True)
    assert Hinv.shape[-1] % 128 == 0
    for g in range(G):
        Hg = acc.H[g].clone()
        if perm is not None:
            Hg = Hg[perm][:, perm]
        _, up, p, fb = ogptq.hinv_with_fallback(Hg, 0.01)
        assert not fb and not ident[g] and abs(p - damp[g]) < 1e-12
        got = Hinv[g, :C, :C].cpu()
        assert rel_fro(got, up) < 2e-5
        assert float(torch.tril(got, -1).abs().max()) == 0.0          # strictly upper, like chol(upper=True)
        # defining property, checked in fp64: U^T U (H + lambda I) = I
        damped = Hg.double() + 0.01 * Hg.double().diagonal().mean() * torch.eye(C, dtype=torch.float64)
        resid = got.double().t() @ got.double() @ damped - torch.eye(C, dtype=torch.float64)
        assert float(resid.abs().max()) < 5e-3


@pytest.mark.parametrize("name", ["plus_frozen_pc", "plus_ragged"])
def test_hinv_factor_from_reference_hessian(golden, name):
    """Same H in (the reference's own), reference's Hinv out."""
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    g = golden("gptq_plus.npz")
    H = torch.from_numpy(g[f"{name}.H"]).to(DEV).contiguous()
    perm = torch.from_numpy(g[f"{name}.perm"]).to(DEV)
    Hinv, damp, ident = fi.hinv_with_fallback(H, perm, 0.01, True)
    C = H.shape[-1]
    assert rel_fro(Hinv[0, :C, :C], torch.from_numpy(g[f"{name}.Hinv0"])) < 2e-5
    assert damp[0] == 0.01


def test_hinv_full_size_property():
    """C = 4096 (benchmark size): U^T U (H + lambda I) = I to fp32 accuracy, no CPU factorisation needed."""
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    C = 4096
    g = torch.Generator(device="cpu").manual_seed(5)
    X = (torch.randn(8192, C, generator=g) * torch.exp(torch.randn(C, generator=g))).to(DEV)
    H = (X.t() @ X / X.shape[0]).reshape(1, C, C).contiguous()
    Hinv, damp, ident = fi.hinv_with_fallback(H, None, 0.01, True)
    assert damp[0] == 0.01 and not ident[0]
    U = Hinv[0].double()
    P = H[0].double() + 0.01 * H[0].double().diagonal().mean() * torch.eye(C, dtype=torch.float64, device=DEV)
    probe = torch.randn(C, 8, dtype=torch.float64, device=DEV)
    back = U.t() @ (U @ (P @ probe))
    assert float((back - probe).norm() / probe.norm()) < 1e-3


def test_hinv_c28672_property():
    """The widest input of the benchmark configurations (Llama-70B down_proj, 28672 channels, one saliency group's
    worth of work): the factor is finite, strictly upper, needs no retry, and U^T U (H + lambda I) v = v in fp64."""
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    C, n = 28672, 57344
    g = torch.Generator(device=DEV).manual_seed(9)
    ch = torch.exp(torch.randn(C, generator=g, device=DEV))
    H = torch.zeros(C, C, device=DEV)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for _ in range(n // 4096):
            x = torch.randn(4096, C, generator=g, device=DEV) * ch
            H.addmm_(x.t(), x)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    H /= n
    H3 = H.reshape(1, C, C)
    Hinv, damp, ident = fi.hinv_with_fallback(H3, None, 0.01, True)
    assert damp[0] == 0.01 and not ident[0]
    assert bool(torch.isfinite(Hinv).all())
    lam = 0.01 * float(H.diagonal().double().mean())
    probe = torch.randn(C, 4, dtype=torch.float64, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
    hv = torch.empty_like(probe)
    for c0 in range(0, C, 4096):                            # H v in fp64 without an fp64 copy of H
        hv[c0:c0 + 4096] = H[c0:c0 + 4096].double() @ probe
    hv += lam * probe
    uv = torch.empty_like(probe)
    for c0 in range(0, C, 4096):
        uv[c0:c0 + 4096] = Hinv[0, c0:c0 + 4096, :C].double() @ hv
    back = torch.zeros_like(probe)
    for c0 in range(0, C, 4096):
        back += Hinv[0, c0:c0 + 4096, :C].double().t() @ uv[c0:c0 + 4096]
    err = float((back - probe).norm() / probe.norm())
    print(f"C=28672: |U^T U (H + lambda I) v - v| / |v| = {err:.3e}")
    assert err < 1e-3
    assert float(torch.tril(Hinv[0, :4096, :4096], -1).abs().max()) == 0.0


def test_nonspd_retries_like_reference(golden):
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    g = golden("faults.npz")
    H = torch.from_numpy(g["nonspd.H"]).reshape(1, 64, 64).to(DEV)
    import logging
    logging.disable(logging.WARNING)
    Hinv, damp, ident = fi.hinv_with_fallback(H, None, 0.01, True)
    logging.disable(logging.NOTSET)
    assert ident[0] == bool(g["nonspd.identity"])
    # the retry count may differ by one step when a pivot sits at the edge of positivity
    assert abs(damp[0] - float(g["nonspd.damp"])) <= 0.0015 * 2 + 1e-9
    if abs(damp[0] - float(g["nonspd.damp"])) < 1e-12:
        assert rel_fro(Hinv[0, :64, :64], torch.from_numpy(g["nonspd.Hinv"])) < 1e-3


def test_hopeless_hessian_falls_back_or_raises():
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    import logging
    H = -torch.eye(128, device=DEV).reshape(1, 128, 128) * 3.0       # negative definite: no damping < 1 helps
    logging.disable(logging.WARNING)
    try:
        Hinv, damp, ident = fi.hinv_with_fallback(H.clone(), None, 0.9, True)
        assert ident[0] and damp[0] >= 1.0
        assert torch.equal(Hinv[0], torch.eye(128, device=DEV))
        with pytest.raises(ValueError):
            fi.hinv_with_fallback(H.clone(), None, 0.9, False)
    finally:
        logging.disable(logging.NOTSET)
    with pytest.raises(ValueError):
        fi.hinv_with_fallback(H.clone(), None, 0.0, True)


# ---------------------------------------------------------------------------- full objects vs the reference
def _code_report(got, ref, order=None):
    """Share of differing codes, rows touched, and per touched row the size of its first deviation in
    processing order (``order`` = the act_order permutation; later deviations follow from the first)."""
    if order is not None:
        got, ref = got[:, order], ref[:, order]
    diff = (got != ref)
    frac = float(diff.float().mean())
    rows_touched = int(diff.any(dim=1).sum())
    first_off = []
    for r in torch.nonzero(diff.any(dim=1)).flatten().tolist():
        j = int(torch.nonzero(diff[r]).flatten()[0])
        first_off.append(abs(float(got[r, j] - ref[r, j])))
    return frac, rows_touched, first_off


POOL = {"n": 0, "bad": 0}


@pytest.mark.parametrize("case", cases.PLUS_CASES, ids=lambda c: c[0])
def test_gptqplus_fasterquant_vs_reference(golden, case):
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    (name, rows, cols, nseq, seqlen, G, bits, gs, act, static, alpha, ref_loss, mode, atomic) = case
    g = golden("gptq_plus.npz")
    W = cases.make_weight(rows, cols, seed=31)
    X = cases.make_acts(nseq, seqlen, cols, seed=31)
    if "ragged" in name:
        X[..., 5] = 0.0
    S = cases.make_saliency(nseq, seqlen, G, seed=31)
    Gr = cases.make_grad(rows, cols, seed=31)
    layer = _layer(W)
    obj = GPTQPlus(layer, S, Gr, G, alpha, ref_loss)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(bits, perchannel=True, sym=True, mse=False)
    obj.add_batch(X[:1].to(DEV), None)
    obj.add_batch(X[1:].to(DEV), None)
    obj.finalize_hessian()
    H_dev, act_sq_dev = obj.H.clone().cpu(), obj.act_square.clone().cpu()
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    fi.KEEP_INTERMEDIATES = True
    seen = []
    try:
        obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static,
                        enable_gradient_update=True, g_update_mode=mode, export_to_et=True,
                        block_atomic_quant=atomic, block_observer=seen.append,
                        gradient_refresh_fn=cases.make_refresh_fn(W, Gr) if mode == "block_backward" else None)
    finally:
        fi.KEEP_INTERMEDIATES = False
    st = obj._last_fasterquant
    if act:
        assert torch.equal(st["perm"].cpu(), torch.from_numpy(g[f"{name}.perm"]))
    if f"{name}.Hinv0" in g:
        assert rel_fro(st["Hinv"][0, :cols, :cols], torch.from_numpy(g[f"{name}.Hinv0"])) < 5e-4
    rg = rows // G
    if mode == "block_backward":
        assert [b["col_end"] for b in seen] == list(range(128, cols + 1, 128))
        assert all(b["mean_refresh_loss"] is not None for b in seen)
    elif alpha > 0:
        assert torch.allclose(st["beta"][:rg].cpu(), torch.from_numpy(g[f"{name}.beta0"]), rtol=1e-3, atol=1e-6)
        assert rel_fro(st["Z"][:rg], torch.from_numpy(g[f"{name}.Z0"])) < 1e-3
        assert rel_fro(st["GHinv_initial"][:rg], torch.from_numpy(g[f"{name}.GHinv0"])) < 1e-3
    scale_ref = torch.from_numpy(g[f"{name}.Scale"])
    dynamic = gs != -1 and not static
    codes_ref = torch.from_numpy(g[f"{name}.W_int"]).float()
    order = st["perm"].cpu() if act else None
    frac, rows_touched, first_off = _code_report(layer.int_weight.cpu(), codes_ref, order)
    print(f"{name}: {frac * 100:.4f}% codes differ in {rows_touched} rows; first deviations {first_off[:8]}")
    POOL["n"] += codes_ref.numel()
    POOL["bad"] += int(frac * codes_ref.numel() + 0.5)
    assert all(d == 1.0 for d in first_off), "a row's first deviation must be a one-step rounding tie"
    assert frac < 0.01
    # rows without a flipped tie carry the reference's scales and weights (dynamic groups range later blocks
    # from the row's own earlier results, so a flipped tie moves that row's later scales)
    same = (layer.int_weight.cpu() == codes_ref).all(dim=1)
    assert int(same.sum()) >= rows - rows_touched
    assert torch.allclose(layer.scale.cpu()[same], scale_ref[same], rtol=1e-4 if dynamic else 1e-6, atol=0)
    assert torch.allclose(layer.weight.data.cpu()[same], torch.from_numpy(g[f"{name}.Q"])[same],
                          rtol=1e-4 if dynamic else 1e-6, atol=0)
    if not dynamic:
        assert torch.allclose(layer.scale.cpu(), scale_ref, rtol=1e-6, atol=0)
    assert layer.weight.dtype == torch.float32
    # the block loop in isolation: the oracle run on the Hessian the device accumulated (which differs from
    # the CPU's in the last bits) must reproduce the device's codes
    from oracle import gptq as og, quantizer as oq
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=True)
    o = og.plus_fasterquant(W, H_dev, act_sq_dev, Gr, q, G, alpha, ref_loss, groupsize=gs, actorder=act,
                            static_groups=static, g_update_mode=mode, block_atomic_quant=atomic,
                            gradient_refresh_fn=cases.make_refresh_fn(W, Gr) if mode == "block_backward" else None)
    frac2, _, first2 = _code_report(layer.int_weight.cpu(), o["W_int"].float(), order)
    print(f"{name}: against the oracle on the device's Hessian {frac2 * 100:.4f}% differ")
    assert frac2 < 0.01 and all(d == 1.0 for d in first2)      # the inverse factors differ at the 1e-5 level


@pytest.mark.parametrize("case", cases.GD_CASES, ids=lambda c: c[0])
def test_gptqplus_block_gd_vs_reference(golden, case):
    """g_update_mode="block_gd": kernels per block, optimizer steps between them.  Against the reference's run
    (rounding ties may flip where the device's Hessian differs in the last bits) and, exactly that isolated, against
    the oracle fed the device's own Hessian."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    from oracle import gptq as og, quantizer as oq
    (name, rows, cols, nseq, seqlen, G, gs, act, static, alpha, ref_loss, atomic, gd) = case
    g = golden("block_gd.npz")
    W = cases.make_weight(rows, cols, seed=37)
    X = cases.make_acts(nseq, seqlen, cols, seed=37)
    S = cases.make_saliency(nseq, seqlen, G, seed=37)
    Gr = cases.make_grad(rows, cols, seed=37)
    layer = _layer(W)
    obj = GPTQPlus(layer, S, Gr, G, alpha, ref_loss)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True, mse=False)
    obj.add_batch(X.to(DEV), None)
    obj.finalize_hessian()
    H_dev, act_sq_dev = obj.H.clone().cpu(), obj.act_square.clone().cpu()
    seen = []
    obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static,
                    enable_gradient_update=True, g_update_mode="block_gd", export_to_et=True,
                    block_atomic_quant=atomic, gradient_refresh_fn=cases.make_refresh_fn(W, Gr),
                    block_observer=seen.append, refresh_full_metrics=True, **gd)
    assert len(seen) == int(g[f"{name}.n_reports"])
    assert np.allclose([r["mean_refresh_loss"] for r in seen], g[f"{name}.refresh_loss"], rtol=2e-2)
    assert all(r["first_order_update_abs_mean"] is not None and r["second_order_update_abs_q99"] is not None
               for r in seen)
    order = obj._last_fasterquant["perm"].cpu() if act else None
    codes_ref = torch.from_numpy(g[f"{name}.W_int"]).float()
    frac, rows_touched, first_off = _code_report(layer.int_weight.cpu(), codes_ref, order)
    print(f"{name}: {frac * 100:.4f}% codes differ from the reference in {rows_touched} rows")
    assert frac < 0.02 and all(d == 1.0 for d in first_off)
    assert torch.allclose(layer.scale.cpu(), torch.from_numpy(g[f"{name}.Scale"]), rtol=1e-6, atol=0)
    q = oq.OracleWeightQuantizer()
    q.configure(4, perchannel=True, sym=True)
    o = og.plus_fasterquant(W, H_dev, act_sq_dev, Gr, q, G, alpha, ref_loss, groupsize=gs, actorder=act,
                            static_groups=static, g_update_mode="block_gd", block_atomic_quant=atomic,
                            gradient_refresh_fn=cases.make_refresh_fn(W, Gr), gd=gd)
    frac2, _, first2 = _code_report(layer.int_weight.cpu(), o["W_int"].float(), order)
    print(f"{name}: against the oracle on the device's Hessian {frac2 * 100:.4f}% differ")
    assert frac2 < 0.01 and all(d == 1.0 for d in first2)


def test_block_gd_argument_checks():
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    W = cases.make_weight(16, 256, seed=1)
    layer = _layer(W)
    obj = GPTQPlus(layer, torch.ones(1, 32, 1), torch.zeros(16, 256), 1, 0.0, 0.0)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True, mse=False)
    obj.add_batch(cases.make_acts(1, 32, 256, seed=1).to(DEV), None)
    obj.finalize_hessian()
    for bad in (dict(grad_optimizer="lion"), dict(grad_reg_strategy="l1"), dict(grad_gate_floor=1.5),
                dict(grad_reg_lambda=-1.0)):
        with pytest.raises(ValueError):
            obj.fasterquant(g_update_mode="block_gd", gradient_refresh_fn=cases.make_refresh_fn(W, W * 0), **bad)
    with pytest.raises(ValueError):                         # the refresh function is mandatory
        obj.fasterquant(g_update_mode="block_gd")


@pytest.mark.parametrize("case", cases.PLAIN_CASES, ids=lambda c: c[0])
def test_plain_gptq_fasterquant_vs_reference(golden, case):
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_utils import GPTQ
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    (name, rows, cols, nseq, seqlen, bits, sym, gs, act, static, bs) = case
    g = golden("plain_gptq.npz")
    W = cases.make_weight(rows, cols, seed=21)
    X = cases.make_acts(nseq, seqlen, cols, seed=21)
    if "ragged" in name:
        X[..., 7] = 0.0
    layer = _layer(W)
    obj = GPTQ(layer)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(bits, perchannel=True, sym=sym, mse="mse" in name)
    for s in range(nseq):
        obj.add_batch(X[s:s + 1].to(DEV), None)
    obj.fasterquant(blocksize=bs, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static, export_to_et=True)
    codes_ref = torch.from_numpy(g[f"{name}.W_int"]).float()
    frac, rows_touched, first_off = _code_report(layer.int_weight.cpu(), codes_ref)
    print(f"{name}: {frac * 100:.4f}% codes differ in {rows_touched} rows; first deviations {first_off[:8]}")
    POOL["n"] += codes_ref.numel()
    POOL["bad"] += int(frac * codes_ref.numel() + 0.5)
    assert all(d == 1.0 for d in first_off)
    assert frac < 0.01
    dynamic = gs != -1 and not static
    # rows without a flipped tie carry the reference's scales (a flip moves the ranges of that row's later dynamic groups)
    same = (layer.int_weight.cpu() == codes_ref).all(dim=1)
    assert same.float().mean() > 0.8
    assert torch.allclose(layer.scale.cpu()[same], torch.from_numpy(g[f"{name}.Scale"])[same],
                          rtol=1e-4 if dynamic else 1e-6, atol=0)
    if frac == 0.0:
        assert torch.allclose(layer.weight.data.cpu(), torch.from_numpy(g[f"{name}.Q"]),
                              rtol=1e-4 if dynamic else 1e-6, atol=0)
    assert not hasattr(obj, "_H") or obj._H is None                 # H is consumed like in the reference


def test_pooled_code_agreement():
    """Over all golden cases together at least 99.9 % of the integer codes equal the reference's."""
    assert POOL["n"] > 100000 - 1
    print(f"pooled: {POOL['bad']} of {POOL['n']} codes differ")
    assert POOL["bad"] / POOL["n"] < 1e-3


def test_mid_size_vs_oracle_bf16_weights():
    """A 512 x 1024 linear with bf16 weights, G = 4, alpha > 0, 8192 calibration tokens (8 per input
    channel, the regime of the benchmark configurations): kernels against the CPU oracle.  With far
    fewer tokens per channel the rounding decisions become so sensitive that the reference disagrees
    with itself at this level when its Hessian is merely accumulated in fp64."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rows, cols, G, nseq, seqlen = 512, 1024, 4, 4, 2048
    W = cases.make_weight(rows, cols, seed=41).bfloat16()
    X = cases.make_acts(nseq, seqlen, cols, seed=41)
    S = cases.make_saliency(nseq, seqlen, G, seed=41)
    Gr = cases.make_grad(rows, cols, seed=41)
    acc = ohess.GroupedHessian(cols, S)
    acc.add_batch(X)
    acc.finalize()
    q = oq.OracleWeightQuantizer()
    q.configure(4, perchannel=True, sym=True)
    ref = ogptq.plus_fasterquant(W.float(), acc.H, acc.act_square, Gr, q, G, 0.25, 0.7, actorder=True,
                                 static_groups=True)
    layer = _layer(W, torch.bfloat16)
    obj = GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True)
    obj.add_batch(X.to(DEV), None)
    obj.finalize_hessian()
    obj.fasterquant(actorder=True, static_groups=True, export_to_et=True)
    assert layer.weight.dtype == torch.bfloat16
    frac, rows_touched, first_off = _code_report(layer.int_weight.cpu(), ref["W_int"])
    print(f"mid-size: {frac * 100:.4f}% codes differ in {rows_touched} rows; first deviations {first_off[:8]}")
    assert frac < 1e-3
    assert all(d == 1.0 for d in first_off)
    assert torch.allclose(layer.scale.cpu(), ref["Scale"], rtol=1e-6, atol=0)


@pytest.mark.parametrize("bs,mse", [(256, False), (128, True)])
def test_gptqplus_dynamic_groups_ranged_by_the_host(bs, mse):
    """GPTQ+ with dynamic weight groups the block kernel cannot range itself (groupsize = blocksize = 256, or the
    shrink-grid search): the host ranges every group between two block launches (gptq_plus_utils.py:1205-1209).
    Checked against the CPU oracle on the Hessian the device accumulated."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rows, cols, G, nseq, seqlen = 32, 512, 2, 4, 1024
    W = cases.make_weight(rows, cols, seed=43)
    X = cases.make_acts(nseq, seqlen, cols, seed=43)
    S = cases.make_saliency(nseq, seqlen, G, seed=43)
    Gr = cases.make_grad(rows, cols, seed=43)
    layer = _layer(W)
    obj = GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True, mse=mse)
    obj.add_batch(X.to(DEV), None)
    obj.finalize_hessian()
    H_dev, act_dev = obj.H.cpu().clone(), obj.act_square.cpu().clone()
    obj.fasterquant(blocksize=bs, groupsize=bs, actorder=True, static_groups=False, export_to_et=True)
    q = oq.OracleWeightQuantizer()
    q.configure(4, perchannel=True, sym=True, mse=mse)
    ref = ogptq.plus_fasterquant(W, H_dev, act_dev, Gr, q, G, 0.25, 0.7, blocksize=bs, groupsize=bs, actorder=True,
                                 static_groups=False)
    frac, rows_touched, first_off = _code_report(layer.int_weight.cpu(), ref["W_int"])
    print(f"host-ranged groups bs={bs} mse={mse}: {frac * 100:.4f}% codes differ in {rows_touched} rows")
    assert frac < 0.01 and all(d == 1.0 for d in first_off)
    same = (layer.int_weight.cpu() == ref["W_int"]).all(dim=1)
    assert same.float().mean() > 0.8
    assert torch.allclose(layer.scale.cpu()[same], ref["Scale"][same], rtol=1e-4, atol=0)
    assert torch.allclose(layer.weight.data.cpu()[same], ref["Q"][same], rtol=1e-4, atol=0)


@pytest.mark.parametrize("case", cases.PLUS_DYNAMIC_CASES, ids=lambda c: c[0])
def test_gptqplus_host_ranged_groups_vs_reference(golden, case):
    """The same modes end to end (device Hessian included) against the unmodified reference's output."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    (name, rows, cols, nseq, seqlen, G, bs, mse, act) = case
    g = golden("gptq_plus_dynamic.npz")
    W = cases.make_weight(rows, cols, seed=43)
    X = cases.make_acts(nseq, seqlen, cols, seed=43)
    S = cases.make_saliency(nseq, seqlen, G, seed=43)
    Gr = cases.make_grad(rows, cols, seed=43)
    layer = _layer(W)
    obj = GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True, mse=mse)
    obj.add_batch(X.to(DEV), None)
    obj.finalize_hessian()
    obj.fasterquant(blocksize=bs, percdamp=0.01, groupsize=bs, actorder=act, static_groups=False, export_to_et=True)
    codes_ref = torch.from_numpy(g[f"{name}.W_int"]).float()
    frac, rows_touched, first_off = _code_report(layer.int_weight.cpu(), codes_ref)
    print(f"{name}: {frac * 100:.4f}% codes differ in {rows_touched} rows; first deviations {first_off[:8]}")
    assert frac < 0.02
    same = (layer.int_weight.cpu() == codes_ref).all(dim=1)
    assert same.float().mean() >= 0.75
    assert torch.allclose(layer.scale.cpu()[same], torch.from_numpy(g[f"{name}.Scale"])[same], rtol=1e-4, atol=0)
    assert torch.allclose(layer.weight.data.cpu()[same], torch.from_numpy(g[f"{name}.Q"])[same], rtol=1e-4, atol=0)


def _compare_summaries(got, ref, path, rtol):
    """Nested dicts / lists of the diagnostics: same keys, ints and bools equal, floats within rtol."""
    if isinstance(ref, dict):
        assert isinstance(got, dict) and set(got) == set(ref), (path, sorted(got), sorted(ref))
        for k in ref:
            _compare_summaries(got[k], ref[k], f"{path}.{k}", rtol)
    elif isinstance(ref, list):
        assert len(got) == len(ref), path
        for i, (a, b) in enumerate(zip(got, ref)):
            _compare_summaries(a, b, f"{path}[{i}]", rtol)
    elif isinstance(ref, bool) or isinstance(ref, int) or ref is None or isinstance(ref, str):
        assert got == ref, (path, got, ref)
    else:
        assert abs(got - ref) <= rtol * max(abs(ref), 1e-12) + 1e-9, (path, got, ref)


@pytest.mark.parametrize("case", ["frozen_pc_act", "online_g128_static_act", "block_g128_dynamic"])
def test_ghinv_diagnostics_vs_reference(case):
    """GPTQPlus.summarize_ghinv / summarize_weight_delta / analyze_ghinv_dynamics against the summaries the
    unmodified reference returns for the same seeded inputs (tests/golden/analysis.json): statistics of row norms,
    so a relative tolerance of 1e-3 (the Hessian and its inverse factor come from this package's kernels)."""
    import json
    import os
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    with open(os.path.join(os.path.dirname(__file__), "golden", "analysis.json")) as f:
        ref = json.load(f)[case]
    gs, act, static, mode = {"frozen_pc_act": (-1, True, True, "frozen"),
                             "online_g128_static_act": (128, True, True, "surrogate_online"),
                             "block_g128_dynamic": (128, False, False, "surrogate_block")}[case]
    rows, cols, nseq, seqlen, G = 64, 256, 4, 96, 4
    W = cases.make_weight(rows, cols, seed=31)
    X = cases.make_acts(nseq, seqlen, cols, seed=31)
    X[..., 5] = 0.0
    S = cases.make_saliency(nseq, seqlen, G, seed=31)
    Gr = cases.make_grad(rows, cols, seed=31)
    other = cases.make_weight(rows, cols, seed=32).to(DEV)
    layer = _layer(W)
    obj = GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True, mse=False)
    obj.add_batch(X.to(DEV), None)
    obj.finalize_hessian()
    before = layer.weight.data.clone()
    got = {
        "summarize_ghinv": obj.summarize_ghinv(actorder=act, max_blocks=1),
        "summarize_ghinv_off": obj.summarize_ghinv(actorder=act, enable_gradient_update=False,
                                                   reference_loss_override=0.3),
        "summarize_weight_delta": obj.summarize_weight_delta(actorder=act, ref_weight_override=other, max_subgroups=3),
        "analyze_ghinv_dynamics": obj.analyze_ghinv_dynamics(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act,
                                                             static_groups=static, g_update_mode=mode),
    }
    assert torch.equal(layer.weight.data, before)                    # diagnostics write nothing back
    _compare_summaries(got, ref, case, 1e-3)
    cache = obj.analyze_ghinv_dynamics(groupsize=gs, actorder=act, static_groups=static, g_update_mode=mode,
                                       max_subgroups=1, max_blocks=1, return_tensors=True)["_tensor_cache"]
    assert len(cache) == 1 and cache[0]["final_raw_eff_ghinv"].shape == (rows // G, 128)


def test_unsupported_modes_are_loud():
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    W = cases.make_weight(8, 128, seed=1)
    layer = _layer(W)
    obj = GPTQPlus(layer, torch.ones(1, 16, 2), torch.zeros(8, 128), 2, 0.0, 0.0)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True)
    obj.add_batch(torch.randn(1, 16, 128, device=DEV), None)
    obj.finalize_hessian()
    with pytest.raises(NotImplementedError):                # the recorder's block tags follow the frozen update
        obj.fasterquant(diagnostic_recorder=object(), g_update_mode="surrogate_block")
    with pytest.raises(NotImplementedError):
        obj.fasterquant(g_update_mode="surrogate_block", blocksize=256)
    with pytest.raises(ValueError):
        obj.fasterquant(g_update_mode="no_such_mode")
    with pytest.raises(ValueError):
        obj.fasterquant(groupsize=64, static_groups=False)


class _Recorder:
    """The three calls the reference's tensor-dump recorder receives (gptq_utils/diagnostics.py)."""

    def __init__(self):
        self.module, self.sub, self.blocks = {}, {}, {}

    def save_module_level(self, tag, t):
        self.module[tag] = t

    def save_subgroup(self, g, tag, t):
        self.sub[(g, tag)] = t

    def save_block(self, g, b, tag, t):
        self.blocks[(g, b, tag)] = t


@pytest.mark.parametrize("gs,static", [(-1, True), (128, False)])
def test_diagnostic_recorder_dumps(gs, static):
    """With a recorder the block loop runs with the host between the launches and hands over the tensors the
    reference dumps (gptq_plus_utils.py:957-972, 1108-1121, 1215-1229, 1377-1387, 1526-1565, 1878-1881); they
    satisfy the identities of the algorithm and the result equals the one of the fused loop."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rows, cols, nseq, seqlen, G = 64, 384, 4, 96, 4
    W = cases.make_weight(rows, cols, seed=31)
    X = cases.make_acts(nseq, seqlen, cols, seed=31)
    S = cases.make_saliency(nseq, seqlen, G, seed=31)
    Gr = cases.make_grad(rows, cols, seed=31)
    results = []
    for rec in (None, _Recorder()):
        layer = _layer(W)
        obj = GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
        obj.quantizer = WeightQuantizer()
        obj.quantizer.configure(4, perchannel=True, sym=True, mse=False)
        for s in range(nseq):
            obj.add_batch(X[s:s + 1].to(DEV), None)
        obj.finalize_hessian()
        obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=static, static_groups=static,
                        export_to_et=True, diagnostic_recorder=rec)
        results.append((layer.weight.data.clone(), layer.int_weight.clone()))
    frac, _, first_off = _code_report(results[1][1].cpu(), results[0][1].cpu())
    assert frac < 5e-3 and all(d == 1.0 for d in first_off)
    for tag in ("original_weight_rotated", "quantizer_scale", "quantizer_maxq", "H_after_accumulate", "act_square",
                "gradients", "reference_loss", "saliencies", "alpha", "Q_final", "W_int_final", "Scale_final"):
        assert tag in rec.module, tag
    assert torch.equal(rec.module["Q_final"], results[1][0])
    assert torch.equal(rec.module["W_int_final"].reshape(rows, cols), results[1][1])
    assert torch.equal(rec.module["Scale_final"] * rec.module["W_int_final"], rec.module["Q_final"])
    rps, nblk = rows // G, cols // 128
    for g in range(G):
        sub = {t: v for (gg, t), v in rec.sub.items() if gg == g}
        for tag in ("W_sub_initial", "gradients_sub", "Hinv_init", "Hinv_upper_cholesky", "hessian_identity_fallback",
                    "beta", "Z_initial", "GHinv_initial", "row_slice"):
            assert tag in sub, tag
        assert sub["row_slice"].tolist() == [g * rps, (g + 1) * rps]
        U = sub["Hinv_upper_cholesky"]
        assert rel_fro(sub["Z_initial"] @ U, sub["GHinv_initial"]) < 1e-4        # GHinv = Z . Hinv (:577)
        for b in range(nblk):
            blk = {t: v for (gg, bb, t), v in rec.blocks.items() if gg == g and bb == b}
            count = 128
            assert blk["block_column_range"].tolist() == [b * 128, b * 128 + count]
            assert torch.equal(blk["Hinv1"], U[b * 128:(b + 1) * 128, b * 128:(b + 1) * 128])
            if b == 0:
                assert torch.equal(blk["W1_start"], sub["W_sub_initial"][:, :128])
                assert torch.equal(blk["GHinv1_at_block_start"], sub["GHinv_initial"][:, :128])
            assert torch.equal(blk["Z1"], sub["Z_initial"][:, b * 128:(b + 1) * 128])
            assert torch.equal(blk["Q1"], blk["Scale1"] * blk["W_int1"])
            # first column of the block: err = (w - q - GHinv) / d (:1340-1343)
            e0 = (blk["W1_start"][:, 0] - blk["Q1"][:, 0] - blk["GHinv1_at_block_start"][:, 0]) / blk["Hinv1"][0, 0]
            assert torch.allclose(blk["Err1"][:, 0], e0, rtol=1e-4, atol=1e-6 * float(e0.abs().max()))
            assert torch.equal(blk["G_Update"], blk["count_times_GHinv_rest"] - blk["einsum_Z1_D_Hinv_term"])
            assert torch.equal(blk["total_outer_update"], blk["second_order_update"] + blk["G_Update"])
            if b + 1 < nblk:
                moved = blk["W_trailing_start"] - blk["W_trailing_after_outer_update"]
                assert rel_fro(moved, blk["total_outer_update"]) < 1e-4
                nxt = {t: v for (gg, bb, t), v in rec.blocks.items() if gg == g and bb == b + 1}
                assert torch.equal(nxt["W1_start"], blk["W_trailing_after_outer_update"][:, :128])


def test_group_owners_quantize_only_owned_rows():
    """With per-group owners a rank quantizes just the rows of its groups, and those rows come out exactly
    as in the run over the whole linear (the groups are independent problems)."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rows, cols, nseq, seqlen, G = 64, 256, 4, 96, 4
    W = cases.make_weight(rows, cols, seed=31)
    X = cases.make_acts(nseq, seqlen, cols, seed=31)
    S = cases.make_saliency(nseq, seqlen, G, seed=31)
    Gr = cases.make_grad(rows, cols, seed=31)
    outs = []
    for owners in (None, [0, 1, 0, 0]):
        layer = _layer(W)
        obj = GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
        obj.quantizer = WeightQuantizer()
        obj.quantizer.configure(4, perchannel=True, sym=True, mse=False)
        obj.add_batch(X.to(DEV), None)
        obj.group_owners = owners
        obj.finalize_hessian()
        obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=128, actorder=True, static_groups=True,
                        export_to_et=True)
        outs.append((layer.weight.data.cpu(), layer.int_weight.cpu(), layer.scale.cpu()))
    rps = rows // G
    (qa, ca, sa), (qb, cb, sb) = outs
    for g in (0, 2, 3):
        r = slice(g * rps, (g + 1) * rps)
        assert torch.equal(qa[r], qb[r]) and torch.equal(ca[r], cb[r]) and torch.equal(sa[r], sb[r])
    r = slice(rps, 2 * rps)
    assert torch.equal(qb[r], W[r]) and not torch.equal(qa[r], W[r])


@pytest.mark.parametrize("cols", [640, 896])
def test_two_level_schedule_with_ragged_last_group(cols):
    """Column counts that leave a partial group of blocks at the end (640 = 512 + 128, 896 = 512 + 384): the
    two-level tensor-core schedule, the one-level CUDA-core schedule and the oracle run on the device's Hessian
    must agree on the codes (up to isolated rounding ties)."""
    from gptq_plus_mp_quant_b200.gptq_utils import fasterquant_impl as fi
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rows, G, nseq, seqlen = 64, 2, 4, 2048
    W = cases.make_weight(rows, cols, seed=51)
    X = cases.make_acts(nseq, seqlen, cols, seed=51)
    S = cases.make_saliency(nseq, seqlen, G, seed=51)
    Gr = cases.make_grad(rows, cols, seed=51)
    got = {}
    H_dev = act_dev = perm = None
    for tensor_cores in (True, False):
        layer = _layer(W)
        obj = GPTQPlus(layer, S, Gr, G, 0.25, 0.7)
        obj.quantizer = WeightQuantizer()
        obj.quantizer.configure(4, perchannel=True, sym=True)
        obj.add_batch(X.to(DEV), None)
        obj.finalize_hessian()
        H_dev, act_dev = obj.H.clone().cpu(), obj.act_square.clone().cpu()
        old = fi.USE_TENSOR_CORES
        fi.USE_TENSOR_CORES = tensor_cores
        try:
            obj.fasterquant(actorder=True, static_groups=True, groupsize=128, export_to_et=True)
        finally:
            fi.USE_TENSOR_CORES = old
        perm = obj._last_fasterquant["perm"].cpu()
        got[tensor_cores] = layer.int_weight.cpu()
    q = oq.OracleWeightQuantizer()
    q.configure(4, perchannel=True, sym=True)
    ref = ogptq.plus_fasterquant(W, H_dev, act_dev, Gr, q, G, 0.25, 0.7, groupsize=128, actorder=True,
                                 static_groups=True)["W_int"].float()
    for name, codes in (("two-level tensor-core", got[True]), ("one-level CUDA-core", got[False])):
        frac, touched, first = _code_report(codes, ref, perm)
        print(f"C={cols} {name}: {frac * 100:.4f}% codes differ in {touched} rows")
        assert frac < 5e-3 and all(d == 1.0 for d in first)


@pytest.mark.parametrize("case", cases.GUIDED_CASES, ids=lambda c: c[0])
def test_gptq_guided_vs_reference(golden, case):
    """GPTQGuided on the device against the reference's outputs, and its block loop against the oracle run on the
    Hessian the device accumulated."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_guided_utils import GPTQGuided
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    (name, rows, cols, nseq, seqlen, G, bits, gs, act, static) = case
    g = golden("guided.npz")
    W = cases.make_weight(rows, cols, seed=61)
    X = cases.make_acts(nseq, seqlen, cols, seed=61)
    S = cases.make_saliency(nseq, seqlen, G, seed=61)
    layer = _layer(W)
    obj = GPTQGuided(layer, S, G)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(bits, perchannel=True, sym=True, mse=False)
    obj.add_batch(X[:1].to(DEV), None)
    obj.add_batch(X[1:].to(DEV), None)
    assert obj.H.shape == (cols, cols, G)
    assert torch.allclose(obj.act_square.cpu(), torch.from_numpy(g[f"{name}.act_square"]), rtol=1e-5)
    assert torch.allclose(torch.einsum("iig->g", obj.H).cpu(), torch.from_numpy(g[f"{name}.H_trace"]), rtol=1e-5)
    H_dev, act_dev = obj.H.clone().cpu(), obj.act_square.clone().cpu()
    obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static, export_to_et=True)
    order = obj._last_fasterquant["perm"].cpu() if act else None
    codes_ref = torch.from_numpy(g[f"{name}.W_int"]).float()
    frac, touched, first = _code_report(layer.int_weight.cpu(), codes_ref, order)
    print(f"{name}: {frac * 100:.4f}% codes differ in {touched} rows")
    assert frac < 0.01 and all(d == 1.0 for d in first)
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=True)
    o = ogptq.guided_fasterquant(W, H_dev, act_dev, q, G, groupsize=gs, actorder=act, static_groups=static)
    frac2, _, first2 = _code_report(layer.int_weight.cpu(), o["W_int"].float(), order)
    print(f"{name}: against the oracle on the device's Hessian {frac2 * 100:.4f}% differ")
    assert frac2 < 0.01 and all(d == 1.0 for d in first2)
    obj.free()
    assert obj.H is None


@pytest.mark.parametrize("case", cases.GPTAQ_CASES, ids=lambda c: c[0])
def test_gptaq_vs_reference(golden, case):
    """GPTAQ on the device: dXXT against the reference's, quantized weights against the reference's and against
    the oracle run on the statistics the device accumulated."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptaq_utils import GPTAQ
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    (name, rows, cols, nseq, seqlen, bits, sym, gs, act, static, alpha) = case
    g = golden("gptaq.npz")
    W = cases.make_weight(rows, cols, seed=71)
    X = cases.make_acts(nseq, seqlen, cols, seed=71)
    Xfp = cases.make_fp_acts(X, seed=72)
    layer = _layer(W)
    obj = GPTAQ(layer)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(bits, perchannel=True, sym=sym, mse=False)
    for s_ in range(nseq):
        obj.fp_inp.append(Xfp[s_].t().contiguous())                # [C, tokens] on the CPU, as the reference queues it
        obj.add_batch(X[s_:s_ + 1].to(DEV), None)
    assert obj.fp_inp == []
    assert rel_fro(obj.dXXT, torch.from_numpy(g[f"{name}.dXXT"])) < 3e-5
    assert torch.allclose(torch.diag(obj.H).cpu(), torch.from_numpy(g[f"{name}.H_diag"]), rtol=1e-5)
    H_dev, d_dev = obj.H.clone().cpu(), obj.dXXT.clone().cpu()
    obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=gs, actorder=act, static_groups=static, alpha=alpha)
    got = layer.weight.data.cpu()
    ref = torch.from_numpy(g[f"{name}.Q"])
    # dynamic groups are ranged from the working weights, whose last bits follow the accumulation order: the scales,
    # and with them every dequantized value of the group, move in the last bits; a flipped code moves a whole step
    tol = 1e-4 * float(ref.abs().max()) if (gs != -1 and not static) else 0.0
    frac = float(((got - ref).abs() > tol).float().mean())
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=sym, mse=False)
    o = ogptq.gptaq_fasterquant(W, H_dev, d_dev, q, groupsize=gs, actorder=act, static_groups=static, alpha=alpha)
    frac2 = float(((got - o["Q"]).abs() > tol).float().mean())
    print(f"{name}: {frac * 100:.4f}% of the quantized weights differ from the reference, {frac2 * 100:.4f}% from the "
          "oracle on the device's statistics")
    assert frac < 0.02 and frac2 < 0.01
    # differing entries are one quantization step away in the row where the first tie flipped, never garbage
    assert float((got - ref).abs().max()) < 16 * float(ref.abs().max()) / (2 ** bits)


def test_w8_asymmetric_codes_beyond_int8():
    """8-bit asymmetric ranges have maxq = 255 (utils/quant_utils.py:309-331) and fake_quantize clamps to
    [-256, 255]: the kernels carry the integer codes in 16 bits.  Plain GPTQ, 64 x 256, against the oracle on the
    device's own Hessian."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_utils import GPTQ
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rows, cols, nseq, seqlen = 64, 256, 4, 512
    W = cases.make_weight(rows, cols, seed=61)
    X = cases.make_acts(nseq, seqlen, cols, seed=61)
    layer = _layer(W)
    obj = GPTQ(layer)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(8, perchannel=True, sym=False, mse=False)
    assert int(obj.quantizer.maxq) == 255
    for s in range(nseq):
        obj.add_batch(X[s:s + 1].to(DEV), None)
    H_dev = obj.H.clone().cpu()
    obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=-1, actorder=True, export_to_et=True)
    q = oq.OracleWeightQuantizer()
    q.configure(8, perchannel=True, sym=False)
    ref = ogptq.plain_fasterquant(W, H_dev, q, blocksize=128, percdamp=0.01, groupsize=-1, actorder=True)
    codes = layer.int_weight.cpu()
    assert float(codes.abs().max()) > 127.0                       # the case does leave the int8 range
    frac, rows_touched, first_off = _code_report(codes, ref["W_int"])
    print(f"W8 asymmetric: {frac * 100:.4f}% codes differ in {rows_touched} rows")
    assert frac < 5e-3 and all(d == 1.0 for d in first_off)
    assert torch.allclose(layer.scale.cpu(), ref["Scale"], rtol=1e-6, atol=0)
