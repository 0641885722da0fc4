"""The CPU oracle against outputs of the unmodified reference (tests/golden/*.npz,
made by tests/golden/make_golden.py).  The oracle uses the same ATen CPU operations in
the same order as the reference, so integer codes must be identical and floating-point
results equal to within a few ulps (tolerances stated per check)."""
import numpy as np
import pytest
import torch

import cases
from oracle import gptq as ogptq
from oracle import hadamard as ohad
from oracle import hessian as ohess
from oracle import quantizer as oq

torch.set_num_threads(1)


def t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("case", cases.QUANTIZER_CASES, ids=lambda c: c[0])
def test_quantizer(golden, case):
    name, rows, cols, bits, pc, sym, mse = case
    g = golden("quantizer.npz")
    W = cases.make_weight(rows, cols, seed=11)
    assert cases.digest(W) == str(g[f"{name}.digest"]), "input generator drifted"
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=pc, sym=sym, mse=mse)
    q.find_params(W)
    assert int(q.maxq) == int(g[f"{name}.maxq"])
    assert torch.equal(q.scale, t(g[f"{name}.scale"]))          # bit-exact: same ops, same order
    assert torch.equal(q.zero, t(g[f"{name}.zero"]))
    deq, codes, _ = q.fake_quantize(W)
    assert torch.equal(codes, t(g[f"{name}.fake_codes"]))
    assert torch.equal(deq, t(g[f"{name}.fake_deq"]))
    assert torch.equal(q.quantize(W), t(g[f"{name}.ste"]))


@pytest.mark.parametrize("case", cases.HADAMARD_CASES, ids=lambda c: c[0])
def test_hadamard(golden, case):
    name, rows, n, dtype = case
    g = golden("hadamard.npz")
    dt = getattr(torch, dtype)
    x = cases.make_acts(1, rows, n, seed=5).reshape(rows, n).to(dt)
    assert cases.digest(x) == str(g[f"{name}.digest"])
    K = ohad.pick_K(n, [int(k) for k in g["table_keys"]])
    assert K == int(g[f"{name}.K"])
    hadK = t(g[f"had{K}"]).float() if K > 1 else None
    y = ohad.rotate(x, hadK, K)
    assert torch.equal(y.float(), t(g[f"{name}.y"]))            # bit-exact restatement
    ys = ohad.rotate_strided(x, hadK, K)
    assert torch.equal(ys.float(), t(g[f"{name}.y_strided"]))
    # the fp64 evaluation is the exact operator: both reference forms sit within their dtype's rounding of it
    exact = ohad.rotate_exact(x, hadK, K)
    tol = {"float32": 2e-6, "bfloat16": 3e-2, "float16": 4e-3}[dtype]
    scale = exact.abs().max()
    assert (y.double() - exact).abs().max() <= tol * scale


def _plain_setup(case):
    (name, rows, cols, nseq, seqlen, bits, sym, gs, act, static, bs) = case
    W = cases.make_weight(rows, cols, seed=21)
    X = cases.make_acts(nseq, seqlen, cols, seed=21)
    if "ragged" in name:
        X[..., 7] = 0.0
    return W, X


@pytest.mark.parametrize("case", cases.PLAIN_CASES, ids=lambda c: c[0])
def test_plain_gptq(golden, case):
    (name, rows, cols, nseq, seqlen, bits, sym, gs, act, static, bs) = case
    g = golden("plain_gptq.npz")
    W, X = _plain_setup(case)
    assert cases.digest(W, X) == str(g[f"{name}.digest"])
    acc = ohess.PlainHessian(cols)
    for s in range(nseq):
        acc.add_batch(X[s:s + 1])
    if f"{name}.H" in g:
        assert torch.equal(acc.H, t(g[f"{name}.H"]))
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=sym, mse="mse" in name)
    out = ogptq.plain_fasterquant(W, acc.H, q, blocksize=bs, percdamp=0.01, groupsize=gs, actorder=act,
                                  static_groups=static)
    assert torch.equal(out["W_int"], t(g[f"{name}.W_int"]).float())
    assert torch.equal(out["Scale"], t(g[f"{name}.Scale"]))
    assert torch.equal(out["Q"], t(g[f"{name}.Q"]))


def _plus_setup(case):
    (name, rows, cols, nseq, seqlen, G, bits, gs, act, static, alpha, ref_loss, mode, atomic) = case
    W = cases.make_weight(rows, cols, seed=31)
    X = cases.make_acts(nseq, seqlen, cols, seed=31)
    if "ragged" in name:
        X[..., 5] = 0.0
    S = cases.make_saliency(nseq, seqlen, G, seed=31)
    Gr = cases.make_grad(rows, cols, seed=31)
    return W, X, S, Gr


@pytest.mark.parametrize("case", cases.PLUS_CASES, ids=lambda c: c[0])
def test_gptq_plus(golden, case):
    (name, rows, cols, nseq, seqlen, G, bits, gs, act, static, alpha, ref_loss, mode, atomic) = case
    g = golden("gptq_plus.npz")
    W, X, S, Gr = _plus_setup(case)
    assert cases.digest(W, X, S, Gr) == str(g[f"{name}.digest"])
    acc = ohess.GroupedHessian(cols, S)
    acc.add_batch(X[:1])
    acc.add_batch(X[1:])
    assert torch.equal(acc.act_square, t(g[f"{name}.act_sum"]))
    acc.finalize()
    if f"{name}.H" in g:
        assert torch.equal(acc.H, t(g[f"{name}.H"]))
    assert torch.equal(acc.act_square, t(g[f"{name}.act_square"]))
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=True, mse=False)
    out = ogptq.plus_fasterquant(W, acc.H, acc.act_square, Gr, q, G, alpha, ref_loss, blocksize=128,
                                 percdamp=0.01, groupsize=gs, actorder=act, static_groups=static,
                                 g_update_mode=mode, block_atomic_quant=atomic,
                                 gradient_refresh_fn=cases.make_refresh_fn(W, Gr) if mode == "block_backward" else None)
    st0 = out["states"][0]
    if act:
        assert torch.equal(out["perm"], t(g[f"{name}.perm"]))
    if f"{name}.Hinv0" in g:
        assert torch.equal(st0["Hinv"], t(g[f"{name}.Hinv0"]))
    assert torch.equal(torch.diagonal(st0["Hinv_init"]), t(g[f"{name}.Hinv_init0_diag"]))
    if mode != "block_backward":                                 # that mode replaces the terms after every block
        assert torch.equal(st0["beta"], t(g[f"{name}.beta0"]))
        assert torch.equal(st0["Z"], t(g[f"{name}.Z0"]))
    assert torch.equal(out["W_int"], t(g[f"{name}.W_int"]).float())
    assert torch.equal(out["Scale"], t(g[f"{name}.Scale"]))
    assert torch.equal(out["Q"], t(g[f"{name}.Q"]))


@pytest.mark.parametrize("case", cases.PLUS_DYNAMIC_CASES, ids=lambda c: c[0])
def test_gptq_plus_dynamic_groups(golden, case):
    """GPTQ+ with dynamic weight groups as wide as a 256-column block, and with the shrink-grid search."""
    (name, rows, cols, nseq, seqlen, G, bs, mse, act) = case
    g = golden("gptq_plus_dynamic.npz")
    W = cases.make_weight(rows, cols, seed=43)
    X = cases.make_acts(nseq, seqlen, cols, seed=43)
    S = cases.make_saliency(nseq, seqlen, G, seed=43)
    Gr = cases.make_grad(rows, cols, seed=43)
    assert cases.digest(W, X, S, Gr) == str(g[f"{name}.digest"])
    acc = ohess.GroupedHessian(cols, S)
    acc.add_batch(X)
    acc.finalize()
    q = oq.OracleWeightQuantizer()
    q.configure(4, perchannel=True, sym=True, mse=mse)
    out = ogptq.plus_fasterquant(W, acc.H, acc.act_square, Gr, q, G, 0.25, 0.7, blocksize=bs, percdamp=0.01,
                                 groupsize=bs, actorder=act, static_groups=False)
    assert torch.equal(out["W_int"], t(g[f"{name}.W_int"]).float())
    assert torch.equal(out["Scale"], t(g[f"{name}.Scale"]))
    assert torch.equal(out["Q"], t(g[f"{name}.Q"]))


@pytest.mark.parametrize("case", cases.GD_CASES, ids=lambda c: c[0])
def test_gptq_plus_block_gd(golden, case):
    """g_update_mode="block_gd" (optimizer steps on the trailing weights between blocks, every regulariser and
    optimizer of the reference) against the reference's own run with the same deterministic refresh function."""
    (name, rows, cols, nseq, seqlen, G, gs, act, static, alpha, ref_loss, atomic, gd) = case
    g = golden("block_gd.npz")
    W = cases.make_weight(rows, cols, seed=37)
    X = cases.make_acts(nseq, seqlen, cols, seed=37)
    S = cases.make_saliency(nseq, seqlen, G, seed=37)
    Gr = cases.make_grad(rows, cols, seed=37)
    assert cases.digest(W, X, S, Gr) == str(g[f"{name}.digest"])
    acc = ohess.GroupedHessian(cols, S)
    acc.add_batch(X)
    acc.finalize()
    q = oq.OracleWeightQuantizer()
    q.configure(4, perchannel=True, sym=True, mse=False)
    out = ogptq.plus_fasterquant(W, acc.H, acc.act_square, Gr, q, G, alpha, ref_loss, blocksize=128, percdamp=0.01,
                                 groupsize=gs, actorder=act, static_groups=static, g_update_mode="block_gd",
                                 block_atomic_quant=atomic, gradient_refresh_fn=cases.make_refresh_fn(W, Gr), gd=gd)
    assert torch.equal(out["W_int"], t(g[f"{name}.W_int"]).float())
    assert torch.equal(out["Scale"], t(g[f"{name}.Scale"]))
    assert torch.equal(out["Q"], t(g[f"{name}.Q"]))
    # the optimizer steps matter: without them other codes come out
    plain = ogptq.plus_fasterquant(W, acc.H, acc.act_square, Gr, q, G, alpha, ref_loss, blocksize=128, percdamp=0.01,
                                   groupsize=gs, actorder=act, static_groups=static, g_update_mode="frozen",
                                   block_atomic_quant=atomic)
    assert int((plain["W_int"] != out["W_int"]).sum()) > 0


def test_sharded_accumulation_matches_single(golden):
    """Token-sharded accumulation followed by a sum of the partial state (what the all-reduce
    in finalize_hessian does) equals the single-process result to fp32 summation noise."""
    case = cases.PLUS_CASES[0]
    (name, rows, cols, nseq, seqlen, G, *_rest) = case
    W, X, S, Gr = _plus_setup(case)
    one = ohess.GroupedHessian(cols, S)
    one.add_batch(X)
    one.finalize()
    parts = []
    for r in range(2):
        sl = slice(r * nseq // 2, (r + 1) * nseq // 2)
        p = ohess.GroupedHessian(cols, S[sl])
        p.add_batch(X[sl])
        parts.append(p)
    merged = ohess.GroupedHessian.merge(parts)
    merged.finalize()
    rel = (merged.H - one.H).norm() / one.H.norm()
    assert rel < 1e-6                                            # relative Frobenius
    assert torch.allclose(merged.act_square, one.act_square, rtol=1e-5)


def test_nonspd_damping_retry(golden):
    g = golden("faults.npz")
    H = t(g["nonspd.H"])
    import logging
    logging.disable(logging.WARNING)
    inv, up, damp, ident = ogptq.hinv_with_fallback(H, 0.01)
    logging.disable(logging.NOTSET)
    assert ident == bool(g["nonspd.identity"])
    assert abs(damp - float(g["nonspd.damp"])) < 1e-12
    assert torch.equal(up, t(g["nonspd.Hinv"]))


def test_nonfinite_hessian_is_zeroed():
    S = torch.ones(1, 4, 1)
    acc = ohess.GroupedHessian(3, S)
    X = torch.tensor([[[1.0, 2.0, float("inf")], [0.5, 1.0, 1.0], [1.0, 0.0, 1.0], [2.0, 1.0, 1.0]]])
    acc.add_batch(X)
    n_nan, n_inf = acc.finalize()
    assert n_nan + n_inf > 0
    assert torch.isfinite(acc.H).all()
    with pytest.raises(RuntimeError):
        acc.add_batch(X)


def test_finalize_before_accumulate_raises():
    acc = ohess.GroupedHessian(3, torch.ones(1, 4, 1))
    with pytest.raises(RuntimeError):
        acc.finalize()


@pytest.mark.parametrize("case", cases.CLIP_CASES, ids=lambda c: c[0])
def test_clip_to_quant_bounds(golden, case):
    """clip_module_weight_to_quant_bounds_ (shrink-grid searched range, then the clamp), bit for bit."""
    name, rows, cols, bits, sym, dtype = case
    g = golden("clip.npz")
    W = cases.make_weight(rows, cols, seed=13).to(getattr(torch, dtype))
    assert cases.digest(W.float()) == str(g[f"{name}.digest"])
    out = oq.clip_weight_to_quant_bounds(W, bits, sym, True)
    assert out.dtype == W.dtype
    assert torch.equal(out.float(), t(g[f"{name}.clipped"]))
    assert int((out.float() != W.float()).sum()) == int(g[f"{name}.changed"]) > 0
    assert oq.clip_weight_to_quant_bounds(W, 16, sym, True) is W and oq.clip_weight_to_quant_bounds(W, bits, sym, False) is W


@pytest.mark.parametrize("case", cases.SALIENCY_CASES, ids=lambda c: c[0])
def test_saliency_hook(golden, case):
    """SaliencyCache's gradient hook (mean squared output gradient per channel group, sink positions dropped)."""
    name, batch, seq, hidden, G, sink, dtype = case
    g = golden("saliency.npz")
    coef = cases.make_out_grad(batch, seq, hidden, seed=17).to(getattr(torch, dtype))
    assert cases.digest(coef.float()) == str(g[f"{name}.digest"])
    sal = ohess.group_mean_square(coef, G, sink)
    assert sal.shape == (batch, seq - sink, G)
    assert torch.equal(sal, t(g[f"{name}.saliency"]))


@pytest.mark.parametrize("n,q", [(8192, 0.99), (100, 0.5), (4097, 0.999), (2, 0.3), (1, 0.99), (65536, 0.01)])
def test_saliency_percentile_clip_is_torch_quantile(n, q):
    """The oracle's restatement of the hook's outlier clip against the library call the reference makes
    (torch.quantile + clamp, gptq_plus_utils.py:2834-2839), on log-normal saliencies with ties."""
    s = cases.make_saliency(1, n, 1, seed=n).flatten()
    s[: n // 7] = s[0]                                              # ties
    ref_cap = torch.quantile(s, q)
    out, cap = ohess.clip_at_percentile(s, q)
    assert torch.equal(cap, ref_cap)
    assert torch.equal(out, torch.clamp(s, max=ref_cap))
    bad = s.clone()
    bad[n // 2] = float("nan")
    _, cap = ohess.clip_at_percentile(bad, q)
    assert torch.isnan(cap) and torch.isnan(torch.quantile(bad, q))


@pytest.mark.parametrize("case", cases.ACT_QUANT_CASES, ids=lambda c: c[0])
def test_act_quantizer(golden, case):
    """ActQuantizer: dynamic per-token / per-token-group ranges and the fake quantization, in the tensor's dtype."""
    name, shape, bits, gs, sym, clip, dtype = case
    g = golden("act_quant.npz")
    x = cases.make_act_tensor(shape, seed=23).to(getattr(torch, dtype))
    assert cases.digest(x.float()) == str(g[f"{name}.digest"])
    scale, zero, maxq = oq.act_find_params(x, bits, gs, sym, clip)
    assert torch.equal(scale.float(), t(g[f"{name}.scale"])) and torch.equal(zero.float(), t(g[f"{name}.zero"]))
    y = oq.act_fake_quant(x, bits, gs, sym, clip)
    assert y.dtype == x.dtype and torch.equal(y.float(), t(g[f"{name}.deq"]))


@pytest.mark.parametrize("case", cases.GUIDED_CASES, ids=lambda c: c[0])
def test_gptq_guided(golden, case):
    """GPTQGuided (GuidedQuant): raw-sum grouped Hessians, the block loop without first-order terms."""
    (name, rows, cols, nseq, seqlen, G, bits, gs, act, static) = case
    g = golden("guided.npz")
    W = cases.make_weight(rows, cols, seed=61)
    X = cases.make_acts(nseq, seqlen, cols, seed=61)
    S = cases.make_saliency(nseq, seqlen, G, seed=61)
    assert cases.digest(W, X, S) == str(g[f"{name}.digest"])
    H = torch.zeros(cols, cols, G)
    act_sq = torch.zeros(cols)
    for sl in (slice(0, 1), slice(1, nseq)):
        inp = X[sl].reshape(-1, cols).float()
        sal = S[sl].reshape(-1, G).float()
        H.add_(torch.einsum("ni,njg->ijg", inp, torch.einsum("nj,ng->njg", inp, sal)))
        act_sq.add_((inp ** 2).sum(0), alpha=1 / inp.shape[0])
    assert torch.equal(act_sq, t(g[f"{name}.act_square"]))
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=True, mse=False)
    out = ogptq.guided_fasterquant(W, H, act_sq, q, G, groupsize=gs, actorder=act, static_groups=static)
    assert torch.equal(out["W_int"], t(g[f"{name}.W_int"]).float())
    assert torch.equal(out["Scale"], t(g[f"{name}.Scale"]))
    assert torch.equal(out["Q"], t(g[f"{name}.Q"]))


@pytest.mark.parametrize("case", cases.GPTAQ_CASES, ids=lambda c: c[0])
def test_gptaq(golden, case):
    """GPTAQ: H / dXXT accumulation from queued full-precision inputs and the block loop with the P term."""
    (name, rows, cols, nseq, seqlen, bits, sym, gs, act, static, alpha) = case
    g = golden("gptaq.npz")
    W = cases.make_weight(rows, cols, seed=71)
    X = cases.make_acts(nseq, seqlen, cols, seed=71)
    Xfp = cases.make_fp_acts(X, seed=72)
    assert cases.digest(W, X, Xfp) == str(g[f"{name}.digest"])
    st = ogptq.AsymCalibState(cols)
    for s_ in range(nseq):
        st.add_batch(X[s_:s_ + 1], Xfp[s_].t().contiguous())
    assert torch.equal(st.dXXT, t(g[f"{name}.dXXT"]))
    assert torch.equal(torch.diag(st.H), t(g[f"{name}.H_diag"]))
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=sym, mse=False)
    out = ogptq.gptaq_fasterquant(W, st.H, st.dXXT, q, groupsize=gs, actorder=act, static_groups=static, alpha=alpha)
    assert torch.equal(out["Q"], t(g[f"{name}.Q"]))


@pytest.mark.parametrize("case", cases.QK_CASES, ids=lambda c: c[0])
def test_qk_rotation_wrapper(golden, case):
    """QKRotationWrapper: head-dim Hadamard of q and k, K-cache fake quantization per token or per head."""
    name, (b, h, kvh, t_, d), bits, gs, sym, clip, dtype = case
    g = golden("qk.npz")
    dt = getattr(torch, dtype)
    q = cases.make_act_tensor((b * h, t_, d), seed=41).reshape(b, h, t_, d).to(dt)
    k = cases.make_act_tensor((b * kvh, t_, d), seed=42).reshape(b, kvh, t_, d).to(dt)
    assert cases.digest(q.float(), k.float()) == str(g[f"{name}.digest"])
    qo, ko = ohad.qk_rotate_quant(q, k, bits, gs, sym, clip)
    assert torch.equal(qo.float(), t(g[f"{name}.q"])) and torch.equal(ko.float(), t(g[f"{name}.k"]))


@pytest.mark.parametrize("case", cases.WGROUP_MSE_CASES, ids=lambda c: c[0])
def test_weight_quantizer_grouped_mse(golden, case):
    """Grouped weight ranges with the shrink-grid search, in the weight's own dtype (an all-zero and a constant
    group included)."""
    name, rows, cols, bits, gs, sym, dtype = case
    g = golden("wgroup_mse.npz")
    W = cases.make_weight(rows, cols, seed=23).to(getattr(torch, dtype))
    W[0, :gs] = 0
    W[1, :gs] = 0.5
    assert cases.digest(W.float()) == str(g[f"{name}.digest"])
    scale, zero, maxq = oq.weight_groupwise_params(W, bits, gs, sym, mse=True)
    assert torch.equal(scale.float(), t(g[f"{name}.scale"])) and torch.equal(zero.float(), t(g[f"{name}.zero"]))
    ste = oq.ste_quantize(W, scale, zero, int(maxq), sym).to(W.dtype)
    assert torch.equal(ste.float(), t(g[f"{name}.ste"]))
    plain, _, _ = oq.weight_groupwise_params(W, bits, gs, sym)
    assert not torch.equal(plain, scale)                                # the search moved some ranges


@pytest.mark.parametrize("case", cases.WGROUP_CASES, ids=lambda c: c[0])
def test_weight_quantizer_grouped(golden, case):
    """WeightQuantizer with weight_groupsize > 0 (round-to-nearest path), evaluated in the weight's own dtype."""
    name, rows, cols, bits, gs, sym, dtype = case
    g = golden("wgroup.npz")
    W = cases.make_weight(rows, cols, seed=19).to(getattr(torch, dtype))
    W[0, :gs] = 0
    assert cases.digest(W.float()) == str(g[f"{name}.digest"])
    fake, codes, scale, zero, ste = oq.weight_groupwise_rtn(W, bits, gs, sym)
    assert torch.equal(scale.float(), t(g[f"{name}.scale"])) and torch.equal(zero.float(), t(g[f"{name}.zero"]))
    assert torch.equal(fake.float(), t(g[f"{name}.fake"])) and torch.equal(codes.float(), t(g[f"{name}.codes"]))
    assert torch.equal(ste.float(), t(g[f"{name}.ste"]))


def test_reference_copy_loads_when_present():
    """oracle/_ref (built by oracle/make_ref.py where the reference is mounted) holds the reference's own modules
    for the CPU arm of the benchmark; when it is there it must import and expose the classes the arm drives."""
    from oracle import ref_loader
    mods = ref_loader.load()
    if mods is None:
        pytest.skip("oracle/_ref has not been built on this machine")
    assert hasattr(mods["gptq_plus_utils"], "GPTQPlus") and hasattr(mods["gptq_utils"], "GPTQ")
    assert hasattr(mods["quant_utils"], "WeightQuantizer")
    assert hasattr(mods["gptq_plus_utils"].GPTQPlus, "_compute_hessian_inverse_with_fallback")
