"""Parity of the sm_100a kernels (through the C ABI) with the CPU oracle and with the golden
outputs of the reference: Hessian accumulation/finalisation, Hadamard rotation, weight
quantizer.  Tolerances: H <= 5e-6 relative Frobenius for sums over a few hundred tokens and
<= 2e-6 from a few thousand tokens on (the split-bf16 rounding terms average out with the
token count; bar: 1e-5), scale/zero <= 1e-6 relative
(bar: 1e-5), integer codes identical, rotation within one rounding of the I/O dtype."""
import math

import numpy as np
import pytest
import torch

import cases
from oracle import hadamard as ohad
from oracle import hessian as ohess
from oracle import quantizer as oq

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def rel_fro(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm())


# ---------------------------------------------------------------------------- Hessian
def _oracle_grouped(X, S):
    acc = ohess.GroupedHessian(X.shape[-1], S)
    acc.add_batch(X)
    return acc


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("C,G,nseq,seqlen,dtype", [
    (128, 1, 1, 64, torch.float32),
    (256, 4, 2, 96, torch.float32),
    (200, 2, 3, 80, torch.float32),          # ragged: C not a multiple of the tile, tokens not of 64
    (384, 4, 2, 128, torch.float32),         # odd number of 128-row tiles
    (512, 4, 2, 200, torch.bfloat16),        # bf16 activations: two-product path
    (640, 3, 1, 130, torch.float16),
])
def test_grouped_hessian_sum(C, G, nseq, seqlen, dtype, variant):
    from gptq_plus_mp_quant_b200 import ops
    X = cases.make_acts(nseq, seqlen, C, seed=3, dtype=dtype)
    S = cases.make_saliency(nseq, seqlen, G, seed=3)
    ref = _oracle_grouped(X.float(), S)
    H = torch.zeros(G, C, C, device=DEV)
    act = torch.zeros(C, device=DEV)
    x2 = X.reshape(-1, C).to(DEV)
    s2 = S.reshape(-1, G).to(DEV)
    ops.hessian_accum(x2, s2, H, act, variant=variant)
    ops.hessian_finalize(H, None)                                   # mirror only
    ops.check_status(torch.device(DEV))
    ref_sym = 0.5 * (ref.H + ref.H.transpose(-1, -2))
    for g in range(G):
        assert rel_fro(H[g], ref_sym[g]) < 5e-6, f"group {g}"
    assert torch.allclose(act.cpu(), ref.act_square, rtol=2e-6, atol=0)
    assert torch.equal(H, H.transpose(-1, -2))                       # exactly symmetric


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("dtype,bound", [(torch.float32, 2e-6), (torch.bfloat16, 1e-6)])
def test_grouped_hessian_many_tokens_is_fp32_faithful(dtype, bound, variant):
    """From a few thousand tokens on the result sits at fp32-GEMM quality."""
    from gptq_plus_mp_quant_b200 import ops
    C, G, nseq, seqlen = 512, 4, 4, 2048
    X = cases.make_acts(nseq, seqlen, C, seed=13, dtype=dtype)
    S = cases.make_saliency(nseq, seqlen, G, seed=13)
    Xd = X.double().reshape(-1, C)
    Sd = S.double().reshape(-1, G)
    exact = torch.stack([Xd.t() @ (Xd * Sd[:, g:g + 1]) for g in range(G)])
    H = torch.zeros(G, C, C, device=DEV)
    ops.hessian_accum(X.reshape(-1, C).to(DEV), S.reshape(-1, G).to(DEV), H, None, variant=variant)
    ops.hessian_finalize(H, None)
    err = rel_fro(H, exact)
    dg = torch.diagonal(H[0]).double().cpu() / torch.diagonal(exact[0]) - 1
    print(f"variant {variant}: diagonal relative error mean {float(dg.mean()):+.3e} std {float(dg.std()):.3e}")
    ref = _oracle_grouped(X.float(), S)                                # the fp32 CPU path, for scale
    err_ref = rel_fro(ref.H, exact)
    print(f"rel. Frobenius vs fp64: kernel {err:.3e}, fp32 CPU path {err_ref:.3e}")
    assert err < bound
    assert err_ref < 1e-6


def test_hessian_chunking_and_accumulation_across_calls():
    """Several calls and several chunks per call give the same sum as one pass."""
    from gptq_plus_mp_quant_b200 import ops
    C, G = 256, 4
    X = cases.make_acts(4, 160, C, seed=9)
    S = cases.make_saliency(4, 160, G, seed=9)
    ref = _oracle_grouped(X, S)
    H = torch.zeros(G, C, C, device=DEV)
    act = torch.zeros(C, device=DEV)
    for s in range(4):
        ops.hessian_accum(X[s].to(DEV), S[s].to(DEV), H, act, chunk_tokens=64)
    ops.hessian_finalize(H, None)
    ref_sym = 0.5 * (ref.H + ref.H.transpose(-1, -2))
    assert rel_fro(H, ref_sym) < 5e-6
    assert torch.allclose(act.cpu(), ref.act_square, rtol=2e-6)


@pytest.mark.parametrize("case", [c for c in cases.PLUS_CASES if c[0] in ("plus_frozen_pc", "plus_ragged")],
                         ids=lambda c: c[0])
def test_gptqplus_add_batch_finalize_vs_reference(golden, case):
    """The drop-in object against the unmodified reference's H and act_square."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    (name, rows, cols, nseq, seqlen, G, bits, gs, act, static, alpha, ref_loss, mode, atomic) = case
    g = golden("gptq_plus.npz")
    W = cases.make_weight(rows, cols, seed=31)
    X = cases.make_acts(nseq, seqlen, cols, seed=31)
    if "ragged" in name:
        X[..., 5] = 0.0
    S = cases.make_saliency(nseq, seqlen, G, seed=31)
    Gr = cases.make_grad(rows, cols, seed=31)
    assert cases.digest(W, X, S, Gr) == str(g[f"{name}.digest"])
    layer = torch.nn.Linear(cols, rows, bias=False, device=DEV)
    layer.weight.data.copy_(W)
    obj = GPTQPlus(layer, S, Gr, G, alpha, ref_loss)
    obj.add_batch(X[:1].to(DEV), None)
    obj.add_batch(X[1:].to(DEV), None)
    obj.finalize_hessian()
    Href = torch.from_numpy(g[f"{name}.H"])
    assert rel_fro(obj.H, Href) < 5e-6
    assert torch.allclose(obj.act_square.cpu(), torch.from_numpy(g[f"{name}.act_square"]), rtol=2e-6)
    if "ragged" in name:
        assert float(obj.H[:, 5, :].abs().max()) == 0.0             # the dead channel stays exactly zero
    with pytest.raises(RuntimeError):
        obj.add_batch(X[:1].to(DEV), None)
    obj.finalize_hessian()                                           # idempotent


def test_plain_gptq_running_mean_vs_reference(golden):
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_utils import GPTQ
    case = [c for c in cases.PLAIN_CASES if c[0] == "plain_pc_act"][0]
    (name, rows, cols, nseq, seqlen, *_r) = case
    g = golden("plain_gptq.npz")
    W = cases.make_weight(rows, cols, seed=21)
    X = cases.make_acts(nseq, seqlen, cols, seed=21)
    layer = torch.nn.Linear(cols, rows, bias=False, device=DEV)
    layer.weight.data.copy_(W)
    obj = GPTQ(layer)
    for s in range(nseq):
        obj.add_batch(X[s:s + 1].to(DEV), None)
    assert obj.nsamples == nseq
    assert rel_fro(obj.H, torch.from_numpy(g[f"{name}.H"])) < 5e-6


def test_finalize_sanitises_nonfinite_and_counts():
    from gptq_plus_mp_quant_b200 import ops
    C, G = 96, 2
    H = torch.randn(G, C, C, device=DEV)
    H[0, 3, 7] = float("nan")
    H[1, 10, 10] = float("inf")
    H[1, 50, 20] = float("nan")                                      # below the diagonal: never read
    act = torch.ones(C, device=DEV) * 6
    counts = ops.hessian_finalize(H, act, div_tokens=2.0, div_scale=4.0, div_seq=3.0, sanitize=True)
    assert counts.tolist() == [2, 1]                                 # (3,7) counted with its mirror
    assert torch.isfinite(H).all()
    assert float(H[0, 3, 7]) == 0.0 and float(H[0, 7, 3]) == 0.0
    assert torch.equal(H, H.transpose(-1, -2))
    assert torch.allclose(act, torch.full((C,), 2.0, device=DEV))


def test_finalize_before_accumulate_raises():
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    layer = torch.nn.Linear(64, 8, bias=False, device=DEV)
    obj = GPTQPlus(layer, torch.ones(1, 4, 2), torch.zeros(8, 64), 2, 0.0, 0.0)
    with pytest.raises(RuntimeError):
        obj.finalize_hessian()


# ---------------------------------------------------------------------------- Hadamard
@pytest.mark.parametrize("case", cases.HADAMARD_CASES, ids=lambda c: c[0])
def test_rotation_vs_reference_and_exact(golden, case):
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    name, rows, n, dtype = case
    g = golden("hadamard.npz")
    dt = getattr(torch, dtype)
    x = cases.make_acts(1, rows, n, seed=5).reshape(rows, n).to(dt)
    hadK, K = hu.get_hadK(n)
    assert K == int(g[f"{name}.K"])
    xd = x.to(DEV)
    keep = xd.clone()
    y = hu.matmul_hadU_cuda(xd, hadK, K)
    assert torch.equal(xd, keep)                                     # input untouched
    exact = ohad.rotate_exact(x, hadK, K)
    scale = float(exact.abs().max())
    # fp32 internals + one rounding to the I/O dtype
    tol = {"float32": 1e-6, "bfloat16": 2.0 ** -8, "float16": 2.0 ** -11}[dtype]
    assert float((y.double().cpu() - exact).abs().max()) <= tol * scale * 1.01
    # and as close to the reference's own output as that output is to the exact operator
    yref = torch.from_numpy(g[f"{name}.y"]).double()
    ref_err = float((yref - exact).abs().max())
    assert float((y.double().cpu() - yref).abs().max()) <= ref_err + tol * scale * 1.01
    y2 = hu.matmul_hadU(xd)
    assert torch.equal(y2, y)


@pytest.mark.parametrize("n", [128, 4096, 12288, 28672])
def test_rotation_full_sizes_are_orthogonal(n):
    """Size-independent properties at the benchmark's row lengths: applying the (symmetric for
    K = 1, transposed for K > 1) rotation twice returns the input; norms are preserved."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    x = torch.randn(64, n, device=DEV)
    hadK, K = hu.get_hadK(n)
    y = hu.matmul_hadU_cuda(x, hadK, K)
    assert torch.allclose(y.norm(dim=1), x.norm(dim=1), rtol=1e-5)
    hadKt, _ = hu.get_hadK(n, transpose=True)
    back = hu.matmul_hadU_cuda(y, hadKt, K)
    assert float((back - x).abs().max()) < 2e-5 * float(x.abs().max()) * 4


@pytest.mark.parametrize("n,rows,dtype", [(12288, 1301, "bfloat16"), (12288, 700, "float32"), (20480, 650, "bfloat16"),
                                          (28672, 650, "bfloat16"), (28672, 330, "float32"), (28672, 37, "float16"),
                                          (24576, 300, "bfloat16"), (49152, 160, "float32"), (4096, 2500, "bfloat16"),
                                          (8192, 700, "float16"), (2048, 3000, "float32")])
def test_rotation_register_resident_kernels_vs_exact_operator(n, rows, dtype):
    """The kernels the benchmark lengths run (K chunks of 1024 / 2048 / 4096 with the tabulated 12 / 20 / 28 mix, and
    the 2048 / 4096 / 8192-long single chunks) against the exact operator in fp64, with enough rows that every CTA
    takes several turns of its grid-stride loop and a row count that no tile size divides: fp32 internals plus one
    rounding to the I/O dtype; also the transposed matrix (a non-tabulated one: the entry-by-entry mix)."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    dt = getattr(torch, dtype)
    x = cases.make_acts(1, rows, n, seed=13).reshape(rows, n).to(dt)
    tol = {"float32": 2e-6, "bfloat16": 2.0 ** -8, "float16": 2.0 ** -11}[dtype]
    for transpose in (False, True):
        hadK, K = hu.get_hadK(n, transpose=transpose)
        if transpose and K == 1:
            continue
        y = hu.matmul_hadU_cuda(x.to(DEV), hadK, K)
        exact = ohad.rotate_exact(x, hadK, K)
        assert float((y.double().cpu() - exact).abs().max()) <= tol * float(exact.abs().max()) * 1.01, (n, transpose)


@pytest.mark.parametrize("K,P,dtype", [(172, 64, "float32"), (172, 64, "bfloat16"), (68, 32, "float16"), (252, 16, "float32"),
                                           (70, 2, "float32"), (172, 1, "float32")])
def test_rotation_with_wide_mix_matrix(K, P, dtype):
    """Orders above 64 (11008 = 172 * 64 and the like): the mix reads its matrix from global memory.  Any +-1
    matrix exercises the arithmetic; compared with the exact operator built from the same matrix."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    g = torch.Generator().manual_seed(K)
    hadK = (torch.randint(0, 2, (K, K), generator=g) * 2 - 1).float()
    n, rows = K * P, 37
    dt = getattr(torch, dtype)
    x = cases.make_acts(1, rows, n, seed=9).reshape(rows, n).to(dt)
    y = hu.matmul_hadU_cuda(x.to(DEV), hadK, K)
    exact = ohad.rotate_exact(x, hadK, K)
    tol = {"float32": 2e-6, "bfloat16": 2.0 ** -8, "float16": 2.0 ** -11}[dtype]
    assert float((y.double().cpu() - exact).abs().max()) <= tol * float(exact.abs().max()) * 1.01
    xin = x.to(DEV).clone()
    hu.fwht(xin, hadK, K, scale=1.0 / math.sqrt(n), out=xin)                      # in place
    assert torch.equal(xin, y)


def test_hadamard_autograd_is_self_adjoint():
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    u = torch.randn(8, 256, device=DEV, requires_grad=True)
    w = torch.randn(8, 256, device=DEV)
    (hu.HadamardTransform.apply(u) * w).sum().backward()
    assert torch.allclose(u.grad, hu.HadamardTransform.apply(w), rtol=1e-5, atol=1e-4)


def test_rotation_empty_and_single_row():
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    assert hu.matmul_hadU_cuda(torch.empty(0, 128, device=DEV), None, 1).shape == (0, 128)
    x = torch.randn(1, 64, device=DEV)
    y = hu.matmul_hadU_cuda(x, None, 1)
    assert torch.allclose(y.cpu(), ohad.rotate_exact(x.cpu(), None, 1).float(), atol=1e-5)


# ---------------------------------------------------------------------------- quantizer
def _range_error(x, scale, zero, maxq, sym, norm=2.4):
    """Per-row sum |q - x|^norm of quantizing x with the given ranges, the quantity the shrink-grid search minimises
    (utils/quant_utils.py:436-448), in fp64."""
    if sym:
        q = scale * torch.clamp(torch.round(x / scale), -(maxq + 1), maxq)
    else:
        q = scale * (torch.clamp(torch.round(x / scale) + zero, 0, maxq) - zero)
    return (q - x).abs().pow(norm).sum(dim=1)


@pytest.mark.parametrize("case", cases.QUANTIZER_CASES, ids=lambda c: c[0])
def test_weight_quantizer_vs_reference(golden, case):
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    name, rows, cols, bits, pc, sym, mse = case
    g = golden("quantizer.npz")
    W = cases.make_weight(rows, cols, seed=11)
    q = WeightQuantizer()
    q.configure(bits, perchannel=pc, sym=sym, mse=mse)
    assert not bool(q.ready())
    q.find_params(W.to(DEV))
    assert bool(q.ready())
    assert int(q.maxq) == int(g[f"{name}.maxq"])
    sref, zref = torch.from_numpy(g[f"{name}.scale"]), torch.from_numpy(g[f"{name}.zero"])
    assert q.scale.shape == sref.shape and q.zero.shape == zref.shape
    if mse:
        # the search compares error sums whose last bits depend on summation order: a near-tie may pick the
        # neighbouring lattice point.  Most rows must agree, and where a row does not, the range the device picked
        # must be as good as the reference's: its error sum, evaluated in fp64, within 1e-5 relative
        same = torch.isclose(q.scale.cpu(), sref, rtol=1e-6).flatten()
        assert float(same.float().mean()) >= 0.9
        Wd = (W if pc else W.flatten().unsqueeze(0)).double()
        err_dev = _range_error(Wd, q.scale.cpu().double().reshape(-1, 1), q.zero.cpu().double().reshape(-1, 1), int(q.maxq), sym)
        err_ref = _range_error(Wd, sref.double().reshape(-1, 1), zref.double().reshape(-1, 1), int(q.maxq), sym)
        assert torch.allclose(err_dev[~same], err_ref[~same], rtol=1e-5, atol=0)
        return
    assert torch.allclose(q.scale.cpu(), sref, rtol=1e-6, atol=0)
    assert torch.equal(q.zero.cpu(), zref)
    deq, codes, scale = q.fake_quantize(W.to(DEV))
    assert torch.equal(codes.cpu(), torch.from_numpy(g[f"{name}.fake_codes"]))
    assert torch.allclose(deq.cpu(), torch.from_numpy(g[f"{name}.fake_deq"]), rtol=1e-6, atol=0)
    assert torch.allclose(q.quantize(W.to(DEV)).cpu(), torch.from_numpy(g[f"{name}.ste"]), rtol=1e-6, atol=0)


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("groupsize", [-1, 128])
def test_shrink_grid_search_vs_oracle_midsize(sym, groupsize):
    """The register-resident search (repeated scales of the symmetric lattice skipped, |d|^2.4 as d^2 * 2^(0.4 log2 d))
    against the oracle's 625 torch passes on 192 x 1024 weights: the chosen lattice point agrees for all but a few
    units, and where it does not the two choices' error sums agree to 1e-5 (a near-tie decided by summation order)."""
    from gptq_plus_mp_quant_b200.utils import quant_utils as qu
    R, C, bits = 192, 1024, 4
    maxq = 2 ** (bits - 1) - 1 if sym else 2 ** bits - 1
    W = cases.make_weight(R, C, seed=77)
    W[3] = 0.0                                                         # an all-zero row
    W[5, :128] = 0.25                                                  # a constant group
    gs = groupsize if groupsize > 0 else C
    scale, zero = qu.find_params_groups(W.to(DEV), gs, maxq, sym, True)
    scale, zero = scale.cpu(), zero.cpu()                              # [groups, R]
    q = oq.OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=sym, mse=True)
    bad = total = 0
    for gi in range(C // gs):
        blk = W[:, gi * gs:(gi + 1) * gs]
        q.find_params(blk)
        s_ref, z_ref = q.scale.flatten(), q.zero.flatten()
        same = (scale[gi] == s_ref) & (zero[gi] == z_ref)
        bad += int((~same).sum())
        total += R
        if not bool(same.all()):
            def err(sc, zr):
                sc, zr = sc.unsqueeze(1), zr.unsqueeze(1)
                if sym:
                    deq = sc * torch.clamp(torch.round(blk / sc), -(maxq + 1), maxq)
                else:
                    deq = sc * (torch.clamp(torch.round(blk / sc) + zr, 0, maxq) - zr)
                return (deq - blk).abs().pow(2.4).sum(1)
            e_dev, e_ref = err(scale[gi], zero[gi]), err(s_ref, z_ref)
            assert torch.allclose(e_dev[~same], e_ref[~same], rtol=1e-5, atol=0)
    print(f"shrink-grid search sym={sym} groupsize={groupsize}: {bad} of {total} units picked another lattice point")
    assert bad <= total // 50


def test_static_group_ranges_match_per_slice_calls():
    from gptq_plus_mp_quant_b200.utils import quant_utils as qu
    W = cases.make_weight(40, 300, seed=4)
    scale, zero = qu.find_params_groups(W.to(DEV), 128, 7, True)
    assert scale.shape == (3, 40)
    for gi in range(3):
        s_ref, z_ref = oq.find_params(W[:, gi * 128:(gi + 1) * 128], 4, perchannel=True, sym=True)
        assert torch.allclose(scale[gi].cpu(), s_ref.flatten(), rtol=1e-6, atol=0)


def test_quantizer_edge_rows():
    """All-zero rows: the symmetric scale clamps at 1e-5/maxq; the asymmetric range becomes (-1, +1)."""
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    W = torch.zeros(4, 32)
    W[1] = torch.linspace(-1, 2, 32)
    for sym in (True, False):
        q = WeightQuantizer()
        q.configure(4, perchannel=True, sym=sym)
        q.find_params(W.to(DEV))
        s_ref, z_ref = oq.find_params(W, 4, perchannel=True, sym=sym)
        assert torch.allclose(q.scale.cpu(), s_ref, rtol=1e-6)
        assert torch.equal(q.zero.cpu(), z_ref)
    q16 = WeightQuantizer()
    q16.configure(16)
    q16.find_params(W.to(DEV))
    assert q16.quantize(W.to(DEV)).equal(W.to(DEV))


def test_ste_gradient_passes_through():
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    W = cases.make_weight(8, 64, seed=2).to(DEV).requires_grad_(True)
    q = WeightQuantizer()
    q.configure(4, perchannel=True, sym=True)
    q.find_params(W.detach())
    q.quantize(W).sum().backward()
    assert torch.equal(W.grad, torch.ones_like(W))


@pytest.mark.gpu
def test_hessian_pipelined_matches_in_order():
    """Packing and contraction on two streams (chunk slots ordered by events) give the bits of the in-order call."""
    from gptq_plus_mp_quant_b200 import ops
    torch.manual_seed(3)
    N, C, G = 3 * 8192 + 640, 384, 2
    x = (torch.randn(N, C, device=DEV) * torch.exp(torch.randn(C, device=DEV))).bfloat16()
    s = torch.exp(torch.randn(N, G, device=DEV))
    outs = []
    for piped in (False, True):
        H = torch.zeros(G, C, C, device=DEV)
        act = torch.zeros(C, device=DEV)
        for part in (x[:N // 2], x[N // 2:]):
            sal = s[:N // 2] if part.data_ptr() == x.data_ptr() else s[N // 2:]
            ops.hessian_accum(part, sal, H, act, pipeline=piped)
        ops.hessian_join(H.device)
        ops.hessian_finalize(H, None)
        outs.append((H.clone(), act.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    ops.check_status(H.device)


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.CLIP_CASES, ids=lambda c: c[0])
def test_clip_module_weight_to_quant_bounds(golden, case):
    """Pre-clip of a linear to its quantizer's range against the reference's output.  The range search may pick the
    neighbouring lattice point in a near-tie (see the quantizer test), which moves that row's bounds: rows whose
    scale matches the oracle's must match bit for bit, and all but a few rows must."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import clip_module_weight_to_quant_bounds_
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    name, rows, cols, bits, sym, dtype = case
    g = golden("clip.npz")
    W = cases.make_weight(rows, cols, seed=13).to(getattr(torch, dtype))
    layer = torch.nn.Linear(cols, rows, bias=False, device=DEV, dtype=W.dtype)
    layer.weight.data.copy_(W)
    clip_module_weight_to_quant_bounds_(layer, bits, sym, True)
    got = layer.weight.data.float().cpu()
    ref = torch.from_numpy(g[f"{name}.clipped"])
    assert layer.weight.dtype == W.dtype
    q_dev = WeightQuantizer()
    q_dev.configure(bits, perchannel=True, sym=sym, mse=True)
    q_dev.find_params(W.float().to(DEV))
    q_ref = oq.OracleWeightQuantizer()
    q_ref.configure(bits, perchannel=True, sym=sym, mse=True)
    q_ref.find_params(W.float())
    same = (q_dev.scale.cpu().flatten() == q_ref.scale.flatten()) & (q_dev.zero.cpu().flatten() == q_ref.zero.flatten())
    assert float(same.float().mean()) >= 0.9
    # rows whose searched range differs from the CPU's are near-ties of the search: equally good ranges
    err_dev = _range_error(W.double(), q_dev.scale.cpu().double().reshape(-1, 1), q_dev.zero.cpu().double().reshape(-1, 1),
                           int(q_dev.maxq), sym)
    err_ref = _range_error(W.double(), q_ref.scale.double().reshape(-1, 1), q_ref.zero.double().reshape(-1, 1),
                           int(q_dev.maxq), sym)
    assert torch.allclose(err_dev[~same], err_ref[~same], rtol=1e-5, atol=0)
    assert torch.equal(got[same], ref[same])
    assert int((got != W.float()).sum()) > 0
    # no-ops
    before = layer.weight.data.clone()
    clip_module_weight_to_quant_bounds_(layer, 16, sym, True)
    clip_module_weight_to_quant_bounds_(layer, bits, sym, False)
    assert torch.equal(before, layer.weight.data)


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.SALIENCY_CASES, ids=lambda c: c[0])
def test_saliency_cache_hook_vs_reference(golden, case):
    """The drop-in SaliencyCache on a CUDA linear whose output gradient is known exactly (loss = sum(out * coef))
    against the reference's cached saliency: fp32 sums of squares in a different order, 2e-6 relative."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import SaliencyCache
    name, batch, seq, hidden, G, sink, dtype = case
    g = golden("saliency.npz")
    dt = getattr(torch, dtype)
    lin = torch.nn.Linear(hidden, hidden, bias=False, device=DEV, dtype=dt)
    x = cases.make_acts(batch, seq, hidden, seed=17).to(dt).to(DEV)
    coef = cases.make_out_grad(batch, seq, hidden, seed=17).to(dt).to(DEV)
    cache = SaliencyCache(["lin"], G, sink_size=sink)
    cache.add_hook({"lin": lin})
    (lin(x) * coef).sum().backward()
    (sal,) = cache.saliency_cache["lin"]
    cache.disable_hooks()
    (lin(x) * coef).sum().backward()
    assert len(cache.saliency_cache["lin"]) == 1                       # disabled hooks record nothing
    cache.clear_hook()
    cache.clear_cache()
    assert cache.saliency_cache["lin"] == [] and cache.handles == []
    ref = torch.from_numpy(g[f"{name}.saliency"])
    assert sal.shape == ref.shape and sal.dtype == torch.float32
    assert torch.allclose(sal.cpu(), ref, rtol=2e-6, atol=0)


@pytest.mark.gpu
@pytest.mark.parametrize("n,q", [(8 * 2048 * 4, 0.99), (100, 0.5), (4097, 0.999), (2, 0.3), (1, 0.99),
                                 (3_000_001, 0.99), (20_000_000, 0.9)])
def test_saliency_percentile_clip_vs_oracle(n, q):
    """Radix selection of the two order statistics + lerp + clamp against the oracle's sort-based restatement of
    torch.quantile: the cap within one rounding (the lerp may or may not contract to a fused multiply-add), every
    element below the cap untouched, the rest equal to the cap.  Sizes beyond torch.quantile's 16M limit work."""
    from gptq_plus_mp_quant_b200 import ops
    s = torch.exp(3.0 * torch.randn(n, generator=torch.Generator().manual_seed(n % 1000)))
    s[: n // 7] = s[0]
    s[n // 3] = -0.0
    _, cap_ref = ohess.clip_at_percentile(s, q)
    x = s.to(DEV)
    cap = ops.clamp_to_quantile_(x, q)
    assert abs(float(cap) - float(cap_ref)) <= 1.2e-7 * abs(float(cap_ref))
    assert torch.equal(x.cpu(), torch.clamp(s, max=cap.cpu()))
    bad = s.clone()
    bad[n // 2] = float("nan")
    xb = bad.to(DEV)
    assert torch.isnan(ops.clamp_to_quantile_(xb, q)) and bool(torch.isnan(xb).all())


@pytest.mark.gpu
def test_saliency_cache_clips_at_percentile():
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import SaliencyCache
    lin = torch.nn.Linear(256, 256, bias=False, device=DEV)
    x = cases.make_acts(2, 300, 256, seed=3).to(DEV)
    coef = cases.make_out_grad(2, 300, 256, seed=3).to(DEV)
    got = []
    for pct in (None, 0.9):
        cache = SaliencyCache(["lin"], 4, clip_percentile=pct)
        cache.add_hook({"lin": lin})
        (lin(x) * coef).sum().backward()
        got.append(cache.saliency_cache["lin"][0].cpu())
        cache.clear_hook()
    ref, _ = ohess.clip_at_percentile(got[0], 0.9)
    assert torch.allclose(got[1], ref, rtol=2e-7, atol=0) and int((got[1] != got[0]).sum()) > 0


@pytest.mark.gpu
def test_fisher_accumulation_vs_oracle():
    """Layer-output Fisher sum grad^T grad / scale over two batches on the tensor-core Gram kernel."""
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import fisher_accumulate_, fisher_finalize_
    hidden, sink = 384, 3
    grads = [cases.make_out_grad(2, 515, hidden, seed=s).bfloat16() for s in (5, 6)]
    ref = sum(ohess.fisher_block(gr, sink) for gr in grads)
    F = torch.zeros(hidden, hidden, device=DEV)
    for gr in grads:
        fisher_accumulate_(F, gr.to(DEV), sink)
    fisher_finalize_(F)
    assert float((F.cpu() - ref).norm() / ref.norm()) < 5e-6
    assert torch.equal(F, F.t())


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.ACT_QUANT_CASES, ids=lambda c: c[0])
def test_act_quantizer_vs_reference(golden, case):
    """The fused activation fake-quant kernel against the reference's ActQuantizer, bit for bit: ranges, dequantized
    values (stored-range forward and the one-pass path) and integer codes."""
    from gptq_plus_mp_quant_b200.utils.quant_utils import ActQuantizer
    name, shape, bits, gs, sym, clip, dtype = case
    g = golden("act_quant.npz")
    x = cases.make_act_tensor(shape, seed=23).to(getattr(torch, dtype)).to(DEV)
    q = ActQuantizer()
    q.configure(bits, groupsize=gs, sym=sym, clip_ratio=clip)
    q.find_params(x)
    assert torch.equal(q.scale.float().cpu(), torch.from_numpy(g[f"{name}.scale"]))
    assert torch.equal(q.zero.float().cpu(), torch.from_numpy(g[f"{name}.zero"]))
    y = q(x)
    assert y.dtype == x.dtype and y.shape == x.shape
    assert torch.equal(y.float().cpu(), torch.from_numpy(g[f"{name}.deq"]))
    assert torch.equal(q.quantize(x)[0].float().cpu(), torch.from_numpy(g[f"{name}.codes"]))
    q.free()
    assert torch.equal(q.fake_quant(x).float().cpu(), torch.from_numpy(g[f"{name}.deq"]))
    q16 = ActQuantizer()
    q16.configure(16)
    assert q16(x) is x


@pytest.mark.gpu
def test_act_quantizer_groupwise_entry_point():
    """ActQuantizer.find_params_per_token_groupwise (utils/quant_utils.py:131-153) is the grouped branch of
    find_params under its own name; without a group size it has nothing to range."""
    from gptq_plus_mp_quant_b200.utils.quant_utils import ActQuantizer
    x = torch.randn(2, 5, 256, device=DEV, dtype=torch.bfloat16)
    a, b = ActQuantizer(), ActQuantizer()
    for q in (a, b):
        q.configure(4, groupsize=64, sym=False, clip_ratio=0.9)
    a.find_params(x)
    b.find_params_per_token_groupwise(x)
    assert torch.equal(a.scale, b.scale) and torch.equal(a.zero, b.zero) and a.scale.shape == x.shape
    assert torch.equal(a(x), b(x))
    c = ActQuantizer()
    c.configure(4, groupsize=-1, sym=True)
    with pytest.raises(ValueError):
        c.find_params_per_token_groupwise(x)


def test_act_quant_wrapper_rotates_and_quantizes():
    """ActQuantWrapper: online Hadamard + 4-bit input fake-quant around a linear equals the same steps done by the
    oracle on the CPU (rotation within one bf16 rounding, hence compared after the quantizer on the kernel's own
    rotated input)."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    from gptq_plus_mp_quant_b200.utils.quant_utils import ActQuantWrapper
    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 64, bias=False, device=DEV, dtype=torch.bfloat16)
    wrap = ActQuantWrapper(lin)
    wrap.online_full_had = True
    wrap.had_K, wrap.K = hu.get_hadK(512)
    wrap.quantizer.configure(4, groupsize=-1, sym=False, clip_ratio=0.9)
    x = cases.make_act_tensor((2, 6, 512), seed=29).bfloat16().to(DEV)
    y = wrap(x)
    xr = hu.matmul_hadU_cuda(x, wrap.had_K, wrap.K)
    xq = oq.act_fake_quant(xr.cpu(), 4, -1, False, 0.9).to(DEV)
    assert torch.equal(y, lin(xq))


@pytest.mark.gpu
@pytest.mark.parametrize("n", [2048, 4096, 8192, 12288, 20480, 28672])
@pytest.mark.parametrize("dtype,sym,clip", [(torch.bfloat16, False, 0.9), (torch.float16, True, 1.0),
                                            (torch.float32, False, 1.0), (torch.bfloat16, True, 0.85)])
def test_fused_rotation_and_act_quant_is_the_two_kernels(n, dtype, sym, clip):
    """rq_fwht_act_quant writes exactly what rq_fwht followed by the per-token rq_act_quant writes (the rotated
    values are rounded to the I/O dtype before the range is taken), including an all-zero and a constant token."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    from gptq_plus_mp_quant_b200.utils.quant_utils import ActQuantizer
    x = cases.make_act_tensor((3, 11, n), seed=n % 97).to(dtype)
    x[0, 0] = 0
    x[1, 3] = 0.5
    x = x.to(DEV)
    hadK, K = hu.get_hadK(n)
    q = ActQuantizer()
    q.configure(4, groupsize=-1, sym=sym, clip_ratio=clip)
    two = q.fake_quant(hu.matmul_hadU_cuda(x, hadK, K))
    one = hu.fwht_act_quant(x, hadK, K, 1.0 / math.sqrt(n), clip, int(q.maxq), sym)
    assert one is not None and one.dtype == dtype
    assert torch.equal(one, two)


@pytest.mark.gpu
def test_act_quant_wrapper_uses_the_fused_kernel_where_it_applies():
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    from gptq_plus_mp_quant_b200.utils.quant_utils import ActQuantWrapper
    assert hu.fwht_act_quant(torch.zeros(4, 1024, device=DEV), None, 1, 1.0, 1.0, 15, True) is None   # not covered
    torch.manual_seed(0)
    lin = torch.nn.Linear(4096, 32, bias=False, device=DEV, dtype=torch.bfloat16)
    wrap = ActQuantWrapper(lin)
    wrap.online_full_had = True
    wrap.had_K, wrap.K = hu.get_hadK(4096)
    wrap.quantizer.configure(4, groupsize=-1, sym=False, clip_ratio=0.9)
    x = cases.make_act_tensor((2, 6, 4096), seed=33).bfloat16().to(DEV)
    y = wrap(x)
    xr = hu.matmul_hadU_cuda(x, wrap.had_K, wrap.K)
    xq = oq.act_fake_quant(xr.cpu(), 4, -1, False, 0.9).to(DEV)
    assert torch.equal(y, lin(xq))


@pytest.mark.gpu
@pytest.mark.parametrize("heads,head_dim,dtype", [(32, 128, torch.bfloat16), (8, 64, torch.float16), (64, 32, torch.float32)])
def test_fwht_across_heads(heads, head_dim, dtype):
    """The online partial rotation: Hadamard across the heads for every position inside a head, against the
    reference's formula evaluated in fp64 (one rounding of the I/O dtype)."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    x = cases.make_act_tensor((2, 5, heads * head_dim), seed=31).to(dtype)
    y = hu.fwht_heads(x.to(DEV), heads, head_dim, None, 1, 1.0 / heads ** 0.5)
    v = x.double().reshape(-1, heads, head_dim).transpose(1, 2)               # [.., D, H]: transform the last dim
    ref = (ohad.fwht_pow2(v.reshape(-1, heads)).reshape(v.shape) / heads ** 0.5).transpose(1, 2).reshape(x.shape)
    assert y.dtype == dtype and y.shape == x.shape
    tol = {torch.float32: 2e-6, torch.float16: 1.5e-3, torch.bfloat16: 1.2e-2}[dtype]
    assert float((y.cpu().double() - ref).abs().max() / ref.abs().max()) < tol
    # dense K x K matrix across the heads (the K != 1 branch): the Sylvester matrix itself must give the same
    if heads <= 32:
        Hm = ohad.fwht_pow2(torch.eye(heads, dtype=torch.float64)).float()
        y2 = hu.fwht_heads(x.to(DEV), heads, head_dim, Hm, heads, 1.0 / heads ** 0.5)
        assert float((y2.cpu().double() - ref).abs().max() / ref.abs().max()) < tol


@pytest.mark.gpu
def test_act_quant_wrapper_partial_rotation():
    from gptq_plus_mp_quant_b200.utils.quant_utils import ActQuantWrapper
    torch.manual_seed(1)
    lin = torch.nn.Linear(512, 32, bias=False, device=DEV, dtype=torch.bfloat16)
    wrap = ActQuantWrapper(lin)
    wrap.online_partial_had, wrap.had_dim, wrap.K = True, 64, 1
    x = cases.make_act_tensor((1, 7, 512), seed=37).bfloat16().to(DEV)
    y = wrap(x)
    v = x.float().reshape(-1, 8, 64).transpose(1, 2)
    xr = (ohad.fwht_pow2(v.cpu().double().reshape(-1, 8)).reshape(v.shape) / 8 ** 0.5).transpose(1, 2).reshape(x.shape)
    assert torch.allclose(y.float().cpu(), lin(xr.to(DEV).bfloat16()).float().cpu(), rtol=0.05, atol=0.05)


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.QK_CASES, ids=lambda c: c[0])
def test_qk_rotation_wrapper_vs_reference(golden, case):
    """The K-cache wrapper on the device against the reference's outputs.  The rotation agrees up to a rare last-bit
    flip of the I/O dtype, which can move a key across a quantization boundary: at most 0.5 % of the entries differ."""
    from gptq_plus_mp_quant_b200.utils.rotation_utils import QKRotationWrapper
    name, (b, h, kvh, t_, d), bits, gs, sym, clip, dtype = case
    g = golden("qk.npz")
    dt = getattr(torch, dtype)
    q = cases.make_act_tensor((b * h, t_, d), seed=41).reshape(b, h, t_, d).to(dt).to(DEV)
    k = cases.make_act_tensor((b * kvh, t_, d), seed=42).reshape(b, kvh, t_, d).to(dt).to(DEV)
    wrap = QKRotationWrapper(lambda a, c: (a, c), d, k_bits=bits, k_groupsize=gs, k_sym=sym, k_clip_ratio=clip)
    qo, ko = wrap(q, k)
    qr, kr = torch.from_numpy(g[f"{name}.q"]), torch.from_numpy(g[f"{name}.k"])
    assert qo.dtype == dt and ko.dtype == dt and qo.shape == q.shape and ko.shape == k.shape
    assert float((qo.float().cpu() != qr).float().mean()) < 0.005
    assert torch.allclose(qo.float().cpu(), qr, rtol=2 ** -7, atol=1e-6)
    assert float((ko.float().cpu() != kr).float().mean()) < 0.005
    with pytest.raises(ValueError):
        wrap.configure_k_quant(head_dim=d * 2)


@pytest.mark.gpu
@pytest.mark.parametrize("bits,cols", [(4, 256), (3, 200), (2, 72), (8, 64)])
def test_packed_export_round_trip(bits, cols):
    """Bit-stream packing of the integer codes and its torch inverse; the packed form of a quantized linear
    dequantizes to the layer's weight."""
    from gptq_plus_mp_quant_b200.utils import export_utils as ex
    g = torch.Generator().manual_seed(bits)
    lo, hi = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
    codes = torch.randint(lo, hi + 1, (37, cols), generator=g).float().to(DEV)
    packed = ex.pack_codes(codes, bits)
    assert packed.shape == (37, (cols + 7) // 8 * bits) and packed.dtype == torch.uint8
    assert torch.equal(ex.unpack_codes(packed, bits, cols).float(), codes)


@pytest.mark.gpu
def test_pack_quantized_linear():
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.utils import export_utils as ex
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    rows, cols, G = 32, 256, 2
    W = cases.make_weight(rows, cols, seed=81)
    X = cases.make_acts(2, 128, cols, seed=81)
    S = cases.make_saliency(2, 128, G, seed=81)
    layer = torch.nn.Linear(cols, rows, bias=False, device=DEV)
    layer.weight.data.copy_(W)
    obj = GPTQPlus(layer, S, cases.make_grad(rows, cols, seed=81), G, 0.25, 0.7)
    obj.quantizer = WeightQuantizer()
    obj.quantizer.configure(4, perchannel=True, sym=True)
    obj.add_batch(X.to(DEV), None)
    obj.finalize_hessian()
    obj.fasterquant(groupsize=128, actorder=True, static_groups=True, export_to_et=True)
    blob = ex.pack_quantized_linear(layer, 4, 128)
    assert blob["qweight"].numel() == rows * cols // 2 and blob["scales"].shape == (rows, 2)
    deq = ex.unpack_codes(blob["qweight"], 4, cols).float() * blob["scales"].repeat_interleave(128, dim=1)
    assert torch.equal(deq, layer.weight.data)


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.WGROUP_CASES, ids=lambda c: c[0])
def test_weight_quantizer_grouped_vs_reference(golden, case):
    """Grouped weight ranges (weight_groupsize > 0) on the device, bit for bit against the reference: ranges,
    fake_quantize (values, codes, row-sliced call) and quantize()."""
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    name, rows, cols, bits, gs, sym, dtype = case
    g = golden("wgroup.npz")
    W = cases.make_weight(rows, cols, seed=19).to(getattr(torch, dtype))
    W[0, :gs] = 0
    Wd = W.to(DEV)
    q = WeightQuantizer()
    q.configure(bits, perchannel=True, sym=sym, mse=False, weight_groupsize=gs)
    q.find_params(Wd)
    assert bool(q.ready()) and q.scale.shape == W.shape and q.scale.dtype == W.dtype
    assert torch.equal(q.scale.float().cpu(), torch.from_numpy(g[f"{name}.scale"]))
    assert torch.equal(q.zero.float().cpu(), torch.from_numpy(g[f"{name}.zero"]))
    deq, codes, scale = q.fake_quantize(Wd)
    assert torch.equal(deq.float().cpu(), torch.from_numpy(g[f"{name}.fake"]))
    assert torch.equal(codes.float().cpu(), torch.from_numpy(g[f"{name}.codes"]))
    assert torch.equal(q.quantize(Wd).float().cpu(), torch.from_numpy(g[f"{name}.ste"]))
    d2, c2, s2 = q.fake_quantize(Wd[4:8], st_idx=4, end_idx=8)
    assert torch.equal(d2, deq[4:8]) and torch.equal(c2, codes[4:8]) and torch.equal(s2, scale[4:8])


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.WGROUP_MSE_CASES, ids=lambda c: c[0])
def test_weight_quantizer_grouped_mse_vs_reference(golden, case):
    """The shrink-grid search over grouped weight ranges on the device against the reference.  Half-precision
    weights: bit for bit (every step is rounded to the dtype, which hides the last bits of powf and of the sum).
    fp32: a candidate whose error sum ties the best within float rounding may be taken or not, so a few groups may
    carry a neighbouring lattice point; those are counted and their error sums checked to be equal to 1e-5."""
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    name, rows, cols, bits, gs, sym, dtype = case
    g = golden("wgroup_mse.npz")
    W = cases.make_weight(rows, cols, seed=23).to(getattr(torch, dtype))
    W[0, :gs] = 0
    W[1, :gs] = 0.5
    Wd = W.to(DEV)
    q = WeightQuantizer()
    q.configure(bits, perchannel=True, sym=sym, mse=True, weight_groupsize=gs)
    q.find_params(Wd)
    assert q.scale.shape == W.shape and q.scale.dtype == W.dtype
    scale_ref, zero_ref = torch.from_numpy(g[f"{name}.scale"]), torch.from_numpy(g[f"{name}.zero"])
    same = (q.scale.float().cpu() == scale_ref) & (q.zero.float().cpu() == zero_ref)
    bad_groups = int((~same).reshape(rows, cols // gs, gs).any(dim=-1).sum())
    print(f"{name}: {bad_groups} of {rows * cols // gs} groups picked another lattice point")
    if dtype != "float32":
        assert bad_groups == 0
        assert torch.equal(q.quantize(Wd).float().cpu(), torch.from_numpy(g[f"{name}.ste"]))
    else:
        assert bad_groups <= max(1, rows * cols // gs // 20)
        ste, ref = q.quantize(Wd).float().cpu(), torch.from_numpy(g[f"{name}.ste"])
        e1 = (ste - W.float()).abs().pow(2.4).reshape(rows, -1, gs).sum(-1)
        e2 = (ref - W.float()).abs().pow(2.4).reshape(rows, -1, gs).sum(-1)
        assert torch.allclose(e1, e2, rtol=1e-5, atol=0)


@pytest.mark.parametrize("C,G,pieces", [(256, 2, 1), (384, 4, 2), (200, 1, 4), (130, 3, 1)])
def test_packed_upper_round_trip(C, G, pieces):
    """pack_upper keeps exactly the entries from each row's 128-block start to the row's end; unpack_upper puts
    them back; everything on or above the diagonal survives the trip bit for bit."""
    from gptq_plus_mp_quant_b200 import ops
    g = torch.Generator(device="cpu").manual_seed(C + G)
    H = torch.randn(G, C, C, generator=g).to(DEV)
    packed = ops.pack_upper(H, pieces)
    n = ops.packed_upper_elems(C)
    assert packed.shape[0] == G and packed.shape[1] >= n and packed.shape[1] % (4 * pieces) == 0
    assert float(packed[:, n:].abs().sum()) == 0.0
    # reference layout built with torch indexing
    ref = torch.cat([H[:, r, (r // 128) * 128:] for r in range(C)], dim=1)
    assert ref.shape[1] == n and torch.equal(packed[:, :n], ref)
    out = torch.full_like(H, float("nan"))
    ops.unpack_upper(packed.clone(), out)
    iu = torch.triu(torch.ones(C, C, dtype=torch.bool, device=DEV))
    assert torch.equal(out[:, iu], H[:, iu])
    kept = torch.zeros(C, C, dtype=torch.bool, device=DEV)
    for r in range(C):
        kept[r, (r // 128) * 128:] = True
    assert bool(torch.isnan(out[:, ~kept]).all())          # nothing else is written


@pytest.mark.parametrize("out_f,in_f,had_dim,output,dtype,use_r2", [
    (96, 1536, -1, False, torch.bfloat16, False),       # full-width rotation of the input side, K = 12
    (1536, 64, -1, True, torch.float16, False),          # full-width rotation of the output side
    (48, 512, 128, False, torch.bfloat16, False),        # per-head rotation (fp64 matmul), input side
    (512, 40, 64, True, torch.float32, False),           # per-head rotation, output side
    (48, 512, 128, False, torch.bfloat16, True),         # caller's own orthogonal matrix R2 instead of the Hadamard
])
def test_apply_exact_had_to_linear(out_f, in_f, had_dim, output, dtype, use_r2):
    """Fusing a rotation into a linear's weight (utils/hadamard_utils.py:133-168) against an fp64 evaluation of the
    same operator: within one rounding of the weight's dtype, dtype and device preserved."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    g = torch.Generator().manual_seed(out_f + in_f)
    W = (torch.randn(out_f, in_f, generator=g) * 0.05).to(dtype)
    lin = torch.nn.Linear(in_f, out_f, bias=False, device=DEV, dtype=dtype)
    lin.weight.data.copy_(W)
    R2 = None
    if use_r2:
        R2 = torch.linalg.qr(torch.randn(had_dim, had_dim, generator=g, dtype=torch.float64))[0].to(DEV)
    hu.apply_exact_had_to_linear(lin, had_dim=had_dim, output=output, R2=R2)
    assert lin.weight.dtype == dtype and lin.weight.device.type == "cuda" and lin.weight.shape == (out_f, in_f)
    Wd = W.double()
    if had_dim == -1:
        n = out_f if output else in_f
        hadK, K = hu.get_hadK(n)
        exact = ohad.rotate_exact(Wd.t().contiguous(), hadK, K).t() if output else ohad.rotate_exact(Wd, hadK, K)
    else:
        Hm = R2.cpu() if use_r2 else ohad.rotate_exact(torch.eye(had_dim, dtype=torch.float64), None, 1)
        src = Wd.t().contiguous() if output else Wd
        rot = (src.reshape(-1, src.shape[-1] // had_dim, had_dim) @ Hm).reshape(src.shape)
        exact = rot.t() if output else rot
    got = lin.weight.data.double().cpu()
    eps = {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -11, torch.float32: 2 ** -22}[dtype]
    assert float((got - exact).abs().max()) <= eps * float(exact.abs().max()) * 1.01 + 1e-12


@pytest.mark.parametrize("size", [128, 1536])
def test_random_hadamard_matrix(size):
    """utils/hadamard_utils.py:76-80: diag(+-1) times the normalised Hadamard matrix, built in fp64.  As in the
    reference the normalisation divides by ``torch.tensor(size).sqrt()``, an fp32 square root, so the entries are
    +-1/sqrt(size) to fp32 accuracy (exactly when size is a power of four) and orthogonality holds to ~1e-7; the
    signs are the generator's."""
    from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu
    gen = torch.Generator().manual_seed(3)
    Q = hu.random_hadamard_matrix(size, DEV, generator=gen)
    assert Q.dtype == torch.float64 and Q.shape == (size, size) and Q.device.type == "cuda"
    eye = torch.eye(size, dtype=torch.float64, device=DEV)
    assert float((Q @ Q.t() - eye).abs().max()) < 1e-6
    assert float((Q.abs() - 1.0 / math.sqrt(size)).abs().max()) < 1e-8
    assert float((Q.abs() - Q.abs()[0, 0]).abs().max()) < 1e-15          # one magnitude throughout
    signs = torch.randint(low=0, high=2, size=(size,), generator=torch.Generator().manual_seed(3)).double() * 2 - 1
    hadK, K = hu.get_hadK(size)
    exact = ohad.rotate_exact(torch.diag(signs), hadK, K)
    assert float((Q.cpu() - exact).abs().max()) < 1e-8
    assert torch.equal(torch.sign(Q.cpu()), torch.sign(exact))
    H = hu.hadamard_matrix(size, DEV)
    assert float((H.double() @ H.double().t() - eye).abs().max()) < 1e-5
