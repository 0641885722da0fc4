"""Oracle: damped inverse-Hessian factor and the ``fasterquant`` block loop.

Test infrastructure (see ``oracle/__init__.py``).  Restates

* plain GPTQ ``fasterquant``                      gptq_utils/gptq_utils.py:45-174
* ``_compute_hessian_inverse_with_fallback``      gptq_utils/gptq_plus_utils.py:494-561
* ``compute_safe_beta_from_reference_loss``       gptq_utils/gptq_plus_utils.py:174-194
* ``_compute_gradient_terms``                     gptq_utils/gptq_plus_utils.py:563-578
* GPTQ+ ``fasterquant`` (set-up, inner column loop, lazy trailing update, epilogue) for
  the modes that need no autograd callback: ``frozen``, ``surrogate_block``,
  ``surrogate_online``, with or without ``block_atomic_quant``
                                                  gptq_utils/gptq_plus_utils.py:910-1896
"""
from __future__ import annotations

import copy
import math

import torch

LinAlgError = torch._C._LinAlgError


# --------------------------------------------------------------------------------------
# damped Cholesky -> inverse -> upper factor
# --------------------------------------------------------------------------------------
def hinv_with_fallback(H_sub: torch.Tensor, percdamp: float = 0.01, step: float = 0.0015):
    """(Hinv_init, Hinv_upper, damp_percent, identity_fallback).

    Damping ``p * mean(diag)`` is added to the *already damped* working matrix on every
    retry and the mean is re-taken from it; a failed or non-finite factorisation bumps
    ``p`` by ``step``; at ``p >= 1`` both results are the identity
    (gptq_plus_utils.py:494-561).
    """
    p = float(percdamp)
    if p <= 0:
        raise ValueError("damp_percent must be positive")
    work = H_sub.clone()
    idx = torch.arange(work.shape[0])
    while 0 < p < 1:
        try:
            work[idx, idx] += p * torch.mean(torch.diag(work))
            low = torch.linalg.cholesky(work)
            inv = torch.cholesky_inverse(low)
            up = torch.linalg.cholesky(inv, upper=True)
            if not torch.isfinite(inv).all() or not torch.isfinite(up).all():
                raise LinAlgError("non-finite inverse")
            return inv, up, p, False
        except LinAlgError:
            p += step
    eye = torch.eye(H_sub.shape[0], dtype=H_sub.dtype)
    return eye, eye.clone(), p, True


def plain_hinv(H: torch.Tensor, percdamp: float = 0.01, step: float = 0.0015) -> torch.Tensor:
    """Upper factor of the damped inverse as plain GPTQ builds it; ``H`` is damped in
    place like the reference; running out of range raises (gptq_utils.py:88-106)."""
    p = percdamp
    n = H.shape[0]
    idx = torch.arange(n)
    while 0 < p < 1:
        try:
            H[idx, idx] += p * torch.mean(torch.diag(H))
            low = torch.linalg.cholesky(H)
            inv = torch.cholesky_inverse(low)
            return torch.linalg.cholesky(inv, upper=True)
        except LinAlgError:
            p += step
    raise ValueError(f"Quantization: `damp_percent` must between 0 and 1. current is {p}")


# --------------------------------------------------------------------------------------
# GPTQ+ first-order terms
# --------------------------------------------------------------------------------------
def safe_beta(grad_sub, hinv_init, reference_loss: float, alpha: float):
    """Per-row beta in [0, 1] and ``G . H^-1`` (gptq_plus_utils.py:174-194)."""
    ghinv_init = grad_sub.matmul(hinv_init)
    if reference_loss <= 0:
        return torch.zeros(grad_sub.shape[0], dtype=grad_sub.dtype), ghinv_init
    c = (grad_sub * ghinv_init).sum(dim=1) - ((ghinv_init ** 2) / torch.diagonal(hinv_init).unsqueeze(0)).mean(1)
    target = 2 * alpha * reference_loss
    c = torch.clamp(c, min=target)
    ratio = torch.where(c > 0, target / c, torch.zeros_like(c))
    ratio = torch.clamp(ratio, min=0.0, max=1.0)
    beta = 1 - torch.sqrt(torch.clamp(1 - ratio, min=0.0))
    return torch.nan_to_num(beta, nan=0.0, posinf=1.0, neginf=0.0), ghinv_init


def gradient_terms(grad_sub, hinv_init, hinv, alpha: float, reference_loss: float,
                   rows: int, columns: int, enable: bool = True):
    """(beta, beta_view, Z, GHinv) with ``alpha_eff = alpha / (rows*columns)``; a
    non-positive alpha or a disabled update gives a single zero beta, hence Z = GHinv = 0
    (gptq_plus_utils.py:563-578)."""
    if enable and alpha > 0:
        beta, _ = safe_beta(grad_sub, hinv_init, reference_loss, alpha / (rows * columns))
    else:
        beta = torch.zeros([1], dtype=grad_sub.dtype)
    bview = beta.unsqueeze(1)
    Z = grad_sub.matmul(hinv.T) * bview
    return beta, bview, Z, Z.matmul(hinv)


# --------------------------------------------------------------------------------------
# plain GPTQ
# --------------------------------------------------------------------------------------
def plain_fasterquant(weight: torch.Tensor, H: torch.Tensor, quantizer, blocksize=128, percdamp=0.01,
                      groupsize=-1, actorder=False, static_groups=False):
    """Returns dict(Q, W_int, Scale, perm) for a plain-GPTQ linear (gptq_utils.py:45-174).

    ``Q`` is un-permuted like the layer weight the reference writes; ``W_int`` and
    ``Scale`` stay in the permuted column order, exactly as the reference registers
    them under ``export_to_et`` (:147-166).
    """
    W = weight.clone().float()
    Scale = weight.clone().float()
    W_int = weight.clone().float()
    columns = W.shape[1]
    if not quantizer.ready():
        quantizer.find_params(W)
    H = H.clone()
    if (H == 0).all():
        H = torch.eye(columns)
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0

    groups = None
    if static_groups:
        groups = []
        for i in range(0, columns, groupsize):
            q = copy.deepcopy(quantizer)
            q.find_params(W[:, i:i + groupsize])
            groups.append(q)

    perm = None
    if actorder:
        perm = torch.argsort(torch.diag(H), descending=True)
        W = W[:, perm]
        H = H[perm][:, perm]
        invperm = torch.argsort(perm)

    Q = torch.zeros_like(W)
    Hinv = plain_hinv(H, percdamp)

    for i1 in range(0, columns, blocksize):
        i2 = min(i1 + blocksize, columns)
        W1 = W[:, i1:i2].clone()
        Q1 = torch.zeros_like(W1)
        Wi1 = torch.zeros_like(W1)
        S1 = torch.zeros_like(W1)
        Err1 = torch.zeros_like(W1)
        Hinv1 = Hinv[i1:i2, i1:i2]
        for i in range(i2 - i1):
            w = W1[:, i]
            d = Hinv1[i, i]
            if groupsize != -1:
                if not static_groups:
                    if (i1 + i) % groupsize == 0:
                        quantizer.find_params(W[:, (i1 + i):(i1 + i + groupsize)])
                else:
                    idx = i1 + i
                    if actorder:
                        idx = perm[idx]
                    quantizer = groups[idx // groupsize]
            q, codes, scale = quantizer.fake_quantize(w.unsqueeze(1))
            q = q.flatten()
            Q1[:, i] = q
            Wi1[:, i] = codes.flatten()
            S1[:, i] = scale.flatten()
            err = (w - q) / d
            W1[:, i:] -= err.unsqueeze(1).matmul(Hinv1[i, i:].unsqueeze(0))
            Err1[:, i] = err
        Q[:, i1:i2] = Q1
        W_int[:, i1:i2] = Wi1
        Scale[:, i1:i2] = S1
        W[:, i2:] -= Err1.matmul(Hinv[i1:i2, i2:])

    if actorder:
        Q = Q[:, invperm]
    return {"Q": Q, "W_int": W_int, "Scale": Scale, "perm": perm, "Hinv": Hinv}


# --------------------------------------------------------------------------------------
# GPTQ+
# --------------------------------------------------------------------------------------
GD_DEFAULTS = dict(grad_lr=1e-3, grad_optimizer="sgd", curvature_damping=0.1, grad_reg_strategy="none",
                   grad_reg_lambda=0.0, grad_gate_floor=0.1, grad_gate_sharpness=1.0, grad_gate_sine_amp=0.0,
                   second_order_scale=1.0, grad_clip=1.0, slide_refresh_start=0, slide_refresh_block_total=None)


def validate_regularizer(gd):
    """gptq_plus_utils.py:666-686."""
    if gd["grad_reg_strategy"] not in ("none", "l2", "hessian", "quant_error_gate", "quant_error_gate_optimized"):
        raise ValueError(f"Unsupported `grad_reg_strategy={gd['grad_reg_strategy']}`.")
    if gd["grad_reg_lambda"] < 0 or gd["grad_gate_sharpness"] < 0 or gd["grad_gate_sine_amp"] < 0:
        raise ValueError("regulariser weights must be non-negative")
    if not 0.0 <= gd["grad_gate_floor"] <= 1.0:
        raise ValueError("`grad_gate_floor` must be in [0, 1]")


def input_curvature_diag(h_diag, damping):
    """Input-only KFAC diagonal of H-Adam (gptq_plus_utils.py:4601-4640 with output_fisher=None): the Hessian
    diagonal clamped at 0, normalised to unit mean, plus the damping; [1, C]."""
    a = h_diag.float().clamp_min(0.0)
    a = a / a.mean().clamp_min(1e-12)
    cur = a.view(1, -1)
    if damping and damping > 0:
        cur = cur + float(damping)
    return cur


def make_optimizer_state(w_sub, kind, curvature=None):
    """gptq_plus_utils.py:586-605."""
    if kind not in ("sgd", "adam", "h_adam"):
        raise ValueError(f"Unsupported `grad_optimizer={kind}`. Expected one of: sgd, adam, h_adam.")
    state = {"type": kind, "step": 0}
    if kind in ("adam", "h_adam"):
        state["m"] = torch.zeros_like(w_sub)
    if kind == "adam":
        state["v"] = torch.zeros_like(w_sub)
    if kind == "h_adam":
        if curvature is None:
            raise ValueError("h_adam requires the curvature diagonal")
        state["curvature"] = curvature
    return state


def clear_optimizer_state(state, c0, c1):
    """gptq_plus_utils.py:607-615."""
    if state is None or c1 <= c0:
        return
    if "m" in state:
        state["m"][:, c0:c1].zero_()
    if "v" in state:
        state["v"][:, c0:c1].zero_()


def optimizer_update(state, grad_sub, col_start, lr, grad_clip=1.0, b1=0.9, b2=0.999, eps=1e-8):
    """Step of the trailing columns (gptq_plus_utils.py:617-663): SGD, Adam, or Adam's first moment preconditioned
    by the fixed curvature diagonal."""
    g = grad_sub[:, col_start:]
    if g.numel() == 0:
        return g
    if grad_clip is not None and grad_clip > 0:
        g = g.clamp(min=-grad_clip, max=grad_clip)
    if state["type"] == "sgd":
        return lr * g
    state["step"] += 1
    m = state["m"][:, col_start:]
    m.mul_(b1).add_(g, alpha=1 - b1)
    bc1 = 1 - b1 ** state["step"]
    if state["type"] == "h_adam":
        denom = state["curvature"][:, col_start:].sqrt() + eps
        return (lr / bc1) * (m / denom)
    v = state["v"][:, col_start:]
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    bc2 = 1 - b2 ** state["step"]
    denom = v.sqrt() / math.sqrt(bc2)
    denom.add_(eps)
    return (lr / bc1) * (m / denom)


def gate_quant_maps(quantizer, w_sub, groupsize, r0, r1, groups=None, perm=None):
    """Per-element scale / zero of the grid each weight will be rounded to (gptq_plus_utils.py:688-722)."""
    gs, gz = torch.zeros_like(w_sub), torch.zeros_like(w_sub)
    if groupsize == -1:
        gs.copy_(quantizer.scale[r0:r1].expand_as(w_sub))
        gz.copy_(quantizer.zero[r0:r1].expand_as(w_sub))
        return gs, gz
    if groups is None:
        raise ValueError("`groups` must be provided when groupsize != -1.")
    ids = (torch.arange(w_sub.shape[1]) if perm is None else perm) // groupsize
    for gid, q in enumerate(groups):
        mask = ids == gid
        n = int(mask.sum())
        if n:
            gs[:, mask] = q.scale[r0:r1].expand(-1, n)
            gz[:, mask] = q.zero[r0:r1].expand(-1, n)
    return gs, gz


def regularized_update(st, current, raw, col_start, gd, maxq, sym):
    """First-order step after the regulariser (gptq_plus_utils.py:730-795)."""
    if raw.numel() == 0:
        return raw
    strategy, lr, lam = gd["grad_reg_strategy"], gd["grad_lr"], gd["grad_reg_lambda"]
    trailing = current[:, col_start:]
    if strategy == "none":
        return raw
    if strategy == "l2":
        return raw + lr * lam * (trailing - st["full_precision"][:, col_start:])
    if strategy == "hessian":
        return raw + lr * lam * (current - st["full_precision"]).matmul(st["hessian_reg"][:, col_start:])
    sc = st["gate_scale"][:, col_start:].clamp(min=1e-8)
    zr = st["gate_zero"][:, col_start:]
    if sym:
        nearest = sc * torch.clamp(torch.round(trailing / sc), -(maxq + 1), maxq)
    else:
        nearest = sc * (torch.clamp(torch.round(trailing / sc) + zr, 0, maxq) - zr)
    distance = (trailing - nearest).abs() / sc
    floor = gd["grad_gate_floor"]
    gate = floor + (1.0 - floor) * (1.0 - torch.exp(-gd["grad_gate_sharpness"] * distance))
    gated = raw * gate
    if strategy == "quant_error_gate":
        return gated
    phase = 2 * math.pi * (trailing / sc) if sym else 2 * math.pi * ((trailing / sc) + zr)
    sine = gd["grad_gate_sine_amp"] * (2 * math.pi / sc) * torch.sin(phase)
    return gated + lr * sine


def _effective_ghinv(base, cur_w, ref_w, bview, mode):
    """gptq_plus_utils.py:580-584."""
    if mode == "frozen":
        return base
    return base + bview * (cur_w - ref_w)


def plus_fasterquant(weight, H, act_square, gradients, quantizer, num_groups, alpha, reference_loss,
                     blocksize=128, percdamp=0.01, groupsize=-1, actorder=False, static_groups=False,
                     enable_gradient_update=True, g_update_mode="frozen", block_atomic_quant=False,
                     gradient_refresh_fn=None, gd=None, group_index_by_position=False):
    """GPTQ+ quantization of one linear (gptq_plus_utils.py:910-1896).  ``gd`` (g_update_mode="block_gd"): dict
    with grad_lr, grad_optimizer, curvature_damping, grad_reg_strategy, grad_reg_lambda, grad_gate_floor,
    grad_gate_sharpness, grad_gate_sine_amp, second_order_scale, grad_clip, slide_refresh_start,
    slide_refresh_block_total (the keyword arguments of the reference's fasterquant, :910-938).  ``H`` is the finalised ``[G, C, C]`` Hessian.  Returns dict(Q, W_int, Scale,
    perm, states) with all three matrices in the layer's natural column order (:1850-1866).
    """
    assert g_update_mode in ("frozen", "surrogate_block", "surrogate_online", "block_backward", "block_gd")
    backward = g_update_mode == "block_backward"
    gd_mode = g_update_mode == "block_gd"
    if gd_mode:
        gd = dict(GD_DEFAULTS, **(gd or {}))
        validate_regularizer(gd)
    so_scale = gd["second_order_scale"] if gd_mode else 1.0
    W = weight.clone().float()
    rows, columns = W.shape
    Q_final = torch.zeros_like(W)
    Wint_final = torch.zeros_like(W)
    Scale_final = torch.zeros_like(W)
    if not quantizer.ready():
        quantizer.find_params(W)

    dynamic_groups = groupsize != -1 and not static_groups
    if dynamic_groups and groupsize != blocksize:
        raise ValueError("`groupsize` must equal `blocksize` when using dynamic groups in GPTQ+.")

    shared_groups = None
    if groupsize != -1 and static_groups:                       # all rows, before dead-zeroing (:995-1002)
        shared_groups = []
        for c0 in range(0, columns, groupsize):
            q = copy.deepcopy(quantizer)
            q.find_params(W[:, c0:min(c0 + groupsize, columns)])
            shared_groups.append(q)

    fast = groupsize == -1 and quantizer.bits < 16 and quantizer.ready()
    maxq = int(quantizer.maxq)
    rps = rows // num_groups
    states = []
    for g in range(num_groups):
        r0, r1 = g * rps, (g + 1) * rps
        W_sub = W[r0:r1].clone()
        H_sub = H[g].clone()
        G_sub = gradients[r0:r1].float().clone()
        dead = torch.diag(H_sub) == 0
        H_sub[dead, dead] = 1
        W_sub[:, dead] = 0
        perm = invperm = None
        if actorder:
            perm = torch.argsort(act_square, descending=True)
            W_sub = W_sub[:, perm]
            H_sub = H_sub[perm][:, perm]
            G_sub = G_sub[:, perm]
            invperm = torch.argsort(perm)
        extra = {}
        if gd_mode:                                                        # :1052-1160
            strategy = gd["grad_reg_strategy"]
            if strategy in ("quant_error_gate", "quant_error_gate_optimized"):
                extra["gate_scale"], extra["gate_zero"] = gate_quant_maps(quantizer, W_sub, groupsize, r0, r1,
                                                                          shared_groups, perm)
            if strategy in ("l2", "hessian"):
                extra["full_precision"] = W_sub.clone()
            if strategy == "hessian":
                extra["hessian_reg"] = H_sub.clone()
            curvature = None
            if gd["grad_optimizer"] == "h_adam":
                curvature = input_curvature_diag(torch.diagonal(H_sub).clone(), gd["curvature_damping"])
            extra["opt"] = make_optimizer_state(W_sub, gd["grad_optimizer"], curvature)
        hinv_init, hinv, damp, ident = hinv_with_fallback(H_sub, percdamp)
        beta, bview, Z, GHinv = gradient_terms(G_sub, hinv_init, hinv, alpha, max(reference_loss, 0),
                                               rows, columns, enable_gradient_update)
        states.append(dict(extra, r0=r0, r1=r1, W_sub=W_sub, Hinv=hinv, Hinv_init=hinv_init, beta=beta, bview=bview,
                           Z=Z, GHinv=GHinv, anchor=W_sub.clone(), Q=torch.zeros_like(W_sub),
                           Wint=torch.zeros_like(W_sub), Scale=torch.zeros_like(W_sub), perm=perm,
                           invperm=invperm, damp=damp, identity=ident,
                           fast_scale=quantizer.scale[r0:r1] if fast else None))

    inner_mode = "surrogate_online" if backward else "frozen" if gd_mode else g_update_mode        # :1190
    outer_mode = "frozen" if g_update_mode in ("frozen", "block_backward", "block_gd") else "surrogate_block"   # :1500
    n_refresh_total = max((columns + blocksize - 1) // blocksize - 1, 0)
    for i1 in range(0, columns, blocksize):
        i2 = min(i1 + blocksize, columns)
        count = i2 - i1
        atomic = block_atomic_quant and not (i2 >= columns)
        D = torch.arange(count - 1, -1, -1).to(W)
        per_block = []
        for st in states:
            W1 = st["W_sub"][:, i1:i2].clone()
            Wref1 = st["anchor"][:, i1:i2]
            Wstart = W1.clone()
            Q1 = torch.zeros_like(W1)
            Wi1 = torch.zeros_like(W1)
            S1 = torch.zeros_like(W1)
            Err1 = torch.zeros_like(W1)
            Hinv1 = st["Hinv"][i1:i2, i1:i2]
            GH1 = st["GHinv"][:, i1:i2].clone()
            Z1 = st["Z"][:, i1:i2]
            online = inner_mode == "surrogate_online"
            GH1_eff = _effective_ghinv(GH1, W1 if online else Wstart, Wref1, st["bview"], inner_mode)
            dyn_q = None
            if dynamic_groups:
                dyn_q = copy.deepcopy(quantizer)
                dyn_q.find_params(Wstart)
            if st["fast_scale"] is not None:
                S1.copy_(st["fast_scale"].expand_as(S1))

            def column_quantizer(i):
                if dyn_q is not None:
                    return dyn_q, None, None
                if groupsize != -1:
                    idx = i1 + i
                    if actorder and not group_index_by_position:
                        idx = st["perm"][idx]
                    return shared_groups[idx // groupsize], st["r0"], st["r1"]
                return quantizer, st["r0"], st["r1"]

            if atomic:
                if groupsize == -1:
                    q, codes, scale = quantizer.fake_quantize(Wstart, st_idx=st["r0"], end_idx=st["r1"])
                    Q1.copy_(q)
                    Wi1.copy_(codes)
                    S1.copy_(scale.expand_as(Wstart))
                else:
                    for i in range(count):
                        qz, a, b = column_quantizer(i)
                        q, codes, scale = qz.fake_quantize(Wstart[:, i].unsqueeze(1), st_idx=a, end_idx=b)
                        Q1[:, i] = q.flatten()
                        Wi1[:, i] = codes.flatten()
                        S1[:, i] = scale.flatten()
                Err1.copy_(torch.linalg.solve_triangular(Hinv1.T, (Wstart - Q1 - GH1_eff).T, upper=False).T)
            else:
                for i in range(count):
                    w = W1[:, i]
                    d = Hinv1[i, i]
                    wc = w.unsqueeze(1)
                    if st["fast_scale"] is not None:
                        codes = torch.clamp(torch.round(wc / st["fast_scale"]), -(maxq + 1), maxq)
                        qf = (st["fast_scale"] * codes).to(wc.dtype)
                    else:
                        qz, a, b = column_quantizer(i)
                        qf, codes, scale = qz.fake_quantize(wc, st_idx=a, end_idx=b)
                        S1[:, i] = scale.flatten()
                    q = qf.flatten()
                    Q1[:, i] = q
                    Wi1[:, i] = codes.flatten()
                    err = (w - q - GH1_eff[:, i]) / d
                    inner = err.unsqueeze(1).matmul(Hinv1[i, i:].unsqueeze(0))
                    if gd_mode:                                                    # :1344-1349
                        W1[:, i:] -= so_scale * (inner + GH1_eff[:, i:])
                    else:
                        W1[:, i:] -= inner + GH1_eff[:, i:]
                    Err1[:, i] = err
                    GH1[:, i:].sub_(Z1[:, i].unsqueeze(1).matmul(Hinv1[i, i:].unsqueeze(0)))
                    if inner_mode != "frozen":
                        GH1_eff = _effective_ghinv(GH1, W1 if online else Wstart, Wref1, st["bview"], inner_mode)
            st["Q"][:, i1:i2] = Q1
            st["Wint"][:, i1:i2] = Wi1
            st["Scale"][:, i1:i2] = S1
            cur = None
            if backward:                                                  # :1392-1396
                cur = st["W_sub"].clone()
                cur[:, :i1] = st["Q"][:, :i1]
                cur[:, i1:i2] = Q1
            per_block.append([st, Err1, Z1, cur])

        if backward and enable_gradient_update:                           # true-gradient refresh (:1408-1460)
            snapshot = weight.clone().float()
            for st, _, _, cur in per_block:
                snapshot[st["r0"]:st["r1"]] = cur[:, st["invperm"]] if actorder else cur
            refreshed, _meta = gradient_refresh_fn(snapshot)
            refreshed = refreshed.float()
            for item in per_block:
                st, cur = item[0], item[3]
                g_sub = refreshed[st["r0"]:st["r1"]]
                if actorder:
                    g_sub = g_sub[:, st["perm"]]
                beta, bview, Z, GHinv = gradient_terms(g_sub, st["Hinv_init"], st["Hinv"], alpha,
                                                       max(reference_loss, 0), rows, columns, enable_gradient_update)
                st.update(beta=beta, bview=bview, Z=Z, GHinv=GHinv, anchor=cur.clone())
                item[2] = Z[:, i1:i2]

        for st, Err1, Z1, _ in per_block:                                 # lazy update (:1500-1570)
            rest = _effective_ghinv(st["GHinv"][:, i2:], st["W_sub"][:, i2:], st["anchor"][:, i2:],
                                    st["bview"], outer_mode)
            g_update = count * rest - torch.einsum("ij,j,jk->ik", Z1, D, st["Hinv"][i1:i2, i2:])
            second = Err1.matmul(st["Hinv"][i1:i2, i2:])
            if gd_mode:                                                           # :1546-1550
                st["W_sub"][:, i2:] -= so_scale * (second + g_update)
            else:
                st["W_sub"][:, i2:] -= second + g_update
            st["GHinv"][:, i2:] -= st["Z"][:, i1:i2].matmul(st["Hinv"][i1:i2, i2:])
            if gd_mode:
                clear_optimizer_state(st["opt"], i1, i2)

        if gd_mode and enable_gradient_update and i2 < columns:                   # :1572-1848
            if gradient_refresh_fn is None:
                raise ValueError("`gradient_refresh_fn` must be provided for g_update_mode='block_gd'.")
            snapshot = weight.clone().float()
            for st in states:
                cur = st["W_sub"].clone()
                cur[:, :i2] = st["Q"][:, :i2]
                snapshot[st["r0"]:st["r1"]] = cur[:, st["invperm"]] if actorder else cur
            total = gd["slide_refresh_block_total"] if gd["slide_refresh_block_total"] is not None else n_refresh_total
            idx = gd["slide_refresh_start"] + i1 // blocksize
            slide_alpha = 1.0 - idx / max(total - 1, 1) if total > 1 else 1.0
            refreshed, _meta = gradient_refresh_fn(snapshot, slide_alpha=slide_alpha)
            refreshed = refreshed.float()
            for st in states:
                g_sub = refreshed[st["r0"]:st["r1"]]
                if actorder:
                    g_sub = g_sub[:, st["perm"]]
                cur = st["W_sub"].clone()
                cur[:, :i2] = st["Q"][:, :i2]
                raw = optimizer_update(st["opt"], g_sub, i2, gd["grad_lr"], gd["grad_clip"])
                upd = regularized_update(st, cur, raw, i2, gd, maxq, quantizer.sym)
                st["pending"] = upd
            for st in states:
                upd = st.pop("pending")
                if upd.numel() > 0:
                    st["W_sub"][:, i2:] -= upd

    for st in states:
        Qs, Wi, Sc = st["Q"], st["Wint"], st["Scale"]
        if actorder:
            Qs, Wi, Sc = Qs[:, st["invperm"]], Wi[:, st["invperm"]], Sc[:, st["invperm"]]
        Q_final[st["r0"]:st["r1"]] = Qs
        Wint_final[st["r0"]:st["r1"]] = Wi
        Scale_final[st["r0"]:st["r1"]] = Sc
    return {"Q": Q_final, "W_int": Wint_final, "Scale": Scale_final,
            "perm": states[0]["perm"], "states": states}


def guided_fasterquant(weight, H_ccg, act_square, quantizer, num_groups, blocksize=128, percdamp=0.01,
                       groupsize=-1, actorder=False, static_groups=False):
    """GPTQGuided.fasterquant (gptq_guided_utils.py:86-259): the GPTQ+ loop without first-order terms on the raw
    Hessian sums ``H_ccg`` [C, C, G]; damping failures raise instead of falling back to the identity."""
    H = H_ccg.permute(2, 0, 1).contiguous()
    for g in range(num_groups):
        if bool((H[g] == 0).all()):
            H[g] = torch.eye(H.shape[-1])
    by_position = False
    if groupsize != -1 and not static_groups and actorder:
        # :186-191 under act_order: W_sub is a permuted COPY, so find_params(W[:, pos:pos+groupsize]) ranges the
        # original (dead-zeroed, un-permuted, never updated) columns at the POSITION being quantized: static ranges
        # looked up by position instead of by the permuted column's own index
        weight = weight.clone().float()
        rps = weight.shape[0] // num_groups
        for g in range(num_groups):
            dead = torch.diag(H[g]) == 0
            weight[g * rps:(g + 1) * rps][:, dead] = 0
        static_groups, by_position = True, True
    out = plus_fasterquant(weight, H, act_square, torch.zeros_like(weight, dtype=torch.float32), quantizer,
                           num_groups, 0.0, 0.0, blocksize=blocksize, percdamp=percdamp, groupsize=groupsize,
                           actorder=actorder, static_groups=static_groups, enable_gradient_update=False,
                           group_index_by_position=by_position)
    if any(st["identity"] for st in out["states"]):
        raise ValueError("Quantization: `damp_percent` must between 0 and 1.")
    return out


# --------------------------------------------------------------------------------------
# GPTAQ
# --------------------------------------------------------------------------------------
class AsymCalibState:
    """H and dXXT of GPTAQ.add_batch (gptaq_utils.py:14-41): running means over sequences of (2/n) X^T X and
    (2/n) (X_fp - X)^T X."""

    def __init__(self, columns):
        self.H = torch.zeros(columns, columns)
        self.dXXT = torch.zeros(columns, columns)
        self.nsamples = 0

    def add_batch(self, inp, fp_inp):
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        tmp = inp.shape[0]
        inp = inp.reshape(-1, inp.shape[-1]).t()
        self.H *= self.nsamples / (self.nsamples + tmp)
        self.dXXT *= self.nsamples / (self.nsamples + tmp)
        self.nsamples += tmp
        inp = math.sqrt(2 / self.nsamples) * inp.float()
        self.H += inp.matmul(inp.t())
        dX = fp_inp.float() * math.sqrt(2 / self.nsamples) - inp       # fp_inp: [C, tokens]
        self.dXXT += dX.matmul(inp.t())


def gptaq_fasterquant(weight, H, dXXT, quantizer, blocksize=128, percdamp=0.01, groupsize=-1, actorder=False,
                      static_groups=False, alpha=0.25):
    """GPTAQ.fasterquant (gptaq_utils.py:43-167): dict(Q, perm, P)."""
    W = weight.clone().float()
    columns = W.shape[1]
    if not quantizer.ready():
        quantizer.find_params(W)
    H = H.clone()
    dXXT = dXXT.clone()
    if (H == 0).all():
        H = torch.eye(columns)
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    dXXT[:, dead] = 0
    groups = None
    if static_groups:
        groups = []
        for i in range(0, columns, groupsize):
            q = copy.deepcopy(quantizer)
            q.find_params(W[:, i:(i + groupsize)])
            groups.append(q)
    perm = invperm = None
    if actorder:
        perm = torch.argsort(torch.diag(H), descending=True)
        W = W[:, perm]
        H = H[perm][:, perm]
        dXXT = dXXT[perm][:, perm]
        invperm = torch.argsort(perm)
    Q = torch.zeros_like(W)
    Hinv = plain_hinv(H, percdamp)
    P = alpha * ((dXXT @ Hinv.T).triu_(diagonal=1)) @ Hinv
    for i1 in range(0, columns, blocksize):
        i2 = min(i1 + blocksize, columns)
        count = i2 - i1
        W1 = W[:, i1:i2].clone()
        Q1 = torch.zeros_like(W1)
        Err1 = torch.zeros_like(W1)
        Hinv1 = Hinv[i1:i2, i1:i2]
        P1 = P[i1:i2, i1:i2]
        for i in range(count):
            w = W1[:, i]
            d = Hinv1[i, i]
            qz = quantizer
            if groupsize != -1:
                if not static_groups:                                   # :126-131, on the working matrix
                    if (i1 + i) % groupsize == 0:
                        quantizer.find_params(W[:, (i1 + i):(i1 + i + groupsize)])
                else:
                    idx = i1 + i
                    if actorder:
                        idx = perm[idx]
                    qz = groups[idx // groupsize]
            q = qz.quantize(w.unsqueeze(1)).flatten()
            Q1[:, i] = q
            err1 = (w - q) / d
            W1[:, i:] -= err1.unsqueeze(1).matmul(Hinv1[i, i:].unsqueeze(0)) - w.unsqueeze(1).matmul(P1[i, i:].unsqueeze(0))
            Err1[:, i] = err1
        Q[:, i1:i2] = Q1
        W[:, i2:] -= Err1.matmul(Hinv[i1:i2, i2:]) - W1.matmul(P[i1:i2, i2:])
    if actorder:
        Q = Q[:, invperm]
    return {"Q": Q, "perm": perm, "P": P}
