"""Diagnostics of ``GPTQPlus``: summaries of the first-order term ``G . H^-1`` and of the weight drift before, inside
and after the blocks of a dry run of the column loop (gptq_plus_utils.py:1898-2367 of the reference: the methods
``analyze_ghinv_dynamics``, ``summarize_ghinv`` and ``summarize_weight_delta``).  They return nested dicts of
Python floats and change nothing: the layer, the Hessian and the quantizer's per-row ranges stay as they are.

None of this is on a timed path.  The damped inverse factor comes from the library (``rq_chol_hinv`` through
``fasterquant_impl.hinv_with_fallback``) and beta / Z / GHinv from ``rq_gptqplus_terms``; the dry run itself is the
reference's own formulation, a per-column loop of small torch operations on the device, because what it reports are
the intermediate states that the fused block kernel keeps in registers.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..utils import quant_utils
from . import fasterquant_impl as fi


def _rows(t: torch.Tensor):
    """Row-norm statistics of a matrix (None when it is empty)."""
    if t.numel() == 0:
        return None
    t = t.float()
    norms = torch.linalg.norm(t, dim=1)
    return {"mean_row_l2": norms.mean().item(), "median_row_l2": norms.median().item(),
            "max_row_l2": norms.max().item(), "fro_norm": torch.linalg.norm(t).item(),
            "abs_mean": t.abs().mean().item()}


def _vector(v: torch.Tensor):
    v = v.float().flatten()
    return {"mean": v.mean().item(), "median": v.median().item(), "min": v.min().item(), "max": v.max().item()}


def selected_column_count(obj, blocksize, max_blocks):
    """gptq_plus_utils.py:489-492."""
    return obj.columns if max_blocks is None else min(obj.columns, max_blocks * blocksize)


def _first_order_state(obj, sub_idx, grads_sub, perm, percdamp, enable, reference_loss, context):
    """Inverse factor U (upper, Hinv = U^T U) of sub-group ``sub_idx`` in the permuted column order, the raw terms
    ``Z_raw = G U^T`` and ``GHinv_raw = Z_raw U`` and, scaled by the safe step beta, Z and GHinv
    (gptq_plus_utils.py:174-194, 563-578).  ``grads_sub`` is already permuted."""
    dev = obj.dev
    Cc = obj.columns
    H3 = obj.H[sub_idx:sub_idx + 1].contiguous()
    Hinv, _, identity = fi.hinv_with_fallback(H3, perm, percdamp, identity_fallback=True, log_context=context)
    U = Hinv[0, :Cc, :Cc]
    Z_raw = grads_sub @ U.t()
    GH_raw = Z_raw @ U
    rps = grads_sub.shape[0]
    if enable and obj.alpha > 0:
        Gp = grads_sub.contiguous()
        Z = torch.empty_like(Gp)
        GH = torch.empty_like(Gp)
        beta = torch.empty(rps, dtype=torch.float32, device=dev)
        hdiag = torch.empty(1, Cc, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check("rq_gptqplus_terms",
                       _lib.lib.rq_gptqplus_terms(_lib.ptr(Gp), _lib.ptr(Hinv), rps, Cc, 1,
                                                  float(obj.alpha / (obj.rows * obj.columns)), float(reference_loss),
                                                  _lib.ptr(Z), _lib.ptr(GH), _lib.ptr(beta), _lib.ptr(hdiag),
                                                  _lib.stream_of(Gp)))
    else:
        beta = torch.zeros(1, dtype=torch.float32, device=dev)
        Z = torch.zeros_like(Z_raw)
        GH = torch.zeros_like(GH_raw)
    return U, bool(identity[0]), beta, Z, GH, Z_raw, GH_raw


def _dead_columns(obj, sub_idx):
    return torch.diagonal(obj.H[sub_idx]) == 0


@torch.no_grad()
def summarize_weight_delta(obj, blocksize=128, actorder=False, max_subgroups=None, max_blocks=None,
                           ref_weight_override=None, weight_override=None, return_tensors=False):
    """gptq_plus_utils.py:2295-2347."""
    current = obj.layer.weight.data.float() if weight_override is None else weight_override.float()
    reference = current if ref_weight_override is None else ref_weight_override.float()
    rps = obj.rows // obj.num_groups
    ncols = selected_column_count(obj, blocksize, max_blocks)
    order = torch.argsort(obj.act_square, descending=True) if actorder else None
    out = {"rows": obj.rows, "columns": obj.columns, "num_groups": obj.num_groups, "subgroups": []}
    kept = []
    for g in range(obj.num_groups if max_subgroups is None else min(obj.num_groups, max_subgroups)):
        delta = current[g * rps:(g + 1) * rps] - reference[g * rps:(g + 1) * rps]
        if order is not None:
            delta = delta[:, order.to(delta.device)]
        delta = delta[:, :ncols]
        out["subgroups"].append({"sub_idx": g, "row_start": g * rps, "row_end": (g + 1) * rps,
                                 "weight_delta": _rows(delta)})
        if return_tensors:
            kept.append({"sub_idx": g, "weight_delta": delta.detach().cpu()})
    if return_tensors:
        out["_tensor_cache"] = kept
    return out


@torch.no_grad()
def summarize_ghinv(obj, percdamp=0.01, blocksize=128, actorder=False, enable_gradient_update=True,
                    gradient_override=None, reference_loss_override=None, max_subgroups=None, max_blocks=None,
                    return_tensors=False):
    """gptq_plus_utils.py:2179-2293: G . H^-1 of every sub-group, raw and scaled by beta, dead input channels
    taken out of the gradient."""
    grads = obj.gradients if gradient_override is None else gradient_override.float()
    ref_loss = obj.reference_loss if reference_loss_override is None else max(float(reference_loss_override), 0.0)
    rps = obj.rows // obj.num_groups
    ncols = selected_column_count(obj, blocksize, max_blocks)
    perm = torch.argsort(obj.act_square, descending=True) if actorder else None
    out = {"rows": obj.rows, "columns": obj.columns, "num_groups": obj.num_groups,
           "enable_gradient_update": bool(enable_gradient_update), "subgroups": []}
    kept = []
    for g in range(obj.num_groups if max_subgroups is None else min(obj.num_groups, max_subgroups)):
        gsub = grads[g * rps:(g + 1) * rps].to(obj.dev).float().clone()
        gsub[:, _dead_columns(obj, g)] = 0
        if perm is not None:
            gsub = gsub[:, perm]
        _, identity, beta, _, GH, _, GH_raw = _first_order_state(
            obj, g, gsub, perm, percdamp, enable_gradient_update, ref_loss, f" summarize_ghinv subgroup={g}")
        out["subgroups"].append({"sub_idx": g, "row_start": g * rps, "row_end": (g + 1) * rps,
                                 "hessian_identity_fallback": identity, "beta": _vector(beta),
                                 "raw_ghinv": _rows(GH_raw[:, :ncols]), "ghinv": _rows(GH[:, :ncols])})
        if return_tensors:
            kept.append({"sub_idx": g, "raw_ghinv": GH_raw[:, :ncols].detach().cpu(),
                         "ghinv": GH[:, :ncols].detach().cpu()})
    if return_tensors:
        out["_tensor_cache"] = kept
    return out


@torch.no_grad()
def analyze_ghinv_dynamics(obj, blocksize=128, percdamp=0.01, groupsize=-1, actorder=False, static_groups=False,
                           enable_gradient_update=True, g_update_mode="frozen", max_subgroups=None, max_blocks=None,
                           return_tensors=False):
    """gptq_plus_utils.py:1898-2177: a dry run of the GPTQ+ column loop that records, block by block, the size of the
    first-order term (as used, ``beta``-scaled, and raw), of the quantization errors and of the drift of the working
    weights from their start values.  Nothing is written back to the layer.

    Quirks of the reference that are kept because the numbers depend on them: the outer update uses ``blocksize`` (not
    the length of a ragged last block) as the count in front of GHinv; dynamic groups are ranged from the layer's
    untouched weight, in natural column order."""
    dev = obj.dev
    W = obj.layer.weight.data.clone().float()
    quantizer = obj.quantizer
    if not quantizer.ready():
        quantizer.find_params(W)
    maxq = int(quantizer.maxq)
    rps = obj.rows // obj.num_groups
    Cc = obj.columns
    perm = torch.argsort(obj.act_square, descending=True) if actorder else None
    ncols = selected_column_count(obj, blocksize, max_blocks)
    surrogate = g_update_mode != "frozen"
    online = g_update_mode == "surrogate_online"
    row_scale = quantizer.scale.to(dev, torch.float32).reshape(-1) if groupsize == -1 else None
    static_tab = None
    if groupsize != -1 and static_groups:
        static_tab, _ = quant_utils.find_params_groups(W, groupsize, maxq, quantizer.sym, quantizer.mse,
                                                       quantizer.norm, quantizer.grid, quantizer.maxshrink)
    out = {"rows": obj.rows, "columns": Cc, "num_groups": obj.num_groups, "blocksize": blocksize,
           "g_update_mode": g_update_mode, "enable_gradient_update": bool(enable_gradient_update), "subgroups": []}
    kept = []
    D = torch.arange(blocksize - 1, -1, -1, device=dev, dtype=torch.float32)

    def code(w, scale):
        return scale * torch.clamp(torch.round(w / scale), -(maxq + 1), maxq)

    for g in range(obj.num_groups if max_subgroups is None else min(obj.num_groups, max_subgroups)):
        r0, r1 = g * rps, (g + 1) * rps
        Wsub = W[r0:r1].clone()
        Wsub[:, _dead_columns(obj, g)] = 0
        gsub = obj.gradients[r0:r1].to(dev).float().clone()
        if perm is not None:
            Wsub = Wsub[:, perm]
            gsub = gsub[:, perm]
        U, identity, beta, Z, GH, Z_raw, GH_raw = _first_order_state(
            obj, g, gsub, perm, percdamp, enable_gradient_update, obj.reference_loss,
            f" analyze_ghinv_dynamics subgroup={g}")
        bcol = beta.unsqueeze(1)
        Wref = Wsub.clone()

        def eff(base, cur, ref, mode, raw=False):
            if mode == "frozen":
                return base
            return base + (cur - ref) if raw else base + bcol * (cur - ref)

        outer_mode = "frozen" if not surrogate else "surrogate_block"
        sub = {"sub_idx": g, "row_start": r0, "row_end": r1, "hessian_identity_fallback": identity,
               "beta": _vector(beta), "initial_raw_ghinv": _rows(GH_raw[:, :ncols]),
               "initial_ghinv": _rows(GH[:, :ncols]), "blocks": []}
        dyn_scale = None
        for i1 in range(0, Cc, blocksize):
            if max_blocks is not None and i1 // blocksize >= max_blocks:
                break
            i2 = min(i1 + blocksize, Cc)
            W1 = Wsub[:, i1:i2].clone()
            Wref1 = Wref[:, i1:i2]
            Wstart = W1.clone()
            Err1 = torch.zeros_like(W1)
            U1 = U[i1:i2, i1:i2]
            G1, G1raw = GH[:, i1:i2].clone(), GH_raw[:, i1:i2].clone()
            Z1, Z1raw = Z[:, i1:i2], Z_raw[:, i1:i2]
            anchor = (lambda: W1) if online else (lambda: Wstart)
            G1eff = eff(G1, anchor(), Wref1, g_update_mode)
            G1eff_raw = eff(G1raw, anchor(), Wref1, g_update_mode, raw=True)
            blk = {"block_idx": i1 // blocksize, "col_start": i1, "col_end": i2,
                   "base_raw_ghinv_before": _rows(GH_raw[:, i1:i2]), "eff_raw_ghinv_before": _rows(G1eff_raw),
                   "base_ghinv_before": _rows(GH[:, i1:i2]), "eff_ghinv_before": _rows(G1eff),
                   "weight_delta_before": _rows(W1 - Wref1)}
            for i in range(i2 - i1):
                col = i1 + i
                if groupsize == -1:
                    scale = row_scale[r0:r1]
                elif static_groups:
                    src = int(perm[col]) if perm is not None else col
                    scale = static_tab[src // groupsize, r0:r1]
                else:
                    if col % groupsize == 0:
                        tab, _ = quant_utils.find_params_groups(W[:, col:col + groupsize].contiguous(), groupsize, maxq,
                                                                quantizer.sym, quantizer.mse, quantizer.norm,
                                                                quantizer.grid, quantizer.maxshrink)
                        dyn_scale = tab[0]
                    scale = dyn_scale[r0:r1]
                w = W1[:, i]
                err = (w - code(w, scale) - G1eff[:, i]) / U1[i, i]
                W1[:, i:] -= err.unsqueeze(1) * U1[i, i:].unsqueeze(0) + G1eff[:, i:]
                Err1[:, i] = err
                G1[:, i:] -= Z1[:, i].unsqueeze(1) * U1[i, i:].unsqueeze(0)
                G1raw[:, i:] -= Z1raw[:, i].unsqueeze(1) * U1[i, i:].unsqueeze(0)
                G1eff = eff(G1, anchor(), Wref1, g_update_mode)
                G1eff_raw = eff(G1raw, anchor(), Wref1, g_update_mode, raw=True)
            blk["eff_raw_ghinv_after_inner"] = _rows(G1eff_raw)
            blk["eff_ghinv_after_inner"] = _rows(G1eff)
            blk["err_after_inner"] = _rows(Err1)
            blk["weight_delta_after_inner"] = _rows(W1 - Wref1)
            rest = eff(GH[:, i2:], Wsub[:, i2:], Wref[:, i2:], outer_mode)
            blk["trailing_eff_raw_ghinv_before"] = _rows(eff(GH_raw[:, i2:], Wsub[:, i2:], Wref[:, i2:], outer_mode, raw=True))
            blk["trailing_eff_ghinv_before"] = _rows(rest)
            far = U[i1:i2, i2:]
            Wsub[:, i2:] -= Err1 @ far + (blocksize * rest - (Z1 * D[:i2 - i1]) @ far)
            GH[:, i2:] -= Z1 @ far
            GH_raw[:, i2:] -= Z1raw @ far
            blk["trailing_eff_raw_ghinv_after"] = _rows(eff(GH_raw[:, i2:], Wsub[:, i2:], Wref[:, i2:], outer_mode, raw=True))
            blk["trailing_eff_ghinv_after"] = _rows(eff(GH[:, i2:], Wsub[:, i2:], Wref[:, i2:], outer_mode))
            sub["blocks"].append(blk)
        final_raw = eff(GH_raw, Wsub, Wref, outer_mode, raw=True)
        sub["final_weight_delta"] = _rows(Wsub - Wref)
        sub["final_raw_eff_ghinv"] = _rows(final_raw[:, :ncols])
        sub["final_base_ghinv"] = _rows(GH[:, :ncols])
        sub["final_eff_ghinv"] = _rows(eff(GH, Wsub, Wref, outer_mode)[:, :ncols])
        out["subgroups"].append(sub)
        if return_tensors:
            # the reference files the raw base term under "initial" after the loop has updated it in place
            kept.append({"sub_idx": g, "initial_raw_ghinv": GH_raw[:, :ncols].detach().cpu(),
                         "final_raw_eff_ghinv": final_raw[:, :ncols].detach().cpu()})
    if return_tensors:
        out["_tensor_cache"] = kept
    return out
