"""Host side of ``fasterquant`` for the ``GPTQ`` and ``GPTQPlus`` objects: sets up the work
matrices, drives the damping-retry loop around the Cholesky kernel and launches the block loop.
All numerical work happens in the kernels of ``librealq_b200.so``; torch supplies the memory,
the ``argsort`` of the act_order key and the stream."""
from __future__ import annotations

import ctypes
import logging
import math
import os
from contextlib import nullcontext

import torch

from .. import _lib, ops
from ..utils import quant_utils

_NULL = nullcontext()


def _sec(rec, name):
    """Section of the caller's profile recorder (the reference's QuantProfileRecorder.section names)."""
    return rec.section(name) if rec is not None else _NULL


BS = 128            # column block of the kernels
_DAMP_STEP = 0.0015
# the factorisation of all groups of a linear shares its launches when their scratch fits this many bytes;
# beyond it (28672-wide inputs with four groups need 79 GB at once) the groups are factorised in smaller batches
CHOL_WORKSPACE_CAP = int(float(os.environ.get("REALQ_CHOL_WORKSPACE_GB", "32")) * (1 << 30))
# GEMM-shaped parts (first-order terms, lazy update) on the tensor cores (split-bf16, four products) or,
# when False, as fp32 FMA tiles on the CUDA cores
USE_TENSOR_CORES = os.environ.get("REALQ_FQ_TENSOR", "1") != "0"
# tests set this to keep a copy of the first-order term as it is before the block loop updates it in place
KEEP_INTERMEDIATES = False


# ----------------------------------------------------------------------------------------------
# damped inverse factor with the reference's retry semantics
# ----------------------------------------------------------------------------------------------
# flag of rq_chol_hinv_flags: bf16 operand planes throughout (REALQ_CHOL_BF16=1 forces it for every call)
CHOL_BF16_ONLY = 1
_CHOL_FLAGS = CHOL_BF16_ONLY if os.environ.get("REALQ_CHOL_BF16", "0") != "0" else 0


def _chol_once(H3: torch.Tensor, perm, factors, Hinv: torch.Tensor, info: torch.Tensor, flags: int | None = None) -> None:
    flags = _CHOL_FLAGS if flags is None else flags
    G, Cc = H3.shape[0], H3.shape[-1]
    need = _lib.lib.rq_chol_workspace_bytes(Cc, G)
    ws = ops._workspace(H3.device, need + 256)
    base = ws.data_ptr()
    aligned = (base + 255) // 256 * 256
    arr = (ctypes.c_float * G)(*[float(f) for f in factors])
    with torch.cuda.device(H3.device):
        rc = _lib.lib.rq_chol_hinv_flags(_lib.ptr(H3), _lib.ptr(perm), arr, _lib.ptr(Hinv), Cc, G, _lib.ptr(info),
                                         aligned, ws.numel() - (aligned - base), int(flags), _lib.stream_of(H3))
    _lib.check("rq_chol_hinv_flags", rc)


def hinv_with_fallback(H3: torch.Tensor, perm, percdamp: float, identity_fallback: bool, log_context: str = ""):
    """``Hinv`` [G, Cp, Cp] (upper factor of the damped inverse of every group), the damping
    fraction each group ended with, and which groups fell back to the identity.

    Retry rule of the reference (gptq_plus_utils.py:519-557, gptq_utils.py:88-106): the damping
    ``p * mean(diag)`` is added to the already-damped matrix, so after attempts p_1..p_k the
    diagonal has grown by ``mean(diag) * (prod(1 + p_i) - 1)``; p grows by 0.0015 per failure;
    at p >= 1 GPTQ+ substitutes the identity while plain GPTQ raises ValueError."""
    if float(percdamp) <= 0:
        raise ValueError(f"Quantization{log_context}: `damp_percent` must be positive. current is {percdamp}")
    G, Cc = H3.shape[0], H3.shape[-1]
    Cp = (Cc + BS - 1) // BS * BS
    Hinv = torch.empty(G, Cp, Cp, dtype=torch.float32, device=H3.device)
    info = torch.zeros(G, dtype=torch.int32, device=H3.device)
    p = [float(percdamp)] * G
    growth = [1.0] * G                                  # prod(1 + p_i) over the attempts so far
    identity = [False] * G
    pending = list(range(G))
    first = True
    while pending:
        todo = [g for g in pending if 0 < p[g] < 1]
        for g in pending:
            if g not in todo:
                identity[g] = True
        if not todo:
            break
        for g in todo:
            growth[g] *= 1.0 + p[g]
        if first and len(todo) == G:
            batch = G
            while batch > 1 and _lib.lib.rq_chol_workspace_bytes(Cc, batch) > CHOL_WORKSPACE_CAP:
                batch = (batch + 1) // 2
            for g0 in range(0, G, batch):
                g1 = min(G, g0 + batch)
                _chol_once(H3[g0:g1], perm, [growth[g] - 1.0 for g in range(g0, g1)], Hinv[g0:g1], info[g0:g1])
            flags = info.tolist()
            # a non-finite result of the fp16-plane route may be an overflowed intermediate of the inverse rather
            # than a failed factorisation: those groups get one more try with bf16 planes at the same damping
            for g in [g for g in range(G) if flags[g] == -1 and _CHOL_FLAGS == 0]:
                sub = torch.zeros(1, dtype=torch.int32, device=H3.device)
                _chol_once(H3[g:g + 1], perm, [growth[g] - 1.0], Hinv[g:g + 1], sub, flags=CHOL_BF16_ONLY)
                flags[g] = int(sub.item())
        else:
            flags = [0] * G
            for g in todo:
                sub = torch.zeros(1, dtype=torch.int32, device=H3.device)
                _chol_once(H3[g:g + 1], perm, [growth[g] - 1.0], Hinv[g:g + 1], sub)
                flags[g] = int(sub.item())
                if flags[g] == -1 and _CHOL_FLAGS == 0:
                    _chol_once(H3[g:g + 1], perm, [growth[g] - 1.0], Hinv[g:g + 1], sub, flags=CHOL_BF16_ONLY)
                    flags[g] = int(sub.item())
        first = False
        pending = []
        if any(flags[g] == -2 for g in todo):
            raise _lib.RealQError("rq_chol_hinv (device wait)", _lib.RQ_ERR_TIMEOUT)
        for g in todo:
            if flags[g] != 0:
                logging.warning("Quantization%s: Current `damp_percent = %.5f` is too low, auto-incrementing by `%.5f`",
                                f"{log_context} subgroup={g}", p[g], _DAMP_STEP)
                p[g] += _DAMP_STEP
                pending.append(g)
    for g in range(G):
        if identity[g]:
            if not identity_fallback:
                raise ValueError(f"Quantization: `damp_percent` must between 0 and 1. current is {p[g]}")
            logging.warning("Quantization%s subgroup=%d: `damp_percent` reached %.5f; falling back to identity "
                            "Hessian inverse for this subgroup.", log_context, g, p[g])
            Hinv[g].zero_()
            Hinv[g].diagonal().fill_(1.0)
    return Hinv, p, identity


# ----------------------------------------------------------------------------------------------
# scale sources
# ----------------------------------------------------------------------------------------------
def _scale_setup(quantizer, W32, groupsize, static_groups, blocksize, perm, dead_zeroed_W=None, rows=None):
    """(mode, scale_row, scale_tab, colgrp, scale_blk, dyn_gs) for the block kernel; ``rows`` restricts
    it to a row slice of the layer (every scale is per row, so a slice is a problem of its own)."""
    dev = W32.device
    if groupsize == -1:
        scale_row = quantizer.scale.to(dev, torch.float32).reshape(-1).contiguous()
        if scale_row.numel() != W32.shape[0]:
            raise ValueError(f"quantizer.scale has {scale_row.numel()} entries for {W32.shape[0]} rows")
        if rows is not None:
            scale_row = scale_row[rows].contiguous()
        return 0, scale_row, None, None, None, 0
    if rows is not None:
        W32 = W32[rows]
        dead_zeroed_W = None if dead_zeroed_W is None else dead_zeroed_W[rows]
    R, Cc = W32.shape
    if not getattr(quantizer, "perchannel", True):
        raise NotImplementedError("grouped quantization needs a per-channel quantizer")
    maxq = int(quantizer.maxq)
    if static_groups:
        src = W32 if dead_zeroed_W is None else dead_zeroed_W
        tab, _ = quant_utils.find_params_groups(src, groupsize, maxq, quantizer.sym, quantizer.mse, quantizer.norm,
                                                quantizer.grid, quantizer.maxshrink)
        cols = perm if perm is not None else torch.arange(Cc, device=dev)
        colgrp = (cols // groupsize).to(torch.int32).contiguous()
        return 1, None, tab, colgrp, None, 0
    # dynamic groups: ranged from the working matrix as it is at the start of the block a group begins in
    # (gptq_utils/gptq_utils.py:123-128; gptq_plus_utils.py:1205-1209).  The kernels' block is 128 columns wide, so
    # that state is reproduced when the reference's block is 128 wide too, or when every group starts at one of
    # the reference's own block boundaries.
    if blocksize != BS and groupsize % blocksize != 0:
        raise NotImplementedError(
            f"dynamic weight groups are ranged from the weights at the start of the reference's block: blocksize "
            f"must be {BS} or divide groupsize; got groupsize={groupsize}, blocksize={blocksize} (use static groups)")
    ng = (Cc + groupsize - 1) // groupsize
    colgrp = (torch.arange(Cc, device=dev) // groupsize).to(torch.int32).contiguous()
    if BS % groupsize == 0 and not quantizer.mse:
        scale_blk = torch.zeros(ng, R, dtype=torch.float32, device=dev)        # ranged inside the block kernel
        return 2, None, None, colgrp, scale_blk, groupsize
    # wider than a block, not a divisor of it, or with the shrink-grid search: the host ranges every group between
    # two block launches (mode 3 = a table indexed by position that fills up as the blocks go by)
    tab = torch.zeros(ng, R, dtype=torch.float32, device=dev)
    return 3, None, tab, colgrp, None, groupsize


# ----------------------------------------------------------------------------------------------
# the shared driver
# ----------------------------------------------------------------------------------------------
_INNER_MODES = {"frozen": 0, "surrogate_block": 1, "surrogate_online": 2}


def _quantize_linear(layer, W32, H3, perm, grads, quantizer, G, alpha_eff, ref_loss, plus, Hinv, mode_pack,
                     export_to_et, permute_export, rec=None, inner_mode=0, atomic=False, refresh=None, gd_pack=None,
                     diag=None, diag_info=None):
    dev = W32.device
    R, Cc = W32.shape
    mode, scale_row, scale_tab, colgrp, scale_blk, dyn_gs = mode_pack
    maxq = int(quantizer.maxq)
    st = _lib.stream_of(W32)
    Wp = torch.empty(R, Cc, dtype=torch.float32, device=dev)
    Gp = torch.empty(R, Cc, dtype=torch.float32, device=dev) if plus else None
    with torch.cuda.device(dev):
        with _sec(rec, "fasterquant.subgroup.slice_inputs"):
            _lib.check("rq_fq_prepare", _lib.lib.rq_fq_prepare(_lib.ptr(W32), _lib.ptr(grads), _lib.ptr(H3),
                                                               _lib.ptr(perm), R, Cc, G, _lib.ptr(Wp), _lib.ptr(Gp), st))
        Z = GH = beta = None
        tc = USE_TENSOR_CORES
        ws_ptr = ws_bytes = 0
        status = _lib.ptr(ops.status_word(dev))
        if tc:
            need = _lib.lib.rq_fq_tc_workspace_bytes(R, Cc, G, 1 if plus else 0)
            ws = ops._workspace(dev, need + 1024, key="fasterquant")
            ws_ptr = (ws.data_ptr() + 1023) // 1024 * 1024
            ws_bytes = ws.numel() - (ws_ptr - ws.data_ptr())
            with _sec(rec, "fasterquant.subgroup.split_hinv"):
                _lib.check("rq_fq_tc_prepare", _lib.lib.rq_fq_tc_prepare(_lib.ptr(Hinv), R, Cc, G, 1 if plus else 0,
                                                                         ws_ptr, ws_bytes, st))
        if plus:
            Z = torch.empty(R, Cc, dtype=torch.float32, device=dev)
            GH = torch.empty(R, Cc, dtype=torch.float32, device=dev)
            beta = torch.empty(R, dtype=torch.float32, device=dev)
            hdiag = torch.empty(G, Cc, dtype=torch.float32, device=dev)
            with _sec(rec, "fasterquant.subgroup.init_ghinv"):
                if tc:
                    _lib.check("rq_gptqplus_terms_tc",
                               _lib.lib.rq_gptqplus_terms_tc(_lib.ptr(Gp), _lib.ptr(Hinv), R, Cc, G, float(alpha_eff),
                                                             float(ref_loss), _lib.ptr(Z), _lib.ptr(GH), _lib.ptr(beta),
                                                             _lib.ptr(hdiag), ws_ptr, ws_bytes, status, st))
                else:
                    _lib.check("rq_gptqplus_terms",
                               _lib.lib.rq_gptqplus_terms(_lib.ptr(Gp), _lib.ptr(Hinv), R, Cc, G, float(alpha_eff),
                                                          float(ref_loss), _lib.ptr(Z), _lib.ptr(GH), _lib.ptr(beta),
                                                          _lib.ptr(hdiag), st))
        GH_initial = GH.clone() if (plus and KEEP_INTERMEDIATES) else None
        if diag is not None:
            _dump_subgroups(diag, diag_info or {}, Wp, Gp, Hinv, perm, G, plus, Z, GH, beta)
        if not plus:
            inner_mode = 0                      # beta = 0: the surrogate term vanishes
        # surrogate modes measure the drift of the weights from their values before the first block
        anchor = Wp.clone() if inner_mode else None
        Q = torch.empty(R, Cc, dtype=torch.float32, device=dev)
        codes = torch.empty(R, Cc, dtype=torch.int16, device=dev)
        Eeff = torch.empty(R, BS, dtype=torch.float32, device=dev)
        with _sec(rec, "fasterquant.block.total"):
            if mode == 3 and (gd_pack is not None or refresh is not None):
                raise NotImplementedError("block_backward / block_gd with dynamic weight groups that the host ranges "
                                          "(shrink-grid search) are not built")
            if gd_pack is not None:
                gd, gd_refresh, gd_groupsize, gd_static = gd_pack
                _block_gd_loop(gd, gd_refresh, quantizer, W32, Wp, GH, Z, Hinv, Q, codes, Eeff, mode_pack, perm, G,
                               plus, 1 if quantizer.sym else 0, maxq, atomic, gd_groupsize, gd_static, H3, st, rec)
            elif refresh is not None:
                beta, Z, GH = _block_backward_loop(
                    refresh, W32, Wp, GH, Z, beta, Hinv, Q, codes, Eeff, mode_pack, perm, G, alpha_eff, ref_loss,
                    plus, 1 if quantizer.sym else 0, maxq, atomic, st, rec)
            elif mode == 3 or diag is not None:
                _host_block_loop(quantizer, Wp, GH, Z, Hinv, Q, codes, Eeff, mode_pack, G, plus,
                                 1 if quantizer.sym else 0, maxq, anchor, beta, inner_mode, atomic, st, rec, diag)
            elif tc:
                _lib.check("rq_fq_run_tc",
                           _lib.lib.rq_fq_run_tc(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Hinv), _lib.ptr(Q),
                                                 _lib.ptr(codes), _lib.ptr(Eeff), _lib.ptr(scale_row),
                                                 _lib.ptr(scale_tab), _lib.ptr(colgrp), _lib.ptr(scale_blk), R, Cc, G,
                                                 mode, dyn_gs, 1 if quantizer.sym else 0, maxq, 1 if plus else 0,
                                                 _lib.ptr(anchor), _lib.ptr(beta) if inner_mode else 0,
                                                 int(inner_mode), 1 if atomic else 0, ws_ptr, ws_bytes, status, st))
            else:
                _lib.check("rq_fq_run",
                           _lib.lib.rq_fq_run(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Hinv), _lib.ptr(Q),
                                              _lib.ptr(codes), _lib.ptr(Eeff), _lib.ptr(scale_row), _lib.ptr(scale_tab),
                                              _lib.ptr(colgrp), _lib.ptr(scale_blk), R, Cc, G, mode, dyn_gs,
                                              1 if quantizer.sym else 0, maxq, 1 if plus else 0,
                                              _lib.ptr(anchor), _lib.ptr(beta) if inner_mode else 0,
                                              int(inner_mode), 1 if atomic else 0, st))
        out = torch.empty(layer.weight.shape, dtype=layer.weight.dtype, device=dev)
        out_codes = out_scale = None
        if export_to_et:
            out_codes = torch.empty(R, Cc, dtype=torch.float32, device=dev)
            out_scale = torch.empty(R, Cc, dtype=torch.float32, device=dev)
        tab = scale_blk if mode == 2 else scale_tab
        with _sec(rec, "fasterquant.write_layer_weight"):
            _lib.check("rq_fq_finish",
                       _lib.lib.rq_fq_finish(_lib.ptr(Q), _lib.ptr(codes), _lib.ptr(perm), R, Cc, _lib.ptr(out),
                                             _lib.dtype_code(out), _lib.ptr(out_codes), _lib.ptr(out_scale),
                                             _lib.ptr(scale_row), _lib.ptr(tab), _lib.ptr(colgrp),
                                             1 if permute_export else 0, st))
    if export_to_et:
        layer.register_buffer("int_weight", out_codes.reshape(layer.weight.shape))
        layer.register_buffer("scale", out_scale)
    layer.weight.data = out
    if diag is not None:                                        # gptq_plus_utils.py:1878-1881, natural column order
        inv = torch.argsort(perm) if perm is not None else slice(None)
        diag.save_module_level("Q_final", Q[:, inv])
        diag.save_module_level("W_int_final", codes.float()[:, inv])
        diag.save_module_level("Scale_final", _scale_matrix(mode_pack, R, Cc)[:, inv])
    return {"beta": beta, "Z": Z, "GHinv_initial": GH_initial}


def _scale_matrix(mode_pack, R, Cc):
    """[R, Cc] scale of every working-matrix position, from whichever source the block kernel used."""
    mode, scale_row, scale_tab, colgrp, scale_blk, _ = mode_pack
    if mode == 0:
        return scale_row[:, None].expand(R, Cc)
    tab = scale_blk if mode == 2 else scale_tab
    return tab[colgrp.long()].t()


def _dump_subgroups(diag, info, Wp, Gp, Hinv, perm, G, plus, Z, GH, beta):
    """Per-subgroup snapshot for the tensor-dump recorder (gptq_plus_utils.py:1108-1121): the permuted weight and
    gradient, both forms of the Hessian inverse and the first-order state before the first block."""
    R, Cc = Wp.shape
    rps = R // G
    grads = Gp
    if grads is None and info.get("gradients") is not None:
        grads = info["gradients"] if perm is None else info["gradients"][:, perm]
    identity = info.get("identity") or [False] * G
    for g in range(G):
        rows = slice(g * rps, (g + 1) * rps)
        U = Hinv[g, :Cc, :Cc]
        diag.save_subgroup(g, "W_sub_initial", Wp[rows].clone())
        if grads is not None:
            diag.save_subgroup(g, "gradients_sub", grads[rows].clone())
        diag.save_subgroup(g, "H_sub_damped_but_original", None)
        diag.save_subgroup(g, "Hinv_init", U.t() @ U)
        diag.save_subgroup(g, "Hinv_upper_cholesky", U.clone())
        diag.save_subgroup(g, "hessian_identity_fallback", torch.tensor(bool(identity[g])))
        diag.save_subgroup(g, "beta", beta[rows].clone() if plus else torch.zeros(1, device=Wp.device))
        diag.save_subgroup(g, "Z_initial", Z[rows].clone() if plus else torch.zeros_like(Wp[rows]))
        diag.save_subgroup(g, "GHinv_initial", GH[rows].clone() if plus else torch.zeros_like(Wp[rows]))
        diag.save_subgroup(g, "row_slice", torch.tensor([g * rps, (g + 1) * rps]))
        if perm is not None:
            diag.save_subgroup(g, "perm", perm)
            diag.save_subgroup(g, "invperm", torch.argsort(perm))


def _host_block_loop(quantizer, Wp, GH, Z, Hinv, Q, codes, Eeff, mode_pack, G, plus, sym, maxq, anchor, beta,
                     inner_mode, atomic, st, rec, diag):
    """The block loop with the host between the launches: one ``rq_fq_block`` and one ``rq_fq_lazy_update`` per 128
    columns.  Used for what needs the working matrix between two blocks:

    * dynamic weight groups that the block kernel cannot range itself (wider than a block, not a divisor of it, or
      with the shrink-grid search): every group that begins inside ``[i1, i2)`` is ranged from ``Wp[:, c:c+groupsize]``
      as it stands before the block is launched, i.e. from the values the reference's global ``W`` holds at that
      point (gptq_utils/gptq_utils.py:123-128; gptq_plus_utils.py:1205-1209);
    * the tensor-dump recorder (gptq_plus_utils.py:1215-1229, 1377-1387, 1526-1565): the block's inputs and outputs
      and the terms of its outer update, per saliency group."""
    dev = Wp.device
    R, Cc = Wp.shape
    mode, scale_row, scale_tab, colgrp, scale_blk, dyn_gs = mode_pack
    kmode = 1 if mode == 3 else mode
    rps = R // G
    for i1 in range(0, Cc, BS):
        count = min(BS, Cc - i1)
        i2 = i1 + count
        blk = i1 // BS
        if mode == 3:
            g0 = (i1 + dyn_gs - 1) // dyn_gs                       # groups that begin in [i1, i2)
            g1 = (i2 + dyn_gs - 1) // dyn_gs
            if g1 > g0:
                with _sec(rec, "fasterquant.block.dynamic_find_params"):
                    span = Wp[:, g0 * dyn_gs:min(Cc, g1 * dyn_gs)]
                    tab, _ = quant_utils.find_params_groups(span, dyn_gs, maxq, quantizer.sym, quantizer.mse,
                                                            quantizer.norm, quantizer.grid, quantizer.maxshrink)
                    scale_tab[g0:g1] = tab
        if diag is not None:
            w_trailing_start = Wp[:, i2:].clone()
            for g in range(G):
                rows = slice(g * rps, (g + 1) * rps)
                diag.save_block(g, blk, "W1_start", Wp[rows, i1:i2].clone())
                diag.save_block(g, blk, "W_trailing_start", w_trailing_start[rows])
                diag.save_block(g, blk, "Hinv1", Hinv[g, i1:i2, i1:i2].clone())
                if plus:
                    diag.save_block(g, blk, "GHinv1_at_block_start", GH[rows, i1:i2].clone())
                    diag.save_block(g, blk, "Z1", Z[rows, i1:i2].clone())
                diag.save_block(g, blk, "block_column_range", torch.tensor([i1, i2]))
        with _sec(rec, "fasterquant.block.inner_loop"):
            _lib.check("rq_fq_block",
                       _lib.lib.rq_fq_block(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Hinv), _lib.ptr(Q),
                                            _lib.ptr(codes), _lib.ptr(Eeff), _lib.ptr(scale_row), _lib.ptr(scale_tab),
                                            _lib.ptr(colgrp), _lib.ptr(scale_blk), R, Cc, G, i1, count, kmode, dyn_gs,
                                            sym, maxq, 1 if plus else 0, _lib.ptr(anchor),
                                            _lib.ptr(beta) if inner_mode else 0, int(inner_mode),
                                            1 if (atomic and i2 < Cc) else 0, 1.0, st))
        if diag is not None:
            Dk = torch.arange(count - 1, -1, -1, device=dev, dtype=torch.float32)
            err = Eeff[:, :count] + (Dk * Z[:, i1:i2] if plus else 0.0)         # the kernel keeps Err - D*Z
            scale1 = _scale_matrix(mode_pack, R, Cc)[:, i1:i2]
            for g in range(G):
                rows = slice(g * rps, (g + 1) * rps)
                far = Hinv[g, i1:i2, i2:Cc]
                second = err[rows] @ far
                diag.save_block(g, blk, "Q1", Q[rows, i1:i2].clone())
                diag.save_block(g, blk, "W_int1", codes[rows, i1:i2].float())
                diag.save_block(g, blk, "Scale1", scale1[rows].contiguous())
                diag.save_block(g, blk, "Err1", err[rows].contiguous())
                total = second
                if plus:
                    gh_rest = GH[rows, i2:].clone()
                    einsum_term = (Z[rows, i1:i2] * Dk) @ far
                    g_update = count * gh_rest - einsum_term
                    total = second + g_update
                    diag.save_block(g, blk, "GHinv_rest_at_outer", gh_rest)
                    diag.save_block(g, blk, "count_times_GHinv_rest", count * gh_rest)
                    diag.save_block(g, blk, "einsum_Z1_D_Hinv_term", einsum_term)
                    diag.save_block(g, blk, "G_Update", g_update)
                diag.save_block(g, blk, "second_order_update", second)
                diag.save_block(g, blk, "total_outer_update", total)
                diag.save_block(g, blk, "W_trailing_before_outer_update", w_trailing_start[rows])
                diag.save_block(g, blk, "applied_second_order_update", second)
        with _sec(rec, "fasterquant.block.outer_update_delta_w"):
            _lib.check("rq_fq_lazy_update",
                       _lib.lib.rq_fq_lazy_update(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Eeff),
                                                  _lib.ptr(Hinv), R, Cc, G, i1, count, 1 if plus else 0,
                                                  _lib.ptr(anchor), _lib.ptr(beta) if inner_mode else 0,
                                                  1 if inner_mode else 0, 1.0, st))
        if diag is not None:
            for g in range(G):
                rows = slice(g * rps, (g + 1) * rps)
                diag.save_block(g, blk, "W_trailing_after_outer_update", Wp[rows, i2:].clone())


_OBSERVER_NONE_KEYS = (
    "second_order_update_abs_mean", "second_order_update_mean_row_l2", "second_order_update_abs_max",
    "second_order_update_abs_q99", "first_order_raw_abs_mean", "first_order_raw_mean_row_l2",
    "first_order_update_abs_mean", "first_order_update_mean_row_l2", "first_order_update_abs_max",
    "first_order_update_abs_q99", "regularizer_update_abs_mean", "regularizer_update_mean_row_l2",
    "sine_regularizer_update_abs_mean", "sine_regularizer_update_mean_row_l2")
_OBSERVER_META_KEYS = ("mean_refresh_loss", "train_mean_refresh_loss", "val_mean_refresh_loss",
                       "refresh_subset_mean_refresh_loss")
_GD_META_KEYS = ("slide_alpha", "mean_refresh_loss_current", "mean_refresh_loss_next")


def _block_backward_loop(refresh, W32, Wp, GH, Z, beta, Hinv, Q, codes, Eeff, mode_pack, perm, G, alpha_eff,
                         ref_loss, plus, sym, maxq, atomic, st, rec):
    """``g_update_mode="block_backward"`` (gptq_plus_utils.py:1190, 1392-1498): every block runs in the kernel
    with the online surrogate term; between the block and its lazy update the host hands the caller's
    ``gradient_refresh_fn`` the current weights (quantized columns up to the block's end, working values to
    the right, natural column order), and the first-order terms are rebuilt from the gradient it returns."""
    refresh_fn, observer, enabled, clip, full_metrics = refresh
    dev = Wp.device
    R, Cc = Wp.shape
    mode, scale_row, scale_tab, colgrp, scale_blk, dyn_gs = mode_pack
    inv = torch.argsort(perm) if perm is not None else None
    anchor = Wp.clone() if plus else None
    hdiag = torch.empty(G, Cc, dtype=torch.float32, device=dev) if plus else None
    for i1 in range(0, Cc, BS):
        count = min(BS, Cc - i1)
        i2 = i1 + count
        with _sec(rec, "fasterquant.block.inner_loop"):
            _lib.check("rq_fq_block",
                       _lib.lib.rq_fq_block(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Hinv), _lib.ptr(Q),
                                            _lib.ptr(codes), _lib.ptr(Eeff), _lib.ptr(scale_row), _lib.ptr(scale_tab),
                                            _lib.ptr(colgrp), _lib.ptr(scale_blk), R, Cc, G, i1, count, mode, dyn_gs,
                                            sym, maxq, 1 if plus else 0, _lib.ptr(anchor), _lib.ptr(beta),
                                            2 if plus else 0, 1 if (atomic and i2 < Cc) else 0, 1.0, st))
        if enabled:
            if refresh_fn is None:
                raise ValueError("`gradient_refresh_fn` must be provided for g_update_mode='block_backward'.")
            with _sec(rec, "fasterquant.block.true_gradient_refresh"):
                current = Wp.clone()
                current[:, :i2] = Q[:, :i2]
                refreshed, meta = refresh_fn(current[:, inv] if inv is not None else current)
                refreshed = refreshed.to(dev).float()
                Gp = (refreshed[:, perm] if perm is not None else refreshed).contiguous()
                if plus:
                    # the kernel left Err - D*Z_old as the lazy update's operand; swap in the refreshed Z
                    Dk = torch.arange(count - 1, -1, -1, device=dev, dtype=torch.float32)
                    err = Eeff[:, :count] + Dk * Z[:, i1:i2]
                    _lib.check("rq_gptqplus_terms",
                               _lib.lib.rq_gptqplus_terms(_lib.ptr(Gp), _lib.ptr(Hinv), R, Cc, G, float(alpha_eff),
                                                          float(ref_loss), _lib.ptr(Z), _lib.ptr(GH), _lib.ptr(beta),
                                                          _lib.ptr(hdiag), st))
                    Eeff[:, :count] = err - Dk * Z[:, i1:i2]
                    anchor = current
                if observer is not None:
                    trailing = Gp[:, i2:] if (full_metrics and i2 < Cc) else None
                    report = {"block_idx": i1 // BS, "col_start": i1, "col_end": i2, "remaining_columns": Cc - i2,
                              "remaining_grad_abs_mean": None, "remaining_grad_clipped_abs_mean": None,
                              "remaining_grad_mean_row_l2": None}
                    if trailing is not None:
                        report["remaining_grad_abs_mean"] = trailing.abs().mean().item()
                        report["remaining_grad_mean_row_l2"] = torch.linalg.norm(trailing, dim=1).mean().item()
                        report["remaining_grad_clipped_abs_mean"] = (
                            trailing.clamp(min=-clip, max=clip).abs().mean().item()
                            if clip is not None and clip > 0 else report["remaining_grad_abs_mean"])
                    report.update({k: None for k in _OBSERVER_NONE_KEYS})
                    report.update({k: None if meta is None else meta.get(k) for k in _OBSERVER_META_KEYS})
                    observer(report)
        with _sec(rec, "fasterquant.block.outer_update_delta_w"):
            _lib.check("rq_fq_lazy_update",
                       _lib.lib.rq_fq_lazy_update(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Eeff),
                                                  _lib.ptr(Hinv), R, Cc, G, i1, count, 1 if plus else 0, 0, 0, 0, 1.0,
                                                  st))
    return beta, Z, GH


# ----------------------------------------------------------------------------------------------
# block_gd: optimizer steps on the trailing weights between blocks (gptq_plus_utils.py:586-795, 1572-1848)
# ----------------------------------------------------------------------------------------------
GD_DEFAULTS = dict(grad_lr=1e-3, grad_optimizer="sgd", curvature_damping=0.1, grad_reg_strategy="none",
                   grad_reg_lambda=0.0, grad_gate_floor=0.1, grad_gate_sharpness=1.0, grad_gate_sine_amp=0.0,
                   second_order_scale=1.0, grad_clip=1.0, slide_refresh_start=0, slide_refresh_block_total=None)
_GD_STRATEGIES = ("none", "l2", "hessian", "quant_error_gate", "quant_error_gate_optimized")


def _validate_gd(gd):
    """gptq_plus_utils.py:586-589, 666-686."""
    if gd["grad_optimizer"] not in ("sgd", "adam", "h_adam"):
        raise ValueError(f"Unsupported `grad_optimizer={gd['grad_optimizer']}`. Expected one of: sgd, adam, h_adam.")
    if gd["grad_reg_strategy"] not in _GD_STRATEGIES:
        raise ValueError(f"Unsupported `grad_reg_strategy={gd['grad_reg_strategy']}`. Expected one of: "
                         f"{', '.join(sorted(_GD_STRATEGIES))}.")
    if gd["grad_reg_lambda"] < 0:
        raise ValueError(f"`grad_reg_lambda` must be non-negative. Got {gd['grad_reg_lambda']}.")
    if not (0.0 <= gd["grad_gate_floor"] <= 1.0):
        raise ValueError(f"`grad_gate_floor` must be in [0, 1]. Got {gd['grad_gate_floor']}.")
    if gd["grad_gate_sharpness"] < 0:
        raise ValueError(f"`grad_gate_sharpness` must be non-negative. Got {gd['grad_gate_sharpness']}.")
    if gd["grad_gate_sine_amp"] < 0:
        raise ValueError(f"`grad_gate_sine_amp` must be non-negative. Got {gd['grad_gate_sine_amp']}.")


class _TrailingOptimizer:
    """SGD / Adam / curvature-preconditioned Adam on the not yet quantized columns of all row groups at once
    (gptq_plus_utils.py:586-663; the groups' states advance in lockstep, so one [G, R/G, C] state serves them).
    ``curvature``: [G, 1, C] for h_adam."""

    def __init__(self, kind, G, Rg, Cc, device, curvature=None):
        self.kind, self.step = kind, 0
        self.m = torch.zeros(G, Rg, Cc, dtype=torch.float32, device=device) if kind != "sgd" else None
        self.v = torch.zeros(G, Rg, Cc, dtype=torch.float32, device=device) if kind == "adam" else None
        self.curvature = curvature

    def clear(self, c0, c1):
        if self.m is not None:
            self.m[:, :, c0:c1].zero_()
        if self.v is not None:
            self.v[:, :, c0:c1].zero_()

    def update(self, grad3, col_start, lr, clip, b1=0.9, b2=0.999, eps=1e-8):
        g = grad3[:, :, col_start:]
        if g.numel() == 0:
            return g
        if clip is not None and clip > 0:
            g = g.clamp(min=-clip, max=clip)
        if self.kind == "sgd":
            return lr * g
        self.step += 1
        m = self.m[:, :, col_start:]
        m.mul_(b1).add_(g, alpha=1 - b1)
        bc1 = 1 - b1 ** self.step
        if self.kind == "h_adam":
            return (lr / bc1) * (m / (self.curvature[:, :, col_start:].sqrt() + eps))
        v = self.v[:, :, col_start:]
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        denom = v.sqrt() / math.sqrt(1 - b2 ** self.step)
        denom.add_(eps)
        return (lr / bc1) * (m / denom)


def _gd_setup(gd, quantizer, W32, Wp, H3, perm, G, groupsize, static_groups):
    """Per-linear state of the regularisers and of h_adam, in the permuted column order of ``Wp`` [R, C]."""
    dev = Wp.device
    R, Cc = Wp.shape
    Rg = R // G
    st = {}
    strategy = gd["grad_reg_strategy"]
    need_h = strategy == "hessian" or gd["grad_optimizer"] == "h_adam"
    if need_h:
        diag = torch.diagonal(H3, dim1=1, dim2=2).clone()                 # [G, C]
        dead = diag == 0
    if gd["grad_optimizer"] == "h_adam":                                   # input-only KFAC diagonal (:4601-4640)
        a = torch.where(dead, torch.ones_like(diag), diag)
        if perm is not None:
            a = a[:, perm]
        a = a.clamp_min(0.0)
        a = a / a.mean(dim=1, keepdim=True).clamp_min(1e-12)
        if gd["curvature_damping"] and gd["curvature_damping"] > 0:
            a = a + float(gd["curvature_damping"])
        st["curvature"] = a.view(G, 1, Cc)
    if strategy in ("l2", "hessian"):
        st["full_precision"] = Wp.clone()
    if strategy == "hessian":                                              # dead-fixed, permuted H (:1062-1064)
        Hr = H3.clone()
        idx = torch.arange(Cc, device=dev)
        Hr[:, idx, idx] = torch.where(dead, torch.ones_like(diag), diag)
        if perm is not None:
            Hr = Hr[:, perm][:, :, perm]
        st["hessian_reg"] = Hr.contiguous()
    if strategy in ("quant_error_gate", "quant_error_gate_optimized"):     # :688-722
        if groupsize == -1:
            st["gate_scale"] = quantizer.scale.to(dev, torch.float32).reshape(R, 1).expand(R, Cc)
            st["gate_zero"] = quantizer.zero.to(dev, torch.float32).reshape(R, 1).expand(R, Cc)
        else:
            if not static_groups:
                raise ValueError("`groups` must be provided when groupsize != -1.")
            tab_s, tab_z = quant_utils.find_params_groups(W32, groupsize, int(quantizer.maxq), quantizer.sym,
                                                          quantizer.mse, quantizer.norm, quantizer.grid,
                                                          quantizer.maxshrink)
            cols = perm if perm is not None else torch.arange(Cc, device=dev)
            ids = (cols // groupsize).long()
            st["gate_scale"] = tab_s[ids].t().contiguous()                 # [R, C]
            st["gate_zero"] = tab_z[ids].t().contiguous()
    st["opt"] = _TrailingOptimizer(gd["grad_optimizer"], G, Rg, Cc, dev, st.get("curvature"))
    return st


def _gd_regularize(gd, st, current, raw, col_start, G, maxq, sym):
    """(update, gate part, sine part) of the first-order step (gptq_plus_utils.py:730-795); ``current`` [R, C] holds
    the quantized columns left of ``col_start`` and the working weights from there on; ``raw`` [R, C - col_start]."""
    strategy, lr, lam = gd["grad_reg_strategy"], gd["grad_lr"], gd["grad_reg_lambda"]
    zero = None
    if raw.numel() == 0 or strategy == "none":
        return raw, zero, zero
    trailing = current[:, col_start:]
    if strategy == "l2":
        reg = lr * lam * (trailing - st["full_precision"][:, col_start:])
        return raw + reg, reg, zero
    if strategy == "hessian":
        R, Cc = current.shape
        diff = (current - st["full_precision"]).view(G, R // G, Cc)
        reg = lr * lam * torch.bmm(diff, st["hessian_reg"][:, :, col_start:]).view(R, Cc - col_start)
        return raw + reg, reg, zero
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
        return gated, gated - raw, zero
    phase = 2 * math.pi * (trailing / sc) if sym else 2 * math.pi * ((trailing / sc) + zr)
    sine = lr * (gd["grad_gate_sine_amp"] * (2 * math.pi / sc) * torch.sin(phase))
    return gated + sine, gated - raw, sine


def _abs_stats(t):
    """(mean |t|, mean row l2) of a [R, n] tensor, or (None, None) when empty."""
    if t is None or t.numel() == 0:
        return None, None
    return t.abs().mean().item(), torch.linalg.norm(t, dim=1).mean().item()


def _block_gd_loop(gd, refresh, quantizer, W32, Wp, GH, Z, Hinv, Q, codes, Eeff, mode_pack, perm, G, plus, sym, maxq,
                   atomic, groupsize, static_groups, H3, st, rec):
    """``g_update_mode="block_gd"`` (gptq_plus_utils.py:1190, 1344-1349, 1546-1848): frozen first-order terms inside
    the kernels, the weight updates scaled by ``second_order_scale``; after every block but the last the caller's
    ``gradient_refresh_fn`` sees the current weights and an optimizer step (with the chosen regulariser) moves the
    columns that are still to be quantized.  Kernels: rq_fq_block / rq_fq_lazy_update per block; the optimizer
    arithmetic is elementwise torch on the device, as in the reference."""
    refresh_fn, observer, enabled, full_metrics = refresh
    dev = Wp.device
    R, Cc = Wp.shape
    Rg = R // G
    mode, scale_row, scale_tab, colgrp, scale_blk, dyn_gs = mode_pack
    inv = torch.argsort(perm) if perm is not None else None
    state = _gd_setup(gd, quantizer, W32, Wp, H3, perm, G, groupsize, static_groups)
    opt = state["opt"]
    so = float(gd["second_order_scale"])
    n_refresh_total = max((Cc + BS - 1) // BS - 1, 0)
    Cp = Hinv.shape[-1]
    for i1 in range(0, Cc, BS):
        count = min(BS, Cc - i1)
        i2 = i1 + count
        with _sec(rec, "fasterquant.block.inner_loop"):
            _lib.check("rq_fq_block",
                       _lib.lib.rq_fq_block(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Hinv), _lib.ptr(Q),
                                            _lib.ptr(codes), _lib.ptr(Eeff), _lib.ptr(scale_row), _lib.ptr(scale_tab),
                                            _lib.ptr(colgrp), _lib.ptr(scale_blk), R, Cc, G, i1, count, mode, dyn_gs,
                                            sym, maxq, 1 if plus else 0, 0, 0, 0,
                                            1 if (atomic and i2 < Cc) else 0, so, st))
        second = None
        if full_metrics and i2 < Cc:                    # applied second-order part of the lazy update, for the report
            err = Eeff[:, :count]
            if plus:
                err = err + torch.arange(count - 1, -1, -1, device=dev, dtype=torch.float32) * Z[:, i1:i2]
            second = so * torch.bmm(err.reshape(G, Rg, count), Hinv.view(G, Cp, Cp)[:, i1:i2, i2:Cc]).view(R, Cc - i2)
        with _sec(rec, "fasterquant.block.outer_update_delta_w"):
            _lib.check("rq_fq_lazy_update",
                       _lib.lib.rq_fq_lazy_update(_lib.ptr(Wp), _lib.ptr(GH), _lib.ptr(Z), _lib.ptr(Eeff),
                                                  _lib.ptr(Hinv), R, Cc, G, i1, count, 1 if plus else 0, 0, 0, 0, so,
                                                  st))
        opt.clear(i1, i2)
        if not (enabled and i2 < Cc):
            continue
        if refresh_fn is None:
            raise ValueError("`gradient_refresh_fn` must be provided for g_update_mode='block_gd'.")
        with _sec(rec, "fasterquant.block.true_gradient_refresh"):
            current = Wp.clone()
            current[:, :i2] = Q[:, :i2]
            total = gd["slide_refresh_block_total"] if gd["slide_refresh_block_total"] is not None else n_refresh_total
            idx = gd["slide_refresh_start"] + i1 // BS
            slide_alpha = 1.0 - idx / max(total - 1, 1) if total > 1 else 1.0
            refreshed, meta = refresh_fn(current[:, inv] if inv is not None else current, slide_alpha=slide_alpha)
            refreshed = refreshed.to(dev).float()
            Gp = (refreshed[:, perm] if perm is not None else refreshed).contiguous()
            raw = opt.update(Gp.view(G, Rg, Cc), i2, gd["grad_lr"], gd["grad_clip"]).reshape(R, Cc - i2)
            update, gate_part, sine_part = _gd_regularize(gd, state, current, raw, i2, G, maxq, bool(sym))
            if observer is not None:
                report = {"block_idx": i1 // BS, "col_start": i1, "col_end": i2, "remaining_columns": Cc - i2,
                          "remaining_grad_abs_mean": None, "remaining_grad_clipped_abs_mean": None,
                          "remaining_grad_mean_row_l2": None}
                report.update({k: None for k in _OBSERVER_NONE_KEYS})
                if full_metrics:
                    trailing = Gp[:, i2:]
                    clip = gd["grad_clip"]
                    report["remaining_grad_abs_mean"], report["remaining_grad_mean_row_l2"] = _abs_stats(trailing)
                    report["remaining_grad_clipped_abs_mean"] = (
                        trailing.clamp(min=-clip, max=clip).abs().mean().item() if clip is not None and clip > 0
                        else report["remaining_grad_abs_mean"])
                    for key, t in (("second_order_update", second), ("first_order_update", update)):
                        report[key + "_abs_mean"], report[key + "_mean_row_l2"] = _abs_stats(t)
                        if t is not None and t.numel() > 0:
                            a = t.abs()
                            report[key + "_abs_max"] = a.max().item()
                            report[key + "_abs_q99"] = ops.clamp_to_quantile_(a.flatten().clone(), 0.99).item()
                    report["first_order_raw_abs_mean"], report["first_order_raw_mean_row_l2"] = _abs_stats(raw)
                    zeros = torch.zeros_like(update)
                    report["regularizer_update_abs_mean"], report["regularizer_update_mean_row_l2"] = _abs_stats(
                        gate_part if gate_part is not None else zeros)
                    (report["sine_regularizer_update_abs_mean"],
                     report["sine_regularizer_update_mean_row_l2"]) = _abs_stats(sine_part if sine_part is not None else zeros)
                report.update({k: None if meta is None else meta.get(k) for k in _OBSERVER_META_KEYS + _GD_META_KEYS})
                observer(report)
        with _sec(rec, "fasterquant.block.outer_update_grad_descent"):
            if update.numel() > 0:
                Wp[:, i2:] -= update


def _check_common(quantizer, blocksize):
    if blocksize % BS != 0:
        raise NotImplementedError(f"blocksize must be a multiple of {BS} (the kernels' column block); got {blocksize}")
    maxq = int(quantizer.maxq)
    if not (0 < maxq <= 32767):
        raise NotImplementedError(f"integer codes are stored as int16: maxq must be in 1..32767, got {maxq}")


class _RowSlice:
    """Stand-in for ``layer`` that lets the shared driver write the result of a row slice."""

    class _Weight:
        def __init__(self, data):
            self.data, self.shape, self.dtype = data, data.shape, data.dtype

    def __init__(self, weight_rows):
        self.weight = self._Weight(weight_rows)
        self.buffers = {}

    def register_buffer(self, name, tensor):
        self.buffers[name] = tensor


def _quantize_owned_groups(obj, W32, H3, perm, grads, alpha_eff, plus, percdamp, groupsize, static_groups, blocksize,
                           export_to_et, rec, inner_mode, atomic):
    """The groups whose owner is this rank, as runs of consecutive groups; rows of other groups stay as they are
    (export buffers: zero there)."""
    from ..utils import dist_utils
    layer = obj.layer
    rank = dist_utils.get_rank()
    G = obj.num_groups
    rps = obj.rows // G
    owned = [g for g in range(G) if obj.group_owners[g] == rank]
    runs = []
    for g in owned:
        if runs and runs[-1][1] == g:
            runs[-1][1] = g + 1
        else:
            runs.append([g, g + 1])
    out = layer.weight.data.clone()
    codes = torch.zeros_like(W32) if export_to_et else None
    scales = torch.zeros_like(W32) if export_to_et else None
    last = {"Hinv": None, "perm": perm, "damp_percent": [None] * G, "identity_fallback": [None] * G}
    for g0, g1 in runs:
        rows = slice(g0 * rps, g1 * rps)
        with _sec(rec, "fasterquant.quantizer_build_groups"):
            mode_pack = _scale_setup(obj.quantizer, W32, groupsize, static_groups, blocksize, perm, None, rows=rows)
        with _sec(rec, "fasterquant.subgroup.compute_hinv"):
            Hinv, damp, identity = hinv_with_fallback(H3[g0:g1], perm, percdamp, identity_fallback=True,
                                                      log_context=f" groups {g0}..{g1 - 1}")
        part = _RowSlice(layer.weight.data[rows])
        _quantize_linear(part, W32[rows], H3[g0:g1], perm, grads[rows] if plus else None, obj.quantizer, g1 - g0,
                         alpha_eff, obj.reference_loss, plus, Hinv, mode_pack, export_to_et, permute_export=True,
                         rec=rec, inner_mode=inner_mode, atomic=atomic)
        out[rows] = part.weight.data
        if export_to_et:
            codes[rows] = part.buffers["int_weight"]
            scales[rows] = part.buffers["scale"]
        last["damp_percent"][g0:g1] = damp
        last["identity_fallback"][g0:g1] = identity
    layer.weight.data = out
    if export_to_et:
        layer.register_buffer("int_weight", codes.reshape(layer.weight.shape))
        layer.register_buffer("scale", scales)
    obj._last_fasterquant = last


def _quantize_row_shard(obj, W32, H3, perm, grads, alpha_eff, plus, percdamp, groupsize, static_groups, blocksize,
                        export_to_et, rec, inner_mode, atomic):
    """Row-parallel mode: this rank's rows ``[r*R/W, (r+1)*R/W)`` only.  They lie in the saliency groups whose summed
    Hessians finalize_hessian left on this rank: whole groups when the world size divides the group count, one
    of ``pieces`` equal row slices of a single group otherwise (the ranks that share a group factorise the same
    Hessian, bit for bit, and split its rows, which are independent given the inverse factor).  The other rows
    of layer.weight keep their values until gather_rows_()."""
    from ..utils import dist_utils
    layer = obj.layer
    G = obj.num_groups
    first, count, piece, pieces = dist_utils.row_parallel_layout(G)
    rps = obj.rows // G
    if rps % pieces != 0:
        raise ValueError(f"row-parallel quantization: {rps} rows per group do not split over {pieces} ranks")
    if pieces == 1:
        rows = slice(first * rps, (first + count) * rps)
    else:
        sub = rps // pieces
        rows = slice(first * rps + piece * sub, first * rps + (piece + 1) * sub)
    with _sec(rec, "fasterquant.quantizer_build_groups"):
        mode_pack = _scale_setup(obj.quantizer, W32, groupsize, static_groups, blocksize, perm, None, rows=rows)
    with _sec(rec, "fasterquant.subgroup.compute_hinv"):
        Hinv, damp, identity = hinv_with_fallback(H3[first:first + count], perm, percdamp, identity_fallback=True,
                                                  log_context=f" groups {first}..{first + count - 1}")
    part = _RowSlice(layer.weight.data[rows])
    _quantize_linear(part, W32[rows], H3[first:first + count], perm, grads[rows] if plus else None, obj.quantizer,
                     count, alpha_eff, obj.reference_loss, plus, Hinv, mode_pack, export_to_et, permute_export=True,
                     rec=rec, inner_mode=inner_mode, atomic=atomic)
    out = layer.weight.data
    if not out.is_contiguous():
        out = out.contiguous()
    out[rows] = part.weight.data
    layer.weight.data = out
    if export_to_et:
        codes, scales = torch.zeros_like(W32), torch.zeros_like(W32)
        codes[rows] = part.buffers["int_weight"]
        scales[rows] = part.buffers["scale"]
        layer.register_buffer("int_weight", codes.reshape(layer.weight.shape))
        layer.register_buffer("scale", scales)
    obj._last_fasterquant = {"Hinv": None, "perm": perm, "damp_percent": damp, "identity_fallback": identity}


# ----------------------------------------------------------------------------------------------
# GuidedQuant (gptq_utils/gptq_guided_utils.py:86-259): grouped Hessians, no first-order terms
# ----------------------------------------------------------------------------------------------
@torch.no_grad()
def guided_fasterquant(obj, H3, blocksize, percdamp, groupsize, actorder, static_groups, export_to_et):
    layer, dev = obj.layer, obj.dev
    W32 = layer.weight.data.float().contiguous()
    G = obj.num_groups
    if not obj.quantizer.ready():
        obj.quantizer.find_params(W32)
    _check_common(obj.quantizer, blocksize)
    empty = (H3.reshape(G, -1) == 0).all(dim=1).tolist()           # no calibration data: round to nearest (:119-121)
    if any(empty):
        H3 = H3.clone()
        for g, e in enumerate(empty):
            if e:
                H3[g] = torch.eye(obj.columns, device=dev)
    perm = torch.argsort(obj.act_square, descending=True) if actorder else None
    if groupsize != -1 and not static_groups and actorder:
        # gptq_guided_utils.py:186-191 under act_order: the working matrix is a permuted copy, so the reference's
        # find_params(W[:, pos:pos+groupsize]) ranges the original columns (dead ones zeroed, never updated) at the
        # POSITION being quantized: a static table looked up by position, not by the permuted column's own index
        Wz = W32.clone()
        rps = W32.shape[0] // G
        dead = torch.diagonal(H3, dim1=1, dim2=2) == 0                                # [G, C]
        Wz.view(G, rps, -1).masked_fill_(dead.unsqueeze(1), 0.0)
        tab, _ = quant_utils.find_params_groups(Wz, groupsize, int(obj.quantizer.maxq), obj.quantizer.sym,
                                                obj.quantizer.mse, obj.quantizer.norm, obj.quantizer.grid,
                                                obj.quantizer.maxshrink)
        colgrp = (torch.arange(W32.shape[1], device=dev) // groupsize).to(torch.int32).contiguous()
        mode_pack = (1, None, tab, colgrp, None, 0)
    else:
        mode_pack = _scale_setup(obj.quantizer, W32, groupsize, static_groups, blocksize, perm, None)
    Hinv, damp, _ = hinv_with_fallback(H3, perm, percdamp, identity_fallback=False)
    _quantize_linear(layer, W32, H3, perm, None, obj.quantizer, G, 0.0, 0.0, False, Hinv, mode_pack, export_to_et,
                     permute_export=True)
    obj._last_fasterquant = {"perm": perm, "damp_percent": damp}


# ----------------------------------------------------------------------------------------------
# plain GPTQ (gptq_utils/gptq_utils.py:45-174)
# ----------------------------------------------------------------------------------------------
@torch.no_grad()
def plain_fasterquant(obj, H, blocksize, percdamp, groupsize, actorder, static_groups, export_to_et):
    layer, dev = obj.layer, obj.dev
    W32 = layer.weight.data.float().contiguous()
    R, Cc = W32.shape
    if not obj.quantizer.ready():
        obj.quantizer.find_params(W32)
    _check_common(obj.quantizer, blocksize)
    if bool((H == 0).all()):                                    # no calibration data: round to nearest
        H = torch.eye(Cc, device=dev)
    H3 = H.reshape(1, Cc, Cc).contiguous()
    diag = torch.diagonal(H3[0])
    dead = diag == 0
    Wz = None
    if groupsize != -1 and static_groups:                      # plain GPTQ ranges the groups after dead-zeroing
        Wz = W32.clone()
        Wz[:, dead] = 0
    perm = None
    if actorder:
        key = torch.where(dead, torch.ones_like(diag), diag)
        perm = torch.argsort(key, descending=True)
    mode_pack = _scale_setup(obj.quantizer, W32, groupsize, static_groups, blocksize, perm, Wz)
    Hinv, _, _ = hinv_with_fallback(H3, perm, percdamp, identity_fallback=False)
    _quantize_linear(layer, W32, H3, perm, None, obj.quantizer, 1, 0.0, 0.0, False, Hinv, mode_pack,
                     export_to_et, permute_export=False)


# ----------------------------------------------------------------------------------------------
# GPTAQ (gptq_utils/gptaq_utils.py:43-167)
# ----------------------------------------------------------------------------------------------
@torch.no_grad()
def gptaq_fasterquant(obj, H, blocksize, percdamp, groupsize, actorder, static_groups, alpha):
    layer, dev = obj.layer, obj.dev
    W32 = layer.weight.data.float().contiguous()
    R, Cc = W32.shape
    quantizer = obj.quantizer
    if not quantizer.ready():
        quantizer.find_params(W32)
    _check_common(quantizer, blocksize)
    dynamic = groupsize != -1 and not static_groups
    if dynamic and (BS % groupsize != 0 or blocksize != BS or quantizer.mse):
        raise NotImplementedError(f"GPTAQ with dynamic weight groups is built for blocksize == {BS}, a groupsize that "
                                  f"divides it and no shrink-grid search; got groupsize={groupsize}, "
                                  f"blocksize={blocksize}, mse={quantizer.mse}")
    if bool((H == 0).all()):                                    # no calibration data: round to nearest
        H = torch.eye(Cc, device=dev)
    H3 = H.reshape(1, Cc, Cc).contiguous()
    diag = torch.diagonal(H3[0])
    dead = diag == 0
    perm = None
    if actorder:
        key = torch.where(dead, torch.ones_like(diag), diag)
        perm = torch.argsort(key, descending=True)
    maxq = int(quantizer.maxq)
    asym = 0 if quantizer.sym else 1
    scale_row = zero_row = scale_tab = zero_tab = colgrp = None
    if groupsize == -1:
        mode = 0
        scale_row = quantizer.scale.to(dev, torch.float32).reshape(-1).contiguous()
        zero_row = quantizer.zero.to(dev, torch.float32).reshape(-1).contiguous()
    elif dynamic:
        mode = 2                                                 # ranged inside the kernel, block by block
    else:
        mode = 1
        Wz = W32.clone()
        Wz[:, dead] = 0                                          # the groups are ranged after dead-zeroing (:70-78)
        scale_tab, zero_tab = quant_utils.find_params_groups(Wz, groupsize, maxq, quantizer.sym, quantizer.mse,
                                                             quantizer.norm, quantizer.grid, quantizer.maxshrink)
        cols = perm if perm is not None else torch.arange(Cc, device=dev)
        colgrp = (cols // groupsize).to(torch.int32).contiguous()
    Hinv, _, _ = hinv_with_fallback(H3, perm, percdamp, identity_fallback=False)
    st = _lib.stream_of(W32)
    Wp = torch.empty(R, Cc, dtype=torch.float32, device=dev)
    Q = torch.empty(R, Cc, dtype=torch.float32, device=dev)
    P = torch.empty(Cc, Cc, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check("rq_fq_prepare", _lib.lib.rq_fq_prepare(_lib.ptr(W32), 0, _lib.ptr(H3), _lib.ptr(perm), R, Cc, 1,
                                                           _lib.ptr(Wp), 0, st))
        need = _lib.lib.rq_gptaq_workspace_bytes(R, Cc)
        ws = ops._workspace(dev, need + 1024, key="gptaq")
        base = (ws.data_ptr() + 1023) // 1024 * 1024
        _lib.check("rq_gptaq_terms", _lib.lib.rq_gptaq_terms(_lib.ptr(obj.dXXT), _lib.ptr(H3), _lib.ptr(perm),
                                                             _lib.ptr(Hinv), Cc, float(alpha), _lib.ptr(P), base, need,
                                                             _lib.ptr(ops.status_word(dev)), st))
        _lib.check("rq_gptaq_run", _lib.lib.rq_gptaq_run(_lib.ptr(Wp), _lib.ptr(Hinv), _lib.ptr(P), _lib.ptr(Q),
                                                         _lib.ptr(scale_row), _lib.ptr(zero_row), _lib.ptr(scale_tab),
                                                         _lib.ptr(zero_tab), _lib.ptr(colgrp), R, Cc, mode,
                                                         groupsize if dynamic else 0, asym, maxq,
                                                         base, need, _lib.ptr(ops.status_word(dev)), st))
        out = torch.empty(layer.weight.shape, dtype=layer.weight.dtype, device=dev)
        _lib.check("rq_fq_finish", _lib.lib.rq_fq_finish(_lib.ptr(Q), 0, _lib.ptr(perm), R, Cc, _lib.ptr(out),
                                                         _lib.dtype_code(out), 0, 0, 0, 0, 0, 0, st))
    layer.weight.data = out
    obj._last_fasterquant = {"perm": perm, "P": P if KEEP_INTERMEDIATES else None}


# ----------------------------------------------------------------------------------------------
# GPTQ+ (gptq_utils/gptq_plus_utils.py:910-1896)
# ----------------------------------------------------------------------------------------------
@torch.no_grad()
def plus_fasterquant(obj, blocksize, percdamp, groupsize, actorder, static_groups, enable_gradient_update,
                     g_update_mode, export_to_et, profile_recorder, gradient_refresh_fn, grad_reg_strategy,
                     second_order_scale, block_atomic_quant, block_observer, diagnostic_recorder, grad_clip=1.0,
                     refresh_full_metrics=False, gd=None):
    if g_update_mode not in _INNER_MODES and g_update_mode not in ("block_backward", "block_gd"):
        raise ValueError(f"Unknown g_update_mode '{g_update_mode}'")
    gd_mode = g_update_mode == "block_gd"
    if gd_mode:
        gd = dict(GD_DEFAULTS, **(gd or {}))
        _validate_gd(gd)
    if (g_update_mode != "frozen" or block_atomic_quant) and blocksize != BS:
        raise NotImplementedError(
            f"surrogate modes and block_atomic_quant depend on the block boundaries: blocksize must be {BS}, "
            f"got {blocksize}")
    diag = diagnostic_recorder
    if diag is not None and (g_update_mode != "frozen" or block_atomic_quant or blocksize != BS):
        raise NotImplementedError(f"the tensor-dump recorder is built for g_update_mode='frozen', blocksize={BS} and "
                                  "no block_atomic_quant (its per-block tags follow the frozen outer update)")
    layer, dev = obj.layer, obj.dev
    rec = profile_recorder
    with _sec(rec, "fasterquant.allocate_outputs"):
        W32 = layer.weight.data.float().contiguous()
    R, Cc = W32.shape
    G = obj.num_groups
    with _sec(rec, "fasterquant.quantizer_find_params_initial"):
        if not obj.quantizer.ready():
            obj.quantizer.find_params(W32)
    _check_common(obj.quantizer, blocksize)
    dynamic_groups = groupsize != -1 and not static_groups
    if dynamic_groups and groupsize != blocksize:
        raise ValueError("`groupsize` must equal `blocksize` when using dynamic groups in GPTQ+. "
                         f"Got groupsize={groupsize}, blocksize={blocksize}.")
    ops.check_status(dev)
    H3 = obj.H
    with _sec(rec, "fasterquant.subgroup.actorder_permute"):
        perm = torch.argsort(obj.act_square, descending=True) if actorder else None
    plus = bool(enable_gradient_update and obj.alpha > 0)
    grads = obj.gradients.to(dev).float().contiguous() if plus else None
    alpha_eff = obj.alpha / (obj.rows * obj.columns) if plus else 0.0
    refresh = ((gradient_refresh_fn, block_observer, bool(enable_gradient_update), grad_clip,
                bool(refresh_full_metrics)) if g_update_mode == "block_backward" else None)
    gd_pack = None
    if gd_mode:
        gd_pack = (gd, (gradient_refresh_fn, block_observer, bool(enable_gradient_update),
                        bool(refresh_full_metrics)), groupsize, static_groups)
    sharded = (getattr(obj, "row_parallel", False) and obj._owned_groups is not None) or \
        getattr(obj, "group_owners", None) is not None
    if diag is not None:
        if sharded:
            raise NotImplementedError("the tensor-dump recorder sees every subgroup: run it without row_parallel / "
                                      "group_owners")
        # gptq_plus_utils.py:957-972
        diag.save_module_level("original_weight_rotated", W32)
        for tag in ("scale", "zero"):
            if hasattr(obj.quantizer, tag):
                diag.save_module_level(f"quantizer_{tag}", getattr(obj.quantizer, tag))
        mq = obj.quantizer.maxq
        diag.save_module_level("quantizer_maxq", mq if isinstance(mq, torch.Tensor) else torch.tensor(float(mq)))
        diag.save_module_level("H_after_accumulate", obj.H)
        diag.save_module_level("act_square", obj.act_square)
        diag.save_module_level("gradients", obj.gradients)
        diag.save_module_level("reference_loss", torch.tensor(obj.reference_loss))
        diag.save_module_level("saliencies", obj.saliencies)
        diag.save_module_level("alpha", torch.tensor(obj.alpha))
    if getattr(obj, "row_parallel", False) and obj._owned_groups is not None:
        if refresh is not None or gd_pack is not None:
            raise NotImplementedError(f"{g_update_mode} needs every row on one rank (the callback sees the whole "
                                      "weight); use hessian_owner instead of row_parallel")
        _quantize_row_shard(obj, W32, H3, perm, grads, alpha_eff, plus, percdamp, groupsize, static_groups,
                            blocksize, export_to_et, rec, _INNER_MODES.get(g_update_mode, 0), bool(block_atomic_quant))
        return
    if getattr(obj, "group_owners", None) is not None:
        if refresh is not None or gd_pack is not None:
            raise NotImplementedError(f"{g_update_mode} needs every row group on one rank (the callback sees the "
                                      "whole weight); use hessian_owner instead of group_owners")
        _quantize_owned_groups(obj, W32, H3, perm, grads, alpha_eff, plus, percdamp, groupsize, static_groups,
                               blocksize, export_to_et, rec, _INNER_MODES.get(g_update_mode, 0),
                               bool(block_atomic_quant))
        return
    with _sec(rec, "fasterquant.quantizer_build_groups"):
        mode_pack = _scale_setup(obj.quantizer, W32, groupsize, static_groups, blocksize, perm, None)
    with _sec(rec, "fasterquant.subgroup.compute_hinv"):
        Hinv, damp, identity = hinv_with_fallback(H3, perm, percdamp, identity_fallback=True)
    state = _quantize_linear(layer, W32, H3, perm, grads, obj.quantizer, G, alpha_eff, obj.reference_loss, plus, Hinv,
                             mode_pack, export_to_et, permute_export=True, rec=rec,
                             inner_mode=_INNER_MODES.get(g_update_mode, 0), atomic=bool(block_atomic_quant),
                             refresh=refresh, gd_pack=gd_pack, diag=diag,
                             diag_info=None if diag is None else {
                                 "identity": identity,
                                 "gradients": None if obj.gradients is None else obj.gradients.to(dev).float()})
    obj._last_fasterquant = {"Hinv": Hinv if KEEP_INTERMEDIATES else None, "perm": perm, "damp_percent": damp,
                             "identity_fallback": identity, **state}
