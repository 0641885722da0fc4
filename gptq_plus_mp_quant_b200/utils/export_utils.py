"""Packed export of a quantized linear.  The reference keeps ``int_weight`` and ``scale`` as fp32 ``[R, C]`` buffers
(gptq_utils/gptq_plus_utils.py:1866-1871) and saves the model's state dict as is (gptq_utils/main.py:66-71); this
module adds a compact form: a bit stream of the codes and one scale per row and column group."""
from __future__ import annotations

import torch

from .. import _lib


def pack_codes(int_weight: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 ``[R, ceil(C/8)*bits]``: every row's codes as a little-endian bit stream, ``bits`` bits each (two's
    complement), eight consecutive codes per ``bits`` bytes."""
    _lib.require_cuda(int_weight)
    assert int_weight.dim() == 2 and int_weight.dtype == torch.float32
    w = int_weight if int_weight.stride(1) == 1 else int_weight.contiguous()
    R, Cc = w.shape
    out = torch.empty(R, _lib.lib.rq_packed_row_bytes(Cc, int(bits)), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        rc = _lib.lib.rq_pack_codes(_lib.ptr(w), R, Cc, w.stride(0), int(bits), _lib.ptr(out), _lib.stream_of(w))
    _lib.check("rq_pack_codes", rc)
    return out


def unpack_codes(packed: torch.Tensor, bits: int, columns: int) -> torch.Tensor:
    """Inverse of pack_codes (plain torch, for consumers and tests): int32 ``[R, columns]`` signed codes."""
    R = packed.shape[0]
    groups = (columns + 7) // 8
    by = packed.reshape(R, groups, bits).to(torch.int64)
    word = torch.zeros(R, groups, dtype=torch.int64, device=packed.device)
    for b in range(bits):
        word |= by[:, :, b] << (8 * b)
    shifts = torch.arange(8, device=packed.device, dtype=torch.int64) * bits
    codes = (word.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    codes = torch.where(codes >= (1 << (bits - 1)), codes - (1 << bits), codes)
    return codes.reshape(R, groups * 8)[:, :columns].to(torch.int32)


def pack_quantized_linear(layer, bits: int, groupsize: int = -1) -> dict:
    """Compact form of a linear quantized with ``export_to_et=True``: ``qweight`` (pack_codes of ``int_weight``),
    ``scales`` ``[R, 1]`` or ``[R, C/groupsize]`` (taken from the first column of every group of ``layer.scale``; the
    groups must be constant in natural column order, i.e. per-row scales or static groups), ``bits``, ``groupsize``,
    ``shape``.  Dequantization: ``unpack_codes(qweight) * scales`` expanded over the groups."""
    int_weight, scale = layer.int_weight, layer.scale
    R, Cc = int_weight.shape
    if groupsize == -1:
        scales = scale[:, :1].contiguous()
        expanded = scales.expand(R, Cc)
    else:
        scales = scale[:, ::groupsize].contiguous()
        expanded = scales.repeat_interleave(groupsize, dim=1)[:, :Cc]
    if not torch.equal(expanded, scale):
        raise ValueError("scales are not constant over the column groups (dynamic groups under act_order cannot be "
                         "stored per group)")
    return {"qweight": pack_codes(int_weight, bits), "scales": scales, "bits": int(bits), "groupsize": int(groupsize),
            "shape": (R, Cc)}
