"""Oracle: weight-quantizer parameter search and round/clamp quantization.

Test infrastructure (see ``oracle/__init__.py``).  Restates
``utils/quant_utils.py`` of the reference:

* ``sym_quant``/``asym_quant`` round-clamp primitives          (:28-57)
* ``STEQuantize`` / ``AsymSTEQuantize`` forward                 (:60-84)
* ``WeightQuantizer.configure``                                 (:309-331)
* ``WeightQuantizer.find_params`` incl. the shrink-grid search  (:390-457)
* ``WeightQuantizer.fake_quantize`` / ``quantize`` / ``ready``  (:460-486)
"""
from __future__ import annotations

import torch


def maxq_for(bits: int, sym: bool) -> int:
    """Largest code: 2^(b-1)-1 symmetric, 2^b-1 asymmetric (quant_utils.py:328-331)."""
    return 2 ** (bits - 1) - 1 if sym else 2 ** bits - 1


def sym_codes(x: torch.Tensor, scale: torch.Tensor, maxq: int) -> torch.Tensor:
    """clamp(round(x / scale), -(maxq+1), maxq); round is half-to-even (quant_utils.py:47-50)."""
    return torch.clamp(torch.round(x / scale), -(maxq + 1), maxq)


def asym_codes(x: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, maxq: int) -> torch.Tensor:
    """clamp(round(x / scale) + zero, 0, maxq) (quant_utils.py:32-36)."""
    return torch.clamp(torch.round(x / scale) + zero, 0, maxq)


def _row_range(x2d: torch.Tensor):
    """Per-row min/max that always contain 0 (quant_utils.py:406-408)."""
    zeros = torch.zeros(x2d.shape[0], dtype=x2d.dtype)
    lo = torch.minimum(x2d.min(1)[0], zeros)
    hi = torch.maximum(x2d.max(1)[0], zeros)
    return lo, hi


def find_params(x: torch.Tensor, bits: int, perchannel: bool = False, sym: bool = True,
                mse: bool = False, norm: float = 2.4, grid: int = 50, maxshrink: float = 0.5):
    """Return (scale, zero), each shaped ``[-1, 1, ...]`` like the reference.

    Follows ``WeightQuantizer.find_params`` (quant_utils.py:390-457) for the
    ``weight_groupsize <= 0`` branch: range always includes 0; symmetric scale
    is ``max(|min|, max).clamp(1e-5) / maxq`` with zero 0; asymmetric scale is
    ``(max - min).clamp(1e-5) / maxq`` with ``zero = round(-min / scale)`` and
    an all-zero row mapped to (-1, +1); the optional search shrinks min and max
    independently on an ``int(maxshrink*grid)``-squared lattice and keeps a
    candidate only when its ``sum |q - x|^norm`` is strictly smaller.
    """
    if bits == 16:
        return None, None
    maxq = maxq_for(bits, sym)
    shape = x.shape
    x2 = x.flatten(1) if perchannel else x.flatten().unsqueeze(0)
    lo, hi = _row_range(x2)

    if sym:
        scale = torch.maximum(lo.abs(), hi).clamp(min=1e-5) / maxq
        zero = torch.zeros_like(scale)
    else:
        flat = (lo == 0) & (hi == 0)
        lo = lo.clone()
        hi = hi.clone()
        lo[flat] = -1
        hi[flat] = +1
        scale = (hi - lo).clamp(min=1e-5) / maxq
        zero = torch.round(-lo / scale)

    if mse:
        best = torch.full([x2.shape[0]], float("inf"))
        steps = int(maxshrink * grid)
        for i in range(steps):
            for j in range(steps):
                lo1 = (1 - i / grid) * lo
                hi1 = (1 - j / grid) * hi
                if sym:
                    s1 = torch.maximum(lo1.abs(), hi1).clamp(min=1e-5) / maxq
                    z1 = torch.zeros_like(s1)
                    deq = s1.unsqueeze(1) * sym_codes(x2, s1.unsqueeze(1), maxq)
                else:
                    s1 = (hi1 - lo1) / maxq
                    z1 = torch.round(-lo1 / s1)
                    deq = s1.unsqueeze(1) * (asym_codes(x2, s1.unsqueeze(1), z1.unsqueeze(1), maxq) - z1.unsqueeze(1))
                err = (deq - x2).abs_().pow_(norm).sum(1)
                better = err < best
                if torch.any(better):
                    best[better] = err[better]
                    scale[better] = s1[better]
                    zero[better] = z1[better]

    if not perchannel:
        scale = scale.repeat(shape[0])
        zero = zero.repeat(shape[0])
    out_shape = [-1] + [1] * (len(shape) - 1)
    return scale.reshape(out_shape), zero.reshape(out_shape)


def ste_quantize(x: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, maxq: int, sym: bool) -> torch.Tensor:
    """Forward value of ``WeightQuantizer.quantize`` (quant_utils.py:60-84,460-468).

    Unlike ``fake_quantize`` this path honours the zero-point when asymmetric.
    """
    if sym:
        return (scale * sym_codes(x, scale, maxq)).to(x.dtype)
    return (scale * (asym_codes(x, scale, zero, maxq) - zero)).to(x.dtype)


def fake_quantize(x: torch.Tensor, scale: torch.Tensor, maxq: int, st_idx=None, end_idx=None):
    """(dequantized, integer codes, scale) as ``WeightQuantizer.fake_quantize``
    (quant_utils.py:471-480): ALWAYS the symmetric clamp, the zero-point is ignored."""
    if st_idx is not None and end_idx is not None:
        scale = scale[st_idx:end_idx]
    codes = sym_codes(x, scale, maxq)
    return (scale * codes).to(x.dtype), codes, scale


class OracleWeightQuantizer:
    """Stateful twin of the reference ``WeightQuantizer`` (quant_utils.py:300-486),
    without the grouped per-token branch.  Used as the injected ``quantizer`` of the
    oracle GPTQ objects."""

    def __init__(self, shape: int = 1):
        self.maxq = torch.tensor(0)
        self.scale = torch.zeros(shape)
        self.zero = torch.zeros(shape)

    def configure(self, bits, perchannel=False, sym=True, mse=False, norm=2.4, grid=50,
                  maxshrink=0.5, weight_groupsize=-1):
        assert weight_groupsize <= 0, "oracle covers the per-channel / per-tensor branch"
        self.bits, self.perchannel, self.sym, self.mse = bits, perchannel, sym, mse
        self.norm, self.grid, self.maxshrink = norm, grid, maxshrink
        self.weight_groupsize = weight_groupsize
        self.maxq = torch.tensor(maxq_for(bits, sym))

    def find_params(self, x):
        if self.bits == 16:
            return
        self.scale, self.zero = find_params(x, self.bits, self.perchannel, self.sym, self.mse,
                                            self.norm, self.grid, self.maxshrink)

    def quantize(self, x):
        if self.ready() and self.bits < 16:
            return ste_quantize(x, self.scale, self.zero, int(self.maxq), self.sym)
        return x

    def fake_quantize(self, x, st_idx=None, end_idx=None):
        if self.ready() and self.bits < 16:
            return fake_quantize(x, self.scale, int(self.maxq), st_idx, end_idx)
        return None, None, None

    def enabled(self):
        return self.maxq > 0

    def ready(self):
        return bool(torch.all(self.scale != 0))


def compute_quant_clip_bounds(scale, zero, maxq, sym):
    """gptq_utils/gptq_plus_utils.py:197-203."""
    scale = scale.clamp(min=1e-8)
    maxq_value = int(maxq.item()) if isinstance(maxq, torch.Tensor) else int(maxq)
    if sym:
        return scale * (-(maxq_value + 1)), scale * maxq_value
    return scale * (-zero), scale * (maxq_value - zero)


def clip_weight_to_quant_bounds(weight, bits, sym, mse):
    """clip_module_weight_to_quant_bounds_ on a bare tensor (gptq_utils/gptq_plus_utils.py:206-225): the clipped
    weight in the input's dtype (the input itself when nothing is to be done)."""
    if bits >= 16 or not mse:
        return weight
    q = OracleWeightQuantizer()
    q.configure(bits, perchannel=True, sym=sym, mse=mse)
    w = weight.float()
    q.find_params(w)
    lo, hi = compute_quant_clip_bounds(q.scale, q.zero, q.maxq, q.sym)
    return torch.minimum(torch.maximum(w, lo.to(w.dtype)), hi.to(w.dtype)).to(weight.dtype)


def act_find_params(x, bits, groupsize=-1, sym=False, clip_ratio=1.0):
    """ActQuantizer.find_params (utils/quant_utils.py:133-206): (scale, zero, maxq), scale / zero of x's shape."""
    maxq = torch.tensor(2 ** (bits - 1) - 1) if sym else torch.tensor(2 ** bits - 1)
    init_shape = x.shape
    if groupsize > 0:
        reshaped_x = x.reshape(-1, x.shape[-2], x.shape[-1] // groupsize, groupsize)
        xmax = torch.amax(reshaped_x, dim=3, keepdim=True) * clip_ratio
        xmin = torch.amin(reshaped_x, dim=3, keepdim=True) * clip_ratio
        if sym:
            xmax = torch.maximum(torch.abs(xmin), xmax)
            tmp = xmax == 0
            scale = xmax / maxq
            scale[tmp] = 1
            zero = torch.zeros_like(scale)
        else:
            tmp = (xmin == 0) & (xmax == 0)
            xmin[tmp] = -1
            xmax[tmp] = +1
            scale = (xmax - xmin) / maxq
            zero = torch.round(-xmin / scale)
        return (scale.repeat(1, 1, 1, groupsize).reshape(init_shape),
                zero.repeat(1, 1, 1, groupsize).reshape(init_shape), maxq)
    reshaped_x = x.reshape((-1, x.shape[-1]))
    tmp = torch.zeros(reshaped_x.shape[0])
    xmin = torch.minimum(reshaped_x.min(1)[0], tmp) * clip_ratio
    xmax = torch.maximum(reshaped_x.max(1)[0], tmp) * clip_ratio
    if sym:
        xmax = torch.maximum(torch.abs(xmin), xmax)
        tmp = xmax == 0
        scale = (xmax / maxq).unsqueeze(1).repeat(1, reshaped_x.shape[-1])
        scale[tmp] = 1
        scale = scale.reshape(init_shape)
        zero = torch.zeros_like(scale)
    else:
        tmp = (xmin == 0) & (xmax == 0)
        xmin[tmp] = -1
        xmax[tmp] = +1
        scale = (xmax - xmin) / maxq
        zero = torch.round(-xmin / scale)
        scale = scale.unsqueeze(1).repeat(1, reshaped_x.shape[-1]).reshape(init_shape)
        zero = zero.unsqueeze(1).repeat(1, reshaped_x.shape[-1]).reshape(init_shape)
    return scale, zero, maxq


def act_fake_quant(x, bits, groupsize=-1, sym=False, clip_ratio=1.0):
    """ActQuantizer.find_params + forward (utils/quant_utils.py:103-110): the fake-quantized activations."""
    if bits == 16:
        return x
    scale, zero, maxq = act_find_params(x, bits, groupsize, sym, clip_ratio)
    if sym:
        q = torch.clamp(torch.round(x / scale), -(maxq + 1), maxq)
        return (scale * q).to(x.dtype)
    q = torch.clamp(torch.round(x / scale) + zero, 0, maxq)
    return (scale * (q - zero)).to(x.dtype)


def weight_groupwise_params(x, bits, groupsize, sym, mse=False, norm=2.4, grid=50, maxshrink=0.5):
    """WeightQuantizer.find_params_weight_groupwise (utils/quant_utils.py:333-388), with the optional shrink-grid
    search: (scale, zero, maxq) with scale / zero of x's shape, in x's dtype."""
    maxq = torch.tensor(2 ** (bits - 1) - 1) if sym else torch.tensor(2 ** bits - 1)
    init_shape = x.shape
    xr = x.reshape(x.shape[-2], x.shape[-1] // groupsize, groupsize)
    xmax = torch.amax(xr, dim=-1, keepdim=True)
    xmin = torch.amin(xr, dim=-1, keepdim=True)
    if sym:
        scale = torch.maximum(torch.abs(xmin), xmax).clamp(min=1e-5) / maxq
        zero = torch.zeros_like(scale)
    else:
        tmp = (xmin == 0) & (xmax == 0)
        xmin[tmp] = -1
        xmax[tmp] = +1
        scale = (xmax - xmin).clamp(min=1e-5) / maxq
        zero = torch.round(-xmin / scale)
    scale = scale.repeat(1, 1, groupsize)
    zero = zero.repeat(1, 1, groupsize)
    if mse:                                                             # :355-385
        best = torch.full([xr.shape[0], xr.shape[1]], float("inf")).type_as(xr)
        steps = int(maxshrink * grid)
        for i in range(steps):
            for j in range(steps):
                lo1 = (1 - i / grid) * xmin
                hi1 = (1 - j / grid) * xmax
                if sym:
                    s1 = (torch.maximum(torch.abs(lo1), hi1).clamp(min=1e-5) / maxq).repeat(1, 1, groupsize)
                    z1 = torch.zeros_like(s1)
                    q = s1 * torch.clamp(torch.round(xr / s1), -(maxq + 1), maxq)
                else:
                    s1 = (hi1 - lo1) / maxq
                    z1 = torch.round(-lo1 / s1).repeat(1, 1, groupsize)
                    s1 = s1.repeat(1, 1, groupsize)
                    q = s1 * (torch.clamp(torch.round(xr / s1) + z1, 0, maxq) - z1)
                q -= xr
                q.abs_()
                q.pow_(norm)
                err = torch.sum(q, -1)
                better = err < best
                if torch.any(better):
                    best[better] = err[better]
                    scale[better] = s1[better]
                    zero[better] = z1[better]
    return scale.reshape(init_shape), zero.reshape(init_shape), maxq


def weight_groupwise_rtn(x, bits, groupsize, sym):
    """Round-to-nearest of a weight with grouped ranges as rtn_fwrd applies it (gptq_utils/gptq_utils.py:339-350):
    fake_quantize (symmetric clamp, zero ignored) -> (dequantized, codes, scale), plus quantize() (zero honoured)."""
    scale, zero, maxq = weight_groupwise_params(x, bits, groupsize, sym)
    q = torch.clamp(torch.round(x / scale), -(maxq + 1), maxq)
    fake = (scale * q).to(x.dtype)
    ste = ste_quantize(x, scale, zero, int(maxq), sym).to(x.dtype)
    return fake, q, scale, zero, ste
