"""Weight quantizer on B200: the ``WeightQuantizer`` / STE interface of the reference's
``utils/quant_utils.py`` (:21-84, :300-486) over the ``rq_find_params`` / ``rq_quantize``
kernels, and the activation-side ``ActQuantizer`` / ``ActQuantWrapper`` (:87-297) over
``rq_act_quant`` and the rotation kernels.  Names, arguments, buffer shapes and error behaviour
follow the reference, including the grouped variant of the weight quantizer
(``weight_groupsize > 0``, :333-388: ranges per row and column group in the weight's dtype, with
or without the shrink-grid search).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import _lib


def get_minq_maxq(bits, sym):
    """quant_utils.py:21-29."""
    if sym:
        maxq = torch.tensor(2 ** (bits - 1) - 1)
        minq = -maxq - 1
    else:
        maxq = torch.tensor(2 ** bits - 1)
        minq = 0
    return minq, maxq


def _row_params(x: torch.Tensor, scale: torch.Tensor, zero):
    """Flatten scale/zero to one fp32 entry per row of ``x`` viewed ``[R, C]`` (or a single entry)."""
    R = x.shape[0] if x.dim() > 1 else 1
    s = scale.to(device=x.device, dtype=torch.float32).reshape(-1)
    z = None if zero is None else zero.to(device=x.device, dtype=torch.float32).reshape(-1)
    if s.numel() == 1:
        return s.contiguous(), (None if z is None else z.contiguous()), 1
    if s.numel() != R:
        raise ValueError(f"scale has {s.numel()} entries for {R} rows")
    return s.contiguous(), (None if z is None else z.contiguous()), 0


def quantize_dequantize(x: torch.Tensor, scale, zero, maxq, honour_zero: bool, want_codes: bool = False):
    """One kernel pass: ``(dequantized in x.dtype, integer codes fp32 or None)``."""
    _lib.require_cuda(x)
    xc = x.contiguous()
    R = xc.shape[0] if xc.dim() > 1 else 1
    Ccols = xc.numel() // R if R else 0
    s, z, pertensor = _row_params(xc, scale, zero if honour_zero else None)
    deq = torch.empty_like(xc)
    codes = torch.empty(xc.shape, dtype=torch.float32, device=xc.device) if want_codes else None
    with torch.cuda.device(xc.device):
        rc = _lib.lib.rq_quantize(_lib.ptr(xc), _lib.ptr(deq), _lib.ptr(codes), _lib.dtype_code(xc), R, Ccols,
                                  _lib.ptr(s), _lib.ptr(z), pertensor, int(maxq), 1 if honour_zero else 0,
                                  _lib.stream_of(xc))
    _lib.check("rq_quantize", rc)
    return deq, codes


def sym_quant(x, scale, maxq):
    """quant_utils.py:47-50."""
    _, q = quantize_dequantize(x, scale, None, maxq, False, want_codes=True)
    return q.to(x.dtype), scale.to(x.device)


def sym_dequant(q, scale):
    return scale * q


def sym_quant_dequant(x, scale, maxq):
    """quant_utils.py:57-58."""
    return quantize_dequantize(x, scale, None, maxq, False)[0]


def asym_quant(x, scale, zero, maxq):
    """quant_utils.py:32-36."""
    _, q = quantize_dequantize(x, scale, zero, maxq, True, want_codes=True)
    return q.to(x.dtype), scale.to(x.device), zero.to(x.device)


def asym_dequant(q, scale, zero):
    return scale * (q - zero)


def asym_quant_dequant(x, scale, zero, maxq):
    """quant_utils.py:43-44."""
    return quantize_dequantize(x, scale, zero, maxq, True)[0]


class STEQuantize(torch.autograd.Function):
    """Symmetric quantize-dequantize with a straight-through gradient (quant_utils.py:60-71)."""

    @staticmethod
    def forward(ctx, x, scale, maxq):
        return quantize_dequantize(x, scale, None, maxq, False)[0]

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None, None


class AsymSTEQuantize(torch.autograd.Function):
    """Asymmetric variant (quant_utils.py:74-84)."""

    @staticmethod
    def forward(ctx, x, scale, zero, maxq):
        return quantize_dequantize(x, scale, zero, maxq, True)[0]

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None, None, None


class ActQuantizer(torch.nn.Module):
    """Dynamic per-token (``groupsize <= 0``) or per-token-group activation quantizer (utils/quant_utils.py:87-206),
    both symmetric and asymmetric.  Ranges and the quantize-dequantize run in one kernel that rounds every
    intermediate to the tensor's dtype exactly as the reference's chain of torch ops does.  The ranges are kept as one
    scale / zero per token (or token group); ``scale`` / ``zero`` expand them to the input's shape on request."""

    def __init__(self) -> None:
        super().__init__()
        self.register_buffer("maxq", torch.tensor(0))
        self._scale = self._zero = None
        self._shape = None
        self.bits = 16

    def free(self) -> None:
        self._scale = self._zero = None
        self._shape = None

    def configure(self, bits: int, groupsize: int = -1, sym: bool = False, clip_ratio: float = 1.0) -> None:
        _, self.maxq = get_minq_maxq(bits, sym)
        self.bits = bits
        self.groupsize = groupsize
        self.sym = sym
        self.clip_ratio = clip_ratio
        assert self.clip_ratio <= 1 and self.clip_ratio > 0, "Clip ratio should be in (0, 1]"

    def _units(self, x):
        n = x.shape[-1]
        if self.groupsize > 0:
            if n % self.groupsize != 0:
                raise ValueError(f"last dimension {n} is not divisible by groupsize {self.groupsize}")
            return x.numel() // self.groupsize, self.groupsize, 0
        return x.numel() // n, n, 1

    def _run(self, x, out, scale_out, zero_out, scale_in, zero_in, codes=False):
        _lib.require_cuda(x)
        units, length, with_zero = self._units(x)
        with torch.cuda.device(x.device):
            rc = _lib.lib.rq_act_quant(_lib.ptr(x), _lib.ptr(out), _lib.dtype_code(x), units, length, with_zero,
                                       float(self.clip_ratio), int(self.maxq), 1 if self.sym else 0,
                                       _lib.ptr(scale_out), _lib.ptr(zero_out), _lib.ptr(scale_in), _lib.ptr(zero_in),
                                       1 if codes else 0, 0 if with_zero else 1, 0, _lib.stream_of(x))
        _lib.check("rq_act_quant", rc)

    def find_params_per_token_groupwise(self, x) -> None:
        """Ranges per token and group of ``groupsize`` channels (utils/quant_utils.py:131-153)."""
        if self.groupsize <= 0:
            raise ValueError("find_params_per_token_groupwise needs groupsize > 0")
        self.find_params(x)

    def find_params(self, x) -> None:
        if self.bits == 16:
            return
        x = x.contiguous()
        units, _, _ = self._units(x)
        self._scale = torch.empty(units, dtype=torch.float32, device=x.device)
        self._zero = torch.zeros(units, dtype=torch.float32, device=x.device)
        self._shape, self._dtype = tuple(x.shape), x.dtype
        self._run(x, None, self._scale, self._zero, None, None)

    def _expand(self, v):
        if v is None:
            return None
        per = 1
        for d in self._shape:
            per *= d
        per //= v.numel()
        # group-wise ranges live in the input's dtype; the per-token path of the reference promotes them to fp32
        dt = self._dtype if self.groupsize > 0 else torch.float32
        return v.to(dt).repeat_interleave(per).reshape(self._shape)

    @property
    def scale(self):
        return self._expand(self._scale)

    @property
    def zero(self):
        return self._expand(self._zero)

    def forward(self, x):
        if self.bits == 16:
            return x
        xc = x.contiguous()
        out = torch.empty_like(xc)
        self._run(xc, out, None, None, self._scale, self._zero)
        return out

    def fake_quant(self, x):
        """find_params + forward + free in one pass (what ActQuantWrapper.forward does around every linear)."""
        if self.bits == 16:
            return x
        xc = x.contiguous()
        out = torch.empty_like(xc)
        self._run(xc, out, None, None, None, None)
        return out

    def quantize(self, x):
        """Integer codes with the stored ranges (utils/quant_utils.py:112-117): (q, scale) or (q, scale, zero)."""
        xc = x.contiguous()
        q = torch.empty_like(xc)
        self._run(xc, q, None, None, self._scale, self._zero, codes=True)
        return (q, self.scale) if self.sym else (q, self.scale, self.zero)


class ActQuantWrapper(torch.nn.Module):
    """Linear wrapped with an optional online Hadamard rotation and dynamic input / output fake quantization
    (utils/quant_utils.py:209-297): rotation and quantization are one kernel each."""

    def __init__(self, module) -> None:
        super().__init__()
        self.module = module
        self.weight = module.weight
        self.bias = module.bias
        self.quantizer = ActQuantizer()
        self.out_quantizer = ActQuantizer()
        self.register_buffer("had_K", torch.tensor(0))
        self._buffers["had_K"] = None
        self.K = 1
        self.online_full_had = False
        self.online_partial_had = False
        self.had_dim = 0
        self.fp32_had = False

    def extra_repr(self) -> str:
        def kind(q):
            return "" if q.bits >= 16 else (" (Symmetric Per-Token)" if q.sym else " (Asymmetric Per-Token)")
        return (f"Input Quantizer Bits: {self.quantizer.bits}{kind(self.quantizer)}"
                f"\nOutput Quantizer Bits: {self.out_quantizer.bits}{kind(self.out_quantizer)}")

    def forward(self, x, R1=None, R2=None, transpose=False):
        from . import hadamard_utils
        x_dtype = x.dtype
        q = self.quantizer
        if (self.online_full_had and q.bits < 16 and q.groupsize <= 0 and self.K == 1 and x.shape[-1] <= 4096
                and (not self.fp32_had or x_dtype == torch.float32)):
            # rotation and per-token quantization in one pass over the activations; the quantizer's correctly rounded
            # divisions take much of the issue bandwidth in either form, and only up to 4096-long rows did the fused
            # kernel measure faster than the two in turn
            import math
            y = hadamard_utils.fwht_act_quant(x, self.had_K, self.K, 1.0 / math.sqrt(x.shape[-1]), q.clip_ratio,
                                              int(q.maxq), q.sym)
            if y is not None:
                x = (self.module(y, R1, R2, transpose) if R1 is not None else self.module(y)).to(x_dtype)
                if self.out_quantizer.bits < 16:
                    x = self.out_quantizer.fake_quant(x).to(x_dtype)
                return x
        if self.online_full_had:
            if self.fp32_had:
                x = hadamard_utils.matmul_hadU_cuda(x.float(), self.had_K, self.K).to(x_dtype)
            else:
                x = hadamard_utils.matmul_hadU_cuda(x, self.had_K, self.K)
        elif self.online_partial_had:
            import math
            heads = x.shape[-1] // self.had_dim
            if self.fp32_had:
                x = x.float()
            if self.K == 1:
                x = hadamard_utils.fwht_heads(x, heads, self.had_dim, None, 1, 1.0 / math.sqrt(heads))
            else:                                           # dense had_K [heads, heads] applied across the heads
                x = hadamard_utils.fwht_heads(x, heads, self.had_dim, self.had_K, heads, 1.0 / math.sqrt(heads))
            if self.fp32_had:
                x = x.to(x_dtype)
        if self.quantizer.bits < 16:
            x = self.quantizer.fake_quant(x).to(x_dtype)
        x = (self.module(x, R1, R2, transpose) if R1 is not None else self.module(x)).to(x_dtype)
        if self.out_quantizer.bits < 16:
            x = self.out_quantizer.fake_quant(x).to(x_dtype)
        return x


def find_params_groups(W: torch.Tensor, groupsize: int, maxq: int, sym: bool, mse: bool = False,
                       norm: float = 2.4, grid: int = 50, maxshrink: float = 0.5):
    """Per-row ranges of every ``groupsize``-wide column group in one launch:
    ``(scale, zero)`` each ``[ngroups, R]``.  Equals ``deepcopy(quantizer).find_params(W[:, g*gs:(g+1)*gs])``
    for every g (gptq_utils/gptq_plus_utils.py:995-1002)."""
    _lib.require_cuda(W)
    assert W.dim() == 2 and W.dtype == torch.float32
    R, Ccols = W.shape
    ng = (Ccols + groupsize - 1) // groupsize if groupsize > 0 else 1
    scale = torch.empty(ng, R, dtype=torch.float32, device=W.device)
    zero = torch.empty(ng, R, dtype=torch.float32, device=W.device)
    Wc = W if W.stride(1) == 1 else W.contiguous()
    with torch.cuda.device(W.device):
        rc = _lib.lib.rq_find_params(_lib.ptr(Wc), R, Ccols, Wc.stride(0), int(groupsize), 1, int(maxq),
                                     1 if sym else 0, 1 if mse else 0, float(norm), int(grid), float(maxshrink),
                                     _lib.ptr(scale), _lib.ptr(zero), _lib.stream_of(W))
    _lib.check("rq_find_params", rc)
    return scale, zero


class WeightQuantizer(torch.nn.Module):
    """Drop-in for the reference ``WeightQuantizer`` (quant_utils.py:300-486)."""

    def __init__(self, shape: int = 1) -> None:
        super().__init__()
        self.register_buffer("maxq", torch.tensor(0))
        self.register_buffer("scale", torch.zeros(shape))
        self.register_buffer("zero", torch.zeros(shape))

    def configure(self, bits, perchannel: bool = False, sym: bool = True, mse: bool = False, norm: float = 2.4,
                  grid: int = 50, maxshrink: float = 0.5, weight_groupsize: int = -1) -> None:
        self.bits = bits
        self.perchannel = perchannel
        self.sym = sym
        self.mse = mse
        self.norm = norm
        self.grid = grid
        self.maxshrink = maxshrink
        self.weight_groupsize = weight_groupsize
        if sym:
            self.maxq = torch.tensor(2 ** (bits - 1) - 1)
        else:
            self.maxq = torch.tensor(2 ** bits - 1)

    def find_params(self, x) -> None:
        if self.bits == 16:
            return
        if self.weight_groupsize > 0:
            self.find_params_weight_groupwise(x)
            return
        self._g_scale = self._g_zero = None
        _lib.require_cuda(x)
        dev = x.device
        self.maxq = self.maxq.to(dev)
        shape = x.shape
        x2 = x.flatten(1) if self.perchannel else x.flatten().unsqueeze(0)
        x2 = x2.float()
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        R, Ccols = x2.shape
        if not self.perchannel and self.mse:
            raise NotImplementedError("the shrink-grid search is provided for per-channel ranges only")
        scale = torch.empty(R, dtype=torch.float32, device=dev)
        zero = torch.empty(R, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.lib.rq_find_params(_lib.ptr(x2), R, Ccols, x2.stride(0), -1, 1, int(self.maxq),
                                         1 if self.sym else 0, 1 if self.mse else 0, float(self.norm),
                                         int(self.grid), float(self.maxshrink), _lib.ptr(scale), _lib.ptr(zero),
                                         _lib.stream_of(x2))
        _lib.check("rq_find_params", rc)
        if not self.perchannel:
            scale = scale.repeat(shape[0])
            zero = zero.repeat(shape[0])
        out_shape = [-1] + [1] * (len(shape) - 1)
        self.scale = scale.reshape(out_shape)
        self.zero = zero.reshape(out_shape)

    # ---- ranges per row and group of ``weight_groupsize`` columns (quant_utils.py:333-388), in the weight's dtype
    def _grouped_call(self, x, out, scale_out, zero_out, scale_in, zero_in, sym, codes=False):
        gs = self.weight_groupsize
        with torch.cuda.device(x.device):
            rc = _lib.lib.rq_act_quant(_lib.ptr(x), _lib.ptr(out), _lib.dtype_code(x), x.numel() // gs, gs, 0, 1.0,
                                       int(self.maxq), 1 if sym else 0, _lib.ptr(scale_out), _lib.ptr(zero_out),
                                       _lib.ptr(scale_in), _lib.ptr(zero_in), 1 if codes else 0, 1, 1, _lib.stream_of(x))
        _lib.check("rq_act_quant", rc)

    def find_params_weight_groupwise(self, x) -> None:
        _lib.require_cuda(x)
        if x.shape[-1] % self.weight_groupsize != 0:
            raise ValueError(f"columns {x.shape[-1]} not divisible by weight_groupsize {self.weight_groupsize}")
        self.maxq = self.maxq.to(x.device)
        xc = x.contiguous()
        units = xc.numel() // self.weight_groupsize
        self._g_scale = torch.empty(units, dtype=torch.float32, device=x.device)
        self._g_zero = torch.zeros(units, dtype=torch.float32, device=x.device)
        if self.mse:
            with torch.cuda.device(x.device):
                rc = _lib.lib.rq_group_mse_search(_lib.ptr(xc), _lib.dtype_code(xc), units, self.weight_groupsize,
                                                  int(self.maxq), 1 if self.sym else 0, float(self.norm),
                                                  int(self.grid), float(self.maxshrink), _lib.ptr(self._g_scale),
                                                  _lib.ptr(self._g_zero), _lib.stream_of(xc))
            _lib.check("rq_group_mse_search", rc)
        else:
            self._grouped_call(xc, None, self._g_scale, self._g_zero, None, None, self.sym)
        expand = lambda v: v.to(x.dtype).repeat_interleave(self.weight_groupsize).reshape(x.shape)   # noqa: E731
        self.scale = expand(self._g_scale)
        self.zero = expand(self._g_zero)

    def quantize(self, x):
        x_dtype = x.dtype
        if getattr(self, "_g_scale", None) is not None and self.bits < 16:
            xc = x.contiguous()
            out = torch.empty_like(xc)
            self._grouped_call(xc, out, None, None, self._g_scale, self._g_zero, self.sym)
            return out
        if self.ready() and self.bits < 16:
            if self.sym:
                return STEQuantize.apply(x, self.scale, self.maxq).to(x_dtype)
            return AsymSTEQuantize.apply(x, self.scale, self.zero, self.maxq).to(x_dtype)
        return x

    def fake_quantize(self, x, st_idx=None, end_idx=None):
        """(dequantized, integer codes, scale): always the symmetric clamp, the zero-point is
        ignored, exactly like the reference (quant_utils.py:471-480)."""
        if getattr(self, "_g_scale", None) is not None and self.bits < 16:
            scale, gsc = self.scale.to(x.device), self._g_scale
            if st_idx is not None and end_idx is not None:
                per_row = scale.shape[-1] // self.weight_groupsize
                scale, gsc = scale[st_idx:end_idx], gsc[st_idx * per_row:end_idx * per_row].contiguous()
            xc = x.contiguous()
            deq, codes = torch.empty_like(xc), torch.empty_like(xc)
            self._grouped_call(xc, deq, None, None, gsc, None, True)
            self._grouped_call(xc, codes, None, None, gsc, None, True, codes=True)
            return deq, codes, scale
        if self.ready() and self.bits < 16:
            scale = self.scale.to(x.device)
            if st_idx is not None and end_idx is not None:
                scale = scale[st_idx:end_idx]
            deq, codes = quantize_dequantize(x, scale, None, self.maxq, False, want_codes=True)
            return deq, codes.to(x.dtype), scale
        return None, None, None

    def enabled(self):
        return self.maxq > 0

    def ready(self):
        return torch.all(self.scale != 0)
