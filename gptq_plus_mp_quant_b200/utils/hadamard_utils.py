"""Hadamard rotation on B200: same names and argument meaning as the reference's
``utils/hadamard_utils.py`` (:11-172), backed by the ``rq_fwht`` kernel.

``y = x . H_n / sqrt(n)`` with ``n = K * 2^m``: a power-of-two Walsh-Hadamard transform along
each contiguous ``n/K`` chunk followed by a ``K x K`` Hadamard mix across the chunks.  The
kernel computes in fp32 whatever the I/O dtype and never modifies its input (the reference's
torch fallback mutates a contiguous input in place, hadamard_utils.py:12,22-25; no caller
relies on that).
"""
from __future__ import annotations

import math
import os
from functools import lru_cache

import torch

from .. import _lib


def is_pow2(n: int) -> bool:
    return (n & (n - 1) == 0) and (n > 0)


# --------------------------------------------------------------------------------------
# K x K Hadamard matrices for the non-power-of-two factor
# --------------------------------------------------------------------------------------
def _is_prime(n: int) -> bool:
    return n > 1 and all(n % p for p in range(2, int(n ** 0.5) + 1))


def _legendre(a: int, q: int) -> int:
    a %= q
    if a == 0:
        return 0
    return 1 if pow(a, (q - 1) // 2, q) == 1 else -1


def _paley1(q: int) -> torch.Tensor:
    """Order q+1, q prime = 3 (mod 4): first row (1, -1, ..., -1), first column ones, core
    ``I + [chi(i-j)]``."""
    K = q + 1
    H = torch.ones(K, K)
    H[0, 1:] = -1
    chi = [_legendre(d, q) for d in range(q)]
    for i in range(q):
        for j in range(q):
            if i != j:
                H[i + 1, j + 1] = chi[(i - j) % q]
    return H


def _paley2(q: int) -> torch.Tensor:
    """Order 2(q+1), q prime = 1 (mod 4): ``[[C+I, C-I], [C-I, -(C+I)]]`` with the symmetric
    conference matrix ``C = [[0, 1], [1, chi(i-j)]]``."""
    m = q + 1
    Cm = torch.ones(m, m)
    Cm[0, 0] = 0
    chi = [_legendre(d, q) for d in range(q)]
    for i in range(q):
        for j in range(q):
            Cm[i + 1, j + 1] = chi[(i - j) % q]
    eye = torch.eye(m)
    top = torch.cat([Cm + eye, Cm - eye], dim=1)
    bot = torch.cat([Cm - eye, -(Cm + eye)], dim=1)
    return torch.cat([top, bot], dim=0)


# orders of the reference's table (utils/had_mat.pt) and how each is obtained here
TABLE_ORDERS = (12, 20, 28, 36, 44, 52, 60, 68, 76, 84, 92, 100, 108, 116, 124, 132, 140, 148, 156, 164,
                172, 180, 188, 204, 212, 220, 228, 236, 244, 252)
_PALEY2_ORDERS = {28: 13, 36: 17, 76: 37, 148: 73, 204: 101, 220: 109}


def _unpack(K: int) -> torch.Tensor:
    import base64

    import numpy as np

    from ._had_tables import PACKED
    bits = np.unpackbits(np.frombuffer(base64.b64decode(PACKED[K]), dtype=np.uint8))[:K * K]
    return torch.from_numpy(bits.astype(np.float32) * 2.0 - 1.0).reshape(K, K)


@lru_cache(maxsize=None)
def hadamard_of_order(K: int) -> torch.Tensor:
    """The K x K (+-1) matrix the reference stores for order K (utils/had_mat.pt).  Orders with a Paley
    construction are generated (and are identical to the stored ones); the other thirteen come from the bit-packed
    table in ``_had_tables.py``."""
    if K in _PALEY2_ORDERS:
        return _paley2(_PALEY2_ORDERS[K])
    if K in TABLE_ORDERS and _is_prime(K - 1) and (K - 1) % 4 == 3 and K not in (212, 228, 252):
        return _paley1(K - 1)
    if K in TABLE_ORDERS:
        return _unpack(K)
    raise ValueError(f"no Hadamard matrix of order {K}: the table holds {TABLE_ORDERS}")


def get_hadK(n, transpose=False):
    """(hadK, K): smallest tabulated K with n % K == 0 and n // K a power of two; (None, 1) for
    powers of two (hadamard_utils.py:37-53)."""
    if is_pow2(n):
        return None, 1
    for k in TABLE_ORDERS:
        if n % k == 0 and is_pow2(n // k):
            hadK = hadamard_of_order(k)
            return (hadK.T if transpose else hadK), k
    raise ValueError(f"Can't find appropriate Hadamard for size {n}!")


# --------------------------------------------------------------------------------------
# kernel wrapper
# --------------------------------------------------------------------------------------
_HADK_DEV = {}


def _hadK_on(device, hadK: torch.Tensor) -> torch.Tensor:
    """Device copy of a K x K mixing matrix.  Only the matrices that hadamard_of_order hands out (kept alive by its
    cache, never modified) are remembered, keyed by their order and orientation; a caller's own matrix is copied on
    every call, so a freed or edited tensor can never be confused with a cached one."""
    K = hadK.shape[0]
    if K in TABLE_ORDERS:
        base = hadamard_of_order(K)
        for tag, cand in (("n", base), ("t", base.T)):
            if hadK.data_ptr() == cand.data_ptr() and hadK.stride() == cand.stride() and hadK.shape == cand.shape:
                key = (str(device), K, tag)
                t = _HADK_DEV.get(key)
                if t is None:
                    t = _HADK_DEV[key] = cand.to(device=device, dtype=torch.float32).contiguous()
                return t
    return hadK.detach().to(device=device, dtype=torch.float32).contiguous()


def fwht(x: torch.Tensor, hadK=None, K: int = 1, scale: float = 1.0, out: torch.Tensor | None = None):
    """``out = (x viewed [-1, K, n/K]) FWHT along last dim, then hadK-mix, times scale``."""
    _lib.require_cuda(x)
    n = x.shape[-1]
    xc = x.contiguous()
    if out is None:
        out = torch.empty_like(xc)
    rows = xc.numel() // n if n else 0
    if rows == 0:
        return out.view(x.shape)
    hk = _hadK_on(x.device, hadK) if K > 1 else None
    with torch.cuda.device(x.device):
        rc = _lib.lib.rq_fwht(_lib.ptr(xc), _lib.ptr(out), _lib.dtype_code(xc), rows, n, K, _lib.ptr(hk),
                              float(scale), _lib.stream_of(xc))
    _lib.check("rq_fwht", rc)
    return out.view(x.shape)


def fwht_act_quant(x: torch.Tensor, hadK, K: int, scale: float, clip_ratio: float, maxq: int, sym: bool):
    """Rotation and per-token fake quantization in one kernel (``rq_fwht_act_quant``); None when the shape is not one
    the fused kernel covers, so that the caller runs the two kernels in turn."""
    _lib.require_cuda(x)
    n = x.shape[-1]
    xc = x.contiguous()
    rows = xc.numel() // n if n else 0
    if rows == 0:
        return torch.empty_like(xc).view(x.shape)
    out = torch.empty_like(xc)
    hk = _hadK_on(x.device, hadK) if K > 1 else None
    with torch.cuda.device(x.device):
        rc = _lib.lib.rq_fwht_act_quant(_lib.ptr(xc), _lib.ptr(out), _lib.dtype_code(xc), rows, n, K, _lib.ptr(hk),
                                        float(scale), float(clip_ratio), int(maxq), 1 if sym else 0, None, None,
                                        _lib.stream_of(xc))
    if rc == _lib.RQ_ERR_UNSUPPORTED:
        return None
    _lib.check("rq_fwht_act_quant", rc)
    return out.view(x.shape)


def fwht_heads(x: torch.Tensor, heads: int, head_dim: int, hadK=None, K: int = 1, scale: float = 1.0) -> torch.Tensor:
    """Hadamard transform across the ``heads`` of ``x[..., heads * head_dim]`` for every position inside a head (the
    online partial rotation of utils/quant_utils.py:258-281), times ``scale``.  ``K == 1``: Sylvester order;
    otherwise ``hadK`` [K, K] mixes the ``heads / K``-long power-of-two chunks (``K == heads``: a dense matrix)."""
    _lib.require_cuda(x)
    assert x.shape[-1] == heads * head_dim
    xc = x.contiguous()
    out = torch.empty_like(xc)
    hk = None
    if K > 1:
        hk = _hadK_on(x.device, hadK)
    with torch.cuda.device(x.device):
        rc = _lib.lib.rq_fwht_heads(_lib.ptr(xc), _lib.ptr(out), _lib.dtype_code(xc), xc.numel() // (heads * head_dim),
                                    int(heads), int(head_dim), int(K), _lib.ptr(hk), float(scale), _lib.stream_of(xc))
    _lib.check("rq_fwht_heads", rc)
    return out


class HadamardTransform(torch.autograd.Function):
    """The unnormalised Hadamard transform over the last (power-of-two) dim; its own adjoint
    (hadamard_utils.py:89-98)."""

    @staticmethod
    def forward(ctx, u):
        return fwht(u)

    @staticmethod
    def backward(ctx, grad):
        return fwht(grad)


def matmul_hadU_cuda(X, hadK, K):
    """hadamard_utils.py:121-130."""
    n = X.shape[-1]
    return fwht(X, hadK, K, scale=1.0 / math.sqrt(n))


def matmul_hadU(X, transpose=False):
    """hadamard_utils.py:101-118 (same operator, picks hadK itself)."""
    n = X.shape[-1]
    hadK, K = get_hadK(n, transpose)
    if X.dtype == torch.float64:                       # offline fp64 callers (random_hadamard_matrix)
        return _matmul_hadU_fp64(X, hadK, K)
    return fwht(X, hadK, K, scale=1.0 / math.sqrt(n))


def _matmul_hadU_fp64(X, hadK, K):
    """Double-precision evaluation with torch ops for the offline construction of rotation
    matrices; the kernel path covers the fp32 / bf16 / fp16 activations and weights."""
    n = X.shape[-1]
    P = n // K
    v = X.reshape(-1, K, P).clone()
    h = 1
    while h < P:
        w = v.view(-1, K, P // (2 * h), 2, h)
        a = w[..., 0, :].clone()
        b = w[..., 1, :].clone()
        w[..., 0, :] = a + b
        w[..., 1, :] = a - b
        h *= 2
    if K > 1:
        v = hadK.to(v) @ v
    return v.reshape(X.shape) / torch.tensor(n).sqrt()


def random_orthogonal_matrix(size, device, generator=None):
    """hadamard_utils.py:56-73: the Q factor of a standard normal fp64 matrix (drawn on the host with
    ``generator``), its columns signed so that the R factor would have a positive diagonal, which makes the result a
    draw from the Haar measure rather than whatever the QR routine's sign convention gives."""
    gauss = torch.randn(size, size, dtype=torch.float64, generator=generator).to(device)
    q, r = torch.linalg.qr(gauss)
    return q * torch.sign(torch.diagonal(r)).unsqueeze(0)


def random_hadamard_matrix(size, device, generator=None):
    """hadamard_utils.py:76-80: rows of the normalised Hadamard matrix with random signs."""
    Q = torch.randint(low=0, high=2, size=(size,), generator=generator).to(torch.float64)
    Q = Q * 2 - 1
    Q = torch.diag(Q)
    return matmul_hadU(Q.to(device)).to(device)


def hadamard_matrix(size, device):
    """hadamard_utils.py:83-86."""
    return matmul_hadU(torch.eye(size, device=device)).to(device)


def apply_exact_had_to_linear(module, had_dim=-1, output=False, R2=None):
    """Fuse a Hadamard rotation into a linear's weight (hadamard_utils.py:133-168): the full-width
    rotation runs through the FWHT kernel in fp32; the per-head variant is an fp64 matmul."""
    assert isinstance(module, torch.nn.Linear)
    in_features, out_features = module.in_features, module.out_features
    if had_dim != -1:
        assert is_pow2(had_dim), "Hadamard dimension must be a power of 2!"
    W_ = module.weight.data
    dtype, dev = W_.dtype, W_.device
    W_ = W_.float().cuda()
    if had_dim == -1:
        if output:
            had_K, K = get_hadK(out_features)
            W_ = matmul_hadU_cuda(W_.t(), had_K, K).t()
        else:
            had_K, K = get_hadK(in_features)
            W_ = matmul_hadU_cuda(W_, had_K, K)
    else:
        hadK = hadamard_matrix(had_dim, "cuda").to(torch.float64)
        if R2 is not None:
            hadK = R2.to(torch.float64)
        if output:
            W_ = W_.t()
            shp = W_.shape
            temp = W_.reshape(-1, shp[-1] // had_dim, had_dim).to(torch.float64) @ hadK
            W_ = temp.reshape(shp).t()
        else:
            shp = W_.shape
            temp = W_.reshape(-1, shp[-1] // had_dim, had_dim).to(torch.float64) @ hadK
            W_ = temp.reshape(shp)
    module.weight.data = W_.to(device=dev, dtype=dtype)
