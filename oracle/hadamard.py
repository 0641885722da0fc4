"""Oracle: Walsh-Hadamard rotation ``y = x . H_n / sqrt(n)`` with ``n = K * 2^m``.

Test infrastructure (see ``oracle/__init__.py``).  Restates
``utils/hadamard_utils.py`` of the reference:

* ``_hadamard_transform_torch``  (:11-28)  unnormalised power-of-two butterflies
* ``matmul_hadU``                (:101-118) butterflies down to K chunks, then the KxK mix
* ``matmul_hadU_cuda``           (:121-130) FWHT on ``[-1, K, n/K]``, ``/sqrt(n)``, ``hadK @``
* ``get_hadK`` selection rule    (:37-53)   smallest K with n % K == 0 and n/K a power of two

The reference's fast path is the third-party ``fast_hadamard_transform`` wheel
(Dao-AILab; not pinned in ``requirements.txt``, not vendored; call sites
:5-8, :31-34).  Its published algorithm is the same unnormalised Sylvester
butterfly network evaluated in fp32, which is what ``fwht_pow2`` computes.
"""
from __future__ import annotations

import math

import torch


def is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def fwht_pow2(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Sylvester-ordered WHT over the last dim (hadamard_utils.py:11-28).

    Returns a new tensor; the input is never modified (the reference fallback
    mutates a contiguous input in place, which callers here must not rely on).
    """
    n = x.shape[-1]
    if not is_pow2(n):
        raise ValueError(f"power-of-two length required, got {n}")
    y = x.reshape(-1, n).clone()
    h = 1
    while h < n:
        v = y.view(-1, n // (2 * h), 2, h)
        a = v[:, :, 0, :].clone()
        b = v[:, :, 1, :].clone()
        v[:, :, 0, :] = a + b
        v[:, :, 1, :] = a - b
        h *= 2
    return y.view(x.shape)


def pick_K(n: int, available) -> int:
    """Smallest tabulated K with n % K == 0 and n // K a power of two; 1 for powers of two
    (hadamard_utils.py:37-53)."""
    if is_pow2(n):
        return 1
    for k in sorted(available):
        if n % k == 0 and is_pow2(n // k):
            return k
    raise ValueError(f"no Hadamard factorisation for size {n}")


def rotate(x: torch.Tensor, hadK: torch.Tensor | None, K: int) -> torch.Tensor:
    """``matmul_hadU_cuda`` (hadamard_utils.py:121-130): FWHT along the contiguous
    ``n/K`` chunks, divide by sqrt(n), then mix the K chunks with ``hadK`` in the
    input dtype."""
    n = x.shape[-1]
    root = torch.tensor(n).sqrt()
    if K == 1:
        return fwht_pow2(x.contiguous()) / root
    v = x.reshape(-1, K, n // K)
    v = fwht_pow2(v.contiguous()) / root
    v = hadK.to(v.dtype) @ v
    return v.reshape(x.shape)


def rotate_exact(x: torch.Tensor, hadK: torch.Tensor | None, K: int) -> torch.Tensor:
    """Same operator evaluated in fp64 from any input dtype: the mathematically
    exact target that a kernel with fp32 internals is compared against."""
    n = x.shape[-1]
    v = x.double().reshape(-1, K, n // K)
    v = fwht_pow2(v)
    if K > 1:
        v = hadK.double() @ v
    return (v / math.sqrt(n)).reshape(x.shape)


def rotate_strided(x: torch.Tensor, hadK: torch.Tensor | None, K: int) -> torch.Tensor:
    """``matmul_hadU`` (hadamard_utils.py:101-118): radix-2 stages on a ``[rows, n, 1]``
    view until K groups remain, ``hadK @`` over those, then ``/sqrt(n)``.  Equal to
    :func:`rotate` up to rounding."""
    n = x.shape[-1]
    src = x.clone().reshape(-1, n, 1)
    dst = src.clone()
    while src.shape[1] > K:
        src = src.view(src.shape[0], src.shape[1] // 2, 2, src.shape[2])
        dst = dst.view(src.shape)
        dst[:, :, 0, :] = src[:, :, 0, :] + src[:, :, 1, :]
        dst[:, :, 1, :] = src[:, :, 0, :] - src[:, :, 1, :]
        dst = dst.view(src.shape[0], src.shape[1], -1)
        src, dst = dst, src
    if K > 1:
        src = hadK.view(1, K, K).to(src) @ src
    return src.view(x.shape) / torch.tensor(n).sqrt()


def qk_rotate_quant(q, k, k_bits=16, k_groupsize=-1, k_sym=False, k_clip_ratio=1.0):
    """QKRotationWrapper.forward after the wrapped function (utils/rotation_utils.py:231-260): head-dim Hadamard of
    q and k in fp32, then token-wise or head-wise fake quantization of k."""
    import math
    from .quantizer import act_fake_quant
    dtype = q.dtype
    q = (fwht_pow2(q.float()).reshape(q.shape) / math.sqrt(q.shape[-1])).to(dtype)
    k = (fwht_pow2(k.float()).reshape(k.shape) / math.sqrt(k.shape[-1])).to(dtype)
    if k_bits >= 16:
        return q, k
    bsz, num_heads, seq_len, head_dim = k.shape
    if k_groupsize == -1:
        tok = k.transpose(1, 2).reshape(-1, num_heads * head_dim)
        k = act_fake_quant(tok, k_bits, -1, k_sym, k_clip_ratio).reshape(bsz, seq_len, num_heads, head_dim).transpose(1, 2).to(q)
    else:
        k = act_fake_quant(k.reshape(-1, head_dim), k_bits, -1, k_sym, k_clip_ratio).reshape(bsz, num_heads, seq_len, head_dim).to(q)
    return q, k
