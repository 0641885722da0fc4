"""Thin torch-facing wrappers of the Hessian entry points of the C ABI: argument checks,
scratch memory taken from torch's caching allocator, current-stream plumbing."""
from __future__ import annotations

import os

import torch

from . import _lib

# tokens packed and contracted per launch pair; the scratch grows with it (about
# (2 + 2G) * C * chunk * 2 bytes)
HESSIAN_CHUNK_TOKENS = int(os.environ.get("REALQ_HESSIAN_CHUNK", "8192"))
# kernel variant of rq_hessian_accum when the caller passes none (see the header: operand layout and
# accumulation window)
HESSIAN_VARIANT = int(os.environ.get("REALQ_HESSIAN_VARIANT", "0"))

# Optional: packing on the caller's stream, tensor-core contraction on one extra stream per device, two rings of
# chunk slots, so that the packing of one linear overlaps the contraction of another.  H is then complete in
# the order of that extra stream: every reader of H calls hessian_join() first.  Off by default: on a part that
# runs against its power cap the overlap was measured to slow the contraction by as much as it hides of the
# packing (0.686 s against 0.683 s per layer); it pays where the clock is not power-limited.
HESSIAN_PIPELINE = os.environ.get("REALQ_HESSIAN_PIPELINE", "0") != "0"
_PIPE_SLOTS = 2             # chunk slots per workspace
_PIPE_RING = 2              # workspaces alternated between calls

_scratch = {}
_status = {}
_pipe = {}


class _PipeState:
    def __init__(self, device):
        self.stream = torch.cuda.Stream(device=device)
        self.turn = 0
        self.free = [None] * _PIPE_RING           # event: the contraction that last read workspace i has finished
        self.dirty = False


def _pipe_state(device) -> "_PipeState":
    st = _pipe.get(device)
    if st is None:
        st = _pipe[device] = _PipeState(device)
    return st


def hessian_join(device) -> None:
    """Make the current stream wait for every Hessian contraction issued so far on ``device``."""
    st = _pipe.get(device)
    if st is not None and st.dirty:
        torch.cuda.current_stream(device).wait_stream(st.stream)


def _workspace(device, nbytes: int, key: str = "main") -> torch.Tensor:
    """Cached scratch buffer per (device, key, current stream); grown on demand, never shrunk.  Keyed by the
    stream so that linears quantized concurrently on different streams never share scratch."""
    k = (device, key, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(k)
    if buf is None or buf.numel() < nbytes:
        _scratch[k] = None
        buf = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        _scratch[k] = buf
    return buf


def release_workspace() -> None:
    _scratch.clear()


def status_word(device) -> torch.Tensor:
    """Device int32 that kernels set when one of their bounded waits ran out."""
    t = _status.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def check_status(device) -> None:
    """Read the status word (synchronises) and raise if a kernel reported a time-out."""
    code = int(status_word(device).item())
    if code != _lib.RQ_OK:
        status_word(device).zero_()
        raise _lib.RealQError("device status", code)


def hessian_accum(x: torch.Tensor, sal, H: torch.Tensor, act_sq, alpha: float = 1.0, beta: float = 1.0,
                  variant: int | None = None, chunk_tokens: int | None = None, pipeline: bool = False) -> None:
    """``H[g] = beta*H[g] + alpha * X^T diag(sal[:, g]) X`` (upper-triangular tiles only) and
    ``act_sq += sum x^2``.  x: [N, C] fp32/bf16/fp16 (row stride free), sal: [N, G] fp32 or None,
    H: [G, C, C] fp32 contiguous (or [C, C] when sal is None).  ``pipeline=True`` issues the contraction on the
    device's extra stream (see HESSIAN_PIPELINE): H is then only complete after hessian_join()."""
    _lib.require_cuda(x, H, sal, act_sq)
    if variant is None:
        variant = HESSIAN_VARIANT
    assert x.dim() == 2, "x must be [tokens, channels]"
    N, Cc = x.shape
    if x.stride(1) != 1:
        x = x.contiguous()
    G = 1 if sal is None else sal.shape[1]
    assert H.is_contiguous() and H.dtype == torch.float32 and H.numel() == G * Cc * Cc
    if sal is not None:
        assert sal.shape[0] == N
        sal = sal.to(dtype=torch.float32).contiguous()
    if act_sq is not None:
        assert act_sq.dtype == torch.float32 and act_sq.is_contiguous() and act_sq.numel() == Cc
    chunk = int(chunk_tokens or HESSIAN_CHUNK_TOKENS)
    chunk = max(64, min(chunk, (N + 63) // 64 * 64))
    if pipeline:
        with torch.cuda.device(x.device):
            ps = _pipe_state(x.device)
            cur = torch.cuda.current_stream(x.device)
            if not ps.dirty:
                ps.stream.wait_stream(cur)        # H as the caller left it (zero-filled, or read back earlier)
            slot_bytes = _lib.lib.rq_hessian_workspace_bytes(chunk, Cc, G, 0 if sal is None else 1)
            ring = ps.turn % _PIPE_RING
            ps.turn += 1
            ws = _workspace(x.device, _PIPE_SLOTS * slot_bytes + 1024, key=f"hpipe{ring}")
            if ps.free[ring] is not None:
                cur.wait_event(ps.free[ring])
            base = ws.data_ptr()
            aligned = (base + 1023) // 1024 * 1024
            rc = _lib.lib.rq_hessian_accum_pipelined(
                _lib.ptr(x), _lib.dtype_code(x), x.stride(0), _lib.ptr(sal), _lib.ptr(H), _lib.ptr(act_sq), N, Cc, G,
                float(alpha), float(beta), aligned, _PIPE_SLOTS * slot_bytes, _lib.ptr(status_word(x.device)),
                int(variant), chunk, cur.cuda_stream, ps.stream.cuda_stream)
            ev = torch.cuda.Event()
            ev.record(ps.stream)
            ps.free[ring] = ev
            ps.dirty = True
        _lib.check("rq_hessian_accum_pipelined", rc)
        return
    with torch.cuda.device(x.device):
        need = _lib.lib.rq_hessian_workspace_bytes(chunk, Cc, G, 0 if sal is None else 1)
        ws = _workspace(x.device, need)              # the cached buffer may be larger: pass `need`, so that the
        base = ws.data_ptr()                         # chunking (hence the bits of H) never depends on its history
        aligned = (base + 1023) // 1024 * 1024
        rc = _lib.lib.rq_hessian_accum(_lib.ptr(x), _lib.dtype_code(x), x.stride(0), _lib.ptr(sal), _lib.ptr(H),
                                       _lib.ptr(act_sq), N, Cc, G, float(alpha), float(beta), aligned,
                                       need, _lib.ptr(status_word(x.device)), int(variant),
                                       _lib.stream_of(x))
    _lib.check("rq_hessian_accum", rc)


def hessian_finalize(H: torch.Tensor, act_sq, div_tokens: float = 1.0, div_scale: float = 1.0,
                     div_seq: float = 1.0, sanitize: bool = False):
    """Scale, mirror the upper triangle into the lower one, optionally zero non-finite entries.
    Returns the device uint64[2] (NaN count, Inf count) when ``sanitize`` else None."""
    _lib.require_cuda(H, act_sq)
    assert H.is_contiguous() and H.dtype == torch.float32
    hessian_join(H.device)
    Cc = H.shape[-1]
    G = H.numel() // (Cc * Cc)
    counts = torch.zeros(2, dtype=torch.int64, device=H.device) if sanitize else None
    with torch.cuda.device(H.device):
        rc = _lib.lib.rq_hessian_finalize(_lib.ptr(H), _lib.ptr(act_sq), Cc, G, float(div_tokens), float(div_scale),
                                          float(div_seq), 1 if sanitize else 0, _lib.ptr(counts), _lib.stream_of(H))
    _lib.check("rq_hessian_finalize", rc)
    return counts


def packed_upper_elems(columns: int) -> int:
    """Floats per group of the packed upper storage (see pack_upper)."""
    return int(_lib.lib.rq_hessian_packed_elems(int(columns)))


def pack_upper(H: torch.Tensor, pieces: int = 1, key: str = "exchange") -> torch.Tensor:
    """The entries on or above the diagonal of every ``H[g]`` (all that an un-finalised sum holds) as ``[G, L]``
    with L = packed_upper_elems(C) rounded up to a multiple of ``4 * pieces``; the buffer comes from the
    workspace cache of the current stream, the padding is zeroed."""
    _lib.require_cuda(H)
    assert H.is_contiguous() and H.dtype == torch.float32 and H.dim() == 3
    G, Cc = H.shape[0], H.shape[-1]
    n = packed_upper_elems(Cc)
    unit = 4 * max(1, int(pieces))
    L = (n + unit - 1) // unit * unit
    ws = _workspace(H.device, G * L * 4 + 1024, key=key)
    off = (-ws.data_ptr()) % 1024
    packed = ws[off:off + G * L * 4].view(torch.float32).view(G, L)
    if L > n:
        packed[:, n:].zero_()
    with torch.cuda.device(H.device):
        rc = _lib.lib.rq_hessian_pack_upper(_lib.ptr(H), Cc, G, _lib.ptr(packed), L, _lib.stream_of(H))
    _lib.check("rq_hessian_pack_upper", rc)
    return packed


def unpack_upper(packed: torch.Tensor, H: torch.Tensor) -> None:
    """Inverse of pack_upper for the groups ``packed`` [g, L] / ``H`` [g, C, C] hold."""
    _lib.require_cuda(packed, H)
    assert H.is_contiguous() and H.dtype == torch.float32 and packed.dtype == torch.float32
    assert packed.stride(-1) == 1 and packed.shape[0] == H.shape[0]
    with torch.cuda.device(H.device):
        rc = _lib.lib.rq_hessian_unpack_upper(_lib.ptr(packed), packed.stride(0), H.shape[-1], H.shape[0], _lib.ptr(H),
                                              _lib.stream_of(H))
    _lib.check("rq_hessian_unpack_upper", rc)


def clamp_to_quantile_(x: torch.Tensor, q: float) -> torch.Tensor:
    """In place ``x = clamp(x, max=torch.quantile(x.flatten(), q))`` for a contiguous fp32 tensor of any size (no
    sort, no 16M-element limit); returns the cap as a 0-dim tensor."""
    _lib.require_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    cap = torch.empty((), dtype=torch.float32, device=x.device)
    need = int(_lib.lib.rq_quantile_workspace_bytes())
    ws = _workspace(x.device, need, key="quantile")
    with torch.cuda.device(x.device):
        rc = _lib.lib.rq_clamp_to_quantile(_lib.ptr(x), x.numel(), float(q), _lib.ptr(cap), _lib.ptr(ws), need,
                                           _lib.stream_of(x))
    _lib.check("rq_clamp_to_quantile", rc)
    return cap


def group_mean_square(grad: torch.Tensor, num_groups: int) -> torch.Tensor:
    """``grad.float().pow(2).view(b, t, G, -1).mean(-1)`` for a ``[batch, seq, hidden]`` gradient (fp32 / bf16 / fp16,
    channels contiguous; the batch and sequence strides are free, so a ``grad[:, sink:]`` slice is taken as is)."""
    _lib.require_cuda(grad)
    assert grad.dim() == 3, "grad must be [batch, seq, hidden]"
    if grad.stride(2) != 1:
        grad = grad.contiguous()
    b, t, hidden = grad.shape
    if hidden % num_groups != 0:
        raise ValueError(f"hidden size {hidden} is not divisible by num_groups {num_groups}")
    out = torch.empty(b, t, num_groups, dtype=torch.float32, device=grad.device)
    with torch.cuda.device(grad.device):
        rc = _lib.lib.rq_group_mean_square(_lib.ptr(grad), _lib.dtype_code(grad), b, t, grad.stride(0), grad.stride(1),
                                           hidden, int(num_groups), _lib.ptr(out), _lib.stream_of(grad))
    _lib.check("rq_group_mean_square", rc)
    return out
