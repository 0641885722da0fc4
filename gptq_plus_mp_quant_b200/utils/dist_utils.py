"""Data-parallel helpers of the quantization path: the subset of the reference's
``utils/dist_utils.py`` (:105-199) that ``finalize_hessian`` and its callers use.  The
collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in CPU tests)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def is_dist_available_and_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size() -> int:
    return dist.get_world_size() if is_dist_available_and_initialized() else 1


def get_rank() -> int:
    return dist.get_rank() if is_dist_available_and_initialized() else 0


def shard_slice(total: int, rank: Optional[int] = None, world: Optional[int] = None) -> slice:
    """Contiguous shard ``[r*total/W, (r+1)*total/W)``; ``total`` must divide evenly (dist_utils.py:105-121)."""
    world = get_world_size() if world is None else world
    rank = get_rank() if rank is None else rank
    if total % world != 0:
        raise ValueError(f"shard_slice: total ({total}) must be divisible by world_size ({world}) "
                         f"— either trim the input or drop to a compatible world_size.")
    chunk = total // world
    return slice(rank * chunk, (rank + 1) * chunk)


def shard_size(total: int, world: Optional[int] = None) -> int:
    world = get_world_size() if world is None else world
    if total % world != 0:
        raise ValueError(f"shard_size: total ({total}) must be divisible by world_size ({world}).")
    return total // world


def allreduce_sum_(tensor: torch.Tensor) -> torch.Tensor:
    """In-place SUM all-reduce; no-op for a single process (dist_utils.py:135-139)."""
    if get_world_size() > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    return tensor


def reduce_sum_(tensor: torch.Tensor, dst: int) -> torch.Tensor:
    """In-place SUM reduce to rank ``dst`` only (the other ranks' buffers are left unspecified)."""
    if get_world_size() > 1:
        dist.reduce(tensor, dst=dst, op=dist.ReduceOp.SUM)
    return tensor


def allreduce_sum_scalar(scalar) -> float:
    """Sum of a Python scalar over ranks in fp64 (dist_utils.py:142-149)."""
    if get_world_size() <= 1:
        return float(scalar)
    device = "cuda" if (torch.cuda.is_available() and dist.get_backend() == "nccl") else "cpu"
    t = torch.tensor([float(scalar)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.item()


def assert_bit_exact(tensor: torch.Tensor, tag: str = "", rtol: float = 0.0, atol: float = 0.0):
    """Every rank must hold rank 0's tensor (dist_utils.py:179-199)."""
    if get_world_size() <= 1:
        return
    ref = tensor.clone().contiguous()
    dist.broadcast(ref, src=0)
    ok = torch.equal(tensor, ref) if (rtol == 0.0 and atol == 0.0) else torch.allclose(tensor, ref, rtol=rtol, atol=atol)
    if not ok:
        diff = (tensor - ref).abs()
        raise RuntimeError(f"[assert_bit_exact] Rank {get_rank()} diverges at `{tag}`: "
                           f"max|diff|={diff.max().item():.3e}, mean|diff|={diff.mean().item():.3e}, "
                           f"shape={tuple(tensor.shape)} dtype={tensor.dtype}")
