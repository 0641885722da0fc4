"""Data-parallel helpers of the quantization path: the reference's ``utils/dist_utils.py`` (:13-199) without
``distribute_model`` (placing a model across devices is the caller's launcher's business), plus the exchanges
of the row-parallel mode.  The collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in
CPU tests)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


_local_only = 0


def is_dist_available_and_initialized() -> bool:
    return dist.is_available() and dist.is_initialized() and _local_only == 0


class local_only:
    """Context in which the helpers of this module behave as in a single process (world size 1, rank 0) although a
    process group exists: for a rank that quantizes something on its own, e.g. a one-rank run of the same data to
    compare a data-parallel result with."""

    def __enter__(self):
        global _local_only
        _local_only += 1

    def __exit__(self, *exc):
        global _local_only
        _local_only -= 1


def init_process_group():
    """Joins the job's process group and waits for the other ranks (dist_utils.py:13-23).  The caller has selected
    its GPU with ``torch.cuda.set_device``; the group is bound to that device so that collectives never guess it.
    NCCL with the reference's 8-hour timeout on GPUs, gloo where there is no GPU."""
    import datetime
    if torch.cuda.is_available():
        dist.init_process_group(backend="nccl", timeout=datetime.timedelta(hours=8),
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    else:
        dist.init_process_group(backend="gloo", timeout=datetime.timedelta(hours=8))
    dist.barrier()


def get_world_size() -> int:
    return dist.get_world_size() if is_dist_available_and_initialized() else 1


def get_rank() -> int:
    return dist.get_rank() if is_dist_available_and_initialized() else 0


def is_main() -> bool:
    return get_rank() == 0


def print_on_main(*args, **kwargs):
    if is_main():
        print(*args, **kwargs)


def barrier():
    if is_dist_available_and_initialized():
        dist.barrier()


def broadcast_parameters(module, src=0, group=None):
    """Every parameter of ``module`` takes rank ``src``'s values (dist_utils.py:47-49)."""
    for param in module.parameters():
        dist.broadcast(param.data, src=src, group=group)


def broadcast_tensor_(tensor: torch.Tensor, src: int = 0) -> torch.Tensor:
    """In-place broadcast; no-op for a single process (dist_utils.py:166-170)."""
    if get_world_size() > 1:
        dist.broadcast(tensor, src=src)
    return tensor


def gather_into_tensor(tensor, dim: int = 0):
    """Rank 0 receives the ranks' tensors concatenated along ``dim`` in rank order; the other ranks get None
    (dist_utils.py:52-62).  A single process gets a copy of its own tensor."""
    world = get_world_size()
    if world == 1:
        return tensor.clone()
    if not is_main():
        dist.gather(tensor, None)
        return None
    pieces = [torch.empty_like(tensor) for _ in range(world)]
    dist.gather(tensor, pieces)
    return torch.cat(pieces, dim=dim)


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


def _reduce_scatter_inplace_(flat: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Sum over ranks of ``flat`` (numel divisible by world), chunk r of the sum delivered into chunk r of rank
    r's own buffer; the other chunks are left unspecified.  Returns this rank's chunk (a view)."""
    chunks = flat.view(world, -1)
    if dist.get_backend() == "nccl":
        dist.reduce_scatter_tensor(chunks[rank], flat, op=dist.ReduceOp.SUM)   # NCCL's in-place layout
    else:                                                                      # gloo has no reduce-scatter
        for s in range(world):
            dist.reduce(chunks[s], dst=s, op=dist.ReduceOp.SUM)
    return chunks[rank]


def group_owner_pattern(num_groups: int, world: int, salt: int = 0):
    """Owners for which reduce_groups_to_owners_ needs one reduce-scatter: ``world`` divides ``num_groups``
    (rank r owns a run of groups) or ``num_groups`` divides ``world`` (group g lands on the ranks
    [g*k, (g+1)*k), k = world / num_groups, and ``salt`` picks which of them owns it, so that successive linears
    load different ranks).  None when neither divides."""
    if world <= 1:
        return [0] * num_groups
    if num_groups % world == 0:
        return [g // (num_groups // world) for g in range(num_groups)]
    if world % num_groups == 0:
        k = world // num_groups
        return [g * k + salt % k for g in range(num_groups)]
    return None


def reduce_groups_to_owners_(H: torch.Tensor, owners) -> None:
    """``H`` [G, ...] holds this rank's partial sums; afterwards rank ``owners[g]`` holds the sum of ``H[g]`` (the
    other ranks' copies of that group are unspecified).  One bandwidth-optimal reduce-scatter when the owners follow
    group_owner_pattern (plus, when several ranks share a group, a gather of its pieces on the owner); one reduce
    per group otherwise."""
    world, rank = get_world_size(), get_rank()
    if world <= 1:
        return
    G = H.shape[0]
    owners = [int(o) for o in owners]
    assert len(owners) == G and H.is_contiguous()
    flat = H.view(-1)
    if G % world == 0 and owners == group_owner_pattern(G, world):
        _reduce_scatter_inplace_(flat, world, rank)
        return
    k = world // G if world % G == 0 else 0
    if k > 1 and flat.numel() % world == 0 and all(g * k <= owners[g] < (g + 1) * k for g in range(G)):
        _reduce_scatter_inplace_(flat, world, rank)            # piece s = g*k + j of the sum now sits on rank s
        chunks = flat.view(world, -1)
        g = rank // k
        ops = []
        if rank == owners[g]:
            ops = [dist.P2POp(dist.irecv, chunks[src], src) for src in range(g * k, (g + 1) * k) if src != rank]
        else:
            ops = [dist.P2POp(dist.isend, chunks[rank], owners[g])]
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        return
    for g, owner in enumerate(owners):
        dist.reduce(H[g], dst=owner, op=dist.ReduceOp.SUM)


def row_parallel_layout(num_groups: int, world: Optional[int] = None, rank: Optional[int] = None):
    """Row-parallel fasterquant: rank r quantizes rows ``[r*R/W, (r+1)*R/W)`` of a linear whose rows fall into
    ``num_groups`` saliency groups, each with a Hessian of its own.  Returns ``(first group, groups, piece, pieces)``:
    the Hessian groups that cover this rank's rows, and which of the ``pieces`` equal row slices of that group the
    rank takes (``pieces`` = ranks per group, 1 when a rank holds whole groups).  ``world`` must divide
    ``num_groups`` or be a multiple of it."""
    world = get_world_size() if world is None else world
    rank = get_rank() if rank is None else rank
    if world <= 1:
        return 0, num_groups, 0, 1
    if num_groups % world == 0:
        n = num_groups // world
        return rank * n, n, 0, 1
    if world % num_groups == 0:
        k = world // num_groups
        return rank // k, 1, rank % k, k
    raise ValueError(f"row-parallel quantization needs world_size ({world}) to divide num_groups ({num_groups}) "
                     "or to be a multiple of it")


_peer_groups = {}


def _group_peers(num_groups: int, world: int):
    """Process groups of the ranks that share one Hessian group (``world`` a multiple of ``num_groups``); created
    once, by every rank, in the same order."""
    key = (num_groups, world)
    if key not in _peer_groups:
        k = world // num_groups
        _peer_groups[key] = [dist.new_group(list(range(g * k, (g + 1) * k))) for g in range(num_groups)]
    return _peer_groups[key]


def exchange_group_sums_(sums: torch.Tensor):
    """``sums`` [G, L]: this rank's partial sums per saliency group (L a multiple of the ranks per group).
    Afterwards rows ``first .. first + groups`` (see row_parallel_layout) hold the sums over all ranks; the other
    rows are unspecified.  One reduce-scatter over all ranks, then, when several ranks share a group, one
    all-gather among those ranks.  Returns ``(first, groups)``."""
    world, rank = get_world_size(), get_rank()
    G = sums.shape[0]
    first, groups, _, k = row_parallel_layout(G, world, rank)
    if world <= 1:
        return first, groups
    assert sums.is_contiguous() and sums.shape[1] % k == 0
    flat = sums.view(-1)
    mine = _reduce_scatter_inplace_(flat, world, rank)
    if k > 1:
        peers = _group_peers(G, world)[first]
        if dist.get_backend() == "nccl":
            dist.all_gather_into_tensor(sums[first], mine, group=peers)          # NCCL's in-place layout
        else:
            parts = [torch.empty_like(mine) for _ in range(k)]
            dist.all_gather(parts, mine.clone(), group=peers)
            sums[first].copy_(torch.cat(parts))
    return first, groups


def allgather_rows_(tensor: torch.Tensor) -> torch.Tensor:
    """``tensor`` [R, ...] with R divisible by the world size: rank r's rows ``[r*R/W, (r+1)*R/W)`` are copied to
    every rank, in place."""
    world, rank = get_world_size(), get_rank()
    if world <= 1:
        return tensor
    assert tensor.is_contiguous() and tensor.shape[0] % world == 0
    n = tensor.shape[0] // world
    if dist.get_backend() == "nccl":
        dist.all_gather_into_tensor(tensor, tensor[rank * n:(rank + 1) * n])
    else:
        parts = [torch.empty_like(tensor[:n]) for _ in range(world)]
        dist.all_gather(parts, tensor[rank * n:(rank + 1) * n].clone())
        tensor.copy_(torch.cat(parts))
    return tensor


def allreduce_sum_scalar(scalar) -> float:
    """Sum of a Python scalar over ranks in fp64 (dist_utils.py:142-149)."""
    if get_world_size() <= 1:
        return float(scalar)
    device = "cuda" if (torch.cuda.is_available() and dist.get_backend() == "nccl") else "cpu"
    t = torch.tensor([float(scalar)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.item()


def allreduce_mean_scalar(scalar, count: int = 1) -> float:
    """Weighted mean over ranks, ``sum(scalar_r * count_r) / sum(count_r)``, in fp64; 0 when the counts sum to 0
    (dist_utils.py:152-163)."""
    if get_world_size() <= 1:
        return float(scalar)
    device = "cuda" if (torch.cuda.is_available() and dist.get_backend() == "nccl") else "cpu"
    pair = torch.tensor([float(scalar) * count, float(count)], device=device, dtype=torch.float64)
    dist.all_reduce(pair, op=dist.ReduceOp.SUM)
    total, weight = pair.tolist()
    return 0.0 if weight == 0 else total / weight


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
