"""Host-side data-parallel logic on CPU with the gloo backend, world size 2: contiguous sharding of
the calibration sequences, summation of the un-normalised partial Hessian state over ranks (the
exchange step of finalize_hessian), reduce-to-owner, the cross-rank bit-exactness assertion and the
assignment of linears to ranks."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cases
        from oracle import hessian as ohess
        from gptq_plus_mp_quant_b200.utils import dist_utils as du
        torch.set_num_threads(1)
        nseq, seqlen, C, G = 4, 64, 96, 2
        X = cases.make_acts(nseq, seqlen, C, seed=7)
        S = cases.make_saliency(nseq, seqlen, G, seed=7)
        sl = du.shard_slice(nseq)
        assert (sl.start, sl.stop) == (rank * 2, rank * 2 + 2)
        assert du.shard_size(nseq) == 2
        with pytest.raises(ValueError):
            du.shard_slice(5)
        part = ohess.GroupedHessian(C, S[sl])
        part.add_batch(X[sl])
        # exchange step exactly as finalize_hessian performs it
        du.allreduce_sum_(part.H)
        du.allreduce_sum_(part.act_square)
        part.index = int(du.allreduce_sum_scalar(part.index))
        part.token_count = int(du.allreduce_sum_scalar(part.token_count))
        part.finalize()
        whole = ohess.GroupedHessian(C, S)
        whole.add_batch(X)
        whole.finalize()
        rel = float((part.H - whole.H).norm() / whole.H.norm())
        assert rel < 1e-6, rel
        assert torch.allclose(part.act_square, whole.act_square, rtol=1e-5)
        du.assert_bit_exact(part.H, "H after all-reduce")            # every rank holds the same bits
        bad = part.H.clone()
        if rank == 1:
            bad[0, 0, 0] += 1.0
            with pytest.raises(RuntimeError):
                du.assert_bit_exact(bad, "perturbed")
        else:
            du.assert_bit_exact(bad, "perturbed")                    # rank 0 is the reference copy
        # reduce-to-owner: only the owner needs the sum
        t = torch.full((8,), float(rank + 1))
        du.reduce_sum_(t, 1)
        if rank == 1:
            assert torch.equal(t, torch.full((8,), 3.0))
        # per-group ownership: group g of the Hessian is summed on its owner only, the owner quantizes that
        # group's rows, the rows travel back by broadcast; equals quantizing everything in one process
        from oracle import gptq as og, quantizer as oq
        rows = 8
        W = cases.make_weight(rows, C, seed=7)
        Gr = cases.make_grad(rows, C, seed=7)
        owners = [1, 0]
        part2 = ohess.GroupedHessian(C, S[sl])
        part2.add_batch(X[sl])
        du.reduce_groups_to_owners_(part2.H, owners)                 # general path: one reduce per group
        du.allreduce_sum_(part2.act_square)
        part2.index = int(du.allreduce_sum_scalar(part2.index))
        part2.token_count = int(du.allreduce_sum_scalar(part2.token_count))
        part2.finalize()
        rps = rows // G
        Wq = W.clone()
        for g, owner in enumerate(owners):
            if owner == rank:
                q = oq.OracleWeightQuantizer()
                q.configure(4, perchannel=True, sym=True)
                r = slice(g * rps, (g + 1) * rps)
                # alpha_eff of the whole layer: alpha / (rows * C) = (alpha / G) / (rps * C)
                o = og.plus_fasterquant(W[r], part2.H[g:g + 1], part2.act_square, Gr[r], q, 1, 0.25 / G, 0.7,
                                        actorder=True, static_groups=True)
                Wq[r] = o["Q"]
        for g, owner in enumerate(owners):
            dist.broadcast(Wq[g * rps:(g + 1) * rps], src=owner)
        q = oq.OracleWeightQuantizer()
        q.configure(4, perchannel=True, sym=True)
        full = og.plus_fasterquant(W, whole.H, whole.act_square, Gr, q, G, 0.25, 0.7, actorder=True,
                                   static_groups=True)["Q"]
        assert float((Wq != full).float().mean()) < 0.02             # summation order differs in the last bit
        du.assert_bit_exact(Wq, "gathered weights")
        # the two reduce-scatter patterns: world divides G (rank r owns a run of groups), and G divides world
        # (pieces of a group land on k ranks and are gathered on the one that owns it)
        assert du.group_owner_pattern(4, 2) == [0, 0, 1, 1] and du.group_owner_pattern(2, 2) == [0, 1]
        assert du.group_owner_pattern(1, 2, salt=0) == [0] and du.group_owner_pattern(1, 2, salt=1) == [1]
        assert du.group_owner_pattern(4, 3) is None
        for owners_p, shape in (([0, 1], (2, 6, 6)), ([0, 0, 1, 1], (4, 5, 4)), ([1], (1, 4, 6)), ([0], (1, 4, 6))):
            gen = torch.Generator().manual_seed(11)
            parts = [torch.randn(shape, generator=gen) for _ in range(world)]
            Hp = parts[rank].clone()
            du.reduce_groups_to_owners_(Hp, owners_p)
            total = parts[0] + parts[1]
            for g, owner in enumerate(owners_p):
                if owner == rank:
                    assert torch.allclose(Hp[g], total[g], rtol=0, atol=1e-6), (owners_p, g)
        # the small helpers of the reference's module (dist_utils.py:38-62, 152-176)
        assert du.is_main() == (rank == 0)
        du.barrier()
        assert du.allreduce_mean_scalar(float(rank + 1)) == 1.5
        assert du.allreduce_mean_scalar(2.0 if rank == 0 else 8.0, count=3 if rank == 0 else 1) == 3.5
        assert du.allreduce_mean_scalar(5.0, count=0) == 0.0
        b = torch.full((3,), float(rank))
        assert torch.equal(du.broadcast_tensor_(b, src=1), torch.ones(3))
        for dim, shape in ((0, (2, 3)), (1, (2, 3))):
            mine = torch.arange(6.0).reshape(shape) + 10 * rank
            got = du.gather_into_tensor(mine, dim=dim)
            if rank == 0:
                want = torch.cat([torch.arange(6.0).reshape(shape), torch.arange(6.0).reshape(shape) + 10], dim=dim)
                assert torch.equal(got, want)
            else:
                assert got is None
        lin = torch.nn.Linear(4, 3)
        with torch.no_grad():
            lin.weight.fill_(float(rank))
            lin.bias.fill_(float(rank))
        du.broadcast_parameters(lin, src=1)
        assert float(lin.weight.min()) == 1.0 and float(lin.bias.max()) == 1.0
        with du.local_only():
            assert du.is_main() and torch.equal(du.gather_into_tensor(b), b) and du.allreduce_mean_scalar(7.0) == 7.0
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_world2_sharded_hessian_and_helpers():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def _row_parallel_worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gptq_plus_mp_quant_b200.utils import dist_utils as du
        torch.set_num_threads(1)
        for G in (1, 2, 4, 8):
            first, count, piece, pieces = du.row_parallel_layout(G)
            # the groups a rank holds cover exactly its row shard [r*R/W, (r+1)*R/W)
            R = 64
            rps = R // G
            lo = first * rps + (piece * (rps // pieces) if pieces > 1 else 0)
            hi = lo + (rps // pieces if pieces > 1 else count * rps)
            assert (lo, hi) == (rank * R // world, (rank + 1) * R // world), (G, lo, hi)
            L = 24
            gen = torch.Generator().manual_seed(5 + G)
            parts = [torch.randn(G, L, generator=gen) for _ in range(world)]
            sums = parts[rank].clone()
            f2, c2 = du.exchange_group_sums_(sums)
            assert (f2, c2) == (first, count)
            total = sum(parts)
            assert torch.allclose(sums[first:first + count], total[first:first + count], rtol=0, atol=1e-5), G
            # ranks that share a group hold the same bits of it
            if pieces > 1:
                same = [torch.empty_like(sums[first]) for _ in range(world)]
                dist.all_gather(same, sums[first].clone())
                k0 = (rank // pieces) * pieces
                assert all(torch.equal(same[k0], same[k0 + j]) for j in range(pieces))
        with pytest.raises(ValueError):
            du.row_parallel_layout(3)
        w = torch.zeros(8, 3)
        n = 8 // world
        w[rank * n:(rank + 1) * n] = float(rank + 1)
        du.allgather_rows_(w)
        assert torch.equal(w[:, 0], torch.arange(1, world + 1).repeat_interleave(n).float())
        with du.local_only():
            assert du.get_world_size() == 1 and du.get_rank() == 0
            assert du.row_parallel_layout(4) == (0, 4, 0, 1)
        assert du.get_world_size() == world
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_row_parallel_exchange(world):
    port = 31500 + (os.getpid() % 2000) + world
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_row_parallel_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {r: "ok" for r in range(world)}
