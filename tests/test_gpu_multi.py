"""Data-parallel quantization on two GPUs over NCCL against a one-GPU run of the same data: the row-parallel
mode of GPTQPlus (packed upper-triangle reduce-scatter, all-gather among the ranks that share a saliency group,
row shards, all-gather of the quantized rows) and the older per-group owner mode.  Skipped on a single GPU.

No rank leaves early and nothing here waits on a flag: the children run the same collectives in the same
order and exit after a barrier."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import cases
        from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
        from gptq_plus_mp_quant_b200.utils import dist_utils as du
        from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
        dev = torch.device("cuda", rank)
        report = {}
        for tag, rows, cols, G, nseq, seqlen in (("g4", 256, 512, 4, 8, 512), ("g1", 128, 384, 1, 4, 1024)):
            W = cases.make_weight(rows, cols, seed=51)
            X = cases.make_acts(nseq, seqlen, cols, seed=51).bfloat16()
            S = cases.make_saliency(nseq, seqlen, G, seed=51)
            Gr = cases.make_grad(rows, cols, seed=51)

            def run(mode):
                layer = torch.nn.Linear(cols, rows, bias=False, device=dev, dtype=torch.bfloat16)
                layer.weight.data.copy_(W)
                sl = slice(0, nseq) if mode == "solo" else du.shard_slice(nseq)
                obj = GPTQPlus(layer, S[sl], Gr, G, 0.25, 0.7)
                obj.quantizer = WeightQuantizer()
                obj.quantizer.configure(4, perchannel=True, sym=True, mse=False)
                obj.row_parallel = mode == "rows"
                for s in range(sl.start, sl.stop, 2):
                    obj.add_batch(X[s:s + 2].to(dev), None)
                if mode == "begin":
                    obj.row_parallel = True
                    side = torch.cuda.Stream()
                    obj.begin_exchange(side)
                obj.finalize_hessian()
                first, count = obj._owned_groups if obj._owned_groups is not None else (0, G)
                H = obj._H[first:first + count].clone()
                obj.fasterquant(blocksize=128, percdamp=0.01, groupsize=128, actorder=True, static_groups=True,
                                export_to_et=True)
                obj.gather_rows_()
                return layer.weight.data.clone(), layer.int_weight.clone(), H, (first, count), obj.act_square.clone()

            with du.local_only():
                w1, c1, h1, _, a1 = run("solo")
            for mode in ("rows", "begin"):
                w2, c2, h2, (first, count), a2 = run(mode)
                du.assert_bit_exact(w2, f"{tag}.{mode}.weight")
                du.assert_bit_exact(c2, f"{tag}.{mode}.codes")
                h_err = float((h2.double() - h1[first:first + count].double()).norm() / h1[first:first + count].double().norm())
                frac = float((c2 != c1).float().mean())
                assert h_err < 2e-6, (tag, mode, h_err)
                assert torch.allclose(a2, a1, rtol=1e-5)
                assert frac < 5e-3, (tag, mode, frac)
                report[f"{tag}.{mode}"] = (h_err, frac)
        dist.barrier()
        results[rank] = report
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_parallel_matches_one_rank():
    import torch.multiprocessing as mp
    world = 2
    port = 33500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert set(results.keys()) == {0, 1}
    print({k: v for k, v in results[0].items()})
