"""The per-layer driver (gptq_utils/layer_loop.py) against the reference's own way of driving the classes
(gptq_plus_utils.py:6930-7530): for every sequential module group, hooks on the group's linears, a full forward of
the partly quantized layer over the calibration batches, finalize_hessian, fasterquant, free; then the replay.
LayerQuantizer leaves each pass early, quantizes the linears of a group concurrently and, with ``stage_fns``, never
recomputes what an earlier pass produced: the quantized weights and the replayed outputs must be the same bits."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup():
    import bench_model as bm
    T, nseq, hidden = 64, 8, 256
    cos, sin = bm.rotary_tables(T, 64, torch.device(DEV), torch.bfloat16)
    x = (torch.randn(nseq, T, hidden, generator=torch.Generator().manual_seed(3)) * 0.5).to(DEV).bfloat16()

    def make_layer():
        return bm.DecoderLayer(hidden=hidden, inter=768, heads=4, kv_heads=2, head_dim=64, device=DEV, seed=11)

    def stats_fn(index, name, module):
        g = torch.Generator(device=DEV)
        g.manual_seed(1000 * index + sum(name.encode()))
        s = torch.exp(torch.randn(nseq, T, 2, generator=g, device=DEV))
        grad = torch.randn(module.weight.shape, generator=g, device=DEV) * 1e-4
        return s, grad, 0.7

    return bm, cos, sin, x, make_layer, stats_fn


def _reference_style(layer, x, cos, sin, stats_fn, bsz):
    from gptq_plus_mp_quant_b200.gptq_utils.gptq_plus_utils import GPTQPlus
    from gptq_plus_mp_quant_b200.gptq_utils.layer_loop import SEQUENTIAL_GROUPS, find_linears
    from gptq_plus_mp_quant_b200.utils.quant_utils import WeightQuantizer
    full = find_linears(layer)
    with torch.no_grad():
        for names in SEQUENTIAL_GROUPS:
            objs, handles = {}, []
            for name in names:
                s, grad, ref_loss = stats_fn(0, name, full[name])
                o = GPTQPlus(full[name], s, grad, 2, 0.25, ref_loss)
                o.quantizer = WeightQuantizer()
                o.quantizer.configure(4, perchannel=True, sym=True, mse=False)
                objs[name] = o
                handles.append(full[name].register_forward_hook(
                    lambda m, inp, out, name=name: objs[name].add_batch(inp[0].data, out.data)))
            for j in range(0, x.shape[0], bsz):
                layer(x[j:j + bsz], cos, sin)
            for h in handles:
                h.remove()
            for name in names:
                objs[name].finalize_hessian()
                objs[name].fasterquant(blocksize=128, percdamp=0.01, groupsize=-1, actorder=True, static_groups=True)
                objs[name].free()
        return torch.cat([layer(x[j:j + bsz], cos, sin) for j in range(0, x.shape[0], bsz)])


@pytest.mark.parametrize("mode", ["early_exit", "staged", "hessian_once"])
def test_layer_quantizer_matches_reference_style_driver(mode):
    from gptq_plus_mp_quant_b200.gptq_utils.layer_loop import LayerQuantizer, find_linears
    bm, cos, sin, x, make_layer, stats_fn = _setup()
    bsz = 4
    ref_layer = make_layer()
    ref_out = _reference_style(ref_layer, x, cos, sin, stats_fn, bsz)
    layer = make_layer()
    before = {n: m.weight.data.clone() for n, m in find_linears(layer).items()}
    lq = LayerQuantizer(stats_fn, lambda l, v: l(v, cos, sin), num_groups=2, alpha=0.25, w_bits=4,
                        hessian_accum_bsz=bsz, row_parallel=False, hessian_once=(mode == "hessian_once"),
                        stage_fns=bm.decoder_layer_stages(cos, sin) if mode == "staged" else None,
                        fasterquant_kwargs=dict(groupsize=-1, actorder=True, static_groups=True))
    lq.events = []
    out = lq.quantize_layer(0, layer, x)
    assert {name for name, _, _ in lq.events} >= {"hessian_pass", "fasterquant", "replay"}
    got, want = find_linears(layer), find_linears(ref_layer)
    assert set(got) == set(want) and len(got) == 7
    for name in got:
        assert not torch.equal(got[name].weight.data, before[name]), name          # every linear was quantized
        if mode == "hessian_once":
            # all Hessians from the unquantized layer: a different (the reference's layer_hessian_once) result for
            # every linear behind the first group, the same for q, k, v
            if name in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                assert torch.equal(got[name].weight.data, want[name].weight.data), name
        else:
            assert torch.equal(got[name].weight.data, want[name].weight.data), name
    if mode != "hessian_once":
        assert torch.equal(out, ref_out)
    # at most 2^4 levels per row survive
    w = got["mlp.down_proj"].weight.data.float()
    assert max(len(torch.unique(w[r])) for r in range(0, w.shape[0], 37)) <= 16


def test_stage_fns_must_cover_every_group():
    from gptq_plus_mp_quant_b200.gptq_utils.layer_loop import LayerQuantizer
    bm, cos, sin, x, make_layer, stats_fn = _setup()
    lq = LayerQuantizer(stats_fn, lambda l, v: l(v, cos, sin), num_groups=2, row_parallel=False,
                        stage_fns=bm.decoder_layer_stages(cos, sin)[:3])
    with pytest.raises(ValueError):
        lq.quantize_layer(0, make_layer(), x)
