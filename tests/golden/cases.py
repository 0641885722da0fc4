"""Seeded input generators shared by the golden-fixture script and the tests.

The value distributions mirror the benchmark configurations at small sizes:
weights ~ N(0, 0.02^2) with a few input columns scaled x10, activations ~ N(0, 1)
times per-channel log-normal(0, 1) scales, per-token per-group saliency ~
log-normal(0, 3) clipped at its 99th percentile (the reference clips the same way,
gptq_utils/gptq_plus_utils.py:2834-2839), weight gradient ~ N(0, 1e-4^2).
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def make_weight(rows: int, cols: int, seed: int, outlier_frac: float = 0.02) -> torch.Tensor:
    g = _gen(seed)
    W = torch.randn(rows, cols, generator=g) * 0.02
    n_out = max(1, int(round(cols * outlier_frac)))
    idx = torch.randperm(cols, generator=g)[:n_out]
    W[:, idx] *= 10.0
    return W


def make_acts(nseq: int, seqlen: int, cols: int, seed: int, dtype=torch.float32) -> torch.Tensor:
    g = _gen(seed + 1000)
    ch = torch.exp(torch.randn(cols, generator=g))
    X = torch.randn(nseq, seqlen, cols, generator=g) * ch
    return X.to(dtype)


def make_saliency(nseq: int, seqlen: int, groups: int, seed: int) -> torch.Tensor:
    g = _gen(seed + 2000)
    s = torch.exp(3.0 * torch.randn(nseq, seqlen, groups, generator=g))
    cap = torch.quantile(s.flatten().double(), 0.99).float()
    return torch.clamp(s, max=cap)


def make_grad(rows: int, cols: int, seed: int, std: float = 1e-4) -> torch.Tensor:
    g = _gen(seed + 3000)
    return torch.randn(rows, cols, generator=g) * std


def digest(*tensors) -> str:
    """Short content hash of the generated inputs; stored in each fixture so that a
    drift of the generators (other torch build, edited code) is reported as such
    rather than as a parity failure."""
    h = hashlib.sha256()
    for t in tensors:
        h.update(np.ascontiguousarray(t.detach().float().numpy()).tobytes())
    return h.hexdigest()[:16]


# ---------------------------------------------------------------------------------------
# case tables (small enough for the pure-CPU reference to finish in seconds)
# ---------------------------------------------------------------------------------------
QUANTIZER_CASES = [
    # name, rows, cols, bits, perchannel, sym, mse
    ("w4_sym_pc", 48, 256, 4, True, True, False),
    ("w4_asym_pc", 48, 256, 4, True, False, False),
    ("w3_sym_pc", 40, 200, 3, True, True, False),
    ("w4_sym_pt", 24, 96, 4, False, True, False),
    ("w4_sym_pc_mse", 32, 128, 4, True, True, True),
    ("w4_asym_pc_mse", 32, 128, 4, True, False, True),
    ("w8_asym_pt", 16, 64, 8, False, False, False),
]

WGROUP_CASES = [
    # name, rows, cols, bits, weight_groupsize, sym, dtype
    ("wg_w4_g128_sym_bf16", 24, 256, 4, 128, True, "bfloat16"),
    ("wg_w4_g64_asym_bf16", 24, 256, 4, 64, False, "bfloat16"),
    ("wg_w3_g128_sym_f32", 16, 384, 3, 128, True, "float32"),
    ("wg_w8_g32_asym_f16", 8, 96, 8, 32, False, "float16"),
]

WGROUP_MSE_CASES = [
    # name, rows, cols, bits, weight_groupsize, sym, dtype  (find_params with mse=True)
    ("wgm_w4_g128_sym_bf16", 12, 256, 4, 128, True, "bfloat16"),
    ("wgm_w4_g64_asym_bf16", 12, 128, 4, 64, False, "bfloat16"),
    ("wgm_w3_g128_sym_f32", 8, 256, 3, 128, True, "float32"),
    ("wgm_w4_g32_asym_f16", 8, 96, 4, 32, False, "float16"),
]

CLIP_CASES = [
    # name, rows, cols, bits, sym, weight dtype
    ("clip_w4_sym_f32", 32, 128, 4, True, "float32"),
    ("clip_w4_asym_bf16", 32, 128, 4, False, "bfloat16"),
    ("clip_w3_sym_bf16", 24, 200, 3, True, "bfloat16"),
]

SALIENCY_CASES = [
    # name, batch, seq, hidden, groups, sink_size, dtype
    ("sal_f32_g4", 2, 24, 256, 4, 0, "float32"),
    ("sal_bf16_g4_sink", 3, 40, 512, 4, 4, "bfloat16"),
    ("sal_bf16_g2_odd", 1, 17, 200, 2, 1, "bfloat16"),
]


def make_out_grad(batch, seq, hidden, seed):
    """Heavy-tailed stand-in for the gradient of a loss with respect to a layer output."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(batch, seq, hidden, generator=g) * torch.exp(2.0 * torch.randn(batch, seq, 1, generator=g)) * 1e-3


QK_CASES = [
    # name, (batch, heads, kv_heads, seq, head_dim), k_bits, k_groupsize (-1 or head_dim), k_sym, clip, dtype
    ("qk_k4_token_asym_bf16", (2, 4, 2, 9, 64), 4, -1, False, 0.95, "bfloat16"),
    ("qk_k4_head_sym_f16", (1, 4, 4, 7, 128), 4, 128, True, 1.0, "float16"),
    ("qk_k16_bf16", (1, 2, 2, 5, 64), 16, -1, False, 1.0, "bfloat16"),
]

GPTAQ_CASES = [
    # name, rows, cols, nseq, seqlen, bits, sym, groupsize, actorder, static, alpha
    ("gptaq_pc_sym_act", 32, 256, 4, 96, 4, True, -1, True, False, 0.25),
    ("gptaq_pc_asym_noact", 24, 256, 3, 80, 4, False, -1, False, False, 0.25),
    ("gptaq_g128_static_act", 32, 384, 4, 96, 4, True, 128, True, True, 0.5),
    ("gptaq_g64_dynamic_asym_act", 16, 256, 3, 80, 4, False, 64, True, False, 0.25),
]


def make_fp_acts(X, seed):
    """Full-precision inputs of GPTAQ: the quantized-path activations plus a few per cent of deviation."""
    g = torch.Generator().manual_seed(seed)
    return X + 0.05 * X.abs().mean() * torch.randn(X.shape, generator=g)


GUIDED_CASES = [
    # name, rows, cols, nseq, seqlen, G, bits, groupsize, actorder, static
    ("guided_pc_act", 32, 256, 4, 96, 4, 4, -1, True, False),
    ("guided_g128_static_act", 32, 256, 4, 96, 2, 4, 128, True, True),
    ("guided_pc_noact", 16, 384, 3, 64, 2, 3, -1, False, False),
    ("guided_g128_dynamic_noact", 16, 256, 3, 64, 2, 4, 128, False, False),
    ("guided_g64_dynamic_act", 16, 256, 3, 64, 2, 4, 64, True, False),
]

ACT_QUANT_CASES = [
    # name, shape, bits, groupsize, sym, clip_ratio, dtype
    ("act_a4_asym_tok_bf16", (2, 9, 256), 4, -1, False, 1.0, "bfloat16"),
    ("act_a4_sym_tok_clip_bf16", (2, 9, 256), 4, -1, True, 0.9, "bfloat16"),
    ("act_a8_asym_g64_f16", (1, 7, 192), 8, 64, False, 0.95, "float16"),
    ("act_a4_sym_g128_bf16", (3, 5, 384), 4, 128, True, 1.0, "bfloat16"),
    ("act_a4_asym_tok_f32_long", (1, 3, 1536), 4, -1, False, 0.9, "float32"),
    ("act_a8_sym_tok_f32", (1, 4, 200), 8, -1, True, 1.0, "float32"),
]


def make_act_tensor(shape, seed):
    """Activations with outlier channels, one all-zero row and one all-positive row."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g) * torch.exp(1.5 * torch.randn(shape[-1], generator=g))
    x[0, 0] = 0.0
    x[0, 1] = x[0, 1].abs() + 0.5
    return x


HADAMARD_CASES = [
    # name, rows, n, dtype
    ("n128_f32", 37, 128, "float32"),
    ("n1024_f32", 9, 1024, "float32"),
    ("n4096_f32", 3, 4096, "float32"),
    ("n96_f32_k12", 21, 96, "float32"),
    ("n1536_f32_k12", 5, 1536, "float32"),
    ("n640_f32_k20", 6, 640, "float32"),
    ("n896_f32_k28", 6, 896, "float32"),
    ("n1024_bf16", 9, 1024, "bfloat16"),
    ("n1536_bf16_k12", 5, 1536, "bfloat16"),
    ("n512_f16", 4, 512, "float16"),
]

PLAIN_CASES = [
    # name, rows, cols, nseq, seqlen, bits, sym, groupsize, actorder, static_groups, blocksize
    ("plain_pc_act", 48, 256, 4, 96, 4, False, -1, True, True, 128),
    ("plain_pc_noact", 48, 256, 4, 96, 4, True, -1, False, False, 128),
    ("plain_g64_static_act", 32, 256, 4, 96, 4, True, 64, True, True, 128),
    ("plain_g128_dynamic", 32, 256, 3, 96, 4, True, 128, False, False, 128),
    ("plain_ragged_block", 24, 200, 3, 80, 3, True, -1, True, True, 128),
    # dynamic groups that do not coincide with the 128-column block ("mse" in the name: shrink-grid search on)
    ("plain_g256_dynamic_act", 32, 512, 3, 96, 4, True, 256, True, False, 128),
    ("plain_g96_dynamic", 24, 384, 3, 96, 4, False, 96, False, False, 128),
    ("plain_g64_dynamic_act", 24, 256, 3, 96, 4, True, 64, True, False, 128),
    ("plain_g64_dynamic_mse", 24, 256, 3, 96, 4, True, 64, False, False, 128),
    ("plain_g256_dynamic_bs256", 32, 512, 3, 96, 4, True, 256, False, False, 256),
]

# GPTQ+ with dynamic weight groups the block kernel cannot range itself: name, rows, cols, nseq, seqlen, G,
# blocksize (= groupsize), shrink-grid search, actorder
PLUS_DYNAMIC_CASES = [
    ("plus_dyn_bs256", 32, 512, 4, 160, 2, 256, False, True),
    ("plus_dyn_bs128_mse", 32, 384, 4, 128, 2, 128, True, False),
]

PLUS_CASES = [
    # name, rows, cols, nseq, seqlen, G, bits, groupsize, actorder, static, alpha, ref_loss, mode, atomic
    ("plus_frozen_pc", 64, 256, 4, 96, 4, 4, -1, True, True, 0.25, 0.7, "frozen", False),
    ("plus_frozen_alpha0", 64, 256, 4, 96, 4, 4, -1, True, True, 0.0, 0.7, "frozen", False),
    ("plus_frozen_g128_static", 32, 256, 4, 96, 2, 4, 128, True, True, 0.25, 0.7, "frozen", False),
    ("plus_frozen_g128_dynamic", 32, 256, 4, 96, 2, 4, 128, False, False, 0.25, 0.7, "frozen", False),
    ("plus_frozen_w3_noact", 32, 384, 3, 64, 4, 3, -1, False, False, 0.5, 0.3, "frozen", False),
    ("plus_surrogate_block", 32, 256, 4, 96, 2, 4, -1, True, True, 0.25, 0.7, "surrogate_block", False),
    ("plus_surrogate_online", 32, 256, 4, 96, 2, 4, -1, True, True, 0.25, 0.7, "surrogate_online", False),
    ("plus_atomic", 32, 256, 4, 96, 2, 4, -1, True, True, 0.25, 0.7, "frozen", True),
    ("plus_ragged", 32, 200, 3, 80, 4, 4, -1, True, True, 0.25, 0.7, "frozen", False),
    ("plus_block_backward", 32, 384, 4, 96, 2, 4, -1, True, True, 0.25, 0.7, "block_backward", False),
]


GD_CASES = [
    # name, rows, cols, nseq, seqlen, G, groupsize, actorder, static, alpha, ref_loss, atomic, block_gd keyword arguments
    ("gd_sgd", 32, 384, 4, 96, 2, -1, True, True, 0.25, 0.7, False,
     dict(grad_lr=5.0, grad_optimizer="sgd", grad_clip=1.0)),
    ("gd_adam_gate_sine", 32, 384, 4, 96, 2, 128, True, True, 0.25, 0.7, False,
     dict(grad_lr=1e-3, grad_optimizer="adam", grad_reg_strategy="quant_error_gate_optimized", grad_gate_floor=0.2,
          grad_gate_sharpness=3.0, grad_gate_sine_amp=1e-9, second_order_scale=0.8, grad_clip=5e-5)),
    ("gd_hadam_l2", 32, 384, 4, 96, 4, -1, False, False, 0.0, 0.7, False,
     dict(grad_lr=1e-3, grad_optimizer="h_adam", curvature_damping=0.1, grad_reg_strategy="l2", grad_reg_lambda=0.3,
          slide_refresh_start=1, slide_refresh_block_total=6)),
    ("gd_adam_hessian_atomic", 32, 384, 4, 96, 2, -1, True, True, 0.25, 0.7, True,
     dict(grad_lr=5e-4, grad_optimizer="adam", grad_reg_strategy="hessian", grad_reg_lambda=0.05)),
    ("gd_adam_gate", 32, 400, 4, 96, 2, -1, True, True, 0.25, 0.7, False,
     dict(grad_lr=1e-3, grad_optimizer="adam", grad_reg_strategy="quant_error_gate", second_order_scale=1.2)),
]


def make_refresh_fn(W0, G0, calls=None):
    """Deterministic stand-in for the model backward that ``block_backward`` calls between blocks: the
    gradient of a diagonal quadratic around the original weights, elementwise in fp32 on the CPU so that
    every implementation sees bit-identical refreshed gradients for identical snapshots."""
    W0 = W0.detach().float().cpu().clone()
    G0 = G0.detach().float().cpu().clone()
    curv = torch.linspace(0.5, 2.0, W0.shape[1]).unsqueeze(0) * 1e-3

    def refresh(weight_snapshot, slide_alpha=None):
        snap = weight_snapshot.detach().float().cpu()
        grad = G0 + (snap - W0) * curv
        if slide_alpha is not None:                       # block_gd passes its loss-window weight
            grad = grad * (0.5 + 0.5 * float(slide_alpha))
        if calls is not None:
            calls.append(snap.clone())
        return grad.to(weight_snapshot.device), {"mean_refresh_loss": float(((snap - W0) ** 2).mean())}

    return refresh
