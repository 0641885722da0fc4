"""Random-init decoder layers in stock PyTorch with the shapes of the benchmark configurations (Qwen3-8B: hidden
4096, intermediate 12288, 32 query / 8 KV heads of 128, RMSNorm, per-head q/k norm, rotary embedding, SwiGLU;
Llama-70B: hidden 8192, intermediate 28672, 64 / 8 heads), used by bench.py to feed the calibration hooks and to
replay quantized layers.  No checkpoint is read: weights ~ N(0, 0.02^2) in bf16.  The down_proj input is rotated
online with the package's Hadamard kernel, as the reference's ActQuantWrapper does for that linear
(utils/quant_utils.py:245-297, utils/rotation_utils.py:151-158); the residual-stream rotation is fused into the
weights offline in the reference and costs nothing at run time."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu


class RMSNorm(torch.nn.Module):
    def __init__(self, dim, eps=1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(dim, device=device, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(x.dtype)


class Attention(torch.nn.Module):
    def __init__(self, hidden, heads, kv_heads, head_dim, qk_norm, device, dtype):
        super().__init__()
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, head_dim
        lin = lambda i, o: torch.nn.Linear(i, o, bias=False, device=device, dtype=dtype)
        self.q_proj, self.k_proj = lin(hidden, heads * head_dim), lin(hidden, kv_heads * head_dim)
        self.v_proj, self.o_proj = lin(hidden, kv_heads * head_dim), lin(heads * head_dim, hidden)
        self.q_norm = RMSNorm(head_dim, device=device, dtype=dtype) if qk_norm else None
        self.k_norm = RMSNorm(head_dim, device=device, dtype=dtype) if qk_norm else None

    def forward(self, x, cos, sin):
        b, t, _ = x.shape
        q = self.q_proj(x).view(b, t, self.heads, self.head_dim)
        k = self.k_proj(x).view(b, t, self.kv_heads, self.head_dim)
        v = self.v_proj(x).view(b, t, self.kv_heads, self.head_dim)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)

        def rope(u):
            h = u.shape[-1] // 2
            rot = torch.cat((-u[..., h:], u[..., :h]), dim=-1)
            return u * cos + rot * sin

        q, k = rope(q), rope(k)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.o_proj(o.transpose(1, 2).reshape(b, t, self.heads * self.head_dim))


class MLP(torch.nn.Module):
    def __init__(self, hidden, inter, device, dtype):
        super().__init__()
        lin = lambda i, o: torch.nn.Linear(i, o, bias=False, device=device, dtype=dtype)
        self.gate_proj, self.up_proj, self.down_proj = lin(hidden, inter), lin(hidden, inter), lin(inter, hidden)
        self.hadK, self.K = hu.get_hadK(inter)

    def forward(self, x):
        a = F.silu(self.gate_proj(x)) * self.up_proj(x)
        a = hu.matmul_hadU_cuda(a, self.hadK, self.K)            # online Hadamard on the down_proj input
        return self.down_proj(a)


class DecoderLayer(torch.nn.Module):
    def __init__(self, hidden=4096, inter=12288, heads=32, kv_heads=8, head_dim=128, qk_norm=True, device=None,
                 dtype=torch.bfloat16, seed=0):
        super().__init__()
        self.input_layernorm = RMSNorm(hidden, device=device, dtype=dtype)
        self.self_attn = Attention(hidden, heads, kv_heads, head_dim, qk_norm, device, dtype)
        self.post_attention_layernorm = RMSNorm(hidden, device=device, dtype=dtype)
        self.mlp = MLP(hidden, inter, device, dtype)
        g = torch.Generator(device=device)
        g.manual_seed(1234 + seed)                                # the same weights on every rank
        for m in self.modules():
            if isinstance(m, torch.nn.Linear):
                m.weight.requires_grad_(False)
                m.weight.data.copy_((torch.randn(m.weight.shape, generator=g, device=device) * 0.02).to(dtype))

    def forward(self, x, cos, sin):
        x = x + self.self_attn(self.input_layernorm(x), cos, sin)
        return x + self.mlp(self.post_attention_layernorm(x))


def decoder_layer_stages(cos, sin):
    """DecoderLayer.forward cut at the inputs of the module groups [q, k, v] -> [o] -> [up, gate] -> [down], for
    ``LayerQuantizer(stage_fns=...)``: every stage applies the linears of the group before it and everything up to
    the next group's inputs, exactly the operations of forward() in the same order."""

    def attention_core(attn, h):
        b, t, _ = h.shape
        q = attn.q_proj(h).view(b, t, attn.heads, attn.head_dim)
        k = attn.k_proj(h).view(b, t, attn.kv_heads, attn.head_dim)
        v = attn.v_proj(h).view(b, t, attn.kv_heads, attn.head_dim)
        if attn.q_norm is not None:
            q, k = attn.q_norm(q), attn.k_norm(k)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)

        def rope(u):
            half = u.shape[-1] // 2
            rot = torch.cat((-u[..., half:], u[..., :half]), dim=-1)
            return u * cos + rot * sin

        o = F.scaled_dot_product_attention(rope(q), rope(k), v, is_causal=True, enable_gqa=True)
        return o.transpose(1, 2).reshape(b, t, attn.heads * attn.head_dim)

    def to_qkv(layer, x):                          # carry: the layer input
        h = layer.input_layernorm(x)
        return {"self_attn.q_proj": h, "self_attn.k_proj": h, "self_attn.v_proj": h}, x

    def to_o(layer, x):                            # carry: layer input and the attention output
        a = attention_core(layer.self_attn, layer.input_layernorm(x))
        return {"self_attn.o_proj": a}, (x, a)

    def to_gate_up(layer, carry):                  # carry: the residual stream after attention
        x, a = carry
        y = x + layer.self_attn.o_proj(a)
        h = layer.post_attention_layernorm(y)
        return {"mlp.up_proj": h, "mlp.gate_proj": h}, y

    def to_down(layer, y):                         # carry: residual stream and the rotated down_proj input
        h = layer.post_attention_layernorm(y)
        d = F.silu(layer.mlp.gate_proj(h)) * layer.mlp.up_proj(h)
        d = hu.matmul_hadU_cuda(d, layer.mlp.hadK, layer.mlp.K)
        return {"mlp.down_proj": d}, (y, d)

    def tail(layer, carry):
        y, d = carry
        return y + layer.mlp.down_proj(d)

    return [to_qkv, to_o, to_gate_up, to_down, tail]


def rotary_tables(seq_len, head_dim, device, dtype, theta=1_000_000.0):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype)[None, None], emb.sin().to(dtype)[None, None]
