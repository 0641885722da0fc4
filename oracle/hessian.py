"""Oracle: Hessian accumulation for plain GPTQ and saliency-grouped GPTQ+.

Test infrastructure (see ``oracle/__init__.py``).  Restates

* ``GPTQ.add_batch``            gptq_utils/gptq_utils.py:33-43
* ``GPTQPlus.add_batch``        gptq_utils/gptq_plus_utils.py:798-857
* ``GPTQPlus.finalize_hessian`` gptq_utils/gptq_plus_utils.py:859-908
"""
from __future__ import annotations

import math

import torch


class PlainHessian:
    """Running-mean Gram matrix of plain GPTQ: after every call
    ``H = (2 / n_seq) * sum_tokens x x^T`` where ``n_seq`` counts *sequences*
    (gptq_utils.py:33-43)."""

    def __init__(self, columns: int):
        self.H = torch.zeros(columns, columns)
        self.nsamples = 0

    def add_batch(self, inp: torch.Tensor):
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        b = inp.shape[0]
        x = inp.reshape(-1, inp.shape[-1]).t()
        self.H *= self.nsamples / (self.nsamples + b)
        self.nsamples += b
        x = math.sqrt(2 / self.nsamples) * x.float()
        self.H += x.matmul(x.t())


class GroupedHessian:
    """Saliency-weighted per-group sums of GPTQ+:

    ``H[g] += X^T diag(s[:, g]) X`` and ``act_square += sum_tokens x^2`` as pure sums
    (gptq_plus_utils.py:798-857); ``finalize`` divides by the token count and the
    saliency scale, divides ``act_square`` by the sequence length, symmetrises and
    zeroes non-finite entries (:859-908).  The cross-rank all-reduce of the
    reference (:875-878) is the caller's business: pass pre-summed state or use
    :func:`merge` to emulate it.
    """

    def __init__(self, columns: int, saliency: torch.Tensor, hessian_saliency_scale: float = 1.0):
        self.G = saliency.shape[2]
        self.saliencies = saliency.float()
        self.H = torch.zeros(self.G, columns, columns)
        self.act_square = torch.zeros(columns)
        self.index = 0
        self.token_count = 0
        self.scale = float(hessian_saliency_scale)
        self.finalized = False

    def add_batch(self, inp: torch.Tensor):
        if self.finalized:
            raise RuntimeError("add_batch called after finalize_hessian")
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        assert inp.dim() == 3
        b = inp.shape[0]
        sal = self.saliencies[self.index:self.index + b]
        self.index += b
        if inp.shape[1] > sal.shape[1]:            # leading "sink" tokens carry no saliency (:833-835)
            inp = inp[:, inp.shape[1] - sal.shape[1]:]
        x = inp.reshape(-1, inp.shape[-1]).float()
        s = sal.reshape(-1, sal.shape[-1]).float()
        weighted = x.unsqueeze(0) * s.t().unsqueeze(-1)                  # [G, N, C]
        self.H += torch.bmm(x.t().unsqueeze(0).expand(self.G, -1, -1), weighted)
        self.act_square += (x ** 2).sum(0)
        self.token_count += x.shape[0]

    @staticmethod
    def merge(parts):
        """Sum the un-normalised state of several shards into the first one: what the
        NCCL all-reduce in ``finalize_hessian`` does across ranks (:875-878)."""
        head = parts[0]
        for p in parts[1:]:
            head.H += p.H
            head.act_square += p.act_square
            head.index += p.index
            head.token_count += p.token_count
        return head

    def finalize(self):
        """Returns (n_nan, n_inf) found before sanitising."""
        if self.finalized:
            return 0, 0
        if self.index <= 0 or self.token_count <= 0:
            raise RuntimeError("finalize_hessian called before any add_batch ran.")
        seq_len = float(self.token_count) / float(self.index)
        self.H.div_(float(self.index) * seq_len)
        if self.scale != 1.0:
            self.H.div_(self.scale)
        self.act_square.div_(seq_len)
        self.H = 0.5 * (self.H + self.H.transpose(-1, -2))
        n_nan = int(torch.isnan(self.H).sum())
        n_inf = int(torch.isinf(self.H).sum())
        if n_nan or n_inf:
            self.H = torch.nan_to_num(self.H, nan=0.0, posinf=0.0, neginf=0.0)
        self.finalized = True
        return n_nan, n_inf


def group_mean_square(grad, num_groups, sink_size=0):
    """The gradient hook of SaliencyCache (gptq_utils/gptq_plus_utils.py:2388-2404): mean squared gradient per
    channel group and token, sink positions dropped."""
    g = grad
    if sink_size > 0 and g.dim() >= 2 and g.shape[1] > sink_size:
        g = g[:, sink_size:]
    bsz, seq_len, hidden_dim = g.shape
    group_size = hidden_dim // num_groups
    return g.float().pow(2).view(bsz, seq_len, num_groups, group_size).mean(dim=-1)


def clip_at_percentile(sal, q):
    """Saliency outlier clip of the calibration hook (gptq_utils/gptq_plus_utils.py:2834-2839):
    ``clamp(sal, max=torch.quantile(sal.flatten(), q))``, with torch.quantile restated: sort, rank = fl32(q) * fl32(n-1),
    two-sided lerp between the neighbouring order statistics.  Returns (clipped, cap)."""
    import numpy as np
    flat = np.sort(sal.detach().float().flatten().numpy())
    n = flat.size
    rank = np.float32(q) * np.float32(n - 1)
    below, above = int(np.floor(rank)), int(np.ceil(rank))
    w = np.float32(rank - np.float32(below))
    lo, hi = flat[below], flat[above]
    cap = lo + w * (hi - lo) if abs(w) < 0.5 else hi - (hi - lo) * (np.float32(1) - w)
    if np.isnan(flat).any():
        cap = np.float32(np.nan)
    cap_t = torch.tensor(cap, dtype=torch.float32)
    return torch.clamp(sal.float(), max=cap_t), cap_t


def fisher_block(grad, sink_size=0, scale=1000.0 * 1000.0):
    """One batch's contribution to the layer-output Fisher sum (gptq_utils/gptq_plus_utils.py:2908-2921)."""
    if sink_size > 0 and grad.dim() >= 2 and grad.shape[1] > sink_size:
        grad = grad[:, sink_size:]
    flat = grad.detach().float().reshape(-1, grad.shape[-1])
    out = flat.t() @ flat
    out.div_(scale)
    return out
