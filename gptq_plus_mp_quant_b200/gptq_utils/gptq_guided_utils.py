"""GuidedQuant on B200: the ``GPTQGuided`` object of the reference's ``gptq_utils/gptq_guided_utils.py``
(:14-271): saliency-grouped Hessians like GPTQ+, no first-order terms, the Hessians used as raw sums.  Same
methods, arguments and attributes; the numerical work runs in the kernels of this package."""
from __future__ import annotations

import logging

import torch

from .. import ops
from . import fasterquant_impl


class GPTQGuided:
    def __init__(self, layer, saliency: torch.Tensor, num_groups: int):
        self.layer = layer
        self.dev = self.layer.weight.device
        self.rows = layer.weight.shape[0]
        self.columns = layer.weight.shape[1]
        self.num_groups = num_groups
        assert self.num_groups == saliency.shape[2], "Number of groups for GuidedQuant must match saliency shape!"
        self.saliencies = saliency.float()
        # kept group-major [G, C, C] for the kernels; ``H`` shows the reference's [C, C, G] layout
        self._H = torch.zeros((self.num_groups, self.columns, self.columns), device=self.dev)
        self._H_upper_only = False
        self.act_square = torch.zeros((self.columns), device=self.dev)
        self._act_batch = torch.zeros((self.columns), device=self.dev)
        self.nsamples = saliency.shape[0]
        self.index = 0
        self.profile_recorder = None
        assert self.rows % self.num_groups == 0, (
            f"Number of rows ({self.rows}) must be divisible by num_groups ({self.num_groups})")

    def _full_H(self):
        if self._H is not None and self._H_upper_only:
            ops.hessian_finalize(self._H, None)
            self._H_upper_only = False
        return self._H

    @property
    def H(self):
        full = self._full_H()
        return None if full is None else full.permute(1, 2, 0)

    @H.setter
    def H(self, value):
        self._H = None if value is None else value.permute(2, 0, 1).contiguous()
        self._H_upper_only = False

    @torch.no_grad()
    def add_batch(self, inp: torch.Tensor, out):
        """``H[..., g] += X^T diag(s_g) X`` and ``act_square += sum x^2 / n_tokens`` (gptq_guided_utils.py:49-81)."""
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        else:
            assert inp.dim() == 3, "Input must be 2D or 3D. Got %dD." % inp.dim()
        bsz = inp.shape[0]
        sal_batch = self.saliencies[self.index: self.index + bsz].to(self.dev)
        self.index += bsz
        inp = inp.reshape(-1, inp.shape[-1])
        sal_batch = sal_batch.reshape(-1, sal_batch.shape[-1])
        n_tokens = inp.shape[0]
        self._act_batch.zero_()
        ops.hessian_accum(inp, sal_batch, self._H, self._act_batch, alpha=1.0, beta=1.0)
        self._H_upper_only = True
        self.act_square.add_(self._act_batch, alpha=1 / n_tokens)

    def __repr__(self):
        return (f"GPTQGuided(H.shape={(self.columns, self.columns, self.num_groups)}, "
                f"index/nsamples={self.index}/{self.nsamples})")

    def fasterquant(self, blocksize=128, percdamp=0.01, groupsize=-1, actorder=False, static_groups=False,
                    export_to_et=False):
        """gptq_guided_utils.py:86-259."""
        ops.check_status(self.dev)
        fasterquant_impl.guided_fasterquant(self, self._full_H(), blocksize, percdamp, groupsize, actorder,
                                            static_groups, export_to_et)
        if torch.any(torch.isnan(self.layer.weight.data)):
            logging.warning("NaN in weights")
            raise ValueError("NaN in weights")

    def free(self):
        ops.hessian_join(self.dev)
        self._H = None
        self.Losses = None
