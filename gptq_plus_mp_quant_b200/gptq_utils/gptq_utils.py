"""Plain GPTQ on B200: the ``GPTQ`` object of the reference's ``gptq_utils/gptq_utils.py``
(:23-180) with the same methods, arguments and attributes, its numerical work done by the
sm_100a kernels of this package."""
from __future__ import annotations

import logging

import torch

from .. import ops
from . import fasterquant_impl


class GPTQ:
    def __init__(self, layer):
        self.layer = layer
        self.dev = self.layer.weight.device
        self.rows = layer.weight.shape[0]
        self.columns = layer.weight.shape[1]
        # The accumulation kernel maintains the tiles on or above the diagonal; the lower
        # triangle is filled in when ``H`` is read.
        self._H = torch.zeros((self.columns, self.columns), device=self.dev)
        self._H_upper_only = False
        self.nsamples = 0

    # ``H`` stays the full symmetric matrix for every reader
    @property
    def H(self):
        if self._H is not None and self._H_upper_only:
            ops.hessian_finalize(self._H, None)
            self._H_upper_only = False
        return self._H

    @H.setter
    def H(self, value):
        self._H = value
        self._H_upper_only = False

    @H.deleter
    def H(self):
        self._H = None

    def add_batch(self, inp, out):
        """``H = H*n/(n+b) + (2/(n+b)) X^T X`` with n, b counted in sequences (gptq_utils.py:33-43)."""
        if len(inp.shape) == 2:
            inp = inp.unsqueeze(0)
        tmp = inp.shape[0]
        if len(inp.shape) == 3:
            inp = inp.reshape((-1, inp.shape[-1]))
        beta = self.nsamples / (self.nsamples + tmp)
        self.nsamples += tmp
        ops.hessian_accum(inp, None, self._H, None, alpha=2.0 / self.nsamples, beta=beta,
                          pipeline=ops.HESSIAN_PIPELINE)
        self._H_upper_only = True

    def fasterquant(self, blocksize=128, percdamp=0.01, groupsize=-1, actorder=False, static_groups=False,
                    export_to_et=False):
        """gptq_utils.py:45-174."""
        ops.check_status(self.dev)
        H = self.H
        del self.H
        fasterquant_impl.plain_fasterquant(self, H, blocksize, percdamp, groupsize, actorder, static_groups,
                                           export_to_et)
        if torch.any(torch.isnan(self.layer.weight.data)):
            logging.warning("NaN in weights")
            raise ValueError("NaN in weights")

    def free(self):
        # Drops the Hessian; unlike the reference this does not return cached blocks to the driver
        # (torch.cuda.empty_cache / cleanup_memory): the next linear re-uses them without a cudaMalloc.
        ops.hessian_join(self.dev)          # no contraction may still be writing the buffer that is released
        self.H = None
        self.Losses = None
