"""GPTAQ on B200: the ``GPTAQ`` object of the reference's ``gptq_utils/gptaq_utils.py`` (:14-167), GPTQ with an
asymmetric-calibration term: besides ``H`` it accumulates ``dXXT`` from the full-precision inputs the caller queues
in ``fp_inp``.  Same methods, arguments and attributes; the numerical work runs in the kernels of this package."""
from __future__ import annotations

import logging
import math

import torch

from .. import _lib, ops
from . import fasterquant_impl


class GPTAQ:
    def __init__(self, layer):
        self.layer = layer
        self.dev = self.layer.weight.device
        self.rows = layer.weight.shape[0]
        self.columns = layer.weight.shape[1]
        self._H = torch.zeros((self.columns, self.columns), device=self.dev)
        self._H_upper_only = False
        self.dXXT = torch.zeros((self.columns, self.columns), device=self.dev)
        self.nsamples = 0
        self.fp_inp = []

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
        """Running means of ``(2/n) X^T X`` and ``(2/n) (X_fp - X)^T X`` with n counted in sequences
        (gptaq_utils.py:26-41); the full-precision input of this batch is taken from the front of ``fp_inp``."""
        if len(inp.shape) == 2:
            inp = inp.unsqueeze(0)
        tmp = inp.shape[0]
        if len(inp.shape) == 3:
            inp = inp.reshape((-1, inp.shape[-1]))
        beta = self.nsamples / (self.nsamples + tmp)
        self.nsamples += tmp
        ops.hessian_accum(inp, None, self._H, None, alpha=2.0 / self.nsamples, beta=beta)
        self._H_upper_only = True
        # the reference queues the full-precision input channel-major, [C, tokens] (gptaq_utils.py:185-189)
        fp = self.fp_inp[0].to(self.dev)
        x = inp if inp.stride(1) == 1 else inp.contiguous()
        N, Cc = x.shape
        assert fp.dim() == 2 and tuple(fp.shape) == (Cc, N), "fp_inp[0] must be the [C, tokens] input of this batch"
        fp = fp if fp.stride(1) == 1 else fp.contiguous()
        with torch.cuda.device(self.dev):
            need = _lib.lib.rq_gptaq_accum_workspace_bytes(N, Cc)
            ws = ops._workspace(self.dev, need + 1024, key="gptaq_accum")
            base = (ws.data_ptr() + 1023) // 1024 * 1024
            rc = _lib.lib.rq_gptaq_accum(_lib.ptr(x), _lib.dtype_code(x), x.stride(0), _lib.ptr(fp), _lib.dtype_code(fp),
                                         fp.stride(0), 1, N, Cc, float(math.sqrt(2 / self.nsamples)), float(beta),
                                         _lib.ptr(self.dXXT), base, need, _lib.ptr(ops.status_word(self.dev)),
                                         _lib.stream_of(x))
        _lib.check("rq_gptaq_accum", rc)
        del self.fp_inp[0]

    def fasterquant(self, blocksize=128, percdamp=0.01, groupsize=-1, actorder=False, static_groups=False, alpha=0.25):
        """gptaq_utils.py:43-167."""
        ops.check_status(self.dev)
        H = self.H
        del self.H
        fasterquant_impl.gptaq_fasterquant(self, H, blocksize, percdamp, groupsize, actorder, static_groups, alpha)
        del self.dXXT
        if torch.any(torch.isnan(self.layer.weight.data)):
            logging.warning("NaN in weights")
            raise ValueError("NaN in weights")

    def free(self):
        ops.hessian_join(self.dev)
        self.H = None
        self.Losses = None
        self.dXXT = None
