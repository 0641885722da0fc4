"""The allocation-free Hessian entry point against the regular one.

rq_hessian_accum_noalloc serves hosts that may not allocate device memory where they feed
calibration batches (for instance a hook that runs while the framework's memory pool is frozen):
its scratch is a fixed 64 MiB array inside the library instead of a caller-provided workspace.
Both entry points run the same kernels, only the token chunking differs, so results must agree to
fp32 summation noise (2e-6 relative Frobenius, the tolerance of the other Hessian tests); two calls
in a row check that the shared array needs no clearing between calls.  Collected last on purpose.
"""
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_fro(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def _noalloc(x, sal, H, act, alpha=1.0, beta=1.0):
    from gptq_plus_mp_quant_b200 import _lib, ops
    N, C = x.shape
    G = sal.shape[1]
    with torch.cuda.device(x.device):
        rc = _lib.lib.rq_hessian_accum_noalloc(_lib.ptr(x), _lib.dtype_code(x), x.stride(0), _lib.ptr(sal), _lib.ptr(H),
                                               _lib.ptr(act), N, C, G, alpha, beta,
                                               _lib.ptr(ops.status_word(x.device)), _lib.stream_of(x))
    return rc


def test_noalloc_matches_regular_entry_point_twice():
    from gptq_plus_mp_quant_b200 import _lib, ops
    assert _lib.lib.rq_hessian_noalloc_scratch_bytes() == 64 * 1024 * 1024
    C, G = 1024, 4
    H_ref = torch.zeros(G, C, C, device=DEV)
    H_new = torch.zeros(G, C, C, device=DEV)
    a_ref = torch.zeros(C, device=DEV)
    a_new = torch.zeros(C, device=DEV)
    for call, (tokens, dtype) in enumerate([(5000, torch.float32), (3000, torch.bfloat16)]):
        X = cases.make_acts(1, tokens, C, seed=50 + call, dtype=dtype).reshape(tokens, C).to(DEV)
        S = cases.make_saliency(1, tokens, G, seed=50 + call).reshape(tokens, G).to(DEV)
        ops.hessian_accum(X, S, H_ref, a_ref)
        assert _noalloc(X, S, H_new, a_new) == _lib.RQ_OK              # several chunks: 64 MiB holds ~3000 tokens here
        torch.cuda.synchronize()
        ops.check_status(torch.device(DEV))
        up = torch.triu(torch.ones(C, C, device=DEV, dtype=torch.bool))  # both maintain the upper triangle
        assert rel_fro(H_new[:, up], H_ref[:, up]) < 2e-6, f"call {call}"
        assert torch.allclose(a_new, a_ref, rtol=2e-6, atol=0)


def test_noalloc_rejects_oversized_problem():
    from gptq_plus_mp_quant_b200 import _lib
    C, G = 65536, 8                                                   # one 64-token chunk would need ~151 MB
    x = torch.zeros(1, 8, device=DEV)                                 # never read: the size check comes first
    rc = _lib.lib.rq_hessian_accum_noalloc(_lib.ptr(x), 0, C, _lib.ptr(x), _lib.ptr(x), 0, 64, C, G, 1.0, 1.0, 0,
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.RQ_ERR_TOO_LARGE
    assert "64 MiB" in _lib.error_string(rc)
