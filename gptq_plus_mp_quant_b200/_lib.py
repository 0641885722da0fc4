"""ctypes binding of ``librealq_b200.so`` (the C ABI declared in ``include/realq_b200.h``).

There is no fallback: if the shared library is absent the import fails, and every wrapper
raises when a kernel reports an error.  Tensors stay owned by torch; the wrappers only pass
raw device pointers, sizes and the current CUDA stream.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# REALQ_B200_LIB names another build of the same library (same exports), e.g. one compiled with different tuning macros
LIB_PATH = os.environ.get("REALQ_B200_LIB") or os.path.join(_HERE, "csrc", "librealq_b200.so")

RQ_OK, RQ_ERR_INVALID, RQ_ERR_CUDA, RQ_ERR_TIMEOUT, RQ_ERR_WORKSPACE, RQ_ERR_UNSUPPORTED, RQ_ERR_TOO_LARGE = range(7)
RQ_F32, RQ_BF16, RQ_F16 = 0, 1, 2
_DTYPES = {torch.float32: RQ_F32, torch.bfloat16: RQ_BF16, torch.float16: RQ_F16}

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "rq_version": (_i, []),
    "rq_error_string": (C.c_char_p, [_i]),
    "rq_profile_enable": (_i, [_i]),
    "rq_profile_read": (_i, [_i, C.POINTER(C.c_double), C.POINTER(C.c_longlong)]),
    "rq_hessian_workspace_bytes": (_sz, [_i64, _i, _i, _i]),
    "rq_hessian_accum": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _i64, _i, _i, _f, _f, _vp, _sz, _vp, _i, _vp]),
    "rq_group_mean_square": (_i, [_vp, _i, _i64, _i64, _i64, _i64, _i, _i, _vp, _vp]),
    "rq_quantile_workspace_bytes": (_sz, []),
    "rq_clamp_to_quantile": (_i, [_vp, _i64, _f, _vp, _vp, _sz, _vp]),
    "rq_gptaq_accum_workspace_bytes": (_sz, [_i64, _i]),
    "rq_gptaq_accum": (_i, [_vp, _i, _i64, _vp, _i, _i64, _i, _i64, _i, _f, _f, _vp, _vp, _sz, _vp, _vp]),
    "rq_gptaq_workspace_bytes": (_sz, [_i, _i]),
    "rq_gptaq_terms": (_i, [_vp, _vp, _vp, _vp, _i, _f, _vp, _vp, _sz, _vp, _vp]),
    "rq_gptaq_run": (_i, [_vp] * 9 + [_i] * 6 + [_vp, _sz, _vp, _vp]),
    "rq_fwht_heads": (_i, [_vp, _vp, _i, _i64, _i, _i, _i, _vp, _f, _vp]),
    "rq_packed_row_bytes": (_i64, [_i64, _i]),
    "rq_pack_codes": (_i, [_vp, _i64, _i64, _i64, _i, _vp, _vp]),
    "rq_act_quant": (_i, [_vp, _vp, _i, _i64, _i, _i, _f, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "rq_group_mse_search": (_i, [_vp, _i, _i64, _i, _i, _i, _f, _i, _f, _vp, _vp, _vp]),
    "rq_clip_to_quant_bounds": (_i, [_vp, _i, _i64, _i64, _i64, _vp, _vp, _i, _i, _vp]),
    "rq_hessian_accum_pipelined": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _i64, _i, _i, _f, _f, _vp, _sz, _vp, _i, _i64,
                                        _vp, _vp]),
    "rq_hessian_noalloc_scratch_bytes": (_sz, []),
    "rq_hessian_accum_noalloc": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _i64, _i, _i, _f, _f, _vp, _vp]),
    "rq_hessian_packed_elems": (_i64, [_i]),
    "rq_hessian_pack_upper": (_i, [_vp, _i, _i, _vp, _i64, _vp]),
    "rq_hessian_unpack_upper": (_i, [_vp, _i64, _i, _i, _vp, _vp]),
    "rq_hessian_finalize": (_i, [_vp, _vp, _i, _i, _f, _f, _f, _i, _vp, _vp]),
    "rq_fwht": (_i, [_vp, _vp, _i, _i64, _i, _i, _vp, _f, _vp]),
    "rq_fwht_act_quant": (_i, [_vp, _vp, _i, _i64, _i, _i, _vp, _f, _f, _i, _i, _vp, _vp, _vp]),
    "rq_find_params": (_i, [_vp, _i64, _i64, _i64, _i, _i, _i, _i, _i, _f, _i, _f, _vp, _vp, _vp]),
    "rq_quantize": (_i, [_vp, _vp, _vp, _i, _i64, _i64, _vp, _vp, _i, _i, _i, _vp]),
    "rq_chol_workspace_bytes": (_sz, [_i, _i]),
    "rq_chol_hinv": (_i, [_vp, _vp, C.POINTER(C.c_float), _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "rq_chol_hinv_flags": (_i, [_vp, _vp, C.POINTER(C.c_float), _vp, _i, _i, _vp, _vp, _sz, _i, _vp]),
    "rq_fq_prepare": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "rq_gptqplus_terms": (_i, [_vp, _vp, _i, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _vp]),
    "rq_fq_block": (_i, [_vp] * 11 + [_i] * 10 + [_vp, _vp, _i, _i, _f, _vp]),
    "rq_fq_lazy_update": (_i, [_vp] * 5 + [_i] * 6 + [_vp, _vp, _i, _f, _vp]),
    "rq_fq_run": (_i, [_vp] * 11 + [_i] * 8 + [_vp, _vp, _i, _i, _vp]),
    "rq_fq_tc_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "rq_fq_tc_prepare": (_i, [_vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "rq_gptqplus_terms_tc": (_i, [_vp, _vp, _i, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "rq_fq_run_tc": (_i, [_vp] * 11 + [_i] * 8 + [_vp, _vp, _i, _i, _vp, _sz, _vp, _vp]),
    "rq_fq_finish": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
}


class RealQError(RuntimeError):
    """A kernel entry point returned a non-zero status."""

    def __init__(self, fn: str, code: int):
        self.code = code
        super().__init__(f"{fn} failed: [{code}] {error_string(code)}")


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built "
            "(run `python -m gptq_plus_mp_quant_b200.csrc.build`); there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)            # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def error_string(code: int) -> str:
    return lib.rq_error_string(int(code)).decode()


def check(fn: str, code: int) -> None:
    if code != RQ_OK:
        raise RealQError(fn, code)


PROF_HESSIAN_UMMA, PROF_HESSIAN_PACK, PROF_FWHT, PROF_CHOL, PROF_BLOCK, PROF_LAZY = 1, 2, 3, 4, 5, 6
PROF_CHOL_DIAG, PROF_CHOL_PANEL, PROF_CHOL_TRAILING, PROF_CHOL_INVERSE, PROF_TERMS = 7, 8, 9, 10, 11


def profile_enable(on: bool) -> None:
    check("rq_profile_enable", lib.rq_profile_enable(1 if on else 0))


def profile_read(tag: int):
    """(total milliseconds, launches) of one tagged kernel since profile_enable(True)."""
    ms, n = C.c_double(0.0), C.c_longlong(0)
    check("rq_profile_read", lib.rq_profile_read(tag, C.byref(ms), C.byref(n)))
    return ms.value, n.value


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("realq_b200 kernels need CUDA tensors: there is no CPU fallback")
