"""Test infrastructure: imports the reference's own modules from ``oracle/_ref/`` (see make_ref.py) for the CPU arm
of the benchmark.  Returns None when that copy is absent; the caller then times the oracle port instead."""
from __future__ import annotations

import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def load():
    """dict(gptq_utils, gptq_plus_utils, quant_utils, hadamard_utils) of the UNMODIFIED reference, or None."""
    if not os.path.isfile(os.path.join(REF, "gptq_utils", "gptq_plus_utils.py")):
        return None
    import torch
    import transformers  # noqa: F401  (must precede the reference's own imports)
    for name, attrs in (("accelerate", ("dispatch_model", "infer_auto_device_map")),
                        ("accelerate.utils", ("get_balanced_memory",)),
                        ("accelerate.hooks", ("remove_hook_from_module",))):
        if name not in sys.modules:
            mod = types.ModuleType(name)
            for a in attrs:
                setattr(mod, a, lambda *args, **kw: None)
            sys.modules[name] = mod
    # the reference's packages are called `utils` and `gptq_utils`: import them with its root first on the path,
    # then take the path entry out again so that nothing else resolves against it
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "utils" or k.startswith("utils.")
             or k == "gptq_utils" or k.startswith("gptq_utils.")}
    sys.path.insert(0, REF)
    try:
        from utils import quant_utils, hadamard_utils, memory_utils
        from gptq_utils import gptq_utils, gptq_plus_utils
    finally:
        sys.path.remove(REF)
    mods = dict(gptq_utils=gptq_utils, gptq_plus_utils=gptq_plus_utils, quant_utils=quant_utils,
                hadamard_utils=hadamard_utils)
    # CPU tensors only: the two CUDA-only housekeeping calls become no-ops (gptq_utils.py:155, memory_utils.py:12-39)
    if not torch.cuda.is_available():
        torch.cuda.synchronize = lambda *a, **k: None
    memory_utils.cleanup_memory = lambda *a, **k: None
    for k, v in saved.items():
        sys.modules.setdefault(k, v)
    return mods
