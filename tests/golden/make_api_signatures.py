"""Records the public call signatures of the reference's classes and functions on the quantization path
(parsed with ``ast``, nothing is imported or executed) into ``api_signatures.json``; ``tests/test_api_surface.py``
holds this package to them.

    python tests/golden/make_api_signatures.py --ref /path/to/reference/checkout
"""
import argparse
import ast
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))

# file -> classes whose public methods are recorded, and whether the module's public functions are recorded
TARGETS = {
    "gptq_utils/gptq_utils.py": (["GPTQ"], False),
    "gptq_utils/gptq_plus_utils.py": (["GPTQPlus", "SaliencyCache"], False),
    "gptq_utils/gptaq_utils.py": (["GPTAQ"], False),
    "gptq_utils/gptq_guided_utils.py": (["GPTQGuided"], False),
    "utils/quant_utils.py": (["WeightQuantizer", "ActQuantizer", "ActQuantWrapper"], False),
    "utils/rotation_utils.py": (["QKRotationWrapper"], False),
    "utils/hadamard_utils.py": ([], True),
    "utils/dist_utils.py": ([], True),
}
# module-level functions of gptq_plus_utils.py that belong to the path
EXTRA_FUNCTIONS = {"gptq_utils/gptq_plus_utils.py": ["clip_module_weight_to_quant_bounds_", "compute_quant_clip_bounds"]}


def signature(fn: ast.FunctionDef):
    a = fn.args
    pos = [x.arg for x in a.posonlyargs + a.args]
    defaults = [None] * (len(pos) - len(a.defaults)) + [ast.unparse(d) for d in a.defaults]
    kwonly = [[x.arg, None if d is None else ast.unparse(d)] for x, d in zip(a.kwonlyargs, a.kw_defaults)]
    return {"args": [[n, d] for n, d in zip(pos, defaults)], "kwonly": kwonly,
            "vararg": a.vararg.arg if a.vararg else None, "kwarg": a.kwarg.arg if a.kwarg else None}


def public(name):
    return not name.startswith("_") or name in ("__init__", "__call__")


def collect(path, classes, functions, extra=()):
    tree = ast.parse(open(path).read())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name in classes:
            out[node.name] = {f.name: signature(f) for f in node.body
                              if isinstance(f, ast.FunctionDef) and public(f.name)}
        elif isinstance(node, ast.FunctionDef) and ((functions and public(node.name)) or node.name in extra):
            out[node.name] = signature(node)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    args = ap.parse_args()
    out = {rel: collect(os.path.join(args.ref, rel), classes, functions, EXTRA_FUNCTIONS.get(rel, ()))
           for rel, (classes, functions) in TARGETS.items()}
    with open(os.path.join(HERE, "api_signatures.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print({k: sorted(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
