"""The drop-in boundary at the Python level: every public method and function the reference offers on the
quantization path exists here under the same name, takes the same arguments in the same order and with the same
defaults (fixture: tests/golden/api_signatures.json, parsed from the reference's sources by
tests/golden/make_api_signatures.py).  Extra keyword arguments after the reference's own are allowed (they must
have defaults); sources are parsed, nothing is imported, so the check runs without the CUDA library."""
import ast
import json
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "gptq_plus_mp_quant_b200")
FIXTURE = json.load(open(os.path.join(ROOT, "tests", "golden", "api_signatures.json")))

# what this package leaves out on purpose, with the reason
OMITTED = {
    ("utils/dist_utils.py", "distribute_model"): "model placement across devices belongs to the caller's launcher",
}


def _sig(fn):
    a = fn.args
    pos = [x.arg for x in a.posonlyargs + a.args]
    defaults = [None] * (len(pos) - len(a.defaults)) + [ast.unparse(d) for d in a.defaults]
    kwonly = {x.arg: (None if d is None else ast.unparse(d)) for x, d in zip(a.kwonlyargs, a.kw_defaults)}
    return list(zip(pos, defaults)), kwonly, bool(a.vararg), bool(a.kwarg)


def _ours(rel):
    tree = ast.parse(open(os.path.join(PKG, rel)).read())
    classes, functions = {}, {}
    for node in tree.body:
        if isinstance(node, ast.ClassDef):
            classes[node.name] = {f.name: f for f in node.body if isinstance(f, ast.FunctionDef)}
        elif isinstance(node, ast.FunctionDef):
            functions[node.name] = node
    return classes, functions


def _norm(default):
    """Defaults compare as source text, up to quoting and float spelling."""
    if default is None:
        return None
    try:
        return repr(ast.literal_eval(default))
    except Exception:
        return default.replace('"', "'")


def _check(where, ref, fn):
    args, kwonly, has_var, has_kw = _sig(fn)
    ref_args = [(n, d) for n, d in ref["args"]]
    assert len(args) >= len(ref_args) or has_var or has_kw, f"{where}: takes fewer arguments than the reference"
    for i, (name, default) in enumerate(ref_args):
        if i >= len(args):
            assert has_kw or has_var, f"{where}: argument {name!r} missing"
            continue
        assert args[i][0] == name, f"{where}: argument {i} is {args[i][0]!r}, the reference has {name!r}"
        if default is not None:
            assert args[i][1] is not None, f"{where}: {name!r} has a default in the reference"
            assert _norm(args[i][1]) == _norm(default), f"{where}: default of {name!r} is {args[i][1]}, reference {default}"
        else:
            assert args[i][1] is None or name == "self", f"{where}: {name!r} is required in the reference"
    for name, default in args[len(ref_args):]:
        assert default is not None, f"{where}: extra argument {name!r} needs a default"
    for name, default in ref["kwonly"]:
        assert name in kwonly or has_kw, f"{where}: keyword-only argument {name!r} missing"


CASES = []
for rel, entries in sorted(FIXTURE.items()):
    for name, body in sorted(entries.items()):
        if "args" in body:                                   # a module-level function
            CASES.append((rel, None, name, body))
        else:
            for meth, sig in sorted(body.items()):
                CASES.append((rel, name, meth, sig))


@pytest.mark.parametrize("rel,cls,name,ref", CASES, ids=lambda v: v if isinstance(v, str) else None)
def test_signature_matches_reference(rel, cls, name, ref):
    if (rel, name) in OMITTED and cls is None:
        pytest.skip(OMITTED[(rel, name)])
    classes, functions = _ours(rel)
    if cls is None:
        assert name in functions, f"{rel}: function {name} missing"
        _check(f"{rel}:{name}", ref, functions[name])
    else:
        assert cls in classes, f"{rel}: class {cls} missing"
        assert name in classes[cls], f"{rel}: {cls}.{name} missing"
        _check(f"{rel}:{cls}.{name}", ref, classes[cls][name])
