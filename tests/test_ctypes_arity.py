"""Every ``b200_*`` entry point Python calls through ctypes is declared in the native sources with the same number of
parameters (no ``argtypes`` are set, so nothing else would notice a call that drifted from its prototype until it ran
on a GPU)."""
import ast
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "deepseek_v4_2080ti_b200")
RET = r"(?:int|void|long long|float|double|const char\s*\*|unsigned long long|size_t)"


def _prototypes() -> dict[str, set[int]]:
    out: dict[str, set[int]] = {}
    for dp, _, fn in os.walk(os.path.join(PKG, "csrc")):
        for f in fn:
            if not f.endswith((".h", ".hpp", ".cuh", ".cu", ".cpp")):
                continue
            src = open(os.path.join(dp, f)).read()
            src = re.sub(r"/\*.*?\*/", "", re.sub(r"//[^\n]*", "", src), flags=re.S)
            for m in re.finditer(r"\b" + RET + r"\s+(b200_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*[;{]", src, flags=re.S):
                args = m.group(2).strip()
                out.setdefault(m.group(1), set()).add(0 if args in ("", "void") else args.count(",") + 1)
    return out


def test_calls_match_their_prototypes():
    protos = _prototypes()
    assert len(protos) > 80
    bad, called = [], set()
    tops = [os.path.join(ROOT, t) for t in ("deepseek_v4_2080ti_b200", "tests", "pocketllm", "baseline")] + [os.path.join(ROOT, "bench.py")]
    for top in tops:
        files = [top] if top.endswith(".py") else [os.path.join(dp, f) for dp, dn, fn in os.walk(top) if "_ref" not in dp for f in fn if f.endswith(".py")]
        for path in files:
            for n in ast.walk(ast.parse(open(path).read(), path)):
                if isinstance(n, ast.Call) and isinstance(n.func, ast.Attribute) and n.func.attr.startswith("b200_"):
                    name = n.func.attr
                    called.add(name)
                    if any(isinstance(a, ast.Starred) for a in n.args) or n.keywords:
                        continue
                    where = f"{os.path.relpath(path, ROOT)}:{n.lineno}"
                    if name not in protos:
                        bad.append(f"{where}: {name} is not declared in the native sources")
                    elif len(n.args) not in protos[name]:
                        bad.append(f"{where}: {name} called with {len(n.args)} arguments, declared with {sorted(protos[name])}")
    assert not bad, "\n".join(bad)
    assert len(called) > 60
