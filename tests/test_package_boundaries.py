"""Layering rules of the package, checked on the import statements (Python) and the include lines (native sources).

Python, module-level imports only - an import inside a function is the sanctioned way to reach upward lazily:

* ``pocketllm`` (control plane) never imports the model package at module level, so importing it stays torch-free.
* ``formats`` and ``encoding`` are leaves: nothing from ``ops / models / components / parallel / runtime / cli``.
* ``ops`` (kernel seam) sees ``formats`` and ``utils`` only; ``parallel`` sees ``ops`` and ``utils``.
* ``components`` do not import ``runtime``, ``parallel`` or ``cli``, and of ``models`` only the pure-math
  ``*_components`` modules.
* ``models`` do not import the loaders (``runtime.loader``, ``runtime.host_runtime``), ``cli`` or ``pocketllm``; the
  storage helpers ``runtime.prefix_cache`` and ``runtime.kv_swap`` are allowed.
* nothing below ``cli`` imports ``cli``; ``utils.canary`` imports nothing from the package.

Native: ``core`` (host runtime) includes no kernel, comm or engine header; ``kernels`` and ``comm`` include nothing from
``core`` or ``engine``; only ``engine`` and ``bindings`` sit on top of everything.

The reference enforces its own layering the same way (tests/test_package_boundaries.py:72-125, cmake/CheckLayering.cmake).
"""
import ast
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "deepseek_v4_2080ti_b200"


def _module_level_imports(path: str, rel: list[str]) -> list[str]:
    """Dotted names (inside PKG, or ``pocketllm...``) imported by statements that are not inside a function."""
    tree = ast.parse(open(path).read(), path)
    out: list[str] = []

    def visit(node, in_func):
        for child in ast.iter_child_nodes(node):
            inside = in_func or isinstance(child, (ast.FunctionDef, ast.AsyncFunctionDef, ast.Lambda))
            if not in_func and isinstance(child, ast.ImportFrom):
                if child.level:
                    base = rel[:-1]
                    base = base[:len(base) - (child.level - 1)] if child.level > 1 else base
                    mod = base + (child.module.split(".") if child.module else [])
                    names = [".".join(mod + [a.name]) for a in child.names] if not child.module or len(mod) <= 1 else [".".join(mod)]
                    out.extend(names)
                elif child.module and child.module.split(".")[0] == PKG:
                    out.append(".".join(child.module.split(".")[1:]) or ".".join(a.name for a in child.names))
                elif child.module and child.module.split(".")[0] == "pocketllm":
                    out.append(child.module)
            elif not in_func and isinstance(child, ast.Import):
                for a in child.names:
                    top = a.name.split(".")[0]
                    if top == PKG:
                        out.append(".".join(a.name.split(".")[1:]))
                    elif top == "pocketllm":
                        out.append(a.name)
            visit(child, inside)
    visit(tree, False)
    return [o for o in out if o]


def _package_files(pkg_dir: str):
    for dp, dn, fn in os.walk(pkg_dir):
        dn[:] = [d for d in dn if d not in ("__pycache__", "csrc", "lib", "bin", "build_tmp")]
        for f in fn:
            if f.endswith(".py"):
                yield os.path.join(dp, f)


def _graph():
    g: dict[str, list[tuple[str, str]]] = {}
    base = os.path.join(ROOT, PKG)
    for path in _package_files(base):
        rel = os.path.relpath(path, base).split(os.sep)
        rel[-1] = rel[-1][:-3]
        layer = rel[0] if len(rel) > 1 else "<top>"
        for name in _module_level_imports(path, rel):
            g.setdefault(layer, []).append((name, os.path.relpath(path, ROOT)))
    return g


RULES = {
    "formats": lambda n: n.split(".")[0] in ("formats",),
    "encoding": lambda n: n.split(".")[0] in ("encoding", "formats"),
    "ops": lambda n: n.split(".")[0] in ("ops", "formats", "utils", "build"),
    "parallel": lambda n: n.split(".")[0] in ("parallel", "ops", "utils"),
    "components": lambda n: n.split(".")[0] in ("components", "ops", "formats", "utils")
    or (n.split(".")[0] == "models" and n.split(".")[1].endswith("_components")),
    "models": lambda n: n.split(".")[0] in ("models", "components", "ops", "formats", "utils", "parallel", "encoding", "build")
    or n in ("runtime.prefix_cache", "runtime.kv_swap"),
    "runtime": lambda n: n.split(".")[0] != "cli" and not n.startswith("pocketllm"),
    "utils": lambda n: n.split(".")[0] != "cli" and not n.startswith("pocketllm"),
}


def test_python_layers_import_downward_only():
    g = _graph()
    assert set(RULES) <= set(g) | {"formats"}, sorted(g)
    bad = [(layer, name, path) for layer, rule in RULES.items() for name, path in g.get(layer, []) if not rule(name)]
    assert not bad, "\n".join(f"{p}: {l} imports {n}" for l, n, p in bad)
    # the guard-band helper is a leaf inside utils
    canary = os.path.join(ROOT, PKG, "utils", "canary.py")
    assert _module_level_imports(canary, ["utils", "canary"]) == []


def test_the_control_plane_reaches_the_model_package_lazily():
    base = os.path.join(ROOT, "pocketllm")
    bad = []
    for path in _package_files(base):
        tree = ast.parse(open(path).read(), path)
        for node in tree.body:                                  # module level only
            names = []
            if isinstance(node, ast.ImportFrom) and not node.level and node.module:
                names = [node.module]
            elif isinstance(node, ast.Import):
                names = [a.name for a in node.names]
            bad += [(os.path.relpath(path, ROOT), n) for n in names if n.split(".")[0] in (PKG, "torch", "numpy")]
    assert not bad, bad


NATIVE = {   # directory -> directories whose headers it may include (besides its own and ptx/)
    "core": set(),
    "ptx": set(),
    "kernels": {"comm"},
    "comm": {"kernels"},
    "cpu": set(),
    "engine": {"core", "kernels", "comm"},
    "bindings": {"core", "kernels", "comm", "engine", "cpu"},
}


def test_native_include_layering():
    csrc = os.path.join(ROOT, PKG, "csrc")
    headers: dict[str, set[str]] = {}
    for d in os.listdir(csrc):
        if os.path.isdir(os.path.join(csrc, d)):
            headers[d] = {f for f in os.listdir(os.path.join(csrc, d)) if f.endswith((".h", ".hpp", ".cuh"))}
    bad = []
    for d, allowed in NATIVE.items():
        for f in sorted(os.listdir(os.path.join(csrc, d))):
            if not f.endswith((".h", ".hpp", ".cuh", ".cu", ".cpp")):
                continue
            for inc in re.findall(r'^\s*#include\s+"([^"]+)"', open(os.path.join(csrc, d, f)).read(), re.M):
                parts = inc.replace("../", "").split("/")
                owner = parts[0] if len(parts) > 1 else next((k for k, v in headers.items() if inc in v and k == d), None) \
                    or next((k for k, v in headers.items() if inc in v), None)
                if owner is None or owner in (d, "ptx") or owner in allowed:
                    continue
                bad.append(f"{d}/{f} includes {inc} (from {owner})")
    assert not bad, "\n".join(bad)
    assert {"core", "kernels", "engine", "comm"} <= set(headers)


@pytest.mark.parametrize("layer", sorted(RULES))
def test_every_ruled_layer_exists(layer):
    assert os.path.isdir(os.path.join(ROOT, PKG, layer))
