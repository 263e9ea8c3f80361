"""Every name a function reads as a global exists at module level (or is a builtin): code that only runs on a GPU, or
only in a failure path, cannot hide a misspelt or missing import from the CPU test run."""
import builtins
import os
import symtable

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KNOWN = set(dir(builtins)) | {"__file__", "__name__", "__doc__", "__spec__", "__path__", "__package__", "__class__"}


def _files():
    for top in ("deepseek_v4_2080ti_b200", "pocketllm", "baseline", "tests"):
        for dp, dn, fn in os.walk(os.path.join(ROOT, top)):
            dn[:] = [d for d in dn if d not in ("__pycache__", "_ref", "csrc", "lib", "bin")]
            for f in fn:
                if f.endswith(".py"):
                    yield os.path.join(dp, f)
    yield os.path.join(ROOT, "bench.py")
    yield os.path.join(ROOT, "__graft_entry__.py")


def _unresolved(path):
    top = symtable.symtable(open(path).read(), path, "exec")
    module = {s.get_name() for s in top.get_symbols() if s.is_assigned() or s.is_imported() or s.is_namespace()}

    def globals_assigned_below(tab):
        for s in tab.get_symbols():
            if s.is_declared_global() and s.is_assigned():
                module.add(s.get_name())
        for c in tab.get_children():
            globals_assigned_below(c)
    globals_assigned_below(top)
    out = []

    def walk(tab):
        if tab.get_type() != "module":
            for s in tab.get_symbols():
                if s.is_referenced() and s.is_global() and s.get_name() not in module and s.get_name() not in KNOWN:
                    out.append(f"{os.path.relpath(path, ROOT)}:{tab.get_lineno()} {tab.get_name()}() reads {s.get_name()}")
        for c in tab.get_children():
            walk(c)
    walk(top)
    return out


def test_no_function_reads_a_global_that_does_not_exist():
    bad = [m for f in _files() for m in _unresolved(f)]
    assert not bad, "\n".join(bad)
    assert sum(1 for _ in _files()) > 100
