"""In-tree native build for the B200 kernel library and the C++ runtime.

Everything is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``)
and the products stay inside the package directory so that a snapshot of the
repository carries them:

* ``lib/libb200_kernels.so``  - every ``csrc/kernels/*.cu`` and ``csrc/comm/*.cu``;
  plain C entry points, loaded with ctypes (no torch headers, so a kernel edit
  rebuilds in seconds).
* ``lib/libb200_core.so`` + ``pocketllm_cpp`` pybind module - the C++ runtime
  (block pool/table, scheduler, command channel, readers, tokenizer, sampler).
* ``lib/libb200_cpu.so`` - AVX2 multi-threaded host kernels (FP4 and INT8 routed experts on the CPU).
* ``bin/pocketllm_engine`` - the native executable.

The reference builds its native plane with CMake for sm_75
(cpp_engine/CMakeLists.txt:95-100) and its torch extensions with setup.py
(setup.py:49-87); this module replaces both.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shlex
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "lib"
BIN = PKG / "bin"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC",
                     "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]
# A compiler that links its C++ runtime statically would otherwise export that runtime's symbols from every module;
# in a process that has already loaded another libstdc++ (torch) the dynamic linker then binds half of a stream or
# locale object to one runtime and half to the other.
PRIVATE_RUNTIME = ["-Wl,--exclude-libs,ALL"]


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write("FAILED: " + " ".join(shlex.quote(c) for c in cmd) + "\n")
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"native build failed: {cmd[0]} {cmd[-1]}")


def _deps_mtime(src: Path) -> float:
    """Newest mtime among the source and every header under csrc/ (coarse but safe)."""
    newest = src.stat().st_mtime
    for pat in ("**/*.h", "**/*.hpp", "**/*.cuh", "**/*.inc"):
        for h in CSRC.glob(pat):
            newest = max(newest, h.stat().st_mtime)
    return newest


def _needs(src: Path, obj: Path) -> bool:
    return (not obj.exists()) or obj.stat().st_mtime < _deps_mtime(src)


def _compile_cu(src: Path) -> Path:
    obj = OBJ / (src.stem + ".cu.o")
    if _needs(src, obj):
        _run([NVCC, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    return obj


def _compile_cpp(src: Path, extra: list[str] | None = None, tag: str = "") -> Path:
    obj = OBJ / (src.stem + tag + ".cpp.o")
    if _needs(src, obj):
        _run([CXX, *CXX_FLAGS, *(extra or []), "-I", str(CSRC), "-I", "/usr/local/cuda/include",
              "-c", str(src), "-o", str(obj)])
    return obj


def build_kernels(jobs: int | None = None) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    srcs = sorted(list((CSRC / "kernels").glob("*.cu")) + list((CSRC / "comm").glob("*.cu")))
    out = LIB / "libb200_kernels.so"
    with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        objs = list(ex.map(_compile_cu, srcs))
    if (not out.exists()) or any(o.stat().st_mtime > out.stat().st_mtime for o in objs):
        _run([NVCC, *ARCH, "-shared", "-o", str(out), *map(str, objs), "-lcudart_static", "-lpthread",
              "-ldl", "-lrt"])
    return out


def build_core(jobs: int | None = None) -> dict[str, Path]:
    """C++ runtime library, pybind module and the engine executable."""
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    BIN.mkdir(exist_ok=True)
    products: dict[str, Path] = {}
    core_srcs = sorted((CSRC / "core").glob("*.cpp"))
    if not core_srcs:
        return products
    with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        core_objs = list(ex.map(_compile_cpp, core_srcs))
    core_lib = LIB / "libb200_core.so"
    if (not core_lib.exists()) or any(o.stat().st_mtime > core_lib.stat().st_mtime for o in core_objs):
        _run([CXX, "-shared", *PRIVATE_RUNTIME, "-o", str(core_lib), *map(str, core_objs), "-pthread"])
    products["core"] = core_lib

    bind_src = CSRC / "bindings" / "core_bindings.cpp"
    if bind_src.exists():
        import pybind11

        ext = sysconfig.get_config_var("EXT_SUFFIX")
        mod = PKG / f"pocketllm_cpp{ext}"
        inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
        bobj = _compile_cpp(bind_src, inc)
        if (not mod.exists()) or bobj.stat().st_mtime > mod.stat().st_mtime or \
                core_lib.stat().st_mtime > mod.stat().st_mtime:
            _run([CXX, "-shared", *PRIVATE_RUNTIME, "-o", str(mod), str(bobj), *map(str, core_objs), "-pthread"])
        products["pybind"] = mod

    main_src = CSRC / "engine" / "main.cpp"
    if main_src.exists():
        eng_srcs = sorted((CSRC / "engine").glob("*.cpp")) + sorted((CSRC / "comm").glob("*.cpp"))
        eng_objs = [_compile_cpp(s, tag=".eng") for s in eng_srcs]
        exe = BIN / "pocketllm_engine"
        kern = LIB / "libb200_kernels.so"
        if (not exe.exists()) or any(o.stat().st_mtime > exe.stat().st_mtime for o in eng_objs + core_objs) \
                or (kern.exists() and kern.stat().st_mtime > exe.stat().st_mtime):
            _run([CXX, "-o", str(exe), *map(str, eng_objs), *map(str, core_objs), "-L", str(LIB),
                  "-lb200_kernels", f"-Wl,-rpath,$ORIGIN/../lib", "-L/usr/local/cuda/lib64",
                  "-lcudart", "-lnccl", "-ldl", "-pthread"])
        products["engine"] = exe
        ebind = CSRC / "bindings" / "engine_bindings.cpp"
        if ebind.exists():
            import pybind11

            ext = sysconfig.get_config_var("EXT_SUFFIX")
            emod = PKG / f"pocketllm_engine_cpp{ext}"
            inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
            eobj = _compile_cpp(ebind, inc)
            lib_objs = [o for o in eng_objs if not o.name.startswith("main.")]
            if (not emod.exists()) or any(o.stat().st_mtime > emod.stat().st_mtime for o in [eobj, *lib_objs, *core_objs]) \
                    or (kern.exists() and kern.stat().st_mtime > emod.stat().st_mtime):
                _run([CXX, "-shared", *PRIVATE_RUNTIME, "-o", str(emod), str(eobj), *map(str, lib_objs), *map(str, core_objs), "-L", str(LIB),
                      "-lb200_kernels", "-Wl,-rpath,$ORIGIN/lib", "-L/usr/local/cuda/lib64", "-lcudart", "-lnccl", "-ldl",
                      "-pthread"])
            products["engine_pybind"] = emod
    return products


def build_selftest(sanitizer: str = "") -> Path:
    """Host-only self-test of the C++ core (csrc/selftest), optionally under a sanitizer:
    ``"address"`` (AddressSanitizer + UBSan) or ``"thread"`` (ThreadSanitizer).  Core sources are recompiled with the
    same flags into one executable ``bin/core_selftest[_asan|_tsan]``."""
    BIN.mkdir(exist_ok=True)
    flags = {"": [], "address": ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g"],
             "thread": ["-fsanitize=thread", "-g"]}[sanitizer]
    suffix = {"": "", "address": "_asan", "thread": "_tsan"}[sanitizer]
    exe = BIN / f"core_selftest{suffix}"
    srcs = sorted((CSRC / "core").glob("*.cpp")) + [CSRC / "selftest" / "core_selftest.cpp"]
    cxx = CXX
    if sanitizer and os.path.exists("/usr/bin/g++"):
        cxx = "/usr/bin/g++"          # the distribution compiler ships the sanitizer runtimes
    if (not exe.exists()) or any(s.stat().st_mtime > exe.stat().st_mtime for s in srcs):
        _run([cxx, "-std=c++17", "-O1", *flags, "-I", str(CSRC), *map(str, srcs), "-o", str(exe), "-pthread"])
    return exe


def build_cpu_selftest(sanitizer: str = "") -> Path:
    """Memory-safety self-test of the AVX2 host kernels (csrc/selftest/cpu_selftest.cpp with csrc/cpu), plain or under
    AddressSanitizer + UBSan: ``bin/cpu_selftest[_asan]``."""
    BIN.mkdir(exist_ok=True)
    flags = {"": [], "address": ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-g"]}[sanitizer]
    exe = BIN / ("cpu_selftest" + ("_asan" if sanitizer else ""))
    srcs = sorted((CSRC / "cpu").glob("*.cpp")) + [CSRC / "selftest" / "cpu_selftest.cpp"]
    cxx = "/usr/bin/g++" if sanitizer and os.path.exists("/usr/bin/g++") else CXX
    if (not exe.exists()) or any(s.stat().st_mtime > exe.stat().st_mtime for s in srcs):
        _run([cxx, "-std=c++17", "-O2", "-mavx2", "-mfma", *flags, "-I", str(CSRC), *map(str, srcs), "-o", str(exe), "-pthread"])
    return exe


def build_cpu() -> Path | None:
    """AVX2 multi-threaded host kernels (csrc/cpu): the CPU path for FP4 and INT8 routed experts."""
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    srcs = sorted((CSRC / "cpu").glob("*.cpp"))
    if not srcs:
        return None
    flags = ["-O3", "-mavx2", "-mfma"]
    objs = [_compile_cpp(s, flags, tag=".cpu") for s in srcs]
    out = LIB / "libb200_cpu.so"
    if (not out.exists()) or any(o.stat().st_mtime > out.stat().st_mtime for o in objs):
        _run([CXX, "-shared", *PRIVATE_RUNTIME, "-o", str(out), *map(str, objs), "-pthread"])
    return out


def build_all() -> dict[str, Path]:
    out = {"kernels": build_kernels()}
    out.update(build_core())
    cpu = build_cpu()
    if cpu is not None:
        out["cpu"] = cpu
    return out


if __name__ == "__main__":
    for k, v in build_all().items():
        print(f"built {k}: {v}")
