"""In-tree build of the native library and the torch extension.

`build_native()` compiles every `.cc` / `.cu` under `csrc/` (except `csrc/torch/`) into
`hccl_b200/lib/libhccl_b200.so` with `nvcc -gencode arch=compute_100a,code=sm_100a`; `build_torch_ext()` compiles the
ProcessGroup binding against the installed torch headers into `hccl_b200/lib/hccl_b200_torch.so`. Both go through a
generated ninja file so rebuilds are incremental and parallel. Nothing is JIT-cached outside the tree: the `.so`
files sit next to the package and are what the Python side loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "hccl_b200" / "lib"
BUILD = ROOT / "build"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _sources(exclude_dirs=("torch",)):
    cc, cu = [], []
    for p in sorted(CSRC.rglob("*")):
        if any(part in exclude_dirs for part in p.relative_to(CSRC).parts[:-1]):
            continue
        if p.suffix == ".cc":
            cc.append(p)
        elif p.suffix == ".cu":
            cu.append(p)
    return cc, cu


def _ninja(build_file: Path, jobs: int | None = None, verbose: bool = False) -> None:
    cmd = [shutil.which("ninja") or "ninja", "-f", str(build_file)]
    if jobs:
        cmd += ["-j", str(jobs)]
    if verbose:
        cmd.append("-v")
    res = subprocess.run(cmd, cwd=str(ROOT), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout[-20000:])
        raise RuntimeError("native build failed")
    if verbose:
        print(res.stdout)


def build_native(verbose: bool = False, ptxas_info: bool = False, flavor: str = "") -> Path:
    """flavor "" = release; "debug" = device-side bounds checks on every heap access (-DHCCL_DEBUG_BOUNDS) and host asserts;
    "asan" / "tsan" / "ubsan" = host code under Address-, Thread- or UndefinedBehaviorSanitizer; "cov" = host code
    instrumented for gcov (run tests with HCCL_B200_LIB pointing at it, then `gcov -o build_cov/obj <source>`). Flavors build into their own directory and library
    (libhccl_b200_<flavor>.so); load one by pointing HCCL_B200_LIB at it."""
    global BUILD
    release_build = BUILD
    if flavor:
        BUILD = ROOT / f"build_{flavor}"
    try:
        return _build_native(verbose, ptxas_info, flavor)
    finally:
        BUILD = release_build


def _build_native(verbose: bool, ptxas_info: bool, flavor: str) -> Path:
    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    cc, cu = _sources()
    inc = [f"-I{ROOT / 'include'}", f"-I{CSRC}", f"-I{CUDA_HOME / 'include'}"]
    cxxflags = ["-O2", "-g1", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"] + inc
    nvflags = (["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
                "--threads", "2"] + ARCH_FLAGS + inc)
    if flavor == "debug":
        cxxflags = [f for f in cxxflags if f != "-O2"] + ["-O1", "-g", "-DHCCL_DEBUG_BOUNDS", "-D_GLIBCXX_ASSERTIONS"]
        nvflags += ["-DHCCL_DEBUG_BOUNDS"]
    elif flavor == "asan":
        cxxflags += ["-fsanitize=address", "-fno-omit-frame-pointer"]
    elif flavor == "cov":
        cxxflags = [f for f in cxxflags if f != "-O2"] + ["-O0", "--coverage"]
    elif flavor == "tsan":
        cxxflags += ["-fsanitize=thread", "-fno-omit-frame-pointer"]
    elif flavor == "ubsan":
        cxxflags += ["-fsanitize=undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"]
    if ptxas_info:
        nvflags += ["-Xptxas", "-v"]
    out = LIBDIR / (f"libhccl_b200_{flavor}.so" if flavor else "libhccl_b200.so")
    lines = [
        "ninja_required_version = 1.3",
        f"builddir = {BUILD}",
        f"cxx = {shutil.which('g++') or 'g++'}",
        f"nvcc = {CUDA_HOME / 'bin' / 'nvcc'}",
        f"cxxflags = {' '.join(cxxflags)}",
        f"nvflags = {' '.join(nvflags)}",
        "rule cxx",
        "  command = $cxx -MMD -MF $out.d $cxxflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule nvcc",
        "  command = $nvcc -MD -MF $out.d $nvflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        "  command = $nvcc -shared -o $out $in -cudart static -lpthread -ldl -lrt -Xlinker -soname=" + out.name + ({"cov": " -Xcompiler --coverage", "asan": " -Xcompiler -fsanitize=address", "tsan": " -Xcompiler -fsanitize=thread", "ubsan": " -Xcompiler -fsanitize=undefined"}.get(flavor, "")),
    ]
    objs = []
    for src in cc + cu:
        obj = BUILD / "obj" / (str(src.relative_to(CSRC)).replace("/", "_") + ".o")
        objs.append(obj)
        lines.append(f"build {obj}: {'cxx' if src.suffix == '.cc' else 'nvcc'} {src}")
    lines.append(f"build {out}: link {' '.join(str(o) for o in objs)}")
    lines.append(f"default {out}")
    bf = BUILD / "native.ninja"
    bf.write_text("\n".join(lines) + "\n")
    _ninja(bf, verbose=verbose)
    return out


def build_torch_ext(verbose: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    srcs = sorted((CSRC / "torch").glob("*.cc"))
    if not srcs:
        raise RuntimeError("no sources under csrc/torch")
    inc = [f"-I{ROOT / 'include'}", f"-I{CSRC}", f"-I{CUDA_HOME / 'include'}"] + [f"-I{p}" for p in ce.include_paths()]
    import sysconfig

    inc.append(f"-I{sysconfig.get_paths()['include']}")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxxflags = ["-O2", "-std=c++17", "-fPIC", "-Wno-unused-function", "-pthread", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                "-DTORCH_EXTENSION_NAME=hccl_b200_torch", "-DTORCH_API_INCLUDE_EXTENSION_H", "-DUSE_C10D_NCCL=0"] + inc
    torch_lib = Path(torch.__file__).parent / "lib"
    out = LIBDIR / "hccl_b200_torch.so"
    ldflags = [f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
               f"-L{LIBDIR}", "-Wl,-rpath,'$$ORIGIN'", "-lhccl_b200"]
    if (torch_lib / "libc10_cuda.so").exists():
        ldflags += ["-lc10_cuda", "-ltorch_cuda"]
    lines = [
        "ninja_required_version = 1.3",
        f"builddir = {BUILD}",
        f"cxx = {shutil.which('g++') or 'g++'}",
        f"cxxflags = {' '.join(cxxflags)}",
        f"ldflags = {' '.join(ldflags)}",
        "rule cxx",
        "  command = $cxx -MMD -MF $out.d $cxxflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        "  command = $cxx -shared -o $out $in $ldflags",
    ]
    objs = []
    for src in srcs:
        obj = BUILD / "obj_torch" / (src.name + ".o")
        objs.append(obj)
        lines.append(f"build {obj}: cxx {src}")
    lines.append(f"build {out}: link {' '.join(str(o) for o in objs)} | {LIBDIR / 'libhccl_b200.so'}")
    lines.append(f"default {out}")
    bf = BUILD / "torch_ext.ninja"
    bf.write_text("\n".join(lines) + "\n")
    _ninja(bf, verbose=verbose)
    return out


def build_all(verbose: bool = False) -> None:
    build_native(verbose=verbose)
    if (CSRC / "torch").is_dir() and any((CSRC / "torch").glob("*.cc")):
        build_torch_ext(verbose=verbose)


def package(dest: Path | None = None) -> Path:
    """dist/hccl_b200-<version>-sm100a.tar.gz: public headers, the built libraries, the Python package, the samples and the docs."""
    import tarfile

    sys.path.insert(0, str(ROOT))
    from hccl_b200 import __version__

    dest = dest or ROOT / "dist"
    dest.mkdir(exist_ok=True)
    name = f"hccl_b200-{__version__}-sm100a"
    out = dest / f"{name}.tar.gz"
    with tarfile.open(out, "w:gz") as tf:
        for rel in ("include", "hccl_b200", "examples", "docs", "README.md"):
            p = ROOT / rel
            if p.exists():
                tf.add(p, arcname=f"{name}/{rel}", filter=lambda ti: None if ("__pycache__" in ti.name or ti.name.endswith("/bin")) else ti)
    return out


if __name__ == "__main__":
    args = sys.argv[1:]
    flavor = next((a.split("=", 1)[1] for a in args if a.startswith("--flavor=")), "")
    if flavor:
        print("built:", build_native(verbose="-v" in args, flavor=flavor))
    else:
        build_all(verbose="-v" in args)
        print("built:", ", ".join(str(p) for p in sorted(LIBDIR.glob("*.so"))))
    if "--pkg" in args:
        print("package:", package())
