"""Ahead-of-time build of the CUDA extension ``vlm_training_b200/ops/_C*.so``.

Kernels are plain ``.cu`` files without framework headers (they compile in
seconds each, for ``sm_100a`` only); ``bindings*.cpp`` are the only files that
include torch headers.  Objects are cached under ``ops/_build`` keyed by a hash
of the source, its local includes and the flags, so an unchanged file is not
recompiled.  The resulting ``.so`` sits in the package directory.

    python -m vlm_training_b200.ops.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import re
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "_build")
EXT_NAME = "_C"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]
NVCC_FLAGS += os.environ.get("VLMT_NVCC_EXTRA", "").split()  # e.g. -DVLMT_ATTN_TRACE for the in-kernel timeline dump
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wno-deprecated-declarations"]


def ext_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, EXT_NAME + suffix)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _local_includes(path: str, seen=None) -> list[str]:
    seen = seen if seen is not None else set()
    out = []
    with open(path) as fh:
        for m in re.finditer(r'#include\s+"([^"]+)"', fh.read()):
            inc = os.path.join(os.path.dirname(path), m.group(1))
            if os.path.exists(inc) and inc not in seen:
                seen.add(inc)
                out.append(inc)
                out.extend(_local_includes(inc, seen))
    return out


def _digest(path: str, flags: list[str]) -> str:
    h = hashlib.sha256(" ".join(flags).encode())
    for p in [path] + sorted(_local_includes(path)):
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths("cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(True):
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    libs = ["-L", lib_dir, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
            "-L", "/usr/local/cuda/lib64", "-lcudart", f"-Wl,-rpath,{lib_dir}"]
    return inc, defs, libs


def _compile_one(src: str, verbose: bool, force: bool) -> tuple[str, str]:
    is_cu = src.endswith(".cu")
    inc, defs, _ = _torch_flags() if not is_cu else ([], [], [])
    flags = NVCC_FLAGS if is_cu else CXX_FLAGS + defs
    obj = os.path.join(BUILD, os.path.basename(src) + "." + _digest(src, flags) + ".o")
    log = ""
    if force or not os.path.exists(obj):
        if is_cu:
            cmd = [_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
        else:
            cmd = [os.environ.get("CXX", "g++")] + CXX_FLAGS + defs + inc + ["-I", "/usr/local/cuda/include", "-I", CSRC,
                                                                            "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        log = res.stdout + res.stderr
        if res.returncode != 0:
            raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{log}")
        if verbose:
            print(log)
    return obj, log


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile_one(s, verbose, force), srcs))
    objs = [o for o, _ in results]
    out = ext_path()
    stamp = hashlib.sha256(" ".join(sorted(objs)).encode()).hexdigest()
    stamp_file = os.path.join(BUILD, "link.stamp")
    if not force and os.path.exists(out) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return out
    _, _, libs = _torch_flags()
    cmd = [os.environ.get("CXX", "g++"), "-shared", "-o", out] + objs + libs
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(cmd)}\n{res.stdout}{res.stderr}")
    with open(stamp_file, "w") as fh:
        fh.write(stamp)
    keep = set(objs)
    for f in os.listdir(BUILD):  # drop objects of older source versions
        p = os.path.join(BUILD, f)
        if f.endswith(".o") and p not in keep:
            os.remove(p)
    return out


def main():
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)


if __name__ == "__main__":
    main()
