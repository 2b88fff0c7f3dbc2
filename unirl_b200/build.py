"""Build the native extension in-tree: ``python -m unirl_b200.build`` → ``unirl_b200/_C.so``.

Each ``.cu`` translation unit is compiled by nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``; cross-compiles without a GPU), ``bindings.cpp`` /
``runtime.cpp`` by the host compiler against the installed PyTorch, and everything is linked into one
shared object next to the package so that it travels with the source tree.  Objects are rebuilt only
when their source (or a header) is newer.
"""

from __future__ import annotations

import os
import shlex
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
TARGET = os.path.join(HERE, "_C.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _run(cmd: List[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(shlex.quote(c) for c in cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout.strip() or r.stderr.strip()):
        print(r.stdout, r.stderr, flush=True)


def _stale(out: str, deps: List[str]) -> bool:
    return not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps)


def _defines_for(src: str, headers: List[str]) -> List[str]:
    """Development switches: ``UNIRL_B200_NVCC_DEFINES=NAME[,NAME=VALUE...]`` adds ``-DNAME`` to the translation units that mention the
    name (directly or through a header of this package), e.g. ``UNIRL_B200_ATTN_DIAG`` (phase timers in the attention kernels) or
    ``UNIRL_B200_SKINNY_DIAG``.  The product build sets none."""
    want = [d for d in os.environ.get("UNIRL_B200_NVCC_DEFINES", "").split(",") if d]
    if not want:
        return []
    text = open(src).read()
    for h in headers:
        if f'"{os.path.basename(h)}"' in text:
            text += open(h).read()
    return [d for d in want if d.split("=")[0] in text]


def _defines_changed(out: str, defs: List[str]) -> bool:
    stamp = out + ".defs"
    old = open(stamp).read() if os.path.exists(stamp) else ""
    return old != ",".join(defs)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    inc = [f"-I{p}" for p in include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    jobs = []
    for f in cu:
        out = os.path.join(OBJ, f + ".o")
        defs = _defines_for(os.path.join(CSRC, f), headers)
        if force or _stale(out, [os.path.join(CSRC, f)] + headers) or _defines_changed(out, defs):
            cmd = [NVCC, "-c", os.path.join(CSRC, f), "-o", out, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", *ARCH,
                   "-Xcompiler", "-fPIC", f"-I{CSRC}", "--expt-relaxed-constexpr", *[f"-D{d}" for d in defs]]
            with open(out + ".defs", "w") as fh:
                fh.write(",".join(defs))
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    for f in cpp:
        out = os.path.join(OBJ, f + ".o")
        if force or _stale(out, [os.path.join(CSRC, f)] + headers):
            jobs.append(["g++", "-c", os.path.join(CSRC, f), "-o", out, "-O2", "-std=c++17", "-fPIC", *inc, f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                         "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", "-Wno-deprecated-declarations"])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    objs = [os.path.join(OBJ, f + ".o") for f in cu + cpp]
    if force or jobs or _stale(TARGET, objs):
        libs = [f"-L{p}" for p in library_paths("cuda")]
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        _run(["g++", "-shared", "-o", TARGET, *objs, *libs, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
              "-lcudart", f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,/usr/local/cuda/lib64"], verbose)
    return TARGET


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv))
