"""In-tree build of the sm_100a extension.

Layout: every ``csrc/*.cu`` holds kernels plus plain C launchers (raw pointers + ``cudaStream_t``);
``csrc/bindings.cpp`` is the only file that sees PyTorch headers and unwraps tensors.  Objects are
cached by content hash (sources + local headers + flags) under ``csrc/build`` and linked into
``_loom_b200.so`` beside this file.  The reference's build driver JIT-compiles through
``torch.utils.cpp_extension.load`` for whatever GPU is visible (``kernels/build.py:262-344``);
here the target is fixed (sm_100a) and nvcc cross-compiles without a GPU.

Run ``python -m loomformer_paraplex_b200.ops.build [-v] [--force]``.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import hashlib
import json
import os
import shutil
import subprocess
import sys
import sysconfig
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(CSRC, "build")
SO = os.path.join(HERE, "_loom_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _hash(paths: List[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as fh:
            h.update(p.encode()); h.update(fh.read())
    return h.hexdigest()[:16]


def _run(cmd: List[str], verbose: bool, log_path: str = None) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log_path:
        with open(log_path, "w") as fh:
            fh.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build failed: " + " ".join(cmd))
    if verbose:
        sys.stderr.write(r.stderr)


def build(verbose: bool = False, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    cus = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    cpps = sorted(glob.glob(os.path.join(CSRC, "*.cpp")))
    if not cus or not cpps:
        raise RuntimeError("no sources under ops/csrc")
    cuda_home = os.path.dirname(os.path.dirname(NVCC))
    inc = ["-I" + CSRC, "-I" + os.path.join(cuda_home, "include")]
    torch_inc = ["-I" + p for p in ce.include_paths()] + ["-I" + sysconfig.get_paths()["include"]]
    jobs, objs = [], []
    for src in cus:
        tag = _hash([src] + headers, " ".join(ARCH + NVCC_FLAGS))
        obj = os.path.join(OUT, f"{os.path.basename(src)}.{tag}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append((NVCC_CMD(src, obj, inc), obj + ".log"))
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_loom_b200",
                 "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for src in cpps:
        tag = _hash([src] + headers, " ".join(cxx_flags) + torch.__version__)
        obj = os.path.join(OUT, f"{os.path.basename(src)}.{tag}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append((["g++", "-c", src, "-o", obj] + cxx_flags + inc + torch_inc, obj + ".log"))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for f in [ex.submit(_run, cmd, verbose, log) for cmd, log in jobs]:
                f.result()
    stamp = os.path.join(OUT, "linked.json")
    want = {"objs": [os.path.basename(o) for o in objs]}
    have = json.load(open(stamp)) if os.path.exists(stamp) else None
    if force or jobs or have != want or not os.path.exists(SO):
        libdirs = ce.library_paths(device_type="cuda")
        link = ["g++", "-shared", "-o", SO] + objs + ["-L" + p for p in libdirs] + \
               ["-Wl,-rpath," + p for p in libdirs] + \
               ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        _run(link, verbose)
        json.dump(want, open(stamp, "w"))
    # drop stale objects
    keep = set(objs) | {o + ".log" for o in objs} | {stamp}
    for p in glob.glob(os.path.join(OUT, "*")):
        if p not in keep:
            os.remove(p)
    return SO


def NVCC_CMD(src: str, obj: str, inc: List[str]) -> List[str]:
    return [NVCC, "-c", src, "-o", obj] + ARCH + NVCC_FLAGS + inc


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output (registers / spills / shared memory) of the last build."""
    out = []
    for log in sorted(glob.glob(os.path.join(OUT, "*.cu.*.o.log"))):
        with open(log) as fh:
            out.append(fh.read())
    return "\n".join(out)


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(path)
