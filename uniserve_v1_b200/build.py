"""Ahead-of-time build of the native libraries, in tree.

Two shared objects are produced under ``uniserve_v1_b200/_lib``:

* ``libus_kernels.so``  every ``csrc/*.cu`` compiled for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``), plain C entry points;
* ``libus_host.so``     every ``csrc/host/*.cpp`` (block manager, batch column
  assembly, media writers): host C++ with plain C entry points.

There is no run-time kernel compilation and no Build Server process: the
reference compiles kernel packages at first start
(crates/build-server, reference project path); here the libraries are built once
and loaded with ctypes.

Usage: ``python -m uniserve_v1_b200.build [--force] [--verbose]``
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _digest(path: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(path.read_bytes())
    for inc in sorted((CSRC / "include").glob("*")):
        h.update(inc.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, flags: list[str], compiler: str, stamp: dict, force: bool,
                 verbose: bool) -> tuple[Path, bool, str]:
    obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
    dig = _digest(src, flags)
    if not force and obj.exists() and stamp.get(str(obj.name)) == dig:
        return obj, False, ""
    cmd = [compiler, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    if proc.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{log}")
    stamp[str(obj.name)] = dig
    if verbose:
        print(log)
    return obj, True, log


def build(force: bool = False, verbose: bool = False) -> dict:
    """Compile what changed and link both libraries; returns the paths."""
    OBJ.mkdir(parents=True, exist_ok=True)
    stamp_path = OBJ / "stamp.json"
    stamp = json.loads(stamp_path.read_text()) if stamp_path.exists() else {}
    nvcc = _nvcc()
    cu = sorted(CSRC.glob("*.cu")) + sorted((CSRC / "fused").glob("*.cu"))
    cpp = sorted((CSRC / "host").glob("*.cpp"))
    logs = {}
    with ThreadPoolExecutor(max_workers=max(1, (os.cpu_count() or 4))) as pool:
        cu_jobs = [pool.submit(_compile_one, s, NVCC_FLAGS, nvcc, stamp, force, verbose) for s in cu]
        cpp_jobs = [pool.submit(_compile_one, s, CXX_FLAGS, "g++", stamp, force, verbose)
                    for s in cpp]
        cu_res = [j.result() for j in cu_jobs]
        cpp_res = [j.result() for j in cpp_jobs]
    for (obj, _, log), src in zip(cu_res, cu):
        logs[src.name] = log
    stamp_path.write_text(json.dumps(stamp, indent=0))
    out = {}
    kern = LIB / "libus_kernels.so"
    if cu_res and (force or not kern.exists() or any(c for _, c, _ in cu_res)):
        tmp = kern.with_suffix(".so.tmp")       # linked aside, then moved into place at once
        cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o, _, _ in cu_res],
               "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed: {proc.stdout}{proc.stderr}")
        os.replace(tmp, kern)
    out["kernels"] = kern
    host = LIB / "libus_host.so"
    if cpp_res and (force or not host.exists() or any(c for _, c, _ in cpp_res)):
        tmp = host.with_suffix(".so.tmp")
        cmd = ["g++", "-shared", "-o", str(tmp), *[str(o) for o, _, _ in cpp_res], "-pthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed: {proc.stdout}{proc.stderr}")
        os.replace(tmp, host)
    out["host"] = host
    out["logs"] = logs
    return out


def main(argv: list[str]) -> int:
    res = build(force="--force" in argv, verbose="--verbose" in argv)
    print("built:", res["kernels"], res["host"])
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
