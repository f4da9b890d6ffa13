"""Builds libllmopt_cuda.so in-tree with nvcc for sm_100a (no JIT cache, no torch)."""

from __future__ import annotations

import os
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PACKAGE_DIR, "csrc")
LIBRARY = os.path.join(PACKAGE_DIR, "libllmopt_cuda.so")
OBJECTS = os.path.join(PACKAGE_DIR, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, name) for name in os.listdir(CSRC) if name.endswith(".cu"))


def _newer(path: str, than: str) -> bool:
    return (not os.path.exists(than)) or os.path.getmtime(path) > os.path.getmtime(than)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile changed translation units and link the shared library."""
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJECTS, exist_ok=True)
    headers = [os.path.join(CSRC, name) for name in os.listdir(CSRC) if name.endswith((".cuh", ".h"))]
    headers.append(os.path.join(PACKAGE_DIR, "..", "include", "llmopt_cuda.h"))
    objects, jobs = [], []
    for source in sources():
        obj = os.path.join(OBJECTS, os.path.basename(source)[:-3] + ".o")
        objects.append(obj)
        stale = force or _newer(source, obj) or any(_newer(h, obj) for h in headers if os.path.exists(h))
        if stale:
            command = [nvcc, *NVCC_FLAGS, "-c", source, "-o", obj]
            if verbose:
                command.insert(1, "-Xptxas=-v")
            jobs.append((source, subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for source, job in jobs:
        output = job.communicate()[0].decode()
        if job.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed for {source}:\n{output}\n")
        elif verbose:
            sys.stderr.write(output)
    if failed:
        raise RuntimeError("libllmopt_cuda.so: compilation failed")
    if jobs or not os.path.exists(LIBRARY):
        subprocess.check_call(
            [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIBRARY, *objects, "-lcudart"]
        )
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
