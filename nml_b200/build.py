"""In-tree build of the sm_100a NVFP4 library with nvcc (cross-compiles without a GPU).

    python -m nml_b200.build [--force] [--verbose]

Produces ``nml_b200/lib/libnml_nvfp4_sm100.so``.  The shared object links the CUDA
runtime statically and resolves the one driver entry point it needs
(cuTensorMapEncodeTiled) at run time, so it loads on machines without a GPU driver.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB_DIR = HERE / "lib"
LIB_PATH = LIB_DIR / "libnml_nvfp4_sm100.so"
SOURCES = ["abi.cu", "embedding.cu", "linear_simt.cu", "linear_umma.cu", "stream.cu", "moe.cu",
           "experts_umma.cu", "ep.cu", "ep_push.cu", "attention_decode.cu", "topk.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the NVFP4 library cannot be built")
    return found


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    inputs = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [
        HERE.parent / "include" / "nml_nvfp4_sm100.h"]
    return any(path.stat().st_mtime > built for path in inputs)


def build(force: bool = False, verbose: bool = False, defines=(), output: Path | None = None) -> Path:
    """Compiles every source and links the shared object.  ``defines`` adds -D flags (for
    example a macro that switches a variant on when tuning) and ``output``
    redirects the result so that a tuning build never replaces the product library."""
    target = Path(output) if output is not None else LIB_PATH
    if output is None and not defines and not force and not _stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    objects = []
    procs = []
    for source in SOURCES:
        obj = LIB_DIR / (source + (".tuning.o" if defines else ".o"))
        cmd = [nvcc(), *ARCH_FLAGS, *[f"-D{d}" for d in defines], "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
               "-Xptxas", "-v" if verbose else "-warn-spills", "-c", str(CSRC / source), "-o",
               str(obj)]
        procs.append((source, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                               stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    failed = False
    for source, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed for {source}\n{out}\n")
        elif verbose and out:
            sys.stderr.write(f"--- {source}\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc(), *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", str(target), *objects]
    subprocess.run(link, check=True)
    for obj in objects:
        os.unlink(obj)
    return target


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--define", action="append", default=[])
    parser.add_argument("--output", type=Path, default=None)
    arguments = parser.parse_args()
    print(build(arguments.force, arguments.verbose, tuple(arguments.define), arguments.output))
