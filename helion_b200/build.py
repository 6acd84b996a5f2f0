"""Builds the C-ABI shared library (``helion_b200/_C/libhelion_b200.so``) with nvcc for sm_100a.

    python -m helion_b200.build [--force] [--verbose]
    python -m helion_b200.build --define HB_SKINNY_TRACE --output helion_b200/_C/libhelion_b200_trace.so

The library is built in-tree so that it travels with the source tree; it is rebuilt only when a
source file is newer than the existing binary.  nvcc cross-compiles without a GPU.  ``--define`` /
``--output`` build a second, instrumented copy beside it (development aids such as the phase stamps of
``python -m helion_b200.chain_trace``); the product library is never built with a define.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT_DIR = PKG_DIR / "_C"
LIB_PATH = OUT_DIR / "libhelion_b200.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

SOURCES = ["api.cu", "fp8_gemm.cu", "fp8_gemm_skinny.cu", "fp8_attention.cu", "fp8_attention_pair.cu", "softmax_ceiling.cu", "attention_16bit.cu", "quantize.cu"]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


def find_nvcc() -> str:
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return nvcc


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE_DIR.glob("*.h"))
    deps.append(Path(__file__))
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False, defines: tuple = (), output: Path | None = None) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library; returns its path.

    With ``defines`` the objects go to a directory of their own and the library to ``output``."""
    variant = bool(defines) or output is not None
    if variant and output is None:
        raise ValueError("an instrumented build needs its own output path")
    lib_path = Path(output).resolve() if variant else LIB_PATH
    if lib_path == LIB_PATH and variant:
        raise ValueError("the product library is not built with extra defines")
    if not variant and not force and not _stale():
        return LIB_PATH
    nvcc = find_nvcc()
    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = OUT_DIR / ("variant_" + "_".join(defines)) if variant else OUT_DIR
    obj_dir.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-I", str(INCLUDE_DIR), "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stdout.write(out)
        if p.returncode != 0:
            failed.append(src)
    if failed:
        raise RuntimeError(f"nvcc failed for: {', '.join(failed)}")
    tmp = lib_path.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", *objs, "-o", str(tmp)]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stdout.write(r.stdout)
        raise RuntimeError("link failed")
    os.replace(tmp, lib_path)
    return lib_path


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print nvcc commands and ptxas resource usage")
    ap.add_argument("--define", action="append", default=[], metavar="NAME", help="instrumented build: -DNAME (needs --output)")
    ap.add_argument("--output", default=None, help="instrumented build: path of the library to write")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose, defines=tuple(args.define),
                output=Path(args.output) if args.output else None))


if __name__ == "__main__":
    main()
