"""Installs the UNMODIFIED reference package into ``oracle/_ref`` (git-ignored test infrastructure).

    python oracle/make_ref.py [--reference <checkout of NanjinLin/LowBitLinear>] [--cpu-only]

``oracle/_ref`` plays two roles, both as checker / baseline only (nothing in ``lowbitlinear_b200``
ever imports it): ``bench.py --impl reference`` and the ``cpu_baseline`` leg time the reference's
own ``linear_int4_reference`` (lowbitlinear/linear.py:43-70) from it on the host cores, and the
tests compare the numpy oracle with it when it is present.  The install is a plain
``pip install --no-index --no-build-isolation --no-deps --target oracle/_ref`` of a scratch copy of
the checkout (pip wants to write into the source tree, the checkout is read-only); no reference
source enters the repository's history.

The reference's ``setup.py`` also compiles its two CUDA kernels whenever a CUDA toolkit is present
(csrc/w4a16_gemv_warp_vec.cu, csrc/cute_w4a16_gemm.cu; CuTe headers from ``CUTLASS_INCLUDE``).
They are built for sm_100a here -- nvcc cross-compiles -- so that the benchmark can also time the
reference's own kernels on the same GPU.  ``--cpu-only`` skips that (the Python files alone).
The reference's ``tests/`` are copied beside the package (``oracle/_ref/reference_tests``) so that
its own suite can be pointed at this library.
"""
import argparse
import importlib.util
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def find_cutlass():
    for package in ("flashinfer", "tilelang", "deep_gemm"):
        spec = importlib.util.find_spec(package)
        if spec is None or not spec.submodule_search_locations:
            continue
        for root in spec.submodule_search_locations:
            for sub in ("data/cutlass/include", "3rdparty/cutlass/include", "include"):
                candidate = Path(root) / sub
                if (candidate / "cute" / "tensor.hpp").is_file():
                    return candidate
    return None


def install(reference, cpu_only=False, verbose=False):
    reference = Path(reference)
    if not (reference / "lowbitlinear" / "linear.py").is_file():
        raise SystemExit(f"{reference} is not a LowBitLinear checkout")
    if TARGET.exists():
        shutil.rmtree(TARGET)
    with tempfile.TemporaryDirectory(prefix="lbl_ref_") as scratch:
        source = Path(scratch) / "src"
        shutil.copytree(reference, source, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", ".git", "assets"))
        env = dict(os.environ)
        cutlass = None if cpu_only else find_cutlass()
        if cutlass is None:
            # Without CuTe headers (or on request) only the Python package is installed: the
            # reference's setup.py takes its CPU-only branch when torch reports no CUDA toolkit.
            (source / "setup.py").write_text("from setuptools import setup\nsetup()\n")
        else:
            env["CUTLASS_INCLUDE"] = str(cutlass)
            env["TORCH_CUDA_ARCH_LIST"] = "10.0a"
            env.setdefault("MAX_JOBS", "4")
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--target", str(TARGET), str(source)]
        result = subprocess.run(cmd, env=env, capture_output=not verbose, text=True)
        if result.returncode != 0:
            if not verbose:
                sys.stderr.write(result.stdout[-4000:] + result.stderr[-4000:])
            raise SystemExit("pip install of the reference failed")
        shutil.copytree(reference / "tests", TARGET / "reference_tests",
                        ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    built = sorted(p.name for p in (TARGET / "lowbitlinear").glob("_C*"))
    (TARGET / "INSTALL.txt").write_text(
        f"reference installed from {reference}\nCUDA kernels: {', '.join(built) if built else 'not built'}\n")
    return TARGET, built


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--reference", default=os.environ.get("LBL_REFERENCE", HERE.parents[1] / "reference"),
                        help="checkout of the reference (default: $LBL_REFERENCE, else ../reference beside this repository)")
    parser.add_argument("--cpu-only", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args(argv)
    target, built = install(args.reference, args.cpu_only, args.verbose)
    print(f"{target}: lowbitlinear installed; CUDA kernels: {built or 'not built'}")


if __name__ == "__main__":
    main()
