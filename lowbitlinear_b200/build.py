"""Builds the native library ``lowbitlinear_b200/_C.so`` for sm_100a with nvcc.

The library is a plain C-ABI shared object (no libtorch, no Python headers): the sources under
``csrc/`` are compiled with ``-gencode arch=compute_100a,code=sm_100a`` and linked with the
static CUDA runtime, in the package directory, where ``_extension.load_cuda_extension`` looks
for it.  nvcc cross-compiles, so no GPU is needed to build.

    python -m lowbitlinear_b200.build [--force] [--verbose] [-D NAME[=VALUE] ...]
"""
import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

try:
    from ._fingerprint import BUILD_DIR, CSRC, DEFINES, INCLUDE, PACKAGE_DIR, STAMP, source_fingerprint
except ImportError:  # run as a plain script
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    from _fingerprint import BUILD_DIR, CSRC, DEFINES, INCLUDE, PACKAGE_DIR, STAMP, source_fingerprint

OUTPUT = PACKAGE_DIR / "_C.so"
SOURCES = ("api.cu", "generic.cu", "skinny.cu", "gemv_decode.cu", "gemv_grouped.cu", "peer_reduce.cu", "gemm_tc.cu", "gemm_tc2.cu", "gemm_tc_small.cu", "gemm_wt.cu", "quantize.cu",
           "tensor_map.cu")
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
COMMON_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v")


def find_nvcc():
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def build(force=False, verbose=False, defines=()):
    """Compile and link ``_C.so``; returns its path.  Skips work when nothing changed."""
    stamp = STAMP
    flags = ARCH_FLAGS + COMMON_FLAGS
    fingerprint = source_fingerprint(flags, defines)
    if not force and OUTPUT.is_file() and stamp.is_file() and stamp.read_text() == fingerprint:
        return OUTPUT
    nvcc = find_nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    define_flags = [f"-D{d}" for d in defines]

    def compile_one(name):
        obj = BUILD_DIR / (Path(name).stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *define_flags, "-I", str(INCLUDE), "-c",
               str(CSRC / name), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        return name, obj, result

    objects = []
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        for name, obj, result in pool.map(compile_one, SOURCES):
            if verbose or result.returncode != 0:
                sys.stderr.write(f"--- {name}\n{result.stdout}{result.stderr}")
            if result.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}")
            (BUILD_DIR / (Path(name).stem + ".ptxas.txt")).write_text(result.stderr)
            objects.append(str(obj))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(OUTPUT), *objects, "-lcudart_static", "-ldl",
            "-lpthread", "-lrt"]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
        raise RuntimeError("link failed")
    DEFINES.write_text("\t".join(flags) + "\n" + "".join(f"{d}\n" for d in defines))
    stamp.write_text(fingerprint)
    return OUTPUT


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("-D", dest="defines", action="append", default=[])
    args = parser.parse_args(argv)
    print(build(force=args.force, verbose=args.verbose, defines=tuple(args.defines)))


if __name__ == "__main__":
    main()
