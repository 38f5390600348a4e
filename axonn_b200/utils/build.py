"""Build the in-tree CUDA library for sm_100a.

``build_library()`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` (object files in
parallel, then one link) into ``axonn_b200/lib/libaxonn_b200.so``.  nvcc
cross-compiles without a GPU.  The library is rebuilt only when a source or
header is newer than it.
"""

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libaxonn_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build axonn_b200's CUDA library")
    return nvcc


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _newest_input():
    files = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    return max(os.path.getmtime(f) for f in files)


def up_to_date():
    return os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_input()


def _compile(src, verbose):
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    hdr_time = max([os.path.getmtime(f) for f in glob.glob(os.path.join(CSRC, "*.cuh")) +
                    glob.glob(os.path.join(CSRC, "*.h"))] + [0])
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
        return obj, ""
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build_variant(out_path, extra_flags, obj_dir):
    """Build a variant of the library (extra nvcc flags, e.g. ``-DAXB_ABLATION``) to ``out_path``; select it
    at run time with ``AXONN_LIB_PATH``.  The default library is not touched."""
    os.makedirs(obj_dir, exist_ok=True)
    objs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        r = subprocess.run([_nvcc()] + NVCC_FLAGS + list(extra_flags) + ["-I", CSRC, "-c", src, "-o", obj],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        objs.append(obj)
    r = subprocess.run([_nvcc(), "-shared", "-o", out_path] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return out_path


def build_library(force=False, verbose=True):
    if not force and up_to_date():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), sources()))
    objs = [o for o, _ in results]
    log = "\n".join(l for _, l in results if l)
    with open(os.path.join(LIB_DIR, "ptxas.log"), "a") as f:
        f.write(log)
    cmd = [_nvcc(), "-shared", "-o", LIB_PATH + ".tmp"] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    if verbose:
        print(f"built {LIB_PATH} from {len(objs)} sources", file=sys.stderr)
    return LIB_PATH


DEBUG_LIB_PATH = os.path.join(LIB_DIR, "libaxonn_b200_debug.so")


def build_debug_library():
    """The bounds-checking build (``-DAXB_DEBUG_BOUNDS``): kernels verify computed offsets into peer memory
    before every store and record violations in the device status word instead of making the access.  Loaded
    instead of the normal library when ``AXONN_DEBUG_BOUNDS=1`` and the file exists."""
    os.makedirs(LIB_DIR, exist_ok=True)
    return build_variant(DEBUG_LIB_PATH, ["-DAXB_DEBUG_BOUNDS"], os.path.join(LIB_DIR, "obj_debug"))


SANITIZER_LIB_PATH = os.path.join(LIB_DIR, "libaxonn_b200_asan.so")


def build_sanitizer_library():
    """The host code of the library (allocators, symmetric heap, launch wrappers, status handling) compiled with
    AddressSanitizer and UndefinedBehaviorSanitizer; device code is unchanged.  Run the CPU tests against it with

        AXONN_LIB_PATH=<this file> LD_PRELOAD="$(gcc -print-file-name=libasan.so) $(gcc -print-file-name=libubsan.so)" \
        ASAN_OPTIONS=detect_leaks=0:abort_on_error=1 UBSAN_OPTIONS=halt_on_error=1 \
        python -m pytest tests/test_arena_cpu.py tests/test_symm_heap_cpu.py tests/test_ops_cpu.py

    (leak detection is off because the Python interpreter itself never frees everything)."""
    os.makedirs(LIB_DIR, exist_ok=True)
    flags = ["-Xcompiler", "-fsanitize=address", "-Xcompiler", "-fsanitize=undefined", "-Xcompiler",
             "-fno-omit-frame-pointer"]
    return build_variant(SANITIZER_LIB_PATH, flags, os.path.join(LIB_DIR, "obj_asan"))


if __name__ == "__main__":
    if "--debug-bounds" in sys.argv:
        print(build_debug_library())
    elif "--sanitize" in sys.argv:
        print(build_sanitizer_library())
    else:
        build_library(force="--force" in sys.argv)
