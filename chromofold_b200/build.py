"""Compile the CUDA sources of this package into chromofold_b200/libchromofold_b200.so (sm_100a only), and the
llama-server multi-sequence bridge (host code, linked against it) into chromofold_b200/libchromofold_b200_llama_ms.so.

Each source is compiled to an object of its own (in parallel, and only when it or a header is newer than its object);
the objects live under chromofold_b200/build/ and are linked into the one shared library."""
import concurrent.futures
import glob
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libchromofold_b200.so")
MS_BRIDGE_LIB = os.path.join(HERE, "libchromofold_b200_llama_ms.so")
OBJ_DIR = os.path.join(HERE, "build")


def sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")) + glob.glob(os.path.join(HERE, "csrc", "*.cpp")))


def bridge_sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc_llama_ms_bridge", "*.cpp")))


def headers():
    return glob.glob(os.path.join(HERE, "csrc", "*.cuh")) + glob.glob(os.path.join(HERE, "csrc", "*.h")) + glob.glob(
        os.path.join(ROOT, "include", "chromofold_b200", "*.h"))


def stale():
    if not os.path.exists(LIB) or not os.path.exists(MS_BRIDGE_LIB):
        return True
    built = min(os.path.getmtime(LIB), os.path.getmtime(MS_BRIDGE_LIB))
    deps = sources() + bridge_sources() + headers()
    return any(os.path.getmtime(f) > built for f in deps)


def _run(cmd, what):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(what + " failed")
    return proc.stderr


def build(force=False, verbose=False, incremental=False):
    """force: recompile everything; incremental: recompile the sources that are newer than their objects (the
    default only asks whether the library is older than any source or header, and then does the same)."""
    if not force and not incremental and not stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    extra = os.environ.get("CFB_NVCC_FLAGS", "").split()  # extra -D switches for tuning experiments
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++20", "--extended-lambda",
             "-Xcompiler", "-fPIC,-fvisibility=default", "-I" + os.path.join(ROOT, "include"),
             "-I" + os.path.join(HERE, "csrc")] + (["-Xptxas", "-v"] if verbose else []) + extra
    tag = hashlib.sha1(" ".join(flags).encode()).hexdigest()[:10]   # objects of another flag set are not reused
    os.makedirs(OBJ_DIR, exist_ok=True)
    newest_header = max([os.path.getmtime(h) for h in headers()] + [os.path.getmtime(__file__)])

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + "." + tag + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), newest_header):
            return obj, ""
        return obj, _run([nvcc] + flags + ["-c", src, "-o", obj], "nvcc on " + os.path.basename(src))

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        results = list(pool.map(compile_one, sources()))
    if verbose:
        sys.stderr.write("".join(log for _, log in results))
    _run([nvcc, "-shared", "-cudart", "static", "-Xlinker", "-Bsymbolic", "-Xcompiler", "-fPIC"] +
         [obj for obj, _ in results] + ["-o", LIB], "linking " + os.path.basename(LIB))
    gxx = shutil.which("g++") or "g++"
    _run([gxx, "-O2", "-std=c++20", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include")] + bridge_sources() +
         ["-o", MS_BRIDGE_LIB, "-L" + HERE, "-lchromofold_b200", "-Wl,-rpath,$ORIGIN", "-Wl,-Bsymbolic"],
         "g++ on the llama-server multi-sequence bridge")
    return LIB


if __name__ == "__main__":
    print(build(force="-f" in sys.argv or "-v" in sys.argv, verbose="-v" in sys.argv, incremental=True))
