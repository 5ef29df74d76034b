"""Compile the CUDA sources of this package into chromofold_b200/libchromofold_b200.so (sm_100a only), and the
llama-server multi-sequence bridge (host code, linked against it) into chromofold_b200/libchromofold_b200_llama_ms.so."""
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libchromofold_b200.so")
MS_BRIDGE_LIB = os.path.join(HERE, "libchromofold_b200_llama_ms.so")


def sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")) + glob.glob(os.path.join(HERE, "csrc", "*.cpp")))


def bridge_sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc_llama_ms_bridge", "*.cpp")))


def stale():
    if not os.path.exists(LIB) or not os.path.exists(MS_BRIDGE_LIB):
        return True
    built = min(os.path.getmtime(LIB), os.path.getmtime(MS_BRIDGE_LIB))
    deps = sources() + bridge_sources() + glob.glob(os.path.join(HERE, "csrc", "*.cuh")) + glob.glob(
        os.path.join(ROOT, "include", "chromofold_b200", "*.h"))
    return any(os.path.getmtime(f) > built for f in deps)


def build(force=False, verbose=False):
    if not force and not stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
           "--extended-lambda", "-Xcompiler", "-fPIC,-fvisibility=default", "-shared", "-cudart", "static",
           "-Xlinker", "-Bsymbolic", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(HERE, "csrc")]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("CFB_NVCC_FLAGS", "").split()  # extra -D switches for tuning experiments
    cmd += sources() + ["-o", LIB]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        sys.stderr.write(proc.stderr)
    gxx = shutil.which("g++") or "g++"
    cmd = [gxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include")] + bridge_sources() + [
        "-o", MS_BRIDGE_LIB, "-L" + HERE, "-lchromofold_b200", "-Wl,-rpath,$ORIGIN", "-Wl,-Bsymbolic"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("g++ failed on the llama-server multi-sequence bridge")
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
