"""This library's headers beside the reference's own (needs the reference checkout; skipped where it is absent):
  * one translation unit includes the reference's headers of the path and then this library's: every prototype this
    library declares must be the reference's (a different parameter list or return type of an extern "C" function is a
    compile error), and this library's headers must stand aside where the reference's types are already defined;
  * sizeof and the offset of every member of every struct these headers define, printed once from this library's
    headers and once from the reference's, must be the same text."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("CF_REFERENCE_ROOT", os.path.abspath(os.path.join(ROOT, "..", "reference")))
REFERENCE_HEADERS = [
    "chromofold/chromofold.h", "chromofold/kv_runtime.h", "chromofold/kv_cuda.h", "chromofold/device_kv_dataplane.h",
    "chromofold/device_kv_seal_attention.h", "chromofold/multisequence_cuda_resolver.h", "chromofold/multisequence_cache.h",
    "chromofold/llama_server_runtime.h", "chromofold/production_attention.h", "chromofold/multigpu_cuda_runtime.h",
    "chromofold_kv_adapter.h", "chromofold_runtime_bridge.h", "chromofold_device_seal_bridge.h", "device_kv_graph_bridge.h",
    "graph/chromofold_graph_contract.h"]
OURS = ["compat_kv.h", "compat_device.h", "compat_ms.h", "compat_mscache.h", "compat_production.h", "compat_multigpu.h",
        "compat_adapter.h", "compat_bridges.h"]
STAND_ASIDE = ["CHROMOFOLD_LLAMA_SERVER_RUNTIME_TYPES", "CHROMOFOLD_PRODUCTION_ATTENTION_TYPES",
               "CHROMOFOLD_MULTIGPU_CUDA_RUNTIME_TYPES"]   # for the reference headers that use #pragma once


def _flags():
    return ["-std=c++20", "-I", os.path.join(REFERENCE, "include"), "-I", os.path.join(REFERENCE, "integrations", "llama.cpp"),
            "-I", os.path.join(ROOT, "include")]


def _need_reference():
    if not os.path.isdir(os.path.join(REFERENCE, "include", "chromofold")) or shutil.which("g++") is None:
        pytest.skip("needs the reference checkout and g++")


def test_prototypes_are_the_references_own(tmp_path):
    _need_reference()
    lines = [f'#include "{h}"' for h in REFERENCE_HEADERS] + [f"#define {m}" for m in STAND_ASIDE]
    lines += [f'#include "chromofold_b200/{h}"' for h in OURS] + ["int main() { return 0; }"]
    src = tmp_path / "both.cpp"
    src.write_text("\n".join(lines) + "\n")
    done = subprocess.run(["g++", "-fsyntax-only", "-Wall"] + _flags() + [str(src)], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]


def test_prototypes_of_the_second_library_are_the_references_own(tmp_path):
    """compat_llama_ms_bridge.h (the llama-server bridges, a library of their own) beside the reference's bridge headers."""
    _need_reference()
    src = tmp_path / "bridges.cpp"
    src.write_text('#include "multisequence/llama_server_multisequence_bridge.h"\n'
                   '#include "multisequence/llama_server_cuda_resolver_bridge.h"\n'
                   '#include "chromofold_b200/compat_llama_ms_bridge.h"\nint main() { return 0; }\n')
    done = subprocess.run(["g++", "-fsyntax-only", "-Wall"] + _flags() + [str(src)], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]


def _structs():
    """(struct name, member names) of every struct with a body in this library's compat headers."""
    found = []
    for h in OURS:
        text = open(os.path.join(ROOT, "include", "chromofold_b200", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for name, body in re.findall(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*\1\s*;", text, flags=re.S):
            members = []
            for decl in body.split(";"):
                decl = decl.strip()
                if not decl:
                    continue
                for piece in decl.split(","):
                    ident = re.findall(r"[A-Za-z_]\w*", re.sub(r"\[.*?\]", "", piece))
                    if ident:
                        members.append(ident[-1])
            found.append((name, members))
    return found


def _layout_text(tmp_path, tag, includes):
    lines = ["#include <cstddef>", "#include <cstdio>"] + [f'#include "{h}"' for h in includes] + ["int main() {"]
    for name, members in _structs():
        lines.append(f'  std::printf("{name} %zu %zu\\n", sizeof({name}), alignof({name}));')
        for m in members:
            lines.append(f'  std::printf("{name}.{m} %zu\\n", offsetof({name}, {m}));')
    lines += ["  return 0;", "}"]
    src, exe = tmp_path / f"layout_{tag}.cpp", tmp_path / f"layout_{tag}"
    src.write_text("\n".join(lines) + "\n")
    done = subprocess.run(["g++", "-Wno-invalid-offsetof"] + _flags() + [str(src), "-o", str(exe)], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]
    return subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout


def test_struct_layouts_are_the_references_own(tmp_path):
    _need_reference()
    structs = _structs()
    assert len(structs) >= 40 and sum(len(m) for _, m in structs) >= 300
    ours = _layout_text(tmp_path, "ours", [f"chromofold_b200/{h}" for h in OURS])
    theirs = _layout_text(tmp_path, "reference", REFERENCE_HEADERS)
    assert ours == theirs
