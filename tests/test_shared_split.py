"""The arithmetic that cuts a shared prefix over the CTAs of the shared-prefix kernel (SharedSplit,
chromofold_b200/csrc/cf_device_common.cuh), checked on the host: the plan kernel, the attention kernel and the combine
kernel each evaluate it on their own, so they must agree on which CTA holds a round and how many partials a row has."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include "cf_device_common.cuh"
#include <cstdio>
using namespace cfb;
int main() {
    long cases = 0;
    for (uint32_t sm : {1u, 4u, 108u, 132u, 148u, 160u})
        for (uint32_t head_tiles = 1; head_tiles <= 300; ++head_tiles)
            for (uint32_t rounds : {1u, 2u, 3u, 7u, 15u, 16u, 17u, 100u, 128u, 1000u}) {
                const uint32_t ctas = shared_split_ctas(rounds, head_tiles, sm, CF_B200_SHARED_CHUNKS_MAX);
                if (ctas == 0 || ctas > sm) return 1;
                const SharedSplit s = {rounds, head_tiles, ctas};
                if (s.first_round(0) != 0 || s.first_round(ctas) != s.total()) return 2;
                uint64_t least = ~0ull, most = 0;
                for (uint32_t b = 0; b < ctas; ++b) {          // every round belongs to exactly one CTA, none is idle
                    const uint64_t lo = s.first_round(b), hi = s.first_round(b + 1);
                    if (hi <= lo) return 3;
                    least = hi - lo < least ? hi - lo : least;
                    most = hi - lo > most ? hi - lo : most;
                    if (s.cta_of(lo) != b || s.cta_of(hi - 1) != b) return 4;
                }
                if (most - least > 1) return 5;                  // equal stretches to within one round
                for (uint32_t t = 0; t < head_tiles; ++t) {      // partial cells of a head-tile fit the workspace
                    const uint64_t first = static_cast<uint64_t>(t) * rounds;
                    if (s.cta_of(first + rounds - 1) - s.cta_of(first) + 1 > CF_B200_SHARED_CHUNKS_MAX) return 6;
                }
                ++cases;
            }
    std::printf("%ld\n", cases);
    return 0;
}
"""


def test_shared_split_covers_every_round_once_and_bounds_the_partials(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    src = tmp_path / "split.cu"
    src.write_text(PROGRAM)
    exe = tmp_path / "split"
    subprocess.run([nvcc, "-std=c++17", "-Wno-deprecated-gpu-targets", "-I", os.path.join(ROOT, "include"), "-I",
                    os.path.join(ROOT, "chromofold_b200", "csrc"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, f"check {out.returncode} failed"
    assert int(out.stdout) == 6 * 300 * 10
