"""The reference's OWN test programs (its tests/*.cpp and tests/*.cu, compiled from where they lie by oracle/Makefile) run
against this repository's library: every C-ABI call they make resolves to libchromofold_b200.so, so a pass means the
reference's own assertions hold for the drop-in. The CUDA tests bring the reference's fixture encoder, CPU reference and
page-upload helper along as their inputs and expected values. The binaries live in oracle/_ref/reftests; where they
were not built (no reference tree at build time) the tests are skipped."""
import subprocess

import pytest

CPU_ONLY = ["kv_runtime_test", "llama_graph_contract_test", "m15_multigpu_cuda_contract"]
NEED_GPU = ["llama_kv_adapter_seam", "device_kv_dataplane_contract", "m9_device_seal_contract",
            "m10_cuda_sequence_resolver_contract", "m10_multisequence_contract", "m10_multisequence_host_contract",
            "m11_pinned_server_contract", "m12_production_attention_contract", "paged_kv_cuda_seam",
            "paged_kv_cuda_correctness", "adapter_attention_test"]


def _run(oracle, name):
    programs = oracle.reference_test_programs()
    if name not in programs:
        pytest.skip("oracle/_ref/reftests was not built (needs the reference tree at build time)")
    done = subprocess.run([programs[name]], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, (name, done.returncode, done.stdout[-800:], done.stderr[-800:])


@pytest.mark.parametrize("name", CPU_ONLY)
def test_reference_test_program_passes_without_a_gpu(native, oracle, name):
    _run(oracle, name)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CPU_ONLY + NEED_GPU)
def test_reference_test_program_passes(native, oracle, name):
    _run(oracle, name)
