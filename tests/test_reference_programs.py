"""The reference's own test programs, linked against the reference rebuilt with its frozen-linear and
LoRA-adapter translation units bound to libcaifq.so (oracle/build_ref_dropin.py), run on the GPU.

Each program is the reference's unmodified tests/<name>.cpp; it prints [PASS]/[FAIL] per case and exits
non-zero if any case failed.  Skipped where the programs have not been built (they are built where the
reference checkout is, and travel as files)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "bin")
PROGRAMS = ("test_device_frozen_linear", "test_device_lora_adapter", "test_device_moe_frozen_expert",
            "test_pluggable_projections")


def _run(name, env=None):
    exe = os.path.join(BIN, name)
    if not os.path.exists(exe):
        pytest.skip("%s has not been built (python oracle/build_ref_dropin.py)" % name)
    full = dict(os.environ)
    full.update(env or {})
    res = subprocess.run([exe], capture_output=True, text=True, timeout=900, env=full)
    return res.returncode, res.stdout + res.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("name", PROGRAMS)
def test_reference_program_passes_on_libcaifq(name):
    code, out = _run(name)
    assert out.count("[PASS]") >= 10, out[-2000:]
    assert "[FAIL]" not in out, out[-2000:]
    assert code == 0


@pytest.mark.gpu
def test_the_programs_compute_through_the_c_abi():
    """With the library told to take nothing but few-token calls, the drop-in frozen-linear program must fail
    (its many-token forwards are this library's calls), while the same program on the unmodified reference
    library does not notice."""
    code, out = _run("test_device_frozen_linear", {"CAIFQ_FORCE_PATH": "decode"})
    assert code != 0 and "[FAIL]" in out
    code, out = _run("test_device_frozen_linear_stock", {"CAIFQ_FORCE_PATH": "decode"})
    assert code == 0 and "[FAIL]" not in out
