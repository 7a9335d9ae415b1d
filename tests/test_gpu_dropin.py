"""The drop-in boundary seen from the reference's side: the reference's own test programs that use only its public
kernel / pool API (the CMake test targets kernels, kv_scale_storage, kv_int8_convert, rope_table and memory), compiled
UNMODIFIED against this library in place of the reference's kernel objects (oracle/Makefile, target `dropin`), must
pass.  The programs are built where the reference tree is present and travel as binaries."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "dropin")


@pytest.mark.parametrize("name", ["test_kernels", "test_kv_scale_storage", "test_kv_int8_convert", "test_rope_table", "test_memory"])
def test_reference_test_program_passes_against_this_library(name):
    exe = os.path.join(BIN, name)
    assert os.path.exists(exe), f"{exe} is missing: run `make -C oracle ref` where the reference tree is present"
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    tail = (r.stdout + r.stderr)[-1500:]
    assert r.returncode == 0, f"{name} exited with {r.returncode}:\n{tail}"
