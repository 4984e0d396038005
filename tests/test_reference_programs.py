"""The reference's own example programs, built from its tree against the CPU tile emulator
(oracle/ref_build.sh), still reproduce the committed fixtures.  Skipped where oracle/_ref/ was
not built (no reference tree on that machine)."""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "oracle" / "_ref"


@pytest.mark.parametrize("name", ["aieml_perf", "multi_tile", "seq_full_col", "multi_kernel", "tutorial_example"])
def test_reference_program_reproduces_fixture(name, golden, tmp_path):
    exe = REF / name
    if not exe.exists():
        pytest.skip("oracle/_ref not built on this machine")
    dump = tmp_path / "dump.bin"
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60,
                         env=dict(os.environ, AIEHLC_REF_DUMP=str(dump)))
    words = np.frombuffer(dump.read_bytes(), dtype="<i4")
    assert [int(v) for v in words] == golden[name]["words_read_back"]
    assert "matches" in res.stdout and "mismatches." not in res.stdout
