#!/usr/bin/env python
"""Generates tests/golden/reference_outputs.json from the aiehlc reference itself.

Runs the reference's own example programs -- compiled from their sources in the reference tree
against the CPU tile emulator (oracle/ref_build.sh -> oracle/_ref/) -- and records what their
kernels wrote back to external memory, plus whether the program's own in-file golden check
passed.  Needs the reference tree; the JSON it writes is committed so the tests do not.

    python tests/golden/make_golden.py [/path/to/aiehlc]
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
REF_BIN = ROOT / "oracle" / "_ref"

PROGRAMS = {
    # name: (source in the reference tree, line that proves the program's own check passed)
    "aieml_perf": ("example/perf/aieml_perf.cc", "CPU result matches vmem_out."),
    "multi_tile": ("example/multi/multi_tile.cpp", "Sucess: CPU result matches AIE."),
    "seq_full_col": ("example/multi/seq_full_col.cpp", "Sucess: CPU result matches AIE."),
    "multi_kernel": ("example/multi/multi_kernel.cc", "Sucess: CPU result matches AIE."),
    "tutorial_example": ("tutorial/example.cpp", "Sucess: CPU result matches AIE."),
}


def main() -> int:
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AIEHLC_REFERENCE")
    if not ref:
        print("usage: make_golden.py /path/to/aiehlc   (or set AIEHLC_REFERENCE)")
        return 2
    subprocess.run(["bash", str(ROOT / "oracle" / "ref_build.sh"), ref], check=True)
    out = {"generator": "tests/golden/make_golden.py", "programs": {}}
    for name, (src, ok_line) in PROGRAMS.items():
        with tempfile.TemporaryDirectory() as td:
            dump = Path(td) / "dump.bin"
            env = dict(os.environ, AIEHLC_REF_DUMP=str(dump))
            res = subprocess.run([str(REF_BIN / name)], capture_output=True, text=True, env=env, timeout=60)
            words = np.frombuffer(dump.read_bytes(), dtype="<i4")
        out["programs"][name] = {
            "source": src,
            "self_check_passed": ok_line in res.stdout and "mismatches." not in res.stdout,
            "self_check_count": res.stdout.count(ok_line),
            "words_read_back": [int(v) for v in words],
        }
    (Path(__file__).parent / "reference_outputs.json").write_text(json.dumps(out, indent=1) + "\n")
    for k, v in out["programs"].items():
        print(k, v["self_check_passed"], len(v["words_read_back"]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
