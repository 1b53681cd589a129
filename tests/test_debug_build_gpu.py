"""The debug build of the kernel library (-DLLMC_DEBUG_CHECKS, selected with LLMC_DEBUG_CHECKS=1): trains cleanly, and reports
an id outside the embedding table and a misaligned 16-byte access through the status word instead of faulting (the stand-in for
the compute-sanitizer runs of the reference's CI)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_debug_library_reports_bad_ids_and_misaligned_accesses():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    env = dict(os.environ, LLMC_DEBUG_CHECKS="1")
    r = subprocess.run([sys.executable, os.path.join(HERE, "debug_build_worker.py")], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["debug_lib"] == 1
    assert out["status_after_training"] == 0 and all(l == l and l < 20 for l in out["losses"]), out
    assert out["status_bad_token"] >> 24 == 4 and out["status_bad_token"] & 0xFFFFFF == 0xE01, out
    assert out["bad_token_output_finite"]
    assert out["status_misaligned"] >> 24 == 4 and (out["status_misaligned"] & 0xFFFF00) == 0xA00, out
    assert out["status_after"] == 0
