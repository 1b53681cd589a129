"""The C++ host library under AddressSanitizer and UndefinedBehaviorSanitizer (the reference runs its data-loader unit test under
-fsanitize=address, .github/workflows/ci_tests.yml:21-28): a sanitized build of csrc/host/host.cpp is exercised through the same
ctypes entry points by a child process that preloads the sanitizer runtime."""
import os
import shutil
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(ROOT, "llm.c_b200", "csrc", "host", "host.cpp")

DRIVER = r"""
import ctypes, os, sys, numpy as np
sys.path.insert(0, %(root)r)
os.environ["LLMC_HOST_LIB"] = %(lib)r
from llmc_b200.utils.dataloader import DataLoader, EvalLoader, write_datafile, write_evalfile
from llmc_b200.utils.rand import MT19937
from llmc_b200.utils.outlier import OutlierDetector
from llmc_b200.utils.schedulers import LearningRateScheduler
d = %(dir)r
for i in range(3):
    write_datafile(os.path.join(d, "s%%d.bin" %% i), np.arange(i * 1000, i * 1000 + 700) %% 60000)
for shuffle in (0, 1):
    dl = DataLoader(os.path.join(d, "s*.bin"), 2, 16, 0, 2, shuffle, prefetch=bool(shuffle))
    seen = 0
    for _ in range(60):
        x, y = dl.next_batch()
        assert x.shape == (2, 16) and int((y[:, :-1] - x[:, 1:]).abs().max()) == 0
        seen += 1
    dl.close()
write_evalfile(os.path.join(d, "e.bin"), [dict(ctx=[1, 2, 3], endings=[[4], [5, 6], [7], [8, 9, 10]], label=2) for _ in range(5)])
el = EvalLoader(os.path.join(d, "e.bin"), 4, 16, 0, 1)
for _ in range(el.num_batches):
    el.next_batch()
el.close()
r = MT19937(7)
assert r.normal(33, 0.0, 1.0).numel() == 33 and r.uniform(5).numel() == 5
od = OutlierDetector()
for i in range(200):
    od.update(float(i %% 7))
s = LearningRateScheduler("cosine", 1e-3, 10, 100, 0.1)
assert s.get_learning_rate(0) > 0
print("sanitized run complete")
"""


def _runtime(name):
    out = subprocess.run(["g++", "-print-file-name=%s" % name], stdout=subprocess.PIPE, text=True).stdout.strip()
    return out if os.path.isabs(out) and os.path.exists(out) else None


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_host_library_is_clean_under_asan_and_ubsan(tmp_path):
    asan, ubsan = _runtime("libasan.so"), _runtime("libubsan.so")
    if asan is None:
        pytest.skip("the AddressSanitizer runtime is not installed")
    lib = str(tmp_path / "libllmc_host_san.so")
    flags = ["-fsanitize=address,undefined" if ubsan else "-fsanitize=address", "-fno-omit-frame-pointer", "-g", "-O1", "-std=c++17", "-fPIC",
             "-pthread", "-shared"]
    build = subprocess.run(["g++"] + flags + [SRC, "-o", lib], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert build.returncode == 0, build.stdout[-3000:]
    script = tmp_path / "driver.py"
    script.write_text(DRIVER % {"root": ROOT, "lib": lib, "dir": str(tmp_path)})
    env = dict(os.environ, LD_PRELOAD=":".join(x for x in (asan, ubsan) if x), ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=23",
               UBSAN_OPTIONS="halt_on_error=1:exitcode=24", LLMC_HOST_LIB=lib)
    run = subprocess.run([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert run.returncode == 0 and "sanitized run complete" in run.stdout, run.stdout[-4000:]
    assert "ERROR: AddressSanitizer" not in run.stdout and "runtime error:" not in run.stdout, run.stdout[-4000:]
