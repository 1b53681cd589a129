"""Placement of optimizer state: device memory first, managed memory when the device allocation fails
(behaviour of cudaMallocConditionallyManaged in the reference, llmc/cuda_utils.cuh:213-229).  The device is faked here."""
import torch

from llmc_b200.utils import memory


def test_host_buffers_are_plain_tensors():
    t, managed = memory.zeros_device_or_managed(100, torch.float32, "cpu")
    assert not managed and t.shape == (100,) and t.dtype == torch.float32 and float(t.abs().sum()) == 0.0


def test_fallback_is_taken_only_when_the_device_is_full(monkeypatch):
    calls, logs = [], []

    def device_ok(numel, dtype, device):
        calls.append("device")
        return torch.zeros(numel, dtype=dtype)

    def device_full(numel, dtype, device):
        calls.append("device")
        raise torch.cuda.OutOfMemoryError("out of memory (faked)")

    def managed(numel, dtype, device, force):
        calls.append("managed force=%d" % force)
        return torch.zeros(numel, dtype=dtype), True

    monkeypatch.setattr(memory, "_managed_zeros", managed)
    monkeypatch.setattr(torch.cuda, "empty_cache", lambda: calls.append("empty_cache"))
    monkeypatch.delenv("LLMC_FORCE_MANAGED", raising=False)

    monkeypatch.setattr(memory, "_device_zeros", device_ok)
    t, m = memory.zeros_device_or_managed(10, torch.float32, "cuda:0", "moments", logs.append)
    assert not m and calls == ["device"] and not logs

    calls.clear()
    monkeypatch.setattr(memory, "_device_zeros", device_full)
    t, m = memory.zeros_device_or_managed(1 << 20, torch.float32, "cuda:0", "moments", logs.append)
    assert m and calls == ["device", "empty_cache", "managed force=0"]
    assert len(logs) == 1 and "moments" in logs[0] and "4.0 MiB" in logs[0] and "managed memory" in logs[0]

    calls.clear()
    monkeypatch.setenv("LLMC_FORCE_MANAGED", "1")
    t, m = memory.zeros_device_or_managed(10, torch.float32, "cuda:0", "moments", None)
    assert m and calls == ["managed force=1"]
