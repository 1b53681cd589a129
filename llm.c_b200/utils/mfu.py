"""Model-FLOPs utilisation and GPU telemetry (reference: llmc/mfu.h).

The reference's table of promised FLOPs stops at Hopper, so on a B200 it prints -100 %.  This table adds the
Blackwell parts (dense bf16 tensor throughput from the public datasheets) and keeps the same lookup-by-name
semantics.  Telemetry reads NVML for the process's own device index."""
import math

# dense bf16 tensor TFLOP/s
PROMISED_BF16_TFLOPS = {
    "NVIDIA B200": 2250.0, "NVIDIA B100": 1800.0, "NVIDIA GB200": 2500.0, "NVIDIA H200": 989.0, "NVIDIA H100 80GB HBM3": 989.0,
    "NVIDIA H100 PCIe": 756.0, "NVIDIA H100": 989.0, "NVIDIA A100-SXM4-80GB": 312.0, "NVIDIA A100-SXM4-40GB": 312.0,
    "NVIDIA A100-PCIE-40GB": 312.0, "NVIDIA A100 80GB PCIe": 312.0, "Tesla V100-SXM2-16GB": 125.0, "NVIDIA GeForce RTX 4090": 165.2,
    "NVIDIA GeForce RTX 3090": 71.0, "NVIDIA L4": 121.0, "NVIDIA L40S": 362.0,
}


def get_flops_promised(device_name, precision="bf16"):
    """TFLOP/s the device promises at the given precision, or -1 if unknown."""
    for key, val in PROMISED_BF16_TFLOPS.items():
        if key in device_name or device_name in key:
            if precision in ("bf16", "fp16"):
                return val
            if precision == "fp32":
                return val / 2.0      # TF32 tensor path
    return -1.0


def measured_peak_tflops(path=None):
    """Sustained bf16 matmul TFLOP/s measured on this machine class, from ``MEASURED_PEAKS.json`` at the repository root (written by
    the benchmark driver: a seconds-long cuBLAS loop under the power cap), or -1 if the file is absent."""
    import json
    import os
    if path is None:
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops_sustained") or d.get("bf16_tflops") or -1.0)
    except (OSError, ValueError):
        return -1.0


def estimate_mfu(flops_per_token, tokens, dt_seconds, device_name, precision="bf16"):
    """(6 N + 6 L C T) * tokens / dt / peak, or -1 if the peak is unknown (reference train_gpt2.cu:1126-1153)."""
    peak = get_flops_promised(device_name, precision)
    if peak <= 0 or dt_seconds <= 0:
        return -1.0
    return flops_per_token * tokens / dt_seconds / (peak * 1e12)


class GPUTelemetry:
    """clock, power, temperature, utilisation and throttle reasons of one device through NVML (read only)."""

    def __init__(self, device_index=0, nvml=None):
        self.ok = False
        try:
            self.nvml = nvml
            if self.nvml is None:
                import pynvml
                self.nvml = pynvml
            self.nvml.nvmlInit()
            self.handle = self.nvml.nvmlDeviceGetHandleByIndex(device_index)
            self.ok = True
        except Exception:
            self.ok = False

    def read(self):
        if not self.ok:
            return None
        n, h = self.nvml, self.handle
        try:
            util = n.nvmlDeviceGetUtilizationRates(h)
            return dict(clock=n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM), max_clock=n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM),
                        power=n.nvmlDeviceGetPowerUsage(h) / 1000.0, power_limit=n.nvmlDeviceGetEnforcedPowerLimit(h) / 1000.0,
                        temperature=n.nvmlDeviceGetTemperature(h, n.NVML_TEMPERATURE_GPU), gpu_utilization=util.gpu,
                        mem_utilization=util.memory, throttle_reasons=int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h)))
        except Exception:
            return None

    @staticmethod
    def format(info):
        if info is None:
            return "GPU telemetry unavailable"
        return ("clock %d/%d MHz | power %.0f/%.0f W | temp %d C | util %d%% | mem util %d%% | throttle 0x%x" %
                (info["clock"], info["max_clock"], info["power"], info["power_limit"], info["temperature"], info["gpu_utilization"],
                 info["mem_utilization"], info["throttle_reasons"]))
