"""Sliding-window z-score detector used to skip updates on loss / gradient-norm spikes (reference: llmc/outlier_detector.h)."""
from . import _hostlib


class OutlierDetector:
    WINDOW = 128

    def __init__(self):
        self._lib = _hostlib.lib()
        self._h = self._lib.llmc_outlier_new()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.llmc_outlier_free(self._h)
            self._h = None

    def update(self, value):
        """Returns the z-score of ``value`` against the last 128 values, or NaN while the window is filling."""
        return float(self._lib.llmc_outlier_update(self._h, float(value)))
