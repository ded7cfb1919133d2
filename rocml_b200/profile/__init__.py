"""Per-kernel timing against the device's limits (``--profile``): see ``profiler`` and ``report``."""
from . import cost
from . import profiler as _profiler
from .peaks import Peaks, load_peaks
from .profiler import OpRecord, Profiler, StepRecord, scope
from .report import build_report, to_human


def active():
    """The profiler that is switched on, or None."""
    return _profiler.ACTIVE


__all__ = ["cost", "Peaks", "load_peaks", "Profiler", "OpRecord", "StepRecord", "scope", "build_report",
           "to_human", "active"]
