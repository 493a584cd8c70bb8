"""`lf.utils`: Logger and Config (lua/luatorch/init.lua:36-39) plus device timing helpers."""
from .config import Config
from .logger import Logger
from .timing import ClockSampler, DeviceTimer
from . import nvtx
from . import debug

__all__ = ["Logger", "Config", "DeviceTimer", "ClockSampler", "nvtx", "debug"]
