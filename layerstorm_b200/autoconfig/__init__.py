from .hwdetect import GpuInfo, HardwareInfo, detect, synthetic
from .solver import AutoconfigRefusal, Levers, PINNABLE, Result, explain_text, solve, write_result
from . import sizing
