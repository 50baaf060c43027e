"""Utilities: checkpoint-format converters, the environment-flag tier, timers, memory monitor."""

from .helpers import (ENV_FLAGS, MemoryMonitor, Timer, Timers, check_bool_flag, describe_env, device_memory, flag,
                      get_logger, nvtx_range)

__all__ = ["ENV_FLAGS", "MemoryMonitor", "Timer", "Timers", "check_bool_flag", "describe_env", "device_memory", "flag",
           "get_logger", "nvtx_range"]
