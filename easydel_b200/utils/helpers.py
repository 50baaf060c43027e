"""Small runtime helpers: the environment-flag tier, timers, a device-memory monitor, NVTX ranges.

Counterparts of easydel/utils/helpers.py (``check_bool_flag`` :437, ``Timer`` / ``Timers`` :99-330,
``get_logger``) and of the memory-usage reporting of easydel/utils/analyze_memory.py. Flags that steer XLA, TPU
transfers or JAX compilation caches in the reference have nothing to act on here and are listed as such in
:data:`ENV_FLAGS` so that a launch script written for the reference can be read against this table.
"""

from __future__ import annotations

import contextlib
import dataclasses
import logging
import os
import threading
import time
import typing as tp

_TRUE = ("true", "yes", "ok", "1", "easy")


def check_bool_flag(name: str, default: bool = True) -> bool:
    """Boolean environment variable; 'true', 'yes', 'ok', '1', 'easy' (any case) count as set."""
    return str(os.getenv(name, "1" if default else "0")).lower() in _TRUE


def env_int(name: str, default: int) -> int:
    try:
        return int(os.getenv(name, default))
    except (TypeError, ValueError):
        return default


def env_float(name: str, default: float) -> float:
    try:
        return float(os.getenv(name, default))
    except (TypeError, ValueError):
        return default


@dataclasses.dataclass(frozen=True)
class EnvFlag:
    name: str
    default: tp.Any
    kind: str            # "bool" | "int" | "float" | "str"
    effect: str          # what it does here; "no effect here: ..." for flags of the reference's XLA / TPU paths

    def value(self):
        if self.kind == "bool":
            return check_bool_flag(self.name, bool(self.default))
        if self.kind == "int":
            return env_int(self.name, self.default)
        if self.kind == "float":
            return env_float(self.name, self.default)
        return os.getenv(self.name, self.default)


#: Every environment variable this package reads, and the reference's that it accepts without effect.
ENV_FLAGS: dict[str, EnvFlag] = {f.name: f for f in (
    EnvFlag("EDL_LIB_PATH", None, "str", "path of another build of the kernel library (e.g. one with bounds checks)"),
    EnvFlag("EDL_FORCE_BUILD", False, "bool", "rebuild the kernel library in-tree on import even if it exists"),
    EnvFlag("EDL_NVCC_EXTRA", "", "str", "extra nvcc flags for csrc/build.py (e.g. -DEDL_BOUNDS_CHECK)"),
    EnvFlag("EDL_GEMM_PAIR", True, "bool", "use the two-CTA (cta_group::2) GEMM for large products"),
    EnvFlag("EDL_GEMM_PAIR128", False, "bool", "skinny products (129-512 rows) may use the CTA-pair GEMM with 256 x 128 "
            "tiles (off: measured the same as the 128-wide kernel)"),
    EnvFlag("EDL_GEMM_PAIR_SPLITK", False, "bool", "plan the two-slice split-K form of the CTA-pair GEMM for skinny "
            "products (off: measured no faster than the 128-wide kernel)"),
    EnvFlag("EDL_TP_TWO_SHOT", True, "bool", "tensor-parallel decode all-reduces of 1-8 MiB run the two-shot peer-memory "
            "kernel (off: NCCL)"),
    EnvFlag("EDL_TP_MULTIMEM", "auto", "str", "peer all-reduce kernels sum and broadcast through the NVLink switch "
            "(multimem): auto = from four ranks up | 1 | 0"),
    EnvFlag("EDL_ESURGE_CUDA_GRAPHS", True, "bool", "replay decode steps from CUDA graphs"),
    EnvFlag("EDL_NVTX", False, "bool", "emit NVTX ranges around trainer steps, engine steps and layers"),
    EnvFlag("EASURGE_MAX_SCHEDULER_ERRORS", 3, "int", "consecutive engine-step errors before in-flight requests fail"),
    EnvFlag("EASURGE_HEARTBEAT_WARN_S", 30.0, "float", "seconds without an engine heartbeat before a warning"),
    EnvFlag("EASURGE_SYNC_INPUTS_FOR_TIMING", False, "bool", "synchronise the device after every engine step "
            "(exact per-step timings, no overlap)"),
    EnvFlag("EASURGE_ENABLE_DP_LOCAL_PAGE_PATH", True, "bool", "KV-page data parallelism: requests keep their pages "
            "on the data-parallel shard that admitted them"),
    EnvFlag("ESURGE_DETOKENIZER_CONTEXT_WINDOW", 6, "int", "tokens of left context the incremental detokenizer keeps"),
    EnvFlag("EP_DISPATCH", "auto", "str", "expert-parallel token exchange: auto | alltoall | allgather"),
    EnvFlag("EP_AUTO_THRESHOLD", 0, "int", "tokens per rank below which 'auto' picks the all-gather exchange"),
    EnvFlag("ENABLE_DISTRIBUTED_INIT", True, "bool", "initialise torch.distributed from RANK / WORLD_SIZE on import "
            "of the parallel runtime"),
    EnvFlag("EASYDEL_FORCE_TORCH_USE_CPU", False, "bool", "build models on the CPU even when a GPU is present"),
    EnvFlag("EASYDEL_AUTO", True, "bool", "no effect here: automatic XLA flag set-up"),
    EnvFlag("EASYDEL_CACHE_COMPILES", False, "bool", "no effect here: JAX compilation cache"),
    EnvFlag("EASYDEL_RECOMPILE_FORCE", False, "bool", "no effect here: forces XLA recompilation"),
    EnvFlag("EASY_SAFE_TRANSFER", True, "bool", "no effect here: TPU host-transfer guard"),
    EnvFlag("EKERNEL_OPS", False, "bool", "no effect here: ejkernel operation registry switch"),
    EnvFlag("EFORMER_CREATE_MESH", True, "bool", "no effect here: eformer mesh construction"),
)}


def flag(name: str):
    """Current value of a documented flag (``KeyError`` for names that are not in :data:`ENV_FLAGS`)."""
    return ENV_FLAGS[name].value()


def describe_env() -> str:
    rows = [f"{f.name:38s} {str(f.value()):>10s}   {f.effect}" for f in ENV_FLAGS.values()]
    return "\n".join(rows)


def get_logger(name: str, level: int | str | None = None) -> logging.Logger:
    lg = logging.getLogger(name)
    if not lg.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s %(name)s %(levelname)s: %(message)s", "%H:%M:%S"))
        lg.addHandler(h)
        lg.propagate = False
    lg.setLevel(level if level is not None else os.getenv("LOGGING_LEVEL_ED", "INFO"))
    return lg


# ------------------------------------------------------------------------------------------------ timers
class Timer:
    """Accumulating wall-clock timer; with ``cuda=True`` the device is synchronised at start and stop."""

    def __init__(self, name: str, cuda: bool = False):
        self.name, self.cuda = name, cuda
        self.elapsed_total = 0.0
        self.calls = 0
        self._t0: float | None = None

    def _sync(self):
        if self.cuda:
            import torch

            if torch.cuda.is_available():
                torch.cuda.synchronize()

    def start(self):
        if self._t0 is not None:
            raise RuntimeError(f"timer {self.name!r} already started")
        self._sync()
        self._t0 = time.perf_counter()

    def stop(self) -> float:
        if self._t0 is None:
            raise RuntimeError(f"timer {self.name!r} was not started")
        self._sync()
        dt = time.perf_counter() - self._t0
        self._t0 = None
        self.elapsed_total += dt
        self.calls += 1
        return dt

    def reset(self):
        self.elapsed_total, self.calls, self._t0 = 0.0, 0, None

    def elapsed(self, reset: bool = True) -> float:
        running = self._t0 is not None
        if running:
            self.stop()
        v = self.elapsed_total
        if reset:
            self.reset()
        if running:
            self.start()
        return v


class Timers:
    """Named timers with ``with timers.timed("x"):`` blocks and a ``log`` that can write to a metrics sink."""

    def __init__(self, use_wandb: bool = False, tensorboard_writer=None, cuda: bool = False):
        self.timers: dict[str, Timer] = {}
        self.use_wandb, self.tb, self.cuda = use_wandb, tensorboard_writer, cuda

    def __call__(self, name: str) -> Timer:
        if name not in self.timers:
            self.timers[name] = Timer(name, self.cuda)
        return self.timers[name]

    @contextlib.contextmanager
    def timed(self, name: str, log: bool = False):
        t = self(name)
        t.start()
        try:
            yield t
        finally:
            dt = t.stop()
            if log:
                get_logger("easydel_b200.timers").info("%s: %.4f s", name, dt)

    def write(self, names: tp.Iterable[str], iteration: int, normalizer: float = 1.0, reset: bool = False) -> dict:
        out = {}
        for n in names:
            v = self.timers[n].elapsed(reset=reset) / normalizer
            out[f"timers/{n}"] = v
            if self.tb is not None:
                self.tb.add_scalar(f"timers/{n}", v, iteration)
        if self.use_wandb:
            try:
                import wandb

                wandb.log(out, step=iteration)
            except Exception:   # metrics sinks never break a run
                pass
        return out

    def log(self, names: tp.Iterable[str] | None = None, normalizer: float = 1.0, reset: bool = True) -> str:
        names = list(names) if names is not None else list(self.timers)
        parts = [f"{n}: {self.timers[n].elapsed(reset=reset) * 1000.0 / normalizer:.2f} ms" for n in names]
        line = " | ".join(parts)
        get_logger("easydel_b200.timers").info(line)
        return line


# ------------------------------------------------------------------------------------------------ memory
def device_memory(device=None) -> dict[str, float]:
    """Allocator and driver view of one GPU's memory in GiB (empty on CPU-only machines)."""
    import torch

    if not torch.cuda.is_available():
        return {}
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    free, total = torch.cuda.mem_get_info(dev)
    g = 2.0 ** 30
    return {"allocated_gib": torch.cuda.memory_allocated(dev) / g, "reserved_gib": torch.cuda.memory_reserved(dev) / g,
            "peak_allocated_gib": torch.cuda.max_memory_allocated(dev) / g, "free_gib": free / g,
            "total_gib": total / g, "used_gib": (total - free) / g}


class MemoryMonitor:
    """Background sampler of device memory (the reference's ``SMPMemoryMonitor``, easydel/utils/analyze_memory.py).
    ``start()`` / ``stop()``; ``peak`` holds the highest driver-side usage seen, ``history`` the samples."""

    def __init__(self, interval: float = 1.0, device=None, keep: int = 3600):
        self.interval, self.device, self.keep = interval, device, keep
        self.history: list[tuple[float, dict[str, float]]] = []
        self.peak = 0.0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def sample(self) -> dict[str, float]:
        m = device_memory(self.device)
        if m:
            self.peak = max(self.peak, m["used_gib"])
            self.history.append((time.time(), m))
            if len(self.history) > self.keep:
                del self.history[: len(self.history) - self.keep]
        return m

    def _run(self):
        while not self._stop.wait(self.interval):
            self.sample()

    def start(self) -> "MemoryMonitor":
        if self._thread is None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, name="edl-memory-monitor", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> float:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
            self._thread = None
        return self.peak

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()

    def summary(self) -> str:
        m = device_memory(self.device)
        if not m:
            return "no CUDA device"
        return (f"used {m['used_gib']:.1f} / {m['total_gib']:.1f} GiB (peak seen {self.peak:.1f}), "
                f"torch allocated {m['allocated_gib']:.1f}, reserved {m['reserved_gib']:.1f}")


# ------------------------------------------------------------------------------------------------ NVTX
@contextlib.contextmanager
def nvtx_range(name: str):
    """An NVTX range around a block when ``EDL_NVTX`` is set (visible in Nsight Systems / Compute timelines); free
    otherwise."""
    if not _NVTX_ON[0]:
        yield
        return
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NVTX_ON = [False]


def refresh_nvtx_flag() -> bool:
    import torch

    _NVTX_ON[0] = bool(check_bool_flag("EDL_NVTX", False) and torch.cuda.is_available())
    return _NVTX_ON[0]


try:   # evaluated once at import; call refresh_nvtx_flag() after changing the environment
    refresh_nvtx_flag()
except Exception:
    pass
