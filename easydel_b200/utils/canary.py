"""Guard bands around device allocations: a stand-in for a memory checker on kernels' output buffers.

Inside ``with CanaryGuard() as guard:`` every CUDA tensor that ``torch.empty`` / ``torch.empty_like`` /
``torch.zeros`` hand out sits between two 4 KiB bands of a known byte pattern, and the tensor's own bytes start out as
that pattern too (so a kernel that skips part of its output leaves a recognisable value behind). ``guard.check()``
(also run on exit) reports every allocation whose bands were written to: an out-of-bounds store of a kernel whose
output came from one of these allocators. Reads out of bounds are not seen, and allocations made by other routes
(``torch.randn``, views of the paged cache) are not wrapped. Not thread-safe: the allocator entry points are patched
process-wide for the duration of the block.

The reference relies on XLA's own buffer assignment and has no counterpart; this exists because the usual tool for
the job (a memory checker under the kernel) is not available where these kernels are developed.
"""

from __future__ import annotations

import torch

PATTERN = 0xA5
BAND = 4096


class CanaryGuard:
    def __init__(self, band: int = BAND):
        self.band = band
        self.live: list[tuple[torch.Tensor, int, str]] = []
        self.violations: list[str] = []
        self._orig: dict = {}

    # -- allocation
    def _alloc(self, shape, dtype, device, zero: bool, what: str) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        item = torch.empty(0, dtype=dtype).element_size()
        nbytes = n * item
        pad = (-nbytes) % 256
        raw = self._orig["empty"](self.band + nbytes + pad + self.band, dtype=torch.uint8, device=device)
        raw.fill_(PATTERN)
        body = raw[self.band:self.band + nbytes]
        if zero:
            body.zero_()
        self.live.append((raw, nbytes, what))
        return body.view(dtype).view(*shape) if n else self._orig["empty"](*shape, dtype=dtype, device=device)

    @staticmethod
    def _shape_of(args, kw):
        if "size" in kw:
            return tuple(kw["size"])
        if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
            return tuple(args[0])
        return tuple(args)

    def _wrap(self, name: str, zero: bool):
        orig = self._orig[name]

        def f(*args, **kw):
            device = kw.get("device")
            dev = torch.device(device) if device is not None else None
            if dev is None or dev.type != "cuda" or kw.get("pin_memory") or kw.get("layout") not in (None, torch.strided) \
                    or kw.get("out") is not None:
                return orig(*args, **kw)
            return self._alloc(self._shape_of(args, kw), kw.get("dtype") or torch.get_default_dtype(), dev, zero,
                               f"torch.{name}{self._shape_of(args, kw)}")

        return f

    def _empty_like(self, t, *args, **kw):
        if not isinstance(t, torch.Tensor) or not t.is_cuda or kw.get("memory_format") not in (
                None, torch.contiguous_format, torch.preserve_format):
            return self._orig["empty_like"](t, *args, **kw)
        return self._alloc(tuple(t.shape), kw.get("dtype") or t.dtype, kw.get("device") or t.device, False,
                           f"torch.empty_like{tuple(t.shape)}")

    # -- checking
    def check(self) -> list[str]:
        """Band bytes that no longer hold the pattern, as messages (also kept in ``violations``)."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = []
        for raw, nbytes, what in self.live:
            pad = (-nbytes) % 256
            front = raw[:self.band]
            back = raw[self.band + nbytes:self.band + nbytes + pad + self.band]
            for side, band in (("before", front), ("after", back)):
                bad = (band != PATTERN).nonzero()
                if bad.numel():
                    first = int(bad[0])
                    off = first - self.band if side == "before" else first
                    out.append(f"{what}: {int(bad.numel())} guard byte(s) written {side} the buffer "
                               f"(first at offset {off} from its {'start' if side == 'before' else 'end'})")
        self.violations = out
        return out

    def __enter__(self) -> "CanaryGuard":
        self._orig = {"empty": torch.empty, "zeros": torch.zeros, "empty_like": torch.empty_like}
        torch.empty = self._wrap("empty", False)
        torch.zeros = self._wrap("zeros", True)
        torch.empty_like = self._empty_like
        return self

    def __exit__(self, exc_type, exc, tb):
        torch.empty, torch.zeros, torch.empty_like = self._orig["empty"], self._orig["zeros"], self._orig["empty_like"]
        if exc_type is None:
            bad = self.check()
            if bad:
                raise AssertionError("out-of-bounds writes detected:\n  " + "\n  ".join(bad))
        self.live.clear()
        return False
