"""Guard regions around freshly allocated tensors: a debugging aid that shows a kernel writing outside
the tensor it was given, without any memory fault.

Inside ``with GuardRegions() as g:`` every tensor that Python code creates with ``torch.empty``,
``torch.empty_like``, ``torch.zeros`` or ``torch.zeros_like`` (which is how the ops layer creates the
outputs and workspaces it hands to kernels) comes from a larger byte buffer whose first and last ``band``
bytes hold a canary pattern.  ``g.check()`` re-reads all bands and returns one record
per damaged band: which allocation (shape, dtype, where it was made), which side, and the offset of the
first changed byte.  A write that overruns an output lands in the band - memory this process owns - so
nothing faults and the offender is named instead of silently corrupting its neighbour.

The interior keeps the allocator's alignment (bands are multiples of 256 bytes, sizes are rounded up to
256), so TMA descriptors and 16-byte vector accesses see what they would see without the guard.  Works
for CPU tensors as well, which is how the mechanism itself is tested.  Off unless the context is entered:
there is no cost in normal runs.
"""
from __future__ import annotations

import traceback
from dataclasses import dataclass
from typing import Any, Optional

import torch

CANARY = 0xA5


@dataclass
class Violation:
    index: int                 # n-th guarded allocation of the context
    side: str                  # "before" or "after" the tensor
    offset: int                # first damaged byte, counted from the tensor's edge outwards
    damaged: int               # damaged bytes in that band
    shape: tuple
    dtype: torch.dtype
    where: str                 # file:line of the allocation

    def __str__(self) -> str:
        return (f"allocation #{self.index} {tuple(self.shape)} {self.dtype} made at {self.where}: {self.damaged} byte(s) "
                f"written {self.side} the tensor, the first {self.offset} byte(s) from its edge")


class GuardRegions:
    def __init__(self, band: int = 4096, device_types: tuple[str, ...] = ("cuda", "cpu"), min_bytes: int = 1) -> None:
        if band % 256:
            raise ValueError("band must be a multiple of 256 bytes")
        self.band = band
        self.device_types = device_types
        self.min_bytes = min_bytes
        self.records: list[tuple[torch.Tensor, int, tuple, torch.dtype, str]] = []   # (raw buffer, payload bytes, shape, dtype, where)
        self._saved: dict[str, Any] = {}

    # ------------------------------------------------------------------ allocation
    def _where(self) -> str:
        for fr in reversed(traceback.extract_stack(limit=8)[:-3]):
            if "utils/guard.py" not in fr.filename and "/torch/" not in fr.filename:
                return f"{fr.filename.rsplit('/', 1)[-1]}:{fr.lineno}"
        return "?"

    def _alloc(self, shape: tuple, dtype: torch.dtype, device: torch.device, zero: bool) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * self._saved["empty"](0, dtype=dtype).element_size()
        padded = (nbytes + 255) // 256 * 256
        raw = self._saved["empty"](self.band + padded + self.band, dtype=torch.uint8, device=device)
        raw.fill_(CANARY)
        inner = raw[self.band:self.band + nbytes]
        if zero:
            inner.zero_()
        self.records.append((raw, nbytes, tuple(shape), dtype, self._where()))
        if n == 0:
            return self._saved["empty"](tuple(shape), dtype=dtype, device=device)
        return inner.view(dtype).reshape(tuple(shape))            # () for a scalar

    def _wants(self, device: Optional[torch.device | str], kw: dict) -> bool:
        if kw.get("pin_memory") or kw.get("memory_format") not in (None, torch.contiguous_format) or kw.get("out") is not None:
            return False
        if kw.get("layout") not in (None, torch.strided) or kw.get("requires_grad"):
            return False
        dev = torch.device(device) if device is not None else self._saved["empty"](0).device
        return dev.type in self.device_types

    @staticmethod
    def _shape(args: tuple) -> tuple:
        if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
            return tuple(args[0])
        return tuple(args)

    def __enter__(self) -> "GuardRegions":
        self._saved = {"empty": torch.empty, "zeros": torch.zeros, "empty_like": torch.empty_like, "zeros_like": torch.zeros_like}
        g = self

        def make(name: str, zero: bool):
            plain = g._saved[name]

            def fn(*args: Any, **kw: Any) -> torch.Tensor:
                if not g._wants(kw.get("device"), kw):
                    return plain(*args, **kw)
                return g._alloc(g._shape(args), kw.get("dtype") or torch.get_default_dtype(), torch.device(kw["device"])
                                if kw.get("device") is not None else g._saved["empty"](0).device, zero)
            return fn

        def make_like(name: str, zero: bool):
            plain = g._saved[name]

            def fn(t: torch.Tensor, **kw: Any) -> torch.Tensor:
                dev = kw.get("device", t.device)
                if not t.is_contiguous() or not g._wants(dev, kw):
                    return plain(t, **kw)
                return g._alloc(tuple(t.shape), kw.get("dtype") or t.dtype, torch.device(dev), zero)
            return fn
        torch.empty, torch.zeros = make("empty", False), make("zeros", True)
        torch.empty_like, torch.zeros_like = make_like("empty_like", False), make_like("zeros_like", True)
        return self

    def __exit__(self, *exc: Any) -> None:
        for name, fn in self._saved.items():
            setattr(torch, name, fn)

    # ------------------------------------------------------------------ checking
    def check(self) -> list[Violation]:
        """All damaged bands so far (synchronises the device).  The records stay, so a later check reports
        them again together with new ones."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out: list[Violation] = []
        for i, (raw, nbytes, shape, dtype, where) in enumerate(self.records):
            before = raw[:self.band]
            after = raw[self.band + nbytes:]                  # includes the rounding slack of the payload
            for side, band in (("before", before.flip(0)), ("after", after)):
                bad = (band != CANARY).nonzero()
                if bad.numel():
                    out.append(Violation(i, side, int(bad[0]), int(bad.numel()), shape, dtype, where))
        return out

    def assert_clean(self) -> None:
        v = self.check()
        if v:
            raise AssertionError("writes outside allocated tensors:\n  " + "\n  ".join(str(x) for x in v))
