"""Guard zones around device allocations: a stand-in for a memory checker on machines where none can be run.

Inside `with GuardedAllocations() as g:` every CUDA tensor created through `torch.empty`, `torch.empty_like`,
`torch.zeros` or `torch.zeros_like` is carved out of a larger buffer with a guard zone of a known byte pattern on
both sides (data start stays 256-byte aligned). The kernels under test then write their outputs into such tensors;
`g.check()` (also run on leaving the block) verifies that no guard byte changed, i.e. that nothing wrote just below
or just above any output, and reports the first tensor whose guard was damaged with the offset of the damage.
Reads past a buffer are not detected; an out-of-range *write* within a few KB of a buffer is.
"""

from __future__ import annotations

import math

import torch

GUARD_BYTES = 4096
PATTERN = 0xA5


class GuardViolation(AssertionError):
    pass


class GuardedAllocations:
    def __init__(self, guard_bytes: int = GUARD_BYTES) -> None:
        if guard_bytes % 256:
            raise ValueError("the guard size must keep 256-byte alignment")
        self.guard = guard_bytes
        self.records: list[tuple[torch.Tensor, int, tuple, torch.dtype]] = []
        self._orig: dict = {}

    # ---- allocation ------------------------------------------------------------------------------
    def _carve(self, shape, dtype, device, zero: bool) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        padded = -(-nbytes // 256) * 256
        base = self._orig["empty"](padded + 2 * self.guard, dtype=torch.uint8, device=device)
        base.fill_(PATTERN)
        body = base[self.guard : self.guard + nbytes]
        if zero:
            body.zero_()
        self.records.append((base, nbytes, shape, dtype))
        return body.view(dtype).view(shape)

    @staticmethod
    def _is_cuda(device) -> bool:
        return device is not None and torch.device(device).type == "cuda"

    def _wrap(self, name: str, zero: bool):
        orig = self._orig[name]

        def alloc(*size, dtype=None, device=None, **kw):
            plain = not kw or set(kw) <= {"requires_grad", "pin_memory"} and not kw.get("pin_memory")
            if self._is_cuda(device) and plain:
                shape = size[0] if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)) else size
                return self._carve(shape, dtype or torch.get_default_dtype(), device, zero)
            return orig(*size, dtype=dtype, device=device, **kw)

        return alloc

    def _wrap_like(self, name: str, zero: bool):
        orig = self._orig[name]

        def alloc_like(t, dtype=None, device=None, **kw):
            dev = device if device is not None else t.device
            if self._is_cuda(dev) and not kw and t.is_contiguous():
                return self._carve(t.shape, dtype or t.dtype, dev, zero)
            return orig(t, dtype=dtype, device=device, **kw)

        return alloc_like

    def __enter__(self) -> "GuardedAllocations":
        for name in ("empty", "zeros", "empty_like", "zeros_like"):
            self._orig[name] = getattr(torch, name)
        torch.empty, torch.zeros = self._wrap("empty", False), self._wrap("zeros", True)
        torch.empty_like, torch.zeros_like = self._wrap_like("empty_like", False), self._wrap_like("zeros_like", True)
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        for name, fn in self._orig.items():
            setattr(torch, name, fn)
        if exc_type is None:
            self.check()
        return False

    # ---- verification ---------------------------------------------------------------------------
    def check(self) -> int:
        """Raises `GuardViolation` for the first damaged guard; returns the number of tensors checked."""
        if self.records:
            torch.cuda.synchronize()
        for i, (base, nbytes, shape, dtype) in enumerate(self.records):
            lo, hi = base[: self.guard], base[self.guard + nbytes :]
            for side, zone in (("below", lo), ("above", hi)):
                bad = (zone != PATTERN).nonzero()
                if bad.numel():
                    off = int(bad[0])
                    where = off - self.guard if side == "below" else nbytes + off
                    raise GuardViolation(f"allocation #{i} {shape} {dtype}: a byte {side} the tensor changed "
                                         f"(offset {where} from its start, {bad.numel()} bytes in all)")  # fmt: skip
        return len(self.records)
