"""Canary regions around device buffers (``csrc/guard.cu``).

``CanaryArena.tensor(shape, dtype)`` hands out a tensor whose storage sits between two guard bands filled with a
position-dependent pattern; ``check()`` scans every band on the device and names the first damaged one.  Kernel tests
allocate their outputs (and inputs) here, so a store past a ragged edge fails the test even when the values inside
the tensor are right.  Reference: the guardrail layer's debug snapshot kernels (native unit N32 there).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import native
from ..ops.kernels import _stream

PATTERN = 0xC0FFEE5A


@dataclass
class CanaryDamage:
    band: int                 # 2 * i = the band before tensor i, 2 * i + 1 = the band after it
    name: str
    first_byte: int           # offset of the first damaged word inside the band
    damaged_words: int

    def __str__(self) -> str:
        side = "after" if self.band & 1 else "before"
        return f"{self.damaged_words} words damaged, first in the band {side} {self.name!r} at byte {self.first_byte}"


class CanaryArena:
    def __init__(self, device, band_bytes: int = 4096) -> None:
        if band_bytes % 256:
            raise ValueError("guard bands are multiples of 256 bytes (tensors stay 256-byte aligned)")
        self.device = torch.device(device)
        self.band = band_bytes
        self._blocks: list[tuple[str, torch.Tensor, int]] = []       # name, raw uint8 storage, offset of the band after
        self._report = torch.zeros(3, dtype=torch.int64, device=self.device)

    def tensor(self, shape, dtype, name: str | None = None) -> torch.Tensor:
        """An uninitialised tensor between two guard bands."""
        n = 1
        for s in shape:
            n *= int(s)
        payload = n * torch.empty((), dtype=dtype).element_size()
        padded = -(-payload // 256) * 256
        raw = torch.empty(self.band + padded + self.band, dtype=torch.uint8, device=self.device)
        lib = native.lib()
        native.check(lib.cb_canary_fill(raw.data_ptr(), self.band, PATTERN, _stream()), "cb_canary_fill")
        # the band after the tensor starts at the first whole word behind the payload: the alignment slack is guarded too
        after = self.band + -(-payload // 4) * 4
        native.check(lib.cb_canary_fill(raw.data_ptr() + after, raw.numel() - after, PATTERN, _stream()), "cb_canary_fill")
        self._blocks.append((name or f"tensor{len(self._blocks)}", raw, after))
        return raw[self.band:self.band + payload].view(dtype).view(*shape)

    def check(self) -> CanaryDamage | None:
        """Scan all bands; returns the first damaged one (lowest band index) or None."""
        lib = native.lib()
        self._report.zero_()
        self._report[1] = -1                                           # all ones: the minimum of nothing
        for i, (_, raw, after) in enumerate(self._blocks):
            native.check(lib.cb_canary_check(raw.data_ptr(), self.band, PATTERN, 2 * i, self._report.data_ptr(), _stream()),
                         "cb_canary_check")
            native.check(lib.cb_canary_check(raw.data_ptr() + after, raw.numel() - after, PATTERN, 2 * i + 1,
                                             self._report.data_ptr(), _stream()), "cb_canary_check")
        bad, key, _ = (int(v) for v in self._report.cpu())
        if not bad:
            return None
        key &= (1 << 64) - 1
        band, word = key >> 40, key & ((1 << 40) - 1)
        return CanaryDamage(band, self._blocks[band // 2][0], word * 4, bad)
