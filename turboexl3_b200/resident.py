"""The resident trunk: a host's opt-in to spend memory on compute.

Mirrors the reference's table (src/core/dense.zig:1323-1530): the host arms it with the trunk trellises it admits
(`residentArm`); the first call past 32 rows on an admitted trellis decodes W_hat once and keeps it (`dequantize`); every
later such call runs a plain tensor-core GEMM on the kept weight; decode rows never touch it; `release` drops every kept
weight (`residentRelease`); `pending` is what is admitted but not kept yet (`residentPending`), which the host bills
against its memory ceiling; `keeps` / `stats` report (`residentKeeps`, `residentStats`). As in the reference a kept weight
is the per-call one bit for bit, and so is every output.
"""
from __future__ import annotations

import torch

from . import api


class ResidentTable:
    def __init__(self):
        self._admitted = {}  # trellis data_ptr -> bytes the kept weight takes
        self._kept = {}      # trellis data_ptr -> (trellis kept alive, W_hat transposed)

    @staticmethod
    def bytes_of(trellis: torch.Tensor) -> int:
        """dense.residentBytesOf (src/core/dense.zig:1342-1345): 2 bytes a weight; 0 for any other shape."""
        if trellis.dim() != 3 or trellis.shape[0] <= 0 or trellis.shape[1] <= 0:
            return 0
        return int(trellis.shape[0]) * 16 * int(trellis.shape[1]) * 16 * 2

    def arm(self, trellises) -> None:
        for t in trellises:
            b = self.bytes_of(t)
            if b:
                self._admitted[t.data_ptr()] = b

    def release(self) -> None:
        self._kept.clear()
        self._admitted.clear()

    def keeps(self, trellis: torch.Tensor) -> bool:
        return trellis.data_ptr() in self._kept

    def pending(self) -> int:
        return sum(b for p, b in self._admitted.items() if p not in self._kept)

    def stats(self) -> dict:
        return {"admitted": len(self._admitted), "kept": len(self._kept),
                "kept_bytes": sum(self._admitted[p] for p in self._kept)}

    def linear(self, x: torch.Tensor, trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor,
               dec: api.Decode = api.Decode.mul1) -> torch.Tensor:
        """root.linear with the table armed: admitted trellises past 32 rows take the kept weight."""
        rows = x.numel() // x.shape[-1]
        key = trellis.data_ptr()
        if rows <= api.DECODE_ROWS_MAX or key not in self._admitted:
            return api.linear(x, trellis, suh, svh, dec)
        if key not in self._kept:
            self._kept[key] = (trellis, api.resident_build(trellis, dec))
        return api.linear_resident(x, self._kept[key][1], suh, svh)
