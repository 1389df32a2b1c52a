"""Flat-buffer layout for ZeRO-1 style partitioning of the Lion step.

All parameters of the optimizer live back to back in one flat buffer, each starting on a
16-byte boundary, and the buffer is padded so that every rank owns an equal, 16-byte aligned
slice.  Because the Lion update is element-wise, a rank's slice may cut through tensors.
Pure arithmetic, no device code: used by the optimizer and tested on CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

ALIGN_ELEMS = 8  # 16 bytes of a 16-bit type; also keeps fp32 tensors 32-byte aligned


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass(frozen=True)
class FlatLayout:
    offsets: Tuple[int, ...]   # start element of each tensor in the flat buffer
    numels: Tuple[int, ...]
    total: int                 # padded length, a multiple of world_size * ALIGN_ELEMS
    world_size: int

    @staticmethod
    def build(numels: Sequence[int], world_size: int) -> "FlatLayout":
        if world_size < 1:
            raise ValueError("world_size must be >= 1")
        offsets: List[int] = []
        cursor = 0
        for n in numels:
            if n < 0:
                raise ValueError("negative numel")
            offsets.append(cursor)
            cursor = _round_up(cursor + n, ALIGN_ELEMS)
        total = _round_up(max(cursor, 1), world_size * ALIGN_ELEMS)
        return FlatLayout(tuple(offsets), tuple(int(n) for n in numels), total, world_size)

    @property
    def shard_size(self) -> int:
        return self.total // self.world_size

    def shard_range(self, rank: int) -> Tuple[int, int]:
        if not 0 <= rank < self.world_size:
            raise ValueError(f"rank {rank} outside [0, {self.world_size})")
        return rank * self.shard_size, (rank + 1) * self.shard_size

    def tensor_slice_in_shard(self, index: int, rank: int) -> Tuple[int, int, int]:
        """Overlap of tensor `index` with rank's shard.

        Returns (start_in_tensor, start_in_shard, length); length 0 when they do not meet.
        """
        b, e = self.shard_range(rank)
        t0, t1 = self.offsets[index], self.offsets[index] + self.numels[index]
        lo, hi = max(b, t0), min(e, t1)
        if hi <= lo:
            return 0, 0, 0
        return lo - t0, lo - b, hi - lo
