"""The expert pool file of a Q4 package, as the reference writes and maps it.

Layout (reference tools/gemma4-mlx4-source.py:1795-1798 writes it, models/gemma4-26b-a4b/src/gemma4_text.c:
1594-1615 and 1765-1780 map it): a 24-byte header ``<QQQ`` = (slot_bytes, layers, experts_per_layer), then
``layers * experts`` slots of ``slot_bytes`` in [layer][expert] order.  A slot is gate | up | down, each
projection being values | scales | biases (tools/gemma4-mlx4-source.py:180-199), which is exactly the
per-expert stride of ``synth.Q4MoeLayer.pool``.  Slots start at 24 + i * slot_bytes, i.e. 8 modulo 16 in the
mapping: a payload used in place is "unaligned" for 16-byte loads, while a payload populated into a
residency seat is 256-byte aligned.
"""
from __future__ import annotations

import mmap
import os
import struct

import numpy as np

from .synth import q4_tensor_bytes

POOL_HEADER = 24


def write_pool(path: str, layers) -> int:
    """Write the experts of ``layers`` (``Q4MoeLayer``, same geometry) as one pool file; returns slot_bytes."""
    slot, experts = layers[0].expert_stride, layers[0].n_experts
    for layer in layers:
        if layer.expert_stride != slot or layer.n_experts != experts or layer.pool.nbytes != slot * experts:
            raise ValueError("layers of one pool share slot_bytes and experts_per_layer")
    with open(path, "wb") as f:
        f.write(struct.pack("<QQQ", slot, len(layers), experts))
        for layer in layers:
            f.write(layer.pool.tobytes())
    return slot


class ExpertPool:
    """Read-only mapping of a pool file; every accessor returns views into the mapping (no copies)."""

    def __init__(self, path: str, hidden: int, inter: int):
        self.hidden, self.inter = hidden, inter
        self._fd = os.open(path, os.O_RDONLY)
        try:
            size = os.fstat(self._fd).st_size
            if size < POOL_HEADER:
                raise ValueError("pool file shorter than its header")
            self._map = mmap.mmap(self._fd, size, access=mmap.ACCESS_READ)
        except Exception:
            os.close(self._fd)
            raise
        self.slot_bytes, self.layers, self.experts = struct.unpack_from("<QQQ", self._map, 0)
        vb, gb = q4_tensor_bytes(inter, hidden)
        self._tensor_bytes = vb + 2 * gb
        if (self.slot_bytes != 3 * self._tensor_bytes or self.layers < 1 or self.experts < 1 or
                size != POOL_HEADER + self.slot_bytes * self.layers * self.experts):
            self.close()
            raise ValueError("pool header does not describe this file (slot_bytes, layers, experts, size)")
        self.bytes = np.frombuffer(self._map, np.uint8)

    def logical_id(self, layer: int, expert: int) -> int:
        """layer * experts + expert (reference gemma4_text.c:1909)."""
        return layer * self.experts + expert

    def payload(self, layer: int, expert: int) -> np.ndarray:
        off = POOL_HEADER + self.logical_id(layer, expert) * self.slot_bytes
        return self.bytes[off:off + self.slot_bytes]

    def tensor(self, layer: int, expert: int, which: int):
        """(values, scales, biases) of gate (0), up (1) or down (2): uint8 views, 8 modulo 16 aligned."""
        vb, gb = q4_tensor_bytes(self.inter, self.hidden)
        p = self.payload(layer, expert)[which * self._tensor_bytes:(which + 1) * self._tensor_bytes]
        return p[:vb], p[vb:vb + gb], p[vb + gb:vb + 2 * gb]

    def close(self):
        self.bytes = None
        try:
            self._map.close()
        except BufferError:      # a caller still holds a view: the mapping goes when the view does
            pass
        finally:
            os.close(self._fd)
