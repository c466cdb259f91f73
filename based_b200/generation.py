"""Inference-time state container shared by the mixers.

Field-for-field mirror of ``InferenceParams`` in the reference (based/generation.py:18-35):
the mixers only read ``seqlen_offset``, ``max_seqlen``, ``max_batch_size``,
``batch_size_offset``, ``lengths_per_sample`` and store their per-layer state in
``key_value_memory_dict[layer_idx]``.  The reference's own class (or any object with these
attributes) can be passed instead; the mixers never check the type.
"""
from dataclasses import dataclass, field
from typing import Optional

from torch import Tensor


@dataclass
class InferenceParams:
    max_seqlen: int
    max_batch_size: int
    seqlen_offset: int = 0
    batch_size_offset: int = 0
    key_value_memory_dict: dict = field(default_factory=dict)
    lengths_per_sample: Optional[Tensor] = None

    def reset(self, max_seqlen, max_batch_size):
        self.max_seqlen = max_seqlen
        self.max_batch_size = max_batch_size
        self.seqlen_offset = 0
        if self.lengths_per_sample is not None:
            self.lengths_per_sample.zero_()
