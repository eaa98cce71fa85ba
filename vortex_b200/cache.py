"""Inference-cache containers with the reference's names, fields and layout
(``vortex/model/cache.py:12-61``).  The engine reads and writes exactly these
dictionaries, keyed by layer index:

* ``fir_state_dict[layer]``        [B, 3D, K3-1]  last featurizer inputs, packed-channel order
* ``fir_inner_state_dict[layer]``  [B, D, K-1]    last k*v samples, oldest first (FIR layers)
* ``state_dict[layer]``            [B, D, S] fp32 modal state, residues not applied (long layers)

Prefill writes the FIR caches in the activation dtype; every decode step returns them in fp32
(``vortex/model/engine.py:427-449``).
"""
from dataclasses import dataclass, field
from typing import Optional

from torch import Tensor


@dataclass
class InferenceParams:
    """Attention KV-cache bookkeeping (kept for interface parity; not touched by the Hyena engine)."""

    max_seqlen: int
    max_batch_size: int
    seqlen_offset: int = 0
    batch_size_offset: int = 0
    key_value_memory_dict: dict = field(default_factory=dict)
    lengths_per_sample: Optional[Tensor] = None

    def reset(self, max_seqlen, max_batch_size):
        self.max_seqlen, self.max_batch_size, self.seqlen_offset = max_seqlen, max_batch_size, 0
        if self.lengths_per_sample is not None:
            self.lengths_per_sample.zero_()


@dataclass
class HyenaCascadeIIRInferenceParams:
    """Caches of the long (modal IIR) Hyena layers."""

    fir_filter_length: int = 3
    state_dim: int = 16
    seqlen_offset: int = 0
    fir_state_dict: dict = field(default_factory=dict)
    state_dict: dict = field(default_factory=dict)

    def reset(self):
        self.fir_filter_length, self.state_dim, self.seqlen_offset = 3, 16, 0


@dataclass
class HyenaCascadeFIRInferenceParams:
    """Caches of the short and medium (explicit FIR) Hyena layers."""

    fir_filter_length: int = 3
    fir_inner_filter_length: int = 4
    seqlen_offset: int = 0
    fir_inner_state_dict: dict = field(default_factory=dict)
    fir_state_dict: dict = field(default_factory=dict)
    state_dict: dict = field(default_factory=dict)

    def reset(self):
        self.fir_filter_length, self.fir_inner_filter_length, self.seqlen_offset = 3, 4, 0
