"""Two mixers side by side on the same input."""
from __future__ import annotations

from typing import Dict

import torch

from .base import MIXERS, CacheNeeds, Mixer, PartSpec, WeightSpec, build_part


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    """out = ( rms_norm(left(h)) * w_left + rms_norm(right(h)) * w_right ) / 2, the norms over the model width with plain
    weights.  ``left`` and ``right`` are mixers of any registered kind; their tensors lie under ``names["left"]`` and
    ``names["right"]``, the two norm weights under ``names["left_out"]`` and ``names["right_out"]``.  The lane holds what
    both need: at most one of them may cache keys, and their per-sequence state must not share names."""

    DEFAULT_NAMES = {"left": "left.", "right": "right.", "left_out": "left.out", "right_out": "right.out"}

    @property
    def recordable_prompt(self) -> bool:
        return bool(self.left.recordable_prompt) and bool(self.right.recordable_prompt)

    def __init__(self, ops, hidden_size: int, left: PartSpec, right: PartSpec, eps: float, names=None):
        super().__init__(ops)
        self.hidden_size, self.eps = int(hidden_size), float(eps)
        self.left, self.right = build_part(MIXERS, left, ops), build_part(MIXERS, right, ops)
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))

    def _sides(self):
        return ((self.names["left"], self.left), (self.names["right"], self.right))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out = {self.names["left_out"]: WeightSpec((self.hidden_size,), "vector"),
               self.names["right_out"]: WeightSpec((self.hidden_size,), "vector")}
        for prefix, part in self._sides():
            for name, spec in part.weight_specs().items():
                out[prefix + name] = spec
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._sides():
            part.load_weights({n: tensors[prefix + n] for n in part.weight_specs()})
        self.w_left = self.ops.keep(tensors[self.names["left_out"]].float().contiguous())
        self.w_right = self.ops.keep(tensors[self.names["right_out"]].float().contiguous())

    def weight_bytes(self) -> int:
        return self.left.weight_bytes() + self.right.weight_bytes() + 8 * self.hidden_size

    def cache_needs(self) -> CacheNeeds:
        a, b = self.left.cache_needs(), self.right.cache_needs()
        if a.kv_heads and b.kv_heads:
            raise ValueError("parallel_mixers: only one of the two mixers may keep keys in the cache")
        keyed, other = (a, b) if a.kv_heads or not b.kv_heads else (b, a)
        return keyed.with_state(other.state)

    def cache_bytes_read(self, kv_len: int) -> int:
        return self.left.cache_bytes_read(kv_len) + self.right.cache_bytes_read(kv_len)

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        a = self.left.forward(ctx, y, lane, writes_cache)
        b = self.right.forward(ctx, y, lane, writes_cache)
        return self.ops.dual_rmsnorm_mean(a, b, self.w_left, self.w_right, self.eps)
