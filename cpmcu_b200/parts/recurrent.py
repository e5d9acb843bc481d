"""Recurrent mixers: a state of fixed size per sequence instead of cached keys."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MIXERS, CacheNeeds, Mixer, WeightSpec


@MIXERS.register("min_gru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token:

        z = sigmoid(Wz h + bz),  u = Wx h + bx,  g(u) = u + 1/2 where u >= 0, sigmoid(u) where u < 0
        S_t = (1 - z) S_{t-1} + z g(u)            (element by element, ``width`` channels)
        out = Wo (S_t * silu(Wg h))

    One product gives Wz h, Wx h and Wg h (32-bit results); the gates, the state and the recurrence are 32-bit.
    The state starts at zero and is per-sequence state of the lane (``gru_state`` [width], 32-bit).  ``names``:
    the tensors' names below the part's prefix, by "z", "z_bias", "x", "x_bias", "g", "o".
    """

    recordable_prompt = True

    DEFAULT_NAMES = {"z": "z.weight", "z_bias": "z.bias", "x": "x.weight", "x_bias": "x.bias", "g": "g.weight", "o": "o.weight"}

    def __init__(self, ops, hidden_size: int, width: int, names=None):
        super().__init__(ops)
        self.hidden_size, self.width = int(hidden_size), int(width)
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))
        self.w_zxg: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_z: Optional[torch.Tensor] = None
        self.b_x: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, w, h = self.names, self.width, self.hidden_size
        return {n["z"]: WeightSpec((w, h)), n["z_bias"]: WeightSpec((w,), "vector"), n["x"]: WeightSpec((w, h)),
                n["x_bias"]: WeightSpec((w,), "vector"), n["g"]: WeightSpec((w, h)), n["o"]: WeightSpec((h, w))}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_zxg = self.ops.keep(torch.cat([tensors[n["z"]], tensors[n["x"]], tensors[n["g"]]], dim=0).contiguous())
        self.w_o = self.ops.keep(tensors[n["o"]].contiguous())
        self.b_z = self.ops.keep(tensors[n["z_bias"]].float().contiguous())
        self.b_x = self.ops.keep(tensors[n["x_bias"]].float().contiguous())

    def weight_bytes(self) -> int:
        return (self.w_zxg.numel() + self.w_o.numel()) * self.w_zxg.element_size() + 8 * self.width

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state={"gru_state": ((self.width,), torch.float32)})

    def cache_bytes_read(self, kv_len: int) -> int:
        return 4 * self.width

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops = self.ops
        proj = ops.linear(y, self.w_zxg, out_f32=True)
        gated = ops.mingru_scan(ctx, proj, self.b_z, self.b_x, lane.state["gru_state"], self.width)
        return ops.linear(gated, self.w_o)
