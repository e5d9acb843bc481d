"""Softmax attention over the paged cache whose weights are mixed across heads after the softmax."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MIXERS, POSITIONS, CacheNeeds, Mixer, PartSpec, WeightSpec, build_part


@MIXERS.register("talking_heads_attention")
class TalkingHeadsAttention(Mixer):
    """Causal grouped-query attention with a temperature per head and a mix of the heads' softmax weights:

        s_g(i, j) = q_g(i) . k_kv(g)(j) * scale * temp[g],   p_g = softmax_j s_g,   w_h = sum_g talk[h][g] p_g
        o_h(i) = sum_j w_h(i, j) v_kv(h)(j),   out = Wo [o_0 | o_1 | ...]

    Queries and keys have ``head_dim`` channels, values ``value_dim``; ``position`` is a rotation of pairs (or "none")
    applied to q and k before keys are cached.  Keys and values live in the paged cache in the compute dtype; scores,
    weights and sums are 32-bit.  ``names``: "q", "k", "v", "o", "temp", "talk".
    """

    DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "temp": "temp", "talk": "talk"}

    @property
    def recordable_prompt(self) -> bool:
        return bool(self.position.recordable_prompt)

    def __init__(self, ops, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int,
                 softmax_scale: float, position: PartSpec, names=None):
        super().__init__(ops)
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot be grouped over {n_kv_heads} key-value heads")
        if n_heads > 128 or value_dim > 256:
            raise ValueError("talking_heads_attention: the kernel takes up to 128 heads and value heads of up to 256 channels")
        self.hidden_size, self.n_heads, self.n_kv = int(hidden_size), int(n_heads), int(n_kv_heads)
        self.d, self.dv, self.scale = int(head_dim), int(value_dim), float(softmax_scale)
        self.position = build_part(POSITIONS, position, ops)
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W, H, G, d, dv = self.names, self.hidden_size, self.n_heads, self.n_kv, self.d, self.dv
        return {n["q"]: WeightSpec((H * d, W)), n["k"]: WeightSpec((G * d, W)), n["v"]: WeightSpec((G * dv, W)),
                n["o"]: WeightSpec((W, H * dv)), n["temp"]: WeightSpec((H,), "vector"), n["talk"]: WeightSpec((H, H), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_qkv = self.ops.keep(torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous())
        self.w_o = self.ops.keep(tensors[n["o"]].contiguous())
        self.temp = self.ops.keep(tensors[n["temp"]].float().contiguous())
        self.talk = self.ops.keep(tensors[n["talk"]].float().contiguous())

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size() + 4 * (self.temp.numel() + self.talk.numel())

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(kv_heads=self.n_kv, head_dim=self.d, value_dim=self.dv if self.dv != self.d else 0)

    def cache_bytes_read(self, kv_len: int) -> int:
        return kv_len * self.n_kv * (self.d + self.dv) * self.ops.element_size

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops = self.ops
        if lane.k is not None:
            ops.set_page_limit(lane.k.shape[0])
        qkv = ops.linear(y, self.w_qkv)
        rot = self.position.rotary()
        if rot is None:
            raise ValueError("talking_heads_attention takes a rotation of pairs or no position encoding")
        inv_freq, magnitude, rot_dim = rot
        if magnitude != 1.0:
            raise ValueError("talking_heads_attention: a rotation with a magnitude factor is not built")
        q = ops.rope_store_dv(ctx, qkv, lane, self.n_heads, self.n_kv, self.d, self.dv, inv_freq if rot_dim else None,
                              rot_dim, writes_cache)
        out = ops.talking_attention(ctx, q, lane, self.n_kv, self.dv, self.scale, self.temp, self.talk)
        return ops.linear(out, self.w_o)
