"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import BLOCKS, Block, CacheNeeds, ResidualStream, WeightSpec, NORMS, build_part, PartSpec


@BLOCKS.register("pre_norm_residual")
class PreNormResidualBlock(Block):
    """x += s * mixer(norm1(x)); x += s * feed_forward(norm2(x)), with one residual scale s.

    The reference scales each part's output by ``scale_depth / sqrt(layers)`` and adds
    it inside the next norm kernel (src/model/layer.cuh:47-67, src/model/norm.cuh:53-99).
    The scale is a parameter of the block; the block does not know where it comes from.
    """

    recordable_prompt = True

    def __init__(self, ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names,
                 residual_scale: float = 1.0):
        super().__init__(ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names)
        self.residual_scale = float(residual_scale)

    def forward(self, ctx, stream: ResidualStream, lane, writes_cache: bool) -> None:
        y = stream.normed(self.mixer_norm)
        a = self.mixer.forward(ctx, y, lane, writes_cache)
        stream.add(a, self.residual_scale)
        if self.feed_forward is None:
            return                                   # a layer of a mixer alone
        y2 = stream.normed(self.feed_forward_norm)
        f = self.feed_forward.forward(ctx, y2)
        stream.add(f, self.residual_scale)


@BLOCKS.register("sandwich_norm_shift")
class SandwichNormShiftBlock(Block):
    """x += post1(mixer(shift(pre1(x)))); x += post2(feed_forward(pre2(x))): a norm before and after each sublayer,
    and a token shift in front of the mixer.

    The shift blends what the mixer reads with the previous token's: h_t <- h_t + (h_{t-1} - h_t) * mix, element by
    element, h = pre1(x) as it was before the blend and zeros before a sequence's first token.  The previous h is
    per-sequence state of every run of the layer (``shift_prev`` [hidden], 32-bit).  The norms after the sublayers
    (``post_mixer_norm``, ``post_feed_forward_norm``) are parts of this block; their tensors are named by
    ``names["post_mixer_norm"]`` and ``names["post_feed_forward_norm"]``, the blend's vector by ``names["shift"]``.
    The residual sum, the norms and the blend are 32-bit; a sublayer's output is added in the kernel that norms it,
    and where a feed-forward follows, that kernel also forms the feed-forward's input.
    """

    recordable_prompt = True

    def __init__(self, ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names, hidden_size: int,
                 post_norm: PartSpec = None):
        super().__init__(ops, mixer, feed_forward, mixer_norm, feed_forward_norm, names)
        self.hidden_size = int(hidden_size)
        if post_norm is None:
            raise ValueError("sandwich_norm_shift needs the specification of its norms after the sublayers")
        self.post_mixer_norm = build_part(NORMS, post_norm, ops)
        self.post_feed_forward_norm = build_part(NORMS, post_norm, ops) if feed_forward is not None else None
        for n in (mixer_norm, feed_forward_norm, self.post_mixer_norm, self.post_feed_forward_norm):
            if n is not None and not (hasattr(n, "shift_forward") and hasattr(n, "add_normed")):
                raise ValueError("sandwich_norm_shift needs norms that offer shift_forward and add_normed (layer_norm)")
        self.mix: Optional[torch.Tensor] = None

    def sub_parts(self):
        parts = super().sub_parts()
        parts.append((self.names.get("post_mixer_norm", "post_mixer_norm."), self.post_mixer_norm))
        if self.post_feed_forward_norm is not None:
            parts.append((self.names.get("post_feed_forward_norm", "post_feed_forward_norm."), self.post_feed_forward_norm))
        return parts

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out = super().weight_specs()
        out[self.names.get("shift", "shift")] = WeightSpec((self.hidden_size,), "vector")
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().load_weights(tensors)
        self.mix = self.ops.keep(tensors[self.names.get("shift", "shift")].float().contiguous())

    def weight_bytes(self) -> int:
        return super().weight_bytes() + 4 * self.hidden_size

    def cache_needs(self) -> CacheNeeds:
        return self.mixer.cache_needs().with_state({"shift_prev": ((self.hidden_size,), torch.float32)})

    def forward(self, ctx, stream: ResidualStream, lane, writes_cache: bool) -> None:
        x = stream.flush()
        h = self.mixer_norm.shift_forward(ctx, x, self.mix, lane.state["shift_prev"])
        a = self.mixer.forward(ctx, h, lane, writes_cache)
        if self.feed_forward is None:
            self.post_mixer_norm.add_normed(x, a)
            return
        y = self.post_mixer_norm.add_normed(x, a, then=self.feed_forward_norm)
        f = self.feed_forward.forward(ctx, y)
        self.post_feed_forward_norm.add_normed(x, f)
