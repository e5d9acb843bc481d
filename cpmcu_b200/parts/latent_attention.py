"""Attention whose keys and values are linear maps of one cached latent per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MIXERS, CacheNeeds, Mixer, WeightSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Queries go through a latent, c_q = rms(Wdq h) * g_q and q = Wuq c_q; keys and values come from a second latent,
    c = rms(Wdkv h) * g_kv (``kv_rank`` values), as k = Wuk c and v = Wuv c, head by head.  No position enters.
    score = (q . k) * scale; a query at position i sees the keys j with 0 <= i - j < window (window None: all
    j <= i); softmax; the heads' outputs go through Wo.

    Only c is cached: one row of ``kv_rank`` values per token, whatever the number of heads.  The attention runs on
    the cached latents themselves, with Wuk moved to the query side (q'_h = Wuk_h^T q_h, so q'_h . c = q_h . k_h) and
    Wuv applied to the weighted sum of latents (Wuv_h sum_j p_j c_j = sum_j p_j v_j): the same arithmetic serves a
    prompt, a portion of one and a single decoded token, and nothing is decompressed.  Norms, scores, softmax and the
    weighted sum are 32-bit, and so are q' and the weighted latents between the kernels.  ``names``: the tensors'
    names below the part's prefix, by "dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "o".
    """

    recordable_prompt = True

    DEFAULT_NAMES = {"dq": "dq.weight", "dq_norm": "dq_norm.weight", "uq": "uq.weight", "dkv": "dkv.weight",
                     "dkv_norm": "dkv_norm.weight", "uk": "uk.weight", "uv": "uv.weight", "o": "o.weight"}

    def __init__(self, ops, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, q_rank: int, kv_rank: int,
                 softmax_scale: float, eps: float, window: Optional[int] = None, names=None):
        super().__init__(ops)
        self.hidden_size, self.n_heads, self.d, self.vd = int(hidden_size), int(n_heads), int(head_dim), int(value_dim)
        self.q_rank, self.kv_rank = int(q_rank), int(kv_rank)
        self.scale, self.eps = float(softmax_scale), float(eps)
        self.window = int(window) if window else 0
        if self.kv_rank > 1024:
            raise ValueError(f"latent_attention: kv_rank {self.kv_rank} is beyond the 1,024 the attention kernels keep per head")
        self.names = dict(self.DEFAULT_NAMES, **(dict(names) if names else {}))
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.g_q = self.g_kv = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, H, h = self.names, self.n_heads, self.hidden_size
        return {n["dq"]: WeightSpec((self.q_rank, h)), n["dq_norm"]: WeightSpec((self.q_rank,), "vector"),
                n["uq"]: WeightSpec((H * self.d, self.q_rank)), n["dkv"]: WeightSpec((self.kv_rank, h)),
                n["dkv_norm"]: WeightSpec((self.kv_rank,), "vector"), n["uk"]: WeightSpec((H * self.d, self.kv_rank)),
                n["uv"]: WeightSpec((H * self.vd, self.kv_rank)), n["o"]: WeightSpec((h, H * self.vd))}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        n, H, keep = self.names, self.n_heads, self.ops.keep
        self.w_down = keep(torch.cat([tensors[n["dq"]], tensors[n["dkv"]]], dim=0).contiguous())      # one product for both latents
        self.w_uq = keep(tensors[n["uq"]].contiguous())
        # per head [k][n] matrices for in[t, h, :] @ w[h]: Wuk_h is [dim, rank] as stored; Wuv_h [vdim, rank] is transposed
        self.w_uk = keep(tensors[n["uk"]].view(H, self.d, self.kv_rank).contiguous())
        self.w_uv = keep(tensors[n["uv"]].view(H, self.vd, self.kv_rank).transpose(1, 2).contiguous())
        self.w_o = keep(tensors[n["o"]].contiguous())
        self.g_q = keep(tensors[n["dq_norm"]].float().contiguous())
        self.g_kv = keep(tensors[n["dkv_norm"]].float().contiguous())

    def weight_bytes(self) -> int:
        mats = (self.w_down, self.w_uq, self.w_uk, self.w_uv, self.w_o)
        return sum(m.numel() for m in mats) * self.w_o.element_size() + 4 * (self.q_rank + self.kv_rank)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(kv_heads=1, head_dim=self.kv_rank, window=self.window or None, values=False)

    def cache_bytes_read(self, kv_len: int) -> int:
        keys = min(kv_len, self.window) if self.window else kv_len
        return keys * self.kv_rank * self.ops.element_size

    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops = self.ops
        ops.set_page_limit(lane.k.shape[0])
        down = ops.linear(y, self.w_down, out_f32=True)                                  # [tokens, q_rank + kv_rank], 32-bit
        c_q = ops.latent_norm_store(ctx, down, self.g_q, self.g_kv, lane, self.q_rank, self.kv_rank, self.eps, writes_cache)
        q = ops.linear(c_q, self.w_uq)                                                   # [tokens, heads * dim]
        q_lat = ops.head_project(q, self.w_uk, self.n_heads, out_f32=True)               # [tokens, heads, kv_rank], 32-bit
        # [tokens, heads, kv_rank]: 32-bit, unless the map that follows is a library product of many tokens, which takes bf16
        narrow = ops.head_project_by_library(ctx.n_tokens) and ops.latent_attention_on_tensor_cores(self.kv_rank)
        o_lat = ops.latent_attention(ctx, q_lat, lane, self.scale, self.window, out_compute_dtype=narrow)
        o = ops.head_project(o_lat, self.w_uv, self.n_heads, out_f32=False)              # [tokens, heads * vdim]
        return ops.linear(o.view(ctx.n_tokens, self.n_heads * self.vd), self.w_o)
