"""The two ends of a model: token embedding into the residual stream, and the output head.

Embedding rows are multiplied by a scale (``scale_emb``, src/model/embedding.cuh:49-52);
the head multiplies the normed state by a scale (``dim_model_base / hidden_size``,
src/model/linear.cuh:86-104, cpmcu/llm.py:68) and returns fp32 logits.  A tied head uses
the embedding matrix itself; the reference copies it (cpmcu/llm.py:136-137).
"""
from __future__ import annotations

from typing import Dict, Optional, Type

import torch

from .base import Part, Registry, WeightSpec

EMBEDDINGS: Registry[Type[Part]] = Registry("embedding")
HEADS: Registry[Type[Part]] = Registry("output head")


@EMBEDDINGS.register("scaled_embedding")
class ScaledEmbedding(Part):
    recordable_prompt = True

    def __init__(self, ops, vocab_size: int, hidden_size: int, scale: float = 1.0, weight_name: str = "weight"):
        super().__init__(ops)
        self.vocab_size, self.hidden_size, self.scale = int(vocab_size), int(hidden_size), float(scale)
        self.weight_name = str(weight_name)      # the table's name below the part's prefix
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size))}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name]
        self.weight = self.ops.keep(w.contiguous()) if self.ops is not None else w

    def forward(self, token_ids: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.embed(token_ids, self.weight, self.scale)


@EMBEDDINGS.register("sinusoidal_scaled_embedding")
class SinusoidalScaledEmbedding(Part):
    """table[id] * scale plus a fixed sinusoidal position vector: entry 2i is sin(p * f_i), entry 2i+1 is
    cos(p * f_i), f_i = base^(-2i / hidden).  The frequencies are made once on the host in 32-bit; angles,
    sines and cosines are 32-bit on the device.  ``weight_name``: the table's name below the part's prefix."""

    recordable_prompt = True

    def __init__(self, ops, vocab_size: int, hidden_size: int, scale: float = 1.0, base: float = 10000.0,
                 weight_name: str = "weight"):
        super().__init__(ops)
        self.vocab_size, self.hidden_size, self.scale = int(vocab_size), int(hidden_size), float(scale)
        if self.hidden_size % 2:
            raise ValueError(f"sinusoidal positions need an even hidden size, got {self.hidden_size}")
        self.base, self.weight_name = float(base), str(weight_name)
        self.weight: Optional[torch.Tensor] = None
        i = torch.arange(self.hidden_size // 2, dtype=torch.float32)
        freq = torch.pow(torch.tensor(self.base, dtype=torch.float32), -2.0 * i / self.hidden_size)
        self.freq = freq.to(ops.device) if ops is not None else freq

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size))}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = self.ops.keep(tensors[self.weight_name].contiguous())

    def forward(self, token_ids: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        if positions is None:
            raise ValueError("sinusoidal_scaled_embedding needs the tokens' positions")
        return self.ops.embed_sinusoid(token_ids, positions, self.weight, self.freq, self.scale)


@HEADS.register("scaled_lm_head")
class ScaledHead(Part):
    recordable_prompt = True

    def __init__(self, ops, vocab_size: int, hidden_size: int, scale: float = 1.0, tied: bool = False,
                 weight_name: str = "weight"):
        super().__init__(ops)
        self.vocab_size, self.hidden_size, self.scale, self.tied = int(vocab_size), int(hidden_size), float(scale), bool(tied)
        self.weight_name = str(weight_name)      # the matrix's name below the part's prefix
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {} if self.tied else {self.weight_name: WeightSpec((self.vocab_size, self.hidden_size))}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = self.ops.keep(tensors[self.weight_name].contiguous())

    def tie(self, embedding_weight: torch.Tensor) -> None:
        self.weight = embedding_weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        """normed rows [n, hidden] -> fp32 logits [n, vocab]."""
        return self.ops.linear(y, self.weight, alpha=self.scale, out_f32=True, result=True)
