"""What happens to the residual stream where a pass through a repeated group of layers begins."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import PASS_ENTRIES, PassEntry, ResidualStream, WeightSpec


@PASS_ENTRIES.register("reinject_with_step")
class ReinjectWithStep(PassEntry):
    """Before every pass but the first, the stream takes the embedding's output once more; before every pass, the
    first too, it takes the pass's own learned vector (row ``number`` of a table [passes, hidden]).  Both additions
    are 32-bit and one kernel."""

    recordable_prompt = True

    def __init__(self, ops, passes: int, hidden_size: int, table_name: str = "step"):
        super().__init__(ops)
        self.passes, self.hidden_size, self.table_name = int(passes), int(hidden_size), str(table_name)
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.table_name: WeightSpec((self.passes, self.hidden_size), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = self.ops.keep(tensors[self.table_name].float().contiguous())

    def weight_bytes(self) -> int:
        return 4 * self.passes * self.hidden_size

    def forward(self, ctx, stream: ResidualStream, number: int, embedded: torch.Tensor) -> None:
        if not 0 <= number < self.passes:
            raise ValueError(f"pass {number} of {self.passes}")
        self.ops.stream_inject(stream.flush(), embedded if number > 0 else None, self.table[number])
