"""What a mixer reads instead of the normed rows themselves.

``token_shift``: a learned blend, per channel, of a token's row with the row of the token before it,
``x_t + (x_(t-1) - x_t) * mix`` with zeros before a sequence's first token.  The last row of a step is
kept per sequence (float32), so prompts cut into steps and decoding continue from it.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import SHIFTS, InputShift, StateNeed, WeightDecl


@SHIFTS.register("token_shift")
class TokenShift(InputShift):
    def __init__(self, dim: int, name: str = "weight"):
        self.dim = int(dim)
        self.name = name                        # what the checkpoint calls the blend weights, behind the part's prefix
        self.mix: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {self.name: WeightDecl((self.dim,))}

    def state_needs(self) -> list[StateNeed]:
        return [StateNeed((self.dim,), torch.float32)]

    def bind(self, tensors, dtype, device) -> None:
        self.mix = tensors[self.name].to(torch.float32).contiguous()

    def vectors(self) -> list[torch.Tensor]:
        return [self.mix]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x, states) -> torch.Tensor:
        out = ctx.scratch("shift.out", tuple(x.shape), x.dtype)
        api.token_shift(x, self.mix, states[0], out, ctx.cu, ctx.slots, ctx.sequences)
        return out
