"""Vectors that a schedule adds to the residual stream between layers."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..weights.spec import ParamSpec
from .base import Part


class PassOffsets(Part):
    """A table [passes, hidden]: row t is added to every position of the stream right before pass t of a stretch of
    layers that runs several times with the same weights (engine.model.ScheduleEntry.pass_index)."""

    def __init__(self, passes: int, hidden: int, param_name: str = "weight"):
        self.passes, self.hidden, self.param_name = passes, hidden, param_name
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.param_name: ParamSpec((self.passes, self.hidden), kind="vector", init="normal")}

    def bind(self, params, compute_dtype):
        self.table = params[self.param_name]

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def row(self, t: int) -> torch.Tensor:
        return self.table[t]

    def add(self, ctx, stream, t: int) -> None:
        stream.flush()
        stream.prepared = None
        kernels.add_row(stream.h, self.table[t])
