"""Mixers side by side."""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer, NormedMean, Part


class _OutWeights(Part):
    """The weights with which the halves' outputs are normed before they are averaged."""

    def __init__(self, hidden: int, names):
        self.hidden, self.names = hidden, list(names)
        self.weights: Dict[str, torch.Tensor] = {}

    def param_specs(self):
        return {n: ParamSpec((self.hidden,), kind="vector", init="ones") for n in self.names}

    def bind(self, params, compute_dtype):
        self.weights = dict(params)


@MIXERS.register("parallel")
class ParallelMixer(Mixer):
    """Several mixers read the same input; the result is the mean of their outputs, each first RMS-normed over the
    width with a weight of its own (used as stored):  mean_b( x_b / sqrt(mean(x_b^2) + eps) * w_b ).

    ``branches``: {name: mixer}; a branch's tensors lie under ``<name>.`` and its out-weight is ``<name>.out``
    (``out_name``).  Each branch keeps what it keeps: the cache request is the dict of the branches' requests, and
    the view this mixer receives is the dict of their views.  Two branches are merged in the kernel that adds the
    result to the stream (the mixer hands out a ``NormedMean``).
    """

    def __init__(self, hidden: int, branches: Dict[str, Mixer], eps: float, out_name: str = "out"):
        if len(branches) != 2:
            raise ValueError("parallel mixer: the merging kernel takes two branches")
        self.hidden, self.branches, self.eps, self.out_name = hidden, dict(branches), float(eps), out_name
        self.outs = _OutWeights(hidden, [f"{name}.{out_name}" for name in self.branches])

    # the halves are leaf parts of their own (their tensors have prefixes of their own)
    def leaf_parts(self) -> Dict[str, Part]:
        out: Dict[str, Part] = {f"{name}.": m for name, m in self.branches.items()}
        out[""] = self.outs
        return out

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def cache_request(self):
        return {name: m.cache_request() for name, m in self.branches.items()}

    def output(self, ctx, y, cache_view):
        return NormedMean([(m.output(ctx, y, cache_view[name]), self.outs.weights[f"{name}.{self.out_name}"])
                           for name, m in self.branches.items()], self.eps)

    def forward(self, ctx, y, cache_view, stream):
        raise NotImplementedError("parallel mixer: its result is merged by the block that holds it (output)")
