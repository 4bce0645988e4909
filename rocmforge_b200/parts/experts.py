"""A feed-forward made of many small ones, of which every token uses a few."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .base import FEED_FORWARDS, FeedForward


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """z = W_router y + b in 32-bit; a token uses the ``top`` experts with the largest z, weighted by the softmax over
    those z alone; an expert is W_down (silu(W_gate y) * (W_up y)) without biases; the result is the weighted sum.

    Nothing of the routing reaches the host.  The (token, choice) pairs are sorted by expert on the device, one grouped
    product over the sorted rows serves gate and up of all experts (the experts' matrices are stacked at load time, gate
    and up interleaved row by row), one the down projections, and the choices of a token are summed in the order of the
    choices, in 32-bit: a token's result does not depend on the rest of the batch.
    Tensors: ``router`` [E, H], ``router.b`` [E], ``e<i>.gate`` / ``.up`` [F, H], ``e<i>.down`` [H, F]
    (``names`` may rename router, router_bias, gate, up, down; ``expert_prefix`` the "e").

    What other designs change, as parameters: ``scoring`` "sigmoid" weights a chosen expert by the sigmoid of its own
    logit, not renormalised (the choice is still by the largest logits); ``weight_on`` "input" multiplies the expert's
    input by the weight instead of its output, out = sum_e expert_e(w_e y) (an expert is not linear, so the two differ;
    the products being linear, w (W y) is formed in the first product's epilogue, in 32-bit, before the activation);
    ``activation`` "clamped_glu" is g sigmoid(glu_alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit).
    """

    def __init__(self, hidden: int, intermediate: int, n_experts: int, top: int, *, router_bias: bool = True,
                 names: Optional[Dict[str, str]] = None, expert_prefix: str = "e", scoring: str = "softmax_of_chosen",
                 weight_on: str = "output", activation: str = "silu", limit: Optional[float] = None, glu_alpha: float = 1.702):
        if not 1 <= top <= n_experts:
            raise ValueError(f"routed experts: top {top} of {n_experts} experts")
        if scoring not in kernels.MOE_SCORINGS:
            raise ValueError(f"routed experts: scoring {scoring!r} (known: {sorted(kernels.MOE_SCORINGS)})")
        if weight_on not in ("output", "input") or activation not in ("silu", "clamped_glu"):
            raise ValueError(f"routed experts: weight_on {weight_on!r} / activation {activation!r} have no kernel")
        if weight_on == "input" and activation == "silu":
            raise ValueError("routed experts: weights on the inputs are built for the clamped activation only")
        if activation == "clamped_glu" and not (limit is not None and limit > 0):
            raise ValueError("routed experts: the clamped activation needs a positive limit")
        self.scoring, self.weight_on, self.activation = scoring, weight_on, activation
        self.limit, self.glu_alpha = (float(limit) if limit is not None else None), float(glu_alpha)
        self.hidden, self.intermediate, self.n_experts, self.top = hidden, intermediate, n_experts, top
        self.router_bias = router_bias
        self.names = {"router": "router", "router_bias": "router.b", "gate": "gate", "up": "up", "down": "down"}
        self.names.update(names or {})
        self.expert_prefix = expert_prefix
        self.router_w = self.router_b = self.gate_up = self.down = None

    def _expert(self, e: int, which: str) -> str:
        return f"{self.expert_prefix}{e}.{self.names[which]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        # random-weights mode: router logits a few units apart, so that a choice rarely hangs on the last bits
        s = {self.names["router"]: ParamSpec((self.n_experts, self.hidden), std=0.5)}
        if self.router_bias:
            s[self.names["router_bias"]] = ParamSpec((self.n_experts,), kind="vector", init="normal", std=0.5)
        for e in range(self.n_experts):
            s[self._expert(e, "gate")] = ParamSpec((self.intermediate, self.hidden))
            s[self._expert(e, "up")] = ParamSpec((self.intermediate, self.hidden))
            s[self._expert(e, "down")] = ParamSpec((self.hidden, self.intermediate))
        return s

    def bind(self, params, compute_dtype):
        self.router_w = params[self.names["router"]]
        self.router_b = params[self.names["router_bias"]].to(torch.float32) if self.router_bias else None
        E, F, H = self.n_experts, self.intermediate, self.hidden
        gu = torch.stack([torch.stack([params[self._expert(e, "gate")], params[self._expert(e, "up")]], dim=1)
                          for e in range(E)])                                # [E, F, 2, H]: row 2j = gate_j, 2j+1 = up_j
        self.gate_up = gu.reshape(E, 2 * F, H).contiguous()
        self.down = torch.stack([params[self._expert(e, "down")] for e in range(E)]).contiguous()      # [E, H, F]

    def cuda_modules(self, compute_dtype):
        return ["elementwise", "gemm_simt", "moe"] + (["gemm_tcgen05"] if compute_dtype == torch.bfloat16 else [])

    def output(self, ctx, y):
        if isinstance(y, ScaledRows):
            y = y.materialize()
        T = y.shape[0]
        z = ctx.matmul(y, self.router_w, self.router_b, out_f32=True)         # 32-bit sums of exact products
        idx, w = kernels.moe_route(z, self.top, self.scoring)
        n = T * self.top
        tc = kernels.tensor_core
        if self.weight_on == "input" or self.activation != "silu":
            return self._output_general(ctx, y, idx, w, n)
        if (ctx.compute_dtype == torch.bfloat16 and ctx.options.tensor_core_gemm
                and tc.grouped_supported(2 * self.intermediate, self.hidden, tc.SWIGLU)
                and tc.grouped_supported(self.hidden, self.intermediate, tc.F32)):
            # tensor cores: the activations once in sorted order, then tiles of 128 sorted rows against their expert's
            # matrices; the gate's silu and the product with up happen in the first product's epilogue
            perm, inv, tiles, max_tiles = kernels.moe_sort(idx, self.n_experts, kernels.MOE_TILE_TC)
            a = tc.gemm_tc_grouped(kernels.moe_gather(y, perm, self.top), self.gate_up, tiles, max_tiles, mode=tc.SWIGLU)
            d = tc.gemm_tc_grouped(a, self.down, tiles, max_tiles, mode=tc.F32)
            return kernels.moe_combine(d, inv, w)
        rows = kernels.MOE_TILE_SMALL if n <= 16 * self.n_experts else kernels.MOE_TILE_LARGE
        perm, inv, tiles, max_tiles = kernels.moe_sort(idx, self.n_experts, rows)
        gu = kernels.gemm_simt_grouped(y, self.gate_up, tiles, max_tiles, rows, n, row_map=perm, row_div=self.top)
        a = kernels.swiglu(gu)                                                               # [n, F], sorted rows
        d = kernels.gemm_simt_grouped(a, self.down, tiles, max_tiles, rows, n, out_f32=True)
        return kernels.moe_combine(d, inv, w)

    def _output_general(self, ctx, y, idx, w, n):
        """Weights on the experts' inputs and/or another activation: each sorted row of the first grouped product is
        scaled by its pair's weight (in 32-bit, before anything is clamped) and the activation applied, in that product's
        epilogue on the tensor-core path and by a kernel of its own otherwise; with the weights spent on the inputs the
        choices of a token are summed plainly."""
        tc = kernels.tensor_core
        on_input = self.weight_on == "input"
        use_tc = (ctx.compute_dtype == torch.bfloat16 and ctx.options.tensor_core_gemm
                  and tc.grouped_supported(2 * self.intermediate, self.hidden, tc.CLAMPGLU)
                  and tc.grouped_supported(self.hidden, self.intermediate, tc.F32))
        rows = kernels.MOE_TILE_TC if use_tc else (kernels.MOE_TILE_SMALL if n <= 16 * self.n_experts else kernels.MOE_TILE_LARGE)
        if on_input:                                  # the sort leaves the pairs' weights in the order of the sorted rows
            perm, inv, tiles, max_tiles, ws = kernels.moe_sort(idx, self.n_experts, rows, weights=w)
        else:
            (perm, inv, tiles, max_tiles), ws = kernels.moe_sort(idx, self.n_experts, rows), None
        if use_tc and self.activation == "clamped_glu":
            # the scale and the activation happen in the first product's epilogue, on its 32-bit sums
            a = tc.gemm_tc_grouped(kernels.moe_gather(y, perm, self.top), self.gate_up, tiles, max_tiles, mode=tc.CLAMPGLU,
                                   row_scale=ws, limit=self.limit, alpha=self.glu_alpha)
        else:
            if use_tc:
                gu = tc.gemm_tc_grouped(kernels.moe_gather(y, perm, self.top), self.gate_up, tiles, max_tiles, mode=tc.STORE)
            else:
                gu = kernels.gemm_simt_grouped(y, self.gate_up, tiles, max_tiles, rows, n, row_map=perm, row_div=self.top)
            a = (kernels.clamped_glu(gu, self.limit, self.glu_alpha, row_scale=ws) if self.activation == "clamped_glu"
                 else kernels.swiglu(gu))
        if use_tc:
            d = tc.gemm_tc_grouped(a, self.down, tiles, max_tiles, mode=tc.F32)
        else:
            d = kernels.gemm_simt_grouped(a, self.down, tiles, max_tiles, rows, n, out_f32=True)
        return kernels.moe_combine(d, inv, None if on_input else w, top=self.top)

    def forward(self, ctx, y, stream):
        stream.add_pending(self.output(ctx, y))
