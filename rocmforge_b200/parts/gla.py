"""Gated linear attention: linear attention whose matrix state decays per key channel, by a factor made from the token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..cache.requests import StateRequest
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer
from .linear import Linear


@MIXERS.register("gla")
class GatedLinearAttention(Mixer):
    """Per head, with q, k of size ``dim`` and v of size ``vdim``:

        alpha_t = sigmoid(z_t)^(1/tau),  z_t = W_a2 (W_a1 x_t) + b      (one decay per key channel, [heads, dim])
        S_t = diag(alpha_t) S_(t-1) + k_t v_t^T                          (S starts at zero, float32, per sequence)
        o_t = S_t^T q_t,  q_t = W_q x_t * q_scale (default dim^-1/2)
        out = W_o (concat_h(rms(o_t) * w) * silu(W_g x))                 (rms over vdim, one weight [vdim] for all heads)

    The projections run in the compute dtype, as one product q | k | v | g | a1 (W_a1 is the narrow first half of the
    decay's low-rank projection) and a second, small one for z, whose result stays 32-bit; q, k, the decay (formed as
    exp(log sigmoid(z) / tau)), the state, o and its norm are 32-bit.  The state is kept as [heads, dim, vdim].  ``names``: the tensors' names below the part's prefix (keys q, k, v, g, o, a1, a2, a2_bias, norm).
    """

    def __init__(self, hidden: int, n_heads: int, dim: int, vdim: int, tau: float, eps: float, *, decay_rank: int,
                 q_scale: Optional[float] = None, names: Optional[Dict[str, str]] = None):
        if not tau > 0:
            raise ValueError(f"gla: tau must be positive, got {tau}")
        if decay_rank < 1:
            raise ValueError(f"gla: the decay's projection needs a rank of at least 1, got {decay_rank}")
        self.hidden, self.n_heads, self.dim, self.vdim = hidden, n_heads, dim, vdim
        self.tau, self.eps, self.decay_rank = float(tau), float(eps), int(decay_rank)
        self.q_scale = float(q_scale) if q_scale is not None else float(dim) ** -0.5
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                      "o": "o_proj.weight", "a1": "a_proj.0.weight", "a2": "a_proj.1.weight", "a2_bias": "a_proj.1.bias",
                      "norm": "norm.weight"}
        self.names.update(names or {})
        self.qk_size, self.v_size = n_heads * dim, n_heads * vdim
        self.proj: Optional[Linear] = None
        self.a2: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        return {n["q"]: ParamSpec((self.qk_size, self.hidden)), n["k"]: ParamSpec((self.qk_size, self.hidden)),
                n["v"]: ParamSpec((self.v_size, self.hidden)), n["g"]: ParamSpec((self.v_size, self.hidden)),
                n["o"]: ParamSpec((self.hidden, self.v_size)),
                n["a1"]: ParamSpec((self.decay_rank, self.hidden)),
                # random-weights mode: decays spread between fast and slow channels
                n["a2"]: ParamSpec((self.qk_size, self.decay_rank), std=1.0),
                n["a2_bias"]: ParamSpec((self.qk_size,), kind="vector", init="normal", std=2.0),
                n["norm"]: ParamSpec((self.vdim,), kind="vector", init="ones")}

    def bind(self, params, compute_dtype):
        n = self.names
        # the narrow decay projection is padded to a multiple of 8 rows so that the second product's input rows stay
        # 16-byte aligned in bfloat16 (the padding's weights are zero and the second matrix has zero columns for it)
        r, rp = self.decay_rank, (self.decay_rank + 7) // 8 * 8
        a1, a2 = params[n["a1"]], params[n["a2"]]
        if rp != r:
            a1 = torch.cat([a1, a1.new_zeros((rp - r, self.hidden))], dim=0)
            a2 = torch.cat([a2, a2.new_zeros((self.qk_size, rp - r))], dim=1)
        self.a1_col = 2 * self.qk_size + 2 * self.v_size
        pad = (-self.a1_col) % 8                     # the a1 columns start on a 16-byte boundary
        blocks = [params[n["q"]], params[n["k"]], params[n["v"]], params[n["g"]]]
        if pad:
            blocks.append(a1.new_zeros((pad, self.hidden)))
            self.a1_col += pad
        self.rank_padded = rp
        self.proj = Linear(torch.cat(blocks + [a1], dim=0).contiguous())
        self.a2 = Linear(a2.contiguous(), params[n["a2_bias"]])
        self.o = Linear(params[n["o"]])
        self.norm_w = params[n["norm"]]

    def cuda_modules(self, compute_dtype):
        return ["elementwise", "retention", "gla"]

    def cache_request(self):
        return StateRequest.of(S=((self.n_heads, self.dim, self.vdim), torch.float32))

    def gated(self, ctx, y, state_view):
        """The gated, normed heads [T, heads*vdim] in the compute dtype (the output product's input)."""
        if isinstance(y, ScaledRows):
            y = y.materialize()
        p = self.proj(ctx, y)                                                # [T, q | k | v | g | a1]
        z = self.a2(ctx, p[:, self.a1_col:self.a1_col + self.rank_padded], out_f32=True)      # [T, heads*dim], 32-bit
        qka = kernels.gla_prepare(p, 0, self.qk_size, z, self.n_heads, self.dim, self.q_scale, self.tau)
        v = p[:, 2 * self.qk_size: 2 * self.qk_size + self.v_size]
        g = p[:, 2 * self.qk_size + self.v_size: 2 * self.qk_size + 2 * self.v_size]
        o = kernels.gla_scan(qka, v, state_view["S"], ctx.cu_q, ctx.seq_slot, self.n_heads, self.dim, self.vdim,
                             one_token=ctx.is_decode)
        return kernels.retention_gate(o, g, self.n_heads, self.vdim, self.eps, weight=self.norm_w)

    def forward(self, ctx, y, cache_view, stream):
        self.o.add_to_stream(ctx, self.gated(ctx, y, cache_view), stream)

    def output(self, ctx, y, cache_view):
        return self.o.f32_parts(ctx, self.gated(ctx, y, cache_view))
