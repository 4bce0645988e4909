"""Plain, slow implementation of the Rifizen decoder, used as the test oracle.

One function per mechanism, whole sequences only, no cache, no batching; everything in
``dtype`` (float64 by default) except the rotation angle, which is formed in 32-bit
(float32(position) * float32(frequency)) like the engine's.  It shares no code with
``rocmforge_b200``: tensors come in as a plain {name: tensor} dict.

Notation: W[name] is stored [out, in] and applied as x @ W.T; rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import math

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- left half: windowed softmax attention

def distance_slopes(heads: int):
    """slope_h = 2^(-8 (h + 1) / heads)."""
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def capped_window_attention(h, W, pre, m, eps):
    """h [T, width] -> [T, width].  ``m``: heads, kv_heads, dim, vdim, scale, softcap, mask.size."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D)
    k = (h @ W[pre + "k"].T).reshape(T, G, D)
    v = (h @ W[pre + "v"].T).reshape(T, G, DV)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    slopes = distance_slopes(H)
    window = int(m["mask"]["size"])
    cap = m.get("softcap")
    out = torch.zeros((T, H, DV), dtype=h.dtype)
    for i in range(T):
        lo = max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            dist = torch.arange(i - lo, -1, -1, dtype=h.dtype)          # i - j for j = lo .. i
            s = s - slopes[hh] * dist
            p = torch.softmax(s, dim=0)
            out[i, hh] = p @ v[lo:i + 1, g]
    return out.reshape(T, H * DV) @ W[pre + "o"].T


# --------------------------------------------------------------------------- right half: retention

def rotate_half_layout(x, positions, dims: int, base: float):
    """x [T, heads, dim]: the first ``dims`` elements of every head turn, element i with element i + dims/2, by the
    angle position * base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (1.0 / torch.pow(torch.tensor(float(base), dtype=torch.float64), 2.0 * i / dims)).to(torch.float32)
    ang = (positions.to(torch.float32)[:, None] * freq[None, :]).to(torch.float64)      # the angle itself is 32-bit
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., dims:]], dim=-1)


def retention(h, W, pre, m, eps, positions=None, state=None):
    """h [T, width] -> ([T, width], final state [heads, dim, vdim]).  ``m``: heads, dim, vdim, decay[], rot{dims, base}."""
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ W[pre + "q"].T).reshape(T, H, D)
    k = (h @ W[pre + "k"].T).reshape(T, H, D)
    v = (h @ W[pre + "v"].T).reshape(T, H, DV)
    gate = silu(h @ W[pre + "g"].T).reshape(T, H, DV)
    q = rotate_half_layout(q, positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half_layout(k, positions, m["rot"]["dims"], m["rot"]["base"]) * D ** -0.5
    S = torch.zeros((H, D, DV), dtype=h.dtype) if state is None else state.clone()
    decay = torch.tensor(m["decay"], dtype=h.dtype)[:, None, None]
    o = torch.zeros((T, H, DV), dtype=h.dtype)
    for t in range(T):
        S = decay * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * gate
    return o.reshape(T, H * DV) @ W[pre + "o"].T, S


def parallel_mixer(h, W, pre, m, eps):
    """Half the sum of the two halves' outputs, each RMS-normed over the width with its own weight."""
    left = capped_window_attention(h, W, pre + "left.", m["left"], eps)
    right, _ = retention(h, W, pre + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, W[pre + "left.out"], eps) + rms_norm(right, W[pre + "right.out"], eps))


# --------------------------------------------------------------------------- feed-forwards

def dense_ff(h, W, pre):
    """W_down relu(W_up h)^2."""
    return torch.relu(h @ W[pre + "up"].T) ** 2 @ W[pre + "down"].T


def routed_ff(h, W, pre, n_experts: int, top: int):
    """Softmax over the ``top`` largest router logits; each chosen expert is W_down (silu(W_gate h) * (W_up h))."""
    z = h @ W[pre + "router"].T + W[pre + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        vals, idx = torch.topk(z[t], top)
        w = torch.softmax(vals, dim=0)
        for wk, e in zip(w, idx.tolist()):
            p = f"{pre}e{e}."
            out[t] += wk * ((silu(h[t] @ W[p + "gate"].T) * (h[t] @ W[p + "up"].T)) @ W[p + "down"].T)
    return out


def feed_forward(h, W, pre, mlp):
    if mlp["kind"] == "dense":
        return dense_ff(h, W, pre)
    return routed_ff(h, W, pre, mlp["router"]["experts"], mlp["router"]["top"])


# --------------------------------------------------------------------------- the model

def layer_order(cfg):
    """[(layer index, pass number or None)] in run order; a pass number marks the first layer of a looped pass."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t if i == loop["start"] else None))
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, tensors, tokens, dtype=torch.float64, trace=None):
    """Logits [T, vocab] of a whole sequence.  ``trace``: a list that receives the stream after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, first_of_pass in layer_order(cfg):
        if first_of_pass is not None:
            x = x + W["loop.step"][first_of_pass]
        L, p = cfg["layers"][i], f"l{i}."
        assert L["type"] == "parallel"
        y = parallel_mixer(rms_norm(x, W[p + "norm1"], eps), W, p + "mix.", L["mixer"], eps)
        x = x + rms_norm(y, W[p + "norm1b"], eps)
        if L.get("mlp"):
            y = feed_forward(rms_norm(x, W[p + "norm2"], eps), W, p + "mlp.", L["mlp"])
            x = x + rms_norm(y, W[p + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T
