"""Plain, slow implementation of the Vilulorn decoder, used as the test oracle.

One function per mechanism, whole sequences only, no cache, no batching; everything in ``dtype`` (float64 by
default) except rotation angles, which are formed in 32-bit (float32(position) * float32(frequency)) like the
engine's.  It shares no code with ``rocmforge_b200``: tensors come in as a plain {name: tensor} dict.

Notation: W[name] is stored [out, in] and applied as x @ W.T; rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis, the weight used as stored."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- embedding

def embed_with_positions(tokens, W, dtype):
    """x_p = embed[token_p] + pos[p], positions from 0."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    return W["embed"].to(dtype)[ids] + W["pos"].to(dtype)[: len(ids)]


# --------------------------------------------------------------------------- mixer 'gla'

def channel_decay(h, W, pre, tau: float):
    """alpha = sigmoid(z)^(1/tau) with z = W_a2 (W_a1 h) + b, one per key channel: [T, heads * dim]."""
    z = (h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def gated_linear_attention(h, W, pre, m, eps):
    """h [T, width] -> [T, width].  ``m``: heads, dim, vdim, tau.

    Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T (S is [dim, vdim], the decay scales the rows), o_t = S_t^T q_t;
    o is RMS-normed per head over vdim with one weight for all heads, gated with silu(W_g h) and projected."""
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, D)
    v = (h @ W[pre + "v"].T).reshape(T, H, DV)
    alpha = channel_decay(h, W, pre, float(m["tau"])).reshape(T, H, D)
    S = torch.zeros((H, D, DV), dtype=h.dtype)
    o = torch.zeros((T, H, DV), dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, W[pre + "norm"], eps).reshape(T, H * DV)
    return (o * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


# --------------------------------------------------------------------------- mixer 'attention'

def scaled_frequencies(dims: int, base: float, scaling):
    """f_i = base^(-2i/dims), then stretched by wavelength: short waves (l < original/high) stay, long ones
    (l > original/low) are divided by ``factor``, in between the two are blended linearly in original/l."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if scaling is None:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for n in range(len(f)):
        wave = 2.0 * math.pi / float(f[n])
        if wave < orig / high:
            continue
        if wave > orig / low:
            out[n] = f[n] / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[n] = (1.0 - s) * f[n] / factor + s * f[n]
    return out


def rotate_neighbours(x, positions, dims: int, freq):
    """x [T, heads, dim]: of the first ``dims`` elements of a head, element 2i turns with element 2i+1 by the angle
    position * freq[i]; the rest pass."""
    ang = (positions.to(torch.float32)[:, None] * freq.to(torch.float32)[None, :]).to(torch.float64)
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, w = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def keys_and_values(h, W, pre, m, eps):
    """The keys (normed per head, rotated) and values of a layer that has projections of its own."""
    T = h.shape[0]
    G, D, DV = m["kv_heads"], m["dim"], m["vdim"]
    k = rms_norm((h @ W[pre + "k"].T).reshape(T, G, D), W[pre + "k.norm"], eps)
    rot = m["rot"]
    k = rotate_neighbours(k, torch.arange(T), int(rot["dims"]), scaled_frequencies(int(rot["dims"]), rot["base"], rot.get("scaling")))
    v = (h @ W[pre + "v"].T).reshape(T, G, DV)
    return k, v


def chunked_attention(h, W, pre, m, eps, kv):
    """h [T, width] -> [T, width].  ``kv``: (keys, values) as ``keys_and_values`` gives them, of this layer or of the
    layer it borrows them from.  Position i sees j <= i inside its own chunk of mask.size positions."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    k, v = kv
    q = rms_norm((h @ W[pre + "q"].T).reshape(T, H, D), W[pre + "q.norm"], eps)
    rot = m["rot"]
    q = rotate_neighbours(q, torch.arange(T), int(rot["dims"]), scaled_frequencies(int(rot["dims"]), rot["base"], rot.get("scaling")))
    size = int(m["mask"]["size"])
    out = torch.zeros((T, H, DV), dtype=h.dtype)
    for i in range(T):
        lo = (i // size) * size
        for hh in range(H):
            g = hh // (H // G)
            p = torch.softmax((k[lo:i + 1, g] @ q[i, hh]) * m["scale"], dim=0)
            out[i, hh] = p @ v[lo:i + 1, g]
    gate = torch.sigmoid(h @ W[pre + "g"].T)
    return (out.reshape(T, H * DV) * gate) @ W[pre + "o"].T


# --------------------------------------------------------------------------- feed-forward

def clamped_expert(x, W, pre, limit: float):
    """g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(x @ W[pre + "gate"].T, max=limit)
    u = torch.clamp(x @ W[pre + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def scored_experts(h, W, pre, mlp, forced=None, chosen=None):
    """Every token uses the ``top`` experts with the largest sigmoid(router logit); an expert's score multiplies its
    input, and the scores are not renormalised: out = sum_e expert_e(s_e h).

    ``forced`` ([T, top] expert indices) replaces the choice (the scores stay this function's own): a comparison with an
    implementation that rounds differently then does not hang on tokens whose best experts are nearly tied.
    ``chosen``: a list that receives, per token, (this function's own choice, the margin between the last chosen and
    the first unchosen logit as a share of the logits' spread)."""
    E, top, limit = mlp["router"]["experts"], mlp["router"]["top"], float(mlp["expert"]["limit"])
    z = h @ W[pre + "router"].T
    s = torch.sigmoid(z)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        # ranked by the logits: the sigmoid keeps their order, but far out it rounds to exactly 1 and would make ties
        ranked = sorted(range(E), key=lambda e: (-float(z[t, e]), e))
        order = ranked[:top]
        if chosen is not None:
            spread = float(z[t].max() - z[t].min()) + 1e-9
            margin = float(z[t, ranked[top - 1]] - z[t, ranked[top]]) / spread if top < E else float("inf")
            chosen.append((order, margin))
        if forced is not None:
            order = [int(e) for e in forced[t]]
        for e in order:
            out[t] += clamped_expert(s[t, e] * h[t], W, f"{pre}e{e}.", limit)
    return out


# --------------------------------------------------------------------------- the model

class PlainVilulorn:
    def __init__(self, config: dict, tensors: dict, dtype=torch.float64):
        self.cfg, self.dtype = config, dtype
        self.W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])

    def logits(self, tokens, layers_out=None, forced=None, chosen=None):
        """[T, vocab] for a whole sequence from position 0; ``layers_out``: a list that receives the stream after
        every layer; ``forced`` {layer: [T, top] expert indices} and ``chosen`` {layer: list}: see ``scored_experts``."""
        W, eps = self.W, self.eps
        x = embed_with_positions(tokens, W, self.dtype)
        kv = {}
        for i, L in enumerate(self.cfg["layers"]):
            pre, m = f"l{i}.mix.", L["mixer"]
            if L["type"] == "gla":
                r = gated_linear_attention(x, W, pre, m, eps)
            elif L["type"] == "attention":
                src = m.get("kv_from")
                if src is None:
                    kv[i] = keys_and_values(x, W, pre, m, eps)
                r = chunked_attention(x, W, pre, m, eps, kv[i if src is None else src])
            else:
                raise ValueError(L["type"])
            x = x + rms_norm(r, W[f"l{i}.norm1"], eps)
            if L.get("mlp") is not None:
                x = x + rms_norm(scored_experts(x, W, f"l{i}.mlp.", L["mlp"], None if forced is None else forced.get(i),
                                                None if chosen is None else chosen.setdefault(i, [])), W[f"l{i}.norm2"], eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        return rms_norm(x, W["final.norm"], eps) @ W["head"].T
