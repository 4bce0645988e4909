"""The Rifizen decoder as a list of parts.

Every layer norms its sub-layers on the way in and on the way out (``sandwich`` block).  Its mixer is two mixers
side by side on the same input (``parallel``): grouped-query softmax attention over a sliding window, without
rotation, with unit-normed query and key heads, scores capped by a tanh and lowered in proportion to the distance
(slope 2^(-8 (h+1) / heads) for head h); and retention, a decaying matrix state per head with rotated q and k.  The
feed-forward is relu(x)^2 between two matrices, a mixture of small gated (silu) experts, or absent.  A stretch of layers
may run several times with the same weights, each pass with a cache and a state of its own and with a learned vector
added to the stream before it.

Tensor names: ``embed``, ``loop.step`` [passes, width], ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.left.q|k|v|o``,
``l<i>.mix.right.q|k|v|g|o``, ``l<i>.mix.left.out|right.out``, ``l<i>.mlp.up|down`` or ``l<i>.mlp.router``,
``.router.b``, ``.e<j>.gate|up|down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.rifizen import RifizenConfig
from ..engine.model import ModelSpec, ScheduleEntry
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.offsets import PassOffsets

NO_POSITION_LIMIT = 1 << 20      # the design has no longest sequence; the cache's size is the only limit


def distance_slopes(heads: int):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def build_rifizen(cfg: RifizenConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps

    def norm():
        return NORMS.build("rmsnorm", size=W, eps=eps, param_name="")

    blocks, prefixes = [], []
    for i, L in enumerate(cfg.layers):
        a, r = L.left, L.right
        left = MIXERS.build("gqa_attention", hidden=W, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
                            v_head_dim=a.vdim, qkv_bias=False, window=a.window, position=None, scale=a.scale,
                            qk_norm_eps=eps, softcap=a.softcap, distance_slopes=distance_slopes(a.heads),
                            names={"q": "q", "k": "k", "v": "v", "o": "o"})
        position = (POSITIONS.build("rope_neox", head_dim=r.dim, theta=r.rot_base, rotary_dim=r.rot_dims)
                    if r.rot_dims > 0 else None)
        right = MIXERS.build("retention", hidden=W, n_heads=r.heads, dim=r.dim, vdim=r.vdim, decay=r.decay, eps=eps,
                             position=position, names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"})
        mixer = MIXERS.build("parallel", hidden=W, branches={"left": left, "right": right}, eps=eps)
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = FEED_FORWARDS.build("relu2_mlp", hidden=W, intermediate=L.mlp.ff, names={"up": "up", "down": "down"})
        elif L.mlp is not None:
            ffn = FEED_FORWARDS.build("routed_experts", hidden=W, intermediate=L.mlp.ff, n_experts=L.mlp.experts,
                                      top=L.mlp.top)
        names = {"norm1": "norm1", "mixer": "mix.", "post1": "norm1b", "norm2": "norm2", "ffn": "mlp.", "post2": "norm2b"}
        blocks.append(BLOCKS.build("sandwich", norm1=norm(), mixer=mixer, post1=norm(),
                                   norm2=norm() if ffn is not None else None, ffn=ffn,
                                   post2=norm() if ffn is not None else None, names=names))
        prefixes.append(f"l{i}.")

    schedule = [ScheduleEntry(layer=i) for i in range(cfg.loop_start if cfg.has_loop else len(cfg.layers))]
    offsets = PassOffsets(cfg.loop_times, W, param_name="") if cfg.loop_given else None
    if cfg.has_loop:
        for t in range(cfg.loop_times):
            for i in range(cfg.loop_start, cfg.loop_stop):
                schedule.append(ScheduleEntry(layer=i, pass_index=t if i == cfg.loop_start else None))
        schedule += [ScheduleEntry(layer=i) for i in range(cfg.loop_stop, len(cfg.layers))]
    return ModelSpec(
        config=cfg, embedding=TokenEmbedding(cfg.vocab, W, param_name=""), embedding_prefix="embed",
        blocks=blocks, block_prefixes=prefixes, final_norm=norm(), final_norm_prefix="final.norm",
        head=OutputHead(cfg.vocab, W, param_name=""), head_prefix="head",
        schedule=schedule, vocab_size=cfg.vocab, hidden_size=W, max_position=NO_POSITION_LIMIT,
        stop_token_ids=[], pass_offsets=offsets, pass_offsets_prefix="loop.step")


register_architecture(RifizenConfig.ARCHITECTURE, RifizenConfig, build_rifizen)
