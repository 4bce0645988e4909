"""The Vilulorn decoder as a list of parts.

x = embed[token] + pos[position].  A layer norms its sub-layers on the way out only, and they read the stream itself:
x += norm1(mixer(x)); x += norm2(ff(x)) (the ``sandwich`` block without its inner norms).  The mixer is, layer by layer,
gated linear attention (``gla``: a matrix state per head that decays per key channel by a factor made from the token) or
grouped-query softmax attention inside chunks of the sequence (``gqa_attention`` with weighted query/key norms, a partly
rotated head with neighbouring pairs and frequencies stretched by wavelength, a sigmoid gate on the heads, and for some
layers the keys and values of an earlier layer).  The feed-forward is a mixture of small experts chosen by the largest
router logits, weighted on their inputs by the sigmoid of their logit, with a clamped gated activation; a layer may have
none.  Final RMS norm, then the head.

Tensor names: ``embed``, ``pos``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v|g|o`` and ``.norm``, ``.a1``, ``.a2``, ``.a2.b``
(gla) or ``.q.norm``, ``.k.norm`` (attention; no k, v, k.norm with ``kv_from``), ``l<i>.mlp.router``, ``.e<j>.gate|up|down``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vilulorn import VilulornConfig
from ..engine.model import ModelSpec, ScheduleEntry
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from ..parts.embedding import LearnedPositions, OutputHead, TokenEmbedding

EXPERT_GATE_SLOPE = 1.702        # g sigmoid(1.702 g): fixed by the design


def build_vilulorn(cfg: VilulornConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps

    def norm():
        return NORMS.build("rmsnorm", size=W, eps=eps, param_name="")

    # an attention layer whose cache other layers read with chunks of another size keeps all of its keys
    readers = {}
    for i, L in enumerate(cfg.layers):
        if L.type == "attention" and L.mixer.kv_from is not None:
            readers.setdefault(L.mixer.kv_from, []).append(L.mixer.chunk)

    blocks, prefixes, schedule = [], [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "gla":
            mixer = MIXERS.build("gla", hidden=W, n_heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau, eps=eps,
                                 decay_rank=m.rank,
                                 names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a1": "a1", "a2": "a2",
                                        "a2_bias": "a2.b", "norm": "norm"})
        else:
            position = (POSITIONS.build("rope_neox", head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims,
                                        interleaved=True, scaling=m.rot_scaling) if m.rot_dims > 0 else None)
            keeps_all = any(c != m.chunk for c in readers.get(i, []))
            mixer = MIXERS.build("gqa_attention", hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                                 v_head_dim=m.vdim, qkv_bias=False, position=position, scale=m.scale, qk_norm_eps=eps,
                                 qk_norm_weight=True, chunk=m.chunk, gate="sigmoid", shares_kv=m.kv_from is not None,
                                 cache_keeps="all" if keeps_all else None,
                                 names={"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm",
                                        "k_norm": "k.norm"})
        ffn = None
        if L.mlp is not None:
            ffn = FEED_FORWARDS.build("routed_experts", hidden=W, intermediate=L.mlp.ff, n_experts=L.mlp.experts,
                                      top=L.mlp.top, router_bias=False, scoring="sigmoid", weight_on="input",
                                      activation="clamped_glu", limit=L.mlp.limit, glu_alpha=EXPERT_GATE_SLOPE)
        names = {"mixer": "mix.", "post1": "norm1", "ffn": "mlp.", "post2": "norm2"}
        blocks.append(BLOCKS.build("sandwich", norm1=None, mixer=mixer, post1=norm(), norm2=None, ffn=ffn,
                                   post2=norm() if ffn is not None else None, names=names))
        prefixes.append(f"l{i}.")
        schedule.append(ScheduleEntry(layer=i, kv_from=m.kv_from if L.type == "attention" else None))
    return ModelSpec(
        config=cfg, embedding=TokenEmbedding(cfg.vocab, W, param_name=""), embedding_prefix="embed",
        blocks=blocks, block_prefixes=prefixes, final_norm=norm(), final_norm_prefix="final.norm",
        head=OutputHead(cfg.vocab, W, param_name=""), head_prefix="head",
        schedule=schedule, vocab_size=cfg.vocab, hidden_size=W, max_position=cfg.max_positions,
        stop_token_ids=[], positions=LearnedPositions(cfg.max_positions, W, param_name=""), positions_prefix="pos")


register_architecture(VilulornConfig.ARCHITECTURE, VilulornConfig, build_vilulorn)
