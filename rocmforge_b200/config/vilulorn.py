"""Typed configuration of the Vilulorn decoder, read from its own config.json keys.

config.json gives every size and every constant that differs between models of the design:

    architecture "Vilulorn"; vocab, width, max_positions; norm.eps
    layers[i]: type "gla":        mixer {heads, dim, vdim, tau}
               type "attention":  mixer {heads, kv_heads, dim, vdim, scale, mask.size, rot {dims, base, scaling
                                  {factor, low, high, original} (optional)}, kv_from (optional: the layer whose keys and
                                  values this one reads)}
               mlp null | {kind "moe", expert {ff, limit}, router {experts, top}}

The rank of a gla layer's decay projection is no key: it is the shape of the layer's ``mix.a1`` tensor, which the
loader hands to ``from_dict`` as ``shapes``.  What the design fixes (activation functions, the constant 1.702 of the
experts' gate, where norms sit, how rotated pairs lie) is in the parts and in the builder.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from .errors import InvalidValue, MissingKey
from .rifizen import _get


@dataclass
class GlaConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int                      # rows of mix.a1


@dataclass
class ChunkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[Dict[str, float]]
    kv_from: Optional[int]


@dataclass
class ExpertsConfig:
    ff: int
    limit: float
    experts: int
    top: int


@dataclass
class VilulornLayer:
    type: str                      # "gla" | "attention"
    mixer: object
    mlp: Optional[ExpertsConfig]


@dataclass
class VilulornConfig:
    architecture: str
    vocab: int
    width: int
    max_positions: int
    eps: float
    layers: List[VilulornLayer]
    raw: dict = field(default_factory=dict, repr=False)

    ARCHITECTURE = "Vilulorn"
    DEFAULT_DECAY_RANK = 16        # where no tensor shapes are at hand (a model made from a configuration alone)
    SHAPES_FROM_TENSORS = True     # the loader passes the folder's tensor shapes to from_dict

    @classmethod
    def from_dict(cls, raw: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "VilulornConfig":
        layers_raw = raw.get("layers")
        if layers_raw is None:
            raise MissingKey("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise InvalidValue("layers", layers_raw, "must be a non-empty list")
        layers: List[VilulornLayer] = []
        for i, L in enumerate(layers_raw):
            p = f"layers[{i}]"
            if not isinstance(L, dict):
                raise InvalidValue(p, L, "must be an object")
            kind = L.get("type")

            def g(path, k, L=L, p=p, **kw):
                return _get(L, path, k, where=p + ".", **kw)
            if kind == "gla":
                rank = None
                if shapes is not None and f"l{i}.mix.a1" in shapes:
                    rank = int(shapes[f"l{i}.mix.a1"][0])
                mixer = GlaConfig(heads=g("mixer.heads", int, minimum=1), dim=g("mixer.dim", int, minimum=1),
                                  vdim=g("mixer.vdim", int, minimum=1), tau=g("mixer.tau", float, positive=True),
                                  rank=int(rank) if rank else cls.DEFAULT_DECAY_RANK)
                if mixer.dim > 256:
                    raise InvalidValue(f"{p}.mixer.dim", mixer.dim, "the recurrence kernel holds at most 256 rows of a state column")
            elif kind == "attention":
                scaling = (L.get("mixer", {}).get("rot", {}) or {}).get("scaling")
                if scaling is not None:
                    scaling = {k: g(f"mixer.rot.scaling.{k}", float, positive=(k != "low")) for k in ("factor", "low", "high", "original")}
                    if not scaling["high"] > scaling["low"]:
                        raise InvalidValue(f"{p}.mixer.rot.scaling", scaling, "needs high > low")
                mixer = ChunkAttentionConfig(
                    heads=g("mixer.heads", int, minimum=1), kv_heads=g("mixer.kv_heads", int, minimum=1),
                    dim=g("mixer.dim", int, minimum=1), vdim=g("mixer.vdim", int, minimum=1),
                    scale=g("mixer.scale", float, positive=True), chunk=g("mixer.mask.size", int, minimum=1),
                    rot_dims=g("mixer.rot.dims", int, minimum=0), rot_base=g("mixer.rot.base", float, positive=True),
                    rot_scaling=scaling, kv_from=g("mixer.kv_from", int, optional=True, minimum=0))
                if mixer.heads % mixer.kv_heads:
                    raise InvalidValue(f"{p}.mixer.kv_heads", mixer.kv_heads, f"must divide heads = {mixer.heads}")
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                    raise InvalidValue(f"{p}.mixer.rot.dims", mixer.rot_dims, f"must be even and at most dim = {mixer.dim}")
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    src = layers[j] if j < i else None
                    if src is None or src.type != "attention" or src.mixer.kv_from is not None:
                        raise InvalidValue(f"{p}.mixer.kv_from", j, "must name an earlier attention layer with keys and values of its own")
                    same = all(getattr(src.mixer, k) == getattr(mixer, k) for k in
                               ("kv_heads", "dim", "vdim", "rot_dims", "rot_base", "rot_scaling"))
                    if not same:
                        raise InvalidValue(f"{p}.mixer.kv_from", j, "the two layers' kv heads, head sizes and rotation must be equal")
            else:
                raise InvalidValue(f"{p}.type", kind, "this design has layers of type 'gla' and 'attention'")
            mlp_raw = L.get("mlp")
            mlp = None
            if mlp_raw is not None:
                mk = mlp_raw.get("kind") if isinstance(mlp_raw, dict) else None
                if mk != "moe":
                    raise InvalidValue(f"{p}.mlp.kind", mk, "must be 'moe' (or mlp null)")
                mlp = ExpertsConfig(ff=g("mlp.expert.ff", int, minimum=1), limit=g("mlp.expert.limit", float, positive=True),
                                    experts=g("mlp.router.experts", int, minimum=1), top=g("mlp.router.top", int, minimum=1))
                if mlp.top > mlp.experts:
                    raise InvalidValue(f"{p}.mlp.router.top", mlp.top, f"there are only {mlp.experts} experts")
                if mlp.top > 16 or mlp.experts > 1024:
                    raise InvalidValue(f"{p}.mlp.router", mlp_raw.get("router"), "the routing kernels take up to 16 of up to 1024 experts")
            layers.append(VilulornLayer(kind, mixer, mlp))
        return cls(architecture=str(raw.get("architecture") or cls.ARCHITECTURE),
                   vocab=_get(raw, "vocab", int, minimum=1), width=_get(raw, "width", int, minimum=1),
                   max_positions=_get(raw, "max_positions", int, minimum=1),
                   eps=_get(raw, "norm.eps", float, positive=True), layers=layers, raw=copy.deepcopy(raw))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)
