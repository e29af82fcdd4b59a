"""Typed view of a Gekitar ``config.json``.

The file lists its layers one by one: ``layers[i] = {"type", "mixer", "mlp"}``.  ``type`` names the mixer
(``latent_attention``, ``latent_attention_2``, ``attention``; a further numeric suffix, as in ``attention_3``, marks
another set of sizes of the same kind), ``mixer`` holds its sizes and constants, ``mlp`` the feed-forward or null for
a layer without one.

* ``latent_attention`` (every earlier position is seen, the heads' outputs are gated element by element) and
  ``latent_attention_2`` (a sliding window ``mask.size``, no gate): ``heads``, ``dim``, ``rot_dim``, ``vdim``,
  ``q_rank``, ``kv_rank``, ``scale``, ``rot.dims`` (= ``rot_dim``), ``rot.base``.  ``kv_from: j`` (on
  ``latent_attention_2``): the layer has no down-projection to the latent of its own and reads what layer j keeps;
  layer j makes its own, and its latent size, ``rot_dim`` and rotation are this layer's.
* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``, ``rot.dims``, ``rot.base`` and
  optionally ``rot.scaling`` = ``{factor, original, fast, slow}``.
* ``mlp.kind`` ``dense``: ``ff``, ``limit``.  ``moe``: ``router.experts``, ``router.top``, ``expert.ff`` and
  optionally ``shared.ff``.

Top level: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``.  Every size and constant is read from the file; a
missing key, a wrong type or an unknown kind is an error that names the key.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .fields import need as _need, positive as _positive
from .model_config import ConfigError

ARCHITECTURE = "Gekitar"


def _rotation(d: dict, where: str, most: int):
    """(dims, base, scaling or None) of a mixer's ``rot``; without ``rot`` nothing is turned."""
    rot = d.get("rot")
    if rot is None:
        return 0, 0.0, None
    w = where + ".rot"
    dims = _need(rot, "dims", int, w)
    if dims < 0 or dims % 2 or dims > most:
        raise ConfigError(f"config.json: '{w}.dims' must be even, not negative and at most {most}")
    base = _need(rot, "base", float, w)
    if dims and (base <= 0 or base == 1.0):
        raise ConfigError(f"config.json: '{w}.base' must be positive and not 1")
    scaling = None
    if rot.get("scaling") is not None:
        sc = _need(rot, "scaling", dict, w)
        scaling = {k: _need(sc, k, float, w + ".scaling") for k in ("factor", "original", "fast", "slow")}
        if scaling["factor"] <= 0 or scaling["original"] <= 0 or scaling["fast"] <= 0 or scaling["slow"] <= 0:
            raise ConfigError(f"config.json: the numbers of '{w}.scaling' must be positive")
    return dims, base, scaling


@dataclass
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_scaling: Optional[dict]
    window: int                       # 0: every earlier position is seen
    gated: bool
    kv_from: Optional[int]            # the layer whose latents this one reads (None: its own)

    @classmethod
    def from_dict(cls, d: dict, where: str, second: bool) -> "LatentConfig":
        heads = _positive(_need(d, "heads", int, where), where + ".heads")
        dim = _positive(_need(d, "dim", int, where), where + ".dim")
        vdim = _positive(_need(d, "vdim", int, where, default=dim, required=False), where + ".vdim")
        rq = _positive(_need(d, "q_rank", int, where), where + ".q_rank")
        rk = _positive(_need(d, "kv_rank", int, where), where + ".kv_rank")
        rot_dim = _need(d, "rot_dim", int, where, default=0, required=False)
        if rot_dim < 0 or rot_dim % 2:
            raise ConfigError(f"config.json: '{where}.rot_dim' must be even and not negative")
        dims, base, scaling = _rotation(d, where, rot_dim)
        if dims != rot_dim:
            raise ConfigError(f"config.json: '{where}.rot.dims' must equal '{where}.rot_dim'")
        window = 0
        if second:
            window = _positive(_need(_need(d, "mask", dict, where), "size", int, where + ".mask"), where + ".mask.size")
        kv_from = d.get("kv_from")
        if kv_from is not None:
            kv_from = _need(d, "kv_from", int, where)
        return cls(heads, dim, rot_dim, vdim, rq, rk, _need(d, "scale", float, where), base, scaling, window,
                   not second, kv_from)


@dataclass
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                    # 0: scores are not capped
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[dict]

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "SinkAttentionConfig":
        heads = _positive(_need(d, "heads", int, where), where + ".heads")
        kv = _positive(_need(d, "kv_heads", int, where, default=heads, required=False), where + ".kv_heads")
        if heads % kv:
            raise ConfigError(f"config.json: '{where}.heads' must be a multiple of '{where}.kv_heads'")
        dim = _positive(_need(d, "dim", int, where), where + ".dim")
        vdim = _positive(_need(d, "vdim", int, where, default=dim, required=False), where + ".vdim")
        dims, base, scaling = _rotation(d, where, dim)
        cap = _need(d, "softcap", float, where, default=0.0, required=False)
        if cap < 0:
            raise ConfigError(f"config.json: '{where}.softcap' must not be negative")
        return cls(heads, kv, dim, vdim, _need(d, "scale", float, where), cap, dims, base, scaling)


@dataclass
class MlpConfig:
    kind: str                         # "dense" | "moe"
    ff: int                           # dense: its width; moe: an expert's
    limit: float = 0.0                # dense: the clamp of both halves
    experts: int = 0
    top: int = 0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MlpConfig":
        kind = _need(d, "kind", str, where)
        if kind == "dense":
            limit = _need(d, "limit", float, where)
            if limit <= 0:
                raise ConfigError(f"config.json: '{where}.limit' must be positive")
            return cls("dense", _positive(_need(d, "ff", int, where), where + ".ff"), limit)
        if kind == "moe":
            r = _need(d, "router", dict, where)
            experts = _positive(_need(r, "experts", int, where + ".router"), where + ".router.experts")
            top = _positive(_need(r, "top", int, where + ".router"), where + ".router.top")
            if top > experts:
                raise ConfigError(f"config.json: '{where}.router.top' must be at most '{where}.router.experts'")
            ff = _positive(_need(_need(d, "expert", dict, where), "ff", int, where + ".expert"), where + ".expert.ff")
            shared = 0
            if d.get("shared") is not None:
                shared = _positive(_need(_need(d, "shared", dict, where), "ff", int, where + ".shared"), where + ".shared.ff")
            return cls("moe", ff, 0.0, experts, top, shared)
        raise ConfigError(f"config.json: '{where}.kind' is {kind!r}; known: dense, moe")


MIXER_KINDS = ("latent_attention", "latent_attention_2", "attention")


def _kind_of(name: str):
    """``latent_attention_2`` is a kind of its own; a further numeric suffix marks another set of sizes."""
    if name in MIXER_KINDS:
        return name
    head, sep, tail = name.rpartition("_")
    if sep and tail.isdigit() and head in MIXER_KINDS:
        return head
    return None


@dataclass
class GekitarLayer:
    type: str
    kind: str
    mixer: object
    mlp: Optional[MlpConfig]


@dataclass
class GekitarConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    eps: float
    embed_scale: float
    layers: list = field(default_factory=list)
    raw: dict = field(default_factory=dict)
    eos_token_id: int = -1

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: dict) -> "GekitarConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            typ = _need(L, "type", str, where)
            kind = _kind_of(typ)
            if kind is None:
                raise ConfigError(f"config.json: '{where}.type' is {typ!r}; known: {', '.join(MIXER_KINDS)} "
                                  "(with a numeric suffix for further sets of sizes)")
            md = _need(L, "mixer", dict, where)
            if kind == "attention":
                mixer = SinkAttentionConfig.from_dict(md, where + ".mixer")
            else:
                mixer = LatentConfig.from_dict(md, where + ".mixer", second=kind == "latent_attention_2")
            mlp = MlpConfig.from_dict(L["mlp"], where + ".mlp") if L.get("mlp") is not None else None
            layers.append(GekitarLayer(typ, kind, mixer, mlp))
        for i, L in enumerate(layers):
            m = L.mixer
            if isinstance(m, LatentConfig) and m.kv_from is not None:
                where = f"layers[{i}].mixer.kv_from"
                j = m.kv_from
                if not (0 <= j < i) or not isinstance(layers[j].mixer, LatentConfig) or layers[j].mixer.kv_from is not None:
                    raise ConfigError(f"config.json: '{where}' must name an earlier latent-attention layer that makes its own latents")
                o = layers[j].mixer
                if (o.kv_rank, o.rot_dim, o.rot_base, o.rot_scaling) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_scaling):
                    raise ConfigError(f"config.json: '{where}': layer {j}'s kv_rank, rot_dim and rot must equal this layer's")
        eps = _need(_need(d, "norm", dict, ""), "eps", float, "norm")
        scale = 1.0
        if d.get("embedding") is not None:
            scale = _need(d["embedding"], "scale", float, "embedding", default=1.0, required=False)
        eos = d.get("eos_token_id", -1)
        return cls(architecture=d.get("architecture", ARCHITECTURE),
                   vocab_size=_positive(_need(d, "vocab", int, ""), "vocab"),
                   hidden_size=_positive(_need(d, "width", int, ""), "width"),
                   eps=eps, embed_scale=scale, layers=layers, raw=dict(d),
                   eos_token_id=int(eos) if isinstance(eos, int) and not isinstance(eos, bool) else -1)

    def to_dict(self) -> dict:
        return dict(self.raw)
