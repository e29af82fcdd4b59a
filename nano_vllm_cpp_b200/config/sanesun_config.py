"""Typed view of a Sanesun ``config.json``.

The file lists its layers one by one: ``layers[i] = {"type", "mixer", "mlp"}``.  ``type`` names the mixer
(``channel_delta``, ``attention``, ``latent_attention``; a numeric suffix, as in ``attention_2``, marks a further set
of sizes of the same kind), ``mixer`` holds its sizes and constants, ``mlp`` the feed-forward
(``{"kind": "dense", "ff"}``) or null for a layer without one.

* ``channel_delta``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps).  The ranks of its two low-rank
  pairs are the tensors' (``decay_rank`` / ``gate_rank`` may name them for random weights).
* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``mask.keep_first``,
  ``rot.dims``, ``rot.base``.  Without ``mask`` every earlier position is seen; without ``rot`` nothing is turned,
  the values neither.
* ``latent_attention``: ``heads``, ``dim``, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``.

Top level: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``.  Every size and constant is read from the file; a
missing key, a wrong type or an unknown kind is an error that names the key.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .fields import need as _need, positive as _positive
from .model_config import ConfigError

ARCHITECTURE = "Sanesun"


@dataclass
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int = 0               # 0: the tensors' own (random weights then take a default)
    gate_rank: int = 0

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ChannelDeltaConfig":
        heads = _positive(_need(d, "heads", int, where), where + ".heads")
        kv = _positive(_need(d, "kv_heads", int, where, default=heads, required=False), where + ".kv_heads")
        if heads % kv:
            raise ConfigError(f"config.json: '{where}.heads' must be a multiple of '{where}.kv_heads'")
        dim = _positive(_need(d, "dim", int, where), where + ".dim")
        vdim = _positive(_need(d, "vdim", int, where, default=dim, required=False), where + ".vdim")
        conv = _positive(_need(d, "conv", int, where), where + ".conv")
        dr = _need(d, "decay_rank", int, where, default=0, required=False)
        gr = _need(d, "gate_rank", int, where, default=0, required=False)
        if dr < 0 or gr < 0:
            raise ConfigError(f"config.json: the ranks of '{where}' must not be negative")
        return cls(heads, kv, dim, vdim, conv, dr, gr)


@dataclass
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                       # 0: every earlier position is seen
    keep_first: int                   # with a window: the first so many positions stay visible
    rot_dims: int                     # 0: q and k are not turned
    rot_base: float                   # 0: no rotation at all (values neither)

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "WindowAttentionConfig":
        heads = _positive(_need(d, "heads", int, where), where + ".heads")
        kv = _positive(_need(d, "kv_heads", int, where, default=heads, required=False), where + ".kv_heads")
        if heads % kv:
            raise ConfigError(f"config.json: '{where}.heads' must be a multiple of '{where}.kv_heads'")
        dim = _positive(_need(d, "dim", int, where), where + ".dim")
        vdim = _positive(_need(d, "vdim", int, where, default=dim, required=False), where + ".vdim")
        window = keep = 0
        if d.get("mask") is not None:
            window = _positive(_need(d["mask"], "size", int, where + ".mask"), where + ".mask.size")
            keep = _need(d["mask"], "keep_first", int, where + ".mask", default=0, required=False)
            if keep < 0:
                raise ConfigError(f"config.json: '{where}.mask.keep_first' must not be negative")
        dims, base = 0, 0.0
        rot = d.get("rot")
        if rot is not None:
            dims = _need(rot, "dims", int, where + ".rot")
            if dims < 0 or dims % 2 or dims > dim:
                raise ConfigError(f"config.json: '{where}.rot.dims' must be even, not negative and at most '{where}.dim'")
            base = _need(rot, "base", float, where + ".rot")
            if base <= 0 or base == 1.0:
                raise ConfigError(f"config.json: '{where}.rot.base' must be positive and not 1")
            if vdim % 2:
                raise ConfigError(f"config.json: '{where}.vdim' must be even (the values are turned in pairs)")
        return cls(heads, kv, dim, vdim, _need(d, "scale", float, where), window, keep, dims, base)


@dataclass
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "LatentAttentionConfig":
        heads = _positive(_need(d, "heads", int, where), where + ".heads")
        dim = _positive(_need(d, "dim", int, where), where + ".dim")
        vdim = _positive(_need(d, "vdim", int, where, default=dim, required=False), where + ".vdim")
        rq = _positive(_need(d, "q_rank", int, where), where + ".q_rank")
        rk = _positive(_need(d, "kv_rank", int, where), where + ".kv_rank")
        return cls(heads, dim, vdim, rq, rk, _need(d, "scale", float, where))


MIXER_KINDS = {"channel_delta": ChannelDeltaConfig, "attention": WindowAttentionConfig,
               "latent_attention": LatentAttentionConfig}
MLP_KINDS = ("dense",)


def _kind_of(name: str, table):
    head, sep, tail = name.rpartition("_")
    if sep and tail.isdigit() and head:
        name = head
    return name if name in table else None


@dataclass
class SanesunLayer:
    type: str
    mixer: object
    mlp_ff: int                       # 0: the layer has no feed-forward


@dataclass
class SanesunConfig:
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
    def from_dict(cls, d: dict) -> "SanesunConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            typ = _need(L, "type", str, where)
            kind = _kind_of(typ, MIXER_KINDS)
            if kind is None:
                raise ConfigError(f"config.json: '{where}.type' is {typ!r}; known: {', '.join(sorted(MIXER_KINDS))} "
                                  "(with a numeric suffix for further sets of sizes)")
            mixer = MIXER_KINDS[kind].from_dict(_need(L, "mixer", dict, where), where + ".mixer")
            ff = 0
            if L.get("mlp") is not None:
                mk = _need(L["mlp"], "kind", str, where + ".mlp")
                if _kind_of(mk, MLP_KINDS) is None:
                    raise ConfigError(f"config.json: '{where}.mlp.kind' is {mk!r}; known: {', '.join(MLP_KINDS)}")
                ff = _positive(_need(L["mlp"], "ff", int, where + ".mlp"), where + ".mlp.ff")
            layers.append(SanesunLayer(typ, mixer, ff))
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
