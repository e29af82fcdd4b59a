"""Sanesun described as parts, layer by layer.

A decoder whose layers read the residual stream once: ``h = rms(x) w``, ``x += mixer(h) + mlp(h)`` (a layer may have
no MLP); the stream starts as the embedding row times a constant.  Three mixers:

* ``channel_delta``: a gated delta rule with short convolutions whose decay is one number per head and key channel
  (through a low-rank pair) and whose output gate is a sigmoid through another low-rank pair;
* ``attention``: grouped-query softmax attention with biased projections, part of q and k turned by the position
  (halves pairing), values turned by their own position over the whole head and the summed output turned back by
  the reader's, scores mixed across heads by a learned matrix before the softmax, a sliding window behind which the
  sequence's first tokens stay visible, and a learned sink per head in the softmax's denominator;
* ``latent_attention``: causal attention without positions whose keys and values are both made from one small
  normed vector per token (the only thing cached), queries through a normed low-rank step, a sigmoid gate per head.

The feed-forward is a dense two-matrix MLP with the xIELU activation (two learned numbers per layer).  Tensor names:
``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.up|down|act``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sanesun_config import (ARCHITECTURE, SanesunConfig, ChannelDeltaConfig, WindowAttentionConfig,
                                     LatentAttentionConfig)
from ..parts import PartSpec, LayerSpec, ModelSpec


def _norm(cfg: SanesunConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.eps, weight_name=name))


def _mixer(cfg: SanesunConfig, m) -> PartSpec:
    W, eps = cfg.hidden_size, cfg.eps
    if isinstance(m, ChannelDeltaConfig):
        return PartSpec("gated_delta_rule", dict(
            hidden_size=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, conv=m.conv, eps=eps,
            channel_decay=True, low_rank_gate=True, gate="sigmoid", decay_rank=m.decay_rank or None,
            gate_rank=m.gate_rank or None))
    if isinstance(m, WindowAttentionConfig):
        position, value_position = PartSpec("none"), None
        if m.rot_base > 0:
            if m.rot_dims:
                position = PartSpec("rotary_neox", dict(rotary_dim=m.rot_dims, theta=m.rot_base))
            value_position = PartSpec("rotary_neox", dict(rotary_dim=m.vdim, theta=m.rot_base))
        names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                 "head_mix": "talk", "sink": "sink"}
        return PartSpec("paged_attention", dict(
            hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim, bias=True,
            scale=m.scale, window=m.window, keep_first=m.keep_first, learned_sink=True, head_mix=True,
            position=position, value_position=value_position, names=names))
    if isinstance(m, LatentAttentionConfig):
        return PartSpec("latent_attention", dict(hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, q_rank=m.q_rank,
                                                 kv_rank=m.kv_rank, scale=m.scale, eps=eps))
    raise TypeError(type(m))


def build_spec(cfg: SanesunConfig) -> ModelSpec:
    layers = []
    for L in cfg.layers:
        parts = {"norm1": _norm(cfg, "norm1"), "mixer": _mixer(cfg, L.mixer)}
        if L.mlp_ff:
            parts["feed_forward"] = PartSpec("dense_mlp", dict(hidden_size=cfg.hidden_size, intermediate_size=L.mlp_ff,
                                                               activation="xielu", up_name="up", down_name="down",
                                                               act_name="act"))
        layers.append(LayerSpec(arrangement="parallel", parts=parts,
                                names={"norm1": "", "mixer": "mix.", "feed_forward": "mlp."}))
    return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers,
                     final_norm=_norm(cfg, "final.norm"), tie_word_embeddings=False, embed_scale=cfg.embed_scale,
                     embed_name="embed", layer_prefix="l{}.", final_norm_prefix="", lm_head_name="head")


register_architecture(ARCHITECTURE, SanesunConfig.from_dict, build_spec)
