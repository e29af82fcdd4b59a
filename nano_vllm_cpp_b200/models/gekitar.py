"""Gekitar described as parts, layer by layer.

A decoder whose layers norm every sublayer's input and output, ``x += n1b(mixer(n1(x))); x += n2b(ff(n2(x)))``, with
RMS norms whose stored weights lie around zero (the multiplier is one plus the weight); the stream starts as the
embedding row times a constant.  Three mixers:

* ``latent_attention``: keys and values made from one small normed vector per token plus a small key part that all
  heads share and that is turned by the position (neighbouring pairs); queries through a normed low-rank step, their
  last elements turned the same way; causal; the concatenated heads gated element by element by a sigmoid;
* ``latent_attention_2``: the same through a sliding window and without the gate; with ``kv_from`` it makes no
  latents of its own and reads the pages of the layer named, with its own up-projections, queries and window;
* ``attention``: grouped-query attention with biases on all four projections, part of a head turned in neighbouring
  pairs with stretched slow frequencies and an amplitude, q and k heads divided by their root mean square after the
  turn, capped scores, and a sink of score zero in the softmax's denominator.

Two feed-forwards: a dense one whose gate and up halves are clamped (``g sigmoid(1.702 g) (u + 1)``), and a mixture
of squared-relu experts (softmax router, the chosen scores renormed) with a shared expert scaled by one sigmoid per
token.  Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.gekitar_config import ARCHITECTURE, GekitarConfig, LatentConfig, SinkAttentionConfig
from ..parts import PartSpec, LayerSpec, ModelSpec
from ..parts.model import LayerCall

GLU_SLOPE = 1.702       # the sigmoid's slope in the dense feed-forward


def _norm(cfg: GekitarConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.eps, weight_offset=1.0, weight_name=name))


def _rotation(dims: int, base: float, scaling) -> PartSpec:
    if not dims:
        return PartSpec("none")
    return PartSpec("rotary_interleaved", dict(rotary_dim=dims, theta=base, scaling=scaling))


def _mixer(cfg: GekitarConfig, i: int) -> PartSpec:
    W, eps, m = cfg.hidden_size, cfg.eps, cfg.layers[i].mixer
    if isinstance(m, SinkAttentionConfig):
        names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                 "o_bias": "o.b"}
        return PartSpec("paged_attention", dict(
            hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim, bias=True,
            out_bias=True, scale=m.scale, position=_rotation(m.rot_dims, m.rot_base, m.rot_scaling), qk_norm_eps=eps,
            qk_norm_weight=False, qk_norm_after_rotation=True, score_softcap=m.softcap, sink_score=0.0,
            round_weights=True, names=names))
    if isinstance(m, LatentConfig):
        # the pages of a layer that others read are kept for the longest window among their readers
        windows = [m.window] + [L.mixer.window for L in cfg.layers
                                if isinstance(L.mixer, LatentConfig) and L.mixer.kv_from == i]
        keep = 0 if min(windows) == 0 else max(windows)
        return PartSpec("latent_attention", dict(
            hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale,
            eps=eps, output_gate=m.gated, gate_each=True, rot_dim=m.rot_dim,
            position=_rotation(m.rot_dim, m.rot_base, m.rot_scaling) if m.rot_dim else None, window=m.window,
            cache_window=keep, own_kv=m.kv_from is None, exact_weights=False))
    raise TypeError(type(m))


def _feed_forward(cfg: GekitarConfig, mlp) -> PartSpec:
    W = cfg.hidden_size
    if mlp.kind == "dense":
        return PartSpec("dense_swiglu", dict(hidden_size=W, intermediate_size=mlp.ff, clamp_limit=mlp.limit,
                                             slope=GLU_SLOPE, names={"gate": "gate", "up": "up", "down": "down"}))
    names = {"router": "router", "expert_up": "e{}.up", "expert_down": "e{}.down", "shared_up": "shared.up",
             "shared_down": "shared.down", "shared_gate": "shared.sg"}
    return PartSpec("sparse_moe_swiglu", dict(
        hidden_size=W, num_experts=mlp.experts, top_k=mlp.top, intermediate_size=mlp.ff,
        shared_intermediate_size=mlp.shared_ff, renormalize=True, expert_activation="relu2", names=names))


def build_spec(cfg: GekitarConfig) -> ModelSpec:
    layers, order = [], []
    for i, L in enumerate(cfg.layers):
        parts = {"norm1": _norm(cfg, "norm1"), "mixer": _mixer(cfg, i), "norm1b": _norm(cfg, "norm1b")}
        if L.mlp is not None:
            parts.update({"norm2": _norm(cfg, "norm2"), "feed_forward": _feed_forward(cfg, L.mlp),
                          "norm2b": _norm(cfg, "norm2b")})
        layers.append(LayerSpec(arrangement="sandwich", parts=parts,
                                names={"norm1": "", "norm1b": "", "norm2": "", "norm2b": "", "mixer": "mix.",
                                       "feed_forward": "mlp."}))
        order.append(LayerCall(i, cache_of=getattr(L.mixer, "kv_from", None)))
    return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers, order=order,
                     final_norm=_norm(cfg, "final.norm"), tie_word_embeddings=False, embed_scale=cfg.embed_scale,
                     embed_name="embed", layer_prefix="l{}.", final_norm_prefix="", lm_head_name="head")


register_architecture(ARCHITECTURE, GekitarConfig.from_dict, build_spec)
