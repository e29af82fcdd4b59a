"""Causal self-attention over paged keys and values, with grouped query heads, an optional
window and a position encoding applied to q and k before the cache write."""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import Mixer, KVCacheSpec, TensorSpec, PartSpec
from .linear import linear
from .registry import register_part, build_part


class PagedAttention(Mixer):
    """Per row t at position p (src/model.cpp:764-786):

    ``q,k,v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv``; rotate q and k; write k and v to the page
    slot of p; ``out = softmax(q K^T * scale) V`` over keys ``[max(0, p+1-window), p]`` of the same
    request read from the cache (so rows of this step see one another through it); ``out Wo^T``.
    Query head h reads kv head ``h // (Hq / Hkv)`` (src/hip_ops.hip:484).  ``scale`` defaults to
    ``1/sqrt(head_dim)`` (src/model.cpp:710).

    Options beyond that, each off by default: values with a head size of their own (``v_head_dim``); an RMS norm
    over every q and k head before the rotation, with one weight vector per side shared by the heads (``qk_norm_eps``);
    a bias on the output projection (``out_bias``); a *sink* in every softmax, a key with the score ``sink_score``
    and no value, so that ``p_j = exp(s_j) / (exp(sink_score) + sum_i exp(s_i))``; a position encoding that pairs
    neighbouring elements or scales its cosines and sines; no value projection at all (``values_from_keys``: a key
    head as projected, before its norm and rotation, is also the value head, and there is no v tensor); softmax
    weights that stay float32 in the product with the values (``exact_weights``; the tensor-core kernels of the
    default path round them to bfloat16).  ``names`` gives the tensors' names where they are not
    the usual ones (keys: q, k, v, o, q_bias, k_bias, v_bias, o_bias, q_norm, k_norm, head_mix, sink).  A layer that
    uses one of these options runs the general kernels (``ops.qk_prepare_store``, ``ops.paged_attention_general``).

    Four more, which also run the general kernels.  ``keep_first``: with a window, the sequence's first so many
    positions stay visible behind it (row i reads j if ``j <= i`` and ``i - j < window or j < keep_first``), at their
    true positions; their pages are held to the request's end.  ``learned_sink``: the sink's score is a learned
    number per query head (tensor ``sink`` [heads]).  ``head_mix``: the heads' scaled scores are mixed before mask
    and softmax, ``s'_h = sum_g M[h, g] s_g`` with the learned ``M`` (tensor ``head_mix`` [heads, heads]); since a
    score is linear in its query, the rows' queries are mixed instead, once per row (``ops.mix_query_heads``), and a
    score becomes one product with all kv heads' keys side by side.  ``value_position`` (a position encoding over
    the whole value head): the value of position j is turned by j before it is stored, and a head's output at
    position i, the weighted sum of such values, is turned back by i, so that a value enters the output turned by
    ``j - i``.

    Three more of the plain general path.  ``qk_norm_weight`` False: the head norm of q and k has no weight
    tensors (a head is divided by its root mean square and nothing else).  ``qk_norm_after_rotation``: that norm
    follows the turn instead of preceding it (with a position encoding whose cosines and sines carry an amplitude,
    or that turns part of a head, the two orders differ).  ``score_softcap`` > 0: a scaled score s becomes
    ``score_softcap * tanh(s / score_softcap)`` before mask and softmax.  ``round_weights``: a bfloat16 run of
    this path rounds the softmax weights (computed in float32) to bfloat16 for their product with the values, as it
    rounds every other operand of a product, instead of taking them in as three bfloat16 terms.
    """

    _NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
              "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias",
              "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "head_mix": "head_mix", "sink": "sink"}

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, bias: bool,
                 position: PartSpec, window: int = 0, scale: float | None = None, v_head_dim: int | None = None,
                 qk_norm_eps: float | None = None, out_bias: bool = False, sink_score: float | None = None,
                 names: dict | None = None, values_from_keys: bool = False, exact_weights: bool = False,
                 keep_first: int = 0, learned_sink: bool = False, head_mix: bool = False,
                 value_position: PartSpec | None = None, qk_norm_weight: bool = True,
                 qk_norm_after_rotation: bool = False, score_softcap: float = 0.0, round_weights: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden, self.Hq, self.Hkv, self.D = hidden_size, num_heads, num_kv_heads, head_dim
        self.Dv = int(v_head_dim) if v_head_dim else head_dim
        self.bias, self.window, self.out_bias = bias, int(window), bool(out_bias)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.sink_score = None if sink_score is None else float(sink_score)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))
        self.position = build_part("position", position) if isinstance(position, PartSpec) else position
        self.names = dict(self._NAMES, **(names or {}))
        self.values_from_keys = bool(values_from_keys)
        self.qk_norm_weight, self.qk_norm_after = bool(qk_norm_weight), bool(qk_norm_after_rotation)
        self.softcap = float(score_softcap)
        self.weight_terms = 1 if round_weights else 3
        if self.softcap < 0:
            raise ValueError("score_softcap must not be negative")
        if self.values_from_keys and self.Dv != self.D:
            raise ValueError("values that are the keys have the keys' head size")
        if self.values_from_keys and bias:
            raise ValueError("values that are the keys: biased projections are not supported")
        self.keep_first = int(keep_first) if self.window > 0 else 0
        self.learned_sink, self.head_mix = bool(learned_sink), bool(head_mix)
        self.value_position = (build_part("position", value_position) if isinstance(value_position, PartSpec)
                               else value_position)
        if self.keep_first < 0:
            raise ValueError("keep_first must not be negative")
        if self.learned_sink and self.sink_score is not None:
            raise ValueError("a sink has a fixed score or a learned one, not both")
        if self.value_position is not None:
            vp = self.value_position
            if self.values_from_keys or vp.pairing != "halves" or vp.amplitude != 1.0 or vp.rotary_dim > self.Dv:
                raise ValueError("turned values: pairs (i, i + dims / 2) over at most the value head, no amplitude, and "
                                 "values of their own")
        # the options that only the general kernels know, whatever the dtype
        self.extended = bool(self.keep_first or self.learned_sink or self.head_mix or self.value_position is not None)
        if self.extended and self.softcap > 0:
            raise ValueError("capped scores are not supported together with kept positions, learned sinks, mixed heads or turned values")
        self.general = (self.extended or self.softcap > 0 or self.values_from_keys or bool(exact_weights) or self.Dv != self.D or self.qk_norm_eps is not None or self.sink_score is not None
                        or self.position.pairing != "halves" or self.position.amplitude != 1.0)
        if self.general:
            if self.extended:
                if head_dim < 1 or self.Dv < 1 or self.Dv > 512:
                    raise ValueError(f"value heads of {self.Dv} elements are not supported: at most 512")
            elif head_dim < 1 or head_dim > 256 or self.Dv < 1 or self.Dv > 256:
                raise ValueError(f"head sizes {head_dim} / {self.Dv} are not supported: the general attention kernels "
                                 "take up to 256 elements per head")
        elif head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take multiples "
                             "of 16 up to 256")

    # ------------------------------------------------------------------ weights
    def tensor_specs(self, available=None):
        H, q, kv, vv, n = self.hidden, self.Hq * self.D, self.Hkv * self.D, self.Hkv * self.Dv, self.names
        s = {n["q"]: TensorSpec((q, H)), n["k"]: TensorSpec((kv, H)),
             n["v"]: TensorSpec((vv, H)), n["o"]: TensorSpec((H, self.Hq * self.Dv))}
        if self.values_from_keys:
            del s[n["v"]]
        if self.bias:
            s.update({n["q_bias"]: TensorSpec((q,), kind="vector"), n["k_bias"]: TensorSpec((kv,), kind="vector"),
                      n["v_bias"]: TensorSpec((vv,), kind="vector")})
        if self.out_bias:
            s[n["o_bias"]] = TensorSpec((H,), kind="vector")
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            s[n["q_norm"]] = TensorSpec((self.D,), init="ones", kind="vector")
            s[n["k_norm"]] = TensorSpec((self.D,), init="ones", kind="vector")
        if self.head_mix:
            s[n["head_mix"]] = TensorSpec((self.Hq, self.Hq), init="identity", kind="vector")
        if self.learned_sink:
            s[n["sink"]] = TensorSpec((self.Hq,), init="zeros", kind="vector")
        s.update(self.position.tensor_specs(available))      # a position encoding may have tensors of its own
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        n = self.names
        self.position.load(fetch, ctx)
        # q, k and v rows are stacked so that one product makes all three (src/model.cpp:508-513)
        self.qkv_weight = _cat([fetch(n["q"]), fetch(n["k"])] + ([] if self.values_from_keys else [fetch(n["v"])]))
        self.qkv_bias = None
        if self.bias:
            self.qkv_bias = _cat([fetch(n["q_bias"]), fetch(n["k_bias"]), fetch(n["v_bias"])])
        self.o_weight = fetch(n["o"])
        self.o_bias = fetch(n["o_bias"]) if self.out_bias else None
        # The tensor-core kernel wants one head size for q, k and v, a multiple of 16: a bfloat16 run of the general
        # path pads the three with zeros up to it (the scores and the sums are the same), and the output
        # projection gets zero columns for the padding.
        self.pad = 0
        self.mix_weight = fetch(n["head_mix"]).float().contiguous() if self.head_mix else None
        self.sinks = fetch(n["sink"]).float().contiguous() if self.learned_sink else None
        if self.value_position is not None:
            self.value_position.load(fetch, ctx)
        if (self.general and not self.extended and ctx.fast_kernels and ctx.act_dtype == torch.bfloat16
                and self.o_weight.dtype == torch.bfloat16):
            self.pad = (max(self.D, self.Dv) + 15) // 16 * 16
            if self.pad != self.Dv:
                w = torch.zeros((self.hidden, self.Hq, self.pad), dtype=self.o_weight.dtype, device=self.o_weight.device)
                w[:, :, :self.Dv] = self.o_weight.view(self.hidden, self.Hq, self.Dv)
                self.o_weight = w.view(self.hidden, self.Hq * self.pad)
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm, self.k_norm = fetch(n["q_norm"]), fetch(n["k_norm"])

    def cache_spec(self):
        if getattr(self, "pad", 0):
            return KVCacheSpec(self.Hkv, self.pad, self.window)
        return KVCacheSpec(self.Hkv, self.D, self.window, 0 if self.Dv == self.D else self.Dv, self.keep_first)

    # ------------------------------------------------------------------ forward
    def forward(self, h, batch, cache):
        ctx = self.ctx
        T = h.shape[0]
        if self.general:
            return self._forward_general(h, batch, cache)
        qkv = linear(ctx, h, self.qkv_weight, ctx.act_dtype, bias=self.qkv_bias)
        bt = batch.block_tables[cache.group]
        ops.rope_store(qkv, batch.positions, self.position.inv_freq(), self.position.rotary_dim, cache.k, cache.v,
                       bt, batch.row_entry, self.Hq, self.Hkv, self.D, cache.write, ctx.err,
                       rot_positions=self.position.rotation_positions(batch), pair_axis=self.position.pair_axis())
        att = torch.empty((T, self.Hq * self.D), dtype=ctx.act_dtype, device=h.device)
        self._attend(qkv, cache, bt, batch, att)
        return linear(ctx, att, self.o_weight, torch.float32, bias=self.o_bias)

    def _forward_general(self, h, batch, cache):
        """The projections come out in float32 (the head norms read them); q after norm and rotation, and the keys
        and values in their pages, are in the activation dtype; scores, weights and sums are float32."""
        ctx, T = self.ctx, h.shape[0]
        Hq, Hkv, D, Dv = self.Hq, self.Hkv, self.D, self.Dv
        proj = linear(ctx, h, self.qkv_weight, torch.float32, bias=self.qkv_bias)
        bt = batch.block_tables[cache.group]
        if self.extended:
            return self._forward_extended(proj, bt, batch, cache)
        P = self.pad
        q = torch.empty((T, Hq * (P or D)), dtype=ctx.act_dtype, device=h.device)
        pos = self.position
        # (values that are the keys are read where the keys are, as projected: the kernel norms and turns its own copy)
        ops.qk_prepare_store(proj, 0, Hq * D, Hq * D if self.values_from_keys else (Hq + Hkv) * D, batch.positions, batch.row_entry, bt, self.q_norm,
                             self.k_norm, self.qk_norm_eps or 0.0, pos.inv_freq(), pos.rotary_dim,
                             pos.pairing == "interleaved", pos.amplitude, q, cache.k, cache.v, Hq, Hkv, D, Dv,
                             cache.write, ctx.err, norm_always=self.qk_norm_eps is not None,
                             norm_after=self.qk_norm_after)
        att = torch.empty((T, Hq * (P or Dv)), dtype=ctx.act_dtype, device=h.device)
        if P:
            # Entries of one row go to the split-key decode kernel (with weights that keep their float32 bits), the
            # others to a tensor-core kernel (tcgen05 for head sizes 64 and 128 without a sink, else mma.sync), where
            # the float32 weights enter the product with the values as three bfloat16 terms; the decode kernel and
            # the mma.sync kernel add the sink to the softmax's denominator.
            single = batch.n_single if ops.attention_decode_usable(cache.k, P) else 0
            if single:
                ops.attention_decode(q, cache.k, cache.v, bt, batch.row_entry, batch.positions, self.scale, self.window,
                                     att, Hq, Hkv, P, batch.max_context if batch.decode_only else batch.max_single_context,
                                     rows=None if batch.decode_only else batch.single_rows, err=ctx.err,
                                     sink_score=self.sink_score, float_weights=self.weight_terms == 3,
                                     softcap=self.softcap)
            if single < batch.S:
                tiles = (batch.T - single) // ops.attention_prefill_tile_rows() + (batch.S - single)
                ops.attention_prefill(q, cache.k, cache.v, bt, batch.cu_rows, batch.entry_pos0, tiles, self.scale,
                                      self.window, att, Hq, Hkv, P, err=ctx.err, min_rows=2 if single else 1,
                                      kernel="mma" if self.sink_score is not None and self.weight_terms == 3 else "auto",
                                      sink_score=self.sink_score, weight_terms=self.weight_terms, softcap=self.softcap)
        else:
            ops.paged_attention_general(q, cache.k, cache.v, bt, batch.row_entry, batch.positions, self.scale,
                                        self.window, att, Hq, Hkv, D, Dv, sink_score=self.sink_score,
                                        softcap=self.softcap)
        return linear(ctx, att, self.o_weight, torch.float32, bias=self.o_bias)

    def _forward_extended(self, proj, bt, batch, cache):
        """Kept first positions, learned sinks, mixed heads, turned values.  The queries stay float32 from the
        projection to the scores (rotation and mixing included); scores, weights and sums are float32; keys and
        values are in their pages in the activation dtype."""
        ctx, T, dev = self.ctx, proj.shape[0], proj.device
        Hq, Hkv, D, Dv = self.Hq, self.Hkv, self.D, self.Dv
        pos, vp = self.position, self.value_position
        span = Hkv if self.head_mix else 1
        # A bfloat16 run whose sizes the tensor-core kernel takes goes there with all its entries, single rows too:
        # the queries are rounded to bfloat16 once, after rotation and mixing.  Else the general kernel, float32
        # queries against the pages.
        fast = (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
                and self.sink_score is None and self.scale > 0 and ops.attention_prefill_wide_usable(D, span, Dv))
        q = torch.empty((T, Hq * D), dtype=torch.bfloat16 if fast and not self.head_mix else torch.float32, device=dev)
        ops.qk_prepare_store(proj, 0, Hq * D, (Hq + Hkv) * D, batch.positions, batch.row_entry, bt, self.q_norm,
                             self.k_norm, self.qk_norm_eps or 0.0, pos.inv_freq(), pos.rotary_dim,
                             pos.pairing == "interleaved", pos.amplitude, q, cache.k, cache.v, Hq, Hkv, D, Dv,
                             cache.write, ctx.err, v_inv_freq=vp.inv_freq() if vp is not None else None,
                             v_rot_dim=vp.rotary_dim if vp is not None else 0)
        if self.head_mix:
            mixed = torch.empty((T, Hq * Hkv * D), dtype=torch.bfloat16 if fast else torch.float32, device=dev)
            ops.mix_query_heads(q, self.mix_weight, mixed, Hq, Hkv, D)
            q = mixed
        turned = vp is not None and vp.rotary_dim > 0
        att = torch.empty((T, Hq * Dv), dtype=torch.float32 if turned else ctx.act_dtype, device=dev)
        if fast:
            # A step that holds entries of one row sends them to a form of their own: where all query heads read the
            # same keys (mixed heads, or one kv head) and are at most 16, a CTA takes all heads of a row and reads
            # its keys once; else the narrow form, which also takes the step's other short entries (up to 16 rows)
            # and in which a CTA's warps share out the keys of one entry and head.  The longer entries go to the form
            # that gives a warp 16 rows of a tile, in the same step if it holds both kinds.
            short = 0
            if batch.n_single:
                by_heads = ops.attention_wide_heads_usable(D, span, Dv, Hq, Hkv, cache.v.shape[1])
                short = 1 if by_heads else ops.attention_wide_narrow_rows()
                context = batch.max_context if batch.decode_only else max(batch.max_single_context, short)
                keys = min(context, self.window + self.keep_first + short) if self.window > 0 else context
                ops.attention_prefill_wide(q, cache.k, cache.v, bt, batch.cu_rows, batch.entry_pos0, batch.S, self.scale,
                                           self.window, att, Hq, Hkv, D, Dv, keep_first=self.keep_first,
                                           sinks=self.sinks, key_span=span, narrow=True, heads=by_heads, max_keys=keys)
            if batch.n_single < batch.S:
                tiles = batch.T // ops.attention_prefill_wide_tile_rows() + batch.S
                ops.attention_prefill_wide(q, cache.k, cache.v, bt, batch.cu_rows, batch.entry_pos0, tiles, self.scale,
                                           self.window, att, Hq, Hkv, D, Dv, keep_first=self.keep_first,
                                           sinks=self.sinks, key_span=span, min_rows=short + 1)
        else:
            ops.paged_attention_general(q, cache.k, cache.v, bt, batch.row_entry, batch.positions, self.scale,
                                        self.window, att, Hq, Hkv, D, Dv, sink_score=self.sink_score, sinks=self.sinks,
                                        keep_first=self.keep_first, key_span=span)
        if turned:
            back = torch.empty((T, Hq * Dv), dtype=ctx.act_dtype, device=dev)
            ops.rotate_heads(att, batch.positions, vp.inv_freq(), vp.rotary_dim, -1.0, back, Hq, Dv)
            att = back
        return linear(ctx, att, self.o_weight, torch.float32, bias=self.o_bias)

    def _attend(self, qkv, cache, bt, batch, att):
        """Which kernel runs which rows.  float32 runs keep the plain kernel for every row, so that their sums have
        one order however the work is cut.  bfloat16 runs send entries of one row to the split-key decode kernel and
        the other entries to the prefill kernel, in the same step if it holds both kinds."""
        ctx = self.ctx
        if not (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16):
            ops.paged_attention_plain(qkv, cache.k, cache.v, bt, batch.row_entry, batch.positions, self.scale,
                                      self.window, att, self.Hq, self.Hkv, self.D)
            return
        single = batch.n_single if ops.attention_decode_usable(cache.k, self.D) else 0
        if single:
            ops.attention_decode(qkv, cache.k, cache.v, bt, batch.row_entry, batch.positions, self.scale, self.window,
                                 att, self.Hq, self.Hkv, self.D,
                                 batch.max_context if batch.decode_only else batch.max_single_context,
                                 rows=None if batch.decode_only else batch.single_rows, err=ctx.err)
        if single < batch.S:
            tm = ops.attention_prefill_tile_rows()
            min_rows = 2 if single else 1
            # an upper bound of the entries' tiles that depends on the step's totals only (CTAs without a tile leave
            # at once): a captured step serves every step with the same totals, however its rows are cut
            tiles = (batch.T - single) // tm + (batch.S - single)
            ops.attention_prefill(qkv, cache.k, cache.v, bt, batch.cu_rows, batch.entry_pos0, tiles, self.scale,
                                  self.window, att, self.Hq, self.Hkv, self.D, err=ctx.err, min_rows=min_rows)


def _cat(ts):
    if len({t.dtype for t in ts}) > 1:
        ts = [t.float() for t in ts]
    return torch.cat(ts, dim=0).contiguous()


register_part("mixer", "paged_attention", PagedAttention)
