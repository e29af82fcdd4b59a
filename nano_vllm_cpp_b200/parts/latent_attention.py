"""Attention whose keys and values are made from one small vector per token, which is all its cache keeps."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, KVCacheSpec, TensorSpec, PartSpec
from .linear import linear
from .registry import register_part, build_part


class LatentAttention(Mixer):
    """Causal softmax attention through latents.  Per row, with ``rms`` the RMS norm (``eps``, plain weights):

        c_q = rms(W_dq h) w_dq;   q_h = W_uq[h] c_q        (heads of ``dim`` elements)
        c   = rms(W_dkv h) w_dkv                           (``kv_rank`` elements: what the cache keeps per token)
        k_h(j) = W_uk[h] c(j);   v_h(j) = W_uv[h] c(j)     (values of ``vdim`` elements)
        o_h = sum_j softmax_j(scale q_h . k_h(j)) v_h(j) over j <= i;   out = W_o (sigmoid(W_g h)_h o_h)

    Keys and values are never formed: ``q_h . k_h(j) = (W_uk[h]^T q_h) . c(j)`` and
    ``sum_j p_j v_h(j) = W_uv[h] sum_j p_j c(j)``, so every head attends with a query of ``kv_rank`` elements over
    the one shared row ``c(j)``, which is key and value at once, and its output is projected by ``W_uv[h]``
    afterwards (``ops.head_project`` does both small products per head, in float32 with the weights as stored).  The
    page pool therefore holds one array of ``kv_rank`` elements per token and layer.  ``output_gate`` False leaves
    the sigmoid gate out.  ``names`` renames the tensors (keys: dq, dq_norm, uq, dkv, dkv_norm, uk, uv, g, o).

    Options, each off by default.

    ``rot_dim`` > 0 with ``position`` (a position encoding over ``rot_dim`` elements): a query head has ``rot_dim``
    further elements behind its ``dim``, ``W_dkv`` has ``rot_dim`` further rows behind the latent's, not normed: one
    key part that all heads share; both are turned by their positions, and a score is
    ``scale (q_h[:dim] . k_h(j) + q_h[dim:] . r(j))``.  The cached row is then ``[c(j), r(j)]`` (the key part after
    its turn), a head's query over it ``[W_uk[h]^T q_h[:dim], turned q_h[dim:]]``, and what the weighted sum of
    the rows holds behind its first ``kv_rank`` elements meets zero rows of ``W_uv[h]``.

    ``window`` > 0: row i reads only ``j`` with ``i - j < window``.  ``cache_window``: the window that the pages are
    kept for, where another layer with a longer one reads them too (0: every page stays; default: ``window``).

    ``gate_each``: the gate has one column per element of the concatenated heads (``W_g`` is
    [heads * vdim, hidden]) instead of one per head.

    ``own_kv`` False: the layer has no ``W_dkv`` and no norm of it; its call reads the pages of an earlier call (whose
    latent size, ``rot_dim`` and position encoding are the same) with its own ``W_uk``, ``W_uv``, queries and
    window, and writes none.

    ``exact_weights`` False: a bfloat16 run rounds the softmax weights (computed in float32) to bfloat16 for their
    product with the cached rows, as it rounds every other operand of a product, instead of taking them in as three
    bfloat16 terms."""

    TC_HEADS_MIN_ROWS = 64      # steps of more rows make the per-head products on the tensor cores (bfloat16 runs)

    _NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
              "uv": "uv", "g": "g", "o": "o"}

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float,
                 eps: float, output_gate: bool = True, names: dict | None = None, rot_dim: int = 0,
                 position: PartSpec | None = None, window: int = 0, cache_window: int | None = None,
                 gate_each: bool = False, own_kv: bool = True, exact_weights: bool = True):
        if min(heads, dim, vdim, q_rank, kv_rank) < 1 or rot_dim < 0 or window < 0:
            raise ValueError("latent attention: every size must be positive")
        if kv_rank + rot_dim > 1024:
            raise ValueError(f"a cached row of {kv_rank + rot_dim} elements is not supported: the attention kernel takes up to 1024")
        self.hidden, self.H, self.D, self.Dv, self.rq, self.rk = hidden_size, heads, dim, vdim, q_rank, kv_rank
        self.scale, self.eps, self.output_gate = float(scale), float(eps), bool(output_gate)
        self.names = dict(self._NAMES, **(names or {}))
        self.R, self.window = int(rot_dim), int(window)
        self.P = self.rk + self.R                                   # elements of a cached row
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window and (not self.window or self.cache_window < self.window):
            raise ValueError("latent attention: the pages must be kept for at least the layer's own window")
        self.gate_each, self.own_kv = bool(gate_each), bool(own_kv)
        self.weight_terms = 3 if exact_weights else 1
        self.position = build_part("position", position) if isinstance(position, PartSpec) else position
        if self.R:
            if self.position is None or self.position.rotary_dim != self.R:
                raise ValueError("latent attention: rot_dim comes with a position encoding over rot_dim elements")
            if self.position.rotation_positions(None) is not None or self.position.pair_axis() is not None:
                raise ValueError("latent attention: the shared key part is turned by the row's place in its sequence")

    def tensor_specs(self, available=None):
        W, H, D, Dv, rq, rk, n = self.hidden, self.H, self.D, self.Dv, self.rq, self.rk, self.names
        s = {n["dq"]: TensorSpec((rq, W)), n["dq_norm"]: TensorSpec((rq,), init="ones", kind="vector"),
             n["uq"]: TensorSpec((H * (D + self.R), rq)), n["uk"]: TensorSpec((H * D, rk)),
             n["uv"]: TensorSpec((H * Dv, rk)), n["o"]: TensorSpec((W, H * Dv))}
        if self.own_kv:
            s[n["dkv"]] = TensorSpec((self.P, W))
            s[n["dkv_norm"]] = TensorSpec((rk,), init="ones", kind="vector")
        if self.output_gate:
            s[n["g"]] = TensorSpec((H * Dv if self.gate_each else H, W))
        if self.position is not None:
            s.update(self.position.tensor_specs(available))
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        n, H, D, Dv, rk, R, P = self.names, self.H, self.D, self.Dv, self.rk, self.R, self.P
        if self.position is not None:
            self.position.load(fetch, ctx)
        parts = [fetch(n["dq"])] + ([fetch(n["dkv"])] if self.own_kv else []) + ([fetch(n["g"])] if self.output_gate else [])
        if len({t.dtype for t in parts}) > 1:
            parts = [t.float() for t in parts]
        self.w_down = torch.cat(parts, dim=0).contiguous()          # one product: query latent | c, key part | gates
        self.gate_col = self.rq + (P if self.own_kv else 0)
        self.dq_norm = fetch(n["dq_norm"])
        self.dkv_norm = fetch(n["dkv_norm"]) if self.own_kv else None
        self.w_uq = fetch(n["uq"])
        uk = fetch(n["uk"]).view(H, D, rk)
        uv = fetch(n["uv"]).view(H, Dv, rk)
        # [h][d][r]: a query head -> its query over the cached rows.  With a turned part the head's last R elements
        # pass as they are (a unit block) behind the kv_rank sums.
        self.w_uk = torch.zeros((H, D + R, P), dtype=uk.dtype, device=uk.device)
        self.w_uk[:, :D, :rk] = uk
        if R:
            self.w_uk[:, D:, rk:] = torch.eye(R, dtype=uk.dtype, device=uk.device)
        # [h][r][v]: the weighted sum of cached rows -> o_h; the rows of the key part are zero
        self.w_uv = torch.zeros((H, P, Dv), dtype=uv.dtype, device=uv.device)
        self.w_uv[:, :rk, :] = uv.transpose(1, 2)
        self.w_out = fetch(n["o"])
        # A bfloat16 run with many rows makes the two small products per head on the tensor cores, all heads in one
        # launch (``ops.gemm_fast_heads``: a tile per token tile and head): the weights as [out, in] per head.
        self._tiles = {}
        self.tc_heads = (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and uk.dtype == torch.bfloat16
                         and (D + R) % 8 == 0 and Dv % 8 == 0 and rk % 8 == 0 and P % 8 == 0)
        if self.tc_heads:
            self.w_uk_t = self.w_uk.transpose(1, 2).contiguous()                     # [h][r][d]
            self.w_uv_n = uv.contiguous()                                            # [h][v][r] over the latent's part of a row

    def _head_tiles(self, T, dev):
        """The tile list of the per-head products for a step of T rows.  Lists are kept for good (a few hundred bytes
        per row count): a captured step names its list by address, and making one copies from the host, which a
        capture does not allow; a shape is captured the second time it is seen, so its list exists by then."""
        key = (T, torch.device(dev))
        tl = self._tiles.get(key)
        if tl is None:
            tl = self._tiles[key] = ops.HeadTiles(T, self.H, dev)
        return tl

    def cache_spec(self):
        return KVCacheSpec(1, self.P, self.cache_window, 0, 0, values=False)

    def forward(self, h, batch, cache):
        ctx, T, dev = self.ctx, h.shape[0], h.device
        H, D, Dv, rq, rk, R, P = self.H, self.D, self.Dv, self.rq, self.rk, self.R, self.P
        pos = self.position
        down = linear(ctx, h, self.w_down, torch.float32)
        bt = batch.block_tables[cache.group]
        if self.own_kv:
            # c normed, the key part turned, both written to the row's place in the pages (the store kernel's key
            # side with one head whose norm covers its first kv_rank elements and whose turn starts behind them)
            ops.qk_prepare_store(down, 0, rq, 0, batch.positions, batch.row_entry, bt, None, self.dkv_norm, self.eps,
                                 pos.inv_freq() if R else self.dkv_norm, R, bool(R) and pos.pairing == "interleaved",
                                 pos.amplitude if R else 1.0, None, cache.k, None, 0, 1, P, P, cache.write, ctx.err,
                                 rot0=rk, k_norm_dim=rk)
        # the queries: norm of the latent, up, and over to the cached rows' space
        cq = torch.empty((T, rq), dtype=ctx.act_dtype, device=dev)
        ops.cols_rmsnorm(down, 0, rq, self.dq_norm, self.eps, cq)
        # A bfloat16 run whose cached row is a head size of the tensor-core kernels attends through them: one shared
        # "kv head" whose pages are keys and values at once (single rows through the split-key decode kernel, the
        # others through the prompt kernel; the softmax weights keep their float32 bits in the product with the
        # values, as three bfloat16 terms).  Else the general kernel, all float32.
        fast = (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
                and P % 16 == 0 and P <= 256)
        mid = torch.bfloat16 if fast else torch.float32
        tc = fast and self.tc_heads and T > self.TC_HEADS_MIN_ROWS
        q_lat = torch.empty((T, H * P), dtype=mid, device=dev)
        if R:
            # the heads' last R elements are turned in float32 and rounded once
            q32 = linear(ctx, cq, self.w_uq, torch.float32)
            q = torch.empty((T, H * (D + R)), dtype=torch.bfloat16 if tc else torch.float32, device=dev)
            ops.qk_prepare_store(q32, 0, 0, 0, batch.positions, batch.row_entry, bt, None, None, self.eps,
                                 pos.inv_freq(), R, pos.pairing == "interleaved", pos.amplitude, q, cache.k, None,
                                 H, 0, D + R, D + R, False, ctx.err, rot0=D)
        else:
            q = linear(ctx, cq, self.w_uq, torch.bfloat16 if tc else torch.float32)
        if tc:
            head_tiles = self._head_tiles(T, dev)
            ops.gemm_fast_heads(q, self.w_uk_t, q_lat, head_tiles, D + R, P, err=ctx.err)
        else:
            ops.head_project(q, self.w_uk, q_lat, H, D + R, P)
        lat = torch.empty((T, H * P), dtype=mid, device=dev)
        if fast:
            single = batch.n_single if ops.attention_decode_usable(cache.k, P) else 0
            if single:
                ops.attention_decode(q_lat, cache.k, cache.k, bt, batch.row_entry, batch.positions, self.scale,
                                     self.window, lat, H, 1, P,
                                     batch.max_context if batch.decode_only else batch.max_single_context,
                                     rows=None if batch.decode_only else batch.single_rows, err=ctx.err,
                                     float_weights=self.weight_terms == 3)
            if single < batch.S:
                tiles = (batch.T - single) // ops.attention_prefill_tile_rows() + (batch.S - single)
                ops.attention_prefill(q_lat, cache.k, cache.k, bt, batch.cu_rows, batch.entry_pos0, tiles, self.scale,
                                      self.window, lat, H, 1, P, err=ctx.err, min_rows=2 if single else 1,
                                      weight_terms=self.weight_terms)
        else:
            ops.paged_attention_general(q_lat, cache.k, None, bt, batch.row_entry, batch.positions, self.scale,
                                        self.window, lat, H, 1, P, P)
        o = torch.empty((T, H * Dv), dtype=ctx.act_dtype, device=dev)
        if tc:
            o32 = torch.empty((T, H * Dv), dtype=torch.float32, device=dev) if self.output_gate else o
            ops.gemm_fast_heads(lat, self.w_uv_n, o32, head_tiles, P, Dv, err=ctx.err)      # (the latent's part of every row)
            if self.output_gate:
                ops.head_gate(o32, down, self.gate_col, o, H, Dv, gate_each=self.gate_each)
        else:
            ops.head_project(lat, self.w_uv, o, H, P, Dv, gate=down if self.output_gate else None,
                             gate_col=self.gate_col, gate_each=self.gate_each)
        return linear(ctx, o, self.w_out, torch.float32)


register_part("mixer", "latent_attention", LatentAttention)
