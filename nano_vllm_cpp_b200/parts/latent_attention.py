"""Attention whose keys and values are made from one small vector per token, which is all its cache keeps."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, KVCacheSpec, TensorSpec
from .linear import linear
from .registry import register_part


class LatentAttention(Mixer):
    """Causal softmax attention through latents, without positions.  Per row, with ``rms`` the RMS norm (``eps``,
    plain weights):

        c_q = rms(W_dq h) w_dq;   q_h = W_uq[h] c_q        (heads of ``dim`` elements)
        c   = rms(W_dkv h) w_dkv                           (``kv_rank`` elements: what the cache keeps per token)
        k_h(j) = W_uk[h] c(j);   v_h(j) = W_uv[h] c(j)     (values of ``vdim`` elements)
        o_h = sum_j softmax_j(scale q_h . k_h(j)) v_h(j) over j <= i;   out = W_o (sigmoid(W_g h)_h o_h)

    Keys and values are never formed: ``q_h . k_h(j) = (W_uk[h]^T q_h) . c(j)`` and
    ``sum_j p_j v_h(j) = W_uv[h] sum_j p_j c(j)``, so every head attends with a query of ``kv_rank`` elements over
    the one shared row ``c(j)``, which is key and value at once, and its output is projected by ``W_uv[h]``
    afterwards (``ops.head_project`` does both small products per head, in float32 with the weights as stored).  The
    page pool therefore holds one array of ``kv_rank`` elements per token and layer.  ``output_gate`` False leaves
    the sigmoid gate out.  ``names`` renames the tensors (keys: dq, dq_norm, uq, dkv, dkv_norm, uk, uv, g, o)."""

    TC_HEADS_MIN_ROWS = 64      # steps of more rows make the per-head products on the tensor cores (bfloat16 runs)

    _NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
              "uv": "uv", "g": "g", "o": "o"}

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float,
                 eps: float, output_gate: bool = True, names: dict | None = None):
        if min(heads, dim, vdim, q_rank, kv_rank) < 1:
            raise ValueError("latent attention: every size must be positive")
        if kv_rank > 512:
            raise ValueError(f"a latent of {kv_rank} elements is not supported: the attention kernel takes up to 512")
        self.hidden, self.H, self.D, self.Dv, self.rq, self.rk = hidden_size, heads, dim, vdim, q_rank, kv_rank
        self.scale, self.eps, self.output_gate = float(scale), float(eps), bool(output_gate)
        self.names = dict(self._NAMES, **(names or {}))

    def tensor_specs(self, available=None):
        W, H, D, Dv, rq, rk, n = self.hidden, self.H, self.D, self.Dv, self.rq, self.rk, self.names
        s = {n["dq"]: TensorSpec((rq, W)), n["dq_norm"]: TensorSpec((rq,), init="ones", kind="vector"),
             n["uq"]: TensorSpec((H * D, rq)), n["dkv"]: TensorSpec((rk, W)),
             n["dkv_norm"]: TensorSpec((rk,), init="ones", kind="vector"), n["uk"]: TensorSpec((H * D, rk)),
             n["uv"]: TensorSpec((H * Dv, rk)), n["o"]: TensorSpec((W, H * Dv))}
        if self.output_gate:
            s[n["g"]] = TensorSpec((H, W))
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        n, H, D, Dv, rk = self.names, self.H, self.D, self.Dv, self.rk
        parts = [fetch(n["dq"]), fetch(n["dkv"])] + ([fetch(n["g"])] if self.output_gate else [])
        if len({t.dtype for t in parts}) > 1:
            parts = [t.float() for t in parts]
        self.w_down = torch.cat(parts, dim=0).contiguous()          # one product: query latent | c | gates
        self.dq_norm, self.dkv_norm = fetch(n["dq_norm"]), fetch(n["dkv_norm"])
        self.w_uq = fetch(n["uq"])
        self.w_uk = fetch(n["uk"]).view(H, D, rk).contiguous()                       # [h][d][r]: q_h -> W_uk[h]^T q_h
        self.w_uv = fetch(n["uv"]).view(H, Dv, rk).transpose(1, 2).contiguous()      # [h][r][v]: latent sum -> o_h
        self.w_out = fetch(n["o"])
        # A bfloat16 run with many rows makes the two small products per head on the tensor cores, head by head
        # on views of the rows: the weights as [out, in] per head.
        self.tc_heads = (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and self.w_uk.dtype == torch.bfloat16
                         and D % 8 == 0 and Dv % 8 == 0 and rk % 8 == 0)
        if self.tc_heads:
            self.w_uk_t = self.w_uk.transpose(1, 2).contiguous()                     # [h][r][d]
            self.w_uv_n = fetch(n["uv"]).view(H, Dv, rk).contiguous()                # [h][v][r]

    def cache_spec(self):
        return KVCacheSpec(1, self.rk, 0, 0, 0, values=False)

    def forward(self, h, batch, cache):
        ctx, T, dev = self.ctx, h.shape[0], h.device
        H, D, Dv, rq, rk = self.H, self.D, self.Dv, self.rq, self.rk
        down = linear(ctx, h, self.w_down, torch.float32)
        bt = batch.block_tables[cache.group]
        # c: normed, and written to the row's place in the pages (the store kernel's key side with one head)
        ops.qk_prepare_store(down, 0, rq, 0, batch.positions, batch.row_entry, bt, None, self.dkv_norm, self.eps,
                             self.dkv_norm, 0, False, 1.0, None, cache.k, None, 0, 1, rk, rk, cache.write, ctx.err)
        # the queries: norm of the latent, up, and over to c's space
        cq = torch.empty((T, rq), dtype=ctx.act_dtype, device=dev)
        ops.cols_rmsnorm(down, 0, rq, self.dq_norm, self.eps, cq)
        # A bfloat16 run whose latent is a head size of the tensor-core kernels attends through them: one shared
        # "kv head" of kv_rank elements whose pages are keys and values at once (single rows through the split-key
        # decode kernel, the others through the prompt kernel; the softmax weights keep their float32 bits in the
        # product with the values, as three bfloat16 terms).  Else the general kernel, all float32.
        fast = (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
                and rk % 16 == 0 and rk <= 256)
        mid = torch.bfloat16 if fast else torch.float32
        tc = fast and self.tc_heads and T > self.TC_HEADS_MIN_ROWS
        q_lat = torch.empty((T, H * rk), dtype=mid, device=dev)
        if tc:
            q = linear(ctx, cq, self.w_uq, torch.bfloat16)
            for h in range(H):
                linear(ctx, q[:, h * D:(h + 1) * D], self.w_uk_t[h], mid, out=q_lat[:, h * rk:(h + 1) * rk])
        else:
            q = linear(ctx, cq, self.w_uq, torch.float32)
            ops.head_project(q, self.w_uk, q_lat, H, D, rk)
        lat = torch.empty((T, H * rk), dtype=mid, device=dev)
        if fast:
            single = batch.n_single if ops.attention_decode_usable(cache.k, rk) else 0
            if single:
                ops.attention_decode(q_lat, cache.k, cache.k, bt, batch.row_entry, batch.positions, self.scale, 0, lat,
                                     H, 1, rk, batch.max_context if batch.decode_only else batch.max_single_context,
                                     rows=None if batch.decode_only else batch.single_rows, err=ctx.err,
                                     float_weights=True)
            if single < batch.S:
                tiles = (batch.T - single) // ops.attention_prefill_tile_rows() + (batch.S - single)
                ops.attention_prefill(q_lat, cache.k, cache.k, bt, batch.cu_rows, batch.entry_pos0, tiles, self.scale,
                                      0, lat, H, 1, rk, err=ctx.err, min_rows=2 if single else 1, weight_terms=3)
        else:
            ops.paged_attention_general(q_lat, cache.k, None, bt, batch.row_entry, batch.positions, self.scale, 0, lat,
                                        H, 1, rk, rk)
        o = torch.empty((T, H * Dv), dtype=ctx.act_dtype, device=dev)
        if tc:
            o32 = torch.empty((T, H * Dv), dtype=torch.float32, device=dev) if self.output_gate else o
            for h in range(H):
                linear(ctx, lat[:, h * rk:(h + 1) * rk], self.w_uv_n[h], o32.dtype, out=o32[:, h * Dv:(h + 1) * Dv])
            if self.output_gate:
                ops.head_gate(o32, down, rq + rk, o, H, Dv)
        else:
            ops.head_project(lat, self.w_uv, o, H, rk, Dv, gate=down if self.output_gate else None, gate_col=rq + rk)
        return linear(ctx, o, self.w_out, torch.float32)


register_part("mixer", "latent_attention", LatentAttention)
