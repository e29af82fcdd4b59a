"""Mixers that keep a fixed-size state per request instead of pages: matrix memories that are updated token by
token.  Their state lives in float32 in the request's state slot, starts at zero with the request's first token
and is carried from step to step; everything that enters the recurrence after the projections is float32."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, StateCacheSpec, CompositeCacheSpec, TensorSpec
from .linear import linear
from .registry import register_part


def _stack(parts: list, dtype_like=None):
    """Rows of several matrices in one, so that one product makes all of them."""
    if len({t.dtype for t in parts}) > 1:
        parts = [t.float() for t in parts]
    return torch.cat(parts, dim=0).contiguous()


class MatrixLSTM(Mixer):
    """The matrix memory of xLSTM (mLSTM) with ``heads`` heads, keys of ``dim`` and values of ``vdim`` elements.

    Per row and head: ``q = Wq h / sqrt(dim)``, ``k = Wk h``, ``v = Wv h``; the log gates
    ``i = cap tanh((Wi h + bi) / cap)`` and ``f = logsigmoid(cap tanh((Wf h + bf) / cap))``.  With a running
    maximum ``m`` (0 at the start):

        m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' = exp(f + m - m') n + exp(i - m') k
        o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

    Every head's ``o`` is divided by its root mean square (``eps``), the heads side by side are multiplied by the
    weight ``norm`` and by ``sigmoid(Wg h)``, and ``Wo`` projects back.  State per request: S, n and m."""

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float):
        if not ops_scan_size_ok(dim, vdim):
            raise ValueError(f"key/value sizes {dim} x {vdim} are not supported: the scan kernel keeps a head's matrix "
                             "in shared memory (values up to 256 wide)")
        self.hidden, self.H, self.dk, self.dv = hidden_size, heads, dim, vdim
        self.cap, self.eps = float(gate_cap), float(eps)

    def tensor_specs(self, available=None):
        W, H, dk, dv = self.hidden, self.H, self.dk, self.dv
        return {"q": TensorSpec((H * dk, W)), "k": TensorSpec((H * dk, W)), "v": TensorSpec((H * dv, W)),
                "g": TensorSpec((H * dv, W)), "o": TensorSpec((W, H * dv)),
                "norm": TensorSpec((H * dv,), init="ones", kind="vector"),
                "i": TensorSpec((H, W)), "i.b": TensorSpec((H,), kind="vector"),
                "f": TensorSpec((H, W)), "f.b": TensorSpec((H,), kind="vector")}

    def load(self, fetch, ctx):
        self.ctx = ctx
        H, dk, dv = self.H, self.dk, self.dv
        # one product for q, k, v, the output gate and the two gates' pre-activations; its result is float32
        self.w_in = _stack([fetch("q"), fetch("k"), fetch("v"), fetch("g"), fetch("i"), fetch("f")])
        self.cols = {"q": 0, "k": H * dk, "v": 2 * H * dk, "g": 2 * H * dk + H * dv, "i": 2 * H * dk + 2 * H * dv,
                     "f": 2 * H * dk + 2 * H * dv + H}
        bias = torch.zeros(self.w_in.shape[0], dtype=torch.float32, device=self.w_in.device)
        bias[self.cols["i"]:self.cols["i"] + H] = fetch("i.b").float()
        bias[self.cols["f"]:self.cols["f"] + H] = fetch("f.b").float()
        self.b_in = bias
        self.norm = fetch("norm")
        self.w_out = fetch("o")

    def cache_spec(self):
        H, dk, dv = self.H, self.dk, self.dv
        return CompositeCacheSpec((StateCacheSpec((H, dk, dv)), StateCacheSpec((H, dk)), StateCacheSpec((H,))))

    def forward(self, h, batch, cache):
        ctx = self.ctx
        proj = linear(ctx, h, self.w_in, torch.float32, bias=self.b_in)
        S, n, m = (p.state for p in cache.parts)
        y = torch.empty((h.shape[0], self.H * self.dv), dtype=ctx.act_dtype, device=h.device)
        ops.mlstm_scan(proj, self.cols, batch, S, n, m, self.H, self.dk, self.dv, self.cap, self.eps, self.norm, y,
                       columns=ctx.fast_kernels)
        return linear(ctx, y, self.w_out, torch.float32)


class GatedDeltaRule(Mixer):
    """A matrix memory with one decay per head and the delta rule, ``heads`` value heads over ``kv_heads`` heads of q
    and k (value head h reads q/k head ``h // (heads / kv_heads)``).

    ``q, k, v = Wq h, Wk h, Wv h``; each passes a causal convolution over time per channel (``taps`` taps, the last
    one the current token's, zeros before the sequence's start) and silu; q and k heads become unit vectors
    (``x / sqrt(sum x^2 + 1e-6)``), q also times ``dim^-1/2``.  ``beta = sigmoid(Wb h)``, ``g = exp(-exp(A_log)
    softplus(Wa h + dt_bias))`` per head.  Per head and row, in this order:

        S = g S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q

    Every head's ``o`` is divided by its root mean square over ``vdim`` (``eps``), multiplied by the weight ``norm``
    (one vector for all heads) and by ``silu(Wg h)``, and ``Wo`` projects back.  State per request: S and the last
    ``taps - 1`` inputs of the convolutions.

    Options.  ``channel_decay``: one decay per head *and key channel*, ``g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 h) +
    dt_bias))`` laid out heads x dim (``dt_bias`` then has heads x dim entries), which multiplies the rows of S:
    ``S = diag(g) S``; its pre-activation comes through a low-rank pair ``a1`` [r, width], ``a2`` [heads * dim, r].
    ``low_rank_gate``: the output gate's pre-activation is ``Wg2 (Wg1 h)`` (``g1`` [r', width], ``g2``
    [heads * vdim, r']).  The two ranks are the files' (``decay_rank`` / ``gate_rank`` say what random weights
    take).  ``gate``: ``silu`` or ``sigmoid``."""

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, eps: float,
                 channel_decay: bool = False, low_rank_gate: bool = False, gate: str = "silu",
                 decay_rank: int | None = None, gate_rank: int | None = None):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if conv < 1:
            raise ValueError("the convolution needs at least one tap")
        if not ops_scan_size_ok(dim, vdim, 2):
            raise ValueError(f"key/value sizes {dim} x {vdim} are not supported: the scan kernel keeps a head's matrix "
                             "in shared memory (values up to 256 wide)")
        self.hidden, self.H, self.G, self.dk, self.dv, self.taps = hidden_size, heads, kv_heads, dim, vdim, conv
        self.eps = float(eps)
        self.C = 2 * kv_heads * dim + heads * vdim          # channels that pass the convolution: q | k | v
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"the output gate is silu or sigmoid, found {gate!r}")
        self.channel_decay, self.low_rank_gate, self.gate = bool(channel_decay), bool(low_rank_gate), gate
        self.decay_rank = int(decay_rank) if decay_rank else max(4, dim // 2)
        self.gate_rank = int(gate_rank) if gate_rank else max(4, vdim // 2)

    def tensor_specs(self, available=None):
        W, H, G, dk, dv, taps = self.hidden, self.H, self.G, self.dk, self.dv, self.taps
        if self.channel_decay or self.low_rank_gate:
            from_file = available is not None       # a rank is the file's; random weights take the constructor's
            s = {"q": TensorSpec((G * dk, W)), "q.conv": TensorSpec((G * dk, taps), kind="vector"),
                 "k": TensorSpec((G * dk, W)), "k.conv": TensorSpec((G * dk, taps), kind="vector"),
                 "v": TensorSpec((H * dv, W)), "v.conv": TensorSpec((H * dv, taps), kind="vector"),
                 "b": TensorSpec((H, W)), "A_log": TensorSpec((H,), init="zeros", kind="vector"),
                 "norm": TensorSpec((dv,), init="ones", kind="vector"), "o": TensorSpec((W, H * dv))}
            if self.channel_decay:
                r = None if from_file else self.decay_rank
                s.update({"a1": TensorSpec((r, W)), "a2": TensorSpec((H * dk, r)),
                          "dt_bias": TensorSpec((H * dk,), init="zeros", kind="vector")})
            else:
                s.update({"a": TensorSpec((H, W)), "dt_bias": TensorSpec((H,), init="zeros", kind="vector")})
            if self.low_rank_gate:
                r = None if from_file else self.gate_rank
                s.update({"g1": TensorSpec((r, W)), "g2": TensorSpec((H * dv, r))})
            else:
                s["g"] = TensorSpec((H * dv, W))
            return s
        return {"q": TensorSpec((G * dk, W)), "q.conv": TensorSpec((G * dk, taps), kind="vector"),
                "k": TensorSpec((G * dk, W)), "k.conv": TensorSpec((G * dk, taps), kind="vector"),
                "v": TensorSpec((H * dv, W)), "v.conv": TensorSpec((H * dv, taps), kind="vector"),
                "b": TensorSpec((H, W)), "a": TensorSpec((H, W)),
                "A_log": TensorSpec((H,), init="zeros", kind="vector"), "dt_bias": TensorSpec((H,), init="zeros", kind="vector"),
                "norm": TensorSpec((dv,), init="ones", kind="vector"),
                "g": TensorSpec((H * dv, W)), "o": TensorSpec((W, H * dv))}

    def load(self, fetch, ctx):
        self.ctx = ctx
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        self.cols = {"q": 0, "k": G * dk, "v": 2 * G * dk}
        if self.channel_decay or self.low_rank_gate:
            # one product for q, k, v, beta and the first halves of the low-rank pairs; the second halves follow
            first = [fetch("q"), fetch("k"), fetch("v"), fetch("b")]
            at = self.C + H
            self.pcols = {"b": self.C}
            self.a2 = self.g2 = None
            if self.channel_decay:
                a1, self.a2 = fetch("a1"), fetch("a2")
                if a1.shape[0] != self.a2.shape[1]:
                    raise ValueError(f"the decay's low-rank pair does not fit: a1 {tuple(a1.shape)}, a2 {tuple(self.a2.shape)}")
                first.append(a1)
                self.a1_cols = (at, at + a1.shape[0])
                at += a1.shape[0]
                self.pcols["a"] = 0                     # column of the second product's result
            else:
                first.append(fetch("a"))
                self.pcols["a"] = at
                at += H
            if self.low_rank_gate:
                g1, self.g2 = fetch("g1"), fetch("g2")
                if g1.shape[0] != self.g2.shape[1]:
                    raise ValueError(f"the gate's low-rank pair does not fit: g1 {tuple(g1.shape)}, g2 {tuple(self.g2.shape)}")
                first.append(g1)
                self.g1_cols = (at, at + g1.shape[0])
                at += g1.shape[0]
                self.pcols["g"] = 0
            else:
                first.append(fetch("g"))
                self.pcols["g"] = at
                at += H * dv
            self.w_in = _stack(first)
        else:
            self.w_in = _stack([fetch("q"), fetch("k"), fetch("v"), fetch("g"), fetch("b"), fetch("a")])
            self.pcols = {"g": self.C, "b": self.C + H * dv, "a": self.C + H * dv + H}
        self.w_conv = torch.cat([fetch("q.conv").float(), fetch("k.conv").float(), fetch("v.conv").float()], dim=0).contiguous()
        self.A_log, self.dt_bias = fetch("A_log"), fetch("dt_bias")
        self.norm = fetch("norm")
        self.w_out = fetch("o")

    def cache_spec(self):
        parts = [StateCacheSpec((self.H, self.dk, self.dv))]
        if self.taps > 1:
            parts.append(StateCacheSpec((self.taps - 1, self.C)))
        return CompositeCacheSpec(tuple(parts))

    def forward(self, h, batch, cache):
        ctx, T = self.ctx, h.shape[0]
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        proj = linear(ctx, h, self.w_in, torch.float32)
        S = cache.parts[0].state
        tail = cache.parts[1].state if self.taps > 1 else S
        qkv = torch.empty((T, self.C), dtype=torch.float32, device=h.device)
        ops.conv_silu_norm(proj, 0, self.C, self.w_conv, self.taps, batch, tail, qkv, unit_heads=2 * G, unit_dim=dk,
                           unit_eps=1e-6, scaled_heads=G, scale=float(dk) ** -0.5)
        if self.taps > 1 and cache.write:
            ops.conv_state_update(proj, 0, self.C, self.taps, batch, tail)
        y = torch.empty((T, H * dv), dtype=ctx.act_dtype, device=h.device)
        if self.channel_decay or self.low_rank_gate or self.gate != "silu":
            # (the second halves read float32 columns of the first product's result: nothing is rounded in between)
            dec = gsrc = None
            if self.channel_decay:
                dec = linear(ctx, proj[:, self.a1_cols[0]:self.a1_cols[1]], self.a2, torch.float32)
            if self.low_rank_gate:
                gsrc = linear(ctx, proj[:, self.g1_cols[0]:self.g1_cols[1]], self.g2, torch.float32)
            ops.gated_delta_scan(qkv, self.cols, G, proj, self.pcols, self.A_log, self.dt_bias, batch, S, H, dk, dv,
                                 self.eps, self.norm, y, columns=ctx.fast_kernels, channel_decay=dec, gate_src=gsrc,
                                 gate=self.gate)
        else:
            ops.gated_delta_scan(qkv, self.cols, G, proj, self.pcols, self.A_log, self.dt_bias, batch, S, H, dk, dv,
                                 self.eps, self.norm, y, columns=ctx.fast_kernels)
        return linear(ctx, y, self.w_out, torch.float32)


def ops_scan_size_ok(dk: int, dv: int, parts: int = 1) -> bool:
    """What ``ops.scan_usable`` checks, without the library: a head's matrix and its helpers fit in 227 KB of
    shared memory and a value is at most 256 wide."""
    if dk < 1 or dv < 1 or dv > 256:
        return False
    rs = max(1, min(256 // dv, dk))
    return 4 * (dk * dv + 3 * dk + (2 + parts) * dv + parts * rs * dv + 8) <= 227 * 1024


register_part("mixer", "matrix_lstm", MatrixLSTM)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
