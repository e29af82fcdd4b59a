"""Feed-forward parts: the dense SwiGLU MLP and the sparse mixture of SwiGLU experts with a
softmax router, top-k routing and an optional sigmoid-gated shared expert."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, RowMix, TensorSpec
from .linear import linear, grouped_linear, small_linear
from .registry import register_part

# Batches of up to this many rows run the shared expert's chunks on a second stream beside the routing.
SIDE_MAX_ROWS = 64
# Prompts: the shared expert's two products run beside the routing chain (router product, top-k, permutation, row
# copy) on a second stream with their grid capped to this share of the multiprocessors, which leaves the chain's
# kernels room; the routed experts' products follow on the first stream.
SIDE_GRID_SHARE = 0.88
# Permutation buffers are kept per batch size; beyond this many sizes the oldest set is dropped.
MAX_ALIGNMENTS = 16


class DenseSwiGLU(FeedForward):
    """``down(silu(gate(h)) * up(h))`` (src/model.cpp:828-832; src/hip_ops.hip:419-429).

    ``clamp_limit`` > 0 makes the pairing of the two halves a clamped one instead, still in the first product's
    epilogue: ``g = min(gate(h), limit)``, ``u = clamp(up(h), -limit, limit)``, ``down(g sigmoid(slope g) (u + 1))``.
    ``names`` renames the tensors (keys: gate, up, down)."""

    _NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, hidden_size: int, intermediate_size: int, clamp_limit: float = 0.0, slope: float = 1.702,
                 names: dict | None = None):
        self.hidden, self.inter = hidden_size, intermediate_size
        if clamp_limit < 0:
            raise ValueError("clamp_limit must not be negative")
        self.pair = ("glu_clamped", float(clamp_limit), float(slope)) if clamp_limit > 0 else None
        self.names = dict(self._NAMES, **(names or {}))

    def tensor_specs(self, available=None):
        H, I, n = self.hidden, self.inter, self.names
        return {n["gate"]: TensorSpec((I, H)), n["up"]: TensorSpec((I, H)), n["down"]: TensorSpec((H, I))}

    def load(self, fetch, ctx):
        self.ctx = ctx
        # gate rows then up rows in one matrix (src/model.cpp:589-596)
        self.gate_up = _cat([fetch(self.names["gate"]), fetch(self.names["up"])])
        self.down = fetch(self.names["down"])

    def forward(self, h, h32, batch):
        act = linear(self.ctx, h, self.gate_up, self.ctx.act_dtype, swiglu=True, act=self.pair)
        return linear(self.ctx, act, self.down, torch.float32)


class DenseMLP(FeedForward):
    """``down(act(up(h)))`` with ``act`` one of ``ops.EPILOGUE_ACTS`` (gelu in its erf or tanh form, silu), taken on
    the up product's float32 sums; its output is in the activation dtype.  Steps of few rows, and float32 runs,
    take the activation in the product's epilogue (one launch less).  A bfloat16 prompt does not: the tensor-core
    product's epilogue is the work of four to eight warps per block, and an erf per value there costs more than
    a pass of its own (measured on 2,048 rows, 2,048 -> 8,192: 0.164 ms fused against 0.066 + 0.055 ms apart).

    ``activation="xielu"``: a learned activation with two numbers (p, q) per layer, the tensor ``act_name`` [2]:
    ``softplus(p) z^2 + z / 2`` for z > 0 and ``(1/2 + softplus(q)) (e^z - 1 - z) + z / 2`` for z <= 0 (continuous with
    slope 1/2 at zero).  The two factors are worked out once, in float64, when the weights are loaded and go to the
    product's epilogue, or to the pass of its own, as two numbers; the rule above holds for it too (measured on
    16,384 rows, 2,048 -> 8,192: 1.85 ms a layer fused against 0.41 + 0.23 ms apart)."""
    FUSED_MAX_ROWS = 32

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "gelu_erf",
                 up_name: str = "up_proj.weight", down_name: str = "down_proj.weight", act_name: str = "act"):
        if activation not in ops.EPILOGUE_ACTS and activation != "xielu":
            raise ValueError(f"activation must be one of {sorted(ops.EPILOGUE_ACTS) + ['xielu']}, found {activation!r}")
        self.hidden, self.inter, self.activation = hidden_size, intermediate_size, activation
        self.up_name, self.down_name, self.act_name = up_name, down_name, act_name
        self.act_params = (0.0, 0.0)

    def tensor_specs(self, available=None):
        s = {self.up_name: TensorSpec((self.inter, self.hidden)), self.down_name: TensorSpec((self.hidden, self.inter))}
        if self.activation == "xielu":
            s[self.act_name] = TensorSpec((2,), kind="vector")
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        self.up, self.down = fetch(self.up_name), fetch(self.down_name)
        if self.activation == "xielu":
            pq = fetch(self.act_name).double().cpu()
            sp = torch.nn.functional.softplus(pq)
            self.act_params = (float(sp[0]), 0.5 + float(sp[1]))

    def forward(self, h, h32, batch):
        ctx = self.ctx
        xielu = self.activation == "xielu"
        if h.shape[0] <= self.FUSED_MAX_ROWS or ctx.act_dtype == torch.float32 or not ctx.fast_kernels:
            act = linear(ctx, h, self.up, ctx.act_dtype,
                         act=("xielu",) + tuple(self.act_params) if xielu else self.activation)
        else:
            z = linear(ctx, h, self.up, torch.float32)
            act = torch.empty(z.shape, dtype=ctx.act_dtype, device=z.device)
            ops.activation(z, act, self.activation, self.act_params)
        return linear(ctx, act, self.down, torch.float32)


class SparseMoeSwiGLU(FeedForward):
    """Per row (src/model.cpp:789-827; src/hip_ops.hip:813-893, 926-934):

    router logits ``r = h Wg^T`` in float32; ``p = softmax(r)`` over all experts; the ``top_k``
    largest (ties to the lower index) with weights ``p`` or ``p / sum`` (``renormalize``);
    ``routed = sum_k w_k * down_e(silu(gate_e(h)) * up_e(h))`` for k in rank order;
    ``shared = sigmoid(h . w_gate) * down_s(silu(gate_s(h)) * up_s(h))`` if there is a shared
    expert; the result is ``shared + routed``.

    Other routers are options.  ``score="sigmoid"``: every expert's score is ``s = sigmoid(r)`` by itself, in
    float32; the ``top_k`` largest ``s + correction`` are chosen (``choice_bias``: a learned vector ``correction``
    [experts] that steers the choice only), and the weights are the chosen experts' ``s`` without it.  ``route_scale``
    multiplies the weights.  ``shared_gate=False``: the shared expert has no gate and is added as it is.  ``names``
    gives the tensors' names where they are not the usual ones (keys: router, correction, shared_gate, and the
    patterns expert_gate, expert_up, expert_down with ``{}`` for the expert's number, shared_gate_proj, shared_up,
    shared_down).

    ``expert_activation`` (one of ``ops.EPILOGUE_ACTS``, for instance ``relu2``): the experts, the shared one too,
    have no gate matrix and are ``down(act(up(h)))``; the activation sits in the first product's epilogue.
    """
    wants_f32_input = True

    _NAMES = {"router": "gate.weight", "correction": "correction", "shared_gate": "shared_expert_gate.weight",
              "expert_gate": "experts.{}.gate_proj.weight", "expert_up": "experts.{}.up_proj.weight",
              "expert_down": "experts.{}.down_proj.weight", "shared_gate_proj": "shared_expert.gate_proj.weight",
              "shared_up": "shared_expert.up_proj.weight", "shared_down": "shared_expert.down_proj.weight"}

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, intermediate_size: int,
                 shared_intermediate_size: int = 0, renormalize: bool = False, score: str = "softmax",
                 route_scale: float = 1.0, choice_bias: bool = False, shared_gate: bool = True,
                 names: dict | None = None, expert_activation: str | None = None):
        if not (1 <= top_k <= num_experts):
            raise ValueError("top_k must lie in 1..num_experts")
        if top_k > 32 or num_experts > 1536:
            raise ValueError("the router kernel takes up to 32 experts per row out of up to 1536")
        self.hidden, self.E, self.K = hidden_size, num_experts, top_k
        self.inter, self.shared_inter, self.renorm = intermediate_size, shared_intermediate_size, renormalize
        if score not in ops.ROUTE_SCORES:
            raise ValueError(f"score must be one of {sorted(ops.ROUTE_SCORES)}, found {score!r}")
        if choice_bias and score != "sigmoid":
            raise ValueError("a choice bias goes with sigmoid scores")
        self.score, self.route_scale, self.choice_bias = score, float(route_scale), bool(choice_bias)
        self.shared_gate = bool(shared_gate) and shared_intermediate_size > 0
        if expert_activation is not None and expert_activation not in ops.EPILOGUE_ACTS:
            raise ValueError(f"expert_activation must be one of {sorted(ops.EPILOGUE_ACTS)}, found {expert_activation!r}")
        self.expert_act = expert_activation
        self.gated = expert_activation is None          # SwiGLU experts: gate and up rows paired in the epilogue
        self.names = dict(self._NAMES, **(names or {}))
        self.rule = None                # what the routing kernels take beyond the softmax rule (set at load)
        self._align = {}
        self._counters = None
        self._captured = {}
        self._static = {}
        self._static_kept = set()
        self.router_and_gate = None
        self.last_alignment = None      # the permutation buffers of the latest forward (for statistics)

    def tensor_specs(self, available=None):
        H, I, E, SI, n = self.hidden, self.inter, self.E, self.shared_inter, self.names
        s = {n["router"]: TensorSpec((E, H))}
        if self.choice_bias:
            s[n["correction"]] = TensorSpec((E,), init="zeros", kind="vector")
        if self.gated and available is not None and available("experts.gate_up_proj"):  # stacked form, src/model.cpp:274-281
            s["experts.gate_up_proj"] = TensorSpec((E, 2 * I, H))
            s["experts.down_proj"] = TensorSpec((E, H, I))
        else:
            for e in range(E):
                if self.gated:
                    s[n["expert_gate"].format(e)] = TensorSpec((I, H))
                s[n["expert_up"].format(e)] = TensorSpec((I, H))
                s[n["expert_down"].format(e)] = TensorSpec((H, I))
        if SI > 0:
            if self.gated:
                s[n["shared_gate_proj"]] = TensorSpec((SI, H))
            s[n["shared_up"]] = TensorSpec((SI, H))
            s[n["shared_down"]] = TensorSpec((H, SI))
            if self.shared_gate:
                s[n["shared_gate"]] = TensorSpec((1, H))
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        H, I, E, SI, n = self.hidden, self.inter, self.E, self.shared_inter, self.names
        self.router = fetch(n["router"])
        bias = fetch(n["correction"]).float().contiguous() if self.choice_bias else None
        if self.score != "softmax" or bias is not None or self.route_scale != 1.0:
            self.rule = (self.score, bias, self.route_scale)
        stacked = self.gated and fetch.has("experts.gate_up_proj")
        G = 2 if self.gated else 1                       # matrices of an expert's first product
        first = fetch("experts.gate_up_proj") if stacked else fetch(n["expert_gate" if self.gated else "expert_up"].format(0))
        # The shared expert as C more experts that every row visits: possible when its width is a whole
        # number of expert widths.  Its chunks then ride in the grouped products and need no launches of
        # their own.  Only the tensor-core path does this; the plain path keeps the shared expert apart.
        C = SI // I if (SI > 0 and SI % I == 0 and SI // I <= 32) else 0
        self.virtual = C if (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and first.dtype == torch.bfloat16
                             and H % 8 == 0 and I % 8 == 0) else 0
        EC = E + self.virtual
        # every expert's [gate; up] rows and down matrix in one block each, indexed by expert
        self.w_gate_up = torch.empty((EC, G * I, H), dtype=first.dtype, device=first.device)
        self.w_down = torch.empty((EC, H, I), dtype=first.dtype, device=first.device)
        if stacked:
            self.w_gate_up[:E].copy_(first)
            self.w_down[:E].copy_(fetch("experts.down_proj"))
        else:
            for e in range(E):
                if self.gated:
                    self.w_gate_up[e, :I].copy_(first if e == 0 else fetch(n["expert_gate"].format(e)))
                    self.w_gate_up[e, I:].copy_(fetch(n["expert_up"].format(e)))
                else:
                    self.w_gate_up[e].copy_(first if e == 0 else fetch(n["expert_up"].format(e)))
                self.w_down[e].copy_(fetch(n["expert_down"].format(e)))
        del first
        if SI > 0:
            su = fetch(n["shared_up"])
            sg = fetch(n["shared_gate_proj"]) if self.gated else su
            sd = fetch(n["shared_down"])
            self.sh_gate = fetch(n["shared_gate"]) if self.shared_gate else None
            # the gate's single row rides along with the router's rows: one product gives both logits
            if self.shared_gate and self.sh_gate.dtype == self.router.dtype:
                self.router_and_gate = torch.cat([self.router, self.sh_gate.reshape(1, -1)], dim=0).contiguous()
            if (self.virtual and sg.dtype == su.dtype == sd.dtype == self.w_gate_up.dtype
                    and (self.router_and_gate is not None or not self.shared_gate)):
                for c in range(self.virtual):
                    if self.gated:
                        self.w_gate_up[E + c, :I].copy_(sg[c * I:(c + 1) * I])
                        self.w_gate_up[E + c, I:].copy_(su[c * I:(c + 1) * I])
                    else:
                        self.w_gate_up[E + c].copy_(su[c * I:(c + 1) * I])
                    self.w_down[E + c].copy_(sd[:, c * I:(c + 1) * I])
            else:
                if self.virtual:                       # mixed storage types: keep the shared expert apart
                    self.w_gate_up, self.w_down = self.w_gate_up[:E].clone(), self.w_down[:E].clone()
                    self.virtual = 0
                self.sh_gate_up = _cat([sg, su]) if self.gated else su
                self.sh_down = sd
        else:
            self.virtual = 0

    def _alignment(self, TK, n_experts, device, fast):
        if fast:    # the down product's tile is the primary list, the SwiGLU product may want a wider one
            tile_m, tile_m2 = ops.grouped_token_tile(TK, n_experts), ops.grouped_token_tile(TK, n_experts, swiglu=True)
        else:
            tile_m, tile_m2 = ops.gemm_plain_tile_m(), 0
        key = (TK, n_experts, tile_m, tile_m2)
        if key in self._captured:
            return self._captured[key]
        al = self._align.pop(key, None)
        if al is None:
            if len(self._align) >= MAX_ALIGNMENTS:
                self._align.pop(next(iter(self._align)))
            al = ops.MoeAlignment(TK, n_experts, tile_m, device, tile_m2)
        if torch.cuda.is_current_stream_capturing():     # a captured step names these buffers by address: kept for good
            self._captured[key] = al
        else:
            self._align[key] = al                        # most recently used last
        return al

    def forward(self, h, h32, batch):
        ctx = self.ctx
        T = h.shape[0]
        dev = h.device
        C = self.virtual
        KT = self.K + C
        gate_logit = None
        if self.router_and_gate is not None:
            both = small_linear(ctx, h32, self.router_and_gate)
            logits, gate_logit = both[:, :self.E], both[:, self.E:]
        else:
            logits = small_linear(ctx, h32, self.router)
        idx = torch.empty((T, KT), dtype=torch.int32, device=dev)
        score = torch.empty((T, KT), dtype=torch.float32, device=dev)
        fast = (ctx.fast_kernels and h.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16
                and self.w_down.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0)
        al = self._alignment(T * KT, self.E + C, dev, fast)
        x_sorted = None
        if (fast and C and T <= SIDE_MAX_ROWS and al.secondary is None
                and ops.moe_route_small_usable(T, self.E, self.K, C, self.hidden)):
            return self._forward_beside(h, logits, gate_logit, idx, score, al)
        if fast and C and T >= 256 and al.secondary is None:
            return self._forward_beside(h, logits, gate_logit, idx, score, al, many=True)
        # (the products' CTAs take their tiles from a counter, as in _forward_beside, unless a handful of pairs split K)
        c0 = c1 = zero = None
        if fast and al.TK > ops.GROUPED_SPLIT_MAX_PAIRS:
            if self._counters is None:
                self._counters = torch.zeros(2, dtype=torch.int32, device=dev)
            zero, c0, c1 = self._counters, self._counters[0:1], self._counters[1:2]
        if fast and al.secondary is None and ops.moe_route_small_usable(T, self.E, self.K, C, self.hidden):
            x_sorted = ops.moe_route_small(logits, self.K, self.renorm, C, gate_logit, idx, score, al, ctx.err,
                                           x=None, zero=zero, rule=self.rule)   # one block copies rows slower than the copy kernel does
        else:
            ops.router_topk(logits, self.K, self.renorm, idx, score, C, gate_logit, rule=self.rule)
            ops.moe_align(idx, KT, al, ctx.err, spread_last=C if fast else 0, zero=zero)
        self.last_alignment = al
        wide = al.secondary                      # the tile list of the SwiGLU product, if it has one of its own
        if x_sorted is not None:
            act = grouped_linear(ctx, x_sorted, self.w_gate_up, ctx.act_dtype, al, swiglu=self.gated, tiles=wide,
                                 counter=c0, act=self.expert_act)
        else:
            act = grouped_linear(ctx, h, self.w_gate_up, ctx.act_dtype, al, a_rows=al.sorted_token, swiglu=self.gated,
                                 tiles=wide, counter=c0, act=self.expert_act)
        # the tile lists were final before the first product started: the second may start beside it
        y = grouped_linear(ctx, act, self.w_down, torch.float32, al, tiles_ready=True, counter=c1)
        shared = None
        if self.shared_inter > 0 and not C:
            sact = linear(ctx, h, self.sh_gate_up, ctx.act_dtype, swiglu=self.gated, act=self.expert_act)
            shared = linear(ctx, sact, self.sh_down, torch.float32)
            if gate_logit is None and self.shared_gate:
                gate_logit = small_linear(ctx, h32, self.sh_gate)
        # the combination (src/hip_ops.hip:873-892) is left to whoever takes the branch: the next norm sums it
        return RowMix(y, al.pair_pos[:T * KT].view(T, KT), score, shared, gate_logit if shared is not None else None)


    def _forward_beside(self, h, logits, gate_logit, idx, score, al, many=False):
        """The shared expert's chunks need no routing, so their two products run on a second stream beside the
        routing and the row copy, which keep few multiprocessors busy; the routed experts' products follow on the
        first stream and write the other rows of the same two buffers.  Few rows (decoding): one launch routes.
        ``many`` rows (a prompt): the routing is three kernels that take a tenth of the layer's time, and the side
        products leave them some multiprocessors."""
        ctx, T, K, C, dev = self.ctx, h.shape[0], self.K, self.virtual, h.device
        KT = K + C
        key = (T, dev)
        st = self._static.get(key)
        if st is None:
            loose = [k for k in self._static if k not in self._static_kept]
            if len(loose) >= MAX_ALIGNMENTS:
                self._static.pop(loose[0])
            st = self._static[key] = ops.StaticTiles(T, K, self.E, C, dev)
        if torch.cuda.is_current_stream_capturing():       # a captured step names these buffers by address
            self._static_kept.add(key)
        act = torch.empty((T * KT, self.inter), dtype=ctx.act_dtype, device=dev)
        y = torch.empty((T * KT, self.hidden), dtype=torch.float32, device=dev)
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        fork, join = torch.cuda.Event(), torch.cuda.Event()
        fork.record(main)
        side.wait_event(fork)
        cap = int(ops.num_sms() * SIDE_GRID_SHARE) if many else 0
        with torch.cuda.stream(side):
            ops.gemm_fast_grouped(h, self.w_gate_up, act, al, swiglu=self.gated, err=ctx.err, tiles=st, tiles_ready=True,
                                  x_rows=st.x_rows, max_ctas=cap, act=self.expert_act)
            ops.gemm_fast_grouped(act, self.w_down, y, al, err=ctx.err, tiles=st, tiles_ready=True, max_ctas=cap)
            join.record(side)
        # The routed products' CTAs take their tiles from a counter: a prompt's start while the side products still hold
        # most multiprocessors, so the ones that start early do more of the work; a decode step's tiles are one to
        # three per CTA, and CTAs that are through with theirs take what is left (measured per decode step: batch 8
        # 3.70 -> 3.63 ms, batch 16 5.42 -> 5.23, batch 32 7.77 -> 7.52, batch 64 10.24 -> 10.18).  A handful of pairs
        # go without: their products split K instead.  A product sets its counter back itself; one that gave up on a
        # wait may not have, so the routing kernel zeroes both.
        c0 = c1 = None
        if many or al.TK > ops.GROUPED_SPLIT_MAX_PAIRS:
            if self._counters is None:
                self._counters = torch.zeros(2, dtype=torch.int32, device=dev)
            c0, c1 = self._counters[0:1], self._counters[1:2]
        if many:
            ops.router_topk(logits, K, self.renorm, idx, score, C, gate_logit, rule=self.rule)
            ops.moe_align(idx, KT, al, ctx.err, static_last=C, zero=self._counters)
        else:
            ops.moe_route_small(logits, K, self.renorm, C, gate_logit, idx, score, al, ctx.err, x=None, static=True,
                                zero=self._counters if c0 is not None else None, rule=self.rule)
        self.last_alignment = al
        x_sorted = ops.permute_rows(h, al.sorted_token, T * K)
        ops.gemm_fast_grouped(x_sorted, self.w_gate_up, act, al, swiglu=self.gated, err=ctx.err, tiles_ready=True,
                              counter=c0, act=self.expert_act)
        ops.gemm_fast_grouped(act, self.w_down, y, al, err=ctx.err, tiles_ready=True, counter=c1)
        main.wait_event(join)
        return RowMix(y, al.pair_pos[:T * KT].view(T, KT), score, None, None)


_side = {}


def _side_stream(dev):
    """One second stream per device for work that runs beside a step's main stream."""
    if ops.timing():                 # per-kernel timers are running: one stream, one kernel after the other
        return torch.cuda.current_stream(dev)
    key = torch.device(dev)
    if key not in _side:
        _side[key] = torch.cuda.Stream(device=key)
    return _side[key]


def _cat(ts):
    if len({t.dtype for t in ts}) > 1:
        ts = [t.float() for t in ts]
    return torch.cat(ts, dim=0).contiguous()


register_part("feed_forward", "dense_swiglu", DenseSwiGLU)
register_part("feed_forward", "dense_mlp", DenseMLP)
register_part("feed_forward", "sparse_moe_swiglu", SparseMoeSwiGLU)
