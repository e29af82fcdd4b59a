"""Arrangements: how a layer's parts are wired around the residual stream.

A layer as data is an arrangement kind plus the parts it names: ``LayerSpec(arrangement, parts, names)``.
Which parts a layer has is the arrangement's business, not ``LayerSpec``'s: the pre-norm block takes four
(``norm1, mixer, norm2, feed_forward``); another arrangement (a parallel block with one norm, a layer without a
feed-forward, a post-norm block) declares its own slots and is registered like any other part:

    class Parallel(Arrangement):
        slots = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}   # slot -> family
        def forward(self, x, pending, batch, cache): ...
    register_part("arrangement", "parallel", Parallel)
    LayerSpec(arrangement="parallel", parts={"norm": ..., "mixer": ..., "feed_forward": ...},
              names={"norm": "ln.", "mixer": "attn.", "feed_forward": "mlp."})
"""
from __future__ import annotations

from .base import PartSpec, StreamRows, BranchSum, NormedBranch, resolve_branch
from .registry import register_part, build_part

_DEFAULT_NAMES = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.",
                  "feed_forward": "mlp."}


class LayerSpec:
    """One layer as data.  ``parts``: slot name -> ``PartSpec``; ``names``: slot name -> prefix of the slot's
    tensors inside the layer (a slot without an entry uses ``<slot>.``).  The slots of the pre-norm block may be
    given as keywords: ``LayerSpec(norm1=..., mixer=..., norm2=..., feed_forward=...)``.  ``params``: constants of
    the arrangement itself."""

    def __init__(self, arrangement: str = "prenorm", parts: dict | None = None, names: dict | None = None,
                 params: dict | None = None, **slots):
        self.arrangement = arrangement
        self.params = dict(params or {})         # the arrangement's own constants (how many copies of the stream, ...)
        self.parts = dict(parts or {})
        for slot, spec in slots.items():
            if not isinstance(spec, PartSpec):
                raise TypeError(f"LayerSpec: {slot!r} must be a PartSpec")
            self.parts[slot] = spec
        self.names = dict(_DEFAULT_NAMES if names is None else names)

    def __getattr__(self, slot):            # spec.mixer, spec.feed_forward, ...: the slot's PartSpec
        parts = self.__dict__.get("parts", {})
        if slot in parts:
            return parts[slot]
        raise AttributeError(slot)

    def prefix(self, slot: str) -> str:
        return self.names.get(slot, slot + ".")


class Arrangement:
    """Base of the arrangements.  ``slots`` maps each slot name to the family its part is built from; the parts
    become attributes of the same names.  ``forward(x, pending, batch, cache) -> pending``: ``x`` is the float32
    residual stream, changed in place; ``pending`` is a branch output that has not been added to it yet (the sum
    is fused with whichever norm runs next), or None; ``cache`` is the layer call's ``CacheView``."""
    slots: dict = {}
    optional: tuple = ()                # slots that a layer may leave out (their attribute is then None)
    cache_slot: str = "mixer"           # the slot whose part says what the layer keeps per request (None: nothing)

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        missing = [s for s in self.slots if s not in spec.parts and s not in self.optional]
        extra = [s for s in spec.parts if s not in self.slots]
        if missing or extra:
            raise ValueError(f"arrangement {spec.arrangement!r} takes the parts {sorted(self.slots)}; "
                             f"missing {missing}, not taken {extra}")
        for slot, family in self.slots.items():
            setattr(self, slot, build_part(family, spec.parts[slot]) if slot in spec.parts else None)

    def parts(self):
        """(tensor-name prefix inside the layer, part) for every part."""
        return [(self.spec.prefix(slot), getattr(self, slot)) for slot in self.slots if getattr(self, slot) is not None]

    def cache_spec(self):
        return getattr(self, self.cache_slot).cache_spec() if self.cache_slot else None

    def forward(self, x, pending, batch, cache):
        raise NotImplementedError


class PreNormBlock(Arrangement):
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (src/model.cpp:762-832).

    The sum into the residual stream is fused with the next norm: a block hands its last branch
    output on as ``pending`` instead of adding it, and every norm adds what is pending first —
    the reference's ``rms_norm_add`` convention (src/hip_ops.hip:395-417).
    """
    slots = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward"}

    def forward(self, x, pending, batch, cache):
        h, _ = self.norm1.forward(x, resolve_branch(self.norm1, pending))
        pending = self.mixer.forward(h, batch, cache)
        h, h32 = self.norm2.forward(x, resolve_branch(self.norm2, pending), want_f32=self.feed_forward.wants_f32_input)
        pending = self.feed_forward.forward(h, h32, batch)
        return pending


register_part("arrangement", "prenorm", PreNormBlock)


class ParallelBlock(Arrangement):
    """One norm, and both sublayers read its output: ``h = norm1(x); x += mixer(h) + feed_forward(h)``.  A layer may
    have no feed-forward.  The sum into the stream is left to whichever norm runs next, which adds both outputs in
    its own kernel (``BranchSum``)."""
    slots = {"norm1": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    optional = ("feed_forward",)

    def forward(self, x, pending, batch, cache):
        ff = self.feed_forward
        h, h32 = self.norm1.forward(x, resolve_branch(self.norm1, pending),
                                    want_f32=ff is not None and ff.wants_f32_input)
        y = self.mixer.forward(h, batch, cache)
        if ff is None:
            return y
        return BranchSum(y, ff.forward(h, h32, batch))


register_part("arrangement", "parallel", ParallelBlock)


class BranchNormBlock(Arrangement):
    """The norm on the sublayer's output only: ``x += norm1(mixer(x)); x += norm2(feed_forward(x))`` and, if the
    layer has one, ``x += norm3(token_input(x))``.  The sublayers read the residual stream itself (its rows in the
    activation dtype; each norm's kernel writes them after its sum).  A layer may have no feed-forward and no
    token input.  Nothing is left pending: the stream is complete when the layer returns, and its rows are handed
    on as ``StreamRows``."""
    slots = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward",
             "norm3": "norm", "token_input": "token_input"}
    optional = ("norm2", "feed_forward", "norm3", "token_input")

    def __init__(self, spec):
        super().__init__(spec)
        if (self.norm2 is None) != (self.feed_forward is None) or (self.norm3 is None) != (self.token_input is None):
            raise ValueError("a branch-norm layer's feed-forward and token input each come with their norm")

    def forward(self, x, pending, batch, cache):
        from .parallel import MixedBranches
        if isinstance(pending, StreamRows):
            h = pending.rows
        elif pending is None:
            h = self.norm1.add_normed(x, [])
        else:
            raise ValueError("a branch-norm layer takes the residual stream with nothing pending")
        y = self.mixer.forward(h, batch, cache)
        if isinstance(y, MixedBranches):
            h = self.norm1.add_normed(x, y.branches, branch_weights=y.weights, mix_scale=y.scale)
        else:
            h = self.norm1.add_normed(x, [y])
        if self.feed_forward is not None:
            h = self.norm2.add_normed(x, [self.feed_forward.forward(h, h, batch)])
        if self.token_input is not None:
            h = self.norm3.add_normed(x, [self.token_input.forward(h, batch)])
        return StreamRows(h)


register_part("arrangement", "branch_norm", BranchNormBlock)


class SandwichBlock(Arrangement):
    """A norm before and after each sublayer: ``x += norm1b(mixer(norm1(x))); x += norm2b(feed_forward(norm2(x)))``.
    A layer may have no feed-forward.  A sublayer's output is handed on as a ``NormedBranch``: the norm that runs
    next (this layer's ``norm2``, the next layer's ``norm1`` or the model's last norm) norms it with the output
    norm's weight, adds it to the stream and norms the stream for its own sublayer, all in one kernel."""
    slots = {"norm1": "norm", "mixer": "mixer", "norm1b": "norm", "norm2": "norm", "feed_forward": "feed_forward",
             "norm2b": "norm"}
    optional = ("norm2", "feed_forward", "norm2b")

    def __init__(self, spec):
        super().__init__(spec)
        if len({self.norm2 is None, self.feed_forward is None, self.norm2b is None}) != 1:
            raise ValueError("a sandwich layer's feed-forward comes with both of its norms")
        for n in (self.norm1b, self.norm2b):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError("a sandwich layer's output norms must be able to norm a branch (RMSNorm)")

    def forward(self, x, pending, batch, cache):
        h, _ = self.norm1.forward(x, resolve_branch(self.norm1, pending))
        pending = NormedBranch(self.mixer.forward(h, batch, cache), self.norm1b)
        ff = self.feed_forward
        if ff is None:
            return pending
        h, h32 = self.norm2.forward(x, resolve_branch(self.norm2, pending), want_f32=ff.wants_f32_input)
        return NormedBranch(ff.forward(h, h32, batch), self.norm2b)


register_part("arrangement", "sandwich", SandwichBlock)


def build_layer(spec: LayerSpec):
    from .registry import ARRANGEMENTS
    try:
        cls = ARRANGEMENTS[spec.arrangement]
    except KeyError:
        raise KeyError(f"no arrangement {spec.arrangement!r} is registered; known: {sorted(ARRANGEMENTS)}") from None
    return cls(spec)
