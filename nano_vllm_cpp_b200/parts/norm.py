"""Norms fused with the residual sum: RMSNorm, and the dynamic tanh, which needs no statistics."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, RowMix, BranchSum, NormedBranch, TensorSpec
from .registry import register_part


class RMSNorm(Norm):
    """``x += branch; y = x * rsqrt(mean(x^2) + eps) * w`` (src/hip_ops.hip:395-417).

    The residual stream and the statistics are float32; ``y`` is written in the activation dtype.
    A branch that is still a ``RowMix`` is summed by the same kernel, and so are the two outputs of a
    ``BranchSum``.  A ``NormedBranch`` (a sublayer output with a norm of its own, ``n``) is taken in by one launch
    that does both norms: ``x += rms_n(branch) * w_n; y = rms(x) * w``.
    """
    accepts_mix = True
    accepts_sum = True
    accepts_normed = True

    def __init__(self, size: int, eps: float, weight_offset: float = 0.0, weight_name: str = "weight"):
        """``weight_offset``: the stored weight lies around zero and the multiplier is ``weight_offset`` + weight
        (1.0 for the "one plus weight" form); the sum is taken once, in float32, when the weight is loaded.
        ``weight_name``: the tensor's name behind the part's prefix."""
        self.size, self.eps = size, float(eps)
        self.weight_offset, self.weight_name = float(weight_offset), weight_name

    def tensor_specs(self, available=None):
        return {self.weight_name: TensorSpec((self.size,), init="near_zero" if self.weight_offset else "ones", kind="vector")}

    def load(self, fetch, ctx):
        self.ctx = ctx
        self.weight = fetch(self.weight_name)
        if self.weight_offset:
            self.weight = (self.weight.float() + self.weight_offset).contiguous()

    def add_normed(self, x, branches, want_rows: bool = True, *, branch_weights=None, mix_scale: float = 1.0):
        """``x += rms(y) * w`` in place, the norm on the branch and not on the stream: ``y`` is the one branch, or
        ``mix_scale`` times the sum of the branches each RMS-normed (this norm's eps) with its own weight.  Returns the
        stream's rows after the sum in the run's activation dtype (the stream itself in a float32 run), which the
        next sublayer's products read; None if not wanted.  No branches: only the rows are made."""
        out = None
        if want_rows:
            out = x if self.ctx.act_dtype == torch.float32 else torch.empty(x.shape, dtype=self.ctx.act_dtype, device=x.device)
        if branches or (out is not None and out is not x):
            ops.branch_norm_add(x, branches, self.weight, self.eps, None if out is x else out,
                                branch_weights=branch_weights, mix_scale=mix_scale)
        return out

    def forward(self, x, branch, want_f32=False):
        out = torch.empty(x.shape, dtype=self.ctx.act_dtype, device=x.device)
        out32 = None
        if want_f32:
            out32 = out if out.dtype == torch.float32 else torch.empty_like(x)
        mix = branch2 = None
        if isinstance(branch, NormedBranch):
            inner, first = branch.branch, branch.norm
            if isinstance(inner, RowMix) and inner.index.shape[1] <= ops.ADD_RMSNORM_MAX_MIX:
                mix, inner = inner.as_tuple(), None
            elif isinstance(inner, (RowMix, BranchSum)):
                inner = inner.sum()
            ops.add_rmsnorm(x, inner, self.weight, self.eps, out, None if out32 is out else out32, mix=mix,
                            branch_weight=first.weight, branch_eps=first.eps)
            return out, out32
        if isinstance(branch, RowMix):
            if branch.index.shape[1] <= ops.ADD_RMSNORM_MAX_MIX:
                mix, branch = branch.as_tuple(), None
            else:
                branch = branch.sum()
        elif isinstance(branch, BranchSum):
            branch, branch2 = branch.first, branch.second
        ops.add_rmsnorm(x, branch, self.weight, self.eps, out, None if out32 is out else out32, mix=mix,
                        branch2=branch2)
        return out, out32


class DynamicTanh(Norm):
    """``y = tanh(alpha * x) * gain + shift``: a norm without mean or variance, every element by itself.  ``alpha`` is
    one number, ``gain`` and ``shift`` are vectors over the width; all three are learned and held in float32, and the
    arithmetic is float32.  The sum of the pending branch into the stream happens in the same kernel.

    ``read_streams`` is the same norm for a model that keeps several copies of its stream (``parts.streams``): the
    kernel brings the copies up to date, reads them with the next sublayer's weights and norms what it read."""
    accepts_mix = True

    def __init__(self, size: int, weight_name: str = "weight", shift_name: str = "bias", alpha_name: str = "alpha"):
        self.size = size
        self.weight_name, self.shift_name, self.alpha_name = weight_name, shift_name, alpha_name

    def tensor_specs(self, available=None):
        return {self.weight_name: TensorSpec((self.size,), init="ones", kind="vector"),
                self.shift_name: TensorSpec((self.size,), init="near_zero", kind="vector"),
                self.alpha_name: TensorSpec((), init="ones", kind="vector")}

    def load(self, fetch, ctx):
        self.ctx = ctx
        self.gain = fetch(self.weight_name).float().contiguous()
        self.shift = fetch(self.shift_name).float().contiguous()
        self.alpha = fetch(self.alpha_name).float().reshape(1).contiguous()

    def _outputs(self, T, device, want_f32):
        out = torch.empty((T, self.size), dtype=self.ctx.act_dtype, device=device)
        out32 = None
        if want_f32:
            out32 = out if out.dtype == torch.float32 else torch.empty((T, self.size), dtype=torch.float32, device=device)
        return out, out32

    def read_streams(self, x, streams: int, branch, carry, write, read, want_f32: bool = False):
        """``x`` [T, streams * size]: the copies, brought up to date in place with ``branch`` (a float32 matrix, a
        ``RowMix`` or None) through ``carry`` and ``write``, then read with ``read`` (None: their plain sum) and
        normed.  Returns (rows in the activation dtype, float32 copy or None)."""
        out, out32 = self._outputs(x.shape[0], x.device, want_f32)
        mix = None
        if isinstance(branch, RowMix):
            if branch.gate_logit is None and branch.index.shape[1] <= ops.STREAM_MAX_MIX:
                mix, branch = branch.as_tuple(), None
            else:
                branch = branch.sum()
        ops.stream_mix_norm(x, streams, branch=branch, mix=mix, carry=carry, write=write, read=read,
                            norm=(self.alpha, self.gain, self.shift), out=out, out32=None if out32 is out else out32)
        return out, out32

    def forward(self, x, branch, want_f32=False):
        return self.read_streams(x, 1, branch, None, None, None, want_f32)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
