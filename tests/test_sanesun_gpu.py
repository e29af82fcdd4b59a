"""The Sanesun decoder and its mechanisms against the plain implementation (tests/plain_sanesun.py): every mixer
and the feed-forward alone, then whole models through the engine's step function, cache manager and scheduler, for
every way of cutting the work into steps.  The configurations are small and of this file's own making; weights are
random, and where random weights would hide a fault (a window's edge, a kept first token, a far key, a sink, one
channel's decay) they are shaped so that it shows."""
import json
import math

import pytest
import torch

import plain_sanesun as ps

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64

CONFIGS = {
    # every mixer twice with different sizes; grouped heads in the delta rule and in attention; value heads wider and
    # narrower than key heads; two windows with different numbers of kept tokens (page groups of their own); part of
    # a head turned and a whole head turned; a layer without a feed-forward; feed-forwards of two widths
    "U": ps.model_config(
        [ps.latent_layer(heads=3, dim=24, vdim=40, q_rank=20, kv_rank=36, scale=0.2, ff=120),
         ps.delta_layer(heads=4, kv_heads=2, dim=24, vdim=40, conv=4, ff=72),
         ps.attention_layer(heads=4, kv_heads=2, dim=32, vdim=48, window=24, keep_first=3, rot_dims=16, base=500.0,
                            scale=0.2, ff=120),
         ps.attention_layer(heads=3, kv_heads=3, dim=48, vdim=16, window=17, keep_first=5, rot_dims=48, base=10000.0,
                            scale=0.11, ff=0, kind="attention_2"),
         ps.delta_layer(heads=3, kv_heads=3, dim=40, vdim=24, conv=2, ff=0, kind="channel_delta_2"),
         ps.latent_layer(heads=2, dim=40, vdim=24, q_rank=48, kv_rank=20, scale=0.15, ff=72, kind="latent_attention_2")],
        width=96, vocab=210, eps=1e-5, embed_scale=4.0),
    # sizes of one: one head everywhere (a 1 x 1 mixing matrix), a convolution of one tap (no kept inputs), a window
    # of one with one kept token, a window longer than any request, no kept tokens, nothing of q and k turned (the
    # values still are), no embedding scale, a head size that is no multiple of sixteen
    "V": ps.model_config(
        [ps.attention_layer(heads=1, kv_heads=1, dim=40, vdim=20, window=1, keep_first=1, rot_dims=0, base=100.0,
                            scale=0.3, ff=48),
         ps.delta_layer(heads=1, kv_heads=1, dim=16, vdim=16, conv=1, ff=48),
         ps.latent_layer(heads=1, dim=16, vdim=16, q_rank=8, kv_rank=8, scale=0.25, ff=0),
         ps.attention_layer(heads=6, kv_heads=1, dim=16, vdim=32, window=500, keep_first=0, rot_dims=16, base=20.0,
                            scale=0.25, ff=48, kind="attention_2"),
         ps.delta_layer(heads=2, kv_heads=1, dim=48, vdim=72, conv=3, ff=0, rank=5, kind="channel_delta_2")],
        width=64, vocab=130),
    # sizes that the tensor-core kernels take: window attention whose mixed key is 128 long with eight heads (a decoded
    # row's heads in one tile) and one with twenty heads (a tile per head), latents of 64 and 128 elements (the
    # prompt kernels of both kinds), per-head products on the tensor cores in steps of more than 64 rows
    "W": ps.model_config(
        [ps.latent_layer(heads=4, dim=32, vdim=48, q_rank=48, kv_rank=64, scale=0.17, ff=256),
         ps.delta_layer(heads=4, kv_heads=2, dim=32, vdim=48, conv=3, ff=256),
         ps.attention_layer(heads=8, kv_heads=2, dim=64, vdim=32, window=48, keep_first=4, rot_dims=32, base=5000.0,
                            scale=0.125, ff=256),
         ps.delta_layer(heads=4, kv_heads=2, dim=32, vdim=48, conv=3, ff=256),
         ps.latent_layer(heads=2, dim=64, vdim=64, q_rank=32, kv_rank=128, scale=0.125, ff=0, kind="latent_attention_2"),
         ps.attention_layer(heads=20, kv_heads=4, dim=16, vdim=16, window=100, keep_first=0, rot_dims=16, base=100.0,
                            scale=0.25, ff=128, kind="attention_2")],
        width=128, vocab=344, eps=1e-6, embed_scale=8.0),
}
SEEDS = {"U": 3, "V": 5, "W": 7}
NAMES = ["U", "V", "W"]
TOL = {"float32": 1e-4, "bfloat16": 4e-2}


def ids_for(name, n, salt=0):
    g = torch.Generator().manual_seed(3000 + 31 * n + salt + ord(name))
    return [int(t) for t in torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g)]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        W = ps.random_weights(cfg, SEEDS[name])
        out[name] = (cfg, W, ps.write_folder(cfg, W, str(tmp_path_factory.mktemp("sane_" + name))))
    return out


_plain = {}


def plain_logits(models, name, ids):
    key = (name, tuple(ids))
    if key not in _plain:
        cfg, W, _ = models[name]
        _plain[key] = ps.forward(cfg, W, ids)
    return _plain[key]


def close(got, want, rel, what):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    err = (got - want).abs().reshape(got.shape[0], -1).max(dim=1).values
    bound = rel * max(1e-3, float(want.abs().max()))
    if bool((err > bound).any()):
        row = int(torch.nonzero(err > bound)[0])
        raise AssertionError(f"{what}: error {float(err[row]):.3g} > {bound:.3g} at row {row} "
                             f"(first of {int((err > bound).sum())})")


def make_runner(folder, dtype, max_tokens, max_requests=4, **kw):
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    return ModelRunner(folder, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests, **kw)


class Steps:
    """Feeds requests through ``ModelRunner.step`` and keeps the logits per (request, position)."""

    def __init__(self, runner):
        from nano_vllm_cpp_b200.engine.batch import StepEntry
        self.runner, self.StepEntry, self.fed, self.logits = runner, StepEntry, {}, {}

    def step(self, parts, end=()):
        entries = [self.StepEntry(rid, list(toks), list(range(len(toks)))) for rid, toks in parts]
        out = self.runner.step(entries).float().cpu()
        r = 0
        for e in entries:
            base = self.fed.get(e.rid, 0)
            for w in e.want:
                self.logits[(e.rid, base + w)] = out[r]
                r += 1
            self.fed[e.rid] = base + len(e.tokens)
        for rid in end:
            self.runner.close(rid)
            self.fed.pop(rid, None)
        self.runner.manager.check()

    def rows(self, rid, n):
        return torch.stack([self.logits[(rid, p)] for p in range(n)])


def check_rows(st, models, name, rid, ids, dtype, what):
    close(st.rows(rid, len(ids)), plain_logits(models, name, ids), TOL[dtype], what)


# ------------------------------------------------------------------------------- the parts alone
def ctx_for(dtype, fast=True):
    from nano_vllm_cpp_b200.csrc import ops
    from nano_vllm_cpp_b200.parts import RunContext
    return RunContext(device=torch.device(DEV), act_dtype=dtype, err=ops.ErrorFlag(DEV), page_size=16, fast_kernels=fast)


class Fetch:
    def __init__(self, tensors, prefix, dtype):
        self.t, self.p, self.dtype = tensors, prefix, dtype

    def __call__(self, name):
        t = self.t[self.p + name]
        small = t.dim() == 1 or name.endswith(".conv") or name in ("talk", "head_mix")
        return t.to(torch.float32 if small else self.dtype).to(DEV)

    def has(self, name):
        return (self.p + name) in self.t


def run_cut(part, cache, xs, cuts, dtype, tables, ctx, slots=None, call=None):
    """``xs``: one [T_i, width] input per request; ``cuts``: per step, the rows every request runs ((lo, hi) or
    None).  Returns per request the float32 outputs of all its rows."""
    from nano_vllm_cpp_b200.engine.batch import StepEntry, EntryInfo
    from batch_builder import build_batch
    outs = [[] for _ in xs]
    slots = slots or list(range(len(xs)))
    width = max(1, max(len(t) for t in tables))
    for cut in cuts:
        ses, infos, tabs, rows, who, row0 = [], [], [], [], [], 0
        for i, c in enumerate(cut):
            if c is None:
                continue
            lo, hi = c
            ses.append(StepEntry(i, [0] * (hi - lo), []))
            infos.append(EntryInfo(i, slots[i], lo, hi - lo, row0))
            tabs.append(tables[i])
            rows.append(xs[i][lo:hi])
            who.append((i, hi - lo))
            row0 += hi - lo
        batch = build_batch(ses, infos, [tabs], width, DEV)
        cache.reset_fresh(batch)
        h = torch.cat(rows).to(dtype).to(DEV)
        y = call(part, h, batch) if call else part.forward(h, batch, cache.view(0))
        ctx.err.check("part")
        at = 0
        for i, n in who:
            outs[i].append(y[at:at + n].float().cpu())
            at += n
    return [torch.cat(o) for o in outs]


def mixer_setup(layer, width, W, dtype, fast=True, pages=48, eps=1e-6):
    """The mixer as the model's own description makes it from a configuration of one layer."""
    from nano_vllm_cpp_b200.config import get_architecture
    from nano_vllm_cpp_b200.parts import build_part
    from nano_vllm_cpp_b200.cache import DeviceCache
    arch = get_architecture("Sanesun")
    cfg = ps.model_config([dict(layer, mlp=None)], width, 8, eps=eps)
    part = build_part("mixer", arch.build_model(arch.config_from_dict(cfg)).layers[0].mixer)
    ctx = ctx_for(dtype, fast)
    part.load(Fetch(W, "m.", dtype), ctx)
    cache = DeviceCache([part.cache_spec()], 16, 4, DEV, dtype)
    cache.allocate(pages, 48)
    return part, cache, ctx


def inputs(width, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(torch.bfloat16).double() for n in lengths]


CUTS = [[(0, 37), (0, 2)], [(37, 38), (2, 19)], [(38, 40), (19, 20)], [(40, 41), (20, 21)], [None, (21, 50)],
        [(41, 64), (50, 51)], [(64, 65), None], [(65, 66), None]]
PAGES = [[7, 3, 11, 0, 9], [5, 2, 8, 10]]
PART_TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}


# ---- the delta rule with a decay per key channel
DELTAS = [ps.delta_layer(heads=4, kv_heads=2, dim=24, vdim=40, conv=4),
          ps.delta_layer(heads=1, kv_heads=1, dim=32, vdim=16, conv=2),
          ps.delta_layer(heads=6, kv_heads=3, dim=40, vdim=72, conv=5, rank=7),
          ps.delta_layer(heads=2, kv_heads=2, dim=16, vdim=16, conv=1),
          ps.delta_layer(heads=2, kv_heads=1, dim=128, vdim=136, conv=3),
          ps.delta_layer(heads=3, kv_heads=1, dim=64, vdim=64, conv=4, rank=1)]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", DELTAS)
def test_channel_delta_alone(dtype, layer, fast):
    """Two requests in state slots of their own, in portions beside single rows; portions shorter than the
    convolution's reach, so that its kept inputs are a mix of old and new ones."""
    width, eps = 80, 1e-5
    W = ps.mixer_weights(layer, width, 21)
    part, cache, ctx = mixer_setup(layer, width, W, dtype, fast, eps=eps)
    xs = inputs(width, [66, 51], 22)
    got = run_cut(part, cache, xs, CUTS, dtype, [[], []], ctx, slots=[1, 3])
    for i, x in enumerate(xs):
        close(got[i], ps.channel_delta(x, W, "m.", layer["mixer"], eps), PART_TOL[dtype], f"request {i}")


@pytest.mark.parametrize("decoded", [False, True])
def test_every_key_channel_has_its_own_decay(decoded):
    """Decay biases that alternate between channels that forget at once and channels that keep everything: a
    kernel that took one decay per head (any one channel's, or their mean) would miss by far more than the
    tolerance, in a prompt and token by token."""
    layer = ps.delta_layer(heads=2, kv_heads=1, dim=24, vdim=32, conv=2)
    width, eps, T = 64, 1e-6, 40
    W = ps.mixer_weights(layer, width, 23)
    sign = torch.tensor([1.0, -1.0], dtype=F64).repeat(24)
    W["m.dt_bias"] = ps.to_bf16(6.0 * sign)
    W["m.a2"] = ps.to_bf16(0.05 * W["m.a2"])
    W["m.A_log"] = ps.to_bf16(torch.tensor([0.5, 1.0], dtype=F64))
    part, cache, ctx = mixer_setup(layer, width, W, torch.float32)
    xs = inputs(width, [T], 24)
    cuts = [[(0, T)]] if not decoded else [[(0, 3)]] + [[(t, t + 1)] for t in range(3, T)]
    got = run_cut(part, cache, xs, cuts, torch.float32, [[]], ctx, slots=[2])
    want = ps.channel_delta(xs[0], W, "m.", layer["mixer"], eps)
    close(got[0], want, 1e-4, "rows")
    flat = dict(W)
    flat["m.dt_bias"] = torch.zeros_like(W["m.dt_bias"])
    other = ps.channel_delta(xs[0], flat, "m.", layer["mixer"], eps)
    assert float((other - want).abs().max()) > 0.1 * float(want.abs().max())


def test_state_slots_are_cleared_when_used_again():
    """A request that takes the slot of a finished one starts from a zero matrix and zero kept inputs."""
    layer = ps.delta_layer(heads=2, kv_heads=2, dim=16, vdim=24, conv=3)
    width = 48
    W = ps.mixer_weights(layer, width, 25)
    part, cache, ctx = mixer_setup(layer, width, W, torch.float32)
    xs = inputs(width, [30, 22], 26)
    got = run_cut(part, cache, xs, [[(0, 30), None], [None, (0, 1)], [None, (1, 22)]], torch.float32, [[], []], ctx,
                  slots=[2, 2])
    for i, x in enumerate(xs):
        close(got[i], ps.channel_delta(x, W, "m.", layer["mixer"], 1e-6), 1e-4, f"request {i}")


def test_long_decoding_keeps_the_state():
    """Three hundred single rows after a short prompt: the matrix and the kept inputs go from step to step."""
    layer = ps.delta_layer(heads=2, kv_heads=1, dim=32, vdim=32, conv=4)
    width, T = 64, 320
    W = ps.mixer_weights(layer, width, 27)
    part, cache, ctx = mixer_setup(layer, width, W, torch.float32)
    xs = inputs(width, [T], 28)
    got = run_cut(part, cache, xs, [[(0, 20)]] + [[(t, t + 1)] for t in range(20, T)], torch.float32, [[]], ctx, slots=[0])
    close(got[0], ps.channel_delta(xs[0], W, "m.", layer["mixer"], 1e-6), 2e-4, "rows")


# ---- window attention with kept first tokens, sinks, mixed heads and turned values
WINDOWS = [ps.attention_layer(heads=4, kv_heads=2, dim=32, vdim=48, window=24, keep_first=3, rot_dims=16, base=500.0, scale=0.2),
           ps.attention_layer(heads=3, kv_heads=3, dim=48, vdim=16, window=17, keep_first=5, rot_dims=48, base=10000.0, scale=0.11),
           ps.attention_layer(heads=1, kv_heads=1, dim=40, vdim=20, window=1, keep_first=1, rot_dims=0, base=100.0, scale=0.3),
           ps.attention_layer(heads=6, kv_heads=1, dim=16, vdim=32, window=500, keep_first=0, rot_dims=16, base=20.0, scale=0.25),
           ps.attention_layer(heads=8, kv_heads=4, dim=64, vdim=64, window=16, keep_first=16, rot_dims=32, base=1e5, scale=0.125),
           ps.attention_layer(heads=2, kv_heads=2, dim=128, vdim=136, window=33, keep_first=2, rot_dims=64, base=3000.0, scale=0.09),
           ps.attention_layer(heads=5, kv_heads=5, dim=24, vdim=24, window=30, keep_first=40, rot_dims=8, base=50.0, scale=0.2),
           ps.attention_layer(heads=4, kv_heads=4, dim=96, vdim=80, window=40, keep_first=2, rot_dims=32, base=1e4, scale=0.1),
           ps.attention_layer(heads=8, kv_heads=2, dim=128, vdim=192, window=20, keep_first=50, rot_dims=128, base=1e6, scale=0.09)]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", WINDOWS)
def test_window_attention_alone(dtype, layer, fast):
    """Two requests on scattered pages, portions beside single rows.  Sizes: grouped heads, value heads wider and
    narrower than key heads, a window of one, a window longer than the requests, no kept tokens, as many kept tokens
    as the window and more, nothing / part / all of a q head turned."""
    width = 80
    W = ps.mixer_weights(layer, width, 31)
    part, cache, ctx = mixer_setup(layer, width, W, dtype, fast)
    xs = inputs(width, [66, 51], 32)
    got = run_cut(part, cache, xs, CUTS, dtype, PAGES, ctx)
    for i, x in enumerate(xs):
        close(got[i], ps.window_attention(x, W, "m.", layer["mixer"]), PART_TOL[dtype], f"request {i}")


@pytest.mark.parametrize("layer", [ps.attention_layer(heads=4, kv_heads=2, dim=32, vdim=48, window=300, keep_first=5, rot_dims=16, base=500.0, scale=0.2),
                                   ps.attention_layer(heads=2, kv_heads=1, dim=64, vdim=32, window=90, keep_first=70, rot_dims=32, base=1e4, scale=0.15),
                                   ps.attention_layer(heads=3, kv_heads=3, dim=128, vdim=144, window=1000, keep_first=0, rot_dims=0, base=50.0, scale=0.1),
                                   ps.attention_layer(heads=20, kv_heads=2, dim=16, vdim=32, window=200, keep_first=9, rot_dims=8, base=300.0, scale=0.25),
                                   ps.attention_layer(heads=16, kv_heads=4, dim=32, vdim=16, window=150, keep_first=1, rot_dims=32, base=1e3, scale=0.2)])
def test_short_entries_far_into_a_sequence(layer):
    """Single rows and portions of 2 to 16 rows hundreds of positions into a sequence, beside a longer portion of
    another request: in a bfloat16 run the short entries' keys are shared out among warps and blocks and merged, and
    with at most 16 query heads a single row's heads are worked on together (sizes: 2 to 20 heads, sixteen heads on
    four value heads, three value heads of one query head each)."""
    width = 80
    W = ps.mixer_weights(layer, width, 41)
    part, cache, ctx = mixer_setup(layer, width, W, torch.bfloat16, True, pages=64)
    xs = inputs(width, [700, 120], 42)
    g = torch.Generator().manual_seed(5)
    order = torch.randperm(60, generator=g).tolist()
    tables = [order[:44], order[44:52]]
    cuts = [[(0, 640), None], [(640, 641), None], [(641, 642), (0, 70)], [(642, 658), (70, 71)], [(658, 660), (71, 72)],
            [(660, 669), (72, 88)], [(669, 670), (88, 120)], [(670, 700), None]]
    got = run_cut(part, cache, xs, cuts, torch.bfloat16, tables, ctx)
    for i, x in enumerate(xs):
        close(got[i], ps.window_attention(x, W, "m.", layer["mixer"]), PART_TOL[torch.bfloat16], f"request {i}")


def edge_case(window, keep, T, i, j, width=64):
    """Weights and inputs for which row i's softmax weight falls on key j and on itself, if it sees j: the q heads
    are copies of the one k head (nothing of them is turned, no biases), row i's input is large, row j's is the same
    plus an equally large part at right angles to it in key space (the same score, another value), the other rows
    are small, and the sinks are far below."""
    layer = ps.attention_layer(heads=2, kv_heads=1, dim=32, vdim=32, window=window, keep_first=keep, rot_dims=0,
                               base=100.0, scale=1.0)
    W = ps.mixer_weights(layer, width, 33)
    W["m.q"] = torch.cat([W["m.k"], W["m.k"]])
    for b in ("m.q.b", "m.k.b"):
        W[b] = torch.zeros_like(W[b])
    W["m.talk"] = ps.to_bf16(torch.tensor([[0.75, 0.25], [0.5, 0.5]], dtype=F64))
    W["m.sink"] = ps.to_bf16(torch.tensor([-3.0, -2.0], dtype=F64))
    g = torch.Generator().manual_seed(34)
    x = 0.05 * torch.randn(T, width, generator=g, dtype=F64)
    big, side = torch.randn(width, generator=g, dtype=F64), torch.randn(width, generator=g, dtype=F64)
    kb, ks = W["m.k"] @ big, W["m.k"] @ side
    side = side - big * float(ks @ kb) / float(kb @ kb)
    big, side = big * (2.5 / float(kb.norm())), side * (2.5 / float((W["m.k"] @ side).norm()))
    x[i], x[j] = big, big + side
    return layer, W, x.to(torch.bfloat16).double()


EDGES = [(24, 3, 50, 27), (24, 3, 50, 26),          # the window's edge
         (24, 3, 50, 2), (24, 3, 50, 3),            # the last kept token and the one after it
         (16, 1, 47, 32), (16, 1, 47, 31),          # the same at page borders
         (16, 16, 47, 15), (16, 16, 47, 16),
         (17, 5, 420, 4), (17, 5, 420, 5),          # a kept token hundreds of positions back
         (400, 0, 430, 31), (400, 0, 430, 30),      # a far key through a long window
         (300, 2, 650, 351), (300, 2, 650, 350), (300, 2, 650, 1)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window,keep,i,j", EDGES)
def test_one_key_stands_out(window, keep, i, j, decoded, dtype):
    """A key just inside the window or among the kept first tokens takes half of row i's weight, the next one
    outside takes none; in a prompt, and when row i is decoded alone after single rows."""
    T = i + 3
    layer, W, x = edge_case(window, keep, T, i, j)
    part, cache, ctx = mixer_setup(layer, 64, W, dtype)
    table = [(5 * p + 3) % 47 for p in range((T + 15) // 16)]
    assert len(set(table)) == len(table)
    cuts = [[(0, T)]] if not decoded else [[(0, i - 2)]] + [[(t, t + 1)] for t in range(i - 2, T)]
    got = run_cut(part, cache, [x], cuts, dtype, [table], ctx)[0]
    m = layer["mixer"]
    want = ps.window_attention(x, W, "m.", m)
    close(got, want, PART_TOL[dtype], "rows")
    # the case shows what it is meant to show: a mask that differs in key j alone moves row i by far more
    if ps.visible(i, j, window, keep):
        flipped = {"size": window, "keep_first": j} if j < keep else {"size": i - j, "keep_first": keep}
    else:
        flipped = {"size": i - j + 1, "keep_first": keep}
    assert ps.visible(i, j, flipped["size"], flipped["keep_first"]) != ps.visible(i, j, window, keep)
    other = ps.window_attention(x, W, "m.", dict(m, mask=flipped))
    assert float((other[i] - want[i]).abs().max()) > 0.2 * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_sink_takes_weight_and_gives_nothing(dtype):
    """One head's sink far above its scores (that head's output nearly vanishes), another's far below (an ordinary
    softmax), a third in between; the sink is neither scaled nor mixed with the other heads' scores."""
    layer = ps.attention_layer(heads=3, kv_heads=1, dim=32, vdim=32, window=20, keep_first=2, rot_dims=16, base=100.0,
                               scale=0.05)
    width = 64
    W = ps.mixer_weights(layer, width, 35)
    W["m.sink"] = ps.to_bf16(torch.tensor([9.0, -30.0, 0.5], dtype=F64))
    part, cache, ctx = mixer_setup(layer, width, W, dtype)
    xs = inputs(width, [45], 36)
    got = run_cut(part, cache, xs, [[(0, 30)]] + [[(t, t + 1)] for t in range(30, 45)], dtype, [[4, 9, 1]], ctx)[0]
    want = ps.window_attention(xs[0], W, "m.", layer["mixer"])
    close(got, want, PART_TOL[dtype], "rows")
    none = dict(W)
    none["m.sink"] = torch.full((3,), -30.0, dtype=F64)
    other = ps.window_attention(xs[0], none, "m.", layer["mixer"])
    assert float((other - want).abs().max()) > 0.2 * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scores_are_mixed_across_heads_before_the_softmax(dtype):
    """A mixing matrix far from the unit matrix (heads that take another head's scores, with signs), with grouped
    key heads: head h's scores are sums over heads that read different key heads."""
    layer = ps.attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=40, keep_first=0, rot_dims=8, base=100.0,
                               scale=0.5)
    width = 64
    W = ps.mixer_weights(layer, width, 37)
    W["m.talk"] = ps.to_bf16(torch.tensor([[0.0, 0.0, 1.5, 0.0], [0.5, 0.0, 0.0, -1.0], [0.0, 1.0, 0.0, 0.0],
                                           [-0.5, 0.5, 0.5, 0.5]], dtype=F64))
    part, cache, ctx = mixer_setup(layer, width, W, dtype)
    xs = inputs(width, [50, 20], 38)
    got = run_cut(part, cache, xs, [[(0, 33), (0, 1)], [(33, 34), (1, 20)]] + [[(t, t + 1), None] for t in range(34, 50)],
                  dtype, [[4, 9, 1, 6], [2, 3]], ctx)
    for i, x in enumerate(xs):
        want = ps.window_attention(x, W, "m.", layer["mixer"])
        close(got[i], want, PART_TOL[dtype], f"request {i}")
    unit = dict(W)
    unit["m.talk"] = torch.eye(4, dtype=F64)
    other = ps.window_attention(xs[1], unit, "m.", layer["mixer"])
    assert float((other - want).abs().max()) > 0.2 * float(want.abs().max())


def test_values_are_turned_by_the_distance():
    """With one value row shared by all positions' inputs apart from the position itself, a value that was turned
    when written and turned back when read enters the output turned by the distance: a kernel that left out either
    turn, or turned only part of the head, would differ by far more than the tolerance."""
    layer = ps.attention_layer(heads=2, kv_heads=1, dim=16, vdim=40, window=64, keep_first=0, rot_dims=0, base=3.0,
                               scale=0.3)
    width = 48
    W = ps.mixer_weights(layer, width, 39)
    part, cache, ctx = mixer_setup(layer, width, W, torch.float32)
    xs = inputs(width, [40], 40)
    got = run_cut(part, cache, xs, [[(0, 25)]] + [[(t, t + 1)] for t in range(25, 40)], torch.float32, [[8, 0, 5]], ctx)[0]
    want = ps.window_attention(xs[0], W, "m.", layer["mixer"])
    close(got, want, 1e-4, "rows")
    # nothing of q and k is turned here, so the base reaches the values alone: with a huge base all pairs but the
    # first stand almost still
    still = ps.window_attention(xs[0], W, "m.", dict(layer["mixer"], rot={"dims": 0, "base": 1e12}))
    assert float((still - want).abs().max()) > 0.2 * float(want.abs().max())


# ---- latent attention
LATENTS = [ps.latent_layer(heads=3, dim=24, vdim=40, q_rank=20, kv_rank=36, scale=0.2),
           ps.latent_layer(heads=1, dim=16, vdim=16, q_rank=8, kv_rank=8, scale=0.25),
           ps.latent_layer(heads=2, dim=40, vdim=24, q_rank=48, kv_rank=20, scale=0.15),
           ps.latent_layer(heads=8, dim=64, vdim=48, q_rank=72, kv_rank=128, scale=0.125),
           ps.latent_layer(heads=5, dim=8, vdim=72, q_rank=4, kv_rank=260, scale=0.3)]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", LATENTS)
def test_latent_attention_alone(dtype, layer, fast):
    width, eps = 80, 1e-5
    W = ps.mixer_weights(layer, width, 41)
    part, cache, ctx = mixer_setup(layer, width, W, dtype, fast, eps=eps)
    xs = inputs(width, [66, 51], 42)
    got = run_cut(part, cache, xs, CUTS, dtype, PAGES, ctx)
    for i, x in enumerate(xs):
        close(got[i], ps.latent_attention(x, W, "m.", layer["mixer"], eps), PART_TOL[dtype], f"request {i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", [LATENTS[3], ps.latent_layer(heads=4, dim=40, vdim=56, q_rank=24, kv_rank=48, scale=0.2),
                                   ps.latent_layer(heads=2, dim=36, vdim=20, q_rank=16, kv_rank=64, scale=0.2)])
def test_latent_attention_steps_of_many_rows(dtype, layer):
    """Steps of hundreds of rows, alone and beside single rows: a bfloat16 run makes the per-head products of such
    steps another way (head by head on the tensor cores where the sizes allow) than those of a few rows."""
    width, eps = 96, 1e-5
    W = ps.mixer_weights(layer, width, 45)
    part, cache, ctx = mixer_setup(layer, width, W, dtype, pages=40, eps=eps)
    xs = inputs(width, [300, 101], 46)
    tables = [[(7 * p + 2) % 19 for p in range(19)], list(range(19, 26))]
    cuts = [[(0, 200), None], [(200, 201), (0, 100)], [(201, 300), (100, 101)]]
    got = run_cut(part, cache, xs, cuts, dtype, tables, ctx)
    for i, x in enumerate(xs):
        close(got[i], ps.latent_attention(x, W, "m.", layer["mixer"], eps), PART_TOL[dtype], f"request {i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("T,i,j", [(600, 590, 3), (600, 590, 0), (330, 320, 16), (330, 320, 15)])
def test_latent_attention_reads_a_far_key(T, i, j, decoded, dtype):
    """Among hundreds of keys the one of row j stands out for row i: queries and keys go through the same maps but
    for a shift of the input's columns, and row j's input is row i's shifted, so that the query latent of row i is
    the key latent of row j and their score is a squared length; row i's own key is as any other.  Without row j
    the output differs by far."""
    layer = ps.latent_layer(heads=2, dim=32, vdim=32, q_rank=32, kv_rank=32, scale=1.0)
    width, eps = 64, 1e-6
    W = ps.mixer_weights(layer, width, 43)
    W["m.dq"], W["m.dq.norm"], W["m.uq"] = torch.roll(W["m.dkv"], -1, dims=1), W["m.dkv.norm"], W["m.uk"]
    g = torch.Generator().manual_seed(44)
    x = torch.randn(T, width, generator=g, dtype=F64)
    x[j] = torch.roll(x[i], 1)
    x = x.to(torch.bfloat16).double()
    part, cache, ctx = mixer_setup(layer, width, W, dtype, pages=48, eps=eps)
    table = [(5 * p + 3) % 47 for p in range((T + 15) // 16)]
    cuts = [[(0, T)]] if not decoded else [[(0, i - 2)]] + [[(t, t + 1)] for t in range(i - 2, T)]
    got = run_cut(part, cache, [x], cuts, dtype, [table], ctx)[0]
    want = ps.latent_attention(x, W, "m.", layer["mixer"], eps)
    close(got, want, PART_TOL[dtype], "rows")
    y = x.clone()
    y[j] = 0.05 * torch.randn(width, generator=g, dtype=F64)
    other = ps.latent_attention(y.to(torch.bfloat16).double(), W, "m.", layer["mixer"], eps)
    assert float((other[i] - want[i]).abs().max()) > 0.2 * float(want.abs().max())


# ---- the feed-forward and the layer
@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff,pq", [(64, 48, (0.3, -0.7)), (96, 120, (-2.0, 1.5)), (256, 320, (0.0, 0.0)),
                                         (80, 8, (3.0, 3.0))])
def test_xielu_mlp_alone(dtype, width, ff, pq, fast):
    """Both branches of the activation with several pairs of its two numbers; one row, a handful and hundreds."""
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    cfg = ps.model_config([ps.delta_layer(heads=1, kv_heads=1, dim=16, vdim=16, conv=1, ff=ff)], width, 8)
    W = {k.replace("l0.mlp.", "m."): v for k, v in ps.random_weights(cfg, 45).items() if k.startswith("l0.mlp.")}
    W["m.act"] = ps.to_bf16(torch.tensor(pq, dtype=F64))
    part = build_part("feed_forward", PartSpec("dense_mlp", dict(hidden_size=width, intermediate_size=ff,
                                                                 activation="xielu", up_name="up", down_name="down",
                                                                 act_name="act")))
    part.load(Fetch(W, "m.", dtype), ctx_for(dtype, fast))
    for T in (1, 5, 70, 300):
        x = 2.0 * inputs(width, [T], 46 + T)[0]
        h32 = x.float().to(DEV)
        y = part.forward(h32.to(dtype), h32, None)
        close(y, ps.dense_mlp(x, W, "m."), PART_TOL[dtype], f"T={T}")


def test_the_activation_alone():
    """The function itself on a grid through zero, large arguments on both sides included."""
    from nano_vllm_cpp_b200.csrc import ops
    z = torch.cat([torch.linspace(-30, 30, 4001, dtype=F64), torch.tensor([0.0, -1e-4, 1e-4, -80.0, 50.0], dtype=F64)])
    for p, q in ((0.3, -0.7), (-2.0, 1.5), (4.0, -5.0)):
        sp = ps.softplus(torch.tensor([p, q], dtype=F64))
        out = torch.empty(z.shape[0], dtype=torch.float32, device=DEV).view(1, -1)
        ops.activation(z.float().to(DEV).view(1, -1), out, "xielu", (float(sp[0]), 0.5 + float(sp[1])))
        want = ps.xielu(z.float().double(), torch.tensor(p, dtype=F64), torch.tensor(q, dtype=F64))
        err = (out.cpu().double().view(-1) - want).abs() / (1.0 + want.abs())
        assert float(err.max()) < 1e-5, (p, q, float(err.max()))


def test_a_layer_reads_the_stream_once():
    """One norm, and both sublayers read its output: the stream after a layer is x + mixer(h) + mlp(h).  Checked on
    the stream after every layer of a model, which the plain implementation lists."""
    from nano_vllm_cpp_b200.engine.batch import StepEntry
    from nano_vllm_cpp_b200.parts.base import BranchSum
    name = "U"
    cfg = CONFIGS[name]
    W = ps.random_weights(cfg, SEEDS[name])
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        runner = make_runner(ps.write_folder(cfg, W, d), "float32", 128)
        seen = []

        def look(k, x, pending):
            # the layer's two outputs wait for the next norm's kernel to add them to the stream
            y = x.detach().clone()
            for part in ((pending.first, pending.second) if isinstance(pending, BranchSum) else (pending,)):
                y += part.float()
            seen.append(y.cpu())

        runner.model.after_call = look
        ids = ids_for(name, 40, salt=50)
        runner.step([StepEntry("s", ids, [])])
        runner.model.after_call = None
    want = []
    ps.forward(cfg, W, ids, layers_out=want)
    assert len(seen) == len(want) == len(cfg["layers"])
    for k, (a, b) in enumerate(zip(seen, want)):
        close(a, b, 1e-4, f"the stream after layer {k}")


# ------------------------------------------------------------------------------- whole models through the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(name, dtype, models):
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    for n in (1, 2, 3, 17, 64, 65, 150):
        ids = ids_for(name, n)
        st.step([(f"w{n}", ids)], end=[f"w{n}"])
        check_rows(st, models, name, f"w{n}", ids, dtype, f"{name} whole n={n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(name, dtype, models):
    """A short prompt in one step, then ninety rows one at a time (the windows pass over decoded tokens; pages
    behind every window go back, the kept first tokens' page stays; steps of the same shape are replayed from a
    captured graph), and a sequence that is decoded from its first token on."""
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    ids = ids_for(name, 100, salt=1)
    st.step([("d", ids[:10])])
    for t in range(10, 100):
        st.step([("d", ids[t:t + 1])])
    check_rows(st, models, name, "d", ids, dtype, f"{name} decode")
    st.step([], end=["d"])
    ids = ids_for(name, 20, salt=2)
    for t in range(20):
        st.step([("e", ids[t:t + 1])])
    check_rows(st, models, name, "e", ids, dtype, f"{name} decode from the first token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_several_sizes(name, dtype, models):
    runner = make_runner(models[name][2], dtype, 256)
    st = Steps(runner)
    ids = ids_for(name, 131, salt=3)
    sizes = [2, 1, 2, 14, 13, 3, 2, 30, 1, 1, 17, 2, 33, 10]
    assert sum(sizes) == 131
    at = 0
    for s in sizes:
        st.step([("p", ids[at:at + s])])
        at += s
    check_rows(st, models, name, "p", ids, dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_unequal_requests_together_with_pages_used_again(name, dtype, models):
    """Three slots and 192 tokens of pages for six requests that need more in turn: portions of some beside single
    rows of others; a finished request's pages and state slot go to the next one.  Every request's logits equal
    those of the request alone."""
    runner = make_runner(models[name][2], dtype, 192, max_requests=3)
    st = Steps(runner)
    L = {"a": 50, "b": 37, "c": 64, "d": 20, "e": 61, "f": 33}
    ids = {r: ids_for(name, n, salt=ord(r)) for r, n in L.items()}
    at = {r: 0 for r in L}

    def take(r, n):
        toks = ids[r][at[r]:at[r] + n]
        at[r] += len(toks)
        return (r, toks)

    def done(*rs):
        return [r for r in rs if at[r] == L[r]]

    st.step([take("a", 30), take("b", 2)])
    st.step([take("a", 1), take("b", 35), take("c", 3)], end=done("b"))
    st.step([take("a", 19), take("c", 1), take("d", 20)], end=done("a", "d"))
    st.step([take("c", 60), take("e", 2), take("f", 1)], end=done("c"))
    st.step([take("e", 1), take("f", 2)])
    st.step([take("e", 58), take("f", 30)], end=done("e", "f"))
    for r, n in L.items():
        assert at[r] == n
        check_rows(st, models, name, r, ids[r], dtype, f"{name} request {r}")


def drawn_config(rng):
    """A model of four to nine layers whose kinds, order and sizes are drawn: every kind at least once, up to two sets
    of sizes per kind, layers without a feed-forward, head counts from 1 to 24, sizes that do and do not fit the
    tensor-core kernels."""
    width, ff = rng.choice([128, 192, 256, 320, 384]), rng.choice([256, 320, 512, 640])
    n = rng.randint(4, 9)
    kinds = [rng.choice(["latent", "delta", "attn"]) for _ in range(n)]
    for must in ("latent", "delta", "attn"):
        if must not in kinds:
            kinds[rng.randrange(n)] = must

    def latent():
        return dict(heads=rng.choice([2, 4, 6, 8, 12]), dim=rng.choice([32, 48, 64, 96]),
                    vdim=rng.choice([32, 48, 64, 80, 96]), q_rank=rng.choice([48, 64, 96, 128]),
                    kv_rank=rng.choice([48, 64, 80, 96, 128, 160]), scale=rng.choice([0.125, 0.1, 0.18]))

    def delta():
        kv = rng.choice([1, 2, 4])
        return dict(heads=kv * rng.choice([1, 2, 3]), kv_heads=kv, dim=rng.choice([16, 32, 48, 64]),
                    vdim=rng.choice([16, 32, 48, 64, 96]), conv=rng.choice([2, 3, 4, 5]), rank=rng.choice([None, 8, 16, 24, 32]))

    def attn():
        kv, dim = rng.choice([1, 2, 3, 4, 6, 8]), rng.choice([32, 64, 96, 128])
        return dict(heads=kv * rng.choice([1, 2, 4]), kv_heads=kv, dim=dim, vdim=rng.choice([32, 64, 96, 128]),
                    window=rng.choice([17, 40, 64, 100, 150, 200]), keep_first=rng.choice([0, 1, 2, 4, 8, 20]),
                    rot_dims=rng.choice([0, 16, 32, dim]), base=rng.choice([1e4, 3e4, 5e5, 100.0]),
                    scale=rng.choice([0.125, 0.09, 0.2]))

    sizes = {"latent": [latent(), latent()], "delta": [delta(), delta()], "attn": [attn(), attn()]}
    make = {"latent": (ps.latent_layer, "latent_attention"), "delta": (ps.delta_layer, "channel_delta"),
            "attn": (ps.attention_layer, "attention")}
    layers = []
    for k in kinds:
        i = rng.randrange(2)
        fn, base = make[k]
        layers.append(fn(ff=rng.choice([ff, ff, ff, 0]), kind=base if i == 0 else base + "_2", **sizes[k][i]))
    return ps.model_config(layers, width=width, vocab=rng.choice([300, 512, 1000]), eps=rng.choice([1e-6, 1e-5]),
                           embed_scale=rng.choice([None, 4.0, 16.0]))


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5])
def test_drawn_models_in_a_mixed_schedule(seed, tmp_path):
    """Drawn models, both dtypes: five unequal requests on three slots and 576 tokens of pages, portions of up to 150
    tokens beside single rows of others, decoding over dozens of steps, finished requests' pages and slots used
    again; every request's logits equal the plain implementation's of the request alone."""
    import random
    cfg = drawn_config(random.Random(seed))
    W = ps.random_weights(cfg, seed)
    one = {"F": (cfg, W, ps.write_folder(cfg, W, str(tmp_path)))}
    L = {"a": 230, "b": 90, "c": 170, "d": 45, "e": 120}
    g = torch.Generator().manual_seed(seed)
    ids = {r: [int(t) for t in torch.randint(0, cfg["vocab"], (n,), generator=g)] for r, n in L.items()}
    for dtype in ("float32", "bfloat16"):
        st = Steps(make_runner(one["F"][2], dtype, 576, max_requests=3))
        at = {r: 0 for r in L}

        def take(r, n):
            toks = ids[r][at[r]:at[r] + n]
            at[r] += len(toks)
            return (r, toks)

        def done(*rs):
            return [r for r in rs if at[r] == L[r]]

        st.step([take("a", 150), take("b", 2)])
        st.step([take("a", 1), take("b", 88), take("c", 3)], end=done("b"))
        for _ in range(30):
            st.step([take("a", 1), take("c", 1)])
        st.step([take("a", 49), take("c", 2), take("d", 45)], end=done("a", "d"))
        st.step([take("c", 135), take("e", 7)], end=done("c"))
        for _ in range(40):
            st.step([take("e", 1)])
        st.step([take("e", 73)], end=done("e"))
        for r, n in L.items():
            assert at[r] == n
            check_rows(st, one, "F", r, ids[r], dtype, f"seed {seed} {dtype} request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_a_row(dtype, models):
    """The same request whole, in portions and beside another request: float32 rows agree to rounding of sums,
    bfloat16 rows to bfloat16 rounding."""
    name = "U"
    ids = ids_for(name, 70, salt=9)
    other = ids_for(name, 40, salt=10)
    runs = []
    for cut in ([70], [33, 1, 2, 34], [64, 6]):
        runner = make_runner(models[name][2], dtype, 256)
        st = Steps(runner)
        at = 0
        for k, s in enumerate(cut):
            st.step([("x", ids[at:at + s])] + ([("o", other[:20] if k == 0 else other[20 + k:21 + k])] if len(cut) == 4 else []))
            at += s
        runs.append(st.rows("x", 70))
    for r in runs[1:]:
        close(r, runs[0], 2e-5 if dtype == "float32" else 3e-2, "the same rows cut another way")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype, models):
    """The engine's own entry point, scheduler and sampling: greedy tokens follow the plain implementation's up
    to the first position where its two best logits are closer than the tolerance."""
    from nano_vllm_cpp_b200 import LLMEngine, SamplingParams
    name = "U"
    cfg, W, folder = models[name]
    prompts = [ids_for(name, 9, salt=20), ids_for(name, 3, salt=21), ids_for(name, 30, salt=22)]
    eng = LLMEngine(folder, max_model_len=96, num_kv_blocks=24, dtype=dtype, max_num_seqs=2, log_stats=False)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for k, tok in enumerate(o["token_ids"]):
            logits = ps.forward(cfg, W, seq)[-1]
            best = int(torch.argmax(logits))
            if best != tok:
                lead = float(logits[best] - logits[tok])
                bound = 2 * TOL[dtype] * float(logits.abs().max())
                assert lead <= bound, f"token {k} of a prompt of {len(p)}: {tok}, plain takes {best} with a lead of {lead:.3g}"
                break
            seq.append(tok)


def test_command_line_serves_the_design(models, tmp_path, capsys):
    """``nanovllm <folder> --tokens ...`` and ``nanovllm --config <json>`` (random weights) run this design as they
    run the others; the greedy tokens from the folder are the plain implementation's."""
    from nano_vllm_cpp_b200 import cli
    name = "V"
    cfg, W, folder = models[name]
    prompt = ids_for(name, 7, salt=30)
    rc = cli.main([folder, "--tokens", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                   "--dtype", "float32", "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0, out
    toks = [int(t) for t in out.strip().splitlines()[-1].split(":")[1].split()]
    assert toks == ps.greedy_generate(cfg, W, prompt, 6)
    path = tmp_path / "config.json"
    path.write_text(json.dumps(CONFIGS["U"]))
    rc = cli.main(["--config", str(path), "--seed", "4", "--tokens", "5,6,7", "--max-tokens", "4", "--temperature", "0",
                   "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0 and len(out.strip().splitlines()[-1].split(":")[1].split()) == 4
