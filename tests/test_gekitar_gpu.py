"""The Gekitar decoder and its mechanisms against the plain implementation (tests/plain_gekitar.py): every mixer and
both feed-forwards alone, the layer's four norms, then whole models through the engine's step function, cache manager
and scheduler, for every way of cutting the work into steps.  The configurations are small and of this file's own
making; weights are random, and where random weights would hide a fault (a window's edge, a far key, the sink, the
cap, the clamp) they are shaped so that it shows."""
import json
import math

import pytest
import torch

import plain_gekitar as pg

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}

CONFIGS = {
    # every mixer with two sets of sizes; a reader of another layer's latents whose window is longer than its owner's
    # and one whose window is shorter; value heads wider and narrower than key heads; part of an attention head turned
    # with stretched frequencies, a whole head turned without; mixtures with and without a shared expert; a layer
    # without a feed-forward
    "P": pg.model_config(
        [pg.latent_layer(heads=3, dim=24, rot_dim=8, vdim=40, q_rank=20, kv_rank=36, scale=0.2, base=500.0,
                         mlp=pg.dense_ff(120, 1.0)),
         pg.latent_layer(heads=2, dim=40, rot_dim=16, vdim=24, q_rank=48, kv_rank=20, scale=0.15, base=1e4, window=24,
                         mlp=pg.moe_ff(5, 2, 24, 40)),
         pg.sink_layer(heads=4, kv_heads=2, dim=32, vdim=48, rot_dims=16, base=300.0, scale=0.3, softcap=5.0,
                       scaling=YARN, mlp=pg.moe_ff(6, 3, 32)),
         pg.latent_layer(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=12, kv_rank=20, scale=0.25, base=1e4, window=40,
                         kv_from=1, mlp=None),
         pg.sink_layer(heads=3, kv_heads=3, dim=48, vdim=16, rot_dims=48, base=1e4, scale=0.11, softcap=30.0,
                       mlp=pg.dense_ff(72, 3.0), kind="attention_2"),
         pg.latent_layer(heads=2, dim=24, rot_dim=16, vdim=32, q_rank=16, kv_rank=20, scale=0.2, base=1e4, window=9,
                         kv_from=1, mlp=pg.dense_ff(48, 0.5), kind="latent_attention_2_2")],
        width=96, vocab=210, eps=1e-5, embed_scale=4.0),
    # sizes of one and values that other models make equal: one head everywhere, a window of one, a window longer than
    # any request, one expert, every expert chosen, a turned part of two elements, no embedding scale, a reader whose
    # owner sees every position
    "Q": pg.model_config(
        [pg.latent_layer(heads=1, dim=16, rot_dim=2, vdim=16, q_rank=8, kv_rank=8, scale=0.25, base=20.0,
                         mlp=pg.moe_ff(1, 1, 16, 8)),
         pg.sink_layer(heads=1, kv_heads=1, dim=40, vdim=20, rot_dims=2, base=100.0, scale=0.3, softcap=1.0,
                       mlp=pg.moe_ff(4, 4, 24)),
         pg.latent_layer(heads=2, dim=8, rot_dim=2, vdim=24, q_rank=4, kv_rank=8, scale=0.3, base=20.0, window=1,
                         kv_from=0, mlp=pg.dense_ff(48, 2.0)),
         pg.latent_layer(heads=5, dim=8, rot_dim=4, vdim=8, q_rank=6, kv_rank=12, scale=0.3, base=50.0, window=500,
                         mlp=None),
         pg.sink_layer(heads=6, kv_heads=1, dim=16, vdim=32, rot_dims=0, base=10.0, scale=0.25, softcap=8.0, mlp=None,
                       kind="attention_2")],
        width=64, vocab=130),
    # sizes that the tensor-core kernels take: cached rows of 64 and 128 elements, attention heads of 64, per-head
    # products on the tensor cores in steps of more than 64 rows, expert widths of 64 with a shared expert of two
    # expert widths (it rides in the grouped products)
    "R": pg.model_config(
        [pg.latent_layer(heads=4, dim=32, rot_dim=16, vdim=48, q_rank=48, kv_rank=48, scale=0.17, base=1e4,
                         mlp=pg.dense_ff(256, 1.5)),
         pg.latent_layer(heads=2, dim=64, rot_dim=32, vdim=64, q_rank=32, kv_rank=96, scale=0.125, base=5e4, window=48,
                         mlp=pg.moe_ff(8, 2, 64, 128)),
         pg.sink_layer(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, base=1e5, scale=0.125, softcap=20.0,
                       scaling=YARN, mlp=pg.moe_ff(8, 3, 64, 96)),
         pg.latent_layer(heads=4, dim=32, rot_dim=32, vdim=32, q_rank=32, kv_rank=96, scale=0.15, base=5e4, window=48,
                         kv_from=1, mlp=pg.dense_ff(128, 1.5))],
        width=128, vocab=344, eps=1e-6, embed_scale=8.0),
}
SEEDS = {"P": 3, "Q": 5, "R": 7}
NAMES = ["P", "Q", "R"]
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
EDGE = 0.01                  # a router margin (the gap between the last chosen and the best unchosen logit, as a fraction
MAX_EDGE_SHARE = 0.25        # of the spread of the row's logits) below which a bfloat16 run may rightly choose otherwise


def ids_for(name, n, salt=0):
    g = torch.Generator().manual_seed(1000 * ord(name) + 7 * n + salt)
    return [int(t) for t in torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g)]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        W = pg.random_weights(cfg, SEEDS[name])
        out[name] = (cfg, W, pg.write_folder(cfg, W, str(tmp_path_factory.mktemp("gekitar_" + name))))
    return out


_plain = {}


def plain_logits(models, name, ids):
    """(logits, per row the smallest router margin of any layer)"""
    key = (name, tuple(ids))
    if key not in _plain:
        cfg, W, _ = models[name]
        margins = []
        lg = pg.forward(cfg, W, ids, margins=margins)
        _plain[key] = (lg, torch.stack(margins).min(dim=0).values if margins else torch.full((len(ids),), math.inf))
    return _plain[key]


def close(got, want, rel, what, margins=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    err = (got - want).abs().reshape(got.shape[0], -1).max(dim=1).values
    bound = rel * max(1e-3, float(want.abs().max()))
    bad = err > bound
    if margins is not None:
        edge = margins < EDGE
        assert int(edge.sum()) <= max(4, MAX_EDGE_SHARE * len(edge)), f"{what}: too many rows on a router's edge"
        if bool(edge.any()):            # every later row may read what an edge row left in the cache
            bad[int(torch.nonzero(edge)[0]):] = False
    if bool(bad.any()):
        row = int(torch.nonzero(bad)[0])
        raise AssertionError(f"{what}: error {float(err[row]):.3g} > {bound:.3g} at row {row} (first of {int(bad.sum())})")


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
    want, margins = plain_logits(models, name, ids)
    close(st.rows(rid, len(ids)), want, TOL[dtype], what, margins if dtype == "bfloat16" else None)


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
        return t.to(torch.float32 if t.dim() == 1 else self.dtype).to(DEV)

    def has(self, name):
        return (self.p + name) in self.t


def run_cut(parts, cache, xs, cuts, dtype, tables, ctx):
    """``parts``: the mixers that run on the same rows, in order, each with the cache view of its index (a reader of
    another's pages after its owner); ``xs``: one [T_i, width] input per request; ``cuts``: per step, the rows every
    request runs ((lo, hi) or None).  Returns per part and request the float32 outputs of all rows."""
    from nano_vllm_cpp_b200.engine.batch import StepEntry, EntryInfo
    from batch_builder import build_batch
    outs = [[[] for _ in xs] for _ in parts]
    width = max(1, max(len(t) for t in tables))
    for cut in cuts:
        ses, infos, tabs, rows, who, row0 = [], [], [], [], [], 0
        for i, c in enumerate(cut):
            if c is None:
                continue
            lo, hi = c
            ses.append(StepEntry(i, [0] * (hi - lo), []))
            infos.append(EntryInfo(i, i, lo, hi - lo, row0))
            tabs.append(tables[i])
            rows.append(xs[i][lo:hi])
            who.append((i, hi - lo))
            row0 += hi - lo
        batch = build_batch(ses, infos, [tabs], width, DEV)
        h = torch.cat(rows).to(dtype).to(DEV)
        for k, part in enumerate(parts):
            y = part.forward(h, batch, cache.view(k))
            ctx.err.check("part")
            at = 0
            for i, n in who:
                outs[k][i].append(y[at:at + n].float().cpu())
                at += n
    return [[torch.cat(o) for o in per] for per in outs]


def mixers_setup(layers, width, Ws, dtype, fast=True, pages=48, eps=1e-6):
    """The mixers as the model's own description makes them from a configuration of these layers, with one cache."""
    from nano_vllm_cpp_b200.config import get_architecture
    from nano_vllm_cpp_b200.parts import build_part
    from nano_vllm_cpp_b200.cache import DeviceCache
    arch = get_architecture("Gekitar")
    cfg = pg.model_config([dict(L, mlp=None) for L in layers], width, 8, eps=eps)
    spec = arch.build_model(arch.config_from_dict(cfg))
    ctx = ctx_for(dtype, fast)
    parts, specs = [], []
    for k, L in enumerate(layers):
        part = build_part("mixer", spec.layers[k].mixer)
        part.load(Fetch(Ws[k], "m.", dtype), ctx)
        parts.append(part)
        src = L["mixer"].get("kv_from")
        specs.append(part.cache_spec() if src is None else ("shared", src))
    cache = DeviceCache(specs, 16, 4, DEV, dtype)
    assert len(cache.windows) == 1
    cache.allocate(pages, 48)
    return parts, cache, ctx


def inputs(width, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(torch.bfloat16).double() for n in lengths]


CUTS = [[(0, 37), (0, 2)], [(37, 38), (2, 19)], [(38, 40), (19, 20)], [(40, 41), (20, 21)], [None, (21, 50)],
        [(41, 64), (50, 51)], [(64, 65), None], [(65, 66), None]]
PAGES = [[7, 3, 11, 0, 9], [5, 2, 8, 10]]
PART_TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}


def plain_latent(x, W, layer, eps, kept=None):
    m = layer["mixer"]
    return pg.latent_attention(x, W, "m.", m, eps, kept=kept, gated=pg.kind_of(layer["type"]) == "latent_attention",
                               window=int(m["mask"]["size"]) if "mask" in m else 0)


# ---- latent attention
LATENTS = [pg.latent_layer(heads=3, dim=24, rot_dim=8, vdim=40, q_rank=20, kv_rank=36, scale=0.2, base=500.0),
           pg.latent_layer(heads=1, dim=16, rot_dim=2, vdim=16, q_rank=8, kv_rank=8, scale=0.25, base=20.0, window=1),
           pg.latent_layer(heads=2, dim=40, rot_dim=16, vdim=24, q_rank=48, kv_rank=20, scale=0.15, window=24),
           pg.latent_layer(heads=4, dim=32, rot_dim=16, vdim=48, q_rank=48, kv_rank=48, scale=0.17),               # rows of 64
           pg.latent_layer(heads=8, dim=64, rot_dim=32, vdim=48, q_rank=72, kv_rank=96, scale=0.125, window=33),   # rows of 128
           pg.latent_layer(heads=2, dim=4, rot_dim=48, vdim=8, q_rank=16, kv_rank=16, scale=0.3, base=100.0),      # the turned part weighs most
           pg.latent_layer(heads=5, dim=8, rot_dim=4, vdim=72, q_rank=4, kv_rank=260, scale=0.3, window=500),
           pg.latent_layer(heads=4, dim=64, rot_dim=64, vdim=64, q_rank=64, kv_rank=192, scale=0.09),              # rows of 256
           pg.latent_layer(heads=3, dim=32, rot_dim=32, vdim=40, q_rank=32, kv_rank=224, scale=0.12, window=70)]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", LATENTS)
def test_latent_attention_alone(dtype, layer, fast):
    """Two requests on scattered pages, portions beside single rows; with and without the gate and the window."""
    width, eps = 80, 1e-5
    W = pg.mixer_weights(layer, width, 41)
    parts, cache, ctx = mixers_setup([layer], width, [W], dtype, fast, eps=eps)
    xs = inputs(width, [66, 51], 42)
    got = run_cut(parts, cache, xs, CUTS, dtype, PAGES, ctx)[0]
    for i, x in enumerate(xs):
        close(got[i], plain_latent(x, W, layer, eps), PART_TOL[dtype], f"request {i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [[300, 101]])
@pytest.mark.parametrize("layer", [LATENTS[3], LATENTS[4], LATENTS[0], LATENTS[7], LATENTS[8]])
def test_latent_attention_steps_of_many_rows(dtype, layer, rows):
    """Steps of hundreds of rows, alone and beside single rows: a bfloat16 run makes the per-head products of such
    steps another way (head by head on the tensor cores where the sizes allow) than those of a few rows."""
    width, eps = 96, 1e-5
    W = pg.mixer_weights(layer, width, 45)
    parts, cache, ctx = mixers_setup([layer], width, [W], dtype, pages=40, eps=eps)
    xs = inputs(width, rows, 46)
    tables = [[(7 * p + 2) % 19 for p in range(19)], list(range(19, 26))]
    cuts = [[(0, 200), None], [(200, 201), (0, 100)], [(201, 300), (100, 101)]]
    got = run_cut(parts, cache, xs, cuts, dtype, tables, ctx)[0]
    for i, x in enumerate(xs):
        close(got[i], plain_latent(x, W, layer, eps), PART_TOL[dtype], f"request {i}")


@pytest.mark.parametrize("kv_rank,rot_dim,window", [(8, 8, 0), (24, 8, 5), (32, 16, 0), (64, 16, 30), (64, 32, 0), (96, 16, 40),
                                                    (128, 32, 96), (160, 32, 0), (128, 64, 50), (192, 32, 0), (224, 16, 33),
                                                    (200, 56, 0), (320, 64, 20), (500, 76, 0)])
def test_cached_rows_of_many_sizes(kv_rank, rot_dim, window):
    """A bfloat16 run picks its attention kernels by the size of the cached row (tcgen05, mma.sync or the general one
    for portions; tensor-core, lane-per-chunk or the general one for single rows): every multiple of sixteen up to
    256 in turn, and rows beyond, in portions beside single rows."""
    width, eps = 64, 1e-5
    layer = pg.latent_layer(heads=3, dim=24, rot_dim=rot_dim, vdim=32, q_rank=16, kv_rank=kv_rank, scale=0.2, window=window)
    W = pg.mixer_weights(layer, width, 61)
    parts, cache, ctx = mixers_setup([layer], width, [W], torch.bfloat16, eps=eps)
    xs = inputs(width, [66, 51], 62)
    got = run_cut(parts, cache, xs, CUTS, torch.bfloat16, PAGES, ctx)[0]
    for i, x in enumerate(xs):
        close(got[i], plain_latent(x, W, layer, eps), PART_TOL[torch.bfloat16], f"request {i}")


@pytest.mark.parametrize("dim,vdim,heads,kv_heads", [(16, 16, 4, 2), (48, 32, 2, 2), (64, 128, 4, 1), (80, 80, 3, 1), (96, 64, 6, 3),
                                                     (128, 64, 8, 2), (192, 192, 2, 1), (256, 256, 2, 2), (256, 128, 4, 2)])
def test_attention_heads_of_many_sizes(dim, vdim, heads, kv_heads):
    """The same for the attention with sink and cap: a bfloat16 run pads keys and values to one head size and picks
    its kernels by it."""
    width, eps = 64, 1e-5
    layer = pg.sink_layer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot_dims=dim // 2, base=1e4, scale=2.0 / dim,
                          softcap=6.0, scaling=YARN)
    W = pg.mixer_weights(layer, width, 63)
    parts, cache, ctx = mixers_setup([layer], width, [W], torch.bfloat16, eps=eps)
    xs = inputs(width, [66, 51], 64)
    got = run_cut(parts, cache, xs, CUTS, torch.bfloat16, PAGES, ctx)[0]
    for i, x in enumerate(xs):
        close(got[i], pg.sink_attention(x, W, "m.", layer["mixer"], eps), PART_TOL[torch.bfloat16], f"request {i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("own,w1,w2", [(24, 40, 9), (0, 30, 1), (17, 17, 64)])
def test_latents_of_another_layer(dtype, own, w1, w2):
    """Two layers read what a third keeps, each with its own up-projections, queries and window (longer and shorter
    than the owner's, and an owner that sees everything); the pages stay for the longest window."""
    width, eps = 80, 1e-5
    owner = pg.latent_layer(heads=2, dim=24, rot_dim=16, vdim=24, q_rank=16, kv_rank=32, scale=0.2, window=own)
    r1 = pg.latent_layer(heads=3, dim=16, rot_dim=16, vdim=40, q_rank=24, kv_rank=32, scale=0.25, window=w1, kv_from=0)
    r2 = pg.latent_layer(heads=4, dim=32, rot_dim=16, vdim=16, q_rank=8, kv_rank=32, scale=0.15, window=w2, kv_from=0)
    layers = [owner, r1, r2]
    Ws = [pg.mixer_weights(L, width, 50 + k) for k, L in enumerate(layers)]
    parts, cache, ctx = mixers_setup(layers, width, Ws, dtype, eps=eps)
    assert cache.windows == [0 if own == 0 else max(own, w1, w2)]
    xs = inputs(width, [66, 51], 52)
    got = run_cut(parts, cache, xs, CUTS, dtype, PAGES, ctx)
    for i, x in enumerate(xs):
        kept = pg.latent_kv(x, Ws[0], "m.", owner["mixer"], eps, torch.arange(x.shape[0]))
        for k, L in enumerate(layers):
            close(got[k][i], plain_latent(x, Ws[k], L, eps, kept=kept), PART_TOL[dtype], f"layer {k} request {i}")


def standout_case(window, T, i, j, width=64, rot_dim=8):
    """Weights and inputs for which row i's weight falls on key j, if it sees it: queries and keys go through the
    same maps but for a shift of the input's columns, and row j's input is row i's shifted, so that the query latent
    of row i is the key latent of row j and their score is a squared length; the turned parts are switched off in the
    queries; row i's own key is as any other."""
    layer = pg.latent_layer(heads=2, dim=32, rot_dim=rot_dim, vdim=32, q_rank=32, kv_rank=32, scale=1.0, window=window)
    W = pg.mixer_weights(layer, width, 43)
    W["m.dq"], W["m.dq.norm"] = torch.roll(W["m.dkv"][:32], -1, dims=1), W["m.dkv.norm"]
    uq = torch.zeros_like(W["m.uq"]).view(2, 32 + rot_dim, 32)
    uq[:, :32] = W["m.uk"].view(2, 32, 32)
    W["m.uq"] = uq.reshape(-1, 32)
    g = torch.Generator().manual_seed(44)
    x = torch.randn(T, width, generator=g, dtype=F64)
    x[j] = torch.roll(x[i], 1)
    return layer, W, x.to(torch.bfloat16).double(), g


EDGES = [(24, 50, 27), (24, 50, 26),            # the window's edge
         (16, 47, 32), (16, 47, 31),            # the same at a page border
         (33, 100, 68), (33, 100, 67),
         (400, 430, 31), (400, 430, 30),        # a far key through a long window
         (0, 590, 3), (0, 590, 0),              # hundreds of positions back without a window
         (0, 320, 16), (0, 320, 15),
         (1, 40, 40), (2, 40, 39), (2, 40, 38)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window,i,j", EDGES)
def test_one_latent_key_stands_out(window, i, j, decoded, dtype):
    """A key just inside the window takes row i's weight, the next one outside takes none; in a prompt, and when
    row i is decoded alone after single rows."""
    T = i + 3
    layer, W, x, g = standout_case(window, T, i, j)
    parts, cache, ctx = mixers_setup([layer], 64, [W], dtype, eps=1e-6)
    table = [(5 * p + 3) % 47 for p in range((T + 15) // 16)]
    assert len(set(table)) == len(table)
    cuts = [[(0, T)]] if not decoded else [[(0, i - 2)]] + [[(t, t + 1)] for t in range(i - 2, T)]
    got = run_cut(parts, cache, [x], cuts, dtype, [table], ctx)[0][0]
    want = plain_latent(x, W, layer, 1e-6)
    close(got, want, PART_TOL[dtype], "rows")
    # the case shows what it is meant to show: a window that differs in key j alone moves row i by far more
    seen = window == 0 or i - j < window
    m = dict(layer["mixer"])
    m["mask"] = {"size": i - j if seen else i - j + 1}
    if seen and i == j:
        return
    other = pg.latent_attention(x, W, "m.", m, 1e-6, gated=window == 0, window=m["mask"]["size"])
    assert float((other[i] - want[i]).abs().max()) > 0.1 * float(want.abs().max())


# ---- attention with capped scores and a sink
SINKS = [pg.sink_layer(heads=4, kv_heads=2, dim=32, vdim=48, rot_dims=16, base=300.0, scale=0.3, softcap=5.0, scaling=YARN),
         pg.sink_layer(heads=3, kv_heads=3, dim=48, vdim=16, rot_dims=48, base=1e4, scale=0.11, softcap=30.0),
         pg.sink_layer(heads=1, kv_heads=1, dim=40, vdim=20, rot_dims=2, base=100.0, scale=0.3, softcap=1.0),
         pg.sink_layer(heads=6, kv_heads=2, dim=64, vdim=64, rot_dims=64, base=1e6, scale=0.125, softcap=20.0,
                       scaling={"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}),
         pg.sink_layer(heads=2, kv_heads=1, dim=128, vdim=128, rot_dims=32, base=1e4, scale=0.09, softcap=50.0),
         pg.sink_layer(heads=20, kv_heads=1, dim=16, vdim=32, rot_dims=0, base=10.0, scale=0.25, softcap=8.0)]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", SINKS)
def test_sink_attention_alone(dtype, layer, fast):
    width, eps = 80, 1e-5
    W = pg.mixer_weights(layer, width, 31)
    parts, cache, ctx = mixers_setup([layer], width, [W], dtype, fast, eps=eps)
    xs = inputs(width, [66, 51], 32)
    got = run_cut(parts, cache, xs, CUTS, dtype, PAGES, ctx)[0]
    for i, x in enumerate(xs):
        close(got[i], pg.sink_attention(x, W, "m.", layer["mixer"], eps), PART_TOL[dtype], f"request {i}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("what", ["sink", "cap", "norm_after_turn"])
def test_what_the_attention_adds_shows(dtype, what):
    """Cases in which leaving one mechanism out moves the output by far more than the tolerance: a scale so small
    that every score is near zero and the sink takes 1 / (n + 1) of the weight; a scale so large that the cap
    flattens the scores; an amplitude of the turned part well above one, which the norm after the turn takes back
    in part."""
    width, eps = 64, 1e-5
    if what == "sink":
        layer = pg.sink_layer(heads=2, kv_heads=1, dim=32, vdim=32, rot_dims=16, base=100.0, scale=1e-3, softcap=10.0)
    elif what == "cap":
        layer = pg.sink_layer(heads=2, kv_heads=1, dim=32, vdim=32, rot_dims=16, base=100.0, scale=3.0, softcap=2.0)
    else:
        layer = pg.sink_layer(heads=2, kv_heads=2, dim=32, vdim=32, rot_dims=16, base=100.0, scale=0.5, softcap=30.0,
                              scaling={"factor": 1000.0, "original": 16, "fast": 4.0, "slow": 1.0})
    W = pg.mixer_weights(layer, width, 35)
    parts, cache, ctx = mixers_setup([layer], width, [W], dtype, eps=eps)
    x = inputs(width, [40], 36)[0]
    cuts = [[(0, 30)]] + [[(t, t + 1)] for t in range(30, 40)]
    got = run_cut(parts, cache, [x], cuts, dtype, [[4, 9, 1]], ctx)[0][0]
    m = layer["mixer"]
    want = pg.sink_attention(x, W, "m.", m, eps)
    close(got, want, PART_TOL[dtype], what)
    T, H, G, D, Dv = 40, m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (x @ W["m.q"].T + W["m.q.b"]).view(T, H, D)
    k = (x @ W["m.k"].T + W["m.k.b"]).view(T, G, D)
    v = (x @ W["m.v"].T + W["m.v.b"]).view(T, G, Dv).repeat_interleave(H // G, dim=1)
    if what == "norm_after_turn":       # the norm before the turn instead
        q, k = pg.rotate_pairs(pg.rms(q, eps), pos, m["rot"]), pg.rotate_pairs(pg.rms(k, eps), pos, m["rot"])
    else:
        q, k = pg.rms(pg.rotate_pairs(q, pos, m["rot"]), eps), pg.rms(pg.rotate_pairs(k, pos, m["rot"]), eps)
    o = pg.attend(q, k.repeat_interleave(H // G, dim=1), v, pos, m["scale"], softcap=0.0 if what == "cap" else m["softcap"],
                  plus_one=what != "sink")
    other = o.reshape(T, H * Dv) @ W["m.o"].T + W["m.o.b"]
    assert float((other - want).abs().max()) > (0.05 if what == "norm_after_turn" else 0.1) * float(want.abs().max())


# ---- the feed-forwards
@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff,limit", [(64, 48, 1.0), (96, 120, 0.25), (256, 320, 7.0), (80, 8, 2.0)])
def test_clamped_glu_alone(dtype, width, ff, limit, fast):
    """Inputs large enough that all three clamps bite (and one limit that none reaches); one row, a handful, hundreds."""
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    cfg = pg.model_config([pg.latent_layer(1, 8, 2, 8, 4, 4, 0.3, mlp=pg.dense_ff(ff, limit))], width, 8)
    W = {k.replace("l0.mlp.", "m."): v for k, v in pg.random_weights(cfg, 45).items() if k.startswith("l0.mlp.")}
    part = build_part("feed_forward", PartSpec("dense_swiglu", dict(hidden_size=width, intermediate_size=ff,
                                                                    clamp_limit=limit, slope=1.702,
                                                                    names={"gate": "gate", "up": "up", "down": "down"})))
    part.load(Fetch(W, "m.", dtype), ctx_for(dtype, fast))
    for T in (1, 5, 70, 300):
        x = 2.0 * inputs(width, [T], 46 + T)[0]
        h32 = x.float().to(DEV)
        y = part.forward(h32.to(dtype), h32, None)
        want = pg.clamped_glu(x, W, "m.", limit)
        close(y, want, PART_TOL[dtype], f"T={T}")
        if limit < 5:
            free = (torch.nn.functional.silu(1.702 * (x @ W["m.gate"].T)) / 1.702 * (x @ W["m.up"].T + 1.0)) @ W["m.down"].T
            assert float((free - want).abs().max()) > 0.1 * float(want.abs().max())


MIXTURES = [(64, pg.moe_ff(5, 2, 24, 40)), (96, pg.moe_ff(8, 8, 16)), (64, pg.moe_ff(1, 1, 32, 8)),
            (80, pg.moe_ff(6, 3, 40)), (128, pg.moe_ff(8, 2, 64, 128)), (128, pg.moe_ff(16, 4, 128, 64))]


@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,mlp", MIXTURES)
def test_expert_mixture_alone(dtype, width, mlp, fast):
    """Squared-relu experts, the chosen scores renormed, a shared expert scaled by one sigmoid per token; all experts
    chosen, a single expert, a shared expert of a whole number of expert widths and of another width."""
    from nano_vllm_cpp_b200.config import get_architecture
    from nano_vllm_cpp_b200.parts import build_part
    arch = get_architecture("Gekitar")
    cfg = pg.model_config([pg.latent_layer(1, 8, 2, 8, 4, 4, 0.3, mlp=mlp)], width, 8)
    part = build_part("feed_forward", arch.build_model(arch.config_from_dict(cfg)).layers[0].feed_forward)
    W = {k.replace("l0.mlp.", "m."): v for k, v in pg.random_weights(cfg, 47).items() if k.startswith("l0.mlp.")}
    part.load(Fetch(W, "m.", dtype), ctx_for(dtype, fast))
    for T in (1, 5, 70, 300):
        x = inputs(width, [T], 48 + T)[0]
        h32 = x.float().to(DEV)
        from nano_vllm_cpp_b200.parts.base import RowMix
        y = part.forward(h32.to(dtype), h32, None)
        y = y.sum() if isinstance(y, RowMix) else y
        margins = []
        want = pg.expert_mixture(x, W, "m.", mlp, margins)
        got, want = y.double().cpu(), want
        err = (got - want).abs().max(dim=1).values
        bad = err > PART_TOL[dtype] * float(want.abs().max())
        if dtype == torch.bfloat16:
            bad &= margins[0] >= EDGE
        assert not bool(bad.any()), f"T={T}: {int(bad.sum())} rows, first {int(torch.nonzero(bad)[0])}, error {float(err[bad].max()):.3g}"


def test_the_routing_weights():
    """The chosen experts' softmax scores divided by their sum, in order of falling score, ties to the lower index."""
    from nano_vllm_cpp_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(50, 7, generator=g) * 2
    logits[3] = 0.0                     # all equal: experts 0, 1, 2
    logits[4, 5] = logits[4, 2] = 9.0   # a tie at the top
    idx = torch.empty((50, 3), dtype=torch.int32, device=DEV)
    w = torch.empty((50, 3), dtype=torch.float32, device=DEV)
    ops.router_topk(logits.to(DEV), 3, True, idx, w)
    s = torch.softmax(logits.double(), dim=-1)
    order = torch.argsort(s, dim=-1, descending=True, stable=True)[:, :3]
    assert idx.cpu().tolist() == order.tolist()
    ws = torch.gather(s, 1, order)
    assert float((w.cpu().double() - ws / ws.sum(-1, keepdim=True)).abs().max()) < 1e-6


# ---- the layer
def test_a_layer_norms_what_goes_in_and_what_comes_out():
    """The stream after every layer of a model (a layer's last output waits for the next norm's kernel, which norms
    it, adds it and norms the sum for its own sublayer), and the two-norm kernel alone with a plain branch and with
    a mixture's rows."""
    from nano_vllm_cpp_b200.engine.batch import StepEntry
    from nano_vllm_cpp_b200.parts.base import NormedBranch
    from nano_vllm_cpp_b200.csrc import ops
    import tempfile
    name = "P"
    cfg = CONFIGS[name]
    W = pg.random_weights(cfg, SEEDS[name])
    with tempfile.TemporaryDirectory() as d:
        runner = make_runner(pg.write_folder(cfg, W, d), "float32", 128)
        seen = []

        def look(k, x, pending):
            assert isinstance(pending, NormedBranch)
            y = x.detach().clone()
            pending.add_to(y)
            seen.append(y.cpu())

        runner.model.after_call = look
        ids = ids_for(name, 40, salt=50)
        runner.step([StepEntry("s", ids, [])])
        runner.model.after_call = None
    want = []
    pg.forward(cfg, W, ids, layers_out=want)
    assert len(seen) == len(want) == len(cfg["layers"])
    for k, (a, b) in enumerate(zip(seen, want)):
        close(a, b, 1e-4, f"the stream after layer {k}")
    g = torch.Generator().manual_seed(9)
    for T, H in ((1, 96), (7, 130), (300, 64)):
        x, y = torch.randn(T, H, generator=g, dtype=F64), 3.0 * torch.randn(T, H, generator=g, dtype=F64)
        w1, w2 = 1 + 0.2 * torch.randn(H, generator=g, dtype=F64), 1 + 0.2 * torch.randn(H, generator=g, dtype=F64)
        rows = torch.randn(2 * T, H, generator=g, dtype=F64)
        index = torch.randint(0, 2 * T, (T, 3), generator=g)
        weight = torch.rand(T, 3, generator=g, dtype=F64)
        dense, gate = torch.randn(T, H, generator=g, dtype=F64), torch.randn(T, 1, generator=g, dtype=F64)
        for mixed in (False, True):
            branch = (torch.sigmoid(gate) * dense + (weight[:, :, None] * rows[index]).sum(1)) if mixed else y
            xn = x + pg.rms(branch, 1e-5) * w1
            xd = x.float().to(DEV)
            out = torch.empty((T, H), dtype=torch.float32, device=DEV)
            f = lambda t: t.float().to(DEV)     # noqa: E731
            mix = (f(rows), index.int().to(DEV), f(weight), f(dense), f(gate)) if mixed else None
            ops.branch_norm_add(xd, [] if mixed else [f(y)], f(w1), 1e-5, out, mix=mix, next_weight=f(w2), next_eps=1e-6)
            close(xd, xn, 1e-5, "the stream")
            close(out, pg.rms(xn, 1e-6) * w2, 1e-5, "the next sublayer's input")
            # the kernel that the layers run: the norm of the stream with the branch's own norm in front
            for dt in (torch.float32, torch.bfloat16):
                xd, out, out32 = f(x), torch.empty((T, H), dtype=dt, device=DEV), torch.empty((T, H), dtype=torch.float32, device=DEV)
                ops.add_rmsnorm(xd, None if mixed else f(y), f(w2), 1e-6, out, out32, mix=mix, branch_weight=f(w1), branch_eps=1e-5)
                close(xd, xn, 1e-5, "the stream")
                close(out32, pg.rms(xn, 1e-6) * w2, 1e-5, "the next sublayer's input")
                close(out, pg.rms(xn, 1e-6) * w2, 1e-5 if dt == torch.float32 else 1e-2, "the next sublayer's input as stored")


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
    """A short prompt in one step, then ninety rows one at a time (the windows pass over decoded tokens and pages
    behind the longest window of a group go back; steps of the same shape are replayed from a captured graph), and
    a sequence that is decoded from its first token on."""
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
@pytest.mark.parametrize("name", ["P", "R"])
def test_steps_of_one_shape_are_replayed(name, dtype, models):
    """Five requests in turn, each as a portion of 100 tokens and a portion of 30 beside a single row of the request
    before: from its second occurrence on a shape runs as a captured graph, the per-head products of many rows and the
    mixtures' permutation buffers among its kernels."""
    runner = make_runner(models[name][2], dtype, 512)
    st = Steps(runner)
    all_ids = [ids_for(name, 131, salt=40 + k) for k in range(5)]
    for k, ids in enumerate(all_ids):
        st.step([(f"g{k}", ids[:100])])
        parts = [(f"g{k}", ids[100:130])]
        if k:
            parts.append((f"g{k - 1}", all_ids[k - 1][130:131]))
        st.step(parts, end=[f"g{k - 1}"] if k else [])
    st.step([("g4", all_ids[4][130:131])], end=["g4"])
    for k, ids in enumerate(all_ids):
        check_rows(st, models, name, f"g{k}", ids, dtype, f"{name} request {k}")


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
    rows of others; a finished request's pages go to the next one.  Every request's logits equal those of the
    request alone."""
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
    """A model of four to nine layers whose kinds, order and sizes are drawn: every mixer kind at least once, up to two
    sets of sizes per kind, windowed latent layers that read an earlier latent layer's pages where one with the same
    latent fits, every feed-forward kind and layers without one, sizes that do and do not fit the tensor-core
    kernels."""
    width = rng.choice([128, 192, 256, 320])
    n = rng.randint(4, 9)
    kinds = [rng.choice(["latent", "window", "attn"]) for _ in range(n)]
    for must in ("latent", "window", "attn"):
        if must not in kinds:
            kinds[rng.randrange(n)] = must

    def latent():
        return dict(heads=rng.choice([2, 4, 6, 8, 12]), dim=rng.choice([16, 32, 48, 64]), vdim=rng.choice([32, 48, 64, 80]),
                    q_rank=rng.choice([48, 64, 96]), scale=rng.choice([0.125, 0.1, 0.18]))

    def kept():       # what two layers must share to share pages
        return dict(kv_rank=rng.choice([48, 64, 96, 112, 160, 192]), rot_dim=rng.choice([16, 32, 64]),
                    base=rng.choice([1e4, 2e4, 2.5e5]))

    def attn():
        kv, dim = rng.choice([1, 2, 3, 4]), rng.choice([32, 64, 96, 128])
        return dict(heads=kv * rng.choice([1, 2, 3, 4]), kv_heads=kv, dim=dim, vdim=rng.choice([32, 64, 96, 128]),
                    rot_dims=rng.choice([16, 32, dim]), base=rng.choice([1e4, 1e6, 100.0]), scale=rng.choice([0.125, 0.09, 0.2]),
                    softcap=rng.choice([10.0, 20.0, 50.0]),
                    scaling=rng.choice([None, {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}, YARN]))

    def mlp():
        k = rng.choice(["dense", "moe", "moe", "none"])
        if k == "dense":
            return pg.dense_ff(rng.choice([128, 256, 320]), rng.choice([1.0, 1.5, 7.0]))
        if k == "moe":
            e = rng.choice([4, 8, 12])
            return pg.moe_ff(e, rng.choice([1, 2, 3, e]), rng.choice([32, 64, 96]), rng.choice([0, 64, 96, 128]))
        return None

    latents, keeps, attns = [latent(), latent()], [kept(), kept()], [attn(), attn()]
    layers, owners = [], {}                 # owners: which layer first made the latents of kept set k
    for at, k in enumerate(kinds):
        i = rng.randrange(2)
        if k == "attn":
            layers.append(pg.sink_layer(mlp=mlp(), kind="attention" if i == 0 else "attention_2", **attns[i]))
            continue
        j = rng.randrange(2)
        window = rng.choice([17, 40, 64, 96, 150]) if k == "window" else 0
        src = owners.get(j) if (k == "window" and rng.random() < 0.6) else None
        if src is None:
            owners.setdefault(j, at)
        kind = ("latent_attention_2" if k == "window" else "latent_attention") + ("" if i == 0 else "_3")
        layers.append(pg.latent_layer(window=window, kv_from=src, mlp=mlp(), kind=kind, **latents[i], **keeps[j]))
    return pg.model_config(layers, width=width, vocab=rng.choice([300, 512, 1000]), eps=rng.choice([1e-6, 1e-5]),
                           embed_scale=rng.choice([None, 4.0, 16.0]))


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5])
def test_drawn_models_in_a_mixed_schedule(seed, tmp_path):
    """Drawn models, both dtypes: five unequal requests on three slots and 576 tokens of pages, portions of up to 150
    tokens beside single rows of others, decoding over dozens of steps, finished requests' pages and slots used
    again; every request's logits equal the plain implementation's of the request alone."""
    import random
    cfg = drawn_config(random.Random(seed))
    W = pg.random_weights(cfg, seed)
    one = {"F": (cfg, W, pg.write_folder(cfg, W, str(tmp_path)))}
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
            want, margins = plain_logits(one, "F", ids[r])
            # (a drawn router may put many rows near an edge: what is held is every row before the first of them)
            got = st.rows(r, n)
            upto = n
            if dtype == "bfloat16" and bool((margins < EDGE).any()):
                upto = int(torch.nonzero(margins < EDGE)[0])
            if upto:
                close(got[:upto], want[:upto], TOL[dtype], f"seed {seed} {dtype} request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_a_row(dtype, models):
    """The same request whole, in portions, and token by token after a prompt, beside another request: the rows agree
    with one another far more closely than with the plain implementation (float32), or within rounding (bfloat16,
    up to the first row on a router's edge)."""
    name = "P"
    folder = models[name][2]
    ids, other = ids_for(name, 70, salt=9), ids_for(name, 40, salt=10)
    _, margins = plain_logits(models, name, ids)
    runs = []
    for cut in ([70], [3, 2, 30, 1, 34], [40] + [1] * 30):
        st = Steps(make_runner(folder, dtype, 256))
        at = 0
        for k, n in enumerate(cut):
            parts = [("x", ids[at:at + n])]
            if k < 4:
                parts.append(("y", other[10 * k:10 * k + 10]))
            st.step(parts)
            at += n
        runs.append(st.rows("x", 70))
    for r in runs[1:]:
        close(r, runs[0], 2e-5 if dtype == "float32" else 3e-2, "the same rows cut another way",
              margins if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype, models):
    """The engine's own entry point, scheduler and sampling: greedy tokens follow the plain implementation's up
    to the first position where its two best logits are closer than the tolerance."""
    from nano_vllm_cpp_b200 import LLMEngine, SamplingParams
    name = "P"
    cfg, W, folder = models[name]
    prompts = [ids_for(name, 9, salt=20), ids_for(name, 3, salt=21), ids_for(name, 30, salt=22)]
    eng = LLMEngine(folder, max_model_len=96, num_kv_blocks=24, dtype=dtype, max_num_seqs=2, log_stats=False)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        seq = list(p)
        assert len(o["token_ids"]) == 12
        for k, tok in enumerate(o["token_ids"]):
            logits = pg.forward(cfg, W, seq)[-1]
            best = int(torch.argmax(logits))
            if best != tok:
                lead = float(logits[best] - logits[tok])
                bound = 2 * TOL[dtype] * float(logits.abs().max())
                if dtype == "float32":
                    assert lead <= bound, f"token {k} of a prompt of {len(p)}: {tok}, plain takes {best} with a lead of {lead:.3g}"
                break
            seq.append(tok)


def test_command_line_serves_the_design(models, tmp_path, capsys):
    """``nanovllm <folder> --tokens ...`` and ``nanovllm --config <json>`` (random weights) run this design as they
    run the others; the greedy tokens from the folder are the plain implementation's."""
    from nano_vllm_cpp_b200 import cli
    name = "Q"
    cfg, W, folder = models[name]
    prompt = ids_for(name, 7, salt=30)
    rc = cli.main([folder, "--tokens", ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                   "--dtype", "float32", "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0, out
    toks = [int(t) for t in out.strip().splitlines()[-1].split(":")[1].split()]
    assert toks == pg.greedy_generate(cfg, W, prompt, 6)
    path = tmp_path / "config.json"
    path.write_text(json.dumps(CONFIGS["P"]))
    rc = cli.main(["--config", str(path), "--seed", "4", "--tokens", "5,6,7", "--max-tokens", "4", "--temperature", "0",
                   "--max-model-len", "64", "--num-kv-blocks", "8", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0 and len(out.strip().splitlines()[-1].split(":")[1].split()) == 4
