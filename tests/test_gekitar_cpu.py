"""Gekitar without a GPU: its configuration and errors, the model as data (tensor names against the plain
implementation's table, what every layer keeps per request, page groups, layers that read another's pages), and the
turned pairs' frequencies."""
import copy

import pytest

import plain_gekitar as pg
from nano_vllm_cpp_b200.config import ConfigError, get_architecture
from nano_vllm_cpp_b200.parts import Model

YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
CFG = pg.model_config(
    [pg.latent_layer(heads=3, dim=24, rot_dim=8, vdim=40, q_rank=20, kv_rank=36, scale=0.2, base=500.0,
                     mlp=pg.dense_ff(120, 1.0)),
     pg.latent_layer(heads=2, dim=40, rot_dim=16, vdim=24, q_rank=48, kv_rank=20, scale=0.15, window=24,
                     mlp=pg.moe_ff(5, 2, 24, 40)),
     pg.sink_layer(heads=4, kv_heads=2, dim=32, vdim=48, rot_dims=16, base=300.0, scale=0.3, softcap=5.0, scaling=YARN,
                   mlp=pg.moe_ff(6, 3, 32)),
     pg.latent_layer(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=12, kv_rank=20, scale=0.25, window=40, kv_from=1),
     pg.latent_layer(heads=2, dim=24, rot_dim=16, vdim=32, q_rank=16, kv_rank=20, scale=0.2, window=9, kv_from=1,
                     mlp=pg.dense_ff(48, 0.5), kind="latent_attention_2_2"),
     pg.latent_layer(heads=1, dim=8, rot_dim=8, vdim=8, q_rank=8, kv_rank=36, scale=0.2, base=500.0, window=7, kv_from=0)],
    width=96, vocab=210, eps=1e-5, embed_scale=4.0)


def build(cfg):
    arch = get_architecture("Gekitar")
    typed = arch.config_from_dict(cfg)
    return typed, Model(arch.build_model(typed))


def test_tensor_names_and_shapes_are_the_plain_table():
    _, model = build(CFG)
    table = pg.tensor_shapes(CFG)
    specs = model.tensor_specs()
    assert set(specs) == set(table)
    for name, (shape, _) in table.items():
        assert tuple(specs[name].shape) == tuple(shape), name
    # a layer that reads another's latents has no down-projection to them; only the first kind has a gate
    assert "l3.mix.dkv" not in specs and "l3.mix.dkv.norm" not in specs and "l1.mix.dkv" in specs
    assert "l0.mix.g" in specs and "l1.mix.g" not in specs
    assert tuple(specs["l0.mix.g"].shape) == (3 * 40, 96)


def test_what_every_layer_keeps_per_request():
    typed, model = build(CFG)
    assert typed.num_hidden_layers == 6 and typed.embed_scale == 4.0 and typed.eps == 1e-5
    l0, l1, att, r1, r2, r0 = model.cache_specs()
    # a latent layer keeps one row per token, the latent and behind it the turned key part, and no values; its
    # pages stay for the longest window of the layers that read them (every page if one of them sees everything)
    assert (l0.num_kv_heads, l0.head_dim, l0.window, l0.values) == (1, 36 + 8, 0, False)
    assert (l1.num_kv_heads, l1.head_dim, l1.window, l1.values) == (1, 20 + 16, 40, False)
    assert (att.num_kv_heads, att.head_dim, att.window, att.v_head_dim) == (2, 32, 0, 48)
    assert r1 == ("shared", 1) and r2 == ("shared", 1) and r0 == ("shared", 0)
    assert model.layers[3].feed_forward is None and model.layers[0].feed_forward is not None
    assert [c.cache_of for c in model.calls] == [None, None, None, 1, 1, 0]
    # the readers attend through their own windows
    assert [model.layers[i].mixer.window for i in (1, 3, 4, 5)] == [24, 40, 9, 7]


def test_page_groups():
    from nano_vllm_cpp_b200.cache import DeviceCache
    _, model = build(CFG)
    cache = DeviceCache(model.cache_specs(), 16, 2, "cpu", None)
    assert cache.windows == [0, 40]


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "mixer", "heads"), 0, "heads"),
    (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 0, "mixer", "rot", "dims"), 6, "rot.dims"),
    (("layers", 1, "mixer", "mask"), None, "mask"),
    (("layers", 2, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 2, "mixer", "rot", "scaling", "factor"), None, "factor"),
    (("layers", 2, "mixer", "softcap"), -1.0, "softcap"),
    (("layers", 3, "mixer", "kv_from"), 2, "kv_from"),
    (("layers", 3, "mixer", "kv_from"), 4, "kv_from"),
    (("layers", 4, "mixer", "kv_rank"), 24, "kv_from"),
    (("layers", 0, "mlp", "limit"), None, "limit"),
    (("layers", 1, "mlp", "router", "top"), 6, "top"),
    (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("layers", 2, "type"), "attention_x", "type"),
    (("norm",), None, "norm"),
    (("width",), 0, "width"),
])
def test_errors_name_the_key(path, value, word):
    d = copy.deepcopy(CFG)
    at = d
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        get_architecture("Gekitar").config_from_dict(d)
    assert word in str(e.value)


def test_a_reader_of_a_reader_is_refused():
    d = copy.deepcopy(CFG)
    d["layers"][4]["mixer"]["kv_from"] = 3
    with pytest.raises(ConfigError):
        get_architecture("Gekitar").config_from_dict(d)


def test_frequencies_of_the_turned_pairs():
    from nano_vllm_cpp_b200.parts.rotary import RotaryInterleaved
    for rot in ({"dims": 16, "base": 300.0, "scaling": YARN}, {"dims": 48, "base": 1e4},
                {"dims": 64, "base": 1e6, "scaling": {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}}):
        part = RotaryInterleaved(rot["dims"], rot["base"], rot.get("scaling"))
        f, amp = pg.pair_frequencies(rot)
        assert max(abs(a - float(b)) for a, b in zip(part.frequencies(), f)) < 1e-15
        assert abs(part.amplitude - amp) < 1e-15
