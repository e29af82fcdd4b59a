"""Sanesun without a GPU: its configuration and errors, the model as data (tensor names against the plain
implementation's table, what every layer keeps per request, page groups), and parts that a file leaves out."""
import copy

import pytest

import plain_sanesun as ps
from nano_vllm_cpp_b200.config import ConfigError, get_architecture
from nano_vllm_cpp_b200.parts import Model

CFG = ps.model_config(
    [ps.latent_layer(heads=3, dim=24, vdim=40, q_rank=20, kv_rank=36, scale=0.2, ff=120),
     ps.delta_layer(heads=4, kv_heads=2, dim=24, vdim=40, conv=4, ff=72, rank=12),
     ps.attention_layer(heads=4, kv_heads=2, dim=32, vdim=48, window=24, keep_first=3, rot_dims=16, base=500.0,
                        scale=0.2, ff=120),
     ps.attention_layer(heads=3, kv_heads=3, dim=48, vdim=16, window=17, keep_first=5, rot_dims=48, base=10000.0,
                        scale=0.11, ff=0, kind="attention_2"),
     ps.delta_layer(heads=3, kv_heads=3, dim=40, vdim=24, conv=2, ff=0, rank=9, kind="channel_delta_2")],
    width=96, vocab=210, eps=1e-5, embed_scale=4.0)


def build(cfg):
    arch = get_architecture("Sanesun")
    typed = arch.config_from_dict(cfg)
    return typed, Model(arch.build_model(typed))


def test_tensor_names_and_shapes_are_the_plain_table():
    _, model = build(CFG)
    table = ps.tensor_shapes(CFG)
    # the ranks of the two low-rank pairs are the tensors' own: the model is told what the file holds
    specs = model.tensor_specs({name: tuple(shape) for name, (shape, _) in table.items()})
    assert set(specs) == set(table)
    for name, (shape, _) in table.items():
        assert len(specs[name].shape) == len(shape), name
        assert all(a is None or a == b for a, b in zip(specs[name].shape, shape)), name      # None: the file's own
    # random weights take the ranks that the configuration names
    d = copy.deepcopy(CFG)
    d["layers"][1]["mixer"].update(decay_rank=12, gate_rank=13)
    specs = build(d)[1].tensor_specs()
    for name in ("l1.mix.a1", "l1.mix.a2", "l1.mix.g1", "l1.mix.g2"):
        assert tuple(specs[name].shape) == tuple(table[name][0]), name


def test_what_every_layer_keeps_per_request():
    typed, model = build(CFG)
    assert typed.num_hidden_layers == 5 and typed.embed_scale == 4.0 and typed.eps == 1e-5
    specs = model.cache_specs()
    lat, d1, a1, a2, d2 = specs
    # the latent layer keeps one vector of kv_rank elements per token and no values
    assert (lat.num_kv_heads, lat.head_dim, lat.window, lat.values) == (1, 36, 0, False)
    # windows with kept first tokens; value heads of their own size
    assert (a1.num_kv_heads, a1.head_dim, a1.window, a1.v_head_dim, a1.keep_first) == (2, 32, 24, 48, 3)
    assert (a2.num_kv_heads, a2.head_dim, a2.window, a2.v_head_dim, a2.keep_first) == (3, 48, 17, 16, 5)
    # the delta rule keeps a matrix per head and the convolution's last inputs, no pages
    for s, m in ((d1, CFG["layers"][1]["mixer"]), (d2, CFG["layers"][4]["mixer"])):
        channels = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
        assert [tuple(p.shape) for p in s.parts] == [(m["heads"], m["dim"], m["vdim"]), (m["conv"] - 1, channels)]
    # a layer without a feed-forward has none
    assert model.layers[3].feed_forward is None and model.layers[0].feed_forward is not None


def test_configuration_errors_name_the_key():
    def broken(path, value, drop=False):
        d = copy.deepcopy(CFG)
        node = d
        for k in path[:-1]:
            node = node[k]
        if drop:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        return d
    arch = get_architecture("Sanesun")
    for path, value, drop, word in [
            (("layers", 1, "mixer", "heads"), 5, False, "kv_heads"),
            (("layers", 1, "mixer", "conv"), 0, False, "conv"),
            (("layers", 1, "mixer", "dim"), None, True, "dim"),
            (("layers", 2, "mixer", "heads"), 5, False, "kv_heads"),
            (("layers", 2, "mixer", "scale"), None, True, "scale"),
            (("layers", 2, "mixer", "rot", "dims"), 34, False, "rot.dims"),
            (("layers", 2, "mixer", "rot", "dims"), 7, False, "rot.dims"),
            (("layers", 2, "mixer", "rot", "base"), 1.0, False, "rot.base"),
            (("layers", 2, "mixer", "mask", "size"), 0, False, "mask.size"),
            (("layers", 2, "mixer", "mask", "keep_first"), -1, False, "keep_first"),
            (("layers", 0, "mixer", "kv_rank"), None, True, "kv_rank"),
            (("layers", 0, "mixer", "q_rank"), 0, False, "q_rank"),
            (("layers", 0, "mlp", "kind"), "mixture", False, "mlp.kind"),
            (("layers", 0, "mlp", "ff"), 0, False, "mlp.ff"),
            (("layers", 3, "type"), "convolution", False, "type"),
            (("width",), None, True, "width"),
            (("vocab",), 0, False, "vocab"),
            (("norm",), None, True, "norm")]:
        with pytest.raises(ConfigError) as e:
            arch.config_from_dict(broken(path, value, drop))
        assert word in str(e.value), (path, str(e.value))
    with pytest.raises(ConfigError):
        arch.config_from_dict(dict(CFG, layers=[]))


def test_parts_a_file_leaves_out_are_switched_off():
    d = copy.deepcopy(CFG)
    del d["embedding"]
    d["layers"][2]["mixer"]["mask"] = None
    d["layers"][3]["mixer"]["rot"] = None
    d["layers"][2]["mixer"]["rot"]["dims"] = 0
    typed, model = build(d)
    assert typed.embed_scale == 1.0
    a1, a2 = model.layers[2].mixer, model.layers[3].mixer
    assert model.cache_specs()[2].window == 0 and a1.keep_first == 0
    # nothing of q and k turned, the values still are
    assert a1.position.rotary_dim == 0 and a1.value_position is not None and a1.value_position.rotary_dim == 48
    # no rotation at all
    assert a2.position.rotary_dim == 0 and a2.value_position is None


def test_a_numeric_suffix_marks_a_further_set_of_sizes():
    typed, _ = build(CFG)
    assert [L.type for L in typed.layers] == ["latent_attention", "channel_delta", "attention", "attention_2",
                                              "channel_delta_2"]
    assert type(typed.layers[2].mixer) is type(typed.layers[3].mixer)


@pytest.mark.parametrize("keep", [1, 16, 17, 40])
def test_pages_of_kept_positions_stay_with_the_request(keep):
    """A window group gives a page back once the window has passed it, but never a page that holds one of the
    sequence's first ``keep`` positions; pages come back to the pool at the request's end and are used again."""
    from nano_vllm_cpp_b200.cache import CacheManager
    m = CacheManager([(16, keep), 16], [12, 12], 16, max_requests=2)
    m.open("r")
    n = 0
    for step in [5, 30, 1, 1, 40, 1, 2, 64, 1, 1]:
        m.extend("r", n, n + step)
        n += step
        m.commit("r", n)
        kept, plain = m.get("r").tables
        first = (min(keep, n) + 15) // 16              # pages that hold a kept position
        assert all(kept[i] >= 0 for i in range(first)), (n, kept)
        assert all(kept[i] >= 0 for i in range(max(0, n - 15) // 16, len(kept)))
        m.check()
    m.extend("r", n, n + 1)                            # the next row's pages are found: the window's passed pages go back
    kept, plain = m.get("r").tables
    first, lo = (keep + 15) // 16, (n - 15) // 16
    assert [i for i, p in enumerate(kept) if p >= 0] == sorted(set(range(first)) | set(range(lo, len(kept))))
    assert [i for i, p in enumerate(plain) if p >= 0] == list(range(lo, len(plain)))
    m.commit("r", n + 1)
    m.check()
    held = {p for p in m.get("r").tables[0] if p >= 0}
    m.close("r")
    m.open("s")
    m.extend("s", 0, 16 * 12)                          # the whole pool again, the kept pages among it
    assert held <= {p for p in m.get("s").tables[0] if p >= 0}
    m.close("s")
    m.check()
