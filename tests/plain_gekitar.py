"""Plain, slow implementation of the Gekitar decoder: whole sequences, no cache, one function per mechanism,
float64 arithmetic on bfloat16-rounded weight values.  It shares no code with the package: it reads the
configuration as a dict and makes and writes its own weights.

Notation.  ``rms(x) = x / sqrt(mean(x^2) + eps)`` over the last axis; a layer's four norms multiply by ``1 + w``.
A layer norms each sublayer's input *and* output:

    x += rms(mixer(rms(x) (1 + w1))) (1 + w1b);    x += rms(ff(rms(x) (1 + w2))) (1 + w2b)

(a layer may have no feed-forward).  Three mixers:

* ``latent_attention``: keys and values made from one normed vector ``c`` per token plus a small turned key part
  that all heads share; queries through a normed low-rank step; every position before the row's is seen; the heads'
  outputs are gated element by element with a sigmoid of a projection of the mixer's input;
* ``latent_attention_2``: the same through a sliding window, without the gate; it may read another layer's ``c`` and
  turned key part instead of making its own (``kv_from``);
* ``attention``: grouped query heads with biased projections, pairs of neighbours turned by a position whose slow
  frequencies are stretched, q and k heads divided by their root mean square after the turn, capped scores, and a
  softmax whose denominator has one added.

Two feed-forwards: a dense one with clamped gate and up halves, and a mixture of squared-relu experts with a softmax
router, renormed top weights and a shared expert scaled by one sigmoid per token.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ------------------------------------------------------------------------------ small functions
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def kind_of(layer_type):
    """``latent_attention_2`` is a kind of its own; any other numeric suffix marks a further set of sizes."""
    if layer_type.startswith("latent_attention_2"):
        rest = layer_type[len("latent_attention_2"):]
        if rest == "" or (rest[0] == "_" and rest[1:].isdigit()):
            return "latent_attention_2"
    head, _, tail = layer_type.rpartition("_")
    return head if head and tail.isdigit() else layer_type


# ------------------------------------------------------------------------------ rotation of neighbouring pairs
def pair_frequencies(rot):
    """f_i for i < dims / 2, with the slow ones stretched if ``rot`` has a ``scaling``; and the amplitude."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def index_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(index_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
        for i in range(len(f)):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=F64), amp


def rotate_pairs(x, positions, rot):
    """x [T, heads, D]: elements (2i, 2i + 1), i < dims / 2, are turned by ``position * f_i``; the rest pass."""
    dims = int(rot["dims"]) if rot else 0
    if dims == 0:
        return x
    f, amp = pair_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------ attention over visible keys
def attend(q, k, v, positions, scale, window=0, softcap=0.0, plus_one=False):
    """q [T, H, D], k [T, H, D], v [T, H, Dv] (already one key head per query head).  Row i reads j <= i, and with a
    window only ``i - j < window``; scores may be capped; ``plus_one`` adds one to the softmax's denominator."""
    T, H = q.shape[0], q.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        pi = int(positions[i])
        js = [j for j in range(T) if int(positions[j]) <= pi and (window <= 0 or pi - int(positions[j]) < window)]
        for h in range(H):
            s = (k[js, h] @ q[i, h]) * scale
            if softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            m = torch.clamp(s.max(), min=0.0) if plus_one else s.max()
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(-m) if plus_one else 0.0)
            out[i, h] = (e / den) @ v[js, h]
    return out


def latent_kv(h, W, p, m, eps, positions):
    """What a cache would keep per token: the normed latent c [T, kv_rank] and the turned shared key part [T, rot_dim]."""
    rk = m["kv_rank"]
    d = h @ W[p + "dkv"].T
    c = rms(d[:, :rk], eps) * W[p + "dkv.norm"]
    kr = rotate_pairs(d[:, None, rk:], positions, m.get("rot"))[:, 0]
    return c, kr


def latent_attention(h, W, p, m, eps, positions=None, kept=None, gated=True, window=0):
    """``kept``: (c, turned key part) of another layer, used instead of this layer's own."""
    T = h.shape[0]
    H, D, R, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    pos = torch.arange(T) if positions is None else positions
    cq = rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, D + R)
    q = torch.cat([q[..., :D], rotate_pairs(q[..., D:], pos, m.get("rot"))], dim=-1)
    c, kr = kept if kept is not None else latent_kv(h, W, p, m, eps, pos)
    k = torch.cat([(c @ W[p + "uk"].T).view(T, H, D), kr[:, None, :].expand(T, H, R)], dim=-1)
    v = (c @ W[p + "uv"].T).view(T, H, Dv)
    out = attend(q, k, v, pos, float(m["scale"]), window=window).reshape(T, H * Dv)
    if gated:
        out = out * torch.sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def sink_attention(h, W, p, m, eps, positions=None):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, Dv)
    q = rms(rotate_pairs(q, pos, m.get("rot")), eps)
    k = rms(rotate_pairs(k, pos, m.get("rot")), eps)
    rep = H // G
    out = attend(q, k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1), pos, float(m["scale"]),
                 softcap=float(m.get("softcap") or 0.0), plus_one=True)
    return out.reshape(T, H * Dv) @ W[p + "o"].T + W[p + "o.b"]


# ------------------------------------------------------------------------------ feed-forward
def clamped_glu(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def relu2_expert(h, W, p):
    return torch.relu(h @ W[p + "up"].T) ** 2 @ W[p + "down"].T


def route(h, W, p, top):
    """(indices [T, top] in order of falling score, weights [T, top], and per row the gap between the last chosen
    and the best unchosen router logit as a fraction of the spread of the row's logits: how near the row is to
    choosing otherwise)."""
    z = h @ W[p + "router"].T
    s = torch.softmax(z, dim=-1)
    order = torch.argsort(s, dim=-1, descending=True, stable=True)
    idx = order[:, :top]
    w = torch.gather(s, 1, idx)
    if top < s.shape[1]:
        zs = torch.gather(z, 1, order)
        margin = (zs[:, top - 1] - zs[:, top]) / (zs[:, 0] - zs[:, -1]).clamp_min(1e-30)
    else:
        margin = torch.full((h.shape[0],), 1.0, dtype=F64)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20), margin


def expert_mixture(h, W, p, mlp, margins=None):
    top = mlp["router"]["top"]
    idx, w, margin = route(h, W, p, top)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for r in range(top):
            out[t] += w[t, r] * relu2_expert(h[t:t + 1], W, f"{p}e{int(idx[t, r])}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * relu2_expert(h, W, p + "shared.")
    return out


def feed_forward(h, W, p, mlp, margins=None):
    if mlp["kind"] == "dense":
        return clamped_glu(h, W, p, float(mlp["limit"]))
    if mlp["kind"] == "moe":
        return expert_mixture(h, W, p, mlp, margins)
    raise ValueError(mlp["kind"])


# ------------------------------------------------------------------------------ the model
def forward(cfg, W, ids, layers_out=None, margins=None):
    """float64 logits [T, vocab] of one whole sequence."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.tensor(list(ids), dtype=torch.long)
    T = ids.shape[0]
    pos = torch.arange(T)
    x = W["embed"][ids] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = norm_one_plus(x, W[p + "norm1"], eps)
        kind = kind_of(L["type"])
        if kind == "attention":
            y = sink_attention(h, W, p + "mix.", m, eps, pos)
        elif kind in ("latent_attention", "latent_attention_2"):
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(h, W, p + "mix.", m, eps, pos)
            y = latent_attention(h, W, p + "mix.", m, eps, pos, kept=kept[i if src is None else src],
                                 gated=kind == "latent_attention",
                                 window=int(m["mask"]["size"]) if kind == "latent_attention_2" else 0)
        else:
            raise ValueError(L["type"])
        x = x + norm_one_plus(y, W[p + "norm1b"], eps)
        if L.get("mlp"):
            h = norm_one_plus(x, W[p + "norm2"], eps)
            x = x + norm_one_plus(feed_forward(h, W, p + "mlp.", L["mlp"], margins), W[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T


def greedy_generate(cfg, W, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]


# ------------------------------------------------------------------------------ weights of our own
def mixer_shapes(kind, m, Wd, x):
    """name -> (shape, kind) for one mixer; kind: 'w' matrix, 'z' vector around zero, 'o' vector around one."""
    out = {}
    if kind == "attention":
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({x + "q": ((H * D, Wd), "w"), x + "q.b": ((H * D,), "z"), x + "k": ((G * D, Wd), "w"),
                    x + "k.b": ((G * D,), "z"), x + "v": ((G * Dv, Wd), "w"), x + "v.b": ((G * Dv,), "z"),
                    x + "o": ((Wd, H * Dv), "w"), x + "o.b": ((Wd,), "z")})
    else:
        H, D, R, Dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        out.update({x + "dq": ((rq, Wd), "w"), x + "dq.norm": ((rq,), "o"), x + "uq": ((H * (D + R), rq), "w"),
                    x + "uk": ((H * D, rk), "w"), x + "uv": ((H * Dv, rk), "w"), x + "o": ((Wd, H * Dv), "w")})
        if m.get("kv_from") is None:
            out.update({x + "dkv": ((rk + R, Wd), "w"), x + "dkv.norm": ((rk,), "o")})
        if kind == "latent_attention":
            out[x + "g"] = ((H * Dv, Wd), "w")
    return out


def mlp_shapes(mlp, Wd, x):
    out = {}
    if mlp["kind"] == "dense":
        ff = mlp["ff"]
        out.update({x + "gate": ((ff, Wd), "w"), x + "up": ((ff, Wd), "w"), x + "down": ((Wd, ff), "w")})
    else:
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            out.update({f"{x}e{e}.up": ((ff, Wd), "w"), f"{x}e{e}.down": ((Wd, ff), "w")})
        out[x + "router"] = ((mlp["router"]["experts"], Wd), "r")
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            out.update({x + "shared.up": ((sf, Wd), "w"), x + "shared.down": ((Wd, sf), "w"),
                        x + "shared.sg": ((1, Wd), "w")})
    return out


def tensor_shapes(cfg):
    Wd, V = cfg["width"], cfg["vocab"]
    out = {"embed": ((V, Wd), "e"), "head": ((V, Wd), "w"), "final.norm": ((Wd,), "z")}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        out.update({p + "norm1": ((Wd,), "z"), p + "norm1b": ((Wd,), "z")})
        out.update(mixer_shapes(kind_of(L["type"]), L["mixer"], Wd, p + "mix."))
        if L.get("mlp"):
            out.update({p + "norm2": ((Wd,), "z"), p + "norm2b": ((Wd,), "z")})
            out.update(mlp_shapes(L["mlp"], Wd, p + "mlp."))
    return out


def to_bf16(t):
    return t.to(torch.float32).to(torch.bfloat16).to(F64)


def random_weights(cfg, seed, std=None, router_std=None):
    """float64 tensors whose values are bfloat16 numbers.  Matrices N(0, 1 / fan_in) so that activations keep their
    size, router rows larger so that the scores differ, stored norm weights around zero."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g, dtype=F64)
        if kind == "w":
            t = r * (std if std is not None else 1.0 / math.sqrt(shape[-1]))
        elif kind == "r":
            t = r * (router_std if router_std is not None else 2.0 / math.sqrt(shape[-1]))
        elif kind == "e":
            t = r / float((cfg.get("embedding") or {}).get("scale", 1.0))
        elif kind == "z":
            t = 0.2 * r
        else:
            t = 1.0 + 0.2 * r
        W[name] = to_bf16(t)
    return W


def _bf16_bits(t):
    u = t.to(torch.float32).contiguous().numpy().view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def write_folder(cfg, W, out_dir):
    """config.json and model.safetensors (BF16): 8 bytes of header length, the JSON header, the data."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name in sorted(W):
        raw = _bf16_bits(W[name]).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(W[name].shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(out_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    return out_dir


# ------------------------------------------------------------------------------ configurations of our own
def dense_ff(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe_ff(experts, top, ff, shared_ff=0):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        d["shared"] = {"ff": shared_ff}
    return d


def latent_layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, window=0, kv_from=None, mlp=None,
                 kind=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"dims": rot_dim, "base": base}}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": kind or ("latent_attention_2" if window else "latent_attention"), "mixer": m, "mlp": mlp}


def sink_layer(heads, kv_heads, dim, vdim, rot_dims, base, scale, softcap, scaling=None, mlp=None, kind="attention"):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "rot": rot}
    return {"type": kind, "mixer": m, "mlp": mlp}


def model_config(layers, width, vocab, eps=1e-6, embed_scale=None):
    cfg = {"architecture": "Gekitar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if embed_scale is not None:
        cfg["embedding"] = {"scale": embed_scale}
    return cfg


def mixer_weights(layer, width, seed, prefix="m."):
    """The tensors of one mixer alone, named ``<prefix><tensor>``."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, (shape, kind) in mixer_shapes(kind_of(layer["type"]), layer["mixer"], width, prefix).items():
        r = torch.randn(shape, generator=g, dtype=F64)
        t = r / math.sqrt(shape[-1]) if kind == "w" else (0.2 * r if kind == "z" else 1.0 + 0.2 * r)
        W[name] = to_bf16(t)
    return W
