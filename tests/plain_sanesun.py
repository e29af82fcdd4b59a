"""Plain, slow implementation of the Sanesun decoder: whole sequences, no cache, one function per mechanism,
float64 arithmetic on bfloat16-rounded weight values.  It shares no code with the package: it reads the
configuration as a dict, makes and writes its own weights, and loops over tokens where the model is recurrent.

Notation.  ``rms(x) = x / sqrt(mean(x^2) + eps)`` over the last axis.  A layer reads the stream once:
``h = rms(x) w1``, ``x += mixer(h) + mlp(h)`` (a layer may have no MLP).  Three mixers:

* ``channel_delta``: a matrix memory per head with the delta rule and one decay per key channel,
* ``attention``: softmax attention through a window that also keeps the first tokens, with a learned sink per
  head, scores mixed across heads before the softmax, part of q and k turned by the position and the values
  turned too (by their own position when written, back by the reader's position after the sum),
* ``latent_attention``: causal attention whose keys and values are both made from one small normed vector per
  token, queries through a normed low-rank step, and a sigmoid gate per head on the output.
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


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.maximum(z, torch.zeros_like(z))


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    ap, an = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(torch.minimum(z, torch.zeros_like(z))) - z) + 0.5 * z)


# ------------------------------------------------------------------------------ rotation of pairs
def rotate_halves(x, positions, dims, base, sign=1.0):
    """x [T, heads, D]: element i < dims/2 is paired with element i + dims/2 and the pair is turned by
    ``sign * position * base^(-2i/dims)``; elements from ``dims`` on pass."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = sign * positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------ window attention with mixed scores
def visible(i, j, size, keep_first):
    """Whether the row at position i reads the key at position j."""
    return j <= i and (i - j < size or j < keep_first)


def window_attention(h, W, p, m, positions=None):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, mask = m.get("rot") or {"dims": 0, "base": 10000.0}, m.get("mask")
    pos = torch.arange(T) if positions is None else positions
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, Dv)
    q = rotate_halves(q, pos, rot["dims"], rot["base"])
    k = rotate_halves(k, pos, rot["dims"], rot["base"])
    v = rotate_halves(v, pos, Dv, rot["base"])                   # every value pair, by the value's own position
    rep = H // G
    raw = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, dim=1)) * float(m["scale"])
    s = torch.einsum("hg,gij->hij", W[p + "talk"], raw)          # the heads' scores are mixed before the softmax
    out = torch.zeros(T, H, Dv, dtype=F64)
    for i in range(T):
        js = [j for j in range(T) if (visible(int(pos[i]), int(pos[j]), mask["size"], mask["keep_first"]) if mask else j <= i)]
        for hd in range(H):
            z = torch.cat([s[hd, i, js], W[p + "sink"][hd:hd + 1]])      # the sink: a score without a value
            w = torch.softmax(z, dim=0)[:-1]
            out[i, hd] = w @ v[js, hd // rep]
    out = rotate_halves(out, pos, Dv, rot["base"], sign=-1.0)    # back by the reader's position
    return out.reshape(T, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------ latent attention
def latent_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    cq = rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, D)
    c = rms(h @ W[p + "dkv"].T, eps) * W[p + "dkv.norm"]          # all that a cache would keep
    k = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, Dv)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    s = s.masked_fill(torch.ones(T, T).triu(1).bool(), float("-inf"))
    out = torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), v)
    out = out * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return out.reshape(T, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------ delta rule with channel decays
def short_conv(x, w):
    """x [T, C], w [C, taps] (the last column is the current token's); zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for d in range(taps):
        y[d:] += x[:T - d] * w[:, taps - 1 - d] if d else x * w[:, taps - 1]
    return y


def channel_delta(h, W, p, m, eps, trace=None):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, dk)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, dk)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    pre = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * softplus(pre).view(T, H, dk))     # [T, H, dk]
    out = torch.zeros(T, H, dv, dtype=F64)
    rep = H // G
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            kk, qq = k[t, hd // rep], q[t, hd // rep]
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kk)
            S = S + torch.outer(kk, u)
            out[t, hd] = S.T @ qq
        if trace is not None:
            trace.append(S)
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, dv)
    y = rms(out, eps) * W[p + "norm"] * gate
    return y.reshape(T, H * dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------ feed-forward
def dense_mlp(h, W, p):
    a = W[p + "act"]
    return xielu(h @ W[p + "up"].T, a[0], a[1]) @ W[p + "down"].T


# ------------------------------------------------------------------------------ the model
def kind_of(layer_type):
    """``attention_2`` is an attention layer with a further set of sizes."""
    head, _, tail = layer_type.rpartition("_")
    return head if head and tail.isdigit() else layer_type


def mixer(L, h, W, p, eps):
    kind = kind_of(L["type"])
    if kind == "channel_delta":
        return channel_delta(h, W, p, L["mixer"], eps)
    if kind == "attention":
        return window_attention(h, W, p, L["mixer"])
    if kind == "latent_attention":
        return latent_attention(h, W, p, L["mixer"], eps)
    raise ValueError(L["type"])


def forward(cfg, W, ids, layers_out=None):
    """float64 logits [T, vocab] of one whole sequence."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.tensor(list(ids), dtype=torch.long)
    x = W["embed"][ids] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * W[p + "norm1"]
        y = mixer(L, h, W, p + "mix.", eps)
        if L.get("mlp"):
            y = y + dense_mlp(h, W, p + "mlp.")
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T


def greedy_generate(cfg, W, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]


# ------------------------------------------------------------------------------ weights of our own
def tensor_shapes(cfg):
    """name -> (shape, kind); kind: 'w' matrix, 'e' embedding, 'z' vector around zero, 'o' vector around one,
    'c' conv taps, 'a' decay rate, 'd' decay bias, 't' head-mixing matrix, 's' sink, 'x' activation numbers."""
    Wd, V = cfg["width"], cfg["vocab"]
    out = {"embed": ((V, Wd), "e"), "head": ((V, Wd), "w"), "final.norm": ((Wd,), "o")}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        x = p + "mix."
        out[p + "norm1"] = ((Wd,), "o")
        kind = kind_of(L["type"])
        if kind == "channel_delta":
            H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            r = m.get("rank", max(4, dk // 2))
            out.update({x + "q": ((G * dk, Wd), "w"), x + "q.conv": ((G * dk, taps), "c"),
                        x + "k": ((G * dk, Wd), "w"), x + "k.conv": ((G * dk, taps), "c"),
                        x + "v": ((H * dv, Wd), "w"), x + "v.conv": ((H * dv, taps), "c"),
                        x + "b": ((H, Wd), "w"), x + "A_log": ((H,), "a"), x + "norm": ((dv,), "o"),
                        x + "a1": ((r, Wd), "w"), x + "a2": ((H * dk, r), "w"), x + "dt_bias": ((H * dk,), "d"),
                        x + "g1": ((r + 1, Wd), "w"), x + "g2": ((H * dv, r + 1), "w"), x + "o": ((Wd, H * dv), "w")})
        elif kind == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({x + "q": ((H * D, Wd), "w"), x + "q.b": ((H * D,), "z"), x + "k": ((G * D, Wd), "w"),
                        x + "k.b": ((G * D,), "z"), x + "v": ((G * Dv, Wd), "w"), x + "v.b": ((G * Dv,), "z"),
                        x + "talk": ((H, H), "t"), x + "sink": ((H,), "s"), x + "o": ((Wd, H * Dv), "w")})
        elif kind == "latent_attention":
            H, D, Dv, rk, rq = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({x + "dq": ((rq, Wd), "w"), x + "dq.norm": ((rq,), "o"), x + "uq": ((H * D, rq), "w"),
                        x + "dkv": ((rk, Wd), "w"), x + "dkv.norm": ((rk,), "o"), x + "uk": ((H * D, rk), "w"),
                        x + "uv": ((H * Dv, rk), "w"), x + "g": ((H, Wd), "w"), x + "o": ((Wd, H * Dv), "w")})
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out.update({p + "mlp.up": ((ff, Wd), "w"), p + "mlp.down": ((Wd, ff), "w"), p + "mlp.act": ((2,), "x")})
    return out


def to_bf16(t):
    return t.to(torch.float32).to(torch.bfloat16).to(F64)


def random_weights(cfg, seed, std=None):
    """float64 tensors whose values are bfloat16 numbers.  Matrices N(0, 1/fan_in) so that activations keep their
    size; norm weights around one; the head-mixing matrix near the unit matrix; decays neither all nor nothing."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g, dtype=F64)
        if kind == "w":
            t = r * (std if std is not None else 1.0 / math.sqrt(shape[-1]))
        elif kind == "e":
            t = r / float((cfg.get("embedding") or {}).get("scale", 1.0))
        elif kind == "z":
            t = 0.2 * r
        elif kind == "o":
            t = 1.0 + 0.2 * r
        elif kind == "c":
            t = 0.5 * r
        elif kind == "a":
            t = -1.0 + 0.5 * r
        elif kind == "t":
            t = torch.eye(shape[0], dtype=F64) + 0.3 * r
        elif kind == "s":
            t = r
        else:
            t = 0.5 * r
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
def delta_layer(heads, kv_heads, dim, vdim, conv, ff=0, rank=None, kind="channel_delta"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if rank is not None:
        m["rank"] = rank
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attention_layer(heads, kv_heads, dim, vdim, window, keep_first, rot_dims, base, scale, ff=0, kind="attention"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": window, "keep_first": keep_first}, "rot": {"dims": rot_dims, "base": base}}
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def latent_layer(heads, dim, vdim, q_rank, kv_rank, scale, ff=0, kind="latent_attention"):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model_config(layers, width, vocab, eps=1e-6, embed_scale=None):
    cfg = {"architecture": "Sanesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if embed_scale is not None:
        cfg["embedding"] = {"scale": embed_scale}
    return cfg


def mixer_weights(layer, width, seed, prefix="m."):
    """The tensors of one mixer alone, named ``<prefix><tensor>``."""
    cfg = model_config([dict(layer, mlp=None)], width, 8)
    W = random_weights(cfg, seed)
    return {k.replace("l0.mix.", prefix): v for k, v in W.items() if k.startswith("l0.mix.")}
