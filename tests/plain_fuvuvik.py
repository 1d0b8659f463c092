"""A plain, slow implementation of the Fuvuvik decoder: one function per mechanism, whole sequences at once, float64 by
default.  It shares no code with the package: it reads ``config.json`` and the safetensors file itself and has no cache,
no state and no batches.

The model: several copies ("streams") of the residual start as the scaled token embedding.  Each sublayer (a mixer, then
a gated feed-forward where the layer has one) reads a weighted sum of the streams through an RMS norm, and its output,
multiplied by a sigmoid gate computed from the same normalised rows, is written back into every stream while the streams
are mixed among themselves.  The mixer reads its rows blended with the row before ("token shift").  Mixers: attention
with short causal convolutions and unit-normed queries and keys; attention in chunks with one added to the softmax's
denominator; a minGRU recurrence.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

DT = torch.float64


# ---- reading a model folder ---------------------------------------------------------------------------------------
def read_model_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    weights = {}
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        index = json.loads(f.read(n))
        base = 8 + n
        kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
        for name, meta in index.items():
            if name == "__metadata__":
                continue
            a, b = meta["data_offsets"]
            f.seek(base + a)
            t = torch.frombuffer(bytearray(f.read(b - a)), dtype=kinds[meta["dtype"]]).reshape(meta["shape"])
            weights[name] = t.to(DT) if t.is_floating_point() else t
    return config, weights


# ---- small pieces ---------------------------------------------------------------------------------------------------
def rms_norm(x, eps, weight=None):
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, mu):
    """Row t becomes h_t + (h_(t-1) - h_t) * mu, with zeros before the first row."""
    before = torch.zeros_like(h)
    before[1:] = h[:-1]
    return h + (before - h) * mu


def short_convolution(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def rotate(x, positions, base, dims):
    """x [T, heads, dim]: the first ``dims`` entries of every head turn, entry i paired with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=DT)
    angle = positions.to(DT)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def attention_weights(q, k, scale, chunk, sink):
    """q [T, H, d], k [T, H, d] -> [H, T, T]: causal, optionally only inside chunks of ``chunk`` positions counted from 0,
    softmax, with 1 added to the denominator when ``sink``."""
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if chunk:
        seen = seen & (i // chunk == j // chunk)
    scores = scores.masked_fill(~seen, float("-inf"))
    top = scores.max(dim=-1, keepdim=True).values
    if sink:
        top = torch.clamp(top, min=0.0)
    e = torch.exp(scores - top)
    total = e.sum(dim=-1, keepdim=True)
    if sink:
        total = total + torch.exp(-top)
    return e / total


# ---- mixers ------------------------------------------------------------------------------------------------------------
def attention_mixer(h, w, p, m, eps, chunked):
    """``chunked`` False: convolutions after the projections, unit-normed queries and keys, every earlier key visible,
    ordinary softmax.  True: no convolution, no norm, chunks of ``mask.size``, the softmax with a sink."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if not chunked:
        q, k, v = (short_convolution(t, w[p + n + ".conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    positions = torch.arange(T)
    q = rotate(q.view(T, H, d), positions, m["rot"]["base"], m["rot"]["dims"])
    k = rotate(k.view(T, G, d), positions, m["rot"]["base"], m["rot"]["dims"])
    if not chunked:
        q, k = rms_norm(q, eps), rms_norm(k, eps)
    v = v.view(T, G, dv)
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    weights = attention_weights(q, k, m["scale"], m["mask"]["size"] if chunked else 0, sink=chunked)
    out = torch.einsum("hij,jhd->ihd", weights, v)
    out = out * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def mingru_mixer(h, w, p):
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    candidate = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    state = torch.zeros(z.shape[1], dtype=DT)
    rows = []
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * candidate[t]
        rows.append(state)
    g = h @ w[p + "g"].T
    return (torch.stack(rows) * (g * torch.sigmoid(g))) @ w[p + "o"].T


def feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---- the model ---------------------------------------------------------------------------------------------------------
def sublayer(streams, w, layer, q, eps, run):
    """Sublayer ``q`` (1 mixer, 2 feed-forward) over the streams [S, T, D]; ``run(h)`` is the mixer or feed-forward."""
    hc = f"{layer}.hc{q}."
    u = torch.einsum("s,std->td", w[hc + "in"], streams)
    h = rms_norm(u, eps, w[f"{layer}.norm{q}"])
    gate = torch.sigmoid(h @ w[f"{layer}.rg{q}"].T + w[f"{layer}.rg{q}.b"])
    y = run(h) * gate
    return torch.einsum("st,sxd->txd", w[hc + "mix"], streams) + w[hc + "out"][:, None, None] * y[None]


def forward_logits(config, weights, ids, layer_sums=None):
    """float64 logits [T, vocab] of the whole sequence ``ids``; ``layer_sums`` (a list) receives the sum of the streams
    after every layer."""
    w = weights
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * config["embedding"]["scale"]
    streams = x[None].repeat(config["streams"], 1, 1)
    for i, spec in enumerate(config["layers"]):
        layer, p, m = f"l{i}", f"l{i}.mix.", spec["mixer"]
        kind = spec["type"]
        if kind == "mingru":
            mixer = lambda h: mingru_mixer(token_shift(h, w[layer + ".shift"]), w, p)
        elif kind in ("attention", "attention_2"):
            mixer = lambda h: attention_mixer(token_shift(h, w[layer + ".shift"]), w, p, m, eps, chunked=kind == "attention_2")
        else:
            raise ValueError(kind)
        streams = sublayer(streams, w, layer, 1, eps, mixer)
        if spec.get("mlp") is not None:
            streams = sublayer(streams, w, layer, 2, eps, lambda h: feed_forward(h, w, f"l{i}.mlp."))
        if layer_sums is not None:
            layer_sums.append(streams.sum(dim=0))
    return rms_norm(streams.sum(dim=0), eps, w["final.norm"]) @ w["head"].T
