"""A plain, slow implementation of the Fuvozen decoder: whole sequences, no cache, float32 on the CPU,
one function per mechanism, written from the design's equations.  It shares no code with the package:
the tests hold the engine (cache, state slots, kernels) to it.

Notation: T tokens, D width, x the residual stream [T, D], h the normalised input of a layer.
"""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open


def read_model_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            weights[name] = t.float() if t.is_floating_point() else t.long()
    return config, weights


def softplus(x):
    return torch.log1p(torch.exp(x))


def group_rms_norm(x, weight, groups: int, eps: float):
    """Every one of ``groups`` equal consecutive parts of a row is divided by its own root mean square."""
    T, D = x.shape
    parts = x.view(T, groups, D // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(T, D) * weight


def rms_unit(x, eps: float):
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def bigram_embedding(config, weights, ids):
    """Token row plus a row of the hashed table of (previous token, token) pairs; the first token takes the last row."""
    spec = config["embedding"]["bigram"]
    buckets, a, b = spec["buckets"], spec["mul_prev"], spec["mul_cur"]
    x = weights["embed"][ids].clone()
    for t, token in enumerate(ids.tolist()):
        row = buckets if t == 0 else (int(ids[t - 1]) * a + token * b) % buckets
        x[t] += weights["bigram"][row]
    return x


def rotate_pairs(x, positions, base: float, dims: int):
    """x [T, ..., d]: the first ``dims`` entries are rotated as pairs (2i, 2i+1) by positions * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=torch.float32)
    freq = base ** (-2.0 * i / dims)
    angle = positions.float()[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = angle.cos().view(shape), angle.sin().view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_attention(h, weights, prefix: str, m, eps: float):
    """Keys and values of all heads are expanded from one small latent per token; one rotated key part is shared."""
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    q = (h @ weights[prefix + "q"].T).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    down = h @ weights[prefix + "dkv"].T
    latent = rms_unit(down[:, :rank], eps) * weights[prefix + "dkv.norm"]
    k_rot = down[:, rank:]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rotate_pairs(q_rot, positions, base, dims)
    k_rot = rotate_pairs(k_rot, positions, base, dims)
    k_plain = (latent @ weights[prefix + "uk"].T).view(T, H, dn)
    value = (latent @ weights[prefix + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("qhd,khd->hqk", q_plain, k_plain) + torch.einsum("qhd,kd->hqk", q_rot, k_rot)) * m["scale"]
    distance = positions[:, None] - positions[None, :]
    visible = distance >= 0
    if m.get("mask"):                            # a sliding window: the token itself and the size - 1 before it
        visible &= distance < m["mask"]["size"]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    out = torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), value).reshape(T, H * dv)
    return out @ weights[prefix + "o"].T


def wkv_mixer(h, weights, prefix: str, m, eps: float):
    """Token-shifted inputs, a per-channel data-dependent decay, and a matrix state per head walked token by token."""
    T, D = h.shape
    H, d = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, D), h[:-1]])

    def mixed(which):
        return h + (before - h) * weights[prefix + "mu." + which]

    r = (mixed("r") @ weights[prefix + "r"].T).view(T, H, d)
    k = (mixed("k") @ weights[prefix + "k"].T).view(T, H, d)
    v = (mixed("v") @ weights[prefix + "v"].T).view(T, H, d)
    g = mixed("g") @ weights[prefix + "g"].T
    gate = g * torch.sigmoid(g)
    lora = torch.tanh(mixed("w") @ weights[prefix + "w1"].T) @ weights[prefix + "w2"].T + weights[prefix + "w0"]
    decay = torch.exp(-torch.exp(lora)).view(T, H, d)
    u = weights[prefix + "u"]
    state = torch.zeros(H, d, d)
    out = torch.zeros(T, H, d)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], state + u[:, :, None] * kv)
        state = decay[t][:, :, None] * state + kv
    out = rms_unit(out, eps).reshape(T, H * d) * weights[prefix + "norm"] * gate
    return out @ weights[prefix + "o"].T


def xielu(z, p, q):
    ap, an = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + 0.5 * z)


def dense_ffn(h, weights, prefix: str):
    p, q = weights[prefix + "act"]
    return xielu(h @ weights[prefix + "up"].T, p, q) @ weights[prefix + "down"].T


def gated_expert(h, weights, prefix: str):
    g = h @ weights[prefix + "gate"].T
    return (g * torch.sigmoid(g) * (h @ weights[prefix + "up"].T)) @ weights[prefix + "down"].T


def moe_ffn(h, weights, prefix: str, spec, gaps=None):
    """``gaps`` (a list) receives, per token, how far the last chosen score lies above the best one left out,
    relative to it: a small gap is a close call that a rounding of h can turn."""
    router = spec["router"]
    scores = torch.softmax(h @ weights[prefix + "router"].T, dim=-1)
    top = torch.topk(scores, router["top"], dim=-1)
    if gaps is not None and router["top"] < scores.shape[-1]:
        ranked = torch.sort(scores, dim=-1, descending=True).values
        gaps.append((ranked[:, router["top"] - 1] - ranked[:, router["top"]]) / ranked[:, router["top"] - 1])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for s, e in zip(top.values[t].tolist(), top.indices[t].tolist()):
            out[t] += s * router["scale"] * gated_expert(h[t:t + 1], weights, f"{prefix}e{e}.")[0]
    if spec.get("shared"):
        out = out + gated_expert(h, weights, prefix + "shared.")
    return out


def forward_logits(config, weights, ids, layers_out=None, gaps=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after every layer,
    ``gaps`` (a list) the routers' gaps per token (see ``moe_ffn``)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x = bigram_embedding(config, weights, ids)
    history = [x]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = group_rms_norm(x, weights[p + "norm1"], groups, eps)
        if layer["type"] == "wkv":
            mixed = wkv_mixer(h, weights, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            mixed = latent_attention(h, weights, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is None:
            fed = 0.0
        elif mlp["kind"] == "dense":
            fed = dense_ffn(h, weights, p + "mlp.")
        else:
            fed = moe_ffn(h, weights, p + "mlp.", mlp, gaps)
        history.append(x + (mixed + fed))
        alpha = weights[p + "dwa"]
        x = sum(alpha[j] * history[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    h = group_rms_norm(x, weights["final.norm"], groups, eps)
    return h @ weights["embed"].T
