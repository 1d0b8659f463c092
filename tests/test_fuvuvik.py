"""The Fuvuvik decoder in the engine against the plain implementation (``plain_fuvuvik``): each mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages and seats used again,
keys at the edges of a chunk and at page borders, a far key among hundreds, memory of the recurrence over hundreds of
tokens, the first tokens, long decoding, other sizes (one stream, one head, value and key sizes that differ, no rotation),
and greedy generation through the engine's entry point.

Everything runs on the CPU with the reference kernels handed to the engine (host logic: plan, cache groups, state
seats, metadata) and, marked ``gpu``, with the CUDA kernels in float32 and bfloat16.
"""
import json
import os
import random
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

import helpers
import kernel_refs
import plain_fuvuvik as plain
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import ConfigError, EngineConfig, resolve
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.engine.runtime import Engine
from flexengine_b200.parts import CacheGroupSpec, PartSpec, RunEntry, build_part
from flexengine_b200.parts.streams import StreamUpdate
from flexengine_b200.weights import load_model, write_random_model

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
CASES = [pytest.param("cpu", "float32", id="cpu-float32"),
         pytest.param("cuda:0", "float32", id="gpu-float32", marks=pytest.mark.gpu),
         pytest.param("cuda:0", "bfloat16", id="gpu-bfloat16", marks=pytest.mark.gpu)]
F64 = torch.float64


def attention(heads, kv_heads, dim, vdim, conv, rot_dims, base=10000.0, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                           "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else 2.0 / dim ** 0.5}}


def chunked(heads, kv_heads, dim, vdim, size, rot_dims, base=10000.0, scale=None):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size},
                                             "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else 1.0 / dim ** 0.5}}


def mingru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(vocab, width, streams, eps, scale, layers):
    return {"architecture": "Fuvuvik", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}


# P: three streams; value heads wider than key heads and the other way round; part of a head rotated; a chunk shorter than a
#    page; a layer without a feed-forward; two recurrences of different widths; two attentions that share no cache group
# Q: one stream, one attention head, no rotation at all, a convolution of one tap and one of five, sizes that are no powers of two
# R: head size 64 (the fast attention kernels in bfloat16), groups of four query heads, a chunk that is no multiple of a page
CONFIGS = {
    "P": config(211, 64, 3, 1e-5, 0.7, [
        (attention(4, 2, 16, 24, 3, 8, base=500.0), dense(96)),
        (mingru(80), dense(48)),
        (chunked(3, 1, 32, 16, 12, 32), None),
        (mingru(40), dense(64)),
        (attention(2, 2, 16, 16, 4, 16), dense(32))]),
    "Q": config(301, 96, 1, 3e-6, 1.0, [
        (mingru(72), dense(112)),
        (chunked(1, 1, 48, 48, 5, 0), dense(40)),
        (attention(1, 1, 24, 40, 1, 0), dense(56)),
        (attention(3, 3, 16, 16, 5, 4, base=77.0), None)]),
    "R": config(400, 128, 4, 1e-6, 2.0, [
        (attention(4, 2, 64, 64, 2, 32), dense(192)),
        (chunked(8, 2, 64, 64, 70, 64, base=50000.0), dense(64)),
        (mingru(128), None),
        (chunked(8, 2, 64, 64, 70, 64, base=50000.0), dense(64))]),
}
PAGE = {"P": 16, "Q": 8, "R": 16}
LENGTHS = {"P": [5, 33, 70, 1, 47], "Q": [2, 40, 77, 23], "R": [150, 64, 90]}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp(f"fuvuvik_{name}")
        write_random_model(cfg, str(d), seed=41 + i)
        out[name] = str(d)
    return out


def ops_for(device):
    if device == "cpu":
        return kernel_refs
    from flexengine_b200 import ops
    return ops


def make_runner(model_dir, dtype, device, pages, page, seats=4):
    _cfg, plan, model = load_model(model_dir, dtype, device)
    cache = CacheManager(plan.cache_groups, pages, page, seats, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], device)
    return ModelRunner(model, cache, ops=ops_for(device))


def plain_logits(model_dir, ids):
    cfg, weights = plain.read_model_folder(model_dir)
    return plain.forward_logits(cfg, weights, ids)


def close(got, want, dtype, what, bars=(3e-5, 6e-2)):
    """Every row within 3e-5 (float32) or 6e-2 (bfloat16) of its own spread, with a tenth of the overall spread as the floor."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, what
    assert torch.isfinite(got).all(), what
    want2, got2 = want.reshape(-1, want.shape[-1]), got.reshape(-1, want.shape[-1])
    floor = max(0.1 * float(want2.std()), 1e-3)
    scale = torch.clamp(want2.std(dim=-1), min=floor)
    err = (got2 - want2).abs().max(dim=-1).values / scale
    bar = bars[0] if dtype == "float32" else bars[1]
    worst = int(err.argmax())
    assert float(err[worst]) <= bar, f"{what}: row {worst} is off by {float(err[worst]):.3e} of its spread (bar {bar:.0e})"


def compare(model_dir, results, requests, dtype, what):
    for rid, ids in requests.items():
        want = plain_logits(model_dir, ids)
        rows = sorted(p for (r, p) in results if r == rid)
        assert rows == list(range(len(ids))), f"{what}: request {rid} misses rows"
        close(torch.stack([results[(rid, p)] for p in rows]), want, dtype, f"{what} request {rid}")


def requests_for(name, seed=3):
    rng = random.Random(seed)
    return {f"r{i}": helpers.random_prompt(rng, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# ---- the plan -----------------------------------------------------------------------------------------------------
def test_plan_reads_every_size_from_the_configuration():
    _typed, plan = resolve(CONFIGS["P"])
    assert plan.architecture == "Fuvuvik" and plan.vocab_size == 211 and plan.hidden_size == 64
    groups = {g.name: g for g in plan.cache_groups}
    # a kept row per layer; heads of 24 values and 16 keys in rows of 32; the chunked layer's rows of 32; histories of 2 and 3 rows
    assert groups["token_shift"].slots == 5 and groups["token_shift"].state_shape == (64,)
    assert (groups["attention_2x32_full"].kind, groups["attention_2x32_full"].head_dim) == ("full", 32)
    assert (groups["attention_1x32_chunk12"].kind, groups["attention_1x32_chunk12"].window) == ("chunk", 12)
    assert groups["conv_history_2x144"].state_shape == (2 * 144,) and groups["conv_history_3x96"].state_shape == (3 * 96,)
    assert groups["mingru_state_80"].state_shape == (80,) and groups["mingru_state_40"].state_shape == (40,)
    assert [layer.feed_forward.kind if layer.feed_forward else None for layer in plan.layers] == ["gated_mlp", "gated_mlp", None, "gated_mlp", "gated_mlp"]
    # two layers of one shape share a group and take a slot each
    _typed, plan = resolve(CONFIGS["R"])
    group = [g for g in plan.cache_groups if g.kind == "chunk"]
    assert len(group) == 1 and group[0].slots == 2 and [e.cache_slot for e in plan.run] == [0, 0, 0, 1]
    # what the design fixes per mixer type
    first, second = plan.layers[0].mixer.params, plan.layers[1].mixer.params
    assert (first["conv"], first["qk_norm"], first["mask"], first["sink"]) == (2, True, "full", False)
    assert (second["conv"], second["qk_norm"], second["mask"], second["mask_size"], second["sink"]) == (0, False, "chunk", 70, True)


def test_configuration_errors_are_named():
    broken = json.loads(json.dumps(CONFIGS["Q"]))
    broken["layers"][1]["type"] = "attention_3"
    with pytest.raises(ConfigError, match="unknown mixer type"):
        resolve(broken)
    broken = json.loads(json.dumps(CONFIGS["Q"]))
    del broken["layers"][1]["mixer"]["mask"]
    with pytest.raises(ConfigError, match="mask.size"):
        resolve(broken)
    broken = json.loads(json.dumps(CONFIGS["Q"]))
    broken["streams"] = 0
    with pytest.raises(ConfigError, match="streams"):
        resolve(broken)


# ---- each mechanism alone -----------------------------------------------------------------------------------------
def step_context(device, dtype, cache, entries, ops):
    runner = ModelRunner.__new__(ModelRunner)                # only build_context is used
    runner.cache, runner.ops, runner.device = cache, ops, cache.device
    runner._ring, runner._ring_at, runner.h2d_bytes = [], 0, 0
    runner.model = types.SimpleNamespace(dtype=dtype)
    return runner.build_context([StepEntry(rid, [0] * n, []) for rid, n in entries])


def drive(run, group_specs, h, cuts, device, dtype, page=4, seats=2, pages=96):
    """``run(ctx, rows)`` over a cache of its own, the sequence cut into ``cuts`` portions; a second request runs in between
    and ends, so that its seat and pages are used again."""
    ops = ops_for(device)
    cache = CacheManager(group_specs, pages, page, seats, dtype, device)
    outs, fed = [], 0
    for n in cuts:
        cache.reserve("r", fed + n)
        ctx = step_context(device, dtype, cache, [("r", n)], ops)
        outs.append(run(ctx, h[fed:fed + n].to(device=device, dtype=dtype).contiguous()).float().cpu())
        cache.commit("r", n)
        fed += n
        if fed == cuts[0]:                                   # a neighbour that comes and goes
            cache.reserve("other", 7)
            ctx = step_context(device, dtype, cache, [("other", 7)], ops)
            run(ctx, torch.randn(7, h.shape[1]).to(device=device, dtype=dtype))
            cache.commit("other", 7)
            cache.free("other")
    cache.assert_invariants()
    return torch.cat(outs)


def bind_by_checkpoint_names(part, weights, prefix, names, device, dtype):
    tensors = {}
    for local, (shape, kind) in part.parameter_shapes().items():
        source = torch.cat([weights[prefix + n].reshape(-1, *weights[prefix + n].shape[1:]) for n in names[local]])
        held = torch.float32 if kind in ("vector", "float32") else dtype
        tensors[local] = source.reshape(shape).to(device=device, dtype=held).contiguous()
    part.bind(tensors)


def bf16_exact(t):
    return t.to(torch.bfloat16).float()


def randn(*shape, seed, scale=1.0):
    return bf16_exact(torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale)


def as64(weights):
    return {k: v.to(F64) for k, v in weights.items()}


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("streams,width", [(1, 40), (2, 40), (3, 42), (5, 40), (8, 36), (9, 40), (16, 24)])
def test_stream_norm_and_update_alone(device, dtype, streams, width):
    """A sublayer's output goes into every stream while they are mixed, then the learned sum is normed: all rows in place,
    and chosen rows without writing anything.  Widths that are and are not multiples of four, up to the most streams."""
    dt = getattr(torch, dtype)
    ops = ops_for(device)
    S, T, D, eps = streams, 9, width, 1e-5
    x = torch.randn(S, T, D, generator=torch.Generator().manual_seed(1))
    y, gate = randn(T, D, seed=2), randn(T, D, seed=3)
    bias, mix = randn(D, seed=4), randn(S, S, seed=5)
    write, read, weight = randn(S, seed=6), randn(S, seed=7), randn(D, seed=8)
    new = torch.einsum("st,snd->tnd", mix.to(F64), x.to(F64)) + write.to(F64)[:, None, None] * (y.to(F64) * torch.sigmoid(gate.to(F64) + bias.to(F64)))[None]
    want = plain.rms_norm(torch.einsum("s,snd->nd", read.to(F64), new), eps, weight.to(F64))
    norm = build_part("norm", PartSpec("stream_rmsnorm", {"hidden_size": D, "eps": eps, "streams": S}))
    norm.bind({"weight": weight.to(device)})
    ctx = types.SimpleNamespace(ops=ops, dtype=dt)
    update = StreamUpdate(y.to(device=device, dtype=dt), gate.to(device=device, dtype=dt), bias.to(device), mix.to(device), write.to(device))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=device)
    streams_dev = x.clone().to(device).contiguous()
    some = norm.forward(ctx, streams_dev, update, rows=rows, read=read.to(device))
    assert torch.equal(streams_dev.cpu(), x)                                  # nothing was written back
    close(some, want[rows.long().cpu()], dtype, "chosen rows", bars=(2e-5, 3e-2))
    got = norm.forward(ctx, streams_dev, update, read=read.to(device))
    close(got, want, dtype, "all rows", bars=(2e-5, 3e-2))
    assert (streams_dev.double().cpu() - new).abs().max() < 1e-4 * float(new.abs().max())
    # a step of one token a request: the token shift of the normed rows in the same kernel; a seat below 0 keeps nothing
    mu = randn(D, seed=9)
    kept_before = randn(T + 2, D, seed=10)
    kept = kept_before.clone().to(device)
    seats = torch.tensor([4, -1, 0, 9, 2, 10, 1, 7, 3], dtype=torch.int32, device=device)
    again = x.clone().to(device).contiguous()
    rows_out, shifted = norm.forward(ctx, again, update, read=read.to(device), shift=(mu.to(device), kept, seats))
    close(rows_out, want, dtype, "rows beside their shift", bars=(2e-5, 3e-2))
    before = torch.stack([kept_before[seat] if seat >= 0 else torch.zeros(D) for seat in seats.tolist()]).to(F64)
    close(shifted, want + (before - want) * mu.to(F64), dtype, "shifted rows", bars=(2e-5, 3e-2))
    for i, seat in enumerate(seats.tolist()):
        if seat >= 0:
            assert torch.equal(kept[seat].cpu(), rows_out[i].float().cpu())
    assert torch.equal(kept[5].cpu(), kept_before[5]) and torch.equal(kept[8].cpu(), kept_before[8])       # nobody's seats
    # no update and the plain sum: what the model's last norm does when nothing is pending
    plain_sum = norm.forward(ctx, streams_dev, None, rows=rows)
    close(plain_sum, plain.rms_norm(new.sum(dim=0), eps, weight.to(F64))[rows.long().cpu()], dtype, "plain sum", bars=(2e-5, 3e-2))


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("width", [24, 30])
def test_token_shift_alone(device, dtype, width):
    from flexengine_b200.parts.streams import TokenShift
    dt = getattr(torch, dtype)
    D, T = width, 19
    mu = randn(D, seed=1)
    h = randn(T, D, seed=2)
    shift = TokenShift(D, 0, 1)
    shift.bind({"mu": mu.to(device)})
    spec = CacheGroupSpec("kept", "state", slots=2, state_shape=(D,))
    want = plain.token_shift(h.to(F64), mu.to(F64))
    for cuts in ([T], [1] * T, [2, 9, 2, 1, 5], [18, 1]):
        close(drive(lambda ctx, rows: shift.forward(ctx, rows), [spec], h, cuts, device, dt), want, dtype, f"token shift {cuts[:4]}", bars=(1e-6, 2e-2))


@pytest.mark.parametrize("device,dtype", CASES)
def test_gated_feed_forward_alone(device, dtype):
    dt = getattr(torch, dtype)
    D, F, T = 48, 72, 13
    weights = {"gate": randn(F, D, seed=1, scale=D ** -0.5), "up": randn(F, D, seed=2, scale=D ** -0.5), "down": randn(D, F, seed=3, scale=F ** -0.5)}
    part = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": F, "activation": "gelu_tanh"}))
    bind_by_checkpoint_names(part, weights, "", {"gate_up.weight": ["gate", "up"], "down.weight": ["down"]}, device, dt)
    h = randn(T, D, seed=4, scale=2.0)                                       # both tails of the gate function
    ctx = types.SimpleNamespace(ops=ops_for(device), dtype=dt)
    want = plain.feed_forward(h.to(F64), as64(weights), "")
    for rows in (T, 5):                                                      # a handful of rows takes another kernel in bfloat16
        got = part.forward(ctx, h[:rows].to(device=device, dtype=dt).contiguous())
        close(got, want[:rows], dtype, f"gated feed-forward, {rows} rows", bars=(2e-5, 4e-2))


def mingru_weights(D, W, seed):
    return {"z": randn(W, D, seed=seed, scale=D ** -0.5), "z.b": randn(W, seed=seed + 1), "x": randn(W, D, seed=seed + 2, scale=2 * D ** -0.5),
            "x.b": randn(W, seed=seed + 3, scale=0.5), "g": randn(W, D, seed=seed + 4, scale=D ** -0.5), "o": randn(D, W, seed=seed + 5, scale=W ** -0.5)}


MINGRU_NAMES = {"zxg.weight": ["z", "x", "g"], "zx.bias": ["z.b", "x.b"], "o.weight": ["o"]}


def mingru_part(D, W, weights, device, dt):
    mixer = build_part("mixer", PartSpec("mingru", {"hidden_size": D, "width": W}))
    bind_by_checkpoint_names(mixer, weights, "", MINGRU_NAMES, device, dt)
    need = mixer.cache_need()
    return mixer, CacheGroupSpec("state", "state", slots=1, state_shape=need["state_shape"], state_dtype=need["state_dtype"])


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("width", [40, 129])
def test_mingru_alone(device, dtype, width):
    """Whole, token by token, and in portions down to two tokens: the state is carried by the seat."""
    dt = getattr(torch, dtype)
    D, T = 32, 37
    weights = mingru_weights(D, width, seed=5)
    mixer, spec = mingru_part(D, width, weights, device, dt)
    h = randn(T, D, seed=6)
    want = plain.mingru_mixer(h.to(F64), as64(weights), "")
    for cuts in ([T], [1] * T, [5, 2, 17, 2, 1, 10], [2, 33, 2]):
        close(drive(lambda ctx, rows: mixer.forward(ctx, rows, RunEntry(0, 0, 0, True)), [spec], h, cuts, device, dt), want, dtype,
              f"mingru cut {cuts[:4]}")


@pytest.mark.parametrize("device,dtype", CASES)
def test_mingru_remembers_over_hundreds_of_tokens(device, dtype):
    """Gates that are almost shut: what token 3 put into the state still decides the output 600 tokens later, through a long
    portion (scanned in blocks on the device), short ones and single tokens.  A state that is lost, zeroed or mixed up
    between seats shows at once."""
    dt = getattr(torch, dtype)
    D, W, T = 32, 48, 640
    weights = mingru_weights(D, W, seed=7)
    weights["z"] *= 0.02
    weights["z.b"] = torch.full((W,), -8.0)
    weights["x"][:, 0] = 0.0
    weights["z"][:, 0] = bf16_exact(torch.full((W,), 3.0))                    # channel 0 of the input opens the gate
    weights["x.b"] = bf16_exact(torch.full((W,), 2.0))
    mixer, spec = mingru_part(D, W, weights, device, dt)
    h = randn(T, D, seed=8, scale=0.1)
    h[:, 0] = 0.0
    h[3, 0] = 4.0                                                             # the one that is remembered
    want = plain.mingru_mixer(h.to(F64), as64(weights), "")
    silent = h.clone()
    silent[3, 0] = 0.0
    assert (plain.mingru_mixer(silent.to(F64), as64(weights), "")[-1] - want[-1]).abs().max() > 0.3 * want[-1].abs().max()
    got = drive(lambda ctx, rows: mixer.forward(ctx, rows, RunEntry(0, 0, 0, True)), [spec], h, [2, 300, 270, 2, 40] + [1] * 26, device, dt)
    close(got, want, dtype, "far memory", bars=(1e-4, 0.1))


@pytest.mark.parametrize("device,dtype", CASES)
def test_mingru_over_a_portion_of_thousands_of_tokens(device, dtype):
    """A portion of 4,200 tokens (on the device: the scan in blocks of 64, chained) and what follows it, against the walk."""
    dt = getattr(torch, dtype)
    D, W, T = 16, 40, 4300
    weights = mingru_weights(D, W, seed=17)
    weights["z.b"] = torch.full((W,), -3.0)                                   # slow gates: the state spans many blocks
    mixer, spec = mingru_part(D, W, weights, device, dt)
    h = randn(T, D, seed=18)
    want = plain.mingru_mixer(h.to(F64), as64(weights), "")
    got = drive(lambda ctx, rows: mixer.forward(ctx, rows, RunEntry(0, 0, 0, True)), [spec], h, [4200, 98, 1, 1], device, dt)
    close(got, want, dtype, "a long portion", bars=(1e-4, 0.1))


def attention_weights(D, m, seed, conv):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"q": randn(H * d, D, seed=seed, scale=D ** -0.5), "k": randn(G * d, D, seed=seed + 1, scale=D ** -0.5),
         "v": randn(G * dv, D, seed=seed + 2, scale=D ** -0.5), "g": randn(H, D, seed=seed + 3, scale=D ** -0.5),
         "o": randn(D, H * dv, seed=seed + 4, scale=(H * dv) ** -0.5)}
    if conv:
        w.update({"q.conv": randn(H * d, conv, seed=seed + 5, scale=0.5), "k.conv": randn(G * d, conv, seed=seed + 6, scale=0.5),
                  "v.conv": randn(G * dv, conv, seed=seed + 7, scale=0.5)})
    return w


ATTENTION_NAMES = {"qkvg.weight": ["q", "k", "v", "g"], "o.weight": ["o"], "conv.weight": ["q.conv", "k.conv", "v.conv"]}


def attention_part(D, m, weights, device, dt, chunk, eps=1e-5):
    """The part and its cache groups (paged rows; the convolution's history)."""
    conv = m.get("conv", 0)
    params = {"hidden_size": D, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
              "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"], "conv": conv, "qk_norm": not chunk, "eps": eps,
              "mask": "chunk" if chunk else "full", "mask_size": m["mask"]["size"] if chunk else 0, "sink": bool(chunk)}
    if conv > 1:
        params.update(conv_group=1, conv_slot=0)
    mixer = build_part("mixer", PartSpec("gated_attention", params))
    bind_by_checkpoint_names(mixer, weights, "", ATTENTION_NAMES, device, dt)
    need = mixer.cache_need()
    specs = [CacheGroupSpec("rows", need["kind"], slots=1, kv_heads=need["kv_heads"], head_dim=need["head_dim"], window=need["window"])]
    if conv > 1:
        specs.append(CacheGroupSpec("history", "state", slots=1, state_shape=((conv - 1) * mixer.channels,)))
    return mixer, specs


def run_attention(mixer):
    return lambda ctx, rows: mixer.forward(ctx, rows, RunEntry(0, 0, 0, True))


# heads, kv_heads, dim, vdim, conv, rot_dims: values wider and narrower than keys, no convolution history (one tap), five taps
# (longer than the shortest portions), no rotation, a whole head rotated, the head size of the fast kernels, one head
@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", [(4, 2, 16, 24, 3, 8), (2, 1, 32, 16, 1, 32), (3, 3, 16, 16, 5, 0), (8, 2, 64, 64, 4, 48), (1, 1, 40, 8, 2, 20),
                                   (2, 1, 16, 12, 2, 8)])
def test_attention_with_convolutions_alone(device, dtype, shape):
    dt = getattr(torch, dtype)
    D, T = 48, 41
    m = attention(*shape, base=300.0)["mixer"]
    weights = attention_weights(D, m, seed=10, conv=shape[4])
    mixer, specs = attention_part(D, m, weights, device, dt, chunk=False)
    h = randn(T, D, seed=11)
    want = plain.attention_mixer(h.to(F64), as64(weights), "", m, 1e-5, chunked=False)
    for cuts in ([T], [1] * T, [7, 2, 19, 2, 1, 10], [2, 37, 2], [1, 1, 2, 1, 36]):
        close(drive(run_attention(mixer), specs, h, cuts, device, dt), want, dtype, f"attention {shape} cut {cuts[:5]}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", [(3, 1, 32, 16, 12, 32), (1, 1, 48, 48, 5, 0), (8, 2, 64, 64, 70, 64), (4, 4, 16, 24, 16, 8), (6, 3, 24, 24, 1, 24)])
def test_chunked_attention_alone(device, dtype, shape):
    """Chunks shorter than, equal to and longer than a page (4), of one position, and no multiple of anything; portions that
    end and begin inside chunks."""
    dt = getattr(torch, dtype)
    D, T = 48, 90
    m = chunked(*shape, base=300.0)["mixer"]
    weights = attention_weights(D, m, seed=20, conv=0)
    mixer, specs = attention_part(D, m, weights, device, dt, chunk=True)
    h = randn(T, D, seed=21)
    want = plain.attention_mixer(h.to(F64), as64(weights), "", m, 1e-5, chunked=True)
    for cuts in ([T], [60] + [1] * 30, [7, 2, 19, 2, 1, 59], [2, 86, 2]):
        close(drive(run_attention(mixer), specs, h, cuts, device, dt), want, dtype, f"chunked attention {shape} cut {cuts[:4]}")


def standing_out(D, m, seed):
    """Weights and inputs in which channel 5 of the input drives one unrotated key entry and channel 9 the same query entry,
    so that a key with channel 5 set takes all of a query's weight with channel 9 set, whenever it is visible."""
    weights = attention_weights(D, m, seed=seed, conv=0)
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    weights["k"][:, 5] = 0.0
    weights["q"][:, 9] = 0.0
    weights["q"][:, 5] = 0.0
    weights["k"][:, 9] = 0.0
    for head in range(G):
        weights["k"][head * d + d - 1, :] = 0.0
        weights["k"][head * d + d - 1, 5] = 8.0
    for head in range(H):
        weights["q"][head * d + d - 1, :] = 0.0
        weights["q"][head * d + d - 1, 9] = 8.0
    return weights


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("key_at,seen", [(24, True), (23, False), (16, False), (35, True), (30, True)])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_key_that_stands_out_at_the_chunks_edge(device, dtype, key_at, seen, decoded):
    """Chunks of 12 in pages of 4: the query at position 35 (the last of chunk 24..35) sees the key at 24 (its chunk's first,
    on a page border), at 30 and itself, and neither 23 (the last of the chunk before) nor 16.  The sink's share shows too:
    where the key is out of sight the scores are small and the sink takes a good part of the weight."""
    dt = getattr(torch, dtype)
    D, size, T = 32, 12, 36
    m = chunked(4, 2, 16, 16, size, 8, scale=0.3)["mixer"]
    weights = standing_out(D, m, seed=12)
    mixer, specs = attention_part(D, m, weights, device, dt, chunk=True)
    h = randn(T, D, seed=13)
    h[:, 5], h[:, 9] = 0.0, 0.0
    h[key_at, 5] = 4.0
    h[-1, 9] = 4.0
    want = plain.attention_mixer(h.to(F64), as64(weights), "", m, 1e-5, chunked=True)
    blind = h.clone()
    blind[key_at, 5] = 0.0
    differs = (plain.attention_mixer(blind.to(F64), as64(weights), "", m, 1e-5, chunked=True)[-1] - want[-1]).abs().max() > 0.05 * want[-1].abs().max()
    assert bool(differs) == seen
    cuts = [T - 1, 1] if decoded else [T - 2, 2]
    close(drive(run_attention(mixer), specs, h, cuts, device, dt), want, dtype, f"key at {key_at}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("decoded", [False, True])
def test_a_far_key_among_hundreds(device, dtype, decoded):
    """Full attention with unit-normed queries and keys: the key at position 3 of 700 has the direction of the last query in
    every head, behind a scale that lets it stand out; it decides the output through portions, pages and single tokens."""
    dt = getattr(torch, dtype)
    D, T = 32, 700
    m = attention(4, 2, 16, 16, 2, 0, scale=24.0)["mixer"]
    weights = attention_weights(D, m, seed=30, conv=2)
    for name in ("q", "k"):                                   # queries and keys read channels 0..15 of the input, head by head the same
        weights[name][:] = 0.0
        for head in range(weights[name].shape[0] // 16):
            weights[name][head * 16:(head + 1) * 16, :16] = torch.eye(16)
    weights["q.conv"][:] = torch.tensor([0.0, 1.0])
    weights["k.conv"][:] = torch.tensor([0.0, 1.0])
    mixer, specs = attention_part(D, m, weights, device, dt, chunk=False)
    h = randn(T, D, seed=31)
    direction = randn(16, seed=32)
    h[3, :16] = direction
    h[-1, :16] = direction
    want = plain.attention_mixer(h.to(F64), as64(weights), "", m, 1e-5, chunked=False)
    blind = h.clone()
    blind[3, :16] = -direction
    assert (plain.attention_mixer(blind.to(F64), as64(weights), "", m, 1e-5, chunked=False)[-1] - want[-1]).abs().max() > 0.2 * want[-1].abs().max()
    cuts = [300, 399, 1] if decoded else [2, 330, 366, 2]
    close(drive(run_attention(mixer), specs, h, cuts, device, dt, page=16, pages=64), want, dtype, "far key")


# ---- the whole model under every way of cutting the work ---------------------------------------------------------------
def scenario(kind, requests, rng):
    if kind == "whole":
        return helpers.steps_whole(requests)
    if kind == "last_decoded":
        return helpers.steps_last_decoded(requests, tail=20)
    if kind == "portions":
        return helpers.steps_portions(requests, rng, sizes=(24, 7, 2, 13, 2, 31, 3, 64, 5))
    doubled = dict(requests)
    doubled.update({rid + "x": ids[::-1] for rid, ids in requests.items()})     # more requests than seats: seats are used again
    return helpers.steps_mixed(doubled, rng, live=4)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("kind", ["whole", "last_decoded", "portions", "mixed"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_model_against_plain(model_dirs, name, kind, device, dtype):
    rng = random.Random(5)
    steps = scenario(kind, requests_for(name), rng)
    page = PAGE[name]
    pages = helpers.peak_pages(steps, page) + (0 if kind == "mixed" else 1)         # just enough: pages are used again
    runner = make_runner(model_dirs[name], dtype, device, pages, page, seats=4)
    results = helpers.run_steps(runner, steps)
    assert runner.cache.used_pages == 0 and len(runner.cache.free_state_slots) == 4
    fed = {}
    for entries, _ in steps:
        for rid, toks, _w in entries:
            fed.setdefault(rid, []).extend(toks)
    compare(model_dirs[name], results, fed, dtype, f"{name}/{kind}/{dtype}")
    if device != "cpu":
        ops_for(device).check_status(device)


def test_layer_sums_against_plain(model_dirs):
    """The sum of the streams after every layer, with what is pending put in: the plain implementation's, layer by layer."""
    name = "P"
    ids = requests_for(name)["r1"]
    cfg, weights = plain.read_model_folder(model_dirs[name])
    sums = []
    plain.forward_logits(cfg, weights, ids, sums)
    _cfg, plan, model = load_model(model_dirs[name], "float32", "cpu")
    cache = CacheManager(plan.cache_groups, 8, 16, 1, torch.float32, "cpu")
    runner = ModelRunner(model, cache, ops=kernel_refs)
    cache.reserve("a", len(ids))
    ctx = runner.build_context([StepEntry("a", ids, [])])
    streams = model.embedding.forward(ctx)
    pending = None
    for at, entry in enumerate(plan.run):
        pending = model.blocks[entry.layer].forward(ctx, streams, pending, entry)
        settled = streams.clone()
        kernel_refs.stream_rmsnorm(settled, None, torch.ones(plan.hidden_size), 1e-6, torch.float32, update=pending)
        assert (settled.sum(dim=0).double() - sums[at]).abs().max() < 2e-5 * float(sums[at].abs().max()), f"layer {at}"


STACKS = {
    "only the recurrence": config(97, 48, 2, 1e-5, 1.0, [(mingru(56), dense(64)), (mingru(24), None)]),
    "only attention": config(97, 48, 2, 1e-5, 0.5, [(attention(2, 1, 16, 16, 3, 8), None), (chunked(2, 2, 16, 32, 9, 16), dense(32))]),
    "one layer": config(50, 32, 1, 1e-5, 1.0, [(mingru(32), None)]),
}


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("stack", list(STACKS))
def test_stacks_of_one_kind(tmp_path, stack, device, dtype):
    """A model without paged groups, one without a recurrence, and one of a single layer without a feed-forward."""
    cfg = STACKS[stack]
    write_random_model(cfg, str(tmp_path), seed=3)
    ids = helpers.random_prompt(random.Random(1), 45, cfg["vocab"])
    runner = make_runner(str(tmp_path), dtype, device, 8, 8)
    got = [runner.step([StepEntry("a", ids[:20], list(range(20)))]), runner.step([StepEntry("a", ids[20:44], list(range(24)))]),
           runner.step([StepEntry("a", ids[44:], [0])])]
    close(torch.cat([g.float().cpu() for g in got]), plain_logits(str(tmp_path), ids), dtype, stack)
    runner.finish("a")
    runner.cache.assert_invariants()


@pytest.mark.parametrize("device,dtype", CASES)
def test_together_and_alone(model_dirs, device, dtype):
    """Unequal requests in one batch against each alone: the same logits (to rounding in bfloat16)."""
    name = "P"
    requests = requests_for(name, seed=9)
    together = make_runner(model_dirs[name], dtype, device, 16, PAGE[name])
    logits = together.step([StepEntry(rid, ids, [len(ids) - 1]) for rid, ids in requests.items()][:4])
    for row, (rid, ids) in enumerate(list(requests.items())[:4]):
        alone = make_runner(model_dirs[name], dtype, device, 8, PAGE[name])
        close(logits[row:row + 1], alone.step([StepEntry(rid, ids, [len(ids) - 1])]), dtype, rid)


@pytest.mark.parametrize("device,dtype", CASES)
def test_first_tokens_and_long_decoding(model_dirs, device, dtype):
    """A prompt of one token, then 150 tokens decoded one by one beside a neighbour that arrives later: every row against the
    whole sequence.  The chunk (12) and the pages pass many times; the chunked group gives pages back."""
    name = "P"
    rng = random.Random(12)
    ids = helpers.random_prompt(rng, 151, CONFIGS[name]["vocab"])
    other = helpers.random_prompt(rng, 60, CONFIGS[name]["vocab"])
    runner = make_runner(model_dirs[name], dtype, device, 16, PAGE[name], seats=2)
    rows, other_rows = [], []
    for p in range(len(ids)):
        entries = [StepEntry("long", ids[p:p + 1], [0])]
        q = p - 40
        if 0 <= q < len(other):
            entries.append(StepEntry("other", other[q:q + 1], [0]))
        logits = runner.step(entries)
        rows.append(logits[0].float().cpu())
        if len(entries) == 2:
            other_rows.append(logits[1].float().cpu())
        if q == len(other) - 1:
            runner.finish("other")
        runner.cache.assert_invariants()
    close(torch.stack(rows), plain_logits(model_dirs[name], ids), dtype, "long decoding")
    close(torch.stack(other_rows), plain_logits(model_dirs[name], other), dtype, "the neighbour")
    chunk_group = [g for _, g in runner.cache.paged if g.spec.kind == "chunk"][0]
    assert chunk_group.pool.used_pages <= 2                  # 151 tokens in chunks of 12 and pages of 16


def test_chunk_groups_give_pages_back():
    """Pages that lie wholly before the chunk of the next token are released at commit, and never a page of that chunk."""
    spec = CacheGroupSpec("rows", "chunk", slots=1, kv_heads=1, head_dim=16, window=10)
    cache = CacheManager([spec], 16, 4, 2, torch.float32, "cpu")
    for upto in (3, 9, 10, 11, 19, 20, 37):
        cache.reserve("a", upto)
        cache.commit("a", upto - cache.tokens_of("a"))
        table = cache.table("a", 0)
        first_needed = upto // 10 * 10
        for j, page in enumerate(table):
            assert (page == -1) == ((j + 1) * 4 <= first_needed), (upto, j, table)
        cache.assert_invariants()
    cache.free("a")
    assert cache.used_pages == 0


# ---- generation through the engine ----------------------------------------------------------------------------------
def greedy(model_dir, prompt, count):
    cfg, weights = plain.read_model_folder(model_dir)
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(plain.forward_logits(cfg, weights, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(model_dirs, device, graphs):
    if graphs and device == "cpu":
        pytest.skip("CUDA graphs need a CUDA device")
    name = "Q"
    rng = random.Random(1)
    prompts = [helpers.random_prompt(rng, n, CONFIGS[name]["vocab"]) for n in (5, 17, 33, 1, 40, 9)]
    cfg = EngineConfig(model=model_dirs[name], device=device, dtype="float32", max_model_len=128, max_num_seqs=3,
                       max_num_batched_tokens=24, prefill_chunk_size=8, kv_block_size=PAGE[name], kv_num_blocks=48,
                       max_output_tokens=16, scheduler_policy="decode_first", cuda_graph=graphs, overlap_steps=device != "cpu")
    engine = Engine.from_model_dir(model_dirs[name], cfg, ops=ops_for(device))
    outputs = engine.generate(prompts, max_tokens=6)
    for prompt, out in zip(prompts, outputs):
        assert out.token_ids == greedy(model_dirs[name], prompt, 6)
    assert engine.cache.used_pages == 0


@pytest.mark.gpu
def test_trace_replay_program(model_dirs, tmp_path):
    """``bin/trace_run`` as a user starts it: steps on standard input, logits in files."""
    name = "P"
    ids = requests_for(name)["r1"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[20:], "want": [len(ids) - 21]}, {"id": "b", "tokens": ids[:3], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": ids[3:5], "want": [1]}], "end": ["b"]}]
    program = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    want = plain_logits(model_dirs[name], ids)
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        done = subprocess.run([sys.executable, program, "--model", model_dirs[name], "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
        vocab = CONFIGS[name]["vocab"]
        rows = [np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, vocab) for n in range(3)]
        close(torch.from_numpy(np.concatenate(rows)), want[[0, 19, len(ids) - 1, 4]], dtype, f"trace_run {dtype}")
