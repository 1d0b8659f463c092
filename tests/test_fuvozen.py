"""The Fuvozen decoder in the engine against the plain implementation (``plain_fuvozen``): each mechanism alone,
whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages and seats
used again, keys at the edges of the window, memory over hundreds of tokens, the first tokens, long decoding,
other sizes, and greedy generation through the engine's entry point.

Everything runs on the CPU with the reference kernels handed to the engine (host logic: plan, cache groups, state
seats, metadata) and, marked ``gpu``, with the CUDA kernels in float32 and bfloat16.
"""
import random
import types

import pytest
import torch

import helpers
import kernel_refs
import plain_fuvozen as plain
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import EngineConfig, resolve
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.engine.runtime import Engine
from flexengine_b200.parts import CacheGroupSpec, PartSpec, RunEntry, build_part
from flexengine_b200.weights import load_model, write_random_model

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
CASES = [pytest.param("cpu", "float32", id="cpu-float32"),
         pytest.param("cuda:0", "float32", id="gpu-float32", marks=pytest.mark.gpu),
         pytest.param("cuda:0", "bfloat16", id="gpu-bfloat16", marks=pytest.mark.gpu)]


def latent(heads, dim, rot_dim, vdim, rank, window, base=10000.0, scale=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
             "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else 0.9 / (dim + rot_dim) ** 0.5}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer}


def wkv(heads, dim):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=0, scale=1.0):
    spec = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        spec["shared"] = {"ff": shared}
    return spec


def config(vocab, width, groups, eps, buckets, muls, layers):
    return {"architecture": "Fuvozen", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": muls[0], "mul_cur": muls[1]}},
            "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}


# P: attention first, a window shorter than a page, two kinds of wkv heads, a layer without a feed-forward, an
#    attention layer that sees everything, a cached row that needs padding (40 + 8 = 48 is a multiple of 16; 20 + 8 is not)
# Q: one norm group, one attention head, every expert chosen, no shared expert, sizes that are no powers of two
# R: head size 64 in the recurrence (state in registers) and a cached row of 128, the sizes of the fast attention kernels
CONFIGS = {
    "P": config(211, 64, 2, 1e-5, 53, (13, 5), [
        (latent(3, 16, 8, 24, 40, 12), moe(5, 2, 24, shared=32, scale=1.5)),
        (wkv(2, 16), dense(96)),
        (wkv(4, 8), None),
        (latent(2, 24, 8, 16, 20, 0, base=500.0), dense(40))]),
    "Q": config(301, 96, 1, 3e-6, 97, (3, 11), [
        (wkv(3, 24), moe(3, 3, 40)),
        (latent(1, 32, 16, 48, 32, 5), dense(112)),
        (wkv(1, 40), moe(6, 1, 16, shared=8, scale=0.7))]),
    "R": config(400, 128, 4, 1e-6, 251, (17, 3), [
        (wkv(2, 64), dense(192)),
        (latent(4, 32, 32, 40, 96, 70), moe(8, 3, 32, shared=64, scale=2.0)),
        (latent(4, 32, 32, 40, 96, 70), dense(64))]),
}
PAGE = {"P": 16, "Q": 8, "R": 16}
LENGTHS = {"P": [5, 33, 70, 1, 47], "Q": [2, 40, 77, 23], "R": [150, 64, 90]}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp(f"fuvozen_{name}")
        write_random_model(cfg, str(d), seed=23 + i)
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


def plain_logits(model_dir, ids, decided=None):
    """``decided`` (a list) receives a mask of the rows at which no router made a close call (the last chosen score
    at least 5 % above the best one left out): bfloat16 may turn a close call, and nothing is asserted there."""
    cfg, weights = plain.read_model_folder(model_dir)
    gaps = []
    logits = plain.forward_logits(cfg, weights, ids, gaps=gaps)
    if decided is not None:
        decided.append(torch.stack(gaps).min(dim=0).values > 0.05 if gaps else torch.ones(len(ids), dtype=torch.bool))
    return logits


def close(got, want, dtype, what, bars=(3e-5, 6e-2), rows=None):
    """Every row within 3e-5 (float32) or 6e-2 (bfloat16) of its own spread (rows differ in size by orders of
    magnitude where one token is made to stand out), with a tenth of the overall spread as the floor.  ``rows``: a
    mask of the rows that are compared in bfloat16 (float32 compares all)."""
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, what
    assert torch.isfinite(got).all(), what
    want2, got2 = want.reshape(-1, want.shape[-1]), got.reshape(-1, want.shape[-1])
    floor = max(0.1 * float(want2.std()), 1e-3)
    scale = torch.clamp(want2.std(dim=-1), min=floor)
    err = (got2 - want2).abs().max(dim=-1).values / scale
    if rows is not None and dtype != "float32":
        assert int(rows.sum()) >= 0.7 * len(rows), f"{what}: too many close calls for the comparison to mean anything"
        err = torch.where(rows, err, torch.zeros_like(err))
    bar = bars[0] if dtype == "float32" else bars[1]
    worst = int(err.argmax())
    assert float(err[worst]) <= bar, f"{what}: row {worst} is off by {float(err[worst]):.3e} of its spread (bar {bar:.0e})"


def compare(model_dir, results, requests, dtype, what):
    for rid, ids in requests.items():
        decided = []
        want = plain_logits(model_dir, ids, decided)
        rows = sorted(p for (r, p) in results if r == rid)
        assert rows == list(range(len(ids))), f"{what}: request {rid} misses rows"
        close(torch.stack([results[(rid, p)] for p in rows]), want, dtype, f"{what} request {rid}", rows=decided[0])


def requests_for(name, seed=3):
    rng = random.Random(seed)
    return {f"r{i}": helpers.random_prompt(rng, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# ---- the plan -----------------------------------------------------------------------------------------------------
def test_plan_reads_every_size_from_the_configuration():
    typed, plan = resolve(CONFIGS["P"])
    assert plan.architecture == "Fuvozen" and plan.vocab_size == 211 and plan.hidden_size == 64
    kinds = [(g.kind, g.slots, g.head_dim, g.window, g.planes) for g in plan.cache_groups]
    # the previous token; rows of 48 under a window of 12; the two shapes of recurrent state; rows of 32 that keep everything
    assert kinds[0][:2] == ("state", 1)
    assert ("window", 1, 48, 12, 1) in kinds and ("full", 1, 32, 0, 1) in kinds
    assert sorted(g.state_shape for g in plan.cache_groups if g.kind == "state") == sorted([(1,), (2 * 16 * 16 + 64,), (4 * 8 * 8 + 64,)])
    assert [layer.feed_forward.kind if layer.feed_forward else None for layer in plan.layers] == \
        ["routed_experts", "xielu_mlp", None, "xielu_mlp"]
    # two layers of one shape share a group and take a slot each
    _typed, plan = resolve(CONFIGS["R"])
    group = [g for g in plan.cache_groups if g.kind == "window"]
    assert len(group) == 1 and group[0].slots == 2 and [e.cache_slot for e in plan.run] == [0, 0, 1]


def test_the_decay_rank_comes_from_the_checkpoint(tmp_path):
    cfg = CONFIGS["Q"]
    _typed, plan = resolve(cfg)
    from flexengine_b200.weights.random_init import checkpoint_tensors, random_tensor
    from flexengine_b200.weights.safetensors_io import write_safetensors
    import json
    tensors = dict(checkpoint_tensors(plan))
    tensors["l0.mix.w1"], tensors["l0.mix.w2"] = (5, 96), (72, 5)           # another rank than a random model's
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(tmp_path / "model.safetensors"), [(n, s, torch.bfloat16) for n, s in tensors.items()],
                      lambda n: random_tensor(plan, n, tensors[n], 1, torch.bfloat16))
    _cfg, _plan, model = load_model(str(tmp_path), "float32", "cpu")
    assert tuple(model.blocks[0].mixer.w1_weight.shape) == (5, 96)
    want = plain_logits(str(tmp_path), [3, 1, 4, 1, 5])
    cache = CacheManager(_plan.cache_groups, 4, 8, 1, torch.float32, "cpu")
    got = ModelRunner(model, cache, ops=kernel_refs).step([StepEntry("a", [3, 1, 4, 1, 5], [0, 1, 2, 3, 4])])
    close(got, want, "float32", "rank 5")


# ---- each mechanism alone -----------------------------------------------------------------------------------------
def step_context(device, dtype, cache, entries, ops):
    runner = ModelRunner.__new__(ModelRunner)                # only build_context is used
    runner.cache, runner.ops, runner.device = cache, ops, cache.device
    runner._ring, runner._ring_at, runner.h2d_bytes = [], 0, 0
    runner.model = types.SimpleNamespace(dtype=dtype)
    return runner.build_context([StepEntry(rid, [0] * n, []) for rid, n in entries])


def drive_mixer(mixer, group_spec, h, cuts, device, dtype, page=4, seats=2):
    """One mixer over a cache of its own, the sequence cut into ``cuts`` portions; a second request runs in between
    and ends, so that its seat and pages are used again."""
    ops = ops_for(device)
    cache = CacheManager([group_spec], 64, page, seats, dtype, device)
    outs, fed = [], 0
    for n in cuts:
        cache.reserve("r", fed + n)
        ctx = step_context(device, dtype, cache, [("r", n)], ops)
        outs.append(mixer.forward(ctx, h[fed:fed + n].to(device=device, dtype=dtype).contiguous(), RunEntry(0, 0, 0, True)).float().cpu())
        cache.commit("r", n)
        fed += n
        if fed == cuts[0]:                                   # a neighbour that comes and goes
            cache.reserve("other", 7)
            ctx = step_context(device, dtype, cache, [("other", 7)], ops)
            mixer.forward(ctx, torch.randn(7, h.shape[1]).to(device=device, dtype=dtype), RunEntry(0, 0, 0, True))
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


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("groups", [1, 2, 5])
def test_group_norm_alone(device, dtype, groups):
    torch.manual_seed(1)
    dt = getattr(torch, dtype)
    norm = build_part("norm", PartSpec("group_rmsnorm", {"hidden_size": 80, "eps": 3e-6, "groups": groups}))
    w = 1 + 0.1 * torch.randn(80)
    norm.bind({"weight": w.to(device)})
    residual, delta = torch.randn(6, 80), bf16_exact(torch.randn(6, 80))
    want = plain.group_rms_norm(residual + delta, w, groups, 3e-6)
    ctx = types.SimpleNamespace(ops=ops_for(device), dtype=dt)
    stream = residual.clone().to(device)
    close(norm.forward(ctx, stream, delta.to(device=device, dtype=dt)), want, dtype, "norm")
    torch.testing.assert_close(stream.cpu(), residual + delta)
    rows = torch.tensor([5, 2], dtype=torch.int32, device=device)
    close(norm.forward(ctx, stream, None, rows=rows), want[[5, 2]], dtype, "rows")


@pytest.mark.parametrize("device", DEVICES)
def test_hashed_pair_embedding_alone(device):
    """Portions of two requests in one step, then their next portions: the token before a portion's first token comes
    from the seat; a request that starts at position 0 takes the table's last row whatever its seat held."""
    torch.manual_seed(2)
    cfg = {"vocab": 50, "embedding": {"bigram": {"buckets": 37, "mul_prev": 31, "mul_cur": 7}}}
    weights = {"embed": bf16_exact(torch.randn(50, 24)), "bigram": bf16_exact(torch.randn(38, 24))}
    part = build_part("embedding", PartSpec("hashed_pairs", {"vocab_size": 50, "hidden_size": 24, "buckets": 37, "mul_prev": 31,
                                                              "mul_cur": 7, "state_group": 0}))
    part.bind({"weight": weights["embed"].to(device), "pairs.weight": weights["bigram"].to(device)})
    spec = CacheGroupSpec("previous", "state", slots=1, state_shape=(1,), state_dtype="int32")
    cache = CacheManager([spec], 1, 4, 2, torch.float32, device)
    ids = {"a": torch.randint(0, 50, (9,)), "b": torch.randint(0, 50, (6,)), "c": torch.randint(0, 50, (3,))}
    want = {k: plain.bigram_embedding(cfg, weights, v) for k, v in ids.items()}
    got = {k: [] for k in ids}
    for step in ([("a", 4), ("b", 1)], [("b", 5), ("a", 1)], [("a", 4)], "free b", [("c", 3)]):
        if step == "free b":
            cache.free("b")                                  # c takes b's seat, which still holds b's last token
            continue
        for rid, _ in step:
            cache.admit(rid)
        ctx = step_context(device, torch.float32, cache, step, ops_for(device))
        tokens = torch.cat([ids[rid][len(got[rid]):len(got[rid]) + n] for rid, n in step]).to(torch.int32).to(device)
        ctx.token_ids = tokens
        out = part.forward(ctx).cpu()
        at = 0
        for rid, n in step:
            got[rid] += list(out[at:at + n])
            cache.commit(rid, n)
            at += n
    for k in ids:
        torch.testing.assert_close(torch.stack(got[k]), want[k], atol=1e-6, rtol=0)


@pytest.mark.parametrize("device,dtype", CASES)
def test_dense_feed_forward_alone(device, dtype):
    torch.manual_seed(3)
    dt = getattr(torch, dtype)
    weights = {"up": bf16_exact(torch.randn(56, 40) * 0.3), "down": bf16_exact(torch.randn(40, 56) * 0.3), "act": torch.tensor([0.4, -0.3])}
    part = build_part("feed_forward", PartSpec("xielu_mlp", {"hidden_size": 40, "intermediate_size": 56}))
    bind_by_checkpoint_names(part, weights, "", {"up.weight": ["up"], "down.weight": ["down"], "act": ["act"]}, device, dt)
    h = bf16_exact(torch.randn(9, 40))
    got = part.forward(types.SimpleNamespace(ops=ops_for(device), dtype=dt), h.to(device=device, dtype=dt))
    close(got, plain.dense_ffn(h, weights, ""), dtype, "xielu mlp")
    z = torch.linspace(-6, 6, 25)
    torch.testing.assert_close(plain.xielu(z, torch.tensor(0.4), torch.tensor(-0.3))[12], torch.tensor(0.0))


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("experts,top,shared,D,F", [(5, 2, 16, 48, 24), (3, 3, 0, 48, 24), (70, 1, 8, 48, 24), (4, 2, 12, 44, 20),
                                                     (6, 2, 0, 136, 72), (3, 2, 0, 1024, 1032)])
def test_routed_feed_forward_alone(device, dtype, experts, top, shared, D, F):
    """Also widths that are no multiples of 8 (rows off 16-byte boundaries), tiles with edges on every side, and a size
    at which the bfloat16 products take the grouped tcgen05 GEMM (1,280 sorted rows, experts of 1,024 x 1,032)."""
    torch.manual_seed(4)
    dt = getattr(torch, dtype)
    T = 70 if D < 100 else (300 if D < 1024 else 640)
    spread = 0.2 * (48 / D) ** 0.5                     # outputs of about the same size whatever the width
    weights = {"router": torch.randn(experts, D) * (48 / D) ** 0.5}          # logits of a few units whatever the width
    names = {"router.weight": ["router"], "experts.gate_up.weight": [], "experts.down.weight": []}
    for e in range(experts):
        for which, shape in (("gate", (F, D)), ("up", (F, D)), ("down", (D, F))):
            weights[f"e{e}.{which}"] = bf16_exact(torch.randn(*shape) * spread)
        names["experts.gate_up.weight"] += [f"e{e}.gate", f"e{e}.up"]
        names["experts.down.weight"].append(f"e{e}.down")
    spec = {"router": {"experts": experts, "top": top, "scale": 1.7}}
    if shared:
        for which, shape in (("gate", (shared, D)), ("up", (shared, D)), ("down", (D, shared))):
            weights[f"shared.{which}"] = bf16_exact(torch.randn(*shape) * spread)
        names.update({"shared.gate_up.weight": ["shared.gate", "shared.up"], "shared.down.weight": ["shared.down"]})
        spec["shared"] = {"ff": shared}
    part = build_part("feed_forward", PartSpec("routed_experts", {"hidden_size": D, "experts": experts, "top": top, "expert_size": F,
                                                                  "scale": 1.7, "shared_size": shared}))
    bind_by_checkpoint_names(part, weights, "", names, device, dt)
    h = bf16_exact(torch.randn(T, D))
    got = part.forward(types.SimpleNamespace(ops=ops_for(device), dtype=dt), h.to(device=device, dtype=dt))
    close(got, plain.moe_ffn(h, weights, "", spec), dtype, "routed experts")
    # a token's output does not depend on its neighbours in the step
    alone = part.forward(types.SimpleNamespace(ops=ops_for(device), dtype=dt), h[11:12].to(device=device, dtype=dt))
    close(alone, got[11:12], dtype, "one token")


def wkv_weights(D, H, d, rank, seed, slow_decay=False):
    g = torch.Generator().manual_seed(seed)
    inner = H * d
    w = {f"mu.{s}": torch.rand(D, generator=g) for s in "rkvgw"}
    for s in "rkvg":
        w[s] = bf16_exact(torch.randn(inner, D, generator=g) / D ** 0.5)
    w["w1"] = torch.randn(rank, D, generator=g) / D ** 0.5
    w["w2"] = torch.randn(inner, rank, generator=g) / rank ** 0.5
    w["w0"] = torch.full((inner,), -7.0) if slow_decay else torch.randn(inner, generator=g) - 1.0
    w["u"] = torch.randn(H, d, generator=g) * 0.3
    w["norm"] = 1 + 0.1 * torch.randn(inner, generator=g)
    w["o"] = bf16_exact(torch.randn(D, inner, generator=g) / inner ** 0.5)
    return w


WKV_NAMES = {"mu": ["mu.r", "mu.k", "mu.v", "mu.g", "mu.w"], "r.weight": ["r"], "k.weight": ["k"], "v.weight": ["v"], "g.weight": ["g"],
             "w1.weight": ["w1"], "w2.weight": ["w2"], "w0": ["w0"], "u": ["u"], "norm.weight": ["norm"], "o.weight": ["o"]}


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("heads,dim", [(2, 16), (1, 64), (3, 24)])
def test_wkv_mixer_alone(device, dtype, heads, dim):
    """Whole, token by token, and in portions down to two tokens: the state and the last row are carried by the seat."""
    dt = getattr(torch, dtype)
    D, rank, T = 40, 6, 37
    weights = wkv_weights(D, heads, dim, rank, seed=5)
    mixer = build_part("mixer", PartSpec("wkv", {"hidden_size": D, "heads": heads, "dim": dim, "decay_rank": rank, "eps": 1e-5}))
    bind_by_checkpoint_names(mixer, weights, "", WKV_NAMES, device, dt)
    need = mixer.cache_need()
    spec = CacheGroupSpec("state", "state", slots=1, state_shape=need["state_shape"], state_dtype=need["state_dtype"])
    h = bf16_exact(torch.randn(T, D, generator=torch.Generator().manual_seed(6)))
    want = plain.wkv_mixer(h, weights, "", {"heads": heads, "dim": dim}, 1e-5)
    for cuts in ([T], [1] * T, [5, 2, 17, 2, 1, 10], [2, 33, 2]):
        close(drive_mixer(mixer, spec, h, cuts, device, dt), want, dtype, f"wkv cut {cuts[:4]}")


@pytest.mark.parametrize("device,dtype", CASES)
def test_wkv_remembers_over_hundreds_of_tokens(device, dtype):
    """A decay close to one: what token 3 wrote into the state still decides the output 300 tokens later, through
    portions and single tokens.  A state that is lost, zeroed or mixed up between seats shows at once."""
    dt = getattr(torch, dtype)
    D, heads, dim, rank, T = 32, 2, 16, 4, 320
    weights = wkv_weights(D, heads, dim, rank, seed=7, slow_decay=True)
    weights["w2"] *= 0.01
    mixer = build_part("mixer", PartSpec("wkv", {"hidden_size": D, "heads": heads, "dim": dim, "decay_rank": rank, "eps": 1e-5}))
    bind_by_checkpoint_names(mixer, weights, "", WKV_NAMES, device, dt)
    spec = CacheGroupSpec("state", "state", slots=1, state_shape=mixer.cache_need()["state_shape"])
    h = bf16_exact(torch.randn(T, D, generator=torch.Generator().manual_seed(8)) * 0.1)
    h[3] = bf16_exact(torch.randn(D, generator=torch.Generator().manual_seed(9)) * 4.0)      # the one that is remembered
    want = plain.wkv_mixer(h, weights, "", {"heads": heads, "dim": dim}, 1e-5)
    silent = h.clone()
    silent[3] = h[2]
    assert (plain.wkv_mixer(silent, weights, "", {"heads": heads, "dim": dim}, 1e-5)[-1] - want[-1]).abs().max() > 0.1 * want[-1].abs().max()
    got = drive_mixer(mixer, spec, h, [2, 60, 130, 2, 100] + [1] * 26, device, dt)
    # hundreds of roundings add up in a state that forgets nothing: wider bars, still far below a lost state's error
    close(got, want, dtype, "far memory", bars=(2e-4, 0.25))


def latent_weights(D, m, seed):
    g = torch.Generator().manual_seed(seed)
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    return {"q": bf16_exact(torch.randn(H * (dn + dr), D, generator=g) / D ** 0.5),
            "dkv": bf16_exact(torch.randn(rank + dr, D, generator=g) / D ** 0.5),
            "dkv.norm": 1 + 0.1 * torch.randn(rank, generator=g),
            "uk": bf16_exact(torch.randn(H * dn, rank, generator=g) / rank ** 0.5),
            "uv": bf16_exact(torch.randn(H * dv, rank, generator=g) / rank ** 0.5),
            "o": bf16_exact(torch.randn(D, H * dv, generator=g) / (H * dv) ** 0.5)}


LATENT_NAMES = {"q.weight": ["q"], "dkv.weight": ["dkv"], "dkv_norm.weight": ["dkv.norm"], "uk.weight": ["uk"], "uv.weight": ["uv"],
                "o.weight": ["o"]}


def latent_mixer(D, m, weights, device, dt):
    mixer = build_part("mixer", PartSpec("latent_attention", {
        "hidden_size": D, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
        "scale": m["scale"], "eps": 1e-5, "window": m.get("mask", {}).get("size", 0), "rot_base": m["rot"]["base"],
        "rot_dims": m["rot"]["dims"]}))
    bind_by_checkpoint_names(mixer, weights, "", LATENT_NAMES, device, dt)
    need = mixer.cache_need()
    spec = CacheGroupSpec("rows", need["kind"], slots=1, kv_heads=1, head_dim=need["head_dim"], window=need["window"], planes=1)
    return mixer, spec


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", [(3, 16, 8, 24, 40, 12), (1, 32, 16, 8, 20, 0), (4, 32, 32, 40, 96, 21), (5, 8, 4, 8, 12, 3),
                                   (2, 16, 16, 24, 272, 9), (20, 16, 8, 8, 24, 14)])      # a row beyond 256; more heads than a decode group takes
def test_latent_attention_alone(device, dtype, shape):
    dt = getattr(torch, dtype)
    D, T = 48, 41
    m = latent(*shape)["mixer"]
    weights = latent_weights(D, m, seed=10)
    mixer, spec = latent_mixer(D, m, weights, device, dt)
    h = bf16_exact(torch.randn(T, D, generator=torch.Generator().manual_seed(11)))
    want = plain.latent_attention(h, weights, "", m, 1e-5)
    for cuts in ([T], [1] * T, [7, 2, 19, 2, 1, 10], [2, 37, 2]):
        close(drive_mixer(mixer, spec, h, cuts, device, dt), want, dtype, f"latent attention {shape} cut {cuts[:4]}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("distance", [0, 1, 11, 12, 13, 200])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_key_that_stands_out_at_the_windows_edge(device, dtype, distance, decoded):
    """One key gets a large entry in the slowest rotated pair (which barely turns) and the last query a large entry
    in the same place, so that this key takes all the weight whenever it is visible: with a window of 12, at distances
    0, 1 and 11 and not at 12, 13 or 200.  The key lies on a page border (position 16) of pages of 4."""
    dt = getattr(torch, dtype)
    D, window = 32, 12
    m = latent(2, 16, 8, 16, 24, window, base=1e7, scale=0.3)["mixer"]
    weights = latent_weights(D, m, seed=12)
    rank, dn, dr = m["kv_rank"], m["dim"], m["rot_dim"]
    marker_k, marker_q = torch.zeros(D), torch.zeros(D)
    marker_k[5], marker_q[9] = 1.0, 1.0
    weights["dkv"][:, 5] = 0.0
    weights["q"][:, 9] = 0.0
    weights["dkv"][rank + dr - 2] = 8.0 * marker_k               # the key's slow pair reads channel 5
    for head in range(m["heads"]):
        weights["q"][head * (dn + dr) + dn + dr - 2] = 8.0 * marker_q
    mixer, spec = latent_mixer(D, m, weights, device, dt)
    key_at, T = 16, 16 + distance + 1
    h = bf16_exact(torch.randn(T, D, generator=torch.Generator().manual_seed(13)))
    h[:, 5], h[:, 9] = 0.0, 0.0
    h[key_at, 5] = 4.0
    h[-1, 9] = 4.0
    want = plain.latent_attention(h, weights, "", m, 1e-5)
    blind = h.clone()
    blind[key_at, 5] = 0.0
    differs = (plain.latent_attention(blind, weights, "", m, 1e-5)[-1] - want[-1]).abs().max() > 0.05 * want[-1].abs().max()
    assert bool(differs) == (distance < window)
    cuts = [T - 1, 1] if decoded else ([T] if distance < 3 else [T - 2, 2])
    if distance == 0 and decoded:
        cuts = [T - 1, 1]
    close(drive_mixer(mixer, spec, h, cuts, device, dt), want, dtype, f"distance {distance}")


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


STACKS = {
    "only the recurrence": config(97, 48, 3, 1e-5, 31, (5, 3), [(wkv(2, 24), dense(64)), (wkv(3, 16), moe(4, 2, 16))]),
    "only attention": config(97, 48, 1, 1e-5, 31, (5, 3), [(latent(2, 16, 8, 16, 24, 6), None), (latent(2, 16, 8, 16, 24, 6), dense(32))]),
    "one layer": config(50, 32, 2, 1e-5, 7, (1, 1), [(wkv(1, 32), None)]),
}


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("stack", list(STACKS))
def test_stacks_of_one_kind(tmp_path, stack, device, dtype):
    """A model without paged groups, one without recurrent state, and one of a single layer without a feed-forward."""
    cfg = STACKS[stack]
    write_random_model(cfg, str(tmp_path), seed=3)
    ids = helpers.random_prompt(random.Random(1), 45, cfg["vocab"])
    runner = make_runner(str(tmp_path), dtype, device, 8, 8)
    got = [runner.step([StepEntry("a", ids[:20], list(range(20)))]), runner.step([StepEntry("a", ids[20:44], list(range(24)))]),
           runner.step([StepEntry("a", ids[44:], [0])])]
    decided = []
    want = plain_logits(str(tmp_path), ids, decided)
    close(torch.cat([g.float().cpu() for g in got]), want, dtype, stack, rows=decided[0])
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
    """A prompt of one token, then 150 tokens decoded one by one beside a neighbour that arrives later: every row
    against the whole sequence.  The window (12) and the pages pass many times; the window group gives pages back."""
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
    decided = []
    close(torch.stack(rows), plain_logits(model_dirs[name], ids, decided), dtype, "long decoding", rows=decided[0])
    close(torch.stack(other_rows), plain_logits(model_dirs[name], other, decided), dtype, "the neighbour", rows=decided[1])
    window_group = [g for _, g in runner.cache.paged if g.spec.kind == "window"][0]
    assert window_group.pool.used_pages <= 2                 # 151 tokens under a window of 12 in pages of 16


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
    import json, os, subprocess, sys
    import numpy as np
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
