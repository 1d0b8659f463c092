"""Fuvozen as a plan of parts: a decoder whose layers alternate, in an order the configuration gives, between a
linear-recurrent mixer ("wkv") and attention over a cached latent with a sliding window ("latent_attention"),
each beside a dense or a routed feed-forward under one grouped RMSNorm, with a learned average over depth after
every layer, a hashed pair table added to the token embedding, and logits from the embedding table.

Checkpoint names: ``embed``, ``bigram``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.dwa``,
``l<i>.mix.*`` and ``l<i>.mlp.*`` (experts ``e<k>.gate|up|down``, ``router``, ``shared.*``).  Matrices are
[out, in].  The five blend vectors ``mu.r|k|v|g|w`` are bound as one tensor, an expert's gate and up as one
matrix, and all experts of a layer as one.

Cache groups: one int32 state group for the previous token of every request (the pair table's key); a float32
state group per distinct (heads, dim) of the wkv layers; a one-plane paged group per distinct
(row width, window) of the latent-attention layers.
"""
from __future__ import annotations

import math
from dataclasses import replace

from ..config.fuvozen_config import DenseMlpConfig, FuvozenConfig, MoeMlpConfig
from ..config.registry import register_architecture
from ..parts.spec import (CacheGroupSpec, LayerSpec, ModelPlan, PartSpec, RunEntry, WeightBinding, WeightSource)


def build_fuvozen_plan(cfg: FuvozenConfig, decay_ranks=None) -> ModelPlan:
    """``decay_ranks``: {layer: rank of its decay's low-rank projection}; a checkpoint gives it by the shape of
    ``l<i>.mix.w1`` (see ``plan_for_checkpoint``), a random model takes the default."""
    D, V = cfg.width, cfg.vocab
    norm = PartSpec("group_rmsnorm", {"hidden_size": D, "eps": cfg.norm_eps, "groups": cfg.norm_groups})
    groups = [CacheGroupSpec(name="previous_token", kind="state", slots=1, state_shape=(1,), state_dtype="int32")]
    group_of: dict = {}            # key -> [group index, slots so far]
    layers, run, bindings = [], [], []
    init = {}

    def src(name, *shape, rule=None):
        fan_in = shape[-1] if len(shape) > 1 else 1
        init[name] = rule or ("normal", 0.0, 1.0 / math.sqrt(max(fan_in, 1)))
        return WeightSource(name, tuple(shape))

    near_one = ("normal", 1.0, 0.1)
    bindings += [WeightBinding(("embedding", "weight"), (src("embed", V, D, rule=("normal", 0.0, 1.0)),)),
                 WeightBinding(("embedding", "pairs.weight"),
                               (src("bigram", cfg.bigram_buckets + 1, D, rule=("normal", 0.0, 0.7)),)),
                 WeightBinding(("final_norm", "weight"), (src("final.norm", D, rule=near_one),), kind="vector"),
                 WeightBinding(("lm_head", "weight"), alias_of=("embedding", "weight"))]
    total = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "wkv":
            rank = (decay_ranks or {}).get(i, min(64, max(8, m.heads * m.dim // 8)))
            mixer = PartSpec("wkv", {"hidden_size": D, "heads": m.heads, "dim": m.dim, "decay_rank": rank, "eps": cfg.norm_eps})
            inner = m.heads * m.dim
            key = ("wkv", m.heads, m.dim)
            need = CacheGroupSpec(name=f"wkv_state_{m.heads}x{m.dim}", kind="state", slots=0,
                                  state_shape=(m.heads * m.dim * m.dim + D,), state_dtype="float32")
            between = ("normal", 0.5, 0.2)
            bindings += [
                WeightBinding(("layer", i, "mixer", "mu"),
                              tuple(src(p + "mix.mu." + s, D, rule=between) for s in ("r", "k", "v", "g", "w")), kind="vector"),
                *[WeightBinding(("layer", i, "mixer", s + ".weight"), (src(p + "mix." + s, inner, D),)) for s in ("r", "k", "v", "g")],
                WeightBinding(("layer", i, "mixer", "w1.weight"), (src(p + "mix.w1", rank, D),), kind="float32"),
                WeightBinding(("layer", i, "mixer", "w2.weight"), (src(p + "mix.w2", inner, rank),), kind="float32"),
                WeightBinding(("layer", i, "mixer", "w0"), (src(p + "mix.w0", inner, rule=("normal", -1.0, 0.7)),), kind="vector"),
                WeightBinding(("layer", i, "mixer", "u"), (src(p + "mix.u", m.heads, m.dim, rule=("normal", 0.3, 0.3)),), kind="vector"),
                WeightBinding(("layer", i, "mixer", "norm.weight"), (src(p + "mix.norm", inner, rule=near_one),), kind="vector"),
                WeightBinding(("layer", i, "mixer", "o.weight"), (src(p + "mix.o", D, inner),)),
            ]
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                "scale": m.scale, "eps": cfg.norm_eps, "window": m.window, "rot_base": m.rot_base, "rot_dims": m.rot_dims})
            row = -(-(m.kv_rank + m.rot_dim) // 16) * 16
            key = ("latent", row, m.window)
            need = CacheGroupSpec(name=f"latent_{row}_window_{m.window}", kind="window" if m.window > 0 else "full", slots=0,
                                  kv_heads=1, head_dim=row, window=m.window, planes=1)
            bindings += [
                WeightBinding(("layer", i, "mixer", "q.weight"), (src(p + "mix.q", m.heads * (m.dim + m.rot_dim), D),)),
                WeightBinding(("layer", i, "mixer", "dkv.weight"), (src(p + "mix.dkv", m.kv_rank + m.rot_dim, D),)),
                WeightBinding(("layer", i, "mixer", "dkv_norm.weight"), (src(p + "mix.dkv.norm", m.kv_rank, rule=near_one),), kind="vector"),
                WeightBinding(("layer", i, "mixer", "uk.weight"), (src(p + "mix.uk", m.heads * m.dim, m.kv_rank),)),
                WeightBinding(("layer", i, "mixer", "uv.weight"), (src(p + "mix.uv", m.heads * m.vdim, m.kv_rank),)),
                WeightBinding(("layer", i, "mixer", "o.weight"), (src(p + "mix.o", D, m.heads * m.vdim),)),
            ]
        if key not in group_of:
            group_of[key] = [len(groups), 0]
            groups.append(need)
        gi, slot = group_of[key]
        group_of[key][1] += 1
        run.append(RunEntry(layer=i, cache_group=gi, cache_slot=slot, write_cache=True))

        mlp = layer.mlp
        if mlp is None:
            feed_forward = None
        elif isinstance(mlp, DenseMlpConfig):
            feed_forward = PartSpec("xielu_mlp", {"hidden_size": D, "intermediate_size": mlp.ff})
            bindings += [
                WeightBinding(("layer", i, "feed_forward", "up.weight"), (src(p + "mlp.up", mlp.ff, D),)),
                WeightBinding(("layer", i, "feed_forward", "down.weight"), (src(p + "mlp.down", D, mlp.ff),)),
                WeightBinding(("layer", i, "feed_forward", "act"), (src(p + "mlp.act", 2, rule=("normal", 0.3, 0.5)),), kind="vector"),
            ]
        else:
            assert isinstance(mlp, MoeMlpConfig)
            f = mlp.expert_ff
            feed_forward = PartSpec("routed_experts", {"hidden_size": D, "experts": mlp.experts, "top": mlp.top, "expert_size": f,
                                                       "scale": mlp.scale, "shared_size": mlp.shared_ff})
            gate_up = tuple(src(f"{p}mlp.e{e}.{which}", f, D) for e in range(mlp.experts) for which in ("gate", "up"))
            bindings += [
                WeightBinding(("layer", i, "feed_forward", "router.weight"), (src(p + "mlp.router", mlp.experts, D),), kind="float32"),
                WeightBinding(("layer", i, "feed_forward", "experts.gate_up.weight"), gate_up),
                WeightBinding(("layer", i, "feed_forward", "experts.down.weight"),
                              tuple(src(f"{p}mlp.e{e}.down", D, f) for e in range(mlp.experts))),
            ]
            if mlp.shared_ff:
                s = mlp.shared_ff
                bindings += [
                    WeightBinding(("layer", i, "feed_forward", "shared.gate_up.weight"),
                                  (src(p + "mlp.shared.gate", s, D), src(p + "mlp.shared.up", s, D))),
                    WeightBinding(("layer", i, "feed_forward", "shared.down.weight"), (src(p + "mlp.shared.down", D, s),)),
                ]
        # the average over depth starts near "take the newest stream"
        bindings.append(WeightBinding(("layer", i, "depth_average", "weight"),
                                      (src(p + "dwa", i + 2, rule=("normal", 1.0 / (i + 2), 0.3)),), kind="vector"))
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, norm=norm, block="parallel_depth_average",
                                block_params={"depth": i, "total": total}))
        bindings.append(WeightBinding(("layer", i, "norm", "weight"), (src(p + "norm1", D, rule=near_one),), kind="vector"))

    counts = {gi: n for gi, n in group_of.values()}
    groups = [replace(g, slots=counts[gi]) if gi in counts else g for gi, g in enumerate(groups)]
    embedding = PartSpec("hashed_pairs", {"vocab_size": V, "hidden_size": D, "buckets": cfg.bigram_buckets,
                                          "mul_prev": cfg.bigram_mul_prev, "mul_cur": cfg.bigram_mul_cur, "state_group": 0})
    return ModelPlan(architecture=FuvozenConfig.ARCHITECTURE, vocab_size=V, hidden_size=D, layers=layers, run=run,
                     cache_groups=groups, final_norm=norm, bindings=bindings, embedding=embedding,
                     head=PartSpec("linear", {"vocab_size": V, "hidden_size": D}),
                     eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id,
                     init={"default": ("normal", 0.0, 0.02), "suffix": init})


def plan_for_checkpoint(cfg: FuvozenConfig, shapes) -> ModelPlan:
    """The plan for a checkpoint whose tensor shapes are ``shapes`` {name: shape}: sizes that only a tensor's shape
    gives (the rank of a decay's projection) are read from there."""
    ranks = {}
    for i, layer in enumerate(cfg.layers):
        shape = shapes.get(f"l{i}.mix.w1")
        if layer.type == "wkv" and shape is not None and len(shape) == 2:
            ranks[i] = int(shape[0])
    return build_fuvozen_plan(cfg, ranks)


register_architecture(FuvozenConfig.ARCHITECTURE, FuvozenConfig, build_fuvozen_plan, refine=plan_for_checkpoint)
