"""Fuvuvik as a plan of parts: a decoder over several residual streams ("hyper-connections").  Every sublayer reads a
learned sum of the streams through an RMSNorm, its output is multiplied by a sigmoid gate of the same normalised rows and
written into all streams while they are mixed among themselves; the mixer reads its rows blended with the row before.
Mixers, in an order the configuration gives: grouped-query attention with short causal convolutions after the
projections and unit-normed queries and keys ("attention"); attention inside chunks of positions with one added to the
softmax's denominator ("attention_2"); a minGRU recurrence ("mingru").  Both attentions rotate the first ``rot.dims``
entries of a head and gate every head's output.  The feed-forward is gated with the tanh form of GELU.

Checkpoint names: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.rg1|rg2`` (+ ``.b``), ``l<i>.shift``, ``l<i>.mix.*`` and ``l<i>.mlp.gate|up|down``.  Matrices are [out, in].
The projections of a mixer that read the same rows are bound as one matrix (q, k, v and the head gate; z, x and g of the
recurrence; gate and up), the three convolutions as one table.

Cache groups: one float32 state group with a slot per layer for the row the token shift keeps; a paged group per
distinct (key/value heads, head size, visibility) of the attention layers (head size: the larger of the query/key and
the value size, in steps of 16; the smaller is padded with zeros); a float32 state group per distinct shape of
convolution history and per distinct width of the recurrence.
"""
from __future__ import annotations

import math
from dataclasses import replace

from ..config.fuvuvik_config import FuvuvikConfig, GatedAttentionConfig
from ..config.registry import register_architecture
from ..parts.spec import (CacheGroupSpec, LayerSpec, ModelPlan, PartSpec, RunEntry, WeightBinding, WeightSource)

SHIFT_GROUP = 0


def build_fuvuvik_plan(cfg: FuvuvikConfig) -> ModelPlan:
    D, V, S = cfg.width, cfg.vocab, cfg.streams
    norm = PartSpec("stream_rmsnorm", {"hidden_size": D, "eps": cfg.norm_eps, "streams": S})
    groups = [CacheGroupSpec(name="token_shift", kind="state", slots=len(cfg.layers), state_shape=(D,), state_dtype="float32")]
    group_of: dict = {}            # key -> [group index, slots so far]
    layers, run, bindings = [], [], []
    init = {}

    def src(name, *shape, rule=None):
        fan_in = shape[-1] if len(shape) > 1 else 1
        init[name] = rule or ("normal", 0.0, 1.0 / math.sqrt(max(fan_in, 1)))
        return WeightSource(name, tuple(shape))

    def slot_in(key, need):
        """(group index, slot) of one more slot in the group of ``key``, made from ``need`` at first use."""
        if key not in group_of:
            group_of[key] = [len(groups), 0]
            groups.append(need)
        gi, slot = group_of[key]
        group_of[key][1] += 1
        return gi, slot

    near_one = ("normal", 1.0, 0.1)
    bindings += [WeightBinding(("embedding", "weight"), (src("embed", V, D, rule=("normal", 0.0, 1.0)),)),
                 WeightBinding(("final_norm", "weight"), (src("final.norm", D, rule=near_one),), kind="vector"),
                 WeightBinding(("lm_head", "weight"), (src("head", V, D),))]
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer

        def target(part, local):
            return ("layer", i, part, local)

        if isinstance(m, GatedAttentionConfig):
            head = -(-max(m.dim, m.vdim) // 16) * 16
            kind = {"full": "full", "chunk": "chunk"}[m.mask]
            gi, slot = slot_in(("paged", m.kv_heads, head, kind, m.mask_size),
                               CacheGroupSpec(name=f"attention_{m.kv_heads}x{head}_{kind}{m.mask_size or ''}", kind=kind, slots=0,
                                              kv_heads=m.kv_heads, head_dim=head, window=m.mask_size))
            channels = (m.heads + m.kv_heads) * m.dim + m.kv_heads * m.vdim
            params = {"hidden_size": D, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                      "rot_base": m.rot_base, "rot_dims": m.rot_dims, "conv": m.conv, "qk_norm": m.qk_norm, "eps": cfg.norm_eps,
                      "mask": m.mask, "mask_size": m.mask_size, "sink": m.sink}
            bindings += [
                WeightBinding(target("mixer", "qkvg.weight"),
                              (src(p + "mix.q", m.heads * m.dim, D), src(p + "mix.k", m.kv_heads * m.dim, D),
                               src(p + "mix.v", m.kv_heads * m.vdim, D), src(p + "mix.g", m.heads, D))),
                WeightBinding(target("mixer", "o.weight"), (src(p + "mix.o", D, m.heads * m.vdim),)),
            ]
            if m.conv > 0:
                # the history of a convolution of ``conv`` taps: the last conv - 1 projected rows of every request
                cg, cs = slot_in(("conv", m.conv - 1, channels),
                                 CacheGroupSpec(name=f"conv_history_{m.conv - 1}x{channels}", kind="state", slots=0,
                                                state_shape=((m.conv - 1) * channels,), state_dtype="float32"))
                params.update(conv_group=cg, conv_slot=cs)
                taps = ("normal", 1.0 / m.conv, 0.5 / m.conv)
                bindings.append(WeightBinding(target("mixer", "conv.weight"),
                                              (src(p + "mix.q.conv", m.heads * m.dim, m.conv, rule=taps),
                                               src(p + "mix.k.conv", m.kv_heads * m.dim, m.conv, rule=taps),
                                               src(p + "mix.v.conv", m.kv_heads * m.vdim, m.conv, rule=taps)), kind="vector"))
            mixer = PartSpec("gated_attention", params)
        else:
            W = m.width
            gi, slot = slot_in(("mingru", W), CacheGroupSpec(name=f"mingru_state_{W}", kind="state", slots=0,
                                                             state_shape=(W,), state_dtype="float32"))
            mixer = PartSpec("mingru", {"hidden_size": D, "width": W})
            bias = ("normal", 0.0, 0.5)
            bindings += [
                WeightBinding(target("mixer", "zxg.weight"), (src(p + "mix.z", W, D), src(p + "mix.x", W, D), src(p + "mix.g", W, D))),
                WeightBinding(target("mixer", "zx.bias"), (src(p + "mix.z.b", W, rule=bias), src(p + "mix.x.b", W, rule=bias)), kind="vector"),
                WeightBinding(target("mixer", "o.weight"), (src(p + "mix.o", D, W),)),
            ]
        run.append(RunEntry(layer=i, cache_group=gi, cache_slot=slot, write_cache=True))

        feed_forward = None
        if layer.mlp is not None:
            f = layer.mlp.ff
            feed_forward = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": f, "activation": "gelu_tanh"})
            bindings += [
                WeightBinding(target("feed_forward", "gate_up.weight"), (src(p + "mlp.gate", f, D), src(p + "mlp.up", f, D))),
                WeightBinding(target("feed_forward", "down.weight"), (src(p + "mlp.down", D, f),)),
            ]
        for q in ("1", "2") if feed_forward is not None else ("1",):
            bindings += [
                WeightBinding(target("norm" + q, "weight"), (src(p + "norm" + q, D, rule=near_one),), kind="vector"),
                WeightBinding(target("hc" + q, "read"), (src(p + f"hc{q}.in", S, rule=("normal", 1.0 / S, 0.3 / S)),), kind="vector"),
                WeightBinding(target("hc" + q, "write"), (src(p + f"hc{q}.out", S, rule=("normal", 1.0, 0.2)),), kind="vector"),
                WeightBinding(target("hc" + q, "mix"), (src(p + f"hc{q}.mix", S, S, rule=("normal", 1.0 / S, 0.3 / S)),), kind="vector"),
                WeightBinding(target("rg" + q, "weight"), (src(p + "rg" + q, D, D),)),
                WeightBinding(target("rg" + q, "bias"), (src(p + f"rg{q}.b", D, rule=("normal", 0.5, 0.5)),), kind="vector"),
            ]
        bindings.append(WeightBinding(target("shift", "mu"), (src(p + "shift", D, rule=("normal", 0.5, 0.2)),), kind="vector"))
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, norm=norm, block="hyper_gated",
                                block_params={"streams": S, "hidden_size": D, "shift_group": SHIFT_GROUP, "shift_slot": i}))

    counts = {gi: n for gi, n in group_of.values()}
    groups = [replace(g, slots=counts[gi]) if gi in counts else g for gi, g in enumerate(groups)]
    embedding = PartSpec("token_table", {"vocab_size": V, "hidden_size": D, "scale": cfg.embedding_scale, "streams": S})
    return ModelPlan(architecture=FuvuvikConfig.ARCHITECTURE, vocab_size=V, hidden_size=D, layers=layers, run=run,
                     cache_groups=groups, final_norm=norm, bindings=bindings, embedding=embedding,
                     head=PartSpec("linear", {"vocab_size": V, "hidden_size": D}),
                     eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id,
                     init={"default": ("normal", 0.0, 0.02), "suffix": init})


register_architecture(FuvuvikConfig.ARCHITECTURE, FuvuvikConfig, build_fuvuvik_plan)
