"""A minGRU mixer: a gated recurrence whose gates read only the current token.

    z = sigmoid(W_z h + b_z);   u = W_x h + b_x;   c = u + 1/2 where u >= 0, sigmoid(u) where u < 0;
    S_t = (1 - z) S_(t-1) + z c   (element by element, ``width`` channels);   out = W_o (S_t * silu(W_g h)).

The three projections are one product whose result stays float32; biases, the gate's sigmoid, the candidate and the
recurrence are float32 whatever the compute dtype.  S of a request lives in a state slot of the cache manager, zero at
admission.  Because S_t is linear in S_(t-1), a long portion is scanned in blocks of tokens that are then chained
(``ops.mingru_scan``).
"""
from __future__ import annotations

from .base import Mixer, register_mixer


class MinGruMixer(Mixer):
    def __init__(self, hidden_size: int, width: int):
        self.hidden_size, self.width = int(hidden_size), int(width)
        self.zxg_weight = self.zx_bias = self.o_weight = None

    def parameter_shapes(self) -> dict:
        D, W = self.hidden_size, self.width
        return {"zxg.weight": ((3 * W, D), "matrix"), "zx.bias": ((2 * W,), "vector"), "o.weight": ((D, W), "matrix")}

    def reads_first(self):
        return self.zxg_weight

    def cache_need(self):
        return {"kind": "state", "state_shape": (self.width,), "state_dtype": "float32"}

    def forward(self, ctx, h, entry):
        ops = ctx.ops
        state = ctx.groups[entry.cache_group].state(entry.cache_slot)        # [seats, width] float32
        zxg = ops.linear(h, self.zxg_weight, None, out_float32=True)
        mixed = ops.mingru_scan(zxg, self.zx_bias, state, ctx.state_slots, ctx.cu_q, self.width, ctx.dtype,
                                max_q_len=ctx.max_q_len)
        return ops.linear(mixed, self.o_weight)


register_mixer("mingru", MinGruMixer)
