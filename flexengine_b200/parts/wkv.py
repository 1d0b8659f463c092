"""A linear-recurrent mixer with a matrix state per head and a data-dependent decay per key channel.

With h' the normalised input of the token before (zeros before the first), each of r, k, v, g, w reads its own
blend h + (h' - h) * mu_s.  r, k, v = W_r, W_k, W_v of their blends, split into heads of ``dim``;
gate = silu(W_g blend_g); decay w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0)), per head and key channel.
Per head, with state S [dim, dim] (key channel x value channel):
    out_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t ;   S_t = diag(w_t) S_{t-1} + k_t v_t^T .
Each head's out is divided by its root mean square, the heads are concatenated, multiplied by a weight and by
the gate, and projected.  The state of a request (S of every head, and the last token's h) lives in a state slot
of the cache manager in float32, zero at admission; the decay with its logarithms and exponentials, the
recurrence and the head norm are float32 whatever the compute dtype.
"""
from __future__ import annotations

from .base import Mixer, register_mixer


class WkvMixer(Mixer):
    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, hidden_size: int, heads: int, dim: int, decay_rank: int, eps: float):
        self.hidden_size, self.heads, self.dim = int(hidden_size), int(heads), int(dim)
        self.decay_rank, self.eps = int(decay_rank), float(eps)
        self.mu = self.r_weight = self.k_weight = self.v_weight = self.g_weight = None
        self.w1_weight = self.w2_weight = self.w0 = self.u = self.norm_weight = self.o_weight = None

    def parameter_shapes(self) -> dict:
        D, inner = self.hidden_size, self.heads * self.dim
        shapes = {"mu": ((len(self.BLENDS) * D,), "vector")}
        for name in ("r", "k", "v", "g"):
            shapes[name + ".weight"] = ((inner, D), "matrix")
        shapes.update({"w1.weight": ((self.decay_rank, D), "float32"), "w2.weight": ((inner, self.decay_rank), "float32"),
                       "w0": ((inner,), "vector"), "u": ((self.heads, self.dim), "vector"), "norm.weight": ((inner,), "vector"),
                       "o.weight": ((D, inner), "matrix")})
        return shapes

    def reads_first(self):
        return self.r_weight

    @property
    def state_elements(self) -> int:
        return self.heads * self.dim * self.dim + self.hidden_size

    def cache_need(self):
        return {"kind": "state", "state_shape": (self.state_elements,), "state_dtype": "float32"}

    def forward(self, ctx, h, entry):
        ops = ctx.ops
        H, d = self.heads, self.dim
        state = ctx.groups[entry.cache_group].state(entry.cache_slot)      # [seats, H d d + D] float32
        matrices = H * d * d
        # the five blends of every token with the token before it (the request's last h of the step before for a
        # portion's first token); the seat then keeps this step's last h
        blends, blend_w = ops.token_shift_blend(h, self.mu, state, matrices, ctx.state_slots, ctx.cu_q, ctx.token_request)
        r = ops.linear(blends[0], self.r_weight)
        k = ops.linear(blends[1], self.k_weight)
        v = ops.linear(blends[2], self.v_weight)
        g = ops.linear(blends[3], self.g_weight)
        lora = ops.activation(ops.linear(blend_w, self.w1_weight, None, out_float32=True), "tanh")
        decay_logits = ops.linear(lora, self.w2_weight, None, out_float32=True)        # w0 is added in the recurrence
        out = ops.wkv_recurrence(r, k, v, decay_logits, self.w0, self.u, state, ctx.state_slots, ctx.cu_q, H, d)
        gated = ops.head_rmsnorm_gate(out, self.norm_weight, g, self.eps, H, ctx.dtype)
        return ops.linear(gated, self.o_weight)


register_mixer("wkv", WkvMixer)
