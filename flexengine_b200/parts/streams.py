"""What a layer over several residual streams is made of besides its norms, mixer and feed-forward.

``HyperConnection``: the learned numbers with which a sublayer reads the streams (``read`` [S]), writes its output into
them (``write`` [S]) and mixes them among themselves (``mix`` [S, S], indexed [from, to]):
    u = sum_s read[s] x_s;   x_t <- sum_s mix[s, t] x_s + write[t] * y   (all streams at once, from the old ones).
``ResidualGate``: a sublayer's output is multiplied, element by element, by sigmoid(W h + b) of the rows it read.
``TokenShift``: the rows a mixer reads are blended with the row of the token before, h + (h' - h) * mu (zeros before a
sequence's first token); a request's last row is kept in a state slot from step to step.
``StreamUpdate``: a sublayer's output on its way into the streams; the norm that reads the streams next puts it there.
"""
from __future__ import annotations

from .base import Part


class HyperConnection(Part):
    def __init__(self, streams: int):
        self.streams = int(streams)
        self.read = self.write = self.mix = None

    def parameter_shapes(self) -> dict:
        s = self.streams
        return {"read": ((s,), "vector"), "write": ((s,), "vector"), "mix": ((s, s), "vector")}


class ResidualGate(Part):
    def __init__(self, hidden_size: int):
        self.hidden_size = int(hidden_size)
        self.weight = self.bias = None

    def parameter_shapes(self) -> dict:
        h = self.hidden_size
        return {"weight": ((h, h), "matrix"), "bias": ((h,), "vector")}

    def reads_first(self):
        return self.weight

    def logits(self, ctx, h):
        """W h, in the compute dtype; the bias and the sigmoid are the work of the kernel that applies the gate."""
        return ctx.ops.linear(h, self.weight)


class TokenShift(Part):
    def __init__(self, hidden_size: int, group: int, slot: int):
        self.hidden_size, self.group, self.slot = int(hidden_size), int(group), int(slot)
        self.mu = None

    def parameter_shapes(self) -> dict:
        return {"mu": ((self.hidden_size,), "vector")}

    @staticmethod
    def cache_need(hidden_size: int):
        return {"kind": "state", "state_shape": (int(hidden_size),), "state_dtype": "float32"}

    def forward(self, ctx, h):
        kept = ctx.groups[self.group].state(self.slot)          # [seats, hidden] float32
        return ctx.ops.token_shift(h, self.mu, kept, ctx.state_slots, ctx.cu_q, ctx.token_request)

    def within_norm(self, ctx):
        """What the norm before needs to do this shift in its own kernel, in a step of one token a request on kernels that
        can (row i is then request i's, and the row before it is the seat's kept one); None otherwise."""
        if ctx.decode_only and getattr(ctx.ops, "FUSES_TOKEN_SHIFT", False):
            return (self.mu, ctx.groups[self.group].state(self.slot), ctx.state_slots)
        return None


class StreamUpdate:
    __slots__ = ("y", "gate", "gate_bias", "mix", "write")

    def __init__(self, y, gate, gate_bias, mix, write):
        self.y, self.gate, self.gate_bias, self.mix, self.write = y, gate, gate_bias, mix, write
