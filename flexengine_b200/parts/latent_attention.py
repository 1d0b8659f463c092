"""Attention over a cached latent: keys and values of all heads are linear maps of one small vector per token.

Per token the cache holds the latent c (``kv_rank`` numbers, RMS-normed) and one rotated key part (``rot_dim``
numbers) that all heads share; nothing per head.  With q = [q_plain | q_rot] per head, the score of a key is
(q_plain . (W_uk c) + q_rot . k_rot) * scale = ((W_uk^T q_plain) . c + q_rot . k_rot) * scale, and the head's
output is W_uv (sum_t p_t c_t).  So the step maps every query into the latent space once (a product of head
size x kv_rank per head), runs attention with ONE key/value head whose rows are the cached vectors
[c | k_rot] themselves (the same paged kernels as grouped-query attention: the heads are one group; the value
is the cached row, of which the first kv_rank columns are used), and expands the result with W_uv.  The
cached vectors are never expanded, whatever the cut of the prompt.

The rotation turns interleaved pairs (2i, 2i+1) of the first ``rot_dims`` entries of the rotated parts by
position * base^(-2i/rot_dims); angles, sines and cosines are float32, and so are the latent's norm, the scores
and the softmax.  Key t is visible to the query at position p iff 0 <= p - t < window (window 0: all).
"""
from __future__ import annotations

import torch

from .base import Mixer, register_mixer


class LatentAttentionMixer(Mixer):
    def __init__(self, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 eps: float, window: int = 0, rot_base: float = 10000.0, rot_dims: int | None = None):
        self.hidden_size, self.heads, self.dim, self.rot_dim = int(hidden_size), int(heads), int(dim), int(rot_dim)
        self.vdim, self.kv_rank, self.scale, self.eps = int(vdim), int(kv_rank), float(scale), float(eps)
        self.window, self.rot_base = int(window), float(rot_base)
        self.rot_dims = int(self.rot_dim if rot_dims is None else rot_dims)
        if self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ValueError("rot_dims must be even and at most rot_dim")
        # a cached row: [latent | rotated key part], padded with zeros to what the attention kernels take
        self.row = -(-(self.kv_rank + self.rot_dim) // 16) * 16
        self.q_weight = self.dkv_weight = self.dkv_norm_weight = self.uk_weight = self.uv_weight = self.o_weight = None
        self._uk_t = self._uv = None
        self._inv_freq = {}

    def parameter_shapes(self) -> dict:
        H, D = self.heads, self.hidden_size
        return {"q.weight": ((H * (self.dim + self.rot_dim), D), "matrix"),
                "dkv.weight": ((self.kv_rank + self.rot_dim, D), "matrix"),
                "dkv_norm.weight": ((self.kv_rank,), "vector"),
                "uk.weight": ((H * self.dim, self.kv_rank), "matrix"),
                "uv.weight": ((H * self.vdim, self.kv_rank), "matrix"),
                "o.weight": ((D, H * self.vdim), "matrix")}

    def bind(self, tensors: dict) -> None:
        super().bind(tensors)
        H = self.heads
        # W_uk^T per head, as the [N, K] matrix of a product that takes a head's plain query part to the latent space
        self._uk_t = self.uk_weight.view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self._uv = self.uv_weight.view(H, self.vdim, self.kv_rank)

    def reads_first(self):
        return self.q_weight

    def cache_need(self):
        return {"kind": "window" if self.window > 0 else "full", "kv_heads": 1, "head_dim": self.row,
                "window": self.window, "planes": 1}

    def inverse_frequencies(self, device):
        key = str(device)
        if key not in self._inv_freq:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            table = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / max(self.rot_dims, 1))
            self._inv_freq[key] = table.to(torch.float32).to(device).contiguous()
        return self._inv_freq[key]

    def forward(self, ctx, h, entry):
        ops = ctx.ops
        group = ctx.groups[entry.cache_group]
        rows, _ = group.kv_slot(entry.cache_slot)               # [pages, 1, page_size, row]
        slot_mapping = group.slot_mapping if entry.write_cache else None
        T, H, dn, dr, rank = h.shape[0], self.heads, self.dim, self.rot_dim, self.kv_rank
        q = ops.linear(h, self.q_weight)                         # [T, H (dn + dr)]
        down = ops.linear(h, self.dkv_weight, None, out_float32=True)
        q_latent = ops.batched_linear(q.view(T, H, dn + dr)[:, :, :dn].transpose(0, 1), self._uk_t)      # [H, T, rank]
        # the queries as the attention kernel takes them, [T, H, row] = [q in latent space | rotated q part | 0],
        # and this step's rows into the cache: the latent through its norm, the key part rotated
        queries = ops.latent_prepare(q, q_latent, down, self.dkv_norm_weight, self.eps, ctx.positions,
                                     self.inverse_frequencies(h.device), self.rot_dims, slot_mapping, rows,
                                     H, dn, dr, rank, self.row, group.page_size)
        mixed = ops.paged_attention(queries, rows, rows, group.block_table, ctx, H, 1, self.row, group.page_size,
                                    self.scale, self.window)
        latent_out = mixed.view(T, H, self.row)[:, :, :rank].transpose(0, 1)                              # [H, T, rank]
        values = ops.batched_linear(latent_out, self._uv, token_major=True)                              # [T, H vdim]
        return ops.linear(values, self.o_weight)


register_mixer("latent_attention", LatentAttentionMixer)
