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

Options: ``q_rank`` > 0 sends the queries through a latent of their own, q = W_uq RMSNorm(W_dq h) (a plain weight, float32
norm); ``shared_latent`` makes a layer that has no W_dkv: it reads the rows another layer's run entry wrote into the cache
slot (its run entry has ``write_cache=False``) through its own W_uk and W_uv.
"""
from __future__ import annotations

import torch

from .base import Mixer, register_mixer


class LatentAttentionMixer(Mixer):
    def __init__(self, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 eps: float, window: int = 0, rot_base: float = 10000.0, rot_dims: int | None = None, q_rank: int = 0,
                 shared_latent: bool = False):
        self.hidden_size, self.heads, self.dim, self.rot_dim = int(hidden_size), int(heads), int(dim), int(rot_dim)
        self.vdim, self.kv_rank, self.scale, self.eps = int(vdim), int(kv_rank), float(scale), float(eps)
        self.window, self.rot_base = int(window), float(rot_base)
        self.q_rank, self.shared_latent = int(q_rank), bool(shared_latent)
        self.rot_dims = int(self.rot_dim if rot_dims is None else rot_dims)
        if self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ValueError("rot_dims must be even and at most rot_dim")
        # a cached row: [latent | rotated key part], padded with zeros to what the attention kernels take
        self.row = -(-(self.kv_rank + self.rot_dim) // 16) * 16
        self.q_weight = self.dkv_weight = self.dkv_norm_weight = self.uk_weight = self.uv_weight = self.o_weight = None
        self.dq_weight = self.dq_norm_weight = self.uq_weight = None
        self._uk_t = self._uv = None
        self._inv_freq = {}

    def parameter_shapes(self) -> dict:
        H, D = self.heads, self.hidden_size
        shapes = {"uk.weight": ((H * self.dim, self.kv_rank), "matrix"),
                  "uv.weight": ((H * self.vdim, self.kv_rank), "matrix"),
                  "o.weight": ((D, H * self.vdim), "matrix")}
        if self.q_rank:
            shapes.update({"dq.weight": ((self.q_rank, D), "matrix"), "dq_norm.weight": ((self.q_rank,), "vector"),
                           "uq.weight": ((H * (self.dim + self.rot_dim), self.q_rank), "matrix")})
        else:
            shapes["q.weight"] = ((H * (self.dim + self.rot_dim), D), "matrix")
        if not self.shared_latent:
            shapes.update({"dkv.weight": ((self.kv_rank + self.rot_dim, D), "matrix"), "dkv_norm.weight": ((self.kv_rank,), "vector")})
        return shapes

    def bind(self, tensors: dict) -> None:
        super().bind(tensors)
        H = self.heads
        # W_uk^T per head, as the [N, K] matrix of a product that takes a head's plain query part to the latent space
        self._uk_t = self.uk_weight.view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self._uv = self.uv_weight.view(H, self.vdim, self.kv_rank)

    def reads_first(self):
        return self.dq_weight if self.q_rank else self.q_weight

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
        slot_mapping = group.slot_mapping if (entry.write_cache and not self.shared_latent) else None
        T, H, dn, dr, rank = h.shape[0], self.heads, self.dim, self.rot_dim, self.kv_rank
        if self.q_rank:
            # the queries' latent: the product stays float32 up to its norm, which rounds once
            low = ops.linear(h, self.dq_weight, None, out_float32=True)
            q = ops.linear(ops.add_rmsnorm(low, None, self.dq_norm_weight, self.eps, ctx.dtype), self.uq_weight)
        else:
            q = ops.linear(h, self.q_weight)                     # [T, H (dn + dr)]
        # a layer that reads another layer's latents makes none: nothing is normed, rotated or written for the keys
        down = None if self.shared_latent else ops.linear(h, self.dkv_weight, None, out_float32=True)
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
