"""Softmax attention inside chunks of positions over the paged cache, with a logarithmic distance
penalty instead of a position encoding.

    q = W_q x [H, dk];  k = W_k x [G, dk];  v = W_v x [G, dv] / rms(v over dv)   (cached so)
    score(i, j) = (q_i . k_j) * scale - r1[h] * log(1 + r2[h] * (i - j))
    i sees j <= i with floor(i / chunk) = floor(j / chunk);  softmax;  out = W_o [heads' results]

Keys and values have sizes of their own (``PagedKVSpec.value_dim``); pages that lie before the
chunk of a request's next position are given back (``PagedKVSpec.chunk``).  Scores, penalty,
weights and the weighted sum are float32 (``csrc/attention_chunk.cu``).
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..kernels import recurrent as rk
from ..kernels.attention_plan import build_plan
from .base import PagedKVSpec, compute_matrix, register_mixer
from .context import StepPrep
from .recurrent import ProjectedMixer, stack_segments, vector32

MAX_DIM = 256


class ChunkAttention(ProjectedMixer):
    kind = "chunk_attention"

    def __init__(self, width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, chunk: int, eps: float, dtype: torch.dtype,
                 device: torch.device) -> None:
        super().__init__(dtype, device)
        if heads % kv_heads:
            raise ValueError(f"chunk_attention: heads ({heads}) must be a multiple of kv_heads "
                             f"({kv_heads})")
        if chunk <= 0:
            raise ValueError(f"chunk_attention: the chunk must be positive, got {chunk}")
        if not (0 < key_dim <= MAX_DIM and 0 < value_dim <= MAX_DIM):
            raise ValueError(f"chunk_attention: key and value sizes up to {MAX_DIM}, got "
                             f"{key_dim} and {value_dim}")
        self.width, self.heads, self.kv_heads = width, heads, kv_heads
        self.dk, self.dv, self.scale, self.chunk, self.eps = key_dim, value_dim, scale, chunk, eps
        self.key = f"chunk_attention/{heads // kv_heads}/{kv_heads}/{key_dim}/{value_dim}"

    def tensors(self):
        d, h, g = self.width, self.heads, self.kv_heads
        return {"q": ((h * self.dk, d), "matrix"), "k": ((g * self.dk, d), "matrix"),
                "v": ((g * self.dv, d), "matrix"), "r1": ((h,), "vector"), "r2": ((h,), "vector"),
                "o": ((d, h * self.dv), "matrix")}

    def load(self, tensors):
        self._host_in, _ = stack_segments([torch.cat((tensors["q"], tensors["k"], tensors["v"]),
                                                     dim=0)])
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.r1, self.r2 = vector32(tensors["r1"], self.device), vector32(tensors["r2"], self.device)
        self.w_in = None

    def input_matrix(self) -> torch.Tensor:
        return self._host_in

    def kernel_modules(self):
        return ("attention_chunk",)

    def cache_spec(self):
        return PagedKVSpec(self.kv_heads, self.dk, None, value_dim=self.dv, chunk=self.chunk)

    @property
    def prepare_key(self) -> str:
        return self.key

    def prepare(self, prep: StepPrep) -> None:
        """The step's tiles of rows (work items of ``kernels.attention_plan``, unsplit: a chunk
        bounds every key range).  Their number depends on the sequences' token counts only."""
        name = self.key + "/items"
        if prep.has(name):
            return
        host = prep.host
        if int(host.seq_qlen.max()) == 1 and rk.chunk_decode_ok(self.dtype, self.heads,
                                                               self.kv_heads, self.dk, self.dv):
            # single tokens only: the kernel that takes a (sequence, kv head) a block, no items
            prep.add(name, np.zeros((0, 8), dtype=np.int32))
            prep.notes[self.key] = 0
            return
        # tiles of 32 rows when the step brings prompt portions, of 8 for single tokens
        rows = rk.chunk_rows_per_tile(self.dtype, self.dk, self.dv,
                                      int(host.seq_qlen.max()) > 1,
                                      rk.long_portion_rows(host.seq_qlen, self.heads, self.kv_heads))
        plan = build_plan(host.seq_qlen, host.seq_pos0, self.heads // self.kv_heads,
                          self.kv_heads, rows, 0, chunk=0)
        prep.add(name, plan.items)
        prep.notes[self.key] = rows

    def run(self, proj, ctx, cache, ahead=None, out_dtype=None):
        if cache is None or cache.kind != "paged":
            raise ValueError("chunk attention needs a paged key/value cache")
        n = proj.shape[0]
        if cache.writes:
            rk.kv_write_normed(proj, self.heads * self.dk, self.kv_heads, self.dk, self.dv,
                               self.eps, cache.k_pages, cache.v_pages, cache.block_table, ctx)
        context = ctx.buffer("chunk_attention.context", (n, self.heads * self.dv))
        if ctx.notes[self.key] == 0:
            rk.chunk_attention_decode(proj, context, cache.k_pages, cache.v_pages,
                                      cache.block_table, self.r1, self.r2, self.heads,
                                      self.kv_heads, self.dk, self.dv, self.scale, self.chunk, ctx)
        else:
            rk.chunk_attention(proj, context, cache.k_pages, cache.v_pages, cache.block_table,
                               ctx.arrays[self.key + "/items"], self.r1, self.r2, self.heads,
                               self.kv_heads, self.dk, self.dv, self.scale, self.chunk, ctx,
                               tile_rows=ctx.notes[self.key])
        return self.project_out(context, "chunk_attention.out", ctx, ahead, out_dtype=out_dtype)


register_mixer("chunk_attention", ChunkAttention)
