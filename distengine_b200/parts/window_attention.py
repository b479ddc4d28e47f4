"""Grouped-query softmax attention over the paged cache with 32-bit scores and weights: a sliding
window that keeps the first tokens of the sequence, a soft cap on the scores, values that are
rotated by position like keys, an output gate, keys and values of different sizes.  Every one of
these is a parameter; with none of them it is plain causal attention.

    q = W_q x [H, dk];  k = W_k x [G, dk];  v = W_v x [G, dv]
    q, k: the first ``rotary_dim`` features turned by position (pairs i, i + rotary_dim / 2) with
          the frequencies theta^(-2i / rotary_dim), optionally rescaled (``scaling``)
    v:    (``rotate_values``) all dv features turned by the key's position with the plain
          frequencies theta^(-2i / dv), cached so; every head's weighted sum is turned back by the
          query's position
    score(i, j) = (q_i . k_j) * scale;  score <- softcap * tanh(score / softcap)
    i sees j <= i with i - j < window or j < keep_first  (``window`` None: every j <= i)
    out = W_o [heads' results * sigmoid(W_g x)]  (``gated``)

``owns_kv`` false: the layer has no key and value matrices; its run reads the cache that another
run wrote (``PlanEntry.reads_cache_of``) with its own queries and mask.  ``cache_window`` /
``cache_keep_first``: what the pages must keep for every run that reads them (the widest window,
None if one of them sees everything, and the most kept tokens among them); they default to the
layer's own.

Frequency rescaling (``scaling`` = (factor, low, high, original)): with wavelength 2 pi / f, f stays
below original / high, becomes f / factor above original / low, and is blended linearly in
original / wavelength between the two.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import ops
from ..kernels import recurrent as rk
from ..kernels.attention_plan import build_plan
from .base import PagedKVSpec, compute_matrix, register_mixer
from .context import StepPrep
from .recurrent import ProjectedMixer, stack_segments

MAX_DIM = 256


def rotary_frequencies(theta: float, dims: int, scaling=None) -> torch.Tensor:
    """float32 [dims / 2], formed in float64."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(theta) ** (-2.0 * i / max(dims, 1))
    if scaling is not None:
        factor, low, high, original = (float(x) for x in scaling)
        wavelength = 2.0 * math.pi / f
        s = (original / wavelength - low) / (high - low)
        blended = (1.0 - s) * f / factor + s * f
        f = torch.where(wavelength < original / high, f,
                        torch.where(wavelength > original / low, f / factor, blended))
    return f.to(torch.float32)


class WindowAttention(ProjectedMixer):
    kind = "window_attention"

    def __init__(self, width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, rotary_dim: int, theta: float, dtype: torch.dtype,
                 device: torch.device, scaling=None, window: "int | None" = None,
                 keep_first: int = 0, softcap: "float | None" = None,
                 rotate_values: bool = False, gated: bool = False, owns_kv: bool = True,
                 cache_window: "int | None | str" = "own",
                 cache_keep_first: "int | None" = None) -> None:
        super().__init__(dtype, device)
        if heads % kv_heads:
            raise ValueError(f"window_attention: heads ({heads}) must be a multiple of kv_heads "
                             f"({kv_heads})")
        if not (0 < key_dim <= MAX_DIM and 0 < value_dim <= MAX_DIM):
            raise ValueError(f"window_attention: key and value sizes up to {MAX_DIM}, got "
                             f"{key_dim} and {value_dim}")
        if rotary_dim % 2 or not 0 <= rotary_dim <= key_dim:
            raise ValueError(f"window_attention: rotary_dim ({rotary_dim}) must be even and at "
                             f"most the key size ({key_dim})")
        if window is not None and window <= 0:
            raise ValueError(f"window_attention: window must be positive or None, got {window}")
        if keep_first < 0 or (softcap is not None and softcap <= 0):
            raise ValueError("window_attention: keep_first >= 0 and softcap > 0 or None")
        if rotate_values and value_dim % 2:
            raise ValueError(f"window_attention: rotated values need an even size, got {value_dim}")
        self.width, self.heads, self.kv_heads = width, heads, kv_heads
        self.dk, self.dv, self.scale = key_dim, value_dim, float(scale)
        self.rotary_dim, self.window, self.keep_first = rotary_dim, window, keep_first
        self.softcap, self.gated, self.owns_kv = softcap, gated, owns_kv
        self.cache_window = window if cache_window == "own" else cache_window
        self.cache_keep_first = keep_first if cache_keep_first is None else cache_keep_first
        self.fk = rotary_frequencies(theta, rotary_dim, scaling).to(device)
        self.fv = rotary_frequencies(theta, value_dim).to(device) if rotate_values else None
        self.key = (f"window_attention/{heads // kv_heads}/{kv_heads}/{key_dim}/{value_dim}")

    def tensors(self):
        d, h, g = self.width, self.heads, self.kv_heads
        out = {"q": ((h * self.dk, d), "matrix"), "o": ((d, h * self.dv), "matrix")}
        if self.owns_kv:
            out["k"] = ((g * self.dk, d), "matrix")
            out["v"] = ((g * self.dv, d), "matrix")
        if self.gated:
            out["g"] = ((h * self.dv, d), "matrix")
        return out

    def load(self, tensors):
        front = [tensors["q"]] + ([tensors["k"], tensors["v"]] if self.owns_kv else [])
        mats = [torch.cat(front, dim=0)] + ([tensors["g"]] if self.gated else [])
        self._host_in, offsets = stack_segments(mats)
        self.g_col = offsets[1] if self.gated else 0
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.w_in = None

    def input_matrix(self) -> torch.Tensor:
        return self._host_in

    def kernel_modules(self):
        return ("attention_chunk",)

    def cache_spec(self):
        return PagedKVSpec(self.kv_heads, self.dk, self.cache_window, value_dim=self.dv,
                           keep_first=self.cache_keep_first if self.cache_window else 0)

    @property
    def prepare_key(self) -> str:
        return self.key

    def prepare(self, prep: StepPrep) -> None:
        """The step's tiles of rows (work items of ``kernels.attention_plan``, unsplit).  Their
        number depends on the sequences' token counts only."""
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
        rows = rk.chunk_rows_per_tile(self.dtype, self.dk, self.dv,
                                      int(host.seq_qlen.max()) > 1,
                                      rk.long_portion_rows(host.seq_qlen, self.heads, self.kv_heads))
        plan = build_plan(host.seq_qlen, host.seq_pos0, self.heads // self.kv_heads,
                          self.kv_heads, rows, 0, chunk=0)
        prep.add(name, plan.items)
        prep.notes[self.key] = rows

    def run(self, proj, ctx, cache, ahead=None, out_dtype=None):
        if cache is None or cache.kind != "paged":
            raise ValueError("window attention needs a paged key/value cache")
        if cache.writes != self.owns_kv:
            raise ValueError("window attention: a layer with key and value matrices writes its "
                             "own cache, one without reads another run's")
        n, H, dv = proj.shape[0], self.heads, self.dv
        context = ctx.buffer("window_attention.context", (n, H * dv))
        if ctx.notes[self.key] == 0:
            # single tokens only: rotation, cache write, attention, back-rotation and gate are
            # one kernel
            gate = proj[:, self.g_col: self.g_col + H * dv] if self.gated else None
            rk.chunk_attention_decode(
                proj, context, cache.k_pages, cache.v_pages, cache.block_table, None, None, H,
                self.kv_heads, self.dk, dv, self.scale, 0, ctx, window=self.window or 0,
                keep_first=self.keep_first if self.window else 0, softcap=self.softcap or 0.0,
                fused=dict(fk=self.fk, rotary_dim=self.rotary_dim, fv=self.fv,
                           write_kv=cache.writes, gate=gate))
            return self.project_out(context, "window_attention.out", ctx, ahead,
                                    out_dtype=out_dtype)
        rk.kv_write_rotated(proj, self.fk, self.rotary_dim, self.fv, H, self.kv_heads, self.dk,
                            dv, cache.k_pages, cache.v_pages, cache.block_table, cache.writes, ctx)
        finish = self.fv is not None or self.gated
        raw = (ctx.buffer("window_attention.raw", (n, H * dv), torch.float32) if finish
               else context)
        sight = dict(window=self.window or 0, keep_first=self.keep_first if self.window else 0,
                     softcap=self.softcap or 0.0)
        rk.chunk_attention(proj, raw, cache.k_pages, cache.v_pages, cache.block_table,
                           ctx.arrays[self.key + "/items"], None, None, H, self.kv_heads,
                           self.dk, dv, self.scale, 0, ctx, tile_rows=ctx.notes[self.key],
                           **sight)
        if finish:
            gate = proj[:, self.g_col: self.g_col + H * dv] if self.gated else None
            rk.attention_finish(raw, self.fv, gate, context, H, dv, ctx)
        return self.project_out(context, "window_attention.out", ctx, ahead, out_dtype=out_dtype)


register_mixer("window_attention", WindowAttention)
