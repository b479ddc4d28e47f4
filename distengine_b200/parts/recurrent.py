"""Mixers that keep a matrix state per head in their request's slot: the gated delta rule with a
decay per key channel, and retention.

Both are *projected* mixers (``ProjectedMixer``): everything they take from the layer's input is
one product against a stacked matrix, so a mixer that runs several of them side by side can stack
their matrices into one (``parts.parallel``).  The segments of a stacked matrix start at multiples
of 8 rows (zero rows between them) so that every segment of the product's output can be the
operand of a further product.

Gated delta rule, per head h with state S [dk, dv] (float32, in the slot):

    q, k, v   = silu(conv(W x))           causal convolution over time per channel, `taps` wide;
                                          query/key head h // (H / G) serves head h
    q, k      unit vectors per head (sum of squares + 1e-6 under the root); q also * dk^-1/2
    beta      = sigmoid(W_b x)            one per head
    g         = exp(-exp(A_log[h]) * softplus(W_a2 (W_a1 x) + dt_bias))   one per head and key channel
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out       = W_o [ o / rms(o) * norm * sigmoid(W_g2 (W_g1 x)) ]        rms over dv, eps inside

Retention, per head with state S [dk, dv]:

    q, k      rotated by position on their first `rotary_dim` features (half-split pairs); k * dk^-1/2
    S <- decay[h] S + k v^T;  o = S^T q
    out       = W_o [ o / rms(o) * silu(W_g x) ]

Generalized delta rule, per head with state S [dk, dv] and the unit key u = k / sqrt(|k|^2 + 1e-6):

    r, k, v   = W_r x, W_k x, W_v x
    w         = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 x) + w0))     decay per head and key channel
    a         = sigmoid(W_a x + a_bias)                               removal rate, likewise
    S <- diag(w) S - (a u) (u^T S) + k v^T      (both first terms read the old S);  o = S^T r
    out       = W_o [ o / rms(o) * norm * sigmoid(W_g x) ]            rms per head, norm [H dv]

Lightning attention, per head with state S [dk, dv]:

    q, k, v   = silu(W_q x), silu(W_k x), silu(W_v x)
    S <- decay[h] S + k v^T;  o = S^T q
    out       = W_o [ heads' o / rms(all heads together) * norm * sigmoid(W_g x) ]

The state, the decays, gates, unit norms, angles and read-outs are float32 in both dtypes; the
projections and what follows the gate are in the activation dtype.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels import recurrent as rk
from .base import Mixer, StateSpec, compute_matrix, register_mixer
from .context import CacheBinding, NormAhead, StepContext, UnscaledRows


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


def stack_segments(mats: "list[torch.Tensor]") -> "tuple[torch.Tensor, list[int]]":
    """The matrices one above the other, each starting at a multiple of 8 rows (zero rows fill
    up); returns the stack and where each starts."""
    rows, offsets, at = [], [], 0
    for m in mats:
        offsets.append(at)
        rows.append(m)
        pad = _up8(m.shape[0]) - m.shape[0]
        if pad:
            rows.append(m.new_zeros(pad, m.shape[1]))
        at += m.shape[0] + pad
    return torch.cat(rows, dim=0), offsets


def vector32(t: torch.Tensor, device: torch.device) -> torch.Tensor:
    return t.to(device=device, dtype=torch.float32).contiguous()


class ProjectedMixer(Mixer):
    """A mixer whose only use of its input is one product: ``input_matrix()`` (host, stored dtype,
    after ``load``) and ``run(proj, ctx, cache)`` on that product's rows (row stride free)."""

    w_in: "torch.Tensor | None" = None

    def kernel_modules(self):
        return ("recurrent",)

    def input_matrix(self) -> torch.Tensor:
        raise NotImplementedError

    def run(self, proj: torch.Tensor, ctx: StepContext, cache: "CacheBinding | None",
            ahead: "NormAhead | None" = None,
            out_dtype: "torch.dtype | None" = None) -> "torch.Tensor | None":
        raise NotImplementedError

    def finish_load(self) -> None:
        """Called by whoever owns the input product once the matrix is on the device elsewhere."""
        self._host_in = None

    def _own_input(self) -> torch.Tensor:
        if self.w_in is None:
            self.w_in = compute_matrix(self.input_matrix(), self.dtype, self.device)
            self.finish_load()
        return self.w_in

    # the norm before the mixer can ride on the input product, the norm after it on the output
    # product (``parts.base.NormRider``), where those go to the weight-streaming kernels
    def takes_unscaled(self, n_rows: int) -> bool:
        return ops.norm_ride_parts(n_rows, self._own_input(), self.dtype) > 0

    def ahead_parts(self, n_rows: int) -> int:
        return ops.norm_ride_parts(n_rows, self.w_o, self.dtype)

    def forward(self, x: "torch.Tensor | UnscaledRows", ctx: StepContext,
                cache: "CacheBinding | None",
                ahead: "NormAhead | None" = None) -> "torch.Tensor | None":
        before = None
        if isinstance(x, UnscaledRows):
            before, x = x, x.rows
        w_in = self._own_input()
        proj = ctx.buffer(f"{self.kind}.proj", (x.shape[0], w_in.shape[0]))
        ops.linear(x, w_in, out=proj, status=ctx.status, before=before)
        return self.run(proj, ctx, cache, ahead=ahead)

    def project_out(self, rows: torch.Tensor, name: str, ctx: StepContext,
                    ahead: "NormAhead | None",
                    out_dtype: "torch.dtype | None" = None) -> "torch.Tensor | None":
        """The output product; with ``ahead`` it joins the residual and does the next norm's
        work (and nothing is returned).  ``out_dtype``: float32 for a result that is combined
        with another before it is rounded."""
        if ahead is not None:
            ops.linear(rows, self.w_o, out=ahead.rows, status=ctx.status, after=ahead)
            return None
        if out_dtype is not None and out_dtype != self.dtype:
            name += ".wide"                       # a buffer of its own: no two dtypes under a name
        out = ctx.buffer(name, (rows.shape[0], self.width), out_dtype)
        ops.linear(rows, self.w_o, out=out, out_dtype=out.dtype, status=ctx.status)
        return out


class GatedDeltaRule(ProjectedMixer):
    kind = "gated_delta_rule"

    def __init__(self, width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                 taps: int, eps: float, dtype: torch.dtype, device: torch.device,
                 rank: "int | None" = None) -> None:
        """``rank``: of the two low-rank projections; None: whatever the weight file holds."""
        super().__init__(dtype, device)
        if heads % kv_heads:
            raise ValueError(f"gated_delta_rule: heads ({heads}) must be a multiple of kv_heads "
                             f"({kv_heads})")
        if key_dim > rk.max_key_dim():
            raise ValueError(f"gated_delta_rule: key size {key_dim} is beyond {rk.max_key_dim()}")
        if taps <= 0:
            raise ValueError("gated_delta_rule: the convolution needs at least one tap")
        self.width, self.heads, self.kv_heads = width, heads, kv_heads
        self.dk, self.dv, self.taps, self.eps, self.rank = key_dim, value_dim, taps, eps, rank
        self.channels = 2 * kv_heads * key_dim + heads * value_dim
        self.state_rows = heads * key_dim * value_dim

    def tensors(self):
        d, r = self.width, -1 if self.rank is None else self.rank
        qk, hv, hk = self.kv_heads * self.dk, self.heads * self.dv, self.heads * self.dk
        return {"q": ((qk, d), "matrix"), "q.conv": ((qk, self.taps), "matrix"),
                "k": ((qk, d), "matrix"), "k.conv": ((qk, self.taps), "matrix"),
                "v": ((hv, d), "matrix"), "v.conv": ((hv, self.taps), "matrix"),
                "b": ((self.heads, d), "matrix"), "A_log": ((self.heads,), "vector"),
                "norm": ((self.dv,), "vector"),
                "a1": ((r, d), "matrix"), "a2": ((hk, r), "matrix"),
                "dt_bias": ((hk,), "vector"),
                "g1": ((r, d), "matrix"), "g2": ((hv, r), "matrix"),
                "o": ((d, hv), "matrix")}

    def load(self, tensors):
        if not (tensors["a1"].shape[0] == tensors["a2"].shape[1]
                and tensors["g1"].shape[0] == tensors["g2"].shape[1]):
            raise ValueError("gated_delta_rule: the two halves of a low-rank projection do not "
                             "have the same rank")
        self._host_in, offsets = stack_segments([
            torch.cat((tensors["q"], tensors["k"], tensors["v"]), dim=0),
            tensors["b"], tensors["a1"], tensors["g1"]])
        _, self.b_col, self.a_col, self.g_col = offsets
        self.a_rank, self.g_rank = tensors["a1"].shape[0], tensors["g1"].shape[0]
        self.w_a2 = compute_matrix(tensors["a2"], self.dtype, self.device)
        self.w_g2 = compute_matrix(tensors["g2"], self.dtype, self.device)
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.conv = vector32(torch.cat((tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]),
                                       dim=0), self.device)
        self.a_log = vector32(tensors["A_log"], self.device)
        self.dt_bias = vector32(tensors["dt_bias"], self.device)
        self.norm = vector32(tensors["norm"], self.device)
        self.w_in = None

    def input_matrix(self) -> torch.Tensor:
        return self._host_in

    def cache_spec(self):
        # the state matrices, then the convolution's last taps - 1 inputs
        return StateSpec((self.state_rows + (self.taps - 1) * self.channels,), torch.float32)

    def run(self, proj, ctx, cache, ahead=None, out_dtype=None):
        if cache is None or cache.kind != "state":
            raise ValueError("the gated delta rule needs a state slot")
        if not cache.writes:
            raise ValueError("the gated delta rule cannot read another run's state: it advances it")
        n, f32 = proj.shape[0], torch.float32
        H, G, dk, dv = self.heads, self.kv_heads, self.dk, self.dv
        a = ctx.buffer("delta.a", (n, H * dk), f32)
        ops.linear(proj[:, self.a_col: self.a_col + self.a_rank], self.w_a2, out=a,
                   out_dtype=f32, status=ctx.status)
        gate = ctx.buffer("delta.gate", (n, H * dv), f32)
        ops.linear(proj[:, self.g_col: self.g_col + self.g_rank], self.w_g2, out=gate,
                   out_dtype=f32, status=ctx.status)
        qn = ctx.buffer("delta.q", (n, G * dk), f32)
        kn = ctx.buffer("delta.k", (n, G * dk), f32)
        vv = ctx.buffer("delta.v", (n, H * dv), f32)
        beta = ctx.buffer("delta.beta", (n, H), f32)
        gdec = ctx.buffer("delta.g", (n, H * dk), f32)
        rk.delta_prep(proj, a, self.conv, self.dt_bias, self.a_log, cache.state, self.state_rows,
                      ctx, qn, kn, vv, beta, gdec, H, G, dk, dv, self.b_col)
        o = ctx.buffer("delta.o", (n, H * dv), f32)
        # (the scan also moves the slot's kept convolution inputs on: the preparation has read them)
        rk.state_scan(qn, kn, vv, cache.state, o, H, G, dk, dv, ctx, g=gdec, beta=beta,
                      keep=(proj, self.state_rows, self.channels, self.taps))
        gated = ctx.buffer("delta.gated", (n, H * dv))
        rk.head_gate(o, gate, self.norm, gated, H, dv, self.eps)
        return self.project_out(gated, "delta.out", ctx, ahead, out_dtype=out_dtype)


class Retention(ProjectedMixer):
    kind = "retention"

    def __init__(self, width: int, heads: int, key_dim: int, value_dim: int, decay, rotary_dim: int,
                 theta: float, eps: float, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype, device)
        if len(decay) != heads:
            raise ValueError(f"retention: {len(decay)} decays for {heads} heads")
        if rotary_dim % 2 or not 0 <= rotary_dim <= key_dim:
            raise ValueError(f"retention: rotary_dim ({rotary_dim}) must be even and at most the "
                             f"key size ({key_dim})")
        if key_dim > rk.max_key_dim():
            raise ValueError(f"retention: key size {key_dim} is beyond {rk.max_key_dim()}")
        self.width, self.heads, self.dk, self.dv, self.eps = width, heads, key_dim, value_dim, eps
        self.rotary_dim = rotary_dim
        self.decay = torch.tensor([float(x) for x in decay], dtype=torch.float32, device=device)
        indices = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
        self.inv_freq = (float(theta) ** (-indices / max(rotary_dim, 1))).to(torch.float32).to(device)

    def tensors(self):
        d, hk, hv = self.width, self.heads * self.dk, self.heads * self.dv
        return {"q": ((hk, d), "matrix"), "k": ((hk, d), "matrix"), "v": ((hv, d), "matrix"),
                "g": ((hv, d), "matrix"), "o": ((d, hv), "matrix")}

    def load(self, tensors):
        self._host_in, offsets = stack_segments([torch.cat((tensors["q"], tensors["k"]), dim=0),
                                                 tensors["v"], tensors["g"]])
        _, self.v_col, self.g_col = offsets
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.w_in = None

    def input_matrix(self) -> torch.Tensor:
        return self._host_in

    def cache_spec(self):
        return StateSpec((self.heads * self.dk * self.dv,), torch.float32)

    def run(self, proj, ctx, cache, ahead=None, out_dtype=None):
        if cache is None or cache.kind != "state":
            raise ValueError("retention needs a state slot")
        if not cache.writes:
            raise ValueError("retention cannot read another run's state: it advances it")
        n, f32, H, dk, dv = proj.shape[0], torch.float32, self.heads, self.dk, self.dv
        qr = ctx.buffer("retention.q", (n, H * dk), f32)
        kr = ctx.buffer("retention.k", (n, H * dk), f32)
        rk.retention_prep(proj, self.inv_freq, self.rotary_dim, H, dk, qr, kr, ctx)
        o = ctx.buffer("retention.o", (n, H * dv), f32)
        rk.state_scan(qr, kr, proj[:, self.v_col: self.v_col + H * dv], cache.state, o, H, H, dk,
                      dv, ctx, decay=self.decay)
        gated = ctx.buffer("retention.gated", (n, H * dv))
        rk.head_gate(o, proj[:, self.g_col: self.g_col + H * dv], None, gated, H, dv, self.eps)
        return self.project_out(gated, "retention.out", ctx, ahead, out_dtype=out_dtype)


class GeneralizedDeltaRule(ProjectedMixer):
    kind = "generalized_delta_rule"

    def __init__(self, width: int, heads: int, key_dim: int, eps: float, dtype: torch.dtype,
                 device: torch.device, rank: "int | None" = None) -> None:
        """Keys, values and read-out vectors all have ``key_dim`` features a head.  ``rank``: of
        the decay's low-rank projection; None: whatever the weight file holds."""
        super().__init__(dtype, device)
        if key_dim > rk.max_key_dim():
            raise ValueError(f"generalized_delta_rule: key size {key_dim} is beyond "
                             f"{rk.max_key_dim()}")
        self.width, self.heads, self.dk, self.eps, self.rank = width, heads, key_dim, eps, rank
        self.rows = heads * key_dim

    def tensors(self):
        d, n, r = self.width, self.rows, -1 if self.rank is None else self.rank
        return {"r": ((n, d), "matrix"), "k": ((n, d), "matrix"), "v": ((n, d), "matrix"),
                "g": ((n, d), "matrix"), "a": ((n, d), "matrix"), "a.b": ((n,), "bias"),
                "w1": ((r, d), "matrix"), "w2": ((n, r), "matrix"), "w0": ((n,), "bias"),
                "norm": ((n,), "vector"), "o": ((d, n), "matrix")}

    def load(self, tensors):
        if tensors["w1"].shape[0] != tensors["w2"].shape[1]:
            raise ValueError("generalized_delta_rule: the two halves of the decay's low-rank "
                             "projection do not have the same rank")
        self._host_in, offsets = stack_segments([
            torch.cat((tensors["r"], tensors["k"], tensors["v"], tensors["g"], tensors["a"]),
                      dim=0), tensors["w1"]])
        self.w1_col, self.w_rank = offsets[1], tensors["w1"].shape[0]
        self.w_w2 = compute_matrix(tensors["w2"], self.dtype, self.device)
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.w0 = vector32(tensors["w0"], self.device)
        self.a_bias = vector32(tensors["a.b"], self.device)
        self.norm = vector32(tensors["norm"], self.device)
        self.w_in = None

    def input_matrix(self) -> torch.Tensor:
        return self._host_in

    def cache_spec(self):
        return StateSpec((self.heads * self.dk * self.dk,), torch.float32)

    def run(self, proj, ctx, cache, ahead=None, out_dtype=None):
        if cache is None or cache.kind != "state":
            raise ValueError("the generalized delta rule needs a state slot")
        if not cache.writes:
            raise ValueError("the generalized delta rule cannot read another run's state: it "
                             "advances it")
        n, f32, H, dk, rows = proj.shape[0], torch.float32, self.heads, self.dk, self.rows
        inner = proj[:, self.w1_col: self.w1_col + self.w_rank]
        ops.activation(inner, inner, "tanh")
        wl = ctx.buffer("gdelta.wl", (n, rows), f32)
        ops.linear(inner, self.w_w2, out=wl, out_dtype=f32, status=ctx.status)
        rr = ctx.buffer("gdelta.r", (n, rows), f32)
        kk = ctx.buffer("gdelta.k", (n, rows), f32)
        ww = ctx.buffer("gdelta.w", (n, rows), f32)
        zz = ctx.buffer("gdelta.z", (n, rows), f32)
        dots = ctx.buffer("gdelta.dots", (n, 2 * H), f32)
        rk.gdelta_prep(proj, 0, rows, 4 * rows, wl, self.w0, self.a_bias, rr, kk, ww, zz, dots,
                       H, dk)
        o = ctx.buffer("gdelta.o", (n, rows), f32)
        rk.state_scan(rr, kk, proj[:, 2 * rows: 3 * rows], cache.state, o, H, H, dk, dk, ctx,
                      g=ww, z=zz, dots=dots)
        gated = ctx.buffer("gdelta.gated", (n, rows))
        rk.head_gate(o, proj[:, 3 * rows: 4 * rows], self.norm, gated, H, dk, self.eps,
                     spanning=True)
        return self.project_out(gated, "gdelta.out", ctx, ahead, out_dtype=out_dtype)


class LightningAttention(ProjectedMixer):
    kind = "lightning_attention"

    def __init__(self, width: int, heads: int, key_dim: int, value_dim: int, decay, eps: float,
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype, device)
        if len(decay) != heads:
            raise ValueError(f"lightning_attention: {len(decay)} decays for {heads} heads")
        if key_dim > rk.max_key_dim():
            raise ValueError(f"lightning_attention: key size {key_dim} is beyond "
                             f"{rk.max_key_dim()}")
        self.width, self.heads, self.dk, self.dv, self.eps = width, heads, key_dim, value_dim, eps
        self.decay = torch.tensor([float(x) for x in decay], dtype=torch.float32, device=device)

    def tensors(self):
        d, hk, hv = self.width, self.heads * self.dk, self.heads * self.dv
        return {"q": ((hk, d), "matrix"), "k": ((hk, d), "matrix"), "v": ((hv, d), "matrix"),
                "g": ((hv, d), "matrix"), "norm": ((hv,), "vector"), "o": ((d, hv), "matrix")}

    def load(self, tensors):
        self._host_in, offsets = stack_segments([
            torch.cat((tensors["q"], tensors["k"], tensors["v"]), dim=0), tensors["g"]])
        self.g_col = offsets[1]
        self.w_o = compute_matrix(tensors["o"], self.dtype, self.device)
        self.norm = vector32(tensors["norm"], self.device)
        self.w_in = None

    def input_matrix(self) -> torch.Tensor:
        return self._host_in

    def cache_spec(self):
        return StateSpec((self.heads * self.dk * self.dv,), torch.float32)

    def run(self, proj, ctx, cache, ahead=None, out_dtype=None):
        if cache is None or cache.kind != "state":
            raise ValueError("lightning attention needs a state slot")
        if not cache.writes:
            raise ValueError("lightning attention cannot read another run's state: it advances it")
        n, f32, H, dk, dv = proj.shape[0], torch.float32, self.heads, self.dk, self.dv
        qkv = ctx.buffer("lightning.qkv", (n, H * (2 * dk + dv)), f32)
        rk.silu_rows(proj[:, : H * (2 * dk + dv)], qkv)
        o = ctx.buffer("lightning.o", (n, H * dv), f32)
        rk.state_scan(qkv[:, : H * dk], qkv[:, H * dk: 2 * H * dk], qkv[:, 2 * H * dk:],
                      cache.state, o, H, H, dk, dv, ctx, decay=self.decay)
        gated = ctx.buffer("lightning.gated", (n, H * dv))
        # one root mean square for all heads together: a single "head" as wide as the row
        rk.head_gate(o, proj[:, self.g_col: self.g_col + H * dv], self.norm, gated, 1, H * dv,
                     self.eps, spanning=True)
        return self.project_out(gated, "lightning.out", ctx, ahead, out_dtype=out_dtype)


register_mixer("generalized_delta_rule", GeneralizedDeltaRule)
register_mixer("lightning_attention", LightningAttention)
register_mixer("gated_delta_rule", GatedDeltaRule)
register_mixer("retention", Retention)
