"""A plain, slow implementation of the Vomotar decoder, one function per mechanism, whole sequences
only, in float64 (or float32) on the CPU.  It shares no code with the engine: the engine's parts
and kernels are compared with it.

``act`` (None or torch.bfloat16) models the engine's bfloat16 mode: the results of matrix
products, the norms' outputs, the gated rows and the cached values are rounded to it (``rnd``);
the residual stream, the states, scores, weights, decays, gates and unit norms are not.

Notation: T tokens, width D.  A weight matrix is stored [out, in]; ``lin`` applies it.  ``w`` maps
tensor names to tensors, ``config`` is the parsed config.json.
"""

from __future__ import annotations

import math

import torch


def rnd(x: torch.Tensor, act) -> torch.Tensor:
    return x if act is None else x.to(act).to(x.dtype)


def lin(x: torch.Tensor, weight: torch.Tensor, act=None) -> torch.Tensor:
    return rnd(x @ weight.to(x.dtype).t(), act)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over the root of (the mean of its squares + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def grouped_rms_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float,
                     act=None) -> torch.Tensor:
    """The last axis is cut into ``groups`` equal consecutive parts; each part is normalised by its
    own root mean square; the whole is multiplied by the weight."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    return rnd(rnd(rms(parts, eps).reshape(shape), act) * weight.to(x.dtype), act)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y[t, c] = sum_j taps[c, j] * x[t - (K - 1) + j, c], zeros before the
    sequence's start; the last column multiplies the current token."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([x.new_zeros(K - 1, C), x], dim=0)
    y = x.new_zeros(T, C)
    for j in range(K):
        y = y + padded[j: j + T] * taps[:, j].to(x.dtype)
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, g):
    """q, k [T, H, dk], v [T, H, dv], beta [T, H], g [T, H, dk] -> o [T, H, dv].
    Per head: S <- g * S (rows are key channels); u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = q.new_zeros(H, dk, dv)
    out = q.new_zeros(T, H, dv)
    for t in range(T):
        S = S * g[t][:, :, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def channel_delta_mixer(h, w, p, m, eps, act=None):
    """The 'channel_delta' mixer on h [T, D]; tensors under prefix p, sizes in m."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(lin(h, w[p + "q"], act), w[p + "q.conv"]))
    k = silu(causal_conv(lin(h, w[p + "k"], act), w[p + "k.conv"]))
    v = silu(causal_conv(lin(h, w[p + "v"], act), w[p + "v.conv"]))
    rep = H // G
    q = unit(q.view(T, G, dk)).repeat_interleave(rep, dim=1) * dk ** -0.5
    k = unit(k.view(T, G, dk)).repeat_interleave(rep, dim=1)
    v = v.view(T, H, dv)
    beta = torch.sigmoid(lin(h, w[p + "b"], act))
    a = lin(lin(h, w[p + "a1"], act), w[p + "a2"]) + w[p + "dt_bias"].to(h.dtype)
    rate = torch.exp(w[p + "A_log"].to(h.dtype))
    g = torch.exp(-rate[None, :, None] * softplus(a).view(T, H, dk))
    o = gated_delta_rule(q, k, v, beta, g)
    gate = torch.sigmoid(lin(lin(h, w[p + "g1"], act), w[p + "g2"])).view(T, H, dv)
    o = rnd(rms(o, eps) * w[p + "norm"].to(h.dtype) * gate, act)
    return lin(o.reshape(T, H * dv), w[p + "o"], act)


def chunked_bias_attention(h, w, p, m, eps, act=None):
    """Softmax attention inside chunks of positions, with a logarithmic distance penalty and
    normalised values."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, scale = m["mask"]["size"], m["scale"]
    q = lin(h, w[p + "q"], act).view(T, H, dk)
    k = lin(h, w[p + "k"], act).view(T, G, dk).repeat_interleave(H // G, dim=1)
    v = rnd(rms(lin(h, w[p + "v"], act).view(T, G, dv), eps), act).repeat_interleave(H // G, dim=1)
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).clamp(min=0).to(h.dtype)
    r1, r2 = w[p + "r1"].to(h.dtype), w[p + "r2"].to(h.dtype)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    scores = scores - r1[:, None, None] * torch.log1p(r2[:, None, None] * dist[None])
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    scores = scores.masked_fill(~seen[None], float("-inf"))
    o = rnd(torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v), act)
    return lin(o.reshape(T, H * dv), w[p + "o"], act)


def rotate_half_layout(x, dims, base):
    """x [T, H, d]: the first ``dims`` features of every head are rotated by position; feature i
    is paired with feature i + dims/2."""
    T = x.shape[0]
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = torch.arange(T, dtype=x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def retention(q, k, v, decay):
    """S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t; no softmax, no denominator."""
    T, H, dk = q.shape
    S = q.new_zeros(H, dk, v.shape[-1])
    out = q.new_zeros(T, H, v.shape[-1])
    for t in range(T):
        S = S * decay[:, None, None] + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def retention_mixer(h, w, p, m, eps, act=None):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = rotate_half_layout(lin(h, w[p + "q"], act).view(T, H, dk), m["rot"]["dims"],
                           m["rot"]["base"])
    k = rotate_half_layout(lin(h, w[p + "k"], act).view(T, H, dk), m["rot"]["dims"],
                           m["rot"]["base"])
    k = k * dk ** -0.5
    v = lin(h, w[p + "v"], act).view(T, H, dv)
    o = retention(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = rnd(rms(o, eps).reshape(T, H * dv) * silu(lin(h, w[p + "g"], act)), act)
    return lin(o, w[p + "o"], act)


def parallel_mixer(h, w, p, m, eps, act=None):
    left = chunked_bias_attention(h, w, p + "left.", m["left"], eps, act)
    right = retention_mixer(h, w, p + "right.", m["right"], eps, act)
    return rnd(0.5 * (rms(left, eps) * w[p + "left.out"].to(h.dtype)
                      + rms(right, eps) * w[p + "right.out"].to(h.dtype)), act)


def dense_feed_forward(h, w, p, act=None):
    # (the engine's fused products keep gate and up in 32-bit up to the activation)
    gate, up = lin(h, w[p + "gate"]), lin(h, w[p + "up"])
    return lin(rnd(silu(gate) * up, act), w[p + "down"], act)


MIXERS = {"channel_delta": channel_delta_mixer, "parallel": parallel_mixer}


def forward(config: dict, w: dict, ids: list[int], dtype=torch.float64, layers_out=None,
            act=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the residual
    stream after every layer; ``act``: see the module's header."""
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x = w["embed"].to(dtype)[torch.tensor(ids)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = grouped_rms_norm(x, w[p + "norm1"], groups, eps, act)
        x = x + MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps, act)
        if layer.get("mlp") is not None:
            h = grouped_rms_norm(x, w[p + "norm2"], groups, eps, act)
            x = x + dense_feed_forward(h, w, p + "mlp.", act)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = grouped_rms_norm(x, w["final.norm"], groups, eps, act)
    return lin(x, w["head"])


def tensor_shapes(config: dict) -> dict:
    """name -> (shape, "matrix" | "vector" | ...) of every tensor of a model of this config."""
    D, out = config["width"], {}
    out["embed"] = (config["vocab"], D)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (D,)
        if layer["type"] == "channel_delta":
            H, G, dk, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            rank = m.get("rank", max(D // 8, 1))
            for name, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + "mix." + name] = (rows, D)
                out[p + "mix." + name + ".conv"] = (rows, K)
            out[p + "mix.b"] = (H, D)
            out[p + "mix.A_log"] = (H,)
            out[p + "mix.norm"] = (dv,)
            out[p + "mix.a1"], out[p + "mix.a2"] = (rank, D), (H * dk, rank)
            out[p + "mix.dt_bias"] = (H * dk,)
            out[p + "mix.g1"], out[p + "mix.g2"] = (rank, D), (H * dv, rank)
            out[p + "mix.o"] = (D, H * dv)
        else:
            a, b = m["left"], m["right"]
            out[p + "mix.left.q"] = (a["heads"] * a["dim"], D)
            out[p + "mix.left.k"] = (a["kv_heads"] * a["dim"], D)
            out[p + "mix.left.v"] = (a["kv_heads"] * a["vdim"], D)
            out[p + "mix.left.r1"], out[p + "mix.left.r2"] = (a["heads"],), (a["heads"],)
            out[p + "mix.left.o"] = (D, a["heads"] * a["vdim"])
            out[p + "mix.right.q"] = (b["heads"] * b["dim"], D)
            out[p + "mix.right.k"] = (b["heads"] * b["dim"], D)
            out[p + "mix.right.v"] = (b["heads"] * b["vdim"], D)
            out[p + "mix.right.g"] = (b["heads"] * b["vdim"], D)
            out[p + "mix.right.o"] = (D, b["heads"] * b["vdim"])
            out[p + "mix.left.out"], out[p + "mix.right.out"] = (D,), (D,)
        if layer.get("mlp") is not None:
            out[p + "norm2"] = (D,)
            ff = layer["mlp"]["ff"]
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (ff, D), (ff, D), (D, ff)
    out["final.norm"] = (D,)
    out["head"] = (config["vocab"], D)
    return out


def random_weights(config: dict, seed: int) -> dict:
    """Random float32 tensors (rounded to bfloat16 values) for a config: matrices so that
    activations stay of order one, vectors and constants in ranges where every mechanism acts."""
    gen = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and leaf != "conv":
            t = torch.randn(shape, generator=gen) * (1.0 / math.sqrt(shape[1]))
            if leaf in ("embed",):
                t = torch.randn(shape, generator=gen)
        elif leaf == "conv":
            t = torch.randn(shape, generator=gen) * 0.5
        elif leaf == "A_log":
            t = torch.rand(shape, generator=gen) * 2.0 - 2.0
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=gen) - 1.0
        elif leaf == "r1":
            t = torch.rand(shape, generator=gen) * 1.5 + 0.2
        elif leaf == "r2":
            t = torch.rand(shape, generator=gen) * 0.9 + 0.1
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w
