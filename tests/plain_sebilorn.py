"""A plain, slow implementation of the Sebilorn decoder, one function per mechanism, whole sequences
only, in float64 (or float32) on the CPU.  It shares no code with the engine: the engine's parts
and kernels are compared with it.

``act`` (None or torch.bfloat16) models the engine's bfloat16 mode: the results of matrix
products, the norms' outputs, rotated queries, cached keys and values, and the rows that enter an
output product are rounded to it (``rnd``); the residual stream, the states, scores, weights,
decays, gates, unit norms and angles are not.

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


def layer_norm(x, weight, bias, eps, act=None):
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight + bias over the last axis."""
    mean = x.mean(dim=-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return rnd(dev / torch.sqrt(var + eps) * weight.to(x.dtype) + bias.to(x.dtype), act)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


# ----------------------------------------------------------------------------- rotation
def frequencies(base: float, dims: int, scaling=None, dtype=torch.float64) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2.  ``scaling`` {factor, low, high, original}: a
    frequency whose wavelength 2 pi / f is below original / high stays, one above original / low
    is divided by factor, between the two it is blended by s = (original / wavelength - low) /
    (high - low): (1 - s) f / factor + s f."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if scaling is not None:
        factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
        original = float(scaling["original"])
        wavelength = 2.0 * math.pi / f
        s = (original / wavelength - low) / (high - low)
        blended = (1.0 - s) * f / factor + s * f
        f = torch.where(wavelength < original / high, f,
                        torch.where(wavelength > original / low, f / factor, blended))
    return f.to(dtype)


def rotate(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, sign: float = 1.0):
    """x [T, heads, d]: the first 2 len(freq) features of every head are turned, feature i paired
    with feature i + len(freq), by the angle sign * position * freq[i]; the rest pass."""
    half = freq.shape[0]
    if half == 0:
        return x
    angle = sign * positions.to(x.dtype)[:, None, None] * freq.to(x.dtype)[None, None, :]
    c, s = torch.cos(angle), torch.sin(angle)
    a, b = x[..., :half], x[..., half: 2 * half]
    return torch.cat((a * c - b * s, b * c + a * s, x[..., 2 * half:]), dim=-1)


# ----------------------------------------------------------------------------- attention
def visible(T: int, window=None, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: query i sees key j <= i; with a window only if i - j < window or
    j < keep_first."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see = see & ((i - j < window) | (j < keep_first))
    return see


def softmax_attention(q, k, v, scale, see, softcap=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; head h reads kv head h // (H/G).
    score = q . k * scale, then softcap * tanh(score / softcap); softmax over the visible keys."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = q.new_zeros(T, H, v.shape[-1])
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].t()) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~see, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = p @ v[:, h // rep]
    return out


def attention_keys_values(h, w, pre, m, positions, act=None):
    """What an attention layer caches: keys rotated by position (scaled frequencies), values
    rotated by position over all their features (plain frequencies)."""
    T = h.shape[0]
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    fk = frequencies(rot["base"], rot["dims"], rot.get("scaling"), h.dtype)
    fv = frequencies(rot["base"], dv, None, h.dtype)
    k = lin(h, w[pre + "k"], act).reshape(T, G, dk)
    v = lin(h, w[pre + "v"], act).reshape(T, G, dv)
    return rnd(rotate(k, positions, fk), act), rnd(rotate(v, positions, fv), act)


def window_attention_mixer(h, w, pre, m, eps, act=None, shared=None):
    """The 'attention' mixer.  ``shared``: (keys, values) of the layer it takes them from.
    Returns (output, (keys, values))."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    positions = torch.arange(T)
    fq = frequencies(rot["base"], rot["dims"], rot.get("scaling"), h.dtype)
    fv = frequencies(rot["base"], dv, None, h.dtype)
    q = rnd(rotate(lin(h, w[pre + "q"], act).reshape(T, H, dk), positions, fq), act)
    kv = shared if shared is not None else attention_keys_values(h, w, pre, m, positions, act)
    mask = m.get("mask") or {}                         # no mask: every earlier token is seen
    see = visible(T, mask.get("size"), mask.get("keep_first", 0))
    o = softmax_attention(q, kv[0], kv[1], m["scale"], see, m.get("softcap"))
    o = rnd(rotate(o, positions, fv, sign=-1.0), act)        # every head's sum turned back
    return lin(o.reshape(T, H * dv), w[pre + "o"], act), kv


def gated_attention_branch(h, w, pre, m, act=None):
    """The left branch of 'parallel': causal softmax attention, rotation on the first rot.dims
    features, the heads' results times sigmoid(W_g h) before the output matrix."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    f = frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"), h.dtype)
    q = rnd(rotate(lin(h, w[pre + "q"], act).reshape(T, H, dk), positions, f), act)
    k = rnd(rotate(lin(h, w[pre + "k"], act).reshape(T, G, dk), positions, f), act)
    v = lin(h, w[pre + "v"], act).reshape(T, G, dv)
    o = softmax_attention(q, k, v, m["scale"], visible(T)).reshape(T, H * dv)
    gate = torch.sigmoid(lin(h, w[pre + "g"], act))
    return lin(rnd(o * gate, act), w[pre + "o"], act)


# ----------------------------------------------------------------------------- recurrences
def generalized_delta_rule(r, k, v, decay, rate):
    """r, k, decay, rate [T, H, dk], v [T, H, dv] -> o [T, H, dv].  Per head, with the unit key
    u = k / sqrt(sum k^2 + 1e-6) and the old state S [dk, dv]:
        S' = decay * S (row by row) - (rate * u) (u^T S) + k v^T;   o = S'^T r."""
    T, H, dk = r.shape
    dv = v.shape[-1]
    S = r.new_zeros(H, dk, dv)
    out = r.new_zeros(T, H, dv)
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(dim=-1, keepdim=True) + 1e-6)
        seen = torch.einsum("hk,hkv->hv", u, S)
        S = (decay[t][:, :, None] * S - (rate[t] * u)[:, :, None] * seen[:, None, :]
             + k[t][:, :, None] * v[t][:, None, :])
        out[t] = torch.einsum("hkv,hk->hv", S, r[t])
    return out


def delta_branch(h, w, pre, m, eps, act=None):
    """The right branch of 'parallel'."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = lin(h, w[pre + "r"], act).reshape(T, H, d)
    k = lin(h, w[pre + "k"], act).reshape(T, H, d)
    v = lin(h, w[pre + "v"], act).reshape(T, H, d)
    inner = rnd(torch.tanh(lin(h, w[pre + "w1"], act)), act)
    logit = inner @ w[pre + "w2"].to(h.dtype).t() + w[pre + "w0"].to(h.dtype)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(logit)).reshape(T, H, d)
    rate = torch.sigmoid(lin(h, w[pre + "a"], act) + w[pre + "a.b"].to(h.dtype)).reshape(T, H, d)
    o = generalized_delta_rule(r, k, v, decay, rate)
    o = rms(o, eps).reshape(T, H * d) * w[pre + "norm"].to(h.dtype)
    o = o * torch.sigmoid(lin(h, w[pre + "g"], act))
    return lin(rnd(o, act), w[pre + "o"], act)


def decayed_state(q, k, v, decay):
    """q, k [T, H, dk], v [T, H, dv], decay [H]: S <- decay S + k v^T, o = S^T q."""
    T, H, dk = q.shape
    S = q.new_zeros(H, dk, v.shape[-1])
    out = q.new_zeros(T, H, v.shape[-1])
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def lightning_mixer(h, w, pre, m, eps, act=None):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(lin(h, w[pre + "q"], act)).reshape(T, H, dk)
    k = silu(lin(h, w[pre + "k"], act)).reshape(T, H, dk)
    v = silu(lin(h, w[pre + "v"], act)).reshape(T, H, dv)
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=h.dtype)
    o = decayed_state(q, k, v, decay).reshape(T, H * dv)
    o = rms(o, eps) * w[pre + "norm"].to(h.dtype) * torch.sigmoid(lin(h, w[pre + "g"], act))
    return lin(rnd(o, act), w[pre + "o"], act)


def parallel_mixer(h, w, pre, m, eps, act=None):
    left = gated_attention_branch(h, w, pre + "left.", m["left"], act)
    right = delta_branch(h, w, pre + "right.", m["right"], eps, act)
    return m["left_scale"] * left + m["right_scale"] * right


def squared_relu_mlp(h, w, pre, act=None):
    up = torch.relu(lin(h, w[pre + "up"], act))
    return lin(rnd(up * up, act), w[pre + "down"], act)


# ----------------------------------------------------------------------------- the model
def forward(config, w, tokens, dtype=torch.float64, act=None, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the residual
    stream after every layer."""
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"].to(dtype)[ids] * config["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps, act)
        if layer["type"] == "attention":
            shared = kept[m["kv_from"]] if m.get("kv_from") is not None else None
            y, kept[i] = window_attention_mixer(h, w, p + "mix.", m, eps, act, shared)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", m, eps, act)
        elif layer["type"] == "lightning":
            y = lightning_mixer(h, w, p + "mix.", m, eps, act)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer["mlp"] is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps, act)
            x = x + squared_relu_mlp(h, w, p + "mlp.", act)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = layer_norm(x, w["final.norm"], w["final.norm.b"], eps, act)
    logits = h @ w["head"].to(dtype).t()
    cap = config.get("logit_softcap")
    if cap is not None:
        logits = cap * torch.tanh(logits / cap)
    return logits


# ----------------------------------------------------------------------------- weights for tests
def tensor_shapes(config) -> dict:
    D, V = config["width"], config["vocab"]
    shapes = {"embed": (V, D), "final.norm": (D,), "final.norm.b": (D,), "head": (V, D)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1.b"] = (D,)
        x = p + "mix."
        if layer["type"] == "attention":
            shapes[x + "q"] = (m["heads"] * m["dim"], D)
            shapes[x + "o"] = (D, m["heads"] * m["vdim"])
            if m.get("kv_from") is None:
                shapes[x + "k"] = (m["kv_heads"] * m["dim"], D)
                shapes[x + "v"] = (m["kv_heads"] * m["vdim"], D)
        elif layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            shapes[x + "left.q"] = (a["heads"] * a["dim"], D)
            shapes[x + "left.k"] = (a["kv_heads"] * a["dim"], D)
            shapes[x + "left.v"] = (a["kv_heads"] * a["vdim"], D)
            shapes[x + "left.g"] = (a["heads"] * a["vdim"], D)
            shapes[x + "left.o"] = (D, a["heads"] * a["vdim"])
            n = b["heads"] * b["dim"]
            rank = b.get("rank", 8)
            for name in ("r", "k", "v", "g", "a"):
                shapes[x + "right." + name] = (n, D)
            shapes[x + "right.a.b"] = shapes[x + "right.w0"] = shapes[x + "right.norm"] = (n,)
            shapes[x + "right.w1"] = (rank, D)
            shapes[x + "right.w2"] = (n, rank)
            shapes[x + "right.o"] = (D, n)
        else:
            for name, rows in (("q", m["dim"]), ("k", m["dim"]), ("v", m["vdim"]),
                               ("g", m["vdim"])):
                shapes[x + name] = (m["heads"] * rows, D)
            shapes[x + "norm"] = (m["heads"] * m["vdim"],)
            shapes[x + "o"] = (D, m["heads"] * m["vdim"])
        if layer["mlp"] is not None:
            shapes[p + "norm2"] = shapes[p + "norm2.b"] = (D,)
            shapes[p + "mlp.up"] = (layer["mlp"]["ff"], D)
            shapes[p + "mlp.down"] = (D, layer["mlp"]["ff"])
    return shapes


def random_weights(config, seed: int = 0, spread: float = 1.0) -> dict:
    """bfloat16 tensors: matrices N(0, spread^2 / in), norm weights near 1, biases small."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        if len(shape) == 2:
            t = torch.randn(shape, generator=g) * (spread / math.sqrt(shape[1]))
            if name == "embed":
                t = torch.randn(shape, generator=g) / config["embedding"]["scale"]
        elif name.endswith(".b") or name.endswith("w0"):
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out
