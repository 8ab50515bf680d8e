"""A plain, slow Redudra in float64 numpy: the oracle of the Redudra tests.

One function per mechanism, whole sequences, no cache, no batching, nothing shared
with the package.  ``cfg`` is the dictionary of a config.json, ``W`` maps tensor
names to float64 arrays.  Notation: X [T, width] the residual stream of one
sequence, t the position (from 0), m the residual multiplier.

    layer:   h = LN1(X);  h'_t = h_t + (h_{t-1} - h_t) * shift  (h_{-1} = 0);  X += m mix(h');  X += m ff(LN2(X))
    LN(x)  = (x - mean) / sqrt(var + eps) * w + b
    loop:    layers [start, stop) run `times` times over the same weights; pass p first adds loop.step[p] to X
    logits = cap * tanh(head(LN(X)) / cap)
"""

from __future__ import annotations

import math

import numpy as np


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, shift):
    """h'_t = h_t + (h_{t-1} - h_t) * shift, with zeros before the sequence."""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (prev - h) * shift


def rotary_frequencies(rot):
    """Angular step of each of the dims/2 pairs, and the factor on cos and sin.

    Plain: f_i = base^(-2i/dims).  With ``scaling`` (factor s, original length L, fast, slow): pairs that turn
    often keep f_i, pairs that turn rarely get f_i / s, and between the two a linear ramp over the pair index,
    from lo = floor(c(fast)) to hi = ceil(c(slow)), c(r) = dims ln(L / (2 pi r)) / (2 ln base), clipped to
    [0, dims-1]; cos and sin are multiplied by 0.1 ln s + 1."""
    dims, base = rot["dims"], float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    s, L = float(sc["factor"]), float(sc["original"])
    c = lambda r: dims * math.log(L / (2.0 * math.pi * r)) / (2.0 * math.log(base))
    lo = max(math.floor(c(float(sc["fast"]))), 0)
    hi = min(math.ceil(c(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / s * ramp + f * (1.0 - ramp), 0.1 * math.log(s) + 1.0


def rotate(x, rot, positions):
    """x [T, heads, dim]: the first rot.dims elements of every head turn by position * f_i, element i paired
    with element i + dims/2; the rest stay."""
    dims = rot["dims"]
    f, mag = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = np.cos(ang)[:, None, :] * mag, np.sin(ang)[:, None, :] * mag
    a, b = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.copy()
    out[..., :dims // 2] = a * cos - b * sin
    out[..., dims // 2:dims] = b * cos + a * sin
    return out


def visible(i, j, size, keep_first):
    """Whether the query at i sees the key at j: causal, and either inside the last ``size`` positions or among
    the first ``keep_first`` of the sequence (``size`` 0: no limit)."""
    if j > i:
        return False
    return size <= 0 or i - j < size or j < keep_first


def windowed_attention(h, W, p, c):
    """Softmax attention of H query heads over G key/value heads (query head a reads head a // (H/G)), rotary
    positions on q and k, score = scale <q, k>, the mask of ``visible``."""
    T = h.shape[0]
    H, G, D, DV = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, G, D)
    v = (h @ W[p + "v"].T).reshape(T, G, DV)
    pos = np.arange(T)
    if c.get("rot"):
        q, k = rotate(q, c["rot"], pos), rotate(k, c["rot"], pos)
    mask = c.get("mask") or {}
    size, keep = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
    scale = float(c.get("scale", D ** -0.5))
    out = np.zeros((T, H, DV))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, size, keep)]
            w = np.exp(s[i, js] - s[i, js].max())
            out[i, a] = (w / w.sum()) @ v[js, g]
    return out.reshape(T, H * DV) @ W[p + "o"].T


def retention(h, W, p, c, eps):
    """Linear attention with a fixed decay per head: S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, k scaled by
    dim^-1/2 after its rotation; each head's o to unit RMS, times silu of the gate projection, then the output
    projection."""
    T = h.shape[0]
    H, D, DV = c["heads"], c["dim"], c["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, DV)
    pos = np.arange(T)
    if c.get("rot"):
        q, k = rotate(q, c["rot"], pos), rotate(k, c["rot"], pos)
    k = k * D ** -0.5
    o = np.zeros((T, H, DV))
    for a in range(H):
        S = np.zeros((D, DV))
        for t in range(T):
            S = float(c["decay"][a]) * S + np.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    o = unit_rms(o, eps).reshape(T, H * DV)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h, W, p, c, eps):
    return (float(c["left_scale"]) * windowed_attention(h, W, p + "left.", c["left"])
            + float(c["right_scale"]) * retention(h, W, p + "right.", c["right"], eps))


def causal_conv(x, taps, bias):
    """y_t[c] = bias[c] + sum_j taps[c, K-1-j] x_{t-j}[c]: the last tap is the current token's, zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    y = np.tile(bias, (T, 1)).astype(np.float64)
    for j in range(K):
        y[j:] += x[:T - j] * taps[:, K - 1 - j]
    return y


def rglru(h, W, p, c):
    """Gated linear recurrence: y = gelu(Wy h + by); u = conv(Wx h + bx); per block b of the channels
    r = sigmoid(Ra_b u_b + ba_b), i = sigmoid(Ri_b u_b + bi_b); a = exp(-8 r softplus(lam));
    S_t = a S_{t-1} + sqrt(1 - a^2) i u (S_{-1} = 0); out = Wo (S * y)."""
    T = h.shape[0]
    C, B = c["width"], c["blocks"]
    y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
    u = causal_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    ub = u.reshape(T, B, C // B)
    r = sigmoid(np.einsum("tbi,boi->tbo", ub, W[p + "ra"]) + W[p + "ra.b"]).reshape(T, C)
    g = sigmoid(np.einsum("tbi,boi->tbo", ub, W[p + "ri"]) + W[p + "ri.b"]).reshape(T, C)
    a = np.exp(-8.0 * r * softplus(W[p + "lam"]))
    S = np.zeros(C)
    out = np.zeros((T, C))
    for t in range(T):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * g[t] * u[t]
        out[t] = S
    return (out * y) @ W[p + "o"].T


def dense_ff(h, W, p):
    gate = h @ W[p + "gate"].T + W[p + "gate.b"]
    up = h @ W[p + "up"].T + W[p + "up.b"]
    return (silu(gate) * up) @ W[p + "down"].T + W[p + "down.b"]


def run_order(cfg):
    """[(layer, pass or None)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop.get("times", 1)) < 1:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(start)]
    for p in range(times):
        order += [(i, p) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def layer(cfg, W, i, X):
    spec = cfg["layers"][i]
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    p = f"l{i}."
    h = token_shift(layer_norm(X, W[p + "norm1"], W[p + "norm1.b"], eps), W[p + "shift"])
    if spec["type"] == "parallel":
        mixed = parallel_mixer(h, W, p + "mix.", spec["mixer"], eps)
    elif spec["type"] == "rglru":
        mixed = rglru(h, W, p + "mix.", spec["mixer"])
    else:
        raise ValueError(spec["type"])
    X = X + m * mixed
    if spec.get("mlp") is not None:
        X = X + m * dense_ff(layer_norm(X, W[p + "norm2"], W[p + "norm2.b"], eps), W, p + "mlp.")
    return X


def forward(cfg, W, tokens, return_streams=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run)."""
    X = W["embed"][np.asarray(tokens)]
    streams = []
    loop = cfg.get("loop")
    first = int(loop["start"]) if loop else -1
    for i, p in run_order(cfg):
        if p is not None and i == first:
            X = X + W["loop.step"][p]
        X = layer(cfg, W, i, X)
        streams.append(X.copy())
    h = layer_norm(X, W["final.norm"], W["final.norm.b"], float(cfg["norm"]["eps"]))
    logits = h @ W["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    if cap > 0.0:
        logits = cap * np.tanh(logits / cap)
    return (logits, streams) if return_streams else logits


def greedy(cfg, W, prompt, n):
    """The n tokens that follow ``prompt`` when the most probable token is always taken (the lowest id on a tie)."""
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(np.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]
