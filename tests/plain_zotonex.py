"""Plain, slow implementation of the Zotonex design: whole sequences, no cache, CPU.

The oracle of the Zotonex tests.  One function for each mechanism, written from
the design's equations; it shares no code with the package and knows nothing of
pages, portions or batches: a sequence goes in whole and logits for every
position come out.  Arithmetic is done in ``dtype`` (float64 by default, so that
the oracle's own rounding is far below anything the tests judge).

The design, in this file's notation (X is the residual stream, one row a token):

    X   = E[token] * embedding.scale
    X  += mix(norm1(X));  X += ff(norm2(X))           for every layer, in order
    out = head(norm_final(X)) * logit_scale
    norm(x) = x / sqrt(mean(x^2) + eps) * w

mix is a differential attention without positions under a chunked causal mask,
ff a mixture of experts with sigmoid scores plus a gated shared expert.
"""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open


def read_folder(folder: str, dtype=torch.float64) -> tuple[dict, dict[str, torch.Tensor]]:
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as fh:
        for name in fh.keys():
            tensors[name] = fh.get_tensor(name).to(dtype)
    return cfg, tensors


# --------------------------------------------------------------------------- mechanisms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def chunk_mask(n: int, size: int | None) -> torch.Tensor:
    """[n, n] bool: query i sees key j when j <= i and both lie in the same chunk of ``size`` positions counted
    from position 0 (no size: every j <= i)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if size:
        seen &= (i // size) == (j // size)
    return seen


def keys_and_values(h: torch.Tensor, w: dict, m: dict, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """What a layer with projections of its own keeps: keys [T, G, 2, dim] after their norm, values [T, G, vdim]."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w["k"].T).view(T, G, 2, dim)
    k = unit_rms(k, eps) * w["k.norm"]
    v = (h @ w["v"].T).view(T, G, vdim)
    return k, v


def diff_lambda(w: dict, diff: float) -> float:
    """exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff: one number for the layer."""
    return math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + diff


def diff_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seen: torch.Tensor, scale: float, lam: float,
              diff: float, eps: float) -> torch.Tensor:
    """q [T, H, 2, dim] and k [S, G, 2, dim] after their norms, v [S, G, vdim], seen [T, S] bool -> [T, H * vdim].
    Each of a head's two maps is a softmax attention of its own over the same values; o = o1 - lam o2, brought to
    unit RMS over the head and multiplied by 1 - diff."""
    H, G = q.shape[1], k.shape[1]
    heads = []
    for hq in range(H):
        g = hq // (H // G)
        maps = []
        for a in range(2):
            s = (q[:, hq, a] @ k[:, g, a].T) * scale
            s = s.masked_fill(~seen, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        heads.append(unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1)


def diff_attention(h: torch.Tensor, w: dict, m: dict, eps: float, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """The mixer for one whole sequence, given the keys and values it reads (its own or another layer's)."""
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, m["heads"], 2, m["dim"])
    q = unit_rms(q, eps) * w["q.norm"]
    seen = chunk_mask(T, (m.get("mask") or {}).get("size"))
    o = diff_core(q, k, v, seen, m["scale"], diff_lambda(w, m["diff"]), m["diff"], eps)
    return o @ w["o"].T


def expert(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = (x @ gate.T).clamp(max=limit)
    u = (x @ up.T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(indices [T, top], weights [T, top]): the experts with the largest sigmoid scores and those scores as they are."""
    s = torch.sigmoid(h @ router.T)
    weights, idx = torch.topk(s, top, dim=-1)
    return idx, weights


def mixture(h: torch.Tensor, w: dict, f: dict) -> torch.Tensor:
    idx, weights = route(h, w["router"], f["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(idx[t].tolist(), weights[t]):
            out[t] += expert(p * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], f["expert"]["limit"])
    if f.get("shared"):
        s = expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], f["shared"]["limit"])
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * s
    return out


# --------------------------------------------------------------------------- the model
def sub(tensors: dict, prefix: str) -> dict:
    return {n[len(prefix):]: t for n, t in tensors.items() if n.startswith(prefix)}


def forward(cfg: dict, tensors: dict, ids, return_layers: bool = False):
    """Logits [T, vocab] of one sequence; with ``return_layers`` also the stream after every layer [L, T, width]."""
    dtype = tensors["embed"].dtype
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(ids, dtype=torch.long)
    x = tensors["embed"][ids] * cfg["embedding"]["scale"]
    kept: dict[int, tuple] = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "attention":
            raise ValueError(f"layer type {layer['type']!r}")
        m = layer["mixer"]
        w = sub(tensors, f"l{i}.mix.")
        h = rms_norm(x, tensors[f"l{i}.norm1"], eps)
        if m.get("kv_from") is None:
            kept[i] = keys_and_values(h, w, m, eps)
        k, v = kept[m["kv_from"] if m.get("kv_from") is not None else i]
        x = x + diff_attention(h, w, m, eps, k, v)
        if layer.get("mlp"):
            h = rms_norm(x, tensors[f"l{i}.norm2"], eps)
            x = x + mixture(h, sub(tensors, f"l{i}.mlp."), layer["mlp"])
        after.append(x.clone())
    logits = (rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T) * cfg["logit_scale"]
    assert logits.dtype == dtype
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(cfg: dict, tensors: dict, prompt, new_tokens: int) -> list[int]:
    """Greedy continuation, the whole sequence run again for every token."""
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(forward(cfg, tensors, ids)[-1].argmax()))
    return ids[len(prompt):]
