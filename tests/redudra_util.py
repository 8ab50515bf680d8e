"""Helpers of the Redudra tests: small configurations, random weights made to show faults, model folders."""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch
from safetensors.torch import save_file


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def left(heads, kv_heads, dim, vdim, size=0, keep=0, rotary=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if size:
        m["mask"] = {"size": size, "keep_first": keep}
    if rotary:
        m["rot"] = rotary
    return m


def right(heads, dim, vdim, decay, rotary=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rotary:
        m["rot"] = rotary
    return m


def parallel(l, r, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": ls, "right_scale": rs},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def rglru(width, blocks, conv, ff):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(which: str) -> dict:
    """A: key rows (16) and value rows (24) of different sizes, 4 heads on 2 kv heads, a window of 20 that keeps 3 first
       tokens, rotary over half of the head with scaling, a recurrence narrower than the model, a layer without
       feed-forward, the first two layers looped three times.
    B: what the other models happen to leave out or make 1: no loop, no soft cap, residual factor 1, both side weights 1, a window
       without kept tokens and a layer without any window, as many kv heads as heads, one block, a convolution of one
       tap, retention without positions, rotary over the whole head without scaling, a sharp softmax.
    C: sizes that are multiples of nothing (width 100, dim 24, vdim 40, 3 heads), a window of 7 (less than a page) that
       keeps 9 (more than the window), five taps, five blocks, the last layer alone looped twice.
    D: sizes that the tensor-core kernels take (dim = vdim = 64 and 128, width 128), windows of 48 and 80 keeping 4 and 16,
       the middle layer looped twice.
    E: see below."""
    if which == "A":
        layers = [parallel(left(4, 2, 16, 24, 20, 3, rot(5000.0, 8, (3.0, 64, 8.0, 1.0))), right(3, 8, 16, (0.9, 0.97, 0.995), rot(300.0, 8)), 0.7, 0.4, 80),
                  rglru(64, 2, 3, 0),
                  parallel(left(2, 1, 16, 8, 33, 1, rot(5000.0, 16, (3.0, 64, 8.0, 1.0))), right(2, 16, 8, (0.95, 0.99), rot(300.0, 4)), 0.5, 0.9, 72)]
        return _model(211, 96, layers, 1e-5, 0.4, 25.0, (0, 2, 3))
    if which == "B":
        layers = [rglru(64, 1, 1, 96),
                  parallel(left(2, 2, 32, 32, 24, 0, rot(10000.0, 32), scale=0.9), right(1, 32, 32, (0.98,)), 1.0, 1.0, 96),
                  parallel(left(2, 2, 32, 32, 0, 0, rot(10000.0, 32), scale=0.9), right(1, 32, 32, (0.98,)), 1.0, 1.0, 96)]
        return _model(300, 64, layers, 1e-6, 1.0, 0.0, None)
    if which == "C":
        layers = [parallel(left(3, 3, 24, 40, 7, 9, rot(777.0, 10, (2.5, 40, 4.0, 0.5))), right(5, 12, 20, (0.8, 0.9, 0.95, 0.99, 0.999), rot(50.0, 12)), 0.3, 1.2, 60),
                  rglru(100, 5, 5, 36)]
        return _model(157, 100, layers, 1e-5, 0.6, 12.0, (1, 2, 2))
    if which == "D":
        layers = [parallel(left(4, 2, 64, 64, 48, 4, rot(30000.0, 64, (3.0, 128, 16.0, 1.0))), right(2, 64, 64, (0.97, 0.995), rot(1000.0, 64)), 0.65, 0.45, 160),
                  rglru(128, 4, 4, 160),
                  parallel(left(2, 1, 128, 128, 80, 16, rot(30000.0, 64)), right(2, 32, 64, (0.9, 0.99), rot(1000.0, 32)), 0.8, 0.3, 0)]
        return _model(320, 128, layers, 1e-6, 0.5, 28.0, (1, 2, 2))
    if which == "E":      # an attention of the tensor-core kernels' sizes beside a retention whose sizes leave the
        # stacked projection's rows unaligned (358 elements) and the output projection's inputs odd (149)
        layers = [parallel(left(2, 1, 64, 64, 40, 2, rot(900.0, 32)), right(3, 10, 7, (0.9, 0.95, 0.99), rot(70.0, 10)), 0.9, 1.1, 56),
                  rglru(48, 3, 2, 0)]
        return _model(131, 72, layers, 1e-5, 0.7, 0.0, (0, 1, 2))
    raise KeyError(which)


def _model(vocab, width, layers, eps, mult, cap, loop) -> dict:
    cfg = {"architecture": "Redudra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if cap:
        cfg["logit_softcap"] = cap
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors by the design's names.  Matrices have unit-variance outputs for unit-variance inputs; norm weights
    lie around 1 with biases of a tenth; shift vectors lie in (0, 1); decay parameters are spread so that some channels
    forget within a few tokens and others keep hundreds; gate biases make the gates neither all open nor all shut."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    bf = lambda t: t.to(torch.bfloat16)
    mat = lambda out, inp, gain=1.0: bf(torch.randn(out, inp, generator=g) * gain / math.sqrt(inp))
    around_one = lambda n: bf(1.0 + 0.2 * torch.randn(n, generator=g))
    small = lambda *n: bf(0.1 * torch.randn(*n, generator=g))
    t = {"embed": bf(torch.randn(V, W, generator=g)), "final.norm": around_one(W), "final.norm.b": small(W), "head": mat(V, W, 3.0)}
    if cfg.get("loop"):
        t["loop.step"] = bf(0.5 * torch.randn(cfg["loop"]["times"], W, generator=g))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        t[p + "norm1"], t[p + "norm1.b"] = around_one(W), small(W)
        t[p + "shift"] = bf(torch.rand(W, generator=g))
        if layer["type"] == "parallel":
            l, r = m["left"], m["right"]
            t[p + "mix.left.q"] = mat(l["heads"] * l["dim"], W)
            t[p + "mix.left.k"] = mat(l["kv_heads"] * l["dim"], W)
            t[p + "mix.left.v"] = mat(l["kv_heads"] * l["vdim"], W)
            t[p + "mix.left.o"] = mat(W, l["heads"] * l["vdim"])
            t[p + "mix.right.q"] = mat(r["heads"] * r["dim"], W)
            t[p + "mix.right.k"] = mat(r["heads"] * r["dim"], W)
            t[p + "mix.right.v"] = mat(r["heads"] * r["vdim"], W)
            t[p + "mix.right.g"] = mat(r["heads"] * r["vdim"], W)
            t[p + "mix.right.o"] = mat(W, r["heads"] * r["vdim"])
        else:
            C, B = m["width"], m["blocks"]
            for n in ("y", "x"):
                t[p + "mix." + n], t[p + "mix." + n + ".b"] = mat(C, W), small(C)
            t[p + "mix.conv"] = bf(torch.randn(C, m["conv"], generator=g) / math.sqrt(m["conv"]))
            t[p + "mix.conv.b"] = small(C)
            for n in ("ra", "ri"):
                t[p + "mix." + n] = bf(torch.randn(B, C // B, C // B, generator=g) / math.sqrt(C // B))
                t[p + "mix." + n + ".b"] = bf(0.5 * torch.randn(B, C // B, generator=g))
            t[p + "mix.lam"] = bf(torch.linspace(-6.0, 1.0, C)[torch.randperm(C, generator=g)])
            t[p + "mix.o"] = mat(W, C)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            t[p + "norm2"], t[p + "norm2.b"] = around_one(W), small(W)
            for n, (o, i_) in (("gate", (F, W)), ("up", (F, W)), ("down", (W, F))):
                t[p + "mlp." + n], t[p + "mlp." + n + ".b"] = mat(o, i_, 1.5 if n != "down" else 1.0), small(o)
    return t


def write_model(folder: str, cfg: dict, seed: int, weights: dict | None = None) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh)
    weights = weights if weights is not None else random_weights(cfg, seed)
    save_file({n: t.contiguous() for n, t in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def read_folder(folder: str):
    """(config dictionary, {name: float64 numpy array}) of a model folder."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json"), encoding="utf-8") as fh:
        cfg = json.load(fh)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k).to(torch.float64).numpy()
    return cfg, tensors


def row_errors(got, want) -> np.ndarray:
    """Per row: the root mean square of the difference, each side's mean taken off, over that of the wanted row."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = (got - got.mean(-1, keepdims=True)) - (want - want.mean(-1, keepdims=True))
    ref = np.maximum(np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean(-1)), 1e-12)
    return np.sqrt((d ** 2).mean(-1)) / ref
