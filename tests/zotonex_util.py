"""Helpers of the Zotonex tests: small configurations, random weights made to show faults, model folders."""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import save_file


def mixer(heads, kv_heads, dim, vdim, size=None, kv_from=None, scale=None, diff=0.35):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if size:
        m["mask"] = {"size": size}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, limit, shared_ff=0, shared_limit=0.0):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return f


def config(which: str) -> dict:
    """A: key rows (2 x 16) and value rows (24) of different sizes, 4 heads on 2 kv heads, chunks of 24, one layer that
       reads another's keys and values, one layer without a feed-forward, two experts of six per token.
    B: one kv head for two heads, value rows as long as key rows, no mask size (every earlier key is seen), one expert
       of three per token, no shared expert, a sharp softmax (a far key that is lost shows).
    C: sizes that are multiples of nothing (width 100, dim 24, vdim 40), chunks of 7, readers whose chunks differ from
       their writer's (10 and none), three experts of five per token.
    D: sizes that the tensor-core kernels take (dim 32 and 64, vdim 64 and 128, width 128), chunks of 48, two heads per
       kv head in one layer and four in the other."""
    if which == "A":
        layers = [{"type": "attention", "mixer": mixer(4, 2, 16, 24, 24), "mlp": moe(6, 2, 40, 1.5, 56, 1.0)},
                  {"type": "attention", "mixer": mixer(4, 2, 16, 24, 24, kv_from=0), "mlp": moe(6, 2, 40, 1.5, 56, 1.0)},
                  {"type": "attention", "mixer": mixer(2, 2, 8, 16, 24), "mlp": None}]
        return _model(211, 96, layers, 1e-5, 9.5, 0.7)
    if which == "B":
        layers = [{"type": "attention", "mixer": mixer(2, 1, 32, 64, None, scale=0.9, diff=0.2), "mlp": moe(3, 1, 48, 2.5)},
                  {"type": "attention", "mixer": mixer(2, 1, 32, 64, None, kv_from=0, scale=0.9, diff=0.2), "mlp": moe(3, 1, 48, 2.5)}]
        return _model(300, 64, layers, 1e-6, 8.0, 1.0)
    if which == "C":
        layers = [{"type": "attention", "mixer": mixer(3, 3, 24, 40, 7), "mlp": moe(5, 3, 36, 1.0, 20, 3.0)},
                  {"type": "attention", "mixer": mixer(3, 3, 24, 40, 10, kv_from=0), "mlp": moe(5, 3, 36, 1.0, 20, 3.0)},
                  {"type": "attention", "mixer": mixer(3, 3, 24, 40, None, kv_from=0), "mlp": None}]
        return _model(157, 100, layers, 1e-5, 10.0, 0.25)
    if which == "D":
        layers = [{"type": "attention", "mixer": mixer(4, 2, 32, 64, 48), "mlp": moe(4, 2, 72, 2.25, 136, 1.25)},
                  {"type": "attention", "mixer": mixer(4, 1, 64, 128, 48), "mlp": moe(4, 2, 72, 2.25, 136, 1.25)},
                  {"type": "attention", "mixer": mixer(4, 1, 64, 128, 80, kv_from=1), "mlp": None}]
        return _model(320, 128, layers, 1e-5, 11.3, 0.5)
    raise KeyError(which)


def _model(vocab, width, layers, eps, emb_scale, logit_scale) -> dict:
    return {"architecture": "Zotonex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb_scale},
            "logit_scale": logit_scale, "layers": layers}


def random_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors by the design's names.  Matrices have unit-variance outputs for unit-variance inputs, so that
    clamps bite, gates are neither all open nor all shut and routers have clear favourites; norm weights lie around 1;
    the lambda vectors are large enough for lambda to differ from ``diff`` in its first digit."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(torch.bfloat16)

    def around_one(n):
        return (1.0 + 0.2 * torch.randn(n, generator=g)).to(torch.bfloat16)

    t = {"embed": (torch.randn(V, W, generator=g) / cfg["embedding"]["scale"]).to(torch.bfloat16), "final.norm": around_one(W),
         "head": mat(V, W)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        t[p + "norm1"] = around_one(W)
        t[p + "mix.q"] = mat(m["heads"] * 2 * m["dim"], W)
        t[p + "mix.q.norm"] = around_one(m["dim"])
        if m.get("kv_from") is None:
            t[p + "mix.k"] = mat(m["kv_heads"] * 2 * m["dim"], W)
            t[p + "mix.v"] = mat(m["kv_heads"] * m["vdim"], W)
            t[p + "mix.k.norm"] = around_one(m["dim"])
        for name in ("lq1", "lk1", "lq2", "lk2"):
            t[p + "mix." + name] = (0.5 * torch.randn(m["dim"], generator=g) / m["dim"] ** 0.25).to(torch.bfloat16)
        t[p + "mix.o"] = mat(W, m["heads"] * m["vdim"])
        f = layer.get("mlp")
        if f:
            t[p + "norm2"] = around_one(W)
            t[p + "mlp.router"] = mat(f["router"]["experts"], W, 2.0)
            for e in range(f["router"]["experts"]):
                t[p + f"mlp.e{e}.gate"] = mat(f["expert"]["ff"], W, 1.5)
                t[p + f"mlp.e{e}.up"] = mat(f["expert"]["ff"], W, 1.5)
                t[p + f"mlp.e{e}.down"] = mat(W, f["expert"]["ff"])
            if f.get("shared"):
                t[p + "mlp.shared.gate"] = mat(f["shared"]["ff"], W, 1.5)
                t[p + "mlp.shared.up"] = mat(f["shared"]["ff"], W, 1.5)
                t[p + "mlp.shared.down"] = mat(W, f["shared"]["ff"])
                t[p + "mlp.shared.sg"] = mat(1, W, 2.0)
    return t


def write_model(folder: str, cfg: dict, seed: int) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh)
    save_file({n: t.contiguous() for n, t in random_weights(cfg, seed).items()}, os.path.join(folder, "model.safetensors"))
    return folder


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: the root mean square of the difference, each side's mean taken off, over that of the wanted row."""
    got, want = got.double(), want.double()
    d = (got - got.mean(-1, keepdim=True)) - (want - want.mean(-1, keepdim=True))
    ref = (want - want.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt().clamp_min(1e-12)
    return d.pow(2).mean(-1).sqrt() / ref
