"""The Redudra design as a plan of parts.

Pre-norm layers (``layernorm`` with weight and bias) over a float32 residual
stream, each with a token shift in front of its mixer and the constant
``residual_mult`` on what it adds.  A ``parallel`` layer's mixer is ``parallel``:
``attention`` (grouped queries, value rows of their own size, rotary positions
with YaRN scaling over part of the head, a sliding window that keeps a request's
first tokens) beside ``retention`` (fixed decay per head, rotary positions, unit
RMS per head, a silu gate), summed with the two weights.  An ``rglru`` layer's
mixer is the gated linear recurrence.  The feed-forward is ``swiglu`` with
biases, or absent.  A looped stretch of layers appears in the schedule once for
every pass, each run with a cache slot of its own, and the first layer of a pass
is preceded by that pass's row of ``loop.step``.

What the design fixes is written here as parameters of the parts; what a model
of the design may choose comes from ``RedudraConfig``.
"""

from __future__ import annotations

from ..config.redudra import MAX_POSITIONS, ParallelSpec, RedudraConfig, RotarySpec
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

RECURRENCE_RATE = 8.0       # a = exp(-8 r softplus(lam)) in the gated recurrence
LOOP_VECTORS = "loop.step"  # [times, width]: row p joins the stream before pass p of the looped layers


def _rotary(rot: RotarySpec | None) -> PartSpec | None:
    if rot is None:
        return None
    return PartSpec("rotary", {"dim": rot.dims, "theta": rot.base, "max_positions": MAX_POSITIONS,
                               "scaling": rot.scaling, "exact": True})


def _parallel(m: ParallelSpec, eps: float) -> PartSpec:
    l, r = m.left, m.right
    left = PartSpec("attention", {
        "num_heads": l.heads, "num_kv_heads": l.kv_heads, "head_dim": l.dim, "value_dim": l.vdim, "scale": l.scale,
        "window": l.window, "keep_first": l.keep_first, "position": _rotary(l.rot) or PartSpec("none"),
        "prefix": "mix.left.", "names": {n: n for n in ("q", "k", "v", "o")}, "bias": False, "out_scale": m.left_scale})
    right = PartSpec("retention", {
        "num_heads": r.heads, "dim": r.dim, "value_dim": r.vdim, "decay": r.decay, "norm_eps": eps,
        "position": _rotary(r.rot), "prefix": "mix.right.", "out_scale": m.right_scale})
    return PartSpec("parallel", {"left": left, "right": right})


def redudra_plan(cfg: RedudraConfig) -> ModelPlan:
    norm = PartSpec("layernorm", {"eps": cfg.norm_eps, "tensor": "", "bias_tensor": ".b"})
    options = {"residual_mult": cfg.residual_mult, "token_shift": "shift"}
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.type == "parallel":
            mixer = _parallel(layer.mixer, cfg.norm_eps)
        else:
            m = layer.mixer
            mixer = PartSpec("rglru", {"width": m.width, "blocks": m.blocks, "conv": m.conv, "rate": RECURRENCE_RATE,
                                       "prefix": "mix."})
        ff = None
        if layer.ff:
            ff = PartSpec("swiglu", {"intermediate_size": layer.ff, "prefix": "mlp.", "bias": True, "names": {
                "gate": "gate", "gate.bias": "gate.b", "up": "up", "up.bias": "up.b", "down": "down", "down.bias": "down.b"}})
        layers.append(LayerSpec(f"l{i}.", "prenorm", mixer, ff, norm, norm_prefixes=("norm1", "norm2"), options=options))
    n = len(layers)
    if cfg.loop is None:
        order = [(i, None) for i in range(n)]
    else:
        start, stop, times = cfg.loop
        order = [(i, None) for i in range(start)]
        for p in range(times):
            order += [(i, p if i == start else None) for i in range(start, stop)]
        order += [(i, None) for i in range(stop, n)]
    # every run of a layer keeps its own pages and states
    schedule = tuple(ScheduleEntry(i, slot, True, (LOOP_VECTORS, p) if p is not None else None)
                     for slot, (i, p) in enumerate(order))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=schedule, final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        head_name="head", tied_head=False, residual_dtype="float32", logit_softcap=cfg.logit_softcap,
        stream_vectors={LOOP_VECTORS: (cfg.loop[2], cfg.width)} if cfg.loop is not None else {})


register_architecture("Redudra", RedudraConfig, redudra_plan)
