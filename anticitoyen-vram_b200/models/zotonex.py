"""The Zotonex design as a plan of parts.

Pre-norm layers over a float32 residual stream; the mixer is ``diff_attention``
(two softmax maps per head over shared values, combined as o1 - lambda o2 and
brought to unit RMS per head) with no position encoding and a chunked causal
mask; a layer whose mixer names ``kv_from`` has no key/value projections and
reads the cache slot that the named layer writes; the feed-forward is ``moe``
(sigmoid scores, the chosen scores as weights on the experts' input, clamped
gated experts, a shared expert behind a sigmoid gate), or absent.  The
embedding is scaled on its way in, the logits on their way out.

What the design fixes is written here as parameters of the parts; what a model
of the design may choose comes from ``ZotonexConfig``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zotonex import MAX_POSITIONS, ZotonexConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

SWISH_ALPHA = 1.702     # of the experts' activation g * sigmoid(alpha g) * (u + 1)


def zotonex_plan(cfg: ZotonexConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps, "tensor": ""})
    layers, schedule = [], []
    slot_of_layer: dict[int, int] = {}
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        own = m.kv_from is None
        if own:
            slot_of_layer[i] = len(slot_of_layer)
        mixer = PartSpec("diff_attention", {
            "num_heads": m.heads, "num_kv_heads": m.kv_heads, "dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
            "diff": m.diff, "norm_eps": cfg.norm_eps, "chunk": m.mask_size, "own_kv": own, "prefix": "mix."})
        ff = None
        if layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec("moe", {
                "experts": f.experts, "top": f.top, "expert_ff": f.ff, "expert_limit": f.limit, "shared_ff": f.shared_ff,
                "shared_limit": f.shared_limit, "alpha": SWISH_ALPHA, "scoring": "sigmoid", "renormalize": False,
                "weight_on": "input", "prefix": "mlp."})
        layers.append(LayerSpec(f"l{i}.", "prenorm", mixer, ff, norm, norm_prefixes=("norm1", "norm2")))
        schedule.append(ScheduleEntry(i, slot_of_layer[i if own else m.kv_from], own))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, embedding_name="embed",
        final_norm_prefix="final.norm", head_name="head", tied_head=False, embedding_scale=cfg.embedding_scale,
        logit_scale=cfg.logit_scale, residual_dtype="float32")


register_architecture("Zotonex", ZotonexConfig, zotonex_plan)
