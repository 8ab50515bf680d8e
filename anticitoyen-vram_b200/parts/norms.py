"""RMS norm with the residual sum fused in."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import Norm, Runtime
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """out = cast(x32 * rsqrt(mean(x32^2) + eps)) * w, the weight being plain ``w``
    (acvram/engine/layers.py:607-630); with ``delta`` the sum x + delta is made first,
    in 32-bit, and written back (acvram/engine/layers.py:633-651)."""

    def __init__(self, hidden_size: int, eps: float, size: int | None = None, tensor: str = "weight") -> None:
        """``tensor``: the weight's name behind the norm's prefix ("" where the prefix is the whole name)."""
        self.size = size or hidden_size
        self.eps = float(eps)
        self.tensor = tensor
        self.weight: torch.Tensor | None = None

    def tensor_needs(self):
        return {self.tensor: TensorNeed((self.size,), "norm")}

    def load(self, tensors, rt: Runtime) -> None:
        self.weight = tensors[self.tensor].to(device=rt.device, dtype=torch.float32).contiguous()

    def decode_layer_spec(self):
        """What the fused decode-layer kernel needs of this norm."""
        return {"weight": self.weight, "eps": self.eps}

    def weight_bytes(self) -> int:
        return 0 if self.weight is None else self.weight.numel() * 4

    def forward(self, x, delta, rows=None, out_dtype=None):
        """A float32 stream beside parts that run in ``out_dtype`` (bfloat16): sum and norm stay 32-bit, the norm's output
        is rounded once."""
        n = rows.shape[0] if rows is not None else x.shape[0]
        out_dtype = out_dtype or (delta.dtype if delta is not None else x.dtype)
        out = torch.empty((n, x.shape[1]), device=x.device, dtype=out_dtype)
        if x.dtype == torch.float32 and out_dtype != torch.float32:
            return ops.add_rmsnorm_f32(x, delta, self.weight, self.eps, out, rows)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
