"""Layer norm with a gain and no bias: ``(x - mean) / sqrt(mean((x - mean)^2) + eps) * gain``, statistics and
scaling in float.  The gain is float32 on the device however it is stored."""

from __future__ import annotations

import torch

from .. import ops
from .base import ParamSpec, Part, bytes_of


class LayerNorm(Part):
    def param_specs(self):
        return {"weight": ParamSpec((self.spec.size,), "gain32")}

    def set_params(self, params):
        self.weight = params["weight"].float().contiguous()

    def for_kernel(self):
        """``(kind, gain, eps)`` as the kernels that fuse a norm take it."""
        return "layernorm", self.weight, self.spec.eps

    def __call__(self, x):
        """The norm of the rows of ``x`` (float32 rows are normed into float32; rows of the working type
        are widened first)."""
        base = x if x.dtype == torch.float32 else x.float()
        return ops.depth_step(base.contiguous(), x.dtype, norm=self.for_kernel())

    def add(self, residual, delta):
        raise TypeError("layer norm stands in arrangements that keep a float32 residual stream; the pre-norm block "
                        "with a stream of the working type fuses RMS norms")

    add_rows = add

    def weight_bytes(self):
        return bytes_of(self.weight)
