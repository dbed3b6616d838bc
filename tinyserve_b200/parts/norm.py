"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in 32-bit, output in the compute
dtype (serve.py:799-809).  ``add_forward`` is the fused residual form of
serve.py:1183-1193 / tinykernels.py:26-61; here the residual stream itself stays in
32-bit between layers, so the residual sum is never rounded."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, ParamSpec, register_norm


class RMSNorm(Norm):
    capturable = True

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.dim = dim
        self.eps = float(eps)
        self.compute_dtype = None

    def prepare(self, runtime):
        self.compute_dtype = runtime.dtype

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), role="vector", init="norm_weight")}

    def forward(self, x, out=None):
        return ops.rmsnorm(x, self.w["weight"], self.eps, out=out)

    def add_forward(self, x, residual, rows=None):
        return ops.add_rmsnorm(x, residual, self.w["weight"], self.eps, self.compute_dtype, rows=rows)

    def rms_parameters(self):
        return self.w["weight"], self.eps


register_norm("rmsnorm", RMSNorm)
