"""RMSNorm as a part: y = (x * (1 / sqrt(mean(x^2) + eps))) * gain.

Formula and order of the multiplications from the reference
(src/main/java/org/robomiri/jllm/cpu/VectorKernels.java:630-634,675-685). The input is the
float32 residual stream; the output has the compute dtype. The gain stays in the dtype it
was stored in (bfloat16 or float32): the kernel reads either.
"""
from __future__ import annotations

from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Norm, register_norm


class RmsNorm(Norm):
    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.eps = float(spec.eps)
        self.dim = dim
        self.gain = tensors[prefix + getattr(spec, "gain_name", "weight")]

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        return {prefix + getattr(spec, "gain_name", "weight"): TensorWant((dim,), "vector", init="gain")}

    def forward(self, x, out, row_index=None, rows=None):
        ops.rmsnorm(x, self.gain, self.eps, out, row_index, rows)


register_norm("rmsnorm", RmsNorm, replace=True)


class DynamicTanh(Norm):
    """y = tanh(a * x) * w + b: a norm without statistics (no mean, no variance, no eps), `a` one stored scalar. The
    tensors lie beside one another under the norm's own name: `<name>` (w), `<name>.b`, `<name>.alpha`."""

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.dim = dim
        self.weight, self.bias = tensors[prefix], tensors[prefix + ".b"]
        if self.bias.dtype != self.weight.dtype:
            self.bias = self.bias.to(self.weight.dtype)
        self.alpha = float(tensors[prefix + ".alpha"].float().item())

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        return {prefix: TensorWant((dim,), "vector", init="gain"), prefix + ".b": TensorWant((dim,), "vector"),
                prefix + ".alpha": TensorWant((), "vector", init="gain")}

    def forward(self, x, out, row_index=None, rows=None):
        ops.dynamic_tanh(x, self.weight, self.bias, self.alpha, out, row_index, rows)


register_norm("dynamic_tanh", DynamicTanh, replace=True)


class LayerNorm(Norm):
    """y = (x - m) / sqrt(v + eps) * g over a row, m its mean and v its mean squared deviation from m; a gain g and no
    bias. Float32 arithmetic; the output has the compute dtype. `out_scale` multiplies the result (1 unless a model sets it)."""

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.eps = float(spec.eps)
        self.dim = dim
        self.gain = tensors[prefix + getattr(spec, "gain_name", "weight")]

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        return {prefix + getattr(spec, "gain_name", "weight"): TensorWant((dim,), "vector", init="gain")}

    def forward(self, x, out, row_index=None, rows=None):
        ops.layernorm(x, self.gain, self.eps, out, row_index, rows, center=True)


register_norm("layernorm", LayerNorm, replace=True)
