"""The dense gated feed-forward: x += Wdown (act(Wgate xb) * (Wup xb)), act = silu or the tanh form of GELU; or, as
`swish_clamped`, x += Wdown (g sigmoid(1.702 g) (u + 1)) with g = min(Wgate xb, limit) and u = clamp(Wup xb, -limit, limit).

Formula from the reference (src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:661-669,
silu at cpu/VectorKernels.java:637-639). As the reference's converter does
(model/ModelConverter.java:380-382), gate and up are stacked into one [2 * hidden, dim]
matrix at load, rows [0, hidden) gate and [hidden, 2 hidden) up, so one product feeds both.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorWant
from .base import FeedForward, register_feed_forward
from .linear import Linear


class DenseGlu(FeedForward):
    can_overwrite = True           # a block that norms the result before adding it asks for x = ... instead of x += ...

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.hidden, self.dim, self.rt = spec.hidden, dim, runtime
        names = getattr(spec, "names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        self.activation = getattr(spec, "activation", "silu")      # silu | gelu_tanh | swish_clamped: the kernels' epilogues take any
        self.limit = float(getattr(spec, "limit", 0.0))
        # what the products' epilogues are told: the activation's number, or for the clamped unit its number and limit
        self.glu = ops.glu_descriptor(self.activation, self.limit)
        self.overwrite = False                                      # True: the result replaces x instead of being added to it
        gate, up = tensors.pop(prefix + names[0]), tensors.pop(prefix + names[1])
        # bfloat16: blocks of 8 gate rows followed by their 8 up rows, so that the product's epilogue holds a
        # gate value and its up value together and applies SwiGLU itself (no [rows, 2 hidden] round trip)
        self.fused = gate.dtype == torch.bfloat16 and dim % 8 == 0 and spec.hidden % 8 == 0
        if self.fused:
            stacked = torch.stack([gate.view(spec.hidden // 8, 8, dim), up.view(spec.hidden // 8, 8, dim)], dim=1)
            self.gate_up = Linear(stacked.reshape(2 * spec.hidden, dim).contiguous())
            del stacked
        else:
            self.gate_up = Linear(torch.cat([gate, up], dim=0).contiguous())
        del gate, up
        self.down = Linear(tensors.pop(prefix + names[2]))

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        names = getattr(spec, "names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        return {prefix + names[0]: TensorWant((spec.hidden, dim)),
                prefix + names[1]: TensorWant((spec.hidden, dim)),
                prefix + names[2]: TensorWant((dim, spec.hidden))}

    def forward(self, xb, x, batch) -> None:
        rows = xb.shape[0]
        h = self.rt.buffer("ffn_hidden", self.hidden)[:rows]
        if self.fused:
            self.gate_up.forward(xb, h, swiglu=self.glu)
        else:
            gate_up = self.rt.buffer("gate_up", 2 * self.hidden)[:rows]
            self.gate_up.forward(xb, gate_up)
            if self.activation == "swish_clamped":
                ops.glu_clamped(gate_up, None, h, 1, self.hidden, self.limit)
            else:
                ops.swiglu(gate_up, h, self.activation)
        self.down.forward(h, x, accumulate=not self.overwrite)


register_feed_forward("dense_glu", DenseGlu, replace=True)


class DenseMlp(FeedForward):
    """x += Wdown act(Wup xb): two matrices and no gate; act the erf form of GELU, applied in place between the products."""
    can_overwrite = True

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.hidden, self.dim, self.rt, self.activation = spec.hidden, dim, runtime, spec.activation
        self.overwrite = False
        self.up = Linear(tensors.pop(prefix + spec.names[0]))
        self.down = Linear(tensors.pop(prefix + spec.names[1]))

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        return {prefix + spec.names[0]: TensorWant((spec.hidden, dim)), prefix + spec.names[1]: TensorWant((dim, spec.hidden))}

    def forward(self, xb, x, batch) -> None:
        h = self.rt.buffer("ffn_hidden", self.hidden)[:xb.shape[0]]
        self.up.forward(xb, h)
        ops.activation(h, self.activation)
        self.down.forward(h, x, accumulate=not self.overwrite)


register_feed_forward("dense_mlp", DenseMlp, replace=True)
