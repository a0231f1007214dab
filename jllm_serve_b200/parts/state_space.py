"""A selective state space as a mixer: a recurrent state per request and head, a step size and inputs that depend on the token.

With h the normed rows, inner = heads x head_dim, N = state, G = groups:

    [z | u | dt] = Win h                      z: inner; u: inner + 2 G N channels (x, B, C); dt: heads
    u_t <- silu(bias + sum_r conv[:, r] u_(t - taps + 1 + r))            a causal convolution per channel, zeros (or the request's
                                                                         last taps - 1 inputs) in front of the rows
    dt <- softplus(dt + dt_bias);  per head, with B and C of group h // (heads / G):
    S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,   y_t = S_t^T C_t + D x_t            (S [N, head_dim], float32)
    x += Wo ( rms_parts(y * silu(z)) * n )                               the gate first, then the norm in `norm_groups` equal parts

The input product leaves in float32, so that the step sizes, the decays and everything else that enters the recurrence
beside the projections are 32-bit numbers in both precisions; the convolution reads and writes float32 too. A
request keeps two states of fixed size: S [heads, N, head_dim] and the convolution's last taps - 1 inputs [taps - 1,
channels], both float32, both zero when the request opens. The recurrence is `ops.scalar_gated_recurrent` (one decay per head
and token; keys B and queries C shared by the heads of a group; the skip D), which other mixers share.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedState
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Mixer, register_mixer
from .linear import Linear


class SelectiveStateSpace(Mixer):
    can_overwrite = True           # a mixer of mixers asks for x = ... instead of x += ...
    takes_out_scale = True         # `out_scale` multiplies the result (applied in front of the output product)

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.overwrite, self.out_scale = False, 1.0
        self.inp = Linear(tensors.pop(prefix + "in"))
        self.conv, self.conv_bias = tensors.pop(prefix + "conv"), tensors.pop(prefix + "conv.b")
        self.dt_bias, self.a_log, self.skip = (tensors.pop(prefix + n) for n in ("dt_bias", "A_log", "D"))
        self.gain = tensors.pop(prefix + "norm")
        self.out = Linear(tensors.pop(prefix + "o"))
        self.width = 2 * spec.inner + 2 * spec.groups * spec.state + spec.heads

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, inner, C = spec.heads, spec.inner, spec.conv_channels
        return {prefix + "in": TensorWant((inner + C + H, dim)), prefix + "conv": TensorWant((C, spec.conv), "vector"),
                prefix + "conv.b": TensorWant((C,), "vector"), prefix + "dt_bias": TensorWant((H,), "vector"),
                prefix + "A_log": TensorWant((H,), "vector"), prefix + "D": TensorWant((H,), "vector", init="gain"),
                prefix + "norm": TensorWant((inner,), "vector", init="gain"), prefix + "o": TensorWant((dim, inner))}

    @classmethod
    def cache_need(cls, spec):
        return (FixedState((spec.heads, spec.state, spec.head_dim), "float32"),
                FixedState((max(spec.conv - 1, 1), spec.conv_channels), "float32"))      # (a row even with one tap: no empty state)

    def decode_bucket_cap(self, rows: int) -> int:
        return 1                       # nothing here looks at the context's length

    def forward(self, xb, x, batch, cache) -> None:
        s, rows = self.spec, xb.shape[0]
        if not cache.writes or len(cache.states) < 2:
            raise ops.KernelError("a state space keeps its own state: a run cannot read another run's")
        H, P, N, G, inner, C = s.heads, s.head_dim, s.state, s.groups, s.inner, s.conv_channels
        proj = self.rt.buffer("ssm_proj", self.width, torch.float32)[:rows]
        self.inp.forward(xb, proj)
        mixed = self.rt.buffer("ssm_conv", C, torch.float32)[:rows]
        ops.causal_conv(proj, inner, C, self.conv, self.conv_bias, cache.states[1], batch, mixed)
        la = self.rt.buffer("recurrence_log_decay", H, torch.float32)[:rows]
        b = self.rt.buffer("recurrence_in_scale", H, torch.float32)[:rows]
        ops.ssm_gates(proj[:, inner + C:inner + C + H], self.dt_bias, self.a_log, la, b)
        y = self.rt.buffer("ssm_out", inner, torch.float32)[:rows]
        # keys B at column inner, queries C at inner + G N, values x at 0 of the convolution's result. Prompt portions in
        # bfloat16 mode with states of 64 or 128 values go through the tensor cores in chunks of 64 tokens; everything else
        # (single rows, float32 mode, other sizes) token by token
        chunked = (not batch.decode_only and self.rt.dtype == torch.bfloat16 and
                   ops.scalar_gated_chunked(mixed, inner + G * N, G, mixed, inner, G, mixed, 0, la, b, cache.states[0], batch, y, H, N,
                                            P, 1.0, skip=self.skip))
        if not chunked:
            ops.scalar_gated_recurrent(mixed, inner + G * N, G, mixed, inner, G, mixed, 0, la, b, cache.states[0], batch, y, H, N,
                                       P, 1.0, skip=self.skip)
        gated = self.rt.buffer("ssm_gated", inner)[:rows]
        ops.gated_head_norm(y, proj[:, :inner], self.gain, s.norm_eps, self.out_scale, gated, s.norm_groups, inner // s.norm_groups,
                            "silu", gate_first=True, gain_per_column=True)
        self.out.forward(gated, x, accumulate=not self.overwrite)


register_mixer("selective_state_space", SelectiveStateSpace, replace=True)
