"""A matrix memory with exponential gates as a mixer: per request and head a matrix S, a normalizer n and a running maximum m.

With h the normed rows, per head (dk key channels, dv value channels):

    q = Wq h / sqrt(dk),  k = Wk h,  v = Wv h
    i = cap tanh((Wi h + bi) / cap),   f = logsigmoid(cap tanh((Wf h + bf) / cap))         log gates, capped
    m_t = max(f + m_(t-1), i)                                                               m starts at 0
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,   n_t likewise with k alone
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    x += Wo ( rms(o_t) per head * n * sigmoid(Wg h) )                                       n: a gain over all heads

One stacked input product (q, k, v, the gate and the two log gates' rows) leaves in float32, so that the gates and all that
enters the recurrence are 32-bit numbers in both precisions (the recurrence reads q, k and v as the product left them).

The normalizer rides through the recurrence as one more value column: n_t is the recurrence of S with a value that is always
1, and n_t . q that column's output. So the values get a column of ones behind them (`ops.memory_values`), the state is
[heads, dk, dvp] with n in column dv (dvp: dv + 1 rounded up to a multiple of 8), the recurrence needs no case of its own
(`ops.scalar_gated_recurrent` token by token; prompt portions in bfloat16 mode with key heads of 64 or 128 channels in chunks
of 64 tokens on the tensor cores, `ops.scalar_gated_chunked`), and `ops.memory_divide` takes the column out again. A request
keeps two states of fixed size, float32, zero when it opens: [S | n] and m [heads]. The gate kernel (`ops.memory_gates`)
shares a request's tokens out in runs whose maps of the running maximum compose.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedState
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Mixer, register_mixer
from .linear import Linear


def _up8(n: int) -> int:
    return -(-n // 8) * 8


class MatrixMemory(Mixer):
    can_overwrite = True
    takes_out_scale = True         # `out_scale` multiplies the result (applied in front of the output product)

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.overwrite, self.out_scale = False, 1.0
        parts = [tensors.pop(prefix + n) for n in ("q", "k", "v", "g", "i", "f")]
        self.offsets, rows, at = [], [], 0
        for w in parts:            # every piece starts at a multiple of 8 columns
            self.offsets.append(at)
            pad = _up8(w.shape[0]) - w.shape[0]
            rows.append(w)
            if pad:
                rows.append(torch.zeros((pad, dim), dtype=w.dtype, device=w.device))
            at += w.shape[0] + pad
        self.width = at
        self.inp = Linear(torch.cat(rows, dim=0).contiguous())
        del parts, rows
        self.i_bias, self.f_bias = tensors.pop(prefix + "i.b"), tensors.pop(prefix + "f.b")
        self.gain = tensors.pop(prefix + "norm")
        self.out = Linear(tensors.pop(prefix + "o"))

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, dk, dv = spec.heads, spec.key_dim, spec.value_dim
        return {prefix + "q": TensorWant((H * dk, dim)), prefix + "k": TensorWant((H * dk, dim)),
                prefix + "v": TensorWant((H * dv, dim)), prefix + "g": TensorWant((H * dv, dim)),
                prefix + "o": TensorWant((dim, H * dv)), prefix + "norm": TensorWant((H * dv,), "vector", init="gain"),
                prefix + "i": TensorWant((H, dim)), prefix + "i.b": TensorWant((H,), "vector"),
                prefix + "f": TensorWant((H, dim)), prefix + "f.b": TensorWant((H,), "vector")}

    @classmethod
    def cache_need(cls, spec):
        return (FixedState((spec.heads, spec.key_dim, cls.padded(spec.value_dim)), "float32"), FixedState((spec.heads,), "float32"))

    @staticmethod
    def padded(value_dim: int) -> int:
        """A head's value columns in the state: its values, the normalizer's column, zeros up to a multiple of 8."""
        return _up8(value_dim + 1)

    def decode_bucket_cap(self, rows: int) -> int:
        return 1

    def forward(self, xb, x, batch, cache) -> None:
        s, rows = self.spec, xb.shape[0]
        if not cache.writes or len(cache.states) < 2:
            raise ops.KernelError("a matrix memory keeps its own state: a run cannot read another run's")
        H, dk, dv = s.heads, s.key_dim, s.value_dim
        q_off, k_off, v_off, g_off, i_off, f_off = self.offsets
        proj = self.rt.buffer("memory_proj", self.width, torch.float32)[:rows]
        self.inp.forward(xb, proj)
        la = self.rt.buffer("recurrence_log_decay", H, torch.float32)[:rows]
        b = self.rt.buffer("recurrence_in_scale", H, torch.float32)[:rows]
        floor = self.rt.buffer("recurrence_floor", H, torch.float32)[:rows]
        ops.memory_gates(proj, i_off, f_off, self.i_bias, self.f_bias, s.gate_cap, cache.states[1], batch, la, b, floor, H)
        dvp = self.padded(dv)
        values = self.rt.buffer("memory_values", H * dvp, torch.float32)[:rows]
        ops.memory_values(proj, v_off, H, dv, dvp, values)
        wide = self.rt.buffer("memory_wide_out", H * dvp, torch.float32)[:rows]
        # (single rows, float32 mode and other sizes token by token: q, k and v are then read as the product left them, in
        # float32; a head's divisor |n . q| may lie near 0, where every rounding of q or k weighs most)
        chunked = (not batch.decode_only and self.rt.dtype == torch.bfloat16 and
                   ops.scalar_gated_chunked(proj, q_off, H, proj, k_off, H, values, 0, la, b, cache.states[0], batch, wide, H, dk,
                                            dvp, dk ** -0.5))
        if not chunked:
            ops.scalar_gated_recurrent(proj, q_off, H, proj, k_off, H, values, 0, la, b, cache.states[0], batch, wide, H, dk,
                                       dvp, dk ** -0.5)
        o = self.rt.buffer("memory_out", H * dv, torch.float32)[:rows]
        ops.memory_divide(wide, floor, o, H, dv, dvp)
        y = self.rt.buffer("memory_gated", H * dv)[:rows]
        ops.gated_head_norm(o, proj[:, g_off:g_off + H * dv], self.gain, s.norm_eps, self.out_scale, y, H, dv, "sigmoid",
                            gain_per_column=True)
        self.out.forward(y, x, accumulate=not self.overwrite)


register_mixer("matrix_memory", MatrixMemory, replace=True)
