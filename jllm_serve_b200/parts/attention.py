"""Grouped-query causal attention over the paged cache, with optional per-head q/k RMSNorm and RoPE.

Order of operations from the reference (src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:
422-458,595-615): q, k, v projections (biases if configured); RMSNorm of every query and key
head with the shared gains `q_norm` / `k_norm`; rotation; keys and values into the cache;
attention of every row over its request's keys [first, position]; `x += att @ Wo^T`.
Query head h reads kv head h // (heads / kv_heads) (cpu/KvCache.java:82,527). q, k and v
are one stacked [Q + 2 KV, dim] matrix, as the reference's fused `matmul3`.

A run that reads another run's cache (`cache.writes == False`) projects queries only.

What a spec may ask for beyond that: value heads of another width than key heads (a cache row is as wide as the wider of
the two); rotation of interleaved pairs; q and k divided by their root mean square behind the rotation; a chunk mask (a row
sees the earlier rows of its own chunk of the sequence only); a sigmoid gate per head, read from the mixer's input by rows
that ride at the end of the stacked projection. These run through the general per-head kernel (`ops.head_prepare`) and
the gate kernel; the attention itself is `ops.attention` for every form.

Further: a window that keeps the sequence's first `keep_first` positions visible to every later row (they keep their true
positions; the cache never gives their pages back); a learned sink per query head, a number whose exponential joins the
softmax's denominator without a key or a value; a sigmoid gate of FULL width (one gate value per value of the concatenated
heads, `gate = "sigmoid"`), whose rows also ride at the end of the stacked projection; and `out_scale`, a factor on the
mixer's result that a mixer of mixers sets (applied together with the gate, in front of the output projection).
"""
from __future__ import annotations

import torch

from ..cache.manager import PagedKeysValues
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Mixer, register_mixer
from .linear import Linear


def _up8(n: int) -> int:
    return -(-n // 8) * 8


class GqaAttention(Mixer):
    can_overwrite = True           # a block that norms the result before adding it asks for x = ... instead of x += ...
    takes_out_scale = True         # `out_scale` multiplies the result (applied in front of the output product)

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, rope=None):
        self.spec, self.dim, self.rt, self.rope = spec, dim, runtime, rope
        self.overwrite, self.out_scale = False, 1.0
        H, Hkv, hd, vd, names = spec.heads, spec.kv_heads, spec.head_dim, spec.v_dim, spec.names
        self.q_width, self.k_width, self.v_width = H * hd, Hkv * hd, Hkv * vd
        self.gated = spec.gate in ("head_sigmoid", "sigmoid")
        self.gate_width = H if spec.gate == "head_sigmoid" else H * vd      # gate values per row
        # the classic form (one head width, pairs (i, i + half), nothing behind the rotation) runs on the fused kernels that
        # were built for it; everything else on the general per-head kernel
        self.classic = (vd == hd and not spec.unit_qk and (rope is None or rope.pairing == "half"))
        if self.classic and spec.gate == "sigmoid" and rope is not None and rope.rotary_dim != hd and hd in (64, 128, 256):
            # a rotation of part of such a head: the general kernel's register form is the faster one (2,048 rows of 16 + 8
            # heads of 128: 14 us against 70)
            self.classic = False
        w = [tensors.pop(prefix + n) for n in (names.q, names.k, names.v)]
        b = [tensors.pop(prefix + n) for n in (names.q_bias, names.k_bias, names.v_bias)] if spec.bias else None
        self.k_off, self.v_off = self.q_width, self.q_width + self.k_width
        self.width = self.q_width + self.k_width + self.v_width
        self.g_off = -1
        if self.gated:
            # the gate's rows ride at the end of the stacked product, from a multiple of 8 columns on
            self.g_off = _up8(self.width)
            g = tensors.pop(prefix + names.gate)
            pad = self.g_off - self.width
            if pad:
                w.append(torch.zeros((pad, dim), dtype=g.dtype, device=g.device))
            w.append(g)
            # (and the row's width stays a multiple of 8 values: the tile kernels read queries by 16-byte pieces)
            tail = _up8(self.gate_width) - self.gate_width
            if tail:
                w.append(torch.zeros((tail, dim), dtype=g.dtype, device=g.device))
            if b:
                b.append(torch.zeros((pad + self.gate_width + tail,), dtype=b[0].dtype, device=b[0].device))
            self.width = self.g_off + self.gate_width + tail
        self.qkv = Linear(torch.cat(w, dim=0).contiguous(), torch.cat(b).contiguous() if b else None)
        self._q_only = None          # the query rows alone, made when a run first reads another run's cache
        del w, b
        self.out = Linear(tensors.pop(prefix + names.o), tensors.pop(prefix + names.o_bias) if spec.out_bias else None)
        self.sink = tensors.pop(prefix + names.sink) if spec.sink else None
        self.keep_first = int(getattr(spec, "keep_first", 0))
        self.q_gain = tensors.pop(prefix + names.q_norm) if spec.qk_norm else None
        self.k_gain = tensors.pop(prefix + names.k_norm) if spec.qk_norm else None
        if rope is not None and rope.rotary_dim > hd:
            raise ValueError(f"rotary_dim={rope.rotary_dim} exceeds head_dim={hd}")
        # what the attention kernels are told about the keys a row sees: 0 all, w > 0 a window, -c < 0 chunks of c positions
        self.span = -spec.chunk if spec.chunk else spec.window

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, Hkv, hd, vd, names = spec.heads, spec.kv_heads, spec.head_dim, spec.v_dim, spec.names
        out = {prefix + names.q: TensorWant((H * hd, dim)),
               prefix + names.k: TensorWant((Hkv * hd, dim)),
               prefix + names.v: TensorWant((Hkv * vd, dim)),
               prefix + names.o: TensorWant((dim, H * vd))}
        if spec.bias:
            out.update({prefix + names.q_bias: TensorWant((H * hd,), "vector"),
                        prefix + names.k_bias: TensorWant((Hkv * hd,), "vector"),
                        prefix + names.v_bias: TensorWant((Hkv * vd,), "vector")})
        if spec.out_bias:
            out[prefix + names.o_bias] = TensorWant((dim,), "vector")
        if spec.qk_norm:
            out[prefix + names.q_norm] = TensorWant((hd,), "vector", init="gain")
            out[prefix + names.k_norm] = TensorWant((hd,), "vector", init="gain")
        if spec.gate == "head_sigmoid":
            out[prefix + names.gate] = TensorWant((H, dim))
        elif spec.gate == "sigmoid":
            out[prefix + names.gate] = TensorWant((H * vd, dim))
        if getattr(spec, "sink", False):
            out[prefix + names.sink] = TensorWant((H,), "vector")
        return out

    @classmethod
    def cache_need(cls, spec):
        # a cache row holds a key in its first head_dim values and a value in its first value_dim; under a chunk mask the
        # pages of chunks that have passed are given back as under a window (the need's window is then -chunk)
        return PagedKeysValues(spec.kv_heads, max(spec.head_dim, spec.v_dim), -spec.chunk if spec.chunk else spec.window,
                               keep_first=int(getattr(spec, "keep_first", 0)))

    def _tiles_fit(self) -> bool:
        s = self.spec
        return (s.v_dim == s.head_dim and ops.attention_decode_fits(self.rt.dtype, s.heads, s.kv_heads, s.head_dim)
                and ops.attention_tiles_take(self.keep_first, self.sink))

    def decode_bucket_cap(self, rows: int) -> int:
        s = self.spec
        if not self._tiles_fit():
            return 1                   # the plain attention's launches do not depend on the context
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        return ops.decode_bucket_cap(rows, s.kv_heads, s.heads, s.head_dim, self.span, scratch)

    def forward(self, xb, x, batch, cache) -> None:
        s, rows = self.spec, xb.shape[0]
        if cache.writes or not self.classic or self.gated:
            qkv = self.rt.buffer("qkv", self.width)[:rows]
            self.qkv.forward(xb, qkv)
        else:
            qkv = self.rt.buffer("q_only", self.q_width)[:rows]
            if self._q_only is None:
                self._q_only = self.qkv.rows(0, self.q_width)
            self._q_only.forward(xb, qkv)
        rope = self.rope
        att = self.rt.buffer("attention_out", s.heads * s.v_dim)[:rows]
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        if (self.classic and not self.gated and cache.writes and batch.decode_only and rope is not None
                and self.sink is None and not self.keep_first and self.out_scale == 1.0
                and ops.attention_decode_fits(qkv.dtype, s.heads, s.kv_heads, s.head_dim)
                and ops.attention_decode_fresh_fits(qkv.dtype, s.heads, s.kv_heads, s.head_dim, rope.rotary_dim)):
            # a step of single rows: the attention kernel norms and rotates its own rows and writes their keys and values
            # (where that pays: it says whether it ran)
            if ops.attention_decode_fresh(qkv, self.q_gain, self.k_gain, s.qk_norm_eps, rope.cos, rope.sin, cache.keys,
                                          cache.values, att, batch.row_seg, batch.positions,
                                          batch.block_tables[cache.group], rows, s.heads, s.kv_heads, s.head_dim,
                                          self.rt.page_size, self.span, s.scale, batch.kv_bucket, scratch):
                return self.out.forward(att, x, accumulate=not self.overwrite)
        slots = batch.slots[cache.group] if cache.writes else None
        if self.classic:
            ops.qk_norm_rope_store(qkv, self.q_gain, self.k_gain, s.qk_norm_eps,
                                   rope.cos if rope else None, rope.sin if rope else None,
                                   rope.rotary_dim if rope else 0, batch.positions, slots, cache.keys, cache.values,
                                   s.heads, s.kv_heads, s.head_dim, self.rt.page_size, write_kv=cache.writes)
        else:
            ops.head_prepare(qkv, 0, self.k_off, self.v_off, self.q_gain, self.k_gain, s.qk_norm_eps,
                             rope.cos if rope else None, rope.sin if rope else None, rope.rotary_dim if rope else 0,
                             rope.pairing if rope else "half", s.unit_qk, batch.positions, slots, cache.keys, cache.values,
                             s.heads, s.kv_heads, s.head_dim, s.v_dim, self.rt.page_size, write_kv=cache.writes)
        ops.attention(qkv, cache.keys, cache.values, att, batch, cache.group, s.heads, s.kv_heads, s.head_dim,
                      self.rt.page_size, self.span, s.scale, scratch, value_dim=s.v_dim, keep_first=self.keep_first,
                      sink=self.sink)
        if s.gate == "sigmoid":
            ops.sigmoid_gate(att, qkv[:, self.g_off:self.g_off + self.gate_width], self.out_scale)
        else:
            if self.gated:
                ops.head_gate(att, qkv[:, self.g_off:self.g_off + s.heads], s.heads, s.v_dim)
            if self.out_scale != 1.0:
                raise ops.KernelError("a factor on the attention's result is built together with the gate of full width")
        self.out.forward(att, x, accumulate=not self.overwrite)


register_mixer("gqa_attention", GqaAttention, replace=True)
