"""Attention over a cached latent as a mixer: one row of `rank` values per position instead of keys and values per head.

With h the normed rows:  q = Wq h (heads x dk),  c_t = rmsnorm(Wd h_t) * n (rank values: all that is cached),
k_j = Wuk c_j and v_j = Wuv c_j per head, p = softmax over j <= t of scale (q . k_j), head output sigmoid(Wg h)_head *
sum_j p_j v_j, x += m Wo [heads side by side]. Nothing rotates.

Since q_h . (Wuk_h c_j) = (Wuk_h^T q_h) . c_j and sum_j p_j Wuv_h c_j = Wuv_h sum_j p_j c_j, the keys and values of
earlier positions are never made: the queries are carried into the latent's space (one small product per head, all heads
in one launch), the engine's paged attention runs with ONE key/value head of width `rank` whose keys and values are the
same cached rows (`PagedKeysValues(1, rank, planes=1)`), and its result goes through Wuv per head, where the gate and the
residual scale m are applied. Scores, softmax and the latent's norm are float32 in both precisions.

What a spec may ask for beyond that (each on its own):

* `query_rank` > 0: the queries go through a latent too, q = Wuq (rmsnorm(Wdq h) * gain) (tensors `dq`, `dq.norm`, `uq`).
* `rope_dim` > 0: the down projection has rank + rope_dim rows; the last rope_dim are not normed but rotated by the position
  and are a key part that all heads share. A query head is [key_dim values, rope_dim rotated values] and its score is
  q[:key_dim] . (Wuk c_j) + rot(q[key_dim:]) . r_j. A cached row is [c_j, r_j]; a head's latent-space query is [Wuk^T
  q[:key_dim], rot(q[key_dim:])], so the score is still ONE dot product with a cached row, and the attention runs with key and
  value heads of rank + rope_dim values: the last rope_dim values of its result are never read (Wuv takes the first rank).
* `own_latent` False: no down projection and no cache of its own; `cache` is another run's, whose rows it reads.
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


class LatentAttention(Mixer):
    takes_residual_scale = True
    can_overwrite = True           # a block that norms the result before adding it asks for x = ... instead of x += ...

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, rope=None):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.residual_scale = 1.0
        self.overwrite = False
        H, dk, dv, R = spec.heads, spec.key_dim, spec.value_dim, spec.rank
        self.q_rank, self.rope_dim, self.own = spec.query_rank, spec.rope_dim, spec.own_latent
        self.plain = not (self.q_rank or self.rope_dim) and self.own       # the form without query latent and rotated part
        self.rope = rope
        if self.rope_dim and (rope is None or rope.pairing != "interleaved" or rope.rotary_dim > self.rope_dim):
            raise ValueError("latent attention: the rotated key part needs a rotary table of neighbouring pairs no wider than it")
        names = (["dq"] if self.q_rank else ["q"]) + (["dkv"] if self.own else []) + (["g"] if spec.gated else [])
        self.offsets, rows, at = {}, [], 0
        for n in names:
            w = tensors.pop(prefix + n)
            self.offsets[n] = at
            pad = _up8(w.shape[0]) - w.shape[0]
            rows.append(w)
            if pad:
                rows.append(torch.zeros((pad, dim), dtype=w.dtype, device=w.device))
            at += w.shape[0] + pad
        self.width = at
        self.inp = Linear(torch.cat(rows, dim=0).contiguous())
        del rows
        self.latent_gain = tensors.pop(prefix + "dkv.norm") if self.own else None
        self.q_gain = tensors.pop(prefix + "dq.norm") if self.q_rank else None
        self.q_up = Linear(tensors.pop(prefix + "uq")) if self.q_rank else None
        # Wuk [heads x dk, rank] as [heads, rank, dk]: the product that carries a head's query into the latent's space
        self.q_to_latent = tensors.pop(prefix + "uk").view(H, dk, R).transpose(1, 2).contiguous()
        self.latent_to_v = tensors.pop(prefix + "uv").view(H, dv, R).contiguous()
        self.out = Linear(tensors.pop(prefix + "o"))

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, dk, dv, R = spec.heads, spec.key_dim, spec.value_dim, spec.rank
        rd, qr = getattr(spec, "rope_dim", 0), getattr(spec, "query_rank", 0)
        out = {prefix + "uk": TensorWant((H * dk, R)), prefix + "uv": TensorWant((H * dv, R)),
               prefix + "o": TensorWant((dim, H * dv))}
        if qr:
            out.update({prefix + "dq": TensorWant((qr, dim)), prefix + "dq.norm": TensorWant((qr,), "vector", init="gain"),
                        prefix + "uq": TensorWant((H * (dk + rd), qr))})
        else:
            out[prefix + "q"] = TensorWant((H * (dk + rd), dim))
        if getattr(spec, "own_latent", True):
            out.update({prefix + "dkv": TensorWant((R + rd, dim)), prefix + "dkv.norm": TensorWant((R,), "vector", init="gain")})
        if spec.gated:
            out[prefix + "g"] = TensorWant((H, dim))
        return out

    @classmethod
    def cache_need(cls, spec):
        return PagedKeysValues(1, spec.rank + getattr(spec, "rope_dim", 0), spec.window, planes=1)

    def decode_bucket_cap(self, rows: int) -> int:
        s = self.spec
        heads, width = min(s.heads, 16), s.rank + self.rope_dim
        if not ops.attention_decode_fits(self.rt.dtype, heads, 1, width):
            return 1
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        return max(ops.decode_bucket_cap(rows, 1, n, width, s.window, scratch)
                   for n in {heads, s.heads % 16 or heads})

    def forward(self, xb, x, batch, cache) -> None:
        if not self.plain:
            return self._forward_general(xb, x, batch, cache)
        s, rows = self.spec, xb.shape[0]
        H, dk, dv, R = s.heads, s.key_dim, s.value_dim, s.rank
        proj = self.rt.buffer("latent_proj", self.width)[:rows]
        self.inp.forward(xb, proj)
        if cache.writes:
            d_off = self.offsets["dkv"]
            ops.latent_norm_store(proj[:, d_off:d_off + R], self.latent_gain, s.norm_eps, batch.slots[cache.group], cache.keys)
        q = self.rt.buffer("latent_queries", H * R)[:rows]
        ops.gemm_heads(proj[:, :H * dk], self.q_to_latent, q)
        att = self.rt.buffer("latent_attended", H * R)[:rows]
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        # the decode kernel shares every key among at most 16 query heads: more heads go in groups of 16, each a launch
        # over the same cached rows
        per = 16 if H > 16 and ops.attention_decode_fits(q.dtype, 16, 1, R) else H
        for h0 in range(0, H, per):
            n = min(per, H - h0)
            ops.attention(q[:, h0 * R:(h0 + n) * R], cache.keys, cache.values, att[:, h0 * R:(h0 + n) * R], batch,
                          cache.group, n, 1, R, self.rt.page_size, s.window, s.scale, scratch)
        y = self.rt.buffer("latent_values", H * dv)[:rows]
        gate = proj[:, self.offsets["g"]:self.offsets["g"] + H] if s.gated else None
        ops.gemm_heads(att, self.latent_to_v, y, gate, self.residual_scale)
        self.out.forward(y, x, accumulate=not self.overwrite)

    def _forward_general(self, xb, x, batch, cache) -> None:
        """The form with a query latent, a rotated key part or a borrowed cache. The stacked down projections leave in
        float32 (their norms are float32 arithmetic), one kernel norms the query latent, norms the latent, rotates the shared
        key part and writes the cached row; a head's query becomes [Wuk^T q, rot(q_rot)] of rank + rope_dim values."""
        s, rows = self.spec, xb.shape[0]
        H, dk, dv, R, rd, qr = s.heads, s.key_dim, s.value_dim, s.rank, self.rope_dim, self.q_rank
        W = R + rd
        if cache.keys is None or cache.keys.shape[-1] != W:
            raise ValueError(f"latent attention: the cache it is handed has rows of "
                             f"{None if cache.keys is None else cache.keys.shape[-1]} values, it reads rows of {W}")
        writes = self.own and cache.writes
        proj = self.rt.buffer("latent_proj32", self.width, torch.float32)[:rows]
        self.inp.forward(xb, proj)
        cq = self.rt.buffer("latent_query_latent", qr)[:rows] if qr else None
        rope = self.rope
        if qr or writes:
            ops.latent_prepare(proj, self.offsets.get("dq", 0), qr, self.q_gain, cq, self.offsets.get("dkv", 0), R, rd,
                               self.latent_gain, rope.cos if rope else None, rope.sin if rope else None,
                               rope.rotary_dim if rope else 0, batch.positions, batch.slots[cache.group] if writes else None,
                               cache.keys if writes else None, s.norm_eps, write_latent=writes)
        if qr:
            q = self.rt.buffer("latent_heads_q", H * (dk + rd))[:rows]
            self.q_up.forward(cq, q)
        else:
            q = self.rt.buffer("latent_heads_q", H * (dk + rd))[:rows]
            q.copy_(proj[:, self.offsets["q"]:self.offsets["q"] + H * (dk + rd)])
        ql = self.rt.buffer("latent_queries", H * W)[:rows]
        # (one more block per row tile and head turns the head's rotated part and puts it behind its latent-space query)
        ops.gemm_heads(q, self.q_to_latent, ql, a_head=dk + rd, out_head=W,
                       rope=(rd, rope.cos, rope.sin, rope.rotary_dim, batch.positions) if rd else None)
        att = self.rt.buffer("latent_attended", H * W)[:rows]
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        per = 16 if H > 16 and ops.attention_decode_fits(ql.dtype, 16, 1, W) else H
        for h0 in range(0, H, per):
            n = min(per, H - h0)
            ops.attention(ql[:, h0 * W:(h0 + n) * W], cache.keys, cache.values, att[:, h0 * W:(h0 + n) * W], batch,
                          cache.group, n, 1, W, self.rt.page_size, s.window, s.scale, scratch)
        y = self.rt.buffer("latent_values", H * dv)[:rows]
        gate = proj_gate = None
        if s.gated:
            proj_gate = self.rt.buffer("latent_gate", _up8(H))[:rows]
            proj_gate.copy_(proj[:, self.offsets["g"]:self.offsets["g"] + _up8(H)])
            gate = proj_gate[:, :H]
        ops.gemm_heads(att, self.latent_to_v, y, gate, self.residual_scale, a_head=W)
        self.out.forward(y, x, accumulate=not self.overwrite)


register_mixer("latent_attention", LatentAttention, replace=True)
