"""The arrangement of one layer: which norm feeds which part, and where results are added.

`pre_norm` is the reference's layer loop (src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:
959-969): x += mixer(norm(x)); x += feed_forward(norm(x)), no norms after the parts. The
residual stream x is float32 in both precisions; the parts add into it themselves (the add
is the epilogue of their last matrix product).

Two things a layer spec may say beyond that: `feed_forward=None` (the layer is its mixer alone, and has no second
norm), and `residual_scale` s (x += s * part(norm(x))). A part that can scale its own result says so
(`takes_residual_scale`; it gets the factor as `residual_scale` and applies it in front of its last product); any other
part adds into a zeroed float32 buffer instead, which is then added to x with the factor.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedState
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Block, part_class, register_block


class PreNormBlock(Block):
    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, position_encodings):
        names = spec.names
        norm_cls = part_class("norm", spec.norm.kind)
        self.rt, self.dim = runtime, dim
        self.mixer_norm = norm_cls(spec.norm, dim, tensors, prefix + names.mixer_norm, runtime)
        mixer_cls = part_class("mixer", spec.mixer.kind)
        table = getattr(spec.mixer, "rope_table", -1)
        extra = {"rope": position_encodings[table]} if table is not None and table >= 0 and position_encodings else {}
        if getattr(mixer_cls, "wants_position_encodings", False):      # a mixer of mixers: its branches pick their tables
            extra = {"position_encodings": position_encodings}
        self.mixer = mixer_cls(spec.mixer, dim, tensors, prefix + names.mixer, runtime, **extra)
        self.ffn_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.ffn_norm = norm_cls(spec.norm, dim, tensors, prefix + names.feed_forward_norm, runtime)
            self.feed_forward = part_class("feed_forward", spec.feed_forward.kind)(
                spec.feed_forward, dim, tensors, prefix + names.feed_forward, runtime)
        self.scale = float(getattr(spec, "residual_scale", 1.0))
        self._scaled_outside = set()
        for part in (self.mixer, self.feed_forward):
            if part is None or self.scale == 1.0:
                continue
            if getattr(part, "takes_residual_scale", False):
                part.residual_scale = self.scale
            else:
                self._scaled_outside.add(id(part))

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in (self.mixer_norm, self.ffn_norm, self.mixer, self.feed_forward)
                   if p is not None)

    def decode_bucket_cap(self, rows: int) -> int:
        # (norms and feed-forwards do not look at the bucket; a mixer that does not say gets the safe answer)
        return getattr(self.mixer, "decode_bucket_cap", lambda _: 32)(rows)

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        names = spec.names
        norm_cls = part_class("norm", spec.norm.kind)
        out = {}
        out.update(norm_cls.wants(spec.norm, dim, prefix + names.mixer_norm))
        out.update(part_class("mixer", spec.mixer.kind).wants(spec.mixer, dim, prefix + names.mixer))
        if spec.feed_forward is not None:
            out.update(norm_cls.wants(spec.norm, dim, prefix + names.feed_forward_norm))
            out.update(part_class("feed_forward", spec.feed_forward.kind).wants(spec.feed_forward, dim,
                                                                                prefix + names.feed_forward))
        return out

    def _into(self, part, x):
        """Where `part` adds its result: x itself, or a zeroed buffer that `_settle` adds to x with the layer's factor."""
        if id(part) not in self._scaled_outside:
            return x
        y = self.rt.buffer("residual_part", self.dim, torch.float32)[:x.shape[0]]
        y.zero_()
        return y

    def _settle(self, x, y) -> None:
        if y is not x:
            ops.add_scaled(x, y, self.scale)

    def forward(self, x, batch, cache) -> None:
        xb = self.rt.buffer("normed", self.dim)[:x.shape[0]]
        self.mixer_norm.forward(x, xb)
        y = self._into(self.mixer, x)
        self.mixer.forward(xb, y, batch, cache)
        self._settle(x, y)
        if self.feed_forward is None:
            return
        self.ffn_norm.forward(x, xb)
        y = self._into(self.feed_forward, x)
        self.feed_forward.forward(xb, y, batch)
        self._settle(x, y)


register_block("pre_norm", PreNormBlock, replace=True)


class ParallelResidualBlock(PreNormBlock):
    """ONE norm whose result feeds both parts, and both results are added to the stream:

        h = norm(x);   x += mixer(h) + feed_forward(h)

    Both parts add into the float32 stream themselves, one after the other (the add is the epilogue of their last products);
    neither reads what the other wrote, because both read h. The layer's one gain is `names.mixer_norm`."""

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, position_encodings):
        if spec.feed_forward is not None and spec.names.feed_forward_norm != spec.names.mixer_norm:
            raise ValueError("one norm feeds both parts: the feed-forward's norm is named like the mixer's")
        super().__init__(spec, dim, tensors, prefix, runtime, position_encodings)
        self.ffn_norm = None           # (built by the base from the same tensor; there is one norm)

    def forward(self, x, batch, cache) -> None:
        xb = self.rt.buffer("normed", self.dim)[:x.shape[0]]
        self.mixer_norm.forward(x, xb)
        y = self._into(self.mixer, x)
        self.mixer.forward(xb, y, batch, cache)
        self._settle(x, y)
        if self.feed_forward is None:
            return
        y = self._into(self.feed_forward, x)
        self.feed_forward.forward(xb, y, batch)
        self._settle(x, y)


register_block("parallel_residual", ParallelResidualBlock, replace=True)


class SandwichNormBlock(PreNormBlock):
    """A norm in front of each part and one behind it, before the residual sum:

        x += post_norm(mixer(norm(x)));   x += post_norm'(feed_forward(norm'(x)))

    The norms behind are RMS norms with gains of their own (`names.mixer_post_norm`, `names.feed_forward_post_norm`). A
    part's result goes into a float32 buffer (the part is told to write instead of add: `overwrite`; one that cannot gets
    the buffer zeroed), and one kernel norms it, adds it to the stream and also makes the normed input of the part that
    follows: the feed-forward's, or the next block's mixer's (`ops.norm_chain`; the model hands a block the next block's
    gain where both arrange their norms this way)."""

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, position_encodings):
        super().__init__(spec, dim, tensors, prefix, runtime, position_encodings)
        if spec.norm.kind != "rmsnorm":
            raise ValueError(f"the norm behind a part is an RMS norm; the layer's norm is {spec.norm.kind!r}")
        if self.scale != 1.0:
            raise ValueError("a residual scale together with norms behind the parts is not built")
        names, gain = spec.names, getattr(spec.norm, "gain_name", "weight")
        self.eps = float(spec.norm.eps)
        self.mixer_post_gain = tensors[prefix + names.mixer_post_norm + gain]
        self.ffn_post_gain = tensors[prefix + names.feed_forward_post_norm + gain] if self.feed_forward is not None else None
        self._zero_first = set()
        for part in (self.mixer, self.feed_forward):
            if part is None:
                continue
            if getattr(part, "can_overwrite", False):
                part.overwrite = True
            else:
                self._zero_first.add(id(part))

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        out = super().wants(spec, dim, prefix)
        names, gain = spec.names, getattr(spec.norm, "gain_name", "weight")
        out[prefix + names.mixer_post_norm + gain] = TensorWant((dim,), "vector", init="gain")
        if spec.feed_forward is not None:
            out[prefix + names.feed_forward_post_norm + gain] = TensorWant((dim,), "vector", init="gain")
        return out

    def _result(self, part, rows):
        y = self.rt.buffer("part_result", self.dim, torch.float32)[:rows]
        if id(part) in self._zero_first:
            y.zero_()
        return y

    chains_norms = True        # `forward` takes `normed` and `next_gain` and says whether it made the next block's input

    def forward(self, x, batch, cache, normed: bool = False, next_gain=None) -> bool:
        """`normed`: the shared buffer of normed rows already holds this block's input (the block in front made it with
        its last launch). `next_gain`: the gain of the norm in front of the block that follows, if that block can take
        its input the same way (same width and eps): this block's last launch then makes it, and True is returned."""
        rows = x.shape[0]
        xb = self.rt.buffer("normed", self.dim)[:rows]
        if not normed:
            self.mixer_norm.forward(x, xb)
        branches = getattr(self.mixer, "forward_branches", None)
        if branches is not None:
            # a mixer of mixers hands over its branches' results as they are: their norms and their sum ride in the same
            # launch as the norm behind the mixer
            a, gain_a, b, gain_b, scale = branches(xb, batch, cache)
        else:
            a, gain_a, b, gain_b, scale = self._result(self.mixer, rows), None, None, None, 1.0
            self.mixer.forward(xb, a, batch, cache)
        nxt = xb if next_gain is not None else None
        if self.feed_forward is None:
            ops.norm_chain(x, a, self.mixer_post_gain, self.eps, b, gain_a, gain_b, scale, next_out=nxt, gain_next=next_gain)
            return nxt is not None
        # ... and so does the norm in front of the feed-forward
        ops.norm_chain(x, a, self.mixer_post_gain, self.eps, b, gain_a, gain_b, scale, next_out=xb, gain_next=self.ffn_norm.gain)
        y = self._result(self.feed_forward, rows)
        self.feed_forward.forward(xb, y, batch)
        ops.norm_chain(x, y, self.ffn_post_gain, self.eps, next_out=nxt, gain_next=next_gain)
        return nxt is not None


register_block("sandwich_norm", SandwichNormBlock, replace=True)


class PostNormBlock(Block):
    """The norm sits behind each part, on the part's result, and the parts read the stream itself:

        x += norm(mixer(h));   x += norm'(feed_forward(x)),   h = x, or with a token shift x_t + (x_(t-1) - x_t) * mu

    The norm is the layer's (`layernorm` or `rmsnorm`, gains `names.mixer_norm` and `names.feed_forward_norm`). A part writes
    its result into a float32 buffer (`overwrite`; one that cannot gets it zeroed) and one kernel norms it, adds it to the
    stream and, in bfloat16, leaves the stream's new rows in the compute type for the part that follows. With a token shift
    the block keeps one row of the stream per request between steps (`cache_need`: a state of `dim` float32 values; the
    cache manager hands a new request a zeroed one), which is what a segment's first row blends with."""

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, position_encodings):
        names, gain = spec.names, getattr(spec.norm, "gain_name", "weight")
        if spec.norm.kind not in ("layernorm", "rmsnorm"):
            raise ValueError(f"the norm behind a part is a layer norm or an RMS norm; the layer's is {spec.norm.kind!r}")
        if float(getattr(spec, "residual_scale", 1.0)) != 1.0:
            raise ValueError("a residual scale together with norms behind the parts is not built")
        self.rt, self.dim, self.eps, self.center = runtime, dim, float(spec.norm.eps), spec.norm.kind == "layernorm"
        self.mixer_gain = tensors[prefix + names.mixer_norm + gain]
        mixer_cls = part_class("mixer", spec.mixer.kind)
        table = getattr(spec.mixer, "rope_table", -1)
        extra = {"rope": position_encodings[table]} if table is not None and table >= 0 and position_encodings else {}
        if getattr(mixer_cls, "wants_position_encodings", False):
            extra = {"position_encodings": position_encodings}
        self.mixer = mixer_cls(spec.mixer, dim, tensors, prefix + names.mixer, runtime, **extra)
        self.ffn_gain = self.feed_forward = None
        if spec.feed_forward is not None:
            self.ffn_gain = tensors[prefix + names.feed_forward_norm + gain]
            self.feed_forward = part_class("feed_forward", spec.feed_forward.kind)(
                spec.feed_forward, dim, tensors, prefix + names.feed_forward, runtime)
        self.shift = tensors[prefix + spec.token_shift] if spec.token_shift else None
        self._zero_first = set()
        for part in (self.mixer, self.feed_forward):
            if part is None:
                continue
            if getattr(part, "can_overwrite", False):
                part.overwrite = True
            else:
                self._zero_first.add(id(part))

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in (self.mixer, self.feed_forward) if p is not None)

    def decode_bucket_cap(self, rows: int) -> int:
        return getattr(self.mixer, "decode_bucket_cap", lambda _: 32)(rows)

    @classmethod
    def cache_need(cls, spec, dim: int):
        """What the arrangement itself keeps between steps, beside its mixer's need."""
        return FixedState((dim,), "float32") if spec.token_shift else None

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        names, gain = spec.names, getattr(spec.norm, "gain_name", "weight")
        out = {prefix + names.mixer_norm + gain: TensorWant((dim,), "vector", init="gain")}
        out.update(part_class("mixer", spec.mixer.kind).wants(spec.mixer, dim, prefix + names.mixer))
        if spec.feed_forward is not None:
            out[prefix + names.feed_forward_norm + gain] = TensorWant((dim,), "vector", init="gain")
            out.update(part_class("feed_forward", spec.feed_forward.kind).wants(spec.feed_forward, dim,
                                                                                prefix + names.feed_forward))
        if spec.token_shift:
            out[prefix + spec.token_shift] = TensorWant((dim,), "vector")
        return out

    def _result(self, part, rows):
        y = self.rt.buffer("part_result", self.dim, torch.float32)[:rows]
        if id(part) in self._zero_first:
            y.zero_()
        return y

    mixes_depth = True         # `forward` takes `shifted` and `tail` and says whether it made the next block's shifted input

    def _last_norm(self, x, a, gain, batch, tail) -> bool:
        """The layer's last norm and residual sum; with `tail` = (stack, weights, n, out, next_shift) also the depth mix
        behind the layer, and, in a step of single rows, the token shift of the block that follows (`next_shift` = its (mu,
        state)); says whether that block's input is made."""
        if tail is None:
            ops.norm_add(x, a, gain, self.eps, center=self.center)
            return False
        stack, weights, n, out, next_shift = tail
        shift = next_shift if batch.decode_only else None
        xb = self.rt.buffer("normed", self.dim)[:x.shape[0]]
        ops.norm_add_mix(x, a, gain, self.eps, stack, weights, n, out, self.center, shift, batch, xb if shift is not None else None)
        return shift is not None

    def forward(self, x, batch, cache, shifted: bool = False, tail=None) -> bool:
        rows = x.shape[0]
        low = self.rt.dtype != torch.float32            # the parts read a copy of the stream in the compute type
        xb = self.rt.buffer("normed", self.dim)[:rows]
        if self.shift is not None:
            if not shifted:                             # (else the block in front made it with its last launch)
                ops.token_shift(x, self.shift, cache.block_states[0], batch, xb)
            h = xb
        elif low:
            xb.copy_(x)
            h = xb
        else:
            h = x
        a = self._result(self.mixer, rows)
        self.mixer.forward(h, a, batch, cache)
        if self.feed_forward is None:
            return self._last_norm(x, a, self.mixer_gain, batch, tail)
        ops.norm_add(x, a, self.mixer_gain, self.eps, next_out=xb if low else None, center=self.center)
        y = self._result(self.feed_forward, rows)
        self.feed_forward.forward(xb if low else x, y, batch)
        return self._last_norm(x, y, self.ffn_gain, batch, tail)


register_block("post_norm", PostNormBlock, replace=True)
