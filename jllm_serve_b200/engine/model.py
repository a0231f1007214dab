"""The generic decoder: embedding, the scheduled layer runs, final norm and head, built from parts.

The model is what a registry entry builds from a `Decoder` spec. It knows the order of
layer runs (data: `spec.schedule`), hands every run the cache it reads or writes, and
computes logits only for the rows that were asked for, as the reference does
(src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:895-928,980-985). The head is the
embedding when `tie_word_embeddings` is set (a `lm_head.weight` that the file still has is
left unread, as the reference's converter drops it: model/ModelConverter.java:663-665), else
`lm_head.weight`, and the embedding again if the file has none (model/ModelWeights.java:37).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import needs_of
from ..config.specs import ConfigError, Decoder
from ..csrc import ops
from ..parts import Linear, RunCache, Runtime, part_class
from ..weights.loader import TensorWant


def cls_prefix(layer, names, index: int) -> str:
    """The checkpoint prefix of a layer: its own if the spec names one (a model whose layers are not numbered in the
    order of their specs), else the model's pattern with the layer's index."""
    own = getattr(layer, "prefix", None)
    return own if own is not None else names.layer.format(index)


class DecoderModel:
    def __init__(self, spec: Decoder, tensors: Dict[str, torch.Tensor], runtime: Runtime):
        self.spec, self.rt = spec, runtime
        core, names = spec.core, spec.names
        tensors = dict(tensors)
        self.embedding = tensors.pop(names.embedding)
        head = None if core.tied else tensors.pop(names.head, None)
        if head is None and not core.tied:
            runtime.notes.append(f"{names.head} is not in the checkpoint: the embedding serves as the head")
        self.head = Linear(self.embedding, keep_plain=True) if head is None else Linear(head)
        self.position_encodings = []
        for t in spec.rope_tables:
            cls = part_class("position", t.kind)
            extra = {"tensors": tensors, "dim": core.dim} if cls.wants(t, core.dim, "") else {}
            self.position_encodings.append(cls(t, runtime.max_positions, runtime.device, **extra))
        self.blocks = []
        for l, layer in enumerate(spec.layers):
            cls = part_class("block", layer.arrangement)
            self.blocks.append(cls(layer, core.dim, tensors, cls_prefix(layer, names, l), runtime, self.position_encodings))
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm, core.dim, tensors,
                                                                   names.final_norm, runtime)
        self.vocab, self.dim = core.vocab, core.dim
        self.logit_scale = float(getattr(core, "logit_scale", 1.0))
        self.embedding_scale = float(getattr(core, "embedding_scale", 1.0))
        # depth mix: what run i hands on is a weighted sum of the embedded rows and of every run's result so far
        self.depth_weights = None
        if getattr(spec, "depth_mix", ""):
            self.depth_weights = [tensors[name] for name in self._depth_names(spec)]
            self._one = torch.ones(1, dtype=torch.float32, device=runtime.device)
        # how many of a run's fixed-size states are its arrangement's own (they follow the mixer's in the run's list)
        self._block_states = [len(needs_of(self._block_need(spec, spec.layers[run.layer]))) for run in spec.schedule]

    @staticmethod
    def _block_need(spec: Decoder, layer):
        need = getattr(part_class("block", layer.arrangement), "cache_need", None)
        return need(layer, spec.core.dim) if need is not None else None

    @staticmethod
    def _depth_names(spec: Decoder) -> List[str]:
        """The tensor of run i's i + 2 depth weights lies under the prefix of the layer that run i runs; a layer that runs
        twice would need two tensors of one name."""
        names = [cls_prefix(spec.layers[run.layer], spec.names, run.layer) + spec.depth_mix for run in spec.schedule]
        if len(set(names)) != len(names):
            raise ConfigError("a depth mix needs weights per layer run, and a layer that runs twice has one tensor")
        return names

    @classmethod
    def wants(cls, spec: Decoder) -> Dict[str, TensorWant]:
        core, names = spec.core, spec.names
        out = {names.embedding: TensorWant((core.vocab, core.dim))}
        if not core.tied:
            out[names.head] = TensorWant((core.vocab, core.dim), optional=True)
        for t in spec.rope_tables:
            out.update(part_class("position", t.kind).wants(t, core.dim, ""))
        for l, layer in enumerate(spec.layers):
            out.update(part_class("block", layer.arrangement).wants(layer, core.dim, cls_prefix(layer, names, l)))
        out.update(part_class("norm", spec.final_norm.kind).wants(spec.final_norm, core.dim, names.final_norm))
        if getattr(spec, "depth_mix", ""):
            for i, name in enumerate(cls._depth_names(spec)):
                out[name] = TensorWant((i + 2,), "vector", init="average")
        return out

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be captured once and replayed: every part says so of itself."""
        return all(b.graph_safe for b in self.blocks) and all(pe.graph_safe for pe in self.position_encodings)

    def decode_bucket_cap(self, rows: int) -> int:
        """The bucket from which on a decode step of `rows` rows no longer changes its launches: the largest the parts name."""
        return max([getattr(b, "decode_bucket_cap", lambda _: 32)(rows) for b in self.blocks] or [1])

    def cache_needs(self) -> List[Optional[object]]:
        """One entry per scheduled run: what it keeps between steps (None if it reads another run's cache; a
        tuple if the mixer keeps several things, say paged keys and values and a state of fixed size)."""
        needs = []
        for run in self.spec.schedule:
            layer = self.spec.layers[run.layer]
            mixer = layer.mixer
            need = None if run.cache_of is not None else part_class("mixer", mixer.kind).cache_need(mixer)
            own = needs_of(self._block_need(self.spec, layer))       # the arrangement's own: kept by every run, borrower or not
            needs.append(tuple(needs_of(need)) + tuple(own) if own else need)
        return needs

    def _run_cache(self, cache, i: int) -> RunCache:
        run = self.spec.schedule[i]
        owner = i if run.cache_of is None else run.cache_of
        out = RunCache(owner, run.cache_of is None)
        if owner in cache.paged_of_run:
            out.group = cache.paged_of_run[owner]
            out.keys, out.values = cache.keys_values(owner)
        mine, theirs = self._block_states[i], self._block_states[owner]
        states = cache.states(owner)
        states = states[:len(states) - theirs] if theirs else states
        if states:
            out.states, out.state = tuple(states), states[0]
        if mine:
            out.block_states = tuple(cache.states(i)[-mine:])
        return out

    def forward(self, batch, cache, logits_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the batch's rows through every scheduled layer; returns float32 logits [wanted rows, vocab]."""
        rows = batch.rows
        schedule, normed, shifted = self.spec.schedule, False, False
        stack = None
        if self.depth_weights is not None:
            # plane 0: the embedded rows; plane j + 1: run j's result, made in place from the mix that run j was handed
            # (which the mix kernel wrote there); the last plane: what the last run hands on
            planes = len(schedule) + 2
            stack = self.rt.buffer("depth_stack", self.dim, torch.float32, rows=planes * self.rt.max_rows)
            stack = stack.view(planes, self.rt.max_rows, self.dim)[:, :rows]
            x = stack[0]
        else:
            x = self.rt.buffer("residual", self.dim, torch.float32)[:rows]
        ops.embed_rows(batch.token_ids, self.embedding, x)
        if self.embedding_scale != 1.0:
            ops.scale_values(x, self.embedding_scale)
        for pe in self.position_encodings:
            pe.on_embedding(x, batch)
        for i, run in enumerate(schedule):
            block = self.blocks[run.layer]
            if stack is not None:
                if i == 0:
                    ops.depth_mix(stack, self._one, 1, stack[1])       # the first run reads the embedded rows themselves
                x = stack[i + 1]
            if getattr(block, "chains_norms", False):
                # an arrangement whose last launch can also make the next block's normed input is given that block's gain
                nxt = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
                gain = nxt.mixer_norm.gain if getattr(nxt, "chains_norms", False) and nxt.eps == block.eps else None
                normed = block.forward(x, batch, self._run_cache(cache, i), normed=normed, next_gain=gain)
            elif stack is not None and getattr(block, "mixes_depth", False):
                # an arrangement whose last launch can also mix the planes (and, in a step of single rows, shift the tokens
                # for the block that follows) is handed the stack and that block's shift vector and state
                nxt = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
                shift = None
                if batch.decode_only and getattr(nxt, "mixes_depth", False) and nxt.shift is not None:
                    shift = (nxt.shift, self._run_cache(cache, i + 1).block_states[0])
                shifted = block.forward(x, batch, self._run_cache(cache, i), shifted=shifted,
                                        tail=(stack, self.depth_weights[i], i + 2, stack[i + 2], shift))
                x = stack[i + 2]
                continue
            else:
                block.forward(x, batch, self._run_cache(cache, i))
                normed = shifted = False
            if stack is not None:
                ops.depth_mix(stack, self.depth_weights[i], i + 2, stack[i + 2])
                x = stack[i + 2]
        n = batch.num_wanted
        if logits_out is None:
            logits_out = torch.empty((n, self.vocab), dtype=torch.float32, device=self.rt.device)
        if n == 0:
            return logits_out[:0]
        hb = self.rt.buffer("head_in", self.dim)[:n]
        self.final_norm.forward(x, hb, row_index=batch.logit_rows, rows=n)
        self.head.forward(hb, logits_out[:n])
        if self.logit_scale != 1.0:
            ops.scale_values(logits_out[:n], self.logit_scale)
        return logits_out[:n]


def build_model(entry, spec, tensors, runtime):
    """What the registry's entry builds: its own builder, else the generic decoder."""
    return (entry.build or DecoderModel)(spec, tensors, runtime)


def model_wants(entry, spec) -> Dict[str, TensorWant]:
    builder = entry.build or DecoderModel
    return builder.wants(spec)
