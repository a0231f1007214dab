"""Routed experts as a feed-forward: x += m sum_e w_e Wdown_e (silu(Wgate_e h) * (Wup_e h)) over a row's chosen experts.

The router (`ops.route_experts`, float32) gives every row a weight per expert, zero for the experts it does not use.
The experts then run as two products for all of them together: gate and up rows of all experts stacked into one
[2 x experts x ff, dim] matrix (with the SwiGLU epilogue of the tensor-core products in bfloat16), and the down matrices
laid side by side along k as one [dim, experts x ff] matrix, whose product adds into the residual stream. Between the
two, a row's hidden values of expert e are multiplied by its weight (and by the residual scale m): an expert the row
does not use contributes exact zeros, and the sum over experts is the product's own float32 accumulation. Every weight
streams once per step however the rows choose; what this costs against running only the chosen experts is experts / top
times the multiply-adds.

`weight_on` "input" (with the clamped gated unit): a row's weight multiplies what the expert READS, y = sum_e expert_e(w_e h).
Both of an expert's first products are linear, so w_e (Wgate_e h) and w_e (Wup_e h) are what it would have computed: the
stacked product runs once on h itself, and one kernel (`ops.glu_clamped`) multiplies, cuts off and gates. An expert that a
row does not use has weight 0 and adds exact zeros, as above. `shared`: a dense gated feed-forward of its own sizes that
every row runs, added to the same result.

What a spec may ask of the router (`ops.route_experts`): `score` "softmax" (the scores are a softmax over all of the router's
entries); `identity` entries behind the experts, chosen like experts, that have no weights and give the row's input itself
times their weight (`ops.add_rows_scaled` with the sum of a row's chosen identity weights); `shared_gate`, a [1, dim] matrix
whose logistic value per row multiplies the shared expert's result: its row rides behind the router's (one float32 matrix,
one launch), and the shared expert rides behind the routed ones in both products as an expert that every row uses with that
weight.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorWant
from .base import FeedForward, part_class, register_feed_forward
from .linear import Linear


class RoutedExperts(FeedForward):
    takes_residual_scale = True
    can_overwrite = True           # a block that norms the result before adding it asks for x = ... instead of x += ...

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.residual_scale = 1.0
        self.overwrite = False
        E, ff = spec.experts, spec.hidden
        self.hidden = E * ff
        self.on_input = getattr(spec, "weight_on", "output") == "input"
        self.shared, self.shared_ff, self.shared_limit = None, 0, 0.0
        shared = getattr(spec, "shared", None)
        gates = [tensors.pop(f"{prefix}e{e}.gate") for e in range(E)]
        ups = [tensors.pop(f"{prefix}e{e}.up") for e in range(E)]
        downs = [tensors.pop(f"{prefix}e{e}.down") for e in range(E)]
        if shared is not None and self.on_input and shared.kind == "dense_glu" and shared.activation == spec.activation:
            # a shared expert of the same kind of unit rides behind the routed ones in both products, as an expert that every
            # row uses with weight 1 (and a limit and size of its own)
            self.shared_ff, self.shared_limit = shared.hidden, float(shared.limit)
            gates.append(tensors.pop(prefix + "shared." + shared.names[0]))
            ups.append(tensors.pop(prefix + "shared." + shared.names[1]))
            downs.append(tensors.pop(prefix + "shared." + shared.names[2]))
        elif shared is not None and getattr(spec, "shared_gate", "") and shared.kind == "dense_glu" and shared.activation == spec.activation:
            # a gated shared expert (weights on the output): behind the routed ones in both products, its weight the row's gate
            self.shared_ff = shared.hidden
            gates.append(tensors.pop(prefix + "shared." + shared.names[0]))
            ups.append(tensors.pop(prefix + "shared." + shared.names[1]))
            downs.append(tensors.pop(prefix + "shared." + shared.names[2]))
        elif shared is not None:
            if getattr(spec, "shared_gate", ""):
                raise ValueError("a gate on a shared expert of another kind of unit than the routed ones is not built")
            self.shared = part_class("feed_forward", shared.kind)(shared, dim, tensors, prefix + "shared.", runtime)
        self.hidden = E * ff + self.shared_ff
        gate, up = torch.cat(gates, dim=0), torch.cat(ups, dim=0)
        del gates, ups
        # (a weight in front of the gated unit rules out the product's own epilogue, which gates what it has summed)
        self.fused = gate.dtype == torch.bfloat16 and dim % 8 == 0 and self.hidden % 8 == 0 and not self.on_input
        if self.fused:      # blocks of 8 gate rows followed by their 8 up rows: the product's epilogue applies SwiGLU
            stacked = torch.stack([gate.view(self.hidden // 8, 8, dim), up.view(self.hidden // 8, 8, dim)], dim=1)
            self.gate_up = Linear(stacked.reshape(2 * self.hidden, dim).contiguous())
            del stacked
        else:
            self.gate_up = Linear(torch.cat([gate, up], dim=0).contiguous())
        del gate, up
        self.down = Linear(torch.cat(downs, dim=1).contiguous())
        del downs
        self.router = tensors.pop(prefix + "router")
        self.correction = tensors.pop(prefix + "correction") if spec.correction else None
        self.identity = int(getattr(spec, "identity", 0))
        self.softmax = getattr(spec, "score", "sigmoid") == "softmax"
        self.gates = 0
        if getattr(spec, "shared_gate", ""):
            self.gates = 1
            self.router = torch.cat([self.router, tensors.pop(prefix + spec.shared_gate).to(self.router.dtype)], dim=0).contiguous()
        # a row's table: the experts' weights, the shared expert's gate, the sum of its chosen identity entries' weights
        self.table = E + self.gates + (1 if self.identity else 0)

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        entries = spec.experts + int(getattr(spec, "identity", 0))
        out = {prefix + "router": TensorWant((entries, dim), "matrix_fp32")}
        if spec.correction:
            out[prefix + "correction"] = TensorWant((entries,), "vector")
        if getattr(spec, "shared_gate", ""):
            out[prefix + spec.shared_gate] = TensorWant((1, dim), "matrix_fp32")
        for e in range(spec.experts):
            out[f"{prefix}e{e}.gate"] = TensorWant((spec.hidden, dim))
            out[f"{prefix}e{e}.up"] = TensorWant((spec.hidden, dim))
            out[f"{prefix}e{e}.down"] = TensorWant((dim, spec.hidden))
        if getattr(spec, "shared", None) is not None:
            out.update(part_class("feed_forward", spec.shared.kind).wants(spec.shared, dim, prefix + "shared."))
        return out

    def forward(self, xb, x, batch) -> None:
        s, rows = self.spec, xb.shape[0]
        weights = self.rt.buffer("expert_weights", self.table, torch.float32)[:rows]
        ops.route_experts(xb, self.router, self.correction, s.top, s.scale * self.residual_scale, s.normalize, weights,
                          identity=self.identity, gates=self.gates, softmax=self.softmax)
        h = self.rt.buffer("experts_hidden", self.hidden)[:rows]
        if self.on_input:
            gate_up = self.rt.buffer("experts_gate_up", 2 * self.hidden)[:rows]
            self.gate_up.forward(xb, gate_up)
            ops.glu_clamped(gate_up, weights, h, s.experts, s.hidden, s.limit, self.shared_ff, self.shared_limit)
        else:
            if self.fused:
                self.gate_up.forward(xb, h, swiglu=True)
            else:
                gate_up = self.rt.buffer("experts_gate_up", 2 * self.hidden)[:rows]
                self.gate_up.forward(xb, gate_up)
                ops.swiglu(gate_up, h)
            ops.scale_expert_hidden(h, weights, s.hidden, s.experts, self.shared_ff)
        self.down.forward(h, x, accumulate=not self.overwrite)
        if self.identity:
            ops.add_rows_scaled(x, xb, weights[:, self.table - 1])
        if self.shared is not None:
            self.shared.forward(xb, x, batch)          # (adds: its `overwrite` stays off)


register_feed_forward("routed_experts", RoutedExperts, replace=True)
