"""The typed configuration: what a model is made of, as plain immutable data.

The vocabulary follows the reference's: a decoder is a core (sizes shared by the whole
model), a list of layer specs and a list of rotary tables
(src/main/java/org/robomiri/jllm/model/Decoder.java:15-33, LayerSpec.java:11-19,
Attention.java:48-50, Mlp.java:7-22, RopeTable.java:20-51, Architecture.java:61-67).
Every size and constant that a part needs is a field here; parts never read
`model_type` and never see config.json.

Two things go beyond the reference's vocabulary, because the order of layers is data:
`Decoder.schedule` lists the layer runs, and a run may name a layer a second time or
read the keys and values of an earlier run instead of writing its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: the message names the key and its value."""


@dataclass(frozen=True)
class RopeScaling:
    """How the inverse frequencies of a rotary table are stretched (Scaling.java:6-78)."""
    kind: str = "none"                     # none | linear | yarn | banded (by wavelength L = 2 pi / f: f where L < original /
                                           # high, f / factor where L > original / low, a blend in between)
    factor: float = 1.0
    original_max_positions: int = 0        # yarn: the trained length
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    attention_factor: float = 0.0          # 0 = derive from factor
    truncate: bool = True
    low: float = 1.0                       # banded: the band's edges, in turns of the original length
    high: float = 4.0


@dataclass(frozen=True)
class RopeTableSpec:
    """One rotary table: `rotary_dim` values of each head are rotated, paired as (i, i + rotary_dim / 2) ("half") or as
    (2i, 2i + 1) ("interleaved"). The table itself (one angle per pair and position) is the same for both; the pairing
    is what the mixer's kernel is told."""
    rotary_dim: int
    theta: float
    scaling: RopeScaling = RopeScaling()
    pairing: str = "half"                  # half: (i, i + rotary_dim/2); interleaved: (2i, 2i + 1)
    kind: str = field(default="rotary", init=False)   # which registered position encoding builds the table

    def __post_init__(self):
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ConfigError(f"rotary_dim={self.rotary_dim} must be even and at least 2")
        if not self.theta > 0:
            raise ConfigError(f"rope_theta={self.theta} must be positive")
        if self.pairing not in ("half", "interleaved"):
            raise ConfigError(f"rope pairing {self.pairing!r} is not built (built: half, interleaved)")


@dataclass(frozen=True)
class NormSpec:
    kind: str = "rmsnorm"                  # rmsnorm | dynamic_tanh (tanh(a x) * w + b: no statistics, eps unused) |
                                           # layernorm ((x - m) / sqrt(v + eps) * g with m the mean and v the mean squared deviation, no bias)
    eps: float = 1e-6
    gain_name: str = "weight"              # rmsnorm: the gain is the tensor <the norm's name> + gain_name ("": the name itself)


@dataclass(frozen=True)
class MixerSpec:
    """Base of every token mixer's spec; `kind` picks the part from the parts registry."""
    kind: str = field(default="", init=False)


@dataclass(frozen=True)
class AttentionNames:
    """Checkpoint names of an attention's tensors, relative to the mixer's prefix."""
    q: str = "q_proj.weight"
    k: str = "k_proj.weight"
    v: str = "v_proj.weight"
    o: str = "o_proj.weight"
    q_bias: str = "q_proj.bias"
    k_bias: str = "k_proj.bias"
    v_bias: str = "v_proj.bias"
    o_bias: str = "o_proj.bias"
    q_norm: str = "q_norm.weight"
    k_norm: str = "k_norm.weight"
    gate: str = "gate.weight"
    sink: str = "sink"


@dataclass(frozen=True)
class GqaAttentionSpec(MixerSpec):
    """Grouped-query causal attention over a paged cache (Attention.java:48-50,68-71). Beyond the reference's: value heads
    of another width than key heads (`value_dim`), rows that see only their own chunk of the sequence (`chunk`), a division
    of every query and key head by its root mean square behind the rotation (`unit_qk`), and a sigmoid gate per head on the
    attention's result, read from the mixer's input by one more projection (`gate`)."""
    kind: str = field(default="gqa_attention", init=False)
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0                        # 0 = all keys; else the last `window` keys
    rope_table: int = 0                    # index into Decoder.rope_tables, -1 = no rotation
    qk_norm: bool = False                  # per-head RMSNorm of q and k before the rotation
    qk_norm_eps: float = 1e-6
    bias: bool = False                     # q, k, v biases
    out_bias: bool = False                 # o_proj bias
    scale: float = 0.0                     # multiplier of q . k
    value_dim: int = 0                     # width of a value head; 0 = head_dim
    chunk: int = 0                         # 0 = none; else position i sees j <= i only if i // chunk == j // chunk
    unit_qk: bool = False                  # q and k over their root mean square (eps qk_norm_eps), after the rotation
    gate: str = "none"                     # none | head_sigmoid: head h's result times sigmoid(Wg x)[h] | sigmoid: every value
                                           # of the concatenated heads times sigmoid(Wg x) of its own (Wg has heads x value_dim rows)
    names: AttentionNames = AttentionNames()
    keep_first: int = 0                    # with a window: the sequence's first keep_first positions stay visible to every row
    sink: bool = False                     # a learned number per query head whose exponential joins the softmax's denominator

    def __post_init__(self):
        if self.heads <= 0:
            raise ConfigError(f"num_attention_heads={self.heads} must be positive")
        if self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"num_key_value_heads={self.kv_heads} must be positive and divide "
                              f"num_attention_heads={self.heads}")
        if self.head_dim <= 0:
            raise ConfigError(f"head_dim must be positive, got {self.head_dim}")
        if self.window < 0:
            raise ConfigError(f"sliding_window={self.window} must not be negative")
        if self.value_dim < 0 or self.chunk < 0:
            raise ConfigError(f"attention: value_dim={self.value_dim} and chunk={self.chunk} must not be negative")
        if self.chunk and self.window:
            raise ConfigError("attention: a window and a chunk mask together are not built")
        if self.gate not in ("none", "head_sigmoid", "sigmoid"):
            raise ConfigError(f"attention: gate {self.gate!r} is not built (built: none, head_sigmoid, sigmoid)")
        if self.keep_first < 0 or (self.keep_first and not self.window):
            raise ConfigError(f"attention: keep_first={self.keep_first} must not be negative and needs a window")

    @property
    def v_dim(self) -> int:
        return self.value_dim or self.head_dim


@dataclass(frozen=True)
class GatedLinearAttentionSpec(MixerSpec):
    """Linear attention with a decay gate per key channel and a recurrent state [heads, key_dim, value_dim] per request:
    S_t = diag(d_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, d_t = sigmoid(W2 (W1 h_t) + b2)^(1 / decay_temperature);
    every head's o_t is RMS-normed (one gain of value_dim values for all heads), gated by silu(Wg h_t) and projected."""
    kind: str = field(default="gated_linear_attention", init=False)
    heads: int = 0
    key_dim: int = 0                       # query and key channels per head
    value_dim: int = 0                     # value channels per head
    decay_rank: int = -1                   # width of the low-rank decay projection (rows of W1); -1: the checkpoint's own
    decay_temperature: float = 1.0         # tau
    norm_eps: float = 1e-6
    query_scale: float = 0.0               # multiplier of q (key_dim^-1/2 in the designs seen so far)

    def __post_init__(self):
        for name in ("heads", "key_dim", "value_dim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"gated linear attention: {name}={getattr(self, name)} must be positive")
        if self.decay_rank == 0 or self.decay_rank < -1:
            raise ConfigError(f"gated linear attention: decay_rank={self.decay_rank} must be positive (or -1: as stored)")
        if not self.decay_temperature > 0:
            raise ConfigError(f"gated linear attention: tau={self.decay_temperature} must be positive")


@dataclass(frozen=True)
class FixedDecayLinearAttentionSpec(MixerSpec):
    """Linear attention with one fixed decay per head and a recurrent state [heads, key_dim, value_dim] per request
    ("lightning" attention): q, k, v = act(Wq h), act(Wk h), act(Wv h); S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T
    (query_scale q_t); the heads' results are RMS-normed (all heads of a row together: `norm_over` "all", or "head" by
    head) with a stored gain, gated by sigmoid(Wg h) (or silu) and projected."""
    kind: str = field(default="fixed_decay_linear_attention", init=False)
    heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    decays: Tuple[float, ...] = ()         # one per head, each in [0, 1]
    activation: str = "silu"               # on q, k and v: silu | none
    query_scale: float = 1.0
    norm_eps: float = 1e-6
    norm_over: str = "all"                 # all: one norm over heads x value_dim values (gain of that many); head: per head
    gate: str = "sigmoid"                  # sigmoid | silu, of Wg h (heads x value_dim values)

    def __post_init__(self):
        for name in ("heads", "key_dim", "value_dim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"linear attention: {name}={getattr(self, name)} must be positive")
        if len(self.decays) != self.heads:
            raise ConfigError(f"linear attention: {len(self.decays)} decays for {self.heads} heads")
        if any(not 0.0 <= d <= 1.0 for d in self.decays):
            raise ConfigError(f"linear attention: every decay must lie in [0, 1], got {list(self.decays)}")
        if self.activation not in ("silu", "none") or self.norm_over not in ("all", "head") or self.gate not in ("sigmoid", "silu"):
            raise ConfigError(f"linear attention: activation={self.activation!r} norm_over={self.norm_over!r} "
                              f"gate={self.gate!r} is not built")


@dataclass(frozen=True)
class SelectiveStateSpaceSpec(MixerSpec):
    """A state space whose step size and inputs depend on the token, with one scalar decay per head (the "state space
    duality" form). One input projection gives [z | x B C | dt] (inner = heads x head_dim; B and C: groups x state each); x,
    B and C pass a causal convolution of `conv` taps per channel and silu; dt = softplus(dt + dt_bias); per head (B, C of
    group h // (heads / groups)) S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t; y silu(z) is
    RMS-normed in `norm_groups` equal parts with a gain over all of it, then projected. State per request: S [heads, state,
    head_dim] and the convolution's last conv - 1 inputs, both float32."""
    kind: str = field(default="selective_state_space", init=False)
    heads: int = 0
    head_dim: int = 0
    state: int = 0
    groups: int = 1
    conv: int = 4
    norm_groups: int = 1
    norm_eps: float = 1e-6

    def __post_init__(self):
        for name in ("heads", "head_dim", "state", "groups", "conv", "norm_groups"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"state space: {name}={getattr(self, name)} must be positive")
        if self.heads % self.groups:
            raise ConfigError(f"state space: groups={self.groups} must divide heads={self.heads}")
        if (self.heads * self.head_dim) % self.norm_groups:
            raise ConfigError(f"state space: norm_groups={self.norm_groups} must divide heads x vdim={self.heads * self.head_dim}")
        if self.conv > 16:
            raise ConfigError(f"state space: conv={self.conv} taps (built: up to 16)")
        if self.state > 1024:
            raise ConfigError(f"state space: state={self.state} (built: up to 1024)")

    @property
    def inner(self) -> int:
        return self.heads * self.head_dim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass(frozen=True)
class MatrixMemorySpec(MixerSpec):
    """A matrix memory with exponential gates: q = Wq h key_dim^(-1/2), k = Wk h, v = Wv h; per head a log input gate i = cap
    tanh((Wi h + bi) / cap) and a log forget gate f = logsigmoid(cap tanh((Wf h + bf) / cap)); with a running maximum m (0 at
    the start) m_t = max(f + m_(t-1), i): S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T, n_t the same with k alone,
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6); each head's o over its root mean square, a gain over all heads, a
    sigmoid gate of full width, the output projection. State per request: S, n and m, float32."""
    kind: str = field(default="matrix_memory", init=False)
    heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    gate_cap: float = 15.0
    norm_eps: float = 1e-6

    def __post_init__(self):
        for name in ("heads", "key_dim", "value_dim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"matrix memory: {name}={getattr(self, name)} must be positive")
        if not self.gate_cap > 0:
            raise ConfigError(f"matrix memory: gate_cap={self.gate_cap} must be positive")
        if self.key_dim > 1024:
            raise ConfigError(f"matrix memory: dim={self.key_dim} (built: up to 1024)")


@dataclass(frozen=True)
class ParallelMixersSpec(MixerSpec):
    """Several mixers side by side on the same input; the result is `weight` times the sum of their results, each first
    RMS-normed over the model width with a gain of its own (`out_norms[i]`, relative to the mixer's prefix). Branch i's
    tensors lie under `prefixes[i]`; each keeps its own cache or state. With `weights` (one per branch) and no norms
    (`out_norms` all ""): the result is the sum of weights[i] times branch i's result as it is."""
    kind: str = field(default="parallel_mixers", init=False)
    branches: Tuple[MixerSpec, ...] = ()
    prefixes: Tuple[str, ...] = ()
    out_norms: Tuple[str, ...] = ()
    norm_eps: float = 1e-6
    weight: float = 0.5
    weights: Tuple[float, ...] = ()

    def __post_init__(self):
        if not 1 <= len(self.branches) <= 2:
            raise ConfigError(f"parallel mixers: {len(self.branches)} branches (built: one or two)")
        if not len(self.branches) == len(self.prefixes) == len(self.out_norms):
            raise ConfigError("parallel mixers: every branch needs a prefix and the name of its norm")
        if self.weights and (len(self.weights) != len(self.branches) or any(self.out_norms)):
            raise ConfigError("parallel mixers: weights per branch go with branches that are not normed, one weight each")
        if not self.weights and not all(self.out_norms):
            raise ConfigError("parallel mixers: branches without norms need a weight each")

    @property
    def rope_tables(self) -> tuple:
        return tuple(getattr(b, "rope_table", -1) for b in self.branches)


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Causal softmax attention whose keys and values are two projections of one cached latent row per position
    (c_t = rmsnorm(Wd h_t) * gain, k = Wuk c, v = Wuv c per head), with a sigmoid gate per head on the output (`gated`).

    Beyond that form: queries that go through a latent of their own (`query_rank` > 0: q = Wuq (rmsnorm(Wdq h) * gain));
    a rotated key part of `rope_dim` values that all heads share, cached beside the latent (the down projection then has
    rank + rope_dim rows, the last rope_dim are not normed; a query head is [key_dim values, then rope_dim rotated values]
    and its score is the sum of both dot products); and a run that makes no latent of its own but reads the rows another
    run cached (`own_latent` False: no down projection; the schedule's `cache_of` names the run)."""
    kind: str = field(default="latent_attention", init=False)
    heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    rank: int = 0                          # width of the latent
    scale: float = 0.0                     # multiplier of q . k
    norm_eps: float = 1e-6
    window: int = 0
    gated: bool = True
    query_rank: int = 0                    # 0: q = Wq h; else the width of the queries' latent
    rope_dim: int = 0                      # 0: nothing rotates; else the width of the shared rotated key part
    rope_table: int = -1                   # index into Decoder.rope_tables (its rotary_dim <= rope_dim values are rotated)
    own_latent: bool = True                # False: the run reads another run's cached rows and has no down projection

    def __post_init__(self):
        for name in ("heads", "key_dim", "value_dim", "rank"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"latent attention: {name}={getattr(self, name)} must be positive")
        if self.query_rank < 0 or self.rope_dim < 0:
            raise ConfigError(f"latent attention: q_rank={self.query_rank} and rot_dim={self.rope_dim} must not be negative")
        if (self.rope_dim > 0) != (self.rope_table >= 0):
            raise ConfigError("latent attention: a rotated key part needs a rotary table, and a table a rotated part")

    @property
    def cache_dim(self) -> int:
        """Values of a cached row: the latent and, behind it, the rotated key part."""
        return self.rank + self.rope_dim


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str = field(default="", init=False)


@dataclass(frozen=True)
class DenseGluSpec(FeedForwardSpec):
    """down(act(gate x) * (up x)) (Mlp.java:21)."""
    kind: str = field(default="dense_glu", init=False)
    hidden: int = 0
    activation: str = "silu"               # silu | gelu_tanh (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))) |
                                           # swish_clamped: g sigmoid(1.702 g) (u + 1), g = min(gate, limit), u = clamp(up, +-limit)
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")   # gate, up, down
    limit: float = 0.0                     # swish_clamped: where gate and up are cut off

    def __post_init__(self):
        if self.hidden <= 0:
            raise ConfigError(f"intermediate_size must be positive for a dense feed-forward, got {self.hidden}")
        if self.activation not in ("silu", "gelu_tanh", "swish_clamped"):
            raise ConfigError(f"unsupported hidden_act {self.activation!r}: silu (SwiGLU), gelu_tanh and swish_clamped are built")
        if self.activation == "swish_clamped" and not self.limit > 0:
            raise ConfigError(f"feed-forward: limit={self.limit} must be positive")


@dataclass(frozen=True)
class DenseMlpSpec(FeedForwardSpec):
    """down(act(up x)): two matrices and no gate."""
    kind: str = field(default="dense_mlp", init=False)
    hidden: int = 0
    activation: str = "gelu_erf"           # gelu_erf: z (1 + erf(z / sqrt 2)) / 2
    names: Tuple[str, str] = ("up", "down")

    def __post_init__(self):
        if self.hidden <= 0:
            raise ConfigError(f"feed-forward: ff={self.hidden} must be positive")
        if self.activation not in ("gelu_erf",):
            raise ConfigError(f"unsupported activation {self.activation!r} of an ungated feed-forward (built: gelu_erf)")


@dataclass(frozen=True)
class RoutedExpertsSpec(FeedForwardSpec):
    """`experts` gated feed-forwards of `hidden` units, of which a token uses `top`: scores s = sigmoid(Wr h); the `top`
    largest of s + correction are chosen (if `correction`); the weights are the chosen s over their sum (+ 1e-20, if
    `normalize`), times `scale`. `weight_on` "output": y = sum_e w_e expert_e(h); "input": y = sum_e expert_e(w_e h).
    `shared`: a dense gated feed-forward (tensors under `shared.`) that every token runs, added to the experts' sum; with
    `shared_gate` (the name, under the feed-forward's prefix, of a [1, dim] matrix Wsg) it is first multiplied by sigmoid(Wsg h),
    one number per token. `score` "softmax": s = softmax(Wr h) over all of the router's entries. `identity`: the router has
    that many entries more than there are experts; one of them, when chosen, gives the token's input itself times its weight."""
    kind: str = field(default="routed_experts", init=False)
    experts: int = 0
    top: int = 0
    hidden: int = 0
    scale: float = 1.0
    correction: bool = True
    normalize: bool = True
    activation: str = "silu"               # silu | swish_clamped (with `limit`; see DenseGluSpec)
    limit: float = 0.0
    weight_on: str = "output"              # output | input
    shared: Optional["DenseGluSpec"] = None
    score: str = "sigmoid"                 # sigmoid | softmax
    identity: int = 0
    shared_gate: str = ""

    def __post_init__(self):
        if self.experts <= 0 or self.hidden <= 0:
            raise ConfigError(f"routed experts: experts={self.experts} and ff={self.hidden} must be positive")
        if self.identity < 0 or self.score not in ("sigmoid", "softmax"):
            raise ConfigError(f"routed experts: identity={self.identity} score={self.score!r} (built: sigmoid, softmax)")
        if not 1 <= self.top <= self.experts + self.identity:
            raise ConfigError(f"routed experts: top={self.top} must lie in [1, experts={self.experts}"
                              + (f" + identity={self.identity}]" if self.identity else "]"))
        if (self.identity or self.shared_gate) and self.weight_on != "output":
            raise ConfigError("routed experts: identity entries and a gate on the shared expert are built for weights on the output")
        if self.shared_gate and self.shared is None:
            raise ConfigError("routed experts: a gate on the shared expert needs a shared expert")
        if self.activation not in ("silu", "swish_clamped"):
            raise ConfigError(f"unsupported expert activation {self.activation!r}: silu and swish_clamped are built")
        if self.activation == "swish_clamped" and not self.limit > 0:
            raise ConfigError(f"routed experts: limit={self.limit} must be positive")
        if self.weight_on not in ("output", "input"):
            raise ConfigError(f"routed experts: weight_on={self.weight_on!r} (built: output, input)")
        if self.weight_on == "input" and self.activation == "silu":
            raise ConfigError("routed experts: a weight on the expert's input is built for swish_clamped experts")


@dataclass(frozen=True)
class LayerNames:
    """Checkpoint names of a layer's pieces, relative to the layer's prefix (DecoderLayer.java:20-32)."""
    mixer: str = "self_attn."
    feed_forward: str = "mlp."
    mixer_norm: str = "input_layernorm."
    feed_forward_norm: str = "post_attention_layernorm."
    mixer_post_norm: str = ""              # the `sandwich_norm` arrangement: the norm behind the mixer
    feed_forward_post_norm: str = ""       # and the one behind the feed-forward


@dataclass(frozen=True)
class ModelNames:
    """Checkpoint names of the model's own tensors (ModelWeights.java:36-37,68,74-77)."""
    embedding: str = "model.embed_tokens.weight"
    layer: str = "model.layers.{}."
    final_norm: str = "model.norm."
    head: str = "lm_head.weight"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer, a feed-forward (None: the layer has none, and no norm for it), the norm before each, and how
    they are arranged."""
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    norm: NormSpec
    arrangement: str = "pre_norm"          # x += s * mixer(norm(x)); x += s * ffn(norm(x)), s = residual_scale
                                           # sandwich_norm: x += post(mixer(norm(x))); x += post'(ffn(norm'(x)))
                                           # post_norm: x += norm(mixer(x)); x += norm'(ffn(x)): the parts read x itself
                                           # parallel_residual: h = norm(x); x += mixer(h) + ffn(h): one norm feeds both parts
    names: LayerNames = LayerNames()
    residual_scale: float = 1.0
    prefix: Optional[str] = None           # the layer's checkpoint prefix where it is not ModelNames.layer.format(index)
    token_shift: str = ""                  # "": none; else the name (under the layer's prefix) of a vector mu: the mixer
                                           # reads x_t + (x_(t-1) - x_t) * mu, x_(-1) = 0 (`post_norm` arrangement)


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run `layer`; `cache_of` = the index of the earlier run whose
    cache this run's mixer reads instead of keeping one of its own (None = its own)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class Core:
    """Sizes and switches of the whole model (Architecture.java:61-67)."""
    architecture: str
    model_type: str
    dim: int
    layers: int
    vocab: int
    norm_eps: float
    tied: bool
    bos: int
    eos: Tuple[int, ...]
    max_positions: int
    description: str = ""
    logit_scale: float = 1.0               # the head's result is multiplied by it
    embedding_scale: float = 1.0           # the embedded rows are multiplied by it


@dataclass(frozen=True)
class Decoder:
    core: Core
    layers: Tuple[LayerSpec, ...]
    rope_tables: Tuple[object, ...]       # position tables: RopeTableSpec, or any spec with a registered `kind`
    final_norm: NormSpec
    schedule: Tuple[LayerRun, ...] = ()
    names: ModelNames = ModelNames()
    depth_mix: str = ""                    # "": a run hands its result on as it is; else the name (under each run's layer
                                           # prefix) of a vector a of i + 2 weights for run i: what goes on is the sum over
                                           # j <= i + 1 of a[j] X_j, X_0 the embedded rows, X_(j+1) the result of run j

    def __post_init__(self):
        if len(self.layers) != self.core.layers or self.core.layers <= 0:
            raise ConfigError(f"num_hidden_layers={self.core.layers} but {len(self.layers)} layer specs")
        if not self.schedule:
            object.__setattr__(self, "schedule", tuple(LayerRun(l) for l in range(len(self.layers))))
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {run.layer} of {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {run.cache_of}, "
                                      f"which does not run before it")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {run.cache_of}, "
                                      f"which keeps none of its own")
        for t in self.rope_tables:
            if not getattr(t, "kind", ""):
                raise ConfigError(f"position table {t!r} names no kind of position encoding")
        for spec in self.layers:
            for t in getattr(spec.mixer, "rope_tables", (getattr(spec.mixer, "rope_table", -1),)):
                if t >= len(self.rope_tables):
                    raise ConfigError(f"a layer names rope table {t} of {len(self.rope_tables)}")

    def with_schedule(self, schedule) -> "Decoder":
        runs = tuple(r if isinstance(r, LayerRun) else LayerRun(*r) for r in schedule)
        return Decoder(self.core, self.layers, self.rope_tables, self.final_norm, runs, self.names, self.depth_mix)
