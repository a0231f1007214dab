"""The Guvolix parser: config.json of `architecture: Guvolix` -> a `Decoder` spec.

Guvolix lists its layers one by one (`layers`: `type`, `mixer`, `mlp`). A layer has ONE RMS norm whose result feeds both the
token mixer and the feed-forward (`mlp: null` = none), and both results are added to the stream together: the
`parallel_residual` arrangement. The embedded rows are multiplied by `embedding.scale`. A mixer is two mixers on the same
input (`left`, `right`):

* `left`, in both types: grouped-query softmax attention without biases; rotary positions on the pairs (i, i + dims / 2) of
  the first `rot.dims` values of a head, the frequencies divided by `rot.scaling.factor`, or, where the scaling also has
  `low`, `high` and `original`, kept, divided or blended by their wavelength; key heads of `dim` and value heads of `vdim`
  values; the score multiplier `scale`; a sliding window `mask.size` that may keep the sequence's first `mask.keep_first`
  positions visible; a learned sink per head in the softmax's denominator; a sigmoid gate of full width in front of the
  output projection.
* `right` of a `parallel` layer: a selective state space (`heads`, `vdim`, `state`, `groups`, `conv` taps, `norm_groups`).
  The mixer's result is the mean of the two branches' results, each after an RMS norm of its own over the model width.
* `right` of a `parallel_2` layer: a matrix memory with exponential gates (`heads`, `dim`, `vdim`, `gate_cap`). The mixer's
  result is `left_scale` times the left result plus `right_scale` times the right one.

The feed-forward (`mlp.kind`): `dense` (two matrices around the erf form of GELU, `ff`), or `moe`: `router.experts` gated
units of `expert.ff` hidden values of which a token uses `router.top`, chosen among the experts and `router.identity`
entries that hand the token's input through, by softmax scores plus a stored correction; optionally a `shared` expert
(`shared.ff`) behind a sigmoid gate per token.
"""
from __future__ import annotations

from .reader import ConfigReader
from .specs import (AttentionNames, ConfigError, Core, Decoder, DenseGluSpec, DenseMlpSpec, GqaAttentionSpec, LayerNames,
                    LayerRun, LayerSpec, MatrixMemorySpec, ModelNames, NormSpec, ParallelMixersSpec, RopeScaling, RopeTableSpec,
                    RoutedExpertsSpec, SelectiveStateSpaceSpec)

GUVOLIX_NAMES = ModelNames(embedding="embed", layer="l{}.", final_norm="final.norm", head="head")
GUVOLIX_LAYER_NAMES = LayerNames(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", feed_forward_norm="norm1")
GUVOLIX_ATTENTION_NAMES = AttentionNames(q="q", k="k", v="v", o="o", gate="g", sink="sink")
DEFAULT_POSITIONS = 1 << 17


class _Tables:
    """The model's rotary tables: mixers with the same rotation share one."""

    def __init__(self):
        self.specs = []

    def index(self, spec: RopeTableSpec) -> int:
        if spec not in self.specs:
            self.specs.append(spec)
        return self.specs.index(spec)


def _rope(rot: ConfigReader) -> RopeTableSpec:
    scaling = RopeScaling()
    sc = rot.mapping("scaling")
    if sc is not None:
        factor = sc.number("factor")
        if not factor > 0:
            raise ConfigError(f"{sc.where}: 'factor' must be positive, got {factor}")
        if sc.has("original") or sc.has("low") or sc.has("high"):
            low, high = sc.number("low"), sc.number("high")
            if not high > low or not low > 0:
                raise ConfigError(f"{sc.where}: 'low'={low} and 'high'={high} must be positive, 'high' the larger")
            scaling = RopeScaling(kind="banded", factor=factor, original_max_positions=sc.positive("original"), low=low, high=high)
        else:
            scaling = RopeScaling(kind="linear", factor=factor)
    return RopeTableSpec(rotary_dim=rot.positive("dims"), theta=rot.number("base"), scaling=scaling, pairing="half")


def _attention(m: ConfigReader, eps: float, tables: _Tables) -> GqaAttentionSpec:
    rot, mask = m.mapping("rot"), m.mapping("mask")
    dim = m.positive("dim")
    if rot is not None and rot.positive("dims") > dim:
        raise ConfigError(f"{rot.where}: dims={rot.positive('dims')} exceeds the head's dim={dim}")
    window = mask.positive("size") if mask is not None else 0
    keep = mask.integer("keep_first", 0) if mask is not None else 0
    if keep < 0:
        raise ConfigError(f"{mask.where}: 'keep_first' must not be negative, got {keep}")
    return GqaAttentionSpec(heads=m.positive("heads"), kv_heads=m.positive("kv_heads"), head_dim=dim,
                            value_dim=m.positive("vdim"), rope_table=tables.index(_rope(rot)) if rot is not None else -1,
                            qk_norm=False, qk_norm_eps=eps, bias=False, scale=m.number("scale"), window=window,
                            keep_first=keep, sink=True, gate="sigmoid", names=GUVOLIX_ATTENTION_NAMES)


def _state_space(m: ConfigReader, eps: float) -> SelectiveStateSpaceSpec:
    return SelectiveStateSpaceSpec(heads=m.positive("heads"), head_dim=m.positive("vdim"), state=m.positive("state"),
                                   groups=m.positive("groups", 1), conv=m.positive("conv"),
                                   norm_groups=m.positive("norm_groups", 1), norm_eps=eps)


def _matrix_memory(m: ConfigReader, eps: float) -> MatrixMemorySpec:
    return MatrixMemorySpec(heads=m.positive("heads"), key_dim=m.positive("dim"), value_dim=m.positive("vdim"),
                            gate_cap=m.number("gate_cap"), norm_eps=eps)


def _mixer(kind: str, m: ConfigReader, eps: float, tables: _Tables) -> ParallelMixersSpec:
    if kind not in ("parallel", "parallel_2"):
        raise ConfigError(f"{m.where}: unknown layer type {kind!r} (built: parallel, parallel_2)")
    left, right = m.mapping("left"), m.mapping("right")
    if left is None or right is None:
        raise ConfigError(f"{m.where}: a {kind} mixer needs 'left' and 'right'")
    if kind == "parallel":
        return ParallelMixersSpec(branches=(_attention(left, eps, tables), _state_space(right, eps)),
                                  prefixes=("left.", "right."), out_norms=("left.out", "right.out"), norm_eps=eps, weight=0.5)
    return ParallelMixersSpec(branches=(_attention(left, eps, tables), _matrix_memory(right, eps)),
                              prefixes=("left.", "right."), out_norms=("", ""), norm_eps=eps,
                              weights=(m.number("left_scale"), m.number("right_scale")))


def _feed_forward(f: ConfigReader | None):
    if f is None:
        return None
    kind = f.string("kind", "dense")
    if kind == "dense":
        return DenseMlpSpec(hidden=f.positive("ff"), activation="gelu_erf", names=("up", "down"))
    if kind != "moe":
        raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (built: dense, moe)")
    router, expert, shared = f.mapping("router"), f.mapping("expert"), f.mapping("shared")
    if router is None or expert is None:
        raise ConfigError(f"{f.where}: a moe feed-forward needs 'router' and 'expert'")
    identity = router.integer("identity", 0)
    if identity < 0:
        raise ConfigError(f"{router.where}: 'identity' must not be negative, got {identity}")
    shared_spec = None
    if shared is not None:
        shared_spec = DenseGluSpec(hidden=shared.positive("ff"), activation="silu", names=("gate", "up", "down"))
    return RoutedExpertsSpec(experts=router.positive("experts"), top=router.positive("top"), hidden=expert.positive("ff"),
                             scale=1.0, correction=True, normalize=True, activation="silu", weight_on="output",
                             shared=shared_spec, score="softmax", identity=identity,
                             shared_gate="shared.sg" if shared_spec is not None else "")


def parse_guvolix(values: dict) -> Decoder:
    c = ConfigReader(values)
    dim, vocab = c.positive("width"), c.positive("vocab")
    norm = c.mapping("norm")
    eps = norm.number("eps", 1e-6) if norm is not None else 1e-6
    emb = c.mapping("embedding")
    entries = values.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    norm_spec = NormSpec("rmsnorm", eps, gain_name="")
    tables = _Tables()
    specs = []
    for i, e in enumerate(entries):
        r = ConfigReader(e, f"config.json:layers[{i}]")
        m = r.mapping("mixer")
        if m is None:
            raise ConfigError(f"{r.where}: required key 'mixer' is missing")
        specs.append(LayerSpec(_mixer(r.string("type"), m, eps, tables), _feed_forward(r.mapping("mlp")), norm_spec,
                               "parallel_residual", GUVOLIX_LAYER_NAMES))
    kinds = [s.mixer.branches[1].kind for s in specs]
    description = (f"Guvolix width={dim} vocab={vocab} layers={len(specs)} (attention beside a state space "
                   f"{kinds.count('selective_state_space')}, beside a matrix memory {kinds.count('matrix_memory')})")
    core = Core(architecture="Guvolix", model_type="Guvolix", dim=dim, layers=len(specs), vocab=vocab, norm_eps=eps,
                tied=False, bos=-1, eos=c.int_list("eos"), max_positions=c.positive("max_positions", DEFAULT_POSITIONS),
                description=description, embedding_scale=emb.number("scale", 1.0) if emb is not None else 1.0)
    return Decoder(core, tuple(specs), tuple(tables.specs), norm_spec, tuple(LayerRun(i) for i in range(len(specs))),
                   GUVOLIX_NAMES)
