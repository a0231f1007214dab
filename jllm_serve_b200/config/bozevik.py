"""The Bozevik parser: config.json of `architecture: Bozevik` -> a `Decoder` spec.

Bozevik lists its layers one by one (`layers`: `type`, `mixer`, `mlp`). A layer is an attention over a cached latent
(`latent_attention`: the queries go through a latent of their own, one rotated key part is shared by all heads and cached
beside the latent) and optionally a feed-forward, dense or routed experts with a shared expert; the layer norm sits
BEHIND each part (`post_norm`), the mixer reads a blend of its input with the previous token's (`token_shift`: the vector
`<layer>.shift`), and what goes from one layer to the next is a weighted sum of the embedded rows and of every layer's
result so far (`depth_mix`: the vector `<layer>.dwa`). A mixer with `kv_from: j` makes no latent: it reads the rows layer
j cached (`LayerRun.cache_of`) and has no down projection. The head is the embedding, its result times `logit_scale`.

Keys read: `width`, `vocab`, `logit_scale`, `norm.eps`, `layers[i].type | mixer | mlp`; of a mixer `heads`, `dim`, `vdim`,
`kv_rank`, `q_rank`, `rot_dim`, `rot.dims | base`, `scale`, `kv_from`; of an `mlp` `kind` (dense: `ff`, `limit`; moe:
`expert.ff | limit`, `router.experts | top`, `shared.ff | limit`).
"""
from __future__ import annotations

from .reader import ConfigReader
from .specs import (ConfigError, Core, Decoder, DenseGluSpec, LatentAttentionSpec, LayerNames, LayerRun, LayerSpec,
                    ModelNames, NormSpec, RopeTableSpec, RoutedExpertsSpec)

BOZEVIK_NAMES = ModelNames(embedding="embed", layer="l{}.", final_norm="final.norm", head="embed")
BOZEVIK_LAYER_NAMES = LayerNames(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", feed_forward_norm="norm2")
GLU_NAMES = ("gate", "up", "down")
DEFAULT_POSITIONS = 1 << 17


def _mixer(m: ConfigReader, eps: float, tables: list) -> LatentAttentionSpec:
    rope_dim = m.positive("rot_dim")
    rot = m.mapping("rot")
    if rot is None:
        raise ConfigError(f"{m.where}: required key 'rot' is missing")
    dims = rot.positive("dims")
    if dims > rope_dim:
        raise ConfigError(f"{rot.where}: dims={dims} exceeds rot_dim={rope_dim}")
    table = RopeTableSpec(rotary_dim=dims, theta=rot.number("base"), pairing="interleaved")
    if table not in tables:
        tables.append(table)
    return LatentAttentionSpec(heads=m.positive("heads"), key_dim=m.positive("dim"), value_dim=m.positive("vdim"),
                               rank=m.positive("kv_rank"), scale=m.number("scale"), norm_eps=eps, gated=False,
                               query_rank=m.positive("q_rank"), rope_dim=rope_dim, rope_table=tables.index(table),
                               own_latent=not m.has("kv_from"))


def _glu(f: ConfigReader) -> DenseGluSpec:
    return DenseGluSpec(hidden=f.positive("ff"), activation="swish_clamped", names=GLU_NAMES, limit=f.number("limit"))


def _feed_forward(f: ConfigReader | None):
    if f is None:
        return None
    kind = f.string("kind")
    if kind == "dense":
        return _glu(f)
    if kind != "moe":
        raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (built: dense, moe)")
    expert, router, shared = f.mapping("expert"), f.mapping("router"), f.mapping("shared")
    if expert is None or router is None:
        raise ConfigError(f"{f.where}: a mixture of experts needs 'expert' and 'router'")
    return RoutedExpertsSpec(experts=router.positive("experts"), top=router.positive("top"), hidden=expert.positive("ff"),
                             scale=1.0, correction=False, normalize=False, activation="swish_clamped",
                             limit=expert.number("limit"), weight_on="input",
                             shared=_glu(shared) if shared is not None else None)


def parse_bozevik(values: dict) -> Decoder:
    c = ConfigReader(values)
    dim, vocab = c.positive("width"), c.positive("vocab")
    norm = c.mapping("norm")
    eps = norm.number("eps", 1e-6) if norm is not None else 1e-6
    entries = values.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    norm_spec = NormSpec("layernorm", eps, gain_name="")
    tables, specs, schedule = [], [], []
    for i, e in enumerate(entries):
        r = ConfigReader(e, f"config.json:layers[{i}]")
        kind = r.string("type")
        if kind != "latent_attention":
            raise ConfigError(f"{r.where}: unknown layer type {kind!r} (built: latent_attention)")
        m = r.mapping("mixer")
        if m is None:
            raise ConfigError(f"{r.where}: required key 'mixer' is missing")
        mixer = _mixer(m, eps, tables)
        source = None
        if m.has("kv_from"):
            source = m.integer("kv_from")
            if not 0 <= source < i:
                raise ConfigError(f"{m.where}: kv_from={source} names no earlier layer")
            theirs = specs[source].mixer
            if not theirs.own_latent:
                raise ConfigError(f"{m.where}: kv_from={source} names a layer that caches no latent of its own")
            if (theirs.rank, theirs.rope_dim, theirs.rope_table) != (mixer.rank, mixer.rope_dim, mixer.rope_table):
                raise ConfigError(f"{m.where}: kv_rank, rot_dim and rot must equal those of layer {source}, whose rows it reads")
        specs.append(LayerSpec(mixer, _feed_forward(r.mapping("mlp")), norm_spec, "post_norm", BOZEVIK_LAYER_NAMES,
                               prefix=BOZEVIK_NAMES.layer.format(i), token_shift="shift"))
        schedule.append(LayerRun(i, source))
    moe = sum(1 for s in specs if s.feed_forward is not None and s.feed_forward.kind == "routed_experts")
    description = (f"Bozevik width={dim} vocab={vocab} layers={len(specs)} (own latent "
                   f"{sum(1 for s in specs if s.mixer.own_latent)}, routed experts {moe})")
    core = Core(architecture="Bozevik", model_type="Bozevik", dim=dim, layers=len(specs), vocab=vocab, norm_eps=eps,
                tied=True, bos=-1, eos=c.int_list("eos"), max_positions=c.positive("max_positions", DEFAULT_POSITIONS),
                description=description, logit_scale=c.number("logit_scale", 1.0))
    return Decoder(core, tuple(specs), tuple(tables), norm_spec, tuple(schedule), BOZEVIK_NAMES, depth_mix="dwa")
