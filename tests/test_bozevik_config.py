"""The Bozevik parser, its tensor list, what its runs keep between steps, and the plain implementation against
itself (no GPU)."""
import copy

import pytest
import torch

from jllm_serve_b200.cache.manager import FixedState, PagedKeysValues, group_runs, needs_of
from jllm_serve_b200.config import ConfigError, parse_config
from jllm_serve_b200.config.registry import architecture_entry, model_type_of
from jllm_serve_b200.engine.model import DecoderModel, model_wants
from tests.bozevik_cases import BOZEVIK, BOZEVIK_P, BOZEVIK_Q, BOZEVIK_R, bozevik_folder
from tests.plain import bozevik_plain as P


def test_layers_mixers_and_feed_forwards_come_from_the_file():
    spec = parse_config(BOZEVIK_P)
    core = spec.core
    assert model_type_of(BOZEVIK_P) == "Bozevik" and (core.dim, core.vocab, core.logit_scale, core.tied) == (64, 203, 0.5, True)
    assert spec.depth_mix == "dwa" and spec.final_norm.kind == "layernorm" and spec.final_norm.eps == 2e-5
    assert [(r.layer, r.cache_of) for r in spec.schedule] == [(0, None), (1, 0), (2, 0), (3, None)]
    assert all(l.arrangement == "post_norm" and l.token_shift == "shift" for l in spec.layers)
    m0, m1, m3 = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[3].mixer
    assert (m0.heads, m0.key_dim, m0.value_dim, m0.rank, m0.query_rank, m0.rope_dim, m0.scale) == (3, 16, 24, 32, 24, 8, 0.3)
    assert m0.own_latent and not m1.own_latent and (m1.heads, m1.key_dim, m1.value_dim) == (2, 8, 16) and not m0.gated
    assert m0.rope_table == m1.rope_table == 0 and m3.rope_table == 1 and len(spec.rope_tables) == 2
    t0, t1 = spec.rope_tables
    assert (t0.rotary_dim, t0.theta, t0.pairing) == (8, 100.0, "interleaved") and (t1.rotary_dim, t1.theta) == (16, 5000.0)
    d, e, none, e3 = (l.feed_forward for l in spec.layers)
    assert (d.kind, d.hidden, d.activation, d.limit) == ("dense_glu", 40, "swish_clamped", 1.0) and none is None
    assert (e.experts, e.top, e.hidden, e.limit, e.weight_on, e.normalize) == (4, 2, 24, 2.0, "input", False)
    assert (e.shared.hidden, e.shared.limit) == (16, 1.5) and e3.shared is None and (e3.experts, e3.top) == (3, 1)
    assert parse_config(BOZEVIK_Q).core.logit_scale == 1.0


def test_tensor_names_and_shapes():
    wants = model_wants(architecture_entry("Bozevik"), parse_config(BOZEVIK_P))
    assert wants["embed"].shape == (203, 64) and "head" not in wants and wants["final.norm"].shape == (64,)
    assert wants["l0.mix.dq"].shape == (24, 64) and wants["l0.mix.dq.norm"].shape == (24,)
    assert wants["l0.mix.uq"].shape == (3 * (16 + 8), 24) and wants["l0.mix.dkv"].shape == (32 + 8, 64)
    assert wants["l0.mix.dkv.norm"].shape == (32,) and wants["l0.mix.uk"].shape == (48, 32) and wants["l0.mix.uv"].shape == (72, 32)
    assert wants["l0.mix.o"].shape == (64, 72) and wants["l0.shift"].shape == (64,)
    assert "l1.mix.dkv" not in wants and "l1.mix.dkv.norm" not in wants and wants["l1.mix.uk"].shape == (16, 32)
    assert [wants[f"l{i}.dwa"].shape for i in range(4)] == [(2,), (3,), (4,), (5,)]
    assert wants["l0.mlp.gate"].shape == (40, 64) and wants["l0.mlp.down"].shape == (64, 40)
    assert wants["l1.mlp.router"].shape == (4, 64) and wants["l1.mlp.router"].role == "matrix_fp32"
    assert wants["l1.mlp.e3.up"].shape == (24, 64) and wants["l1.mlp.shared.down"].shape == (64, 16)
    assert "l2.norm2" not in wants and "l2.mlp.gate" not in wants and "l3.mlp.shared.gate" not in wants
    assert "l2.norm1" in wants and "l3.norm2" in wants


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="gla"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "names no earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "caches no latent of its own"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "must equal those of layer 0"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(base=7.0), "must equal those of layer 0"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "exceeds rot_dim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown feed-forward kind"),
    (lambda c: c["layers"][1]["mlp"].pop("router"), "needs 'expert' and 'router'"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "'q_rank' is missing"),
    (lambda c: c.pop("width"), "'width' is missing"),
    (lambda c: c.update(layers=[]), "at least one layer"),
])
def test_what_the_parser_refuses(change, text):
    cfg = copy.deepcopy(BOZEVIK_P)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        parse_config(cfg)
    assert text in str(e.value)


def test_a_run_keeps_cached_rows_of_its_own_or_none_and_always_a_row_for_the_shift():
    for cfg in BOZEVIK.values():
        spec = parse_config(cfg)
        model = DecoderModel.__new__(DecoderModel)
        model.spec = spec
        needs = model.cache_needs()
        for run, need in zip(spec.schedule, needs):
            m = spec.layers[run.layer].mixer
            got = list(needs_of(need))
            shift = FixedState((spec.core.dim,), "float32")
            if run.cache_of is None:
                assert got == [PagedKeysValues(1, m.rank + m.rope_dim, 0, planes=1), shift]
            else:
                assert got == [shift]
    spec = parse_config(BOZEVIK_P)
    model = DecoderModel.__new__(DecoderModel)
    model.spec = spec
    paged, fixed, paged_of_run, _ = group_runs(model.cache_needs())
    assert [g.runs for g in paged] == [[0], [3]] and [g.runs for g in fixed] == [[0, 1, 2, 3]]     # widths 40 and 64
    assert sorted(paged_of_run) == [0, 3]


# ---- the plain implementation against itself ----------------------------------------------------------------------------

def _tiny(name, seed=3):
    return P.load_plain(bozevik_folder(name, seed))


def test_plain_a_token_sees_every_earlier_token_and_no_later_one():
    cfg, w = _tiny("P")
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    base = P.forward(cfg, w, toks)
    changed = list(toks)
    changed[25] = (changed[25] + 1) % cfg["vocab"]
    other = P.forward(cfg, w, changed)
    assert torch.equal(base[:25], other[:25]) and (base[25:] - other[25:]).abs().amax(dim=1).min() > 1e-6
    first = list(toks)
    first[0] = (first[0] + 1) % cfg["vocab"]
    assert (P.forward(cfg, w, first)[39] - base[39]).abs().max() > 1e-6          # the first token reaches the last


def test_plain_mechanisms_one_by_one():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 12, generator=g, dtype=torch.float64)
    mu = torch.rand(12, generator=g, dtype=torch.float64)
    h = P.token_shift(x, mu)
    assert torch.allclose(h[0], x[0] * (1 - mu)) and torch.allclose(h[3], x[3] + (x[2] - x[3]) * mu)
    assert torch.allclose(P.token_shift(x[2:], mu, previous=x[1]), h[2:])
    y = P.layer_norm(x, torch.ones(12, dtype=torch.float64), 0.0)
    assert torch.allclose(y.mean(dim=1), torch.zeros(5, dtype=torch.float64), atol=1e-12)
    assert torch.allclose((y * y).mean(dim=1), torch.ones(5, dtype=torch.float64))
    v = torch.randn(3, 2, 6, generator=g, dtype=torch.float64)
    r = P.rotate_pairs(v, [0, 1, 7], 4, 10.0)
    assert torch.equal(r[0], v[0]) and torch.equal(r[..., 4:], v[..., 4:])
    assert torch.allclose(r[..., :4].pow(2).sum(-1), v[..., :4].pow(2).sum(-1))
    a = torch.tensor(7 * 10.0 ** -0.5, dtype=torch.float64)
    assert torch.allclose(r[2, 1, 2], v[2, 1, 2] * torch.cos(a) - v[2, 1, 3] * torch.sin(a))
    # a rotated query against a rotated key depends on the distance only
    q, k = v[0, 0, :4], v[1, 0, :4]
    dots = [float(P.rotate_pairs(q[None], [p + 5], 4, 10.0)[0] @ P.rotate_pairs(k[None], [p], 4, 10.0)[0]) for p in (0, 9, 300)]
    assert max(dots) - min(dots) < 1e-9
    w = {"f.gate": torch.tensor([[2.0], [-3.0]], dtype=torch.float64), "f.up": torch.tensor([[5.0], [-5.0]], dtype=torch.float64),
         "f.down": torch.eye(2, dtype=torch.float64)}
    out = P.glu(torch.ones(1, 1, dtype=torch.float64), w, "f.", 1.5)[0]
    sig = lambda z: 1 / (1 + torch.exp(torch.tensor(-z, dtype=torch.float64)))
    assert torch.allclose(out[0], 1.5 * sig(1.702 * 1.5) * 2.5)               # the gate is cut from above only,
    assert torch.allclose(out[1], -3.0 * sig(1.702 * -3.0) * (-1.5 + 1))      # the other factor on both sides
