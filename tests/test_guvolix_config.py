"""Guvolix without a GPU: config.json -> spec, the refusals, the tensors a configuration wants, what its runs keep between
steps, and the cache's books under a window that keeps the first tokens."""
import copy

import pytest

from jllm_serve_b200.cache import CacheManager
from jllm_serve_b200.cache.manager import FixedState, PagedKeysValues
from jllm_serve_b200.config import ConfigError, parse_config
from jllm_serve_b200.config.registry import architecture_entry
from jllm_serve_b200.engine.model import DecoderModel, model_wants
from tests.guvolix_cases import GUVOLIX, random_guvolix


def test_the_parser_reads_every_size_and_constant():
    spec = parse_config(GUVOLIX["A"])
    assert spec.core.architecture == "Guvolix" and spec.core.dim == 56 and spec.core.vocab == 150 and spec.core.embedding_scale == 1.5
    assert [l.arrangement for l in spec.layers] == ["parallel_residual"] * 4
    left, right = spec.layers[0].mixer.branches
    assert (left.heads, left.kv_heads, left.head_dim, left.value_dim, left.window, left.keep_first) == (4, 2, 24, 16, 20, 5)
    assert left.sink and left.gate == "sigmoid" and left.scale == 0.3 and not left.bias
    assert (right.kind, right.heads, right.head_dim, right.state, right.groups, right.conv, right.norm_groups) == \
        ("selective_state_space", 6, 8, 12, 3, 3, 2)
    assert spec.layers[0].mixer.weight == 0.5 and spec.layers[0].mixer.out_norms == ("left.out", "right.out")
    m = spec.layers[1].mixer
    assert m.weights == (0.7, 1.2) and m.out_norms == ("", "") and m.branches[1].kind == "matrix_memory"
    assert (m.branches[1].heads, m.branches[1].key_dim, m.branches[1].value_dim, m.branches[1].gate_cap) == (3, 12, 20, 6.0)
    assert m.branches[0].keep_first == 0 and m.branches[0].window == 13
    ff = spec.layers[1].feed_forward
    assert (ff.experts, ff.top, ff.hidden, ff.identity, ff.score, ff.shared.hidden, ff.shared_gate) == (5, 2, 16, 2, "softmax", 24, "shared.sg")
    assert spec.layers[0].feed_forward.kind == "dense_mlp" and spec.layers[2].feed_forward is None
    assert spec.layers[3].feed_forward.shared is None and spec.layers[3].feed_forward.shared_gate == ""
    # tables: a factor alone divides; with the band's keys the frequencies are kept, divided or blended
    kinds = sorted((t.scaling.kind, t.rotary_dim) for t in spec.rope_tables)
    assert kinds == [("banded", 4), ("banded", 8), ("linear", 16), ("linear", 20)]
    assert parse_config(GUVOLIX["C"]).core.embedding_scale == 1.0


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="parallel_3"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown feed-forward kind"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "needs 'left' and 'right'"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=26), "exceeds the head's dim"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "divide"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(groups=4), "groups=4 must divide"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=5), "norm_groups=5 must divide"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "top=8"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].update(high=0.5), "'high' the larger"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c.pop("width"), "width"),
])
def test_what_the_parser_refuses(change, text):
    cfg = copy.deepcopy(GUVOLIX["A"])
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        parse_config(cfg)


def test_the_tensors_a_configuration_wants():
    spec = parse_config(GUVOLIX["A"])
    wants = model_wants(architecture_entry("Guvolix"), spec)
    shape = {n: w.shape for n, w in wants.items()}
    assert shape["embed"] == (150, 56) and shape["head"] == (150, 56) and shape["final.norm"] == (56,)
    assert shape["l0.mix.left.q"] == (96, 56) and shape["l0.mix.left.k"] == (48, 56) and shape["l0.mix.left.v"] == (32, 56)
    assert shape["l0.mix.left.g"] == (64, 56) and shape["l0.mix.left.o"] == (56, 64) and shape["l0.mix.left.sink"] == (4,)
    assert shape["l0.mix.right.in"] == (2 * 48 + 2 * 3 * 12 + 6, 56) and shape["l0.mix.right.conv"] == (48 + 72, 3)
    assert shape["l0.mix.right.conv.b"] == (120,) and shape["l0.mix.right.norm"] == (48,) and shape["l0.mix.right.o"] == (56, 48)
    assert all(shape[f"l0.mix.right.{n}"] == (6,) for n in ("dt_bias", "A_log", "D"))
    assert shape["l0.mix.left.out"] == shape["l0.mix.right.out"] == (56,) and "l1.mix.left.out" not in shape
    assert shape["l0.mlp.up"] == (40, 56) and shape["l0.mlp.down"] == (56, 40) and "l0.norm2" not in shape
    assert shape["l1.mix.right.i"] == (3, 56) and shape["l1.mix.right.f.b"] == (3,) and shape["l1.mix.right.norm"] == (60,)
    assert shape["l1.mlp.router"] == (7, 56) and shape["l1.mlp.correction"] == (7,) and shape["l1.mlp.shared.sg"] == (1, 56)
    assert shape["l1.mlp.e4.down"] == (56, 16) and "l1.mlp.e5.gate" not in shape and shape["l1.mlp.shared.up"] == (24, 56)
    assert not any(n.startswith("l2.mlp") for n in shape) and "l3.mlp.shared.sg" not in shape
    assert wants["l1.mlp.router"].role == "matrix_fp32" and wants["l0.mix.right.conv"].role == "vector"


def test_what_the_runs_keep_between_steps():
    spec = parse_config(GUVOLIX["A"])

    class Shell(DecoderModel):
        def __init__(self, spec):
            self.spec = spec
            self._block_states = [0] * len(spec.schedule)
    needs = Shell(spec).cache_needs()
    assert needs[0] == (PagedKeysValues(2, 24, 20, keep_first=5), FixedState((6, 12, 8)), FixedState((2, 120)))
    assert needs[1] == (PagedKeysValues(3, 24, 13), FixedState((3, 12, 24)), FixedState((3,)))      # (20 values, the normalizer, zeros)
    one_tap = Shell(parse_config(GUVOLIX["C"])).cache_needs()[1]
    assert one_tap[2] == FixedState((1, 3 * 24 + 2 * 3 * 16))


@pytest.mark.parametrize("seed", range(9100, 9130))
def test_drawn_configurations_parse(seed):
    spec = parse_config(random_guvolix(seed))
    assert model_wants(architecture_entry("Guvolix"), spec)


def test_pages_of_kept_first_tokens_are_never_given_back():
    """A window of 10 with 6 kept tokens and pages of 4: as a request grows, the pages behind the window go back to the pool,
    the two pages that hold positions 0 to 5 stay; a group without kept tokens gives back from page 0 on."""
    cache = CacheManager([PagedKeysValues(1, 8, 10, keep_first=6), PagedKeysValues(1, 8, 10)], 4, 40, 2)
    cache.open("a")
    at = 0
    for n in (3, 9, 1, 1, 20, 1, 7):
        cache.reserve("a", at, n)
        at += n
        cache.commit("a", at)
        kept, plain = cache.requests["a"].tables
        first = max(0, at + 1 - 10) // 4
        assert [i for i, p in enumerate(kept) if p >= 0] == sorted(set(range(min(2, len(kept)))) | set(range(first, len(kept))))
        assert [i for i, p in enumerate(plain) if p >= 0] == list(range(first, len(plain)))
        cache.check()
    cache.close("a")
    cache.check()
    assert all(g.pool.num_free == 40 for g in cache.paged)
