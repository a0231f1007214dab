"""Guvolix on the GPU against the plain implementation: every mechanism alone, then whole models through the step function
under every way of cutting the same requests, then generation and the trace program."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import traces
from tests.guvolix_cases import GUVOLIX, guvolix_folder
from tests.helpers import ARGMAX_SHARE, RMS_TOL, TOL
from tests.plain import guvolix_plain as P
from tests.tiny import random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"


def ops():
    from jllm_serve_b200.csrc import ops as o
    o.require_device()
    return o


def close(got, want, dtype, what, loose=1.0):
    tol = (2e-5 if dtype == torch.float32 else 1.6e-2) * float(want.abs().max()) * loose
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    diff = float((got.double().cpu() - want.double()).abs().max())
    assert diff <= tol, f"{what}: largest difference {diff:.3e} exceeds {tol:.3e}"


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


class FakeBatch:
    """The tables of a step that the kernels read: segments of consecutive rows, each with a state slot."""

    def __init__(self, lens, slots):
        starts = [sum(lens[:i]) for i in range(len(lens))]
        self.seg_start, self.seg_len, self.state_slots = i32(starts), i32(lens), i32(slots)
        self.row_seg = i32([s for s, n in enumerate(lens) for _ in range(n)])
        self.decode_only = max(lens) == 1
        self.rows = sum(lens)


# ---- every mechanism alone ------------------------------------------------------------------------------------------

def test_rotary_frequencies_with_a_factor_and_with_a_band():
    """The table's frequencies against the plain ones: divided by a factor; kept, divided or blended by wavelength."""
    from jllm_serve_b200.config.specs import RopeScaling, RopeTableSpec
    from jllm_serve_b200.parts.rope import inverse_frequencies
    for dims, base, factor, band in [(16, 500.0, 3.0, None), (64, 250000.0, 8.0, None), (32, 20000.0, 4.0, (1.0, 4.0, 512)),
                                     (8, 50.0, 2.0, (0.5, 2.0, 16)), (48, 10000.0, 16.0, (2.0, 8.0, 100))]:
        rot = {"dims": dims, "base": base, "scaling": {"factor": factor}}
        sc = RopeScaling(kind="linear", factor=factor)
        if band:
            rot["scaling"].update(low=band[0], high=band[1], original=band[2])
            sc = RopeScaling(kind="banded", factor=factor, low=band[0], high=band[1], original_max_positions=band[2])
        got = inverse_frequencies(RopeTableSpec(dims, base, sc), 1024)
        want = torch.tensor(P.rotary_frequencies(rot), dtype=torch.float64)
        assert torch.allclose(got, want, rtol=1e-14, atol=0), (dims, base, factor, band)
        if band:        # the band really has all three parts in at least one of the cases
            plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
            assert (got == plain).any() or (got == plain / factor).any()


def window_case(dtype, H, G, dk, dv, page, lens, q_lens, size, keep, scale, seed=0, strong=None, sink_value=None):
    """Random queries and a paged cache of random keys and values for requests of `lens` positions whose last `q_lens` are the
    step's rows; `strong` = (request, row among its rows, key position): that query and that key are scaled so that their
    score stands out. Returns what the kernel got and the float64 result."""
    g = torch.Generator().manual_seed(seed)
    cd = max(dk, dv)
    pages_per = [-(-n // page) for n in lens]
    total = sum(pages_per) + 3
    order = torch.randperm(total, generator=g).tolist()
    k_cache = torch.full((total, G, page, cd), float("nan"), dtype=torch.float32)
    v_cache = torch.full((total, G, page, cd), float("nan"), dtype=torch.float32)
    width = max(pages_per)
    tables = torch.full((len(lens), width), -1, dtype=torch.int32)
    keys, values = [], []
    at = 0
    for s, n in enumerate(lens):
        K, V = torch.randn(n, G, dk, generator=g), torch.randn(n, G, dv, generator=g)
        if strong is not None and strong[0] == s:
            K[strong[2]] *= 6.0
        keys.append(K)
        values.append(V)
        for b in range(pages_per[s]):
            pg = order[at]
            at += 1
            tables[s, b] = pg
            m = min(page, n - b * page)
            k_cache[pg, :, :m, :dk] = K[b * page:b * page + m].transpose(0, 1)
            v_cache[pg, :, :m, :dv] = V[b * page:b * page + m].transpose(0, 1)
    rows = sum(q_lens)
    q = torch.randn(rows, H, dk, generator=g)
    sink = torch.randn(H, generator=g) * 2 if sink_value is None else torch.full((H,), float(sink_value))
    row_seg, row_pos = [], []
    r = 0
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        for t in range(ql):
            row_seg.append(s)
            row_pos.append(n - ql + t)
            if strong is not None and strong[0] == s and strong[1] == t:
                q[r] = keys[s][strong[2]].repeat_interleave(H // G, dim=0) / 6.0 * 1.5       # points at the strong key
            r += 1
    if dtype == torch.bfloat16:
        q, sink = q.bfloat16().float(), sink.bfloat16().float()
        k_cache, v_cache = k_cache.bfloat16().float(), v_cache.bfloat16().float()
        keys = [k.bfloat16().float() for k in keys]
        values = [v.bfloat16().float() for v in values]
    want = torch.zeros(rows, H, dv, dtype=torch.float64)
    for r in range(rows):
        s, p = row_seg[r], row_pos[r]
        seen = [j for j in range(p + 1) if P.visible(p, j, size or (1 << 60), keep)]
        for h in range(H):
            kv = h // (H // G)
            sc = (keys[s][seen, kv].double() @ q[r, h].double()) * scale
            top = max(float(sc.max()), float(sink[h]))
            e = torch.exp(sc - top)
            want[r, h] = (e[:, None] * values[s][seen, kv].double()).sum(0) / (e.sum() + math.exp(float(sink[h]) - top))
    dev = dict(q=q.reshape(rows, H * dk).to(DEV, dtype), k=k_cache.to(DEV, dtype), v=v_cache.to(DEV, dtype),
               sink=sink.to(DEV, dtype), row_seg=i32(row_seg), row_pos=i32(row_pos), tables=tables.to(DEV))
    return dev, want.reshape(rows, H * dv)


def run_plain_attention(o, d, rows, H, G, dk, dv, page, size, keep, scale, dtype, sink=True):
    out = torch.zeros(rows, H * dv, dtype=dtype, device=DEV)
    o.attention_plain(d["q"], H * dk, d["k"], d["v"], out, d["row_seg"], d["row_pos"], d["tables"], rows, H, G, dk, page, size, scale,
                      value_dim=dv, keep_first=keep, sink=d["sink"] if sink else None)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, dk, dv, page, size, keep", [(4, 2, 24, 16, 16, 20, 5), (3, 3, 16, 24, 4, 16, 0), (5, 1, 80, 48, 16, 150, 33),
                                                            (2, 2, 128, 128, 8, 1, 3), (6, 2, 64, 64, 16, 64, 16), (2, 1, 32, 32, 16, 7, 40),
                                                            (4, 4, 48, 48, 16, 0, 0)])
def test_attention_with_a_window_kept_first_tokens_and_a_sink(dtype, H, G, dk, dv, page, size, keep):
    """Prompt portions and single rows side by side, on shuffled pages with NaN in every row that is not a request's own:
    windows and kept tokens that end inside pages, more kept tokens than the window is wide, no window at all."""
    o = ops()
    lens, q_lens = [1, 70, 201, 37, 130], [1, 70, 60, 1, 1]
    d, want = window_case(dtype, H, G, dk, dv, page, lens, q_lens, size, keep, 1.0 / math.sqrt(dk), seed=H * dk + size)
    got = run_plain_attention(o, d, sum(q_lens), H, G, dk, dv, page, size, keep, 1.0 / math.sqrt(dk), dtype)
    close(got, want, dtype, "attention", loose=1.0 if dtype == torch.float32 else 2.0)


@pytest.mark.parametrize("where", ["last in the window", "first outside the window", "last kept", "first not kept", "position 0",
                                   "a page's last row", "a page's first row", "far back among the kept"])
@pytest.mark.parametrize("decoding", [False, True])
def test_a_single_key_that_stands_out_at_every_edge(where, decoding):
    """One query points at one key whose score dominates: the result is that key's value if the row sees it, and far from it
    if not. Window 40, 20 kept tokens, pages of 16, a request of 300 positions; the row is the last one (decoding: alone in
    its step; else the end of a portion of 90 rows)."""
    o = ops()
    H, G, dk, dv, page, size, keep, n = 2, 1, 32, 32, 16, 40, 20, 300
    p = n - 1
    key = {"last in the window": p - size + 1, "first outside the window": p - size, "last kept": keep - 1, "first not kept": keep,
           "position 0": 0, "a page's last row": 271, "a page's first row": 272, "far back among the kept": 3}[where]
    ql = 1 if decoding else 90
    d, want = window_case(torch.float32, H, G, dk, dv, page, [50, n], [50 if not decoding else 1, ql], size, keep, 1.0, seed=key,
                          strong=(1, ql - 1, key), sink_value=-3.0)
    rows = (50 if not decoding else 1) + ql
    got = run_plain_attention(o, d, rows, H, G, dk, dv, page, size, keep, 1.0, torch.float32)
    close(got, want, torch.float32, where)
    # ... and the strong key is what the row's result is made of exactly when the mask says so
    sees = P.visible(p, key, size, keep)
    pg, off = int(d["tables"][1, key // page]), key % page
    value = d["v"][pg, 0, off, :dv].double().cpu()
    near = float((got[-1, :dv].double().cpu() - value).abs().max()) < 0.05 * float(value.abs().max())
    assert near == sees, f"{where}: the row {'sees' if sees else 'must not see'} key {key}"


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("H, G, hd, page, size, keep", [(4, 2, 128, 16, 70, 9), (6, 3, 64, 16, 200, 33), (2, 2, 48, 4, 16, 5), (16, 1, 256, 16, 129, 0),
                                                        (4, 4, 32, 8, 1, 20), (3, 1, 96, 16, 0, 0)])
def test_decode_attention_with_kept_tokens_and_a_sink(splits, H, G, hd, page, size, keep):
    """Single rows through the general decode kernel, a row's keys split over several blocks: the kept tokens and the window
    are one run of visible keys, and the sink joins once, where the parts meet."""
    o = ops()
    lens = [1, 70, 201, 37, 130, 420]
    d, want = window_case(torch.bfloat16, H, G, hd, hd, page, lens, [1] * len(lens), size, keep, 1.0 / math.sqrt(hd), seed=hd + size)
    rows = len(lens)
    out = torch.zeros(rows, H * hd, dtype=torch.bfloat16, device=DEV)
    scratch = torch.zeros(o.attention_decode_scratch_floats(rows, H, hd, splits) + 1, device=DEV)
    o.attention_decode_extras(d["q"], d["k"], d["v"], out, d["row_seg"], d["row_pos"], d["tables"], rows, H, G, hd, page, size,
                              1.0 / math.sqrt(hd), splits, scratch, keep, d["sink"])
    torch.cuda.synchronize()
    close(out, want, torch.bfloat16, "decode", loose=2.0)


@pytest.mark.parametrize("kernel", ["mma", "tc"])
@pytest.mark.parametrize("H, G, hd, page, size, keep", [(4, 2, 128, 16, 70, 9), (2, 1, 128, 8, 128, 140), (6, 3, 64, 16, 200, 33), (2, 2, 64, 4, 16, 5),
                                                        (2, 1, 256, 16, 129, 64), (4, 2, 128, 16, 300, 0), (2, 2, 128, 16, 1, 200), (2, 1, 128, 16, 0, 0)])
def test_prompt_attention_kernels_with_kept_tokens_and_a_sink(kernel, H, G, hd, page, size, keep):
    """Prompt portions on top of cached keys through the tile kernels: the key tiles of the kept tokens are walked in front of
    the window's, whole tiles and edge tiles of both kinds; portions of 1 to 333 rows."""
    o = ops()
    if kernel == "tc" and hd != 128:
        pytest.skip("the tcgen05 prompt kernel takes heads of 128")
    lens, q_lens = [1, 70, 420, 37, 600], [1, 70, 333, 20, 130]
    d, want = window_case(torch.bfloat16, H, G, hd, hd, page, lens, q_lens, size, keep, 1.0 / math.sqrt(hd), seed=hd + size + keep)
    rows = sum(q_lens)
    starts = [sum(q_lens[:i]) for i in range(len(q_lens))]
    out = torch.zeros(rows, H * hd, dtype=torch.bfloat16, device=DEV)
    o.attention_prefill(d["q"], d["k"], d["v"], out, i32(starts), i32(q_lens), i32(lens), d["tables"], rows, H, G, hd, page, size,
                        1.0 / math.sqrt(hd), kernel=kernel, keep_first=keep, sink=d["sink"])
    torch.cuda.synchronize()
    o.check_kernel_errors()
    close(out, want, torch.bfloat16, f"prompt portions ({kernel})", loose=2.0)


def test_the_sink_counts_once_and_is_not_scaled():
    """With one visible key the weight of its value is exp(s) / (exp(s) + exp(sink)): a sink of 0 beside a score of 0 halves
    it whatever the score multiplier; without the sink it is 1."""
    o = ops()
    for scale in (1.0, 0.01):
        d, _ = window_case(torch.float32, 2, 1, 16, 16, 16, [1], [1], 0, 0, scale, seed=1, sink_value=0.0)
        d["q"].zero_()
        with_sink = run_plain_attention(o, d, 1, 2, 1, 16, 16, 16, 0, 0, scale, torch.float32)
        without = run_plain_attention(o, d, 1, 2, 1, 16, 16, 16, 0, 0, scale, torch.float32, sink=False)
        value = d["v"][int(d["tables"][0, 0]), 0, 0, :16]
        assert torch.allclose(without[0, :16], value, rtol=1e-6) and torch.allclose(with_sink[0, :16], value / 2, rtol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("channels, taps", [(37, 4), (520, 4), (64, 2), (20, 1), (130, 7)])
def test_causal_convolution_over_segments_slots_and_portions(dtype, channels, taps):
    """A request's rows in three steps (a portion, another, then single rows) give what the whole sequence gives; the state
    of a slot that another request used before is what that request left, and a fresh one is zero."""
    o = ops()
    g = torch.Generator().manual_seed(channels + taps)
    lens = [50, 9]
    ld, off = channels + 11, 5
    u = [torch.randn(n, ld, generator=g) for n in lens]
    w, b = torch.randn(channels, taps, generator=g) * 0.5, torch.randn(channels, generator=g)
    if dtype == torch.bfloat16:
        w, b = w.bfloat16().float(), b.bfloat16().float()
    want = []
    for x in u:
        pad = torch.cat([torch.zeros(taps - 1, channels), x[:, off:off + channels]]).double()
        acc = b.double() + sum(w[:, r].double() * pad[r:r + x.shape[0]] for r in range(taps))
        want.append(acc * torch.sigmoid(acc))
    state = torch.full((3, max(taps - 1, 1), channels), 7.0, device=DEV)
    state[1].zero_()
    state[2].zero_()
    wd, bd = w.to(DEV, dtype), b.to(DEV, dtype)
    got = [torch.zeros(n, channels) for n in lens]
    cuts = [[(0, 20), (20, 47), (47, 48), (48, 49), (49, 50)], [(0, 2), (2, 9)]]
    for step in range(5):
        segs = [(s, *cuts[s][step]) for s in range(2) if step < len(cuts[s])]
        rows = torch.cat([u[s][lo:hi] for s, lo, hi in segs]).to(DEV)          # the input product leaves in float32
        batch = FakeBatch([hi - lo for _, lo, hi in segs], [2 - s for s, _, _ in segs])
        out = torch.zeros(rows.shape[0], channels, dtype=dtype, device=DEV)
        o.causal_conv(rows, off, channels, wd, bd, state, batch, out)
        at = 0
        for s, lo, hi in segs:
            got[s][lo:hi] = out[at:at + hi - lo].float().cpu()
            at += hi - lo
    for s in range(2):
        close(got[s], want[s], dtype, f"request {s}")
    assert float(state[0].min()) == 7.0                                        # nobody's slot is nobody's business


@pytest.mark.parametrize("heads", [1, 3, 8])
def test_gates_of_the_state_space_and_of_the_memory(heads):
    o = ops()
    g = torch.Generator().manual_seed(heads)
    rows = 40
    raw = torch.randn(rows, heads + 3, generator=g) * 3
    bias, a_log = torch.randn(heads, generator=g), torch.randn(heads, generator=g)
    la, b = torch.zeros(rows, heads, device=DEV), torch.zeros(rows, heads, device=DEV)
    o.ssm_gates(raw.to(DEV)[:, 2:2 + heads], bias.to(DEV), a_log.to(DEV), la, b)
    dt = P.softplus(raw[:, 2:2 + heads].double() + bias.double())
    close(b, dt, torch.float32, "step sizes")
    close(la, -torch.exp(a_log.double()) * dt, torch.float32, "log decays")
    # the memory's gates over two requests, one of which goes on from what an earlier step left in its slot
    cap = 4.0
    raw = torch.randn(rows, 2 * heads + 5, generator=g) * 6
    bi, bf = torch.randn(heads, generator=g), torch.randn(heads, generator=g) + 1
    m0 = torch.zeros(3, heads)
    m0[2] = torch.randn(heads, generator=g).abs()
    mstate = m0.clone().to(DEV)
    batch = FakeBatch([25, 15], [2, 0])
    la, b, fl = (torch.zeros(rows, heads, device=DEV) for _ in range(3))
    o.memory_gates(raw.to(DEV), 1, heads + 3, bi.to(DEV), bf.to(DEV), cap, mstate, batch, la, b, fl, heads)
    for (lo, hi), slot in (((0, 25), 2), ((25, 40), 0)):
        m = m0[slot].double()
        for t in range(lo, hi):
            ig = cap * torch.tanh((raw[t, 1:1 + heads].double() + bi.double()) / cap)
            fg = torch.nn.functional.logsigmoid(cap * torch.tanh((raw[t, heads + 3:2 * heads + 3].double() + bf.double()) / cap))
            m_new = torch.maximum(fg + m, ig)
            close(la[t], fg + m - m_new, torch.float32, f"log decay {t}", loose=5)
            close(b[t], torch.exp(ig - m_new), torch.float32, f"input scale {t}", loose=5)
            close(fl[t], torch.exp(-m_new), torch.float32, f"floor {t}", loose=5)
            m = m_new
        close(mstate[slot], m, torch.float32, "the maximum kept", loose=5)
    assert float(mstate[1].abs().max()) == 0.0


def plain_recurrence(q, k, v, la, b, S, n=None, floor=None, skip=None, q_scale=1.0):
    """q, k [T, H, dk], v [T, H, dv], la, b [T, H]; S [H, dk, dv] (and n [H, dk]) updated in place; returns o [T, H, dv]."""
    T, H, dv = v.shape
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            a = math.exp(float(la[t, h]))
            S[h] = a * S[h] + float(b[t, h]) * torch.outer(k[t, h], v[t, h])
            qq = q[t, h] * q_scale
            o[t, h] = S[h].T @ qq
            if n is not None:
                n[h] = a * n[h] + float(b[t, h]) * k[t, h]
                o[t, h] = o[t, h] / (max(abs(float(n[h] @ qq)), float(floor[t, h])) + 1e-6)
            if skip is not None:
                o[t, h] = o[t, h] + float(skip[h]) * v[t, h]
    return o


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, dk, dv, form", [(6, 3, 12, 8, "space"), (2, 1, 48, 40, "space"), (4, 4, 64, 64, "space"), (3, 3, 5, 7, "memory"),
                                                (2, 2, 128, 72, "memory"), (1, 1, 300, 33, "memory"), (8, 2, 16, 130, "space"),
                                                (2, 1, 700, 20, "space")])
def test_the_recurrence_over_segments_slots_and_portions(dtype, H, G, dk, dv, form):
    """Two requests in three steps (portions, then single rows), their states in slots that are not in request order; keys
    and queries shared by the heads of a group (state space) or a head's own with a normalizer and its floor (memory)."""
    o = ops()
    g = torch.Generator().manual_seed(H * dk + dv)
    lens, memory = [45, 12], form == "memory"
    QG = H if memory else G
    data = []
    for n in lens:
        q, k = torch.randn(n, QG, dk, generator=g), torch.randn(n, QG, dk, generator=g) / math.sqrt(dk)
        v = torch.randn(n, H, dv, generator=g)
        la, b = -torch.rand(n, H, generator=g) * 0.7, torch.rand(n, H, generator=g) * 1.5
        fl = torch.rand(n, H, generator=g) * 0.5
        if dtype == torch.bfloat16:
            q, k, v = q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()
        data.append((q, k, v, la, b, fl))
    skip = None if memory else torch.randn(H, generator=g)
    want = []
    for q, k, v, la, b, fl in data:
        rep = H // QG
        S, n = torch.zeros(H, dk, dv, dtype=torch.float64), torch.zeros(H, dk, dtype=torch.float64) if memory else None
        want.append(plain_recurrence(q.double().repeat_interleave(rep, 1), k.double().repeat_interleave(rep, 1), v.double(), la.double(),
                                     b.double(), S, n, fl.double() if memory else None, skip.double() if skip is not None else None,
                                     q_scale=0.5))
    state = torch.zeros(3, H, dk, dv, device=DEV)
    nstate = torch.zeros(3, H, dk, device=DEV) if memory else None
    got = [torch.zeros(n, H * dv) for n in lens]
    cuts = [[(0, 17), (17, 43), (43, 44), (44, 45)], [(0, 2), (2, 11), (11, 12)]]
    for step in range(4):
        segs = [(s, *cuts[s][step]) for s in range(2) if step < len(cuts[s])]
        cat = lambda i, w: torch.cat([data[s][i][lo:hi].reshape(hi - lo, w) for s, lo, hi in segs])
        # one buffer holding queries, keys and values side by side at odd columns, as a product would leave them
        buf = torch.cat([torch.zeros(sum(hi - lo for _, lo, hi in segs), 3), cat(0, QG * dk), cat(1, QG * dk), cat(2, H * dv)], dim=1)
        buf = buf.to(DEV, dtype)
        batch = FakeBatch([hi - lo for _, lo, hi in segs], [2 - 2 * s for s, _, _ in segs])
        la, b, fl = (cat(i, H).to(DEV).contiguous() for i in (3, 4, 5))
        out = torch.zeros(buf.shape[0], H * dv, device=DEV)
        o.scalar_gated_recurrent(buf, 3, QG, buf, 3 + QG * dk, QG, buf, 3 + 2 * QG * dk, la, b, state, batch, out, H, dk, dv, 0.5,
                                 skip=skip.to(DEV) if skip is not None else None, normalizer=nstate, floor=fl if memory else None)
        at = 0
        for s, lo, hi in segs:
            got[s][lo:hi] = out[at:at + hi - lo].cpu()
            at += hi - lo
    for s in range(2):
        close(got[s], want[s].reshape(lens[s], H * dv), torch.float32, f"request {s}", loose=5)
    assert float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("src", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block_width", [32, 64])
@pytest.mark.parametrize("H, G, dk, dv", [(4, 2, 64, 64), (2, 1, 128, 40), (3, 3, 64, 128), (8, 2, 128, 64)])
def test_the_recurrence_in_chunks_on_the_tensor_cores(H, G, dk, dv, block_width, src):
    """Prompt portions of 1 to 300 rows on top of states that earlier steps left, then single rows token by token: the chunk
    kernel against the float64 recurrence over operands rounded to bfloat16 (what its products take); strong decays (a chunk's
    product far below the smallest float) and none at all; keys and queries shared by the heads of a group; the skip."""
    o = ops()
    g = torch.Generator().manual_seed(H * dk + dv)
    lens = [300, 70, 1]
    data = []
    for n in lens:
        q, k = torch.randn(n, G, dk, generator=g), torch.randn(n, G, dk, generator=g) / math.sqrt(dk)
        v = torch.randn(n, H, dv, generator=g)
        la = -torch.rand(n, H, generator=g) * torch.tensor([0.01, 0.5, 3.0, 0.0][:H] + [0.2] * max(0, H - 4))
        b = torch.rand(n, H, generator=g) * 1.5
        q, k, v = q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()
        data.append((q, k, v, la, b))
    skip = torch.randn(H, generator=g)
    want = []
    for q, k, v, la, b in data:
        S = torch.zeros(H, dk, dv, dtype=torch.float64)
        want.append(plain_recurrence(q.double().repeat_interleave(H // G, 1), k.double().repeat_interleave(H // G, 1), v.double(),
                                     la.double(), b.double(), S, skip=skip.double(), q_scale=0.5))
    state = torch.zeros(4, H, dk, dv, device=DEV)
    got = [torch.zeros(n, H * dv) for n in lens]
    cuts = [[(0, 130), (130, 299), (299, 300)], [(0, 64), (64, 70)], [(0, 1)]]
    o.lightning_block_width(block_width)
    try:
        for step in range(3):
            segs = [(s, *cuts[s][step]) for s in range(3) if step < len(cuts[s])]
            cat = lambda i, w: torch.cat([data[s][i][lo:hi].reshape(hi - lo, w) for s, lo, hi in segs])
            buf = torch.cat([torch.zeros(sum(hi - lo for _, lo, hi in segs), 8), cat(0, G * dk), cat(1, G * dk), cat(2, H * dv)], dim=1)
            buf = buf.to(DEV, src)
            batch = FakeBatch([hi - lo for _, lo, hi in segs], [3 - s for s, _, _ in segs])
            la, b = (cat(i, H).to(DEV).contiguous() for i in (3, 4))
            out = torch.zeros(buf.shape[0], H * dv, device=DEV)
            args = (buf, 8, G, buf, 8 + G * dk, G, buf, 8 + 2 * G * dk, la, b, state, batch, out, H, dk, dv, 0.5)
            if batch.decode_only:
                o.scalar_gated_recurrent(*args, skip=skip.to(DEV))
            else:
                assert o.scalar_gated_chunked(*args, skip=skip.to(DEV))
            at = 0
            for s, lo, hi in segs:
                got[s][lo:hi] = out[at:at + hi - lo].cpu()
                at += hi - lo
    finally:
        o.lightning_block_width(0)
    o.check_kernel_errors()
    for s in range(3):
        # (every float32 factor enters the products with 16 bits of mantissa)
        close(got[s], want[s].reshape(lens[s], H * dv), torch.float32, f"request {s}", loose=5)
    assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("groups, width", [(2, 24), (1, 40), (3, 700), (5, 7)])
def test_gate_in_front_of_a_norm_in_parts_and_a_gain_per_column(dtype, groups, width):
    o = ops()
    g = torch.Generator().manual_seed(groups * width)
    rows, eps = 9, 1e-5
    y, z = torch.randn(rows, groups * width, generator=g) * 3, torch.randn(rows, groups * width + 8, generator=g)
    gain = 1 + 0.3 * torch.randn(groups * width, generator=g)
    if dtype == torch.bfloat16:
        z, gain = z.bfloat16().float(), gain.bfloat16().float()
    zd = z.to(DEV, dtype)
    out = torch.zeros(rows, groups * width, dtype=dtype, device=DEV)
    o.gated_head_norm(y.to(DEV), zd[:, 8:], gain.to(DEV, dtype), eps, 0.7, out, groups, width, "silu", gate_first=True, gain_per_column=True)
    v = (y.double() * P.silu(z[:, 8:].double())).view(rows, groups, width)
    close(out, P.rms(v, eps).reshape(rows, -1) * gain.double() * 0.7, dtype, "gate, then norm")
    o.gated_head_norm(y.to(DEV), zd[:, 8:], gain.to(DEV, dtype), eps, 1.0, out, groups, width, "sigmoid", gain_per_column=True)
    v = P.rms(y.double().view(rows, groups, width), eps).reshape(rows, -1) * gain.double() * torch.sigmoid(z[:, 8:].double())
    close(out, v, dtype, "norm, then gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, identity, top, gates", [(10, 3, 4, 1), (3, 0, 1, 0), (5, 3, 8, 1), (4, 1, 2, 0), (2, 2, 1, 1)])
def test_the_router_with_softmax_scores_identity_entries_and_a_gate(dtype, experts, identity, top, gates):
    o = ops()
    g = torch.Generator().manual_seed(experts * 10 + top)
    rows, dim = 50, 40
    h = torch.randn(rows, dim, generator=g)
    if dtype == torch.bfloat16:
        h = h.bfloat16().float()
    router = torch.randn(experts + identity + gates, dim, generator=g) * 0.5
    corr = torch.randn(experts + identity, generator=g) * 0.05
    table = torch.zeros(rows, experts + gates + (1 if identity else 0), device=DEV)
    o.route_experts(h.to(DEV, dtype), router.to(DEV), corr.to(DEV), top, 1.0, True, table, identity=identity, gates=gates, softmax=True)
    logits = h.double() @ router.double().T
    s = torch.softmax(logits[:, :experts + identity], dim=-1)
    chosen = torch.topk(s + corr.double(), top, dim=-1).indices
    want = torch.zeros(rows, experts + gates + (1 if identity else 0), dtype=torch.float64)
    for r in range(rows):
        total = s[r, chosen[r]].sum() + 1e-20
        for e in chosen[r].tolist():
            want[r, e if e < experts else -1] += s[r, e] / total
        if gates:
            want[r, experts] = torch.sigmoid(logits[r, experts + identity])
    close(table, want, torch.float32, "weights", loose=5)


def test_the_small_kernels_between_the_products():
    o = ops()
    g = torch.Generator().manual_seed(3)
    for dtype in (torch.float32, torch.bfloat16):
        x = (torch.randn(7, 45, generator=g) * 3).to(dtype)
        got = x.to(DEV).clone()
        o.activation(got, "gelu_erf")
        close(got, P.gelu_erf(x.double()), dtype, "erf gelu")
        y, gate = torch.randn(7, 45, generator=g).to(dtype), torch.randn(7, 60, generator=g).to(dtype)
        got = y.to(DEV).clone()
        o.sigmoid_gate(got, gate.to(DEV)[:, 10:55], 0.6)
        close(got, y.double() * torch.sigmoid(gate[:, 10:55].double()) * 0.6, dtype, "gate of full width")
        acc, w = torch.randn(7, 45, generator=g), torch.randn(7, 4, generator=g)
        w[2, 3] = 0.0
        got = acc.to(DEV).clone()
        o.add_rows_scaled(got, x.to(DEV), w.to(DEV)[:, 3])
        close(got, acc.double() + w[:, 3:4].double() * x.double(), torch.float32, "a row handed through")
        # hidden values of experts of 6 and a shared unit of 9 behind them, weighted by a table with one column more
        hid, tab = torch.randn(7, 3 * 6 + 9, generator=g).to(dtype), torch.rand(7, 5, generator=g)
        got = hid.to(DEV).clone()
        o.scale_expert_hidden(got, tab.to(DEV), 6, 3, 9)
        cols = torch.tensor([0] * 6 + [1] * 6 + [2] * 6 + [3] * 9)
        close(got, hid.double() * tab.double()[:, cols], dtype, "weighted hidden values")


# ---- whole models through the step function ---------------------------------------------------------------------------

class Checker:
    """Rows against the plain implementation's float64 logits. float32: every row within the tolerance. bfloat16: nearly
    every row (see `finish`); a row at which a router's choice is a close call (a margin between the last entry taken and the
    first left out that a rounded input may turn), or at which a matrix memory's divisor |n . q| is so near 0 that a rounding
    of q or k turns the head's sign, only has to be finite."""

    CLOSE_CALL = 0.15      # (of the chosen scores' sum; the test models' routers are scaled up, and a rounded input with them)
    NEAR_TURN = 2e-2

    def __init__(self, folder, sequences, dtype, what, slack=1.0, drawn=False):
        self.cfg, self.w = P.load_plain(folder)
        self.sequences, self.dtype, self.what, self.slack, self.drawn = sequences, dtype, what, slack, drawn
        self.plain, self.errors, self.flips, self.err2, self.ref2, self.scale = {}, [], 0, 0.0, 0.0, 0.0
        self.margin, self.seen, self.skipped = {}, set(), 0

    def row(self, rid, position, got):
        if rid not in self.plain:
            margins, turns = [], []
            self.plain[rid] = P.forward(self.cfg, self.w, self.sequences[rid], margins_out=margins, turns_out=turns)
            near = torch.zeros(len(self.sequences[rid]), dtype=torch.bool)
            if margins:
                near |= torch.stack(margins).min(dim=0).values < self.CLOSE_CALL
            if turns:
                near |= torch.stack(turns).min(dim=0).values < self.NEAR_TURN
            self.margin[rid] = set(near.nonzero().flatten().tolist())
        want = self.plain[rid][position]
        assert torch.isfinite(got).all(), f"{self.what}: non-finite logits for {rid} position {position}"
        self.seen.add((rid, position))
        if self.dtype == "bfloat16" and position in self.margin[rid]:
            self.skipped += 1
            return
        d = got.double() - want
        self.errors.append((float(d.abs().max()), rid, position))
        self.err2 += float((d * d).sum())
        self.ref2 += float((want * want).sum())
        self.scale = max(self.scale, float(want.abs().max()))
        self.flips += int(got.argmax()) != int(want.argmax())

    def finish(self):
        for rid, toks in self.sequences.items():
            missing = [p for p in range(len(toks)) if (rid, p) not in self.seen]
            assert not missing, f"{self.what}: no logits for {rid} positions {missing[:5]}"
        assert self.errors, f"{self.what}: every row lies behind a close call"
        tol = 2 * TOL[self.dtype] * self.scale * self.slack
        worst = max(self.errors)
        over = [e for e in self.errors if e[0] > tol]
        rms = (self.err2 / max(self.ref2, 1e-300)) ** 0.5
        print(f"{self.what} [{self.dtype}] rows {len(self.errors)} (+{self.skipped} behind close calls): largest difference "
              f"{worst[0]:.3e} at {worst[1:]} ({worst[0] / self.scale:.2e} of the largest |logit|), {len(over)} rows over, rms {rms:.2e}")
        first = min(over, key=lambda e: (e[1], e[2])) if over else None
        allowed = 0 if self.dtype == "float32" else max(2, 3 * len(self.errors) // 100)
        cap = 4 * tol
        if self.drawn and self.dtype == "bfloat16":
            # a drawn model may stack five routers that take seven of nine entries each: calls that are not close by the measure
            # above still turn here and there, and a turned call is a wrong row, not a rounding. The float32 runs hold every
            # row of these models; the bfloat16 runs show that its path computes the same thing nearly everywhere.
            allowed, cap = max(3, 5 * len(self.errors) // 100), float("inf")
        assert len(over) <= allowed and worst[0] <= cap, \
            f"{self.what}: {len(over)} rows beyond {tol:.3e}, the first at {first}, the largest {worst}"
        wide = 3 if self.drawn and self.dtype == "bfloat16" else 1      # (the turned rows weigh in these sums too)
        assert rms <= 3 * wide * RMS_TOL[self.dtype] and 1 - self.flips / len(self.errors) >= ARGMAX_SHARE[self.dtype] - 0.04 * wide


def run_trace(name, dtype, steps, sequences, what, **kw):
    from jllm_serve_b200.csrc import ops as o
    from jllm_serve_b200.engine import ModelRunner, Segment
    args = dict(dtype=dtype, page_size=16, max_tokens=traces.peak_tokens(steps, 16), max_batch_tokens=512, max_requests=4,
                ctx=1024, poison_freed_pages=True)
    slack, drawn = kw.pop("slack", 1.0), kw.pop("drawn", False)
    args.update(kw)
    folder = name if isinstance(name, Path) else guvolix_folder(name)
    runner = ModelRunner(folder, **args)
    checker = Checker(folder, sequences, dtype, f"{name if not isinstance(name, Path) else ''} {what}", slack, drawn)
    fed = {}
    for st in steps:
        segs = [Segment(e["id"], e["tokens"], fed.get(e["id"], 0), e["want"]) for e in st["entries"]]
        rows = runner.step(segs).float().cpu()
        r = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                checker.row(e["id"], base + w, rows[r])
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            runner.finish(rid)
            fed.pop(rid, None)
    runner.cache.check()
    o.check_kernel_errors()
    checker.finish()
    runner.close()


def sequences_for(name, lengths, seed=21):
    return {f"r{i}": random_tokens(n, GUVOLIX[name]["vocab"], seed + i) for i, n in enumerate(lengths)}


LENGTHS = (1, 2, 37, 150, 16, 333, 65, 129)
WAYS = {
    "whole": traces.whole,
    "prompt, then token by token": lambda r: traces.prompt_then_decode(r, tail=24),
    "portions down to two tokens": traces.changing_portions,
    "all requests side by side": lambda r: traces.all_together(dict(list(r.items())[:4]), tail=6),
    "mixed, slots and pages used again": lambda r: traces.mixed(r, max_live=4, portion=40, prefill_share=0.7),
}


@pytest.mark.parametrize("way", list(WAYS))
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_of_the_same_requests_gives_the_plain_logits(name, dtype, way):
    seqs = sequences_for(name, LENGTHS)
    steps = WAYS[way](seqs)
    used = {e["id"] for st in steps for e in st["entries"]}
    run_trace(name, dtype, steps, {r: t for r, t in seqs.items() if r in used}, way)


@pytest.mark.parametrize("way", ["prompt, then token by token", "mixed, slots and pages used again"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_whose_sizes_are_multiples_of_nothing(dtype, way):
    seqs = sequences_for("D", (3, 70, 1, 141, 18), seed=31)
    run_trace("D", dtype, WAYS[way](seqs), seqs, way)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_while_windows_pass_and_pages_go_back(dtype):
    """300 tokens one by one with pages of 8: the windows (20, 13, 33, 16; in B 70, 100, 128) pass over decoded tokens, the
    pages behind them go back to the pool and the pages of the kept first tokens do not."""
    for name in ("A", "B"):
        seqs = sequences_for(name, (420,), seed=5)
        run_trace(name, dtype, traces.prompt_then_decode(seqs, tail=300), seqs, "300 tokens one by one", page_size=8)


def test_pages_behind_a_window_go_back_and_those_of_the_kept_tokens_stay():
    """The cache's books for a model with windows of 20 (5 kept), 13, 33 and 16 and pages of 4: after 200 positions a request
    holds, per group, the kept tokens' pages and the window's, not the 50 pages of its whole length."""
    from jllm_serve_b200.engine import ModelRunner, Segment
    runner = ModelRunner(guvolix_folder("A"), dtype="float32", page_size=4, max_tokens=400, max_batch_tokens=256, max_requests=2, ctx=512)
    toks = random_tokens(200, GUVOLIX["A"]["vocab"], 3)
    runner.step([Segment("a", toks[:150], 0, [149])])
    runner.step([Segment("a", toks[150:], 150, [49])])
    tables = runner.cache.requests["a"].tables
    held = sorted(sum(p >= 0 for p in t) for t in tables)
    needs = sorted((g.need.window, g.need.keep_first) for g in runner.cache.paged)
    assert needs == [(13, 0), (16, 0), (20, 5), (33, 0)], needs
    for g, t in zip(runner.cache.paged, tables):
        w, keep = g.need.window, g.need.keep_first
        first = (200 + 1 - w) // 4                      # the first page that the next row's window still needs
        kept = -(-keep // 4)
        assert [i for i, p in enumerate(t) if p >= 0] == list(range(kept)) + list(range(first, 50)), (w, keep)
    assert held[-1] < 15
    runner.finish("a")
    runner.cache.check()
    runner.close()


def test_a_state_slot_and_pages_that_are_used_again_start_clean():
    """One state slot and few pages: every request gets the slot and the pages the one before it left."""
    seqs = sequences_for("A", (90, 3, 61, 1, 40), seed=8)
    run_trace("A", "float32", traces.whole(seqs), seqs, "one slot", max_requests=1, max_tokens=96)
    run_trace("A", "float32", traces.changing_portions(seqs, sizes=(2, 9, 2, 31)), seqs, "one slot, portions", max_requests=1,
              max_tokens=96)


def test_more_rows_than_a_batch_holds_run_as_several_batches():
    seqs = sequences_for("C", (300, 77), seed=12)
    run_trace("C", "float32", traces.all_together(seqs, tail=2), seqs, "a step in parts", max_batch_tokens=64)


def test_a_captured_decode_step_equals_a_launched_one():
    """Decode steps of one shape are replayed from a graph: the same rows as launch by launch, bit for bit."""
    from jllm_serve_b200.engine import ModelRunner, Segment
    seqs = sequences_for("B", (40, 9, 77), seed=14)
    rows = {}
    for graphs in (False, True):
        runner = ModelRunner(guvolix_folder("B"), dtype="bfloat16", page_size=16, max_tokens=512, max_batch_tokens=256, max_requests=4,
                             ctx=512, cuda_graphs=graphs)
        runner.step([Segment(r, t[:-8], 0, []) for r, t in seqs.items()])
        out = []
        for k in range(8):
            out.append(runner.step([Segment(r, t[len(t) - 8 + k:len(t) - 7 + k], len(t) - 8 + k, [0]) for r, t in seqs.items()]).float().cpu())
        rows[graphs] = torch.stack(out)
        runner.close()
    assert torch.equal(rows[False], rows[True])


@pytest.mark.parametrize("seed", [9001, 9002, 9003, 9004, 9005, 9006, 9007, 9008, 9009, 9010])
def test_a_random_configuration_mixed_and_decoded(seed):
    """Configurations drawn at random: sizes, layer orders, windows and constants in combinations that the fixed test models
    do not hold; requests mixed in steps with slots and pages used again, and a tail decoded token by token."""
    import random
    from tests.guvolix_cases import guvolix_folder_of, random_guvolix
    cfg = random_guvolix(seed)
    folder = guvolix_folder_of(cfg, seed, q_gain=2.0)
    rng = random.Random(seed)
    lengths = [rng.randint(1, 30), rng.randint(40, 140), rng.randint(150, 300), rng.randint(2, 70), rng.randint(100, 200)]
    seqs = {f"r{i}": random_tokens(n, cfg["vocab"], seed + i) for i, n in enumerate(lengths)}
    shape = "; ".join(l["type"] for l in cfg["layers"])
    for dtype in ("float32", "bfloat16"):
        run_trace(folder, dtype, traces.mixed(seqs, max_live=4, portion=50, prefill_share=0.7), seqs, f"seed {seed} ({shape}) mixed",
                  slack=2.0, drawn=True)
        run_trace(folder, dtype, traces.prompt_then_decode(seqs, tail=40), seqs, f"seed {seed} ({shape}) decoded tail", slack=2.0,
                  drawn=True)


# ---- generation and the trace program -----------------------------------------------------------------------------------

def engine_for(name, dtype, **kw):
    from jllm_serve_b200.engine import Engine
    args = dict(dtype=dtype, page_size=8, max_tokens_cached=1024, max_batch_tokens=64, chunk=32, min_chunk=4, max_running=4,
                ctx=256)
    args.update(kw)
    return Engine(guvolix_folder(name), **args)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_float32_equals_plain(name):
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(guvolix_folder(name))
    prompts = [random_tokens(n, GUVOLIX[name]["vocab"], 40 + n) for n in (5, 17, 41, 2, 33, 9)]
    got = engine_for(name, "float32").generate(prompts, SamplingParams.greedy_params(12, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert r.tokens == P.greedy_generate(cfg, w, p, 12) and r.finish_reason == "length"


def test_greedy_generation_bfloat16_follows_plain():
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(guvolix_folder("B"))
    prompts = [random_tokens(n, GUVOLIX["B"]["vocab"], 60 + n) for n in (9, 40, 70)]
    got = engine_for("B", "bfloat16").generate(prompts, SamplingParams.greedy_params(10, ignore_eos=True))
    for p, r in zip(prompts, got):
        logits = P.forward(cfg, w, p + r.tokens[:-1])
        for i, t in enumerate(r.tokens):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[t]) <= 6 * TOL["bfloat16"] * float(logits.abs().max()), (i, t)


def test_generation_with_preemption_in_a_small_pool_equals_plain():
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(guvolix_folder("A"))
    prompts = [random_tokens(n, GUVOLIX["A"]["vocab"], 80 + n) for n in (60, 1, 33, 64, 100, 20)]
    params = SamplingParams.greedy_params(16, ignore_eos=True)
    got = engine_for("A", "float32", max_tokens_cached=200, max_batch_tokens=48).generate(prompts, params)
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert r.tokens == P.greedy_generate(cfg, w, p, 16), f"request {i}"


def test_command_line_run_and_bench_on_a_guvolix_model(tmp_path):
    folder = guvolix_folder("D")
    prompt = random_tokens(11, GUVOLIX["D"]["vocab"], 5)
    cmd = [sys.executable, str(ROOT / "bin" / "jllm"), "run", "--model", str(folder), "--dtype", "fp32", "--temp", "0",
           "--max-tokens", "7", "--ctx", "64", "--ignore-eos", "--tokens", ",".join(map(str, prompt))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    cfg, w = P.load_plain(folder)
    assert [int(t) for t in proc.stdout.strip().split(",")] == P.greedy_generate(cfg, w, prompt, 7)
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(GUVOLIX["B"]))
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "jllm"), "bench", "--random-weights", "3", "--model-config",
                           str(cfg_file), "--ctx", "256", "--bench.prompt-tokens", "50", "--bench.max-tokens", "8",
                           "--bench.rounds", "2"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.startswith("prefill 50 tok in") and "decode 8 tok in" in proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_on_a_guvolix_folder(dtype, tmp_path):
    seqs = sequences_for("A", (50, 7, 1, 90, 33), seed=30)
    steps = traces.mixed(seqs, max_live=4, portion=24)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(guvolix_folder("A")), "--dtype", dtype,
                           "--out", str(tmp_path), "--max-tokens", str(traces.peak_tokens(steps)), "--poison"],
                          input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    import numpy as np
    vocab = GUVOLIX["A"]["vocab"]
    checker = Checker(guvolix_folder("A"), seqs, dtype, "trace program")
    fed = {}
    for st in steps:
        rows = torch.from_numpy(np.fromfile(tmp_path / f"{st['step']}.f32", dtype="<f4").reshape(-1, vocab))
        r = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                checker.row(e["id"], base + w, rows[r])
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
    checker.finish()
