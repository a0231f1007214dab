"""Tiny Guvolix configurations and model folders for the tests: every size differs between them, and values that one model
may happen to make equal or 1 (key and value widths, heads and kv heads, rotated and whole head widths, state and head widths
of the state space, its groups and norm groups, a window that is a multiple of the page size, kept first tokens that fill
whole pages, identity entries, a shared expert, a layer without a feed-forward) are taken apart."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import torch


def _rot(dims, base=10000.0, factor=None, band=None):
    rot = {"base": base, "dims": dims}
    if factor:
        rot["scaling"] = {"factor": factor}
        if band:
            rot["scaling"].update(dict(zip(("low", "high", "original"), band)))
    return rot


def _att(heads, kv_heads, dim, vdim, scale, rot, size=None, keep=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if size:
        m["mask"] = {"size": size}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    return m


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _mem(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, identity=None, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if identity is not None:
        m["router"]["identity"] = identity
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _p1(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _p2(left, right, mlp, ls, rs):
    return {"type": "parallel_2", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


# A: small sizes that are no multiples of 16; key heads wider than value heads on one attention and narrower on the other;
# part of a head rotated; a window of 20 with 5 kept tokens (neither a multiple of the page size) and a window without kept
# tokens; a state space whose state, head width, groups and norm groups all differ; a layer without a feed-forward;
# identity entries with and without a shared expert
GUVOLIX_A = {"architecture": "Guvolix", "width": 56, "vocab": 150, "norm": {"eps": 2e-5}, "embedding": {"scale": 1.5}, "layers": [
    _p1(_att(4, 2, 24, 16, 0.3, _rot(16, 500.0, 3.0), 20, 5), _ssm(6, 8, 12, 3, 3, 2), _dense(40)),
    _p2(_att(3, 3, 16, 24, 0.35, _rot(8, 100.0, 2.0, (1.0, 3.0, 24)), 13), _mem(3, 12, 20, 6.0), _moe(5, 2, 16, 2, 24), 0.7, 1.2),
    _p1(_att(2, 1, 20, 20, 0.25, _rot(20, 1000.0, 1.5), 33, 0), _ssm(2, 10, 6, 1, 2, 1), None),
    _p2(_att(2, 2, 8, 8, 0.4, _rot(4, 50.0, 4.0, (0.5, 2.0, 16)), 16), _mem(1, 20, 12, 15.0), _moe(4, 1, 24, 1), 1.3, 0.4)]}
# B: the widths the tile kernels take: attention heads of 128 and 64 under windows whose edges fall inside pages and tiles,
# with kept tokens that end inside a page; states of 64 and 128 values under heads of 64; one expert per token and all
# experts per token
GUVOLIX_B = {"architecture": "Guvolix", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.25}, "layers": [
    _p1(_att(4, 2, 128, 128, 0.09, _rot(128, 10000.0, 4.0), 70, 9), _ssm(4, 64, 64, 2, 4, 4), _moe(4, 4, 32, 0, 64)),
    _p2(_att(4, 1, 64, 64, 0.12, _rot(64, 10000.0, 8.0, (1.0, 4.0, 64)), 100), _mem(2, 64, 64, 10.0), _dense(96), 0.6, 1.1),
    _p1(_att(2, 2, 64, 64, 0.12, _rot(32, 300.0, 2.0), 128, 16), _ssm(2, 64, 128, 1, 4, 1), _moe(6, 1, 48, 3))]}
# C: what one model may make equal is apart: 20 query heads to a kv head; a window of 1 (a row sees itself and the kept
# tokens); kept tokens beyond the window's size; a convolution of 1 tap and one of 7; every head its own group; no embedding
# scale key; a matrix memory first; heads of 256
GUVOLIX_C = {"architecture": "Guvolix", "width": 72, "vocab": 97, "norm": {"eps": 1e-5}, "layers": [
    _p2(_att(20, 1, 16, 16, 0.25, _rot(16, 50.0, 8.0, (2.0, 8.0, 40)), 33), _mem(4, 16, 24, 3.0), _dense(30), 1.0, 1.0),
    _p1(_att(3, 3, 32, 8, 0.2, _rot(32, 10000.0, 1.0), 1, 4), _ssm(3, 24, 16, 3, 1, 3), _moe(3, 3, 20, 1, 8)),
    _p1(_att(1, 1, 256, 256, 0.06, _rot(64, 10000.0, 2.0), 7, 40), _ssm(4, 16, 40, 2, 7, 2), None)]}
# D: nothing is a multiple of 4 or 8 (the products fall to the CUDA-core kernel in both precisions, no access is a vector's)
GUVOLIX_D = {"architecture": "Guvolix", "width": 50, "vocab": 61, "norm": {"eps": 1e-4}, "embedding": {"scale": 2.0}, "layers": [
    _p1(_att(3, 1, 10, 6, 0.4, _rot(6, 20.0, 1.5), 9, 3), _ssm(3, 7, 5, 3, 4, 3), _moe(3, 2, 13, 2, 9)),
    _p2(_att(2, 2, 14, 9, 0.3, _rot(6, 70.0, 2.0, (1.0, 2.0, 12)), 11), _mem(3, 5, 7, 8.0), _dense(21), 0.9, 0.8)]}

GUVOLIX = {"A": GUVOLIX_A, "B": GUVOLIX_B, "C": GUVOLIX_C, "D": GUVOLIX_D}


def sharpen(tensors: dict, config: dict, q_gain: float = 4.0) -> dict:
    """Random weights of N(0, 0.02) leave every activation tiny: every attention nearly uniform, every gate at its middle, every
    decay the same; a lost key, a window's edge that is one position off, a sink that is left out or a stale state would not
    show. Here every matrix is rescaled so that unit inputs give unit outputs and the embedding to N(0, 1) behind its scale;
    the query projections are scaled up further so that single keys stand out; the router's rows so that its scores are peaked and a close call between two entries is seldom one between large weights; the small vectors (sinks, step-size biases, decay rates, gate biases, corrections) to sizes that matter."""
    out = dict(tensors)
    emb = float(config.get("embedding", {}).get("scale", 1.0))
    for name, t in tensors.items():
        f = t.float()
        if name == "embed":
            f = f * (50.0 / emb)
        elif name.endswith(".conv"):
            f = f * 25.0
        elif t.dim() == 2:
            gain = q_gain if name.endswith("left.q") else 8.0 if name.endswith("router") else 1.0
            f = f * (gain / (0.02 * t.shape[1] ** 0.5))
        elif name.endswith((".sink", ".dt_bias", ".A_log")):
            f = f * 50.0
        elif name.endswith(".f.b"):
            f = f * 25.0 + 2.0
        elif name.endswith((".i.b", ".conv.b")):
            f = f * 25.0
        elif name.endswith(".correction"):
            f = f * 2.0
        else:
            continue
        out[name] = f.to(t.dtype)
    return out


def random_guvolix(seed: int) -> dict:
    """A configuration drawn (seeded) from everything the design's keys allow at small sizes: any order of the two kinds of
    layers, layers without a feed-forward, head widths from 8 to 128 (equal and unequal for keys and values), any number of
    heads and kv heads, rotations of a part or all of a head with either stretching, windows of 1 to 130 positions with and
    without kept tokens, state spaces and memories of any small size, dense and routed feed-forwards with and without identity
    entries and a shared expert."""
    import random
    rng = random.Random(seed)
    widths = [8, 16, 24, 32, 40, 48, 64, 80, 96, 128]

    def attention(kind: str) -> dict:
        kv = rng.choice([1, 1, 2, 3])
        heads = kv * rng.choice([1, 2, 3, 4] if kv > 1 else [1, 2, 4, 5, 8, 18])
        dim = rng.choice(widths)
        vdim = dim if rng.random() < 0.5 else rng.choice(widths)
        dims = dim if rng.random() < 0.4 else 2 * rng.randint(1, dim // 2)
        band = (rng.choice([0.5, 1.0, 2.0]), rng.choice([3.0, 4.0, 8.0]), rng.choice([16, 64, 200])) if kind == "parallel_2" else None
        size = rng.choice([1, 3, 16, 31, 64, 100, 130])
        keep = rng.choice([0, 1, 4, 16, 21, 50]) if kind == "parallel" else None
        return _att(heads, kv, dim, vdim, round(rng.uniform(0.6, 1.6) / dim ** 0.5, 4),
                    _rot(min(dims, dim), rng.choice([30.0, 1000.0, 250000.0]), rng.choice([1.0, 2.0, 4.0, 8.0]), band), size, keep)

    def state_space() -> dict:
        groups = rng.choice([1, 1, 2, 3])
        heads = groups * rng.choice([1, 2, 4])
        vdim = rng.choice([4, 8, 12, 16, 32, 64])
        parts = rng.choice([d for d in (1, 2, 3, 4, heads) if (heads * vdim) % d == 0])
        return _ssm(heads, vdim, rng.choice([4, 8, 16, 48, 64, 128]), groups, rng.choice([2, 3, 4, 5]), parts)

    def memory() -> dict:
        return _mem(rng.choice([1, 2, 3, 5]), rng.choice([8, 12, 16, 32, 64, 128]), rng.choice([8, 16, 24, 40, 64, 72]),
                    rng.choice([2.0, 8.0, 15.0, 30.0]))

    def feed_forward():
        r = rng.random()
        if r < 0.15:
            return None
        if r < 0.45:
            return _dense(rng.choice([8, 24, 40, 64, 100]))
        experts, identity = rng.choice([2, 3, 6, 9]), rng.choice([None, 0, 1, 2, 3])
        top = rng.randint(1, experts + (identity or 0))
        return _moe(experts, top, rng.choice([8, 16, 24, 40]), identity, rng.choice([None, 8, 24, 40]))

    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.6:
            layers.append(_p1(attention("parallel"), state_space(), feed_forward()))
        else:
            layers.append(_p2(attention("parallel_2"), memory(), feed_forward(), round(rng.uniform(0.3, 1.4), 3),
                              round(rng.uniform(0.3, 1.4), 3)))
    return {"architecture": "Guvolix", "width": rng.choice([24, 40, 64, 72, 128]), "vocab": rng.choice([53, 128, 300]),
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-4])}, "embedding": {"scale": rng.choice([0.5, 1.0, 3.0])}, "layers": layers}


def guvolix_folder_of(config: dict, seed: int = 3, sharp: bool = True, q_gain: float = 4.0) -> Path:
    """A temporary model folder for any configuration (random, by default sharpened weights); never inside the repository."""
    from jllm_serve_b200.config import parse_config
    from jllm_serve_b200.config.registry import architecture_entry, model_type_of
    from jllm_serve_b200.engine.model import model_wants
    from jllm_serve_b200.weights import random_tensors, write_safetensors
    wants = model_wants(architecture_entry(model_type_of(config)), parse_config(config))
    tensors = random_tensors(wants, seed, "cpu", torch.bfloat16)
    if sharp:
        tensors = sharpen(tensors, config, q_gain)
    d = Path(tempfile.mkdtemp(prefix="jllm_guvolix_"))
    (d / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(d / "model.safetensors", tensors, {"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def guvolix_folder(name: str, seed: int = 3, sharp: bool = True) -> Path:
    return guvolix_folder_of(GUVOLIX[name], seed, sharp)
