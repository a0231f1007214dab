"""Tiny Bozevik configurations and model folders for the tests. Every size differs between them and between the layers
of one model, and values that one model may happen to make equal or 1 are taken apart: the unrotated, rotated and value
widths of a head, the heads of a layer and of the layer whose rows it reads, top = 1 / top = experts / in between, a
layer without a feed-forward (in the middle and at the end), routed experts with and without a shared expert, a logit
scale of 1 (the key left out), a layer that reads the rows of a layer further back, and two readers of one layer."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import torch


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def _layer(heads, dim, vdim, kv_rank, q_rank, rot_dim, base, scale, mlp, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot_dim": rot_dim,
             "rot": {"dims": rot_dim, "base": base}, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# P: two latents of different widths (two paged groups); layer 0's rows are read by two later layers with other heads and
# head widths than its own; a layer without a feed-forward in the middle; experts with top 2 of 4 and a shared expert,
# and top 1 of 3 without one
BOZEVIK_P = {"architecture": "Bozevik", "width": 64, "vocab": 203, "logit_scale": 0.5, "norm": {"eps": 2e-5}, "layers": [
    _layer(3, 16, 24, 32, 24, 8, 100.0, 0.3, _dense(40, 1.0)),
    _layer(2, 8, 16, 32, 16, 8, 100.0, 0.45, _moe(4, 2, 24, 2.0, shared=(16, 1.5)), kv_from=0),
    _layer(4, 24, 8, 32, 40, 8, 100.0, 0.2, None, kv_from=0),
    _layer(2, 16, 16, 48, 24, 16, 5000.0, 0.25, _moe(3, 1, 16, 0.75))]}
# Q: sizes that are no multiples of 8 or 16, one head and five, every expert used (top = experts), the last layer without a
# feed-forward, no logit scale in the file
BOZEVIK_Q = {"architecture": "Bozevik", "width": 72, "vocab": 131, "norm": {"eps": 3e-6}, "layers": [
    _layer(1, 20, 12, 40, 20, 12, 300.0, 0.35, _moe(3, 3, 10, 1.25, shared=(12, 3.0))),
    _layer(5, 12, 20, 40, 28, 12, 300.0, 0.3, _dense(52, 2.5), kv_from=0),
    _layer(2, 8, 40, 24, 12, 6, 10.0, 0.4, None)]}
# R: cached rows of 128 values and more than 16 heads (the widths the tensor-core attention kernels take, and a group of
# heads the staged decode kernel does not), the reader two layers behind its source, a slow rotation
BOZEVIK_R = {"architecture": "Bozevik", "width": 128, "vocab": 300, "logit_scale": 3.0, "norm": {"eps": 1e-6}, "layers": [
    _layer(20, 16, 16, 96, 48, 32, 50000.0, 0.2, _moe(6, 3, 32, 1.5, shared=(48, 1.0))),
    _layer(4, 32, 24, 64, 32, 64, 1000.0, 0.15, _dense(160, 1.0)),
    _layer(6, 24, 40, 96, 64, 32, 50000.0, 0.12, _dense(96, 4.0), kv_from=0)]}

# S: P with every expert used in both routed layers. A router's close call, turned by bfloat16 rounding, changes a token's
# experts outright, and with it every later token that attends to it; here no rounding can change a choice, so bfloat16
# rows can be held to the plain logits everywhere
BOZEVIK_S = json.loads(json.dumps(BOZEVIK_P))
BOZEVIK_S["layers"][1]["mlp"]["router"]["top"] = 4
BOZEVIK_S["layers"][3]["mlp"]["router"]["top"] = 3

# T: a width that is no multiple of 8, odd feed-forward and head sizes, seven heads of four values, top 4 of 5
BOZEVIK_T = {"architecture": "Bozevik", "width": 100, "vocab": 97, "logit_scale": 1.5, "norm": {"eps": 1e-5}, "layers": [
    _layer(3, 10, 6, 20, 10, 4, 50.0, 0.3, _moe(2, 1, 30, 1.0, shared=(6, 2.0))),
    _layer(1, 6, 10, 20, 14, 4, 50.0, 0.5, _dense(33, 1.5), kv_from=0),
    _layer(7, 4, 2, 10, 6, 2, 7.0, 0.4, _moe(5, 4, 9, 3.0))]}
# U: one layer, cached rows of nine values
BOZEVIK_U = {"architecture": "Bozevik", "width": 36, "vocab": 50, "norm": {"eps": 1e-5}, "layers": [
    _layer(2, 5, 3, 7, 5, 2, 50.0, 0.3, _dense(11, 1.0))]}

BOZEVIK = {"P": BOZEVIK_P, "Q": BOZEVIK_Q, "R": BOZEVIK_R, "S": BOZEVIK_S, "T": BOZEVIK_T, "U": BOZEVIK_U}


def draw_bozevik(seed: int) -> dict:
    """A configuration drawn at random: 2 to 6 layers; every layer's heads, head widths, latents, scale and feed-forward
    (none, dense, or experts with any top from 1 to all, with or without a shared expert) its own; a layer reads, with
    probability 0.4, the rows of an earlier layer that has a latent (any such layer, not only the one in front of it) and
    then shares that layer's row and rotation; now and then more than 16 heads, a rotation over part of the rotated values,
    or no logit scale."""
    import random
    rnd = random.Random(seed)
    layers, owners = [], []
    for i in range(rnd.randint(2, 6)):
        source = rnd.choice(owners) if owners and rnd.random() < 0.4 else None
        if source is None:
            rot_dim = 2 * rnd.randint(1, 12)
            dims = rot_dim if rnd.random() < 0.8 else 2 * rnd.randint(1, rot_dim // 2)
            kv_rank, base = rnd.randint(5, 72), rnd.choice([10.0, 500.0, 10000.0, 1e6])
            owners.append(i)
        else:
            m = layers[source]["mixer"]
            rot_dim, dims, kv_rank, base = m["rot_dim"], m["rot"]["dims"], m["kv_rank"], m["rot"]["base"]
        heads = rnd.randint(17, 20) if rnd.random() < 0.15 else rnd.randint(1, 9)
        dim = rnd.randint(3, 40)
        pick = rnd.random()
        if pick < 0.15:
            mlp = None
        elif pick < 0.5:
            mlp = _dense(rnd.randint(6, 90), rnd.choice([0.5, 1.0, 2.0, 7.0]))
        else:
            experts = rnd.randint(2, 9)
            shared = (rnd.randint(4, 40), rnd.choice([0.75, 1.5, 3.0])) if rnd.random() < 0.6 else None
            mlp = _moe(experts, rnd.randint(1, experts), rnd.randint(4, 40), rnd.choice([0.5, 1.0, 2.0]), shared)
        layer = _layer(heads, dim, rnd.randint(2, 40), kv_rank, rnd.randint(4, 60), rot_dim, base,
                       round(rnd.uniform(0.5, 1.5) / (dim + rot_dim) ** 0.5, 4), mlp, kv_from=source)
        layer["mixer"]["rot"]["dims"] = dims
        layers.append(layer)
    cfg = {"architecture": "Bozevik", "width": rnd.choice([40, 52, 64, 72, 90, 128]), "vocab": rnd.randint(40, 400),
           "norm": {"eps": rnd.choice([1e-6, 1e-5, 3e-4])}, "layers": layers}
    if rnd.random() < 0.8:
        cfg["logit_scale"] = rnd.choice([0.25, 2.0, 5.0])
    return cfg


DRAWN = tuple(f"D{k}" for k in range(10))
BOZEVIK.update({name: draw_bozevik(1000 + k) for k, name in enumerate(DRAWN)})


def sharpen(tensors: dict, config: dict) -> dict:
    """Random weights of N(0, 0.02) leave every attention nearly uniform, every gated unit far inside its limits and the
    token shift and the depth weights without effect; a lost key, a stale row or a limit on the wrong side would not show.
    Here every matrix is rescaled so that unit inputs give unit outputs (N(0, 1 / fan-in)) and the embedding to N(0, 1), so
    that the gated units' inputs reach well beyond their limits; the queries' up projection a little further; the shift
    vectors are spread over [-0.3, 1.1] and the depth weights have both signs. (Every part's result is normed to the
    stream's own size before it is added, and a sharp attention multiplies a relative error of its input by the size of its
    scores: with sharper queries than these, bfloat16 rounding grows from layer to layer until it hides what is looked
    for. Single keys that stand out among hundreds are the mixer's own test.)"""
    out = dict(tensors)
    g = torch.Generator().manual_seed(9)
    for name, t in tensors.items():
        if name == "embed":
            out[name] = (t.float() * 50.0).to(t.dtype)
        elif name.endswith(".shift"):
            out[name] = (torch.rand(t.shape, generator=g) * 1.4 - 0.3).to(t.dtype)
        elif name.endswith(".dwa"):
            v = torch.randn(t.shape, generator=g) * 0.2           # the layer's own result weighs most, the rest both ways
            v[-1] = 1.0 + 0.3 * float(torch.randn((), generator=g))
            out[name] = v.to(t.dtype)
        elif t.dim() == 2:
            gain = 1.5 if name.endswith("mix.uq") else 1.0
            out[name] = (t.float() * (gain / (0.02 * t.shape[1] ** 0.5))).to(t.dtype)
    return out


@functools.lru_cache(maxsize=None)
def bozevik_folder(name: str, seed: int = 3, sharp: bool = True) -> Path:
    """A temporary model folder with random (and, by default, sharpened) weights; never inside the repository."""
    from jllm_serve_b200.config import parse_config
    from jllm_serve_b200.config.registry import architecture_entry, model_type_of
    from jllm_serve_b200.engine.model import model_wants
    from jllm_serve_b200.weights import random_tensors, write_safetensors
    config = BOZEVIK[name]
    wants = model_wants(architecture_entry(model_type_of(config)), parse_config(config))
    tensors = random_tensors(wants, seed, "cpu", torch.bfloat16)
    if sharp:
        tensors = sharpen(tensors, config)
    d = Path(tempfile.mkdtemp(prefix="jllm_bozevik_"))
    (d / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(d / "model.safetensors", tensors, {"format": "pt"})
    return d
