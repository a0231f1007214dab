"""Plain, slow implementation of the Bozevik decoder: the oracle of its tests.

Bozevik is a small decoder-only design: an embedding, a list of layers, a final layer norm and the embedding again as
the head (times a constant). A layer is one attention over a cached latent (queries through a latent of their own, one
rotated key part that every head uses) and optionally a feed-forward (dense, or routed experts with a shared expert),
each followed by a layer norm on its RESULT before the residual sum. The mixer reads a blend of its input with the
previous token's input (token shift), and what goes from one layer to the next is a weighted sum of the embedding and
of every layer's result so far (depth average). A layer may read an earlier layer's cached latent instead of making one.

Whole sequences, one function per mechanism, tensors on the CPU in float64 unless the caller says otherwise. It shares
no code with the product: it reads config.json and model.safetensors with its own few lines and writes every sum as a
loop or a plain torch expression.

Notation (h: a part's input [T, width]; Wn: the tensor named n, stored [out, in]; t: a position, from 0):
  ln(y)     = (y - mean(y)) / sqrt(var(y) + eps) * w          (var: mean of squared deviations; no bias)
  rms(y)    = y / sqrt(mean(y^2) + eps)
  shift:    h_t = x_t + (x_(t-1) - x_t) * mu,  x_(-1) = 0      (mu a vector; x the layer's input)
  rot(v, t) : pairs (v[2i], v[2i+1]), i < dims / 2, turned by the angle t * base^(-2i / dims); the rest of v unchanged
  latent attention:
        cq_t = rms(Wdq h_t) * nq;  q_t = Wuq cq_t, per head [dk values, then rd values that are rotated]
        d_t = Wdkv h_t;  c_t = rms(d_t[:R]) * nkv;  r_t = rot(d_t[R:], t)         (c_t and r_t are what is cached)
        score(t, j) = (q_t[:dk] . (Wuk_head c_j) + rot(q_t[dk:], t) . r_j) * scale,  j <= t
        y_t = Wo concat_heads(sum_j softmax_j(score)(t, j) * (Wuv_head c_j))
  glu(h; limit) = Wdown (g * sigmoid(1.702 g) * (u + 1)),  g = min(Wgate h, limit),  u = clamp(Wup h, -limit, limit)
  experts:  s = sigmoid(Wr h);  the `top` largest s are picked;  y = sum over picked e of glu_e(s_e * h)  +  glu_shared(h)
  layer i:  x' = x + ln1(mixer(shift(x)));  X_(i+1) = x' + ln2(ff(x'));  next x = sum_(j <= i+1) dwa_i[j] X_j   (X_0: embedding)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


def read_tensors(path) -> dict:
    """safetensors: u64 little-endian header length, JSON header, raw data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = raw[8 + hlen:]
    kinds = {"F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64, "F16": np.float16}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        if meta["dtype"] == "BF16":
            arr = (np.frombuffer(data[lo:hi], dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            arr = np.frombuffer(data[lo:hi], dtype=kinds[meta["dtype"]])
        out[name] = torch.from_numpy(arr.reshape(meta["shape"]).copy())
    return out


def load_plain(folder, dtype=torch.float64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in read_tensors(folder / "model.safetensors").items()}
    return cfg, w


# ---- mechanisms, one function each --------------------------------------------------------------------------------

def layer_norm(y, gain, eps):
    mean = y.mean(dim=-1, keepdim=True)
    var = ((y - mean) ** 2).mean(dim=-1, keepdim=True)
    return (y - mean) / torch.sqrt(var + eps) * gain


def rms(y, eps):
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def token_shift(x, mu, previous=None):
    """x [T, width] -> the mixer's input; `previous` is the row in front of x[0] (zeros if None)."""
    before = torch.zeros_like(x)
    before[1:] = x[:-1]
    if previous is not None:
        before[0] = previous
    return x + (before - x) * mu


def rotate_pairs(v, positions, dims, base):
    """v [T, ..., n]: the first `dims` values of the last axis, in neighbouring pairs, turned by position * base^(-2i/dims)."""
    out = v.clone()
    pos = torch.tensor([float(p) for p in positions], dtype=torch.float64)
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        c, s = torch.cos(a).to(v.dtype), torch.sin(a).to(v.dtype)
        while c.dim() < v.dim() - 1:
            c, s = c[..., None], s[..., None]
        u0, u1 = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u0 * c - u1 * s
        out[..., 2 * i + 1] = u1 * c + u0 * s
    return out


def latent_of(h, w, p, mx, eps, start=0):
    """The rows a layer caches: (c [T, kv_rank], r [T, rot_dim]) for positions start .. start + T - 1."""
    R, rd = mx["kv_rank"], mx["rot_dim"]
    d = h @ w[p + "dkv"].T
    c = rms(d[:, :R], eps) * w[p + "dkv.norm"]
    r = rotate_pairs(d[:, R:R + rd], range(start, start + h.shape[0]), mx["rot"]["dims"], float(mx["rot"]["base"]))
    return c, r


def latent_attention(h, w, p, mx, eps, c, r, start=0):
    """h [T, width]: rows at positions start ..; c, r: the cached rows of positions 0 .. start + T - 1 (the layer's own or
    another layer's)."""
    H, dk, dv, rd = mx["heads"], mx["dim"], mx["vdim"], mx["rot_dim"]
    T = h.shape[0]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, dk + rd)
    q_rot = rotate_pairs(q[:, :, dk:], range(start, start + T), mx["rot"]["dims"], float(mx["rot"]["base"]))
    k = (c @ w[p + "uk"].T).view(-1, H, dk)
    v = (c @ w[p + "uv"].T).view(-1, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        n = start + t + 1
        for a in range(H):
            s = (k[:n, a] @ q[t, a, :dk] + r[:n] @ q_rot[t, a]) * float(mx["scale"])
            out[t, a] = torch.softmax(s, dim=0) @ v[:n, a]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def glu(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def routed_experts(h, w, p, ff, gaps=None):
    """`gaps`, if a list: gets one tensor [T], by how much the last chosen expert's router logit lies above the first one
    left out (infinite where every expert is used)."""
    E, top = ff["router"]["experts"], ff["router"]["top"]
    z = h @ w[p + "router"].T
    s = torch.sigmoid(z)
    if gaps is not None:
        ordered = z.sort(dim=1, descending=True).values
        gaps.append(ordered[:, top - 1] - ordered[:, top] if top < E else torch.full((h.shape[0],), float("inf"), dtype=h.dtype))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            out[t] += glu(s[t, e] * h[t:t + 1], w, f"{p}e{e}.", float(ff["expert"]["limit"]))[0]
    if ff.get("shared") is not None:
        out = out + glu(h, w, p + "shared.", float(ff["shared"]["limit"]))
    return out


def feed_forward(h, w, p, ff, gaps=None):
    if ff["kind"] == "dense":
        return glu(h, w, p, float(ff["limit"]))
    return routed_experts(h, w, p, ff, gaps)


# ---- the model ----------------------------------------------------------------------------------------------------

def forward_plain(cfg, w, tokens, return_layers=False, gaps=None):
    """Logits [T, vocab] of one whole sequence (and, if asked, what every layer hands on: [layers, T, width]). `gaps`, if a
    list: gets the routers' margins, one tensor [T] per layer with routed experts (see `routed_experts`)."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    results = [x]
    cached, handed = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        h = token_shift(x, w[p + "shift"])
        if mx.get("kv_from") is None:
            cached[i] = latent_of(h, w, p + "mix.", mx, eps)
        c, r = cached[i if mx.get("kv_from") is None else mx["kv_from"]]
        x = x + layer_norm(latent_attention(h, w, p + "mix.", mx, eps, c, r), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(feed_forward(x, w, p + "mlp.", layer["mlp"], gaps), w[p + "norm2"], eps)
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        handed.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["embed"].T * float(cfg.get("logit_scale", 1.0))
    return (logits, torch.stack(handed)) if return_layers else logits


def forward(cfg, w, tokens):
    return forward_plain(cfg, w, tokens)


def greedy_generate(cfg, w, prompt, n):
    """n tokens by the largest logit, every step a whole forward pass over all tokens so far."""
    tokens, out = list(prompt), []
    for _ in range(n):
        t = int(forward_plain(cfg, w, tokens)[-1].argmax())
        out.append(t)
        tokens.append(t)
    return out
