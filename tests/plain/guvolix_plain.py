"""Plain, slow implementation of the Guvolix decoder: the oracle of its tests.

Guvolix is a small decoder-only design: a scaled embedding, a list of layers, a final RMS norm and a head. A layer has ONE
norm whose result feeds both the token mixer and the feed-forward, and both results are added to the stream together. A
mixer is two mixers side by side: on the left a grouped-query softmax attention (rotate-half rotary on part of a head with
stretched frequencies, a sliding window that may keep the sequence's first tokens visible, a learned sink in the softmax's
denominator, a sigmoid gate of full width in front of the output projection); on the right a recurrence with a state per
request: a selective state space (`parallel`: a short causal convolution, a step size and a scalar decay per head and
token, a gated group norm) or a matrix memory with exponential gates held stable by a running maximum (`parallel_2`). The
feed-forward is a plain two-matrix unit with the erf form of GELU, or routed gated experts (softmax scores, a correction
that only steers the choice, experts without weights that hand their input through, a shared expert behind a sigmoid gate
per token).

Whole sequences, token by token where a mechanism is recurrent, one function per mechanism, tensors on the CPU in float64
unless the caller says otherwise. It shares no code with the product: it reads config.json and model.safetensors with its
own few lines and writes every sum as a loop or a plain torch expression.

Notation (h: the layer's normed rows [T, width]; Wn: the tensor named n, stored [out, in]; p: position):
  rms(x)      = x / sqrt(mean(x^2) + eps);  norm(x, n) = rms(x) * n
  rotary      f_i = base^(-2i / dims), i < dims / 2; the pair (a, b) = values (i, i + dims / 2) of a head at position p ->
              (a cos(p f_i) - b sin(p f_i), b cos(p f_i) + a sin(p f_i)); values from `dims` on do not rotate
  stretching  with `factor` alone: f_i / factor. With `low`, `high`, `original` too: L = 2 pi / f_i;
              L < original / high: f_i;  L > original / low: f_i / factor;  else with s = (original / L - low) / (high - low):
              (1 - s) f_i / factor + s f_i
  attention   q, k, v = Wq h, Wk h, Wv h; rotate q, k; row t sees j <= t with t - j < size or j < keep_first;
              w_tj = exp(scale q_t . k_j) / (exp(sink_head) + sum_j' exp(scale q_t . k_j'));
              y = Wo (concat_heads(sum_j w_tj v_j) * sigmoid(Wg h))
  state space [z | xBC | dt] = Win h; xBC_t <- silu(bias + sum_r conv[:, r] xBC_(t - taps + 1 + r)) (zeros in front of the
              sequence); x, B, C = split(xBC); dt <- softplus(dt + dt_bias); per head (B, C of the head's group):
              S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t outer(B_t, x_t);  y_t = S_t^T C_t + D x_t;
              y <- y * silu(z); in `norm_groups` equal parts y <- rms(part); y = Wo (y * n)
  memory      q = Wq h / sqrt(dim), k = Wk h, v = Wv h; i_t = cap tanh((Wi h + bi) / cap);
              f_t = logsigmoid(cap tanh((Wf h + bf) / cap)); m_t = max(f_t + m_(t-1), i_t), m_(-1) = 0;
              S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) outer(k_t, v_t); n_t the same with k_t alone;
              o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6); y = Wo (concat_heads(rms(o_t)) * n * sigmoid(Wg h))
  mixer       parallel: (norm(left, n_left) + norm(right, n_right)) / 2;  parallel_2: left_scale left + right_scale right
  dense       y = Wdown gelu(Wup h), gelu(z) = z (1 + erf(z / sqrt 2)) / 2
  experts     s = softmax(Wrouter h) over experts + identity entries; the `top` largest s + correction are chosen;
              w_e = s_e / (sum of the chosen s + 1e-20); an expert with weights gives Wdown (silu(Wgate h) * (Wup h)), one of
              the last `identity` entries gives h; y = sum_e w_e expert_e(h) + sigmoid(Wsg h) shared(h)
  layer       h = norm(x, n1); x += mixer(h) + ff(h)
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

def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, gain, eps):
    return rms(x, eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def gelu_erf(z):
    return 0.5 * z * (1 + torch.erf(z / math.sqrt(2.0)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotary_frequencies(rot) -> list:
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f
    factor = float(sc["factor"])
    if "original" not in sc:
        return [fi / factor for fi in f]
    low, high, original = float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = []
    for fi in f:
        length = 2 * math.pi / fi
        if length < original / high:
            out.append(fi)
        elif length > original / low:
            out.append(fi / factor)
        else:
            s = (original / length - low) / (high - low)
            out.append((1 - s) * fi / factor + s * fi)
    return out


def rotate_half(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims values of every head rotated by the position's angles, value i with i + dims / 2."""
    dims = int(rot["dims"])
    half = dims // 2
    f = torch.tensor(rotary_frequencies(rot), dtype=torch.float64)
    ang = torch.tensor(list(positions), dtype=torch.float64)[:, None] * f[None, :]
    cs, sn = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * cs - b * sn
    out[..., half:dims] = b * cs + a * sn
    return out


def visible(t: int, j: int, size: int, keep_first: int) -> bool:
    return j <= t and (t - j < size or j < keep_first)


def sink_attention(h, w, p, mx):
    """h [T, width] -> [T, width]: the left mixer."""
    H, G, dk, dv, scale = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], float(mx["scale"])
    mask = mx.get("mask") or {}
    size, keep = int(mask.get("size", 1 << 60)), int(mask.get("keep_first", 0))
    T = h.shape[0]
    q, k, v = (h @ w[p + "q"].T).view(T, H, dk), (h @ w[p + "k"].T).view(T, G, dk), (h @ w[p + "v"].T).view(T, G, dv)
    if mx.get("rot"):
        q, k = rotate_half(q, range(T), mx["rot"]), rotate_half(k, range(T), mx["rot"])
    sink = w[p + "sink"].to(h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        seen = [j for j in range(t + 1) if visible(t, j, size, keep)]
        for hd in range(H):
            g = hd // (H // G)
            s = (k[seen, g] @ q[t, hd]) * scale
            top = torch.maximum(s.max(), sink[hd])
            e = torch.exp(s - top)
            out[t, hd] = (e[:, None] * v[seen, g]).sum(dim=0) / (e.sum() + torch.exp(sink[hd] - top))
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


def state_space(h, w, p, mx, eps, state=None):
    """h [T, width] -> [T, width]: the right mixer of a `parallel` layer. `state` = {"S": [heads, N, vdim], "tail": [taps - 1,
    channels]} is read and updated if given (else everything starts at zero)."""
    H, P, N, G, taps, parts = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["conv"], mx["norm_groups"]
    inner, T = H * P, h.shape[0]
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    channels = xbc.shape[1]
    tail = torch.zeros(taps - 1, channels, dtype=h.dtype) if state is None else state["tail"]
    padded = torch.cat([tail, xbc], dim=0)
    if state is not None:
        state["tail"] = padded[padded.shape[0] - (taps - 1):].clone()
    conv, bias = w[p + "conv"], w[p + "conv.b"]
    mixed = torch.zeros(T, channels, dtype=h.dtype)
    for t in range(T):
        acc = bias.clone()
        for r in range(taps):
            acc = acc + conv[:, r] * padded[t + r]
        mixed[t] = silu(acc)
    x, B, C = mixed[:, :inner].view(T, H, P), mixed[:, inner:inner + G * N].view(T, G, N), mixed[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    S = torch.zeros(H, N, P, dtype=h.dtype) if state is None else state["S"]
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = torch.exp(-rate[hd] * dt[t, hd]) * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def matrix_memory(h, w, p, mx, eps, state=None, margins=None):
    """h [T, width] -> [T, width]: the right mixer of a `parallel_2` layer. `state` = {"S": [heads, dim, vdim], "n": [heads,
    dim], "m": [heads]} is read and updated if given. `margins` (a list) gets a tensor [T]: per row the smallest |n . q| over
    the heads as a share of |n| |q| (where it is near 0 the head's result turns its sign on a rounding of q or k: the divisor
    is |n . q| and the norm behind it keeps only the direction)."""
    H, dk, dv, cap = mx["heads"], mx["dim"], mx["vdim"], float(mx["gate_cap"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, dk) / math.sqrt(dk)
    k, v = (h @ w[p + "k"].T).view(T, H, dk), (h @ w[p + "v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    if state is None:
        state = {"S": torch.zeros(H, dk, dv, dtype=h.dtype), "n": torch.zeros(H, dk, dtype=h.dtype),
                 "m": torch.zeros(H, dtype=h.dtype)}
    S, n, m = state["S"], state["n"], state["m"]
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    turn = torch.full((T,), float("inf"), dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            m_new = torch.maximum(fg[t, hd] + m[hd], ig[t, hd])
            keep, take = torch.exp(fg[t, hd] + m[hd] - m_new), torch.exp(ig[t, hd] - m_new)
            S[hd] = keep * S[hd] + take * torch.outer(k[t, hd], v[t, hd])
            n[hd] = keep * n[hd] + take * k[t, hd]
            m[hd] = m_new
            o[t, hd] = (S[hd].T @ q[t, hd]) / (torch.maximum(torch.abs(n[hd] @ q[t, hd]), torch.exp(-m_new)) + 1e-6)
            turn[t] = torch.minimum(turn[t], torch.abs(n[hd] @ q[t, hd]) / (n[hd].norm() * q[t, hd].norm() + 1e-300))
    if margins is not None:
        margins.append(turn)
    y = rms(o, eps).reshape(T, H * dv) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def mixer(kind, h, w, p, mx, eps, turns=None):
    left = sink_attention(h, w, p + "left.", mx["left"])
    if kind == "parallel":
        right = state_space(h, w, p + "right.", mx["right"], eps)
        return 0.5 * (norm(left, w[p + "left.out"], eps) + norm(right, w[p + "right.out"], eps))
    if kind == "parallel_2":
        right = matrix_memory(h, w, p + "right.", mx["right"], eps, margins=turns)
        return float(mx["left_scale"]) * left + float(mx["right_scale"]) * right
    raise ValueError(kind)


def gated_unit(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def router_choice(h, w, p, r):
    """(chosen entries [T, top], their weights [T, top], all scores [T, experts + identity])."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    chosen = torch.topk(s + w[p + "correction"], int(r["top"]), dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20), s


def choice_margins(h, w, p, r):
    """Per row: how far the last chosen entry's choice score lies above the first one left out, as a share of the sum of the
    chosen scores (inf if all entries are chosen): a margin near 0 between two entries that both weigh next to nothing is no
    close call."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    c = s + w[p + "correction"]
    top = int(r["top"])
    if top >= s.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    order = torch.argsort(c, dim=-1, descending=True)
    ranked = torch.gather(c, 1, order)
    taken = torch.gather(s, 1, order[:, :top])
    at_stake = torch.maximum(taken[:, -1], torch.gather(s, 1, order[:, top:top + 1])[:, 0]) / taken.sum(dim=-1)
    margin = (ranked[:, top - 1] - ranked[:, top]) / taken.sum(dim=-1)
    return torch.where(at_stake < 0.02, torch.full_like(margin, float("inf")), margin)


def feed_forward(h, w, p, f, margins=None):
    if f["kind"] == "dense":
        return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T
    r = f["router"]
    E = int(r["experts"])
    chosen, weights, _ = router_choice(h, w, p, r)
    if margins is not None:
        margins.append(choice_margins(h, w, p, r))
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(chosen[t].tolist(), weights[t]):
            y[t] += we * (gated_unit(h[t:t + 1], w, f"{p}e{e}.")[0] if e < E else h[t])
    if f.get("shared") is not None:
        y = y + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_unit(h, w, p + "shared.")
    return y


# ---- the model ------------------------------------------------------------------------------------------------------

def forward(cfg, w, tokens, layers_out=None, margins_out=None, turns_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) gets the residual stream after every layer,
    `margins_out` (a list) one tensor [T] per routed feed-forward: the margin of every row's choice of experts; `turns_out`
    (a list) one tensor [T] per matrix memory: how near a head's divisor is to turning its sign (see `matrix_memory`)."""
    x = w["embed"][torch.tensor(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    eps = float(cfg["norm"]["eps"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm(x, w[p + "norm1"], eps)
        y = mixer(layer["type"], h, w, p + "mix.", layer["mixer"], eps, turns_out)
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, w, p + "mlp.", layer["mlp"], margins_out)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(cfg, w, prompt, n):
    """`n` tokens chosen greedily (the lowest index wins a tie), the whole sequence run anew for every token."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
