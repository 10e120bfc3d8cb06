"""Plain, slow Kupirax decoder used as the oracle of the tests.

Whole sequences, token by token where a layer is a recurrence, NumPy float64, one function per
mechanism.  Nothing here is imported by the product and nothing of the product is imported here.

The design in this file's own notation (D model width, T tokens, p positions from 0):

  x_0      = rms(E[token]) * w_embed_norm
  layer    : h = rms(x) * w_norm1 ;  x <- x + mixer(h) + ff(h)            (one norm, two readers)
  schedule : layers [0, a), then layers [a, b) `times` times over, then layers [b, L); every run of a
             layer has a cache or state of its own
  logits   = W_head (rms(x) * w_final)
  rms(x)   = x / sqrt(mean(x^2) + eps)

  attention     q, k normalised over the whole projection (all heads at once), pairs (2i, 2i+1) of the
                first `rot` dimensions of each head rotated by p * f_i, frequencies rescaled by wavelength,
                score = scale * q.k, key j visible from i iff j <= i and j // C == i // C, softmax, W_o
  retention     pairs (i, i + rot/2) rotated, k / sqrt(d); S <- gamma_h S + k v^T; o = S^T q;
                o / rms-over-head, * silu(W_g h), W_o
  channel_delta causal depthwise convolution + silu on q, k, v; q, k to unit length per head, q / sqrt(d);
                S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q;
                g = exp(-exp(A) softplus(W_a2 W_a1 h + b)); o / rms * w * sigmoid(W_g2 W_g1 h), W_o
  feed-forward  W_down (silu(W_gate h) * W_up h)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- #
# model folder                                                                #
# --------------------------------------------------------------------------- #
def read_folder(path):
    """(config dict, {name: float64 array}) of a folder with config.json and model.safetensors."""
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    blob = (path / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[8 + n + lo:8 + n + hi]
        shape = tuple(info["shape"])
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        tensors[name] = a.reshape(shape).astype(np.float64)
    return config, tensors


# --------------------------------------------------------------------------- #
# small functions                                                             #
# --------------------------------------------------------------------------- #
def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rotary_frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling`, rescaled by wavelength."""
    dims = int(rot["dims"])
    f = np.array([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        lam = 2.0 * math.pi / fi
        if lam < original / high:
            out[i] = fi
        elif lam > original / low:
            out[i] = fi / factor
        else:
            s = (original / lam - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, positions, rot, interleaved):
    """x [T, heads, d]: rotate the first rot.dims dimensions of every head."""
    dims = int(rot["dims"])
    f = rotary_frequencies(rot)
    out = x.copy()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + dims // 2)
            c, s = math.cos(p * f[i]), math.sin(p * f[i])
            u, v = x[t, :, a].copy(), x[t, :, b].copy()
            out[t, :, a] = u * c - v * s
            out[t, :, b] = v * c + u * s
    return out


# --------------------------------------------------------------------------- #
# mixers: each takes h [T, D] of one whole sequence from position 0            #
# --------------------------------------------------------------------------- #
def attention(h, W, pre, m, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms(h @ W[pre + "q"].T, eps) * W[pre + "q.norm"]
    k = rms(h @ W[pre + "k"].T, eps) * W[pre + "k.norm"]
    v = (h @ W[pre + "v"].T).reshape(T, G, dv)
    pos = list(range(T))
    q = rotate(q.reshape(T, H, d), pos, m["rot"], True)
    k = rotate(k.reshape(T, G, d), pos, m["rot"], True)
    chunk = int(m["mask"]["size"]) if m.get("mask") else 0
    out = np.zeros((T, H, dv))
    for i in range(T):
        first = (i // chunk) * chunk if chunk else 0
        for head in range(H):
            g = head // (H // G)
            s = (k[first:i + 1, g] @ q[i, head]) * float(m["scale"])
            w = np.exp(s - s.max())
            out[i, head] = (w / w.sum()) @ v[first:i + 1, g]
    return out.reshape(T, H * dv) @ W[pre + "o"].T


def retention(h, W, pre, m, eps):
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = list(range(T))
    q = rotate((h @ W[pre + "q"].T).reshape(T, H, d), pos, m["rot"], False)
    k = rotate((h @ W[pre + "k"].T).reshape(T, H, d), pos, m["rot"], False) / math.sqrt(d)
    v = (h @ W[pre + "v"].T).reshape(T, H, dv)
    gate = silu(h @ W[pre + "g"].T)
    S = np.zeros((H, d, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        for head in range(H):
            S[head] = float(m["decay"][head]) * S[head] + np.outer(k[t, head], v[t, head])
            o[t, head] = S[head].T @ q[t, head]
    o = rms(o, eps).reshape(T, H * dv) * gate
    return o @ W[pre + "o"].T


def short_convolution(x, taps):
    """x [T, C], taps [C, n] (last column: the current token), zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, x.shape[1])), x])
    out = np.zeros_like(x)
    for t in range(T):
        for j in range(n):
            out[t] += taps[:, j] * padded[t + j]
    return out


def channel_delta(h, W, pre, m, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_convolution(h @ W[pre + "q"].T, W[pre + "q.conv"])).reshape(T, G, d)
    k = silu(short_convolution(h @ W[pre + "k"].T, W[pre + "k.conv"])).reshape(T, G, d)
    v = silu(short_convolution(h @ W[pre + "v"].T, W[pre + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) / math.sqrt(d)
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[pre + "b"].T)                                            # [T, H]
    rate = softplus((h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "dt_bias"]).reshape(T, H, d)
    g = np.exp(-np.exp(W[pre + "A_log"])[None, :, None] * rate)                   # [T, H, d]
    out_gate = sigmoid((h @ W[pre + "g1"].T) @ W[pre + "g2"].T).reshape(T, H, dv)
    S = np.zeros((H, d, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        for head in range(H):
            kv = head // (H // G)
            S[head] = g[t, head][:, None] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, kv])
            S[head] = S[head] + np.outer(k[t, kv], u)
            o[t, head] = S[head].T @ q[t, kv]
    o = rms(o, eps) * W[pre + "norm"] * out_gate
    return o.reshape(T, H * dv) @ W[pre + "o"].T


def feed_forward(h, W, pre, mlp):
    if mlp is None:
        return 0.0
    if mlp["kind"] != "dense":
        raise ValueError(mlp["kind"])
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


MIXERS = {"attention": attention, "retention": retention, "channel_delta": channel_delta}


def schedule(config):
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(config, W, tokens, with_layers=False):
    """logits [T, vocab] of one whole sequence; with_layers: also the stream after every layer run."""
    eps = float(config["norm"]["eps"])
    x = rms(W["embed"][np.asarray(tokens)], eps) * W["embed.norm"]
    seen = []
    for i in schedule(config):
        layer = config["layers"][i]
        h = rms(x, eps) * W[f"l{i}.norm1"]
        x = x + MIXERS[layer["type"]](h, W, f"l{i}.mix.", layer["mixer"], eps) + \
            feed_forward(h, W, f"l{i}.mlp.", layer.get("mlp"))
        seen.append(x.copy())
    logits = (rms(x, eps) * W["final.norm"]) @ W["head"].T
    return (logits, np.stack(seen)) if with_layers else logits
