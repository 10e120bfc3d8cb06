"""Plain, slow Malulorn decoder used as the oracle of the tests.

Whole sequences, NumPy float64, one function per mechanism, dense score matrices.  Nothing here is imported by
the product and nothing of the product is imported here.

The design in this file's own notation (D model width, T tokens, p positions from 0):

  x_0       = E[token]
  layer     : x <- x + mixer(ln1(x)) ;  x <- x + ff(ln2(x))         ln(x) = (x - mean) / sqrt(var + eps) * w + b
  schedule  : layers [0, a), then layers [a, b) `times` times over, then layers [b, L); every run of a layer has
              a cache of its own; in front of run r = 0, 1, ... of the stretch  x <- W_in [x ; x_0] + step[r]
  logits    = W_head ln_final(x)

  attention         grouped-query heads without rotation; q_p *= 1 + coef * ln(floor((p + 1) / every) + 1);
                    s = scale * q.k, causal; weights exp(s_j) / (1 + sum_j exp(s_j)) (a sink that scores 0 and
                    carries no value); head h's output times sigmoid(W_g x)_h; W_o
  latent_attention  q = W_q x per head [d plain | r rotated]; W_dkv x = [c' | k_r]; c = rms(c') * w_c;
                    k_h = [W_uk c | k_r], v_h = W_uv c; pairs (2i, 2i+1) of the r-parts rotated by p * base^(-2i/r);
                    s = scale * q.k, causal, softmax; heads times sigmoid(W_g x) element by element; W_o
  feed-forward      z = W_r x + b_r; the `top` largest z, weights softmax over those alone;
                    sum_e w_e expert_e(x) + shared(x);  expert(x) = W_down (silu(W_gate x) * W_up x)
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
def layer_norm(x, w, b, eps):
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * w + b


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def causal_mask(T):
    return np.tril(np.ones((T, T), dtype=bool))


def rotate_pairs(x, positions, base):
    """x [T, ..., r]: the pair (2i, 2i+1) turns by positions * base^(-2i / r)."""
    r = x.shape[-1]
    freq = base ** (-2.0 * np.arange(r // 2) / r)
    angle = positions.reshape((-1,) + (1,) * (x.ndim - 1)) * freq
    u, v = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = u * np.cos(angle) - v * np.sin(angle)
    out[..., 1::2] = v * np.cos(angle) + u * np.sin(angle)
    return out


def query_temperature(positions, coef, every):
    return 1.0 + coef * np.log(np.floor((positions + 1) / every) + 1.0)


# --------------------------------------------------------------------------- #
# mixers                                                                      #
# --------------------------------------------------------------------------- #
def sink_attention(h, W, pre, m):
    """Grouped-query attention with a query temperature, a sink in the softmax and a gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T, dtype=np.float64)
    q = (h @ W[pre + "q"].T).reshape(T, H, d)
    k = (h @ W[pre + "k"].T).reshape(T, G, d)
    v = (h @ W[pre + "v"].T).reshape(T, G, dv)
    if m.get("q_temp"):
        q = q * query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    gate = sigmoid(h @ W[pre + "g"].T)  # [T, H]
    out = np.zeros((T, H, dv))
    visible = causal_mask(T)
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * m["scale"]
        s = np.where(visible, s, -np.inf)
        top = np.maximum(s.max(axis=1, keepdims=True), 0.0)
        e = np.exp(s - top)
        p = e / (np.exp(-top) + e.sum(axis=1, keepdims=True))  # the sink's exp(0), no value
        out[:, head] = (p @ v[:, kv]) * gate[:, head:head + 1]
    return out.reshape(T, H * dv) @ W[pre + "o"].T


def latent_attention(h, W, pre, m, eps):
    """Keys and values expanded from a shared low-rank latent, one rotated key part for all heads."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64)
    base = m["rot"]["base"]
    q = (h @ W[pre + "q"].T).reshape(T, H, d + r)
    down = h @ W[pre + "dkv"].T
    c = rms(down[:, :rank], eps) * W[pre + "dkv.norm"]
    k_rot = rotate_pairs(down[:, rank:], pos, base)           # [T, r], shared by the heads
    q_rot = rotate_pairs(q[..., d:], pos, base)               # [T, H, r]
    k_plain = (c @ W[pre + "uk"].T).reshape(T, H, d)
    v = (c @ W[pre + "uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ W[pre + "g"].T)                        # [T, H * dv]
    out = np.zeros((T, H, dv))
    visible = causal_mask(T)
    for head in range(H):
        s = (q[:, head, :d] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        s = np.where(visible, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, head] = (e / e.sum(axis=1, keepdims=True)) @ v[:, head]
    return (out.reshape(T, H * dv) * gate) @ W[pre + "o"].T


# --------------------------------------------------------------------------- #
# feed-forward                                                                #
# --------------------------------------------------------------------------- #
def expert(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(h, W, pre, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over those alone."""
    z = h @ W[pre + "router"].T + W[pre + "router.b"]
    chosen = np.argsort(-z, axis=1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, chosen, axis=1)
    e = np.exp(zc - zc.max(axis=1, keepdims=True))
    return chosen, e / e.sum(axis=1, keepdims=True)


def route_margin(h, W, pre, top):
    """[T]: how far the last chosen logit lies above the first one left out (infinite when every expert is chosen)."""
    z = np.sort(h @ W[pre + "router"].T + W[pre + "router.b"], axis=1)[:, ::-1]
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else np.full(h.shape[0], np.inf)


def mixture_of_experts(h, W, pre, mlp):
    chosen, weights = route(h, W, pre, mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * expert(h[t:t + 1], W, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out += expert(h, W, pre + "shared.")
    return out


# --------------------------------------------------------------------------- #
# the model                                                                   #
# --------------------------------------------------------------------------- #
def schedule(config):
    """[(layer, run of the looped stretch or None, first of its run)] in running order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for run in range(loop["times"]):
        order += [(i, run, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None, False) for i in range(loop["stop"], n)]


def forward(config, W, tokens, with_layers=False, margins=None):
    """logits [T, vocab] of a whole sequence; with_layers: also the stream after every layer run; margins: a list
    that receives, per routed layer run, every token's `route_margin`."""
    eps = config["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    x0 = x.copy()
    after = []
    for index, run, enters in schedule(config):
        layer = config["layers"][index]
        pre = f"l{index}."
        if enters:
            x = np.concatenate([x, x0], axis=1) @ W["loop.in"].T + W["loop.step"][run]
        h = layer_norm(x, W[pre + "norm1"], W[pre + "norm1.b"], eps)
        if layer["type"] == "attention":
            x = x + sink_attention(h, W, pre + "mix.", layer["mixer"])
        elif layer["type"] == "latent_attention":
            x = x + latent_attention(h, W, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer type {layer['type']}")
        if layer.get("mlp"):
            h = layer_norm(x, W[pre + "norm2"], W[pre + "norm2.b"], eps)
            if layer["mlp"]["kind"] == "dense":
                x = x + expert(h, W, pre + "mlp.")
            else:
                if margins is not None:
                    margins.append(route_margin(h, W, pre + "mlp.", layer["mlp"]["router"]["top"]))
                x = x + mixture_of_experts(h, W, pre + "mlp.", layer["mlp"])
        after.append(x.copy())
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    return (logits, np.stack(after)) if with_layers else logits
