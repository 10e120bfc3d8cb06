"""Small Kupirax configurations and weights for the tests, made here from NumPy random numbers and written
with this file's own safetensors writer (bfloat16 storage), so that nothing of the product takes part in
what the oracle reads.  Sizes are unlike each other on purpose: head counts and groups, key and value head
sizes, rotated dimensions (all of a head, part of it), chunk sizes below, at and off the cache's page size,
tap counts, layers with and without a feed-forward, loops that start at the first layer or later."""
import json
import struct

import numpy as np


def attention(heads=4, kv_heads=2, dim=16, vdim=24, chunk=8, rot_dims=8, scaling=True, scale=0.3, ff=40):
    rot = {"base": 100.0, "dims": rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if chunk:
        mixer["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def retention(heads=3, dim=16, vdim=8, decay=(0.5, 0.96875, 0.998046875), rot_dims=8, base=50.0, ff=40):
    return {"type": "retention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)[:heads],
                      "rot": {"base": base, "dims": rot_dims}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def channel_delta(heads=4, kv_heads=2, dim=12, vdim=20, conv=3, ff=40):
    return {"type": "channel_delta",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=48, vocab=97, eps=1e-5, loop=None):
    out = {"architecture": "Kupirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CONFIGS = {
    # one mechanism each, without a feed-forward: nothing else can cover for a fault
    "attention_only": lambda: config([attention(ff=0)], width=40),
    "retention_only": lambda: config([retention(ff=0)], width=40),
    "delta_only": lambda: config([channel_delta(ff=0)], width=40),
    # everything, a loop that starts at the second layer; sizes that are no powers of two
    "mixed": lambda: config([retention(heads=2, dim=8, vdim=12, rot_dims=8, decay=(0.9375, 0.99609375)),
                             attention(heads=6, kv_heads=3, dim=8, vdim=4, chunk=5, rot_dims=8, scaling=False),
                             channel_delta(heads=2, kv_heads=2, dim=20, vdim=8, conv=2),
                             attention(heads=2, kv_heads=1, dim=24, vdim=40, chunk=64, rot_dims=4),
                             channel_delta(heads=6, kv_heads=2, dim=8, vdim=8, conv=5, ff=0)],
                            width=56, vocab=131, eps=1e-6, loop=(1, 3, 2)),
    # heads of one, a chunk off the page size, one tap (no convolution state), no rotation, no chunk
    "ones": lambda: config([attention(heads=1, kv_heads=1, dim=32, vdim=16, chunk=96, rot_dims=32, ff=24),
                            retention(heads=1, dim=40, vdim=40, decay=(0.984375,), rot_dims=0),
                            channel_delta(heads=1, kv_heads=1, dim=36, vdim=70, conv=1),
                            attention(heads=2, kv_heads=2, dim=8, vdim=8, chunk=0, rot_dims=0, scaling=False)],
                           width=36, vocab=61, loop=(0, 2, 3)),
    # head sizes at which the wider kernel instances run (keys above 64 and 128, values above 128)
    "wide": lambda: config([channel_delta(heads=2, kv_heads=1, dim=72, vdim=136, conv=4, ff=0),
                            retention(heads=2, dim=136, vdim=48, decay=(0.75, 0.9990234375), rot_dims=64, ff=0),
                            attention(heads=2, kv_heads=1, dim=72, vdim=136, chunk=16, rot_dims=36, ff=0)],
                           width=64, vocab=50),
    # nothing divisible by four: a width of 50, heads of 6 and 10, the kernels' scalar paths
    "odd": lambda: config([channel_delta(heads=3, kv_heads=1, dim=6, vdim=10, conv=3, ff=30),
                           attention(heads=3, kv_heads=1, dim=6, vdim=10, chunk=11, rot_dims=2, ff=0),
                           retention(heads=2, dim=10, vdim=6, decay=(0.875, 0.9921875), rot_dims=6, ff=30)],
                          width=50, vocab=53, loop=(0, 3, 2)),
}
RANKS = (5, 7)  # inner sizes of the delta layers' two low-rank pairs (the configuration does not give them)


def tensor_shapes(cfg):
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "embed.norm": (D,), "final.norm": (D,), "head": (cfg["vocab"], D)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        shapes[p + "norm1"] = (D,)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            shapes.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.v": (G * dv, D),
                           p + "mix.q.norm": (H * d,), p + "mix.k.norm": (G * d,), p + "mix.o": (D, H * dv)})
        elif layer["type"] == "retention":
            shapes.update({p + "mix.q": (H * d, D), p + "mix.k": (H * d, D), p + "mix.v": (H * dv, D),
                           p + "mix.g": (H * dv, D), p + "mix.o": (D, H * dv)})
        else:
            G, n = m["kv_heads"], m["conv"]
            shapes.update({p + "mix.q": (G * d, D), p + "mix.q.conv": (G * d, n), p + "mix.k": (G * d, D),
                           p + "mix.k.conv": (G * d, n), p + "mix.v": (H * dv, D), p + "mix.v.conv": (H * dv, n),
                           p + "mix.b": (H, D), p + "mix.A_log": (H,), p + "mix.norm": (dv,),
                           p + "mix.a1": (RANKS[0], D), p + "mix.a2": (H * d, RANKS[0]), p + "mix.dt_bias": (H * d,),
                           p + "mix.g1": (RANKS[1], D), p + "mix.g2": (H * dv, RANKS[1]), p + "mix.o": (D, H * dv)})
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "mlp.gate": (ff, D), p + "mlp.up": (ff, D), p + "mlp.down": (D, ff)})
    return shapes


def to_bf16_bits(a):
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def make_weights(cfg, seed):
    """name -> float32 array holding bfloat16 values.  Scales are chosen so that every mechanism matters: norm
    weights far from 1, query/key norms that make the softmax pick single keys, decays of the delta layers spread
    from fast to slow, convolution taps of order 1."""
    rng = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[-1]
        fan_in = shape[-1]
        if leaf in ("norm1", "norm", "mix.norm") or name in ("embed.norm", "final.norm"):
            a = 1.0 + 0.3 * rng.randn(*shape)
        elif leaf == "mix.q.norm":
            a = 2.0 + 0.5 * rng.randn(*shape)     # peaky scores: a key that is wrongly seen or missed shows
        elif leaf == "mix.k.norm":
            a = 1.5 + 0.5 * rng.randn(*shape)
        elif leaf.endswith(".conv"):
            a = 0.6 * rng.randn(*shape)
        elif leaf == "mix.A_log":
            a = rng.uniform(-3.0, 0.5, size=shape)
        elif leaf == "mix.dt_bias":
            a = rng.uniform(-2.0, 1.0, size=shape)
        elif name == "embed":
            a = rng.randn(*shape)
        elif leaf in ("mix.o", "mlp.down"):
            a = 0.5 * rng.randn(*shape) / np.sqrt(fan_in)
        else:
            a = 1.5 * rng.randn(*shape) / np.sqrt(fan_in)
        bits = to_bf16_bits(a)
        out[name] = (bits.astype(np.uint32) << 16).view(np.float32).reshape(shape)
    return out


def write_folder(cfg, weights, folder):
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    header, blobs, at = {}, [], 0
    for name, a in weights.items():
        raw = to_bf16_bits(a).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(folder / "model.safetensors", "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)
    return str(folder)


def make_folder(name, folder, seed=0):
    cfg = CONFIGS[name]()
    weights = make_weights(cfg, seed)
    return write_folder(cfg, weights, folder), cfg, {k: v.astype(np.float64) for k, v in weights.items()}


def tokens(cfg, length, seed):
    return [int(t) for t in np.random.RandomState(seed).randint(0, cfg["vocab"], size=length)]
