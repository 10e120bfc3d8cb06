"""Small Malulorn configurations and weights for the tests, made here from NumPy random numbers and written with
this file's own safetensors writer (bfloat16 storage), so that nothing of the product takes part in what the
oracle reads.  Sizes are unlike each other on purpose: head counts and groups, key and value head sizes that
differ, latent ranks and rotated parts, temperature periods of a few tokens (so that its steps fall inside short
prompts), expert counts that are no powers of two, one expert per token and all experts per token, layers with
and without a feed-forward or a shared expert, loops that start at the first layer or later and run once, twice
or three times, and models without a loop."""
import json
import struct

import numpy as np


def moe(experts=5, top=2, ff=24, shared=16):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared} if shared else None}


def attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.35, temp=(0.5, 8), mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if temp:
        mixer["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.3, base=100.0, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}},
            "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, loop=None):
    out = {"architecture": "Malulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CONFIGS = {
    # one mechanism each, nothing else that could cover for a fault (no feed-forward, no loop)
    "sink_only": lambda: config([attention()], width=40),
    "latent_only": lambda: config([latent()], width=40),
    # the routed feed-forward behind a small mixer, and the re-entry around one layer run three times
    "routed": lambda: config([attention(heads=2, kv_heads=1, dim=8, vdim=8, temp=None, mlp=moe(experts=6, top=3, ff=20))],
                             width=32, vocab=71),
    "reentry": lambda: config([latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16)], width=32, vocab=71, loop=(0, 1, 3)),
    # everything; the loop starts at the second layer; sizes that are no powers of two
    "mixed": lambda: config([latent(heads=2, dim=24, rot_dim=8, vdim=16, kv_rank=48, mlp=moe(7, 3, 24, 40)),
                             attention(heads=6, kv_heads=3, dim=8, vdim=16, temp=(0.3, 5), mlp=moe(7, 2, 16, 0)),
                             attention(heads=3, kv_heads=3, dim=24, vdim=8, temp=(0.7, 64), mlp=None),
                             latent(heads=4, dim=8, rot_dim=16, vdim=24, kv_rank=24, base=10000.0, mlp=moe(3, 1, 32, 8))],
                            width=56, vocab=131, eps=1e-6, loop=(1, 3, 2)),
    # heads of one, one expert per token, every expert per token, a single expert, a loop of one pass, a dense layer
    "ones": lambda: config([attention(heads=1, kv_heads=1, dim=32, vdim=16, temp=(0.5, 1), mlp=moe(4, 1, 16, 8)),
                            latent(heads=1, dim=40, rot_dim=2, vdim=40, kv_rank=8, mlp=moe(3, 3, 8, 0)),
                            attention(heads=2, kv_heads=1, dim=8, vdim=8, temp=None, mlp=moe(1, 1, 24, 24)),
                            latent(heads=2, dim=8, rot_dim=8, vdim=4, kv_rank=72, mlp={"kind": "dense", "ff": 24})],
                           width=36, vocab=61, loop=(2, 4, 1)),
    # sizes at which the wider kernel instances run: cache rows beyond 256, keys above 64, values above 128
    "wide": lambda: config([latent(heads=2, dim=72, rot_dim=32, vdim=136, kv_rank=264, mlp=None),
                            attention(heads=2, kv_heads=1, dim=72, vdim=136, temp=(0.2, 16), mlp=moe(9, 2, 72, 0)),
                            latent(heads=4, dim=32, rot_dim=64, vdim=32, kv_rank=136, mlp=None)],
                           width=64, vocab=50),
    # head sizes of 64 and 128 for keys and values alike: in bfloat16 the sink layers run on the tcgen05 prompt kernel
    # and the TMA-fed decode kernel, at 32 on the mma.sync decode kernel; a latent row of exactly 256
    "tensor": lambda: config([attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.2, temp=(0.3, 32), mlp=moe(4, 2, 32, 16)),
                              attention(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.15, temp=None, mlp=None),
                              latent(heads=4, dim=32, rot_dim=64, vdim=32, kv_rank=192, scale=0.1, mlp=moe(8, 2, 64, 0)),
                              attention(heads=4, kv_heads=4, dim=32, vdim=32, scale=0.3, temp=(0.5, 100), mlp=None)],
                             width=128, vocab=89, loop=(0, 2, 2)),
    # nothing divisible by four: a width of 50, heads of 6 and 10, the kernels' scalar paths
    "odd": lambda: config([attention(heads=3, kv_heads=1, dim=6, vdim=10, temp=(0.4, 7), mlp=moe(5, 2, 30, 14)),
                           latent(heads=3, dim=6, rot_dim=2, vdim=10, kv_rank=10, mlp=moe(5, 4, 6, 0))],
                          width=50, vocab=53, loop=(0, 2, 2)),
}


def tensor_shapes(cfg):
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "final.norm": (D,), "final.norm.b": (D,), "head": (cfg["vocab"], D)}
    loop = cfg.get("loop")
    if loop and loop["stop"] > loop["start"]:
        shapes["loop.in"] = (D, 2 * D)
        shapes["loop.step"] = (loop["times"], D)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        shapes.update({p + "norm1": (D,), p + "norm1.b": (D,)})
        if layer["type"] == "attention":
            G = m["kv_heads"]
            shapes.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.v": (G * dv, D),
                           p + "mix.g": (H, D), p + "mix.o": (D, H * dv)})
        else:
            r, rank = m["rot_dim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * (d + r), D), p + "mix.dkv": (rank + r, D), p + "mix.dkv.norm": (rank,),
                           p + "mix.uk": (H * d, rank), p + "mix.uv": (H * dv, rank), p + "mix.g": (H * dv, D),
                           p + "mix.o": (D, H * dv)})
        mlp = layer["mlp"]
        if mlp is None:
            continue  # and no second norm either: nothing would read it
        shapes.update({p + "norm2": (D,), p + "norm2.b": (D,)})
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], D), p + "mlp.up": (mlp["ff"], D), p + "mlp.down": (D, mlp["ff"])})
            continue
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        shapes.update({p + "mlp.router": (E, D), p + "mlp.router.b": (E,)})
        for e in range(E):
            shapes.update({f"{p}mlp.e{e}.gate": (ff, D), f"{p}mlp.e{e}.up": (ff, D), f"{p}mlp.e{e}.down": (D, ff)})
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            shapes.update({p + "mlp.shared.gate": (sf, D), p + "mlp.shared.up": (sf, D), p + "mlp.shared.down": (D, sf)})
    return shapes


def to_bf16_bits(a):
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def make_weights(cfg, seed):
    """name -> float32 array holding bfloat16 values.  Scales are chosen so that every mechanism matters: norm
    weights far from 1 and biases far from 0, queries large enough that single keys win and the sink's share
    moves between almost nothing and almost everything, router logits a few units apart, re-entry vectors of the
    stream's own size, gates that are neither open nor shut."""
    rng = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[-1]
        fan_in = shape[-1]
        if leaf in ("norm1", "norm2", "mix.dkv.norm") or name == "final.norm":
            a = 1.0 + 0.3 * rng.randn(*shape)
        elif name.endswith(".b") and leaf != "mlp.router.b":
            a = 0.3 * rng.randn(*shape)
        elif leaf == "mlp.router.b":
            a = 0.7 * rng.randn(*shape)
        elif leaf == "mlp.router":
            a = 2.0 * rng.randn(*shape) / np.sqrt(fan_in)
        elif leaf == "mix.q":
            a = 2.0 * rng.randn(*shape) / np.sqrt(fan_in)
        elif name in ("embed", "loop.step"):
            a = rng.randn(*shape)
        elif name == "loop.in":
            a = 1.2 * rng.randn(*shape) / np.sqrt(fan_in / 2)
        elif leaf in ("mix.o",) or leaf.endswith(".down"):
            a = 0.7 * rng.randn(*shape) / np.sqrt(fan_in)
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
