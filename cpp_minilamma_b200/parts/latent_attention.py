"""Attention whose keys and values are expanded from a shared low-rank latent.

    q_h     = W_q h per head: d plain columns, then r rotated ones
    [c'|k'] = W_dkv h: the first `rank` columns normalised to c = c' / rms(c') * w_c, the last r columns one rotated
              key part k_r that every head shares
    k_h     = [W_uk,h c | k_r],  v_h = W_uv,h c            what a head's key and value are
    score   = scale * (q_plain . W_uk,h c + q_r . k_r), causal softmax
    out     = W_o (concat_heads(sum_j p_j v_h,j) * sigmoid(W_g h))      (the gate is optional)

Only [c | k_r] is cached: one row of rank + r columns per position, whatever the number of heads.  Keys and values
are never expanded.  Both are linear in c, so the plain part of a query goes through W_uk,h^T once,
q~_h = W_uk,h^T q_plain, after which the layer is attention of H query heads over one key/value head whose key rows
are the cache rows and whose value rows are their leading `rank` columns (the kernels of the chunked attention take
exactly that: `v_in_k`); a head's result, still in the latent's coordinates, goes through W_uv,h afterwards.  The two
per-head products are batched library products over the heads.  The rotated parts turn by position * base^(-2i/r)
in pairs (2i, 2i + 1) or (i, i + r/2), from the same tables as every other rotary layer.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, CacheNeed, KVNeed, Mixer, WeightSpec, register_part
from .linear import Linear
from .rope import shared_position_encoding


class LatentAttention(Mixer):
    """params:
      n_heads, head_dim, rot_dim, v_head_dim, kv_rank   sizes (head_dim: the plain part of a query / key head)
      scale                                             factor on the scores
      position                                          PartSpec of a rotary encoding over rot_dim dimensions (None if rot_dim is 0)
      eps                                               of the latent's norm
      gate                                              True: the heads are multiplied by sigmoid(W_g h) element by element
      names                                             {"q","dkv","dkv_norm","uk","uv","o"} (and "g"): tensor names
    """

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.n_heads = int(params["n_heads"])
        self.d = int(params["head_dim"])
        self.rot = int(params.get("rot_dim") or 0)
        self.dv = int(params["v_head_dim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        self.gate = bool(params.get("gate", False))
        self.names = dict(params["names"])
        if self.rot % 2:
            raise ValueError(f"latent attention: {self.rot} rotated dimensions")
        if self.rank + self.rot > 1024:
            raise ValueError(f"latent attention: cache rows of {self.rank + self.rot} exceed the 1024 the kernels take")
        self.position = shared_position_encoding(params["position"], ctx) if self.rot else None
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.c_weight = self.w_uk = self.w_uv_t = None

    @property
    def row(self) -> int:
        return self.rank + self.rot

    def weight_specs(self) -> List[WeightSpec]:
        D, H = self.ctx.hidden_size, self.n_heads
        specs = [WeightSpec(self.names["q"], (H * (self.d + self.rot), D)),
                 WeightSpec(self.names["dkv"], (self.row, D)),
                 WeightSpec(self.names["dkv_norm"], (self.rank,), kind="vector", init="norm"),
                 WeightSpec(self.names["uk"], (H * self.d, self.rank)),
                 WeightSpec(self.names["uv"], (H * self.dv, self.rank)),
                 WeightSpec(self.names["o"], (D, H * self.dv))]
        if self.gate:
            specs.append(WeightSpec(self.names["g"], (H * self.dv, D)))
        return specs

    def bind(self, store) -> None:
        mats = [store.take(self.names[p]) for p in (("q", "dkv", "g") if self.gate else ("q", "dkv"))]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.proj = Linear(torch.cat(mats, dim=0), self.names["q"] + "+dkv" + ("+g" if self.gate else ""))
        del mats
        self.c_weight = store.take(self.names["dkv_norm"])
        act = self.ctx.act_dtype
        # per head: q~ = q_plain W_uk,h  ([d] x [d, rank]),  out = o_latent W_uv,h^T  ([rank] x [rank, dv])
        self.w_uk = store.take(self.names["uk"]).to(act).view(self.n_heads, self.d, self.rank).contiguous()
        self.w_uv_t = store.take(self.names["uv"]).to(act).view(self.n_heads, self.dv, self.rank).transpose(1, 2).contiguous()
        self.o = Linear(store.take(self.names["o"]), self.names["o"])

    def parameter_bytes(self) -> int:
        return (self.proj.parameter_bytes() + self.o.parameter_bytes()
                + (self.w_uk.numel() + self.w_uv_t.numel()) * self.w_uk.element_size())

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kv=KVNeed(1, self.row, 0, self.rank, v_in_k=True))

    def step_metadata_key(self):
        # the tile list of prompt steps on tensor cores, shared with the chunked attention's layers
        return ("chunked_attention.tiles", K.PREFILL_TILE) if self.ctx.act_dtype == torch.bfloat16 else None

    def prepare_step(self, shape):
        if shape.all_decode:
            return {}
        lists = {"tile_seq": [], "tile_row0": [], "wide_seq": [], "wide_row0": []}
        wide = []
        for i in sorted(range(shape.n_seqs), key=lambda i: -shape.lens[i]):
            for row0 in range(0, shape.lens[i], K.PREFILL_TILE):
                lists["tile_seq"].append(i)
                lists["tile_row0"].append(row0)
            for row0 in range(0, shape.lens[i], 2 * K.PREFILL_TILE):
                wide.append((shape.starts[i] + min(shape.lens[i], row0 + 2 * K.PREFILL_TILE), i, row0))
        wide.sort()
        lists["wide_seq"] = [i for _, i, _ in wide]
        lists["wide_row0"] = [row0 for _, _, row0 in wide]
        return lists

    def forward(self, step, h, cache):
        T, H = h.shape[0], self.n_heads
        act = self.ctx.act_dtype
        if cache.k is None:
            raise RuntimeError("latent attention: the cache view has no storage")
        if act == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
            raise RuntimeError("latent attention: TF32 is enabled; the float32 path needs true 32-bit products")
        proj = self.proj.forward(step, h, "latent.proj")
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        q = step.ws.buffer("latent.q", (T, H * self.row), act)
        K.latent_prepare(proj, self.c_weight, cos, sin, step.tok_pos, step.tok_seq, step.seq_slot, cache.block_table,
                         q, cache.k, H, self.d, self.rot, self.rank,
                         bool(self.position.interleaved) if self.position is not None else False, self.eps)
        # q~_h = q_plain,h W_uk,h into the first `rank` columns of every head's query row (a strided batched product)
        q_plain = proj[:, :H * (self.d + self.rot)].view(T, H, self.d + self.rot)[:, :, :self.d].transpose(0, 1)
        torch.bmm(q_plain, self.w_uk, out=q.view(T, H, self.row)[:, :, :self.rank].transpose(0, 1))
        latent = step.ws.buffer("latent.o", (T, H * self.rank), act)
        tiles = step.meta.get(self.step_metadata_key()) if not step.all_decode else None
        if step.all_decode and K.local_attention_mma_supported(act, self.row, self.rank):
            # single tokens: all heads read the one latent row per position, so they are the rows of one tile
            splits = K.local_attention_heads_splits(T, -(-H // 64), self.ctx.multiprocessors)
            scratch = step.ws.buffer("latent.parts", (K.local_attention_heads_scratch(T, H, self.rank, splits),),
                                     torch.float32) if splits > 1 else None
            K.local_attention_heads(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen,
                                    cache.block_table, latent, T, H, 1, self.row, self.rank, 0, 0, self.scale, v_in_k=True,
                                    n_splits=splits, scratch=scratch)
        elif tiles and K.local_attention_mma_supported(act, self.row, self.rank):
            K.local_attention_tiles(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen,
                                    tiles["tile_seq"], tiles["tile_row0"], cache.block_table, latent, H, 1, self.row,
                                    self.rank, 0, 0, self.scale, v_in_k=True)
        else:
            K.local_attention(q, cache.k, cache.v, step.tok_pos, step.tok_seq, step.seq_slot, cache.block_table, latent,
                              H, 1, self.row, self.rank, 0, 0, self.scale, v_in_k=True)
        # out_h = o_latent,h W_uv,h^T, written token-major
        out = step.ws.buffer("attn", (T, H * self.dv), act)
        torch.bmm(latent.view(T, H, self.rank).transpose(0, 1), self.w_uv_t, out=out.view(T, H, self.dv).transpose(0, 1))
        if self.gate:
            K.heads_gate(out, proj, H * (self.d + self.rot) + self.row, out, H, self.dv, per_head=False)
        return self.o.forward(step, out, "o")


register_part("mixer", "latent_attention", LatentAttention)
