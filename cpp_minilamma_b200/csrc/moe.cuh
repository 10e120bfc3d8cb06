// What the kernels of the routed feed-forward share (moe.cu, moe_mma.cu).
#pragma once

#define MOE_SIMT_BM 16  // rows of a tile in the plain products

namespace mll {

// The (token, choice) pairs of a step sorted by expert, on the device.
struct MoePlan {
  int* order;        // [pairs] place -> pair (= token * top + choice)
  int* offsets;      // [experts + 1] first place of every expert
  int* tile_expert;  // [max tiles] tiles of up to BM consecutive places of one expert
  int* tile_row0;    // [max tiles] a tile's first place
  int* n_tiles;      // [1] how many tiles the step really has
};

struct MoeProductArgs {
  const void* a;             // activations: [tokens, k] gathered by pair (gate_up) or [pairs, k] by place (down)
  const void* w;             // [experts, n or 2 n, k]
  void* out;
  const float* pair_weight;  // [pairs] (down)
  MoePlan plan;
  int k, n, top;
};

}  // namespace mll
