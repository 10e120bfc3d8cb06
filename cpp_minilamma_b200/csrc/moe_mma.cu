// The two products of the routed feed-forward (moe.cu) on tensor cores, bfloat16: tiles of 64 rows of one expert
// times 128 weight rows, mma.sync m16n8k16 with float32 accumulation, operands through a four-stage cp.async
// ring (64 columns of k a stage, 108 KB of shared memory: two blocks a multiprocessor keep about 80 KB of weights
// in flight, which a decode step - every touched expert's weights streamed once - needs to fill the memory pipe).
// Four warps as 2 x 2: a warp owns 32 of the tile's rows.
//   gate_up  the 128 weight rows are 64 gate rows and the 64 up rows of the same activation columns; a warp's
//            eight 8-column tiles are four of gate and the same four of up, so silu(gate) * up happens in the
//            accumulator registers; rows are gathered from the step's tokens by (token, choice) pair.
//   down     the 128 weight rows are output columns; a row's result is multiplied by its pair's routing weight
//            and written as float32 to the pair's row (summed over a token's choices by the combine kernel).
// Rows past a tile's end and columns past the matrices' edges are zero-filled in shared memory.
#include "attention_decode.cuh"
#include "common.cuh"
#include "moe.cuh"

namespace mll {

constexpr int MMA_BK = 64, MMA_STAGES = 4, MMA_LD = MMA_BK + 8;  // 144-byte rows: ldmatrix without bank conflicts
constexpr size_t MMA_SMEM = (size_t)MMA_STAGES * (MOE_MMA_BM + 128) * MMA_LD * sizeof(__nv_bfloat16);

template <bool GATE_UP>
__global__ void __launch_bounds__(128) moe_mma_kernel(MoeProductArgs a) {
  const int tile = blockIdx.x;
  if (tile >= a.plan.n_tiles[0]) return;
  extern __shared__ __align__(16) unsigned char moe_smem[];
  typedef __nv_bfloat16 (*ATile)[MOE_MMA_BM][MMA_LD];
  typedef __nv_bfloat16 (*BTile)[128][MMA_LD];
  ATile a_s = reinterpret_cast<ATile>(moe_smem);
  BTile b_s = reinterpret_cast<BTile>(moe_smem + (size_t)MMA_STAGES * MOE_MMA_BM * MMA_LD * sizeof(__nv_bfloat16));
  __shared__ int row_src[MOE_MMA_BM];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;
  const int g = lane >> 2, t = lane & 3;
  const int e = a.plan.tile_expert[tile], row0 = a.plan.tile_row0[tile];
  const int rows = min(MOE_MMA_BM, a.plan.offsets[e + 1] - row0);
  const int K = a.k, N = a.n;
  const int n0 = blockIdx.y * (GATE_UP ? 64 : 128);  // first activation column (gate_up) or output column (down)
  if (tid < MOE_MMA_BM) row_src[tid] = tid < rows ? (GATE_UP ? a.plan.order[row0 + tid] / a.top : row0 + tid) : -1;
  __syncthreads();
  const __nv_bfloat16* act = (const __nv_bfloat16*)a.a;
  const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)e * (GATE_UP ? 2 * N : N) * K;

  auto load = [&](int kt, int stage) {
    const int k0 = kt * MMA_BK;
    for (int c = tid; c < MOE_MMA_BM * (MMA_BK / 8); c += 128) {
      const int r = c / (MMA_BK / 8), cc = c % (MMA_BK / 8);
      const int src = row_src[r];
      const bool in = src >= 0 && k0 + cc * 8 < K;
      cp_async16_zfill(&a_s[stage][r][cc * 8], act + (in ? (size_t)src * K + k0 + cc * 8 : 0), in);
    }
    for (int c = tid; c < 128 * (MMA_BK / 8); c += 128) {
      const int r = c / (MMA_BK / 8), cc = c % (MMA_BK / 8);
      // gate_up: rows 0..63 are gate rows n0 + r, rows 64..127 the up rows of the same columns
      const int col = GATE_UP ? n0 + (r & 63) : n0 + r;
      const size_t wrow = GATE_UP ? (size_t)(r >> 6) * N + col : (size_t)col;
      const bool in = col < N && k0 + cc * 8 < K;
      cp_async16_zfill(&b_s[stage][r][cc * 8], w + (in ? wrow * K + k0 + cc * 8 : 0), in);
    }
  };

  float acc[2][8][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;

  const int nk = (K + MMA_BK - 1) / MMA_BK;
#pragma unroll
  for (int s = 0; s < MMA_STAGES - 1; ++s) {
    if (s < nk) load(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<MMA_STAGES - 2>();
    __syncthreads();
    if (kt + MMA_STAGES - 1 < nk) load(kt + MMA_STAGES - 1, (kt + MMA_STAGES - 1) % MMA_STAGES);
    cp_async_commit();
    const int stage = kt % MMA_STAGES;
#pragma unroll
    for (int ks = 0; ks < MMA_BK / 16; ++ks) {
      unsigned af[2][4];
#pragma unroll
      for (int m = 0; m < 2; ++m)
        ldmatrix_x4(af[m], &a_s[stage][wm * 32 + m * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)][ks * 16 + ((lane >> 4) << 3)]);
#pragma unroll
      for (int n = 0; n < 8; n += 2) {
        // the warp's n-th 8-column tile: gate_up 0..3 gate, 4..7 up, both at columns wn * 32 + (n & 3) * 8
        const int brow = GATE_UP ? (n >> 2) * 64 + wn * 32 + (n & 3) * 8 : wn * 64 + n * 8;
        unsigned bf[4];
        ldmatrix_x4(bf, &b_s[stage][brow + (lane & 7) + ((lane >> 4) << 3)][ks * 16 + (((lane >> 3) & 1) << 3)]);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          mma_16816(acc[m][n], af[m], bf[0], bf[1]);
          mma_16816(acc[m][n + 1], af[m], bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + m * 16 + g + 8 * half;
      if (r >= rows) continue;
      const int place = row0 + r;
      if (GATE_UP) {
        __nv_bfloat16* dst = (__nv_bfloat16*)a.out + (size_t)place * N;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int col = n0 + wn * 32 + n * 8 + 2 * t;
          if (col >= N) continue;  // N is even: a pair is inside or outside as a whole
          const float g0 = acc[m][n][2 * half], g1 = acc[m][n][2 * half + 1];
          const float u0 = acc[m][n + 4][2 * half], u1 = acc[m][n + 4][2 * half + 1];
          *reinterpret_cast<__nv_bfloat162*>(dst + col) =
              __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
        }
      } else {
        const int pair = a.plan.order[place];
        const float pw = a.pair_weight[pair];
        float* dst = (float*)a.out + (size_t)pair * N;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int col = n0 + wn * 64 + n * 8 + 2 * t;
          if (col >= N) continue;
          *reinterpret_cast<float2*>(dst + col) = make_float2(pw * acc[m][n][2 * half], pw * acc[m][n][2 * half + 1]);
        }
      }
    }
}

template <bool GATE_UP>
int moe_mma_reserve() {
  cudaError_t err = cudaFuncSetAttribute(moe_mma_kernel<GATE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MMA_SMEM);
  if (err != cudaSuccess) {
    mll_set_error("moe (mma): cannot reserve %zu bytes of shared memory: %s", MMA_SMEM, cudaGetErrorString(err));
    return -1;
  }
  return 0;
}

}  // namespace mll

MLL_API int mll_moe_mma_rows() { return MOE_MMA_BM; }

// bfloat16 only; rows of 16-byte words on both sides of both products.
MLL_API int mll_moe_mma_supported(int width, int inter) { return width > 0 && inter > 0 && width % 8 == 0 && inter % 8 == 0; }

MLL_API int mll_moe_gate_up_mma(const void* h, const void* w, void* act, const int* order, const int* offsets,
                                const int* tile_expert, const int* tile_row0, const int* n_tiles, int max_tiles,
                                int width, int inter, int top, cudaStream_t stream) {
  MLL_REQUIRE(mll_moe_mma_supported(width, inter) && max_tiles > 0 && top > 0, "moe gate_up (mma): sizes %d / %d", width, inter);
  MLL_REQUIRE((inter + 63) / 64 <= 65535, "moe gate_up (mma): %d columns are too many for one launch", inter);
  mll::MoeProductArgs a{h, w, act, nullptr, mll::MoePlan{(int*)order, (int*)offsets, (int*)tile_expert, (int*)tile_row0,
                                                         (int*)n_tiles}, width, inter, top};
  if (mll::moe_mma_reserve<true>() != 0) return -1;
  MLL_LAUNCH((mll::moe_mma_kernel<true>), dim3(max_tiles, (inter + 63) / 64), 128, mll::MMA_SMEM, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_moe_down_mma(const void* act, const void* w, float* y, const float* pair_weight, const int* order,
                             const int* offsets, const int* tile_expert, const int* tile_row0, const int* n_tiles,
                             int max_tiles, int inter, int width, int top, cudaStream_t stream) {
  MLL_REQUIRE(mll_moe_mma_supported(width, inter) && max_tiles > 0 && top > 0, "moe down (mma): sizes %d / %d", width, inter);
  MLL_REQUIRE((width + 127) / 128 <= 65535, "moe down (mma): %d columns are too many for one launch", width);
  mll::MoeProductArgs a{act, w, y, pair_weight, mll::MoePlan{(int*)order, (int*)offsets, (int*)tile_expert,
                                                             (int*)tile_row0, (int*)n_tiles}, inter, width, top};
  if (mll::moe_mma_reserve<false>() != 0) return -1;
  MLL_LAUNCH((mll::moe_mma_kernel<false>), dim3(max_tiles, (width + 127) / 128), 128, mll::MMA_SMEM, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}
