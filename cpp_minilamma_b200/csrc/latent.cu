// Attention over a shared low-rank latent: what a layer caches per position is one row [c | k_r] - the
// normalised latent c (rank columns) and one rotated key part k_r (rot columns) that every head shares.  A head's
// key is [W_uk,h c | k_r] and its value W_uv,h c; because both are linear in c, the query's plain part is taken
// through W_uk,h^T once (q~_h = W_uk,h^T q_h, a batched product outside this file) and the scores become
// [q~_h | q_r,h] . [c | k_r]: attention of H query heads over ONE key/value head whose keys have rank + rot
// columns and whose values are the keys' leading rank columns.  The head's output, still in the latent's
// coordinates, goes through W_uv,h afterwards (another batched product).
//
// The kernel here prepares a step's tokens, one block per token, float32 arithmetic:
//   c   = c' / sqrt(mean(c'^2) + eps) * w          c' = the first `rank` columns of the down projection
//   k_r = the last `rot` columns of it, pairs (2i, 2i + 1) (or (i, i + rot/2)) rotated by position * f_i
//   the cache row [c | k_r] is written into the token's page;
//   q_r of every head rotated the same way and written behind the head's q~ columns of the query buffer.
#include "common.cuh"

namespace mll {

struct LatentPrepArgs {
  const void* proj;        // [T, ld]: H heads of (d plain + rot rotated) query columns, then rank + rot down-projection columns
  const float* c_weight;   // [rank]
  const float* cos_table;  // [max_pos, rot / 2]
  const float* sin_table;
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const int* block_table;
  void* q_out;             // [T, H, rank + rot]: only the last rot columns of every head are written here
  void* kv_cache;          // [pages, 1, PAGE, rank + rot]
  int ld, n_heads, d, rot, rank, interleaved, max_blocks;
  float eps;
};

template <typename T>
__device__ __forceinline__ float rotated(const T* src, int e, int rot, int interleaved, const float* cs, const float* sn) {
  const int half = rot >> 1;
  int pair, partner;
  bool first;
  if (interleaved) {
    pair = e >> 1; first = !(e & 1); partner = e ^ 1;
  } else {
    first = e < half; pair = first ? e : e - half; partner = first ? e + half : e - half;
  }
  const float x = to_float(src[e]), y = to_float(src[partner]);
  return first ? x * cs[pair] - y * sn[pair] : x * cs[pair] + y * sn[pair];
}

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(LatentPrepArgs a) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int nq = a.n_heads * (a.d + a.rot), row_w = a.rank + a.rot;
  const T* row = (const T*)a.proj + (size_t)t * a.ld;
  const T* down = row + nq;
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
    const float v = to_float(down[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float f = 1.f / sqrtf(ss / (float)a.rank + a.eps);
  const int pos = a.tok_pos[t];
  const int slot = a.seq_slot[a.tok_seq[t]];
  const int page = a.block_table[(size_t)slot * a.max_blocks + pos / MLL_PAGE];
  T* cache_row = (T*)a.kv_cache + ((size_t)page * MLL_PAGE + pos % MLL_PAGE) * row_w;
  const float* cs = a.cos_table + (size_t)pos * (a.rot >> 1);
  const float* sn = a.sin_table + (size_t)pos * (a.rot >> 1);
  for (int i = threadIdx.x; i < a.rank; i += blockDim.x)
    cache_row[i] = from_float<T>(to_float(down[i]) * f * a.c_weight[i]);
  for (int i = threadIdx.x; i < a.rot; i += blockDim.x)
    cache_row[a.rank + i] = from_float<T>(rotated(down + a.rank, i, a.rot, a.interleaved, cs, sn));
  for (int i = threadIdx.x; i < a.n_heads * a.rot; i += blockDim.x) {
    const int h = i / a.rot, e = i % a.rot;
    ((T*)a.q_out)[((size_t)t * a.n_heads + h) * row_w + a.rank + e] =
        from_float<T>(rotated(row + (size_t)h * (a.d + a.rot) + a.d, e, a.rot, a.interleaved, cs, sn));
  }
}

}  // namespace mll

MLL_API int mll_latent_prepare(const void* proj, const float* c_weight, const float* cos_table, const float* sin_table,
                               const int* tok_pos, const int* tok_seq, const int* seq_slot, const int* block_table,
                               void* q_out, void* kv_cache, int dtype, int n_tokens, int ld, int n_heads, int d, int rot,
                               int rank, int interleaved, int max_blocks, float eps, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && d > 0 && rank > 0, "latent prepare: bad sizes");
  MLL_REQUIRE(rot >= 0 && rot % 2 == 0, "latent prepare: %d rotated dimensions", rot);
  MLL_REQUIRE(ld >= n_heads * (d + rot) + rank + rot, "latent prepare: row stride %d too short", ld);
  MLL_REQUIRE(rot == 0 || (cos_table && sin_table), "latent prepare: rotated dimensions without tables");
  if (n_tokens == 0) return 0;
  mll::LatentPrepArgs a{proj, c_weight, cos_table, sin_table, tok_pos, tok_seq, seq_slot, block_table, q_out, kv_cache,
                        ld, n_heads, d, rot, rank, interleaved, max_blocks, eps};
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::latent_prepare_kernel<float>), n_tokens, 256, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::latent_prepare_kernel<__nv_bfloat16>), n_tokens, 256, 0, stream, a);
  else
    MLL_REQUIRE(false, "latent prepare: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}
