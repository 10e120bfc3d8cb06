// Attention whose keys and values have head sizes of their own (d for queries and keys, dv for
// values), with an explicit score scale, an optional norm of the whole q and k projections, rotary
// encoding of the first `rot` dimensions of a head only, and a mask that is causal inside chunks:
// query i sees key j iff j <= i and j / chunk == i / chunk (chunk 0: every earlier key), and with a
// window w > 0 only keys j > i - w.  Chunks count from position 0 of the sequence, whatever portion of it
// a step brings.
//
// Two kernels, for prompts and single tokens alike:
//   * prepare: one block per token.  q and k are each divided by the root mean square of their whole
//     projection (all heads at once) and multiplied by a weight, the pairs of the first `rot`
//     dimensions of every head are rotated by position * frequency (cos / sin from a table), q goes to
//     a buffer and k, v into the pages of the cache.  All arithmetic in float32.
//   * attend: one warp per (token, query head).  Lanes take one key each for the scores (float32 dot
//     products over the head), the softmax runs online in float32, and for the values every lane owns
//     output columns lane, lane + 32, ...  Any d and dv (16-byte loads where rows allow them).
#include "common.cuh"

namespace mll {

struct LocalPrepArgs {
  const void* qkv;        // [T, ld]: q (Hq * d), k (Hk * d), v (Hk * dv)
  const float* q_weight;  // [Hq * d] or null: no norm of the projections
  const float* k_weight;  // [Hk * d]
  const float* cos_table; // [max_pos, rot / 2] or null
  const float* sin_table;
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const int* block_table;
  void* q_out;            // [T, Hq * d]
  void* k_cache;          // [pages, Hk, PAGE, d]
  void* v_cache;          // [pages, Hk, PAGE, dv]
  int ld, n_heads, n_kv_heads, d, dv, rot, interleaved, max_blocks;
  float eps;
};

template <typename T>
__global__ void __launch_bounds__(256) local_prepare_kernel(LocalPrepArgs a) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int d = a.d, nq = a.n_heads * d, nk = a.n_kv_heads * d, nv = a.n_kv_heads * a.dv;
  const T* row = (const T*)a.qkv + (size_t)t * a.ld;
  float fq = 1.f, fk = 1.f;
  if (a.q_weight) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
      const float v = to_float(row[i]);
      sq += v * v;
    }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
      const float v = to_float(row[nq + i]);
      sk += v * v;
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    fq = 1.f / sqrtf(sq / (float)nq + a.eps);
    fk = 1.f / sqrtf(sk / (float)nk + a.eps);
  }
  const int pos = a.tok_pos[t];
  const int slot = a.seq_slot[a.tok_seq[t]];
  const int page = a.block_table[(size_t)slot * a.max_blocks + pos / MLL_PAGE];
  const int in_page = pos % MLL_PAGE;
  const int half = a.rot >> 1;
  const float* cs = a.cos_table ? a.cos_table + (size_t)pos * half : nullptr;
  const float* sn = a.cos_table ? a.sin_table + (size_t)pos * half : nullptr;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const bool is_q = i < nq;
    const int c = is_q ? i : i - nq;  // column within the q or k projection
    const int head = c / d, e = c % d;
    const float* w = is_q ? a.q_weight : a.k_weight;
    const float f = is_q ? fq : fk;
    const T* src = row + (is_q ? 0 : nq) + head * d;
    float x = to_float(src[e]) * f;
    if (w) x *= w[c];
    if (cs && e < a.rot) {
      int pair, partner;
      bool first;
      if (a.interleaved) {
        pair = e >> 1; first = !(e & 1); partner = e ^ 1;
      } else {
        first = e < half; pair = first ? e : e - half; partner = first ? e + half : e - half;
      }
      float y = to_float(src[partner]) * f;
      if (w) y *= w[head * d + partner];
      const float co = cs[pair], si = sn[pair];
      x = first ? x * co - y * si : x * co + y * si;
    }
    if (is_q)
      ((T*)a.q_out)[(size_t)t * nq + c] = from_float<T>(x);
    else
      ((T*)a.k_cache)[(((size_t)page * a.n_kv_heads + head) * MLL_PAGE + in_page) * d + e] = from_float<T>(x);
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int head = i / a.dv, e = i % a.dv;
    ((T*)a.v_cache)[(((size_t)page * a.n_kv_heads + head) * MLL_PAGE + in_page) * a.dv + e] = row[nq + nk + i];
  }
}

struct LocalAttnArgs {
  const void* q;         // [T, Hq * d]
  const void* k_cache;
  const void* v_cache;
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const int* block_table;
  void* out;             // [T, Hq * dv]
  int n_tokens, n_heads, n_kv_heads, d, dv, chunk, window, max_blocks;
  float scale;
};

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ k, const float* __restrict__ q, int d, bool vec);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ k, const float* __restrict__ q, int d,
                                                bool vec) {
  float s = 0.f;
  if (vec) {
    for (int e = 0; e < d; e += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(k + e);
      const float4 qv = *reinterpret_cast<const float4*>(q + e);
      s = fmaf(kv.x, qv.x, s); s = fmaf(kv.y, qv.y, s); s = fmaf(kv.z, qv.z, s); s = fmaf(kv.w, qv.w, s);
    }
  } else {
    for (int e = 0; e < d; ++e) s = fmaf(k[e], q[e], s);
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ k,
                                                        const float* __restrict__ q, int d, bool vec) {
  float s = 0.f;
  if (vec) {
    for (int e = 0; e < d; e += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + e);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        s = fmaf(f.x, q[e + 2 * i], s);
        s = fmaf(f.y, q[e + 2 * i + 1], s);
      }
    }
  } else {
    for (int e = 0; e < d; ++e) s = fmaf(__bfloat162float(k[e]), q[e], s);
  }
  return s;
}

constexpr int LOCAL_WARPS = 4;

// grid (ceil(T / LOCAL_WARPS), Hq); dynamic shared memory LOCAL_WARPS * d_padded floats.
template <typename T, int NACC>
__global__ void __launch_bounds__(32 * LOCAL_WARPS) local_attention_kernel(LocalAttnArgs a) {
  extern __shared__ __align__(16) float q_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * LOCAL_WARPS + warp;
  if (t >= a.n_tokens) return;  // whole warps leave; nothing below synchronises the block
  const int h = blockIdx.y;
  const int kvh = h / (a.n_heads / a.n_kv_heads);
  const int d = a.d, dv = a.dv;
  const int d_pad = (d + 3) & ~3;
  float* qs = q_smem + warp * d_pad;
  const T* qrow = (const T*)a.q + ((size_t)t * a.n_heads + h) * d;
  for (int e = lane; e < d; e += 32) qs[e] = to_float(qrow[e]) * a.scale;
  __syncwarp();
  const int pos = a.tok_pos[t];
  int first = a.chunk > 0 ? (pos / a.chunk) * a.chunk : 0;
  if (a.window > 0) first = max(first, pos - a.window + 1);
  const int* table = a.block_table + (size_t)a.seq_slot[a.tok_seq[t]] * a.max_blocks;
  const bool kvec = (d * sizeof(T)) % 16 == 0;

  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  for (int j0 = first; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= pos;
    int page = 0;
    float s = -INFINITY;
    if (valid) {
      page = table[j / MLL_PAGE];
      const T* krow = (const T*)a.k_cache + (((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE + j % MLL_PAGE) * d;
      s = dot_row<T>(krow, qs, d, kvec);
    }
    const float m_new = fmaxf(m_run, warp_max(s));  // lane 0 of the step is always valid: finite
    const float alpha = expf(m_run - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l_run = l_run * alpha + warp_sum(p);
    m_run = m_new;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
    const int count = min(32, pos - j0 + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int pg = __shfl_sync(0xffffffffu, page, jj);
      const T* vrow = (const T*)a.v_cache + (((size_t)pg * a.n_kv_heads + kvh) * MLL_PAGE + (j0 + jj) % MLL_PAGE) * dv;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) acc[i] = fmaf(pj, to_float(vrow[c]), acc[i]);
      }
    }
  }
  const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
  T* orow = (T*)a.out + ((size_t)t * a.n_heads + h) * dv;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) orow[c] = from_float<T>(acc[i] * inv);
  }
}

template <typename T>
int launch_local_attention(const LocalAttnArgs& a, cudaStream_t stream) {
  const dim3 grid((a.n_tokens + LOCAL_WARPS - 1) / LOCAL_WARPS, a.n_heads);
  const size_t smem = (size_t)LOCAL_WARPS * ((a.d + 3) & ~3) * sizeof(float);
  const int nacc = (a.dv + 31) / 32;
  if (nacc <= 1)
    MLL_LAUNCH((local_attention_kernel<T, 1>), grid, 32 * LOCAL_WARPS, smem, stream, a);
  else if (nacc <= 2)
    MLL_LAUNCH((local_attention_kernel<T, 2>), grid, 32 * LOCAL_WARPS, smem, stream, a);
  else if (nacc <= 4)
    MLL_LAUNCH((local_attention_kernel<T, 4>), grid, 32 * LOCAL_WARPS, smem, stream, a);
  else
    MLL_LAUNCH((local_attention_kernel<T, 8>), grid, 32 * LOCAL_WARPS, smem, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

}  // namespace mll

MLL_API int mll_local_attention_prepare(const void* qkv, const float* q_weight, const float* k_weight,
                                        const float* cos_table, const float* sin_table, const int* tok_pos,
                                        const int* tok_seq, const int* seq_slot, const int* block_table, void* q_out,
                                        void* k_cache, void* v_cache, int dtype, int n_tokens, int ld, int n_heads,
                                        int n_kv_heads, int d, int dv, int rot, int interleaved, int max_blocks,
                                        float eps, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && d > 0 && dv > 0, "local attention prepare: bad sizes");
  MLL_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "local attention prepare: %d rotated dimensions of %d", rot, d);
  MLL_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "local attention prepare: one norm weight without the other");
  MLL_REQUIRE(ld >= n_heads * d + n_kv_heads * (d + dv), "local attention prepare: row stride %d too short", ld);
  if (n_tokens == 0) return 0;
  mll::LocalPrepArgs a{qkv, q_weight, k_weight, rot > 0 ? cos_table : nullptr, sin_table, tok_pos, tok_seq, seq_slot,
                       block_table, q_out, k_cache, v_cache, ld, n_heads, n_kv_heads, d, dv, rot, interleaved,
                       max_blocks, eps};
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::local_prepare_kernel<float>), n_tokens, 256, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::local_prepare_kernel<__nv_bfloat16>), n_tokens, 256, 0, stream, a);
  else
    MLL_REQUIRE(false, "local attention prepare: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_local_attention(const void* q, const void* k_cache, const void* v_cache, const int* tok_pos,
                                const int* tok_seq, const int* seq_slot, const int* block_table, void* out, int dtype,
                                int n_tokens, int n_heads, int n_kv_heads, int d, int dv, int chunk, int window,
                                int max_blocks, float scale, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "local attention: bad head counts");
  MLL_REQUIRE(d > 0 && d <= 1024 && dv > 0 && dv <= 256, "local attention: head sizes %d / %d (at most 1024 / 256)", d, dv);
  MLL_REQUIRE(chunk >= 0 && window >= 0, "local attention: negative chunk or window");
  MLL_REQUIRE(n_heads <= 65535, "local attention: too many heads for one launch");
  if (n_tokens == 0) return 0;
  mll::LocalAttnArgs a{q, k_cache, v_cache, tok_pos, tok_seq, seq_slot, block_table, out, n_tokens, n_heads,
                       n_kv_heads, d, dv, chunk, window, max_blocks, scale};
  if (dtype == MLL_F32) return mll::launch_local_attention<float>(a, stream);
  if (dtype == MLL_BF16) return mll::launch_local_attention<__nv_bfloat16>(a, stream);
  MLL_REQUIRE(false, "local attention: unknown dtype %d", dtype);
  return -1;
}
