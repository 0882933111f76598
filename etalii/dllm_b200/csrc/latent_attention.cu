// Attention over a latent cache: a position keeps one row [ c (rank) | r (rot) ] for ALL heads, c a normed latent from
// which every head's keys and values are linear maps, r a rotated key part the heads share. With per head
// k_h = [W_uk,h c | r] and v_h = W_uv,h c the score q_h . k_h = (W_uk,h^T q_h,plain) . c + q_h,rot . r, so a query is
// first taken into the latent's coordinates ("absorbed") and attention then runs over the cached rows themselves:
// every head reads the same rows, its weighted sum of c is mapped to the head's values afterwards.
//
//   latent_prepare:  per token, from the down projections' float32 rows: the query latent normed (with its weight) for
//                    the up projection, the key latent normed and r rotated into the token's place in the cache.
//   latent_queries:  per (token, head): [ W_uk,h^T q_plain | rotate(q_rot) ] * scale, float32.
//   latent_attention: causal softmax attention of every (token, head) over its sequence's rows; the general kernel, a
//                    warp per pair, float32 arithmetic whatever the cache's type. With `sinks` the softmax's
//                    denominator also holds exp(sinks[head]): a learned score per head that has no key and no value.
//   latent_values:   per (token, head): W_uv,h (weighted sum of c) * sigmoid(gate), in the activation type.
//
// Cache layout (keys only): [page][row][rank + rot] in the cache's type; page_table[slot * max_pages + i] is the page
// of positions i * page_size ...
#include "common.cuh"

namespace {

struct LatentCache {
  void* base;
  const int* page_table;
  int max_pages, page_size, width;  // width = rank + rot
};

template <typename T>
__device__ __forceinline__ T* cache_row(const LatentCache& c, int slot, int pos) {
  int page = c.page_table[(size_t)slot * c.max_pages + pos / c.page_size];
  return (T*)c.base + ((size_t)page * c.page_size + pos % c.page_size) * c.width;
}

__device__ __forceinline__ float block_total(float v, float* scratch) {
  v = warp_sum(v);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = lane < warps ? scratch[lane] : 0.f;
  return warp_sum(total);
}

__device__ __forceinline__ float sigmoid_exact(float g) {
  if (g >= 0.f) return 1.0f / (1.0f + expf(-g));
  float e = expf(g);
  return e / (1.0f + e);
}

// rows[t] = [ ... | cq (q_rank) at cq_at | ... | c (rank) r (rot) at c_at | ... ] float32.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(
    const float* __restrict__ rows, int stride, int cq_at, int q_rank, int c_at, int rank, int rot,
    const float* __restrict__ wq, const float* __restrict__ wc, float eps, const float* __restrict__ table,
    T* __restrict__ cq_out, LatentCache cache, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
    const int* __restrict__ slots, int write_cache) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = rows + (size_t)t * stride;
  if (q_rank > 0) {
    float s = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) s = fmaf(row[cq_at + i], row[cq_at + i], s);
    float inv = 1.0f / sqrtf(block_total(s, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      cq_out[(size_t)t * q_rank + i] = from_float<T>(row[cq_at + i] * inv * wq[i]);
  }
  if (!write_cache) return;
  const int pos = tok_pos[t], slot = slots[tok_seq[t]];
  T* dst = cache_row<T>(cache, slot, pos);
  float s = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) s = fmaf(row[c_at + i], row[c_at + i], s);
  float inv = 1.0f / sqrtf(block_total(s, scratch) / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(row[c_at + i] * inv * wc[i]);
  const int half = rot / 2;
  const float* r = row + c_at + rank;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float cs = table[((size_t)pos * half + i) * 2], sn = table[((size_t)pos * half + i) * 2 + 1];
    float u = r[i], v = r[i + half];
    dst[rank + i] = from_float<T>(u * cs - v * sn);
    dst[rank + half + i] = from_float<T>(v * cs + u * sn);
  }
}

// q [tokens, heads * (dim + rot)] float32, head by head [plain (dim) | rotated part (rot)]; uk [heads * dim, rank].
// out [tokens, heads, rank + rot] float32 = [ uk_h^T q_plain | rotate(q_rot) ] * scale.
template <typename W>
__global__ void __launch_bounds__(128) latent_queries_kernel(
    const float* __restrict__ q, const W* __restrict__ uk, const float* __restrict__ table, float* __restrict__ out,
    int heads, int dim, int rot, int rank, float scale, const int* __restrict__ tok_pos) {
  extern __shared__ float plain[];  // dim
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* row = q + ((size_t)t * heads + h) * (dim + rot);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) plain[i] = row[i];
  __syncthreads();
  float* dst = out + ((size_t)t * heads + h) * (rank + rot);
  const W* w = uk + (size_t)h * dim * rank;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) {
    float s = 0.f;
    for (int d = 0; d < dim; ++d) s = fmaf(to_float(w[(size_t)d * rank + j]), plain[d], s);
    dst[j] = s * scale;
  }
  const int half = rot / 2, pos = tok_pos[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float cs = table[((size_t)pos * half + i) * 2], sn = table[((size_t)pos * half + i) * 2 + 1];
    float u = row[dim + i], v = row[dim + i + half];
    dst[rank + i] = (u * cs - v * sn) * scale;
    dst[rank + half + i] = (v * cs + u * sn) * scale;
  }
}

// A warp per (token, head): tiles of 32 positions, a position a lane for the scores (the query from shared memory),
// running maximum and sum, then the weighted sum of the rows' first `rank` values with the lanes across the columns.
constexpr int ATT_WARPS = 4;
constexpr int MAX_COLS = 16;  // rank <= 32 * MAX_COLS

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32) latent_attention_kernel(
    const float* __restrict__ q, float* __restrict__ out, LatentCache cache, int heads, int rank,
    const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ slots, int tokens,
    const float* __restrict__ sinks) {
  extern __shared__ float queries[];  // ATT_WARPS x width
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long pair = (long long)blockIdx.x * ATT_WARPS + warp;
  if (pair >= (long long)tokens * heads) return;
  const int t = (int)(pair / heads), width = cache.width;
  float* mine = queries + (size_t)warp * width;
  const float* src = q + (size_t)pair * width;
  for (int i = lane; i < width; i += 32) mine[i] = src[i];
  __syncwarp();
  const int pos = tok_pos[t], slot = slots[tok_seq[t]];
  const int* pages = cache.page_table + (size_t)slot * cache.max_pages;
  float acc[MAX_COLS];
#pragma unroll
  for (int i = 0; i < MAX_COLS; ++i) acc[i] = 0.f;
  // (a sink is a score without a key or a value that counts once in the denominator: the walk starts from it)
  float top = -INFINITY, total = 0.f;
  if (sinks != nullptr) {
    top = sinks[pair % heads];
    total = 1.0f;
  }
  for (int j0 = 0; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    float score = -INFINITY;
    if (j <= pos) {
      const T* key = (const T*)cache.base + ((size_t)pages[j / cache.page_size] * cache.page_size +
                                             j % cache.page_size) * width;
      float s = 0.f;
      for (int d = 0; d < width; ++d) s = fmaf(mine[d], to_float(key[d]), s);
      score = s;
    }
    float tile_top = warp_max(score);
    float new_top = fmaxf(top, tile_top);
    float correction = expf(top - new_top);  // (exp(-inf) = 0 at the first tile)
    float p = j <= pos ? expf(score - new_top) : 0.f;
    total = total * correction + warp_sum(p);
    top = new_top;
#pragma unroll
    for (int i = 0; i < MAX_COLS; ++i) acc[i] *= correction;
    const int here = min(32, pos + 1 - j0);
    for (int jj = 0; jj < here; ++jj) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      int at = j0 + jj;
      const T* value = (const T*)cache.base + ((size_t)pages[at / cache.page_size] * cache.page_size +
                                               at % cache.page_size) * width;
#pragma unroll
      for (int i = 0; i < MAX_COLS; ++i)
        if (lane + 32 * i < rank) acc[i] = fmaf(pj, to_float(value[lane + 32 * i]), acc[i]);
    }
  }
  float inv = 1.0f / total;
  float* dst = out + (size_t)pair * rank;
#pragma unroll
  for (int i = 0; i < MAX_COLS; ++i)
    if (lane + 32 * i < rank) dst[lane + 32 * i] = acc[i] * inv;
}

// mixed [tokens, heads, rank] float32; uv [heads * vdim, rank]; gates: a float32 row per token, head h at column h.
// out [tokens, heads * vdim] = (uv_h mixed_h) * sigmoid(gate_h).
template <typename W, typename T>
__global__ void __launch_bounds__(128) latent_values_kernel(
    const float* __restrict__ mixed, const W* __restrict__ uv, const float* __restrict__ gates, int gate_stride,
    T* __restrict__ out, int heads, int rank, int vdim) {
  extern __shared__ float latent[];  // rank
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* src = mixed + ((size_t)t * heads + h) * rank;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) latent[i] = src[i];
  __syncthreads();
  float gate = gates != nullptr ? sigmoid_exact(gates[(size_t)t * gate_stride + h]) : 1.0f;
  for (int e = warp; e < vdim; e += blockDim.x >> 5) {
    const W* w = uv + ((size_t)h * vdim + e) * rank;
    float s = 0.f;
    for (int j = lane; j < rank; j += 32) s = fmaf(to_float(w[j]), latent[j], s);
    s = warp_sum(s);
    if (lane == 0) out[(size_t)t * heads * vdim + h * vdim + e] = from_float<T>(s * gate);
  }
}

}  // namespace

DLLM_EXPORT int dllm_latent_prepare(const float* rows, int stride, int cq_at, int q_rank, int c_at, int rank, int rot,
                                    const float* wq, const float* wc, float eps, const float* table, void* cq_out,
                                    void* cache_base, const int* page_table, int max_pages, int page_size,
                                    const int* tok_seq, const int* tok_pos, const int* slots, int tokens,
                                    int write_cache, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (rank <= 0 || rot < 0 || rot % 2 || q_rank < 0 || stride <= 0) return DLLM_UNSUPPORTED_SIZE;
  if (!rows || !wc || (q_rank > 0 && (!wq || !cq_out)) || (rot > 0 && !table) || !cache_base || !page_table ||
      !tok_seq || !tok_pos || !slots)
    return DLLM_BAD_ARGUMENT;
  LatentCache cache = {cache_base, page_table, max_pages, page_size, rank + rot};
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(latent_prepare_kernel<float>, dim3(tokens), dim3(128), 0, stream, rows, stride, cq_at,
                           q_rank, c_at, rank, rot, wq, wc, eps, table, (float*)cq_out, cache, tok_seq, tok_pos, slots,
                           write_cache);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(latent_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, rows, stride,
                           cq_at, q_rank, c_at, rank, rot, wq, wc, eps, table, (__nv_bfloat16*)cq_out, cache, tok_seq,
                           tok_pos, slots, write_cache);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_latent_queries(const float* q, const void* uk, const float* table, float* out, int tokens,
                                    int heads, int dim, int rot, int rank, float scale, const int* tok_pos,
                                    int weight_dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || heads > 65535 || dim <= 0 || dim > 8192 || rot < 0 || rot % 2 || rank <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  if (!q || !uk || !out || !tok_pos || (rot > 0 && !table)) return DLLM_BAD_ARGUMENT;
  dim3 grid(tokens, heads);
  size_t bytes = (size_t)dim * sizeof(float);
  if (weight_dtype == DLLM_F32)
    return dllm_launch_pdl(latent_queries_kernel<float>, grid, dim3(128), bytes, stream, q, (const float*)uk, table,
                           out, heads, dim, rot, rank, scale, tok_pos);
  if (weight_dtype == DLLM_BF16)
    return dllm_launch_pdl(latent_queries_kernel<__nv_bfloat16>, grid, dim3(128), bytes, stream, q,
                           (const __nv_bfloat16*)uk, table, out, heads, dim, rot, rank, scale, tok_pos);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_latent_attention(const float* q, float* out, void* cache_base, const int* page_table,
                                      int max_pages, int page_size, int heads, int rank, int rot,
                                      const int* tok_seq, const int* tok_pos, const int* slots, int tokens,
                                      int cache_dtype, const float* sinks, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || rank <= 0 || rank > 32 * MAX_COLS || rot < 0 || (size_t)(rank + rot) * ATT_WARPS * 4 > 48 * 1024)
    return DLLM_UNSUPPORTED_SIZE;
  if (!q || !out || !cache_base || !page_table || !tok_seq || !tok_pos || !slots) return DLLM_BAD_ARGUMENT;
  LatentCache cache = {cache_base, page_table, max_pages, page_size, rank + rot};
  long long pairs = (long long)tokens * heads;
  dim3 grid((unsigned)((pairs + ATT_WARPS - 1) / ATT_WARPS));
  size_t bytes = (size_t)ATT_WARPS * (rank + rot) * sizeof(float);
  if (cache_dtype == DLLM_F32)
    return dllm_launch_pdl(latent_attention_kernel<float>, grid, dim3(ATT_WARPS * 32), bytes, stream, q, out, cache,
                           heads, rank, tok_seq, tok_pos, slots, tokens, sinks);
  if (cache_dtype == DLLM_BF16)
    return dllm_launch_pdl(latent_attention_kernel<__nv_bfloat16>, grid, dim3(ATT_WARPS * 32), bytes, stream, q, out,
                           cache, heads, rank, tok_seq, tok_pos, slots, tokens, sinks);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_latent_values(const float* mixed, const void* uv, const float* gates, int gate_stride, void* out,
                                   int tokens, int heads, int rank, int vdim, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || heads > 65535 || rank <= 0 || rank > 8192 || vdim <= 0) return DLLM_UNSUPPORTED_SIZE;
  if (!mixed || !uv || !out) return DLLM_BAD_ARGUMENT;
  dim3 grid(tokens, heads);
  size_t bytes = (size_t)rank * sizeof(float);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(latent_values_kernel<float, float>, grid, dim3(128), bytes, stream, mixed, (const float*)uv,
                           gates, gate_stride, (float*)out, heads, rank, vdim);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(latent_values_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(128), bytes, stream, mixed,
                           (const __nv_bfloat16*)uv, gates, gate_stride, (__nv_bfloat16*)out, heads, rank, vdim);
  return DLLM_BAD_ARGUMENT;
}
