// Embedding gather, RMSNorm (optionally of gathered rows), rotary position encoding fused with the cache write,
// and the residual add. The residual stream is float32 in both precisions; norms and rotations are computed in
// float32 and rounded once to the output type.
#include "common.cuh"

// ---- embedding: x[r, :] = float(table[token_r, :]) ----------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ tokens,
                             int hidden, int vocab, float scale, int* __restrict__ status) {
  int row = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  int token = tokens[row];
  if (token < 0 || token >= vocab) {  // refused, never read out of range
    if (threadIdx.x == 0) *(volatile int*)status = 64;  // (a word in device or pinned host memory)
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)row * hidden + i] = 0.f;
    return;
  }
  const T* src = table + (size_t)token * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)row * hidden + i] = to_float(src[i]) * scale;
}

// x[r, :] = float(table[token_r, :]) * scale (the product in float32; scale 1 is the plain gather).
DLLM_EXPORT int dllm_embed_scaled(float* out, const void* table, const int* tokens, int rows, int hidden, int vocab,
                                  int dtype, float scale, int* status, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (hidden <= 0 || vocab <= 0) return DLLM_BAD_ARGUMENT;
  int threads = hidden >= 256 ? 256 : 64;
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(embed_kernel<float>, dim3(rows), dim3(threads), 0, stream, out, (const float*)table,
                           tokens, hidden, vocab, scale, status);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(embed_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, out,
                           (const __nv_bfloat16*)table, tokens, hidden, vocab, scale, status);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_embed(float* out, const void* table, const int* tokens, int rows, int hidden, int vocab,
                           int dtype, int* status, cudaStream_t stream) {
  return dllm_embed_scaled(out, table, tokens, rows, hidden, vocab, dtype, 1.0f, status, stream);
}

// ---- RMSNorm: out[r] = x[rows ? rows[r] : r] * (1 / sqrt(mean(x^2) + eps)) * w ---------------------------------------
// One block per row; each thread sums a strided part, then a fixed-order block reduction, so a row's result does not
// depend on which other rows are in the launch.
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ weight,
                               const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float partial[32];
  int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = src[i];
    sum = fmaf(v, v, sum);
  }
  sum = warp_sum(sum);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) partial[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float v = lane < warps ? partial[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) partial[0] = 1.0f / sqrtf(v / (float)hidden + eps);
  }
  __syncthreads();
  float inv = partial[0];
  T* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_float<T>(src[i] * inv * weight[i]);
}

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
  *reinterpret_cast<uint2*>(dst) = packed;
}

// Narrow rows (hidden a multiple of 4, at most 4096 floats): one warp per row, the row kept in registers between
// the sum and the scaling, 16-byte loads. Lane l holds floats 4*(l + 32*i) ..; the sum is a fixed tree.
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_warp_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                           const float* __restrict__ weight,
                                                           const int* __restrict__ rows, int n_rows, int hidden,
                                                           float eps) {
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * hidden);
  int vecs = hidden >> 2;
  float4 v[32];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int idx = lane + 32 * i;
    if (idx < vecs) {
      v[i] = src[idx];
      sum = fmaf(v[i].x, v[i].x, sum); sum = fmaf(v[i].y, v[i].y, sum);
      sum = fmaf(v[i].z, v[i].z, sum); sum = fmaf(v[i].w, v[i].w, sum);
    }
  }
  sum = warp_sum(sum);
  float inv = 1.0f / sqrtf(sum / (float)hidden + eps);
  const float4* wv = reinterpret_cast<const float4*>(weight);
  T* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int idx = lane + 32 * i;
    if (idx < vecs) {
      float4 w4 = wv[idx];
      store4(dst + 4 * idx, v[i].x * inv * w4.x, v[i].y * inv * w4.y, v[i].z * inv * w4.z, v[i].w * inv * w4.w);
    }
  }
}

DLLM_EXPORT int dllm_rmsnorm(void* out, const float* x, const float* weight, const int* rows, int n_rows, int hidden,
                             float eps, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return DLLM_OK;
  if (hidden <= 0) return DLLM_BAD_ARGUMENT;
  if ((hidden & 3) == 0 && hidden <= 4096) {  // whatever the number of rows, so a row has the same bits everywhere
    int blocks = (n_rows + 7) / 8;
    if (out_dtype == DLLM_F32)
      return dllm_launch_pdl(rmsnorm_warp_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, x, weight, rows,
                             n_rows, hidden, eps);
    if (out_dtype == DLLM_BF16)
      return dllm_launch_pdl(rmsnorm_warp_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                             (__nv_bfloat16*)out, x, weight, rows, n_rows, hidden, eps);
    return DLLM_BAD_ARGUMENT;
  }
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (out_dtype == DLLM_F32)
    rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>((float*)out, x, weight, rows, hidden, eps);
  else if (out_dtype == DLLM_BF16)
    rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>((__nv_bfloat16*)out, x, weight, rows, hidden, eps);
  else
    return DLLM_BAD_ARGUMENT;
  return dllm_launch_status();
}

// ---- what a norm folded around the next product needs of the first rows of a step -------------------------------
// copy[r] = bfloat16(x[r]) and ssq[r] = sum of x[r]^2 (one part a row): a warp a row, any width that is a multiple
// of 4 (see NormArgs in gemm_common.cuh; later rows come from the epilogue of the products that write the residual).
__global__ void __launch_bounds__(256) cast_ssq_kernel(__nv_bfloat16* __restrict__ copy, float* __restrict__ ssq,
                                                       const float* __restrict__ x, int n_rows, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)r * hidden);
  float sum = 0.f;
  for (int idx = lane; idx < (hidden >> 2); idx += 32) {
    float4 v = src[idx];
    sum = fmaf(v.x, v.x, sum); sum = fmaf(v.y, v.y, sum);
    sum = fmaf(v.z, v.z, sum); sum = fmaf(v.w, v.w, sum);
    store4(copy + (size_t)r * hidden + 4 * idx, v.x, v.y, v.z, v.w);
  }
  sum = warp_sum(sum);
  if (lane == 0) ssq[r] = sum;
}

DLLM_EXPORT int dllm_cast_ssq(void* copy, float* ssq, const float* x, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return DLLM_OK;
  if (hidden <= 0 || (hidden & 3) || copy == nullptr || ssq == nullptr) return DLLM_UNSUPPORTED_SIZE;
  return dllm_launch_pdl(cast_ssq_kernel, dim3((n_rows + 7) / 8), dim3(256), 0, stream, (__nv_bfloat16*)copy, ssq, x,
                         n_rows, hidden);
}

// ---- rotary encoding + cache write --------------------------------------------------------------------------------
// qkv is the float32 output of the fused q/k/v projection, [tokens, (heads + 2 kv_heads) * head_dim]. Queries and
// keys rotate pairs (i, i + rotary_dim/2) by the angle whose cosine and sine the table holds for the token's
// position; dimensions beyond rotary_dim pass through. Queries go to q_out, keys and values into the token's
// place in the paged cache (page_table[slot][pos / page_size], row pos % page_size). With parts > 1, qkv is that
// many partial results of the projection, `part_stride` floats apart, and a value is their sum in order.
template <typename T>
__global__ void rope_cache_kernel(const float* __restrict__ qkv, T* __restrict__ q_out, KvLayout cache,
                                  const float2* __restrict__ table, int rotary_dim, int heads,
                                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                  const int* __restrict__ slots, int write_cache, int parts, size_t part_stride) {
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x, h = blockIdx.y;
  int hd = cache.head_dim, nkv = cache.kv_heads;
  if (!write_cache && h >= heads) return;
  int pos = tok_pos[t];
  const float* src = qkv + ((size_t)t * (heads + 2 * nkv) + h) * hd;
  T* dst;
  bool rotate = h < heads + nkv && table != nullptr;
  if (h < heads) {
    dst = q_out + ((size_t)t * heads + h) * hd;
  } else {
    int which = h < heads + nkv ? 0 : 1;
    int g = h - heads - which * nkv;
    int slot = slots[tok_seq[t]];
    int page = cache.page_table[(size_t)slot * cache.max_pages + pos / cache.page_size];
    dst = (T*)cache.base + kv_offset(cache, page, which, g, pos % cache.page_size);
  }
  int half = rotary_dim / 2;
  auto value = [&](int i) {
    float sum = src[i];
    for (int p = 1; p < parts; ++p) sum += src[(size_t)p * part_stride + i];
    return sum;
  };
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    float v = value(i);
    if (rotate && i < rotary_dim) {
      int j = i < half ? i : i - half;
      float2 cs = table[(size_t)pos * half + j];
      float a = value(j), b = value(j + half);
      v = i < half ? fmaf(a, cs.x, -(b * cs.y)) : fmaf(a, cs.y, b * cs.x);
    }
    dst[i] = from_float<T>(v);
  }
}

DLLM_EXPORT int dllm_rope_cache_write(const float* qkv, void* q_out, void* cache_base, const int* page_table,
                                      int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                      const float* table, int rotary_dim, const int* tok_seq, const int* tok_pos,
                                      const int* slots, int tokens, int write_cache, int dtype, int parts,
                                      long long part_stride, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || head_dim <= 0 || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) ||
      parts < 1 || part_stride < 0)
    return DLLM_BAD_ARGUMENT;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  dim3 grid(tokens, heads + 2 * kv_heads);
  int threads = head_dim >= 128 ? 128 : (head_dim > 32 ? 64 : 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(rope_cache_kernel<float>, grid, dim3(threads), 0, stream, qkv, (float*)q_out, cache,
                           (const float2*)table, rotary_dim, heads, tok_seq, tok_pos, slots, write_cache, parts,
                           (size_t)part_stride);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(rope_cache_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, qkv,
                           (__nv_bfloat16*)q_out, cache, (const float2*)table, rotary_dim, heads, tok_seq, tok_pos,
                           slots, write_cache, parts, (size_t)part_stride);
  return DLLM_BAD_ARGUMENT;
}

// ---- residual += update (float32 sum) -----------------------------------------------------------------------------
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ residual, const T* __restrict__ update, size_t count) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) residual[i] += to_float(update[i]);
}

DLLM_EXPORT int dllm_add_residual(float* residual, const void* update, long long count, int dtype,
                                  cudaStream_t stream) {
  if (count <= 0) return DLLM_OK;
  unsigned blocks = (unsigned)((count + 255) / 256);
  if (dtype == DLLM_F32)
    add_residual_kernel<float><<<blocks, 256, 0, stream>>>(residual, (const float*)update, (size_t)count);
  else if (dtype == DLLM_BF16)
    add_residual_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(residual, (const __nv_bfloat16*)update,
                                                                    (size_t)count);
  else
    return DLLM_BAD_ARGUMENT;
  return dllm_launch_status();
}

// ---- residual += parts[0] + parts[1] + ... (the partial results of a product whose reduction was cut) ------------
// parts holds `k_split` float32 arrays of `count` values one behind the other; they are summed in that order, then
// added to the residual. count must be a multiple of 4 and the arrays 16-byte aligned.
__global__ void __launch_bounds__(256) sum_parts_residual_kernel(float* __restrict__ residual,
                                                                 const float* __restrict__ parts, int k_split,
                                                                 size_t count) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= count) return;
  float4 old = *reinterpret_cast<const float4*>(residual + i);
  float4 sum = __ldcg(reinterpret_cast<const float4*>(parts + i));
  for (int s = 1; s < k_split; ++s) {
    float4 p = __ldcg(reinterpret_cast<const float4*>(parts + (size_t)s * count + i));
    sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
  }
  old.x += sum.x; old.y += sum.y; old.z += sum.z; old.w += sum.w;
  *reinterpret_cast<float4*>(residual + i) = old;
}

DLLM_EXPORT int dllm_sum_parts_residual(float* residual, const float* parts, int k_split, long long count,
                                        cudaStream_t stream) {
  if (count <= 0) return DLLM_OK;
  if (k_split < 1 || (count & 3) || ((uintptr_t)residual & 15) || ((uintptr_t)parts & 15)) return DLLM_UNSUPPORTED_SIZE;
  unsigned blocks = (unsigned)((count / 4 + 255) / 256);
  return dllm_launch_pdl(sum_parts_residual_kernel, dim3(blocks), dim3(256), 0, stream, residual, parts, k_split,
                         (size_t)count);
}

// ---- decode feedback: the chosen tokens become the next step's input, positions move on by one -------------------
// Lets single-token steps follow one another on the device without the host: tokens[b] = chosen[b], positions and
// cached lengths + 1, and the chosen tokens are appended to `history` ([capacity, batch]) at row *counter.
__global__ void decode_advance_kernel(int* __restrict__ tokens, int* __restrict__ tok_pos, int* __restrict__ start,
                                      const int* __restrict__ chosen, int* __restrict__ history,
                                      int* __restrict__ counter, int batch, int capacity) {
  pdl_wait();
  int row = *counter;
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    int token = chosen[b];
    tokens[b] = token;
    tok_pos[b] += 1;
    start[b] += 1;
    if (row < capacity) history[(size_t)row * batch + b] = token;
  }
  __syncthreads();
  if (threadIdx.x == 0) *counter = row + 1;
}

DLLM_EXPORT int dllm_decode_advance(int* tokens, int* tok_pos, int* start, const int* chosen, int* history,
                                    int* counter, int batch, int capacity, cudaStream_t stream) {
  if (batch <= 0) return DLLM_OK;
  return dllm_launch_pdl(decode_advance_kernel, dim3(1), dim3(256), 0, stream, tokens, tok_pos, start, chosen,
                         history, counter, batch, capacity);
}

// A copy from pinned host memory to the device on the given stream (the host side of a step makes two small ones: the
// step's metadata and the page-table rows that changed; through this entry point each costs the host a few
// microseconds less than through the tensor library's dispatch).
DLLM_EXPORT int dllm_copy_to_device(void* dst, const void* src, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return DLLM_OK;
  if (dst == nullptr || src == nullptr) return DLLM_BAD_ARGUMENT;
  return cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, stream) == cudaSuccess ? DLLM_OK
                                                                                                 : DLLM_LAUNCH_FAILED;
}

// Takes token ids out of the choice while an output is shorter than it has to be: logits[row, ids[i]] = -inf for
// every row, if *produced + *steps < min_tokens (`produced`: tokens every sequence of the batch has so far when a run
// of steps begins; `steps`: the steps of that run so far, or null). A probability of exactly zero is never drawn and
// never the largest, so what is chosen is what a choice among the other tokens alone would choose.
__global__ void mask_tokens_kernel(float* __restrict__ logits, int rows, int vocab, const int* __restrict__ ids,
                                   int n_ids, const int* __restrict__ produced, const int* __restrict__ steps,
                                   int min_tokens) {
  pdl_wait();
  int have = *produced + (steps != nullptr ? *steps : 0);
  if (have >= min_tokens) return;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * n_ids; i += gridDim.x * blockDim.x) {
    int id = ids[i % n_ids];
    if (id >= 0 && id < vocab) logits[(size_t)(i / n_ids) * vocab + id] = -INFINITY;
  }
}

DLLM_EXPORT int dllm_mask_tokens(float* logits, int rows, int vocab, const int* ids, int n_ids, const int* produced,
                                 const int* steps, int min_tokens, cudaStream_t stream) {
  if (rows <= 0 || n_ids <= 0 || min_tokens <= 0) return DLLM_OK;
  if (vocab <= 0 || logits == nullptr || ids == nullptr || produced == nullptr) return DLLM_BAD_ARGUMENT;
  return dllm_launch_pdl(mask_tokens_kernel, dim3(1), dim3(256), 0, stream, logits, rows, vocab, ids, n_ids, produced,
                         steps, min_tokens);
}

// ---- layer norm without a bias: out[r] = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w -------------------------
// One block per row: the mean first, then the mean of the squared deviations (two passes, as the definition reads;
// not E[x^2] - mean^2), both in float32 with a fixed-order block reduction, so a row's bits do not depend on the
// other rows of the launch. `rows` gathers as in the RMS norm.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  __syncthreads();  // (scratch may still be read from the sum before)
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = lane < warps ? scratch[lane] : 0.f;
  return warp_sum(total);
}

template <typename T>
__global__ void layernorm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ weight,
                                 const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) sum += src[i];
  float mean = block_sum(sum, scratch) / (float)hidden;
  float squares = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float d = src[i] - mean;
    squares = fmaf(d, d, squares);
  }
  float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)hidden + eps);
  T* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_float<T>((src[i] - mean) * inv * weight[i]);
}

// Narrow rows (hidden a multiple of 4, at most 4096 floats): one warp per row, the row kept in registers between the
// mean, the squared deviations and the scaling (one pass over memory), 16-byte loads, sums in a fixed tree.
template <typename T>
__global__ void __launch_bounds__(256) layernorm_warp_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                             const float* __restrict__ weight,
                                                             const int* __restrict__ rows, int n_rows, int hidden,
                                                             float eps) {
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31;
  int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * hidden);
  int vecs = hidden >> 2;
  float4 v[32];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int idx = lane + 32 * i;
    if (idx < vecs) {
      v[i] = src[idx];
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  float mean = warp_sum(sum) / (float)hidden;
  float squares = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int idx = lane + 32 * i;
    if (idx < vecs) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
      squares = fmaf(v[i].x, v[i].x, squares); squares = fmaf(v[i].y, v[i].y, squares);
      squares = fmaf(v[i].z, v[i].z, squares); squares = fmaf(v[i].w, v[i].w, squares);
    }
  }
  float inv = 1.0f / sqrtf(warp_sum(squares) / (float)hidden + eps);
  const float4* wv = reinterpret_cast<const float4*>(weight);
  T* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    int idx = lane + 32 * i;
    if (idx < vecs) {
      float4 w4 = wv[idx];
      store4(dst + 4 * idx, v[i].x * inv * w4.x, v[i].y * inv * w4.y, v[i].z * inv * w4.z, v[i].w * inv * w4.w);
    }
  }
}

DLLM_EXPORT int dllm_layernorm(void* out, const float* x, const float* weight, const int* rows, int n_rows, int hidden,
                               float eps, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return DLLM_OK;
  if (hidden <= 0) return DLLM_BAD_ARGUMENT;
  if ((hidden & 3) == 0 && hidden <= 4096) {  // whatever the number of rows, so a row has the same bits everywhere
    int blocks = (n_rows + 7) / 8;
    if (out_dtype == DLLM_F32)
      return dllm_launch_pdl(layernorm_warp_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, x, weight,
                             rows, n_rows, hidden, eps);
    if (out_dtype == DLLM_BF16)
      return dllm_launch_pdl(layernorm_warp_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                             (__nv_bfloat16*)out, x, weight, rows, n_rows, hidden, eps);
    return DLLM_BAD_ARGUMENT;
  }
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (out_dtype == DLLM_F32)
    return dllm_launch_pdl(layernorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (float*)out, x, weight,
                           rows, hidden, eps);
  if (out_dtype == DLLM_BF16)
    return dllm_launch_pdl(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream,
                           (__nv_bfloat16*)out, x, weight, rows, hidden, eps);
  return DLLM_BAD_ARGUMENT;
}

// ---- gated unit with clamped inputs ------------------------------------------------------------------------------
// in[r] = gate_0, up_0, gate_1, up_1, ... as the product of the interleaved weight left them; g = min(gate, limit),
// u = clamp(up, -limit, limit); out[r, i] = g * sigmoid(alpha * g) * (u + shift), computed in float32, rounded once.
template <typename T>
__global__ void glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ in, long long total, int width,
                                   float limit, float alpha, float shift) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i / width;
    int c = (int)(i - r * width);
    float g = fminf(to_float(in[r * 2 * width + 2 * c]), limit);
    float u = fminf(fmaxf(to_float(in[r * 2 * width + 2 * c + 1]), -limit), limit);
    float s = 1.0f / (1.0f + expf(-alpha * g));
    out[i] = from_float<T>(g * s * (u + shift));
  }
}

// Four outputs a thread from eight inputs (width a multiple of 4: rows start on 16 bytes).
__device__ __forceinline__ void load8(const float* p, float* v) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(pairs[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename T>
__global__ void glu_clamped_vector_kernel(T* __restrict__ out, const T* __restrict__ in, long long quads, float limit,
                                          float alpha, float shift) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < quads;
       i += (long long)gridDim.x * blockDim.x) {
    float v[8], y[4];
    load8(in + 8 * i, v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float g = fminf(v[2 * j], limit);
      float u = fminf(fmaxf(v[2 * j + 1], -limit), limit);
      y[j] = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift);
    }
    store4(out + 4 * i, y[0], y[1], y[2], y[3]);
  }
}

template <typename T>
static int launch_glu_clamped(T* out, const T* in, int rows, int width, float limit, float alpha, float shift,
                              cudaStream_t stream) {
  long long total = (long long)rows * width;
  if ((width & 3) == 0) {
    long long quads = total / 4;
    int blocks = (int)((quads + 255) / 256 < 148 * 16 ? (quads + 255) / 256 : 148 * 16);
    return dllm_launch_pdl(glu_clamped_vector_kernel<T>, dim3(blocks), dim3(256), 0, stream, out, in, quads, limit,
                           alpha, shift);
  }
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return dllm_launch_pdl(glu_clamped_kernel<T>, dim3(blocks), dim3(256), 0, stream, out, in, total, width, limit, alpha,
                         shift);
}

DLLM_EXPORT int dllm_glu_clamped(void* out, const void* in, int rows, int width, float limit, float alpha, float shift,
                                 int dtype, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (width <= 0 || out == nullptr || in == nullptr) return DLLM_BAD_ARGUMENT;
  if (dtype == DLLM_F32)
    return launch_glu_clamped((float*)out, (const float*)in, rows, width, limit, alpha, shift, stream);
  if (dtype == DLLM_BF16)
    return launch_glu_clamped((__nv_bfloat16*)out, (const __nv_bfloat16*)in, rows, width, limit, alpha, shift, stream);
  return DLLM_BAD_ARGUMENT;
}

// ---- sum of RMS-normed branches into the residual ----------------------------------------------------------------
// residual[r] += factor * (a[r] / rms(a[r]) * wa + b[r] / rms(b[r]) * wb), everything float32; one block per row.
__global__ void norm_sum_residual_kernel(float* __restrict__ residual, const float* __restrict__ a,
                                         const float* __restrict__ wa, const float* __restrict__ b,
                                         const float* __restrict__ wb, int hidden, float eps, float factor) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  size_t base = (size_t)blockIdx.x * hidden;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float va = a[base + i], vb = b[base + i];
    sa = fmaf(va, va, sa);
    sb = fmaf(vb, vb, sb);
  }
  float inv_a = 1.0f / sqrtf(block_sum(sa, scratch) / (float)hidden + eps);
  float inv_b = 1.0f / sqrtf(block_sum(sb, scratch) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    residual[base + i] += factor * (a[base + i] * inv_a * wa[i] + b[base + i] * inv_b * wb[i]);
}

DLLM_EXPORT int dllm_norm_sum_residual(float* residual, const float* a, const float* wa, const float* b, const float* wb,
                                       int rows, int hidden, float eps, float factor, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (hidden <= 0) return DLLM_BAD_ARGUMENT;
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  return dllm_launch_pdl(norm_sum_residual_kernel, dim3(rows), dim3(threads), 0, stream, residual, a, wa, b, wb, hidden,
                         eps, factor);
}

// ---- one RMS-normed sublayer output into the residual -------------------------------------------------------------
// residual[r] += y[r] / sqrt(mean(y[r]^2) + eps) * w, everything float32; one block per row. The arrangement that
// norms a sublayer's output instead of its input ends both of its sublayers with this. With `copy`, the new rows are
// also written there as bfloat16: they are the next sublayer's operand, which then needs no kernel to round them.
__global__ void norm_add_residual_kernel(float* __restrict__ residual, const float* __restrict__ y,
                                         const float* __restrict__ w, __nv_bfloat16* __restrict__ copy, int hidden,
                                         float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  size_t base = (size_t)blockIdx.x * hidden;
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = y[base + i];
    s = fmaf(v, v, s);
  }
  float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = residual[base + i] + y[base + i] * inv * w[i];
    residual[base + i] = v;
    if (copy != nullptr) copy[base + i] = __float2bfloat16_rn(v);
  }
}

DLLM_EXPORT int dllm_norm_add_residual(float* residual, const float* y, const float* w, void* copy, int rows, int hidden,
                                       float eps, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (hidden <= 0 || residual == nullptr || y == nullptr || w == nullptr) return DLLM_BAD_ARGUMENT;
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  return dllm_launch_pdl(norm_add_residual_kernel, dim3(rows), dim3(threads), 0, stream, residual, y, w,
                         (__nv_bfloat16*)copy, hidden, eps);
}

// ---- the float32 stream as an operand: out = bfloat16(x) ----------------------------------------------------------
// For a sublayer that reads the stream itself, with no norm in front whose kernel would do the rounding.
__global__ void cast_rows_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ x, long long pairs,
                                 long long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
       i += (long long)gridDim.x * blockDim.x) {
    if (2 * i + 1 < total) {
      float2 v = *reinterpret_cast<const float2*>(x + 2 * i);
      *reinterpret_cast<__nv_bfloat162*>(out + 2 * i) = __floats2bfloat162_rn(v.x, v.y);
    } else {
      out[2 * i] = __float2bfloat16_rn(x[2 * i]);
    }
  }
}

DLLM_EXPORT int dllm_cast_rows(void* out, const float* x, long long total, cudaStream_t stream) {
  if (total <= 0) return DLLM_OK;
  if (out == nullptr || x == nullptr || ((uintptr_t)x & 7) || ((uintptr_t)out & 3)) return DLLM_BAD_ARGUMENT;
  long long pairs = (total + 1) / 2;
  int blocks = (int)((pairs + 255) / 256 < 148 * 16 ? (pairs + 255) / 256 : 148 * 16);
  return dllm_launch_pdl(cast_rows_kernel, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, x, pairs, total);
}

// ---- the stream beside a kept copy, as one operand ---------------------------------------------------------------
// both[r] = [x[r] | kept[r]] in the activation type (the operand of the product that mixes the two), and then
// x[r] = start (one row for all): the product adds into x in its epilogue, so x ends as start + W [x | kept].
template <typename T>
__global__ void concat_restart_kernel(T* __restrict__ both, float* __restrict__ x, const float* __restrict__ kept,
                                      const float* __restrict__ start, long long total, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i / hidden;
    int c = (int)(i - r * hidden);
    both[r * 2 * hidden + c] = from_float<T>(x[i]);
    both[r * 2 * hidden + hidden + c] = from_float<T>(kept[i]);
    x[i] = start != nullptr ? start[c] : 0.f;
  }
}

DLLM_EXPORT int dllm_concat_restart(void* both, float* x, const float* kept, const float* start, int rows, int hidden,
                                    int dtype, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (hidden <= 0 || both == nullptr || x == nullptr || kept == nullptr) return DLLM_BAD_ARGUMENT;
  long long total = (long long)rows * hidden;
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(concat_restart_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)both, x, kept,
                           start, total, hidden);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(concat_restart_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                           (__nv_bfloat16*)both, x, kept, start, total, hidden);
  return DLLM_BAD_ARGUMENT;
}

// ---- RMS norm followed by a short causal convolution over time ------------------------------------------------------
// h_t = x_t / sqrt(mean(x_t^2) + eps) * w;  out_t = h_t + sum_j taps[:, j] h_(t - n_taps + 1 + j): every channel is
// filtered over the sequence's own earlier tokens (zeros before its start), the last tap on the token itself. The
// normed rows of tokens before the step come from `history` [slots, n_taps - 1, hidden] (float32, the oldest first),
// those of the step are normed again here from the stream (a row's norm costs one pass over it). A block per token;
// everything float32, rounded once to the output type. In a step of single tokens the block also moves the history
// on; otherwise `norm_conv_history_kernel` does, after every block has read the old one. A step of few tokens deals
// each token's channels to several blocks (blockIdx.y; every one of them sums the row's squares for itself), so that
// a block's loads of history, taps and weights are one round and not a chain of them.
#define CONV_MAX_TAPS 8

template <typename T>
__global__ void __launch_bounds__(256) norm_conv_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                        const float* __restrict__ w, const float* __restrict__ taps,
                                                        int n_taps, float* __restrict__ history,
                                                        const int* __restrict__ tok_seq,
                                                        const int* __restrict__ cu_seqlens,
                                                        const int* __restrict__ slots, int hidden, float eps,
                                                        int single) {
  __shared__ float scratch[32];
  __shared__ float inv[CONV_MAX_TAPS];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, seq = tok_seq[t], local = t - cu_seqlens[seq], slot = slots[seq];
  const int kept = n_taps - 1;
  for (int back = 0; back < n_taps && back <= local; ++back) {  // the rows of this step: their norms
    const float* row = x + (size_t)(t - back) * hidden;
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) s = fmaf(row[i], row[i], s);
    float total = block_sum(s, scratch);
    if (threadIdx.x == 0) inv[back] = 1.0f / sqrtf(total / (float)hidden + eps);
  }
  __syncthreads();
  float* old = history + (size_t)slot * kept * hidden;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
    float h[CONV_MAX_TAPS];  // h[j]: the input `kept - j` tokens back
    for (int j = 0; j < n_taps; ++j) {
      int back = kept - j;
      h[j] = back <= local ? x[(size_t)(t - back) * hidden + i] * inv[back] * w[i]
                           : old[(size_t)(kept - (back - local)) * hidden + i];
    }
    float sum = h[kept];
    for (int j = 0; j < n_taps; ++j) sum = fmaf(taps[(size_t)i * n_taps + j], h[j], sum);
    out[(size_t)t * hidden + i] = from_float<T>(sum);
    if (single)
      for (int j = 0; j < kept; ++j) old[(size_t)j * hidden + i] = h[j + 1];
  }
}

// The history after a step of any lengths: the last n_taps - 1 normed rows of each sequence, from the step's rows
// where it has that many and from the old history before them. A block per sequence and kept row; a thread reads
// what it needs of the old history before the block writes (a row r only reads rows >= r).
__global__ void __launch_bounds__(256) norm_conv_history_kernel(const float* __restrict__ x,
                                                                const float* __restrict__ w,
                                                                float* __restrict__ history,
                                                                const int* __restrict__ cu_seqlens,
                                                                const int* __restrict__ slots, int n_taps, int hidden,
                                                                float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, first = cu_seqlens[seq], count = cu_seqlens[seq + 1] - first, slot = slots[seq];
  const int kept = n_taps - 1;
  float* old = history + (size_t)slot * kept * hidden;
  for (int r = 0; r < kept; ++r) {  // in order: row r's source, where it is old history, is a row behind r
    int at = count - kept + r;      // index among the step's tokens of this sequence
    if (at >= 0) {
      const float* row = x + (size_t)(first + at) * hidden;
      float s = 0.f;
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) s = fmaf(row[i], row[i], s);
      float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) old[(size_t)r * hidden + i] = row[i] * inv * w[i];
    } else {
      for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        old[(size_t)r * hidden + i] = old[(size_t)(r + count) * hidden + i];
    }
  }
}

// out[tokens, hidden] = norm(x) + conv(norm(x)) as above; taps [hidden, n_taps] float32; history [slots, n_taps - 1,
// hidden] float32 (may be null for one tap); `single`: every sequence of the step has one token.
DLLM_EXPORT int dllm_norm_conv(void* out, const float* x, const float* w, const float* taps, int n_taps,
                               float* history, const int* tok_seq, const int* cu_seqlens, const int* slots, int tokens,
                               int sequences, int hidden, float eps, int single, int out_dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (hidden <= 0 || n_taps < 1 || n_taps > CONV_MAX_TAPS) return DLLM_UNSUPPORTED_SIZE;
  if (!out || !x || !w || !taps || !tok_seq || !cu_seqlens || !slots || (n_taps > 1 && !history))
    return DLLM_BAD_ARGUMENT;
  int threads = hidden >= 1024 ? 256 : 128;
  int slices = 1;
  if (tokens <= 64) slices = (hidden + threads - 1) / threads < 32 ? (hidden + threads - 1) / threads : 32;
  dim3 grid(tokens, slices);
  int status;
  if (out_dtype == DLLM_F32)
    status = dllm_launch_pdl(norm_conv_kernel<float>, grid, dim3(threads), 0, stream, (float*)out, x, w, taps,
                             n_taps, history, tok_seq, cu_seqlens, slots, hidden, eps, single);
  else if (out_dtype == DLLM_BF16)
    status = dllm_launch_pdl(norm_conv_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream,
                             (__nv_bfloat16*)out, x, w, taps, n_taps, history, tok_seq, cu_seqlens, slots, hidden, eps,
                             single);
  else
    return DLLM_BAD_ARGUMENT;
  if (status != DLLM_OK || single || n_taps == 1) return status;
  return dllm_launch_pdl(norm_conv_history_kernel, dim3(sequences), dim3(threads), 0, stream, x, w, history, cu_seqlens,
                         slots, n_taps, hidden, eps);
}

// ---- bias, activation and a gate per row behind a product -----------------------------------------------------------
// out[r, i] = act(in[r, i] + bias[i]) * (gated ? sigmoid(in[r, width]) : 1) for i < width; `in` float32 rows of
// `stride` values (a product's float32 output: with a gate, its column `width` is the row's gate pre-activation).
// act 0: none, 1: gelu (erf), 2: gelu (tanh form), 3: relu squared. Float32, rounded once to the output type. `out` has
// rows of out_width >= width values; the columns behind `width` are set to zero (a padded reduction width).
__device__ __forceinline__ float activate(float z, int kind) {
  if (kind == 1) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (kind == 2) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  if (kind == 3) { float r = fmaxf(z, 0.f); return r * r; }
  return z;
}
__device__ __forceinline__ float sigmoid_f(float g) {
  if (g >= 0.f) return 1.0f / (1.0f + expf(-g));
  float e = expf(g);
  return e / (1.0f + e);
}

template <typename T>
__global__ void __launch_bounds__(256) bias_act_kernel(T* __restrict__ out, const float* __restrict__ in,
                                                       const float* __restrict__ bias, int width, int out_width,
                                                       int stride, int kind, int gated) {
  pdl_launch_dependents();
  pdl_wait();
  const float* row = in + (size_t)blockIdx.x * stride;
  float gate = gated ? sigmoid_f(row[width]) : 1.0f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < out_width; i += gridDim.y * blockDim.x) {
    float v = 0.f;
    if (i < width) v = activate(row[i] + (bias != nullptr ? bias[i] : 0.f), kind) * gate;
    out[(size_t)blockIdx.x * out_width + i] = from_float<T>(v);
  }
}

DLLM_EXPORT int dllm_bias_act(void* out, const float* in, const float* bias, int rows, int width, int out_width,
                              int stride, int kind, int gated, int out_dtype, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (width <= 0 || out_width < width || stride < width + (gated ? 1 : 0) || kind < 0 || kind > 3)
    return DLLM_UNSUPPORTED_SIZE;
  if (!out || !in) return DLLM_BAD_ARGUMENT;
  dim3 grid(rows, (width + 1023) / 1024 > 64 ? 64 : (width + 1023) / 1024);
  if (out_dtype == DLLM_F32)
    return dllm_launch_pdl(bias_act_kernel<float>, grid, dim3(256), 0, stream, (float*)out, in, bias, width, out_width,
                           stride, kind, gated);
  if (out_dtype == DLLM_BF16)
    return dllm_launch_pdl(bias_act_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)out, in, bias,
                           width, out_width, stride, kind, gated);
  return DLLM_BAD_ARGUMENT;
}

// residual[r, :] += row (float32): a bias behind a product that has added into the stream.
__global__ void __launch_bounds__(256) add_row_kernel(float* __restrict__ residual, const float* __restrict__ row,
                                                      long long total, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    residual[i] += row[i % hidden];
}

DLLM_EXPORT int dllm_add_row(float* residual, const float* row, int rows, int hidden, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (hidden <= 0 || !residual || !row) return DLLM_BAD_ARGUMENT;
  long long total = (long long)rows * hidden;
  int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  return dllm_launch_pdl(add_row_kernel, dim3(blocks), dim3(256), 0, stream, residual, row, total, hidden);
}

// ---- a token's own embedding part times an activated gate -----------------------------------------------------------
// out[r, i] = act(z[r, i]) * table[tokens[r], offset + i] for i < width (z float32 rows of `stride` values; the table
// in T, rows of `table_width` values); columns width .. out_width - 1 of `out` are set to zero (a reduction width
// padded for the product that follows). A token outside the table gives a zero row and sets the status word.
template <typename T>
__global__ void __launch_bounds__(128) gate_embed_kernel(T* __restrict__ out, const float* __restrict__ z, int stride,
                                                         const T* __restrict__ table, int table_width, int vocab,
                                                         int offset, const int* __restrict__ tokens, int width,
                                                         int out_width, int kind, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, token = tokens[r];
  const bool ok = token >= 0 && token < vocab;
  if (!ok && threadIdx.x == 0) *(volatile int*)status = 64;
  for (int i = threadIdx.x; i < out_width; i += blockDim.x) {
    float v = 0.f;
    if (ok && i < width)
      v = activate(z[(size_t)r * stride + i], kind) * to_float(table[(size_t)token * table_width + offset + i]);
    out[(size_t)r * out_width + i] = from_float<T>(v);
  }
}

DLLM_EXPORT int dllm_gate_embed(void* out, const float* z, int stride, const void* table, int table_width, int vocab,
                                int offset, const int* tokens, int rows, int width, int out_width, int kind,
                                int dtype, int* status, cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (width <= 0 || out_width < width || offset < 0 || offset + width > table_width || kind < 0 || kind > 3)
    return DLLM_UNSUPPORTED_SIZE;
  if (!out || !z || !table || !tokens || !status) return DLLM_BAD_ARGUMENT;
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(gate_embed_kernel<float>, dim3(rows), dim3(128), 0, stream, (float*)out, z, stride,
                           (const float*)table, table_width, vocab, offset, tokens, width, out_width, kind, status);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(gate_embed_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, (__nv_bfloat16*)out, z,
                           stride, (const __nv_bfloat16*)table, table_width, vocab, offset, tokens, width, out_width,
                           kind, status);
  return DLLM_BAD_ARGUMENT;
}

// ---- a norm without statistics ---------------------------------------------------------------------------------------
// out[r, i] = tanh(alpha * x[row(r), i]) * weight[i] + bias[i] in float32, rounded once to the output type; row(r) =
// rows[r] where `rows` is given (a gather of the wanted rows), else r. Four values a thread where rows start on 16
// bytes.
template <typename T>
__global__ void __launch_bounds__(256) dynamic_tanh_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                           const float* __restrict__ weight,
                                                           const float* __restrict__ bias,
                                                           const int* __restrict__ rows, int hidden, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  T* dst = out + (size_t)r * hidden;
  if ((hidden & 3) == 0) {
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < hidden; i += gridDim.y * blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(src + i), w = *reinterpret_cast<const float4*>(weight + i),
             b = *reinterpret_cast<const float4*>(bias + i);
      store4(dst + i, fmaf(tanhf(alpha * v.x), w.x, b.x), fmaf(tanhf(alpha * v.y), w.y, b.y),
             fmaf(tanhf(alpha * v.z), w.z, b.z), fmaf(tanhf(alpha * v.w), w.w, b.w));
    }
    return;
  }
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x)
    dst[i] = from_float<T>(fmaf(tanhf(alpha * src[i]), weight[i], bias[i]));
}

DLLM_EXPORT int dllm_dynamic_tanh(void* out, const float* x, const float* weight, const float* bias, const int* rows,
                                  int n_rows, int hidden, float alpha, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return DLLM_OK;
  if (hidden <= 0 || !out || !x || !weight || !bias) return DLLM_BAD_ARGUMENT;
  int across = (hidden + 1023) / 1024;
  dim3 grid(n_rows, across > 64 ? 64 : across);
  if (out_dtype == DLLM_F32)
    return dllm_launch_pdl(dynamic_tanh_kernel<float>, grid, dim3(256), 0, stream, (float*)out, x, weight, bias, rows,
                           hidden, alpha);
  if (out_dtype == DLLM_BF16)
    return dllm_launch_pdl(dynamic_tanh_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)out, x,
                           weight, bias, rows, hidden, alpha);
  return DLLM_BAD_ARGUMENT;
}

// ---- gated unit with an activation by kind ---------------------------------------------------------------------------
// in[r] = gate_0, up_0, gate_1, up_1, ... float32, as the product of the interleaved weight left them;
// out[r, i] = act(gate_i) * up_i (kinds as `activate`), computed in float32, rounded once.
template <typename T>
__global__ void __launch_bounds__(256) glu_act_kernel(T* __restrict__ out, const float* __restrict__ in,
                                                      long long total, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float2 v = *reinterpret_cast<const float2*>(in + 2 * i);
    out[i] = from_float<T>(activate(v.x, kind) * v.y);
  }
}

DLLM_EXPORT int dllm_glu_act(void* out, const float* in, int rows, int width, int kind, int out_dtype,
                             cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (width <= 0 || kind < 0 || kind > 3) return DLLM_UNSUPPORTED_SIZE;
  if (!out || !in) return DLLM_BAD_ARGUMENT;
  long long total = (long long)rows * width;
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (out_dtype == DLLM_F32)
    return dllm_launch_pdl(glu_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, in, total, kind);
  if (out_dtype == DLLM_BF16)
    return dllm_launch_pdl(glu_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, in,
                           total, kind);
  return DLLM_BAD_ARGUMENT;
}
