// Attention without a softmax: the weight of a visible key is sigmoid(q . k * scale - slope_h * (i - j) + b_h), the
// heads' weights are then mixed by a matrix, weight_h(i, j) <- sum_g M[h, g] weight_g(i, j), and head h applies its
// mixed weights to the values of its own key/value head; the concatenated heads are multiplied by sigmoid(gate).
// Nothing is normalised over the keys, so the sums over stretches of keys simply add up.
//
// Position i sees j <= i with i - j < window, and the sequence's first `keep` positions whatever their distance.
// Queries and keys may be RMS-normed over the WHOLE projection (all heads at once, one weight per coordinate) and have
// biases; there is no rotation: positions enter through the distance penalty alone.
//
//   sigmoid_prepare:    a block per token, from the fused projection's float32 row: biases, the two whole-row norms,
//                       queries to their buffer, keys and values into the token's place in the cache.
//   sigmoid_attention:  the general kernel: a block per token (and stretch of keys), all heads of the token together,
//                       tiles of 32 keys: scores with a key a lane, mixing through shared memory, then the weighted
//                       sum of the values with the threads across (head, value coordinate). float32 arithmetic
//                       whatever the cache's type.
//   sigmoid_combine:    sums the stretches' partial outputs in order, applies the gate, rounds.
//
// Cache entry: [page][ keys: kv_head, row, dim | values: kv_head, row, vdim ] (wide_kv.cuh).
#include "wide_kv.cuh"

namespace {

constexpr int TJ = 32;        // keys of a tile (pages are multiples of it: a tile lies in one page)
constexpr int MAX_OUT = 8;    // outputs a thread accumulates

struct SigmoidArgs {
  const void* q;        // [tokens, heads * dim] in the cache's type
  WideKv cache;
  const float* mix;     // [heads, heads] or null (no mixing)
  const float* slopes;  // [heads] or null (no distance penalty)
  const float* head_bias;  // [heads] or null
  const float* gates;   // gates[token * gate_ld + o], o < heads * vdim, or null
  int gate_ld;
  void* out;            // [tokens, heads * vdim] in the cache's type
  float* part;          // splits > 1: [split][token][heads * vdim]
  int heads, window, keep, tokens, splits;
  float scale;
  const int* tok_seq;
  const int* tok_pos;
  const int* slots;
};

__device__ __forceinline__ float sigmoid_exact(float g) {
  if (g >= 0.f) return 1.0f / (1.0f + expf(-g));
  float e = expf(g);
  return e / (1.0f + e);
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

// q . key over `dim` values: q float32 in shared memory, the key in the cache's type; 16-byte loads where rows allow.
__device__ __forceinline__ float dot_key(const float* q, const float* key, int dim, bool wide) {
  float s = 0.f;
  if (wide) {
    for (int d = 0; d < dim; d += 4) {
      float4 k = *reinterpret_cast<const float4*>(key + d);
      s = fmaf(q[d], k.x, s); s = fmaf(q[d + 1], k.y, s); s = fmaf(q[d + 2], k.z, s); s = fmaf(q[d + 3], k.w, s);
    }
    return s;
  }
  for (int d = 0; d < dim; ++d) s = fmaf(q[d], key[d], s);
  return s;
}
__device__ __forceinline__ float dot_key(const float* q, const __nv_bfloat16* key, int dim, bool wide) {
  float s = 0.f;
  if (wide) {
    for (int d = 0; d < dim; d += 8) {
      uint4 raw = *reinterpret_cast<const uint4*>(key + d);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(pairs[i]);
        s = fmaf(q[d + 2 * i], f.x, s);
        s = fmaf(q[d + 2 * i + 1], f.y, s);
      }
    }
    return s;
  }
  for (int d = 0; d < dim; ++d) s = fmaf(q[d], __bfloat162float(key[d]), s);
  return s;
}

// rows[t] = [ ... q (heads * dim) at q_at ... k (kv_heads * dim) at k_at ... v (kv_heads * vdim) at v_at ... ].
template <typename T>
__global__ void __launch_bounds__(256) sigmoid_prepare_kernel(
    const float* __restrict__ rows, int stride, int q_at, int k_at, int v_at, int heads,
    const float* __restrict__ q_bias, const float* __restrict__ k_bias, const float* __restrict__ v_bias,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps, T* __restrict__ q_out,
    WideKv cache, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ slots,
    int write_cache) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, dim = cache.key_dim, vdim = cache.value_dim;
  const float* row = rows + (size_t)t * stride;
  const int q_size = heads * dim, k_size = cache.kv_heads * dim, v_size = cache.kv_heads * vdim;
  {
    float inv = 1.0f;
    if (q_weight != nullptr) {
      float s = 0.f;
      for (int i = threadIdx.x; i < q_size; i += blockDim.x) {
        float x = row[q_at + i] + (q_bias != nullptr ? q_bias[i] : 0.f);
        s = fmaf(x, x, s);
      }
      inv = 1.0f / sqrtf(block_total(s, scratch) / (float)q_size + eps);
    }
    for (int i = threadIdx.x; i < q_size; i += blockDim.x) {
      float x = row[q_at + i] + (q_bias != nullptr ? q_bias[i] : 0.f);
      q_out[(size_t)t * q_size + i] = from_float<T>(q_weight != nullptr ? x * inv * q_weight[i] : x);
    }
  }
  if (!write_cache) return;
  const int pos = tok_pos[t], slot = slots[tok_seq[t]];
  const int page = cache.page_table[(size_t)slot * cache.max_pages + pos / cache.page_size];
  const int at = pos % cache.page_size;
  float inv = 1.0f;
  if (k_weight != nullptr) {
    float s = 0.f;
    for (int i = threadIdx.x; i < k_size; i += blockDim.x) {
      float x = row[k_at + i] + (k_bias != nullptr ? k_bias[i] : 0.f);
      s = fmaf(x, x, s);
    }
    inv = 1.0f / sqrtf(block_total(s, scratch) / (float)k_size + eps);
  }
  for (int i = threadIdx.x; i < k_size; i += blockDim.x) {
    float x = row[k_at + i] + (k_bias != nullptr ? k_bias[i] : 0.f);
    int g = i / dim, d = i - g * dim;
    ((T*)cache.base)[key_at(cache, page, g, at) + d] = from_float<T>(k_weight != nullptr ? x * inv * k_weight[i] : x);
  }
  for (int i = threadIdx.x; i < v_size; i += blockDim.x) {
    float x = row[v_at + i] + (v_bias != nullptr ? v_bias[i] : 0.f);
    int g = i / vdim, d = i - g * vdim;
    ((T*)cache.base)[value_at(cache, page, g, at) + d] = from_float<T>(x);
  }
}

// The tiles of TJ keys a token at `pos` walks: those that hold kept first positions, then those of its window (a tile
// that holds both counts once). Tile number `index` of the walk -> the tile's first key.
struct TileWalk {
  int kept_tiles, window_first, count;
  __device__ __forceinline__ TileWalk(int pos, int window, int keep) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    int kept_end = min(keep, lo);
    kept_tiles = (kept_end + TJ - 1) / TJ;
    window_first = max(lo / TJ, kept_tiles);
    count = kept_tiles + pos / TJ - window_first + 1;
  }
  __device__ __forceinline__ int first_key(int index) const {
    return (index < kept_tiles ? index : window_first + index - kept_tiles) * TJ;
  }
};

template <typename T>
__global__ void sigmoid_attention_kernel(SigmoidArgs a) {
  extern __shared__ float smem[];
  const int heads = a.heads, dim = a.cache.key_dim, vdim = a.cache.value_dim, group = heads / a.cache.kv_heads;
  float* q_s = smem;                       // heads * dim
  float* mix_s = q_s + heads * dim;        // heads * heads
  float* w_s = mix_s + heads * heads;      // heads * TJ
  float* mixed_s = w_s + heads * TJ;       // heads * TJ
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5, threads = blockDim.x;
  pdl_launch_dependents();
  if (a.mix != nullptr)
    for (int i = tid; i < heads * heads; i += threads) mix_s[i] = a.mix[i];
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = a.tok_pos[t], slot = a.slots[a.tok_seq[t]];
  {
    const T* src = (const T*)a.q + (size_t)t * heads * dim;
    for (int i = tid; i < heads * dim; i += threads) q_s[i] = to_float(src[i]);
  }
  const int* pages = a.cache.page_table + (size_t)slot * a.cache.max_pages;
  const bool wide = (dim * sizeof(T)) % 16 == 0;
  const int outputs = heads * vdim;
  float acc[MAX_OUT];
#pragma unroll
  for (int r = 0; r < MAX_OUT; ++r) acc[r] = 0.f;

  const TileWalk walk(pos, a.window, a.keep);
  int begin = 0, end = walk.count;
  if (a.splits > 1) {
    int per = (walk.count + a.splits - 1) / a.splits;
    begin = blockIdx.y * per;
    end = min(walk.count, begin + per);
  }
  __syncthreads();
  for (int index = begin; index < end; ++index) {
    const int j0 = walk.first_key(index);
    const int page = pages[j0 / a.cache.page_size], row0 = j0 % a.cache.page_size;
    {
      const int j = j0 + lane;
      const bool visible = j <= pos && (a.window <= 0 || pos - j < a.window || j < a.keep);
      for (int h = warp; h < heads; h += warps) {
        float w = 0.f;
        if (visible) {
          const T* key = (const T*)a.cache.base + key_at(a.cache, page, h / group, row0 + lane);
          float s = dot_key(q_s + h * dim, key, dim, wide) * a.scale;
          if (a.slopes != nullptr) s -= a.slopes[h] * (float)(pos - j);
          if (a.head_bias != nullptr) s += a.head_bias[h];
          w = sigmoid_exact(s);
        }
        w_s[h * TJ + lane] = w;
      }
    }
    __syncthreads();
    const float* use = w_s;
    if (a.mix != nullptr) {
      for (int i = tid; i < heads * TJ; i += threads) {
        int h = i / TJ, j = i - h * TJ;
        float s = 0.f;
        for (int g = 0; g < heads; ++g) s = fmaf(mix_s[h * heads + g], w_s[g * TJ + j], s);
        mixed_s[i] = s;
      }
      __syncthreads();
      use = mixed_s;
    }
    const int here = min(TJ, pos + 1 - j0);
#pragma unroll
    for (int r = 0; r < MAX_OUT; ++r) {
      int o = tid + r * threads;
      if (o < outputs) {
        int h = o / vdim, e = o - h * vdim;
        const T* value = (const T*)a.cache.base + value_at(a.cache, page, h / group, row0) + e;
        const float* wh = use + h * TJ;
        float s = acc[r];
        for (int jj = 0; jj < here; ++jj) s = fmaf(wh[jj], to_float(value[(size_t)jj * vdim]), s);
        acc[r] = s;
      }
    }
    if (a.mix == nullptr) __syncthreads();  // (with mixing, the barrier behind the next tile's scores does this)
  }
#pragma unroll
  for (int r = 0; r < MAX_OUT; ++r) {
    int o = tid + r * threads;
    if (o >= outputs) continue;
    if (a.splits > 1) {
      a.part[((size_t)blockIdx.y * a.tokens + t) * outputs + o] = acc[r];
    } else {
      float g = a.gates != nullptr ? sigmoid_exact(a.gates[(size_t)t * a.gate_ld + o]) : 1.0f;
      ((T*)a.out)[(size_t)t * outputs + o] = from_float<T>(acc[r] * g);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) sigmoid_combine_kernel(SigmoidArgs a, int outputs) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int o = blockIdx.y * blockDim.x + threadIdx.x; o < outputs; o += gridDim.y * blockDim.x) {
    float s = 0.f;
    for (int z = 0; z < a.splits; ++z) s += a.part[((size_t)z * a.tokens + t) * outputs + o];
    float g = a.gates != nullptr ? sigmoid_exact(a.gates[(size_t)t * a.gate_ld + o]) : 1.0f;
    ((T*)a.out)[(size_t)t * outputs + o] = from_float<T>(s * g);
  }
}

template <typename T>
int launch_attention(const SigmoidArgs& a, cudaStream_t stream) {
  const int outputs = a.heads * a.cache.value_dim;
  int threads = 256;
  while (threads < 1024 && threads * MAX_OUT < outputs) threads *= 2;
  if (threads * MAX_OUT < outputs) return DLLM_UNSUPPORTED_SIZE;
  size_t smem = ((size_t)a.heads * a.cache.key_dim + (size_t)a.heads * a.heads + 2 * (size_t)a.heads * TJ) * sizeof(float);
  if (smem > 200 * 1024) return DLLM_UNSUPPORTED_SIZE;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(sigmoid_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = smem;
  }
  int status = dllm_launch_pdl(sigmoid_attention_kernel<T>, dim3(a.tokens, a.splits), dim3(threads), smem, stream, a);
  if (status != DLLM_OK || a.splits == 1) return status;
  int across = (outputs + 255) / 256;
  return dllm_launch_pdl(sigmoid_combine_kernel<T>, dim3(a.tokens, across > 16 ? 16 : across), dim3(256), 0, stream,
                         a, outputs);
}

}  // namespace

DLLM_EXPORT int dllm_sigmoid_prepare(const float* rows, int stride, int q_at, int k_at, int v_at, int heads,
                                     int kv_heads, int dim, int vdim, const float* q_bias, const float* k_bias,
                                     const float* v_bias, const float* q_weight, const float* k_weight, float eps,
                                     void* q_out, void* cache_base, const int* page_table, int max_pages,
                                     int page_size, const int* tok_seq, const int* tok_pos, const int* slots,
                                     int tokens, int write_cache, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || stride <= 0 || page_size <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  if (!rows || !q_out || !cache_base || !page_table || !tok_seq || !tok_pos || !slots) return DLLM_BAD_ARGUMENT;
  WideKv cache{cache_base, page_table, max_pages, page_size, kv_heads, dim, vdim};
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(sigmoid_prepare_kernel<float>, dim3(tokens), dim3(256), 0, stream, rows, stride, q_at, k_at,
                           v_at, heads, q_bias, k_bias, v_bias, q_weight, k_weight, eps, (float*)q_out, cache, tok_seq,
                           tok_pos, slots, write_cache);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(sigmoid_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, rows, stride,
                           q_at, k_at, v_at, heads, q_bias, k_bias, v_bias, q_weight, k_weight, eps,
                           (__nv_bfloat16*)q_out, cache, tok_seq, tok_pos, slots, write_cache);
  return DLLM_BAD_ARGUMENT;
}

// out[t, o] = (sum over splits of part[split][t][o]) * sigmoid(gates[t * gate_ld + o]), rounded to `dtype`: the second
// step of an attention kernel that dealt the keys to several blocks (this library's, or the tile kernel's).
DLLM_EXPORT int dllm_sigmoid_combine(const float* part, const float* gates, int gate_ld, void* out, int tokens,
                                     int outputs, int splits, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (outputs <= 0 || splits < 1) return DLLM_UNSUPPORTED_SIZE;
  if (!part || !out) return DLLM_BAD_ARGUMENT;
  SigmoidArgs a{};
  a.part = const_cast<float*>(part);
  a.gates = gates;
  a.gate_ld = gate_ld;
  a.out = out;
  a.tokens = tokens;
  a.splits = splits;
  int across = (outputs + 255) / 256;
  dim3 grid(tokens, across > 16 ? 16 : across);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(sigmoid_combine_kernel<float>, grid, dim3(256), 0, stream, a, outputs);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(sigmoid_combine_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, a, outputs);
  return DLLM_BAD_ARGUMENT;
}

// window <= 0: every earlier position is seen. splits > 1: `part` holds splits x tokens x heads x vdim floats.
DLLM_EXPORT int dllm_sigmoid_attention(const void* q, void* out, void* cache_base, const int* page_table,
                                       int max_pages, int page_size, int heads, int kv_heads, int dim, int vdim,
                                       const float* mix, const float* slopes, const float* head_bias,
                                       const float* gates, int gate_ld, float scale, int window, int keep,
                                       const int* tok_seq, const int* tok_pos, const int* slots, int tokens,
                                       int splits, float* part, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || page_size <= 0 || page_size % TJ ||
      keep < 0 || splits < 1 || splits > 65535)
    return DLLM_UNSUPPORTED_SIZE;
  if (!q || !out || !cache_base || !page_table || !tok_seq || !tok_pos || !slots || (splits > 1 && !part))
    return DLLM_BAD_ARGUMENT;
  SigmoidArgs a{q, WideKv{cache_base, page_table, max_pages, page_size, kv_heads, dim, vdim}, mix, slopes, head_bias,
                gates, gate_ld, out, part, heads, window, keep, tokens, splits, scale, tok_seq, tok_pos, slots};
  if (dtype == DLLM_F32) return launch_attention<float>(a, stream);
  if (dtype == DLLM_BF16) return launch_attention<__nv_bfloat16>(a, stream);
  return DLLM_BAD_ARGUMENT;
}
