// The experts' products of a prompt-sized step as grouped tile products on the tensor cores (bfloat16, mma.sync
// m16n8k16). The (token, choice) pairs are first put in expert order on the device (`moe_sort`: counts, offsets, each
// pair's place; one block, no host involved, so the step's launches do not depend on what the router chose). Then
//
//   grouped<GLU>:     act[place] = glu(W_gate_up[expert] h[token of the pair at place])   (rows gathered on the way in)
//   grouped<SCATTER>: y[pair]    = W_down[expert] act[place]                              (float32, scattered by pair)
//   moe_combine:      out[token] (+)= sum over the token's choices of weight * y[pair]
//
// A block owns a tile of 128 places of ONE expert x 128 output features; it finds its expert and rows from the offsets
// (tiles past the last expert's rows return at once: the grid is sized for the worst case). Operands go through three
// cp.async stages of 64 reduction values; eight warps of 64 x 32 outputs each. A pair's result does not depend on its
// place or on its tile mates, so the arbitrary order inside an expert's list changes no bit.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 128, BN = 128, BK = 64, STAGES = 3, THREADS = 256, LDS = BK + 8;
constexpr int MAX_EXPERTS = 256;
constexpr int EPI_GLU = 0, EPI_SCATTER = 1, EPI_ACT = 2;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- pairs in expert order ------------------------------------------------------------------------------------------
// chosen[pairs] -> offsets[experts + 1] (where each expert's places begin) and place_pair[place] = pair.
// One block: counts in shared memory, a serial prefix over at most 256 experts, then every pair takes the next free
// place of its expert.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ chosen, int pairs, int experts,
                                                        int* __restrict__ offsets, int* __restrict__ place_pair) {
  __shared__ int counts[MAX_EXPERTS], cursor[MAX_EXPERTS];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&counts[chosen[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      cursor[e] = at;
      offsets[e] = at;
      at += counts[e];
    }
    offsets[experts] = at;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) place_pair[atomicAdd(&cursor[chosen[i]], 1)] = i;
}

struct GroupedArgs {
  const bf16* a;          // rows of activations
  int lda;
  const int* place_pair;  // place -> pair
  int a_by_token;         // 1: the row of a place is a[pair / top] (gathered); 0: a[place]
  int top;
  const bf16* w;          // [experts, n, k]
  int n, k, experts;
  const int* offsets;
  bf16* act;              // EPI_GLU: [places, n / 2]; EPI_ACT: [places, n]
  float* y;               // EPI_SCATTER: [pairs, n]
  float limit, alpha, shift;
  int kind;               // EPI_ACT: 1 gelu (erf), 2 gelu (tanh form), 3 the square of relu
};

__device__ __forceinline__ float plain_activation(float z, int kind) {
  if (kind == 1) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (kind == 2) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  float r = fmaxf(z, 0.f);
  return r * r;
}

template <int EPI>
__global__ void __launch_bounds__(THREADS) grouped_kernel(GroupedArgs g) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* a_s = reinterpret_cast<bf16*>(smem_raw);        // [STAGES][BM][LDS]
  bf16* b_s = a_s + STAGES * BM * LDS;                  // [STAGES][BN][LDS]
  __shared__ int src_row[BM];
  pdl_launch_dependents();
  pdl_wait();
  // which expert and which of its rows
  int id = blockIdx.x, expert = -1, m0 = 0, rows = 0;
  for (int e = 0, before = 0; e < g.experts; ++e) {
    int begin = g.offsets[e], count = g.offsets[e + 1] - begin;
    int tiles = (count + BM - 1) / BM;
    if (id < before + tiles) {
      expert = e;
      m0 = begin + (id - before) * BM;
      rows = min(BM, begin + count - m0);
      break;
    }
    before += tiles;
  }
  if (expert < 0) return;
  int n0 = blockIdx.y * BN;
  for (int r = threadIdx.x; r < BM; r += THREADS) {
    int place = m0 + min(r, rows - 1);
    src_row[r] = g.a_by_token ? g.place_pair[place] / g.top : place;
  }
  __syncthreads();
  const bf16* w = g.w + (size_t)expert * g.n * g.k;
  int k_tiles = (g.k + BK - 1) / BK;
  auto load = [&](int stage, int kt) {
    int k0 = kt * BK;
#pragma unroll
    for (int i = 0; i < BM * (BK / 8) / THREADS; ++i) {
      int idx = threadIdx.x + i * THREADS;
      int r = idx / (BK / 8), c = (idx % (BK / 8)) * 8;
      bool ok = r < rows && k0 + c < g.k;
      cp_async_16(a_s + (stage * BM + r) * LDS + c, ok ? g.a + (size_t)src_row[r] * g.lda + k0 + c : g.a, ok);
    }
#pragma unroll
    for (int i = 0; i < BN * (BK / 8) / THREADS; ++i) {
      int idx = threadIdx.x + i * THREADS;
      int r = idx / (BK / 8), c = (idx % (BK / 8)) * 8;
      bool ok = n0 + r < g.n && k0 + c < g.k;
      cp_async_16(b_s + (stage * BN + r) * LDS + c, ok ? w + (size_t)(n0 + r) * g.k + k0 + c : w, ok);
    }
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < k_tiles) load(s, s);
    cp_async_commit();
  }
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int warp_m = warp >> 2, warp_n = warp & 3;  // 2 x 4 warps of 64 x 32 outputs
  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.f;

  for (int kt = 0; kt < k_tiles; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();  // this tile has landed, and everyone is done with the stage the next load overwrites
    if (kt + STAGES - 1 < k_tiles) load((kt + STAGES - 1) % STAGES, kt + STAGES - 1);
    cp_async_commit();
    const bf16* at = a_s + (kt % STAGES) * BM * LDS;
    const bf16* bt = b_s + (kt % STAGES) * BN * LDS;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      unsigned a_frag[4][4], b_frag[2][4];
#pragma unroll
      for (int mi = 0; mi < 4; ++mi)
        ldmatrix_x4(a_frag[mi], at + (warp_m * 64 + mi * 16 + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8);
      int mat = lane >> 3;
#pragma unroll
      for (int jp = 0; jp < 2; ++jp)
        ldmatrix_x4(b_frag[jp], bt + (warp_n * 32 + jp * 16 + (mat >> 1) * 8 + (lane & 7)) * LDS + ks * 16 + (mat & 1) * 8);
#pragma unroll
      for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int nj = 0; nj < 4; ++nj)
          mma_bf16(acc[mi][nj], a_frag[mi], b_frag[nj >> 1][(nj & 1) * 2], b_frag[nj >> 1][(nj & 1) * 2 + 1]);
    }
  }
  cp_async_wait<0>();
  int gq = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 4; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      int r = warp_m * 64 + mi * 16 + gq + half * 8;
      if (r >= rows) continue;
      int place = m0 + r;
      if (EPI == EPI_GLU) {
        bf16* dst = g.act + (size_t)place * (g.n / 2);
#pragma unroll
        for (int nj = 0; nj < 4; ++nj) {
          int n = n0 + warp_n * 32 + nj * 8 + tq * 2;  // (even: gate at n, up at n + 1)
          if (n + 1 < g.n) {
            float gate = fminf(acc[mi][nj][half * 2], g.limit);
            float up = fminf(fmaxf(acc[mi][nj][half * 2 + 1], -g.limit), g.limit);
            dst[n / 2] = __float2bfloat16_rn(gate / (1.0f + expf(-g.alpha * gate)) * (up + g.shift));
          }
        }
      } else if (EPI == EPI_ACT) {
        bf16* dst = g.act + (size_t)place * g.n;
#pragma unroll
        for (int nj = 0; nj < 4; ++nj) {
          int n = n0 + warp_n * 32 + nj * 8 + tq * 2;
          float lo = plain_activation(acc[mi][nj][half * 2], g.kind), hi = plain_activation(acc[mi][nj][half * 2 + 1], g.kind);
          if (n + 1 < g.n) *reinterpret_cast<__nv_bfloat162*>(dst + n) = __floats2bfloat162_rn(lo, hi);
          else if (n < g.n) dst[n] = __float2bfloat16_rn(lo);
        }
      } else {
        float* dst = g.y + (size_t)g.place_pair[place] * g.n;
#pragma unroll
        for (int nj = 0; nj < 4; ++nj) {
          int n = n0 + warp_n * 32 + nj * 8 + tq * 2;
          if (n + 1 < g.n) *reinterpret_cast<float2*>(dst + n) = make_float2(acc[mi][nj][half * 2], acc[mi][nj][half * 2 + 1]);
          else if (n < g.n) dst[n] = acc[mi][nj][half * 2];
        }
      }
    }
}

__global__ void __launch_bounds__(256) moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y,
                                                          const float* __restrict__ weights, int width, int top,
                                                          long long total, int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i / width;
    int n = (int)(i - t * width);
    float sum = 0.f;
    for (int k = 0; k < top; ++k) sum = fmaf(weights[t * top + k], y[(t * top + k) * width + n], sum);
    out[i] = accumulate ? out[i] + sum : sum;
  }
}

template <int EPI>
int launch_grouped(const GroupedArgs& g, int pairs, cudaStream_t stream) {
  size_t smem = (size_t)STAGES * (BM + BN) * LDS * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(grouped_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  // every expert's rows in tiles of BM: at most pairs / BM + experts tiles
  dim3 grid(pairs / BM + g.experts, (g.n + BN - 1) / BN);
  return dllm_launch_pdl(grouped_kernel<EPI>, grid, dim3(THREADS), smem, stream, g);
}
}  // namespace

DLLM_EXPORT int dllm_moe_sort(const int* chosen, int pairs, int experts, int* offsets, int* place_pair,
                              cudaStream_t stream) {
  if (pairs <= 0) return DLLM_OK;
  if (experts <= 0 || experts > MAX_EXPERTS) return DLLM_UNSUPPORTED_SIZE;
  return dllm_launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, chosen, pairs, experts, offsets, place_pair);
}

// act [pairs, ff] bfloat16 in expert order = glu(W_gate_up[expert] h[token]); h [tokens, width] bfloat16.
DLLM_EXPORT int dllm_moe_grouped_up(void* act, const void* h, int width, const void* w_gate_up, int ff, int experts,
                                    int top, int tokens, const int* offsets, const int* place_pair, float limit,
                                    float alpha, float shift, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || (width & 7) || ff <= 0 || experts <= 0 || experts > MAX_EXPERTS || top <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  GroupedArgs g{(const bf16*)h, width, place_pair, 1, top, (const bf16*)w_gate_up, 2 * ff, width, experts, offsets,
                (bf16*)act, nullptr, limit, alpha, shift, 0};
  return launch_grouped<EPI_GLU>(g, tokens * top, stream);
}

// act [pairs, ff] bfloat16 in expert order = activation(W_up[expert] h[token]) for experts without a gate matrix;
// w_up [experts, ff, width]; ff even (a pair of values a store).
DLLM_EXPORT int dllm_moe_grouped_up_plain(void* act, const void* h, int width, const void* w_up, int ff, int experts,
                                          int top, int tokens, const int* offsets, const int* place_pair, int kind,
                                          cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || (width & 7) || ff <= 0 || (ff & 1) || experts <= 0 || experts > MAX_EXPERTS || top <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  if (kind < 1 || kind > 3) return DLLM_BAD_ARGUMENT;
  GroupedArgs g{(const bf16*)h, width, place_pair, 1, top, (const bf16*)w_up, ff, width, experts, offsets, (bf16*)act,
                nullptr, 0.f, 0.f, 0.f, kind};
  return launch_grouped<EPI_ACT>(g, tokens * top, stream);
}

// y [pairs, width] float32 by pair = W_down[expert] act[place]; act [pairs, ff] bfloat16 in expert order.
DLLM_EXPORT int dllm_moe_grouped_down(float* y, const void* act, int ff, const void* w_down, int width, int experts,
                                      int top, int tokens, const int* offsets, const int* place_pair,
                                      cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || (width & 1) || ff <= 0 || (ff & 7) || experts <= 0 || experts > MAX_EXPERTS || top <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  GroupedArgs g{(const bf16*)act, ff, place_pair, 0, top, (const bf16*)w_down, width, ff, experts, offsets, nullptr, y,
                0.f, 0.f, 0.f, 0};
  return launch_grouped<EPI_SCATTER>(g, tokens * top, stream);
}

DLLM_EXPORT int dllm_moe_combine(float* out, const float* y, const float* weights, int width, int top, int tokens,
                                 int accumulate, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || top <= 0) return DLLM_UNSUPPORTED_SIZE;
  long long total = (long long)tokens * width;
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return dllm_launch_pdl(moe_combine_kernel, dim3(blocks), dim3(256), 0, stream, out, y, weights, width, top, total,
                         accumulate);
}
