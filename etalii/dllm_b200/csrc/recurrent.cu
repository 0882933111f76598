// Mixers whose memory is a matrix per head instead of a list of keys: S [dim, vdim] in float32 per (sequence, head),
// carried from token to token in the cache's fixed-size state.
//
//   decayed outer products:  S <- decay_h S + k_t v_t^T;                          o_t = S^T q_t
//   gated delta rule:        S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//   gated outer products:    S <- a_t S + b_t k_t v_t^T  (a_t, b_t per token and head);   o_t = S^T q_t, and the
//                            same sum with v = 1 as one more column of S (the normaliser n_t), read out as n_t . q_t
//
// One kernel serves prompts and single tokens: a block owns 16 columns of one head's S for one sequence and walks
// that sequence's new tokens in order, from the state the cache holds to the state it leaves there. A column's
// recurrence does not involve the other columns, so columns are the parallel dimension besides heads and sequences.
// Inside a warp a lane holds `RPL` consecutive rows of one column (8 or 16 lanes a column): the sums over
// rows (S^T q, S^T k) are RPL multiply-adds a lane and three or four shuffles. The tokens' q, k and v come through two
// shared-memory stages filled by cp.async (16-byte pieces where the rows allow it), so global latency is paid once per
// 16 tokens and hidden behind the arithmetic of the stage before. Everything is float32: inputs, state, sums.
//
// State layout: [slot][head][column][row], a column's rows contiguous (a lane's rows are one or more 16-byte loads).
#include "common.cuh"

#define SCAN_COLS 16  // columns of S a block owns

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float silu_exact(float g) {
  float s;
  if (g >= 0.f) {
    s = 1.0f / (1.0f + expf(-g));
  } else {
    float e = expf(g);
    s = e / (1.0f + e);
  }
  return g * s;
}
__device__ __forceinline__ float sigmoid_exact(float g) {
  if (g >= 0.f) return 1.0f / (1.0f + expf(-g));
  float e = expf(g);
  return e / (1.0f + e);
}

struct ScanArgs {
  const float* q;        // rows of `stride` floats; a token's q of head j starts at q + token * stride + j * dim
  const float* k;
  const float* v;        // a token's v of head h starts at v + token * stride + h * vdim
  int stride;
  int heads, qk_heads;   // head h reads q/k head h / (heads / qk_heads)
  int dim, vdim;
  float* state;          // [slots][heads][vdim][dim]
  const int* cu_seqlens; // sequence s has the tokens cu_seqlens[s] .. cu_seqlens[s + 1] - 1 of the step
  const int* slots;
  float* out;            // [tokens][heads * vdim]
  int vector;            // q, k, v and their rows are 16-byte aligned and dim, vdim multiples of 4: 16-byte copies
  // decayed outer products
  const float* decay;    // [heads]
  float out_scale;       // the read-out is multiplied by this (a scale of the keys, which the sums are linear in)
  // gated delta rule: per token [g (heads) | beta (heads) | k.q (qk_heads)], `aux_stride` floats a token
  const float* aux;
  int aux_stride;
  // gated outer products: aux holds per token [a (heads) | b (heads) | -]; the state has vdim + 1 columns, the last
  // one written with v = 1, and its read-out goes to nq [tokens][heads]
  float* nq;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}

// MODE 0: decayed outer products; MODE 1: gated delta rule; MODE 2: gated outer products. TOKENS: tokens a stage. LPC lanes share a column (8 or
// 16), each with RPL rows of it: the block has 16 * LPC threads. Few lanes a column mean few shuffles and few
// instructions a token; many lanes mean more warps to hide latency behind, which is what a step with few sequences
// and heads needs (one warp per scheduler issues a dependent instruction every four cycles and no faster).
template <int RPL, int LPC, int MODE, int TOKENS, int STAGES>
__global__ void __launch_bounds__(SCAN_COLS * LPC) scan_kernel(ScanArgs a) {
  constexpr int DIMP = RPL * LPC;  // rows a stage holds per token (the head's dim rounded up)
  constexpr int CPW = 32 / LPC;    // columns a warp owns
  constexpr int SCAN_THREADS = SCAN_COLS * LPC;
  constexpr int PER_TOKEN = 2 * DIMP + SCAN_COLS + 4;
  constexpr int PIECES = PER_TOKEN / 4;  // 16-byte pieces of a token's stage row
  extern __shared__ __align__(16) float stage[];  // [STAGES][TOKENS][PER_TOKEN]: k | q | v (16 columns) | g, beta, k.q, -
  pdl_launch_dependents();
  const int head = blockIdx.y, seq = blockIdx.z, col0 = blockIdx.x * SCAN_COLS;
  const int qk_head = head / (a.heads / a.qk_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = lane / CPW, cc = lane % CPW;
  const int col = col0 + warp * CPW + cc;
  const float decay = MODE == 0 ? a.decay[head] : 0.f;
  const int state_cols = a.vdim + (MODE == 2 ? 1 : 0);
  pdl_wait();
  const int first = a.cu_seqlens[seq], count = a.cu_seqlens[seq + 1] - first;
  const int slot = a.slots[seq];
  float* my_state = a.state + (((size_t)slot * a.heads + head) * state_cols + col) * (size_t)a.dim + rg * RPL;

  float S[RPL];  // (dim is a multiple of 4 and so is a lane's first row: a piece of 4 rows is inside the head or not)
#pragma unroll
  for (int j = 0; j < RPL; j += 4) {
    float4 s4 = (col < state_cols && rg * RPL + j < a.dim) ? *reinterpret_cast<const float4*>(my_state + j)
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
    S[j] = s4.x; S[j + 1] = s4.y; S[j + 2] = s4.z; S[j + 3] = s4.w;
  }

  auto fill = [&](int chunk, int buffer) {
    float* dst = stage + (size_t)buffer * TOKENS * PER_TOKEN;
    const int t0 = chunk * TOKENS, here = min(TOKENS, count - t0);
    if (a.vector) {
      // (the chunk's first rows once, 32-bit offsets from there: the copies are most of what a token costs besides
      // its arithmetic)
      const float* k0 = a.k + (size_t)(first + t0) * a.stride + qk_head * a.dim;
      const float* q0 = a.q + (size_t)(first + t0) * a.stride + qk_head * a.dim;
      const float* v0 = a.v + (size_t)(first + t0) * a.stride + head * a.vdim + col0;
      for (int i = tid; i < here * PIECES; i += SCAN_THREADS) {
        int t = i / PIECES, e = (i - t * PIECES) * 4;
        float* to = dst + t * PER_TOKEN + e;
        int row = t * a.stride;
        const float* src = nullptr;
        if (e < DIMP) {
          if (e < a.dim) src = k0 + row + e;
        } else if (e < 2 * DIMP) {
          if (e - DIMP < a.dim) src = q0 + row + (e - DIMP);
        } else if (e < 2 * DIMP + SCAN_COLS) {
          if (col0 + e - 2 * DIMP < a.vdim) src = v0 + row + (e - 2 * DIMP);
        } else if (MODE >= 1) {
          const float* aux = a.aux + (size_t)(first + t0 + t) * a.aux_stride;
          cp_async4(to, aux + head);
          cp_async4(to + 1, aux + a.heads + head);
          cp_async4(to + 2, aux + 2 * a.heads + qk_head);
          continue;
        }
        if (src != nullptr) cp_async16(to, src);
        else *reinterpret_cast<float4*>(to) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      for (int i = tid; i < here * PER_TOKEN; i += SCAN_THREADS) {
        int t = i / PER_TOKEN, e = i - t * PER_TOKEN;
        size_t token = (size_t)(first + t0 + t);
        const float* src = nullptr;
        if (e < DIMP) {
          if (e < a.dim) src = a.k + token * a.stride + qk_head * a.dim + e;
        } else if (e < 2 * DIMP) {
          if (e - DIMP < a.dim) src = a.q + token * a.stride + qk_head * a.dim + (e - DIMP);
        } else if (e < 2 * DIMP + SCAN_COLS) {
          int c = col0 + e - 2 * DIMP;
          if (c < a.vdim) src = a.v + token * a.stride + head * a.vdim + c;
        } else if (MODE >= 1) {
          int which = e - 2 * DIMP - SCAN_COLS;
          if (which == 0) src = a.aux + token * a.aux_stride + head;
          else if (which == 1) src = a.aux + token * a.aux_stride + a.heads + head;
          else if (which == 2) src = a.aux + token * a.aux_stride + 2 * a.heads + qk_head;
        }
        if (src != nullptr) cp_async4(dst + i, src);
        else dst[i] = 0.f;
      }
    }
    cp_async_commit();
  };

  // one token of the decayed sum: the state moves on, the lane's part of S^T q comes back. Two rows an instruction
  // (the packed float32 multiply-add of sm_100: the same roundings as two single ones, half the issue slots).
  auto decayed = [&](const float* row) -> float {
    float v = row[2 * DIMP + warp * CPW + cc];
    float keep = decay;
    if (MODE == 2) {  // this token's own factors; the column behind the values is written with v = 1
      keep = row[2 * DIMP + SCAN_COLS];
      v = (col == a.vdim ? 1.0f : v) * row[2 * DIMP + SCAN_COLS + 1];
    }
    const float2 vv = make_float2(v, v), dd = make_float2(keep, keep);
    float2 p = make_float2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < RPL; j += 4) {
      float4 k4 = *reinterpret_cast<const float4*>(row + rg * RPL + j);
      float4 q4 = *reinterpret_cast<const float4*>(row + DIMP + rg * RPL + j);
      float2 s01 = __ffma2_rn(dd, make_float2(S[j], S[j + 1]), __fmul2_rn(make_float2(k4.x, k4.y), vv));
      float2 s23 = __ffma2_rn(dd, make_float2(S[j + 2], S[j + 3]), __fmul2_rn(make_float2(k4.z, k4.w), vv));
      S[j] = s01.x; S[j + 1] = s01.y; S[j + 2] = s23.x; S[j + 3] = s23.y;
      p = __ffma2_rn(s01, make_float2(q4.x, q4.y), p);
      p = __ffma2_rn(s23, make_float2(q4.z, q4.w), p);
    }
    return p.x + p.y;
  };

  const int chunks = (count + TOKENS - 1) / TOKENS;
  const int out_width = a.heads * a.vdim;
  // STAGES - 1 chunks are on their way while one is worked on (a long prompt: the rows come from L2 or memory, a
  // microsecond away, and a chunk's arithmetic is shorter than that); every round commits one group, empty or not
  for (int ahead = 0; ahead < STAGES - 1; ++ahead) {
    if (ahead < chunks) fill(ahead, ahead);
    else cp_async_commit();
  }
  for (int chunk = 0; chunk < chunks; ++chunk) {
    int buffer = chunk % STAGES;
    if (chunk + STAGES - 1 < chunks) fill(chunk + STAGES - 1, (chunk + STAGES - 1) % STAGES);
    else cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const float* base = stage + (size_t)buffer * TOKENS * PER_TOKEN;
    const int here = min(TOKENS, count - chunk * TOKENS);
    float* out = a.out + (size_t)(first + chunk * TOKENS) * out_width + head * a.vdim + col;
    const bool writes = rg == 0 && col < a.vdim;
    int t = 0;
    if (MODE == 0 || MODE == 2) {
      // The decayed sum's read-out does not feed the state, so its sum over the rows need not be finished token by
      // token: every lane leaves its part in shared memory and goes on to the next token (nothing but the state's
      // own multiply-add links two tokens); after the chunk the block adds the parts up, a thread per token and
      // column, and writes whole pieces of rows.
      float* parts = stage + (size_t)STAGES * TOKENS * PER_TOKEN;  // [TOKENS][16 columns][LPC + 4]
      constexpr int PADL = LPC + 4;
      // a group of tokens at a time: all their rows are asked of shared memory first (the loads do not depend on the
      // state), then the state walks through them
      constexpr int GROUP = RPL <= 8 ? 4 : 2;
      int u = 0;
      for (; u + GROUP <= here; u += GROUP) {
        float4 kq[GROUP][RPL / 2];
        float v[GROUP], keep[GROUP];
#pragma unroll
        for (int w = 0; w < GROUP; ++w) {
          const float* row = base + (u + w) * PER_TOKEN;
          v[w] = row[2 * DIMP + warp * CPW + cc];
          keep[w] = decay;
          if (MODE == 2) {
            keep[w] = row[2 * DIMP + SCAN_COLS];
            v[w] = (col == a.vdim ? 1.0f : v[w]) * row[2 * DIMP + SCAN_COLS + 1];
          }
#pragma unroll
          for (int j = 0; j < RPL; j += 4) {
            kq[w][j / 2] = *reinterpret_cast<const float4*>(row + rg * RPL + j);
            kq[w][j / 2 + 1] = *reinterpret_cast<const float4*>(row + DIMP + rg * RPL + j);
          }
        }
#pragma unroll
        for (int w = 0; w < GROUP; ++w) {
          const float2 vv = make_float2(v[w], v[w]), dd = make_float2(keep[w], keep[w]);
          float2 p = make_float2(0.f, 0.f);
#pragma unroll
          for (int j = 0; j < RPL; j += 4) {
            float4 k4 = kq[w][j / 2], q4 = kq[w][j / 2 + 1];
            float2 s01 = __ffma2_rn(dd, make_float2(S[j], S[j + 1]), __fmul2_rn(make_float2(k4.x, k4.y), vv));
            float2 s23 = __ffma2_rn(dd, make_float2(S[j + 2], S[j + 3]), __fmul2_rn(make_float2(k4.z, k4.w), vv));
            S[j] = s01.x; S[j + 1] = s01.y; S[j + 2] = s23.x; S[j + 3] = s23.y;
            p = __ffma2_rn(s01, make_float2(q4.x, q4.y), p);
            p = __ffma2_rn(s23, make_float2(q4.z, q4.w), p);
          }
          parts[((u + w) * SCAN_COLS + warp * CPW + cc) * PADL + rg] = p.x + p.y;
        }
      }
      for (; u < here; ++u)
        parts[(u * SCAN_COLS + warp * CPW + cc) * PADL + rg] = decayed(base + u * PER_TOKEN);
      __syncthreads();
      for (int i = tid; i < here * SCAN_COLS; i += SCAN_THREADS) {
        int u = i / SCAN_COLS, c = i % SCAN_COLS;
        const float4* mine = reinterpret_cast<const float4*>(parts + i * PADL);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < LPC / 4; ++j) {
          float4 p4 = mine[j];
          sum += (p4.x + p4.y) + (p4.z + p4.w);
        }
        if (col0 + c < a.vdim)
          a.out[(size_t)(first + chunk * TOKENS + u) * out_width + head * a.vdim + col0 + c] = sum * a.out_scale;
        else if (MODE == 2 && col0 + c == a.vdim)
          a.nq[(size_t)(first + chunk * TOKENS + u) * a.heads + head] = sum * a.out_scale;
      }
      t = here;
    }
    for (; t < here; ++t) {  // (the delta rule: its sums over the rows feed the state, token by token)
      const float* row = base + t * PER_TOKEN;
      float o;
      {
        float v = row[2 * DIMP + warp * CPW + cc];
        float g = row[2 * DIMP + SCAN_COLS], beta = row[2 * DIMP + SCAN_COLS + 1], kq = row[2 * DIMP + SCAN_COLS + 2];
        float2 kk[RPL / 2];
        float2 sk2 = make_float2(0.f, 0.f), sq2 = make_float2(0.f, 0.f);  // S^T k and S^T q before this token
#pragma unroll
        for (int j = 0; j < RPL; j += 4) {
          float4 k4 = *reinterpret_cast<const float4*>(row + rg * RPL + j);
          float4 q4 = *reinterpret_cast<const float4*>(row + DIMP + rg * RPL + j);
          kk[j / 2] = make_float2(k4.x, k4.y);
          kk[j / 2 + 1] = make_float2(k4.z, k4.w);
          float2 s01 = make_float2(S[j], S[j + 1]), s23 = make_float2(S[j + 2], S[j + 3]);
          sk2 = __ffma2_rn(s01, kk[j / 2], sk2);
          sq2 = __ffma2_rn(s01, make_float2(q4.x, q4.y), sq2);
          sk2 = __ffma2_rn(s23, kk[j / 2 + 1], sk2);
          sq2 = __ffma2_rn(s23, make_float2(q4.z, q4.w), sq2);
        }
        float sk = sk2.x + sk2.y, sq = sq2.x + sq2.y;
#pragma unroll
        for (int o2 = CPW; o2 <= 16; o2 <<= 1) {
          sk += __shfl_xor_sync(0xffffffffu, sk, o2);
          sq += __shfl_xor_sync(0xffffffffu, sq, o2);
        }
        // (g S + k u^T)^T q = g S^T q + u (k . q): the read-out of the state after the write, without a second sum
        float u = beta * (v - g * sk);
        o = fmaf(g, sq, u * kq);
        const float2 uu = make_float2(u, u), gg = make_float2(g, g);
#pragma unroll
        for (int j = 0; j < RPL; j += 2) {
          float2 next = __ffma2_rn(kk[j / 2], uu, __fmul2_rn(gg, make_float2(S[j], S[j + 1])));
          S[j] = next.x; S[j + 1] = next.y;
        }
      }
      if (writes) out[(size_t)t * out_width] = o;
    }
    __syncthreads();  // the stage is filled again in the next round
  }
#pragma unroll
  for (int j = 0; j < RPL; j += 4)
    if (col < state_cols && rg * RPL + j < a.dim)
      *reinterpret_cast<float4*>(my_state + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
}

template <int RPL, int LPC, int MODE, int TOKENS, int STAGES>
static int launch_scan_case(const ScanArgs& a, dim3 grid, cudaStream_t stream) {
  size_t bytes = (size_t)STAGES * TOKENS * (2 * RPL * LPC + SCAN_COLS + 4) * sizeof(float);
  if (MODE != 1) bytes += (size_t)TOKENS * SCAN_COLS * (LPC + 4) * sizeof(float);  // the parts of the read-out
  static bool allowed = false;  // (more than 48 KB of dynamic shared memory has to be asked for once)
  if (bytes > 48 * 1024 && !allowed) {
    if (cudaFuncSetAttribute(scan_kernel<RPL, LPC, MODE, TOKENS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)bytes) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    allowed = true;
  }
  return dllm_launch_pdl(scan_kernel<RPL, LPC, MODE, TOKENS, STAGES>, grid, dim3(SCAN_COLS * LPC), bytes, stream, a);
}

// `longest`: the most new tokens a sequence of the step has (the host knows; the kernel reads the real counts).
template <int MODE>
static int launch_scan(const ScanArgs& a, int sequences, int longest, cudaStream_t stream) {
  dim3 grid((a.vdim + (MODE == 2 ? 1 : 0) + SCAN_COLS - 1) / SCAN_COLS, a.heads, sequences);
  // Lanes a column: 8 where the step has blocks enough to give every scheduler several warps (many sequences or
  // heads), else 16, which doubles the warps (measured on one prompt of 2,048 tokens, 16 heads of 128 x 128: 477 us
  // with 8 lanes, 397 with 16, 427 with 32, whose warps each read all of k and q from shared memory again).
  long long blocks = (long long)grid.x * grid.y * grid.z;
  int dimp = a.dim <= 32 ? 32 : (a.dim <= 64 ? 64 : (a.dim <= 128 ? 128 : 256));
  int lanes = (blocks * 4 >= 148 * 16 || dimp / 16 < 4) ? 8 : 16;
  bool deep = longest > 32;  // four stages for prompts, two for steps of single tokens and short portions
#define SCAN_CASE(RPL, LPC, TOKENS)                                                                 \
  if (dimp == RPL * LPC && lanes == LPC)                                                            \
    return deep ? launch_scan_case<RPL, LPC, MODE, TOKENS, 4>(a, grid, stream)                      \
                : launch_scan_case<RPL, LPC, MODE, TOKENS, 2>(a, grid, stream);
  SCAN_CASE(4, 8, 16)
  SCAN_CASE(8, 8, 16) SCAN_CASE(4, 16, 16)
  SCAN_CASE(16, 8, 16) SCAN_CASE(8, 16, 16)
  SCAN_CASE(32, 8, 8) SCAN_CASE(16, 16, 8)
#undef SCAN_CASE
  return DLLM_UNSUPPORTED_SIZE;
}

static bool scan_sizes_ok(int heads, int qk_heads, int dim, int vdim, int stride) {
  return heads > 0 && qk_heads > 0 && heads % qk_heads == 0 && dim > 0 && dim <= 256 && dim % 4 == 0 && vdim > 0 &&
         stride > 0 && heads < 65536;
}

static int scan_vector(const float* q, const float* k, const float* v, int stride, int dim, int vdim) {
  return (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0 && stride % 4 == 0 && dim % 4 == 0 && vdim % 4 == 0;
}

// Decayed outer products over the new tokens of every sequence of the step. q, k, v: pointers to the first token's
// first head inside rows of `stride` floats (float32). Head h decays by decay[h] per token. The keys count k_scale
// times: the sums are linear in them, so the state holds the unscaled sum and the read-out is multiplied instead.
DLLM_EXPORT int dllm_decay_scan(const float* q, const float* k, const float* v, int stride, int heads, int dim,
                                int vdim, const float* decay, float k_scale, float* state,
                                const int* cu_seqlens, const int* slots, int sequences, int longest, float* out,
                                cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (!scan_sizes_ok(heads, heads, dim, vdim, stride) || sequences >= 65536) return DLLM_UNSUPPORTED_SIZE;
  if (!q || !k || !v || !decay || !state || !cu_seqlens || !slots || !out) return DLLM_BAD_ARGUMENT;
  ScanArgs a = {};
  a.q = q; a.k = k; a.v = v; a.stride = stride; a.heads = heads; a.qk_heads = heads; a.dim = dim; a.vdim = vdim;
  a.state = state; a.cu_seqlens = cu_seqlens; a.slots = slots; a.out = out; a.decay = decay;
  a.out_scale = k_scale; a.vector = scan_vector(q, k, v, stride, dim, vdim);
  return launch_scan<0>(a, sequences, longest, stream);
}

// The gated delta rule over the new tokens of every sequence. q and k are unit vectors (q scaled) per q/k head, v
// the values per head, all float32 in rows of `stride` floats; aux holds per token the heads' decays g, the heads'
// step sizes beta and the q/k heads' k.q (see `dllm_delta_prepare`).
DLLM_EXPORT int dllm_delta_scan(const float* q, const float* k, const float* v, int stride, int heads, int qk_heads,
                                int dim, int vdim, const float* aux, int aux_stride, float* state,
                                const int* cu_seqlens, const int* slots, int sequences, int longest, float* out,
                                cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (!scan_sizes_ok(heads, qk_heads, dim, vdim, stride) || sequences >= 65536) return DLLM_UNSUPPORTED_SIZE;
  if (!q || !k || !v || !aux || !state || !cu_seqlens || !slots || !out) return DLLM_BAD_ARGUMENT;
  ScanArgs a = {};
  a.q = q; a.k = k; a.v = v; a.stride = stride; a.heads = heads; a.qk_heads = qk_heads; a.dim = dim; a.vdim = vdim;
  a.state = state; a.cu_seqlens = cu_seqlens; a.slots = slots; a.out = out; a.aux = aux; a.aux_stride = aux_stride;
  a.out_scale = 1.0f; a.vector = scan_vector(q, k, v, stride, dim, vdim);
  return launch_scan<1>(a, sequences, longest, stream);
}

// Gated outer products over the new tokens of every sequence: S <- a_t S + b_t k_t v_t^T per head, out = S^T q times
// q_scale, and the same recurrence with v = 1 in one more column of the state, whose read-out n_t . q_t (times
// q_scale) goes to nq [tokens][heads]. aux [tokens][aux_stride] holds a (heads) then b (heads). state [slots][heads]
// [vdim + 1][dim].
DLLM_EXPORT int dllm_gated_scan(const float* q, const float* k, const float* v, int stride, int heads, int dim, int vdim,
                                const float* aux, int aux_stride, float q_scale, float* state, const int* cu_seqlens,
                                const int* slots, int sequences, int longest, float* out, float* nq,
                                cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (!scan_sizes_ok(heads, heads, dim, vdim, stride) || sequences >= 65536 || aux_stride < 3 * heads)
    return DLLM_UNSUPPORTED_SIZE;
  if (!q || !k || !v || !aux || !state || !cu_seqlens || !slots || !out || !nq) return DLLM_BAD_ARGUMENT;
  ScanArgs a = {};
  a.q = q; a.k = k; a.v = v; a.stride = stride; a.heads = heads; a.qk_heads = heads; a.dim = dim; a.vdim = vdim;
  a.state = state; a.cu_seqlens = cu_seqlens; a.slots = slots; a.out = out; a.aux = aux; a.aux_stride = aux_stride;
  a.nq = nq; a.out_scale = q_scale; a.vector = scan_vector(q, k, v, stride, dim, vdim);
  return launch_scan<2>(a, sequences, longest, stream);
}

// ---- the gates of the gated outer products under a running maximum ------------------------------------------------
// Per token and head, from pre-activations zi, zf (float32 columns of the projected rows) and biases: the log input
// gate i = cap tanh((zi + bi) / cap) and the log forget gate f = logsigmoid(cap tanh((zf + bf) / cap)); with the running
// maximum m' = max(f + m, i) (m carried per sequence and head in `m_state` [slots][heads], zero at a sequence's start):
// aux[t] = [ a = exp(f + m - m') | b = exp(i - m') | e = exp(-m') ], each `heads` wide. A warp per (sequence, head) walks
// the step's tokens 32 at a time: the map m -> max(m + F, I) of a token composes associatively, (F1, I1) then (F2, I2)
// giving (F1 + F2, max(I1 + F2, I2)), so a chunk is a prefix scan over the lanes.
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void __launch_bounds__(128) running_max_gates_kernel(
    const float* __restrict__ zi, const float* __restrict__ zf, int stride, const float* __restrict__ bi,
    const float* __restrict__ bf, float cap, float* __restrict__ m_state, const int* __restrict__ cu_seqlens,
    const int* __restrict__ slots, int sequences, int heads, float* __restrict__ aux, int aux_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= (long long)sequences * heads) return;
  const int seq = (int)(unit / heads), head = (int)(unit - (long long)seq * heads);
  const int first = cu_seqlens[seq], count = cu_seqlens[seq + 1] - first;
  float* kept = m_state + (size_t)slots[seq] * heads + head;
  float m = *kept;
  const float add_i = bi != nullptr ? bi[head] : 0.f, add_f = bf != nullptr ? bf[head] : 0.f;
  for (int t0 = 0; t0 < count; t0 += 32) {
    const int t = t0 + lane;
    float gi = -INFINITY, gf = 0.f;  // (a lane beyond the end is the identity map)
    if (t < count) {
      gi = cap * tanhf((zi[(size_t)(first + t) * stride + head] + add_i) / cap);
      gf = log_sigmoid(cap * tanhf((zf[(size_t)(first + t) * stride + head] + add_f) / cap));
    }
    float F = gf, I = gi;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {  // the maps of the lanes before, composed with this one
      float pf = __shfl_up_sync(0xffffffffu, F, o), pi = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) { I = fmaxf(pi + F, I); F = pf + F; }
    }
    float mine = fmaxf(m + F, I);
    float before = __shfl_up_sync(0xffffffffu, mine, 1);
    if (lane == 0) before = m;
    if (t < count) {
      float* dst = aux + (size_t)(first + t) * aux_stride + head;
      dst[0] = expf(gf + before - mine);
      dst[heads] = expf(gi - mine);
      dst[2 * heads] = expf(-mine);
    }
    m = __shfl_sync(0xffffffffu, mine, min(31, count - 1 - t0));
  }
  if (lane == 0) *kept = m;
}

DLLM_EXPORT int dllm_running_max_gates(const float* zi, const float* zf, int stride, const float* bi, const float* bf,
                                       float cap, float* m_state, const int* cu_seqlens, const int* slots,
                                       int sequences, int heads, float* aux, int aux_stride, cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (heads <= 0 || stride <= 0 || aux_stride < 3 * heads || !(cap > 0.f)) return DLLM_UNSUPPORTED_SIZE;
  if (!zi || !zf || !m_state || !cu_seqlens || !slots || !aux) return DLLM_BAD_ARGUMENT;
  long long units = (long long)sequences * heads;
  return dllm_launch_pdl(running_max_gates_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream, zi, zf,
                         stride, bi, bf, cap, m_state, cu_seqlens, slots, sequences, heads, aux, aux_stride);
}

// The read-out of the gated outer products: x [tokens, heads * vdim] is divided per head by max(|nq|, floor) + 1e-6
// (nq [tokens][heads]; floor = the e of `aux`), then by its root mean square over the head (eps), times weight
// [heads * vdim] if given, times sigmoid(z) with z the token's gate pre-activations; rounded once to the output type.
template <typename T>
__global__ void __launch_bounds__(128) normalised_readout_kernel(
    T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ nq, const float* __restrict__ floor_,
    int floor_stride, const float* __restrict__ weight, const float* __restrict__ gate, int gate_stride, int tokens,
    int heads, int vdim, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= (long long)tokens * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit - (long long)t * heads);
  const float* row = x + ((size_t)t * heads + h) * vdim;
  float below = fmaxf(fabsf(nq[(size_t)t * heads + h]), floor_[(size_t)t * floor_stride + h]) + 1e-6f;
  float inv_below = 1.0f / below;
  float ss = 0.f;
  for (int i = lane; i < vdim; i += 32) {
    float v = row[i] * inv_below;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  float inv = inv_below / sqrtf(ss / (float)vdim + eps);
  const float* z = gate + (size_t)t * gate_stride + h * vdim;
  for (int i = lane; i < vdim; i += 32) {
    float value = row[i] * inv;
    if (weight != nullptr) value *= weight[h * vdim + i];
    out[((size_t)t * heads + h) * vdim + i] = from_float<T>(value * sigmoid_exact(z[i]));
  }
}

DLLM_EXPORT int dllm_normalised_readout(void* out, const float* x, const float* nq, const float* floor_,
                                        int floor_stride, const float* weight, const float* gate, int gate_stride,
                                        int tokens, int heads, int vdim, float eps, int out_dtype,
                                        cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || vdim <= 0) return DLLM_UNSUPPORTED_SIZE;
  if (!out || !x || !nq || !floor_ || !gate) return DLLM_BAD_ARGUMENT;
  long long units = (long long)tokens * heads;
  dim3 grid((unsigned)((units + 3) / 4));
  if (out_dtype == DLLM_F32)
    return dllm_launch_pdl(normalised_readout_kernel<float>, grid, dim3(128), 0, stream, (float*)out, x, nq, floor_,
                           floor_stride, weight, gate, gate_stride, tokens, heads, vdim, eps);
  if (out_dtype == DLLM_BF16)
    return dllm_launch_pdl(normalised_readout_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (__nv_bfloat16*)out,
                           x, nq, floor_, floor_stride, weight, gate, gate_stride, tokens, heads, vdim, eps);
  return DLLM_BAD_ARGUMENT;
}

// ---- what the delta rule needs of a token before its scan --------------------------------------------------------
// proj[t] = [q (qk_heads x dim) | k (qk_heads x dim) | v (heads x vdim) | ... | b (heads) | a (heads)] float32, the
// first `channels` = 2 qk_heads dim + heads vdim of them pass a causal convolution over time per channel
// (taps[channel][j], the last column multiplying the token itself; inputs before the step come from
// conv_state[slot][taps - 1][channels], zeros before the sequence's start) and silu; q and k are then divided by
// sqrt(sum of squares + 1e-6) per head, q also multiplied by dim^(-1/2). Written: prepared[t][channels] and
// aux[t] = [g (heads) | beta (heads) | k.q (qk_heads)] with beta = sigmoid(b), g = exp(-exp(A_log) softplus(a +
// dt_bias)). In a step of single tokens (`single` != 0) the block also moves the convolution's history on.
#define DELTA_MAX_TAPS 16

struct DeltaPrepareArgs {
  const float* proj; int stride; int b_off, a_off;
  const float* taps; int n_taps;
  const float* a_log; const float* dt_bias;
  float* conv_state;
  const int* tok_seq; const int* cu_seqlens; const int* slots;
  int heads, qk_heads, dim, vdim;
  float* prepared; float* aux;
  int single;
};

// A block serves one token and one unit of its channels: q/k head j (both vectors: their norms and their product), or
// the values of head h with that head's decay and step size. A thread owns the channels it convolves.
__device__ __forceinline__ float delta_channel(const DeltaPrepareArgs& a, const float* row, float* kept, int channels,
                                               int local, int ch) {
  const int history = a.n_taps - 1;
  float x[DELTA_MAX_TAPS];
  for (int j = 0; j < a.n_taps; ++j) {
    int back = history - j;  // how many tokens before this one
    x[j] = back <= local ? row[ch - (ptrdiff_t)back * a.stride]
                         : kept[(size_t)(history - (back - local)) * channels + ch];
  }
  float sum = 0.f;
  for (int j = 0; j < a.n_taps; ++j) sum = fmaf(a.taps[(size_t)ch * a.n_taps + j], x[j], sum);
  if (a.single)  // the history moves on by this token: this thread alone reads and writes the channel
    for (int j = 0; j < history; ++j) kept[(size_t)j * channels + ch] = x[j + 1];
  return silu_exact(sum);
}

__global__ void __launch_bounds__(128) delta_prepare_kernel(DeltaPrepareArgs a) {
  __shared__ float values[2 * 256];  // q | k of one head (dim at most 256)
  __shared__ float scale[2];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, unit = blockIdx.y;
  const int seq = a.tok_seq[t], local = t - a.cu_seqlens[seq], slot = a.slots[seq];
  const int qk = a.qk_heads * a.dim, channels = 2 * qk + a.heads * a.vdim, history = a.n_taps - 1;
  const float* row = a.proj + (size_t)t * a.stride;
  float* kept = a.conv_state + (size_t)slot * history * channels;
  float* prepared = a.prepared + (size_t)t * channels;
  float* aux = a.aux + (size_t)t * (2 * a.heads + a.qk_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (unit >= a.qk_heads) {  // the values of one head, and the head's decay and step size
    const int h = unit - a.qk_heads;
    for (int i = threadIdx.x; i < a.vdim; i += blockDim.x) {
      int ch = 2 * qk + h * a.vdim + i;
      prepared[ch] = delta_channel(a, row, kept, channels, local, ch);
    }
    if (threadIdx.x == 0) {
      float z = row[a.a_off + h] + a.dt_bias[h];
      float softplus = z > 20.f ? z : log1pf(expf(z));
      aux[h] = expf(-expf(a.a_log[h]) * softplus);
      aux[a.heads + h] = sigmoid_exact(row[a.b_off + h]);
    }
    return;
  }
  for (int i = threadIdx.x; i < 2 * a.dim; i += blockDim.x) {
    int ch = i < a.dim ? unit * a.dim + i : qk + unit * a.dim + (i - a.dim);
    values[i] = delta_channel(a, row, kept, channels, local, ch);
  }
  __syncthreads();
  if (warp < 2) {  // warp 0: q, warp 1: k
    const float* p = values + warp * a.dim;
    float ss = 0.f;
    for (int i = lane; i < a.dim; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + 1e-6f);
    if (warp == 0) inv *= 1.0f / sqrtf((float)a.dim);
    if (lane == 0) scale[warp] = inv;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * a.dim; i += blockDim.x) {
    float value = values[i] * scale[i < a.dim ? 0 : 1];
    values[i] = value;
    prepared[i < a.dim ? unit * a.dim + i : qk + unit * a.dim + (i - a.dim)] = value;
  }
  __syncthreads();
  if (warp == 0) {
    float dot = 0.f;
    for (int i = lane; i < a.dim; i += 32) dot = fmaf(values[i], values[a.dim + i], dot);
    dot = warp_sum(dot);
    if (lane == 0) aux[2 * a.heads + unit] = dot;
  }
}

// The convolution's history after a step of any lengths: the last taps - 1 inputs of each sequence, from the step's
// rows where it has that many and from the old history before them. A thread owns a channel: it reads all it
// needs before it writes.
__global__ void __launch_bounds__(256) delta_history_kernel(DeltaPrepareArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, first = a.cu_seqlens[seq], count = a.cu_seqlens[seq + 1] - first, slot = a.slots[seq];
  const int channels = 2 * a.qk_heads * a.dim + a.heads * a.vdim, history = a.n_taps - 1;
  float* kept = a.conv_state + (size_t)slot * history * channels;
  for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
    float x[DELTA_MAX_TAPS];
    for (int r = 0; r < history; ++r) {
      int at = count - history + r;  // index among the step's tokens of this sequence
      x[r] = at >= 0 ? a.proj[(size_t)(first + at) * a.stride + ch] : kept[(size_t)(r + count) * channels + ch];
    }
    for (int r = 0; r < history; ++r) kept[(size_t)r * channels + ch] = x[r];
  }
}

DLLM_EXPORT int dllm_delta_prepare(const float* proj, int stride, int b_off, int a_off, const float* taps, int n_taps,
                                   const float* a_log, const float* dt_bias, float* conv_state, const int* tok_seq,
                                   const int* cu_seqlens, const int* slots, int tokens, int sequences, int heads,
                                   int qk_heads, int dim, int vdim, float* prepared, float* aux, int single,
                                   cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (n_taps < 1 || n_taps > DELTA_MAX_TAPS || !scan_sizes_ok(heads, qk_heads, dim, vdim, stride))
    return DLLM_UNSUPPORTED_SIZE;
  size_t channels = 2 * (size_t)qk_heads * dim + (size_t)heads * vdim;
  if (qk_heads + heads >= 65536) return DLLM_UNSUPPORTED_SIZE;
  if (!proj || !taps || !a_log || !dt_bias || !tok_seq || !cu_seqlens || !slots || !prepared || !aux ||
      (n_taps > 1 && !conv_state))
    return DLLM_BAD_ARGUMENT;
  DeltaPrepareArgs a = {proj, stride, b_off, a_off, taps, n_taps, a_log, dt_bias, conv_state, tok_seq, cu_seqlens,
                        slots, heads, qk_heads, dim, vdim, prepared, aux, single};
  int status = dllm_launch_pdl(delta_prepare_kernel, dim3(tokens, qk_heads + heads), dim3(128), 0, stream, a);
  if (status != DLLM_OK || single || n_taps == 1) return status;
  int across = (int)((channels + 255) / 256);
  return dllm_launch_pdl(delta_history_kernel, dim3(sequences, across), dim3(256), 0, stream, a);
}

// ---- read-out: norm, weight and gate ----------------------------------------------------------------------------
// x [tokens, width] float32 is normed in groups of `group` values (a head's vdim, or the whole width): divided by
// sqrt(mean square + eps), times weight[i % group] if a weight is given, times gate(z) with z the token's gate
// pre-activations (rows of `gate_stride` floats; gate 1: silu, 2: sigmoid), rounded once to the output type.
template <typename T>
__device__ __forceinline__ void gated_store(T* dst, const float* row, const float* weight, const float* z, int i,
                                            int group, float inv, int gate_kind) {
  float value = row[i] * inv;
  if (weight != nullptr) value *= weight[i % group];
  value *= gate_kind == 1 ? silu_exact(z[i]) : sigmoid_exact(z[i]);
  dst[i] = from_float<T>(value);
}

// groups narrower than the row (a head's values): a warp per token and group
template <typename T>
__global__ void __launch_bounds__(128) gated_norm_groups_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                                const float* __restrict__ weight,
                                                                const float* __restrict__ gate, int gate_stride,
                                                                int tokens, int width, int group, float eps,
                                                                int gate_kind) {
  pdl_launch_dependents();
  pdl_wait();
  const int groups = width / group, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= (long long)tokens * groups) return;
  const int t = (int)(unit / groups), g = (int)(unit - (long long)t * groups);
  const float* row = x + (size_t)t * width;
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) ss = fmaf(row[g * group + i], row[g * group + i], ss);
  ss = warp_sum(ss);
  float inv = 1.0f / sqrtf(ss / (float)group + eps);
  for (int i = lane; i < group; i += 32)
    gated_store<T>(out + (size_t)t * width, row, weight, gate + (size_t)t * gate_stride, g * group + i, group, inv,
                   gate_kind);
}

// one group over the whole row: a block per token
template <typename T>
__global__ void __launch_bounds__(512) gated_norm_row_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                             const float* __restrict__ weight,
                                                             const float* __restrict__ gate, int gate_stride,
                                                             int width, float eps, int gate_kind) {
  __shared__ float scratch[16];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const float* row = x + (size_t)t * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  ss = warp_sum(ss);
  if (lane == 0) scratch[warp] = ss;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < warps; ++w) total += scratch[w];
  float inv = 1.0f / sqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    gated_store<T>(out + (size_t)t * width, row, weight, gate + (size_t)t * gate_stride, i, width, inv, gate_kind);
}

template <typename T>
static int launch_gated_norm(T* out, const float* x, const float* weight, const float* gate, int gate_stride,
                             int tokens, int width, int group, float eps, int gate_kind, cudaStream_t stream) {
  if (group == width) {
    int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    return dllm_launch_pdl(gated_norm_row_kernel<T>, dim3(tokens), dim3(threads), 0, stream, out, x, weight, gate,
                           gate_stride, width, eps, gate_kind);
  }
  long long units = (long long)tokens * (width / group);
  return dllm_launch_pdl(gated_norm_groups_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream, out, x,
                         weight, gate, gate_stride, tokens, width, group, eps, gate_kind);
}

DLLM_EXPORT int dllm_gated_norm(void* out, const float* x, const float* weight, const float* gate, int gate_stride,
                                int tokens, int width, int group, float eps, int gate_kind, int out_dtype,
                                cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || group <= 0 || width % group || (gate_kind != 1 && gate_kind != 2)) return DLLM_UNSUPPORTED_SIZE;
  if (!out || !x || !gate) return DLLM_BAD_ARGUMENT;
  if (out_dtype == DLLM_F32)
    return launch_gated_norm((float*)out, x, weight, gate, gate_stride, tokens, width, group, eps, gate_kind, stream);
  if (out_dtype == DLLM_BF16)
    return launch_gated_norm((__nv_bfloat16*)out, x, weight, gate, gate_stride, tokens, width, group, eps, gate_kind,
                             stream);
  return DLLM_BAD_ARGUMENT;
}

// ---- silu in place on the first `columns` values of every row (q, k and v of a mixer whose inputs are activated) ---
__global__ void silu_columns_kernel(float* __restrict__ rows, long long total, int columns, int stride) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i / columns;
    float* at = rows + r * stride + (i - r * columns);
    *at = silu_exact(*at);
  }
}

// (columns and stride multiples of 4: 16 bytes a thread)
__global__ void silu_columns_vector_kernel(float* __restrict__ rows, long long quads, int columns, int stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = columns >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < quads;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i / per_row;
    float4* at = reinterpret_cast<float4*>(rows + r * stride + 4 * (i - r * per_row));
    float4 v = *at;
    *at = make_float4(silu_exact(v.x), silu_exact(v.y), silu_exact(v.z), silu_exact(v.w));
  }
}

DLLM_EXPORT int dllm_silu_columns(float* rows, int n_rows, int columns, int stride, cudaStream_t stream) {
  if (n_rows <= 0 || columns <= 0) return DLLM_OK;
  if (rows == nullptr || stride < columns) return DLLM_BAD_ARGUMENT;
  long long total = (long long)n_rows * columns;
  if ((columns & 3) == 0 && (stride & 3) == 0 && ((uintptr_t)rows & 15) == 0) {
    long long quads = total / 4;
    int blocks = (int)((quads + 255) / 256 < 148 * 16 ? (quads + 255) / 256 : 148 * 16);
    return dllm_launch_pdl(silu_columns_vector_kernel, dim3(blocks), dim3(256), 0, stream, rows, quads, columns, stride);
  }
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return dllm_launch_pdl(silu_columns_kernel, dim3(blocks), dim3(256), 0, stream, rows, total, columns, stride);
}
