// Attention over a latent cache on the tensor cores (bfloat16 operands, mma.sync m16n8k16, float32 accumulators),
// for prompt-sized steps and single tokens alike. A position's cache row [ c (rank) | r (rot) ] serves every head, as
// key (all of it) and as value (its first `rank` places), so the heads of a token are just more query rows over the
// same keys: a sequence's new (token, head) pairs, token-major, form one tall query matrix [pairs, rank + rot], and a
// block takes 64 consecutive rows of it. Row p belongs to token p / heads at position pos, sees keys 0 .. pos. The
// block walks the sequence's cache in tiles of 32 positions (cp.async, two stages), each warp holds 16 rows: scores
// S = Q K^T, an online softmax in float32 (running maximum and sum per row, weights rounded to bfloat16 only as the
// operand of the second product), O += P C with the key tile's first `rank` columns as the values.
//
// The queries arrive as float32 rows [rank + rot] per pair in the latent's coordinates, scale included; with a table
// the last `rot` places are still unrotated and are rotated here (halves) on the way into shared memory. The output is
// the weighted sum of c per pair: float32, or multiplied by the pair's gate sigmoid(z) and rounded to bfloat16 (the
// operand of a product over all heads' sums).
//
// Few rows over a long context (single tokens) would leave most multiprocessors idle: with `splits` > 1 the key tiles of
// a sequence are dealt to that many blocks, each leaves its rows' unnormalised sums with their maximum and total in
// scratch, and `latent_combine` merges them (and applies gate and rounding).
//
// rank: a multiple of 8, at most 256 (a warp keeps 16 x rank sums in registers; instantiated for 64, 128, 256).
// rank + rot: a multiple of 8 (cache rows are copied in 16-byte pieces). page_size: a multiple of 32.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 64, BN = 32, WARPS = 4, THREADS = WARPS * 32;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

struct TiledArgs {
  const float* q;      // [tokens, heads, rank + rot] float32
  const float* table;  // [positions, rot / 2, (cos, sin)], or null: the rotated part arrives rotated
  const float* gates;  // gates[token * gate_ld + head], or null
  const float* sinks;  // sinks[head]: a score without key or value that counts once in the denominator, or null
  int gate_ld;
  void* out;           // [tokens, heads, rank]: float32, or bfloat16 with out_bf16
  int out_bf16;
  const bf16* cache;   // [page][row][rank + rot]
  const int* page_table;
  int max_pages, page_size;
  const int* cu_seqlens;
  const int* tok_pos;
  const int* slots;
  int heads, rank, rot, ld;  // ld: elements of a shared-memory row
  int splits;                // blocks that share a sequence's keys (blockIdx.z)
  float* part_o;             // splits > 1: [pair][split][rank] unnormalised sums
  float* part_ml;            // splits > 1: [pair][split][2] maximum (in units of log2 e) and total
};

template <int RANK>
__global__ void __launch_bounds__(THREADS) latent_tiled_kernel(TiledArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ld = a.ld, width = a.rank + a.rot, heads = a.heads;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [BM][ld]
  bf16* k_s = q_s + (size_t)BM * ld;              // [2][BN][ld]
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const int tok0 = a.cu_seqlens[b], n_new = a.cu_seqlens[b + 1] - tok0;
  const long long pairs = (long long)n_new * heads;
  // (the last rows of a sequence see the most keys: they go first, so that the longest blocks do not end the kernel)
  const long long p0 = (long long)(gridDim.x - 1 - blockIdx.x) * BM;
  if (p0 >= pairs) return;
  const int rows = (int)min((long long)BM, pairs - p0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int first_pos = a.tok_pos[tok0];  // positions of a sequence's new tokens are consecutive

  // the places of a shared-memory row behind rank + rot are zeros in queries and keys (nothing else writes them);
  // rows beyond the tile's own keep what they hold: their scores are masked, their sums never stored
  {
    const int pad = ld - width;
    for (int i = tid; i < (BM + 2 * BN) * pad; i += THREADS)
      q_s[(size_t)(i / pad) * ld + width + i % pad] = __float2bfloat16_rn(0.f);
  }

  const int* pages = a.page_table + (size_t)a.slots[b] * a.max_pages;
  const int pieces = width >> 3;
  auto load_keys = [&](int stage, int kt) {
    int at = kt * BN;
    const bf16* src = a.cache + ((size_t)pages[at / a.page_size] * a.page_size + at % a.page_size) * width;
    bf16* dst = k_s + (size_t)stage * BN * ld;
    for (int idx = tid; idx < BN * pieces; idx += THREADS) {
      int r = idx / pieces, c = idx - r * pieces;
      cp_async_16(dst + (size_t)r * ld + c * 8, src + (size_t)r * width + c * 8);
    }
  };
  const int last_pos = first_pos + (int)((p0 + rows - 1) / heads);
  int kt_begin = 0, kt_end = last_pos / BN;
  if (a.splits > 1) {
    int per = (kt_end + a.splits) / a.splits;  // ceil((kt_end + 1) / splits)
    kt_begin = blockIdx.z * per;
    kt_end = min(kt_end, kt_begin + per - 1);
    if (kt_begin > kt_end) {  // nothing left for this block: its rows count for nothing
      for (int i = tid; i < rows; i += THREADS) {
        float* ml = a.part_ml + (((size_t)tok0 * heads + p0 + i) * a.splits + blockIdx.z) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
      return;
    }
  }
  load_keys(0, kt_begin);
  cp_async_commit();

  // the queries, rotated where that is still to do, as bfloat16 (four places a thread: rank and rot are even, rank +
  // rot a multiple of 8)
  {
    const float* src = a.q + ((size_t)tok0 * heads + p0) * width;
    const int half = a.rot >> 1, rank = a.rank, quads = width >> 2;
    for (int idx = tid; idx < rows * quads; idx += THREADS) {
      int r = idx / quads, c = (idx - r * quads) * 4;
      const float* at = src + (size_t)r * width + c;
      float4 v4 = *reinterpret_cast<const float4*>(at);
      float v[4] = {v4.x, v4.y, v4.z, v4.w};
      if (a.table != nullptr && c + 3 >= rank) {
        int pos = first_pos + (int)((p0 + r) / heads);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int i = c + e - rank;
          if (i < 0) continue;
          int pair = i < half ? i : i - half;
          const float* cs = a.table + ((size_t)pos * half + pair) * 2;
          float other = at[e + (i < half ? half : -half)];
          v[e] = i < half ? v[e] * cs[0] - other * cs[1] : v[e] * cs[0] + other * cs[1];
        }
      }
      *reinterpret_cast<uint2*>(q_s + (size_t)r * ld + c) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
    }
  }

  float o_acc[RANK / 8][4];
#pragma unroll
  for (int i = 0; i < RANK / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int gq = lane >> 2, tq = lane & 3, mat = lane >> 3;
  int row_pos[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int r = warp * 16 + gq + 8 * i;
    row_pos[i] = r < rows ? first_pos + (int)((p0 + r) / heads) : -1;  // (a row beyond the tile sees nothing)
  }
  if (a.sinks != nullptr && kt_begin == 0) {
    // the walk over the keys starts from the sink: running maximum = the sink, running sum = its own weight, 1 (the
    // sum is kept in four parts a row that meet at the end: the first takes it); with the keys dealt to several
    // blocks, the block of the first keys has it
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int r = warp * 16 + gq + 8 * i;
      if (r < rows) {
        m_run[i] = a.sinks[(int)((p0 + r) % heads)] * LOG2E;
        l_run[i] = tq == 0 ? 1.0f : 0.f;
      }
    }
  }
  const int warp_rows = min(16, rows - warp * 16);  // <= 0: the warp has no row
  const int warp_first_pos = warp_rows > 0 ? first_pos + (int)((p0 + warp * 16) / heads) : -1;
  const int warp_last_pos = warp_rows > 0 ? first_pos + (int)((p0 + warp * 16 + warp_rows - 1) / heads) : -1;
  const int k_steps = (width + 15) >> 4;

  for (int kt = kt_begin; kt <= kt_end; ++kt) {
    const int stage = (kt - kt_begin) & 1;
    if (kt + 1 <= kt_end) load_keys(stage ^ 1, kt + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();  // (also: the queries are in shared memory)
    const int key0 = kt * BN;
    if (key0 <= warp_last_pos) {
      const bf16* kb = k_s + (size_t)stage * BN * ld;
      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) s[j][r] = 0.f;
#pragma unroll 2
      for (int ks = 0; ks < k_steps; ++ks) {
        unsigned qf[4];
        ldmatrix_x4(qf, q_s + (size_t)(warp * 16 + (lane & 15)) * ld + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int jp = 0; jp < BN / 16; ++jp) {
          unsigned bfr[4];
          ldmatrix_x4(bfr, kb + (size_t)(jp * 16 + (mat >> 1) * 8 + (lane & 7)) * ld + ks * 16 + (mat & 1) * 8);
          mma_bf16(s[2 * jp], qf, bfr[0], bfr[1]);
          mma_bf16(s[2 * jp + 1], qf, bfr[2], bfr[3]);
        }
      }
      const bool need_mask = key0 + BN - 1 > warp_first_pos || warp_rows < 16;
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float v = s[j][r] * LOG2E;
          if (need_mask && key0 + j * 8 + tq * 2 + (r & 1) > row_pos[r >> 1]) v = -INFINITY;
          s[j][r] = v;
        }
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[j][r]);
      float corr[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
        tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
        float m_new = fmaxf(m_run[i], tile_max[i]);
        float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen nothing yet
        corr[i] = fast_exp2(m_run[i] - m_use);
        m_run[i] = m_new;
        tile_max[i] = m_use;
      }
      float row_sum[2] = {0.f, 0.f};
      unsigned p_frag[BN / 16][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
        float p0f = fast_exp2(s[j][0] - tile_max[0]), p1f = fast_exp2(s[j][1] - tile_max[0]);
        float p2f = fast_exp2(s[j][2] - tile_max[1]), p3f = fast_exp2(s[j][3] - tile_max[1]);
        row_sum[0] += p0f + p1f;
        row_sum[1] += p2f + p3f;
        p_frag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0f, p1f);
        p_frag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2f, p3f);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + row_sum[i];
#pragma unroll
      for (int i = 0; i < RANK / 8; ++i) {
        o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
        o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
      }
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < RANK / 16; ++np) {
          unsigned bfr[4];
          ldmatrix_x4_trans(bfr, kb + (size_t)(kk * 16 + (mat & 1) * 8 + (lane & 7)) * ld + np * 16 + (mat >> 1) * 8);
          mma_bf16(o_acc[2 * np], p_frag[kk], bfr[0], bfr[1]);
          mma_bf16(o_acc[2 * np + 1], p_frag[kk], bfr[2], bfr[3]);
        }
      }
    }
    __syncthreads();  // the stage is free for the load after next
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  if (a.splits > 1) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      int r = warp * 16 + gq + half * 8;
      if (r >= rows) continue;
      size_t at = ((size_t)tok0 * heads + p0 + r) * a.splits + blockIdx.z;
      if (tq == 0) {
        a.part_ml[at * 2] = m_run[half];
        a.part_ml[at * 2 + 1] = l_run[half];
      }
#pragma unroll
      for (int i = 0; i < RANK / 8; ++i) {
        int d = i * 8 + tq * 2;
        if (d < a.rank)
          *reinterpret_cast<float2*>(a.part_o + at * a.rank + d) = make_float2(o_acc[i][half * 2], o_acc[i][half * 2 + 1]);
      }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    int r = warp * 16 + gq + half * 8;
    if (r >= rows) continue;
    long long p = p0 + r;
    float factor = 1.0f / l_run[half];
    if (a.gates != nullptr) {
      float z = a.gates[(size_t)(tok0 + p / heads) * a.gate_ld + (int)(p % heads)];
      factor *= z >= 0.f ? 1.0f / (1.0f + expf(-z)) : expf(z) / (1.0f + expf(z));
    }
    size_t at = ((size_t)tok0 * heads + p) * a.rank;
#pragma unroll
    for (int i = 0; i < RANK / 8; ++i) {
      int d = i * 8 + tq * 2;
      if (d >= a.rank) continue;
      float x = o_acc[i][half * 2] * factor, y = o_acc[i][half * 2 + 1] * factor;
      if (a.out_bf16) *reinterpret_cast<__nv_bfloat162*>((bf16*)a.out + at + d) = __floats2bfloat162_rn(x, y);
      else *reinterpret_cast<float2*>((float*)a.out + at + d) = make_float2(x, y);
    }
  }
}

// A block per (token, head) pair: the splits' sums weighted by 2^(their maximum - the largest), divided by the total.
// The first 64 threads take a split each (weights and total through shared memory), then a thread a column.
__global__ void __launch_bounds__(128) latent_combine_kernel(TiledArgs a, long long pairs) {
  __shared__ float weight[64];
  __shared__ float scratch[4];
  pdl_launch_dependents();
  pdl_wait();
  const long long p = blockIdx.x;
  if (p >= pairs) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* ml = a.part_ml + (size_t)p * a.splits * 2;
  float m = -INFINITY, l = 0.f;
  if (tid < a.splits) {
    m = ml[2 * tid];
    l = ml[2 * tid + 1];
  }
  float top = warp_max(m);
  if (lane == 0) scratch[warp] = top;
  __syncthreads();
  top = fmaxf(fmaxf(scratch[0], scratch[1]), fmaxf(scratch[2], scratch[3]));
  float w = m == -INFINITY ? 0.f : fast_exp2(m - top);
  if (tid < 64) weight[tid] = w;
  float total = warp_sum(w * l);
  __syncthreads();
  if (lane == 0) scratch[warp] = total;
  __syncthreads();
  float factor = 1.0f / (scratch[0] + scratch[1] + scratch[2] + scratch[3]);
  if (a.gates != nullptr) {
    float z = a.gates[(size_t)(p / a.heads) * a.gate_ld + (int)(p % a.heads)];
    factor *= z >= 0.f ? 1.0f / (1.0f + expf(-z)) : expf(z) / (1.0f + expf(z));
  }
  const float* o = a.part_o + (size_t)p * a.splits * a.rank;
  for (int d = tid; d < a.rank; d += blockDim.x) {
    float sum = 0.f;
#pragma unroll 8
    for (int z = 0; z < a.splits; ++z) {
      float wz = weight[z];
      if (wz != 0.f) sum = fmaf(wz, o[(size_t)z * a.rank + d], sum);  // (a split without keys wrote no sums)
    }
    sum *= factor;
    if (a.out_bf16) ((bf16*)a.out)[(size_t)p * a.rank + d] = __float2bfloat16_rn(sum);
    else ((float*)a.out)[(size_t)p * a.rank + d] = sum;
  }
}

template <int RANK>
int launch(const TiledArgs& a, int tiles, int n_seqs, cudaStream_t stream) {
  size_t smem = (size_t)(BM + 2 * BN) * a.ld * sizeof(bf16);
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(latent_tiled_kernel<RANK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = smem;
  }
  return dllm_launch_pdl(latent_tiled_kernel<RANK>, dim3(tiles, n_seqs, a.splits), dim3(THREADS), smem, stream, a);
}
}  // namespace

// max_new: the most new tokens any sequence of the step has (the grid covers that many pairs for every sequence;
// blocks beyond a sequence's own pairs leave at once). splits > 1: part_o [pairs, splits, rank] and part_ml [pairs,
// splits, 2] float32 scratch, pairs = the step's tokens x heads.
DLLM_EXPORT int dllm_latent_attention_tiled(const float* q, const float* table, const float* gates, int gate_ld,
                                            const float* sinks,
                                            void* out, int out_bf16, const void* cache, const int* page_table,
                                            int max_pages, int page_size, int heads, int rank, int rot,
                                            const int* cu_seqlens, const int* tok_pos, const int* slots, int n_seqs,
                                            int max_new, int splits, float* part_o, float* part_ml, long long pairs,
                                            cudaStream_t stream) {
  if (n_seqs <= 0 || max_new <= 0) return DLLM_OK;
  if (heads <= 0 || rank <= 0 || rank > 256 || (rank & 7) || rot < 0 || (rot & 1) || ((rank + rot) & 7) ||
      page_size <= 0 || page_size % BN || n_seqs > 65535)
    return DLLM_UNSUPPORTED_SIZE;
  if (!q || !out || !cache || !page_table || !cu_seqlens || !tok_pos || !slots) return DLLM_BAD_ARGUMENT;
  int padded_rank = rank <= 64 ? 64 : (rank <= 128 ? 128 : 256);
  int k_width = ((rank + rot + 15) / 16) * 16;
  int ld = (k_width > padded_rank ? k_width : padded_rank) + 8;
  if ((size_t)(BM + 2 * BN) * ld * sizeof(bf16) > 200 * 1024) return DLLM_UNSUPPORTED_SIZE;
  TiledArgs a{q, rot > 0 ? table : nullptr, gates, sinks, gate_ld, out, out_bf16, (const bf16*)cache, page_table, max_pages,
              page_size, cu_seqlens, tok_pos, slots, heads, rank, rot, ld, splits, part_o, part_ml};
  if (splits < 1 || splits > 64 || (splits > 1 && (!part_o || !part_ml || pairs <= 0))) return DLLM_BAD_ARGUMENT;
  long long most = (long long)max_new * heads;
  int tiles = (int)((most + BM - 1) / BM);
  int status = rank <= 64 ? launch<64>(a, tiles, n_seqs, stream)
                          : (rank <= 128 ? launch<128>(a, tiles, n_seqs, stream) : launch<256>(a, tiles, n_seqs, stream));
  if (status != DLLM_OK || splits == 1) return status;
  return dllm_launch_pdl(latent_combine_kernel, dim3((unsigned)pairs), dim3(128), 0, stream, a, pairs);
}
