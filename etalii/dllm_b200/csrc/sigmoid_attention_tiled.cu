// Attention with sigmoid weights mixed across heads (see sigmoid_attention.cu) for prompt-sized steps on the tensor
// cores (bfloat16 operands, mma.sync m16n8k16, float32 accumulators).
//
// A block takes 16 consecutive new tokens of one sequence and ALL heads, because the mixing needs every head's weight
// of a (query, key) pair in one place. It walks the keys the 16 tokens can see (the kept first positions, then the
// window) in tiles of 32; per tile
//   1. keys and values of every kv head arrive in shared memory (cp.async, two stages where they fit),
//   2. each warp computes S_h = Q_h K^T for ITS heads and leaves w_h = sigmoid(S_h scale - slope_h (i - j) + b_h), zero
//      where j is not visible, in shared memory as bfloat16 [head][query][key],
//   3. the mixing w'_h = sum_g M[h, g] w_g is itself a product on the tensor cores: M (bfloat16 fragments that every
//      warp holds in registers for the whole kernel) times the [head] x [query, key] matrix of weights, each warp a
//      stretch of the tile's (query, key) pairs; the mixed weights go back to shared memory as bfloat16,
//   4. each warp adds w'_h V for its heads to their sums.
// Without a mixing matrix step 3 is left out. The epilogue multiplies by sigmoid(gate) and rounds. Nothing is
// normalised over the keys, so there is no running maximum and no rescaling. Warp w owns heads w * HPW .. w * HPW +
// HPW - 1. (With the mixing as float32 multiply-adds out of shared memory, a head's 16 x 32 weights from all heads'
// at 8 multiply-adds per load, a warp spent 1,000 of its 2,500 instructions a tile there and 800 on exact sigmoids.)
//
// Where the queries of all heads, a tile of all kv heads and all heads' weights do not fit one block's shared memory (32
// heads of 128), a cluster of two blocks takes the 16 tokens: each block owns half the heads with their kv heads
// (queries, keys, values and sums of its own heads only), writes the weights of its heads into BOTH blocks' shared
// memory (`st.shared::cluster`), and mixes and sums for its own heads after a cluster barrier; a second cluster
// barrier at the end of a tile keeps a block from writing the next tile's weights while the other still reads.
//
// dim and vdim: multiples of 16, at most 128 (vdim) and 256 (dim). page_size: a multiple of 32.
#include "wide_kv.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 16, BN = 32, W_LD = 40;
constexpr int W_PLANE = BM * W_LD + 8;  // a head's weights; the 8 keep ldmatrix over eight heads off one bank
constexpr int MAX_HEAD_TILES = 2;       // the mixing matrix in registers: up to 32 heads

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
constexpr float LOG2E = 1.4426950408889634f;
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// 1 / (1 + 2^x) with the hardware's approximations (x = -score * log2 e; 2^x = inf gives 0).
__device__ __forceinline__ float sigmoid_of_exp2(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(1.0f + fast_exp2(x)));
  return y;
}
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Four bytes to the same shared-memory place in block `rank` of the cluster.
__device__ __forceinline__ void store_remote(const void* local, unsigned rank, unsigned value) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote), "r"(value) : "memory");
}
__device__ __forceinline__ float sigmoid_exact(float g) {
  if (g >= 0.f) return 1.0f / (1.0f + expf(-g));
  float e = expf(g);
  return e / (1.0f + e);
}

struct TiledArgs {
  const bf16* q;        // [tokens, heads * dim]
  WideKv cache;         // bfloat16
  const float* mix;     // [heads, heads] or null
  const float* slopes;  // [heads] or null
  const float* head_bias;  // [heads] or null
  const float* gates;   // gates[token * gate_ld + o] or null
  int gate_ld;
  bf16* out;            // [tokens, heads * vdim]
  float* part;          // splits > 1: [split][token][heads * vdim] float32 sums, no gate (sigmoid_combine finishes)
  int splits, tokens;   // blocks that share a block's tiles of keys (blockIdx.z); the step's tokens
  int heads, window, keep, stages;
  int cluster;          // blocks that share a block of 16 tokens, each with its share of the heads (1 or 2)
  float scale;
  const int* cu_seqlens;
  const int* tok_pos;
  const int* slots;
};

template <int HPW, int VD>
__global__ void __launch_bounds__(HPW == 1 && VD == 64 ? 512 : 256) sigmoid_tiled_kernel(TiledArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // `all_heads` is the model's; heads, groups: this block's own (all of them, or its half in a cluster of two), which
  // start at head h0 and kv head g0
  const int all_heads = a.heads, share = all_heads / a.cache.kv_heads;
  const unsigned crank = a.cluster > 1 ? cluster_rank() : 0;
  const int heads = all_heads / a.cluster, groups = a.cache.kv_heads / a.cluster;
  const int h0 = (int)crank * heads, g0 = (int)crank * groups;
  const int dim = a.cache.key_dim, vdim = a.cache.value_dim;
  const int k_ld = dim + 8, v_ld = vdim + 8;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                 // [heads][BM][k_ld]
  bf16* k_s = q_s + (size_t)heads * BM * k_ld;                   // [stages][groups][BN][k_ld]
  bf16* v_s = k_s + (size_t)a.stages * groups * BN * k_ld;       // [stages][groups][BN][v_ld]
  const int head_tiles = (all_heads + 15) >> 4, own_tiles = (heads + 15) >> 4;
  bf16* w_s = v_s + (size_t)a.stages * groups * BN * v_ld;       // [16 head_tiles][W_PLANE]: ALL heads' weights
  // ... and this block's heads' weights after the mixing (without a mixing matrix: its own planes of w_s)
  bf16* p_s = a.mix != nullptr ? w_s + (size_t)head_tiles * 16 * W_PLANE : w_s + (size_t)h0 * W_PLANE;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, threads = blockDim.x, warps = threads >> 5;
  const int gq = lane >> 2, tq = lane & 3, mat = lane >> 3;
  pdl_launch_dependents();
  // the mixing matrix as the left operand's fragments: tile (mt, kt) holds M[16 mt + row][16 kt + column]
  unsigned m_frag[MAX_HEAD_TILES][MAX_HEAD_TILES][4];
  if (a.mix != nullptr) {
#pragma unroll
    for (int mt = 0; mt < MAX_HEAD_TILES; ++mt)
#pragma unroll
      for (int kt = 0; kt < MAX_HEAD_TILES; ++kt)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          int h = mt * 16 + gq + 8 * (x & 1), g = kt * 16 + tq * 2 + 8 * (x >> 1);  // (h: among this block's heads)
          float lo = h < heads && g < all_heads ? a.mix[(h0 + h) * all_heads + g] : 0.f;
          float hi = h < heads && g + 1 < all_heads ? a.mix[(h0 + h) * all_heads + g + 1] : 0.f;
          m_frag[mt][kt][x] = pack_bf16(lo, hi);
        }
    // heads beyond the model's (the padding of the last tile of 16) have weights of zero for good
    for (int i = tid; i < (head_tiles * 16 - all_heads) * W_PLANE; i += threads)
      w_s[(size_t)all_heads * W_PLANE + i] = __float2bfloat16_rn(0.f);
  }
  pdl_wait();
  const int b = blockIdx.y;
  const int tok0 = a.cu_seqlens[b], n_new = a.cu_seqlens[b + 1] - tok0;
  // (the last tokens of a sequence see the most keys: they go first)
  const int m0 = (gridDim.x / a.cluster - 1 - blockIdx.x / a.cluster) * BM;
  if (m0 >= n_new) return;
  const int rows = min(BM, n_new - m0);
  const int pos_lo = a.tok_pos[tok0] + m0, pos_hi = pos_lo + rows - 1;  // positions of new tokens are consecutive
  const int* pages = a.cache.page_table + (size_t)a.slots[b] * a.cache.max_pages;

  // the tiles this block walks: those of the kept first positions that lie before the first row's window, then from
  // the first row's window to the last row's own position
  const int lo = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
  const int kept_tiles = (min(a.keep, lo) + BN - 1) / BN;
  const int window_first = max(lo / BN, kept_tiles);
  const int count = kept_tiles + pos_hi / BN - window_first + 1;
  auto first_key = [&](int index) { return (index < kept_tiles ? index : window_first + index - kept_tiles) * BN; };

  int begin = 0, end = count;
  if (a.splits > 1) {
    const int per = (count + a.splits - 1) / a.splits;
    begin = blockIdx.z * per;
    end = min(count, begin + per);
    if (begin >= end) {  // nothing left for this block: its heads' sums of its rows are zeros
      const int outputs = all_heads * vdim, mine = heads * vdim;
      for (int i = tid; i < rows * mine; i += threads)
        a.part[((size_t)blockIdx.z * a.tokens + tok0 + m0 + i / mine) * outputs + h0 * vdim + i % mine] = 0.f;
      return;
    }
  }
  // A row of keys (or values) of one kv head is copied by a power-of-two stretch of a warp's lanes, 16 bytes a lane, so
  // that finding a lane's row and piece takes shifts only.
  const int k_pieces = dim >> 3, v_pieces = vdim >> 3;
  int k_shift = 0, v_shift = 0;
  while ((1 << k_shift) < k_pieces) ++k_shift;
  while ((1 << v_shift) < v_pieces) ++v_shift;
  auto load_rows = [&](bf16* dst, int ld, int pieces, int shift, int width, size_t first, size_t per_group) {
    const int piece = lane & ((1 << shift) - 1), rows_at_once = 32 >> shift;
    if (piece >= pieces) return;
    const bf16* base = (const bf16*)a.cache.base + first + piece * 8;
    for (int rr = warp * rows_at_once + (lane >> shift); rr < groups * BN; rr += warps * rows_at_once) {
      const int g = rr / BN, r = rr % BN;  // (BN is a power of two)
      cp_async_16(dst + (size_t)rr * ld + piece * 8, base + g * per_group + (size_t)r * width);
    }
  };
  auto load_tile = [&](int stage, int index) {
    const int j0 = first_key(index);
    const int page = pages[j0 / a.cache.page_size], row0 = j0 % a.cache.page_size;
    load_rows(k_s + (size_t)stage * groups * BN * k_ld, k_ld, k_pieces, k_shift, dim, key_at(a.cache, page, g0, row0),
              (size_t)a.cache.page_size * dim);
    load_rows(v_s + (size_t)stage * groups * BN * v_ld, v_ld, v_pieces, v_shift, vdim,
              value_at(a.cache, page, g0, row0), (size_t)a.cache.page_size * vdim);
  };
  load_tile(0, begin);
  cp_async_commit();

  // the block's queries: [head][row][dim]; rows beyond the sequence's tokens are zeros
  for (int idx = tid; idx < heads * BM * k_pieces; idx += threads) {
    int h = idx / (BM * k_pieces), rest = idx - h * BM * k_pieces, r = rest / k_pieces, c = rest - r * k_pieces;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows)
      v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(tok0 + m0 + r) * all_heads + h0 + h) * dim + c * 8);
    *reinterpret_cast<uint4*>(q_s + ((size_t)h * BM + r) * k_ld + c * 8) = v;
  }

  float o_acc[HPW][VD / 8][4];
#pragma unroll
  for (int e = 0; e < HPW; ++e)
#pragma unroll
    for (int i = 0; i < VD / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o_acc[e][i][j] = 0.f;
  int row_pos[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) row_pos[i] = gq + 8 * i < rows ? pos_lo + gq + 8 * i : -1;
  const int k_steps = dim >> 4, nv16 = vdim >> 4;
  // -(score) in units of log2 e: x = S * (-scale log2 e) + c_row + slope' * (column), with the row's constant
  // c_row = (slope (i - j0) - bias) log2 e and slope' = -slope log2 e
  float slope_of[HPW], bias_of[HPW];
#pragma unroll
  for (int e = 0; e < HPW; ++e) {
    const int h = h0 + min(warp * HPW + e, heads - 1);
    slope_of[e] = a.slopes != nullptr ? a.slopes[h] * LOG2E : 0.f;
    bias_of[e] = a.head_bias != nullptr ? a.head_bias[h] * LOG2E : 0.f;
  }
  if (a.cluster > 1) cluster_sync();  // (the other block runs, and has cleared its padding, before anyone writes to it)

  for (int index = begin; index < end; ++index) {
    const int stage = a.stages == 2 ? ((index - begin) & 1) : 0;
    if (a.stages == 2) {
      if (index + 1 < end) load_tile(stage ^ 1, index + 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();  // the tile (and, the first time, the queries) is in shared memory
    const int j0 = first_key(index);
    const bf16* kb = k_s + (size_t)stage * groups * BN * k_ld;
    const bf16* vb = v_s + (size_t)stage * groups * BN * v_ld;
    // 2. this warp's heads: scores, weights, into shared memory
#pragma unroll
    for (int e = 0; e < HPW; ++e) {
      const int h = warp * HPW + e;
      if (h >= heads) break;
      const bf16* kg = kb + (size_t)(h / share) * BN * k_ld;
      const bf16* qh = q_s + (size_t)h * BM * k_ld;
      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) s[j][r] = 0.f;
#pragma unroll 2
      for (int ks = 0; ks < k_steps; ++ks) {
        unsigned qf[4];
        ldmatrix_x4(qf, qh + (size_t)(lane & 15) * k_ld + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int jp = 0; jp < BN / 16; ++jp) {
          unsigned bfr[4];
          ldmatrix_x4(bfr, kg + (size_t)(jp * 16 + (mat >> 1) * 8 + (lane & 7)) * k_ld + ks * 16 + (mat & 1) * 8);
          mma_bf16(s[2 * jp], qf, bfr[0], bfr[1]);
          mma_bf16(s[2 * jp + 1], qf, bfr[2], bfr[3]);
        }
      }
      const float slope = slope_of[e], bias = bias_of[e], scale = -a.scale * LOG2E;
      bf16* wh = w_s + (size_t)(h0 + h) * W_PLANE;
      // a tile all of whose keys every row sees needs no mask
      const bool open = j0 + BN - 1 <= pos_lo && rows == BM &&
                        (a.window <= 0 || pos_hi - j0 < a.window || j0 + BN <= a.keep);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = row_pos[half];
        const float c_row = fmaf(slope, (float)(i - j0 - tq * 2), -bias);
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
          float w[2];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            w[c] = sigmoid_of_exp2(fmaf(s[j][half * 2 + c], scale, fmaf(-slope, (float)(j * 8 + c), c_row)));
            if (!open) {
              const int key = j0 + j * 8 + tq * 2 + c;
              if (!(key <= i && (a.window <= 0 || i - key < a.window || key < a.keep))) w[c] = 0.f;
            }
          }
          bf16* at = wh + (size_t)(gq + 8 * half) * W_LD + j * 8 + tq * 2;
          const unsigned both = pack_bf16(w[0], w[1]);
          *reinterpret_cast<unsigned*>(at) = both;
          if (a.cluster > 1) store_remote(at, crank ^ 1, both);
        }
      }
    }
    if (a.cluster > 1) cluster_sync(); else __syncthreads();
    // 3. the mixing as a product: P[h][pair] = sum_g M[h][g] W[g][pair], pairs = the tile's (query, key) places; a warp
    // takes every warps-th stretch of 16 keys of a query row
    if (a.mix != nullptr) {
      for (int item = warp; item < BM * (BN / 16); item += warps) {
        const int row = item / (BN / 16), col = (item - row * (BN / 16)) * 16;
        float d[MAX_HEAD_TILES][2][4];
#pragma unroll
        for (int mt = 0; mt < MAX_HEAD_TILES; ++mt)
#pragma unroll
          for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int x = 0; x < 4; ++x) d[mt][n][x] = 0.f;
#pragma unroll
        for (int kt = 0; kt < MAX_HEAD_TILES; ++kt) {
          if (kt < head_tiles) {
            unsigned bfr[4];  // heads 16 kt + (0..7 | 8..15) x keys col + (0..7 | 8..15)
            ldmatrix_x4_trans(bfr, w_s + (size_t)(kt * 16 + (mat & 1) * 8 + (lane & 7)) * W_PLANE + row * W_LD + col +
                                       (mat >> 1) * 8);
#pragma unroll
            for (int mt = 0; mt < MAX_HEAD_TILES; ++mt) {
              if (mt < own_tiles) {
                mma_bf16(d[mt][0], m_frag[mt][kt], bfr[0], bfr[1]);
                mma_bf16(d[mt][1], m_frag[mt][kt], bfr[2], bfr[3]);
              }
            }
          }
        }
#pragma unroll
        for (int mt = 0; mt < MAX_HEAD_TILES; ++mt)
#pragma unroll
          for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int h = mt * 16 + gq + 8 * half;
              if (mt < own_tiles && h < heads)
                *reinterpret_cast<unsigned*>(p_s + (size_t)h * W_PLANE + row * W_LD + col + n * 8 + tq * 2) =
                    pack_bf16(d[mt][n][half * 2], d[mt][n][half * 2 + 1]);
            }
      }
      __syncthreads();
    }
    // 4. this warp's heads: add the weighted values
#pragma unroll
    for (int e = 0; e < HPW; ++e) {
      const int h = warp * HPW + e;
      if (h >= heads) break;
      const bf16* ph = p_s + (size_t)h * W_PLANE;
      const bf16* vg = vb + (size_t)(h / share) * BN * v_ld;
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        unsigned p_frag[4];
        ldmatrix_x4(p_frag, ph + (size_t)(lane & 15) * W_LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < VD / 16; ++np) {
          if (np < nv16) {
            unsigned bfr[4];
            ldmatrix_x4_trans(bfr, vg + (size_t)(kk * 16 + (mat & 1) * 8 + (lane & 7)) * v_ld + np * 16 + (mat >> 1) * 8);
            mma_bf16(o_acc[e][2 * np], p_frag, bfr[0], bfr[1]);
            mma_bf16(o_acc[e][2 * np + 1], p_frag, bfr[2], bfr[3]);
          }
        }
      }
    }
    // the tile's stage and the weights are free again (in a cluster: also for the other block's next weights)
    if (a.cluster > 1) cluster_sync(); else __syncthreads();
    if (a.stages == 1 && index + 1 < end) {
      load_tile(0, index + 1);
      cp_async_commit();
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int e = 0; e < HPW; ++e) {
    const int h = warp * HPW + e;
    if (h >= heads) break;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = gq + 8 * half;
      if (r >= rows) continue;
      const size_t t = (size_t)tok0 + m0 + r;
#pragma unroll
      for (int i = 0; i < VD / 8; ++i) {
        const int d = i * 8 + tq * 2;
        if (d >= vdim) continue;
        const size_t o = (size_t)(h0 + h) * vdim + d;
        float x = o_acc[e][i][half * 2], y = o_acc[e][i][half * 2 + 1];
        if (a.splits > 1) {
          *reinterpret_cast<float2*>(a.part + ((size_t)blockIdx.z * a.tokens + t) * all_heads * vdim + o) =
              make_float2(x, y);
          continue;
        }
        if (a.gates != nullptr) {
          float2 z = *reinterpret_cast<const float2*>(a.gates + t * a.gate_ld + o);
          x *= sigmoid_exact(z.x);
          y *= sigmoid_exact(z.y);
        }
        *reinterpret_cast<__nv_bfloat162*>(a.out + t * all_heads * vdim + o) = __floats2bfloat162_rn(x, y);
      }
    }
  }
}

// A block's shared memory: the queries of its `heads` (all of them, or half in a cluster of two), `stages` tiles of
// its kv heads, the weights of ALL heads and its own heads' mixed weights.
size_t shared_bytes(int all_heads, int groups, int dim, int vdim, int stages, int cluster) {
  int heads = all_heads / cluster;
  size_t planes = (size_t)((all_heads + 15) / 16) * 16 + (size_t)((heads + 15) / 16) * 16;
  return ((size_t)heads * BM * (dim + 8) + (size_t)stages * (groups / cluster) * BN * (dim + 8 + vdim + 8) +
          planes * W_PLANE) * sizeof(bf16);
}

template <int HPW, int VD>
int launch(const TiledArgs& a, int warps, size_t smem, int tiles, int n_seqs, cudaStream_t stream) {
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(sigmoid_tiled_kernel<HPW, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = smem;
  }
  if (a.cluster == 1)
    return dllm_launch_pdl(sigmoid_tiled_kernel<HPW, VD>, dim3(tiles, n_seqs, a.splits), dim3(warps * 32), smem,
                           stream, a);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(tiles * a.cluster, n_seqs, a.splits);
  config.blockDim = dim3(warps * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = a.cluster;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = dllm_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, sigmoid_tiled_kernel<HPW, VD>, a) == cudaSuccess ? DLLM_OK : DLLM_LAUNCH_FAILED;
}

// Heads a warp owns, of a block's `heads`: the fewest that give at most eight warps (a thread of these kernels takes
// up to 255 registers, which is what 256 threads may have); values of up to 64 take a head a warp up to sixteen warps
// (128 registers a thread). 0: these sizes do not run here, because a warp's sums would not fit its registers (heads x
// padded vdim above 256).
int heads_per_warp(int heads, int vdim) {
  int padded = vdim <= 64 ? 64 : 128;
  if (padded == 64 && heads <= 16) return 1;
  int hpw = heads <= 8 ? 1 : (heads <= 16 ? 2 : 4);
  if (hpw * padded > 256 || (heads + hpw - 1) / hpw > 8) return 0;
  return hpw;
}

// Blocks that share 16 tokens: 1 where one block holds everything, 2 where two halves of the heads do (whole tiles of
// 16 heads and whole kv heads each), 0 where neither does.
int blocks_for(int heads, int kv_heads, int dim, int vdim) {
  if (heads > 16 * MAX_HEAD_TILES) return 0;
  if (heads_per_warp(heads, vdim) != 0 && shared_bytes(heads, kv_heads, dim, vdim, 1, 1) <= 220 * 1024) return 1;
  if (heads % 32 == 0 && kv_heads % 2 == 0 && (heads / 2) % (heads / kv_heads) == 0 &&
      heads_per_warp(heads / 2, vdim) != 0 && shared_bytes(heads, kv_heads, dim, vdim, 1, 2) <= 220 * 1024)
    return 2;
  return 0;
}
}  // namespace

// 1 where the kernel below runs these sizes, else 0.
DLLM_EXPORT int dllm_sigmoid_attention_tiled_fits(int heads, int kv_heads, int dim, int vdim, int page_size) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim > 256 || (dim & 15) || vdim <= 0 ||
      vdim > 128 || (vdim & 15) || page_size <= 0 || page_size % BN)
    return 0;
  return blocks_for(heads, kv_heads, dim, vdim) != 0 ? 1 : 0;
}

// max_new: the most new tokens any sequence of the step has (the grid covers that many for every sequence; blocks
// beyond a sequence's own tokens leave at once). gates: float32, rows of gate_ld values, 8-byte aligned. splits > 1:
// the tiles of keys a block of 16 tokens walks are dealt to that many blocks, which leave float32 sums in `part`
// [splits][tokens][heads x vdim] for `dllm_sigmoid_combine` (sigmoid_attention.cu) to add, gate and round; `out` and
// `gates` are then not used here.
DLLM_EXPORT int dllm_sigmoid_attention_tiled(const void* q, void* out, const void* cache_base, const int* page_table,
                                             int max_pages, int page_size, int heads, int kv_heads, int dim, int vdim,
                                             const float* mix, const float* slopes, const float* head_bias,
                                             const float* gates, int gate_ld, float scale, int window, int keep,
                                             const int* cu_seqlens, const int* tok_pos, const int* slots, int n_seqs,
                                             int max_new, int splits, float* part, int tokens, cudaStream_t stream) {
  if (n_seqs <= 0 || max_new <= 0) return DLLM_OK;
  if (!dllm_sigmoid_attention_tiled_fits(heads, kv_heads, dim, vdim, page_size) || keep < 0 || n_seqs > 65535 ||
      (gates != nullptr && ((gate_ld & 1) || ((uintptr_t)gates & 7))))
    return DLLM_UNSUPPORTED_SIZE;
  if (!q || !out || !cache_base || !page_table || !cu_seqlens || !tok_pos || !slots) return DLLM_BAD_ARGUMENT;
  if (splits < 1 || splits > 65535 || (splits > 1 && (!part || tokens <= 0))) return DLLM_BAD_ARGUMENT;
  int cluster = blocks_for(heads, kv_heads, dim, vdim);
  // two stages where two blocks a multiprocessor still fit, or where only one fits either way
  size_t one = shared_bytes(heads, kv_heads, dim, vdim, 1, cluster), two = shared_bytes(heads, kv_heads, dim, vdim, 2, cluster);
  int stages = (two <= 110 * 1024 || (two <= 220 * 1024 && one > 110 * 1024)) ? 2 : 1;
  TiledArgs a{(const bf16*)q, WideKv{(void*)cache_base, page_table, max_pages, page_size, kv_heads, dim, vdim}, mix,
              slopes, head_bias, gates, gate_ld, (bf16*)out, part, splits, tokens, heads, window, keep, stages, cluster,
              scale, cu_seqlens, tok_pos, slots};
  size_t smem = stages == 2 ? two : one;
  int own = heads / cluster;
  int hpw = heads_per_warp(own, vdim), warps = (own + hpw - 1) / hpw;
  int tiles = (max_new + BM - 1) / BM;
  bool narrow = vdim <= 64;
  if (hpw == 1) return narrow ? launch<1, 64>(a, warps, smem, tiles, n_seqs, stream)
                              : launch<1, 128>(a, warps, smem, tiles, n_seqs, stream);
  if (hpw == 2) return narrow ? launch<2, 64>(a, warps, smem, tiles, n_seqs, stream)
                              : launch<2, 128>(a, warps, smem, tiles, n_seqs, stream);
  return launch<4, 64>(a, warps, smem, tiles, n_seqs, stream);
}
