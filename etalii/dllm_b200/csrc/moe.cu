// A mixture of gated feed-forward experts, token by token: every token goes to the `top` experts with the largest router
// logits, weighted by the softmax over those logits only.
//
//   moe_route:  a block per token: logits = W_r x + b in float32 from the float32 stream, `top` rounds of arg-max (the
//               lower expert on ties), then the weights.
//               With `all_experts` the weights are instead the chosen experts' shares of the softmax over ALL experts'
//               logits, as they are (they do not add up to one).
//   moe_up:     per (token, choice): the chosen expert's gate and up rows times the token's activations, then the
//               clamped gated unit g sigmoid(alpha g) (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit).
//               Gate and up rows interleave in the stacked weight [experts, 2 ff, width].
//   moe_up_plain: the same for experts without a gate: act(W_up[expert] h), act by kind (relu squared, gelu).
//   moe_down:   per token: sum over its choices of weight * W_down[expert] act, stored (or added) in float32.
//
// A warp owns a few output values: its lanes split the reduction in 16-byte pieces (the rows' loads asked for together),
// sums in float32. These kernels read an
// expert's weights once per token that chose it, which is what a step of few tokens needs.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int MAX_EXPERTS = 256;
constexpr int MAX_TOP = 16;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ float piece(const float* a, const float* b) {
  float4 x = *(const float4*)a, y = *(const float4*)b;
  return fmaf(x.w, y.w, fmaf(x.z, y.z, fmaf(x.y, y.y, x.x * y.x)));
}
// This lane's share of a . b over n values (the warp's shares add up to the dot product).
template <typename T>
__device__ __forceinline__ float lane_dot(const T* a, const T* b, int n, int lane) {
  float s = 0.f;
  if (n % Vec<T>::N == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
    for (int d = lane * Vec<T>::N; d < n; d += 32 * Vec<T>::N) s += piece(a + d, b + d);
  } else {
    for (int d = lane; d < n; d += 32) s = fmaf(to_float(a[d]), to_float(b[d]), s);
  }
  return s;
}

// This lane's shares of R dot products at once: rows w, w + stride, ... against the same b. The R rows' pieces are
// asked for together (and b's piece once), so a warp keeps R loads in flight where one row after another keeps one.
template <int R, typename T>
__device__ __forceinline__ void lane_dots(const T* w, size_t stride, const T* b, int n, int lane, float* out) {
#pragma unroll
  for (int r = 0; r < R; ++r) out[r] = 0.f;
  bool pieces = n % Vec<T>::N == 0 && (((uintptr_t)w | (uintptr_t)b | (uintptr_t)(stride * sizeof(T))) & 15) == 0;
  if (pieces) {
    constexpr int N = Vec<T>::N;
    for (int d = lane * N; d < n; d += 32 * N) {
      struct alignas(16) Piece { T v[N]; };
      Piece held[R], mine;
#pragma unroll
      for (int r = 0; r < R; ++r) held[r] = *reinterpret_cast<const Piece*>(w + r * stride + d);
      mine = *reinterpret_cast<const Piece*>(b + d);
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < N; ++i) out[r] = fmaf(to_float(held[r].v[i]), to_float(mine.v[i]), out[r]);
    }
  } else {
    for (int d = lane; d < n; d += 32) {
      float x = to_float(b[d]);
#pragma unroll
      for (int r = 0; r < R; ++r) out[r] = fmaf(to_float(w[r * stride + d]), x, out[r]);
    }
  }
}

// The router's weights are float32 whatever the activations are.
template <typename X>
__device__ __forceinline__ float lane_dot_router(const float* w, const X* x, int n, int lane) {
  float s = 0.f;
  for (int d = lane; d < n; d += 32) s = fmaf(w[d], to_float(x[d]), s);
  return s;
}
template <>
__device__ __forceinline__ float lane_dot_router<float>(const float* w, const float* x, int n, int lane) {
  return lane_dot(w, x, n, lane);
}

template <typename X>
__global__ void __launch_bounds__(WARPS * 32) moe_route_kernel(
    const X* __restrict__ x, int width, const float* __restrict__ w, const float* __restrict__ bias, int experts,
    int top, int tokens, int* __restrict__ chosen, float* __restrict__ weights, int all_experts) {
  // a block per token: its warps share the experts' logits out, warp 0 then chooses
  __shared__ float logits[MAX_EXPERTS];
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int t = blockIdx.x;
  const X* row = x + (size_t)t * width;
  for (int e = warp; e < experts; e += WARPS) {
    float s = warp_sum(lane_dot_router(w + (size_t)e * width, row, width, lane));
    if (lane == 0) logits[e] = s + (bias != nullptr ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  float kept[MAX_TOP];
  float largest = 0.f, total = 0.f, everyone = 0.f;
  if (all_experts) {  // the softmax's denominator over every expert, before the chosen logits are struck out
    float most = -INFINITY;
    for (int e = lane; e < experts; e += 32) most = fmaxf(most, logits[e]);
    most = warp_max(most);
    for (int e = lane; e < experts; e += 32) everyone += expf(logits[e] - most);
    everyone = warp_sum(everyone);
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int where = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      float v = logits[e];
      if (v > best) { best = v; where = e; }  // (ascending e: the first of equals stays)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int ow = __shfl_xor_sync(0xffffffffu, where, o);
      if (ov > best || (ov == best && ow < where)) { best = ov; where = ow; }
    }
    if (where == 0x7fffffff) where = k;  // (only rows without a finite logit)
    if (k == 0) largest = best;
    kept[k] = expf(best - largest);
    total += kept[k];
    if (lane == 0) {
      chosen[(size_t)t * top + k] = where;
      logits[where] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0)
    for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] = kept[k] / (all_experts ? everyone : total);
}

constexpr int UP_PER_WARP = 2;    // gated values a warp of moe_up owns (four rows of W)
constexpr int DOWN_PER_WARP = 4;  // output values a warp of moe_down owns

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) moe_up_kernel(
    T* __restrict__ act, const T* __restrict__ h, int width, const T* __restrict__ w_gate_up, int ff, int top,
    const int* __restrict__ chosen, float limit, float alpha, float shift) {
  pdl_launch_dependents();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int f = (blockIdx.y * WARPS + warp) * UP_PER_WARP;
  if (f >= ff) return;
  pdl_wait();
  int a = blockIdx.x;
  int e = chosen[a];
  const T* row = h + (size_t)(a / top) * width;
  const T* wg = w_gate_up + ((size_t)e * 2 * ff + 2 * f) * width;  // rows: gate f, up f, gate f + 1, up f + 1
  float sums[2 * UP_PER_WARP];
  if (f + UP_PER_WARP <= ff) {
    lane_dots<2 * UP_PER_WARP>(wg, (size_t)width, row, width, lane, sums);
  } else {  // (an odd ff: the last value alone)
    lane_dots<2>(wg, (size_t)width, row, width, lane, sums);
    sums[2] = sums[3] = 0.f;
  }
#pragma unroll
  for (int r = 0; r < 2 * UP_PER_WARP; ++r) sums[r] = warp_sum(sums[r]);
  if (lane < UP_PER_WARP && f + lane < ff) {
    float g = fminf(lane == 0 ? sums[0] : sums[2], limit);
    float u = fminf(fmaxf(lane == 0 ? sums[1] : sums[3], -limit), limit);
    act[(size_t)a * ff + f + lane] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
  }
}

__device__ __forceinline__ float plain_activation(float z, int kind) {
  if (kind == 1) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
  if (kind == 2) return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  float r = fmaxf(z, 0.f);
  return r * r;
}

constexpr int PLAIN_PER_WARP = 4;  // activated values a warp of moe_up_plain owns

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) moe_up_plain_kernel(
    T* __restrict__ act, const T* __restrict__ h, int width, const T* __restrict__ w_up, int ff, int top,
    const int* __restrict__ chosen, int kind) {
  pdl_launch_dependents();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int f = (blockIdx.y * WARPS + warp) * PLAIN_PER_WARP;
  if (f >= ff) return;
  pdl_wait();
  int a = blockIdx.x;
  int e = chosen[a];
  const T* row = h + (size_t)(a / top) * width;
  const T* w = w_up + ((size_t)e * ff + f) * width;
  int count = min(PLAIN_PER_WARP, ff - f);
  float sums[PLAIN_PER_WARP];
  if (count == PLAIN_PER_WARP) {
    lane_dots<PLAIN_PER_WARP>(w, (size_t)width, row, width, lane, sums);
  } else {
#pragma unroll
    for (int r = 0; r < PLAIN_PER_WARP; ++r) {
      sums[r] = 0.f;
      if (r < count) lane_dots<1>(w + (size_t)r * width, (size_t)width, row, width, lane, &sums[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < PLAIN_PER_WARP; ++r) sums[r] = warp_sum(sums[r]);
  if (lane < count) {
    float mine = sums[0];
#pragma unroll
    for (int r = 1; r < PLAIN_PER_WARP; ++r)
      if (lane == r) mine = sums[r];
    act[(size_t)a * ff + f + lane] = from_float<T>(plain_activation(mine, kind));
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) moe_down_kernel(
    float* __restrict__ out, const T* __restrict__ act, int ff, const T* __restrict__ w_down, int width, int top,
    const int* __restrict__ chosen, const float* __restrict__ weights, int accumulate) {
  pdl_launch_dependents();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int n = (blockIdx.y * WARPS + warp) * DOWN_PER_WARP;
  if (n >= width) return;
  pdl_wait();
  int t = blockIdx.x;
  int count = min(DOWN_PER_WARP, width - n);
  float total[DOWN_PER_WARP];
#pragma unroll
  for (int r = 0; r < DOWN_PER_WARP; ++r) total[r] = 0.f;
  for (int k = 0; k < top; ++k) {
    int a = t * top + k;
    int e = chosen[a];
    const T* w = w_down + ((size_t)e * width + n) * ff;
    float sums[DOWN_PER_WARP];
    if (count == DOWN_PER_WARP) {
      lane_dots<DOWN_PER_WARP>(w, (size_t)ff, act + (size_t)a * ff, ff, lane, sums);
    } else {
#pragma unroll
      for (int r = 0; r < DOWN_PER_WARP; ++r) {
        sums[r] = 0.f;
        if (r < count) lane_dots<1>(w + (size_t)r * ff, (size_t)ff, act + (size_t)a * ff, ff, lane, &sums[r]);
      }
    }
    float weight = weights[a];
#pragma unroll
    for (int r = 0; r < DOWN_PER_WARP; ++r) total[r] = fmaf(weight, warp_sum(sums[r]), total[r]);
  }
  if (lane < count) {
    float mine = total[0];
#pragma unroll
    for (int r = 1; r < DOWN_PER_WARP; ++r)
      if (lane == r) mine = total[r];
    size_t at = (size_t)t * width + n + lane;
    out[at] = accumulate ? out[at] + mine : mine;
  }
}
}  // namespace

DLLM_EXPORT int dllm_moe_route(const void* x, int width, const float* w, const float* bias, int experts, int top,
                               int tokens, int* chosen, float* weights, int all_experts, int dtype,
                               cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (experts <= 0 || experts > MAX_EXPERTS || top <= 0 || top > MAX_TOP || top > experts || width <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  if (x == nullptr || w == nullptr || chosen == nullptr || weights == nullptr) return DLLM_BAD_ARGUMENT;
  dim3 grid(tokens), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(moe_route_kernel<float>, grid, block, 0, stream, (const float*)x, width, w, bias, experts,
                           top, tokens, chosen, weights, all_experts);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(moe_route_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, width, w,
                           bias, experts, top, tokens, chosen, weights, all_experts);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_moe_up(void* act, const void* h, int width, const void* w_gate_up, int ff, int top, int tokens,
                            const int* chosen, float limit, float alpha, float shift, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || ff <= 0 || top <= 0 || ff > 65535 * WARPS) return DLLM_UNSUPPORTED_SIZE;
  dim3 grid(tokens * top, (ff + WARPS * UP_PER_WARP - 1) / (WARPS * UP_PER_WARP)), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(moe_up_kernel<float>, grid, block, 0, stream, (float*)act, (const float*)h, width,
                           (const float*)w_gate_up, ff, top, chosen, limit, alpha, shift);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(moe_up_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)act,
                           (const __nv_bfloat16*)h, width, (const __nv_bfloat16*)w_gate_up, ff, top, chosen, limit, alpha,
                           shift);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_moe_down(float* out, const void* act, int ff, const void* w_down, int width, int top, int tokens,
                              const int* chosen, const float* weights, int accumulate, int dtype,
                              cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || ff <= 0 || top <= 0 || width > 65535 * WARPS) return DLLM_UNSUPPORTED_SIZE;
  dim3 grid(tokens, (width + WARPS * DOWN_PER_WARP - 1) / (WARPS * DOWN_PER_WARP)), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(moe_down_kernel<float>, grid, block, 0, stream, out, (const float*)act, ff,
                           (const float*)w_down, width, top, chosen, weights, accumulate);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(moe_down_kernel<__nv_bfloat16>, grid, block, 0, stream, out, (const __nv_bfloat16*)act, ff,
                           (const __nv_bfloat16*)w_down, width, top, chosen, weights, accumulate);
  return DLLM_BAD_ARGUMENT;
}

// act[t, k] = activation(W_up[chosen[t, k]] h[t]); W_up [experts, ff, width]; kind 1: gelu (erf), 2: gelu (tanh form),
// 3: relu squared.
DLLM_EXPORT int dllm_moe_up_plain(void* act, const void* h, int width, const void* w_up, int ff, int top, int tokens,
                                  const int* chosen, int kind, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || ff <= 0 || top <= 0 || ff > 65535 * WARPS || kind < 1 || kind > 3) return DLLM_UNSUPPORTED_SIZE;
  dim3 grid(tokens * top, (ff + WARPS * PLAIN_PER_WARP - 1) / (WARPS * PLAIN_PER_WARP)), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(moe_up_plain_kernel<float>, grid, block, 0, stream, (float*)act, (const float*)h, width,
                           (const float*)w_up, ff, top, chosen, kind);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(moe_up_plain_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)act,
                           (const __nv_bfloat16*)h, width, (const __nv_bfloat16*)w_up, ff, top, chosen, kind);
  return DLLM_BAD_ARGUMENT;
}
