// Routed experts: the router with groups, and the experts' two products for the (token, expert) pairs of a step.
//
// Router, per token, in 32-bit: z = W_r h; s = softmax(z) over all experts; the experts form `groups` equal
// groups of neighbours, a group's score is its largest s, only experts of the `keep` best groups can be
// chosen; the `top` largest s among those are chosen (the lower index wins a tie); their weights are
// s / (sum of the chosen s + 1e-20) * scale.
// Experts: y_t = sum_j weight_j * W_down[e_j] act(W_up[e_j] h_t), act = exact gelu (erf) here.
// The pair kernels read each chosen expert's rows once per pair: the form for steps of few tokens, where the
// weights stream from memory once and every token adds its experts in the order of its choices.
#include "common.cuh"

#define MOE_MAX_EXPERTS 1024

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, int ld, const float* __restrict__ wr, int n_tokens, int width,
                                 int E, int groups, int keep, int top, float scale, int* __restrict__ idx,
                                 float* __restrict__ wts) {
  extern __shared__ float sm[];           // E scores per warp, then `groups` group scores per warp
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + wib;
  if (t >= n_tokens) return;
  float* s = sm + (size_t)wib * E;
  const T* x = h + (size_t)t * ld;
  for (int e = 0; e < E; ++e) {
    const float* w = wr + (size_t)e * width;
    float part = 0.f;
    for (int k = lane; k < width; k += 32) part += to_f32(x[k]) * w[k];
    part = warp_sum(part);
    if (lane == 0) s[e] = part;
  }
  __syncwarp();
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(s[e] - mx);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
  __syncwarp();
  // groups: the experts of groups that are not kept are struck out (-1, below every score)
  const int per = E / groups;
  if (keep < groups) {
    float* gs = sm + (size_t)(blockDim.x >> 5) * E + (size_t)wib * groups;
    for (int g = lane; g < groups; g += 32) {
      float v = -1.f;
      for (int j = 0; j < per; ++j) v = fmaxf(v, s[g * per + j]);
      gs[g] = v;
    }
    __syncwarp();
    for (int pick = 0; pick < keep; ++pick) {
      float best = -0.5f;
      int bg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] > best) { best = gs[g]; bg = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (ob > best || (ob == best && og < bg)) { best = ob; bg = og; }
      }
      if (lane == 0 && bg != 0x7fffffff) gs[bg] = -2.f;      // kept
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / per] != -2.f) s[e] = -1.f;
    __syncwarp();
  }
  float chosen_sum = 0.f;
  for (int pick = 0; pick < top; ++pick) {
    float best = -0.5f;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = s[e];
      if (v > best) { best = v; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if (be == 0x7fffffff) { be = 0; best = 0.f; }      // nothing left to choose (or the row holds no numbers)
    chosen_sum += best;
    if (lane == 0) {
      idx[(size_t)t * top + pick] = be;
      wts[(size_t)t * top + pick] = best;
      s[be] = -1.f;                                    // taken
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = scale / (chosen_sum + 1e-20f);
    for (int j = 0; j < top; ++j) wts[(size_t)t * top + j] *= inv;
  }
}

AB_API int ab_moe_route(const void* h, int dtype, int ld, const float* wr, int n_tokens, int width, int E, int groups,
                        int keep, int top, float scale, int* idx, float* wts, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (E <= 0 || E > MOE_MAX_EXPERTS || groups <= 0 || E % groups || keep <= 0 || keep > groups || top <= 0 ||
      top > keep * (E / groups))
    return AB_BAD_ARG;
  const int wpb = 4;
  const unsigned blocks = (unsigned)((n_tokens + wpb - 1) / wpb);
  const size_t smem = (size_t)wpb * (E + groups) * sizeof(float);
  if (dtype == AB_F32)
    moe_route_kernel<float><<<blocks, wpb * 32, smem, stream>>>((const float*)h, ld, wr, n_tokens, width, E, groups,
                                                                 keep, top, scale, idx, wts);
  else if (dtype == AB_BF16)
    moe_route_kernel<bf16><<<blocks, wpb * 32, smem, stream>>>((const bf16*)h, ld, wr, n_tokens, width, E, groups, keep,
                                                                top, scale, idx, wts);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f)); }
__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// act[p, j] = f(W_up[e_p][j] . h[t_p]) for pair p = t * top + k.  One warp per (pair, j).
template <typename T>
__global__ void moe_up_pairs_kernel(const T* __restrict__ h, int ld, const T* __restrict__ w_up, const int* __restrict__ idx,
                                    T* __restrict__ act, int n_pairs, int top, int width, int ff, int activation) {
  const int lane = threadIdx.x & 31;
  const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long long)n_pairs * ff) return;
  const int p = (int)(id / ff), j = (int)(id - (long long)p * ff);
  const int e = idx[p];
  const T* x = h + (size_t)(p / top) * ld;
  const T* w = w_up + ((size_t)e * ff + j) * width;
  float part = 0.f;
  for (int k = lane; k < width; k += 32) part += to_f32(x[k]) * to_f32(w[k]);
  part = warp_sum(part);
  if (lane == 0) {
    act[(size_t)p * ff + j] = from_f32<T>(activation == 0 ? gelu_erf(part) : silu(part));
  }
}

// out[t, i] = sum_k wts[t, k] * (W_down[e_k][i] . act[t * top + k]).  One warp per (token, i).
template <typename T>
__global__ void moe_down_pairs_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ idx,
                                      const float* __restrict__ wts, T* __restrict__ out, int n_tokens, int top, int width,
                                      int ff) {
  const int lane = threadIdx.x & 31;
  const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (id >= (long long)n_tokens * width) return;
  const int t = (int)(id / width), i = (int)(id - (long long)t * width);
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    const int e = idx[(size_t)t * top + k];
    const T* a = act + ((size_t)t * top + k) * ff;
    const T* w = w_down + ((size_t)e * width + i) * ff;
    float part = 0.f;
    for (int j = lane; j < ff; j += 32) part += to_f32(a[j]) * to_f32(w[j]);
    total += wts[(size_t)t * top + k] * warp_sum(part);
  }
  if (lane == 0) out[(size_t)t * width + i] = from_f32<T>(total);
}

AB_API int ab_moe_pairs(const void* h, int dtype, int ld, const void* w_up, const void* w_down, const int* idx,
                        const float* wts, void* act, void* out, int n_tokens, int top, int width, int ff, int E,
                        int activation, cudaStream_t stream) {
  if (n_tokens <= 0) return AB_OK;
  if (top <= 0 || width <= 0 || ff <= 0 || E <= 0 || (activation != 0 && activation != 1)) return AB_BAD_ARG;
  const int wpb = 8;
  const long long up_warps = (long long)n_tokens * top * ff, down_warps = (long long)n_tokens * width;
  const long long up_blocks = (up_warps + wpb - 1) / wpb, down_blocks = (down_warps + wpb - 1) / wpb;
  if (up_blocks > 0x7fffffffLL || down_blocks > 0x7fffffffLL) return AB_BAD_ARG;
  if (dtype == AB_F32) {
    moe_up_pairs_kernel<float><<<(unsigned)up_blocks, wpb * 32, 0, stream>>>(
        (const float*)h, ld, (const float*)w_up, idx, (float*)act, n_tokens * top, top, width, ff, activation);
    moe_down_pairs_kernel<float><<<(unsigned)down_blocks, wpb * 32, 0, stream>>>(
        (const float*)act, (const float*)w_down, idx, wts, (float*)out, n_tokens, top, width, ff);
  } else if (dtype == AB_BF16) {
    moe_up_pairs_kernel<bf16><<<(unsigned)up_blocks, wpb * 32, 0, stream>>>(
        (const bf16*)h, ld, (const bf16*)w_up, idx, (bf16*)act, n_tokens * top, top, width, ff, activation);
    moe_down_pairs_kernel<bf16><<<(unsigned)down_blocks, wpb * 32, 0, stream>>>(
        (const bf16*)act, (const bf16*)w_down, idx, wts, (bf16*)out, n_tokens, top, width, ff);
  } else {
    return AB_BAD_ARG;
  }
  return ab_launch_status();
}
