// The matrix-memory recurrence (mLSTM) over packed sequences, 32-bit arithmetic throughout.
//
// Per head, with log input gate gi_t = cap tanh((zi_t + bi) / cap) and log forget gate
// gf_t = logsigmoid(cap tanh((zf_t + bf) / cap)), a running maximum m (m_0 = 0) and S_0 = 0, n_0 = 0:
//   m_t = max(gf_t + m_{t-1}, gi_t)
//   S_t = exp(gf_t + m_{t-1} - m_t) S_{t-1} + exp(gi_t - m_t) k_t v_t^T        [D, V]
//   n_t = (the same two factors) n_{t-1}, k_t                                     [D]
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t scaled by qscale
// Three kernels:
//   gates    one warp per (sequence, head) walks the tokens: the two factors and the denominator of every
//            token (n and m live here);
//   state    one CTA per (sequence, head, tile of columns of S): each thread owns one column of S, in
//            registers when D is 16, 32, 64 or 128 and in shared memory otherwise, and walks the tokens;
//            columns need nothing from each other, so no barrier is inside the loop;
//   output   per (token, head): o divided by its root mean square, times a weight, times sigmoid(gate).
// The state of a sequence is read when the step starts and written back when it ends, so a prompt can be
// cut anywhere and a decode step is the same code with one token.  A row of the state per (slot, head):
// S [D][V] | n [D] | m | padding to a multiple of 4 floats.
// The projections come as one float32 row per token: q | k | v | g | zi | zf at given offsets.
#include "common.cuh"

struct MlstmArgs {
  const float* proj;       // [T, ld]
  int ld, off_q, off_k, off_v, off_g, off_i, off_f;
  const float* bias_i;     // [H]
  const float* bias_f;     // [H]
  float* state;            // [slots, H, row]
  int row;                 // floats per (slot, head)
  int H, D, V;
  const int* cu_q;         // [B + 1]
  const int* slots;        // [B]
  const int* tok_seq;      // [T], -1: a row without a sequence
  float cap, qscale;
  float* coef;             // [T, H, 3]: keep, add, denominator
  float* o_raw;            // [T, H, V]
  int write_state;
};

__device__ __forceinline__ float log_sigmoid(float x) {
  return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x));
}

// DPL: dims of n per lane
template <int DPL>
__global__ void mlstm_gates_kernel(MlstmArgs a, int n_pairs) {
  const int lane = threadIdx.x & 31;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_pairs) return;
  const int b = w / a.H, h = w - b * a.H;
  const int t0 = a.cu_q[b], t1 = a.cu_q[b + 1];
  const int slot = a.slots[b];
  if (slot < 0 || t1 <= t0 || a.tok_seq[t0] < 0) return;
  float* st = a.state + ((size_t)slot * a.H + h) * a.row;
  float* sn = st + (size_t)a.D * a.V;
  float n[DPL];
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    const int d = lane + 32 * j;
    n[j] = d < a.D ? sn[d] : 0.f;
  }
  float m = sn[a.D];
  const float bi = a.bias_i[h], bf = a.bias_f[h];
  for (int t = t0; t < t1; ++t) {
    const float* p = a.proj + (size_t)t * a.ld;
    const float gi = a.cap * tanhf((p[a.off_i + h] + bi) / a.cap);
    const float gf = log_sigmoid(a.cap * tanhf((p[a.off_f + h] + bf) / a.cap));
    const float m_new = fmaxf(gf + m, gi);
    const float keep = expf(gf + m - m_new), add = expf(gi - m_new);
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int d = lane + 32 * j;
      if (d < a.D) {
        n[j] = keep * n[j] + add * p[a.off_k + h * a.D + d];
        part += n[j] * (p[a.off_q + h * a.D + d] * a.qscale);
      }
    }
    const float nq = warp_sum(part);
    m = m_new;
    if (lane == 0) {
      float* c = a.coef + ((size_t)t * a.H + h) * 3;
      c[0] = keep;
      c[1] = add;
      c[2] = fmaxf(fabsf(nq), expf(-m_new)) + 1e-6f;
    }
  }
  if (a.write_state) {
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int d = lane + 32 * j;
      if (d < a.D) sn[d] = n[j];
    }
    if (lane == 0) sn[a.D] = m;
  }
}

// One thread per column of S.  DR > 0: the column's D = DR entries live in registers; DR = 0: in shared
// memory, [d][column of the tile].
template <int DR>
__global__ void mlstm_state_kernel(MlstmArgs a) {
  extern __shared__ float smem[];
  const int b = blockIdx.x, h = blockIdx.y;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  const int t0 = a.cu_q[b], t1 = a.cu_q[b + 1];
  const int slot = a.slots[b];
  if (slot < 0 || t1 <= t0 || a.tok_seq[t0] < 0) return;
  const bool live = c < a.V;
  const int D = DR > 0 ? DR : a.D;
  float* st = a.state + ((size_t)slot * a.H + h) * a.row;
  float reg[DR > 0 ? DR : 1];
  float* col = smem + threadIdx.x;      // entry d at col[d * blockDim.x]
  const int cs = blockDim.x;
  if (live) {
    if (DR > 0) {
#pragma unroll
      for (int d = 0; d < DR; ++d) reg[d] = st[(size_t)d * a.V + c];
    } else {
      for (int d = 0; d < D; ++d) col[d * cs] = st[(size_t)d * a.V + c];
    }
  }
  for (int t = t0; t < t1; ++t) {
    const float* p = a.proj + (size_t)t * a.ld;
    const float* cf = a.coef + ((size_t)t * a.H + h) * 3;
    const float keep = cf[0], add = cf[1], den = cf[2];
    const float* kk = p + a.off_k + h * D;
    const float* qq = p + a.off_q + h * D;
    if (!live) continue;
    const float av = add * p[a.off_v + h * a.V + c];
    float acc = 0.f;
    if (DR > 0) {
#pragma unroll
      for (int d = 0; d < DR; d += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kk + d);
        const float4 q4 = *reinterpret_cast<const float4*>(qq + d);
        reg[d] = keep * reg[d] + av * k4.x;
        acc += reg[d] * q4.x;
        reg[d + 1] = keep * reg[d + 1] + av * k4.y;
        acc += reg[d + 1] * q4.y;
        reg[d + 2] = keep * reg[d + 2] + av * k4.z;
        acc += reg[d + 2] * q4.z;
        reg[d + 3] = keep * reg[d + 3] + av * k4.w;
        acc += reg[d + 3] * q4.w;
      }
    } else {
      for (int d = 0; d < D; ++d) {
        const float s = keep * col[d * cs] + av * kk[d];
        col[d * cs] = s;
        acc += s * qq[d];
      }
    }
    a.o_raw[((size_t)t * a.H + h) * a.V + c] = acc * a.qscale / den;
  }
  if (a.write_state && live) {
    if (DR > 0) {
#pragma unroll
      for (int d = 0; d < DR; ++d) st[(size_t)d * a.V + c] = reg[d];
    } else {
      for (int d = 0; d < D; ++d) st[(size_t)d * a.V + c] = col[d * cs];
    }
  }
}

// out[t, h*V + c] = o / rms(o over the head) * weight[h*V + c] * sigmoid(g[t, h*V + c]); one warp per (token, head)
template <typename T>
__global__ void mlstm_output_kernel(const float* __restrict__ o_raw, const float* __restrict__ proj, int ld, int off_g,
                                    const float* __restrict__ weight, const int* __restrict__ tok_seq, T* __restrict__ out,
                                    int n_tokens, int H, int V, float eps) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * H) return;
  const int t = (int)(w / H), h = (int)(w - (long long)t * H);
  T* y = out + ((size_t)t * H + h) * V;
  if (tok_seq[t] < 0) {
    for (int c = lane; c < V; c += 32) y[c] = from_f32<T>(0.f);
    return;
  }
  const float* o = o_raw + ((size_t)t * H + h) * V;
  float ss = 0.f;
  for (int c = lane; c < V; c += 32) ss += o[c] * o[c];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  const float* g = proj + (size_t)t * ld + off_g + h * V;
  for (int c = lane; c < V; c += 32) {
    const float gate = 1.0f / (1.0f + expf(-g[c]));
    y[c] = from_f32<T>(o[c] * inv * weight[h * V + c] * gate);
  }
}

AB_API int ab_mlstm_step(const float* proj, int ld, int off_q, int off_k, int off_v, int off_g, int off_i, int off_f,
                         const float* bias_i, const float* bias_f, float* state, int row, int H, int D, int V,
                         const int* cu_q, const int* slots, const int* tok_seq, int n_seqs, int n_tokens, float cap,
                         float qscale, float* coef, float* o_raw, const float* weight, float eps, void* out,
                         int out_dtype, int write_state, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return AB_OK;
  if (H <= 0 || D <= 0 || V <= 0 || D > 1024 || row < D * V + D + 1) return AB_BAD_ARG;
  MlstmArgs a{proj, ld, off_q, off_k, off_v, off_g, off_i, off_f, bias_i, bias_f, state, row, H, D, V, cu_q, slots,
              tok_seq, cap, qscale, coef, o_raw, write_state};
  {
    const int pairs = n_seqs * H, wpb = 4;
    const unsigned blocks = (unsigned)((pairs + wpb - 1) / wpb);
    const int dpl = (D + 31) / 32;
    if (dpl <= 1) mlstm_gates_kernel<1><<<blocks, wpb * 32, 0, stream>>>(a, pairs);
    else if (dpl <= 2) mlstm_gates_kernel<2><<<blocks, wpb * 32, 0, stream>>>(a, pairs);
    else if (dpl <= 4) mlstm_gates_kernel<4><<<blocks, wpb * 32, 0, stream>>>(a, pairs);
    else if (dpl <= 8) mlstm_gates_kernel<8><<<blocks, wpb * 32, 0, stream>>>(a, pairs);
    else mlstm_gates_kernel<32><<<blocks, wpb * 32, 0, stream>>>(a, pairs);
    int rc = ab_launch_status();
    if (rc) return rc;
  }
  {
    // columns per CTA: few, so that a prompt of one sequence still spreads over many processors
    const int tile = V >= 256 ? 64 : 32;
    dim3 grid((unsigned)n_seqs, (unsigned)H, (unsigned)((V + tile - 1) / tile));
    const bool aligned = D % 4 == 0 && (off_q % 4 == 0) && (off_k % 4 == 0) && (ld % 4 == 0);
    if (aligned && D == 16) mlstm_state_kernel<16><<<grid, tile, 0, stream>>>(a);
    else if (aligned && D == 32) mlstm_state_kernel<32><<<grid, tile, 0, stream>>>(a);
    else if (aligned && D == 64) mlstm_state_kernel<64><<<grid, tile, 0, stream>>>(a);
    else if (aligned && D == 128) mlstm_state_kernel<128><<<grid, tile, 0, stream>>>(a);
    else {
      const size_t smem = (size_t)D * tile * sizeof(float);
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(mlstm_state_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return AB_CUDA_ERR + (int)e;
      }
      mlstm_state_kernel<0><<<grid, tile, smem, stream>>>(a);
    }
    int rc = ab_launch_status();
    if (rc) return rc;
  }
  {
    const long long warps = (long long)n_tokens * H;
    const int wpb = 4;
    const unsigned blocks = (unsigned)((warps + wpb - 1) / wpb);
    if (out_dtype == AB_F32)
      mlstm_output_kernel<float><<<blocks, wpb * 32, 0, stream>>>(o_raw, proj, ld, off_g, weight, tok_seq, (float*)out,
                                                                   n_tokens, H, V, eps);
    else if (out_dtype == AB_BF16)
      mlstm_output_kernel<bf16><<<blocks, wpb * 32, 0, stream>>>(o_raw, proj, ld, off_g, weight, tok_seq, (bf16*)out,
                                                                  n_tokens, H, V, eps);
    else
      return AB_BAD_ARG;
  }
  return ab_launch_status();
}
