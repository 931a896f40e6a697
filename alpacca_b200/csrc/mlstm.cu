// The matrix-memory recurrence (mLSTM) over packed sequences, 32-bit arithmetic throughout.
//
// Per head, with log input gate gi_t = cap tanh((zi_t + bi) / cap) and log forget gate
// gf_t = logsigmoid(cap tanh((zf_t + bf) / cap)), a running maximum m (m_0 = 0) and S_0 = 0, n_0 = 0:
//   m_t = max(gf_t + m_{t-1}, gi_t)
//   S_t = exp(gf_t + m_{t-1} - m_t) S_{t-1} + exp(gi_t - m_t) k_t v_t^T        [D, V]
//   n_t = (the same two factors) n_{t-1}, k_t                                     [D]
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t scaled by qscale
// Three kernels, in two forms.  The form for D a multiple of 16 up to 256 (rows 16-byte aligned):
//   scan     one warp per (sequence, head): the gates of 32 tokens at a time, in parallel, the running maximum
//            by a scan over the warp; leaves (keep, add, m) per token;
//   state    one CTA per (sequence, head, 8 or 32 columns of [S | n]): n is one more column of S, the one whose
//            value is 1.  A column's D entries are spread over 16 (4) threads' registers; q, k, v and the
//            factors of 4 to 16 tokens at a time are brought to shared memory by cp.async, three buffers, so
//            that the walk over the tokens does not wait for memory; leaves S^T q and n . q;
//   output   per (token, head): the denominator from n . q and m, o divided by its root mean square, times a
//            weight, times sigmoid(gate).
// The general form (any D up to 1024): `gates` (one warp per (sequence, head) walks the tokens and keeps n) and a
// `state` whose threads each own one whole column, in shared memory; it leaves o already divided.
// The state of a sequence is read when the step starts and written back when it ends, so a prompt can be
// cut anywhere and a decode step is the same code with one token.  A row of the state per (slot, head):
// S [D][V] | n [D] | m | padding to a multiple of 4 floats.
// The projections come as one float32 row per token: q | k | v | g | zi | zf at given offsets.
#include "common.cuh"
#include "launch.cuh"

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
  float* coef;             // [T, H, 3]: keep, add, and the denominator (general form) or m (fast form)
  float* o_raw;            // [T, H, V + 1]
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
    a.o_raw[((size_t)t * a.H + h) * (a.V + 1) + c] = acc * a.qscale / den;
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

// ---------------------------------------------------------------------------------------------
// the fast form
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void mlstm_scan_kernel(MlstmArgs a, int n_pairs) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= n_pairs) return;
  const int b = w / a.H, h = w - b * a.H;
  const int t0 = a.cu_q[b], t1 = a.cu_q[b + 1];
  const int slot = a.slots[b];
  if (slot < 0 || t1 <= t0 || a.tok_seq[t0] < 0) return;
  float* sm_ = a.state + ((size_t)slot * a.H + h) * a.row + (size_t)a.D * a.V + a.D;
  float m = *sm_;
  const float bi = a.bias_i[h], bf = a.bias_f[h];
  for (int base = t0; base < t1; base += 32) {
    const int t = base + lane;
    float gi = 0.f, gf = 0.f;
    if (t < t1) {
      const float* p = a.proj + (size_t)t * a.ld;
      gi = a.cap * tanhf((p[a.off_i + h] + bi) / a.cap);
      gf = log_sigmoid(a.cap * tanhf((p[a.off_f + h] + bf) / a.cap));
    }
    // m' = max(m + gf, gi) is the map m -> max(m + A, B); two such maps in a row are one again,
    // (A1 + A2, max(B1 + A2, B2)), so the 32 tokens' maps are combined by a scan over the warp
    float A = t < t1 ? gf : 0.f, B = t < t1 ? gi : -INFINITY;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float pa = __shfl_up_sync(0xffffffffu, A, o), pb = __shfl_up_sync(0xffffffffu, B, o);
      if (lane >= o) { B = fmaxf(pb + A, B); A = pa + A; }
    }
    const float m_after = fmaxf(m + A, B);
    float m_before = __shfl_up_sync(0xffffffffu, m_after, 1);
    if (lane == 0) m_before = m;
    m = __shfl_sync(0xffffffffu, m_after, 31);      // lanes past the end hold the identity map
    if (t < t1) {
      float* c = a.coef + ((size_t)t * a.H + h) * 3;
      c[0] = expf(gf + m_before - m_after);
      c[1] = expf(gi - m_after);
      c[2] = m_after;
    }
  }
  if (a.write_state && lane == 0) *sm_ = m;
}

// A column's D entries are spread over DG threads of a warp, DQ = D / DG each (DG 16 when D is a multiple of
// 64, else 4); a warp holds 32 / DG columns, the CTA of four warps COLS = 128 / DG.  TB tokens per buffer.
// Per token a thread updates its DQ entries and leaves its share of the column's dot product with q in shared
// memory; the shares of a buffer's tokens are added after its last token, so that the walk over the tokens
// has neither a shuffle nor a barrier in it.
template <int DQ, int DG, int TB>
__global__ void __launch_bounds__(128) mlstm_state_fast_kernel(MlstmArgs a) {
  constexpr int NBUF = 3;                               // buffers of TB tokens: two are on their way while one is read
  constexpr int D = DQ * DG;
  constexpr int COLS = 128 / DG;
  constexpr int SP = ((DQ / 4) & 1) ? DQ : DQ + 4;      // floats between two threads' parts: 4 x odd, no bank met twice
  constexpr int KP = DG * SP;
  __shared__ __align__(16) float ks[NBUF][TB][KP];
  __shared__ __align__(16) float qs[NBUF][TB][KP];
  __shared__ float vs[NBUF][TB][COLS];
  __shared__ float cs[NBUF][TB][2];
  __shared__ float part[TB][COLS][DG + 1];
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dg = lane % DG;                         // which part of the column
  const int col = warp * (32 / DG) + lane / DG;     // column within the CTA's COLS
  const int c = blockIdx.z * COLS + col;            // column of [S | n]: c == V is n
  const int t0 = a.cu_q[b], t1 = a.cu_q[b + 1];
  const int slot = a.slots[b];
  if (slot < 0 || t1 <= t0 || a.tok_seq[t0] < 0) return;
  const int V = a.V;
  const bool live = c <= V;
  float* st = a.state + ((size_t)slot * a.H + h) * a.row;
  float* sn = st + (size_t)D * V;
  float reg[DQ];
#pragma unroll
  for (int d = 0; d < DQ; ++d) {
    const int dd = dg * DQ + d;
    reg[d] = !live ? 0.f : (c < V ? st[(size_t)dd * V + c] : sn[dd]);
  }
  const int n_blocks = (t1 - t0 + TB - 1) / TB;
  auto stage = [&](int blk) {          // every call closes one group of copies, an empty one past the end
    const int buf = blk % NBUF;
    const int tb0 = t0 + blk * TB;
    const int n = blk < n_blocks ? min(TB, t1 - tb0) : 0;
    for (int i = tid; i < n * (D / 4); i += 128) {
      const int tok = i / (D / 4), ch = i - tok * (D / 4);
      const int p_ = (ch * 4) / DQ, within = ch * 4 - p_ * DQ;
      const float* p = a.proj + (size_t)(tb0 + tok) * a.ld;
      cp_async_16(&ks[buf][tok][p_ * SP + within], p + a.off_k + h * D + ch * 4);
      cp_async_16(&qs[buf][tok][p_ * SP + within], p + a.off_q + h * D + ch * 4);
    }
    for (int i = tid; i < n * COLS; i += 128) {
      const int tok = i / COLS, cc = i - tok * COLS;
      const int gc = blockIdx.z * COLS + cc;
      if (gc < V) cp_async_4(&vs[buf][tok][cc], a.proj + (size_t)(tb0 + tok) * a.ld + a.off_v + h * V + gc);
    }
    for (int i = tid; i < n * 2; i += 128) {
      const int tok = i >> 1, j = i & 1;
      cp_async_4(&cs[buf][tok][j], a.coef + ((size_t)(tb0 + tok) * a.H + h) * 3 + j);
    }
    cp_async_commit();
  };
  for (int blk = 0; blk < NBUF - 1; ++blk) stage(blk);
  for (int blk = 0; blk < n_blocks; ++blk) {
    const int buf = blk % NBUF;
    stage(blk + NBUF - 1);             // into the buffer that the barrier at the end of the last round set free
    cp_async_wait<NBUF - 1>();         // all but the latest NBUF - 1 groups have landed: this round's buffer has
    __syncthreads();
    const int tb0 = t0 + blk * TB;
    const int n = min(TB, t1 - tb0);
#pragma unroll 4
    for (int i = 0; i < n; ++i) {
      const float keep = cs[buf][i][0], add = cs[buf][i][1];
      const float av = !live ? 0.f : add * (c < V ? vs[buf][i][col] : 1.0f);
      const float* kk = &ks[buf][i][dg * SP];
      const float* qq = &qs[buf][i][dg * SP];
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int d = 0; d < DQ; d += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kk + d);
        const float4 q4 = *reinterpret_cast<const float4*>(qq + d);
        reg[d] = keep * reg[d] + av * k4.x;
        acc0 += reg[d] * q4.x;
        reg[d + 1] = keep * reg[d + 1] + av * k4.y;
        acc1 += reg[d + 1] * q4.y;
        reg[d + 2] = keep * reg[d + 2] + av * k4.z;
        acc0 += reg[d + 2] * q4.z;
        reg[d + 3] = keep * reg[d + 3] + av * k4.w;
        acc1 += reg[d + 3] * q4.w;
      }
      part[i][col][dg] = acc0 + acc1;
    }
    __syncthreads();
    for (int i = tid; i < n * COLS; i += 128) {
      const int tok = i / COLS, cc = i - tok * COLS;
      const int gc = blockIdx.z * COLS + cc;
      if (gc <= V) {
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < DG; ++j) sum += part[tok][cc][j];
        a.o_raw[((size_t)(tb0 + tok) * a.H + h) * (V + 1) + gc] = sum * a.qscale;
      }
    }
    __syncthreads();
  }
  if (a.write_state && live) {
#pragma unroll
    for (int d = 0; d < DQ; ++d) {
      const int dd = dg * DQ + d;
      if (c < V) st[(size_t)dd * V + c] = reg[d]; else sn[dd] = reg[d];
    }
  }
}

// out[t, h*V + c] = o / rms(o over the head) * weight[h*V + c] * sigmoid(g[t, h*V + c]); one warp per (token, head)
// raw: o_raw holds S^T q and, in column V, n . q, and coef's third number is m: the denominator is formed here.
template <typename T>
__global__ void mlstm_output_kernel(const float* __restrict__ o_raw, const float* __restrict__ proj, int ld, int off_g,
                                    const float* __restrict__ weight, const int* __restrict__ tok_seq, T* __restrict__ out,
                                    int n_tokens, int H, int V, float eps, const float* __restrict__ coef, int raw) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * H) return;
  const int t = (int)(w / H), h = (int)(w - (long long)t * H);
  T* y = out + ((size_t)t * H + h) * V;
  if (tok_seq[t] < 0) {
    for (int c = lane; c < V; c += 32) y[c] = from_f32<T>(0.f);
    return;
  }
  const float* o = o_raw + ((size_t)t * H + h) * (V + 1);
  float scale = 1.0f;
  if (raw) scale = 1.0f / (fmaxf(fabsf(o[V]), expf(-coef[((size_t)t * H + h) * 3 + 2])) + 1e-6f);
  float ss = 0.f;
  for (int c = lane; c < V; c += 32) ss += (o[c] * scale) * (o[c] * scale);
  ss = warp_sum(ss);
  const float inv = scale / sqrtf(ss / (float)V + eps);
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
  const bool fast = D % 16 == 0 && D <= 256 && off_q % 4 == 0 && off_k % 4 == 0 && ld % 4 == 0;
  if (fast) {
    const int pairs = n_seqs * H, wpb = 4;
    ab_launch(mlstm_scan_kernel, dim3((unsigned)((pairs + wpb - 1) / wpb)), dim3(wpb * 32), 0, stream, a, pairs);
    int rc = ab_launch_status();
    if (rc) return rc;
    const int cols = D % 64 == 0 ? 8 : 32;
    dim3 grid((unsigned)n_seqs, (unsigned)H, (unsigned)((V + 1 + cols - 1) / cols));
    switch (D / 16) {
#define AB_FAST(N, DQ, DG, TB) \
  case N: ab_launch(mlstm_state_fast_kernel<DQ, DG, TB>, grid, dim3(128), 0, stream, a); break;
      AB_FAST(1, 4, 4, 16) AB_FAST(2, 8, 4, 16) AB_FAST(3, 12, 4, 16) AB_FAST(4, 4, 16, 16) AB_FAST(5, 20, 4, 8)
      AB_FAST(6, 24, 4, 8) AB_FAST(7, 28, 4, 8) AB_FAST(8, 8, 16, 8) AB_FAST(9, 36, 4, 4) AB_FAST(10, 40, 4, 4)
      AB_FAST(11, 44, 4, 4) AB_FAST(12, 12, 16, 8) AB_FAST(13, 52, 4, 4) AB_FAST(14, 56, 4, 4) AB_FAST(15, 60, 4, 4)
      AB_FAST(16, 16, 16, 4)
#undef AB_FAST
      default: return AB_BAD_ARG;
    }
    rc = ab_launch_status();
    if (rc) return rc;
  } else {
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
    const int tile = (V >= 256 && (size_t)D * 64 * sizeof(float) <= 160 * 1024) ? 64 : 32;   // [D][tile] floats must fit
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
  }
  {
    const long long warps = (long long)n_tokens * H;
    const int wpb = 4;
    const unsigned blocks = (unsigned)((warps + wpb - 1) / wpb);
    if (out_dtype == AB_F32)
      ab_launch(mlstm_output_kernel<float>, dim3(blocks), dim3(wpb * 32), 0, stream, (const float*)o_raw, proj, ld, off_g,
                weight, tok_seq, (float*)out, n_tokens, H, V, eps, (const float*)coef, fast ? 1 : 0);
    else if (out_dtype == AB_BF16)
      ab_launch(mlstm_output_kernel<bf16>, dim3(blocks), dim3(wpb * 32), 0, stream, (const float*)o_raw, proj, ld, off_g,
                weight, tok_seq, (bf16*)out, n_tokens, H, V, eps, (const float*)coef, fast ? 1 : 0);
    else
      return AB_BAD_ARG;
  }
  return ab_launch_status();
}
