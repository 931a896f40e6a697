// Small kernels on the float32 residual stream that are not a norm before a sub-layer:
//
//   add_row        x[t, :] += row[:]                       a learned vector added to every token (a pass of a loop)
//   stream_cast    x += delta (if given); y = cast(x)      the stream itself as the input of a product
//   token_gate     a[t, j] = act(z[t, j]) * table[token_t, off + j]    a product gated by a per-token table row;
//                  act = gelu_tanh: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   add_unit_norm  x[t, :] += y[t, :] / sqrt(mean(y[t, :]^2) + eps) * w[:]
//
// Arithmetic is 32-bit; rows whose sequence index is negative (padding of a captured step) are left alone by
// the kernels that write the stream.
#include "common.cuh"
#include "launch.cuh"

__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ row, const int* __restrict__ tok_seq,
                               size_t total, int width) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / width;
  if (tok_seq[t] < 0) return;
  x[i] += row[i - t * width];
}

template <typename T>
__global__ void stream_cast_kernel(float* __restrict__ x, const T* __restrict__ delta, T* __restrict__ y, size_t total) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = x[i];
  if (delta != nullptr) {
    v += to_f32(delta[i]);
    x[i] = v;
  }
  y[i] = from_f32<T>(v);
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ z, const T* __restrict__ table, int table_width, int off,
                                  const int* __restrict__ tokens, const int* __restrict__ tok_seq, T* __restrict__ out,
                                  size_t total, int dim) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / dim;
  const int j = (int)(i - t * dim);
  if (tok_seq[t] < 0) { out[i] = from_f32<T>(0.f); return; }
  const float e = to_f32(table[(size_t)tokens[t] * table_width + off + j]);
  out[i] = from_f32<T>(gelu_tanh_f(to_f32(z[i])) * e);
}

// a block per row
__global__ void add_unit_norm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w,
                                     const int* __restrict__ tok_seq, int width, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (tok_seq[t] < 0) return;
  const float* yr = y + (size_t)t * width;
  float ss = 0.f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) ss += yr[j] * yr[j];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  float* xr = x + (size_t)t * width;
  for (int j = threadIdx.x; j < width; j += blockDim.x) xr[j] += yr[j] * inv * w[j];
}

AB_API int ab_add_row(float* x, const float* row, const int* tok_seq, int n_rows, int width, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return AB_OK;
  ab_launch(add_row_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, row, tok_seq, total, width);
  return ab_launch_status();
}

AB_API int ab_stream_cast(float* x, const void* delta, void* y, int dtype, int n_rows, int width, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return AB_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == AB_F32)
    ab_launch(stream_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (const float*)delta, (float*)y, total);
  else if (dtype == AB_BF16)
    ab_launch(stream_cast_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, (const bf16*)delta, (bf16*)y, total);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

AB_API int ab_token_gate(const void* z, const void* table, int table_width, int off, const int* tokens,
                         const int* tok_seq, void* out, int dtype, int n_rows, int dim, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * dim;
  if (total == 0) return AB_OK;
  if (off < 0 || off + dim > table_width) return AB_BAD_ARG;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == AB_F32)
    ab_launch(token_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)z, (const float*)table,
              table_width, off, tokens, tok_seq, (float*)out, total, dim);
  else if (dtype == AB_BF16)
    ab_launch(token_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)z, (const bf16*)table,
              table_width, off, tokens, tok_seq, (bf16*)out, total, dim);
  else
    return AB_BAD_ARG;
  return ab_launch_status();
}

AB_API int ab_add_unit_norm(float* x, const float* y, const float* w, const int* tok_seq, int n_rows, int width, float eps,
                            cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return AB_OK;
  const int threads = width >= 2048 ? 256 : 128;
  ab_launch(add_unit_norm_kernel, dim3((unsigned)n_rows), dim3(threads), 0, stream, x, y, w, tok_seq, width, eps);
  return ab_launch_status();
}
