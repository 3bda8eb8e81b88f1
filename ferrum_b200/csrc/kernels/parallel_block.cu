// Elementwise steps of a block whose sublayers read ONE norm of the residual row and whose results are
// scaled on their way into the float32 residual stream x:
//
// scaled_sum:       x <- x + mult * (y1 + y2)     (y2 may be absent); optionally also x in the compute
//                   type, for a product that reads the new row.
// gated_table_rows: g[t][j] = gelu_tanh(s[t][j]) * table[token[t]][offset + j]   (the per-layer part of a
//                   second embedding table, gated by a projection of the row), compute type out.
// norm_scaled_add:  x <- x + mult * y / sqrt(mean(y^2) + eps) * w    (an RMS norm of the branch's result,
//                   not of x).
// All arithmetic is float32; one block per token for the norm, with a fixed reduction tree.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
scaled_sum_kernel(float* __restrict__ x, const float* __restrict__ y1, const float* __restrict__ y2, float mult,
                  T* __restrict__ xc, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = y1[i];
  if (y2 != nullptr) s += y2[i];
  const float v = fmaf(mult, s, x[i]);
  x[i] = v;
  if (xc != nullptr) xc[i] = from_f32<T>(v);
}

__device__ __forceinline__ float pb_gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_table_rows_kernel(const float* __restrict__ s, int lds, const T* __restrict__ table, int ldt, int n_vocab,
                        const int* __restrict__ token_ids, int offset, int dim, T* __restrict__ out, int ldo, int n_tokens,
                        int* __restrict__ err) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_tokens * dim) return;
  const int t = (int)(i / dim), j = (int)(i % dim);
  const int tok = token_ids[t];
  if (tok < 0 || tok >= n_vocab) {
    atomicExch(err, 1);
    return;
  }
  const float e = to_f32<T>(table[(size_t)tok * ldt + offset + j]);
  out[(size_t)t * ldo + j] = from_f32<T>(pb_gelu_tanh(s[(size_t)t * lds + j]) * e);
}

__global__ void __launch_bounds__(256)
norm_scaled_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, float mult, float eps,
                       int E) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* yr = y + (size_t)t * E;
  float ss = 0.f;
  for (int i = threadIdx.x; i < E; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)E + eps);
  for (int i = threadIdx.x; i < E; i += blockDim.x) x[(size_t)t * E + i] = fmaf(mult, yr[i] * r * w[i], x[(size_t)t * E + i]);
}

FERRUM_API int ferrum_scaled_sum(float* x, const float* y1, const float* y2, float mult, void* xc, int dtype, int n_tokens,
                                 int E, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  const long long n = (long long)n_tokens * E;
  FERRUM_DISPATCH_DTYPE(dtype, T, (scaled_sum_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, y1, y2, mult, (T*)xc, n)));
  FERRUM_CHECK_LAUNCH("scaled_sum");
  return 0;
}

FERRUM_API int ferrum_gated_table_rows(const float* s, int lds, const void* table, int ldt, int n_vocab, const int* token_ids,
                                       int offset, int dim, void* out, int ldo, int dtype, int n_tokens, int* err,
                                       cudaStream_t stream) {
  FERRUM_CHECK_ARG(dim > 0 && offset >= 0 && offset + dim <= ldt, "gated_table_rows: columns %d..%d are outside a row of %d",
                   offset, offset + dim, ldt);
  if (n_tokens == 0) return 0;
  const long long n = (long long)n_tokens * dim;
  FERRUM_DISPATCH_DTYPE(dtype, T, (gated_table_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
      s, lds, (const T*)table, ldt, n_vocab, token_ids, offset, dim, (T*)out, ldo, n_tokens, err)));
  FERRUM_CHECK_LAUNCH("gated_table_rows");
  return 0;
}

FERRUM_API int ferrum_norm_scaled_add(float* x, const float* y, const float* w, float mult, float eps, int n_tokens, int E,
                                      cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  norm_scaled_add_kernel<<<n_tokens, 256, 0, stream>>>(x, y, w, mult, eps, E);
  FERRUM_CHECK_LAUNCH("norm_scaled_add");
  return 0;
}
