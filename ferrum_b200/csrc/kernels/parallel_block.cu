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
#include "partials.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
scaled_sum_kernel(float* __restrict__ x, const float* __restrict__ y1, const float* __restrict__ y2, float mult,
                  T* __restrict__ xc, long long n) {
  pdl_launch();      // the product that follows may fetch its weights meanwhile
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = y1[i];
  if (y2 != nullptr) s += y2[i];
  const float v = fmaf(mult, s, x[i]);
  x[i] = v;
  if (xc != nullptr) xc[i] = from_f32<T>(v);
}

// The same for a few tokens whose sublayers left their last products as partials (either may instead
// be a plain buffer, the second may be absent): a row is shared out between gridDim.y blocks.
template <typename T>
__global__ void __launch_bounds__(256)
scaled_sum_partials_kernel(float* __restrict__ x, int E, const float* __restrict__ y1, const float* __restrict__ y2, float mult,
                           T* __restrict__ xc, const PartialLayout L1, const PartialLayout L2) {
  pdl_launch();      // the product that follows may fetch its weights meanwhile
  __shared__ PartialTable tab1, tab2;
  if (L1.ws != nullptr) build_partial_table(L1, tab1);
  if (L2.ws != nullptr) build_partial_table(L2, tab2);
  const int t = blockIdx.x;
  const int per = (E + gridDim.y - 1) / gridDim.y;
  const int lo = blockIdx.y * per, hi = min(E, lo + per);
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float s = L1.ws != nullptr ? partial_sum(L1, tab1, t, i) : y1[(size_t)t * E + i];
    if (L2.ws != nullptr) s += partial_sum(L2, tab2, t, i);
    else if (y2 != nullptr) s += y2[(size_t)t * E + i];
    const float v = fmaf(mult, s, x[(size_t)t * E + i]);
    x[(size_t)t * E + i] = v;
    if (xc != nullptr) xc[(size_t)t * E + i] = from_f32<T>(v);
  }
}

__device__ __forceinline__ float pb_gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_table_rows_kernel(const float* __restrict__ s, int lds, const T* __restrict__ table, int ldt, int n_vocab,
                        const int* __restrict__ token_ids, int offset, int dim, T* __restrict__ out, int ldo, int n_tokens,
                        int* __restrict__ err, const PartialLayout L) {
  pdl_launch();      // the product that follows may fetch its weights meanwhile
  __shared__ PartialTable tab;
  if (L.ws != nullptr) build_partial_table(L, tab);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_tokens * dim) return;
  const int t = (int)(i / dim), j = (int)(i % dim);
  const int tok = token_ids[t];
  if (tok < 0 || tok >= n_vocab) {
    atomicExch(err, 1);
    return;
  }
  const float e = to_f32<T>(table[(size_t)tok * ldt + offset + j]);
  const float z = L.ws != nullptr ? partial_sum(L, tab, t, j) : s[(size_t)t * lds + j];
  out[(size_t)t * ldo + j] = from_f32<T>(pb_gelu_tanh(z) * e);
}

// y comes from a plain buffer or from partials; `hold`: the row is kept in shared memory (E floats)
// between the sum of squares and the update (always with partials; a wider row is read twice).
__global__ void __launch_bounds__(256)
norm_scaled_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, float mult, float eps,
                       int E, const PartialLayout L, int hold) {
  pdl_launch();      // the product that follows may fetch its weights meanwhile
  extern __shared__ float pb_row[];
  __shared__ float red[32];
  __shared__ PartialTable tab;
  if (L.ws != nullptr) build_partial_table(L, tab);
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    const float v = L.ws != nullptr ? partial_sum(L, tab, t, i) : y[(size_t)t * E + i];
    if (hold) pb_row[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)E + eps);
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    const float v = hold ? pb_row[i] : y[(size_t)t * E + i];
    x[(size_t)t * E + i] = fmaf(mult, v * r * w[i], x[(size_t)t * E + i]);
  }
}

static int pb_layout(const float* partials, const int* layout, int n_tokens, int width, PartialLayout* L) {
  *L = PartialLayout{nullptr, 0, 0, 0, 0};
  if (partials == nullptr) return 0;
  if (int r = partial_make_layout(partials, layout, L)) return r;
  FERRUM_CHECK_ARG(width <= L->tiles * 128 && n_tokens <= L->acc_cols, "the partials do not cover the rows");
  return 0;
}

// y1 / y2: float32 [n_tokens, E] buffers, or null where partials1 / partials2 (with their layouts) stand in.
FERRUM_API int ferrum_scaled_sum(float* x, const float* y1, const float* y2, float mult, void* xc, int dtype, int n_tokens,
                                 int E, const float* partials1, const int* layout1, const float* partials2,
                                 const int* layout2, cudaStream_t stream) {
  FERRUM_CHECK_ARG(y1 != nullptr || partials1 != nullptr, "scaled_sum: no first term");
  if (n_tokens == 0) return 0;
  if (partials1 != nullptr || partials2 != nullptr) {
    PartialLayout L1, L2;
    if (int r = pb_layout(partials1, layout1, n_tokens, E, &L1)) return r;
    if (int r = pb_layout(partials2, layout2, n_tokens, E, &L2)) return r;
    const int slices = n_tokens <= 64 ? max(1, min(16, E / 256)) : 1;
    FERRUM_DISPATCH_DTYPE(dtype, T, (scaled_sum_partials_kernel<T><<<dim3(n_tokens, slices), 256, 0, stream>>>(
        x, E, y1, y2, mult, (T*)xc, L1, L2)));
    FERRUM_CHECK_LAUNCH("scaled_sum_partials");
    return 0;
  }
  const long long n = (long long)n_tokens * E;
  FERRUM_DISPATCH_DTYPE(dtype, T, (scaled_sum_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, y1, y2, mult, (T*)xc, n)));
  FERRUM_CHECK_LAUNCH("scaled_sum");
  return 0;
}

FERRUM_API int ferrum_gated_table_rows(const float* s, int lds, const void* table, int ldt, int n_vocab, const int* token_ids,
                                       int offset, int dim, void* out, int ldo, int dtype, int n_tokens, int* err,
                                       const float* partials, const int* layout, cudaStream_t stream) {
  FERRUM_CHECK_ARG(dim > 0 && offset >= 0 && offset + dim <= ldt, "gated_table_rows: columns %d..%d are outside a row of %d",
                   offset, offset + dim, ldt);
  FERRUM_CHECK_ARG(s != nullptr || partials != nullptr, "gated_table_rows: no gate input");
  if (n_tokens == 0) return 0;
  PartialLayout L;
  if (int r = pb_layout(partials, layout, n_tokens, dim, &L)) return r;
  const long long n = (long long)n_tokens * dim;
  FERRUM_DISPATCH_DTYPE(dtype, T, (gated_table_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
      s, lds, (const T*)table, ldt, n_vocab, token_ids, offset, dim, (T*)out, ldo, n_tokens, err, L)));
  FERRUM_CHECK_LAUNCH("gated_table_rows");
  return 0;
}

constexpr int PB_MAX_ROW = 11264;      // floats of a row that the norm holds in shared memory

FERRUM_API int ferrum_norm_scaled_add_max_width() { return PB_MAX_ROW; }

FERRUM_API int ferrum_norm_scaled_add(float* x, const float* y, const float* w, float mult, float eps, int n_tokens, int E,
                                      const float* partials, const int* layout, cudaStream_t stream) {
  FERRUM_CHECK_ARG(y != nullptr || partials != nullptr, "norm_scaled_add: no input");
  FERRUM_CHECK_ARG(E > 0 && (partials == nullptr || E <= PB_MAX_ROW), "norm_scaled_add: a row of %d from partials is wider than %d",
                   E, PB_MAX_ROW);
  if (n_tokens == 0) return 0;
  PartialLayout L;
  if (int r = pb_layout(partials, layout, n_tokens, E, &L)) return r;
  const int hold = E <= PB_MAX_ROW;
  norm_scaled_add_kernel<<<n_tokens, 256, hold ? (size_t)E * 4 : 0, stream>>>(x, y, w, mult, eps, E, L, hold);
  FERRUM_CHECK_LAUNCH("norm_scaled_add");
  return 0;
}
