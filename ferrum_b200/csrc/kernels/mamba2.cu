// A selective state-space mixer with a scalar decay per head (the Mamba-2 recurrence), after its
// input product.  A token's float32 product row is [z: inner | x: inner | B: G N | C: G N | dt: heads]
// with inner = heads * P.  Per request the state row keeps, in float32,
//   S [heads][P][N]                      the recurrent state (element (n, p) of head h at (h P + p) N + n)
//   u [taps - 1][channels]               the last inputs of the short convolution (channels = inner + 2 G N)
//
// mamba_conv:        xBC <- silu(bias + sum_j w[c][j] * input(t - (taps - 1 - j))[c]); an input before the
//                    portion's first token comes from u, which is all zero before a sequence's first token.
// mamba_conv_state:  u <- the last taps - 1 inputs after this portion (old rows move up when the portion
//                    is shorter than that).  A launch of its own, so that nobody reads u while it changes.
// mamba_scan:        per (request, head, p) one warp walks the portion's tokens in order; lane l holds
//                    S[n] for n = l, l + 32, ...:
//                      dt = softplus(dt_raw + dt_bias[h]);  S[n] <- exp(-exp(A_log[h]) dt) S[n] + dt B[n] x[p]
//                      y[p] = sum_n S[n] C[n] + D[h] x[p]
//                    The sum over n has one fixed tree, and the walk is token by token whatever the
//                    portion: a token's result does not depend on how the sequence was cut.
// mamba_gate_norm:   v = y * silu(z); each of `norm_groups` equal parts of the row is divided by its own
//                    root mean square and multiplied by the weight; out in the compute type.
#include "common.cuh"

constexpr int MS_WARPS = 8;
constexpr int MS_MAX_TAPS = 16;

__device__ __forceinline__ float ms_silu(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float ms_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

__global__ void __launch_bounds__(256)
mamba_conv_kernel(const float* __restrict__ proj, int ldp, int off_xbc, int C, int taps, const float* __restrict__ w,
                  const float* __restrict__ bias, const float* __restrict__ state, long long state_stride,
                  long long conv_off, const int* __restrict__ req_of_token, const int* __restrict__ q_start,
                  const int* __restrict__ slots, float* __restrict__ out, int n_tokens) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * C) return;
  const int t = (int)(idx / C), c = (int)(idx % C);
  const int r = req_of_token[t];
  const int t0 = q_start[r];
  const int local = t - t0;
  const float* u = state + (long long)slots[r] * state_stride + conv_off;
  float acc = bias[c];
  for (int j = 0; j < taps; ++j) {
    const int src = local - (taps - 1 - j);
    const float v = src >= 0 ? proj[(size_t)(t0 + src) * ldp + off_xbc + c] : u[(size_t)(taps - 1 + src) * C + c];
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  out[(size_t)t * C + c] = ms_silu(acc);
}

__global__ void __launch_bounds__(256)
mamba_conv_state_kernel(const float* __restrict__ proj, int ldp, int off_xbc, int C, int taps, float* __restrict__ state,
                        long long state_stride, long long conv_off, const int* __restrict__ q_start,
                        const int* __restrict__ slots, int n_reqs) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_reqs * C) return;
  const int r = (int)(idx / C), c = (int)(idx % C);
  const int t0 = q_start[r], n = q_start[r + 1] - t0;
  float* u = state + (long long)slots[r] * state_stride + conv_off;
  float keep[MS_MAX_TAPS];
#pragma unroll
  for (int s = 0; s < MS_MAX_TAPS; ++s) {
    if (s < taps - 1) {
      const int src = n - (taps - 1) + s;            // position within the portion of the input that row s will hold
      keep[s] = src >= 0 ? proj[(size_t)(t0 + src) * ldp + off_xbc + c] : u[(size_t)(taps - 1 + src) * C + c];
    }
  }
#pragma unroll
  for (int s = 0; s < MS_MAX_TAPS; ++s)
    if (s < taps - 1) u[(size_t)s * C + c] = keep[s];
}

template <int NK>
__global__ void __launch_bounds__(MS_WARPS * 32)
mamba_scan_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ proj, int ldp, int off_dt,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                  const int* __restrict__ slots, float* __restrict__ y, int heads, int P, int N, int groups) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = blockIdx.x * MS_WARPS + warp, h = blockIdx.y, r = blockIdx.z;
  if (p >= P) return;
  const int inner = heads * P;
  const int g = h / (heads / groups);
  const int t0 = q_start[r], t1 = q_start[r + 1];
  float* S = state + (long long)slots[r] * state_stride + ((long long)h * P + p) * N;
  float s[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) s[k] = lane + 32 * k < N ? S[lane + 32 * k] : 0.f;
  const float a = expf(a_log[h]), db = dt_bias[h], dsk = d_skip[h];
  const int off_b = inner + g * N, off_c = inner + groups * N + g * N;
#pragma unroll 2
  for (int t = t0; t < t1; ++t) {
    const float* row = xbc + (size_t)t * C;
    const float dt = ms_softplus(proj[(size_t)t * ldp + off_dt + h] + db);
    const float decay = expf(-a * dt);
    const float x = row[h * P + p];
    const float dtx = dt * x;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < NK; ++k) {
      const int n = lane + 32 * k;
      const float b = n < N ? row[off_b + n] : 0.f, c = n < N ? row[off_c + n] : 0.f;
      s[k] = fmaf(decay, s[k], dtx * b);
      acc = fmaf(s[k], c, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)t * inner + h * P + p] = fmaf(dsk, x, acc);
  }
#pragma unroll
  for (int k = 0; k < NK; ++k)
    if (lane + 32 * k < N) S[lane + 32 * k] = s[k];
}

template <typename T>
__global__ void __launch_bounds__(256)
mamba_gate_norm_kernel(const float* __restrict__ y, int inner, const float* __restrict__ proj, int ldp, int off_z,
                       const float* __restrict__ w, T* __restrict__ out, int ldo, int norm_groups, float eps) {
  __shared__ float red[32];
  const int t = blockIdx.x, grp = blockIdx.y;
  const int width = inner / norm_groups;
  const float* yr = y + (size_t)t * inner + (size_t)grp * width;
  const float* zr = proj + (size_t)t * ldp + off_z + (size_t)grp * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = yr[i] * ms_silu(zr[i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float mult = 1.f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = yr[i] * ms_silu(zr[i]);
    out[(size_t)t * ldo + (size_t)grp * width + i] = from_f32<T>(v * mult * w[(size_t)grp * width + i]);
  }
}

// proj: the input product's float32 rows; xbc [n_tokens, C] and y [n_tokens, inner]: float32 scratch;
// out [n_tokens, inner] in `dtype`; state: the requests' float32 state rows (see the top of the file).
FERRUM_API int ferrum_mamba2_mix(const float* proj, int ldp, int n_tokens, int n_reqs, const int* req_of_token,
                                 const int* q_start, const int* slots, const float* conv_w, const float* conv_b, int taps,
                                 const float* dt_bias, const float* a_log, const float* d_skip, const float* norm_w,
                                 int heads, int P, int N, int groups, int norm_groups, float eps, float* state,
                                 long long state_stride, float* xbc, float* y, void* out, int ldo, int dtype,
                                 cudaStream_t stream) {
  FERRUM_CHECK_ARG(heads > 0 && P > 0 && N > 0 && groups > 0 && heads % groups == 0, "mamba2: bad sizes");
  FERRUM_CHECK_ARG(N <= 256, "mamba2: a state of %d per head and element is more than 256", N);
  FERRUM_CHECK_ARG(taps >= 1 && taps <= MS_MAX_TAPS, "mamba2: %d convolution taps are outside [1, %d]", taps, MS_MAX_TAPS);
  const int inner = heads * P;
  FERRUM_CHECK_ARG(norm_groups > 0 && inner % norm_groups == 0, "mamba2: %d norm groups do not divide %d", norm_groups, inner);
  FERRUM_CHECK_ARG(heads <= 65535 && n_reqs <= 65535 && norm_groups <= 65535, "mamba2: too many heads, requests or groups");
  if (n_tokens == 0) return 0;
  const int C = inner + 2 * groups * N;
  const int off_xbc = inner, off_dt = inner + C;
  const long long conv_off = (long long)inner * N;
  {
    const long long n = (long long)n_tokens * C;
    mamba_conv_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(proj, ldp, off_xbc, C, taps, conv_w, conv_b, state,
                                                                      state_stride, conv_off, req_of_token, q_start, slots,
                                                                      xbc, n_tokens);
    FERRUM_CHECK_LAUNCH("mamba_conv");
  }
  if (taps > 1) {
    const long long n = (long long)n_reqs * C;
    mamba_conv_state_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(proj, ldp, off_xbc, C, taps, state, state_stride,
                                                                            conv_off, q_start, slots, n_reqs);
    FERRUM_CHECK_LAUNCH("mamba_conv_state");
  }
  {
    const dim3 grid((P + MS_WARPS - 1) / MS_WARPS, heads, n_reqs);
#define MS_SCAN(NK_)                                                                                                   \
  mamba_scan_kernel<NK_><<<grid, MS_WARPS * 32, 0, stream>>>(xbc, C, proj, ldp, off_dt, dt_bias, a_log, d_skip, state, \
                                                            state_stride, q_start, slots, y, heads, P, N, groups)
    if (N <= 32) MS_SCAN(1);
    else if (N <= 64) MS_SCAN(2);
    else if (N <= 128) MS_SCAN(4);
    else MS_SCAN(8);
#undef MS_SCAN
    FERRUM_CHECK_LAUNCH("mamba_scan");
  }
  {
    const dim3 grid(n_tokens, norm_groups);
    FERRUM_DISPATCH_DTYPE(dtype, T, (mamba_gate_norm_kernel<T><<<grid, 256, 0, stream>>>(y, inner, proj, ldp, 0, norm_w, (T*)out,
                                                                                         ldo, norm_groups, eps)));
    FERRUM_CHECK_LAUNCH("mamba_gate_norm");
  }
  return 0;
}
