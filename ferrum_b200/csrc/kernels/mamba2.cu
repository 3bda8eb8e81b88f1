// A selective state-space mixer with a scalar decay per head (the Mamba-2 recurrence), after its
// input product.  A token's float32 product row is [z: inner | x: inner | B: G N | C: G N | dt: heads]
// with inner = heads * P.  Per request the state row keeps, in float32,
//   S [heads][N][P]                      the recurrent state (element (n, p) of head h at (h N + n) P + p)
//   u [taps - 1][channels]               the last inputs of the short convolution (channels = inner + 2 G N)
//
// mamba_conv:        xBC <- silu(bias + sum_j w[c][j] * input(t - (taps - 1 - j))[c]); an input before the
//                    portion's first token comes from u, which is all zero before a sequence's first token.
// mamba_conv_state:  u <- the last taps - 1 inputs after this portion (old rows move up when the portion
//                    is shorter than that).  A launch of its own, so that nobody reads u while it changes.
// mamba_scan:        per (request, head) and 32 values of p one block walks the portion's tokens in order:
//                      dt = softplus(dt_raw + dt_bias[h]);  S[n] <- exp(-exp(A_log[h]) dt) S[n] + dt B[n] x[p]
//                      y[p] = sum_n S[n] C[n] + D[h] x[p]
//                    The sum over n has one fixed tree, and the walk is token by token whatever the
//                    portion: a token's result does not depend on how the sequence was cut.
// mamba_gate_norm:   v = y * silu(z); each of `norm_groups` equal parts of the row is divided by its own
//                    root mean square and multiplied by the weight; out in the compute type.
#include "common.cuh"

constexpr int MS_TC = 32;        // tokens per chunk that the walk stages in shared memory (4 when no request brings more)
constexpr int MS_WARPS = 8;      // warps of the walk's block: each owns an eighth of a head's state elements
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

// Shared memory of the walk for 8 * NQ >= N state elements per (head, p): two buffers of a chunk's
// B and C rows (zero past N), x of the block's 32 p, step size and decay per token; the eight warps'
// parts of y for a chunk.
template <int NQ, int TC>
struct MsTile {
  static constexpr int W = 8 * NQ;
  static constexpr int OFF_B = 0;
  static constexpr int OFF_C = OFF_B + 2 * TC * W;
  static constexpr int OFF_X = OFF_C + 2 * TC * W;
  static constexpr int OFF_DT = OFF_X + 2 * TC * 32;
  static constexpr int OFF_DECAY = OFF_DT + 2 * TC;
  static constexpr int OFF_Y = OFF_DECAY + 2 * TC;
  static constexpr int SMEM_BYTES = (OFF_Y + MS_WARPS * TC * 32) * 4;
};

__device__ __forceinline__ void ms_cp_async(void* smem, const void* gmem, int bytes, int src_bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}

// A block of eight warps walks the tokens of one (request, head) for 32 values of p: lane l of warp w
// holds S[n] for p = 32 blockIdx.x + l and n in [w NQ, (w + 1) NQ) in registers.  A token's B and C
// values are the same for all lanes of a warp (one broadcast read serves 32 p), x differs by lane.  Each
// warp leaves its part of y[p] per token in shared memory, and after a chunk the block adds the eight
// parts in warp order (one fixed tree) and writes y.  The tokens' x, B, C arrive in chunks of TC
// through two shared-memory buffers (cp.async, the next chunk on its way while this one is walked);
// step size and decay of a chunk's tokens are worked out by one thread per token, off the serial
// chain, which is one fused multiply-add per state element and token.
template <int NQ, int TC>
__global__ void __launch_bounds__(MS_WARPS * 32)
mamba_scan_kernel(const float* __restrict__ xbc, int C, const float* __restrict__ proj, int ldp, int off_dt,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                  const int* __restrict__ slots, float* __restrict__ y, int heads, int P, int N, int groups, int vec) {
  using Tile = MsTile<NQ, TC>;
  constexpr int W = Tile::W, NT = MS_WARPS * 32;
  extern __shared__ __align__(16) float ms_smem[];
  float* const sB = ms_smem + Tile::OFF_B;
  float* const sC = ms_smem + Tile::OFF_C;
  float* const sX = ms_smem + Tile::OFF_X;
  float* const sDt = ms_smem + Tile::OFF_DT;
  float* const sDecay = ms_smem + Tile::OFF_DECAY;
  float* const sY = ms_smem + Tile::OFF_Y;          // [warp][token][32]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int p0 = blockIdx.x * 32, h = blockIdx.y, r = blockIdx.z;
  const int p = p0 + lane, n0 = warp * NQ;
  const int inner = heads * P;
  const int g = h / (heads / groups);
  const int t0 = q_start[r], t1 = q_start[r + 1];
  const int n_chunks = (t1 - t0 + TC - 1) / TC;
  float* S = state + (long long)slots[r] * state_stride + ((long long)h * N + n0) * P + p;      // (n + 1: P further)
  float s[NQ];
#pragma unroll
  for (int k = 0; k < NQ; ++k) s[k] = (p < P && n0 + k < N) ? S[(long long)k * P] : 0.f;
  const float a = expf(a_log[h]), db = dt_bias[h], dsk = d_skip[h];
  const int off_b = inner + g * N, off_c = inner + groups * N + g * N;

  auto stage = [&](int c, int b) {          // chunk c on its way into buffer b (the caller commits the group)
    const int base = t0 + c * TC;
    const int cnt = min(TC, t1 - base);          // (rows past the chunk's last token are never read)
    if (vec) {
      for (int idx = tid; idx < cnt * (W / 4); idx += NT) {
        const int t = idx / (W / 4), n = (idx % (W / 4)) * 4;
        const bool there = n < N;                              // (N is a multiple of 4 here)
        const float* row = xbc + (size_t)(base + t) * C;
        ms_cp_async(&sB[(b * TC + t) * W + n], row + off_b + (there ? n : 0), 16, there ? 16 : 0);
        ms_cp_async(&sC[(b * TC + t) * W + n], row + off_c + (there ? n : 0), 16, there ? 16 : 0);
      }
    } else {
      for (int idx = tid; idx < cnt * W; idx += NT) {
        const int t = idx / W, n = idx % W;
        const bool there = n < N;
        const float* row = xbc + (size_t)(base + t) * C;
        ms_cp_async(&sB[(b * TC + t) * W + n], row + off_b + (there ? n : 0), 4, there ? 4 : 0);
        ms_cp_async(&sC[(b * TC + t) * W + n], row + off_c + (there ? n : 0), 4, there ? 4 : 0);
      }
    }
    for (int idx = tid; idx < cnt * 32; idx += NT) {
      const int t = idx >> 5, i = idx & 31;
      const bool there = p0 + i < P;
      ms_cp_async(&sX[(b * TC + t) * 32 + i], xbc + (size_t)(base + t) * C + h * P + (there ? p0 + i : 0), 4, there ? 4 : 0);
    }
  };
  auto raw_dt = [&](int c) {                // thread t: the step-size input of token t of chunk c
    const int t = t0 + c * TC + tid;
    return (tid < TC && t < t1) ? proj[(size_t)t * ldp + off_dt + h] : 0.f;
  };
  auto finish_dt = [&](float raw, int b) {
    if (tid < TC) {
      const float dt = ms_softplus(raw + db);
      sDt[b * TC + tid] = dt;
      sDecay[b * TC + tid] = expf(-a * dt);
    }
  };

  if (n_chunks > 0) {
    stage(0, 0);
    finish_dt(raw_dt(0), 0);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int c = 0; c < n_chunks; ++c) {
    const int b = c & 1;
    const bool more = c + 1 < n_chunks;
    float raw_next = 0.f;
    if (more) {
      stage(c + 1, b ^ 1);                  // (its buffer was last read for chunk c - 1, before the barrier that ended it)
      raw_next = raw_dt(c + 1);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const int nt = min(TC, t1 - t0 - c * TC);
#pragma unroll 2
    for (int t = 0; t < nt; ++t) {
      const float decay = sDecay[b * TC + t];
      const float xr = sX[(b * TC + t) * 32 + lane];
      const float xd = xr * sDt[b * TC + t];
      const float4* bp = reinterpret_cast<const float4*>(&sB[(b * TC + t) * W + n0]);
      const float4* cp = reinterpret_cast<const float4*>(&sC[(b * TC + t) * W + n0]);
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;      // four chains, added in one fixed order
#pragma unroll
      for (int k4 = 0; k4 < NQ / 4; ++k4) {
        const float4 bb = bp[k4], cc = cp[k4];
        s[4 * k4 + 0] = fmaf(decay, s[4 * k4 + 0], bb.x * xd);
        a0 = fmaf(s[4 * k4 + 0], cc.x, a0);
        s[4 * k4 + 1] = fmaf(decay, s[4 * k4 + 1], bb.y * xd);
        a1 = fmaf(s[4 * k4 + 1], cc.y, a1);
        s[4 * k4 + 2] = fmaf(decay, s[4 * k4 + 2], bb.z * xd);
        a2 = fmaf(s[4 * k4 + 2], cc.z, a2);
        s[4 * k4 + 3] = fmaf(decay, s[4 * k4 + 3], bb.w * xd);
        a3 = fmaf(s[4 * k4 + 3], cc.w, a3);
      }
      const float part = (a0 + a1) + (a2 + a3);
      sY[(warp * TC + t) * 32 + lane] = warp == 0 ? fmaf(dsk, xr, part) : part;      // (the skip term rides on the first part)
    }
    __syncthreads();
    for (int idx = tid; idx < nt * 32; idx += NT) {
      const int t = idx >> 5, i = idx & 31;
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < MS_WARPS; ++w) acc += sY[(w * TC + t) * 32 + i];
      if (p0 + i < P) y[(size_t)(t0 + c * TC + t) * inner + h * P + p0 + i] = acc;
    }
    if (more) finish_dt(raw_next, b ^ 1);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int k = 0; k < NQ; ++k)
    if (p < P && n0 + k < N) S[(long long)k * P] = s[k];
}

template <typename T>
__global__ void __launch_bounds__(256)
mamba_gate_norm_kernel(const float* __restrict__ y, int inner, const float* __restrict__ proj, int ldp, int off_z,
                       const float* __restrict__ w, T* __restrict__ out, int ldo, int norm_groups, float eps) {
  pdl_launch();      // the product that follows may fetch its weights meanwhile
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

// max_q_len: the most tokens any request brings in this step (it only chooses the chunk size of the walk).
// proj: the input product's float32 rows; xbc [n_tokens, C] and y [n_tokens, inner]: float32 scratch;
// out [n_tokens, inner] in `dtype`; state: the requests' float32 state rows (see the top of the file).
FERRUM_API int ferrum_mamba2_mix(const float* proj, int ldp, int n_tokens, int n_reqs, const int* req_of_token,
                                 const int* q_start, const int* slots, const float* conv_w, const float* conv_b, int taps,
                                 const float* dt_bias, const float* a_log, const float* d_skip, const float* norm_w,
                                 int heads, int P, int N, int groups, int norm_groups, float eps, float* state,
                                 long long state_stride, float* xbc, float* y, void* out, int ldo, int dtype,
                                 int max_q_len, cudaStream_t stream) {
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
    const dim3 grid((P + 31) / 32, heads, n_reqs);
    // rows of B and C start on 16-byte borders: 16-byte copies
    const int vec = N % 4 == 0 && C % 4 == 0 && inner % 4 == 0 && ((uintptr_t)xbc & 15) == 0;
#define MS_SCAN2(NQ_, TC_)                                                                                                \
  do {                                                                                                                     \
    static bool configured = false;                                                                                        \
    if (!configured) {                                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(mamba_scan_kernel<NQ_, TC_>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                           MsTile<NQ_, TC_>::SMEM_BYTES);                                                  \
      FERRUM_CHECK_ARG(e == cudaSuccess, "mamba2: cannot reserve %d bytes of shared memory: %s",                           \
                       MsTile<NQ_, TC_>::SMEM_BYTES, cudaGetErrorString(e));                                               \
      configured = true;                                                                                                   \
    }                                                                                                                      \
    mamba_scan_kernel<NQ_, TC_><<<grid, MS_WARPS * 32, MsTile<NQ_, TC_>::SMEM_BYTES, stream>>>(                            \
        xbc, C, proj, ldp, off_dt, dt_bias, a_log, d_skip, state, state_stride, q_start, slots, y, heads, P, N, groups, vec); \
  } while (0)
#define MS_SCAN(NQ_)                  \
  do {                                \
    if (max_q_len <= 4) MS_SCAN2(NQ_, 4); \
    else MS_SCAN2(NQ_, MS_TC);        \
  } while (0)
    if (N <= 32) MS_SCAN(4);
    else if (N <= 64) MS_SCAN(8);
    else if (N <= 128) MS_SCAN(16);
    else MS_SCAN(32);
#undef MS_SCAN
#undef MS_SCAN2
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
