// Kernels around attention over a cached latent.  A token keeps one row of R + Rr elements: a
// normalised latent c (R elements; every head's keys and values are linear maps of it) and one
// rotated key part (Rr elements) shared by all heads.  With the key map folded into the query,
//   q'_h = [ U_k,h^T q_h,plain | rot(q_h,rot) ],   score_h(j) = q'_h . row_j * scale,
//   o_h = sum_j softmax_j(score_h) c_j,            head output = U_v,h o_h,
// attention runs on the cached rows directly: one "KV head" of R + Rr key elements whose first R
// elements are also the values.
//
// latent_prep: from the float32 down-projections of a token: the normalised query latent, the
//   cache row (normalised latent, rotated key part) written to the token's page, and the sigmoid
//   of the output-gate logits.
// latent_q_rope: the rotated part of every query head, moved behind the folded part.
// attention_latent: the attention itself, float32 arithmetic, for float32 and 16-bit storage.
#include "common.cuh"
#include "partials.cuh"

constexpr int LAT_THREADS = 256;

// pairing (i, i + dims/2) of the first `dims` elements; the others pass unchanged
__device__ __forceinline__ float latent_rotated(const float* v, int i, int dims, const float* cs) {
  const int half = dims >> 1;
  if (i >= dims) return v[i];
  if (i < half) return v[i] * cs[2 * i] - v[i + half] * cs[2 * i + 1];
  const int k = i - half;
  return v[i] * cs[2 * k] + v[k] * cs[2 * k + 1];
}

template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
latent_prep_kernel(const float* __restrict__ proj, int ld, int off_q, int q_rank, const float* __restrict__ wq, int off_kv, int kv_rank,
                   int rot_dim, const float* __restrict__ wkv, int off_gate, int n_gate, const int* __restrict__ positions,
                   const int* __restrict__ req_of_token, const int* __restrict__ block_table, int table_width,
                   const float* __restrict__ cos_sin, int n_pos, int rope_dims, T* __restrict__ plane, long long page_stride,
                   int page_size, T* __restrict__ cq, int ld_cq, float* __restrict__ gate, float eps, int* __restrict__ err,
                   int n_in, const PartialLayout L) {
  __shared__ float red[32];
  __shared__ PartialTable tab;
  extern __shared__ __align__(16) float lp_row[];      // the token's n_in projections
  if (L.ws != nullptr) build_partial_table(L, tab);
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  // the row once into shared memory: from the product's output, or summed from its partials
  for (int i = threadIdx.x; i < n_in; i += blockDim.x) lp_row[i] = L.ws != nullptr ? partial_sum(L, tab, t, i) : proj[(size_t)t * ld + i];
  __syncthreads();
  const float* row = lp_row;
  if (q_rank > 0) {
    const float* p = row + off_q;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(p[i], p[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)t * ld_cq + i] = from_f32<T>(p[i] * inv * wq[i]);
  }
  for (int i = threadIdx.x; i < n_gate; i += blockDim.x) gate[(size_t)t * n_gate + i] = 1.0f / (1.0f + expf(-row[off_gate + i]));
  if (off_kv < 0) return;
  const int pos = positions[t];
  const int lp = pos / page_size;
  int page = -1;
  if (pos < 0 || (rope_dims > 0 && pos >= n_pos)) {
    if (threadIdx.x == 0) atomicExch(err, 2);
  } else if (lp >= table_width) {
    if (threadIdx.x == 0) atomicExch(err, 3);
  } else {
    page = block_table[(size_t)req_of_token[t] * table_width + lp];
    if (page < 0 && threadIdx.x == 0) atomicExch(err, 4);
  }
  const float* p = row + off_kv;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss = fmaf(p[i], p[i], ss);
  ss = block_sum(ss, red);
  if (page < 0) return;
  const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  T* dst = plane + (size_t)page * page_stride + (size_t)(pos % page_size) * (kv_rank + rot_dim);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_f32<T>(p[i] * inv * wkv[i]);
  const float* cs = rope_dims > 0 ? cos_sin + (size_t)pos * rope_dims : nullptr;      // [dims/2][2]
  for (int i = threadIdx.x; i < rot_dim; i += blockDim.x)
    dst[kv_rank + i] = from_f32<T>(rope_dims > 0 ? latent_rotated(p + kv_rank, i, rope_dims, cs) : p[kv_rank + i]);
}

// With `partials` (a product left in deferred mode, see partials.cuh) the projections are summed from
// them instead of read from proj.
// proj: [T, ld] float32 rows holding the query down-projection at off_q (q_rank elements; 0: none),
// the key/value down-projection at off_kv (kv_rank + rot_dim elements; off_kv < 0: this layer
// writes no cache) and n_gate gate logits at off_gate.  A cache page holds page_size rows of
// kv_rank + rot_dim elements.  cos_sin: [n_pos, rope_dims / 2, 2].
FERRUM_API int ferrum_latent_prep(const float* proj, int ld, int n_tokens, int off_q, int q_rank, const float* wq, int off_kv,
                                  int kv_rank, int rot_dim, const float* wkv, int off_gate, int n_gate, const int* positions,
                                  const int* req_of_token, const int* block_table, int table_width, const float* cos_sin,
                                  int n_pos, int rope_dims, void* plane, long long page_stride, int page_size, void* cq,
                                  int ld_cq, int dtype, float* gate, float eps, int* err_flag, const float* partials,
                                  const int* layout, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && q_rank >= 0 && kv_rank > 0 && rot_dim >= 0 && n_gate >= 0, "latent prep: bad sizes");
  int n_in = off_q + q_rank;
  if (off_kv >= 0 && off_kv + kv_rank + rot_dim > n_in) n_in = off_kv + kv_rank + rot_dim;
  if (off_gate + n_gate > n_in) n_in = off_gate + n_gate;
  FERRUM_CHECK_ARG(n_in * 4 <= 200 * 1024 && (partials != nullptr || (proj != nullptr && ld >= n_in)), "latent prep: %d projections a token", n_in);
  PartialLayout L{nullptr, 0, 0, 0, 0};
  if (partials != nullptr) {
    if (int r = partial_make_layout(partials, layout, &L)) return r;
    FERRUM_CHECK_ARG(n_in <= L.tiles * 128 && n_tokens <= L.acc_cols, "latent prep: the partials do not cover the rows");
  }
  FERRUM_CHECK_ARG(rope_dims >= 0 && rope_dims % 2 == 0 && rope_dims <= rot_dim, "latent prep: %d rotated dimensions of %d", rope_dims, rot_dim);
  FERRUM_CHECK_ARG(off_kv < 0 || (plane != nullptr && page_size > 0 && table_width > 0), "latent prep: cache arguments missing");
  FERRUM_CHECK_ARG(eps > 0.f, "latent prep: eps must be positive");
  if (n_tokens == 0) return 0;
  FERRUM_DISPATCH_DTYPE(dtype, T, {
    if (n_in * 4 > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(latent_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, n_in * 4);
      FERRUM_CHECK_ARG(e == cudaSuccess, "latent prep: cannot reserve %d bytes of shared memory: %s", n_in * 4, cudaGetErrorString(e));
    }
    launch_kernel(latent_prep_kernel<T>, n_tokens, LAT_THREADS, (size_t)n_in * 4, stream, proj, ld, off_q, q_rank, wq, off_kv, kv_rank,
                  rot_dim, wkv, off_gate, n_gate, positions, req_of_token, block_table, table_width, cos_sin, n_pos, rope_dims,
                  (T*)plane, page_stride, page_size, (T*)cq, ld_cq, gate, eps, err_flag, n_in, L);
  });
  FERRUM_CHECK_LAUNCH("latent_prep");
  return 0;
}

// q: [T, ldq], head h at h * (Dn + Rr): Dn plain elements then Rr to rotate.  qf: [T, ldf], head h at
// h * (R + Rr): the rotated part lands at R .. R + Rr (the first R elements belong to the folded
// product).
template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
latent_q_rope_kernel(const T* __restrict__ q, int ldq, T* __restrict__ qf, int ldf, const int* __restrict__ positions,
                     const float* __restrict__ cos_sin, int n_pos, int rope_dims, int H, int Dn, int Rr, int R, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (rope_dims > 0 && (pos < 0 || pos >= n_pos)) {
    if (threadIdx.x == 0) atomicExch(err, 2);
    return;
  }
  const float* cs = rope_dims > 0 ? cos_sin + (size_t)pos * rope_dims : nullptr;
  const int half = rope_dims >> 1;
  for (int idx = threadIdx.x; idx < H * Rr; idx += blockDim.x) {
    const int h = idx / Rr, i = idx % Rr;
    const T* src = q + (size_t)t * ldq + (size_t)h * (Dn + Rr) + Dn;
    float v = to_f32<T>(src[i]);
    if (i < rope_dims) {
      if (i < half) v = v * cs[2 * i] - to_f32<T>(src[i + half]) * cs[2 * i + 1];
      else v = v * cs[2 * (i - half)] + to_f32<T>(src[i - half]) * cs[2 * (i - half) + 1];
    }
    qf[(size_t)t * ldf + (size_t)h * (R + Rr) + R + i] = from_f32<T>(v);
  }
}

FERRUM_API int ferrum_latent_q_rope(const void* q, int ldq, void* qf, int ldf, int dtype, int n_tokens, const int* positions,
                                    const float* cos_sin, int n_pos, int rope_dims, int H, int Dn, int Rr, int R, int* err_flag,
                                    cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && H > 0 && Dn >= 0 && Rr >= 0 && R > 0, "latent q rope: bad sizes");
  FERRUM_CHECK_ARG(rope_dims >= 0 && rope_dims % 2 == 0 && rope_dims <= Rr, "latent q rope: %d rotated dimensions of %d", rope_dims, Rr);
  FERRUM_CHECK_ARG(ldq >= H * (Dn + Rr) && ldf >= H * (R + Rr), "latent q rope: a row stride is too short");
  if (n_tokens == 0 || Rr == 0) return 0;
  FERRUM_DISPATCH_DTYPE(dtype, T, launch_kernel(latent_q_rope_kernel<T>, n_tokens, LAT_THREADS, 0, stream, (const T*)q, ldq, (T*)qf, ldf,
                                                positions, cos_sin, n_pos, rope_dims, H, Dn, Rr, R, err_flag));
  FERRUM_CHECK_LAUNCH("latent_q_rope");
  return 0;
}

// ================================================================= attention over the cached rows
// A CTA of eight warps takes up to TQ = TH * TW consecutive tokens of ONE request and HW heads
// (HW * TW = 8): warp w works for head w % HW and tokens (w / HW) * TH .. + TH - 1 of the chunk.
// Tiles of TK cached rows go to shared memory as float32, one tile ahead; a tile serves every
// head and token of the CTA, as keys (all Dk elements) and as values (the first Dv).  Lane j forms
// the scores of key j for its warp's rows (no reduction across lanes), the warp takes maximum
// and sum by shuffles and leaves the weights in shared memory, lane e adds the weighted values of
// elements e, e + 32, ... in key order.  Max, sum and the weighted values are float32 registers.
// Prompt portions run HW = 4, TW = 2; steps of single tokens run HW = 8, TW = 1, TH = 1.
// A query at position p sees keys max(0, p - window + 1) .. p (window 0: from key 0).
__device__ __forceinline__ void lat_cp_async16(void* smem, const void* gmem, int src_bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void lat_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void lat_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T>
__device__ __forceinline__ float4 lat_load4(const T* row, int d, int D, bool vec) {
  float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec) {
    if (d < D) {
      if constexpr (sizeof(T) == 4) {
        r = *reinterpret_cast<const float4*>(row + d);
      } else {
        const uint2 u = *reinterpret_cast<const uint2*>(row + d);
        const T* e = reinterpret_cast<const T*>(&u);
        r = make_float4(to_f32<T>(e[0]), to_f32<T>(e[1]), to_f32<T>(e[2]), to_f32<T>(e[3]));
      }
    }
  } else {
    if (d < D) r.x = to_f32<T>(row[d]);
    if (d + 1 < D) r.y = to_f32<T>(row[d + 1]);
    if (d + 2 < D) r.z = to_f32<T>(row[d + 2]);
    if (d + 3 < D) r.w = to_f32<T>(row[d + 3]);
  }
  return r;
}

constexpr int LAT_WARPS = 8;
constexpr int LAT_SPLIT = 128;      // keys per split of a single token's key range

struct LatSmem {
  int DK8, KS, off_q, off_p, off_row, bytes;
};
inline LatSmem lat_smem(int Dk, int TK, int TQ, int HW) {
  LatSmem s;
  s.DK8 = (Dk + 7) / 8 * 8;
  s.KS = s.DK8 + 4;                       // (KS / 4 odd: a quarter warp's 16-byte reads of eight rows hit different banks)
  s.off_q = 2 * TK * s.KS + 32;           // (the value loop may read up to 31 floats past a row's Dv elements)
  s.off_p = s.off_q + TQ * HW * s.DK8;
  s.off_row = (s.off_p + HW * TQ * TK + 1) / 2 * 2;
  s.bytes = (s.off_row + 2 * TK * 2) * 4;
  return s;
}

template <typename T, int DVI, int TH, int HW>
__global__ void __launch_bounds__(LAT_WARPS * 32)
attention_latent_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo, const float* __restrict__ gate,
                        const int* __restrict__ positions, const int* __restrict__ q_start, int n_reqs,
                        const int* __restrict__ block_table, int table_width, const T* __restrict__ plane, long long page_stride,
                        int page_size, int H, int Dk, int Dv, float scale, int window, int* __restrict__ err, int vec, int TK,
                        int DK8, int off_q, int off_p, int off_row, float* __restrict__ part, int split_slots) {
  constexpr int TW = LAT_WARPS / HW, TQ = TH * TW;
  extern __shared__ __align__(16) float lat_sm[];
  const int KS = DK8 + 4;
  float* const sm_k = lat_sm;
  float* const sm_q = lat_sm + off_q;
  float* const sm_p = lat_sm + off_p;
  long long* const sm_row = reinterpret_cast<long long*>(lat_sm + off_row);
  __shared__ int chunk_req, chunk_t0, chunk_nt;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp = wid % HW;                 // the head (within the CTA's heads) this warp works for
  const int i0 = (wid / HW) * TH;            // the first of its tokens
  const int hchunks = (H + HW - 1) / HW;
  const int c = blockIdx.x / hchunks, hchunk = blockIdx.x % hchunks;
  pdl_wait();
  if (threadIdx.x == 0) {
    int left = c, r = 0, t0 = 0, nt = 0;
    for (; r < n_reqs; ++r) {
      const int a = q_start[r], len = q_start[r + 1] - a;
      const int n = (len + TQ - 1) / TQ;
      if (left < n) {
        t0 = a + left * TQ;
        nt = min(TQ, a + len - t0);
        break;
      }
      left -= n;
    }
    chunk_req = r;
    chunk_t0 = t0;
    chunk_nt = nt;
  }
  __syncthreads();
  const int req = chunk_req, t0 = chunk_t0, nt = chunk_nt;
  if (nt == 0) return;
  const int h0 = hchunk * HW;
  const int nh = min(HW, H - h0);
  int k_begin = 0x7fffffff, k_end = 0;
#pragma unroll
  for (int i = 0; i < TQ; ++i) {
    if (i < nt) {
      const int p = positions[t0 + i];
      k_begin = min(k_begin, window > 0 ? max(0, p - window + 1) : 0);
      k_end = max(k_end, p + 1);
    }
  }
  if (part != nullptr) {
    // (one token per CTA) the token's keys are cut at multiples of LAT_SPLIT in absolute positions:
    // where a cut falls depends on the position alone, never on the batch
    const int s = k_begin / LAT_SPLIT + blockIdx.y;
    if (s * LAT_SPLIT >= k_end) return;
    k_begin = max(k_begin, s * LAT_SPLIT);
    k_end = min(k_end, (s + 1) * LAT_SPLIT);
  }
  int pos[TH], lo[TH];
#pragma unroll
  for (int i = 0; i < TH; ++i) {
    pos[i] = i0 + i < nt ? positions[t0 + i0 + i] : -1;
    lo[i] = i0 + i < nt ? (window > 0 ? max(0, pos[i] - window + 1) : 0) : 0x7fffffff;
  }
  const int* bt = block_table + (size_t)req * table_width;
  const bool vec_ok = vec != 0;
  const bool async_rows = vec_ok && sizeof(T) == 4;
  const int n_tiles = (k_end - k_begin + TK - 1) / TK;
  const int d4 = DK8 / 4;

  auto find_rows = [&](int n) {
    if (threadIdx.x < TK) {
      const int key = k_begin + n * TK + threadIdx.x;
      long long off = -1;
      if (key < k_end) {
        const int lp = key / page_size;
        const int page = lp < table_width ? bt[lp] : -1;
        if (page < 0) atomicExch(err, 5);
        else off = (long long)page * page_stride + (long long)(key % page_size) * Dk;
      }
      sm_row[(n & 1) * TK + threadIdx.x] = off;
    }
  };
  auto load_tile = [&](int n) {
    const int b = n & 1;
    float* const kb = sm_k + b * TK * KS;
    for (int idx = threadIdx.x; idx < TK * d4; idx += LAT_WARPS * 32) {
      const int j = idx / d4, d = (idx % d4) * 4;
      const long long off = sm_row[b * TK + j];
      if (async_rows) {
        const bool there = off >= 0 && d < Dk;
        lat_cp_async16(&kb[j * KS + d], plane + (there ? off + d : 0), there ? 16 : 0);
      } else {
        float4 kk = make_float4(0.f, 0.f, 0.f, 0.f);
        if (off >= 0) kk = lat_load4<T>(plane + off, d, Dk, vec_ok);
        *reinterpret_cast<float4*>(&kb[j * KS + d]) = kk;
      }
    }
  };

  // the chunk's queries [token][head][DK8], zero past Dk and for rows that do not exist
  for (int idx = threadIdx.x; idx < TQ * HW * d4; idx += LAT_WARPS * 32) {
    const int i = idx / (HW * d4), g = (idx / d4) % HW, d = (idx % d4) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < nt && g < nh) v = lat_load4<T>(q + (size_t)(t0 + i) * ldq + (size_t)(h0 + g) * Dk, d, Dk, vec_ok && ldq % 4 == 0);
    *reinterpret_cast<float4*>(&sm_q[(i * HW + g) * DK8 + d]) = v;
  }
  find_rows(0);
  __syncthreads();
  load_tile(0);
  lat_cp_async_commit();

  float m[TH], l[TH], acc[TH][DVI];
#pragma unroll
  for (int i = 0; i < TH; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int e = 0; e < DVI; ++e) acc[i][e] = 0.f;
  }

  for (int n = 0; n < n_tiles; ++n) {
    const int b = n & 1;
    const bool more = n + 1 < n_tiles;
    if (more) find_rows(n + 1);
    __syncthreads();
    if (more) load_tile(n + 1);
    lat_cp_async_commit();
    lat_cp_async_wait<1>();
    const bool have = lane < TK && sm_row[b * TK + lane] >= 0;
    __syncthreads();
    if (warp < nh && i0 < nt) {
      const float* const kb = sm_k + b * TK * KS;
      const int key = k_begin + n * TK + lane;
      float sc[TH];
#pragma unroll
      for (int i = 0; i < TH; ++i) sc[i] = 0.f;
      {
        const float4* kr = reinterpret_cast<const float4*>(&kb[(lane < TK ? lane : 0) * KS]);
#pragma unroll 4
        for (int cc = 0; cc < d4; ++cc) {
          const float4 k4 = kr[cc];
#pragma unroll
          for (int i = 0; i < TH; ++i) {
            const float4 a = *reinterpret_cast<const float4*>(&sm_q[((i0 + i) * HW + warp) * DK8 + cc * 4]);
            sc[i] = fmaf(a.x, k4.x, sc[i]);
            sc[i] = fmaf(a.y, k4.y, sc[i]);
            sc[i] = fmaf(a.z, k4.z, sc[i]);
            sc[i] = fmaf(a.w, k4.w, sc[i]);
          }
        }
      }
      float corr[TH];
      __syncwarp();
#pragma unroll
      for (int i = 0; i < TH; ++i) {
        const bool seen = have && key <= pos[i] && key >= lo[i];
        const float sv = seen ? sc[i] * scale : -INFINITY;
        const float m_new = fmaxf(m[i], warp_max(sv));
        float cr = 1.f, pj = 0.f;
        if (m_new != -INFINITY) {
          cr = m[i] == -INFINITY ? 0.f : expf(m[i] - m_new);
          pj = sv == -INFINITY ? 0.f : expf(sv - m_new);
        }
        l[i] = l[i] * cr + warp_sum(pj);
        m[i] = m_new;
        corr[i] = cr;
        if (lane < TK) sm_p[(warp * TQ + i0 + i) * TK + lane] = pj;
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < TH; ++i)
#pragma unroll
        for (int e = 0; e < DVI; ++e) acc[i][e] *= corr[i];
#pragma unroll 1
      for (int j4 = 0; j4 < TK / 4; ++j4) {
        float vv[4][DVI];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int e = 0; e < DVI; ++e) vv[jj][e] = kb[(j4 * 4 + jj) * KS + lane + 32 * e];
#pragma unroll
        for (int i = 0; i < TH; ++i) {
          const float4 pw = *reinterpret_cast<const float4*>(&sm_p[(warp * TQ + i0 + i) * TK + j4 * 4]);
#pragma unroll
          for (int e = 0; e < DVI; ++e) {
            float a = acc[i][e];
            a = fmaf(pw.x, vv[0][e], a);
            a = fmaf(pw.y, vv[1][e], a);
            a = fmaf(pw.z, vv[2][e], a);
            a = fmaf(pw.w, vv[3][e], a);
            acc[i][e] = a;
          }
        }
      }
    }
  }
  lat_cp_async_wait<0>();
  pdl_launch();
  if (warp >= nh) return;
  const int h = h0 + warp;
#pragma unroll
  for (int i = 0; i < TH; ++i) {
    if (i0 + i >= nt) break;
    const int t = t0 + i0 + i;
    if (part != nullptr) {
      float* p = part + (((size_t)t * H + h) * split_slots + blockIdx.y) * (Dv + 2);
      if (lane == 0) {
        p[0] = m[i];
        p[1] = l[i];
      }
#pragma unroll
      for (int e = 0; e < DVI; ++e) {
        const int d = lane + 32 * e;
        if (d < Dv) p[2 + d] = acc[i][e];
      }
      continue;
    }
    const float f = (l[i] > 0.f ? 1.0f / l[i] : 0.f) * (gate != nullptr ? gate[(size_t)t * H + h] : 1.0f);
#pragma unroll
    for (int e = 0; e < DVI; ++e) {
      const int d = lane + 32 * e;
      if (d < Dv) out[(size_t)t * ldo + (size_t)h * Dv + d] = from_f32<T>(acc[i][e] * f);
    }
  }
}

// Folds the splits of every (token, head) and applies the gate: one block of four warps each.  The
// first warp reads every split's (max, sum), takes the overall maximum and leaves each split's factor
// exp(max_s - max) in shared memory; then thread d adds the splits' weighted values of element d,
// d + 128, ... in ascending key order (independent loads: the splits are not walked as a chain).
constexpr int LAT_COMB_THREADS = 128, LAT_COMB_MAX = 1024;
template <typename T>
__global__ void __launch_bounds__(LAT_COMB_THREADS)
attention_latent_combine_kernel(T* __restrict__ out, int ldo, const float* __restrict__ part, const float* __restrict__ gate,
                                const int* __restrict__ positions, int H, int Dv, int window, int split_slots) {
  __shared__ float factor[LAT_COMB_MAX];
  __shared__ float total;
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n = min(min(pos / LAT_SPLIT - lo / LAT_SPLIT + 1, split_slots), LAT_COMB_MAX);
  const float* base = part + ((size_t)t * H + h) * split_slots * (Dv + 2);
  if (threadIdx.x < 32) {
    float mx = -INFINITY;
    for (int s = threadIdx.x; s < n; s += 32) mx = fmaxf(mx, base[(size_t)s * (Dv + 2)]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int s = threadIdx.x; s < n; s += 32) {
      const float ms = base[(size_t)s * (Dv + 2)];
      const float f = ms == -INFINITY ? 0.f : expf(ms - mx);
      factor[s] = f;
      sum += base[(size_t)s * (Dv + 2) + 1] * f;
    }
    sum = warp_sum(sum);
    if (threadIdx.x == 0) total = sum;
  }
  __syncthreads();
  const float L = total;
  const float f = (L > 0.f ? 1.0f / L : 0.f) * (gate != nullptr ? gate[(size_t)t * H + h] : 1.0f);
  for (int d = threadIdx.x; d < Dv; d += LAT_COMB_THREADS) {
    float o = 0.f;
    for (int s = 0; s < n; ++s) o = fmaf(base[(size_t)s * (Dv + 2) + 2 + d], factor[s], o);
    out[(size_t)t * ldo + (size_t)h * Dv + d] = from_f32<T>(o * f);
  }
}

FERRUM_API int ferrum_attention_latent_split() { return LAT_SPLIT; }

// out[t, h] = gate[t, h] * (the fold of the splits' partials [t][h][slot][Dv + 2] in ascending key order).
FERRUM_API int ferrum_attention_latent_combine(void* out, int ldo, int dtype, const float* part, const float* gate, int n_tokens,
                                               const int* positions, int H, int Dv, int window, int split_slots, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && H > 0 && H <= 65535 && Dv > 0 && split_slots > 0 && split_slots <= LAT_COMB_MAX && part != nullptr,
                   "latent attention merge: bad arguments (at most %d splits)", LAT_COMB_MAX);
  if (n_tokens == 0) return 0;
  FERRUM_DISPATCH_DTYPE(dtype, T, launch_kernel(attention_latent_combine_kernel<T>, dim3(n_tokens, H), dim3(LAT_COMB_THREADS), 0, stream, (T*)out, ldo,
                                                part, gate, positions, H, Dv, window, split_slots));
  FERRUM_CHECK_LAUNCH("attention_latent_combine");
  return 0;
}

constexpr int LAT_MAX_DK = 1024, LAT_MAX_DV = 512, LAT_SMEM_LIMIT = 200 * 1024;

// q: [T, ldq], head h at h * Dk, already scaled by nothing (the kernel multiplies scores by `scale`).
// out: [T, ldo], head h at h * Dv: the weighted sum of the first Dv elements of the seen rows,
// times gate[t, h] where gate (float32 [T, H]) is given.  single_tokens != 0: every request brings
// one token (the head-major shape); else tokens of a request that follow each other share tiles.
FERRUM_API int ferrum_attention_latent(const void* q, int ldq, void* out, int ldo, int dtype, const float* gate, int n_tokens,
                                       const int* positions, const int* q_start, int n_reqs, const int* block_table,
                                       int table_width, const void* plane, long long page_stride, int page_size, int H, int Dk,
                                       int Dv, float scale, int window, int single_tokens, float* part, int split_slots,
                                       int* err_flag, cudaStream_t stream) {
  FERRUM_CHECK_ARG(part == nullptr || (single_tokens && split_slots > 0 && split_slots <= 65535),
                   "latent attention: key splits are for steps of single tokens (slots %d)", split_slots);
  FERRUM_CHECK_ARG(n_tokens >= 0 && n_reqs > 0 && H > 0, "latent attention: bad sizes T=%d requests=%d H=%d", n_tokens, n_reqs, H);
  FERRUM_CHECK_ARG(Dk > 0 && Dk <= LAT_MAX_DK && Dv > 0 && Dv <= Dk && Dv <= LAT_MAX_DV,
                   "latent attention: key size %d (at most %d) or value size %d (at most %d and the key size)", Dk, LAT_MAX_DK, Dv, LAT_MAX_DV);
  FERRUM_CHECK_ARG(page_size > 0 && table_width > 0 && window >= 0, "latent attention: bad cache arguments");
  FERRUM_CHECK_ARG(ldq >= H * Dk && ldo >= H * Dv, "latent attention: a row stride is too short");
  if (n_tokens == 0) return 0;
  const int esize = dtype == FERRUM_F32 ? 4 : 2;
  const int vec = Dk % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)plane & 15) == 0 && page_stride % 4 == 0 &&
                  (Dk * esize) % (esize == 4 ? 16 : 8) == 0;
  const int dvi = Dv <= 32 ? 1 : Dv <= 64 ? 2 : Dv <= 128 ? 4 : Dv <= 256 ? 8 : 16;
#define LAT_LAUNCH(DVI_, TH_, HW_)                                                                                          \
  do {                                                                                                                      \
    constexpr int TQ_ = TH_ * (LAT_WARPS / HW_);                                                                            \
    int TK = 32;                                                                                                            \
    LatSmem s = lat_smem(Dk, TK, TQ_, HW_);                                                                                 \
    if (s.bytes > LAT_SMEM_LIMIT) {                                                                                         \
      TK = 16;                                                                                                              \
      s = lat_smem(Dk, TK, TQ_, HW_);                                                                                       \
    }                                                                                                                       \
    FERRUM_CHECK_ARG(s.bytes <= LAT_SMEM_LIMIT, "latent attention: %d bytes of shared memory", s.bytes);                    \
    const long long chunks = single_tokens ? n_tokens : (n_tokens + TQ_ - 1) / TQ_ + n_reqs;                                \
    const long long ctas = chunks * ((H + HW_ - 1) / HW_);                                                                  \
    FERRUM_CHECK_ARG(ctas < (1LL << 31), "latent attention: too many rows");                                                \
    FERRUM_DISPATCH_DTYPE(dtype, T, {                                                                                       \
      static int configured = 0;                                                                                            \
      if (configured < s.bytes) {                                                                                           \
        cudaError_t e = cudaFuncSetAttribute(attention_latent_kernel<T, DVI_, TH_, HW_>,                                    \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, s.bytes);                         \
        FERRUM_CHECK_ARG(e == cudaSuccess, "latent attention: cannot reserve %d bytes of shared memory: %s", s.bytes,       \
                         cudaGetErrorString(e));                                                                            \
        configured = s.bytes;                                                                                               \
      }                                                                                                                     \
      launch_kernel(attention_latent_kernel<T, DVI_, TH_, HW_>, dim3((unsigned)ctas, part ? split_slots : 1),               \
                    dim3(LAT_WARPS * 32), (size_t)s.bytes,                                                                  \
                    stream, (const T*)q, ldq, (T*)out, ldo, gate, positions, q_start, n_reqs, block_table, table_width,     \
                    (const T*)plane, page_stride, page_size, H, Dk, Dv, scale, window, err_flag, vec, TK, s.DK8, s.off_q,    \
                    s.off_p, s.off_row, part, split_slots);                                                                 \
    });                                                                                                                     \
  } while (0)
#define LAT_SHAPES(DVI_)                               \
  do {                                                 \
    if (single_tokens) LAT_LAUNCH(DVI_, 1, 8);         \
    else if (DVI_ <= 8) LAT_LAUNCH(DVI_, 4, 4);        \
    else LAT_LAUNCH(DVI_, 2, 4);                       \
  } while (0)
  switch (dvi) {
    case 1: LAT_SHAPES(1); break;
    case 2: LAT_SHAPES(2); break;
    case 4: LAT_SHAPES(4); break;
    case 8: LAT_SHAPES(8); break;
    default: LAT_SHAPES(16); break;
  }
#undef LAT_SHAPES
#undef LAT_LAUNCH
  FERRUM_CHECK_LAUNCH("attention_latent");
  if (part != nullptr) return ferrum_attention_latent_combine(out, ldo, dtype, part, gate, n_tokens, positions, H, Dv, window, split_slots, stream);
  return 0;
}

// ================================================================= one small product per head, few tokens
// y[t, h * ldyh + n] = sum_k x[t, h * ldxh + k] * w[h][n][k] for n < N, k < K: every head has its own
// [N, K] matrix (k contiguous).  For steps of a few tokens the time is the weights' read: a warp
// owns one output feature of one head, reads its weight row once (8 bytes a lane where the rows
// allow) and keeps up to HL_TOK tokens' sums, which the lanes fold in a butterfly; more tokens
// take further passes over the (cached) row.  A sum walks k in an order that depends on K alone.
constexpr int HL_WARPS = 8, HL_TOK = 8;

template <typename T, bool VEC>
__global__ void __launch_bounds__(HL_WARPS * 32)
head_linear_kernel(const T* __restrict__ x, int ldx, int ldxh, const T* __restrict__ w, T* __restrict__ y, int ldy, int ldyh,
                   int M, int N, int K) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * HL_WARPS + warp, h = blockIdx.y;
  if (n >= N) return;
  const T* wr = w + ((size_t)h * N + n) * K;
  for (int t0 = 0; t0 < M; t0 += HL_TOK) {
    float acc[HL_TOK];
#pragma unroll
    for (int i = 0; i < HL_TOK; ++i) acc[i] = 0.f;
    if constexpr (VEC) {
      for (int k = lane * 4; k < K; k += 128) {
        float wv[4];
        if constexpr (sizeof(T) == 4) {
          const float4 u = *reinterpret_cast<const float4*>(wr + k);
          wv[0] = u.x; wv[1] = u.y; wv[2] = u.z; wv[3] = u.w;
        } else {
          const uint2 u = *reinterpret_cast<const uint2*>(wr + k);
          const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) wv[j] = to_f32<T>(e[j]);
        }
#pragma unroll
        for (int i = 0; i < HL_TOK; ++i) {
          if (t0 + i < M) {
            const T* xr = x + (size_t)(t0 + i) * ldx + (size_t)h * ldxh + k;
            float xv[4];
            if constexpr (sizeof(T) == 4) {
              const float4 u = *reinterpret_cast<const float4*>(xr);
              xv[0] = u.x; xv[1] = u.y; xv[2] = u.z; xv[3] = u.w;
            } else {
              const uint2 u = *reinterpret_cast<const uint2*>(xr);
              const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
              for (int j = 0; j < 4; ++j) xv[j] = to_f32<T>(e[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i] = fmaf(xv[j], wv[j], acc[i]);
          }
        }
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float wv = to_f32<T>(wr[k]);
#pragma unroll
        for (int i = 0; i < HL_TOK; ++i)
          if (t0 + i < M) acc[i] = fmaf(to_f32<T>(x[(size_t)(t0 + i) * ldx + (size_t)h * ldxh + k]), wv, acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < HL_TOK; ++i) {
      const float s = warp_sum(acc[i]);
      if (lane == 0 && t0 + i < M) y[(size_t)(t0 + i) * ldy + (size_t)h * ldyh + n] = from_f32<T>(s);
    }
  }
}

FERRUM_API int ferrum_head_linear_max_tokens() { return 64; }

FERRUM_API int ferrum_head_linear(const void* x, int ldx, int ldxh, const void* w, void* y, int ldy, int ldyh, int dtype, int M,
                                  int H, int N, int K, cudaStream_t stream) {
  FERRUM_CHECK_ARG(M >= 0 && H > 0 && H <= 65535 && N > 0 && K > 0, "head linear: bad sizes M=%d H=%d N=%d K=%d", M, H, N, K);
  FERRUM_CHECK_ARG(ldxh >= 0 && ldyh >= N && ldx >= (H - 1) * ldxh + K && ldy >= (H - 1) * ldyh + N, "head linear: a stride is too short");
  if (M == 0) return 0;
  const int esize = dtype == FERRUM_F32 ? 4 : 2;
  const int al = esize == 4 ? 16 : 8;
  const bool vec = K % 4 == 0 && ldx % 4 == 0 && ldxh % 4 == 0 && ((uintptr_t)x % al) == 0 && ((uintptr_t)w % al) == 0;
  const dim3 grid((N + HL_WARPS - 1) / HL_WARPS, H);
  FERRUM_DISPATCH_DTYPE(dtype, T, {
    if (vec) launch_kernel(head_linear_kernel<T, true>, grid, dim3(HL_WARPS * 32), 0, stream, (const T*)x, ldx, ldxh, (const T*)w, (T*)y, ldy, ldyh, M, N, K);
    else launch_kernel(head_linear_kernel<T, false>, grid, dim3(HL_WARPS * 32), 0, stream, (const T*)x, ldx, ldxh, (const T*)w, (T*)y, ldy, ldyh, M, N, K);
  });
  FERRUM_CHECK_LAUNCH("head_linear");
  return 0;
}
