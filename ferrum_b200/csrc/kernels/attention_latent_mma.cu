// Attention over cached latent rows on the tensor cores (mma.sync m16n8k16), for 16-bit storage.
//
// Every head of a token reads the same cached rows (keys: all Dk elements of a row, values: its
// first Dv), so a tile of 16 rows packs the heads of one token (or of 16 / HB tokens where the
// model has fewer than 16 heads: HB = heads per tile, a power of two).  The output of a row
// tile is 16 x Dv float32, too wide for one warp's registers: FOUR warps share a row tile.  For
// a stage of 64 or 32 keys each of them forms the scores of ITS quarter of the keys (Q K^T over Dk) and keeps them in
// registers; the warps exchange their row maxima through shared memory, each takes the softmax
// step for its own keys (max and sums in float32 registers; a warp's sum covers its keys, the four
// meet once at the end), rounds its weights to the 16-bit type into a shared [16][64] operand tile,
// and then every warp multiplies the whole tile with ITS quarter of the value columns (the key rows
// read through
// ldmatrix.trans).  A CTA has one row tile (steps of single tokens: 4 warps) or up to three (prompt
// portions: 12 warps on one key stage).  Key stages arrive by cp.async one stage
// ahead.  Single tokens may cut their key range at multiples of 128 absolute positions among CTAs
// (partials folded by attention_latent_combine, the same as the CUDA-core kernel's).
// Needs Dk % 16 == 0, Dv % 32 == 0, Dv <= 512 and 16-byte aligned rows; the CUDA-core kernel takes
// everything else and float32.
#include "common.cuh"

#include <type_traits>

// keys per stage: a template parameter TK (64: a warp forms the scores of 16 keys; 32: of 8)
constexpr int LM_SPLIT = 128;      // keys per split (the CUDA-core kernel's and the merge kernel's)
constexpr int LM_SMEM_LIMIT = 225 * 1024;
// row stride of the weights' operand tile: TK + 8 16-bit elements

__device__ __forceinline__ void lm_cp_async16(void* smem, const void* gmem, int src_bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
template <typename T>
__device__ __forceinline__ void lm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

struct LmSmem {
  int DKP, off_k, off_s, off_row, bytes;     // offsets in bytes
};
inline LmSmem lm_smem(int Dk, int NRT, int TK) {
  LmSmem s;
  s.DKP = Dk + 8;                                    // (rows 16 bytes apart modulo 128: ldmatrix reads eight rows without bank conflicts)
  s.off_k = NRT * 16 * s.DKP * 2;
  s.off_s = s.off_k + 2 * TK * s.DKP * 2;                // per row tile: 64 + 64 floats (maxima, sums), then its weights tile
  s.off_row = s.off_s + NRT * (128 * 4 + 16 * (TK + 8) * 2);
  s.bytes = s.off_row + 2 * TK * 8;
  return s;
}

// NV: n-tiles of 8 value columns per warp (Dv / 32 <= NV).  NRT: row tiles per CTA.
template <typename T, int NV, int NRT, int TK>
__global__ void __launch_bounds__(128 * NRT)
attention_latent_mma_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo, const float* __restrict__ gate,
                            const int* __restrict__ positions, const int* __restrict__ q_start, int n_reqs,
                            const int* __restrict__ block_table, int table_width, const T* __restrict__ plane,
                            long long page_stride, int page_size, int H, int HB, int Dk, int Dv, float scale, int window,
                            int* __restrict__ err, int DKP, int off_k, int off_s, int off_row, float* __restrict__ part,
                            int split_slots) {
  extern __shared__ __align__(16) unsigned char lm_sm[];
  T* const sQ = reinterpret_cast<T*>(lm_sm);
  T* const sK = reinterpret_cast<T*>(lm_sm + off_k);
  float* const sS = reinterpret_cast<float*>(lm_sm + off_s);                        // [NRT][64] maxima, [NRT][64] sums
  T* const sP = reinterpret_cast<T*>(lm_sm + off_s + NRT * 128 * 4);                // [NRT * 16][LM_PS]
  long long* const sRow = reinterpret_cast<long long*>(lm_sm + off_row);
  __shared__ int chunk_req, chunk_t0, chunk_nt;
  constexpr int THREADS = 128 * NRT;
  constexpr int KW = TK / 4;                   // keys per warp of a stage's scores
  constexpr int LM_PS = TK + 8;
  static_assert(TK == 64 || TK == 32, "a stage has 64 or 32 keys");
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rt = wid >> 2, quarter = wid & 3;
  const int TT = 16 / HB;                       // tokens per row tile
  const int TQ = TT * NRT;                      // tokens per CTA
  const int hchunks = (H + HB - 1) / HB;
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
  const int h0 = hchunk * HB;
  int k_begin = 0x7fffffff, k_end = 0;
  for (int i = 0; i < nt; ++i) {
    const int p = positions[t0 + i];
    k_begin = min(k_begin, window > 0 ? max(0, p - window + 1) : 0);
    k_end = max(k_end, p + 1);
  }
  if (part != nullptr) {
    const int s = k_begin / LM_SPLIT + blockIdx.y;
    if (s * LM_SPLIT >= k_end) return;
    k_begin = max(k_begin, s * LM_SPLIT);
    k_end = min(k_end, (s + 1) * LM_SPLIT);
  }
  // this thread's two rows of its row tile: lane / 4 and lane / 4 + 8
  int r_tok[2], r_head[2], r_pos[2], r_lo[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = (lane >> 2) + 8 * j;
    const int i = rt * TT + r / HB, h = h0 + r % HB;
    const bool there = i < nt && h < H;
    r_tok[j] = there ? t0 + i : -1;
    r_head[j] = h;
    r_pos[j] = there ? positions[t0 + i] : -1;
    r_lo[j] = there ? (window > 0 ? max(0, r_pos[j] - window + 1) : 0) : 0x7fffffff;
  }
  const int* bt = block_table + (size_t)req * table_width;
  const int n_tiles = (k_end - k_begin + TK - 1) / TK;
  const int chunks16 = Dk / 8;                  // 16-byte pieces of a row (the queries' load)

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
      sRow[(n & 1) * TK + threadIdx.x] = off;
    }
  };
  // a warp per row, a lane per 16-byte piece (no index division in the loop that runs every stage)
  auto load_tile = [&](int n) {
    const int b = n & 1;
    T* const kb = sK + (size_t)b * TK * DKP;
    for (int j = wid; j < TK; j += THREADS / 32) {
      const long long off = sRow[b * TK + j];
      const T* src = plane + (off >= 0 ? off : 0);
      T* dst = kb + j * DKP;
      const int bytes = off >= 0 ? 16 : 0;
      for (int d = lane * 8; d < Dk; d += 256) lm_cp_async16(dst + d, src + d, bytes);
    }
  };

  // the CTA's query rows, zero where a row does not exist
  for (int idx = threadIdx.x; idx < NRT * 16 * chunks16; idx += THREADS) {
    const int r = idx / chunks16, d = (idx % chunks16) * 8;
    const int i = (r >> 4) * TT + (r & 15) / HB, h = h0 + (r & 15) % HB;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (i < nt && h < H) v = *reinterpret_cast<const uint4*>(q + (size_t)(t0 + i) * ldq + (size_t)h * Dk + d);
    *reinterpret_cast<uint4*>(&sQ[r * DKP + d]) = v;
  }
  find_rows(0);
  __syncthreads();
  load_tile(0);
  lm_commit();

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  const int nv = Dv / 32;                       // this warp's n-tiles: value columns quarter * Dv/4 + j * 8
  const int vbase = quarter * (Dv / 4);

  for (int n = 0; n < n_tiles; ++n) {
    const int b = n & 1;
    const bool more = n + 1 < n_tiles;
    if (more) find_rows(n + 1);
    __syncthreads();                 // tile n - 1 has been read by everyone; the next rows' offsets are visible
    if (more) load_tile(n + 1);
    lm_commit();
    lm_wait<1>();
    __syncthreads();                 // tile n is in shared memory
    const T* const kb = sK + (size_t)b * TK * DKP;
    // ---- scores of this warp's 16 keys for the row tile's 16 rows
    {
      // (two accumulator sets over alternate k-steps: four independent chains of products per warp instead of two)
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, u0[4] = {0.f, 0.f, 0.f, 0.f}, u1[4] = {0.f, 0.f, 0.f, 0.f};
      const T* qa = sQ + (size_t)(rt * 16 + (lane & 15)) * DKP + (lane >> 4) * 8;
      const int nks = Dk / 16;
      if constexpr (KW == 16) {
        const T* kr = kb + (size_t)(quarter * 16 + (lane & 7) + ((lane >> 4) << 3)) * DKP + ((lane >> 3) & 1) * 8;
#pragma unroll 2
        for (int ks = 0; ks + 1 < nks; ks += 2) {
          uint32_t a[4], bq[4], a2[4], bq2[4];
          lm_ldmatrix_x4(a, qa + ks * 16);
          lm_ldmatrix_x4(bq, kr + ks * 16);
          lm_ldmatrix_x4(a2, qa + ks * 16 + 16);
          lm_ldmatrix_x4(bq2, kr + ks * 16 + 16);
          lm_mma<T>(s0, a, bq[0], bq[1]);
          lm_mma<T>(s1, a, bq[2], bq[3]);
          lm_mma<T>(u0, a2, bq2[0], bq2[1]);
          lm_mma<T>(u1, a2, bq2[2], bq2[3]);
        }
        if (nks & 1) {
          uint32_t a[4], bq[4];
          lm_ldmatrix_x4(a, qa + (nks - 1) * 16);
          lm_ldmatrix_x4(bq, kr + (nks - 1) * 16);
          lm_mma<T>(s0, a, bq[0], bq[1]);
          lm_mma<T>(s1, a, bq[2], bq[3]);
        }
      } else {
        // eight keys per warp: one ldmatrix.x4 brings the key operands of TWO k-steps (keys x k 0-7, 8-15, 16-23, 24-31)
        const T* kr = kb + (size_t)(quarter * 8 + (lane & 7)) * DKP + (lane >> 3) * 8;
#pragma unroll 2
        for (int ks = 0; ks + 1 < nks; ks += 2) {
          uint32_t a[4], a2[4], bq[4];
          lm_ldmatrix_x4(a, qa + ks * 16);
          lm_ldmatrix_x4(a2, qa + ks * 16 + 16);
          lm_ldmatrix_x4(bq, kr + ks * 16);
          lm_mma<T>(s0, a, bq[0], bq[1]);
          lm_mma<T>(u0, a2, bq[2], bq[3]);
        }
        if (nks & 1) {
          uint32_t a[4], bq[4];
          lm_ldmatrix_x4(a, qa + (nks - 1) * 16);
          lm_ldmatrix_x4(bq, kr + (nks - 1) * 16 - ((lane >> 4) << 4));     // (lanes 16-31 repeat the first two pieces: stay inside the row)
          lm_mma<T>(s0, a, bq[0], bq[1]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s0[e] += u0[e];
        s1[e] += u1[e];
      }
      // ---- this warp's share of the softmax step: its KW keys of the thread's two rows, in registers.
      // s0: keys cc, cc + 1 (rows r0 | r0 + 8); with 16 keys per warp s1: keys cc + 8, cc + 9
      constexpr int NE = KW / 4;                   // score elements per thread and row
      const int key = k_begin + n * TK + quarter * KW + (lane & 3) * 2;
      float sv[2][4];
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float vals[4] = {s0[2 * j], s0[2 * j + 1], s1[2 * j], s1[2 * j + 1]};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ke = key + (e & 1) + (e >> 1) * 8;
          const bool seen = e < NE && ke < k_end && ke <= r_pos[j] && ke >= r_lo[j];
          sv[j][e] = seen ? vals[e] * scale : -INFINITY;
          mx[j] = fmaxf(mx[j], sv[j][e]);
        }
        mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 1));
        mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 2));
      }
      float* const sMx = sS + rt * 64;                       // [quarter][16 rows]: the warps' row maxima of this stage
      if ((lane & 3) == 0) {
        sMx[quarter * 16 + (lane >> 2)] = mx[0];
        sMx[quarter * 16 + (lane >> 2) + 8] = mx[1];
      }
      __syncthreads();               // the four warps' maxima are there
      float corr[2];
      uint32_t pw[2][2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int r = (lane >> 2) + 8 * j;
        const float tile_max = fmaxf(fmaxf(sMx[r], sMx[16 + r]), fmaxf(sMx[32 + r], sMx[48 + r]));
        const float m_new = fmaxf(m[j], tile_max);
        corr[j] = (m_new == -INFINITY || m[j] == -INFINITY) ? (m_new == -INFINITY ? 1.f : 0.f) : expf(m[j] - m_new);
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = sv[j][e] == -INFINITY ? 0.f : expf(sv[j][e] - m_new);
          sv[j][e] = p;
          sum += p;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[j] = l[j] * corr[j] + sum;               // (this warp's keys only; the four warps' sums meet at the end)
        m[j] = m_new;
        pw[j][0] = pack2<T>(sv[j][0], sv[j][1]);
        pw[j][1] = pack2<T>(sv[j][2], sv[j][3]);
      }
      // the weights, rounded to the storage type, into the row tile's [16][TK] operand tile
      T* const sPt = sP + rt * 16 * LM_PS;
      const int r0 = lane >> 2, cc = quarter * KW + (lane & 3) * 2;
      *reinterpret_cast<uint32_t*>(&sPt[r0 * LM_PS + cc]) = pw[0][0];
      *reinterpret_cast<uint32_t*>(&sPt[(r0 + 8) * LM_PS + cc]) = pw[1][0];
      if constexpr (KW == 16) {
        *reinterpret_cast<uint32_t*>(&sPt[r0 * LM_PS + cc + 8]) = pw[0][1];
        *reinterpret_cast<uint32_t*>(&sPt[(r0 + 8) * LM_PS + cc + 8]) = pw[1][1];
      }
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        acc[j][0] *= corr[0];
        acc[j][1] *= corr[0];
        acc[j][2] *= corr[1];
        acc[j][3] *= corr[1];
      }
    }
    __syncthreads();                 // the row tile's weights are complete
    uint32_t pa[TK / 16][4];
#pragma unroll
    for (int kk = 0; kk < TK / 16; ++kk)
      lm_ldmatrix_x4(pa[kk], sP + (size_t)(rt * 16 + (lane & 15)) * LM_PS + kk * 16 + (lane >> 4) * 8);
    // ---- weighted values of this warp's quarter of the columns
#pragma unroll
    for (int kk = 0; kk < TK / 16; ++kk) {
      const T* vr = kb + (size_t)(kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * DKP + vbase + (lane >> 4) * 8;
#pragma unroll
      for (int j = 0; j < NV; j += 2) {
        if (j < nv) {
          uint32_t bv[4];
          lm_ldmatrix_x4_trans(bv, vr + j * 8);
          lm_mma<T>(acc[j], pa[kk], bv[0], bv[1]);
          if (j + 1 < nv) lm_mma<T>(acc[j + 1], pa[kk], bv[2], bv[3]);
        }
      }
    }
  }
  lm_wait<0>();
  pdl_launch();
  // the row sums of the four warps (each over its own keys, on the same sequence of maxima) in a fixed order
  {
    float* const sL = sS + NRT * 64 + rt * 64;
    __syncthreads();
    if ((lane & 3) == 0) {
      sL[quarter * 16 + (lane >> 2)] = l[0];
      sL[quarter * 16 + (lane >> 2) + 8] = l[1];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = (lane >> 2) + 8 * j;
      l[j] = (sL[r] + sL[16 + r]) + (sL[32 + r] + sL[48 + r]);
    }
  }
#pragma unroll
  for (int j2 = 0; j2 < 2; ++j2) {
    const int t = r_tok[j2];
    if (t < 0) continue;
    const int h = r_head[j2];
    if (part != nullptr) {
      float* p = part + (((size_t)t * H + h) * split_slots + blockIdx.y) * (Dv + 2);
      if (quarter == 0 && (lane & 3) == 0) {
        p[0] = m[j2];
        p[1] = l[j2];
      }
#pragma unroll
      for (int j = 0; j < NV; ++j)
        if (j < nv) {
          const int d = vbase + j * 8 + (lane & 3) * 2;
          p[2 + d] = acc[j][2 * j2];
          p[2 + d + 1] = acc[j][2 * j2 + 1];
        }
      continue;
    }
    const float f = (l[j2] > 0.f ? 1.0f / l[j2] : 0.f) * (gate != nullptr ? gate[(size_t)t * H + h] : 1.0f);
    T* o = out + (size_t)t * ldo + (size_t)h * Dv;
#pragma unroll
    for (int j = 0; j < NV; ++j)
      if (j < nv) {
        const int d = vbase + j * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(o + d) = pack2<T>(acc[j][2 * j2] * f, acc[j][2 * j2 + 1] * f);
      }
  }
}

// 1 where this kernel takes the shape and the pointers, else 0 (the CUDA-core kernel runs).
FERRUM_API int ferrum_attention_latent_mma_supported(int dtype, int Dk, int Dv, int ldq, int ldo, long long page_stride,
                                                     const void* q, const void* out, const void* plane) {
  return ferrum_is_16bit(dtype) && Dk % 16 == 0 && Dv % 32 == 0 && Dv <= 512 && Dv <= Dk && Dk <= 1024 && ldq % 8 == 0 && ldo % 2 == 0 &&
         page_stride % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)plane & 15) == 0 && ((uintptr_t)out & 3) == 0;
}

// For tests and measurements: 32 or 64 forces the stage size wherever it fits, 0 restores the rule.
static int g_force_stage = 0;
FERRUM_API void ferrum_attention_latent_mma_stage(int keys) { g_force_stage = (keys == 32 || keys == 64) ? keys : 0; }

FERRUM_API int ferrum_attention_latent_mma(const void* q, int ldq, void* out, int ldo, int dtype, const float* gate, int n_tokens,
                                           const int* positions, const int* q_start, int n_reqs, const int* block_table,
                                           int table_width, const void* plane, long long page_stride, int page_size, int H, int Dk,
                                           int Dv, float scale, int window, int single_tokens, float* part, int split_slots,
                                           int* err_flag, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && n_reqs > 0 && H > 0, "latent attention: bad sizes T=%d requests=%d H=%d", n_tokens, n_reqs, H);
  FERRUM_CHECK_ARG(ferrum_attention_latent_mma_supported(dtype, Dk, Dv, ldq, ldo, page_stride, q, out, plane),
                   "latent attention (tensor cores): shape Dk=%d Dv=%d or alignment not supported", Dk, Dv);
  FERRUM_CHECK_ARG(page_size > 0 && table_width > 0 && window >= 0, "latent attention: bad cache arguments");
  FERRUM_CHECK_ARG(ldq >= H * Dk && ldo >= H * Dv, "latent attention: a row stride is too short");
  FERRUM_CHECK_ARG(part == nullptr || (single_tokens && split_slots > 0 && split_slots <= 65535),
                   "latent attention: key splits are for steps of single tokens (slots %d)", split_slots);
  if (n_tokens == 0) return 0;
  int HB = 16;
  while (HB > 1 && HB / 2 >= H) HB /= 2;        // heads per row tile: the least power of two that holds H, at most 16
  const int TT = 16 / HB;
  const int hchunks = (H + HB - 1) / HB;
  const int nvq = Dv / 32;
#define LM_LAUNCH(NV_, NRT_, TK_)                                                                                              \
  do {                                                                                                                       \
    const LmSmem s = lm_smem(Dk, NRT_, TK_);                                                                                   \
    const int TQ_ = TT * NRT_;                                                                                               \
    const long long chunks = TQ_ == 1 ? n_tokens : (n_tokens + TQ_ - 1) / TQ_ + n_reqs;                                      \
    const long long ctas = chunks * hchunks;                                                                                 \
    FERRUM_CHECK_ARG(ctas < (1LL << 31), "latent attention: too many rows");                                                 \
    FERRUM_DISPATCH_16BIT(dtype, T, {                                                                                        \
      static int configured = 0;                                                                                             \
      if (configured < s.bytes) {                                                                                            \
        cudaError_t e = cudaFuncSetAttribute(attention_latent_mma_kernel<T, NV_, NRT_, TK_>,                                      \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, s.bytes);                          \
        FERRUM_CHECK_ARG(e == cudaSuccess, "latent attention: cannot reserve %d bytes of shared memory: %s", s.bytes,        \
                         cudaGetErrorString(e));                                                                             \
        configured = s.bytes;                                                                                                \
      }                                                                                                                      \
      launch_kernel(attention_latent_mma_kernel<T, NV_, NRT_, TK_>, dim3((unsigned)ctas, part ? split_slots : 1), dim3(128 * NRT_), \
                    (size_t)s.bytes, stream, (const T*)q, ldq, (T*)out, ldo, gate, positions, q_start, n_reqs, block_table,    \
                    table_width, (const T*)plane, page_stride, page_size, H, HB, Dk, Dv, scale, window, err_flag, s.DKP,       \
                    s.off_k, s.off_s, s.off_row, part, split_slots);                                                          \
    });                                                                                                                      \
  } while (0)
  // Prompt portions: three row tiles (12 warps) on stages of 64 keys where shared memory holds them, else
  // two, else (a very long key row) two on stages of 32 keys.  Single tokens: one row tile; stages of 32
  // keys let two CTAs share an SM, which pays once the grid has more than two CTAs per SM; a
  // smaller grid runs stages of 64 keys (fewer barriers per key).  (Measured at 16 heads, rows of
  // 576: prompt of 2,048 tokens 559 us against 684 us with four row tiles on stages of 32 keys; 8
  // single tokens over 8,192 keys 71 against 88 us, over 2,048 keys 32 against 26 us.)
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  bool big_grid = (long long)n_tokens * hchunks * (part ? split_slots : 1) > 2LL * sms;
  int fit64 = lm_smem(Dk, 3, 64).bytes <= LM_SMEM_LIMIT ? 3 : (lm_smem(Dk, 2, 64).bytes <= LM_SMEM_LIMIT ? 2 : 0);
  if (g_force_stage == 32) big_grid = true, fit64 = 0;
  if (g_force_stage == 64) big_grid = false;
#define LM_SHAPES(NV_)                                                          \
  do {                                                                          \
    if (single_tokens) {                                                        \
      if (big_grid || lm_smem(Dk, 1, 64).bytes > LM_SMEM_LIMIT) LM_LAUNCH(NV_, 1, 32); \
      else LM_LAUNCH(NV_, 1, 64);                                               \
    } else if (fit64 == 3) LM_LAUNCH(NV_, 3, 64);                               \
    else if (fit64 == 2) LM_LAUNCH(NV_, 2, 64);                                 \
    else LM_LAUNCH(NV_, 2, 32);                                                 \
  } while (0)
  if (nvq <= 4) LM_SHAPES(4);
  else if (nvq <= 8) LM_SHAPES(8);
  else LM_SHAPES(16);
#undef LM_SHAPES
#undef LM_LAUNCH
  FERRUM_CHECK_LAUNCH("attention_latent_mma");
  return 0;
}

// ================================================================= one product per head, many tokens
// y[t, h * ldyh + n] = sum_k x[t, h * ldxh + k] * w[h][n][k] on mma.sync: the per-head maps around
// the attention above (the key map folded into the queries, the value map after the weighted sum)
// for prompt-sized steps, all heads in ONE launch (grid z = head).  A CTA of eight warps makes a
// tile of 128 tokens x 128 features, k in steps of 32 through two shared-memory stages (cp.async);
// a warp owns 32 x 64 of the tile.  Needs K % 8 == 0 and 16-byte aligned rows.
constexpr int HM_BM = 128, HM_BN = 128, HM_BK = 32, HM_LD = HM_BK + 8;

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_mma_kernel(const T* __restrict__ x, int ldx, int ldxh, const T* __restrict__ w, T* __restrict__ y, int ldy, int ldyh,
                       int M, int N, int K) {
  __shared__ __align__(16) T sA[2][HM_BM * HM_LD];
  __shared__ __align__(16) T sB[2][HM_BN * HM_LD];
  pdl_launch();
  pdl_wait();
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = wid >> 1, wn = wid & 1;                 // warp rows wm * 32 .., columns wn * 64 ..
  const int m0 = blockIdx.x * HM_BM, n0 = blockIdx.y * HM_BN, h = blockIdx.z;
  const T* xh = x + (size_t)h * ldxh;
  const T* wh = w + (size_t)h * N * K;
  const int nk = (K + HM_BK - 1) / HM_BK;
  auto load = [&](int kb, int buf) {
    const int k0 = kb * HM_BK;
    for (int idx = threadIdx.x; idx < (HM_BM + HM_BN) * 4; idx += 256) {
      const bool isA = idx < HM_BM * 4;
      const int r = (isA ? idx : idx - HM_BM * 4) >> 2, kc = ((idx & 3) << 3);
      const bool there = k0 + kc < K && (isA ? m0 + r < M : n0 + r < N);
      const T* src = isA ? xh + (size_t)(m0 + r) * ldx + k0 + kc : wh + (size_t)(n0 + r) * K + k0 + kc;
      T* dst = (isA ? sA[buf] : sB[buf]) + r * HM_LD + kc;
      lm_cp_async16(dst, there ? src : (isA ? x : w), there ? 16 : 0);
    }
  };
  float acc[2][8][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
  load(0, 0);
  lm_commit();
  for (int kb = 0; kb < nk; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nk) load(kb + 1, buf ^ 1);
    lm_commit();
    lm_wait<1>();
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < HM_BK / 16; ++ks) {
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        lm_ldmatrix_x4(a[i], &sA[buf][(wm * 32 + i * 16 + (lane & 15)) * HM_LD + ks * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t b[4];
        lm_ldmatrix_x4(b, &sB[buf][(wn * 64 + j * 8 + (lane & 7) + ((lane >> 4) << 3)) * HM_LD + ks * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          lm_mma<T>(acc[i][j], a[i], b[0], b[1]);
          lm_mma<T>(acc[i][j + 1], a[i], b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  lm_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int t = m0 + wm * 32 + i * 16 + (lane >> 2) + half * 8;
      if (t >= M) continue;
      T* yr = y + (size_t)t * ldy + (size_t)h * ldyh;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = n0 + wn * 64 + j * 8 + (lane & 3) * 2;
        if (n + 1 < N) *reinterpret_cast<uint32_t*>(yr + n) = pack2<T>(acc[i][j][half * 2], acc[i][j][half * 2 + 1]);
        else if (n < N) yr[n] = from_f32<T>(acc[i][j][half * 2]);
      }
    }
}

FERRUM_API int ferrum_head_linear_mma_supported(int dtype, int K, int ldx, int ldxh, int ldy, int ldyh, const void* x, const void* w,
                                                const void* y) {
  return ferrum_is_16bit(dtype) && K % 8 == 0 && ldx % 8 == 0 && ldxh % 8 == 0 && ldy % 2 == 0 && ldyh % 2 == 0 &&
         ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)y & 3) == 0;
}

FERRUM_API int ferrum_head_linear_mma(const void* x, int ldx, int ldxh, const void* w, void* y, int ldy, int ldyh, int dtype, int M,
                                      int H, int N, int K, cudaStream_t stream) {
  FERRUM_CHECK_ARG(M >= 0 && H > 0 && H <= 65535 && N > 0 && K > 0, "head linear: bad sizes M=%d H=%d N=%d K=%d", M, H, N, K);
  FERRUM_CHECK_ARG(ferrum_head_linear_mma_supported(dtype, K, ldx, ldxh, ldy, ldyh, x, w, y), "head linear (tensor cores): K=%d or alignment not supported", K);
  FERRUM_CHECK_ARG(ldyh >= N && ldx >= (H - 1) * ldxh + K && ldy >= (H - 1) * ldyh + N, "head linear: a stride is too short");
  if (M == 0) return 0;
  const dim3 grid((M + HM_BM - 1) / HM_BM, (N + HM_BN - 1) / HM_BN, H);
  FERRUM_CHECK_ARG(grid.y <= 65535, "head linear: too many features");
  FERRUM_DISPATCH_16BIT(dtype, T, launch_kernel(head_linear_mma_kernel<T>, grid, dim3(256), 0, stream, (const T*)x, ldx, ldxh, (const T*)w,
                                                (T*)y, ldy, ldyh, M, N, K));
  FERRUM_CHECK_LAUNCH("head_linear_mma");
  return 0;
}
