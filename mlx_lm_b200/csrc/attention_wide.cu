// Attention over the paged cache where one CTA takes a query token with a whole group of heads, 32-bit math.
//
// What it serves that the per-head kernels do not:
//   * scores mixed across heads before the softmax ("talking heads"): s'_h = sum_g talk[h, g] s_g, where
//     s_g = scale * q_g . k_kv(g) is head g's raw score for the same (query, key) pair.  All heads of the
//     query must then be in one CTA (the group is all heads);
//   * fewer value heads than key heads (Hv of them: key heads c * Hkv/Hv .. read value head c; several score maps
//     over the same values);
//   * keys and values of different widths, and values that are a prefix of the key row itself (v_pool may be
//     k_pool: a cache of latent rows [c | rotated part] read as keys of width Dk and as values of width Dv);
//   * the visible keys of position p given by a window (p - window < j <= p), by chunks counted from position
//     0 of the sequence (floor(j / chunk) = floor(p / chunk), j <= p), or both; beside a window, the first
//     `keep_first` positions of the sequence stay visible to every later position (j < keep_first);
//   * scores bounded by a soft cap: s <- cap * tanh(s / cap), after the scale and before the softmax;
//   * an output gate: head h's output times sigmoid(gate[t, h]), or, with `gate_cols`, every output column with a
//     gate of its own, sigmoid(gate[t, h * Dv + d]).
//
// The query arrives in float32 (q + t*ldq + h*qhs, Dk values); a key row lies at
// ((pg*Hkv + c)*page + row)*krs in k_pool, a value row at the same index times vrs in v_pool.
//
// A CTA walks the visible keys in blocks of 64 from the first visible one upwards (kept first positions that the
// window has passed come first, in blocks of 64 from position 0):
//   A  one thread per (key, head): the dot product, times scale               -> raw scores in shared memory
//   A' (with talk) one thread per (key, head): the mix over heads             -> mixed scores
//   B  one warp per head: running maximum, weights exp(s - m), running sum, the correction of what was summed
//   C  one thread per (head, pair of value columns): o = o * corr + sum_j w_j v_j over the block's keys
// and divides by the sum at the end.  The order of additions for a token depends on its position and the
// layer's sizes only, so a token's result is the same bits whether it came alone or inside a portion.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int AW_THREADS = 256;
constexpr int AW_KB = 64;      // keys per block
constexpr int AW_MAXO = 8;     // (head, column group) items a thread accumulates
constexpr int AW_MAXH = 64;    // heads a CTA takes at most

template <typename T>
struct KVec;   // 16 bytes of keys
template <>
struct KVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
  }
};
template <>
struct KVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    unpack8(*reinterpret_cast<const uint4*>(p), v);
  }
};

template <typename T>
__device__ __forceinline__ void load2(const T* p, float& a, float& b);
template <>
__device__ __forceinline__ void load2<float>(const float* p, float& a, float& b) {
  const float2 u = *reinterpret_cast<const float2*>(p);
  a = u.x; b = u.y;
}
template <>
__device__ __forceinline__ void load2<__nv_bfloat16>(const __nv_bfloat16* p, float& a, float& b) {
  const unsigned u = *reinterpret_cast<const unsigned*>(p);
  a = __uint_as_float(u << 16);
  b = __uint_as_float(u & 0xffff0000u);
}

template <typename T, typename TO, bool VECK, bool VECV>
__global__ void __launch_bounds__(AW_THREADS)
attention_wide_kernel(const float* q, int ldq, int qhs, const int* __restrict__ positions,
                      const int* __restrict__ token_req, const int* __restrict__ block_table, int max_pages,
                      int n_pages, int page, int Hq, int Hkv, int HB, int Dk, int Dv, int krs, int vrs, int window,
                      int chunk, float scale, const float* __restrict__ talk, const T* k_pool, const T* v_pool,
                      const T* gate, int ldg, TO* __restrict__ out, int ldo, int ohs, const int* __restrict__ rows,
                      int* __restrict__ status, float softcap, int keep_first, int gate_cols, int Hv) {
  extern __shared__ __align__(16) unsigned char aw_smem[];
  const int DkP = (Dk + 3) & ~3;
  long long* sRow = reinterpret_cast<long long*>(aw_smem);   // [KB] row of the key in head 0 of its page, or -1
  long long* sRowV = sRow + AW_KB;                           // [KB] the same among the value heads
  float* sq = reinterpret_cast<float*>(sRowV + AW_KB);       // [HB][DkP]
  float* sS = sq + HB * DkP;                                 // [HB][KB] raw scores
  float* sP = sS + HB * AW_KB;                               // [HB][KB] mixed scores, then weights
  float* sT = sP + HB * AW_KB;                               // [HB][HB] the mixing matrix
  float* sM = sT + HB * HB;                                  // [HB] running maximum
  float* sC = sM + HB;                                       // [HB] correction of this block
  float* sL = sC + HB;                                       // [HB] running sum
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ti = blockIdx.x, h0 = blockIdx.y * HB;
  const int t = rows ? rows[ti] : ti;
  const int r = token_req[t];
  if (r < 0) return;   // a row that pads the step
  const int p = positions[t];
  if (talk)
    for (int e = tid; e < HB * HB; e += AW_THREADS) sT[e] = talk[e];
  for (int e = tid; e < HB; e += AW_THREADS) { sM[e] = -INFINITY; sL[e] = 0.f; sC[e] = 0.f; }
  pdl_wait();
  pdl_trigger();
  q = after_wait(q);
  k_pool = after_wait(k_pool);
  v_pool = after_wait(v_pool);
  gate = after_wait(gate);
  for (int e = tid; e < HB * DkP; e += AW_THREADS) {
    const int hh = e / DkP, d = e - hh * DkP;
    sq[e] = d < Dk ? q[(size_t)t * ldq + (size_t)(h0 + hh) * qhs + d] : 0.f;
  }
  const int* bt = block_table + (size_t)r * max_pages;
  const int rep = Hq / Hkv, vrep = rep * (Hkv / Hv);       // query heads a key head, and a value head, serves
  int lo = 0;
  if (window > 0 && p - window + 1 > lo) lo = p - window + 1;
  if (chunk > 0 && (p / chunk) * chunk > lo) lo = (p / chunk) * chunk;

  constexpr int VV = VECV ? 2 : 1;
  const int DvV = Dv / VV, n_items = HB * DvV;
  float o[AW_MAXO][2];
  int item_h[AW_MAXO], item_d[AW_MAXO];
#pragma unroll
  for (int i = 0; i < AW_MAXO; ++i) {
    o[i][0] = o[i][1] = 0.f;
    const int it = tid + i * AW_THREADS;
    item_h[i] = it < n_items ? it / DvV : 0;
    item_d[i] = it < n_items ? (it - item_h[i] * DvV) * VV : 0;
  }

  const int kf = min(keep_first, lo);        // kept first positions that lie before the window
  int j0 = kf > 0 ? 0 : lo, j_end = kf > 0 ? kf - 1 : p;
  for (;;) {
    const int nk = min(AW_KB, j_end - j0 + 1);
    __syncthreads();        // the block before is done with sRow and sP (first pass: sq, sM are written)
    if (tid < AW_KB) {
      long long row = -1, vrow = -1;
      if (tid < nk) {
        const int j = j0 + tid, lp = j / page;
        const int pg = lp < max_pages ? bt[lp] : -1;
        if (pg >= n_pages) atomicOr(status, MLXB_ST_PAGE_RANGE);
        else if (pg < 0) atomicOr(status, MLXB_ST_POSITION_RANGE);   // a key inside the range has no page
        else { row = (long long)pg * Hkv * page + (j % page); vrow = (long long)pg * Hv * page + (j % page); }
      }
      sRow[tid] = row;
      sRowV[tid] = vrow;
    }
    __syncthreads();
    // A: raw scores
    for (int it = tid; it < HB * AW_KB; it += AW_THREADS) {
      const int hh = it / AW_KB, jj = it - hh * AW_KB;
      float s = -INFINITY;
      const long long row = sRow[jj];
      if (row >= 0) {
        const int c = (h0 + hh) / rep;
        const T* kp = k_pool + (size_t)(row + (long long)c * page) * krs;
        const float* qh = sq + hh * DkP;
        float a = 0.f;
        if (VECK) {
          constexpr int N = KVec<T>::N;
          for (int d = 0; d < Dk; d += N) {
            float kv[N];
            KVec<T>::load(kp + d, kv);
#pragma unroll
            for (int e = 0; e < N; e += 4) {
              const float4 qq = *reinterpret_cast<const float4*>(qh + d + e);
              a = fmaf(qq.x, kv[e], a);
              a = fmaf(qq.y, kv[e + 1], a);
              a = fmaf(qq.z, kv[e + 2], a);
              a = fmaf(qq.w, kv[e + 3], a);
            }
          }
        } else {
          for (int d = 0; d < Dk; ++d) a = fmaf(qh[d], to_f(kp[d]), a);
        }
        s = a * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      }
      (talk ? sS : sP)[it] = s;
    }
    if (talk) {
      __syncthreads();
      for (int it = tid; it < HB * AW_KB; it += AW_THREADS) {
        const int hh = it / AW_KB, jj = it - hh * AW_KB;
        float s = -INFINITY;
        if (sRow[jj] >= 0) {
          s = 0.f;
          for (int g = 0; g < HB; ++g) s = fmaf(sT[hh * HB + g], sS[g * AW_KB + jj], s);
        }
        sP[it] = s;
      }
    }
    __syncthreads();
    // B: per head, the block's maximum and weights
    for (int hh = warp; hh < HB; hh += AW_THREADS / 32) {
      float* ph = sP + hh * AW_KB;
      const float s0 = ph[lane], s1 = ph[lane + 32];
      const float m_old = sM[hh];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
      const float p0 = s0 == -INFINITY ? 0.f : expf(s0 - m_new);
      const float p1 = s1 == -INFINITY ? 0.f : expf(s1 - m_new);
      const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
      const float sum = warp_sum(p0 + p1);
      ph[lane] = p0;
      ph[lane + 32] = p1;
      if (lane == 0) {
        sM[hh] = m_new;
        sC[hh] = corr;
        sL[hh] = sL[hh] * corr + sum;
      }
    }
    __syncthreads();
    // C: values
#pragma unroll
    for (int i = 0; i < AW_MAXO; ++i) {
      if (tid + i * AW_THREADS < n_items) {
        const float corr = sC[item_h[i]];
        o[i][0] *= corr;
        o[i][1] *= corr;
      }
    }
    for (int jj = 0; jj < nk; ++jj) {
      const long long row = sRowV[jj];
      if (row < 0) continue;
#pragma unroll
      for (int i = 0; i < AW_MAXO; ++i) {
        if (tid + i * AW_THREADS < n_items) {
          const int hh = item_h[i];
          const float w = sP[hh * AW_KB + jj];
          const T* vp = v_pool + (size_t)(row + (long long)((h0 + hh) / vrep) * page) * vrs + item_d[i];
          if (VECV) {
            float a, b;
            load2<T>(vp, a, b);
            o[i][0] = fmaf(w, a, o[i][0]);
            o[i][1] = fmaf(w, b, o[i][1]);
          } else {
            o[i][0] = fmaf(w, to_f(vp[0]), o[i][0]);
          }
        }
      }
    }
    j0 += AW_KB;
    if (j0 > j_end) {
      if (j_end == p) break;
      j0 = lo;             // the kept positions are done: on to the window
      j_end = p;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < AW_MAXO; ++i) {
    if (tid + i * AW_THREADS < n_items) {
      const int hh = item_h[i], h = h0 + hh;
      const float l = sL[hh];
      const float f = l > 0.f ? 1.f / l : 0.f;
      float g0 = 1.f, g1 = 1.f;
      if (gate) {
        const T* gp = gate + (size_t)t * ldg + (gate_cols ? (size_t)h * Dv + item_d[i] : (size_t)h);
        g0 = 1.f / (1.f + expf(-to_f(gp[0])));
        g1 = (VECV && gate_cols) ? 1.f / (1.f + expf(-to_f(gp[1]))) : g0;
      }
      TO* op = out + (size_t)t * ldo + (size_t)h * ohs + item_d[i];
      op[0] = from_f<TO>(o[i][0] * f * g0);
      if (VECV) op[1] = from_f<TO>(o[i][1] * f * g1);
    }
  }
}

template <typename T, typename TO>
static int aw_launch(const float* q, int ldq, int qhs, const int* positions, const int* token_req,
                     const int* block_table, int max_pages, int n_pages, int page, int Hq, int Hkv, int HB, int Dk,
                     int Dv, int krs, int vrs, int window, int chunk, float scale, const float* talk,
                     const void* k_pool, const void* v_pool, const void* gate, int ldg, void* out, int ldo, int ohs,
                     const int* rows, int n_tokens, int* status, float softcap, int keep_first, int gate_cols, int Hv,
                     cudaStream_t stream) {
  constexpr int NK = KVec<T>::N;
  const bool veck = Dk % NK == 0 && krs % NK == 0 && ((uintptr_t)k_pool & 15) == 0;
  const bool vecv = Dv % 2 == 0 && vrs % 2 == 0 && ((uintptr_t)v_pool & (2 * sizeof(T) - 1)) == 0;
  const int items = HB * (vecv ? Dv / 2 : Dv);
  if (items > AW_MAXO * AW_THREADS)
    return mlxb_fail(MLXB_BAD_ARG, "attention (wide): %d heads of %d value columns are more than a CTA takes", HB, Dv);
  const int DkP = (Dk + 3) & ~3;
  const size_t smem = sizeof(long long) * 2 * AW_KB +
                      sizeof(float) * ((size_t)HB * DkP + 2 * (size_t)HB * AW_KB + (size_t)HB * HB + 3 * (size_t)HB);
  const dim3 grid(n_tokens, Hq / HB), block(AW_THREADS);
#define AW_GO(VK, VV)                                                                                                  \
  do {                                                                                                                 \
    auto kern = attention_wide_kernel<T, TO, VK, VV>;                                                                  \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
      if (e != cudaSuccess)                                                                                            \
        return mlxb_fail((int)e, "attention (wide): %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));    \
    }                                                                                                                  \
    launch_pdl(kern, grid, block, smem, stream, q, ldq, qhs, positions, token_req, block_table, max_pages, n_pages,    \
               page, Hq, Hkv, HB, Dk, Dv, krs, vrs, window, chunk, scale, talk, (const T*)k_pool, (const T*)v_pool,    \
               (const T*)gate, ldg, (TO*)out, ldo, ohs, rows, status, softcap, keep_first, gate_cols, Hv);                 \
  } while (0)
  if (veck && vecv) AW_GO(true, true);
  else if (veck) AW_GO(true, false);
  else if (vecv) AW_GO(false, true);
  else AW_GO(false, false);
#undef AW_GO
  return mlxb_check_launch("attention (wide)");
}

// q: float32 [*, ldq], head h from column h*qhs, Dk values; pools in `dtype` with rows krs / vrs wide; talk: float32
// [Hq, Hq] or null; gate: `dtype` [*, ldg] (one column per head) or null; out: `dtype`, or float32 if out_f32, head h
// from column h*ohs, Dv values; rows: int32 [n_tokens] token rows to take, or null for 0..n_tokens-1;
// window, chunk <= 0: none; softcap <= 0: none; keep_first: positions 0 .. keep_first-1 stay visible beside the window;
// gate_cols: gate has Hq * Dv columns, one per output column.  Hv: heads of v_pool (0: Hkv).
MLXB_EXPORT int mlxb_attention_wide(int dtype, int out_f32, const float* q, int ldq, int qhs, const int* positions,
                                    const int* token_req, const int* block_table, int max_pages, int n_pages, int page,
                                    int Hq, int Hkv, int Dk, int Dv, int krs, int vrs, int window, int chunk,
                                    float scale, const float* talk, const void* k_pool, const void* v_pool,
                                    const void* gate, int ldg, void* out, int ldo, int ohs, const int* rows,
                                    int n_tokens, int* status, float softcap, int keep_first, int gate_cols, int Hv,
                                    cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (Hv <= 0) Hv = Hkv;
  if (Hkv % Hv) return mlxb_fail(MLXB_BAD_ARG, "attention (wide): %d key heads over %d value heads", Hkv, Hv);
  if (page <= 0 || (page & (page - 1)) || Hq <= 0 || Hkv <= 0 || Hq % Hkv || Dk <= 0 || Dv <= 0 || krs < Dk || vrs < Dv ||
      qhs < Dk || ohs < Dv)
    return mlxb_fail(MLXB_BAD_ARG, "attention (wide): %d/%d heads, sizes %d/%d in rows of %d/%d, page %d", Hq, Hkv, Dk,
                     Dv, krs, vrs, page);
  int HB = Hq;
  if (talk) {
    if (Hq > AW_MAXH) return mlxb_fail(MLXB_BAD_ARG, "attention (wide): scores mixed over %d heads (at most %d)", Hq, AW_MAXH);
  } else {
    // independent heads: as many a CTA as its threads have accumulators for, and no more than 8
    while (HB > 1 && (HB > 8 || HB * ((Dv + 1) / 2) > AW_MAXO * AW_THREADS || Hq % HB)) --HB;
  }
  if (dtype == MLXB_F32)
    return aw_launch<float, float>(q, ldq, qhs, positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv, HB,
                                   Dk, Dv, krs, vrs, window, chunk, scale, talk, k_pool, v_pool, gate, ldg, out, ldo, ohs,
                                   rows, n_tokens, status, softcap, keep_first, gate_cols, Hv, stream);
  if (dtype == MLXB_BF16 && out_f32)
    return aw_launch<__nv_bfloat16, float>(q, ldq, qhs, positions, token_req, block_table, max_pages, n_pages, page, Hq,
                                           Hkv, HB, Dk, Dv, krs, vrs, window, chunk, scale, talk, k_pool, v_pool, gate,
                                           ldg, out, ldo, ohs, rows, n_tokens, status, softcap, keep_first, gate_cols, Hv, stream);
  if (dtype == MLXB_BF16)
    return aw_launch<__nv_bfloat16, __nv_bfloat16>(q, ldq, qhs, positions, token_req, block_table, max_pages, n_pages,
                                                   page, Hq, Hkv, HB, Dk, Dv, krs, vrs, window, chunk, scale, talk, k_pool,
                                                   v_pool, gate, ldg, out, ldo, ohs, rows, n_tokens, status, softcap, keep_first, gate_cols, Hv, stream);
  return mlxb_fail(MLXB_BAD_DTYPE, "attention (wide): dtype code %d", dtype);
}
