// Queries, keys and values on their way from the projection into the attention kernels:
//   q, k   optional RMS norm over the WHOLE projection of a token (all heads at once, one weight per
//          column, eps inside the root), then a rotation by position of the first 2*half dimensions of
//          every head: dimension i is paired with i + half, the pair (u, v) at position p becomes
//          (u cos a - v sin a, v cos a + u sin a) with a = p * freq[i]; the other dimensions pass.
//   q      goes to a buffer [tokens, Hq*Dh]; k and v go into the token's page.  Heads are laid out Dh
//          wide there (values: Dvr wide), Dh >= dk, Dvr >= dv, the columns beyond a head's own size are written as zeros, so
//          that attention kernels built for one head size serve keys and values of different sizes
//          (zeros add nothing to a score, and the value columns they produce are never read).
//   Options: the pairs of a rotation may be neighbours instead ((2i, 2i+1), `interleaved`); cosine and sine may both
//   carry a factor (`mscale`, what a stretched rotation multiplies them with); every head of q and of k may be divided
//   by its root mean square over its dk columns after the rotation (no weight, `head_eps` >= 0); the values may have
//   fewer heads than the keys (Hv of them, [n_pages, Hv, page, Dvr]: several key heads then read one value head); every value head may be
//   divided by its root mean square over its dv columns (no weight, `v_eps` >= 0) before it enters the page; q may
//   leave in float32 whatever the activation dtype is (for attention kernels that take float32 queries).
// Norm, angle, sine and cosine are float32 (the angle is the float32 product of the position and a
// float32 frequency, reduced accurately by sincosf).
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

template <typename T, typename TQ>
__global__ void qkv_prepare_kernel(const T* proj, int ld, int q_off, int k_off, int v_off, int Hq, int Hkv, int dk,
                                   int dv, int Dh, const float* __restrict__ wq, const float* __restrict__ wk,
                                   float eps, const float* __restrict__ freq, int half,
                                   const int* __restrict__ positions, const int* __restrict__ token_req,
                                   const int* __restrict__ block_table, int max_pages, int n_pages, int page,
                                   TQ* __restrict__ q_out, int ldq, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                   int write, int* __restrict__ status, int interleaved, float v_eps, int Dvr, int Hv,
                                   float mscale, float head_eps) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int r = token_req[t];
  if (r < 0) return;
  const int p = positions[t];
  long long slot = -1;      // the token's row in head 0 of its page, counted in rows
  long long vslot = -1;     // the same among the value heads (Hv of them)
  if (write) {
    const int lp = p / page;
    if (p < 0 || lp >= max_pages) {
      if (threadIdx.x == 0) atomicOr(status, MLXB_ST_POSITION_RANGE);
    } else {
      const int pg = block_table[(size_t)r * max_pages + lp];
      if (pg >= n_pages) {
        if (threadIdx.x == 0) atomicOr(status, MLXB_ST_PAGE_RANGE);
      } else if (pg >= 0) {
        slot = (long long)pg * Hkv * page + (p % page);
        vslot = (long long)pg * Hv * page + (p % page);
      }
    }
  }
  pdl_wait();
  pdl_trigger();
  proj = after_wait(proj);
  const T* row = proj + (size_t)t * ld;
  float rq = 1.f, rk = 1.f;
  if (wq) {
    float s = 0.f;
    for (int e = threadIdx.x; e < Hq * dk; e += blockDim.x) { const float v = to_f(row[q_off + e]); s = fmaf(v, v, s); }
    rq = 1.f / sqrtf(block_sum(s, red) / (float)(Hq * dk) + eps);
  }
  if (wk) {
    float s = 0.f;
    for (int e = threadIdx.x; e < Hkv * dk; e += blockDim.x) { const float v = to_f(row[k_off + e]); s = fmaf(v, v, s); }
    rk = 1.f / sqrtf(block_sum(s, red) / (float)(Hkv * dk) + eps);
  }
  const float fp = (float)p;
  if (head_eps >= 0.f) {
    // every head of q and of k divided by its root mean square AFTER the rotation: a warp a head, which forms the
    // head's values twice (for the sum of squares, then to write them)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int hh = warp; hh < Hq + Hkv; hh += nw) {
      const bool is_q = hh < Hq;
      const int h = is_q ? hh : hh - Hq;
      if (!is_q && slot < 0) continue;
      const T* src = row + (is_q ? q_off : k_off) + (size_t)h * dk;
      const float* w = is_q ? wq : wk;
      const float rn = is_q ? rq : rk;
      auto value = [&](int i) {
        float x = to_f(src[i]) * rn;
        if (w) x *= w[h * dk + i];
        if (i >= 2 * half) return x;
        const bool lower = interleaved ? !(i & 1) : i < half;
        const int partner = interleaved ? (i ^ 1) : (lower ? i + half : i - half);
        float y = to_f(src[partner]) * rn;
        if (w) y *= w[h * dk + partner];
        float sn, cs;
        sincosf(fp * freq[interleaved ? i >> 1 : (lower ? i : i - half)], &sn, &cs);
        cs *= mscale;
        sn *= mscale;
        return lower ? x * cs - y * sn : x * cs + y * sn;
      };
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) { const float a = value(i); ss = fmaf(a, a, ss); }
      const float rinv = 1.f / sqrtf(warp_sum(ss) / (float)dk + head_eps);
      for (int i = lane; i < Dh; i += 32) {
        const float a = i < dk ? value(i) * rinv : 0.f;
        if (is_q) q_out[(size_t)t * ldq + (size_t)h * Dh + i] = from_f<TQ>(a);
        else k_pool[(size_t)(slot + (long long)h * page) * Dh + i] = from_f<T>(a);
      }
    }
  }
  // one thread per (head, dimension below Dh) of q and of k; the lower partner of a pair computes both
  for (int e = threadIdx.x; e < (head_eps >= 0.f ? 0 : (Hq + Hkv) * Dh); e += blockDim.x) {
    const int hh = e / Dh, i = e - hh * Dh;
    const bool is_q = hh < Hq;
    const int h = is_q ? hh : hh - Hq;
    const int off = is_q ? q_off : k_off;
    const float* w = is_q ? wq : wk;
    const float rn = is_q ? rq : rk;
    TQ* dq = nullptr;
    T* dk_ = nullptr;
    if (is_q) dq = q_out + (size_t)t * ldq + (size_t)h * Dh;
    else if (slot >= 0) dk_ = k_pool + (size_t)(slot + (long long)h * page) * Dh;
    else continue;
    float a = 0.f, b = 0.f;     // what goes to column i and, for the lower partner of a pair, to column j
    int j = -1;
    if (i < dk) {
      const bool rotated = i < 2 * half;
      if (rotated && (interleaved ? (i & 1) : i >= half)) continue;      // written by its partner
      const int c = h * dk + i;
      float u = to_f(row[off + c]) * rn;
      if (w) u *= w[c];
      if (rotated) {
        const int step = interleaved ? 1 : half;
        float v = to_f(row[off + c + step]) * rn;
        if (w) v *= w[c + step];
        float sn, cs;
        sincosf(fp * freq[interleaved ? i >> 1 : i], &sn, &cs);
        cs *= mscale;
        sn *= mscale;
        a = u * cs - v * sn;
        b = v * cs + u * sn;
        j = i + step;
      } else {
        a = u;
      }
    }
    if (is_q) {
      dq[i] = from_f<TQ>(a);
      if (j >= 0) dq[j] = from_f<TQ>(b);
    } else {
      dk_[i] = from_f<T>(a);
      if (j >= 0) dk_[j] = from_f<T>(b);
    }
  }
  if (slot >= 0 && v_eps >= 0.f) {
    // every value head divided by its root mean square: a warp a head
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = warp; h < Hv; h += nw) {
      float s = 0.f;
      for (int i = lane; i < dv; i += 32) { const float v = to_f(row[v_off + h * dv + i]); s = fmaf(v, v, s); }
      const float rv = 1.f / sqrtf(warp_sum(s) / (float)dv + v_eps);
      for (int i = lane; i < Dvr; i += 32)
        v_pool[(size_t)(vslot + (long long)h * page) * Dvr + i] = from_f<T>(i < dv ? to_f(row[v_off + h * dv + i]) * rv : 0.f);
    }
  } else if (slot >= 0) {
    for (int e = threadIdx.x; e < Hv * Dvr; e += blockDim.x) {
      const int h = e / Dvr, i = e - h * Dvr;
      v_pool[(size_t)(vslot + (long long)h * page) * Dvr + i] = i < dv ? row[v_off + h * dv + i] : from_f<T>(0.f);
    }
  }
}

// proj: [n_tokens, ...] at row stride ld holding q (Hq*dk columns from q_off), k (Hkv*dk from k_off) and v (Hkv*dv
// from v_off); interleaved: pairs (2i, 2i+1) instead of (i, i+half); v_eps >= 0: value heads divided by their root mean
// square with this eps; Hv: value heads (0: as many as key heads); mscale: factor on cosine and sine; head_eps >= 0: q and k
// heads divided by their root mean square after the rotation; q_f32: q_out is float32 whatever dtype says; wq / wk: float32 norm weights over the whole q / k projection, or null for no norm; freq: float32
// [half] rotation frequencies (half may be 0); k_pool [n_pages, Hkv, page, Dh], v_pool [n_pages, Hkv, page, Dvr]; q_out [n_tokens, Hq*Dh] at row stride ldq.
MLXB_EXPORT int mlxb_qkv_prepare(int dtype, const void* proj, int ld, int q_off, int k_off, int v_off, int Hq, int Hkv,
                                 int dk, int dv, int Dh, const float* wq, const float* wk, float eps, const float* freq,
                                 int half, const int* positions, const int* token_req, const int* block_table,
                                 int max_pages, int n_pages, int page, void* q_out, int ldq, void* k_pool, void* v_pool,
                                 int write, int n_tokens, int* status, int interleaved, float v_eps, int q_f32, int Dvr,
                                 int Hv, float mscale, float head_eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (Hv <= 0) Hv = Hkv;
  if (Hq <= 0 || Hkv <= 0 || dk <= 0 || dv <= 0 || Dh < dk || Dvr < dv || 2 * half > dk || half < 0 || page <= 0 ||
      (half > 0 && freq == nullptr) || ldq < Hq * Dh)
    return mlxb_fail(MLXB_BAD_ARG, "qkv_prepare: %d/%d heads, sizes %d/%d in %d, %d rotated pairs, page %d", Hq, Hkv, dk,
                     dv, Dh, half, page);
  const int work = (Hq + Hkv) * Dh;
  const int threads = work >= 2048 ? 256 : (work >= 512 ? 128 : 64);
#define QKVP_GO(T, TQ)                                                                                                  \
  launch_pdl(qkv_prepare_kernel<T, TQ>, dim3(n_tokens), dim3(threads), 0, stream, (const T*)proj, ld, q_off, k_off, v_off, \
             Hq, Hkv, dk, dv, Dh, wq, wk, eps, freq, half, positions, token_req, block_table, max_pages, n_pages, page,  \
             (TQ*)q_out, ldq, (T*)k_pool, (T*)v_pool, write, status, interleaved, v_eps, Dvr, Hv, mscale, head_eps)
  if (dtype == MLXB_F32) QKVP_GO(float, float);
  else if (dtype == MLXB_BF16 && q_f32) QKVP_GO(__nv_bfloat16, float);
  else if (dtype == MLXB_BF16) QKVP_GO(__nv_bfloat16, __nv_bfloat16);
  else return mlxb_fail(MLXB_BAD_DTYPE, "qkv_prepare: dtype code %d", dtype);
#undef QKVP_GO
  return mlxb_check_launch("qkv_prepare");
}
