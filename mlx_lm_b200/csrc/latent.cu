// Attention over a cache of latent rows (keys and values of all heads compressed into one short vector per
// token): what stands around the attention kernel.
//
// latent_prepare  From a fused projection of a token, [q | down]: `down` holds R latent columns and dr columns of a
//                 rotated key part that all heads share.  The latent columns are divided by their root mean square
//                 and multiplied by a weight (c); the key part is rotated by the position; [c | rotated part | 0..]
//                 becomes the token's row in the pages (one "head", Dh >= R + dr wide).  Of every query head
//                 ([d unrotated | dr rotated] in the projection) the rotated part is rotated the same way and put,
//                 in float32, behind the R columns that head_linear fills: q_lat[t, h] = [W_uk_h^T q_h | rotated q].
//                 Pairs of a rotation: (2i, 2i+1) (`interleaved`) or (i, i + dr/2); angle p * freq[i], float32; cosine
//                 and sine both times `mscale` (what a stretched rotation multiplies them with; 1: a plain one).
// head_linear     out[t, h, n] = sum_k x[t, h, k] * w[h, n, k]: a product per head, each head with its own matrix.
//                 Absorbs the keys' up-projection into the queries (q_h -> W_uk_h^T q_h, so that scores are taken
//                 against the latent rows directly) and applies the values' up-projection to the attention's output
//                 over latent rows.  float32 accumulation in a fixed order (k ascending); x and out may be float32
//                 beside bfloat16 weights, so that nothing is rounded between the attention and these products.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

template <typename T>
__global__ void latent_prepare_kernel(const T* proj, int ld, int q_off, int c_off, int H, int d, int dr, int R,
                                      const float* __restrict__ w, float eps, const float* __restrict__ freq,
                                      int interleaved, const int* __restrict__ positions,
                                      const int* __restrict__ token_req, const int* __restrict__ block_table,
                                      int max_pages, int n_pages, int page, int Dh, T* __restrict__ pool, int write,
                                      float* __restrict__ q_lat, int ldq, int qhs, int* __restrict__ status,
                                      float mscale) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int r = token_req[t];
  if (r < 0) return;
  const int p = positions[t];
  long long slot = -1;
  if (write) {
    const int lp = p / page;
    if (p < 0 || lp >= max_pages) {
      if (threadIdx.x == 0) atomicOr(status, MLXB_ST_POSITION_RANGE);
    } else {
      const int pg = block_table[(size_t)r * max_pages + lp];
      if (pg >= n_pages) {
        if (threadIdx.x == 0) atomicOr(status, MLXB_ST_PAGE_RANGE);
      } else if (pg >= 0) {
        slot = ((long long)pg * page + (p % page)) * Dh;
      }
    }
  }
  pdl_wait();
  pdl_trigger();
  proj = after_wait(proj);
  const T* row = proj + (size_t)t * ld;
  const int half = dr / 2;
  const float fp = (float)p;
  // rotated parts: H query heads, then the shared key part
  for (int e = threadIdx.x; e < (H + 1) * half; e += blockDim.x) {
    const int hh = e / half, i = e - hh * half;
    const int lo = interleaved ? 2 * i : i, hi = interleaved ? 2 * i + 1 : i + half;
    const T* src = hh < H ? row + q_off + (size_t)hh * (d + dr) + d : row + c_off + R;
    const float u = to_f(src[lo]), v = to_f(src[hi]);
    float sn, cs;
    sincosf(fp * freq[i], &sn, &cs);
    cs *= mscale;
    sn *= mscale;
    const float a = u * cs - v * sn, b = v * cs + u * sn;
    if (hh < H) {
      float* dst = q_lat + (size_t)t * ldq + (size_t)hh * qhs + R;
      dst[lo] = a;
      dst[hi] = b;
    } else if (slot >= 0) {
      pool[slot + R + lo] = from_f<T>(a);
      pool[slot + R + hi] = from_f<T>(b);
    }
  }
  if (slot < 0) return;
  float s = 0.f;
  for (int e = threadIdx.x; e < R; e += blockDim.x) { const float v = to_f(row[c_off + e]); s = fmaf(v, v, s); }
  const float rinv = 1.f / sqrtf(block_sum(s, red) / (float)R + eps);
  for (int e = threadIdx.x; e < R; e += blockDim.x) pool[slot + e] = from_f<T>(to_f(row[c_off + e]) * rinv * w[e]);
  for (int e = R + dr + threadIdx.x; e < Dh; e += blockDim.x) pool[slot + e] = from_f<T>(0.f);
}

MLXB_EXPORT int mlxb_latent_prepare(int dtype, const void* proj, int ld, int q_off, int c_off, int H, int d, int dr, int R,
                                    const float* w, float eps, const float* freq, int interleaved, const int* positions,
                                    const int* token_req, const int* block_table, int max_pages, int n_pages, int page,
                                    int Dh, void* pool, int write, float* q_lat, int ldq, int qhs, int n_tokens,
                                    int* status, float mscale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || d < 0 || dr < 0 || dr % 2 || R <= 0 || Dh < R + dr || qhs < R + dr || page <= 0 || (dr > 0 && !freq))
    return mlxb_fail(MLXB_BAD_ARG, "latent_prepare: %d heads of %d + %d, %d latent columns in rows of %d", H, d, dr, R, Dh);
  const int threads = R >= 512 ? 256 : 128;
  if (dtype == MLXB_F32)
    launch_pdl(latent_prepare_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)proj, ld, q_off,
               c_off, H, d, dr, R, w, eps, freq, interleaved, positions, token_req, block_table, max_pages, n_pages, page,
               Dh, (float*)pool, write, q_lat, ldq, qhs, status, mscale);
  else if (dtype == MLXB_BF16)
    launch_pdl(latent_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream,
               (const __nv_bfloat16*)proj, ld, q_off, c_off, H, d, dr, R, w, eps, freq, interleaved, positions, token_req,
               block_table, max_pages, n_pages, page, Dh, (__nv_bfloat16*)pool, write, q_lat, ldq, qhs, status, mscale);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "latent_prepare: dtype code %d", dtype);
  return mlxb_check_launch("latent_prepare");
}

// ---------------------------------------------------------------- a product per head

constexpr int HL_TM = 64, HL_TN = 64, HL_TK = 16;

// Tile of 64 tokens x 64 outputs of one head, 256 threads with 4 x 4 results each; x and w go through shared
// memory 16 columns of k at a time.  Every result adds its k in ascending order.
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_linear_kernel(const TX* x, int ldx, int xhs, const TW* __restrict__ w, TO* __restrict__ out, int ldo, int ohs,
                   int M, int N, int K, const int* __restrict__ token_req) {
  __shared__ float sx[HL_TK][HL_TM + 4];
  __shared__ float sw[HL_TK][HL_TN + 4];
  const int h = blockIdx.z, m0 = blockIdx.y * HL_TM, n0 = blockIdx.x * HL_TN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  const TX* xh = x + (size_t)h * xhs;
  const TW* wh = w + (size_t)h * N * K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HL_TK) {
    __syncthreads();
    for (int e = tid; e < HL_TM * HL_TK; e += 256) {
      const int mm = e / HL_TK, kk = e - mm * HL_TK;
      const int m = m0 + mm, k = k0 + kk;
      sx[kk][mm] = (m < M && k < K) ? to_f(xh[(size_t)m * ldx + k]) : 0.f;
    }
    for (int e = tid; e < HL_TN * HL_TK; e += 256) {
      const int nn = e / HL_TK, kk = e - nn * HL_TK;
      const int n = n0 + nn, k = k0 + kk;
      sw[kk][nn] = (n < N && k < K) ? to_f(wh[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HL_TK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&sx[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&sw[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M || (token_req && token_req[m] < 0)) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * ldo + (size_t)h * ohs + n] = from_f<TO>(acc[i][j]);
    }
  }
}

// The same on tensor cores (mma.sync, bfloat16 weights) for steps of many rows: a tile of 64 tokens x 64 outputs of one
// head a CTA, four warps with 16 tokens each, k in pieces of 64 through shared memory.  A float32 x is used as two
// bfloat16 halves (hi + lo, two products per tile), so nothing of it is lost; sums are float32.
__device__ __forceinline__ unsigned hl_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void hl_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void hl_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int HT_KC = 64, HT_LD = HT_KC + 8;

template <typename TX, typename TO, bool VEC>
__global__ void __launch_bounds__(128)
head_linear_tc_kernel(const TX* x, int ldx, int xhs, const __nv_bfloat16* __restrict__ w, TO* __restrict__ out, int ldo,
                      int ohs, int M, int N, int K, const int* __restrict__ token_req) {
  constexpr bool SPLIT = sizeof(TX) == 4;
  __shared__ __align__(16) __nv_bfloat16 sxh[64 * HT_LD];
  __shared__ __align__(16) __nv_bfloat16 sxl[SPLIT ? 64 * HT_LD : 8];
  __shared__ __align__(16) __nv_bfloat16 sw[64 * HT_LD];
  const int h = blockIdx.z, m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  const TX* xh = x + (size_t)h * xhs;
  const __nv_bfloat16* wh = w + (size_t)h * N * K;
  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HT_KC) {
    __syncthreads();
    if (VEC) {
      // eight k of a row a thread, 16 bytes a load (two for a float32 x); K is a multiple of 8: a piece is all in or out
      for (int e = tid; e < 64 * (HT_KC / 8); e += 128) {
        const int rr = e / (HT_KC / 8), kk = (e - rr * (HT_KC / 8)) * 8;
        const int m = m0 + rr, n = n0 + rr, k = k0 + kk;
        uint4 wv = make_uint4(0u, 0u, 0u, 0u);
        if (n < N && k < K) wv = *reinterpret_cast<const uint4*>(wh + (size_t)n * K + k);
        *reinterpret_cast<uint4*>(sw + rr * HT_LD + kk) = wv;
        if (SPLIT) {
          float xv[8], hi[8], lo[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) xv[i] = 0.f;
          if (m < M && k < K) {
            const float* xp = reinterpret_cast<const float*>(xh) + (size_t)m * ldx + k;
            *reinterpret_cast<float4*>(xv) = *reinterpret_cast<const float4*>(xp);
            *reinterpret_cast<float4*>(xv + 4) = *reinterpret_cast<const float4*>(xp + 4);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            hi[i] = __bfloat162float(__float2bfloat16_rn(xv[i]));
            lo[i] = xv[i] - hi[i];
          }
          *reinterpret_cast<uint4*>(sxh + rr * HT_LD + kk) = pack8(hi);
          *reinterpret_cast<uint4*>(sxl + rr * HT_LD + kk) = pack8(lo);
        } else {
          uint4 xv = make_uint4(0u, 0u, 0u, 0u);
          if (m < M && k < K) xv = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(xh) + (size_t)m * ldx + k);
          *reinterpret_cast<uint4*>(sxh + rr * HT_LD + kk) = xv;
        }
      }
    } else
    for (int e = tid; e < 64 * HT_KC; e += 128) {
      const int rr = e / HT_KC, kk = e - rr * HT_KC;
      const int m = m0 + rr, n = n0 + rr, k = k0 + kk;
      const float xv = (m < M && k < K) ? to_f(xh[(size_t)m * ldx + k]) : 0.f;
      const __nv_bfloat16 hi = __float2bfloat16_rn(xv);
      sxh[rr * HT_LD + kk] = hi;
      if (SPLIT) sxl[rr * HT_LD + kk] = __float2bfloat16_rn(xv - __bfloat162float(hi));
      sw[rr * HT_LD + kk] = (n < N && k < K) ? wh[(size_t)n * K + k] : __float2bfloat16_rn(0.f);
    }
    __syncthreads();
    const unsigned ah = hl_smem(sxh + (warp * 16 + (lane & 15)) * HT_LD + (lane >> 4) * 8);
    const unsigned al = hl_smem(sxl + (SPLIT ? (warp * 16 + (lane & 15)) * HT_LD + (lane >> 4) * 8 : 0));
    // weights: a group of four 8 x 8 pieces is two output tiles by two halves of a k step
    const unsigned wb = hl_smem(sw + ((lane & 7) + ((lane >> 4) & 1) * 8) * HT_LD + ((lane >> 3) & 1) * 8);
#pragma unroll
    for (int ks = 0; ks < HT_KC; ks += 16) {
      unsigned a[4], a2[4];
      hl_ldmatrix_x4(a, ah + ks * 2);
      if (SPLIT) hl_ldmatrix_x4(a2, al + ks * 2);
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        unsigned b[4];
        hl_ldmatrix_x4(b, wb + (jp * 16 * HT_LD + ks) * 2);
        hl_mma(acc[2 * jp], a, b[0], b[1]);
        hl_mma(acc[2 * jp + 1], a, b[2], b[3]);
        if (SPLIT) {
          hl_mma(acc[2 * jp], a2, b[0], b[1]);
          hl_mma(acc[2 * jp + 1], a2, b[2], b[3]);
        }
      }
    }
  }
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = m0 + warp * 16 + g + half * 8;
    if (m >= M || (token_req && token_req[m] < 0)) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + j * 8 + t4 * 2;
      TO* op = out + (size_t)m * ldo + (size_t)h * ohs + n;
      if (n < N) op[0] = from_f<TO>(acc[j][half * 2]);
      if (n + 1 < N) op[1] = from_f<TO>(acc[j][half * 2 + 1]);
    }
  }
}

// The same for steps of few rows (single-token entries): a warp per output column and eight rows, the lanes side by
// side along k (the weights are read once, in whole lines), partial sums added across the warp.
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_linear_rows_kernel(const TX* x, int ldx, int xhs, const TW* __restrict__ w, TO* __restrict__ out, int ldo, int ohs,
                        int M, int N, int K, const int* __restrict__ token_req) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp, h = blockIdx.y, m0 = blockIdx.z * 8;
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  if (n >= N) return;
  const TW* wr = w + ((size_t)h * N + n) * K;
  const TX* xh = x + (size_t)h * xhs;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float wv = to_f(wr[k]);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (m0 + i < M) acc[i] = fmaf(to_f(xh[(size_t)(m0 + i) * ldx + k]), wv, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float v = warp_sum(acc[i]);
    const int m = m0 + i;
    if (lane == 0 && m < M && !(token_req && token_req[m] < 0)) out[(size_t)m * ldo + (size_t)h * ohs + n] = from_f<TO>(v);
  }
}

// x: [M, .] at row stride ldx, head h from column h*xhs (K values), float32 if x_f32 else `dtype`; w: `dtype`
// [H, N, K]; out: [M, .] at row stride ldo, head h from column h*ohs (N values), float32 if out_f32 else `dtype`;
// token_req: int32 [M] or null: rows whose entry is negative are not written.
MLXB_EXPORT int mlxb_head_linear(int dtype, int x_f32, int out_f32, const void* x, int ldx, int xhs, const void* w,
                                 void* out, int ldo, int ohs, int M, int N, int K, int H, const int* token_req,
                                 cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N <= 0 || K <= 0 || H <= 0 || xhs < K || ohs < N || H > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "head_linear: %d heads of %d x %d, head strides %d / %d", H, N, K, xhs, ohs);
  // (float32 runs keep the tiled kernel whatever the step's size: a row's sum is then the same bits in every step)
  const bool few = M <= 16 && dtype != MLXB_F32;
  const dim3 grid((N + HL_TN - 1) / HL_TN, (M + HL_TM - 1) / HL_TM, H), rgrid((N + 7) / 8, H, (M + 7) / 8), block(256);
  const bool tc = dtype == MLXB_BF16 && M > 16 && getenv("MLXB_HEAD_LINEAR_SIMT") == nullptr;
  if (tc) {
    const dim3 tgrid((N + 63) / 64, (M + 63) / 64, H), tblock(128);
    const int xa = x_f32 ? 4 : 8;          // elements of x in 16 bytes
    const bool vec = K % 8 == 0 && ldx % xa == 0 && xhs % xa == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0;
#define HT_GO(TX, TO)                                                                                                 \
  if (vec)                                                                                                            \
    launch_pdl(head_linear_tc_kernel<TX, TO, true>, tgrid, tblock, 0, stream, (const TX*)x, ldx, xhs,                 \
               (const __nv_bfloat16*)w, (TO*)out, ldo, ohs, M, N, K, token_req);                                      \
  else                                                                                                                \
    launch_pdl(head_linear_tc_kernel<TX, TO, false>, tgrid, tblock, 0, stream, (const TX*)x, ldx, xhs,                \
               (const __nv_bfloat16*)w, (TO*)out, ldo, ohs, M, N, K, token_req)
    if (x_f32 && out_f32) { HT_GO(float, float); }
    else if (x_f32) { HT_GO(float, __nv_bfloat16); }
    else if (out_f32) { HT_GO(__nv_bfloat16, float); }
    else { HT_GO(__nv_bfloat16, __nv_bfloat16); }
#undef HT_GO
    return mlxb_check_launch("head_linear");
  }
#define HL_GO(TX, TW, TO)                                                                                             \
  if (few)                                                                                                            \
    launch_pdl(head_linear_rows_kernel<TX, TW, TO>, rgrid, block, 0, stream, (const TX*)x, ldx, xhs, (const TW*)w,   \
               (TO*)out, ldo, ohs, M, N, K, token_req);                                                               \
  else                                                                                                                \
    launch_pdl(head_linear_kernel<TX, TW, TO>, grid, block, 0, stream, (const TX*)x, ldx, xhs, (const TW*)w, (TO*)out, \
               ldo, ohs, M, N, K, token_req)
  if (dtype == MLXB_F32) { HL_GO(float, float, float); }
  else if (dtype != MLXB_BF16) return mlxb_fail(MLXB_BAD_DTYPE, "head_linear: dtype code %d", dtype);
  else if (x_f32 && out_f32) { HL_GO(float, __nv_bfloat16, float); }
  else if (x_f32) { HL_GO(float, __nv_bfloat16, __nv_bfloat16); }
  else if (out_f32) { HL_GO(__nv_bfloat16, __nv_bfloat16, float); }
  else { HL_GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); }
#undef HL_GO
  return mlxb_check_launch("head_linear");
}
