// The attention of attention_wide.cu on tensor cores (mma.sync, bfloat16 pages, float32 accumulation).
//
// A CTA takes 32 rows (64 for portions where the shared memory allows it: two halves that share the key tiles): TQ consecutive tokens of one request times HG neighbouring heads that share a value head
// (TQ * HG = 32; a single-token entry: one token, HG heads, the other rows empty), and walks the keys in blocks of
// 64 positions that start at multiples of 64, so the order of additions for a row depends on its position only.
//
// Queries arrive in float32 and are used as two bfloat16 halves (hi + lo, two products per tile): nothing is
// lost of them.  Scores mixed across heads (talk [H, H]) are computed as products of MIXED QUERIES: with
// s'_h = sum_g talk[h, g] scale q_g . k_kv(g), grouping the heads g by their key head c gives
// s'_h = scale sum_c (sum_{g in c} talk[h, g] q_g) . k_c, an ordinary score of a query of G*dk dimensions against the
// token's G key heads laid side by side; the mixed query is made in float32 when the CTA loads its queries.
//
// Per block of keys: the K tile (and the V tile, unless the values are the first Dv columns of the key rows) comes
// into shared memory by 16-byte cp.async through the block table, the next block's while this block is computed
// where two buffers fit; warp w takes the scores of keys 8w .. 8w+7 for
// all 32 rows (S = Q K^T), masked and scaled into shared memory in float32; eight threads a row keep the running
// maximum and sum and write the weights as bfloat16; warp w then takes every eighth 8-column tile of the values
// (O = O * corr + P V) in registers.  Masks: causal, a window, runs of `chunk` positions counted from 0; beside a
// window the first `keep_first` positions stay visible (their blocks, counted from position 0, are walked before the
// window's).  Scores may be bounded by a soft cap (cap * tanh(s / cap)) before the softmax.  The gate is one number
// per head or, with `gate_cols`, one per output column.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int TC_M = 32, TC_N = 64, TC_THREADS = 256, TC_WARPS = 8;
constexpr int TC_NT = 8;      // 8-column value tiles a warp accumulates: Dv <= 8 * 8 * TC_NT = 512
constexpr int TC_SPAD = 4, TC_PPAD = 8;

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

// tiles: int32 [n_tiles, 4] = (first token row, queries, block-table row, first position); a CTA takes tokens
// sub*TQ .. of tile blockIdx.x / subs.  DkE: columns of a (mixed) query and of a key tile row, a multiple of 16;
// seg: columns one key head gives (talk: dk, G segments side by side; else the key's columns rounded up to 8, one
// segment).  shared_v: values are columns 0 .. Dv-1 of the key tile.  MP: the CTA takes 32 * MP rows with 8 * MP warps
// (two halves that share the key tiles).  nbuf = 2: the next block's tiles are fetched while this block is computed.
template <typename TO, int MP>
__global__ void __launch_bounds__(TC_THREADS * MP, MP == 1 ? 2 : 1)
attention_wide_tc_kernel(const float* q, int ldq, int qhs, const int* __restrict__ tiles, int subs, int TQ, int HG,
                         const int* __restrict__ block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                         int Dk, int Dv, int DkE, int seg, int n_seg, int krs, int vrs, int shared_v, int window,
                         int chunk, float scale, const float* __restrict__ talk, const __nv_bfloat16* k_pool,
                         const __nv_bfloat16* v_pool, const __nv_bfloat16* gate, int ldg, TO* __restrict__ out, int ldo,
                         int ohs, int* __restrict__ status, int bps, int n_rel, float* __restrict__ scratch, int nbuf,
                         float softcap, int keep_first, int gate_cols, int Hv) {
  constexpr int M = TC_M * MP, THREADS = TC_THREADS * MP;
  extern __shared__ __align__(16) unsigned char tc_smem[];
  const int ldk = DkE + 8, ldv = shared_v ? ldk : Dv + 8;
  float* sS = reinterpret_cast<float*>(tc_smem);                            // [M][TC_N + TC_SPAD]
  float* sCorr = sS + M * (TC_N + TC_SPAD);                                 // [M]
  float* sL = sCorr + M;                                                    // [M]
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sL + M);             // [M][TC_N + TC_PPAD]
  __nv_bfloat16* sQh = sP + M * (TC_N + TC_PPAD);                           // [M][ldk]
  __nv_bfloat16* sQl = sQh + M * ldk;                                       // [M][ldk]
  __nv_bfloat16* sK0 = sQl + M * ldk;                                       // [nbuf][TC_N][ldk]
  __nv_bfloat16* sV0 = shared_v ? sK0 : sK0 + nbuf * TC_N * ldk;            // [nbuf][TC_N][ldv]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mp = warp / TC_WARPS, w8 = warp % TC_WARPS;                     // which half of the rows, which warp of it
  const int tile = blockIdx.x / subs, sub = blockIdx.x - tile * subs;
  const int t_first = tiles[4 * tile], n_tile = tiles[4 * tile + 1], bt_row = tiles[4 * tile + 2];
  const int nq = min(TQ, n_tile - sub * TQ);
  if (nq <= 0) return;
  const int t0 = t_first + sub * TQ, pos0 = tiles[4 * tile + 3] + sub * TQ;
  const int h0 = blockIdx.y * HG, rep = Hq / Hkv, cv = h0 / rep;
  const int* bt = block_table + (size_t)bt_row * max_pages;
  int lo_min = 0;                                            // first visible key of the first token: the smallest of the CTA
  if (window > 0 && pos0 - window + 1 > lo_min) lo_min = pos0 - window + 1;
  if (chunk > 0 && (pos0 / chunk) * chunk > lo_min) lo_min = (pos0 / chunk) * chunk;
  int p_max = pos0 + nq - 1;
  int j_first = (lo_min / TC_N) * TC_N;
  // kept first positions: the blocks 0 .. that lie wholly before the window's first block are walked first
  int kept_end = min((min(keep_first, lo_min) + TC_N - 1) / TC_N * TC_N, j_first);      // a multiple of TC_N
  int j_start = kept_end > 0 ? 0 : j_first;
  if (bps > 0) {
    // single rows with their keys split over the CTAs of grid.z: first the splits of the kept blocks (bps blocks
    // each, counted from position 0), then those of the window: split z takes the blocks bps*za .. bps*za + bps - 1,
    // counted from position 0; each leaves an unnormalised partial result for the merge kernel
    const int kz = (kept_end / TC_N + bps - 1) / bps;
    if ((int)blockIdx.z < kz) {
      j_start = blockIdx.z * bps * TC_N;
      p_max = min(kept_end, j_start + bps * TC_N) - 1;
      kept_end = p_max + 1;
      j_first = kept_end;                                    // nothing of the window
    } else {
      const int za = (lo_min / TC_N) / bps + (blockIdx.z - kz);
      if (za * bps * TC_N > p_max) return;                   // a split without keys
      j_first = max(j_first, za * bps * TC_N);
      p_max = min(p_max, (za + 1) * bps * TC_N - 1);
      kept_end = 0;
      j_start = j_first;
    }
  }
  // the block after the one that starts at j0
  auto next_block = [&](int j0) { const int n = j0 + TC_N; return (n >= kept_end && n < j_first) ? j_first : n; };
  pdl_wait();
  pdl_trigger();
  q = after_wait(q);
  k_pool = after_wait(k_pool);
  v_pool = after_wait(v_pool);
  gate = after_wait(gate);

  // The tiles of the block of keys that starts at j0, into buffer `buf`: 16-byte pieces through the block table;
  // zeros where a key lies outside lo_min .. p_max, where a column pads the tile, or where a page is missing.
  auto load_tiles = [&](int j0, int buf) {
    __nv_bfloat16* dK = sK0 + buf * TC_N * ldk;
    const int per_key = DkE / 8;
    for (int e = tid; e < TC_N * per_key; e += THREADS) {
      const int jj = e / per_key, col = (e - jj * per_key) * 8, j = j0 + jj;
      const int c = col / seg, d = col - c * seg;
      const __nv_bfloat16* src = nullptr;
      if ((j >= lo_min || j < keep_first) && j <= p_max && c < n_seg) {
        const int lp = j / page;
        const int pg = lp < max_pages ? bt[lp] : -1;
        if (pg >= n_pages) atomicOr(status, MLXB_ST_PAGE_RANGE);
        else if (pg < 0) atomicOr(status, MLXB_ST_POSITION_RANGE);     // a key inside the range has no page
        else src = k_pool + (((size_t)pg * Hkv + (talk ? c : cv)) * page + (j % page)) * krs + d;
      }
      if (src) cp_async16(dK + jj * ldk + col, src);
      else *reinterpret_cast<uint4*>(dK + jj * ldk + col) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (!shared_v) {
      __nv_bfloat16* dV = sV0 + buf * TC_N * ldv;
      const int per_v = Dv / 8;
      for (int e = tid; e < TC_N * per_v; e += THREADS) {
        const int jj = e / per_v, col = (e - jj * per_v) * 8, j = j0 + jj;
        const __nv_bfloat16* src = nullptr;
        if ((j >= lo_min || j < keep_first) && j <= p_max) {
          const int lp = j / page;
          const int pg = lp < max_pages ? bt[lp] : -1;
          if (pg >= 0 && pg < n_pages) src = v_pool + (((size_t)pg * Hv + cv / (Hkv / Hv)) * page + (j % page)) * vrs + col;
        }
        if (src) cp_async16(dV + jj * ldv + col, src);
        else *reinterpret_cast<uint4*>(dV + jj * ldv + col) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_tiles(j_start, 0);

  // ---- queries: float32 -> hi + lo; with talk, the heads' queries mixed into the key heads' segments
  const int rows_used = nq * HG;                             // rows 0 .. rows_used - 1 carry a (token, head)
  for (int e = tid; e < rows_used * DkE; e += THREADS) {
    const int r = e / DkE, col = e - r * DkE;
    const int tq = r / HG, h = h0 + r % HG;
    float v = 0.f;
    const float* qt = q + (size_t)(t0 + tq) * ldq;
    if (talk) {
      const int c = col / seg, d = col - c * seg;
      if (c < n_seg)
        for (int i = 0; i < rep; ++i) v = fmaf(talk[h * Hq + c * rep + i], qt[(size_t)(c * rep + i) * qhs + d], v);
    } else if (col < Dk) {
      v = qt[(size_t)h * qhs + col];
    }
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    sQh[r * ldk + col] = hi;
    sQl[r * ldk + col] = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
  for (int e = rows_used * (ldk / 8) + tid; e < M * (ldk / 8); e += THREADS) {      // the empty rows: zeros
    reinterpret_cast<uint4*>(sQh)[e] = make_uint4(0u, 0u, 0u, 0u);
    reinterpret_cast<uint4*>(sQl)[e] = make_uint4(0u, 0u, 0u, 0u);
  }
  // the rows' visible ranges
  const int my_row = tid >> 3, my_sub = tid & 7;             // softmax: eight threads a row
  const int my_tq = my_row / HG;
  const int my_p = my_tq < nq ? min(pos0 + my_tq, p_max) : -1;
  int my_lo = 0;
  {
    const int p_own = pos0 + my_tq;
    if (window > 0 && p_own - window + 1 > my_lo) my_lo = p_own - window + 1;
    if (chunk > 0 && (p_own / chunk) * chunk > my_lo) my_lo = (p_own / chunk) * chunk;
  }
  float m_run = -INFINITY, l_run = 0.f;
  float o[TC_NT][2][4];
#pragma unroll
  for (int i = 0; i < TC_NT; ++i)
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int x = 0; x < 4; ++x) o[i][m][x] = 0.f;
  const int n_vt = Dv / 8;                                   // 8-column tiles of the values
  const int g = lane >> 2, tq4 = lane & 3;
  const int row0 = mp * TC_M;                                // this warp's rows: row0 .. row0 + 31

  int buf = 0;
  for (int j0 = j_start; j0 <= p_max; j0 = next_block(j0)) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                         // this block's tiles have landed; the block before is done with
    const int j_next = next_block(j0);
    const bool more = j_next <= p_max;
    if (nbuf == 2 && more) load_tiles(j_next, buf ^ 1);
    const __nv_bfloat16* sK = sK0 + buf * TC_N * ldk;
    const __nv_bfloat16* sV = sV0 + buf * TC_N * ldv;
    // ---- S = Q K^T for keys 8 w8 .. 8 w8 + 7 and this half's rows
    {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const unsigned kb = smem_addr(sK + (w8 * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8);
      const unsigned qh = smem_addr(sQh + (row0 + (lane & 15)) * ldk + (lane >> 4) * 8);
      const unsigned ql = smem_addr(sQl + (row0 + (lane & 15)) * ldk + (lane >> 4) * 8);
      for (int k0 = 0; k0 < DkE; k0 += 16) {
        // the five fragment loads of a step go out together, then its four products
        unsigned b[2], ah[2][4], al[2][4];
        ldmatrix_x2(b, kb + k0 * 2);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          ldmatrix_x4(ah[m], qh + (m * 16 * ldk + k0) * 2);
          ldmatrix_x4(al[m], ql + (m * 16 * ldk + k0) * 2);
        }
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          mma_bf16(s[m], ah[m], b);
          mma_bf16(s[m], al[m], b);
        }
      }
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int r = row0 + m * 16 + g + (x >> 1) * 8, jj = w8 * 8 + tq4 * 2 + (x & 1);
          float sc = s[m][x] * scale;
          if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
          sS[r * (TC_N + TC_SPAD) + jj] = sc;
        }
    }
    __syncthreads();
    // ---- weights: eight threads a row, eight keys each
    {
      float sv[8];
      float mb = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int jj = my_sub * 8 + i, j = j0 + jj;
        sv[i] = (j <= my_p && (j >= my_lo || j < keep_first)) ? sS[my_row * (TC_N + TC_SPAD) + jj] : -INFINITY;
        mb = fmaxf(mb, sv[i]);
      }
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
      const float m_new = fmaxf(m_run, mb);
      const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
      float sum = 0.f;
      __nv_bfloat16* pr = sP + my_row * (TC_N + TC_PPAD) + my_sub * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float pw = sv[i] == -INFINITY ? 0.f : expf(sv[i] - m_new);
        const __nv_bfloat16 pb = __float2bfloat16_rn(pw);
        pr[i] = pb;
        sum += __bfloat162float(pb);                         // the sum of what the values are weighted with
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      l_run = l_run * corr + sum;
      m_run = m_new;
      if (my_sub == 0) sCorr[my_row] = corr;
    }
    __syncthreads();
    // ---- O = O corr + P V for this warp's value tiles
    {
      float cr[2][2];
#pragma unroll
      for (int m = 0; m < 2; ++m) { cr[m][0] = sCorr[row0 + m * 16 + g]; cr[m][1] = sCorr[row0 + m * 16 + g + 8]; }
      unsigned a[2][4][4];                                   // P: two row tiles x four key steps
      const unsigned pb = smem_addr(sP + (row0 + (lane & 15)) * (TC_N + TC_PPAD) + (lane >> 4) * 8);
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) ldmatrix_x4(a[m][ks], pb + (m * 16 * (TC_N + TC_PPAD) + ks * 16) * 2);
#pragma unroll
      for (int i = 0; i < TC_NT; ++i) {
        const int nt = w8 + i * TC_WARPS;
        if (nt < n_vt) {
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            o[i][m][0] *= cr[m][0]; o[i][m][1] *= cr[m][0];
            o[i][m][2] *= cr[m][1]; o[i][m][3] *= cr[m][1];
          }
          const unsigned vb = smem_addr(sV + (lane & 15) * ldv + nt * 8);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            unsigned b[2];
            ldmatrix_x2_trans(b, vb + ks * 16 * ldv * 2);
            mma_bf16(o[i][0], a[0][ks], b);
            mma_bf16(o[i][1], a[1][ks], b);
          }
        }
      }
    }
    if (nbuf == 2) {
      buf ^= 1;
    } else if (more) {
      __syncthreads();                                       // one buffer: everybody is done with it before it is refilled
      load_tiles(j_next, 0);
    }
  }
  if (my_sub == 0) sL[my_row] = l_run;
  __syncthreads();
  if (bps > 0) {
    // partial results (one token: row r is head h0 + r): [tile, head, split][Dv values | maximum | sum]
    const size_t stride = (size_t)Dv + 2;
    if (my_sub == 0 && my_row < HG) {
      float* sp = scratch + (((size_t)tile * Hq + h0 + my_row) * n_rel + blockIdx.z) * stride;
      sp[Dv] = m_run;
      sp[Dv + 1] = l_run;
    }
#pragma unroll
    for (int i = 0; i < TC_NT; ++i) {
      const int nt = w8 + i * TC_WARPS;
      if (nt >= n_vt) continue;
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = row0 + m * 16 + g + half * 8;
          if (r >= HG) continue;
          float* sp = scratch + (((size_t)tile * Hq + h0 + r) * n_rel + blockIdx.z) * stride + nt * 8 + tq4 * 2;
          sp[0] = o[i][m][half * 2];
          sp[1] = o[i][m][half * 2 + 1];
        }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < TC_NT; ++i) {
    const int nt = w8 + i * TC_WARPS;
    if (nt >= n_vt) continue;
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = row0 + m * 16 + g + half * 8;
        const int tq = r / HG, h = h0 + r % HG;
        if (tq >= nq) continue;
        const float l = sL[r];
        const float f = l > 0.f ? 1.f / l : 0.f;
        const int t = t0 + tq, col = nt * 8 + tq4 * 2;
        float g0 = 1.f, g1 = 1.f;
        if (gate) {
          const __nv_bfloat16* gp = gate + (size_t)t * ldg + (gate_cols ? (size_t)h * Dv + col : (size_t)h);
          g0 = 1.f / (1.f + expf(-__bfloat162float(gp[0])));
          g1 = gate_cols ? 1.f / (1.f + expf(-__bfloat162float(gp[1]))) : g0;
        }
        TO* op = out + (size_t)t * ldo + (size_t)h * ohs + col;
        op[0] = from_f<TO>(o[i][m][half * 2] * f * g0);
        op[1] = from_f<TO>(o[i][m][half * 2 + 1] * f * g1);
      }
  }
}

// The partial results of a single row's splits, merged in the order of the splits: one block per (tile, head).
template <typename TO>
__global__ void attention_wide_merge_kernel(const int* __restrict__ tiles, int Hq, int Dv, int window, int chunk, int bps,
                                            int n_rel, const float* scratch, const __nv_bfloat16* gate, int ldg,
                                            TO* __restrict__ out, int ldo, int ohs, int keep_first, int gate_cols) {
  const int tile = blockIdx.x, h = blockIdx.y;
  if (tiles[4 * tile + 1] <= 0) return;
  const int t = tiles[4 * tile], p = tiles[4 * tile + 3];
  int lo = 0;
  if (window > 0 && p - window + 1 > lo) lo = p - window + 1;
  if (chunk > 0 && (p / chunk) * chunk > lo) lo = (p / chunk) * chunk;
  const int kept_end = min((min(keep_first, lo) + TC_N - 1) / TC_N * TC_N, (lo / TC_N) * TC_N);
  const int nz = (kept_end / TC_N + bps - 1) / bps + (p / TC_N) / bps - (lo / TC_N) / bps + 1;
  pdl_wait();
  pdl_trigger();
  scratch = after_wait(scratch);
  gate = after_wait(gate);
  const size_t stride = (size_t)Dv + 2;
  const float* sp = scratch + ((size_t)tile * Hq + h) * n_rel * stride;
  float M = -INFINITY;
  for (int z = 0; z < nz; ++z) M = fmaxf(M, sp[z * stride + Dv]);
  float L = 0.f;
  for (int z = 0; z < nz; ++z) {
    const float mz = sp[z * stride + Dv];
    if (mz != -INFINITY) L = fmaf(expf(mz - M), sp[z * stride + Dv + 1], L);
  }
  const float f = L > 0.f ? 1.f / L : 0.f;
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < nz; ++z) {
      const float mz = sp[z * stride + Dv];
      if (mz != -INFINITY) a = fmaf(expf(mz - M), sp[z * stride + c], a);
    }
    float gt = 1.f;
    if (gate) gt = 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)t * ldg + (gate_cols ? (size_t)h * Dv + c : (size_t)h)])));
    out[(size_t)t * ldo + (size_t)h * ohs + c] = from_f<TO>(a * f * gt);
  }
}

constexpr int TC_BPS = 1;     // key blocks a CTA of a split single row takes: a constant, never a function of the batch

// Blocks of keys a single row can touch: the positions it can see, in blocks, and one more for a ragged start.
static int tc_blocks(int window, int chunk, int max_len, int keep_first = 0) {
  int span = max_len > 0 ? max_len : 1;
  if (window > 0 && window < span) span = window;
  if (chunk > 0 && chunk < span) span = chunk;
  int kept = 0;
  if (keep_first > 0 && window > 0) kept = (keep_first + TC_N - 1) / TC_N;
  return (span + TC_N - 1) / TC_N + 1 + kept;
}
// Rows that see at most three blocks are not split; the others have room for this many partial results.
static bool tc_splits_rows(int window, int chunk, int max_len, int keep_first = 0) {
  return tc_blocks(window, chunk, max_len, keep_first) > 3;
}
static int tc_splits(int window, int chunk, int max_len, int keep_first = 0) {
  return (tc_blocks(window, chunk, max_len, keep_first) + TC_BPS - 1) / TC_BPS + 1;
}

// Floats of scratch memory that single rows need (0: rows that see few keys are not split).
MLXB_EXPORT long long mlxb_attention_wide_tc_scratch(int n_rows, int Hq, int Dv, int window, int chunk, int max_len,
                                                     int keep_first) {
  if (!tc_splits_rows(window, chunk, max_len, keep_first)) return 0;
  return (long long)n_rows * Hq * tc_splits(window, chunk, max_len, keep_first) * (Dv + 2);
}

// How a launch is laid out, or false if the sizes are not served (the caller then takes the kernel on the CUDA
// cores): key and value widths in whole 16-byte pieces, at most 512 value columns, heads that group.  Portions take
// 64 rows a CTA and two buffers for the key tiles where the shared memory allows it, else 32 rows, else one buffer.
struct TcPlan { int DkE, seg, n_seg, HG, MP, nbuf; long long smem; };
static bool tc_plan(int Hq, int Hkv, int Dk, int Dv, int krs, int vrs, int talk, int shared_v, bool portions, TcPlan* p) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Dv % 8 || Dv > 64 * TC_NT || krs % 8 || vrs % 8) return false;
  const int rep = Hq / Hkv;
  if (talk) {
    if (Dk % 8) return false;
    p->seg = Dk;
    p->n_seg = Hkv;
  } else {
    p->seg = (Dk + 7) / 8 * 8;          // the pool's rows are zero beyond Dk
    if (p->seg > krs) return false;
    p->n_seg = 1;
  }
  p->DkE = (p->seg * p->n_seg + 15) / 16 * 16;
  if (shared_v && Dv > p->DkE) return false;
  int hg = 1;
  while (hg * 2 <= TC_M && rep % (hg * 2) == 0) hg *= 2;
  p->HG = hg;
  const int ldk = p->DkE + 8, ldv = shared_v ? ldk : Dv + 8;
  auto bytes_of = [&](int MP, int nbuf) {
    const int M = TC_M * MP;
    return 4LL * (M * (TC_N + TC_SPAD) + 2 * M) + 2LL * M * (TC_N + TC_PPAD) + 2LL * 2 * M * ldk +
           (long long)nbuf * (2LL * TC_N * ldk + (shared_v ? 0LL : 2LL * TC_N * ldv));
  };
  const long long whole = 220 * 1024, half = 110 * 1024;      // what one CTA, and what each of two CTAs of an SM, may take
  // portions: 64 rows and two buffers; single rows: two CTAs an SM come before the second buffer
  const int tries[5][3] = {{2, 2, 0}, {1, 2, 1}, {1, 1, 1}, {1, 2, 0}, {1, 1, 0}};
  for (int i = portions ? 0 : 1; i < 5; ++i) {
    const long long bytes = bytes_of(tries[i][0], tries[i][1]);
    if (bytes <= (tries[i][2] ? half : whole)) {
      p->MP = tries[i][0];
      p->nbuf = tries[i][1];
      p->smem = bytes;
      return true;
    }
  }
  return false;
}

MLXB_EXPORT int mlxb_attention_wide_tc_supported(int Hq, int Hkv, int Dk, int Dv, int krs, int vrs, int talk, int shared_v) {
  TcPlan p;
  return tc_plan(Hq, Hkv, Dk, Dv, krs, vrs, talk, shared_v, false, &p) ? 1 : 0;
}

// The arguments of mlxb_attention_wide with bfloat16 pools, and instead of the token rows a list of tiles: int32
// [n_tiles, 4] = (first token row, queries, block-table row, first position), each of at most tile_q queries.  Hv: heads
// of v_pool (0: Hkv); with fewer, key heads c * Hkv/Hv .. read value head c.
MLXB_EXPORT int mlxb_attention_wide_tc(int out_f32, const float* q, int ldq, int qhs, const int* tiles, int n_tiles,
                                       int tile_q, const int* block_table, int max_pages, int n_pages, int page, int Hq,
                                       int Hkv, int Dk, int Dv, int krs, int vrs, int window, int chunk, float scale,
                                       const float* talk, const void* k_pool, const void* v_pool, const void* gate,
                                       int ldg, void* out, int ldo, int ohs, int* status, float* scratch, int max_len,
                                       float softcap, int keep_first, int gate_cols, int Hv, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (Hv <= 0) Hv = Hkv;
  if (Hkv % Hv || (Hv != Hkv && v_pool == k_pool))
    return mlxb_fail(MLXB_BAD_ARG, "attention (wide, tensor cores): %d key heads over %d value heads", Hkv, Hv);
  TcPlan pl;
  const int shared_v = v_pool == k_pool;
  if (!tc_plan(Hq, Hkv, Dk, Dv, krs, vrs, talk != nullptr, shared_v, tile_q > 1, &pl) || page <= 0 || (page & (page - 1)) ||
      tile_q <= 0 || qhs < Dk || ohs < Dv)
    return mlxb_fail(MLXB_BAD_ARG, "attention (wide, tensor cores): %d/%d heads, sizes %d/%d in rows of %d/%d", Hq, Hkv,
                     Dk, Dv, krs, vrs);
  // single rows with scratch memory: their keys split over grid.z, then merged
  if (window <= 0) keep_first = 0;           // without a window every earlier position is visible anyway
  const int n_rel = tc_splits(window, chunk, max_len, keep_first);
  // (only while the rows alone leave SMs idle: with more CTAs than SMs a split adds work and nothing else; a row's
  // result is the same up to the rounding of the merge either way)
  const bool split = tile_q == 1 && scratch != nullptr && tc_splits_rows(window, chunk, max_len, keep_first) && (long long)n_tiles * (Hq / pl.HG) < mlxb_sm_count();
  const int TQ = split ? 1 : TC_M * pl.MP / pl.HG;
  const int subs = (tile_q + TQ - 1) / TQ;
  const int bps = split ? TC_BPS : 0;
  const long long smem = pl.smem;
  const dim3 grid((unsigned)n_tiles * subs, Hq / pl.HG, split ? n_rel : 1), block(TC_THREADS * pl.MP);
#define TCW_GO(TO, MPV)                                                                                                \
  do {                                                                                                                 \
    auto kern = attention_wide_tc_kernel<TO, MPV>;                                                                     \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
      if (e != cudaSuccess)                                                                                            \
        return mlxb_fail((int)e, "attention (wide, tensor cores): %lld bytes of shared memory: %s", smem,              \
                         cudaGetErrorString(e));                                                                       \
    }                                                                                                                  \
    launch_pdl(kern, grid, block, (size_t)smem, stream, q, ldq, qhs, tiles, subs, TQ, pl.HG, block_table, max_pages,   \
               n_pages, page, Hq, Hkv, Dk, Dv, pl.DkE, pl.seg, pl.n_seg, krs, vrs, shared_v, window, chunk, scale, talk, \
               (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (const __nv_bfloat16*)gate, ldg, (TO*)out,  \
               ldo, ohs, status, bps, n_rel, scratch, pl.nbuf, softcap, keep_first, gate_cols, Hv);                        \
    if (split) {                                                                                                       \
      if (int e = mlxb_check_launch("attention (wide, tensor cores)")) return e;                                       \
      launch_pdl(attention_wide_merge_kernel<TO>, dim3(n_tiles, Hq), dim3(Dv >= 128 ? 128 : 64), 0, stream, tiles, Hq, \
                 Dv, window, chunk, bps, n_rel, (const float*)scratch, (const __nv_bfloat16*)gate, ldg, (TO*)out, ldo, \
                 ohs, keep_first, gate_cols);                                                                          \
    }                                                                                                                  \
  } while (0)
  if (pl.MP == 2) {
    if (out_f32) TCW_GO(float, 2);
    else TCW_GO(__nv_bfloat16, 2);
  } else {
    if (out_f32) TCW_GO(float, 1);
    else TCW_GO(__nv_bfloat16, 1);
  }
#undef TCW_GO
  return mlxb_check_launch("attention (wide, tensor cores)");
}
