// A feed-forward made of many small experts, of which every token uses a few.
//
// moe_route   one warp per token: scores s = f(router logits) in float32 (f: sigmoid, or a softmax over the experts),
//             the `top` largest (ties: the lower expert), their scores as weights (optionally divided by their sum).
//             sel_expert[t * top + c], sel_weight[t * top + c]; a row that pads the step gets expert -1.  Options: a
//             correction per expert added to the scores for the choice only; groups of neighbouring experts of which
//             only the best few stay in the race; identity experts (no tensors; marked -2); weights scaled.
// moe_combine x[t] += the sum of the token's choices' rows, an identity expert's choice being its weight times the input.
// moe_plan    one CTA: the (token, choice) slots sorted by expert, and a list of tiles of at most `tile_rows` slots of
//             one expert each: tile_info[i] = (expert, first place in the sorted list, slots).  How many tiles there are
//             depends on the data; the kernels that follow are launched for the most there can be and read the count.
// moe_gemm    per tile and block of output columns: out[slot, n] = sum_k A[row(slot), k] W[expert][n, k], the rows
//             gathered through the sorted list (row(slot) = slot / a_div: the token's row where the input is shared by
//             a token's choices, the slot's own row where it is not).  GATED: W holds [gate | up] rows (2 N of them);
//             with the routing weight w of the slot the result is silu(w g) * (w u), which is what the gated unit
//             makes of the expert's input scaled by w (the products are linear in it, so w is applied to the float32
//             sums instead of to the rounded input), or the bounded unit times w (gated_unit.cuh).  bfloat16 runs on tensor cores (mma.sync m16n8k16, float32
//             accumulation; 64 x 64 tiles, 16-byte cp.async in two stages), float32 (and inner sizes that are no
//             multiple of 8) on the CUDA cores with float32 FMAs in the order of k.  A step of a few tokens (decoding)
//             takes tiles of 4 slots and a warp per output column instead (moe_rows_kernel).
// A slot's result does not depend on which tile it lands in or on its place there: every output element is a sum over
// k in a fixed order.  The sum over a token's choices is taken by the caller in the order of the choices.
#include "common.cuh"
#include "gated_unit.cuh"

MLXB_DEFINE_LAST_ERROR()

enum { MOE_SIGMOID = 0, MOE_SOFTMAX = 1 };

// Shared memory: per warp E scores, E choice scores, n_groups group maxima and n_groups flags.
__global__ void moe_route_kernel(const float* logits, int ldl, const int* __restrict__ token_req, int T, int E, int top,
                                 int score, int renorm, int* __restrict__ sel_expert, float* __restrict__ sel_weight,
                                 const float* __restrict__ correction, int n_groups, int keep_groups, int n_real,
                                 float renorm_eps, float out_scale) {
  extern __shared__ float mr_smem[];
  pdl_wait();
  pdl_trigger();
  logits = after_wait(logits);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  if (token_req && token_req[t] < 0) {
    for (int c = lane; c < top; c += 32) { sel_expert[(size_t)t * top + c] = -1; sel_weight[(size_t)t * top + c] = 0.f; }
    return;
  }
  float* sS = mr_smem + (size_t)warp * (2 * E + 2 * n_groups);     // [E] scores
  float* sC = sS + E;                                              // [E] what the choice goes by
  float* sG = sC + E;                                              // [n_groups] the largest choice score of a group
  int* sKeep = reinterpret_cast<int*>(sG + n_groups);              // [n_groups] is the group among the best?
  const float* z = logits + (size_t)t * ldl;
  float zmax = -INFINITY, zsum = 1.f;
  if (score == MOE_SOFTMAX) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) s += expf(z[e] - zmax);
    zsum = warp_sum(s);
  }
  for (int e = lane; e < E; e += 32) {
    const float s = score == MOE_SOFTMAX ? expf(z[e] - zmax) / zsum : 1.f / (1.f + expf(-z[e]));
    sS[e] = s;
    sC[e] = correction ? s + correction[e] : s;
  }
  __syncwarp();
  if (n_groups > 1 && keep_groups < n_groups) {
    // groups of neighbours: only experts of the keep_groups groups with the largest best choice score stay in the race
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float m = -INFINITY;
      for (int i = 0; i < per; ++i) m = fmaxf(m, sC[g * per + i]);
      sG[g] = m;
      sKeep[g] = 0;
    }
    __syncwarp();
    for (int c = 0; c < keep_groups; ++c) {
      float best = -INFINITY;
      int best_g = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32)
        if (!sKeep[g] && (sG[g] > best || (sG[g] == best && g < best_g))) { best = sG[g]; best_g = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
      }
      if (lane == 0 && best_g < n_groups) sKeep[best_g] = 1;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (!sKeep[e / per]) sC[e] = -INFINITY;
    __syncwarp();
  }
  float last_s = INFINITY;
  int last_e = -1;
  float wsum = 0.f;
  for (int c = 0; c < top; ++c) {
    // the largest choice score that comes after (last_s, last_e) in the order (score descending, expert ascending)
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float s = sC[e];
      const bool after = s < last_s || (s == last_s && e > last_e);
      if (after && (s > best || (s == best && e < best_e))) { best = s; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    last_s = best;
    last_e = best_e;
    const float w = best_e < E ? sS[best_e] : 0.f;      // the weight is the score itself, whatever the choice went by
    wsum += w;
    if (lane == 0) {
      // an expert from n_real on has no tensors (its output is its input): marked -2, which the plan passes over
      sel_expert[(size_t)t * top + c] = best_e < n_real ? best_e : (best_e < E ? -2 : -1);
      sel_weight[(size_t)t * top + c] = w;
    }
  }
  __syncwarp();
  if (renorm) {
    const float d = wsum + renorm_eps;
    for (int c = lane; c < top; c += 32) sel_weight[(size_t)t * top + c] = sel_weight[(size_t)t * top + c] / d * out_scale;
  } else if (out_scale != 1.f) {
    for (int c = lane; c < top; c += 32) sel_weight[(size_t)t * top + c] *= out_scale;
  }
}

// correction: float32 [E] added to the scores for the choice only, or null; n_groups > 1: the experts form n_groups
// equal groups of neighbours of which the keep_groups best (by their largest choice score) stay in the race; n_real:
// experts n_real .. E-1 are identity experts, chosen like the others and marked -2 in sel_expert; renorm: the weights
// are divided by (their sum + renorm_eps); every weight is multiplied by out_scale.
MLXB_EXPORT int mlxb_moe_route(const float* logits, int ldl, const int* token_req, int T, int E, int top, int score,
                               int renorm, int* sel_expert, float* sel_weight, const float* correction, int n_groups,
                               int keep_groups, int n_real, float renorm_eps, float out_scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || ldl < E || score < 0 || score > 1 || n_groups < 1 || E % n_groups ||
      keep_groups < 1 || keep_groups > n_groups || n_real < 0 || n_real > E || top > keep_groups * (E / n_groups))
    return mlxb_fail(MLXB_BAD_ARG, "moe_route: %d of %d experts (%d with tensors), score %d, %d of %d groups", top, E,
                     n_real, score, keep_groups, n_groups);
  const size_t per_warp = sizeof(float) * (2 * (size_t)E + 2 * (size_t)n_groups);
  if (per_warp > 48 * 1024) return mlxb_fail(MLXB_BAD_ARG, "moe_route: %d experts are more than a warp keeps", E);
  const int warps = 4 * per_warp <= 48 * 1024 ? 4 : 1;
  launch_pdl(moe_route_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), warps * per_warp, stream, logits, ldl,
             token_req, T, E, top, score, renorm, sel_expert, sel_weight, correction, n_groups, keep_groups, n_real,
             renorm_eps, out_scale);
  return mlxb_check_launch("moe_route");
}

// x[t] += sum over the token's choices, in their order: the expert's row y[t * top + c] for a choice with tensors,
// sel_weight * h[t] for an identity expert (sel_expert -2).  Rows that pad the step are passed over.
template <typename T>
__global__ void moe_combine_kernel(float* x, int ldx, const float* y, int ldy, const int* sel_expert,
                                   const float* sel_weight, const T* h, int ldh, const int* __restrict__ token_req,
                                   int top, int D) {
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  y = after_wait(y);
  sel_expert = after_wait(sel_expert);
  sel_weight = after_wait(sel_weight);
  h = after_wait(h);
  const int t = blockIdx.x;
  if (token_req && token_req[t] < 0) return;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int slot = t * top + k, e = sel_expert[slot];
      if (e >= 0) acc += y[(size_t)slot * ldy + c];
      else if (e == -2) acc = fmaf(sel_weight[slot], to_f(h[(size_t)t * ldh + c]), acc);
    }
    x[(size_t)t * ldx + c] += acc;
  }
}

MLXB_EXPORT int mlxb_moe_combine(int dtype, float* x, int ldx, const float* y, int ldy, const int* sel_expert,
                                 const float* sel_weight, const void* h, int ldh, const int* token_req, int T, int top,
                                 int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0 || top <= 0 || ldx < D || ldy < D || ldh < D)
    return mlxb_fail(MLXB_BAD_ARG, "moe_combine: width %d, %d choices, strides %d / %d / %d", D, top, ldx, ldy, ldh);
  const int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : 64);
  if (dtype == MLXB_F32)
    launch_pdl(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, x, ldx, y, ldy, sel_expert, sel_weight,
               (const float*)h, ldh, token_req, top, D);
  else if (dtype == MLXB_BF16)
    launch_pdl(moe_combine_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, ldx, y, ldy, sel_expert,
               sel_weight, (const __nv_bfloat16*)h, ldh, token_req, top, D);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "moe_combine: dtype code %d", dtype);
  return mlxb_check_launch("moe_combine");
}

// sorted [S]; tile_info [max_tiles][3]; n_tiles [1].  Shared memory: 3 E + 1 ints.
__global__ void moe_plan_kernel(const int* sel_expert, int S, int E, int tile_rows, int max_tiles,
                                int* __restrict__ sorted, int* __restrict__ tile_info, int* __restrict__ n_tiles) {
  extern __shared__ int mp_smem[];
  int* cnt = mp_smem;          // [E]
  int* off = cnt + E;          // [E]
  int* cur = off + E;          // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
  pdl_wait();
  pdl_trigger();
  sel_expert = after_wait(sel_expert);
  __syncthreads();
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    const int e = sel_expert[i];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = acc;
      for (int r0 = 0; r0 < cnt[e] && nt < max_tiles; r0 += tile_rows) {
        tile_info[3 * nt] = e;
        tile_info[3 * nt + 1] = acc + r0;
        tile_info[3 * nt + 2] = min(tile_rows, cnt[e] - r0);
        ++nt;
      }
      acc += cnt[e];
    }
    n_tiles[0] = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    const int e = sel_expert[i];
    if (e >= 0 && e < E) sorted[off[e] + atomicAdd(&cur[e], 1)] = i;
  }
}

MLXB_EXPORT int mlxb_moe_plan(const int* sel_expert, int S, int E, int tile_rows, int max_tiles, int* sorted,
                              int* tile_info, int* n_tiles, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (E <= 0 || tile_rows <= 0 || max_tiles < (S + tile_rows - 1) / tile_rows + E || E > 8192)
    return mlxb_fail(MLXB_BAD_ARG, "moe_plan: %d slots, %d experts, tiles of %d, room for %d", S, E, tile_rows, max_tiles);
  launch_pdl(moe_plan_kernel, dim3(1), dim3(S >= 4096 ? 1024 : 256), sizeof(int) * 3 * (size_t)E, stream, sel_expert, S,
             E, tile_rows, max_tiles, sorted, tile_info, n_tiles);
  return mlxb_check_launch("moe_plan");
}

// ---------------------------------------------------------------- CUDA cores: any sizes, float32 or bfloat16 inputs
constexpr int MS_BM = 16, MS_BN = 64, MS_BK = 32, MS_THREADS = 256;

template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(MS_THREADS)
moe_gemm_simt_kernel(const T* A, int lda, int a_div, const T* __restrict__ W, long long w_stride, int N, int K,
                     const int* sorted, const int* tile_info, const int* n_tiles, const float* sel_weight,
                     TO* __restrict__ out, int ldo, int act, float limit) {
  __shared__ float sA[MS_BM][MS_BK + 1];
  __shared__ float sW[GATED ? 2 : 1][MS_BN][MS_BK + 1];
  __shared__ int sSlot[MS_BM];
  pdl_wait();
  pdl_trigger();
  A = after_wait(A);
  sorted = after_wait(sorted);
  tile_info = after_wait(tile_info);
  n_tiles = after_wait(n_tiles);
  sel_weight = after_wait(sel_weight);
  const int tile = blockIdx.x;
  if (tile >= n_tiles[0]) return;
  const int e = tile_info[3 * tile], first = tile_info[3 * tile + 1], rows = tile_info[3 * tile + 2];
  const int n0 = blockIdx.y * MS_BN, tid = threadIdx.x;
  if (tid < MS_BM) sSlot[tid] = tid < rows ? sorted[first + tid] : -1;
  __syncthreads();
  const T* We = W + (size_t)e * w_stride;
  const int r = tid / 16, cb = tid % 16;          // this thread: row r, columns cb + 16 i
  float acc[GATED ? 2 : 1][4];
#pragma unroll
  for (int h = 0; h < (GATED ? 2 : 1); ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[h][i] = 0.f;
  for (int k0 = 0; k0 < K; k0 += MS_BK) {
    for (int x = tid; x < MS_BM * MS_BK; x += MS_THREADS) {
      const int rr = x / MS_BK, kk = x - rr * MS_BK;
      const int slot = sSlot[rr];
      sA[rr][kk] = (slot >= 0 && k0 + kk < K) ? to_f(A[(size_t)(slot / a_div) * lda + k0 + kk]) : 0.f;
    }
    for (int x = tid; x < (GATED ? 2 : 1) * MS_BN * MS_BK; x += MS_THREADS) {
      const int h = x / (MS_BN * MS_BK), y = x - h * MS_BN * MS_BK;
      const int nn = y / MS_BK, kk = y - nn * MS_BK;
      sW[h][nn][kk] = (n0 + nn < N && k0 + kk < K) ? to_f(We[(size_t)(h * N + n0 + nn) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < MS_BK; ++kk) {
      const float a = sA[r][kk];
#pragma unroll
      for (int h = 0; h < (GATED ? 2 : 1); ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] = fmaf(a, sW[h][cb + 16 * i][kk], acc[h][i]);
    }
    __syncthreads();
  }
  const int slot = sSlot[r];
  if (slot < 0) return;
  const float w = GATED ? sel_weight[slot] : 1.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = n0 + cb + 16 * i;
    if (n >= N) continue;
    float v = acc[0][i];
    if (GATED) v = mlxb_gated_unit(act, acc[0][i], acc[GATED ? 1 : 0][i], w, limit);
    out[(size_t)slot * ldo + n] = from_f<TO>(v);
  }
}

// ---------------------------------------------------------------- few slots (decoding): bfloat16, K a multiple of 8
// A tile is up to MV_ROWS slots of one expert.  The CTA keeps their rows in shared memory; a warp takes an output
// column at a time, reads its row of W (and, gated, the up row of the same column) once with 16 bytes a lane, and
// forms the column's sum for every slot of the tile: lanes over k, then a butterfly over the lanes.  The weights are
// streamed by many small CTAs with all of a row's loads in flight, which is what a step of a few tokens needs.
constexpr int MV_ROWS = 4, MV_COLS = 32, MV_THREADS = 256;

template <typename TO, bool GATED>
__global__ void __launch_bounds__(MV_THREADS)
moe_rows_kernel(const __nv_bfloat16* A, int lda, int a_div, const __nv_bfloat16* __restrict__ W, long long w_stride, int N,
                int K, const int* sorted, const int* tile_info, const int* n_tiles, const float* sel_weight,
                TO* __restrict__ out, int ldo, int act, float limit) {
  extern __shared__ uint4 mv_rows[];          // [MV_ROWS][K / 8]
  __shared__ int sSlot[MV_ROWS];
  pdl_wait();
  pdl_trigger();
  A = after_wait(A);
  sorted = after_wait(sorted);
  tile_info = after_wait(tile_info);
  n_tiles = after_wait(n_tiles);
  sel_weight = after_wait(sel_weight);
  const int tile = blockIdx.x;
  if (tile >= n_tiles[0]) return;
  const int e = tile_info[3 * tile], first = tile_info[3 * tile + 1], rows = tile_info[3 * tile + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k8 = K >> 3;
  if (tid < MV_ROWS) sSlot[tid] = tid < rows ? sorted[first + tid] : -1;
  __syncthreads();
  for (int x = tid; x < MV_ROWS * k8; x += MV_THREADS) {
    const int rr = x / k8, c = x - rr * k8;
    const int slot = sSlot[rr];
    mv_rows[x] = slot >= 0 ? reinterpret_cast<const uint4*>(A + (size_t)(slot / a_div) * lda)[c] : make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  const __nv_bfloat16* We = W + (size_t)e * w_stride;
#pragma unroll 1
  for (int j = 0; j < MV_COLS / 8; ++j) {
    const int n = blockIdx.y * MV_COLS + j * 8 + warp;
    if (n >= N) continue;
    const uint4* wg = reinterpret_cast<const uint4*>(We + (size_t)n * K);
    const uint4* wu = reinterpret_cast<const uint4*>(We + (size_t)(N + n) * K);
    float acc[GATED ? 2 : 1][MV_ROWS];
#pragma unroll
    for (int h = 0; h < (GATED ? 2 : 1); ++h)
#pragma unroll
      for (int rr = 0; rr < MV_ROWS; ++rr) acc[h][rr] = 0.f;
#pragma unroll 4
    for (int c = lane; c < k8; c += 32) {
      float g[8], u[8];
      unpack8(wg[c], g);
      if (GATED) unpack8(wu[c], u);
#pragma unroll
      for (int rr = 0; rr < MV_ROWS; ++rr) {
        float a[8];
        unpack8(mv_rows[rr * k8 + c], a);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[0][rr] = fmaf(a[i], g[i], acc[0][rr]);
          if (GATED) acc[1][rr] = fmaf(a[i], u[i], acc[1][rr]);
        }
      }
    }
#pragma unroll
    for (int h = 0; h < (GATED ? 2 : 1); ++h)
#pragma unroll
      for (int rr = 0; rr < MV_ROWS; ++rr) acc[h][rr] = warp_sum(acc[h][rr]);
    if (lane < MV_ROWS) {
      const int slot = sSlot[lane];
      if (slot >= 0) {
        float v = 0.f, v2 = 0.f;
#pragma unroll
        for (int rr = 0; rr < MV_ROWS; ++rr)
          if (rr == lane) { v = acc[0][rr]; v2 = acc[GATED ? 1 : 0][rr]; }
        if (GATED) {
          v = mlxb_gated_unit(act, v, v2, sel_weight[slot], limit);
        }
        out[(size_t)slot * ldo + n] = from_f<TO>(v);
      }
    }
  }
}

// ---------------------------------------------------------------- tensor cores: bfloat16, K a multiple of 8
constexpr int MG_BM = 64, MG_BN = 64, MG_BK = 32, MG_THREADS = 128, MG_LD = MG_BK + 8;

__device__ __forceinline__ unsigned mg_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mg_ldm_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mg_ldm_x2(unsigned (&r)[2], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mg_mma(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mg_cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(mg_smem(dst)), "l"(src) : "memory");
}

template <typename TO, bool GATED>
__global__ void __launch_bounds__(MG_THREADS)
moe_gemm_tc_kernel(const __nv_bfloat16* A, int lda, int a_div, const __nv_bfloat16* __restrict__ W, long long w_stride,
                   int N, int K, const int* sorted, const int* tile_info, const int* n_tiles, const float* sel_weight,
                   TO* __restrict__ out, int ldo, int act, float limit) {
  constexpr int NH = GATED ? 2 : 1;
  __shared__ __align__(16) __nv_bfloat16 sA[2][MG_BM][MG_LD];
  __shared__ __align__(16) __nv_bfloat16 sW[2][NH][MG_BN][MG_LD];
  __shared__ int sSlot[MG_BM];
  pdl_wait();
  pdl_trigger();
  A = after_wait(A);
  sorted = after_wait(sorted);
  tile_info = after_wait(tile_info);
  n_tiles = after_wait(n_tiles);
  sel_weight = after_wait(sel_weight);
  const int tile = blockIdx.x;
  if (tile >= n_tiles[0]) return;
  const int e = tile_info[3 * tile], first = tile_info[3 * tile + 1], rows = tile_info[3 * tile + 2];
  const int n0 = blockIdx.y * MG_BN, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < MG_BM) sSlot[tid] = tid < rows ? sorted[first + tid] : -1;
  __syncthreads();
  const __nv_bfloat16* We = W + (size_t)e * w_stride;

  auto load_stage = [&](int k0, int buf) {
    constexpr int CH = MG_BK / 8;                       // 16-byte pieces per row
    for (int x = tid; x < MG_BM * CH; x += MG_THREADS) {
      const int rr = x / CH, kk = (x - rr * CH) * 8;
      const int slot = sSlot[rr];
      __nv_bfloat16* dst = &sA[buf][rr][kk];
      if (slot >= 0 && k0 + kk < K) mg_cp16(dst, A + (size_t)(slot / a_div) * lda + k0 + kk);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int x = tid; x < NH * MG_BN * CH; x += MG_THREADS) {
      const int h = x / (MG_BN * CH), y = x - h * MG_BN * CH;
      const int nn = y / CH, kk = (y - nn * CH) * 8;
      __nv_bfloat16* dst = &sW[buf][h][nn][kk];
      if (n0 + nn < N && k0 + kk < K) mg_cp16(dst, We + (size_t)(h * N + n0 + nn) * K + k0 + kk);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[NH][MG_BN / 8][4];
#pragma unroll
  for (int h = 0; h < NH; ++h)
#pragma unroll
    for (int j = 0; j < MG_BN / 8; ++j)
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[h][j][x] = 0.f;

  load_stage(0, 0);
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                     // this stage has landed; everybody is done with the other one
    if (k0 + MG_BK < K) load_stage(k0 + MG_BK, buf ^ 1);
#pragma unroll
    for (int ks = 0; ks < MG_BK; ks += 16) {
      unsigned a[4];
      mg_ldm_x4(a, mg_smem(&sA[buf][warp * 16 + (lane & 15)][ks + (lane >> 4) * 8]));
#pragma unroll
      for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int j = 0; j < MG_BN / 8; ++j) {
          unsigned b[2];
          mg_ldm_x2(b, mg_smem(&sW[buf][h][j * 8 + (lane & 7)][ks + ((lane >> 3) & 1) * 8]));
          mg_mma(acc[h][j], a, b);
        }
    }
    buf ^= 1;
  }
  const int g = lane >> 2, q4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int slot = sSlot[warp * 16 + g + half * 8];
    if (slot < 0) continue;
    const float w = GATED ? sel_weight[slot] : 1.f;
#pragma unroll
    for (int j = 0; j < MG_BN / 8; ++j)
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int n = n0 + j * 8 + q4 * 2 + x;
        if (n >= N) continue;
        float v = acc[0][j][half * 2 + x];
        if (GATED) v = mlxb_gated_unit(act, v, acc[NH - 1][j][half * 2 + x], w, limit);
        out[(size_t)slot * ldo + n] = from_f<TO>(v);
      }
  }
}

// A: `dtype` [*, lda]; W: `dtype` [E][(gated ? 2 : 1) * N][K] at w_stride elements an expert; out: `dtype`, or float32
// with out_f32, [S, ldo]; max_tiles: the tiles the plan had room for (the grid); tile_rows: what the plan was made with,
// mlxb_moe_tile_rows(1) for the tensor-core kernel (bfloat16, every inner size a multiple of 8) or
// mlxb_moe_tile_rows(0) for the kernel on the CUDA cores, mlxb_moe_tile_rows(2) for the kernel for few slots (bfloat16,
// inner sizes multiples of 8 up to 6144); the products of one feed-forward share a plan.
MLXB_EXPORT int mlxb_moe_tile_rows(int tensor_cores) { return tensor_cores == 2 ? MV_ROWS : tensor_cores ? MG_BM : MS_BM; }

MLXB_EXPORT int mlxb_moe_gemm(int dtype, int out_f32, int gated, const void* A, int lda, int a_div, const void* W,
                              long long w_stride, int N, int K, const int* sorted, const int* tile_info,
                              const int* n_tiles, int max_tiles, int tile_rows, const float* sel_weight, void* out,
                              int ldo, int act, float limit, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (N <= 0 || K <= 0 || a_div <= 0 || lda < K || ldo < N || (gated && !sel_weight) ||
      (tile_rows != MG_BM && tile_rows != MS_BM && tile_rows != MV_ROWS) ||
      ((tile_rows == MG_BM || tile_rows == MV_ROWS) && dtype != MLXB_BF16))
    return mlxb_fail(MLXB_BAD_ARG, "moe_gemm: %d x %d, strides %d / %d, tiles of %d rows", N, K, lda, ldo, tile_rows);
#define MOE_SIMT(T, TO, G)                                                                                             \
  launch_pdl(moe_gemm_simt_kernel<T, TO, G>, dim3(max_tiles, (N + MS_BN - 1) / MS_BN), dim3(MS_THREADS), 0, stream,    \
             (const T*)A, lda, a_div, (const T*)W, w_stride, N, K, sorted, tile_info, n_tiles, sel_weight, (TO*)out, ldo, act, limit)
#define MOE_TC(TO, G)                                                                                                  \
  launch_pdl(moe_gemm_tc_kernel<TO, G>, dim3(max_tiles, (N + MG_BN - 1) / MG_BN), dim3(MG_THREADS), 0, stream,         \
             (const __nv_bfloat16*)A, lda, a_div, (const __nv_bfloat16*)W, w_stride, N, K, sorted, tile_info, n_tiles, \
             sel_weight, (TO*)out, ldo, act, limit)
  if (dtype == MLXB_F32) {
    if (gated) MOE_SIMT(float, float, true); else MOE_SIMT(float, float, false);
  } else if (dtype == MLXB_BF16) {
    const bool tc = K % 8 == 0 && lda % 8 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0 && w_stride % 8 == 0;
    if ((tile_rows == MG_BM || tile_rows == MV_ROWS) && !tc)
      return mlxb_fail(MLXB_BAD_ARG, "moe_gemm: rows of %d elements at stride %d are not in whole 16 bytes", K, lda);
    if (tile_rows == MV_ROWS) {
      const size_t smem = (size_t)MV_ROWS * K * sizeof(__nv_bfloat16);
      if (smem > 48 * 1024) return mlxb_fail(MLXB_BAD_ARG, "moe_gemm (few slots): rows of %d elements", K);
#define MOE_ROWS(TO, G)                                                                                                \
  launch_pdl(moe_rows_kernel<TO, G>, dim3(max_tiles, (N + MV_COLS - 1) / MV_COLS), dim3(MV_THREADS), smem, stream,     \
             (const __nv_bfloat16*)A, lda, a_div, (const __nv_bfloat16*)W, w_stride, N, K, sorted, tile_info, n_tiles, \
             sel_weight, (TO*)out, ldo, act, limit)
      if (gated) { if (out_f32) MOE_ROWS(float, true); else MOE_ROWS(__nv_bfloat16, true); }
      else { if (out_f32) MOE_ROWS(float, false); else MOE_ROWS(__nv_bfloat16, false); }
#undef MOE_ROWS
    } else if (tile_rows == MG_BM) {
      if (gated) { if (out_f32) MOE_TC(float, true); else MOE_TC(__nv_bfloat16, true); }
      else { if (out_f32) MOE_TC(float, false); else MOE_TC(__nv_bfloat16, false); }
    } else {
      if (gated) { if (out_f32) MOE_SIMT(__nv_bfloat16, float, true); else MOE_SIMT(__nv_bfloat16, __nv_bfloat16, true); }
      else { if (out_f32) MOE_SIMT(__nv_bfloat16, float, false); else MOE_SIMT(__nv_bfloat16, __nv_bfloat16, false); }
    }
  } else {
    return mlxb_fail(MLXB_BAD_DTYPE, "moe_gemm: dtype code %d", dtype);
  }
#undef MOE_SIMT
#undef MOE_TC
  return mlxb_check_launch("moe_gemm");
}
