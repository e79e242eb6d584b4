// The experts' products of moe.cu for many slots (prompt portions), on the 5th-generation tensor cores.
//
// moe_gather      the rows of a step's (token, choice) slots in the plan's order: dst[i] = src[sorted[i] / a_div], so that
//                 the rows of one expert lie together and a tile of them is one TMA copy.
// moe_gemm_tc05   per tile of the plan (up to 128 slots of one expert, rows first .. first + slots - 1 of the gathered
//                 matrix) and block of output columns: out = A . W[expert]^T.  bfloat16 operands, float32 accumulation.
//                 A tile takes BN = 128 or 256 rows of W (chosen on the host by what the rounds of tiles over the SMs
//                 cost).  GATED: W holds [gate | up] rows; a CTA takes BN / 2 gate rows and the up rows of the same
//                 columns as one BN-wide operand, and the epilogue writes silu(w g) * (w u) (w: the slot's routing
//                 weight, applied to the float32 sums) as bfloat16 rows IN THE PLAN'S ORDER, ready to be the second
//                 product's operand.  Not gated: BN output columns a CTA, float32 rows written to the slot's own row
//                 (out[sorted[i]]).
//
// The kernel is persistent (one CTA per SM walks over the (tile, column block) pairs; how many tiles there are is read
// from the plan on the device) and has the roles of the linear kernel in gemm_tcgen05.cu: warp 0 is the TMA producer
// (a ring of stages of a 128 x 64 tile of A and BN / 64 boxes of 64 x 64 of W, 128-byte swizzle), warp 1 owns the
// tensor memory and issues tcgen05.mma into one of two 128 x BN float32 accumulators, warps 2-9 are the epilogue (two
// per quadrant of TMEM lanes).  Rows of a tile beyond the expert's slots hold another expert's rows or zeros; they are
// computed and not stored.  Every wait on an mbarrier is bounded; a timeout raises MLXB_ST_WAIT_TIMEOUT and all roles
// leave through the common exit, where the tensor memory is freed.
// A slot's result does not depend on which tile it lands in or on its place there: the sum over K runs stage by
// stage in a fixed order.
#include "tcgen05.cuh"
#include "gated_unit.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int MT_BM = 128, MT_BK = 64;
constexpr int MT_EPI_WARPS = 8;
constexpr int MT_THREADS = 64 + 32 * MT_EPI_WARPS;
// BN: rows of W a tile takes (128 or 256); a wider tile moves fewer bytes a flop, a narrower one leaves fewer SMs idle
// in the last round of a small problem.
constexpr int mt_stages(int bn) { return bn == 256 ? 4 : 6; }

template <int BN>
struct MoeSmem {
  alignas(1024) __nv_bfloat16 a[mt_stages(BN)][MT_BM * MT_BK];
  alignas(1024) __nv_bfloat16 b[mt_stages(BN)][BN * MT_BK];
  alignas(8) uint64_t full[mt_stages(BN)];
  uint64_t empty[mt_stages(BN)];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t drained;
  uint32_t tmem_base;
  int abort_flag;
};


// dst [*, ldd] <- src [*, lds], `cols` columns (a multiple of 8): one warp a row, 16 bytes a lane and step.
__global__ void moe_gather_kernel(const __nv_bfloat16* src, int lds, int a_div, const int* sorted, const int* tile_info,
                                  const int* n_tiles, int cols, __nv_bfloat16* __restrict__ dst, int ldd) {
  pdl_wait();
  pdl_trigger();
  src = after_wait(src);
  sorted = after_wait(sorted);
  tile_info = after_wait(tile_info);
  const int t = blockIdx.x;
  if (t >= after_wait(n_tiles)[0]) return;
  const int first = tile_info[3 * t + 1], cnt = tile_info[3 * t + 2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  // the tile's rows are spread over the CTAs of a grid column; a lane has up to four 16-byte pieces of a row in flight
  for (int r = blockIdx.y * warps + warp; r < cnt; r += gridDim.y * warps) {
    const int slot = sorted[first + r];
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)(slot / a_div) * lds);
    uint4* d = reinterpret_cast<uint4*>(dst + (size_t)(first + r) * ldd);
    const int n16 = cols / 8;
    for (int c = lane; c < n16; c += 128) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + 32 * j < n16) v[j] = s[c + 32 * j];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + 32 * j < n16) d[c + 32 * j] = v[j];
    }
  }
}

template <bool GATED, int BN>
__global__ void __launch_bounds__(MT_THREADS)
moe_gemm_tc05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     const int* sorted, const int* tile_info, const int* n_tiles_p, int NW, int N, int K,
                     const float* sel_weight, void* out_v, int ldo, int* __restrict__ status, int act,
                     float limit) {
  extern __shared__ uint8_t smem_raw[];
  MoeSmem<BN>& sm = *reinterpret_cast<MoeSmem<BN>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int MT_BN = BN, MT_STAGES = mt_stages(BN), HALF = BN / 2;
  constexpr uint32_t MT_STAGE_BYTES = (MT_BM + BN) * MT_BK * sizeof(__nv_bfloat16);
  constexpr uint32_t MT_TMEM_COLS = 2 * BN;   // two accumulators
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + MT_BK - 1) / MT_BK;
  constexpr int COLS = GATED ? MT_BN / 2 : MT_BN;        // output columns a CTA's tile makes
  const int n_blocks = (N + COLS - 1) / COLS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MT_STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&sm.acc_full[b], 1); mbar_init(&sm.acc_empty[b], 32 * MT_EPI_WARPS); }
    mbar_init(&sm.drained, 1);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(MT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  volatile int* abort_flag = &sm.abort_flag;
  pdl_trigger();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sm.tmem_base;
  pdl_wait();   // the plan, the gathered rows and the routing weights come from the kernels before
  sorted = after_wait(sorted);
  tile_info = after_wait(tile_info);
  sel_weight = after_wait(sel_weight);
  const int n_tiles = after_wait(n_tiles_p)[0];
  const int n_work = n_tiles * n_blocks;
  // work item w: tile w % n_tiles, column block w / n_tiles (neighbouring CTAs share an expert's rows of W)

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const int t = w % n_tiles, nb = w / n_tiles;
        const int expert = tile_info[3 * t], first = tile_info[3 * t + 1];
        const int w0 = expert * NW + nb * COLS;                    // gate rows, or the first half of the output rows
        const int w1 = GATED ? w0 + NW / 2 : w0 + HALF;            // up rows of the same columns, or the second half
        for (int kt = 0; kt < k_tiles; ++kt, ++issued) {
          const int s = issued % MT_STAGES;
          const uint32_t ph = (issued / MT_STAGES) & 1;
          if (issued >= MT_STAGES && !mbar_wait(&sm.empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&sm.full[s], MT_STAGE_BYTES);
          tma_load_2d(sm.a[s], &map_a, kt * MT_BK, first, &sm.full[s]);
#pragma unroll
          for (int i = 0; i < HALF / 64; ++i) {   // boxes of 64 rows: in the 128-byte swizzle simply consecutive 8-row groups
            tma_load_2d(sm.b[s] + (64 * i) * MT_BK, &map_w, kt * MT_BK, w0 + 64 * i, &sm.full[s]);
            tma_load_2d(sm.b[s] + (HALF + 64 * i) * MT_BK, &map_w, kt * MT_BK, w1 + 64 * i, &sm.full[s]);
          }
        }
      }
      if (*abort_flag) {   // gave up: let the copies already issued land before the CTA exits
        for (int i = issued > MT_STAGES ? issued - MT_STAGES : 0; i < issued; ++i) {
          const uint32_t addr = smem_u32(&sm.full[i % MT_STAGES]);
          for (uint32_t p = 0; p < (1u << 20); ++p) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"((uint32_t)((i / MT_STAGES) & 1))
                         : "memory");
            if (done) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(MT_BM, MT_BN);
      int consumed = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++it) {
        const int b = it & 1;
        ok = mbar_wait(&sm.acc_empty[b], ((it >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + (uint32_t)(b * MT_BN);
        for (int kt = 0; kt < k_tiles; ++kt, ++consumed) {
          const int s = consumed % MT_STAGES;
          const uint32_t ph = (consumed / MT_STAGES) & 1;
          ok = mbar_wait(&sm.full[s], ph, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t da = umma_desc(smem_u32(sm.a[s])), db = umma_desc(smem_u32(sm.b[s]));
#pragma unroll
          for (int k = 0; k < MT_BK / 16; ++k)
            umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          umma_commit(&sm.empty[s]);
        }
        if (ok) umma_commit(&sm.acc_full[b]);
      }
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31; the two warps of a quadrant split the columns
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int it = 0;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x, ++it) {
      const int b = it & 1;
      const int t = w % n_tiles, nb = w / n_tiles;
      const int first = tile_info[3 * t + 1], cnt = tile_info[3 * t + 2];
      const int r = q * 32 + lane;
      const bool live = r < cnt;
      const int slot = live ? sorted[first + r] : -1;
      const float wgt = (GATED && live) ? sel_weight[slot] : 1.f;
      if (!mbar_wait(&sm.acc_full[b], (it >> 1) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * MT_BN);
      if (GATED) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_v) + (size_t)(first + r) * ldo;
#pragma unroll 1
        for (int c0 = 0; c0 < HALF / 2; c0 += 32) {   // this warp's output columns: gate and up of a column in one lane
          uint32_t g[32], u[32];
          tmem_ld32(taddr + (uint32_t)(HALF / 2 * half + c0), g);
          tmem_ld32(taddr + (uint32_t)(HALF + HALF / 2 * half + c0), u);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (c0 + 32 >= HALF / 2) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sm.acc_empty[b]);
          }
          if (live) {
            const int n0 = nb * COLS + HALF / 2 * half + c0;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              const int n8 = n0 + 8 * g8;
              if (n8 >= N) break;                 // N is a multiple of 8: a group is whole or absent
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i)
                v[i] = mlxb_gated_unit(act, __uint_as_float(g[8 * g8 + i]), __uint_as_float(u[8 * g8 + i]), wgt, limit);
              *reinterpret_cast<uint4*>(o + n8) = pack8(v);
            }
          }
        }
      } else {
        float* o = reinterpret_cast<float*>(out_v) + (size_t)(live ? slot : 0) * ldo;
#pragma unroll 1
        for (int c0 = 0; c0 < MT_BN / 2; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(taddr + (uint32_t)(MT_BN / 2 * half + c0), v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (c0 + 32 >= MT_BN / 2) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sm.acc_empty[b]);
          }
          if (live) {
            const int n0 = nb * COLS + MT_BN / 2 * half + c0;
#pragma unroll
            for (int g4 = 0; g4 < 8; ++g4) {
              const int n4 = n0 + 4 * g4;
              if (n4 >= N) break;               // N is a multiple of 8
              *reinterpret_cast<float4*>(o + n4) =
                  make_float4(__uint_as_float(v[4 * g4]), __uint_as_float(v[4 * g4 + 1]), __uint_as_float(v[4 * g4 + 2]),
                              __uint_as_float(v[4 * g4 + 3]));
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  const bool aborted = sm.abort_flag != 0;
  if (threadIdx.x == 0 && aborted) atomicOr(status, MLXB_ST_WAIT_TIMEOUT);
  if (warp == 1) {
    if (lane == 0 && aborted) {
      // products this thread issued may still run on the tensor memory that is freed below: one more commit arrives
      // when all of them have completed; wait for it, bounded
      umma_commit(&sm.drained);
      const uint32_t addr = smem_u32(&sm.drained);
      for (uint32_t p = 0; p < (1u << 20); ++p) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"(0u) : "memory");
        if (done) break;
      }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(MT_TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host side

static int mt_make_map(CUtensorMap* map, const void* base, long long rows, int cols, int ld, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__nv_bfloat16)};
  const cuuint32_t box[2] = {(cuuint32_t)MT_BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    const char* msg = nullptr;
    cuGetErrorString(r, &msg);
    return mlxb_fail(MLXB_BAD_ARG, "moe_gemm (tensor cores): cuTensorMapEncodeTiled(%lld x %d, ld %d): %s", rows, cols, ld,
                     msg ? msg : "?");
  }
  return 0;
}

static int mt_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

struct MtLaunch {
  CUtensorMap ma, mw;
  const int *sorted, *tile_info, *n_tiles;
  int NW, N, K;
  const float* sel_weight;
  void* out;
  int ldo;
  int* status;
  int max_tiles;
  cudaStream_t stream;
  int act;
  float limit;
};

template <bool GATED, int BN>
static int mt_launch(const MtLaunch& l) {
  static_assert(sizeof(MoeSmem<BN>) + 1024 <= 227 * 1024, "the stages fit a CTA's shared memory");
  auto kern = moe_gemm_tc05_kernel<GATED, BN>;
  const size_t smem = sizeof(MoeSmem<BN>) + 1024;
  static bool raised = false;   // once per kernel, and never for the first time inside a stream capture
  if (!raised) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess)
      return mlxb_fail((int)err, "moe_gemm (tensor cores): %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    raised = true;
  }
  const int cols = GATED ? BN / 2 : BN;
  const long long work = (long long)l.max_tiles * ((l.N + cols - 1) / cols);
  const dim3 grid((unsigned)(work < mt_sm_count() ? work : mt_sm_count()));
  launch_pdl(kern, grid, dim3(MT_THREADS), smem, l.stream, l.ma, l.mw, l.sorted, l.tile_info, l.n_tiles, l.NW, l.N, l.K,
             l.sel_weight, l.out, l.ldo, l.status, l.act, l.limit);
  return mlxb_check_launch("moe_gemm (tensor cores)");
}

MLXB_EXPORT int mlxb_moe_tc05_tile_rows() { return MT_BM; }

// src bfloat16 [*, lds]; dst bfloat16 [S, ldd]: dst[i] = src[sorted[i] / a_div] for the places of the plan's tiles.
MLXB_EXPORT int mlxb_moe_gather(const void* src, int lds, int a_div, const int* sorted, const int* tile_info,
                                const int* n_tiles, int max_tiles, int cols, void* dst, int ldd, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (cols <= 0 || (cols & 7) || (lds & 7) || (ldd & 7) || a_div <= 0 || (((uintptr_t)src | (uintptr_t)dst) & 15))
    return mlxb_fail(MLXB_BAD_ARG, "moe_gather: rows of %d columns at strides %d -> %d are not in whole 16 bytes", cols, lds, ldd);
  launch_pdl(moe_gather_kernel, dim3(max_tiles, 16), dim3(256), 0, stream, (const __nv_bfloat16*)src, lds, a_div, sorted,
             tile_info, n_tiles, cols, (__nv_bfloat16*)dst, ldd);
  return mlxb_check_launch("moe_gather");
}

// How many rows of W a tile takes: the width whose rounds of tiles over the SMs cost least, a tile's cost being the
// rows it streams per K step (128 of A plus BN of W).  How many tiles the plan holds is known on the device only: the
// estimate is full tiles plus half a tile an expert.  The second product stays at 128: its epilogue writes float32 rows,
// four times the bytes a column of the gated product's, and with 256 columns a tile the two accumulators no longer
// hide it (measured: 24.6 against 20.1 us at width 1024, 43.8 against 41.0 at width 2048).
static int mt_tile_width(int S, int E, int N, bool gated) {
  if (const char* force = getenv("MLXB_MOE_BN")) return atoi(force) == 256 ? 256 : 128;   // experiments and tests
  if (!gated) return 128;
  const long long tiles = (S + MT_BM - 1) / MT_BM + (E + 1) / 2;
  int best = 128;
  long long best_cost = -1;
  for (int bn : {256, 128}) {
    const int cols = gated ? bn / 2 : bn;
    const long long work = tiles * ((N + cols - 1) / cols);
    const long long cost = ((work + mt_sm_count() - 1) / mt_sm_count()) * (MT_BM + bn);
    if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
  }
  return best;
}

// A: bfloat16 [S, lda], rows in the plan's order; W: bfloat16 [E][NW][K] contiguous, NW = 2 N (gated: gate rows, then up
// rows) or N.  gated: out bfloat16 [S, ldo] in the plan's order = the gated unit of kind `act` (gated_unit.cuh); else out float32 [S, ldo], row
// sorted[i] = the product of row i.  The plan was made with tiles of mlxb_moe_tc05_tile_rows() slots.
// K, N, lda, ldo multiples of 8; A, W, out 16-byte aligned.
MLXB_EXPORT int mlxb_moe_gemm_tc05(int gated, const void* A, int lda, int S, const void* W, int E, int NW, int N, int K,
                                   const int* sorted, const int* tile_info, const int* n_tiles, int max_tiles,
                                   const float* sel_weight, void* out, int ldo, int* status, int act, float limit,
                                   cudaStream_t stream) {
  if (max_tiles <= 0 || S <= 0) return 0;
  if (N <= 0 || K <= 0 || E <= 0 || (K & 7) || (N & 7) || (lda & 7) || (ldo & 7) || lda < K || ldo < N ||
      NW != (gated ? 2 : 1) * N || (gated && !sel_weight) || (((uintptr_t)A | (uintptr_t)W | (uintptr_t)out) & 15) ||
      (long long)E * NW > 0x7fffffffLL)
    return mlxb_fail(MLXB_BAD_ARG, "moe_gemm (tensor cores): %d experts of %d x %d, strides %d / %d", E, NW, K, lda, ldo);
  MtLaunch l = {{}, {}, sorted, tile_info, n_tiles, NW, N, K, sel_weight, out, ldo, status, max_tiles, stream, act, limit};
  if (int e = mt_make_map(&l.ma, A, S, K, lda, MT_BM)) return e;
  if (int e = mt_make_map(&l.mw, W, (long long)E * NW, K, K, 64)) return e;
  const int bn = mt_tile_width(S, E, N, gated != 0);
  if (bn == 256) return gated ? mt_launch<true, 256>(l) : mt_launch<false, 256>(l);
  return gated ? mt_launch<true, 128>(l) : mt_launch<false, 128>(l);
}
