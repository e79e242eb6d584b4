// Layers with a state of fixed size per request: short causal convolutions, the selective
// state-space scan (Mamba-2) and the gated delta rule.  A step brings each request's next tokens as
// a run of rows (req_first_token[r] .. , as many as carry the request's index in token_req); the state
// of request r lives in row slots[r] of a float32 pool, is read at the start of the run and written
// back at its end, so a sequence may be cut into steps anywhere.  All state and everything that feeds
// a recurrence (step sizes, decays, gates, unit norms) is float32; inputs arrive in the activation
// dtype.  The order of additions for a token depends on the layer's sizes only, never on the batch.
//
// conv_silu          out[t, c] = silu(bias[c] + sum_j w[c, taps-1-j] * in(t - j, c)),  j = 0 .. taps-1 (act = 0: the sum
//                    as it is, without the silu),
//                    where in(t - j) is a row of this step if the run reaches that far back, else one of
//                    the request's last taps-1 inputs kept in the state (zeros before the sequence starts).
// conv_state_update  moves the last taps-1 inputs of every run into the state (launched after conv_silu).
// mamba2_scan        per (request, head): S <- exp(-exp(A_log) dt) S + dt B x^T,  y = S^T C + D x,
//                    dt = softplus(dt_raw + dt_bias); S is N x V (kept column by column in the pool).
// gated_delta_scan   per (request, head): S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with
//                    q and k divided by sqrt(|.|^2 + 1e-6) (q also by sqrt(dim)), beta = sigmoid(b_raw),
//                    g = exp(-exp(A_log) softplus(a_raw + dt_bias)); S is K x V (kept column by column).
//
// Both scans give a thread one column v of the state and 16 consecutive rows of it, in registers; the NS
// threads of a column are neighbouring lanes and add their partial sums by shuffles.  The inputs of 16 tokens
// at a time are staged in shared memory by the whole block, laid out so that a thread fetches its 16 values
// with four 16-byte loads; four tokens at a time go through the recurrence, their read-outs reduced together.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// Rows t0 .. t1-1 that belong to request r (they come first in the range).  Every thread of the block calls it.
__device__ __forceinline__ int request_rows(const int* __restrict__ token_req, int t0, int t1, int r) {
  int n = 0;
  for (int base = t0; base < t1; base += blockDim.x) {
    const int t = base + threadIdx.x;
    n += __syncthreads_count(t < t1 && token_req[t] == r);
  }
  return n;
}

// ---------------------------------------------------------------- short convolution

template <typename T>
__global__ void conv_silu_kernel(const T* in, int ldi, const float* __restrict__ w, const float* __restrict__ bias,
                                 int taps, int C, const float* state, const int* __restrict__ slots,
                                 const int* __restrict__ positions, const int* __restrict__ token_req,
                                 const int* __restrict__ req_first_position, T* __restrict__ out, int ldo, int act) {
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = token_req[t];
  if (r < 0 || c >= C) return;
  const int i = positions[t] - req_first_position[r];   // rows of this run before t
  const int slot = slots[r];
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  state = after_wait(state);
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    float v;
    if (j <= i) v = to_f(in[(size_t)(t - j) * ldi + c]);
    else v = state[((size_t)slot * (taps - 1) + (taps - 1 + i - j)) * C + c];
    acc = fmaf(w[(size_t)c * taps + taps - 1 - j], v, acc);
  }
  out[(size_t)t * ldo + c] = from_f<T>(act ? silu_f(acc) : acc);
}

// The same with VEC = 16 / sizeof(T) neighbouring channels a thread and 16-byte accesses (C, the strides and the
// bases must allow them); a channel's taps are added in the same order, so the results are the same bits.  It
// reads the weights tap by tap ([taps, C]: neighbouring channels side by side), a copy the caller keeps.
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) { unpack8(*reinterpret_cast<const uint4*>(p), v); }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) { *reinterpret_cast<uint4*>(p) = pack8(v); }
};

template <typename T>
__global__ void conv_silu_vec_kernel(const T* in, int ldi, const float* __restrict__ wt, const float* __restrict__ bias,
                                     int taps, int C, const float* state, const int* __restrict__ slots,
                                     const int* __restrict__ positions, const int* __restrict__ token_req,
                                     const int* __restrict__ req_first_position, T* __restrict__ out, int ldo, int act) {
  constexpr int VEC = Vec16<T>::N;
  const int t = blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int r = token_req[t];
  if (r < 0 || c >= C) return;
  const int i = positions[t] - req_first_position[r];
  const int slot = slots[r];
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  state = after_wait(state);
  float acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = bias ? bias[c + e] : 0.f;
  for (int j = 0; j < taps; ++j) {
    float v[VEC];
    if (j <= i) {
      Vec16<T>::load(in + (size_t)(t - j) * ldi + c, v);
    } else {
      const float* sp = state + ((size_t)slot * (taps - 1) + (taps - 1 + i - j)) * C + c;
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {
        const float4 q = *reinterpret_cast<const float4*>(sp + e);
        v[e] = q.x; v[e + 1] = q.y; v[e + 2] = q.z; v[e + 3] = q.w;
      }
    }
    const float* wp = wt + (size_t)(taps - 1 - j) * C + c;
#pragma unroll
    for (int e = 0; e < VEC; e += 4) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(wp + e));
      acc[e] = fmaf(q.x, v[e], acc[e]);
      acc[e + 1] = fmaf(q.y, v[e + 1], acc[e + 1]);
      acc[e + 2] = fmaf(q.z, v[e + 2], acc[e + 2]);
      acc[e + 3] = fmaf(q.w, v[e + 3], acc[e + 3]);
    }
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = act ? silu_f(acc[e]) : acc[e];
  Vec16<T>::store(out + (size_t)t * ldo + c, acc);
}

template <typename T>
__global__ void conv_state_update_kernel(const T* in, int ldi, int taps, int C, float* state,
                                         const int* __restrict__ slots, const int* __restrict__ token_req,
                                         const int* __restrict__ req_first_token) {
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = req_first_token[r], t1 = req_first_token[r + 1];
  const int n = request_rows(token_req, t0, t1, r);
  if (n == 0 || c >= C) return;
  const int keep = taps - 1;
  float* st = state + (size_t)slots[r] * keep * C + c;
  float nv[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    if (s < keep) {
      const int li = n - keep + s;
      nv[s] = li >= 0 ? to_f(in[(size_t)(t0 + li) * ldi + c]) : st[(size_t)(s + n) * C];
    }
  }
#pragma unroll
  for (int s = 0; s < 8; ++s)
    if (s < keep) st[(size_t)s * C] = nv[s];
}

template <typename T>
static int conv_launch(const void* in, int ldi, const float* w, const float* wt, const float* bias, int taps, int C, float* state,
                       const int* slots, const int* positions, const int* token_req, const int* req_first_token,
                       const int* req_first_position, void* out, int ldo, int n_tokens, int n_requests,
                       int act, cudaStream_t stream) {
  const int threads = 128;
  constexpr int VEC = 16 / (int)sizeof(T);
  // (with few rows the launch is a matter of latency, and more, lighter threads are the quicker: decode steps of
  // up to 31 rows keep one channel a thread; the results are the same bits either way)
  const bool vec = wt != nullptr && n_tokens >= 32 && C % VEC == 0 && ldi % VEC == 0 && ldo % VEC == 0 && C % 4 == 0 &&
                   (((uintptr_t)in | (uintptr_t)out | (uintptr_t)state | (uintptr_t)wt) & 15) == 0;
  if (vec) {
    const int tv = C / VEC >= 128 ? 128 : 64;
    launch_pdl(conv_silu_vec_kernel<T>, dim3((C / VEC + tv - 1) / tv, n_tokens), dim3(tv), 0, stream, (const T*)in, ldi,
               wt, bias, taps, C, (const float*)state, slots, positions, token_req, req_first_position, (T*)out, ldo, act);
  } else {
    launch_pdl(conv_silu_kernel<T>, dim3((C + threads - 1) / threads, n_tokens), dim3(threads), 0, stream, (const T*)in,
               ldi, w, bias, taps, C, (const float*)state, slots, positions, token_req, req_first_position, (T*)out, ldo, act);
  }
  if (int e = mlxb_check_launch("conv_silu")) return e;
  if (taps == 1) return 0;          // nothing of earlier tokens is read: no state
  launch_pdl(conv_state_update_kernel<T>, dim3((C + threads - 1) / threads, n_requests), dim3(threads), 0, stream,
             (const T*)in, ldi, taps, C, state, slots, token_req, req_first_token);
  return mlxb_check_launch("conv_state_update");
}

// in: [n_tokens, >= C] at row stride ldi (activation dtype); w: float32 [C, taps]; wt: the same tap by tap, float32
// [taps, C], or null (with it, and sizes that allow 16-byte accesses, the vector kernel runs); bias: float32 [C] or null;
// state: float32 [slots, taps-1, C]; out: [n_tokens, C] at row stride ldo; act: 1 silu, 0 none.  Two launches: the convolution, then the
// state's update (which must not overtake the convolution's reads of the state).
MLXB_EXPORT int mlxb_conv_silu(int dtype, const void* in, int ldi, const float* w, const float* wt, const float* bias, int taps, int C,
                               float* state, const int* slots, const int* positions, const int* token_req,
                               const int* req_first_token, const int* req_first_position, void* out, int ldo,
                               int n_tokens, int n_requests, int act, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return 0;
  if (taps < 1 || taps > 9 || C <= 0 || ldi < C || ldo < C || n_tokens > 65535 * 32 || n_requests > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "conv: %d taps (1..9), %d channels, strides %d / %d, %d tokens of %d requests", taps, C,
                     ldi, ldo, n_tokens, n_requests);
  if (n_tokens > 65535) return mlxb_fail(MLXB_BAD_ARG, "conv: %d tokens are too many for one call", n_tokens);
  if (dtype == MLXB_F32)
    return conv_launch<float>(in, ldi, w, wt, bias, taps, C, state, slots, positions, token_req, req_first_token,
                              req_first_position, out, ldo, n_tokens, n_requests, act, stream);
  if (dtype == MLXB_BF16)
    return conv_launch<__nv_bfloat16>(in, ldi, w, wt, bias, taps, C, state, slots, positions, token_req, req_first_token,
                                      req_first_position, out, ldo, n_tokens, n_requests, act, stream);
  return mlxb_fail(MLXB_BAD_DTYPE, "conv: dtype code %d", dtype);
}

// ---------------------------------------------------------------- scans

constexpr int SCAN_NPT = 16;               // consecutive rows of a state column a thread holds
constexpr int SCAN_SEG = SCAN_NPT + 4;     // floats such a run of 16 inputs takes in shared memory: 4 of padding, so that
                                           // the 16-byte loads of a warp's threads fall on different banks
constexpr int SCAN_CHUNK = 16;             // tokens staged at a time

struct ScanShape {
  int NS, VB, threads, zblocks;
};

// n_rows: rows of the state (N or K); V: its columns; pairs: (request, head) pairs of the launch.  A block takes all
// columns of a pair when there are pairs enough to fill the SMs; with fewer the columns are cut into several
// blocks, each of which stages the pair's inputs for itself, but never below four warps a block.
static inline ScanShape scan_shape(int n_rows, int V, long long pairs) {
  ScanShape s;
  s.NS = 1;
  while (s.NS * SCAN_NPT < n_rows) s.NS <<= 1;
  const int lanes = 32 / s.NS;                       // columns per warp
  const int vmax = 512 / s.NS;                       // columns per block at most
  int vb = (V + lanes - 1) / lanes * lanes;
  if (vb > vmax) vb = vmax;
  const long long want = mlxb_sm_count();
  while (vb > lanes && pairs * ((V + vb - 1) / vb) < want) {
    int half = (vb / 2 + lanes - 1) / lanes * lanes;
    if (half >= vb || half * s.NS < 128) break;
    vb = half;
  }
  s.VB = vb;
  s.threads = vb * s.NS;
  s.zblocks = (V + vb - 1) / vb;
  return s;
}

// where row nn of a token's staged vector lies: runs of SCAN_NPT rows, SCAN_SEG floats apart
__device__ __forceinline__ int seg_index(int nn) { return (nn / SCAN_NPT) * SCAN_SEG + (nn % SCAN_NPT); }

__device__ __forceinline__ void load16(const float* p, float (&v)[SCAN_NPT]) {
#pragma unroll
  for (int j = 0; j < SCAN_NPT / 4; ++j) {
    const float4 q = reinterpret_cast<const float4*>(p)[j];
    v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
  }
}

// A thread's 16 rows of its column, to and from the pool.  The pool keeps a head's state column by column
// ([V][rows]: a thread's rows are consecutive floats, a warp's threads read neighbouring runs), so that a decode
// step, which is little more than reading and writing every state once, moves whole 16-byte pieces.
__device__ __forceinline__ void state_load(const float* col, int first, int n_rows, bool valid, float (&S)[SCAN_NPT]) {
  if ((n_rows & 3) == 0) {
#pragma unroll
    for (int j = 0; j < SCAN_NPT / 4; ++j) {
      float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid && first + 4 * j < n_rows) q = *reinterpret_cast<const float4*>(col + first + 4 * j);
      S[4 * j] = q.x; S[4 * j + 1] = q.y; S[4 * j + 2] = q.z; S[4 * j + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < SCAN_NPT; ++i) S[i] = (valid && first + i < n_rows) ? col[first + i] : 0.f;
  }
}
__device__ __forceinline__ void state_store(float* col, int first, int n_rows, bool valid, const float (&S)[SCAN_NPT]) {
  if (!valid) return;
  if ((n_rows & 3) == 0) {
#pragma unroll
    for (int j = 0; j < SCAN_NPT / 4; ++j)
      if (first + 4 * j < n_rows)
        *reinterpret_cast<float4*>(col + first + 4 * j) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < SCAN_NPT; ++i)
      if (first + i < n_rows) col[first + i] = S[i];
  }
}

// Thread (s, v) holds rows 16 s .. 16 s + 15 of column v of the state; rows beyond the state's own stay zero (their
// staged inputs are zeros).  NS threads (neighbouring lanes) share a column.
template <typename T, int NS>
__global__ void __launch_bounds__(512, 1)
mamba2_scan_kernel(const T* xbc, int ldx, int x_off, int b_off, int c_off, const T* dt_raw, int lddt,
                   const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                   const float* __restrict__ Dskip, float* state, const int* __restrict__ slots,
                   const int* __restrict__ token_req, const int* __restrict__ req_first_token, float* __restrict__ y,
                   int ldy, int H, int G, int N, int V, int VB) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NP = NS * SCAN_SEG;        // floats of a token's staged B (or C)
  float* sB = sm;                          // [CHUNK][NP]
  float* sC = sB + SCAN_CHUNK * NP;        // [CHUNK][NP]
  float* sx = sC + SCAN_CHUNK * NP;        // [CHUNK][VB]
  float* sdt = sx + SCAN_CHUNK * VB;       // [CHUNK]
  float* sa = sdt + SCAN_CHUNK;            // [CHUNK]
  const int h = blockIdx.x, r = blockIdx.y, vb = blockIdx.z;
  const int t0 = req_first_token[r], t1 = req_first_token[r + 1];
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int s = tid % NS, vl = tid / NS, v = vb * VB + vl;
  const bool valid = v < V;
  const int g = h / (H / G);
  // The state was last written by a step before this one (a cache is touched by one launch a step), so it can
  // be on its way before the wait for the kernel that wrote this step's inputs.
  float* st = state + ((size_t)slots[r] * H + h) * N * V + (size_t)(valid ? v : 0) * N;   // this thread's column
  float S[SCAN_NPT];
  state_load(st, s * SCAN_NPT, N, valid, S);
  pdl_wait();
  pdl_trigger();
  xbc = after_wait(xbc);
  dt_raw = after_wait(dt_raw);
  const int n = request_rows(token_req, t0, t1, r);
  if (n == 0) return;
  const float negA = -expf(A_log[h]), skip = Dskip[h], bias = dt_bias[h];
  for (int c0 = 0; c0 < n; c0 += SCAN_CHUNK) {
    const int nc = min(SCAN_CHUNK, n - c0);
    __syncthreads();
    // eight elements a thread at a time: their loads go out together, then the stores (one element per
    // iteration would wait for memory once per element)
    for (int base = tid; base < nc * NS * SCAN_NPT; base += nthreads * 8) {
      T bq[8], cq[8];
      int at[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int idx = base + j * nthreads;
        const int tt = idx / (NS * SCAN_NPT), nn = idx - tt * (NS * SCAN_NPT);
        at[j] = (idx < nc * NS * SCAN_NPT && nn < N) ? tt * NP + seg_index(nn) : -1 - (tt * NP + seg_index(nn));
        if (at[j] >= 0) {
          const T* row = xbc + (size_t)(t0 + c0 + tt) * ldx;
          bq[j] = row[b_off + g * N + nn];
          cq[j] = row[c_off + g * N + nn];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int idx = base + j * nthreads;
        if (idx < nc * NS * SCAN_NPT) {
          const int pos = at[j] >= 0 ? at[j] : -1 - at[j];
          sB[pos] = at[j] >= 0 ? to_f(bq[j]) : 0.f;
          sC[pos] = at[j] >= 0 ? to_f(cq[j]) : 0.f;
        }
      }
    }
    for (int idx = tid; idx < nc * VB; idx += nthreads) {
      const int tt = idx / VB, vv = idx - tt * VB, col = vb * VB + vv;
      sx[idx] = col < V ? to_f(xbc[(size_t)(t0 + c0 + tt) * ldx + x_off + h * V + col]) : 0.f;
    }
    for (int tt = tid; tt < nc; tt += nthreads) {
      const float d = softplus_f(to_f(dt_raw[(size_t)(t0 + c0 + tt) * lddt + h]) + bias);
      sdt[tt] = d;
      sa[tt] = expf(negA * d);
    }
    __syncthreads();
    // Four tokens at a time: the state's update of a token needs only the update before it (one multiply-add
    // deep), while a token's read-out ends in a chain of shuffles; the four read-outs of a group are reduced
    // together, so that their latencies overlap instead of adding up.
    for (int tt0 = 0; tt0 < nc; tt0 += 4) {
      float acc[4], xs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int tt = tt0 + u;
        const bool in = tt < nc;
        const int tc = in ? tt : tt0;
        const float a = in ? sa[tc] : 1.f, xv = sx[tc * VB + vl], dtx = in ? sdt[tc] * xv : 0.f;   // beyond the chunk: S stays
        float bv[SCAN_NPT], cv[SCAN_NPT];
        load16(sB + tc * NP + s * SCAN_SEG, bv);
        load16(sC + tc * NP + s * SCAN_SEG, cv);
        float acc0 = 0.f, acc1 = 0.f;    // two chains, added at the end: even and odd rows of the thread's share
#pragma unroll
        for (int i = 0; i < SCAN_NPT; ++i) {
          S[i] = fmaf(a, S[i], dtx * bv[i]);
          if (i & 1) acc1 = fmaf(S[i], cv[i], acc1);
          else acc0 = fmaf(S[i], cv[i], acc0);
        }
        acc[u] = acc0 + acc1;
        xs[u] = xv;
      }
#pragma unroll
      for (int o = NS >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (s == 0 && valid && tt0 + u < nc) y[(size_t)(t0 + c0 + tt0 + u) * ldy + h * V + v] = fmaf(skip, xs[u], acc[u]);
    }
  }
  state_store(st, s * SCAN_NPT, N, valid, S);
}

// xbc: the convolution's output [n_tokens, ...] (activation dtype) holding x (H*V columns from x_off), B and C (G*N
// columns each from b_off / c_off); dt_raw: [n_tokens, >= H] at row stride lddt; state: float32 [slots, H, V, N] (column by column);
// y: float32 [n_tokens, H*V] at row stride ldy.
MLXB_EXPORT int mlxb_mamba2_scan(int dtype, const void* xbc, int ldx, int x_off, int b_off, int c_off,
                                 const void* dt_raw, int lddt, const float* dt_bias, const float* A_log,
                                 const float* Dskip, float* state, const int* slots, const int* token_req,
                                 const int* req_first_token, float* y, int ldy, int H, int G, int N, int V,
                                 int n_requests, cudaStream_t stream) {
  if (n_requests <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || N <= 0 || V <= 0 || N > 32 * SCAN_NPT || n_requests > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "mamba2_scan: %d heads in %d groups, state %d x %d (at most %d rows)", H, G, N, V,
                     32 * SCAN_NPT);
  const ScanShape sh = scan_shape(N, V, (long long)H * n_requests);
  const size_t smem = (size_t)(SCAN_CHUNK * (2 * sh.NS * SCAN_SEG + sh.VB + 2)) * sizeof(float);
  const dim3 grid(H, n_requests, sh.zblocks);
  if (dtype != MLXB_F32 && dtype != MLXB_BF16) return mlxb_fail(MLXB_BAD_DTYPE, "mamba2_scan: dtype code %d", dtype);
  cudaError_t e = cudaSuccess;
#define M2_GO(T_, NS_)                                                                                                   \
  {                                                                                                                      \
    static size_t allowed = 48 * 1024;   /* per kernel: raised once, outside any stream capture that comes later */     \
    if (smem > allowed) {                                                                                                \
      e = cudaFuncSetAttribute(mamba2_scan_kernel<T_, NS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
      if (e == cudaSuccess) allowed = smem;                                                                              \
    }                                                                                                                    \
    if (e == cudaSuccess)                                                                                                \
      launch_pdl(mamba2_scan_kernel<T_, NS_>, grid, dim3(sh.threads), smem, stream, (const T_*)xbc, ldx, x_off, b_off,   \
                 c_off, (const T_*)dt_raw, lddt, dt_bias, A_log, Dskip, state, slots, token_req, req_first_token, y,     \
                 ldy, H, G, N, V, sh.VB);                                                                                \
  }
#define M2_NS(NS_) { if (dtype == MLXB_F32) M2_GO(float, NS_) else M2_GO(__nv_bfloat16, NS_) }
  switch (sh.NS) {
    case 1: M2_NS(1) break;
    case 2: M2_NS(2) break;
    case 4: M2_NS(4) break;
    case 8: M2_NS(8) break;
    case 16: M2_NS(16) break;
    default: M2_NS(32) break;
  }
#undef M2_NS
#undef M2_GO
  if (e != cudaSuccess) return mlxb_fail((int)e, "mamba2_scan: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  return mlxb_check_launch("mamba2_scan");
}

template <typename T, int NS>
__global__ void __launch_bounds__(512, 1)
gated_delta_scan_kernel(const T* qkv, int ldq, int q_off, int k_off, int v_off, const T* b_raw, int ldb,
                        const T* a_raw, int lda, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                        float* state, const int* __restrict__ slots, const int* __restrict__ token_req,
                        const int* __restrict__ req_first_token, float* __restrict__ o, int ldo, int H, int G, int K,
                        int V, int VB) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NP = NS * SCAN_SEG;        // floats of a token's staged q (or k)
  float* sq = sm;                          // [CHUNK][NP]
  float* sk = sq + SCAN_CHUNK * NP;        // [CHUNK][NP]
  float* sv = sk + SCAN_CHUNK * NP;        // [CHUNK][VB]
  float* sbeta = sv + SCAN_CHUNK * VB;     // [CHUNK]
  float* sg = sbeta + SCAN_CHUNK;          // [CHUNK]
  const int h = blockIdx.x, r = blockIdx.y, vb = blockIdx.z;
  const int t0 = req_first_token[r], t1 = req_first_token[r + 1];
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
  const int s = tid % NS, vl = tid / NS, v = vb * VB + vl;
  const bool valid = v < V;
  const int g = h / (H / G);
  // older than this step (see mamba2_scan_kernel): asked for before the wait
  float* st = state + ((size_t)slots[r] * H + h) * K * V + (size_t)(valid ? v : 0) * K;   // this thread's column
  float S[SCAN_NPT];
  state_load(st, s * SCAN_NPT, K, valid, S);
  pdl_wait();
  pdl_trigger();
  qkv = after_wait(qkv);
  b_raw = after_wait(b_raw);
  a_raw = after_wait(a_raw);
  const int n = request_rows(token_req, t0, t1, r);
  if (n == 0) return;
  const float negA = -expf(A_log[h]), bias = dt_bias[h], q_scale = 1.f / sqrtf((float)K);
  for (int c0 = 0; c0 < n; c0 += SCAN_CHUNK) {
    const int nc = min(SCAN_CHUNK, n - c0);
    __syncthreads();
    // eight elements a thread at a time: their loads go out together, then the stores
    for (int base = tid; base < nc * NS * SCAN_NPT; base += nthreads * 8) {
      T qq[8], kq[8];
      int at[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int idx = base + j * nthreads;
        const int tt = idx / (NS * SCAN_NPT), kk = idx - tt * (NS * SCAN_NPT);
        at[j] = (idx < nc * NS * SCAN_NPT && kk < K) ? tt * NP + seg_index(kk) : -1 - (tt * NP + seg_index(kk));
        if (at[j] >= 0) {
          const T* row = qkv + (size_t)(t0 + c0 + tt) * ldq;
          qq[j] = row[q_off + g * K + kk];
          kq[j] = row[k_off + g * K + kk];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int idx = base + j * nthreads;
        if (idx < nc * NS * SCAN_NPT) {
          const int pos = at[j] >= 0 ? at[j] : -1 - at[j];
          sq[pos] = at[j] >= 0 ? to_f(qq[j]) : 0.f;
          sk[pos] = at[j] >= 0 ? to_f(kq[j]) : 0.f;
        }
      }
    }
    for (int idx = tid; idx < nc * VB; idx += nthreads) {
      const int tt = idx / VB, vv = idx - tt * VB, col = vb * VB + vv;
      sv[idx] = col < V ? to_f(qkv[(size_t)(t0 + c0 + tt) * ldq + v_off + h * V + col]) : 0.f;
    }
    for (int tt = tid; tt < nc; tt += nthreads) {
      const size_t row = (size_t)(t0 + c0 + tt);
      sbeta[tt] = 1.f / (1.f + expf(-to_f(b_raw[row * ldb + h])));
      sg[tt] = expf(negA * softplus_f(to_f(a_raw[row * lda + h]) + bias));
    }
    __syncthreads();
    for (int tt = warp; tt < nc; tt += nwarps) {     // a warp per token: q and k of the head become unit vectors
      float q2 = 0.f, k2 = 0.f;
      for (int kk = lane; kk < K; kk += 32) {
        const float qv = sq[tt * NP + seg_index(kk)], kv = sk[tt * NP + seg_index(kk)];
        q2 = fmaf(qv, qv, q2);
        k2 = fmaf(kv, kv, k2);
      }
      q2 = warp_sum(q2);
      k2 = warp_sum(k2);
      const float rq = q_scale / sqrtf(q2 + 1e-6f), rk = 1.f / sqrtf(k2 + 1e-6f);
      for (int kk = lane; kk < K; kk += 32) {
        sq[tt * NP + seg_index(kk)] *= rq;
        sk[tt * NP + seg_index(kk)] *= rk;
      }
    }
    __syncthreads();
    // Four tokens at a time.  What the next token waits for is this token's write to S, and that needs the reduced
    // S^T k; the read-out S^T q is only written out, so its shuffles are put off to the end of the group, where
    // the four of them overlap.
    for (int tt0 = 0; tt0 < nc; tt0 += 4) {
      float outs[4];
#pragma unroll
      for (int w4 = 0; w4 < 4; ++w4) {
        const int tt = tt0 + w4;
        const bool in = tt < nc;
        const int tc = in ? tt : tt0;
        const float gg = in ? sg[tc] : 1.f, beta = in ? sbeta[tc] : 0.f, vv = sv[tc * VB + vl];   // beyond the chunk: S stays
        float kr[SCAN_NPT], qr[SCAN_NPT];
        load16(sk + tc * NP + s * SCAN_SEG, kr);
        load16(sq + tc * NP + s * SCAN_SEG, qr);
        float acc0 = 0.f, acc1 = 0.f;      // two chains each, added at the end
#pragma unroll
        for (int i = 0; i < SCAN_NPT; ++i) {
          S[i] *= gg;
          if (i & 1) acc1 = fmaf(S[i], kr[i], acc1);
          else acc0 = fmaf(S[i], kr[i], acc0);
        }
        float acc = acc0 + acc1;
#pragma unroll
        for (int w = NS >> 1; w > 0; w >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
        const float u = beta * (vv - acc);
        float out0 = 0.f, out1 = 0.f;
#pragma unroll
        for (int i = 0; i < SCAN_NPT; ++i) {
          S[i] = fmaf(kr[i], u, S[i]);
          if (i & 1) out1 = fmaf(S[i], qr[i], out1);
          else out0 = fmaf(S[i], qr[i], out0);
        }
        outs[w4] = out0 + out1;
      }
#pragma unroll
      for (int w = NS >> 1; w > 0; w >>= 1) {
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) outs[w4] += __shfl_xor_sync(0xffffffffu, outs[w4], w);
      }
#pragma unroll
      for (int w4 = 0; w4 < 4; ++w4)
        if (s == 0 && valid && tt0 + w4 < nc) o[(size_t)(t0 + c0 + tt0 + w4) * ldo + h * V + v] = outs[w4];
    }
  }
  state_store(st, s * SCAN_NPT, K, valid, S);
}

// qkv: the convolutions' output [n_tokens, ...] (activation dtype): q and k (G*K columns each from q_off / k_off),
// v (H*V columns from v_off); b_raw, a_raw: [n_tokens, >= H] at row strides ldb / lda; state: float32 [slots, H, V, K] (column by column);
// o: float32 [n_tokens, H*V] at row stride ldo.
MLXB_EXPORT int mlxb_gated_delta_scan(int dtype, const void* qkv, int ldq, int q_off, int k_off, int v_off,
                                      const void* b_raw, int ldb, const void* a_raw, int lda, const float* dt_bias,
                                      const float* A_log, float* state, const int* slots, const int* token_req,
                                      const int* req_first_token, float* o, int ldo, int H, int G, int K, int V,
                                      int n_requests, cudaStream_t stream) {
  if (n_requests <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || K <= 0 || V <= 0 || K > 32 * SCAN_NPT || n_requests > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "gated_delta_scan: %d heads over %d key heads, state %d x %d (at most %d rows)", H, G,
                     K, V, 32 * SCAN_NPT);
  const ScanShape sh = scan_shape(K, V, (long long)H * n_requests);
  const size_t smem = (size_t)(SCAN_CHUNK * (2 * sh.NS * SCAN_SEG + sh.VB + 2)) * sizeof(float);
  const dim3 grid(H, n_requests, sh.zblocks);
  if (dtype != MLXB_F32 && dtype != MLXB_BF16) return mlxb_fail(MLXB_BAD_DTYPE, "gated_delta_scan: dtype code %d", dtype);
  cudaError_t e = cudaSuccess;
#define GD_GO(T_, NS_)                                                                                                    \
  {                                                                                                                       \
    static size_t allowed = 48 * 1024;                                                                                    \
    if (smem > allowed) {                                                                                                 \
      e = cudaFuncSetAttribute(gated_delta_scan_kernel<T_, NS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess) allowed = smem;                                                                               \
    }                                                                                                                     \
    if (e == cudaSuccess)                                                                                                 \
      launch_pdl(gated_delta_scan_kernel<T_, NS_>, grid, dim3(sh.threads), smem, stream, (const T_*)qkv, ldq, q_off,      \
                 k_off, v_off, (const T_*)b_raw, ldb, (const T_*)a_raw, lda, dt_bias, A_log, state, slots, token_req,     \
                 req_first_token, o, ldo, H, G, K, V, sh.VB);                                                             \
  }
#define GD_NS(NS_) { if (dtype == MLXB_F32) GD_GO(float, NS_) else GD_GO(__nv_bfloat16, NS_) }
  switch (sh.NS) {
    case 1: GD_NS(1) break;
    case 2: GD_NS(2) break;
    case 4: GD_NS(4) break;
    case 8: GD_NS(8) break;
    case 16: GD_NS(16) break;
    default: GD_NS(32) break;
  }
#undef GD_NS
#undef GD_GO
  if (e != cudaSuccess) return mlxb_fail((int)e, "gated_delta_scan: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  return mlxb_check_launch("gated_delta_scan");
}
