// Dynamic Tanh: a norm without statistics, and the update of a float32 residual stream through it.
//
// dyt_norm      out[r, c] = (tanh(alpha * x[row(r), c]) * w[c] + b[c]) * out_scale
//               x is float32, the result has the activation dtype (or float32); `alpha` is one float32 number in
//               device memory, w and b float32 [D] (b may be null); rows: int32 list of source rows or null.
// dyt_residual  y[t, c]  = sum over k < terms of branch[t * terms + k, c]        (added in the order of k)
//               x[t, c] += tanh(alpha * y[t, c]) * w[c] + b[c]                    (with w null: x += y)
//               next[t, c] = tanh(alpha2 * x[t, c]) * w2[c] + b2[c]               (optional: the norm of the
//               sublayer that reads the stream next, in the activation dtype, so that it costs no launch)
//               branch is float32 [T * terms, D]: what a sublayer's last product wrote; with terms > 1 a token's
//               rows are the results of the experts it was routed to.
// All arithmetic is float32 (tanhf).  Rows whose token_req is negative (they pad a step) are skipped by
// dyt_residual where token_req is given.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

template <typename TO>
__device__ __forceinline__ void store4(TO* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&a);
  u.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// VEC: four columns a thread (D, the strides and the bases allow 16-byte accesses), else one.
template <typename TO, int VEC>
__global__ void dyt_norm_kernel(const float* x, int ldx, const int* __restrict__ rows, int n_src_rows,
                                const float* __restrict__ alpha, const float* __restrict__ w,
                                const float* __restrict__ b, float out_scale, TO* __restrict__ out, int ldo, int D,
                                int R) {
  const float a = alpha[0];
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  const int per_row = D / VEC;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)R * per_row) return;
  const int r = (int)(idx / per_row), c = (int)(idx - (long long)r * per_row) * VEC;
  const int src = rows ? rows[r] : r;
  float v[VEC];
  if (src < 0 || src >= n_src_rows) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = 0.f;
  } else {
    const float* xr = x + (size_t)src * ldx + c;
    if (VEC == 4) {
      const float4 u = *reinterpret_cast<const float4*>(xr);
      v[0] = u.x; v[VEC > 1 ? 1 : 0] = u.y; v[VEC > 2 ? 2 : 0] = u.z; v[VEC > 3 ? 3 : 0] = u.w;
    } else {
      v[0] = xr[0];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = (tanhf(a * v[e]) * w[c + e] + (b ? b[c + e] : 0.f)) * out_scale;
  }
  TO* o = out + (size_t)r * ldo + c;
  if (VEC == 4) {
    float q[4] = {v[0], v[VEC > 1 ? 1 : 0], v[VEC > 2 ? 2 : 0], v[VEC > 3 ? 3 : 0]};
    store4<TO>(o, q);
  } else {
    o[0] = from_f<TO>(v[0]);
  }
}

MLXB_EXPORT int mlxb_dyt_norm(int out_dtype, const float* x, int ldx, const int* rows, int n_src_rows,
                              const float* alpha, const float* w, const float* b, float out_scale, void* out, int ldo,
                              int R, int D, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || ldx < D || ldo < D || !alpha || !w)
    return mlxb_fail(MLXB_BAD_ARG, "dyt_norm: width %d, strides %d / %d", D, ldx, ldo);
  const int osz = out_dtype == MLXB_F32 ? 4 : 2;
  const bool vec = D % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)x & 15) == 0 &&
                   ((uintptr_t)out & (4 * osz - 1)) == 0 && ((uintptr_t)w & 15) == 0;
  const int threads = 256;
  const long long total = (long long)R * (vec ? D / 4 : D);
  const dim3 grid((unsigned)((total + threads - 1) / threads));
#define DYT_GO(TO, V)                                                                                                 \
  launch_pdl(dyt_norm_kernel<TO, V>, grid, dim3(threads), 0, stream, x, ldx, rows, n_src_rows, alpha, w, b, out_scale, \
             (TO*)out, ldo, D, R)
  if (out_dtype == MLXB_F32) { if (vec) DYT_GO(float, 4); else DYT_GO(float, 1); }
  else if (out_dtype == MLXB_BF16) { if (vec) DYT_GO(__nv_bfloat16, 4); else DYT_GO(__nv_bfloat16, 1); }
  else return mlxb_fail(MLXB_BAD_DTYPE, "dyt_norm: dtype code %d", out_dtype);
#undef DYT_GO
  return mlxb_check_launch("dyt_norm");
}

template <typename TO, int VEC>
__global__ void dyt_residual_kernel(float* x, int ldx, const float* branch, int ldb, int terms,
                                    const int* __restrict__ token_req, const float* __restrict__ alpha,
                                    const float* __restrict__ w, const float* __restrict__ b,
                                    const float* __restrict__ alpha2, const float* __restrict__ w2,
                                    const float* __restrict__ b2, TO* __restrict__ next, int ldn, int D, int T) {
  const float a = w ? alpha[0] : 0.f, a2 = next ? alpha2[0] : 0.f;
  const int per_row = D / VEC;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = idx < (long long)T * per_row;
  const int t = live ? (int)(idx / per_row) : 0, c = live ? (int)(idx - (long long)t * per_row) * VEC : 0;
  float wv[VEC], bv[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    wv[e] = (live && w) ? w[c + e] : 1.f;
    bv[e] = (live && w && b) ? b[c + e] : 0.f;
  }
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  branch = after_wait(branch);
  if (!live || (token_req && token_req[t] < 0)) return;
  float y[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) y[e] = 0.f;
  for (int k = 0; k < terms; ++k) {
    const float* br = branch + ((size_t)t * terms + k) * ldb + c;
    if (VEC == 4) {
      const float4 u = *reinterpret_cast<const float4*>(br);
      y[0] += u.x; y[VEC > 1 ? 1 : 0] += u.y; y[VEC > 2 ? 2 : 0] += u.z; y[VEC > 3 ? 3 : 0] += u.w;
    } else {
      y[0] += br[0];
    }
  }
  float* xr = x + (size_t)t * ldx + c;
  float v[VEC];
  if (VEC == 4) {
    const float4 u = *reinterpret_cast<const float4*>(xr);
    v[0] = u.x; v[VEC > 1 ? 1 : 0] = u.y; v[VEC > 2 ? 2 : 0] = u.z; v[VEC > 3 ? 3 : 0] = u.w;
  } else {
    v[0] = xr[0];
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) v[e] += w ? tanhf(a * y[e]) * wv[e] + bv[e] : y[e];
  if (VEC == 4) *reinterpret_cast<float4*>(xr) = make_float4(v[0], v[VEC > 1 ? 1 : 0], v[VEC > 2 ? 2 : 0], v[VEC > 3 ? 3 : 0]);
  else xr[0] = v[0];
  if (next) {
    float q[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int e = 0; e < VEC; ++e) q[e] = tanhf(a2 * v[e]) * w2[c + e] + (b2 ? b2[c + e] : 0.f);
    TO* o = next + (size_t)t * ldn + c;
    if (VEC == 4) store4<TO>(o, q);
    else o[0] = from_f<TO>(q[0]);
  }
}

MLXB_EXPORT int mlxb_dyt_residual(int next_dtype, float* x, int ldx, const float* branch, int ldb, int terms,
                                  const int* token_req, const float* alpha, const float* w, const float* b,
                                  const float* alpha2, const float* w2, const float* b2, void* next, int ldn, int T,
                                  int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0 || ldx < D || ldb < D || terms <= 0 || (w && !alpha) || (next && (!alpha2 || !w2 || ldn < D)))
    return mlxb_fail(MLXB_BAD_ARG, "dyt_residual: width %d, %d terms, strides %d / %d / %d", D, terms, ldx, ldb, ldn);
  const int osz = next_dtype == MLXB_F32 ? 4 : 2;
  const bool vec = D % 4 == 0 && ldx % 4 == 0 && ldb % 4 == 0 && (!next || ldn % 4 == 0) && ((uintptr_t)x & 15) == 0 &&
                   ((uintptr_t)branch & 15) == 0 && ((uintptr_t)next & (4 * osz - 1)) == 0;
  const int threads = 256;
  const long long total = (long long)T * (vec ? D / 4 : D);
  const dim3 grid((unsigned)((total + threads - 1) / threads));
#define DYTR_GO(TO, V)                                                                                                 \
  launch_pdl(dyt_residual_kernel<TO, V>, grid, dim3(threads), 0, stream, x, ldx, branch, ldb, terms, token_req, alpha, \
             w, b, alpha2, w2, b2, (TO*)next, ldn, D, T)
  if (next_dtype == MLXB_F32) { if (vec) DYTR_GO(float, 4); else DYTR_GO(float, 1); }
  else if (next_dtype == MLXB_BF16) { if (vec) DYTR_GO(__nv_bfloat16, 4); else DYTR_GO(__nv_bfloat16, 1); }
  else return mlxb_fail(MLXB_BAD_DTYPE, "dyt_residual: dtype code %d", next_dtype);
#undef DYTR_GO
  return mlxb_check_launch("dyt_residual");
}
