// Root-mean-square norms over float32 rows, and the update of a float32 residual stream.
//
// rmsnorm          out[r, c] = x[row(r), c] / sqrt(mean_g(x^2) + eps) * (offset + w[c % period])
//                  The row is cut into `groups` equal parts, each divided by its own root mean square.
//                  The weight repeats with `period` columns (the width: one weight per column; the width
//                  of a part: the parts share one weight), is stored as it is (offset 0) or as its distance
//                  from one (offset 1).  A gate g (activation dtype) may come in: mode 1 multiplies x by
//                  silu(g) BEFORE the statistics, mode 2 multiplies the normed value by silu(g).
//                  x is float32; the result has the activation dtype.  All arithmetic is float32.
// residual_update  x[r, :] += scale * (f1(y1[r, :]) + f2(y2[r, :])),  f_i = rmsnorm with weight w_i over the
//                  whole row, or the identity where w_i is null; y2 may be null.  Optionally a copy of the new
//                  row in the activation dtype is left in `cast_out` for the products that read it next.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

template <typename TO>
__global__ void rmsnorm_kernel(const float* x, int ldx, const int* __restrict__ rows, int n_src_rows,
                               const float* __restrict__ w, float offset, int period, const TO* gate, int ldg,
                               int gate_mode, TO* __restrict__ out, int ldo, int D, int groups, float eps) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  gate = after_wait(gate);
  const int r = blockIdx.x, g = blockIdx.y;
  const int src = rows ? rows[r] : r;
  const int Dg = D / groups;
  TO* o = out + (size_t)r * ldo + (size_t)g * Dg;
  if (src < 0 || src >= n_src_rows) {
    for (int c = threadIdx.x; c < Dg; c += blockDim.x) o[c] = from_f<TO>(0.f);
    return;
  }
  const float* xr = x + (size_t)src * ldx + (size_t)g * Dg;
  const TO* gr = gate ? gate + (size_t)src * ldg + (size_t)g * Dg : nullptr;
  float s = 0.f;
  for (int c = threadIdx.x; c < Dg; c += blockDim.x) {
    float v = xr[c];
    if (gate_mode == 1) v *= silu_f(to_f(gr[c]));
    s = fmaf(v, v, s);
  }
  const float rinv = 1.f / sqrtf(block_sum(s, red) / (float)Dg + eps);
  for (int c = threadIdx.x; c < Dg; c += blockDim.x) {
    float v = xr[c];
    if (gate_mode == 1) v *= silu_f(to_f(gr[c]));
    v = v * rinv * (offset + w[(g * Dg + c) % period]);
    if (gate_mode == 2) v *= silu_f(to_f(gr[c]));
    o[c] = from_f<TO>(v);
  }
}

MLXB_EXPORT int mlxb_rmsnorm(int out_dtype, const float* x, int ldx, const int* rows, int n_src_rows, const float* w,
                             float offset, int period, const void* gate, int ldg, int gate_mode, void* out, int ldo,
                             int R, int D, int groups, float eps, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || groups <= 0 || D % groups || period <= 0 || ldx < D || ldo < D)
    return mlxb_fail(MLXB_BAD_ARG, "rmsnorm: width %d in %d parts, weight period %d, strides %d / %d", D, groups, period,
                     ldx, ldo);
  if (gate_mode < 0 || gate_mode > 2 || ((gate_mode != 0) != (gate != nullptr)))
    return mlxb_fail(MLXB_BAD_ARG, "rmsnorm: gate mode %d %s a gate", gate_mode, gate ? "with" : "without");
  if (groups > 65535) return mlxb_fail(MLXB_BAD_ARG, "rmsnorm: %d parts", groups);
  const int Dg = D / groups;
  const int threads = Dg >= 2048 ? 256 : (Dg >= 512 ? 128 : (Dg >= 128 ? 64 : 32));
  const dim3 grid(R, groups);
  if (out_dtype == MLXB_F32)
    launch_pdl(rmsnorm_kernel<float>, grid, dim3(threads), 0, stream, x, ldx, rows, n_src_rows, w, offset, period,
               (const float*)gate, ldg, gate_mode, (float*)out, ldo, D, groups, eps);
  else if (out_dtype == MLXB_BF16)
    launch_pdl(rmsnorm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, x, ldx, rows, n_src_rows, w, offset,
               period, (const __nv_bfloat16*)gate, ldg, gate_mode, (__nv_bfloat16*)out, ldo, D, groups, eps);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "rmsnorm: dtype code %d", out_dtype);
  return mlxb_check_launch("rmsnorm");
}

template <typename TO>
__global__ void residual_update_kernel(float* x, int ldx, const float* y1, const float* __restrict__ w1,
                                       const float* y2, const float* __restrict__ w2, int ldy, float scale, float eps,
                                       TO* __restrict__ cast_out, int ldc, int D) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  x = after_wait(x);
  y1 = after_wait(y1);
  y2 = after_wait(y2);
  const int r = blockIdx.x;
  float* xr = x + (size_t)r * ldx;
  const float* a = y1 + (size_t)r * ldy;
  const float* b = y2 ? y2 + (size_t)r * ldy : nullptr;
  float ra = 1.f, rb = 1.f;
  if (w1) {
    float s = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) s = fmaf(a[c], a[c], s);
    ra = 1.f / sqrtf(block_sum(s, red) / (float)D + eps);
  }
  if (b && w2) {
    float s = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) s = fmaf(b[c], b[c], s);
    rb = 1.f / sqrtf(block_sum(s, red) / (float)D + eps);
  }
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float v = w1 ? a[c] * ra * w1[c] : a[c];
    if (b) v += w2 ? b[c] * rb * w2[c] : b[c];
    const float nx = xr[c] + scale * v;
    xr[c] = nx;
    if (cast_out) cast_out[(size_t)r * ldc + c] = from_f<TO>(nx);
  }
}

MLXB_EXPORT int mlxb_residual_update(int cast_dtype, float* x, int ldx, const float* y1, const float* w1,
                                     const float* y2, const float* w2, int ldy, float scale, float eps, void* cast_out,
                                     int ldc, int R, int D, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || ldx < D || ldy < D || y1 == nullptr || (cast_out && ldc < D))
    return mlxb_fail(MLXB_BAD_ARG, "residual_update: width %d, strides %d / %d / %d", D, ldx, ldy, ldc);
  const int threads = D >= 2048 ? 256 : (D >= 512 ? 128 : 64);
  if (cast_dtype == MLXB_F32)
    launch_pdl(residual_update_kernel<float>, dim3(R), dim3(threads), 0, stream, x, ldx, y1, w1, y2, w2, ldy, scale,
               eps, (float*)cast_out, ldc, D);
  else if (cast_dtype == MLXB_BF16)
    launch_pdl(residual_update_kernel<__nv_bfloat16>, dim3(R), dim3(threads), 0, stream, x, ldx, y1, w1, y2, w2, ldy,
               scale, eps, (__nv_bfloat16*)cast_out, ldc, D);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "residual_update: dtype code %d", cast_dtype);
  return mlxb_check_launch("residual_update");
}

// Two score maps over the same values, combined per head: with a1 and a2 the two maps' outputs of head h,
// o = a1 - lambda * a2, divided by its root mean square over the head's Dv columns (eps inside the root, no weight),
// times `post`.  a: float32 [T, lda] in which the heads of key/value group g lie as [map 1: rep heads | map 2: rep heads]
// (head h = g * rep + r has its first map at column ((2 g) rep + r) Dv and its second at ((2 g + 1) rep + r) Dv).
// One warp per (token, head).
template <typename TO>
__global__ void head_difference_kernel(const float* a, int lda, const int* __restrict__ token_req, int H, int rep, int Dv,
                                       float lambda, float eps, float post, TO* __restrict__ out, int ldo, int T) {
  pdl_wait();
  pdl_trigger();
  a = after_wait(a);
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  if (token_req && token_req[t] < 0) return;
  const int g = h / rep, r = h - g * rep;
  const float* a1 = a + (size_t)t * lda + (size_t)((2 * g) * rep + r) * Dv;
  const float* a2 = a1 + (size_t)rep * Dv;
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) { const float o = a1[d] - lambda * a2[d]; ss = fmaf(o, o, ss); }
  const float f = post / sqrtf(warp_sum(ss) / (float)Dv + eps);
  TO* op = out + (size_t)t * ldo + (size_t)h * Dv;
  for (int d = lane; d < Dv; d += 32) op[d] = from_f<TO>((a1[d] - lambda * a2[d]) * f);
}

MLXB_EXPORT int mlxb_head_difference(int out_dtype, const float* a, int lda, const int* token_req, int H, int rep, int Dv,
                                     float lambda, float eps, float post, void* out, int ldo, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || rep <= 0 || H % rep || Dv <= 0 || lda < 2 * H * Dv || ldo < H * Dv)
    return mlxb_fail(MLXB_BAD_ARG, "head_difference: %d heads in groups of %d, %d columns, strides %d / %d", H, rep, Dv, lda, ldo);
  const int warps = 4;
  const dim3 grid((unsigned)(((long long)T * H + warps - 1) / warps));
  if (out_dtype == MLXB_F32)
    launch_pdl(head_difference_kernel<float>, grid, dim3(32 * warps), 0, stream, a, lda, token_req, H, rep, Dv, lambda, eps,
               post, (float*)out, ldo, T);
  else if (out_dtype == MLXB_BF16)
    launch_pdl(head_difference_kernel<__nv_bfloat16>, grid, dim3(32 * warps), 0, stream, a, lda, token_req, H, rep, Dv,
               lambda, eps, post, (__nv_bfloat16*)out, ldo, T);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "head_difference: dtype code %d", out_dtype);
  return mlxb_check_launch("head_difference");
}
