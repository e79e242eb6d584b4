// Small row-wise kernels between the products of a layer.
//   gated_unit      out[t, j] = unit(in[t, j], in[t, F + j]): the two halves of a fused [gate | up] projection through
//                   the gated unit of kind `act` (gated_unit.cuh: silu(g) * u, or the bounded unit with `limit`);
//                   float32 arithmetic, rounded once.
//   scale_by_rows   out[t, j] = in[t, j] * table[index[t], first + j]: a per-token vector looked up in a table.
//   xielu           out[t, j] = f(in[t, j]) with two learned numbers (a, b) of the layer, read from device memory:
//                   z > 0: softplus(a) z^2 + z/2;  z <= 0: (1/2 + softplus(b)) (exp(z) - 1 - z) + z/2.  In place if out = in.
//   join_rows       out[t] = [a[t] | b[t]] in the activation dtype from float32 rows (b may be null: a plain cast).
#include "common.cuh"
#include "gated_unit.cuh"

MLXB_DEFINE_LAST_ERROR()

template <typename T>
__global__ void gated_unit_kernel(const T* in, int ldi, T* __restrict__ out, int ldo, int F, int n, int act, float limit) {
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * F) return;
  const int t = (int)(idx / F), j = (int)(idx - (long long)t * F);
  const T* row = in + (size_t)t * ldi;
  out[(size_t)t * ldo + j] = from_f<T>(mlxb_gated_unit(act, to_f(row[j]), to_f(row[F + j]), 1.f, limit));
}

// Eight elements a thread (bfloat16 rows whose halves, strides and bases allow 16-byte accesses).
__global__ void gated_unit_bf16x8_kernel(const __nv_bfloat16* in, int ldi, __nv_bfloat16* __restrict__ out, int ldo, int F,
                                         int n, int act, float limit) {
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  const int per_row = F / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * per_row) return;
  const int t = (int)(idx / per_row), j = (int)(idx - (long long)t * per_row) * 8;
  const __nv_bfloat16* row = in + (size_t)t * ldi;
  float g[8], u[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(row + j), g);
  unpack8(*reinterpret_cast<const uint4*>(row + F + j), u);
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = mlxb_gated_unit(act, g[e], u[e], 1.f, limit);
  *reinterpret_cast<uint4*>(out + (size_t)t * ldo + j) = pack8(o);
}

MLXB_EXPORT int mlxb_gated_unit(int dtype, const void* in, int ldi, void* out, int ldo, int F, int n_rows, int act,
                                float limit, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (F <= 0 || ldi < 2 * F || ldo < F) return mlxb_fail(MLXB_BAD_ARG, "gated_unit: %d columns, strides %d / %d", F, ldi, ldo);
  const long long total = (long long)n_rows * F;
  const int threads = 256;
  const dim3 grid((unsigned)((total + threads - 1) / threads));
  if (dtype == MLXB_F32)
    launch_pdl(gated_unit_kernel<float>, grid, dim3(threads), 0, stream, (const float*)in, ldi, (float*)out, ldo, F, n_rows, act, limit);
  else if (dtype == MLXB_BF16 && F % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0)
    launch_pdl(gated_unit_bf16x8_kernel, dim3((unsigned)((total / 8 + threads - 1) / threads)), dim3(threads), 0, stream,
               (const __nv_bfloat16*)in, ldi, (__nv_bfloat16*)out, ldo, F, n_rows, act, limit);
  else if (dtype == MLXB_BF16)
    launch_pdl(gated_unit_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)in, ldi,
               (__nv_bfloat16*)out, ldo, F, n_rows, act, limit);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "gated_unit: dtype code %d", dtype);
  return mlxb_check_launch("gated_unit");
}

template <typename T>
__global__ void scale_by_rows_kernel(const T* in, int ldi, const int* __restrict__ index, const T* __restrict__ table,
                                     int ldt, int n_table_rows, int first, T* __restrict__ out, int ldo, int F, int n,
                                     int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * F) return;
  const int t = (int)(idx / F), j = (int)(idx - (long long)t * F);
  const int id = index[t];
  float e = 0.f;
  if (id < 0 || id >= n_table_rows) { if (j == 0) atomicOr(status, MLXB_ST_TOKEN_RANGE); }
  else e = to_f(table[(size_t)id * ldt + first + j]);
  out[(size_t)t * ldo + j] = from_f<T>(to_f(in[(size_t)t * ldi + j]) * e);
}

MLXB_EXPORT int mlxb_scale_by_rows(int dtype, const void* in, int ldi, const int* index, const void* table, int ldt,
                                   int n_table_rows, int first, void* out, int ldo, int F, int n_rows, int* status,
                                   cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (F <= 0 || ldi < F || ldo < F || first < 0 || first + F > ldt)
    return mlxb_fail(MLXB_BAD_ARG, "scale_by_rows: columns %d..%d of %d, strides %d / %d", first, first + F, ldt, ldi, ldo);
  const long long total = (long long)n_rows * F;
  const int threads = 256;
  const dim3 grid((unsigned)((total + threads - 1) / threads));
  if (dtype == MLXB_F32)
    launch_pdl(scale_by_rows_kernel<float>, grid, dim3(threads), 0, stream, (const float*)in, ldi, index,
               (const float*)table, ldt, n_table_rows, first, (float*)out, ldo, F, n_rows, status);
  else if (dtype == MLXB_BF16)
    launch_pdl(scale_by_rows_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)in, ldi, index,
               (const __nv_bfloat16*)table, ldt, n_table_rows, first, (__nv_bfloat16*)out, ldo, F, n_rows, status);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "scale_by_rows: dtype code %d", dtype);
  return mlxb_check_launch("scale_by_rows");
}

template <typename T>
__global__ void join_rows_kernel(const float* a, const float* b, int D, T* __restrict__ out, int ldo, int n) {
  pdl_wait();
  pdl_trigger();
  a = after_wait(a);
  b = after_wait(b);
  const int W = b ? 2 * D : D;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * W) return;
  const int t = (int)(idx / W), j = (int)(idx - (long long)t * W);
  const float v = j < D ? a[(size_t)t * D + j] : b[(size_t)t * D + j - D];
  out[(size_t)t * ldo + j] = from_f<T>(v);
}

// Eight elements a thread into bfloat16 rows (D a multiple of 8, 16-byte aligned bases and strides).
__global__ void join_rows_bf16x8_kernel(const float* a, const float* b, int D, __nv_bfloat16* __restrict__ out, int ldo, int n) {
  pdl_wait();
  pdl_trigger();
  a = after_wait(a);
  b = after_wait(b);
  const int W = b ? 2 * D : D, per_row = W / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * per_row) return;
  const int t = (int)(idx / per_row), j = (int)(idx - (long long)t * per_row) * 8;
  const float* src = j < D ? a + (size_t)t * D + j : b + (size_t)t * D + j - D;
  const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
  const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  *reinterpret_cast<uint4*>(out + (size_t)t * ldo + j) = pack8(v);
}

// a, b: float32 [n_rows, D] contiguous (b may be null); out: [n_rows, D or 2D] at row stride ldo.
MLXB_EXPORT int mlxb_join_rows(int dtype, const float* a, const float* b, int D, void* out, int ldo, int n_rows,
                               cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int W = b ? 2 * D : D;
  if (D <= 0 || ldo < W) return mlxb_fail(MLXB_BAD_ARG, "join_rows: width %d into stride %d", W, ldo);
  const long long total = (long long)n_rows * W;
  const int threads = 256;
  const dim3 grid((unsigned)((total + threads - 1) / threads));
  if (dtype == MLXB_F32)
    launch_pdl(join_rows_kernel<float>, grid, dim3(threads), 0, stream, a, b, D, (float*)out, ldo, n_rows);
  else if (dtype == MLXB_BF16 && D % 8 == 0 && ldo % 8 == 0 &&
           (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0)
    launch_pdl(join_rows_bf16x8_kernel, dim3((unsigned)((total / 8 + threads - 1) / threads)), dim3(threads), 0, stream, a, b,
               D, (__nv_bfloat16*)out, ldo, n_rows);
  else if (dtype == MLXB_BF16)
    launch_pdl(join_rows_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, a, b, D, (__nv_bfloat16*)out, ldo, n_rows);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "join_rows: dtype code %d", dtype);
  return mlxb_check_launch("join_rows");
}

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T>
__global__ void xielu_kernel(const T* in, int ldi, T* out, int ldo, int F, int n, const float* __restrict__ act) {
  const float ap = softplus_f(act[0]), aq = 0.5f + softplus_f(act[1]);
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * F) return;
  const int t = (int)(idx / F), j = (int)(idx - (long long)t * F);
  const float z = to_f(in[(size_t)t * ldi + j]);
  const float y = z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
  out[(size_t)t * ldo + j] = from_f<T>(y);
}

// Eight elements a thread (bfloat16 rows whose width, strides and bases allow 16-byte accesses).
__global__ void xielu_bf16x8_kernel(const __nv_bfloat16* in, int ldi, __nv_bfloat16* out, int ldo, int F, int n,
                                    const float* __restrict__ act) {
  const float ap = softplus_f(act[0]), aq = 0.5f + softplus_f(act[1]);
  pdl_wait();
  pdl_trigger();
  in = after_wait(in);
  const int per_row = F / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * per_row) return;
  const int t = (int)(idx / per_row), j = (int)(idx - (long long)t * per_row) * 8;
  float z[8], y[8];
  unpack8(*reinterpret_cast<const uint4*>(in + (size_t)t * ldi + j), z);
#pragma unroll
  for (int e = 0; e < 8; ++e) y[e] = z[e] > 0.f ? fmaf(ap * z[e], z[e], 0.5f * z[e]) : fmaf(aq, expm1f(z[e]) - z[e], 0.5f * z[e]);
  *reinterpret_cast<uint4*>(out + (size_t)t * ldo + j) = pack8(y);
}

// act: float32 [2] on the device, the layer's two numbers before their softplus.
MLXB_EXPORT int mlxb_xielu(int dtype, const void* in, int ldi, void* out, int ldo, int F, int n_rows, const float* act,
                           cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (F <= 0 || ldi < F || ldo < F || !act) return mlxb_fail(MLXB_BAD_ARG, "xielu: %d columns, strides %d / %d", F, ldi, ldo);
  const long long total = (long long)n_rows * F;
  const int threads = 256;
  const dim3 grid((unsigned)((total + threads - 1) / threads));
  if (dtype == MLXB_F32)
    launch_pdl(xielu_kernel<float>, grid, dim3(threads), 0, stream, (const float*)in, ldi, (float*)out, ldo, F, n_rows, act);
  else if (dtype == MLXB_BF16 && F % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0)
    launch_pdl(xielu_bf16x8_kernel, dim3((unsigned)((total / 8 + threads - 1) / threads)), dim3(threads), 0, stream,
               (const __nv_bfloat16*)in, ldi, (__nv_bfloat16*)out, ldo, F, n_rows, act);
  else if (dtype == MLXB_BF16)
    launch_pdl(xielu_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)in, ldi,
               (__nv_bfloat16*)out, ldo, F, n_rows, act);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "xielu: dtype code %d", dtype);
  return mlxb_check_launch("xielu");
}
