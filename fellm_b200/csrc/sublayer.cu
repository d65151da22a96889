// What stands between a sublayer and the residual stream in designs that norm a sublayer's OUTPUT, and the small
// element-wise steps of their sublayers.
//
//   layernorm        y = (x - mean) / sqrt(var + eps) * w + b, float32 in, activation dtype out, optional row gather
//   add_layernorm    x += LN(y) in place (float32); optionally leaves the new rows in the activation dtype too
//   cast_rows        float32 rows -> activation dtype
//   act_mul          [gate | up] rows -> act(gate) * up, act = SiLU or the tanh form of GELU
//   gate_mul         a *= sigmoid(g), element by element (an output gate on concatenated heads)
//   relu2            max(z, 0)^2, float32 in, activation dtype out (a plain expert's activation)
//
// Every row is reduced by one warp in an order that depends on the row's length alone: a token's result does not
// depend on the batch it is in.  Means, variances and the sums into the stream are float32.
#include "common.cuh"

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// A warp per row.  The mean first, then the variance as the mean of the squared deviations (not E[x^2] - mean^2:
// no cancellation), both from the row held in registers where it fits (VPL values a lane), re-read otherwise.
template <int VPL>
__device__ __forceinline__ void row_stats(const float* __restrict__ r, int d, int lane, float keep[VPL], float& mean, float& rstd, float eps) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) { int i = lane + j * 32; keep[j] = i < d ? r[i] : 0.f; s += keep[j]; }
  for (int i = lane + VPL * 32; i < d; i += 32) s += r[i];
  mean = warp_sum(s) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) { int i = lane + j * 32; if (i < d) { float c = keep[j] - mean; q = fmaf(c, c, q); } }
  for (int i = lane + VPL * 32; i < d; i += 32) { float c = r[i] - mean; q = fmaf(c, c, q); }
  rstd = 1.0f / sqrtf(warp_sum(q) / (float)d + eps);
}

#define LN_VPL 16     // rows of up to 512 stay in registers
#define LN_WARPS 4

// d % 4 == 0: the same with 16-byte loads, VPL vectors of a lane (rows of up to 128 * VPL) in registers.
template <int VPL>
__device__ __forceinline__ void row_stats4(const float4* __restrict__ r, int nv, int d, int lane, float4 keep[VPL], float& mean, float& rstd, float eps) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int i = lane + j * 32;
    keep[j] = i < nv ? r[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (keep[j].x + keep[j].y) + (keep[j].z + keep[j].w);
  }
  for (int i = lane + VPL * 32; i < nv; i += 32) { const float4 v = r[i]; s += (v.x + v.y) + (v.z + v.w); }
  mean = warp_sum(s) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    if (lane + j * 32 < nv) {
      const float a = keep[j].x - mean, b = keep[j].y - mean, c = keep[j].z - mean, e = keep[j].w - mean;
      q = fmaf(a, a, fmaf(b, b, fmaf(c, c, fmaf(e, e, q))));
    }
  }
  for (int i = lane + VPL * 32; i < nv; i += 32) {
    const float4 v = r[i];
    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, e = v.w - mean;
    q = fmaf(a, a, fmaf(b, b, fmaf(c, c, fmaf(e, e, q))));
  }
  rstd = 1.0f / sqrtf(warp_sum(q) / (float)d + eps);
}

__device__ __forceinline__ void put4(float* o, float4 v) { *(float4*)o = v; }
__device__ __forceinline__ void put4(bf16* o, float4 v) {
  __nv_bfloat162 p0 = __floats2bfloat162_rn(v.x, v.y), p1 = __floats2bfloat162_rn(v.z, v.w);
  uint2 u; u.x = *(unsigned*)&p0; u.y = *(unsigned*)&p1;
  *(uint2*)o = u;
}
__device__ __forceinline__ float4 ln4(float4 v, float mean, float rstd, float4 w, float4 b) {
  return make_float4(fmaf((v.x - mean) * rstd, w.x, b.x), fmaf((v.y - mean) * rstd, w.y, b.y),
                     fmaf((v.z - mean) * rstd, w.z, b.z), fmaf((v.w - mean) * rstd, w.w, b.w));
}

// x (may be null: the plain norm) += LN(y rows); out / cast (may be null) gets the result in TO.
template <typename TO, int VPL>
__global__ void __launch_bounds__(LN_WARPS * 32)
layernorm_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, const float* __restrict__ b,
                     TO* __restrict__ out, const int* __restrict__ rows, int n_rows, int d, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int orow = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  if (orow >= n_rows) return;
  const int nv = d >> 2;
  const float4* r = (const float4*)(y + (size_t)(rows ? rows[orow] : orow) * d);
  const float4* w4 = (const float4*)w; const float4* b4 = (const float4*)b;
  float4 keep[VPL];
  float mean, rstd;
  row_stats4<VPL>(r, nv, d, lane, keep, mean, rstd, eps);
  float4* xr = x ? (float4*)(x + (size_t)orow * d) : nullptr;
  TO* o = out ? out + (size_t)orow * d : nullptr;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int i = lane + j * 32;
    if (i < nv) {
      float4 v = ln4(keep[j], mean, rstd, w4[i], b4[i]);
      if (xr) { const float4 a = xr[i]; v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; xr[i] = v; }
      if (o) put4(o + 4 * i, v);
    }
  }
  for (int i = lane + VPL * 32; i < nv; i += 32) {
    float4 v = ln4(r[i], mean, rstd, w4[i], b4[i]);
    if (xr) { const float4 a = xr[i]; v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; xr[i] = v; }
    if (o) put4(o + 4 * i, v);
  }
}

template <typename TO>
static int launch_ln_vec(float* x, const float* y, const float* w, const float* b, TO* out, const int* rows, int n_rows, int d,
                         float eps, cudaStream_t stream) {
  dim3 grid(ceil_div(n_rows, LN_WARPS));
  const int cls = launch_class_for_rows(n_rows, 0);
  if (d <= 1024) return launch_k_class(cls, layernorm_vec_kernel<TO, 8>, grid, dim3(LN_WARPS * 32), 0, stream, 1, x, y, w, b, out, rows, n_rows, d, eps);
  return launch_k_class(cls, layernorm_vec_kernel<TO, 16>, grid, dim3(LN_WARPS * 32), 0, stream, 1, x, y, w, b, out, rows, n_rows, d, eps);
}
static inline bool ln_vec_ok(const void* a, const void* b, const void* c, const void* e, const void* f, int d) {
  return d % 4 == 0 && d >= 128 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)e | (uintptr_t)f) & 15) == 0;
}

template <typename TO>
__global__ void __launch_bounds__(LN_WARPS * 32)
layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out,
                 const int* __restrict__ rows, int n_rows, int d, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int orow = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  if (orow >= n_rows) return;
  const float* r = x + (size_t)(rows ? rows[orow] : orow) * d;
  float keep[LN_VPL], mean, rstd;
  row_stats<LN_VPL>(r, d, lane, keep, mean, rstd, eps);
  TO* o = out + (size_t)orow * d;
#pragma unroll
  for (int j = 0; j < LN_VPL; ++j) { int i = lane + j * 32; if (i < d) o[i] = from_f<TO>(fmaf((keep[j] - mean) * rstd, w[i], b[i])); }
  for (int i = lane + LN_VPL * 32; i < d; i += 32) o[i] = from_f<TO>(fmaf((r[i] - mean) * rstd, w[i], b[i]));
}

FELLM_API int fellm_layernorm(const float* x, const float* w, const float* b, void* out, int out_is_bf16, const int* rows,
                              int n_out_rows, int d, float eps, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (!x || !w || !b || !out || d < 1) return FELLM_ERR_ARG;
  if (ln_vec_ok(x, w, b, out, nullptr, d)) {
    if (out_is_bf16) return launch_ln_vec<bf16>(nullptr, x, w, b, (bf16*)out, rows, n_out_rows, d, eps, stream);
    return launch_ln_vec<float>(nullptr, x, w, b, (float*)out, rows, n_out_rows, d, eps, stream);
  }
  dim3 grid(ceil_div(n_out_rows, LN_WARPS));
  const int cls = launch_class_for_rows(n_out_rows, 0);
  if (out_is_bf16) return launch_k_class(cls, layernorm_kernel<bf16>, grid, dim3(LN_WARPS * 32), 0, stream, 1, x, w, b, (bf16*)out, rows, n_out_rows, d, eps);
  return launch_k_class(cls, layernorm_kernel<float>, grid, dim3(LN_WARPS * 32), 0, stream, 1, x, w, b, (float*)out, rows, n_out_rows, d, eps);
}

// x[t, :] += LN(y[t, :]); `cast` (may be null): the new row of x in the activation dtype, for the sublayer that reads
// the stream itself next.
template <typename TO>
__global__ void __launch_bounds__(LN_WARPS * 32)
add_layernorm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, const float* __restrict__ b,
                     TO* __restrict__ cast, int n_rows, int d, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const float* r = y + (size_t)row * d;
  float keep[LN_VPL], mean, rstd;
  row_stats<LN_VPL>(r, d, lane, keep, mean, rstd, eps);
  float* xr = x + (size_t)row * d;
  TO* c = cast ? cast + (size_t)row * d : nullptr;
#pragma unroll
  for (int j = 0; j < LN_VPL; ++j) {
    int i = lane + j * 32;
    if (i < d) { float v = xr[i] + fmaf((keep[j] - mean) * rstd, w[i], b[i]); xr[i] = v; if (c) c[i] = from_f<TO>(v); }
  }
  for (int i = lane + LN_VPL * 32; i < d; i += 32) {
    float v = xr[i] + fmaf((r[i] - mean) * rstd, w[i], b[i]); xr[i] = v; if (c) c[i] = from_f<TO>(v);
  }
}

FELLM_API int fellm_add_layernorm(float* x, const float* y, const float* w, const float* b, void* cast, int cast_is_bf16,
                                  int n_rows, int d, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (!x || !y || !w || !b || d < 1) return FELLM_ERR_ARG;
  if (ln_vec_ok(x, y, w, b, cast, d)) {
    if (cast_is_bf16) return launch_ln_vec<bf16>(x, y, w, b, (bf16*)cast, nullptr, n_rows, d, eps, stream);
    return launch_ln_vec<float>(x, y, w, b, (float*)cast, nullptr, n_rows, d, eps, stream);
  }
  dim3 grid(ceil_div(n_rows, LN_WARPS));
  const int cls = launch_class_for_rows(n_rows, 0);
  if (cast_is_bf16) return launch_k_class(cls, add_layernorm_kernel<bf16>, grid, dim3(LN_WARPS * 32), 0, stream, 1, x, y, w, b, (bf16*)cast, n_rows, d, eps);
  return launch_k_class(cls, add_layernorm_kernel<float>, grid, dim3(LN_WARPS * 32), 0, stream, 1, x, y, w, b, (float*)cast, n_rows, d, eps);
}

// ---------------------------------------------------------------- float32 -> bfloat16 rows
__global__ void cast_rows_kernel(const float* __restrict__ x, bf16* __restrict__ out, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(x[i]);
}

static inline int ew_blocks(long long n) {
  long long b = (n + 255) / 256, cap = (long long)fellm_sm_count() * 16;
  return (int)(b > cap ? cap : (b < 1 ? 1 : b));
}

FELLM_API int fellm_cast_rows(const float* x, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!x || !out) return FELLM_ERR_ARG;
  return launch_k_class(launch_class_for_rows(n / 256, 0), cast_rows_kernel, dim3(ew_blocks(n)), dim3(256), 0, stream, 1, x, (bf16*)out, n);
}

// ---------------------------------------------------------------- act(gate) * up
// gu [T, ld]: gate in columns [0, F), up in [F, 2F); out [T, F].  act 0: SiLU; 1: GELU, tanh form.
template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ gu, int ld, T* __restrict__ out, int rows, int F, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t n = (size_t)rows * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / F; const int c = (int)(i - r * F);
    const float g = to_f(gu[r * ld + c]), u = to_f(gu[r * ld + F + c]);
    out[i] = from_f<T>((act == 1 ? gelu_tanh_f(g) : g / (1.0f + expf(-g))) * u);
  }
}

// bfloat16, F % 8 == 0, rows 16-byte aligned: eight elements a thread.
__global__ void act_mul_vec_kernel(const bf16* __restrict__ gu, int ld, bf16* __restrict__ out, int rows, int F, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int per = F >> 3;
  const size_t n = (size_t)rows * per;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / per; const int c = (int)(i - r * per) << 3;
    const uint4 gr = *(const uint4*)(gu + r * ld + c), ur = *(const uint4*)(gu + r * ld + F + c);
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&gr; const __nv_bfloat162* u2 = (const __nv_bfloat162*)&ur;
    uint4 o; __nv_bfloat162* o2 = (__nv_bfloat162*)&o;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      const float a0 = act == 1 ? gelu_tanh_f(g.x) : g.x / (1.0f + expf(-g.x)), a1 = act == 1 ? gelu_tanh_f(g.y) : g.y / (1.0f + expf(-g.y));
      o2[e] = __floats2bfloat162_rn(a0 * u.x, a1 * u.y);
    }
    *(uint4*)(out + r * F + c) = o;
  }
}

FELLM_API int fellm_act_mul(const void* gu, int ld, void* out, int is_bf16, int rows, int F, int act, cudaStream_t stream) {
  if (rows <= 0 || F <= 0) return 0;
  if (!gu || !out || act < 0 || act > 1 || ld < 2 * F) return FELLM_ERR_ARG;
  if (is_bf16 && F % 8 == 0 && ld % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0)
    return launch_k_class(launch_class_for_rows(rows, 0), act_mul_vec_kernel, dim3(ew_blocks((long long)rows * (F >> 3))), dim3(256), 0, stream, 1,
                          (const bf16*)gu, ld, (bf16*)out, rows, F, act);
  const int blocks = ew_blocks((long long)rows * F), cls = launch_class_for_rows(rows, 0);
  if (is_bf16) return launch_k_class(cls, act_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1, (const bf16*)gu, ld, (bf16*)out, rows, F, act);
  return launch_k_class(cls, act_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, (const float*)gu, ld, (float*)out, rows, F, act);
}

// ---------------------------------------------------------------- a *= sigmoid(g)
// a [T, N] contiguous, g [T, ldg] (the gate's logits); the sigmoid and the product in float32.
template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ a, const T* __restrict__ g, int ldg, int rows, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t n = (size_t)rows * N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / N; const int c = (int)(i - r * N);
    a[i] = from_f<T>(to_f(a[i]) / (1.0f + expf(-to_f(g[r * ldg + c]))));
  }
}

// bfloat16, N % 8 == 0, 16-byte aligned rows: eight elements a thread.
__global__ void gate_mul_vec_kernel(bf16* __restrict__ a, const bf16* __restrict__ g, int ldg, int rows, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int per = N >> 3;
  const size_t n = (size_t)rows * per;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / per; const int c = (int)(i - r * per) << 3;
    uint4 av = *(const uint4*)(a + r * N + c);
    const uint4 gv = *(const uint4*)(g + r * ldg + c);
    __nv_bfloat162* a2 = (__nv_bfloat162*)&av; const __nv_bfloat162* g2 = (const __nv_bfloat162*)&gv;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(a2[e]), z = __bfloat1622float2(g2[e]);
      a2[e] = __floats2bfloat162_rn(x.x / (1.0f + expf(-z.x)), x.y / (1.0f + expf(-z.y)));
    }
    *(uint4*)(a + r * N + c) = av;
  }
}

FELLM_API int fellm_gate_mul(void* a, const void* g, int ldg, int is_bf16, int rows, int N, cudaStream_t stream) {
  if (rows <= 0 || N <= 0) return 0;
  if (!a || !g || ldg < N) return FELLM_ERR_ARG;
  if (is_bf16 && N % 8 == 0 && ldg % 8 == 0 && (((uintptr_t)a | (uintptr_t)g) & 15) == 0)
    return launch_k_class(launch_class_for_rows(rows, 0), gate_mul_vec_kernel, dim3(ew_blocks((long long)rows * (N >> 3))), dim3(256), 0, stream, 1,
                          (bf16*)a, (const bf16*)g, ldg, rows, N);
  const int blocks = ew_blocks((long long)rows * N), cls = launch_class_for_rows(rows, 0);
  if (is_bf16) return launch_k_class(cls, gate_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1, (bf16*)a, (const bf16*)g, ldg, rows, N);
  return launch_k_class(cls, gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, (float*)a, (const float*)g, ldg, rows, N);
}

// ---------------------------------------------------------------- max(z, 0)^2
template <typename TO>
__global__ void relu2_kernel(const float* __restrict__ z, TO* __restrict__ out, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(z[i], 0.f);
    out[i] = from_f<TO>(v * v);
  }
}

FELLM_API int fellm_relu2(const float* z, void* out, int out_is_bf16, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!z || !out) return FELLM_ERR_ARG;
  const int cls = launch_class_for_rows(n / 256, 0);
  if (out_is_bf16) return launch_k_class(cls, relu2_kernel<bf16>, dim3(ew_blocks(n)), dim3(256), 0, stream, 1, z, (bf16*)out, n);
  return launch_k_class(cls, relu2_kernel<float>, dim3(ew_blocks(n)), dim3(256), 0, stream, 1, z, (float*)out, n);
}
