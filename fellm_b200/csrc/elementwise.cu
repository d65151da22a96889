// Embedding gather (times a constant), RMSNorm, SiLU-gate, row gather, a vector added to every row, scaled and
// soft-capped logits.
//
// FeLLM counterparts (plugins/cuda_kernels/src/oxide_kernels.rs): embedding_bf16_rows (3140),
// rmsnorm_group (165), silu_gate (67).  The residual stream is float32 in both engine dtypes;
// norms read it and write the engine's activation dtype.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                  float* __restrict__ out, int d, int vocab, int* __restrict__ status, float scale) {
  FELLM_TRACE_SCOPE(TRACE_EMBED_ROWS);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();                 // the residual buffer may still be read by the step before
  int row = blockIdx.x;
  int tok = tokens[row];
  float* o = out + (size_t)row * d;
  if (tok < 0 || tok >= vocab) {          // never read outside the table: record and write zeros
    if (threadIdx.x == 0 && status) atomicExch(status, 1);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* src = table + (size_t)tok * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f(src[i]) * scale;
}

FELLM_API int fellm_embed_rows(const int* tokens, const void* table, int table_is_bf16, float* out,
                               int rows, int d, int vocab, int* status, float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!tokens || !table || !out) return FELLM_ERR_ARG;
  int threads = d >= 256 ? 256 : (d >= 128 ? 128 : 64);
  if (table_is_bf16)
    return launch_k_class(launch_class_for_rows(rows, 2), embed_rows_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, 1, tokens, (const bf16*)table, out, d, vocab, status, scale);
  return launch_k_class(launch_class_for_rows(rows, 2), embed_rows_kernel<float>, dim3(rows), dim3(threads), 0, stream, 1, tokens, (const float*)table, out, d, vocab, status, scale);
}

// ---------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w, product order (x*scale)*w, all in float32.
// One block per output row; the reduction order depends on d and the block size only, so a row's
// result does not depend on which other rows are in the batch.
template <typename TO, int THREADS>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               TO* __restrict__ out, const int* __restrict__ rows, int d, float eps) {
  FELLM_TRACE_SCOPE(TRACE_RMSNORM);
  __shared__ float partial[THREADS / 32];
  __shared__ float scale_s;
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  int orow = blockIdx.x;
  int irow = rows ? rows[orow] : orow;
  const float* xr = x + (size_t)irow * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += THREADS) { float v = xr[i]; ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) t += partial[i];
    scale_s = 1.0f / sqrtf(t / (float)d + eps);
  }
  __syncthreads();
  float scale = scale_s;
  TO* o = out + (size_t)orow * d;
  for (int i = threadIdx.x; i < d; i += THREADS) o[i] = from_f<TO>((xr[i] * scale) * w[i]);
}

__device__ __forceinline__ void store4(float* o, float a, float b, float c, float e) { *(float4*)o = make_float4(a, b, c, e); }
__device__ __forceinline__ void store4(bf16* o, float a, float b, float c, float e) {
  __nv_bfloat162 p0 = __floats2bfloat162_rn(a, b), p1 = __floats2bfloat162_rn(c, e);
  uint2 v; v.x = *(unsigned*)&p0; v.y = *(unsigned*)&p1;
  *(uint2*)o = v;
}

// d % 4 == 0: a warp per row, 16-byte loads; up to VPL vectors of a lane stay in registers between
// the sum and the scaling (rows longer than 128*VPL are read a second time).  A row's sum has the
// same order whatever else is in the batch.
template <typename TO, int VPL>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   TO* __restrict__ out, const int* __restrict__ rows, int n_rows, int d, float eps) {
  FELLM_TRACE_SCOPE(TRACE_RMSNORM_VEC);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  const int lane = threadIdx.x & 31;
  const int orow = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (orow >= n_rows) return;
  const int irow = rows ? rows[orow] : orow;
  const float4* xr = (const float4*)(x + (size_t)irow * d);
  const float4* wr = (const float4*)w;
  const int nv = d >> 2;
  float4 keep[VPL];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int i = lane + j * 32;
    keep[j] = i < nv ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j)
    ss = fmaf(keep[j].x, keep[j].x, fmaf(keep[j].y, keep[j].y, fmaf(keep[j].z, keep[j].z, fmaf(keep[j].w, keep[j].w, ss))));
  for (int i = lane + VPL * 32; i < nv; i += 32) {
    float4 v = xr[i];
    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)d + eps);
  TO* o = out + (size_t)orow * d;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int i = lane + j * 32;
    if (i < nv) {
      float4 g = wr[i];
      store4(o + 4 * i, (keep[j].x * scale) * g.x, (keep[j].y * scale) * g.y, (keep[j].z * scale) * g.z, (keep[j].w * scale) * g.w);
    }
  }
  for (int i = lane + VPL * 32; i < nv; i += 32) {
    float4 v = xr[i], g = wr[i];
    store4(o + 4 * i, (v.x * scale) * g.x, (v.y * scale) * g.y, (v.z * scale) * g.z, (v.w * scale) * g.w);
  }
}

// RMSNorm as a kernel of its own runs where the products do not take it in (17 rows and more): launched as a
// programmatic dependent from FELLM_B200_NORM_PDL_ROWS rows on, its launch hides under the product in front.
static int norm_class(int rows) {
  static int from = -1;
  if (from < 0) { const char* e = getenv("FELLM_B200_NORM_PDL_ROWS"); from = e ? atoi(e) : 17; }
  return rows >= from ? 1 : 0;
}

FELLM_API int fellm_rmsnorm(const float* x, const float* w, void* out, int out_is_bf16,
                            const int* rows, int n_out_rows, int d, float eps, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (!x || !w || !out) return FELLM_ERR_ARG;
  if (d % 4 == 0 && d >= 128) {
    const int warps = 4;
    dim3 vgrid((n_out_rows + warps - 1) / warps);
    if (d <= 1024) {
      if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<bf16, 8>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (bf16*)out, rows, n_out_rows, d, eps);
      return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<float, 8>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (float*)out, rows, n_out_rows, d, eps);
    }
    if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<bf16, 16>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (bf16*)out, rows, n_out_rows, d, eps);
    return launch_k_class(norm_class(n_out_rows), rmsnorm_vec_kernel<float, 16>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (float*)out, rows, n_out_rows, d, eps);
  }
  dim3 grid(n_out_rows);
  if (d >= 512) {
    if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<bf16, 256>, grid, dim3(256), 0, stream, 1, x, w, (bf16*)out, rows, d, eps);
    return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<float, 256>, grid, dim3(256), 0, stream, 1, x, w, (float*)out, rows, d, eps);
  }
  if (out_is_bf16) return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<bf16, 64>, grid, dim3(64), 0, stream, 1, x, w, (bf16*)out, rows, d, eps);
  return launch_k_class(norm_class(n_out_rows), rmsnorm_kernel<float, 64>, grid, dim3(64), 0, stream, 1, x, w, (float*)out, rows, d, eps);
}

// ---------------------------------------------------------------- SiLU gate
// in [T, 2F]: gate in columns [0,F), up in [F,2F); out [T,F] = gate/(1+exp(-gate)) * up.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int F) {
  FELLM_TRACE_SCOPE(TRACE_SILU_MUL);
  pdl_launch_dependents();
  pdl_wait(); FELLM_TRACE_WAITED();
  size_t n = (size_t)rows * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / F; int c = (int)(i - r * F);
    float g = to_f(gu[r * 2 * F + c]);
    float u = to_f(gu[r * 2 * F + F + c]);
    out[i] = from_f<T>((g / (1.0f + expf(-g))) * u);
  }
}

FELLM_API int fellm_silu_mul(const void* gu, void* out, int is_bf16, int rows, int F, cudaStream_t stream) {
  if (rows <= 0) return 0;
  size_t n = (size_t)rows * F;
  int blocks = (int)((n + 255) / 256); if (blocks > fellm_sm_count() * 16) blocks = fellm_sm_count() * 16;
  if (is_bf16) return launch_k_class(launch_class_for_rows(rows, 0), silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1, (const bf16*)gu, (bf16*)out, rows, F);
  return launch_k_class(launch_class_for_rows(rows, 0), silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, (const float*)gu, (float*)out, rows, F);
}

// ---------------------------------------------------------------- Dynamic Tanh norm
// y = tanh(alpha * x) * w + b: no mean, no variance, nothing that couples the elements of a row.
template <typename TO>
__global__ void dyt_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                float alpha, TO* __restrict__ out, const int* __restrict__ rows, int n_rows, int d) {
  pdl_launch_dependents();
  pdl_wait();
  size_t n = (size_t)n_rows * d;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / d; int c = (int)(i - r * d);
    size_t src = rows ? (size_t)rows[r] : r;
    out[i] = from_f<TO>(fmaf(tanhf(alpha * x[src * d + c]), w[c], b[c]));
  }
}

FELLM_API int fellm_dyt_norm(const float* x, const float* w, const float* b, float alpha, void* out, int out_is_bf16,
                             const int* rows, int n_out_rows, int d, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (!x || !w || !b || !out) return FELLM_ERR_ARG;
  size_t n = (size_t)n_out_rows * d;
  int blocks = (int)((n + 255) / 256); if (blocks > fellm_sm_count() * 16) blocks = fellm_sm_count() * 16;
  if (out_is_bf16) return launch_k_class(launch_class_for_rows(n_out_rows, 0), dyt_norm_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1, x, w, b, alpha, (bf16*)out, rows, n_out_rows, d);
  return launch_k_class(launch_class_for_rows(n_out_rows, 0), dyt_norm_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, x, w, b, alpha, (float*)out, rows, n_out_rows, d);
}

// ---------------------------------------------------------------- [a | b] rows in the activation dtype
// out[t, 0:d] = a[t, :], out[t, d:2d] = b[t, :] (float32 in): the input of a product over two streams.
template <typename TO>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out,
                                   int rows, int d) {
  pdl_launch_dependents();
  pdl_wait();
  size_t n = (size_t)rows * 2 * d;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / (2 * d); int c = (int)(i - r * 2 * d);
    out[i] = from_f<TO>(c < d ? a[r * d + c] : b[r * d + c - d]);
  }
}

FELLM_API int fellm_concat_cast(const float* a, const float* b, void* out, int out_is_bf16, int rows, int d,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!a || !b || !out) return FELLM_ERR_ARG;
  size_t n = (size_t)rows * 2 * d;
  int blocks = (int)((n + 255) / 256); if (blocks > fellm_sm_count() * 16) blocks = fellm_sm_count() * 16;
  if (out_is_bf16) return launch_k_class(launch_class_for_rows(rows, 0), concat_cast_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1, a, b, (bf16*)out, rows, d);
  return launch_k_class(launch_class_for_rows(rows, 0), concat_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, a, b, (float*)out, rows, d);
}

// ---------------------------------------------------------------- a vector added to every row
// x[t, :] += v   (float32; what opens a pass of a looped run of layers)
__global__ void add_row_vector_kernel(float* __restrict__ x, const float* __restrict__ v, long long n, int d) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += v[i % d];
}

FELLM_API int fellm_add_row_vector(float* x, const float* v, int rows, int d, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!x || !v || d < 1) return FELLM_ERR_ARG;
  long long n = (long long)rows * d;
  add_row_vector_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, v, n, d);
  return launch_status();
}

// ---------------------------------------------------------------- logits: scale, then soft cap
// z <- cap * tanh(z * scale / cap)   (cap <= 0: z <- z * scale), float32 in place
__global__ void scale_softcap_kernel(float* __restrict__ z, long long n, float scale, float cap) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = z[i] * scale;
  z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

FELLM_API int fellm_scale_softcap(float* z, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!z) return FELLM_ERR_ARG;
  scale_softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(z, n, scale, cap);
  return launch_status();
}

// ---------------------------------------------------------------- a block's sum, the same order for every row
// Sum of v over the block (blockDim.x a multiple of 32, at most 1024): lanes by a butterfly, warps in order.
__device__ __forceinline__ float block_sum(float v, float* scratch /* [33] */) {
  v = warp_sum(v);
  __syncthreads();                          // the scratch may still be read from the call before
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += scratch[i];
    scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---------------------------------------------------------------- RMSNorm in groups
// The row in `groups` equal consecutive parts, each over its own root mean square, then the weight:
// y[c] = x[c] / sqrt(mean over c's part of x^2 + eps) * w[c].  A block per (row, part); float32 in, activation dtype out.
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_groups_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                      const int* __restrict__ rows, int d, int groups, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int orow = blockIdx.x, g = blockIdx.y, per = d / groups;
  const int irow = rows ? rows[orow] : orow;
  const float* xr = x + (size_t)irow * d + (size_t)g * per;
  float ss = 0.f;
  for (int i = threadIdx.x; i < per; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
  const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)per + eps);
  TO* o = out + (size_t)orow * d + (size_t)g * per;
  const float* wg = w + (size_t)g * per;
  for (int i = threadIdx.x; i < per; i += blockDim.x) o[i] = from_f<TO>((xr[i] * scale) * wg[i]);
}

// Parts of a multiple of 4 elements up to 2,048: a warp per (row, part), the part read once with 16-byte loads and
// kept in registers between the sum and the scaling (a lane's share in order, then a butterfly: the same order whatever
// else the step holds).
template <typename TO, int VPL>
__global__ void rmsnorm_groups_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                                          const int* __restrict__ rows, int n_rows, int d, int groups, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)n_rows * groups) return;
  const int orow = (int)(unit / groups), g = (int)(unit - (long long)orow * groups), per = d / groups;
  const int irow = rows ? rows[orow] : orow;
  const float4* xr = (const float4*)(x + (size_t)irow * d + (size_t)g * per);
  const float4* wr = (const float4*)(w + (size_t)g * per);
  const int nv = per >> 2;
  float4 keep[VPL];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int i = lane + j * 32;
    keep[j] = i < nv ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j)
    ss = fmaf(keep[j].x, keep[j].x, fmaf(keep[j].y, keep[j].y, fmaf(keep[j].z, keep[j].z, fmaf(keep[j].w, keep[j].w, ss))));
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)per + eps);
  TO* o = out + (size_t)orow * d + (size_t)g * per;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int i = lane + j * 32;
    if (i < nv) {
      const float4 gw = wr[i];
      store4(o + 4 * i, (keep[j].x * scale) * gw.x, (keep[j].y * scale) * gw.y, (keep[j].z * scale) * gw.z, (keep[j].w * scale) * gw.w);
    }
  }
}

FELLM_API int fellm_rmsnorm_groups(const float* x, const float* w, void* out, int out_is_bf16, const int* rows,
                                   int n_out_rows, int d, int groups, float eps, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (!x || !w || !out) return FELLM_ERR_ARG;
  if (groups < 1 || d % groups || groups > 65535) return FELLM_ERR_SIZE;
  if ((d / groups) % 4 == 0 && d / groups <= 2048 && (((size_t)x | (size_t)w | (size_t)out) & 15) == 0) {
    const int warps = 4, cls = launch_class_for_rows(n_out_rows, 0);
    const long long units = (long long)n_out_rows * groups;
    dim3 vgrid((unsigned)((units + warps - 1) / warps));
#define GROUPS_VEC(TO_, VPL_) return launch_k_class(cls, rmsnorm_groups_vec_kernel<TO_, VPL_>, vgrid, dim3(warps * 32), 0, stream, 1, x, w, (TO_*)out, rows, n_out_rows, d, groups, eps)
    if (d / groups <= 512) { if (out_is_bf16) GROUPS_VEC(bf16, 4); GROUPS_VEC(float, 4); }
    if (d / groups <= 1024) { if (out_is_bf16) GROUPS_VEC(bf16, 8); GROUPS_VEC(float, 8); }
    if (out_is_bf16) GROUPS_VEC(bf16, 16);
    GROUPS_VEC(float, 16);
#undef GROUPS_VEC
  }
  const int per = d / groups, threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
  dim3 grid(n_out_rows, groups);
  if (out_is_bf16) return launch_k_class(launch_class_for_rows(n_out_rows, 0), rmsnorm_groups_kernel<bf16>, grid, dim3(threads), 0, stream, 1, x, w, (bf16*)out, rows, d, groups, eps);
  return launch_k_class(launch_class_for_rows(n_out_rows, 0), rmsnorm_groups_kernel<float>, grid, dim3(threads), 0, stream, 1, x, w, (float*)out, rows, d, groups, eps);
}

// ---------------------------------------------------------------- polynomial activation over unit powers
// out = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(v) = v / sqrt(mean(v^2) + eps) over the row;
// coef = (a, b, c, e) on the device.  z float32 [T, F] (the product's sums as they are; rows ldz apart), out in the activation dtype.
template <typename TO>
__global__ void __launch_bounds__(256)
poly_norm_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ coef, TO* __restrict__ out, int F, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* zr = z + (size_t)blockIdx.x * ldz;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = zr[i], v2 = v * v, v3 = v2 * v;
    s1 = fmaf(v, v, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
  }
  const float r1 = coef[0] / sqrtf(block_sum(s1, scratch) / (float)F + eps);
  const float r2 = coef[1] / sqrtf(block_sum(s2, scratch) / (float)F + eps);
  const float r3 = coef[2] / sqrtf(block_sum(s3, scratch) / (float)F + eps);
  const float e = coef[3];
  TO* o = out + (size_t)blockIdx.x * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float v = zr[i], v2 = v * v;
    o[i] = from_f<TO>(fmaf(v, r1, fmaf(v2, r2, fmaf(v2 * v, r3, e))));
  }
}

// Rows of a multiple of 4 elements up to 256 x 4 x KEEP: the row is read once, 16 bytes a lane, and stays in registers
// between the three sums and the result (the sums: a thread's share in order, warps in order, as above).
template <typename TO, int KEEP>
__global__ void __launch_bounds__(256)
poly_norm_vec_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ coef, TO* __restrict__ out, int F, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float4* zr = (const float4*)(z + (size_t)blockIdx.x * ldz);
  const int nv = F >> 2;
  float4 keep[KEEP];
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int i = threadIdx.x + j * 256;
    keep[j] = i < nv ? zr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const float v[4] = {keep[j].x, keep[j].y, keep[j].z, keep[j].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float v2 = v[e] * v[e], v3 = v2 * v[e];
      s1 = fmaf(v[e], v[e], s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
    }
  }
  const float r1 = coef[0] / sqrtf(block_sum(s1, scratch) / (float)F + eps);
  const float r2 = coef[1] / sqrtf(block_sum(s2, scratch) / (float)F + eps);
  const float r3 = coef[2] / sqrtf(block_sum(s3, scratch) / (float)F + eps);
  const float e0 = coef[3];
  TO* o = out + (size_t)blockIdx.x * F;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < nv) {
      const float4 v = keep[j];
      store4(o + 4 * i, fmaf(v.x, r1, fmaf(v.x * v.x, r2, fmaf(v.x * v.x * v.x, r3, e0))),
             fmaf(v.y, r1, fmaf(v.y * v.y, r2, fmaf(v.y * v.y * v.y, r3, e0))),
             fmaf(v.z, r1, fmaf(v.z * v.z, r2, fmaf(v.z * v.z * v.z, r3, e0))),
             fmaf(v.w, r1, fmaf(v.w * v.w, r2, fmaf(v.w * v.w * v.w, r3, e0))));
    }
  }
}

FELLM_API int fellm_poly_norm(const float* z, int ldz, const float* coef, void* out, int out_is_bf16, int rows, int F, float eps,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!z || !coef || !out || F < 1 || ldz < F) return FELLM_ERR_ARG;
  if (F % 4 == 0 && ldz % 4 == 0 && F <= 256 * 4 * 16 && F >= 1024 && (((size_t)z | (size_t)out) & 15) == 0) {
    const int cls = launch_class_for_rows(rows, 0);
#define POLY_VEC(TO_, K_) return launch_k_class(cls, poly_norm_vec_kernel<TO_, K_>, dim3(rows), dim3(256), 0, stream, 1, z, ldz, coef, (TO_*)out, F, eps)
    if (F <= 256 * 4 * 4) { if (out_is_bf16) POLY_VEC(bf16, 4); POLY_VEC(float, 4); }
    if (F <= 256 * 4 * 8) { if (out_is_bf16) POLY_VEC(bf16, 8); POLY_VEC(float, 8); }
    if (out_is_bf16) POLY_VEC(bf16, 16);
    POLY_VEC(float, 16);
#undef POLY_VEC
  }
  const int threads = F >= 1024 ? 256 : 128;
  if (out_is_bf16) return launch_k_class(launch_class_for_rows(rows, 0), poly_norm_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, 1, z, ldz, coef, (bf16*)out, F, eps);
  return launch_k_class(launch_class_for_rows(rows, 0), poly_norm_kernel<float>, dim3(rows), dim3(threads), 0, stream, 1, z, ldz, coef, (float*)out, F, eps);
}

// ---------------------------------------------------------------- sublayers through sigmoid gates into the stream
// x[t, c] += sum over the n sublayers s of y_s[t, c] * sigmoid(zg[t, s * d + c])   (zg: the gates' logits, bias
// included, float32 [T, ldg]; y_s float32 [T, d]; n = 1 or 2; the sublayers are added up first, in order)
__global__ void gated_add_kernel(float* __restrict__ x, const float* __restrict__ y0, const float* __restrict__ y1,
                                 const float* __restrict__ zg, int ldg, long long n, int d) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / d; const int c = (int)(i - t * d);
    const float* g = zg + t * ldg;
    float v = y0[i] / (1.0f + expf(-g[c]));
    if (y1) v += y1[i] / (1.0f + expf(-g[d + c]));
    x[i] += v;
  }
}

FELLM_API int fellm_gated_add(float* x, const float* y0, const float* y1, const float* zg, int ldg, int rows, int d,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!x || !y0 || !zg || d < 1) return FELLM_ERR_ARG;
  const long long n = (long long)rows * d;
  long long blocks = (n + 255) / 256; if (blocks > fellm_sm_count() * 16) blocks = fellm_sm_count() * 16;
  return launch_k_class(launch_class_for_rows(rows, 0), gated_add_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, 1, x, y0, y1, zg, ldg, n, d);
}

// ---------------------------------------------------------------- what a token adds to the stream by itself
// e = table[token, off : off + m];  g = gelu_tanh(Wg x) * e;  y = Wp g;  x += y / sqrt(mean(y^2) + eps) * w
// (Wg [m, d], Wp [d, m], w float32 [d]; x float32, updated in place).  A block per row, float32 sums: every dot
// product over d is a lane's share in order and a butterfly, every sum over m runs in order.
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
template <typename TW>
__global__ void __launch_bounds__(256)
token_side_kernel(float* __restrict__ x, const int* __restrict__ tokens, const TW* __restrict__ table, int ldt, int off,
                  int vocab, const TW* __restrict__ Wg, const TW* __restrict__ Wp, const float* __restrict__ w, int d, int m,
                  float eps, int* __restrict__ status) {
  extern __shared__ float sh[];            // [d] the row, then its y; [m] g
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  float* xs = sh; float* gs = sh + d;
  float* xr = x + (size_t)blockIdx.x * d;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < d; i += blockDim.x) xs[i] = xr[i];
  int tok = tokens[blockIdx.x];
  const bool bad = tok < 0 || tok >= vocab;
  if (bad) { if (threadIdx.x == 0 && status) atomicExch(status, 1); tok = 0; }
  __syncthreads();
  for (int j = warp; j < m; j += nw) {
    const TW* wr = Wg + (size_t)j * d;
    float s = 0.f;
    for (int k = lane; k < d; k += 32) s = fmaf(xs[k], to_f(wr[k]), s);
    s = warp_sum(s);
    if (lane == 0) gs[j] = bad ? 0.f : gelu_tanh_f(s) * to_f(table[(size_t)tok * ldt + off + j]);
  }
  __syncthreads();
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const TW* pr = Wp + (size_t)i * m;
    float y = 0.f;
    for (int j = 0; j < m; ++j) y = fmaf(gs[j], to_f(pr[j]), y);
    xs[i] = y;                              // (a thread overwrites only the elements it owns; the row was read before the barrier)
    ss = fmaf(y, y, ss);
  }
  const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) xr[i] += (xs[i] * scale) * w[i];
}

FELLM_API int fellm_token_side(float* x, const int* tokens, const void* table, int ldt, int off, int vocab, const void* Wg,
                               const void* Wp, int w_bf16, const float* w, int rows, int d, int m, float eps, int* status,
                               cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!x || !tokens || !table || !Wg || !Wp || !w) return FELLM_ERR_ARG;
  const size_t smem = (size_t)(d + m) * sizeof(float);
  if (d < 1 || m < 1 || smem > 200 * 1024) return FELLM_ERR_SIZE;
  const int cls = launch_class_for_rows(rows, 0);
  if (w_bf16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(token_side_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_k_class(cls, token_side_kernel<bf16>, dim3(rows), dim3(256), smem, stream, 1, x, tokens, (const bf16*)table, ldt, off, vocab,
                          (const bf16*)Wg, (const bf16*)Wp, w, d, m, eps, status);
  }
  if (smem > 48 * 1024) cudaFuncSetAttribute(token_side_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_k_class(cls, token_side_kernel<float>, dim3(rows), dim3(256), smem, stream, 1, x, tokens, (const float*)table, ldt, off, vocab,
                        (const float*)Wg, (const float*)Wp, w, d, m, eps, status);
}

// The same on tensor cores (bfloat16 tables, mma.sync.m16n8k16, float32 sums): a block takes 16 rows.  Its 8 warps
// share the gate product's m outputs by tiles of 8 (the rows' x rounded to bfloat16 in shared memory, W_gate's
// fragments read in place), g goes through shared memory as bfloat16, and each warp then owns d / 8 columns of
// y = W_proj g, NT tiles of 8 in registers, so that a row's mean square is a sum over the warps and x is read and
// written once.  A row's sums run in the same order whatever else the step holds.
__device__ __forceinline__ void ts_ldsm_x4(unsigned* r, const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ts_mma16816(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NT, int W>
__global__ void __launch_bounds__(32 * W)
token_side_mma_kernel(float* __restrict__ x, const float* __restrict__ y0, const float* __restrict__ y1,
                      const float* __restrict__ zg, int ldz, const int* __restrict__ tokens, const bf16* __restrict__ table,
                      int ldt, int off, int vocab, const bf16* __restrict__ Wg, const bf16* __restrict__ Wp,
                      const float* __restrict__ w, int T, int d, int m, float eps, int* __restrict__ status) {
  extern __shared__ __align__(16) unsigned char ts_smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int ldx = d + 8, ldg = m + 8;                       // (16 bytes of padding a row spread the banks)
  constexpr int LDP = 72;
  bf16* Xs = (bf16*)ts_smem;                               // [16][d + 8]
  bf16* Gs = Xs + 16 * ldx;                                // [16][m + 8]
  float* part = (float*)(Gs + 16 * ldg);                   // [W warps][16 rows][64 + 8]: the warps' shares of a gate product
  float* red = part + W * 16 * LDP;                        // [W warps][16 rows]
  int* toks = (int*)(red + W * 16);                        // [16]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int row0 = blockIdx.x * 16;
  // the rows of x, with what the layer's gated sublayers add taken in on the way (y0 != null): x is written back
  // with it, and every product below reads the sum
#pragma unroll 4
  for (int i = tid; i < 16 * (d / 4); i += 32 * W) {
    const int r = i / (d / 4), k = 4 * (i - r * (d / 4));
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < T) {
      float* px = x + (size_t)(row0 + r) * d + k;
      v = *(const float4*)px;
      if (y0) {
        const float* gz = zg + (size_t)(row0 + r) * ldz + k;
        const float4 a = *(const float4*)(y0 + (size_t)(row0 + r) * d + k), ga = *(const float4*)gz;
        float4 s = make_float4(a.x / (1.0f + expf(-ga.x)), a.y / (1.0f + expf(-ga.y)), a.z / (1.0f + expf(-ga.z)), a.w / (1.0f + expf(-ga.w)));
        if (y1) {
          const float4 b = *(const float4*)(y1 + (size_t)(row0 + r) * d + k), gb = *(const float4*)(gz + d);
          s.x += b.x / (1.0f + expf(-gb.x)); s.y += b.y / (1.0f + expf(-gb.y));
          s.z += b.z / (1.0f + expf(-gb.z)); s.w += b.w / (1.0f + expf(-gb.w));
        }
        v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w;
        *(float4*)px = v;
      }
    }
    *(__nv_bfloat162*)(Xs + r * ldx + k) = __floats2bfloat162_rn(v.x, v.y);
    *(__nv_bfloat162*)(Xs + r * ldx + k + 2) = __floats2bfloat162_rn(v.z, v.w);
  }
  if (tid < 16) {
    int tok = row0 + tid < T ? tokens[row0 + tid] : 0;
    if (tok < 0 || tok >= vocab) { if (status) atomicExch(status, 1); tok = -1; }
    toks[tid] = tok;
  }
  __syncthreads();
  // g = gelu_tanh(x W_gate^T) * e, 64 outputs at a time: warp w takes the k16 steps w, w + 8, ... of every output,
  // the warps' shares are added in the order of the warps
  for (int nc0 = 0; nc0 < m; nc0 += 64) {
    const int ntc = min(8, (m - nc0) / 8);
    float z[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) z[n][0] = z[n][1] = z[n][2] = z[n][3] = 0.f;
    for (int ks = warp; ks < d / 16; ks += W) {
      unsigned b[8][2];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const bf16* wr = Wg + (size_t)(nc0 + min(n, ntc - 1) * 8 + g) * d + 16 * ks + 2 * c;
        b[n][0] = *(const unsigned*)wr; b[n][1] = *(const unsigned*)(wr + 8);
      }
      unsigned af[4];
      ts_ldsm_x4(af, Xs + (lane & 15) * ldx + 16 * ks + 8 * (lane >> 4));
#pragma unroll
      for (int n = 0; n < 8; ++n) ts_mma16816(z[n], af, b[n][0], b[n][1]);
    }
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      *(float2*)(part + (warp * 16 + g) * LDP + 8 * n + 2 * c) = make_float2(z[n][0], z[n][1]);
      *(float2*)(part + (warp * 16 + g + 8) * LDP + 8 * n + 2 * c) = make_float2(z[n][2], z[n][3]);
    }
    __syncthreads();
    for (int i = tid; i < 16 * 64; i += 32 * W) {
      const int r = i >> 6, cl = i & 63;
      if (cl < ntc * 8) {
        float sum = 0.f;
#pragma unroll
        for (int ww = 0; ww < W; ++ww) sum += part[(ww * 16 + r) * LDP + cl];
        const int tok = toks[r];
        const float e = tok >= 0 ? to_f(table[(size_t)tok * ldt + off + nc0 + cl]) : 0.f;
        Gs[r * ldg + nc0 + cl] = __float2bfloat16_rn(gelu_tanh_f(sum) * e);
      }
    }
    __syncthreads();
  }
  // y = g W_proj^T: this warp's columns [warp d / W, (warp + 1) d / W), n_tiles tiles of 8 (tiles beyond them repeat the last)
  const int n_tiles = d / (8 * W), col0 = warp * (d / W);
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll 2
  for (int ks = 0; ks < m / 16; ++ks) {
    unsigned b[NT][2];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const bf16* pr = Wp + (size_t)(col0 + 8 * min(n, n_tiles - 1) + g) * m + 16 * ks + 2 * c;
      b[n][0] = *(const unsigned*)pr; b[n][1] = *(const unsigned*)(pr + 8);
    }
    unsigned af[4];
    ts_ldsm_x4(af, Gs + (lane & 15) * ldg + 16 * ks + 8 * (lane >> 4));
#pragma unroll
    for (int n = 0; n < NT; ++n) ts_mma16816(acc[n], af, b[n][0], b[n][1]);
  }
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    if (n < n_tiles) {
      ss0 = fmaf(acc[n][0], acc[n][0], fmaf(acc[n][1], acc[n][1], ss0));
      ss1 = fmaf(acc[n][2], acc[n][2], fmaf(acc[n][3], acc[n][3], ss1));
    }
  }
  ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
  ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
  if (c == 0) { red[warp * 16 + g] = ss0; red[warp * 16 + g + 8] = ss1; }
  __syncthreads();
  float t0 = 0.f, t1 = 0.f;
#pragma unroll
  for (int i = 0; i < W; ++i) { t0 += red[i * 16 + g]; t1 += red[i * 16 + g + 8]; }
  const float sc0 = 1.0f / sqrtf(t0 / (float)d + eps), sc1 = 1.0f / sqrtf(t1 / (float)d + eps);
  // (the loads of a few tiles first, then their sums and stores: the loads are in flight together)
  constexpr int NB = NT < 4 ? NT : 4;
  const bool in0 = row0 + g < T, in1 = row0 + g + 8 < T;
  float* x0 = x + (size_t)(row0 + g) * d;
  float* x1 = x + (size_t)(row0 + g + 8) * d;
#pragma unroll
  for (int n0 = 0; n0 < NT; n0 += NB) {
    float2 wv[NB], v0[NB], v1[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int col = col0 + 8 * min(n0 + j, n_tiles - 1) + 2 * c;
      wv[j] = *(const float2*)(w + col);
      v0[j] = in0 ? *(const float2*)(x0 + col) : make_float2(0.f, 0.f);
      v1[j] = in1 ? *(const float2*)(x1 + col) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int n = n0 + j, col = col0 + 8 * n + 2 * c;
      if (n < n_tiles) {
        if (in0) *(float2*)(x0 + col) = make_float2(v0[j].x + (acc[n][0] * sc0) * wv[j].x, v0[j].y + (acc[n][1] * sc0) * wv[j].y);
        if (in1) *(float2*)(x1 + col) = make_float2(v1[j].x + (acc[n][2] * sc1) * wv[j].x, v1[j].y + (acc[n][3] * sc1) * wv[j].y);
      }
    }
  }
}

template <int NT, int W>
static int launch_token_side_mma(float* x, const float* y0, const float* y1, const float* zg, int ldz, const int* tokens,
                                 const bf16* table, int ldt, int off, int vocab, const bf16* Wg, const bf16* Wp, const float* w,
                                 int rows, int d, int m, float eps, int* status, cudaStream_t stream) {
  const size_t smem = (size_t)16 * (d + 8) * 2 + (size_t)16 * (m + 8) * 2 + (W * 16 * 72 + W * 16) * sizeof(float) + 16 * sizeof(int);
  auto kern = token_side_mma_kernel<NT, W>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_k_class(launch_class_for_rows(rows, 0), kern, dim3((rows + 15) / 16), dim3(32 * W), smem, stream, 1, x, y0, y1, zg, ldz,
                        tokens, table, ldt, off, vocab, Wg, Wp, w, rows, d, m, eps, status);
}

// bfloat16 tables; d a multiple of 64 up to 2048, m a multiple of 16 up to 512, tables that start on 4 bytes.
// y0 (and y1) float32 [rows, d] with zg float32 [rows, >= d (2 d)]: x += y0 sigmoid(zg[:, :d]) (+ y1 sigmoid(zg[:, d:2d]))
// first, in the same launch (what gated_add does), and the side input is computed from that sum.
// Up to 16 rows (one block, a decode step): 16 warps where d is a multiple of 128, which halves the block's chains
// (the order of a row's sums then differs from the 8-warp form's: rounding).
FELLM_API int fellm_token_side_mma(float* x, const float* y0, const float* y1, const float* zg, int ldz, const int* tokens,
                                   const void* table, int ldt, int off, int vocab, const void* Wg, const void* Wp, const float* w,
                                   int rows, int d, int m, float eps, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!x || !tokens || !table || !Wg || !Wp || !w || (y0 && !zg) || (y1 && !y0)) return FELLM_ERR_ARG;
  if (d < 64 || d % 64 || d > 2048 || m < 16 || m % 16 || m > 512) return FELLM_ERR_SIZE;
  if ((((size_t)Wg | (size_t)Wp) & 3) || (((size_t)x | (size_t)y0 | (size_t)y1 | (size_t)zg) & 15) || ((size_t)w & 7) || (y0 && (ldz & 3))) return FELLM_ERR_ARG;
#define TS_LAUNCH(N_, W_) return launch_token_side_mma<N_, W_>(x, y0, y1, zg, ldz, tokens, (const bf16*)table, ldt, off, vocab, (const bf16*)Wg, (const bf16*)Wp, w, rows, d, m, eps, status, stream)
  if (rows <= 16 && d % 128 == 0) {
    const int nt = d / 128;
    if (nt <= 2) TS_LAUNCH(2, 16);
    if (nt <= 4) TS_LAUNCH(4, 16);
    if (nt <= 8) TS_LAUNCH(8, 16);
    TS_LAUNCH(16, 16);
  }
  const int nt = d / 64;
  if (nt <= 2) TS_LAUNCH(2, 8);
  if (nt <= 4) TS_LAUNCH(4, 8);
  if (nt <= 8) TS_LAUNCH(8, 8);
  if (nt <= 16) TS_LAUNCH(16, 8);
  TS_LAUNCH(32, 8);
#undef TS_LAUNCH
}

// ---------------------------------------------------------------- one stream added to another
// x += y   (float32; the embedding's output added again where a pass of a looped run of layers opens)
__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ y, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] += y[i];
}

FELLM_API int fellm_add_rows(float* x, const float* y, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!x || !y) return FELLM_ERR_ARG;
  long long blocks = (n + 255) / 256; if (blocks > fellm_sm_count() * 16) blocks = fellm_sm_count() * 16;
  add_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, y, n);
  return launch_status();
}
