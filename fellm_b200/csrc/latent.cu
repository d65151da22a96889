// What a latent-attention layer does between its products: the cache keeps, per token, ONE normed key-value latent
// of rk elements followed by ONE rotated key part of dr elements, shared by all heads; queries come from a normed
// latent of their own.
//
//   latent_prep       z [T, ldz] float32, the sums of the layer's down projections: the query latent (rq elements at
//                     q_off) over its root mean square times a weight -> cq in the activation dtype; the key-value
//                     latent (rk at c_off) likewise -> elements [0, rk) of the token's cache row; the key part (dr at
//                     r_off), rotated by the token's position -> elements [rk, rk + dr) of the cache row.
//   latent_rotate_q   the rotated part (dr elements behind the dn unrotated ones) of every head's query, rotated by
//                     the row's position, into elements [rk, rk + dr) of the head's row of q_abs [T, H, rk + dr], whose
//                     first rk elements a per-head product fills (the query taken into the latent's space).
//
// Rotation: pairs (2i, 2i + 1) for i < n_rot / 2; angle = float(position) * freq[i] in float32; cos and sin times
// `mag`; elements from n_rot on pass unchanged.  freq is a table the host made (scaled frequencies included).
// Norms, angles and the rotation are float32 in both engines.
#include "common.cuh"

// (u, v) at pair i of a row at position pos
__device__ __forceinline__ void rotate_pair(float& u, float& v, int pos, float f, float mag) {
  float sn, cs;
  sincosf((float)pos * f, &sn, &cs);
  sn *= mag; cs *= mag;
  const float a = u * cs - v * sn, b = v * cs + u * sn;
  u = a; v = b;
}

template <typename TO, typename TC>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const float* __restrict__ z, int ldz, int q_off, int rq, int c_off, int rk, int r_off, int dr,
                   const float* __restrict__ wq, const float* __restrict__ wc, float eps,
                   const float* __restrict__ freq, int n_rot, float mag,
                   const int* __restrict__ positions, const int* __restrict__ row_slot,
                   const int* __restrict__ block_table, int max_pages, TC* __restrict__ pool, int page_tokens, int layer,
                   int layers_in_group, TO* __restrict__ cq, int* __restrict__ status) {
  __shared__ float scratch[68];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const float* zr = z + (size_t)row * ldz;
  // (the page's number is asked for first: its two dependent loads run under the sums)
  const int pos = positions[row];
  const int page = block_table[(size_t)row_slot[row] * max_pages + pos / page_tokens];
  // both latents' sums of squares in one reduction: a thread's share in order, the warps in order
  float sq_ = 0.f, sc_ = 0.f;
  for (int i = threadIdx.x; i < rq; i += blockDim.x) { const float v = zr[q_off + i]; sq_ = fmaf(v, v, sq_); }
  for (int i = threadIdx.x; i < rk; i += blockDim.x) { const float v = zr[c_off + i]; sc_ = fmaf(v, v, sc_); }
  sq_ = warp_sum(sq_); sc_ = warp_sum(sc_);
  if ((threadIdx.x & 31) == 0) { scratch[threadIdx.x >> 5] = sq_; scratch[32 + (threadIdx.x >> 5)] = sc_; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) { a += scratch[i]; b += scratch[32 + i]; }
    scratch[64] = a; scratch[65] = b;
  }
  __syncthreads();
  const float sq = 1.0f / sqrtf(scratch[64] / (float)rq + eps), sc = 1.0f / sqrtf(scratch[65] / (float)rk + eps);
  // the query latent
  for (int i = threadIdx.x; i < rq; i += blockDim.x) cq[(size_t)row * rq + i] = from_f<TO>((zr[q_off + i] * sq) * wq[i]);
  // the key-value latent and the rotated key part into the token's cache row
  if (page < 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, 2);
    return;
  }
  const int D = rk + dr;
  TC* rec = pool + (((size_t)page * layers_in_group + layer) * page_tokens + (pos % page_tokens)) * D;
  for (int i = threadIdx.x; i < rk; i += blockDim.x) rec[i] = from_f<TC>((zr[c_off + i] * sc) * wc[i]);
  for (int i = threadIdx.x; i < n_rot / 2; i += blockDim.x) {
    float u = zr[r_off + 2 * i], v = zr[r_off + 2 * i + 1];
    rotate_pair(u, v, pos, freq[i], mag);
    rec[rk + 2 * i] = from_f<TC>(u); rec[rk + 2 * i + 1] = from_f<TC>(v);
  }
  for (int i = n_rot + threadIdx.x; i < dr; i += blockDim.x) rec[rk + i] = from_f<TC>(zr[r_off + i]);
}

FELLM_API int fellm_latent_prep(const float* z, int ldz, int q_off, int rq, int c_off, int rk, int r_off, int dr,
                                const float* wq, const float* wc, float eps, const float* freq, int n_rot, float mag,
                                const int* positions, const int* row_slot, const int* block_table, int max_pages,
                                void* pool, int bf16_, int page_tokens, int layer, int layers_in_group, void* cq, int T,
                                int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!z || !wq || !wc || !positions || !row_slot || !block_table || !pool || !cq) return FELLM_ERR_ARG;
  if (rq < 1 || rk < 1 || dr < 0 || n_rot < 0 || n_rot > dr || (n_rot & 1) || (n_rot && !freq)) return FELLM_ERR_SIZE;
  const int cls = launch_class_for_rows(T, 0);
  if (bf16_)
    return launch_k_class(cls, latent_prep_kernel<bf16, bf16>, dim3(T), dim3(128), 0, stream, 1, z, ldz, q_off, rq, c_off, rk, r_off, dr,
                          wq, wc, eps, freq, n_rot, mag, positions, row_slot, block_table, max_pages, (bf16*)pool, page_tokens,
                          layer, layers_in_group, (bf16*)cq, status);
  return launch_k_class(cls, latent_prep_kernel<float, float>, dim3(T), dim3(128), 0, stream, 1, z, ldz, q_off, rq, c_off, rk, r_off, dr,
                        wq, wc, eps, freq, n_rot, mag, positions, row_slot, block_table, max_pages, (float*)pool, page_tokens,
                        layer, layers_in_group, (float*)cq, status);
}

template <typename TA>
__global__ void __launch_bounds__(128)
latent_rotate_q_kernel(const TA* __restrict__ q, int ldq, int H, int dn, int dr, TA* __restrict__ q_abs, int rk,
                       const float* __restrict__ freq, int n_rot, float mag, const int* __restrict__ positions) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, pos = positions[row];
  const TA* qr = q + (size_t)row * ldq;
  TA* o = q_abs + (size_t)row * H * (rk + dr);
  const int half = n_rot / 2, rest = dr - n_rot;
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    const TA* src = qr + (size_t)h * (dn + dr) + dn + 2 * p;
    float u = to_f(src[0]), v = to_f(src[1]);
    rotate_pair(u, v, pos, freq[p], mag);
    TA* dst = o + (size_t)h * (rk + dr) + rk + 2 * p;
    dst[0] = from_f<TA>(u); dst[1] = from_f<TA>(v);
  }
  for (int i = threadIdx.x; i < H * rest; i += blockDim.x) {
    const int h = i / rest, p = n_rot + (i - h * rest);
    o[(size_t)h * (rk + dr) + rk + p] = qr[(size_t)h * (dn + dr) + dn + p];
  }
}

FELLM_API int fellm_latent_rotate_q(const void* q, int bf16_, int ldq, int H, int dn, int dr, void* q_abs, int rk,
                                    const float* freq, int n_rot, float mag, const int* positions, int T,
                                    cudaStream_t stream) {
  if (T <= 0 || dr == 0) return 0;
  if (!q || !q_abs || !positions) return FELLM_ERR_ARG;
  if (H < 1 || dn < 0 || dr < 0 || rk < 1 || n_rot < 0 || n_rot > dr || (n_rot & 1) || (n_rot && !freq)) return FELLM_ERR_SIZE;
  const int cls = launch_class_for_rows(T, 0);
  if (bf16_)
    return launch_k_class(cls, latent_rotate_q_kernel<bf16>, dim3(T), dim3(128), 0, stream, 1, (const bf16*)q, ldq, H, dn, dr,
                          (bf16*)q_abs, rk, freq, n_rot, mag, positions);
  return launch_k_class(cls, latent_rotate_q_kernel<float>, dim3(T), dim3(128), 0, stream, 1, (const float*)q, ldq, H, dn, dr,
                        (float*)q_abs, rk, freq, n_rot, mag, positions);
}
