// Causal GQA attention over the paged cache on CUDA cores, float32 arithmetic: the engine's
// 32-bit attention, and the yardstick of the tensor-core kernels.
//
// FeLLM counterpart: attention_paged_batch_heads, one thread per (row, head) with a serial
// online softmax over the row's length (plugins/cuda_kernels/src/oxide_kernels.rs:4271-4360;
// formulas crates/fellm-plugin-abi/src/attention_provider.rs:175-237): s_j = (q.k_j)*scale,
// m' = max(m, s), l = l*exp(m-m') + sum exp(s-m'), acc = acc*exp(m-m') + sum p_j v_j, out = acc/l.
//
// One block per (row, head), one to eight warps.  Keys are taken in tiles of 32 that start at the first visible
// position (0, position-window+1, or the start of the query's block of `chunk` positions), so the
// order of every sum depends on the query's position alone: not on the cut of the prompt, the
// batch, or the pages.
//
// Beyond FeLLM's attention the kernel takes: values of another size than keys (vd; a page-layer record is
// K [G][tokens][hd] followed by V [G][tokens][vd]), queries read in place from a wider row (ldq), a soft cap on
// the scores (cap * tanh(s / cap)), blocks of `chunk` positions that a query does not look out of, and a gate
// per (row, head) whose sigmoid scales the head's output; a bias by distance, slope[h] * (query position - key
// position) taken off the scaled score; a query temperature by position, q times
// 1 + coef * ln(floor((p + 1) / every) + 1); and values that ARE the keys (vd == 0 in the record: a page-layer
// record then holds the keys alone and the read-out has the keys' size).  kv_write puts a step's keys and values,
// as the product left them, into their pages; in a decode step the attention kernel does that itself (new_k_off).
// A sink per head: exp(sink) joins the softmax's denominator, with no key and no value; and, with values that are
// the keys, a read-out of only the first `od` elements of a key (a cache of latents with a positional tail: the
// tail enters the scores alone).
#include "common.cuh"

#define MAX_HD 1024

// A block per (row, head); its `nw` warps take the row's key tiles by turns (warp w: tiles w, w + nw, ...) and their
// partial results are added in the order of the warps.  nw is the caller's constant for a layer (from its window), never
// the batch's or the context's: the order of every sum depends on the query's position alone.
__device__ __forceinline__ void load8(const bf16* p, float* f) {
  const uint4 raw = *(const uint4*)p;
  const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
  for (int e = 0; e < 4; ++e) { float2 v = __bfloat1622float2(h[e]); f[2 * e] = v.x; f[2 * e + 1] = v.y; }
}
__device__ __forceinline__ void load8(const float* p, float* f) {
  *(float4*)f = *(const float4*)p;
  *(float4*)(f + 4) = *(const float4*)(p + 4);
}

// NACC: registers a lane keeps of the read-out (elements lane, lane + 32, ...): the value size over 32, rounded up.
template <typename TA, typename TC, bool VEC, int NACC>
__global__ void __launch_bounds__(256)
paged_attention_simt_kernel(const TA* __restrict__ q, const TC* __restrict__ pool,
                            const int* __restrict__ block_table, int max_pages,
                            const int* __restrict__ positions, const int* __restrict__ row_slot,
                            TA* __restrict__ out, int T, int H, int G, int hd, int page_tokens, int layer,
                            int layers_in_group, float scale, int window, int vd, int ldq, float softcap, int chunk,
                            const float* __restrict__ gate, int ldg, const float* __restrict__ slopes,
                            float qt_coef, int qt_every, int new_k_off, int new_v_off, int* __restrict__ status,
                            const float* __restrict__ sinks, int od) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_SIMT);
  // new_k_off >= 0: a decode step, every row its request's only row.  The row's own key (and value) is read from the
  // row itself, at columns new_k_off (new_v_off) of q's rows, and written into its page here by the first head of
  // its kv head: no kernel in front has to write the cache, and no block reads what another writes.
  const bool fused = new_k_off >= 0;
  extern __shared__ __align__(16) float qs[];       // [hd rounded up to 8] the query; then [nw][vd + 2] the warps' parts
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int row = blockIdx.x / H, h = blockIdx.x - row * H;
  const int g = h / (H / G);
  const TA* qr = q + (size_t)row * ldq + (size_t)h * hd;
  int pos = positions[row];
  const float qt = qt_every > 0 ? 1.0f + qt_coef * logf((float)((pos + 1) / qt_every + 1)) : 1.0f;
  for (int e = threadIdx.x; e < hd; e += blockDim.x) qs[e] = to_f(qr[e]) * qt;
  __syncthreads();
  const float slope = slopes ? slopes[h] : 0.f;
  const bool v_is_k = vd == 0;          // the values are the keys: nothing else is stored
  if (v_is_k) vd = hd;
  const int ov = (v_is_k && od > 0) ? od : vd;       // elements of a value that are read out (values that are keys: the first od)
  float* parts = qs + ((hd + 7) & ~7);
  const int* bt = block_table + (size_t)row_slot[row] * max_pages;
  int k_begin = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) k_begin = max(k_begin, (pos / chunk) * chunk);
  const size_t record = (size_t)G * page_tokens * (v_is_k ? hd : hd + vd);       // one page of one layer: keys, then values

  float m = -INFINITY, l = 0.f;
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

  for (int k0 = k_begin + 32 * w; k0 <= pos; k0 += 32 * nw) {
    int kj = k0 + lane;
    float s = -INFINITY;
    const TC* vrow = nullptr;
    if (kj <= pos) {
      int page = max(bt[kj / page_tokens], 0);      // an unmapped entry (-1) must never become an address
      const TC* rec = pool + ((size_t)page * layers_in_group + layer) * record;
      size_t tok = (size_t)g * page_tokens + (kj % page_tokens);
      const TC* krow = rec + tok * hd;
      vrow = v_is_k ? krow : rec + (size_t)G * page_tokens * hd + tok * vd;
      const bool own = fused && kj == pos;
      if (own) {
        krow = (const TC*)(q + (size_t)row * ldq + new_k_off + (size_t)g * hd);
        vrow = v_is_k ? krow : (const TC*)(q + (size_t)row * ldq + new_v_off + (size_t)g * vd);
      }
      float dot = 0.f;
      if (VEC && !own) {
        for (int e0 = 0; e0 < hd; e0 += 8) {
          float kf[8];
          load8(krow + e0, kf);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(qs[e0 + e], kf[e], dot);
        }
      } else {
        for (int e = 0; e < hd; ++e) dot = fmaf(qs[e], to_f(krow[e]), dot);
      }
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      s -= slope * (float)(pos - kj);
    }
    float m_new = fmaxf(m, warp_max(s));
    float p = kj <= pos ? expf(s - m_new) : 0.f;
    float corr = expf(m - m_new);                  // m = -inf on the first tile: exp(-inf) = 0
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    int n_valid = pos - k0 + 1 < 32 ? pos - k0 + 1 : 32;
#pragma unroll 4
    for (int j = 0; j < n_valid; ++j) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      const TC* vj = (const TC*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        int e = lane + 32 * i;
        if (e < ov) acc[i] = fmaf(pj, to_f(vj[e]), acc[i]);
      }
    }
  }
  if (fused && h % (H / G) == 0) {
    const int page = bt[pos / page_tokens];
    if (page < 0) {
      if (threadIdx.x == 0 && status) atomicExch(status, 2);
    } else {
      TC* rec = const_cast<TC*>(pool) + ((size_t)page * layers_in_group + layer) * record;
      const size_t tok = (size_t)g * page_tokens + (pos % page_tokens);
      const TA* kn = q + (size_t)row * ldq + new_k_off + (size_t)g * hd;
      for (int e = threadIdx.x; e < hd; e += blockDim.x) rec[tok * hd + e] = from_f<TC>(to_f(kn[e]));
      if (!v_is_k) {
        const TA* vn = q + (size_t)row * ldq + new_v_off + (size_t)g * vd;
        TC* vrec = rec + (size_t)G * page_tokens * hd;
        for (int e = threadIdx.x; e < vd; e += blockDim.x) vrec[tok * vd + e] = from_f<TC>(to_f(vn[e]));
      }
    }
  }
  if (nw > 1) {
    // the warps' parts, added in the order of the warps (a warp without a tile holds m = -inf, l = 0)
    float* mine = parts + (size_t)w * (ov + 2);
#pragma unroll
    for (int i = 0; i < NACC; ++i) { int e = lane + 32 * i; if (e < ov) mine[e] = acc[i]; }
    if (lane == 0) { mine[ov] = m; mine[ov + 1] = l; }
    __syncthreads();
    if (w != 0) return;
    float M = -INFINITY;
    for (int u = 0; u < nw; ++u) M = fmaxf(M, parts[(size_t)u * (ov + 2) + ov]);
    l = 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    for (int u = 0; u < nw; ++u) {
      const float* pu = parts + (size_t)u * (ov + 2);
      const float f = expf(pu[ov] - M);
      l = fmaf(pu[ov + 1], f, l);
#pragma unroll
      for (int i = 0; i < NACC; ++i) { int e = lane + 32 * i; if (e < ov) acc[i] = fmaf(pu[e], f, acc[i]); }
    }
    m = M;
  }
  if (sinks) {
    // a sink: one more term exp(sink) in the softmax's denominator, with no key and no value
    const float sk = sinks[h], M2 = fmaxf(m, sk), f = expf(m - M2);
    l = fmaf(l, f, expf(sk - M2));
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= f;
  }
  TA* o = out + ((size_t)row * H + h) * ov;
  float inv_l = 1.0f / l;
  if (gate) inv_l *= 1.0f / (1.0f + expf(-gate[(size_t)row * ldg + h]));
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    int e = lane + 32 * i;
    if (e < ov) o[e] = from_f<TA>(acc[i] * inv_l);
  }
}

// Keys and values of a step's rows into their pages: k at column k_off of a row of `src` (G x hd), v at v_off
// (G x vd).  A row whose page is not mapped writes nothing and sets the status word to 2.
template <typename TA, typename TC>
__global__ void kv_write_kernel(const TA* __restrict__ src, int ld, int k_off, int v_off, TC* __restrict__ pool,
                                const int* __restrict__ block_table, int max_pages, const int* __restrict__ positions,
                                const int* __restrict__ row_slot, int G, int hd, int vd, int page_tokens, int layer,
                                int layers_in_group, int* __restrict__ status) {
  const int row = blockIdx.x;
  const int pos = positions[row];
  const int page = block_table[(size_t)row_slot[row] * max_pages + pos / page_tokens];
  if (page < 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, 2);
    return;
  }
  const size_t record = (size_t)G * page_tokens * (hd + vd);
  TC* rec = pool + ((size_t)page * layers_in_group + layer) * record;
  const int in_page = pos % page_tokens;
  const TA* s = src + (size_t)row * ld;
  for (int e = threadIdx.x; e < G * hd; e += blockDim.x) {
    int g = e / hd, c = e - g * hd;
    rec[((size_t)g * page_tokens + in_page) * hd + c] = from_f<TC>(to_f(s[k_off + e]));
  }
  TC* vrec = rec + (size_t)G * page_tokens * hd;
  for (int e = threadIdx.x; e < G * vd; e += blockDim.x) {
    int g = e / vd, c = e - g * vd;
    vrec[((size_t)g * page_tokens + in_page) * vd + c] = from_f<TC>(to_f(s[v_off + e]));
  }
}

FELLM_API int fellm_kv_write(const void* src, int act_bf16, int ld, int k_off, int v_off, void* pool, int cache_bf16,
                             const int* block_table, int max_pages, const int* positions, const int* row_slot, int T,
                             int G, int hd, int vd, int page_tokens, int layer, int layers_in_group, int* status,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!src || !pool || !block_table || !positions || !row_slot) return FELLM_ERR_ARG;
  if (act_bf16 != cache_bf16) return FELLM_ERR_ARG;
  if (act_bf16)
    kv_write_kernel<bf16, bf16><<<T, 128, 0, stream>>>((const bf16*)src, ld, k_off, v_off, (bf16*)pool, block_table, max_pages,
                                                       positions, row_slot, G, hd, vd, page_tokens, layer, layers_in_group, status);
  else
    kv_write_kernel<float, float><<<T, 128, 0, stream>>>((const float*)src, ld, k_off, v_off, (float*)pool, block_table,
                                                         max_pages, positions, row_slot, G, hd, vd, page_tokens, layer,
                                                         layers_in_group, status);
  return launch_status();
}

FELLM_API int fellm_paged_attention_general(const void* q, int act_bf16, const void* pool, int cache_bf16,
                                            const int* block_table, int max_pages, const int* positions,
                                            const int* row_slot, void* out, int T, int H, int G, int hd,
                                            int page_tokens, int layer, int layers_in_group, float scale,
                                            int window, int vd, int ldq, float softcap, int chunk, const float* gate,
                                            int ldg, const float* slopes, float qt_coef, int qt_every, int warps,
                                            int new_k_off, int new_v_off, int* status, const float* sinks, int od,
                                            cudaStream_t stream) {
  // sinks float32 [H] or null: exp(sinks[h]) joins head h's softmax denominator.  od: with values that are the keys
  // (vd == 0), only the first od elements of a key are read out (0: all hd).
  if (T <= 0) return 0;
  if (hd < 1 || hd > MAX_HD || vd < 0 || vd > MAX_HD || warps < 1 || warps > 8) return FELLM_ERR_SIZE;
  if (od < 0 || od > hd || (od && vd)) return FELLM_ERR_SIZE;
  if (G < 1 || H % G) return FELLM_ERR_SIZE;
  if (!q || !pool || !block_table || !positions || !row_slot || !out) return FELLM_ERR_ARG;
  if (act_bf16 != cache_bf16) return FELLM_ERR_ARG;
  const int out_d = vd ? vd : (od ? od : hd);
  const size_t smem = ((size_t)((hd + 7) & ~7) + (size_t)warps * (out_d + 2)) * sizeof(float);
  const unsigned blocks = (unsigned)((long long)T * H);
  // 16 bytes of a key at a time where every key row starts on such a boundary
  const bool vec = hd % 8 == 0 && ((uintptr_t)pool % 16) == 0 && (vd == 0 || vd % 8 == 0);
#define PA(TA_, VEC_, NACC_) paged_attention_simt_kernel<TA_, TA_, VEC_, NACC_><<<blocks, warps * 32, smem, stream>>>((const TA_*)q, \
        (const TA_*)pool, block_table, max_pages, positions, row_slot, (TA_*)out, T, H, G, hd, page_tokens, \
        layer, layers_in_group, scale, window, vd, ldq, softcap, chunk, gate, ldg, slopes, qt_coef, qt_every, \
        new_k_off, new_v_off, status, sinks, od)
#define PA_N(TA_, VEC_) do { if (out_d <= 32) PA(TA_, VEC_, 1); else if (out_d <= 64) PA(TA_, VEC_, 2); \
                             else if (out_d <= 128) PA(TA_, VEC_, 4); else if (out_d <= 256) PA(TA_, VEC_, 8); \
                             else if (out_d <= 512) PA(TA_, VEC_, 16); else PA(TA_, VEC_, 32); } while (0)
  if (act_bf16) { if (vec) PA_N(bf16, true); else PA_N(bf16, false); }
  else { if (vec) PA_N(float, true); else PA_N(float, false); }
#undef PA_N
#undef PA
  return launch_status();
}

FELLM_API int fellm_paged_attention_simt(const void* q, int act_bf16, const void* pool, int cache_bf16,
                                         const int* block_table, int max_pages, const int* positions,
                                         const int* row_slot, void* out, int T, int H, int G, int hd,
                                         int page_tokens, int layer, int layers_in_group, float scale,
                                         int window, cudaStream_t stream) {
  return fellm_paged_attention_general(q, act_bf16, pool, cache_bf16, block_table, max_pages, positions, row_slot, out,
                                       T, H, G, hd, page_tokens, layer, layers_in_group, scale, window, hd, H * hd, 0.f,
                                       0, nullptr, 0, nullptr, 0.f, 0, 1, -1, -1, nullptr, nullptr, 0, stream);
}
