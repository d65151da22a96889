// Latent attention over the paged cache on tensor cores (mma.sync.m16n8k16, ldmatrix, cp.async): bfloat16 queries and
// cache rows, float32 scores, softmax and sums.  Compiled for one pair of sizes: -DLAT_RK (the latent, a multiple of
// 32 up to 512) and -DLAT_DR (the rotated key part; LAT_RK + LAT_DR a multiple of 16).
//
// A token's cache row is [c (RK) | rotated key part (DR)], one for all heads; a query row is [W_uk,h^T qn (RK) |
// rotated qr (DR)] per (token, head).  score = scale (query . row); the value of a key is the first RK elements of
// its row.  So all H heads of a token are rows of ONE product against the same keys: a CTA takes MQ = 16 NG
// consecutive (token, head) rows of one item, walks the keys its rows can see in tiles of KT = 16 NC, and its NG x NC
// warps split a tile two ways: warp (i, j) computes the scores of row group i against keys [16 j, 16 j + 16) of the
// tile and leaves them in shared memory; after a barrier it reads its group's scores for the whole tile, does the
// online softmax for them (the NC warps of a group do the same arithmetic and hold the same m and l), and adds
// P V for the value elements [j RK / NC, (j + 1) RK / NC), which it alone accumulates: a row's read-out of RK
// float32 sums lies across NC warps' registers.
//
//   NG = 4, NC = 2   portions of prompts: 64 rows, key tiles of 32 through a two-stage cp.async ring
//   NG = 1, NC = 4   single tokens (16 rows = the heads of a token), key tiles of 64; NC = 2 where RK / 4 is not a
//                    multiple of 16.  The key range can be split over gridDim.z CTAs, which leave (m, l, sums) in a
//                    scratch buffer that latent_merge_kernel puts together (a block a row: 8 x the parallelism of
//                    a merge by the CTA that finishes last, which was tried and cost 40 us a layer).
//
// A key counts for the row of a token at position p iff p - window < key <= p (window 0: every key up to p).  A
// sink per head joins the denominator once: exp(sink_h), not scaled, no value.  Rows of an item have consecutive
// positions; key tiles start at multiples of KT, so a tile lies in one page (page_tokens % KT == 0).
#include "common.cuh"

#ifndef LAT_RK
#define LAT_RK 512
#endif
#ifndef LAT_DR
#define LAT_DR 64
#endif

constexpr int RK = LAT_RK, DR = LAT_DR, D = RK + DR;
static_assert(RK % 32 == 0 && RK >= 32 && RK <= 512 && DR >= 0 && D % 16 == 0, "latent sizes the tensor-core kernel takes");
constexpr int CPR = D / 8;                          // 16-byte chunks per row
constexpr bool SWZ = (CPR % 8 == 0);                // rows of whole 128-byte lines: XOR swizzle
constexpr int ROWB = D * 2 + (SWZ ? 0 : 16);        // else 16 bytes of padding spread the banks
constexpr int KS = D / 16;                          // k16 steps over a row
constexpr float LOG2E = 1.4426950408889634f;
constexpr int MAX_SPLITS = 32;                     // ranges a single token's key walk is split into, at most

__device__ __forceinline__ int tile_off(int row, int chunk) {
  return row * ROWB + ((SWZ ? (chunk ^ (row & 7)) : chunk) << 4);
}
__device__ __forceinline__ void cp_async16(unsigned smem_addr, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem));
}
__device__ __forceinline__ void st_shared_zero16(unsigned smem_addr) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(smem_addr), "r"(0u));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
__device__ __forceinline__ void ldsm_x4(unsigned* r, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned* r, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(unsigned*)&v;
}

struct LatArgs {
  const bf16* q;            // [rows of all items][H][D]; with qsrc: [rows][H][RK], the rotated part comes from qsrc
  const bf16* qsrc;         // or null: [rows][ldq], head h's rotated part (DR elements, not yet rotated) at column h q_head + q_rot_off
  int ldq, q_head, q_rot_off, n_rot;
  const float* freq; float mag;      // pairs (2i, 2i + 1), i < n_rot / 2: angle = float(position) freq[i], cos and sin times mag
  const bf16* pool;         // [pages][layers_in_group][page_tokens][D]
  const int* block_table; int max_pages;
  const int* positions; const int* row_slot; const int* item_start;
  bf16* out;                // [rows][H][RK]
  float* scratch;           // n_splits > 1: [rows * H][n_splits][RK + 2]
  const float* sinks;       // [H] or null
  int H, page_tokens, layer, layers_in_group, window, n_splits;
  float scale_log2;
};

template <int NG, int NC>
__global__ void __launch_bounds__(NG * NC * 32, 1) latent_attention_kernel(LatArgs a) {
  constexpr int KT = 16 * NC, MQ = 16 * NG, NTH = NG * NC * 32, DVW = RK / NC, NT = DVW / 8, SLD = KT + 8, KK = KT / 16;
  static_assert(DVW % 16 == 0, "a warp's share of the value elements is a multiple of 16");
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, wi = warp / NC, wj = warp % NC, g = lane >> 2, c = lane & 3;
  const int item = blockIdx.y, H = a.H;
  const int r_begin = a.item_start[item];
  const int n_rows = (a.item_start[item + 1] - r_begin) * H;
  // (an item's last rows see the most keys: their CTAs start first, the short walks of its first rows fill the tail)
  const int R0 = (int)(gridDim.x - 1 - blockIdx.x) * MQ;
  if (R0 >= n_rows) return;
  const int rows_here = min(MQ, n_rows - R0);
  const int pos0 = a.positions[r_begin];
  const int* bt = a.block_table + (size_t)a.row_slot[r_begin] * a.max_pages;
  const int pos_lo = pos0 + R0 / H, pos_hi = pos0 + (R0 + rows_here - 1) / H;
  int key_begin = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
  key_begin &= ~(KT - 1);
  const int n_tiles = (pos_hi + 1 - key_begin + KT - 1) / KT;
  const int per = (n_tiles + a.n_splits - 1) / a.n_splits;
  const int t_begin = blockIdx.z * per, t_end = min(n_tiles, t_begin + per);

  const unsigned q_s = (unsigned)__cvta_generic_to_shared(smem), k_s = q_s + MQ * ROWB;
  float* S_s = (float*)(smem + (MQ + 2 * KT) * ROWB);

  // the CTA's query rows (rows beyond the item's end are zeros)
  {
    const int q_ld = a.qsrc ? RK : D;
    const bf16* qg = a.q + ((size_t)r_begin * H + R0) * q_ld;
    for (int ch = tid; ch < MQ * CPR; ch += NTH) {
      const int r = ch / CPR, cc = ch - r * CPR;
      if (r >= rows_here) st_shared_zero16(q_s + tile_off(r, cc));
      else if (cc < RK / 8 || !a.qsrc) cp_async16(q_s + tile_off(r, cc), qg + (size_t)r * q_ld + cc * 8);
      else {
        // eight elements of the head's rotated part, rotated by the row's position on their way in
        const int R = R0 + r, t = R / H, h = R - t * H, e0 = (cc - RK / 8) * 8;
        uint4 raw = *(const uint4*)(a.qsrc + (size_t)(r_begin + t) * a.ldq + (size_t)h * a.q_head + a.q_rot_off + e0);
        __nv_bfloat162* pr = (__nv_bfloat162*)&raw;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (e0 + 2 * i < a.n_rot) {
            float2 uv = __bfloat1622float2(pr[i]);
            float sn, cs;
            sincosf((float)(pos0 + t) * a.freq[(e0 >> 1) + i], &sn, &cs);
            sn *= a.mag; cs *= a.mag;
            pr[i] = __floats2bfloat162_rn(uv.x * cs - uv.y * sn, uv.y * cs + uv.x * sn);
          }
        }
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(q_s + tile_off(r, cc)), "r"(raw.x), "r"(raw.y), "r"(raw.z), "r"(raw.w));
      }
    }
  }
  // keys beyond the last visible one are zeros: they are masked, but a value of a freed page's bits must not
  // reach a product (0 * NaN)
  auto load_tile = [&](int t, int buf) {
    const int k0 = key_begin + t * KT;
    const int page = max(bt[k0 / a.page_tokens], 0);
    const bf16* src = a.pool + (((size_t)page * a.layers_in_group + a.layer) * a.page_tokens + (k0 % a.page_tokens)) * D;
    const unsigned dst = k_s + buf * KT * ROWB;
    const int n_keys = min(KT, pos_hi + 1 - k0);
    for (int ch = tid; ch < KT * CPR; ch += NTH) {
      const int r = ch / CPR, cc = ch - r * CPR;
      if (r < n_keys) cp_async16(dst + tile_off(r, cc), src + (size_t)r * D + cc * 8);
      else st_shared_zero16(dst + tile_off(r, cc));
    }
  };

  // rows g and g + 8 of the warp's group
  const int Rg0 = R0 + wi * 16 + g, Rg1 = Rg0 + 8;
  const int hi0 = pos0 + min(Rg0, n_rows - 1) / H, hi1 = pos0 + min(Rg1, n_rows - 1) / H;
  const int lo0 = a.window > 0 ? hi0 - a.window + 1 : 0, lo1 = a.window > 0 ? hi1 - a.window + 1 : 0;
  const int grp_lo = pos0 + min(R0 + wi * 16, n_rows - 1) / H, grp_hi = pos0 + min(R0 + wi * 16 + 15, n_rows - 1) / H;
  const int grp_first = a.window > 0 ? grp_lo - a.window + 1 : 0;

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  if (t_begin < t_end) load_tile(t_begin, 0);
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    const int buf = (t - t_begin) & 1;
    cp_async_wait_all();
    __syncthreads();                   // tile t has landed; everyone is done with the other buffer and with S_s
    if (t + 1 < t_end) load_tile(t + 1, buf ^ 1);
    cp_async_commit();
    const int k0 = key_begin + t * KT;
    const bool live = k0 <= grp_hi && k0 + KT - 1 >= grp_first;        // some row of the group sees some key of the tile
    const unsigned kb = k_s + buf * KT * ROWB;
    if (live) {
      float s[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 6
      for (int ks = 0; ks < KS; ++ks) {
        unsigned af[4], bq[4];
        ldsm_x4(af, q_s + tile_off(wi * 16 + (lane & 15), 2 * ks + (lane >> 4)));
        ldsm_x4(bq, kb + tile_off(wj * 16 + (lane & 7) + ((lane >> 4) << 3), 2 * ks + ((lane >> 3) & 1)));
        mma16816(s[0], af, bq[0], bq[1]);
        mma16816(s[1], af, bq[2], bq[3]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float* d0 = S_s + (wi * 16 + g) * SLD + wj * 16 + 8 * i + 2 * c;
        *(float2*)d0 = make_float2(s[i][0], s[i][1]);
        *(float2*)(d0 + 8 * SLD) = make_float2(s[i][2], s[i][3]);
      }
    }
    __syncthreads();
    if (!live) continue;
    // the group's scores for the whole tile, in the layout of the P V product's first operand
    float p0[KK][4], p1[KK][4];
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int col = 16 * kk + 8 * hf + 2 * c;
        const float2 v0 = *(const float2*)(S_s + (wi * 16 + g) * SLD + col);
        const float2 v1 = *(const float2*)(S_s + (wi * 16 + g + 8) * SLD + col);
        const int kj = k0 + col;
        p0[kk][2 * hf] = (kj <= hi0 && kj >= lo0) ? v0.x * a.scale_log2 : -INFINITY;
        p0[kk][2 * hf + 1] = (kj + 1 <= hi0 && kj + 1 >= lo0) ? v0.y * a.scale_log2 : -INFINITY;
        p1[kk][2 * hf] = (kj <= hi1 && kj >= lo1) ? v1.x * a.scale_log2 : -INFINITY;
        p1[kk][2 * hf + 1] = (kj + 1 <= hi1 && kj + 1 >= lo1) ? v1.y * a.scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(p0[kk][2 * hf], p0[kk][2 * hf + 1]));
        mx1 = fmaxf(mx1, fmaxf(p1[kk][2 * hf], p1[kk][2 * hf + 1]));
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;      // a row that has seen nothing yet
    const float corr0 = exp2f(m0 - mu0), corr1 = exp2f(m1 - mu1);
    m0 = mn0; m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
    unsigned pa[KK][4];
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p0[kk][e] = exp2f(p0[kk][e] - mu0); sum0 += p0[kk][e];
        p1[kk][e] = exp2f(p1[kk][e] - mu1); sum1 += p1[kk][e];
      }
      pa[kk][0] = pack_bf16(p0[kk][0], p0[kk][1]); pa[kk][1] = pack_bf16(p1[kk][0], p1[kk][1]);
      pa[kk][2] = pack_bf16(p0[kk][2], p0[kk][3]); pa[kk][3] = pack_bf16(p1[kk][2], p1[kk][3]);
    }
    l0 = l0 * corr0 + sum0; l1 = l1 * corr1 + sum1;
#pragma unroll
    for (int n = 0; n < NT; ++n) { o[n][0] *= corr0; o[n][1] *= corr0; o[n][2] *= corr1; o[n][3] *= corr1; }
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        unsigned vb[4];
        ldsm_x4_trans(vb, kb + tile_off(16 * kk + (lane & 7) + (((lane >> 3) & 1) << 3), wj * (DVW / 8) + 2 * n2 + (lane >> 4)));
        mma16816(o[2 * n2], pa[kk], vb[0], vb[1]);
        mma16816(o[2 * n2 + 1], pa[kk], vb[2], vb[3]);
      }
    }
  }
  cp_async_wait_all();

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const size_t row_g0 = (size_t)r_begin * H + Rg0;         // the (token, head) row among all rows of the step
  if (a.n_splits == 1) {
    if (a.sinks) {
      l0 += exp2f(a.sinks[Rg0 % H] * LOG2E - m0);
      l1 += exp2f(a.sinks[Rg1 % H] * LOG2E - m1);
    }
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int col = wj * DVW + 8 * n + 2 * c;
      if (Rg0 < n_rows) *(__nv_bfloat162*)(a.out + row_g0 * RK + col) = __floats2bfloat162_rn(o[n][0] * inv0, o[n][1] * inv0);
      if (Rg1 < n_rows) *(__nv_bfloat162*)(a.out + (row_g0 + 8) * RK + col) = __floats2bfloat162_rn(o[n][2] * inv1, o[n][3] * inv1);
    }
  } else {
    float* r0 = a.scratch + (row_g0 * a.n_splits + blockIdx.z) * (RK + 2);
    float* r1 = a.scratch + ((row_g0 + 8) * a.n_splits + blockIdx.z) * (RK + 2);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int col = wj * DVW + 8 * n + 2 * c;
      if (Rg0 < n_rows) *(float2*)(r0 + col) = make_float2(o[n][0], o[n][1]);
      if (Rg1 < n_rows) *(float2*)(r1 + col) = make_float2(o[n][2], o[n][3]);
    }
    if (wj == 0 && c == 0) {
      if (Rg0 < n_rows) { r0[RK] = m0; r0[RK + 1] = l0; }
      if (Rg1 < n_rows) { r1[RK] = m1; r1[RK + 1] = l1; }
    }
  }
}

// The ranges of a split key walk put together, in the order of the ranges: out = sum_s O_s 2^(m_s - m) / (sum_s l_s
// 2^(m_s - m) + 2^(sink - m)), m = max_s m_s.  A block per (token, head) row.
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ scratch, bf16* __restrict__ out,
                                                           const float* __restrict__ sinks, int H, int n_splits) {
  __shared__ float sm_m[MAX_SPLITS], sm_w[MAX_SPLITS];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* base = scratch + row * n_splits * (RK + 2);
  if (threadIdx.x < n_splits) {                    // every range's (m, l) at once
    sm_m[threadIdx.x] = base[(size_t)threadIdx.x * (RK + 2) + RK];
    sm_w[threadIdx.x] = base[(size_t)threadIdx.x * (RK + 2) + RK + 1];
  }
  __syncthreads();
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, sm_m[s]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += sm_m[s] > -INFINITY ? sm_w[s] * exp2f(sm_m[s] - m) : 0.f;
  if (sinks) L += exp2f(sinks[row % H] * LOG2E - m);
  const float inv = 1.0f / L;
  __syncthreads();
  if (threadIdx.x < n_splits) sm_w[threadIdx.x] = sm_m[threadIdx.x] > -INFINITY ? exp2f(sm_m[threadIdx.x] - m) : 0.f;
  __syncthreads();
  for (int e = threadIdx.x; e < RK; e += blockDim.x) {
    float acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < n_splits; ++s) acc = fmaf(base[(size_t)s * (RK + 2) + e], sm_w[s], acc);
    out[row * RK + e] = __float2bfloat16_rn(acc * inv);
  }
}

template <int NG, int NC>
static int launch_latent(const LatArgs& a, int n_items, int max_item_rows, int rows_total, cudaStream_t stream) {
  constexpr int KT = 16 * NC, MQ = 16 * NG;
  if (a.page_tokens % KT) return FELLM_ERR_SIZE;
  const size_t smem = (size_t)(MQ + 2 * KT) * ROWB + (size_t)MQ * (KT + 8) * sizeof(float);
  auto kern = latent_attention_kernel<NG, NC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(ceil_div(max_item_rows * a.H, MQ), n_items, a.n_splits);
  const int cls = launch_class_for_rows(rows_total, 0);
  int rc = launch_k_class(cls, kern, grid, dim3(NG * NC * 32), smem, stream, 1, a);
  if (rc || a.n_splits == 1) return rc;
  return launch_k_class(cls, latent_merge_kernel, dim3(rows_total * a.H), dim3(128), 0, stream, 1, (const float*)a.scratch, a.out,
                        a.sinks, a.H, a.n_splits);
}

FELLM_API int fellm_latent_attention_rk() { return RK; }
FELLM_API int fellm_latent_attention_dr() { return DR; }
// the key tile of a variant (0: portions, 1: single tokens): pages hold a multiple of it
FELLM_API int fellm_latent_attention_key_tile(int variant) { return variant != 1 ? 32 : (RK % 64 == 0 ? 64 : 32); }

// variant 0: 64 rows a CTA (portions of prompts), n_splits must be 1; variant 1: 16 rows a CTA (single tokens),
// qsrc (or null): the queries' rotated parts are read from there and rotated in the kernel, and q holds the RK
// elements of a (token, head) row alone.  n_splits >= 1 (up to 32) with scratch of rows * H * n_splits * (RK + 2) floats when above 1.
FELLM_API int fellm_latent_attention_mma(const void* q, const void* pool, const int* block_table, int max_pages,
                                         const int* positions, const int* row_slot, const int* item_start, int n_items,
                                         int max_item_rows, int rows_total, void* out, float* scratch, int n_splits, int H,
                                         int page_tokens, int layer, int layers_in_group, float scale, int window,
                                         const float* sinks, int variant, const void* qsrc, int ldq, int q_head, int q_rot_off,
                                         const float* freq, int n_rot, float mag, cudaStream_t stream) {
  if (n_items <= 0 || rows_total <= 0 || max_item_rows <= 0) return 0;
  if (!q || !pool || !block_table || !positions || !row_slot || !item_start || !out) return FELLM_ERR_ARG;
  if (H < 1 || page_tokens < 1 || n_splits < 1 || n_splits > MAX_SPLITS || (n_splits > 1 && (!scratch || variant != 1))) return FELLM_ERR_ARG;
  if (qsrc && ((ldq | q_head | q_rot_off) % 8 || ((size_t)qsrc & 15) || n_rot < 0 || n_rot > DR || (n_rot & 1) || (n_rot && !freq))) return FELLM_ERR_SIZE;
  LatArgs a;
  a.qsrc = DR ? (const bf16*)qsrc : nullptr; a.ldq = ldq; a.q_head = q_head; a.q_rot_off = q_rot_off; a.n_rot = n_rot; a.freq = freq; a.mag = mag;
  a.q = (const bf16*)q; a.pool = (const bf16*)pool; a.block_table = block_table; a.max_pages = max_pages;
  a.positions = positions; a.row_slot = row_slot; a.item_start = item_start; a.out = (bf16*)out; a.scratch = scratch;
  a.sinks = sinks; a.H = H; a.page_tokens = page_tokens; a.layer = layer; a.layers_in_group = layers_in_group;
  a.window = window > 0 ? window : 0; a.n_splits = n_splits; a.scale_log2 = scale * LOG2E;
  if (variant == 0) return launch_latent<4, 2>(a, n_items, max_item_rows, rows_total, stream);
  if constexpr (RK % 64 == 0) return launch_latent<1, 4>(a, n_items, max_item_rows, rows_total, stream);
  else return launch_latent<1, 2>(a, n_items, max_item_rows, rows_total, stream);
}
