// Recurrent mixers: what runs between their matrix products.
//
//   causal_conv_act    short causal convolution per channel over portions, then SiLU; history in a state slot
//   token_shift_mix    h + (h_prev - h) * mu_s for several mixes s; the previous row in a state slot
//   lowrank_expand     out = f_out(W2 f_in(z) + bias): the second factor of a low-rank projection, float32
//   delta_scan         gated delta rule:  S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q
//   decay_bonus_scan   o = (S + diag(u) k v^T)^T r; S = diag(w) S + k v^T   (per-channel decay, bonus for the current token)
//   retention_scan     S = decay_h S + k v^T; o = S^T q, q and k rotated by position
//   gated_write_scan   S = diag(f) S + (1 - f) v^T; o = S^T q: the forget gate also weighs what is written
//   token_shift        h + (h_prev - h) * mu from float32 rows into the activation dtype
//   head_norm_gate     per head: o / rms(o) * weight * act(gate)
//   branch_combine     x += mean over branches of rms_unit(branch) * weight
//
// FeLLM's GatedDeltaNet keeps the same two things between steps, a convolution history and a matrix
// (crates/fellm-model/src/graph.rs:792-806), and runs one token per request and step; here a request
// brings a portion of any length and its state after the portion equals the state after the same
// tokens one by one: every sum below runs in an order that depends on the sizes alone, not on where
// a prompt was cut, on the batch, or on the slot.
//
// States, decays, gates of the recurrences, unit norms and every sum are float32 in both engine dtypes.
#include "common.cuh"

#define MAX_TAPS 8
#define CH_TILE 32

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------- short causal convolution + activation
// grid (channel tiles, items, row tiles), block (CH_TILE, row lanes).  out[t, c] = act(sum_j taps[c, j] in[t - (L-1) + j, c]);
// inputs before the portion come from the slot's history (the last L-1 inputs; zeros for a new request).  The block of
// row tile 0 is the only one that touches the slot: it reads the history before its rows and, behind a barrier, writes
// the portion's last L-1 inputs there (no other block reads the slot, so no block can see the new history too early).
#define ROW_TILE 64
template <typename TA>
__global__ void causal_conv_act_kernel(const TA* __restrict__ x, int ldx, const float* __restrict__ taps, int L,
                                       float* __restrict__ state, long long slot_stride,
                                       const int* __restrict__ item_start, const int* __restrict__ item_slot,
                                       TA* __restrict__ out, int ldo, int C, int act) {
  __shared__ float hist[MAX_TAPS - 1][CH_TILE];
  const int item = blockIdx.y, tx = threadIdx.x;
  const int c = blockIdx.x * CH_TILE + tx;
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  const int tile0 = blockIdx.z * ROW_TILE;
  if (tile0 >= n && blockIdx.z > 0) return;
  const bool first = blockIdx.z == 0;
  float* st = state + (size_t)item_slot[item] * slot_stride;
  const bool live = c < C;
  if (first) {
    if (threadIdx.y == 0 && live)
      for (int j = 0; j < L - 1; ++j) hist[j][tx] = st[(size_t)j * C + c];
    __syncthreads();
  }
  float w[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) w[j] = (live && j < L) ? taps[(size_t)c * L + j] : 0.f;
  if (live) {
    const int r_end = min(n, tile0 + ROW_TILE);
    for (int r = tile0 + threadIdx.y; r < r_end; r += blockDim.y) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < MAX_TAPS; ++j) {
        if (j < L) {
          int idx = r - (L - 1) + j;
          float v = idx >= 0 ? to_f(x[(size_t)(r0 + idx) * ldx + c]) : hist[L - 1 + idx][tx];     // (idx < 0 only in row tile 0)
          acc = fmaf(w[j], v, acc);
        }
      }
      out[(size_t)(r0 + r) * ldo + c] = from_f<TA>(act == 1 ? silu_f(acc) : acc);
    }
  }
  if (!first) return;
  __syncthreads();
  if (threadIdx.y == 0 && live) {
    float keep[MAX_TAPS - 1];
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j) {
      if (j < L - 1) {
        int idx = n - (L - 1) + j;
        keep[j] = idx >= 0 ? to_f(x[(size_t)(r0 + idx) * ldx + c]) : hist[L - 1 + idx][tx];
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
      if (j < L - 1) st[(size_t)j * C + c] = keep[j];
  }
}

FELLM_API int fellm_causal_conv_act(const void* x, int is_bf16, int ldx, const float* taps, int L, float* state,
                                    long long slot_stride, const int* item_start, const int* item_slot, void* out,
                                    int ldo, int n_items, int C, int act, int max_item_rows, cudaStream_t stream) {
  if (n_items <= 0 || C <= 0) return 0;
  if (L < 1 || L > MAX_TAPS) return FELLM_ERR_SIZE;
  if (!x || !taps || (!state && L > 1) || !item_start || !item_slot || !out) return FELLM_ERR_ARG;
  if (max_item_rows < 1) max_item_rows = 1;
  dim3 grid(ceil_div(C, CH_TILE), n_items, ceil_div(max_item_rows, ROW_TILE)), block(CH_TILE, max_item_rows == 1 ? 1 : 8);
  if (is_bf16)
    causal_conv_act_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)x, ldx, taps, L, state, slot_stride, item_start,
                                                             item_slot, (bf16*)out, ldo, C, act);
  else
    causal_conv_act_kernel<float><<<grid, block, 0, stream>>>((const float*)x, ldx, taps, L, state, slot_stride, item_start,
                                                              item_slot, (float*)out, ldo, C, act);
  return launch_status();
}

// ---------------------------------------------------------------- token shift
// out[s][t][c] = h[t][c] + (h[t-1][c] - h[t][c]) * mu[s][c]; the row before a portion is the slot's state, which
// then takes the portion's last row.  Same grid as the convolution; row tile 0 reads the slot and then writes it.
template <typename TA, typename TO = TA>
__global__ void token_shift_mix_kernel(const TA* __restrict__ h, const float* __restrict__ mu, int n_mix,
                                       float* __restrict__ state, long long slot_stride,
                                       const int* __restrict__ item_start, const int* __restrict__ item_slot,
                                       TO* __restrict__ out, int T, int d) {
  const int item = blockIdx.y;
  const int c = blockIdx.x * CH_TILE + threadIdx.x;
  if (c >= d) return;
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  const int tile0 = blockIdx.z * ROW_TILE;
  if (tile0 >= n) return;
  float* st = state + (size_t)item_slot[item] * slot_stride;
  const bool owner = blockIdx.z == 0 && threadIdx.y == 0;       // row 0 is this thread's, and so is the slot
  const float first_prev = owner ? st[c] : 0.f;
  const int r_end = min(n, tile0 + ROW_TILE);
  for (int r = tile0 + threadIdx.y; r < r_end; r += blockDim.y) {
    float cur = to_f(h[(size_t)(r0 + r) * d + c]);
    float prev = r > 0 ? to_f(h[(size_t)(r0 + r - 1) * d + c]) : first_prev;
    float diff = prev - cur;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * T + r0 + r) * d + c] = from_f<TO>(fmaf(diff, mu[(size_t)s * d + c], cur));
  }
  if (owner) st[c] = to_f(h[(size_t)(r0 + n - 1) * d + c]);
}

FELLM_API int fellm_token_shift_mix(const void* h, int is_bf16, const float* mu, int n_mix, float* state,
                                    long long slot_stride, const int* item_start, const int* item_slot, void* out,
                                    int T, int n_items, int d, int max_item_rows, cudaStream_t stream) {
  if (n_items <= 0 || d <= 0) return 0;
  if (!h || !mu || !state || !item_start || !item_slot || !out || n_mix < 1) return FELLM_ERR_ARG;
  if (max_item_rows < 1) max_item_rows = 1;
  dim3 grid(ceil_div(d, CH_TILE), n_items, ceil_div(max_item_rows, ROW_TILE)), block(CH_TILE, max_item_rows == 1 ? 1 : 8);
  if (is_bf16)
    token_shift_mix_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)h, mu, n_mix, state, slot_stride, item_start,
                                                             item_slot, (bf16*)out, T, d);
  else
    token_shift_mix_kernel<float><<<grid, block, 0, stream>>>((const float*)h, mu, n_mix, state, slot_stride, item_start,
                                                              item_slot, (float*)out, T, d);
  return launch_status();
}

// The same from float32 rows (a residual stream that a sublayer reads as it is) into the activation dtype: the slot keeps
// the float32 row, the mix is rounded once.
// d % 4 == 0 and the rows' items known (row_item): a thread four channels of a row, 16-byte loads.  The thread of an item's
// FIRST row is the only one that touches the slot: it reads the row in front from there and then leaves the item's last row.
template <typename TO>
__global__ void __launch_bounds__(256)
token_shift_vec_kernel(const float* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state, long long slot_stride,
                       const int* __restrict__ item_start, const int* __restrict__ item_slot, const int* __restrict__ row_item,
                       TO* __restrict__ out, int T, int d) {
  const int nv = d >> 2;
  const size_t n = (size_t)T * nv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / nv), c = (int)(i - (size_t)row * nv);
    const int item = row_item[row], r0 = item_start[item];
    const float4 cur = ((const float4*)(h + (size_t)row * d))[c], m = ((const float4*)mu)[c];
    float4 prev;
    if (row == r0) {
      float4* st = (float4*)(state + (size_t)item_slot[item] * slot_stride) + c;
      prev = *st;
      *st = ((const float4*)(h + (size_t)(item_start[item + 1] - 1) * d))[c];
    } else {
      prev = ((const float4*)(h + (size_t)(row - 1) * d))[c];
    }
    const float4 o = make_float4(fmaf(prev.x - cur.x, m.x, cur.x), fmaf(prev.y - cur.y, m.y, cur.y),
                                 fmaf(prev.z - cur.z, m.z, cur.z), fmaf(prev.w - cur.w, m.w, cur.w));
    TO* op = out + (size_t)row * d + 4 * c;
    if (sizeof(TO) == 4) {
      *(float4*)op = o;
    } else {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(o.x, o.y), p1 = __floats2bfloat162_rn(o.z, o.w);
      uint2 u; u.x = *(unsigned*)&p0; u.y = *(unsigned*)&p1;
      *(uint2*)op = u;
    }
  }
}

FELLM_API int fellm_token_shift(const float* h, const float* mu, float* state, long long slot_stride, const int* item_start,
                                const int* item_slot, const int* row_item, void* out, int out_is_bf16, int T, int n_items, int d,
                                int max_item_rows, cudaStream_t stream) {
  if (n_items <= 0 || d <= 0) return 0;
  if (!h || !mu || !state || !item_start || !item_slot || !out) return FELLM_ERR_ARG;
  if (row_item && d % 4 == 0 && slot_stride % 4 == 0 &&
      (((uintptr_t)h | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)out) & 15) == 0) {
    const size_t n = (size_t)T * (d >> 2);
    size_t blocks = (n + 255) / 256, cap = (size_t)fellm_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (out_is_bf16)
      token_shift_vec_kernel<bf16><<<(unsigned)blocks, 256, 0, stream>>>(h, mu, state, slot_stride, item_start, item_slot, row_item, (bf16*)out, T, d);
    else
      token_shift_vec_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(h, mu, state, slot_stride, item_start, item_slot, row_item, (float*)out, T, d);
    return launch_status();
  }
  if (max_item_rows < 1) max_item_rows = 1;
  dim3 grid(ceil_div(d, CH_TILE), n_items, ceil_div(max_item_rows, ROW_TILE)), block(CH_TILE, max_item_rows == 1 ? 1 : 8);
  if (out_is_bf16)
    token_shift_mix_kernel<float, bf16><<<grid, block, 0, stream>>>(h, mu, 1, state, slot_stride, item_start, item_slot, (bf16*)out, T, d);
  else
    token_shift_mix_kernel<float, float><<<grid, block, 0, stream>>>(h, mu, 1, state, slot_stride, item_start, item_slot, (float*)out, T, d);
  return launch_status();
}

// ---------------------------------------------------------------- second factor of a low-rank projection
// out[t, n] = f_out(bias[n] + sum_r W2[n, r] f_in(z[t, r])), float32.  f_in: 0 identity, 1 tanh.
// f_out: 0 identity; 1 exp(-exp(v)) (a decay from its double logarithm); 2 exp(-exp(rate[n / per]) softplus(v)).
#define LR_ROWS 8
template <typename TW>
__global__ void __launch_bounds__(128)
lowrank_expand_kernel(const float* __restrict__ z, int ldz, const TW* __restrict__ W2, const float* __restrict__ bias,
                      const float* __restrict__ rate, int per, float* __restrict__ out, int T, int N, int R,
                      int f_in, int f_out) {
  extern __shared__ float zs[];                      // [LR_ROWS][R]
  const int t0 = blockIdx.y * LR_ROWS;
  for (int e = threadIdx.x; e < LR_ROWS * R; e += blockDim.x) {
    int i = e / R, r = e - i * R;
    float v = t0 + i < T ? z[(size_t)(t0 + i) * ldz + r] : 0.f;
    zs[e] = f_in == 1 ? tanhf(v) : v;
  }
  __syncthreads();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float acc[LR_ROWS];
#pragma unroll
  for (int i = 0; i < LR_ROWS; ++i) acc[i] = 0.f;
  const TW* wr = W2 + (size_t)n * R;
  for (int r = 0; r < R; ++r) {
    float w = to_f(wr[r]);
#pragma unroll
    for (int i = 0; i < LR_ROWS; ++i) acc[i] = fmaf(zs[i * R + r], w, acc[i]);
  }
  const float b = bias ? bias[n] : 0.f;
  const float rt = f_out == 2 ? expf(rate[n / per]) : 0.f;
#pragma unroll
  for (int i = 0; i < LR_ROWS; ++i) {
    if (t0 + i >= T) break;
    float v = acc[i] + b;
    if (f_out == 1) v = expf(-expf(v));
    else if (f_out == 2) v = expf(-rt * softplus_f(v));
    out[(size_t)(t0 + i) * N + n] = v;
  }
}

FELLM_API int fellm_lowrank_expand(const float* z, int ldz, const void* W2, int w_bf16, const float* bias,
                                   const float* rate, int per, float* out, int T, int N, int R, int f_in, int f_out,
                                   cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (!z || !W2 || !out || R < 1 || (f_out == 2 && (!rate || per < 1))) return FELLM_ERR_ARG;
  if (R > 1024) return FELLM_ERR_SIZE;
  dim3 grid(ceil_div(N, 128), ceil_div(T, LR_ROWS));
  size_t smem = (size_t)LR_ROWS * R * sizeof(float);
  if (w_bf16)
    lowrank_expand_kernel<bf16><<<grid, 128, smem, stream>>>(z, ldz, (const bf16*)W2, bias, rate, per, out, T, N, R, f_in, f_out);
  else
    lowrank_expand_kernel<float><<<grid, 128, smem, stream>>>(z, ldz, (const float*)W2, bias, rate, per, out, T, N, R, f_in, f_out);
  return launch_status();
}

// ---------------------------------------------------------------- the two scans
// One kernel for both recurrences.  Per head the state is a matrix S [dk, dv]; its columns do not meet, so a
// warp owns CPW = 32 / KS of them and spreads a column's dk rows over KS lanes, four rows at a time (row
// 4 (ks + KS r4) + e belongs to lane ks: a float4 of the staged vectors per lane, consecutive lanes on consecutive
// float4s).  Sums over dk run over (r4, e) in a thread, then over the KS lanes by a butterfly.
//
// Both recurrences have the form, per token and column j,
//     d1 = sum_i S[i,j] A_i        d2 = sum_i S[i,j] B_i          (from the state BEFORE the token)
//     u  = beta (v_j - d1)   (delta rule)       or   u = v_j      (decay and bonus)
//     o_j = d2 + u c
//     S[i,j] <- G_i S[i,j] + K_i u
// with per-token vectors A, B, G, K [dk] and scalars beta, c that do not depend on S:
//   delta rule (k^ = k / |k|, q^ = q / |q| / sqrt(dk), decay g per head or per channel):
//       A = g k^,  B = g q^,  G = g,  K = k^,  c = k^ . q^      (S^T q after the write = g S^T q + u (k.q))
//   decay and bonus:  B = r,  G = w,  K = k,  c = sum_i r_i u_i k_i,  A unused
//   gated write (q = SiLU(q raw), f = l + (1 - l) sigmoid(f raw + bias), l a lower bound per channel):
//       B = f q,  G = f,  K = 1 - f,  c = sum_i (1 - f_i) q_i      (S^T q after the write = S^T (f q) + v c)
//   the same, prepared (mode 5): a kernel in front has left f q and f where q raw and f raw stood and c beside them, once a
//   token and head; the producers then only copy (every column tile of a head repeats the staging, and with the gate's
//   exponentials in it the staging was two thirds of the kernel's instructions)
// so the chain from token to token is one reduction and one multiply-add per element.  Eight producer warps stage
// these vectors for the next tokens (loads, unit norms, decays, sigmoids) in shared memory while four consumer
// warps run the chain over the tokens staged before: one block barrier per stage.  KS is chosen from the model's
// sizes alone (enough lanes a column that one prompt's columns fill the SMs), never from the batch: the order of
// every sum is the same in every step.
#define SC_CONSUMERS 4
#define SC_PRODUCERS 8
#define SC_THREADS ((SC_CONSUMERS + SC_PRODUCERS) * 32)
#define SC_MAX_TOK 32

struct ScanArgs {
  // delta rule: q at qkv, k at qkv + k_off, v at qkv + v_off of a row (ld elements); decay and bonus: r, k, v rows
  const void* q; const void* k; const void* v; int ld, k_off, v_off;
  const float* small; int lds, b_off, a_off;           // delta: beta's logit (and the per-head decay's)
  const float* A_log; const float* dt_bias;            // delta, decay per head
  const float* gch;                                    // delta per channel: g; decay and bonus: w   [T, H*dk]
  const float* bonus;                                  // decay and bonus: u [H, dk]
  float* state; long long slot_stride;
  const int* item_start; const int* item_slot;
  float* out;
  int H, G, dk, dv, KS, tc;
  int vec;                                             // q, k (and the decay) can be read 16 bytes at a time
  // retention: the rows' positions, the rotary frequencies [rot / 2], how many leading elements of a head are rotated,
  // the decay of each head, and what the rotated keys are multiplied by
  const int* pos; const float* inv_freq; int rot; const float* decay_h; float kscale;
  // gated write: the forget gate's lower bound and its bias, [H, dk] each
  const float* lower; const float* fbias;
  // a portion in blocks of `blk` tokens that run side by side (recurrences whose write does not read the state: S_t =
  // G_t S_(t-1) + K_t v_t^T is linear in the state in front of it).  phase 1: every block from a state of zeros, no
  // outputs; it leaves its end state in blk_state [item][block][H][dv][dk] and the product of its G in blk_decay
  // [item][block][H][dk].  scan_blocks_kernel then walks an item's blocks in order and turns blk_state into the states
  // IN FRONT of the blocks (and moves the slot's state on).  phase 3: every block again from that state, with outputs.
  int phase, blk; float* blk_state; float* blk_decay;
};

template <int VE> __device__ __forceinline__ void load_vec(const float* p, float* out) {
  *(float4*)out = *(const float4*)p;
}
template <int VE> __device__ __forceinline__ void load_vec(const bf16* p, float* out) {
  const uint4 raw = *(const uint4*)p;
  const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
  for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(h[e]); out[2 * e] = f.x; out[2 * e + 1] = f.y; }
}

__device__ __forceinline__ void producers_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(SC_PRODUCERS * 32) : "memory");
}

// The producers' share of a stage.  First the raw vectors of all its tokens, every thread with several loads in flight
// (a token's vectors are short: taken token by token, each load's latency would stand alone); then, behind a barrier of
// the producers, a warp per token turns them into A, B, G, K and the token's scalars.
template <int MODE, typename TA>
__device__ __forceinline__ void scan_stage(const ScanArgs& a, float* buf, int DKP, int COLS, int h, int col0, int row0,
                                           int n_tok, int ptid) {
  float* A = buf; float* B = A + a.tc * DKP; float* Gd = B + a.tc * DKP; float* KK = Gd + a.tc * DKP;
  float* V = KK + a.tc * DKP; float* beta = V + a.tc * COLS; float* cc = beta + a.tc;
  const int dk = a.dk;
  constexpr int PT = SC_PRODUCERS * 32, U = 4;
  const int total = n_tok * DKP;
  const int g = MODE == 2 ? h : h / (a.H / a.G);
  const TA* x0p = (const TA*)a.q + (size_t)g * dk;                                         // q, or r
  const TA* x1p = MODE == 2 ? (const TA*)a.k + (size_t)h * dk : x0p + a.k_off;             // k
  const float* x2p = (MODE == 0 || MODE >= 3) ? nullptr : a.gch + (size_t)h * dk;           // the decay per channel
  // The values of this block's columns and the tokens' logits are asked for first and stored last: their latency
  // runs under the vectors' loads.
  constexpr int VMAX = (SC_MAX_TOK * 32 * SC_CONSUMERS + PT - 1) / PT;
  const TA* vp = MODE == 2 ? (const TA*)a.v + (size_t)h * dk : (const TA*)a.q + a.v_off + (size_t)h * a.dv;
  float vreg[VMAX];
#pragma unroll
  for (int u = 0; u < VMAX; ++u) {
    const int idx = ptid + u * PT;
    vreg[u] = 0.f;
    if (idx < n_tok * COLS) {
      const int t = idx / COLS, x = idx - t * COLS;
      if (col0 + x < a.dv) vreg[u] = to_f(vp[(size_t)(row0 + t) * a.ld + col0 + x]);
    }
  }
  float logit_b = 0.f, logit_a = 0.f;
  if (MODE < 2 && ptid < n_tok) {
    const size_t row = (size_t)(row0 + ptid);
    logit_b = a.small[row * a.lds + a.b_off + h];
    if (MODE == 0) logit_a = a.small[row * a.lds + a.a_off + h];
  }
  if (MODE == 5 && ptid < n_tok) { logit_b = 1.f; logit_a = a.small[(size_t)(row0 + ptid) * a.lds + h]; }      // beta, c
  if (a.vec) {
    // eight (bfloat16) or four (float32) elements a load: 16 bytes of q, of k and, where there is one, of the decay
    constexpr int VE = sizeof(TA) == 2 ? 8 : 4;
    constexpr int UV = sizeof(TA) == 2 ? 2 : 4;          // vectors a thread keeps in flight: a stage's loads are ONE round trip to memory
    const int per_tok = DKP / VE, nvec = n_tok * per_tok;
    for (int base = ptid; base < nvec; base += PT * UV) {
      float x0[UV][VE], x1[UV][VE], x2[UV][VE];
#pragma unroll
      for (int u = 0; u < UV; ++u) {
#pragma unroll
        for (int e = 0; e < VE; ++e) x0[u][e] = x1[u][e] = x2[u][e] = 0.f;
        const int idx = base + u * PT;
        if (idx < nvec) {
          const int t = idx / per_tok, i = (idx - t * per_tok) * VE;
          if (i < dk) {
            const size_t row = (size_t)(row0 + t);
            load_vec<VE>(x0p + row * a.ld + i, x0[u]);
            load_vec<VE>(x1p + row * a.ld + i, x1[u]);
            if (MODE == 1 || MODE == 2) {
#pragma unroll
              for (int e = 0; e < VE; e += 4) *(float4*)(x2[u] + e) = *(const float4*)(x2p + row * ((size_t)a.H * dk) + i + e);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UV; ++u) {
        const int idx = base + u * PT;
        if (idx < nvec) {
          const int t = idx / per_tok, i = (idx - t * per_tok) * VE;
          const int o = t * DKP + i;
#pragma unroll
          for (int e = 0; e < VE; e += 4) {
            *(float4*)(B + o + e) = *(float4*)(x0[u] + e);
            *(float4*)(KK + o + e) = *(float4*)(x1[u] + e);
            *(float4*)(Gd + o + e) = *(float4*)(x2[u] + e);
          }
        }
      }
    }
  } else {
    for (int base = ptid; base < total; base += PT * U) {
      float x0[U], x1[U], x2[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * PT;
        x0[u] = x1[u] = x2[u] = 0.f;
        if (idx < total) {
          const int t = idx / DKP, i = idx - t * DKP;
          if (i < dk) {
            const size_t row = (size_t)(row0 + t);
            x0[u] = to_f(x0p[row * a.ld + i]);
            x1[u] = to_f(x1p[row * a.ld + i]);
            if (MODE == 1 || MODE == 2) x2[u] = x2p[row * ((size_t)a.H * dk) + i];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * PT;
        if (idx < total) { B[idx] = x0[u]; KK[idx] = x1[u]; Gd[idx] = x2[u]; }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < VMAX; ++u) {
    const int idx = ptid + u * PT;
    if (idx < n_tok * COLS) V[idx] = vreg[u];
  }
  if ((MODE < 2 || MODE == 5) && ptid < n_tok) { beta[ptid] = logit_b; cc[ptid] = logit_a; }
  producers_sync();
  // a warp takes TPW tokens at once: their sums and butterflies are independent chains
  constexpr int TPW = SC_MAX_TOK / SC_PRODUCERS;
  const int pw = ptid >> 5, lane = ptid & 31;
  const float rate = MODE == 0 ? expf(a.A_log[h]) : 0.f, bias_a = MODE == 0 ? a.dt_bias[h] : 0.f;
  if (MODE == 2) {
    const float* ur = a.bonus + (size_t)h * dk;
    float c[TPW];
#pragma unroll
    for (int u = 0; u < TPW; ++u) c[u] = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const float b = ur[i];
#pragma unroll
      for (int u = 0; u < TPW; ++u) {
        const int t = pw + u * SC_PRODUCERS;
        if (t < n_tok) c[u] = fmaf(B[t * DKP + i] * b, KK[t * DKP + i], c[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < TPW; ++u) c[u] = warp_sum(c[u]);
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int t = pw + u * SC_PRODUCERS;
      if (t < n_tok && lane == 0) { cc[t] = c[u]; beta[t] = 1.f; }
    }
  } else if (MODE == 5) {
    // gated write, prepared: B = f q is staged as it is, KK holds f: G = f, K = 1 - f (rows behind dk: zeros)
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int t = pw + u * SC_PRODUCERS;
      if (t >= n_tok) continue;
      float* Gt = Gd + t * DKP; float* Kt = KK + t * DKP;
      for (int i = lane; i < DKP; i += 32) {
        const float f = Kt[i];
        Gt[i] = f; Kt[i] = i < dk ? 1.0f - f : 0.f;
      }
    }
  } else if (MODE == 4) {
    // gated write: everything of the gate in float32; rows behind dk keep K = 0, so the state's padding stays zero
    const float* lo = a.lower + (size_t)h * dk; const float* fb = a.fbias + (size_t)h * dk;
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int t = pw + u * SC_PRODUCERS;
      if (t >= n_tok) continue;
      float* Bt = B + t * DKP; float* Gt = Gd + t * DKP; float* Kt = KK + t * DKP;
      float c = 0.f;
      for (int i = lane; i < DKP; i += 32) {
        float fq = 0.f, f = 0.f, w = 0.f;
        if (i < dk) {
          const float q = silu_f(Bt[i]), l = lo[i];
          f = fmaf(1.0f - l, sigmoid_f(Kt[i] + fb[i]), l);
          w = 1.0f - f; fq = f * q;
          c = fmaf(w, q, c);
        }
        Bt[i] = fq; Gt[i] = f; Kt[i] = w;
      }
      c = warp_sum(c);
      if (lane == 0) { cc[t] = c; beta[t] = 1.f; }
    }
  } else if (MODE == 3) {
    // retention: rotate the leading `rot` elements of q and k (element i with i + rot/2, angle = position * frequency i),
    // k times kscale after the rotation; B = decay q, K = k, G = decay, c = k . q  (S^T q after the write is
    // decay S^T q + v (k . q))
    const int half = a.rot >> 1;
    const float gam = a.decay_h[h];
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int t = pw + u * SC_PRODUCERS;
      if (t >= n_tok) continue;
      float* Bt = B + t * DKP; float* Gt = Gd + t * DKP; float* Kt = KK + t * DKP;
      const float p = (float)a.pos[row0 + t];
      for (int i = lane; i < half; i += 32) {
        float sn, cs;
        sincosf(p * a.inv_freq[i], &sn, &cs);
        const float qu = Bt[i], qv = Bt[i + half], ku = Kt[i], kv = Kt[i + half];
        Bt[i] = qu * cs - qv * sn; Bt[i + half] = qv * cs + qu * sn;
        Kt[i] = ku * cs - kv * sn; Kt[i + half] = kv * cs + ku * sn;
      }
      __syncwarp();
      float kq = 0.f;
      for (int i = lane; i < DKP; i += 32) {
        const float kk = Kt[i] * a.kscale, qq = Bt[i];
        kq = fmaf(kk, qq, kq);
        Kt[i] = kk; Bt[i] = gam * qq; Gt[i] = gam;
      }
      kq = warp_sum(kq);
      if (lane == 0) { cc[t] = kq; beta[t] = 1.f; }
    }
  } else {
    float sq[TPW], sk[TPW], kq[TPW];
#pragma unroll
    for (int u = 0; u < TPW; ++u) sq[u] = sk[u] = kq[u] = 0.f;
    for (int i = lane; i < DKP; i += 32) {
#pragma unroll
      for (int u = 0; u < TPW; ++u) {
        const int t = pw + u * SC_PRODUCERS;
        if (t < n_tok) {
          const float q = B[t * DKP + i], k = KK[t * DKP + i];
          sq[u] = fmaf(q, q, sq[u]); sk[u] = fmaf(k, k, sk[u]); kq[u] = fmaf(k, q, kq[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < TPW; ++u) { sq[u] = warp_sum(sq[u]); sk[u] = warp_sum(sk[u]); kq[u] = warp_sum(kq[u]); }
#pragma unroll
    for (int u = 0; u < TPW; ++u) {
      const int t = pw + u * SC_PRODUCERS;
      if (t >= n_tok) continue;
      float* At = A + t * DKP; float* Bt = B + t * DKP; float* Gt = Gd + t * DKP; float* Kt = KK + t * DKP;
      const float kn = 1.0f / sqrtf(sk[u] + 1e-6f);
      const float qn = 1.0f / (sqrtf(sq[u] + 1e-6f) * sqrtf((float)dk));
      float gs = 0.f;
      if (MODE == 0) gs = expf(-rate * softplus_f(cc[t] + bias_a));
      for (int i = lane; i < DKP; i += 32) {
        const float kk = Kt[i] * kn, qq = Bt[i] * qn;
        const float gi = MODE == 1 ? Gt[i] : gs;
        At[i] = gi * kk; Bt[i] = gi * qq; Gt[i] = gi; Kt[i] = kk;
      }
      __syncwarp();
      if (lane == 0) { cc[t] = kq[u] * kn * qn; beta[t] = sigmoid_f(beta[t]); }
    }
  }
}

// KST: the lanes a column as a compile-time constant (0: read from the arguments).
template <int MODE, int R4, int KST, typename TA>
__global__ void __launch_bounds__(SC_THREADS) scan_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float sc_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KS = KST > 0 ? KST : a.KS;
  const int CPW = 32 / KS, COLS = SC_CONSUMERS * CPW, DKP = 4 * KS * R4;
  const int col_tiles = (a.dv + COLS - 1) / COLS;
  const int h = blockIdx.x / col_tiles, col0 = (blockIdx.x - h * col_tiles) * COLS;
  const int item = blockIdx.y;
  int row_begin = a.item_start[item], n = a.item_start[item + 1] - row_begin;
  const int per_buf = a.tc * (4 * DKP + COLS + 4);          // (a multiple of four floats: the second buffer stays 16-byte aligned)
  const bool consumer = warp < SC_CONSUMERS;
  const int ks = lane % KS, cw = warp * CPW + lane / KS;          // (consumers) this thread's lane of rows and column
  const int j = col0 + cw;
  const bool live = consumer && j < a.dv;
  float* Sg = a.state + (size_t)a.item_slot[item] * a.slot_stride + (size_t)h * a.dk * a.dv;
  constexpr bool BLOCKS = MODE == 4 || MODE == 5;                       // (the modes that run portions in blocks)
  const int phase = BLOCKS ? a.phase : 0;
  float* Dg = nullptr;
  if (BLOCKS && phase) {
    const int off = blockIdx.z * a.blk;
    if (off >= n) return;                                  // (the whole CTA: this item has no such block)
    row_begin += off; n = min(a.blk, n - off);
    const size_t at = ((size_t)item * gridDim.z + blockIdx.z) * a.H + h;
    Sg = a.blk_state + at * a.dk * a.dv;
    Dg = a.blk_decay + at * a.dk;
  }
  float S[4 * R4];
  float Dp[BLOCKS ? 4 * R4 : 1];
  if (BLOCKS) {
#pragma unroll
    for (int e = 0; e < 4 * R4; ++e) Dp[e] = 1.f;
  }
  // In memory a head's state is kept column by column (element (i, j) at j * dk + i): a thread's four rows are one
  // 16-byte load and a warp's lanes read a column's rows side by side.  Nothing but this kernel reads the layout.
  const bool s_vec = (a.dk & 3) == 0;
  if (consumer) {
#pragma unroll
    for (int r4 = 0; r4 < R4; ++r4) {
      const int i0 = 4 * (ks + KS * r4);
      if (phase == 1) {
#pragma unroll
        for (int e = 0; e < 4; ++e) S[4 * r4 + e] = 0.f;
      } else if (live && s_vec && i0 < a.dk) {
        const float4 t = *(const float4*)(Sg + (size_t)j * a.dk + i0);
        S[4 * r4] = t.x; S[4 * r4 + 1] = t.y; S[4 * r4 + 2] = t.z; S[4 * r4 + 3] = t.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) S[4 * r4 + e] = (live && i0 + e < a.dk) ? Sg[(size_t)j * a.dk + i0 + e] : 0.f;
      }
    }
  }
  const int n_stages = (n + a.tc - 1) / a.tc;
  if (!consumer) scan_stage<MODE, TA>(a, sc_smem, DKP, COLS, h, col0, row_begin, min(a.tc, n), (int)threadIdx.x - SC_CONSUMERS * 32);
  __syncthreads();
  for (int s = 0; s < n_stages; ++s) {
    float* buf = sc_smem + (s & 1) * per_buf;
    const int t0 = s * a.tc, n_tok = min(a.tc, n - t0);
    if (!consumer) {
      if (s + 1 < n_stages)
        scan_stage<MODE, TA>(a, sc_smem + ((s + 1) & 1) * per_buf, DKP, COLS, h, col0, row_begin + t0 + a.tc,
                             min(a.tc, n - t0 - a.tc), (int)threadIdx.x - SC_CONSUMERS * 32);
    } else {
      const float4* A4 = (const float4*)buf;
      const float4* B4 = (const float4*)(buf + a.tc * DKP);
      const float4* G4 = (const float4*)(buf + 2 * a.tc * DKP);
      const float4* K4 = (const float4*)(buf + 3 * a.tc * DKP);
      const float* V = buf + 4 * a.tc * DKP;
      const float* beta = V + a.tc * COLS;
      const float* cc = beta + a.tc;
      const int dq = DKP / 4;
      // the vectors of token t + 1 are asked for before token t's chain starts: nothing of them depends on S
      float4 nA[R4], nB[R4], nG[R4], nK[R4];
      float nv, nbeta, ncc;
      constexpr bool AHEAD = R4 <= 4;              // (with 32 rows a thread the second set of vectors would spill)
      auto fetch = [&](int t) {
#pragma unroll
        for (int r4 = 0; r4 < R4; ++r4) {
          const int at = t * dq + ks + KS * r4;
          if (MODE < 2) nA[r4] = A4[at];
          nB[r4] = B4[at]; nG[r4] = G4[at]; nK[r4] = K4[at];
        }
        nv = V[t * COLS + cw]; nbeta = beta[t]; ncc = cc[t];
      };
      // Recurrences whose write does not read the state (u = v): four tokens a round.  The state's chain from token to
      // token is one multiply-add an element; what takes long is the butterfly that sums a column's lanes, and the four
      // tokens' butterflies are independent: they go round together.  Same operations, same order, same numbers as the
      // token-by-token loop below.
      constexpr bool ROUNDS = MODE >= 2;
      if (ROUNDS) {
        constexpr int TB = 4;
        for (int t = 0; t < n_tok; t += TB) {
          float d2[TB], vv[TB], ctt[TB];
#pragma unroll
          for (int b = 0; b < TB; ++b) {
            d2[b] = 0.f; vv[b] = 0.f; ctt[b] = 0.f;
            if (t + b < n_tok) {
              const int tt = t + b;
              const float v = V[tt * COLS + cw];
              float p2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
              for (int r4 = 0; r4 < R4; ++r4) {
                const int at = tt * dq + ks + KS * r4;
                const float4 cB = B4[at], cG = G4[at], cK = K4[at];
                p2[0] = fmaf(S[4 * r4], cB.x, p2[0]); p2[1] = fmaf(S[4 * r4 + 1], cB.y, p2[1]);
                p2[2] = fmaf(S[4 * r4 + 2], cB.z, p2[2]); p2[3] = fmaf(S[4 * r4 + 3], cB.w, p2[3]);
                S[4 * r4] = fmaf(cK.x, v, cG.x * S[4 * r4]);
                S[4 * r4 + 1] = fmaf(cK.y, v, cG.y * S[4 * r4 + 1]);
                S[4 * r4 + 2] = fmaf(cK.z, v, cG.z * S[4 * r4 + 2]);
                S[4 * r4 + 3] = fmaf(cK.w, v, cG.w * S[4 * r4 + 3]);
                if (BLOCKS && phase == 1) {
                  Dp[4 * r4] *= cG.x; Dp[4 * r4 + 1] *= cG.y; Dp[4 * r4 + 2] *= cG.z; Dp[4 * r4 + 3] *= cG.w;
                }
              }
              d2[b] = (p2[0] + p2[1]) + (p2[2] + p2[3]); vv[b] = v; ctt[b] = cc[tt];
            }
          }
          for (int o = 1; o < KS; o <<= 1) {
#pragma unroll
            for (int b = 0; b < TB; ++b) d2[b] += __shfl_xor_sync(0xffffffffu, d2[b], o);
          }
#pragma unroll
          for (int b = 0; b < TB; ++b)
            if (t + b < n_tok && ks == 0 && live && phase != 1)
              a.out[(size_t)(row_begin + t0 + t + b) * ((size_t)a.H * a.dv) + (size_t)h * a.dv + j] = fmaf(vv[b], ctt[b], d2[b]);
        }
      }
      if (AHEAD && !ROUNDS) fetch(0);
#pragma unroll 2
      for (int t = 0; t < (ROUNDS ? 0 : n_tok); ++t) {
        if (!AHEAD) fetch(t);
        float4 cA[R4], cB[R4], cG[R4], cK[R4];
#pragma unroll
        for (int r4 = 0; r4 < R4; ++r4) { if (MODE < 2) cA[r4] = nA[r4]; cB[r4] = nB[r4]; cG[r4] = nG[r4]; cK[r4] = nK[r4]; }
        const float v = nv, bt = nbeta, ct = ncc;
        if (AHEAD && t + 1 < n_tok) fetch(t + 1);
        float p1[4] = {0.f, 0.f, 0.f, 0.f}, p2[4] = {0.f, 0.f, 0.f, 0.f};      // four short chains a dot, added in a fixed order
#pragma unroll
        for (int r4 = 0; r4 < R4; ++r4) {
          p2[0] = fmaf(S[4 * r4], cB[r4].x, p2[0]); p2[1] = fmaf(S[4 * r4 + 1], cB[r4].y, p2[1]);
          p2[2] = fmaf(S[4 * r4 + 2], cB[r4].z, p2[2]); p2[3] = fmaf(S[4 * r4 + 3], cB[r4].w, p2[3]);
          if (MODE < 2) {
            p1[0] = fmaf(S[4 * r4], cA[r4].x, p1[0]); p1[1] = fmaf(S[4 * r4 + 1], cA[r4].y, p1[1]);
            p1[2] = fmaf(S[4 * r4 + 2], cA[r4].z, p1[2]); p1[3] = fmaf(S[4 * r4 + 3], cA[r4].w, p1[3]);
          }
        }
        float d1 = (p1[0] + p1[1]) + (p1[2] + p1[3]), d2 = (p2[0] + p2[1]) + (p2[2] + p2[3]);
        for (int o = 1; o < KS; o <<= 1) {
          d2 += __shfl_xor_sync(0xffffffffu, d2, o);
          if (MODE < 2) d1 += __shfl_xor_sync(0xffffffffu, d1, o);
        }
        const float u = MODE >= 2 ? v : bt * (v - d1);
        const float o = fmaf(u, ct, d2);
#pragma unroll
        for (int r4 = 0; r4 < R4; ++r4) {
          S[4 * r4] = fmaf(cK[r4].x, u, cG[r4].x * S[4 * r4]);
          S[4 * r4 + 1] = fmaf(cK[r4].y, u, cG[r4].y * S[4 * r4 + 1]);
          S[4 * r4 + 2] = fmaf(cK[r4].z, u, cG[r4].z * S[4 * r4 + 2]);
          S[4 * r4 + 3] = fmaf(cK[r4].w, u, cG[r4].w * S[4 * r4 + 3]);
          if (BLOCKS && phase == 1) {
            Dp[4 * r4] *= cG[r4].x; Dp[4 * r4 + 1] *= cG[r4].y; Dp[4 * r4 + 2] *= cG[r4].z; Dp[4 * r4 + 3] *= cG[r4].w;
          }
        }
        if (ks == 0 && live && phase != 1) a.out[(size_t)(row_begin + t0 + t) * ((size_t)a.H * a.dv) + (size_t)h * a.dv + j] = o;
      }
    }
    __syncthreads();
  }
  if (BLOCKS && phase == 1 && consumer && col0 == 0 && cw == 0) {
#pragma unroll
    for (int r4 = 0; r4 < R4; ++r4)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * (ks + KS * r4) + e;
        if (i < a.dk) Dg[i] = Dp[4 * r4 + e];
      }
  }
  if (live && phase != 3) {
#pragma unroll
    for (int r4 = 0; r4 < R4; ++r4) {
      const int i0 = 4 * (ks + KS * r4);
      if (s_vec && i0 < a.dk) {
        *(float4*)(Sg + (size_t)j * a.dk + i0) = make_float4(S[4 * r4], S[4 * r4 + 1], S[4 * r4 + 2], S[4 * r4 + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (i0 + e < a.dk) Sg[(size_t)j * a.dk + i0 + e] = S[4 * r4 + e];
      }
    }
  }
}

// The walk between the two passes of a portion in blocks: per item and state element, over the item's blocks in order,
// S_b = the state in front of block b (written where the block's end state stood), S_(b+1) = D_b S_b + L_b; the slot then
// holds the state behind the last block.  A thread an element: the order of the sums is the order of the blocks.
__global__ void __launch_bounds__(256)
scan_blocks_kernel(float* __restrict__ blk_state, const float* __restrict__ blk_decay, float* __restrict__ state,
                   long long slot_stride, const int* __restrict__ item_start, const int* __restrict__ item_slot,
                   int n_blocks, int blk, int H, int dk, int dv) {
  const int item = blockIdx.y;
  const size_t per_head = (size_t)dk * dv, per_item = per_head * H;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per_item) return;
  const int h = (int)(e / per_head), i = (int)((e - (size_t)h * per_head) % dk);
  const int n = item_start[item + 1] - item_start[item];
  const int nb = (n + blk - 1) / blk;
  float* slot = state + (size_t)item_slot[item] * slot_stride + e;
  float S = *slot;
  for (int b = 0; b < nb; ++b) {
    const size_t at = (size_t)item * n_blocks + b;
    float* L = blk_state + at * per_item + e;
    const float D = blk_decay[(at * H + h) * dk + i], l = *L;
    *L = S;
    S = fmaf(D, S, l);
  }
  *slot = S;
}

template <int MODE, typename TA>
static int scan_launch(ScanArgs& a, int n_items, int max_item_rows, cudaStream_t stream) {
  int KS = 1;
  while (KS < 32 && a.dk > 16 * KS) KS <<= 1;                // up to 16 rows a thread while dk <= 512
  // more lanes a column while one item's blocks do not fill the device and a lane keeps four rows or more (a portion in
  // blocks fills the device by its blocks: it keeps the fewest lanes a column, the most work a thread)
  while (!a.phase && KS < 32 && 8 * KS <= a.dk && a.H * ((a.dv * KS + 32 * SC_CONSUMERS - 1) / (32 * SC_CONSUMERS)) < 120) KS <<= 1;
  int r4 = (a.dk + 4 * KS - 1) / (4 * KS), R4 = 1;
  while (R4 < r4) R4 <<= 1;
  if (R4 > 8) return FELLM_ERR_SIZE;
  a.KS = KS;
  {
    const int ve = sizeof(TA) == 2 ? 8 : 4;
    const size_t esz = sizeof(TA);
    bool ok = a.dk % ve == 0 && a.ld % ve == 0 && (4 * KS * R4) % ve == 0 && ((uintptr_t)a.q % 16) == 0;
    if (MODE == 2) ok = ok && ((uintptr_t)a.k % 16) == 0;
    else ok = ok && a.k_off % ve == 0;
    if (MODE == 1 || MODE == 2) ok = ok && ((uintptr_t)a.gch % 16) == 0;
    (void)esz;
    a.vec = ok ? 1 : 0;
  }
  const int CPW = 32 / KS, COLS = SC_CONSUMERS * CPW, DKP = 4 * KS * R4;
  const int per_tok = (4 * DKP + COLS + 4) * (int)sizeof(float);
  int tc = 81920 / per_tok;          // (two buffers: up to 160 KB a CTA; a stage is as long as the producers' round trip to memory is worth)
  a.tc = tc < 1 ? 1 : (tc > SC_MAX_TOK ? SC_MAX_TOK : tc);
  if (max_item_rows > 0 && max_item_rows < a.tc) a.tc = max_item_rows;      // a decode step stages one token: 4 KB a block, not 67
  if (a.phase && a.tc > 8) a.tc = 8;                                        // blocks side by side: less shared memory, more CTAs an SM
  const size_t smem = (size_t)2 * a.tc * per_tok;
  const int n_blocks = a.phase ? (max_item_rows + a.blk - 1) / a.blk : 1;
  dim3 grid(a.H * ((a.dv + COLS - 1) / COLS), n_items, n_blocks);
  void (*kern)(ScanArgs) = nullptr;
#define SCAN_PICK(R4_, KS_) if (R4 == R4_ && KS == KS_) kern = scan_kernel<MODE, R4_, KS_, TA>
  SCAN_PICK(1, 8); SCAN_PICK(2, 8); SCAN_PICK(4, 8); SCAN_PICK(1, 16); SCAN_PICK(2, 16); SCAN_PICK(4, 16);
  SCAN_PICK(1, 32); SCAN_PICK(2, 32); SCAN_PICK(4, 32);
#undef SCAN_PICK
  if (!kern) kern = R4 == 1 ? scan_kernel<MODE, 1, 0, TA> : R4 == 2 ? scan_kernel<MODE, 2, 0, TA>
                  : R4 == 4 ? scan_kernel<MODE, 4, 0, TA> : scan_kernel<MODE, 8, 0, TA>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kern<<<grid, SC_THREADS, smem, stream>>>(a);
  if (a.phase == 1) {
    // the walk over the blocks, then every block again from the state in front of it
    const size_t per_item = (size_t)a.H * a.dk * a.dv;
    scan_blocks_kernel<<<dim3((unsigned)((per_item + 255) / 256), n_items), 256, 0, stream>>>(
        a.blk_state, a.blk_decay, a.state, a.slot_stride, a.item_start, a.item_slot, n_blocks, a.blk, a.H, a.dk, a.dv);
    a.phase = 3;
    kern<<<grid, SC_THREADS, smem, stream>>>(a);
  }
  return launch_status();
}

// Gated delta rule.  qkv [T, ldq]: q heads at column 0 (G x dk), k at k_off, v at v_off (H x dv), after their
// convolutions and SiLU.  small [T, lds]: beta's logit at column b_off + h; per-head decay: logit at a_off + h,
// g = exp(-exp(A_log[h]) softplus(logit + dt_bias[h])); per-channel decay: gch [T, H*dk] holds g itself.
FELLM_API int fellm_delta_scan(const void* qkv, int is_bf16, int ldq, int k_off, int v_off, const float* small, int lds,
                               int b_off, int a_off, const float* A_log, const float* dt_bias, const float* gch,
                               float* state, long long slot_stride, const int* item_start, const int* item_slot,
                               float* out, int n_items, int H, int G, int dk, int dv, int max_item_rows, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (dk < 1 || dk > 1024 || dv < 1 || G < 1 || H % G) return FELLM_ERR_SIZE;
  if (!qkv || !small || !state || !item_start || !item_slot || !out || (!gch && (!A_log || !dt_bias))) return FELLM_ERR_ARG;
  ScanArgs a = {};
  a.q = qkv; a.ld = ldq; a.k_off = k_off; a.v_off = v_off; a.small = small; a.lds = lds; a.b_off = b_off; a.a_off = a_off;
  a.A_log = A_log; a.dt_bias = dt_bias; a.gch = gch; a.state = state; a.slot_stride = slot_stride;
  a.item_start = item_start; a.item_slot = item_slot; a.out = out; a.H = H; a.G = G; a.dk = dk; a.dv = dv;
  if (gch) return is_bf16 ? scan_launch<1, bf16>(a, n_items, max_item_rows, stream) : scan_launch<1, float>(a, n_items, max_item_rows, stream);
  return is_bf16 ? scan_launch<0, bf16>(a, n_items, max_item_rows, stream) : scan_launch<0, float>(a, n_items, max_item_rows, stream);
}

// Decay-and-bonus recurrence.  r, k, v [T, ld] (H x dk each), w float32 [T, H*dk] (the decay itself), u [H, dk].
FELLM_API int fellm_decay_bonus_scan(const void* r, const void* k, const void* v, int is_bf16, int ld, const float* w,
                                     const float* u, float* state, long long slot_stride, const int* item_start,
                                     const int* item_slot, float* out, int n_items, int H, int dk, int max_item_rows,
                                     cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (dk < 1 || dk > 1024 || H < 1) return FELLM_ERR_SIZE;
  if (!r || !k || !v || !w || !u || !state || !item_start || !item_slot || !out) return FELLM_ERR_ARG;
  ScanArgs a = {};
  a.q = r; a.k = k; a.v = v; a.ld = ld; a.gch = w; a.bonus = u; a.state = state; a.slot_stride = slot_stride;
  a.item_start = item_start; a.item_slot = item_slot; a.out = out; a.H = H; a.G = H; a.dk = dk; a.dv = dk;
  return is_bf16 ? scan_launch<2, bf16>(a, n_items, max_item_rows, stream) : scan_launch<2, float>(a, n_items, max_item_rows, stream);
}

// Retention: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, q and k rotated by position (the first `rot` elements
// of a head, element i paired with i + rot/2), k times kscale after the rotation.  qkv [T, ld]: q heads at column 0
// (H x dk), k at k_off (H x dk), v at v_off (H x dv), as their products left them.
FELLM_API int fellm_retention_scan(const void* qkv, int is_bf16, int ld, int k_off, int v_off, const int* positions,
                                   const float* inv_freq, int rot, const float* decay, float kscale, float* state,
                                   long long slot_stride, const int* item_start, const int* item_slot, float* out,
                                   int n_items, int H, int dk, int dv, int max_item_rows, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (dk < 1 || dk > 1024 || dv < 1 || H < 1 || rot < 0 || rot > dk || (rot & 1)) return FELLM_ERR_SIZE;
  if (!qkv || !positions || !decay || !state || !item_start || !item_slot || !out || (rot && !inv_freq)) return FELLM_ERR_ARG;
  ScanArgs a = {};
  a.q = qkv; a.ld = ld; a.k_off = k_off; a.v_off = v_off; a.state = state; a.slot_stride = slot_stride;
  a.item_start = item_start; a.item_slot = item_slot; a.out = out; a.H = H; a.G = H; a.dk = dk; a.dv = dv;
  a.pos = positions; a.inv_freq = inv_freq; a.rot = rot; a.decay_h = decay; a.kscale = kscale;
  return is_bf16 ? scan_launch<3, bf16>(a, n_items, max_item_rows, stream) : scan_launch<3, float>(a, n_items, max_item_rows, stream);
}

// In front of the prepared form: a warp a (token, head) turns q raw into f q and f raw into f where they stand and leaves
// c = sum_i (1 - f_i) q_i in cc [T, H]: the same operations in the same order as the unprepared stage's, so both forms
// hand the consumers the same numbers.
__global__ void __launch_bounds__(128)
gated_write_prep_kernel(float* __restrict__ z, int ld, int f_off, const float* __restrict__ lower, const float* __restrict__ fbias,
                        float* __restrict__ cc, int T, int H, int dk) {
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (warp >= T * H) return;
  const int t = warp / H, h = warp - t * H;
  float* qr = z + (size_t)t * ld + (size_t)h * dk;
  float* fr = qr + f_off;
  const float* lo = lower + (size_t)h * dk; const float* fb = fbias + (size_t)h * dk;
  float c = 0.f;
  for (int i = lane; i < dk; i += 32) {
    const float q = silu_f(qr[i]), l = lo[i];
    const float f = fmaf(1.0f - l, sigmoid_f(fr[i] + fb[i]), l);
    const float w = 1.0f - f;
    c = fmaf(w, q, c);
    qr[i] = f * q; fr[i] = f;
  }
  c = warp_sum(c);
  if (lane == 0) cc[(size_t)t * H + h] = c;
}

// Gated write: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t with q = SiLU(q raw) and
// f = lower + (1 - lower) sigmoid(f raw + bias).  z float32 [T, ld]: q raw at column 0 (H x dk), f raw at f_off (H x dk),
// v at v_off (H x dv), as their product left them; lower, bias float32 [H * dk].
// blk > 0 (with scratch of n_items * ceil(max_item_rows / blk) * H * (dk * dv + dk) floats): the portions run in blocks of
// blk tokens side by side (two passes and a walk over the blocks' states between them; sums in another order than the
// plain scan's, equal up to float32 rounding).
// prep (float32 [T, H], with T the rows of z): the gates are computed once a token and head by a kernel in front, IN PLACE
// (z's q and f columns then hold f q and f), and the scan's producers only copy: for portions; a decode step's single
// tokens keep the one launch.
FELLM_API int fellm_gated_write_scan(float* z, int ld, int f_off, int v_off, const float* lower, const float* bias,
                                     float* state, long long slot_stride, const int* item_start, const int* item_slot,
                                     float* out, int n_items, int H, int dk, int dv, int max_item_rows, int blk,
                                     float* scratch, float* prep, int T, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (dk < 1 || dk > 1024 || dv < 1 || H < 1) return FELLM_ERR_SIZE;
  if (!z || !lower || !bias || !state || !item_start || !item_slot || !out) return FELLM_ERR_ARG;
  ScanArgs a = {};
  a.q = z; a.ld = ld; a.k_off = f_off; a.v_off = v_off; a.state = state; a.slot_stride = slot_stride;
  a.item_start = item_start; a.item_slot = item_slot; a.out = out; a.H = H; a.G = H; a.dk = dk; a.dv = dv;
  a.lower = lower; a.fbias = bias;
  if (blk > 0 && scratch && max_item_rows > blk) {
    const size_t n_blocks = (size_t)(max_item_rows + blk - 1) / blk;
    a.phase = 1; a.blk = blk; a.blk_state = scratch; a.blk_decay = scratch + (size_t)n_items * n_blocks * H * dk * dv;
  }
  if (prep && T > 0) {
    gated_write_prep_kernel<<<(unsigned)(((long long)T * H + 3) / 4), 128, 0, stream>>>(z, ld, f_off, lower, bias, prep, T, H, dk);
    a.small = prep; a.lds = H;
    return scan_launch<5, float>(a, n_items, max_item_rows, stream);
  }
  return scan_launch<4, float>(a, n_items, max_item_rows, stream);
}

// ---------------------------------------------------------------- per-head norm and gate
// y[t, h, e] = o[t, h, e] / sqrt(mean_e o^2 + eps) * w[(per_head ? h * dv : 0) + e] * act(gate[t, h*dv + e]);
// act: 0 no gate, 1 SiLU, 2 sigmoid.  One warp per (t, h).
template <typename TO, typename TG>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int per_head,
                      const TG* __restrict__ gate, int ldg, int act, TO* __restrict__ y, int T, int H, int dv, float eps) {
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (warp >= T * H) return;
  const int t = warp / H, h = warp - t * H;
  const float* orow = o + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int e = lane; e < dv; e += 32) { float v = orow[e]; ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)dv + eps);
  const float* wr = w ? w + (per_head ? (size_t)h * dv : 0) : nullptr;       // no weight: the unit norm alone
  TO* yr = y + ((size_t)t * H + h) * dv;
  for (int e = lane; e < dv; e += 32) {
    float v = orow[e] * scale;
    if (wr) v *= wr[e];
    if (act) {
      float gz = to_f(gate[(size_t)t * ldg + (size_t)h * dv + e]);
      v *= act == 1 ? silu_f(gz) : sigmoid_f(gz);
    }
    yr[e] = from_f<TO>(v);
  }
}

FELLM_API int fellm_head_norm_gate(const float* o, const float* w, int per_head, const void* gate, int gate_bf16, int ldg,
                                   int act, void* y, int y_bf16, int T, int H, int dv, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!o || !y || (act && !gate)) return FELLM_ERR_ARG;
  unsigned blocks = (unsigned)(((long long)T * H + 3) / 4);
#define HNG(TO_, TG_) head_norm_gate_kernel<TO_, TG_><<<blocks, 128, 0, stream>>>(o, w, per_head, (const TG_*)gate, ldg, act, (TO_*)y, T, H, dv, eps)
  if (y_bf16) { if (gate_bf16) HNG(bf16, bf16); else HNG(bf16, float); }
  else { if (gate_bf16) HNG(float, bf16); else HNG(float, float); }
#undef HNG
  return launch_status();
}

// ---------------------------------------------------------------- branches of a parallel mixer
// x[t, :] += (1 / n) * sum_b branch_b[t, :] / sqrt(mean(branch_b[t]^2) + eps) * w_b.  One block per row.
#define MAX_BRANCHES 4
struct Branches { const float* o[MAX_BRANCHES]; const float* w[MAX_BRANCHES]; };

__global__ void __launch_bounds__(256)
branch_combine_kernel(Branches br, int n_br, float* __restrict__ x, int d, float eps) {
  __shared__ float part[MAX_BRANCHES][8];
  __shared__ float scale[MAX_BRANCHES];
  const int t = blockIdx.x;
  for (int b = 0; b < n_br; ++b) {
    const float* o = br.o[b] + (size_t)t * d;
    float ss = 0.f;
    for (int e = threadIdx.x; e < d; e += blockDim.x) ss = fmaf(o[e], o[e], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[b][threadIdx.x >> 5] = ss;
  }
  __syncthreads();
  if (threadIdx.x < n_br) {
    float s = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += part[threadIdx.x][i];
    scale[threadIdx.x] = 1.0f / sqrtf(s / (float)d + eps);
  }
  __syncthreads();
  const float inv = 1.0f / (float)n_br;
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float s = 0.f;
    for (int b = 0; b < n_br; ++b) s += (br.o[b][(size_t)t * d + e] * scale[b]) * br.w[b][e];
    x[(size_t)t * d + e] += s * inv;
  }
}

FELLM_API int fellm_branch_combine(const float* const* outs, const float* const* weights, int n_br, float* x, int T, int d,
                                   float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_br < 1 || n_br > MAX_BRANCHES) return FELLM_ERR_SIZE;
  if (!outs || !weights || !x) return FELLM_ERR_ARG;
  Branches br;
  for (int b = 0; b < MAX_BRANCHES; ++b) { br.o[b] = b < n_br ? outs[b] : nullptr; br.w[b] = b < n_br ? weights[b] : nullptr; }
  branch_combine_kernel<<<T, 256, 0, stream>>>(br, n_br, x, d, eps);
  return launch_status();
}
