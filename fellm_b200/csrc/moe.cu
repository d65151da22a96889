// Routed experts (a mixture of small gated feed-forwards): everything between the router's logits and the sum
// that goes into the residual stream, without a word to the host.
//
//   moe_route     softmax over the experts in float32, the `top` largest per token (ties: the lower expert), their
//                 scores as they are (or renormalised to sum 1)
//   moe_plan      (three kernels) the (token, choice) pairs sorted by expert: a count per tile of pairs and expert,
//                 an exclusive scan in the order (expert, tile), each pair's place; and the table of row tiles
//                 (expert, first row, rows) that the grouped products walk
//   moe_gemm      grouped product over the table: C[r, :] = A[row(r), :] W[e]^T, with the input rows gathered by
//                 token (first product, SiLU(gate) * up in the epilogue) or taken in sorted order (second product)
//   moe_combine   x[t, :] += sum_c score[t, c] * y[place(t, c), :], c in order
//
// A row's arithmetic depends on the row alone: a pair's place among its expert's rows moves it inside a tile, never
// into another sum; every sum over K runs in the order of K; the sum over a token's experts runs in the order of the
// choices.  So a token's result does not depend on the batch, and no atomics touch data.
#include "common.cuh"

#define MOE_MAX_TOP 16
#define PLAN_TILE 1024

// ---------------------------------------------------------------- routing
// One warp: softmax over z[0..E) in float32, the `top` largest (ties: the lower expert) into idx / w.
__device__ __forceinline__ void route_warp(const float* z, int E, int top, int renorm, int* idx, float* w, int lane) {
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) sum += expf(z[e] - m);
  sum = warp_sum(sum);
  int taken[MOE_MAX_TOP];
  float tw[MOE_MAX_TOP];
  float chosen = 0.f;
#pragma unroll
  for (int c = 0; c < MOE_MAX_TOP; ++c) {
    if (c >= top) break;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool free_ = true;
#pragma unroll
      for (int p = 0; p < MOE_MAX_TOP; ++p) if (p < c && taken[p] == e) free_ = false;
      const float v = z[e];
      if (free_ && (v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    taken[c] = bi;
    tw[c] = expf(best - m) / sum;
    chosen += tw[c];
  }
  if (lane == 0) {
#pragma unroll
    for (int c = 0; c < MOE_MAX_TOP; ++c) {
      if (c >= top) break;
      idx[c] = taken[c];
      w[c] = renorm ? tw[c] / chosen : tw[c];
    }
  }
}

// One warp, the sigmoid form: scores s_e = sigmoid(z_e); the choice looks at s_e + corr_e (corr may be null) and only
// inside the `keep` groups (of n_groups equal groups of neighbouring experts) whose `gtop` largest choice scores sum
// highest (ties: the lower group); the `top` largest choice scores among those (ties: the lower expert); weights = the
// chosen experts' plain scores, over their sum + 1e-20 when renorm.  work: shared memory of E + n_groups floats.
__device__ __forceinline__ void route_sigmoid_warp(const float* z, const float* corr, int E, int top, int renorm,
                                                   int n_groups, int keep, int gtop, float* work, int* idx, float* w, int lane) {
  float* choice = work;                 // [E]
  float* gscore = work + E;             // [n_groups]; -inf once a group is taken, then +inf marks the kept ones
  for (int e = lane; e < E; e += 32) choice[e] = 1.0f / (1.0f + expf(-z[e])) + (corr ? corr[e] : 0.f);
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      // the sum of the group's gtop largest choice scores: gtop passes over the group, each taking the next largest
      float sum = 0.f;
      int last_i = -1; float last_v = INFINITY;
      for (int c = 0; c < gtop && c < per; ++c) {
        float best = -INFINITY; int bi = -1;
        for (int i = 0; i < per; ++i) {
          const float v = choice[g * per + i];
          const bool after = v < last_v || (v == last_v && i > last_i);      // not yet taken, in (value desc, index asc) order
          if (after && (bi < 0 || v > best)) { best = v; bi = i; }
        }
        sum += best; last_v = best; last_i = bi;
      }
      gscore[g] = sum;
    }
    __syncwarp();
    for (int c = 0; c < keep; ++c) {
      float best = -INFINITY; int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gscore[g];
        if (v != INFINITY && (bi == 0x7fffffff || v > best || (v == best && g < bi))) { best = v; bi = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
      }
      if (lane == 0 && bi != 0x7fffffff) gscore[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32) if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  int taken[MOE_MAX_TOP];
  float tw[MOE_MAX_TOP];
  float chosen = 0.f;
#pragma unroll
  for (int c = 0; c < MOE_MAX_TOP; ++c) {
    if (c >= top) break;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool free_ = true;
#pragma unroll
      for (int p = 0; p < MOE_MAX_TOP; ++p) if (p < c && taken[p] == e) free_ = false;
      const float v = choice[e];
      if (free_ && (bi == 0x7fffffff || v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
    }
    taken[c] = bi;
    tw[c] = 1.0f / (1.0f + expf(-z[bi]));
    chosen += tw[c];
  }
  if (lane == 0) {
#pragma unroll
    for (int c = 0; c < MOE_MAX_TOP; ++c) {
      if (c >= top) break;
      idx[c] = taken[c];
      w[c] = renorm ? tw[c] / (chosen + 1e-20f) : tw[c];
    }
  }
}

// One warp per token.  logits float32 [T, ld]; idx [T, top] int32; w [T, top] float32.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int ld, int T, int E, int top, int renorm,
                 int* __restrict__ idx, float* __restrict__ w) {
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (warp >= T) return;
  route_warp(logits + (size_t)warp * ld, E, top, renorm, idx + (size_t)warp * top, w + (size_t)warp * top, lane);
}

FELLM_API int fellm_moe_route(const float* logits, int ld, int T, int E, int top, int renorm, int* idx, float* w,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 1 || top < 1 || top > E || top > MOE_MAX_TOP) return FELLM_ERR_SIZE;
  if (!logits || !idx || !w) return FELLM_ERR_ARG;
  moe_route_kernel<<<(T + 3) / 4, 128, 0, stream>>>(logits, ld, T, E, top, renorm, idx, w);
  return launch_status();
}

// The router's product and the routing in one kernel: a block per token, its warps take the experts by turns
// (z_e = sum_k h[k] Wr[e, k] in float32: a lane sums its share of k in order, the lanes are added by a butterfly: the
// order depends on K alone), then the first warp routes.  h [T, ldh] and Wr [E, K] bfloat16 or float32.
#define ROUTER_WARPS 4
template <typename TA, typename TW>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
moe_router_kernel(const TA* __restrict__ h, int ldh, const TW* __restrict__ Wr, int K, int E, int top, int renorm,
                  int* __restrict__ idx, float* __restrict__ w, int sigmoid, const float* __restrict__ corr,
                  int n_groups, int keep, int gtop, const float* __restrict__ bias) {
  extern __shared__ float zs[];                 // [E]; the sigmoid form: + [E + n_groups]
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TA* hr = h + (size_t)t * ldh;
  for (int e = warp; e < E; e += ROUTER_WARPS) {
    const TW* wr = Wr + (size_t)e * K;
    float s = 0.f;
    for (int k = lane; k < K; k += 32) s = fmaf(to_f(hr[k]), to_f(wr[k]), s);
    s = warp_sum(s);
    if (lane == 0) zs[e] = bias ? s + bias[e] : s;
  }
  __syncthreads();
  if (warp == 0) {
    if (sigmoid) route_sigmoid_warp(zs, corr, E, top, renorm, n_groups, keep, gtop, zs + E, idx + (size_t)t * top, w + (size_t)t * top, lane);
    else route_warp(zs, E, top, renorm, idx + (size_t)t * top, w + (size_t)t * top, lane);
  }
}

FELLM_API int fellm_moe_router(const void* h, int h_bf16, int ldh, const void* Wr, int w_bf16, int T, int K, int E, int top,
                               int renorm, int* idx, float* w, int sigmoid, const float* corr, int n_groups, int keep,
                               int gtop, const float* bias, cudaStream_t stream) {
  // bias (float32 [E] or null) is added to the logits before anything looks at them.
  // sigmoid = 0: softmax scores over all experts.  sigmoid = 1: sigmoid scores, a correction added for the choice
  // (corr float32 [E] or null), the choice limited to `keep` of n_groups groups ranked by their gtop best choice scores.
  if (T <= 0) return 0;
  if (n_groups < 1) n_groups = 1;
  if (E < 1 || top < 1 || top > E || top > MOE_MAX_TOP || (size_t)(2 * E + n_groups) * sizeof(float) > 48 * 1024) return FELLM_ERR_SIZE;
  if (sigmoid && (E % n_groups || keep < 1 || keep > n_groups || gtop < 1 || top > (E / n_groups) * keep)) return FELLM_ERR_SIZE;
  if (!h || !Wr || !idx || !w) return FELLM_ERR_ARG;
  const size_t sh = (size_t)(sigmoid ? 2 * E + n_groups : E) * sizeof(float);
#define ROUTER(TA_, TW_) moe_router_kernel<TA_, TW_><<<T, ROUTER_WARPS * 32, sh, stream>>>((const TA_*)h, ldh, (const TW_*)Wr, K, E, top, renorm, idx, w, sigmoid, corr, n_groups, keep, gtop, bias)
  if (h_bf16) { if (w_bf16) ROUTER(bf16, bf16); else ROUTER(bf16, float); }
  else { if (w_bf16) ROUTER(float, bf16); else ROUTER(float, float); }
#undef ROUTER
  return launch_status();
}

// ---------------------------------------------------------------- the plan
// Pairs p = t * top + c, P of them.  Tile i of PLAN_TILE pairs: counts[i][e] and each pair's rank among the pairs of
// its tile that chose the same expert before it.
__global__ void __launch_bounds__(PLAN_TILE)
moe_count_kernel(const int* __restrict__ idx, int P, int E, int* __restrict__ counts, int* __restrict__ rank) {
  __shared__ int ex[PLAN_TILE];
  const int p = blockIdx.x * PLAN_TILE + threadIdx.x;
  const int e = p < P ? idx[p] : -1;
  ex[threadIdx.x] = e;
  for (int i = threadIdx.x; i < E; i += PLAN_TILE) counts[(size_t)blockIdx.x * E + i] = 0;
  __syncthreads();
  if (e < 0) return;
  int r = 0;
  for (int j = 0; j < (int)threadIdx.x; ++j) r += ex[j] == e;
  rank[p] = r;
  // the last pair of its expert in the tile knows the count
  bool last = true;
  for (int j = threadIdx.x + 1; j < PLAN_TILE && last; ++j) last = ex[j] != e;
  if (last) counts[(size_t)blockIdx.x * E + e] = r + 1;
}

// One block.  base[i][e] = first sorted row of tile i's pairs of expert e (experts in order, tiles in order inside an
// expert); row tiles of BM rows: table[n] = (expert, first row, rows), n_tiles.
__global__ void __launch_bounds__(1024)
moe_scan_kernel(const int* __restrict__ counts, int n_plan_tiles, int E, int BM, int* __restrict__ base,
                int* __restrict__ table, int* __restrict__ n_tiles) {
  extern __shared__ int sh[];            // [E] rows of an expert, then [E] its first row, then [E] its first row tile
  int* rows = sh; int* first = sh + E; int* first_tile = sh + 2 * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int n = 0;
    for (int i = 0; i < n_plan_tiles; ++i) n += counts[(size_t)i * E + e];
    rows[e] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) { first[e] = at; first_tile[e] = tiles; at += rows[e]; tiles += (rows[e] + BM - 1) / BM; }
    *n_tiles = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int at = first[e];
    for (int i = 0; i < n_plan_tiles; ++i) { base[(size_t)i * E + e] = at; at += counts[(size_t)i * E + e]; }
    int n = first_tile[e];
    for (int r = 0; r < rows[e]; r += BM, ++n) {
      table[3 * n] = e; table[3 * n + 1] = first[e] + r; table[3 * n + 2] = min(BM, rows[e] - r);
    }
  }
}

// sorted[place] = pair, place_of[pair] = place
__global__ void moe_place_kernel(const int* __restrict__ idx, const int* __restrict__ rank, const int* __restrict__ base,
                                 int P, int E, int* __restrict__ sorted, int* __restrict__ place_of) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= P) return;
  const int place = base[(size_t)(p / PLAN_TILE) * E + idx[p]] + rank[p];
  sorted[place] = p;
  place_of[p] = place;
}

// Up to PLAN_TILE pairs (a decode step): count, scan and places in one block.
__global__ void __launch_bounds__(PLAN_TILE)
moe_plan_small_kernel(const int* __restrict__ idx, int P, int E, int BM, int* __restrict__ sorted, int* __restrict__ place_of,
                      int* __restrict__ table, int* __restrict__ n_tiles) {
  __shared__ int ex[PLAN_TILE];
  extern __shared__ int sh[];            // [E] rows of an expert, then [E] its first row
  int* rows = sh; int* first = sh + E;
  const int p = threadIdx.x;
  const int e = p < P ? idx[p] : -1;
  ex[p] = e;
  for (int i = p; i < E; i += PLAN_TILE) rows[i] = 0;
  __syncthreads();
  int r = 0;
  if (e >= 0) {
    for (int j = 0; j < p; ++j) r += ex[j] == e;
    bool last = true;
    for (int j = p + 1; j < P && last; ++j) last = ex[j] != e;
    if (last) rows[e] = r + 1;
  }
  __syncthreads();
  if (p == 0) {
    int at = 0, tiles = 0;
    for (int i = 0; i < E; ++i) {
      first[i] = at;
      for (int q = 0; q < rows[i]; q += BM, ++tiles) {
        table[3 * tiles] = i; table[3 * tiles + 1] = at + q; table[3 * tiles + 2] = min(BM, rows[i] - q);
      }
      at += rows[i];
    }
    *n_tiles = tiles;
  }
  __syncthreads();
  if (e >= 0) {
    const int place = first[e] + r;
    sorted[place] = p;
    place_of[p] = place;
  }
}

// scratch (int32): counts [tiles][E] | base [tiles][E] | rank [P]
FELLM_API int fellm_moe_plan(const int* idx, int P, int E, int BM, int* scratch, int* sorted, int* place_of, int* table,
                             int* n_tiles, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E < 1 || BM < 1) return FELLM_ERR_SIZE;
  if (!idx || !scratch || !sorted || !place_of || !table || !n_tiles) return FELLM_ERR_ARG;
  if (P <= PLAN_TILE && (size_t)2 * E * sizeof(int) <= 40 * 1024) {
    moe_plan_small_kernel<<<1, PLAN_TILE, (size_t)2 * E * sizeof(int), stream>>>(idx, P, E, BM, sorted, place_of, table, n_tiles);
    return launch_status();
  }
  const int tiles = (P + PLAN_TILE - 1) / PLAN_TILE;
  int* counts = scratch; int* base = counts + (size_t)tiles * E; int* rank = base + (size_t)tiles * E;
  moe_count_kernel<<<tiles, PLAN_TILE, 0, stream>>>(idx, P, E, counts, rank);
  const size_t sh = (size_t)3 * E * sizeof(int);
  if (sh > 48 * 1024) return FELLM_ERR_SIZE;
  moe_scan_kernel<<<1, 1024, sh, stream>>>(counts, tiles, E, BM, base, table, n_tiles);
  moe_place_kernel<<<(P + 255) / 256, 256, 0, stream>>>(idx, rank, base, P, E, sorted, place_of);
  return launch_status();
}

// ---------------------------------------------------------------- grouped products, float32 FMA
// Every output is ONE chain of fused multiply-adds over k = 0..K-1: the 32-bit engine's product, and the bfloat16
// engine's where the tensor-core kernel below does not take a size.
// GATED: W[e] is [2N, K]; the epilogue stores SiLU(gate) * up.  inter = 0: the N gate rows first, then the N up
// rows; inter = 1: blocks of 8 gate rows and 8 up rows by turns (the layout the tcgen05 product's epilogue reads).
// Rows of A: gather[row] / top when gather is given (a pair's token), else the sorted row itself.
__device__ __forceinline__ int gate_row(int n, int inter) { return inter ? ((n >> 3) << 4) + (n & 7) : n; }
__device__ __forceinline__ int up_row(int n, int N, int inter) { return inter ? ((n >> 3) << 4) + 8 + (n & 7) : N + n; }
#define FB 64
#define FK 16
template <typename TA, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_fma_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ gather, int top,
                    const TW* __restrict__ W, TO* __restrict__ C, int ldc, int N, int K,
                    const int* __restrict__ table, const int* __restrict__ n_tiles, int inter, float act_limit, float act_alpha) {
  if ((int)blockIdx.x >= *n_tiles) return;
  __shared__ float As[FK][FB + 1];
  __shared__ float Ws[GATED ? 2 : 1][FK][FB + 1];
  __shared__ int arow[FB];
  const int e = table[3 * blockIdx.x], row0 = table[3 * blockIdx.x + 1], rows = table[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * FB;
  const TW* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
  for (int r = threadIdx.x; r < FB; r += 256)
    arow[r] = r < rows ? (gather ? gather[row0 + r] / top : row0 + r) : -1;
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 4 columns x 4 rows a thread
  float acc[4][4], acc2[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = acc2[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += FK) {
    for (int i = threadIdx.x; i < FB * FK; i += 256) {
      const int r = i / FK, k = i - r * FK;
      const int ar = arow[r];
      As[k][r] = (ar >= 0 && k0 + k < K) ? to_f(A[(size_t)ar * lda + k0 + k]) : 0.f;
      const int n = n0 + r;
      const bool ok = n < N && k0 + k < K;
      Ws[0][k][r] = ok ? to_f(We[(size_t)(GATED ? gate_row(n, inter) : n) * K + k0 + k]) : 0.f;
      if (GATED) Ws[1][k][r] = ok ? to_f(We[(size_t)up_row(n, N, inter) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < FK; ++k) {
      float a[4], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { b[j] = Ws[0][k][tx * 4 + j]; if (GATED) b2[j] = Ws[1][k][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (GATED) {
        // in the bfloat16 engine gate and up are activations like those of the dense feed-forward: rounded first
        float g = to_f(from_f<TA>(v)), u = to_f(from_f<TA>(acc2[i][j]));
        v = glu_act(g, u, act_limit, act_alpha);
      }
      C[(size_t)(row0 + r) * ldc + n] = from_f<TO>(v);
    }
  }
}

// ---------------------------------------------------------------- grouped products, bfloat16 tensor cores
// 64 rows x 64 columns a CTA (x 2 column sets when GATED), K in steps of 32 through shared memory (rows padded to 40
// elements: the fragment loads of a warp fall on different banks), four warps of 16 rows each, mma.m16n8k16 with
// float32 accumulators.  A token's sum over K is the same chain of MMAs wherever the row lies in its tile.
#define TB 64
#define TK 32
#define TLD 40
__device__ __forceinline__ void mma16816(float* d, const unsigned* a, const unsigned* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename TO, bool GATED>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ gather, int top,
                    const bf16* __restrict__ W, TO* __restrict__ C, int ldc, int N, int K,
                    const int* __restrict__ table, const int* __restrict__ n_tiles, int inter, float act_limit, float act_alpha) {
  if ((int)blockIdx.x >= *n_tiles) return;
  __shared__ __align__(16) bf16 As[2][TB * TLD];
  __shared__ __align__(16) bf16 Ws[2][(GATED ? 2 : 1) * TB * TLD];
  __shared__ int arow[TB];
  const int e = table[3 * blockIdx.x], row0 = table[3 * blockIdx.x + 1], rows = table[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * TB;
  const bf16* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
  for (int r = threadIdx.x; r < TB; r += 128)
    arow[r] = r < rows ? (gather ? gather[row0 + r] / top : row0 + r) : -1;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  constexpr int NB = GATED ? 16 : 8;                   // blocks of 8 columns a warp: 64 columns (and 64 of the up set)
  float acc[NB][4];
#pragma unroll
  for (int j = 0; j < NB; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  // a thread copies 16 bytes at a time: 64 rows x 4 vectors of A, and of each column set of W
  auto stage = [&](int buf, int k0) {
    for (int i = threadIdx.x; i < TB * 4; i += 128) {
      const int r = i >> 2, kv = (i & 3) * 8;
      uint4 va = make_uint4(0, 0, 0, 0), vw = make_uint4(0, 0, 0, 0), vw2 = make_uint4(0, 0, 0, 0);
      const int ar = arow[r];
      if (ar >= 0 && k0 + kv < K) va = *(const uint4*)(A + (size_t)ar * lda + k0 + kv);
      const int n = n0 + r;
      if (n < N && k0 + kv < K) {
        vw = *(const uint4*)(We + (size_t)(GATED ? gate_row(n, inter) : n) * K + k0 + kv);
        if (GATED) vw2 = *(const uint4*)(We + (size_t)up_row(n, N, inter) * K + k0 + kv);
      }
      *(uint4*)(&As[buf][r * TLD + kv]) = va;
      *(uint4*)(&Ws[buf][r * TLD + kv]) = vw;
      if (GATED) *(uint4*)(&Ws[buf][(TB + r) * TLD + kv]) = vw2;
    }
  };
  const int n_k = (K + TK - 1) / TK;
  stage(0, 0);
  __syncthreads();
  for (int kb = 0; kb < n_k; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < n_k) stage(buf ^ 1, (kb + 1) * TK);
    const bf16* as = As[buf] + (warp * 16) * TLD;
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      unsigned a[4];
      a[0] = *(const unsigned*)(as + gid * TLD + kk + tig * 2);
      a[1] = *(const unsigned*)(as + (gid + 8) * TLD + kk + tig * 2);
      a[2] = *(const unsigned*)(as + gid * TLD + kk + 8 + tig * 2);
      a[3] = *(const unsigned*)(as + (gid + 8) * TLD + kk + 8 + tig * 2);
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const bf16* ws = Ws[buf] + (j * 8 + gid) * TLD + kk + tig * 2;
        unsigned b[2];
        b[0] = *(const unsigned*)ws;
        b[1] = *(const unsigned*)(ws + 8);
        mma16816(acc[j], a, b);
      }
    }
    __syncthreads();
  }
  // c0, c1: row gid, columns 2 tig, 2 tig + 1; c2, c3: row gid + 8
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = warp * 16 + gid + half * 8;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int n = n0 + j * 8 + tig * 2 + c;
        if (n >= N) continue;
        float v = acc[j][half * 2 + c];
        if (GATED) {
          const float g = to_f(from_f<bf16>(v)), u = to_f(from_f<bf16>(acc[8 + j][half * 2 + c]));
          v = glu_act(g, u, act_limit, act_alpha);
        }
        C[(size_t)(row0 + r) * ldc + n] = from_f<TO>(v);
      }
    }
  }
}

// Few rows (a decode step): the product is bound by reading each chosen expert's matrix once.  A warp owns one
// output column of a row tile (and, GATED, the column's up partner): it streams the column's weight row(s) 16 bytes a
// lane at a time against up to VR rows of A at once (more rows: again, the weights then come from L1 / L2), the lanes'
// sums are added by a butterfly.  bfloat16 only; K a multiple of 8.
#define VW 8            // warps a block
#define VR 4            // rows at once
__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* h = (const __nv_bfloat162*)&raw;
#pragma unroll
  for (int e = 0; e < 4; ++e) { float2 v = __bfloat1622float2(h[e]); f[2 * e] = v.x; f[2 * e + 1] = v.y; }
}
// A warp's columns: n and, GATED, its up partner; not gated: n and n + 1 (two weight rows against the same rows of A).
template <typename TO, bool GATED>
__global__ void __launch_bounds__(VW * 32)
moe_gemv_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ gather, int top,
                const bf16* __restrict__ W, TO* __restrict__ C, int ldc, int N, int K,
                const int* __restrict__ table, const int* __restrict__ n_tiles, int inter, float act_limit, float act_alpha) {
  if ((int)blockIdx.x >= *n_tiles) return;
  const int e = table[3 * blockIdx.x], row0 = table[3 * blockIdx.x + 1], rows = table[3 * blockIdx.x + 2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = GATED ? blockIdx.y * VW + warp : 2 * (blockIdx.y * VW + warp);
  if (n >= N) return;
  const bool two = !GATED && n + 1 < N;
  const bf16* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
  const bf16* w0 = We + (size_t)(GATED ? gate_row(n, inter) : n) * K;
  const bf16* w1 = GATED ? We + (size_t)up_row(n, N, inter) * K : (two ? w0 + K : w0);
  for (int r0 = 0; r0 < rows; r0 += VR) {
    const bf16* ar[VR];
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      const int r = min(r0 + i, rows - 1);
      ar[i] = A + (size_t)(gather ? gather[row0 + r] / top : row0 + r) * lda;
    }
    const int nr = min(VR, rows - r0);
    float s0[VR], s1[VR];
#pragma unroll
    for (int i = 0; i < VR; ++i) s0[i] = s1[i] = 0.f;
    // two steps of K at once: four 16-byte loads of weights in flight a lane before the first is used
    for (int k = lane * 8; k < K; k += 512) {
      const bool second = k + 256 < K;
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const uint4 ra0 = *(const uint4*)(w0 + k), rb0 = *(const uint4*)(w1 + k);
      const uint4 ra1 = second ? *(const uint4*)(w0 + k + 256) : zero, rb1 = second ? *(const uint4*)(w1 + k + 256) : zero;
      uint4 xa[VR], xb[VR];
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        xa[i] = i < nr ? *(const uint4*)(ar[i] + k) : zero;
        xb[i] = (i < nr && second) ? *(const uint4*)(ar[i] + k + 256) : zero;
      }
      float f0[8], f1[8], g0[8], g1[8];
      unpack8(ra0, f0); unpack8(rb0, f1); unpack8(ra1, g0); unpack8(rb1, g1);
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        float fa[8], fb[8];
        unpack8(xa[i], fa); unpack8(xb[i], fb);
#pragma unroll
        for (int j = 0; j < 8; ++j) { s0[i] = fmaf(fa[j], f0[j], s0[i]); s1[i] = fmaf(fa[j], f1[j], s1[i]); }
#pragma unroll
        for (int j = 0; j < 8; ++j) { s0[i] = fmaf(fb[j], g0[j], s0[i]); s1[i] = fmaf(fb[j], g1[j], s1[i]); }
      }
    }
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      float a = warp_sum(s0[i]), b = warp_sum(s1[i]);
      if (lane == 0 && r0 + i < rows) {
        if (GATED) {
          a = to_f(from_f<bf16>(a)); b = to_f(from_f<bf16>(b));
          C[(size_t)(row0 + r0 + i) * ldc + n] = from_f<TO>(glu_act(a, b, act_limit, act_alpha));
        } else {
          C[(size_t)(row0 + r0 + i) * ldc + n] = from_f<TO>(a);
          if (two) C[(size_t)(row0 + r0 + i) * ldc + n + 1] = from_f<TO>(b);
        }
      }
    }
  }
}

// A [*, lda] (bfloat16 or float32), W [E][(gated ? 2 : 1) * N][K] of the same kind; C [P, ldc]: bfloat16 or float32
// when gated (the activation), float32 otherwise.  max_tiles: the table's capacity = the launch's first extent.
FELLM_API int fellm_moe_gemm(const void* A, int a_bf16, int lda, const int* gather, int top, const void* W, int w_bf16,
                             void* C, int c_bf16, int ldc, int N, int K, int gated, const int* table, const int* n_tiles,
                             int max_tiles, int use_mma, int inter, int few_rows, float act_limit, float act_alpha, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  if (N < 1 || K < 1 || top < 1) return FELLM_ERR_SIZE;
  if (!A || !W || !C || !table || !n_tiles) return FELLM_ERR_ARG;
  if (a_bf16 != w_bf16 || (!gated && c_bf16) || (gated && c_bf16 != a_bf16)) return FELLM_ERR_ARG;
  const bool mma = use_mma && a_bf16 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0;
  if (mma && few_rows) {
    dim3 grid(max_tiles, gated ? (N + VW - 1) / VW : (N + 2 * VW - 1) / (2 * VW));
    if (gated)
      moe_gemv_kernel<bf16, true><<<grid, VW * 32, 0, stream>>>((const bf16*)A, lda, gather, top, (const bf16*)W, (bf16*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
    else
      moe_gemv_kernel<float, false><<<grid, VW * 32, 0, stream>>>((const bf16*)A, lda, gather, top, (const bf16*)W, (float*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
    return launch_status();
  }
  if (mma) {
    dim3 grid(max_tiles, (N + TB - 1) / TB);
    if (gated)
      moe_gemm_mma_kernel<bf16, true><<<grid, 128, 0, stream>>>((const bf16*)A, lda, gather, top, (const bf16*)W, (bf16*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
    else
      moe_gemm_mma_kernel<float, false><<<grid, 128, 0, stream>>>((const bf16*)A, lda, gather, top, (const bf16*)W, (float*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
    return launch_status();
  }
  dim3 grid(max_tiles, (N + FB - 1) / FB);
  if (a_bf16) {
    if (gated)
      moe_gemm_fma_kernel<bf16, bf16, bf16, true><<<grid, 256, 0, stream>>>((const bf16*)A, lda, gather, top, (const bf16*)W, (bf16*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
    else
      moe_gemm_fma_kernel<bf16, bf16, float, false><<<grid, 256, 0, stream>>>((const bf16*)A, lda, gather, top, (const bf16*)W, (float*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
  } else {
    if (gated)
      moe_gemm_fma_kernel<float, float, float, true><<<grid, 256, 0, stream>>>((const float*)A, lda, gather, top, (const float*)W, (float*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
    else
      moe_gemm_fma_kernel<float, float, float, false><<<grid, 256, 0, stream>>>((const float*)A, lda, gather, top, (const float*)W, (float*)C, ldc, N, K, table, n_tiles, inter, act_limit, act_alpha);
  }
  return launch_status();
}

// ---------------------------------------------------------------- rows in sorted order
// out[r, :] = a[sorted[r] / top, :]   (bfloat16, K a multiple of 8: 16 bytes a thread): the input of the tcgen05
// grouped product, whose TMA boxes want an expert's rows side by side.
__global__ void moe_gather_kernel(const bf16* __restrict__ a, int lda, const int* __restrict__ sorted, int top,
                                  bf16* __restrict__ out, int K) {
  const int r = blockIdx.x;
  const bf16* src = a + (size_t)(sorted[r] / top) * lda;
  bf16* dst = out + (size_t)r * K;
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) *(uint4*)(dst + k) = *(const uint4*)(src + k);
}

FELLM_API int fellm_moe_gather(const void* a, int lda, const int* sorted, int top, void* out, int P, int K, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (!a || !sorted || !out) return FELLM_ERR_ARG;
  if (K % 8 || lda % 8 || ((uintptr_t)a % 16) || ((uintptr_t)out % 16)) return FELLM_ERR_SIZE;
  moe_gather_kernel<<<P, 128, 0, stream>>>((const bf16*)a, lda, sorted, top, (bf16*)out, K);
  return launch_status();
}

// ---------------------------------------------------------------- the weighted sum into the residual stream
// x[t, :] += sum_c w[t, c] * y[place_of[t * top + c], :], c = 0 .. top-1 in order, float32 (store: x[t, :] = the sum).
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, const int* __restrict__ place_of,
                                   const float* __restrict__ w, int top, int d, int store) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float s = 0.f;
    for (int c = 0; c < top; ++c) s = fmaf(w[(size_t)t * top + c], y[(size_t)place_of[(size_t)t * top + c] * d + i], s);
    x[(size_t)t * d + i] = store ? s : x[(size_t)t * d + i] + s;
  }
}

FELLM_API int fellm_moe_combine(float* x, const float* y, const int* place_of, const float* w, int T, int top, int d,
                                int store, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!x || !y || !place_of || !w) return FELLM_ERR_ARG;
  moe_combine_kernel<<<T, d >= 256 ? 256 : 128, 0, stream>>>(x, y, place_of, w, top, d, store);
  return launch_status();
}
