// A feed-forward of routed experts: the router's choice, the sort of (token, expert) pairs into
// tiles of one expert each, the two grouped products, and the weighted sum.
//
//   route:    s = sigmoid(z), or softmax(z) over all experts (score_kind 1); choice = s + correction;
//             experts in equal groups of neighbours, a group's score the sum of its `group_top` (1 or
//             2) largest choice scores, the best `group_keep` groups stay; of their experts the `top`
//             largest choice scores win (ties: the lower index); weight_j = s_j / (sum of the chosen
//             s + eps) * scale, or s_j * scale (normalize 0).  One warp per token, float32.
//   sort:     pairs p = t * top + j are placed, by expert, into tiles of `tile` rows; an expert's
//             rows are filled up to whole tiles (row -> pair or -1; tile -> expert or -1).
//   gate/up:  hidden[row] = silu(x[token] Wg_e^T) * (x[token] Wu_e^T), rounded once to x's type.
//   down:     per_pair[pair] = hidden[row] Wd_e^T, float32.
//   combine:  out[t] = sum_j weight[t, j] per_pair[t * top + j] (in the order of j)
//                      + sigmoid(logits[t, col]) * shared[t] (col < 0: + shared[t]).
//
// A row's sums never depend on the other rows of its tile, on the tile's size or on where the row
// sits in it: bfloat16 products run on the tensor cores (mma.sync m16n8k16, float32 accumulators,
// k in ascending steps of 32), everything else on the CUDA cores with k in ascending order.
#include "source.cuh"

namespace {

constexpr float NEG_INF = -__builtin_huge_valf();

// ---- the router ------------------------------------------------------------------------------
// (value, index) of the larger; ties go to the lower index
__device__ __forceinline__ void arg_best(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
__device__ __forceinline__ void warp_arg_best(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    arg_best(v, i, ov, oi);
  }
}

constexpr int ROUTE_WARPS = 4;
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(Source logits, long long row_width, const float* __restrict__ correction, int* __restrict__ ids,
                 float* __restrict__ weights, int T, int E, int top, int groups, int keep, float scale, float eps,
                 int score_kind, int group_top, int normalize) {
  extern __shared__ float smem[];            // per warp: s [E], choice [E], group score [groups]
  pdl_prologue(logits.p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* s = smem + (size_t)warp * (2 * E + groups);
  float* choice = s + E;
  float* gscore = choice + E;
  const int per = E / groups;
  if (score_kind == 1) {
    // softmax over all experts: the largest logit, then the sum of the exponentials in a fixed order
    float mx = NEG_INF;
    for (int e = lane; e < E; e += 32) {
      const float z = source_load(logits, (long long)t * row_width + e);
      s[e] = z;
      mx = fmaxf(mx, z);
    }
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = expf(s[e] - mx);
      s[e] = v;
      den = __fadd_rn(den, v);
    }
    den = warp_sum(den);
    for (int e = lane; e < E; e += 32) {
      const float v = s[e] / den;
      s[e] = v;
      choice[e] = __fadd_rn(v, correction[e]);
    }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float v = sigmoid_f32(source_load(logits, (long long)t * row_width + e));
      s[e] = v;
      choice[e] = __fadd_rn(v, correction[e]);
    }
  }
  __syncwarp();
  if (groups > 1) {
    for (int g = lane; g < groups; g += 32) {
      float a = NEG_INF, b = NEG_INF;        // the largest and the second largest of the group
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) { b = a; a = c; }
        else if (c > b) b = c;
      }
      gscore[g] = (per > 1 && group_top > 1) ? __fadd_rn(a, b) : a;
    }
    __syncwarp();
    // the best `keep` groups, one after the other; a kept group's score is replaced by +infinity
    for (int n = 0; n < keep; ++n) {
      float v = NEG_INF;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float c = gscore[g];
        if (c != __builtin_huge_valf()) arg_best(v, at, c, g);
      }
      warp_arg_best(v, at);
      if (lane == 0 && at < groups) gscore[at] = __builtin_huge_valf();
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gscore[e / per] != __builtin_huge_valf()) choice[e] = NEG_INF;
    __syncwarp();
  }
  float sum = 0.f, mine = 0.f;               // lane j keeps the j-th chosen expert's score
  int mine_id = 0;
  for (int n = 0; n < top; ++n) {
    float v = NEG_INF;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = choice[e];
      if (s[e] >= 0.f) arg_best(v, at, c, e);      // (a taken expert's s is set below zero)
    }
    warp_arg_best(v, at);
    if (at >= E) at = 0;                     // (cannot happen: top <= keep * per)
    const float sv = s[at];
    sum = __fadd_rn(sum, sv);
    if (lane == n) { mine = sv; mine_id = at; }
    __syncwarp();
    if (lane == 0) s[at] = -1.f;
    __syncwarp();
  }
  if (lane < top) {
    ids[(long long)t * top + lane] = mine_id;
    weights[(long long)t * top + lane] = normalize ? mine / __fadd_rn(sum, eps) * scale : __fmul_rn(mine, scale);
  }
}

// ---- the sort -----------------------------------------------------------------------------------
// order: int32 [max_tiles * tile] row -> pair (-1: padding), then [max_tiles] tile -> expert (-1: unused), then
// one entry: the number of tiles in use (they are the first ones).
// One block.  Where a pair lands inside its expert's rows depends on the order in which threads arrive,
// which no result depends on (a row's sums do not know the row's place).
constexpr int SORT_THREADS = 1024;
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int* __restrict__ ids, int pairs, int E, int tile, int max_tiles, int* __restrict__ order) {
  __shared__ int count[SORT_THREADS], first_tile[SORT_THREADS + 1], scan[SORT_THREADS];
  pdl_prologue(ids);
  const int e = threadIdx.x;
  count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += SORT_THREADS) {
    const int x = ids[i];
    if (x >= 0 && x < E) atomicAdd(&count[x], 1);
  }
  __syncthreads();
  const int my_tiles = e < E ? (count[e] + tile - 1) / tile : 0;
  scan[e] = my_tiles;
  __syncthreads();
  for (int o = 1; o < SORT_THREADS; o <<= 1) {        // inclusive scan
    const int v = e >= o ? scan[e - o] : 0;
    __syncthreads();
    scan[e] += v;
    __syncthreads();
  }
  first_tile[e + 1] = scan[e];
  if (e == 0) first_tile[0] = 0;
  count[e] = 0;                                       // now the expert's cursor
  __syncthreads();
  int* tile_expert = order + (long long)max_tiles * tile;
  for (int i = threadIdx.x; i < max_tiles * tile; i += SORT_THREADS) order[i] = -1;
  for (int i = threadIdx.x; i < max_tiles; i += SORT_THREADS) tile_expert[i] = -1;
  __syncthreads();
  if (e < E)
    for (int k = first_tile[e]; k < first_tile[e + 1] && k < max_tiles; ++k) tile_expert[k] = e;
  if (e == 0) tile_expert[max_tiles] = first_tile[E] < max_tiles ? first_tile[E] : max_tiles;   // tiles in use: the first ones
  for (int i = threadIdx.x; i < pairs; i += SORT_THREADS) {
    const int x = ids[i];
    if (x < 0 || x >= E) continue;
    const long long at = (long long)first_tile[x] * tile + atomicAdd(&count[x], 1);
    if (at < (long long)max_tiles * tile) order[at] = i;
  }
}

// ---- the grouped products -------------------------------------------------------------------------
// mode 0 (gate and up): A row r = x[pair / top] (K = the model's width), B = the expert's [2F][K] (gate
// rows, then up rows), out hidden[row][F] = silu(gate) * up in T.
// mode 1 (down): A row r = hidden[row] (K = F), B = the expert's [N][K], out per_pair[pair][N] float32.

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Tensor-core form, bfloat16, K a multiple of 8.  A CTA of four warps takes one tile of MT * 16 rows and,
// per warp, NJ blocks of 8 columns (mode 0: NJ / 2 of the gate and the same columns of up).  A thread
// fetches 8 consecutive k of a weight row with one 16-byte load; the four threads of a column cover a
// step of 32 k.  Inside a step the products are handed to the tensor cores in a fixed permutation of k
// (a thread's first four k to one instruction, its last four to the next), the same for A and B, so
// the step's sum is that of all 32 products; the A rows of the step come from shared memory, 16 bytes
// a thread and row.
constexpr int GP_THREADS = 128, GP_PAD = 32;      // (rows 64 bytes apart modulo 128: a quarter warp's 16-byte loads meet no bank twice)
template <int MT, int NJ>
__global__ void __launch_bounds__(GP_THREADS)
moe_product_mma_kernel(const __nv_bfloat16* __restrict__ a_rows, const int* __restrict__ order, int max_tiles,
                       int tile, int top, const __nv_bfloat16* __restrict__ w, void* out, int K, int N, int KC,
                       int mode) {
  extern __shared__ __align__(16) unsigned char gp_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gp_smem);     // [MT * 16][KC + GP_PAD]
  __shared__ int row_pair[MT * 16];
  pdl_prologue(a_rows, order);
  const int tl = blockIdx.x;
  const int expert = order[(long long)max_tiles * tile + tl];
  if (expert < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  constexpr int ROWS = MT * 16;
  for (int r = threadIdx.x; r < ROWS; r += GP_THREADS) row_pair[r] = r < tile ? order[(long long)tl * tile + r] : -1;
  // this warp's column blocks: rows of B
  const int rows_b = mode == 0 ? 2 * N : N;
  const __nv_bfloat16* wb = w + (long long)expert * rows_b * K;
  const int n0 = mode == 0 ? (blockIdx.y * 4 + warp) * (NJ / 2) * 8 : (blockIdx.y * 4 + warp) * NJ * 8;
  const __nv_bfloat16* brow[NJ];
  bool bok[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    int n;                 // the column of the output this thread's B row feeds
    long long rb;          // its row in B
    if (mode == 0) { n = n0 + (j % (NJ / 2)) * 8 + g; rb = j < NJ / 2 ? n : (long long)N + n; }
    else { n = n0 + j * 8 + g; rb = n; }
    bok[j] = n < N;
    brow[j] = wb + (bok[j] ? rb : 0) * K + tig * 8;
  }
  float acc[MT][NJ][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f;
  const int as = KC + GP_PAD;
  __syncthreads();
  for (int kc = 0; kc < K; kc += KC) {
    const int klen = K - kc < KC ? K - kc : KC;                    // a multiple of 8
    const int kpad = (klen + 31) / 32 * 32;
    if (kc > 0) __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * (kpad / 8); idx += GP_THREADS) {
      const int r = idx / (kpad / 8), c8 = idx - r * (kpad / 8);
      const int pair = row_pair[r];
      uint4 v = make_uint4(0, 0, 0, 0);
      if (pair >= 0 && c8 * 8 < klen) {
        const long long arow = mode == 0 ? pair / top : (long long)tl * tile + r;
        v = *reinterpret_cast<const uint4*>(a_rows + arow * K + kc + c8 * 8);
      }
      *reinterpret_cast<uint4*>(As + r * as + c8 * 8) = v;
    }
    __syncthreads();
    // (tiles of 16 rows are bound by the weight loads in flight: four steps' loads are issued ahead)
#pragma unroll(MT == 1 ? 4 : 2)
    for (int k = 0; k < kpad; k += 32) {
      uint4 b[NJ];
      const bool kin = k + tig * 8 < klen;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        b[j] = (bok[j] && kin) ? __ldg(reinterpret_cast<const uint4*>(brow[j] + kc + k)) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4 lo = *reinterpret_cast<const uint4*>(As + (m * 16 + g) * as + k + tig * 8);
        const uint4 hi = *reinterpret_cast<const uint4*>(As + (m * 16 + g + 8) * as + k + tig * 8);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          mma_bf16_16816(acc[m][j], lo.x, hi.x, lo.y, hi.y, b[j].x, b[j].y);
          mma_bf16_16816(acc[m][j], lo.z, hi.z, lo.w, hi.w, b[j].z, b[j].w);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = m * 16 + g + 8 * hh;
      const int pair = row_pair[r];
      if (pair < 0) continue;
      if (mode == 0) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + ((long long)tl * tile + r) * N;
#pragma unroll
        for (int j = 0; j < NJ / 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int n = n0 + j * 8 + tig * 2 + e;
            const float gt = acc[m][j][2 * hh + e], up = acc[m][j + NJ / 2][2 * hh + e];
            if (n < N) dst[n] = __float2bfloat16_rn(gt * sigmoid_f32(gt) * up);
          }
      } else {
        float* dst = reinterpret_cast<float*>(out) + (long long)pair * N;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int n = n0 + j * 8 + tig * 2 + e;
            if (n < N) dst[n] = acc[m][j][2 * hh + e];
          }
      }
    }
}

// CUDA-core form: any type, any sizes.  A CTA takes 16 rows of a tile (blockIdx.z picks them) and 128
// columns, a thread a column (mode 0: of the gate and of up); k in ascending order, one chain per sum.
constexpr int GC_ROWS = 16, GC_COLS = 128, GC_K = 128;
template <typename T>
__global__ void __launch_bounds__(GC_COLS)
moe_product_kernel(const T* __restrict__ a_rows, const int* __restrict__ order, int max_tiles, int tile, int top,
                   const T* __restrict__ w, void* out, int K, int N, int mode) {
  __shared__ float xs[GC_ROWS][GC_K];
  __shared__ int row_pair[GC_ROWS];
  pdl_prologue(a_rows, order);
  const int tl = blockIdx.x;
  const int expert = order[(long long)max_tiles * tile + tl];
  if (expert < 0) return;
  const int r0 = blockIdx.z * GC_ROWS;
  if (threadIdx.x < GC_ROWS)
    row_pair[threadIdx.x] = r0 + threadIdx.x < tile ? order[(long long)tl * tile + r0 + threadIdx.x] : -1;
  const int n = blockIdx.y * GC_COLS + threadIdx.x;
  const int rows_b = mode == 0 ? 2 * N : N;
  const T* w0 = w + ((long long)expert * rows_b + (n < N ? n : 0)) * K;
  const T* w1 = w0 + (long long)N * K;               // (mode 0: the column's up row)
  float acc0[GC_ROWS], acc1[GC_ROWS];
#pragma unroll
  for (int r = 0; r < GC_ROWS; ++r) acc0[r] = acc1[r] = 0.f;
  __syncthreads();
  for (int kc = 0; kc < K; kc += GC_K) {
    const int klen = K - kc < GC_K ? K - kc : GC_K;
    if (kc > 0) __syncthreads();
    for (int idx = threadIdx.x; idx < GC_ROWS * GC_K; idx += GC_COLS) {
      const int r = idx / GC_K, k = idx - r * GC_K;
      const int pair = row_pair[r];
      float v = 0.f;
      if (pair >= 0 && k < klen) {
        const long long arow = mode == 0 ? pair / top : (long long)tl * tile + r0 + r;
        v = Elem<T>::load(a_rows + arow * K + kc + k);
      }
      xs[r][k] = v;
    }
    __syncthreads();
    if (n < N)
      for (int k = 0; k < klen; ++k) {
        const float b0 = Elem<T>::load(w0 + kc + k);
        const float b1 = mode == 0 ? Elem<T>::load(w1 + kc + k) : 0.f;
#pragma unroll
        for (int r = 0; r < GC_ROWS; ++r) {
          acc0[r] = __fmaf_rn(xs[r][k], b0, acc0[r]);
          if (mode == 0) acc1[r] = __fmaf_rn(xs[r][k], b1, acc1[r]);
        }
      }
  }
  if (n >= N) return;
#pragma unroll
  for (int r = 0; r < GC_ROWS; ++r) {
    const int pair = row_pair[r];
    if (pair < 0) continue;
    if (mode == 0)
      Elem<T>::store(reinterpret_cast<T*>(out) + ((long long)tl * tile + r0 + r) * N + n,
                     acc0[r] * sigmoid_f32(acc0[r]) * acc1[r]);
    else
      reinterpret_cast<float*>(out)[(long long)pair * N + n] = acc0[r];
  }
}

// out[t, c] = sum_j weights[t, j] * per_pair[t * top + j, c], j ascending, + sigmoid(gate[t]) * shared[t, c]
// (gate_col < 0: the shared expert has no gate and is added as it is)
__global__ void moe_combine_kernel(const float* __restrict__ per_pair, const float* __restrict__ weights, Source shared,
                                   Source logits, long long logit_row, int gate_col, float* __restrict__ out, int T,
                                   int top, int W) {
  pdl_prologue(per_pair, weights, shared.p, logits.p);
  const long long n = (long long)T * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / W, c = i - t * W;
    float v = 0.f;
    for (int j = 0; j < top; ++j) v = __fmaf_rn(weights[t * top + j], per_pair[(t * top + j) * W + c], v);
    if (shared.p != nullptr)
      v = gate_col < 0 ? __fadd_rn(v, source_load(shared, i))
                       : __fmaf_rn(sigmoid_f32(source_load(logits, t * logit_row + gate_col)), source_load(shared, i), v);
    out[i] = v;
  }
}

template <int MT, int NJ>
int launch_product_mma(const void* a_rows, const int* order, int max_tiles, int tile, int top, const void* w, void* out,
                       int K, int N, int mode, cudaStream_t st) {
  // the A rows' k are staged in runs of KC (a multiple of 64) that fit 64 KB; tiles of 16 rows (decoded
  // tokens: the product is bound by how many weight loads an SM keeps in flight) in runs that fit 16 KB,
  // so that an SM holds many CTAs.  The runs do not change the order of a sum.
  int KC = ((MT == 1 ? 16 : 64) * 1024 / (MT * 16 * 2) - GP_PAD) / 64 * 64;
  if (KC > (K + 63) / 64 * 64) KC = (K + 63) / 64 * 64;
  const size_t smem = (size_t)MT * 16 * (KC + GP_PAD) * 2;
  static DeviceOnce once;
  if (smem > 48 * 1024 && !once.done()) {
    if (cudaFuncSetAttribute(moe_product_mma_kernel<MT, NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) !=
        cudaSuccess)
      return DIB_LAUNCH_FAILED;
    once.mark();
  }
  const int per_cta = mode == 0 ? 16 * NJ : 32 * NJ;
  dib_launch(moe_product_mma_kernel<MT, NJ>, dim3(max_tiles, (N + per_cta - 1) / per_cta), dim3(GP_THREADS), smem, st,
             (const __nv_bfloat16*)a_rows, order, max_tiles, tile, top, (const __nv_bfloat16*)w, out, K, N, KC, mode);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// mode 0: gate and up; 1: down.  dtype 0 float32, 1 bfloat16.
int moe_product(const void* a_rows, int dtype, const int* order, int max_tiles, int tile, int top, const void* w,
                void* out, int K, int N, int mode, cudaStream_t st) {
  if (max_tiles == 0) return DIB_OK;
  if (K < 1 || N < 1 || tile < 1 || tile % GC_ROWS || top < 1) return DIB_BAD_SIZE;
  if (dtype == 1 && K % 8 == 0 && (tile == 16 || tile == 64)) {
    if (tile == 16) return launch_product_mma<1, 4>(a_rows, order, max_tiles, tile, top, w, out, K, N, mode, st);
    return launch_product_mma<4, 4>(a_rows, order, max_tiles, tile, top, w, out, K, N, mode, st);
  }
  const dim3 grid(max_tiles, (N + GC_COLS - 1) / GC_COLS, tile / GC_ROWS);
  if (dtype == 0)
    dib_launch(moe_product_kernel<float>, grid, dim3(GC_COLS), 0, st, (const float*)a_rows, order, max_tiles, tile, top,
               (const float*)w, out, K, N, mode);
  else if (dtype == 1)
    dib_launch(moe_product_kernel<__nv_bfloat16>, grid, dim3(GC_COLS), 0, st, (const __nv_bfloat16*)a_rows, order,
               max_tiles, tile, top, (const __nv_bfloat16*)w, out, K, N, mode);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// ---- the sorted rows as matrices of their own (for the tensor-core product of whole tiles) ----------
// a_sorted[row] = x[order[row] / top] (a padding row: zeros); 16 bytes a thread and step.
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ order, long long rows,
                                       int top, int vecs, uint4* __restrict__ a_sorted) {
  pdl_prologue(order);
  const long long n = rows * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vecs;
    const int v = (int)(i - row * vecs);
    const int pair = order[row];
    a_sorted[i] = pair >= 0 ? x[(long long)(pair / top) * vecs + v] : make_uint4(0u, 0u, 0u, 0u);
  }
}
// per_pair[order[row]] = y_sorted[row]
__global__ void moe_scatter_rows_kernel(const float4* __restrict__ y_sorted, const int* __restrict__ order, long long rows,
                                        int vecs, float4* __restrict__ per_pair) {
  pdl_prologue(y_sorted);
  const long long n = rows * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vecs;
    const int pair = order[row];
    if (pair >= 0) per_pair[(long long)pair * vecs + (i - row * vecs)] = y_sorted[i];
  }
}

}  // namespace

extern "C" {

// x bfloat16 [T, W] (W a multiple of 8) -> a_sorted bfloat16 [rows, W] in the order of `order`
int dib_moe_gather_rows(const void* x, const int* order, long long rows, int top, int W, void* a_sorted,
                        cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (W < 8 || W % 8 != 0 || top < 1) return DIB_BAD_SIZE;
  const long long n = rows * (W / 8);
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  dib_launch(moe_gather_rows_kernel, dim3(blocks), dim3(256), 0, st, (const uint4*)x, order, rows, top, W / 8,
             (uint4*)a_sorted);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// y_sorted float32 [rows, W] (W a multiple of 4) -> per_pair float32 [pairs, W]
int dib_moe_scatter_rows(const float* y_sorted, const int* order, long long rows, int W, float* per_pair,
                         cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (W < 4 || W % 4 != 0) return DIB_BAD_SIZE;
  const long long n = rows * (W / 4);
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  dib_launch(moe_scatter_rows_kernel, dim3(blocks), dim3(256), 0, st, (const float4*)y_sorted, order, rows, W / 4,
             (float4*)per_pair);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_moe_route(const void* logits, int kind, int splits, long long stride, long long row_width,
                  const float* correction, int* ids, float* weights, int T, int E, int top, int groups, int keep,
                  float scale, float eps, int score_kind, int group_top, int normalize, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (E < 1 || E > 1024 || top < 1 || top > 32 || groups < 1 || E % groups || keep < 1 || keep > groups ||
      top > keep * (E / groups) || score_kind < 0 || score_kind > 1 || group_top < 1 || group_top > 2)
    return DIB_BAD_SIZE;
  const size_t smem = sizeof(float) * ROUTE_WARPS * (2 * (size_t)E + groups);
  dib_launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, st,
             make_source(logits, kind, splits, stride), row_width, correction, ids, weights, T, E, top, groups, keep,
             scale, eps, score_kind, group_top, normalize);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// order: int32 [max_tiles * tile + max_tiles + 1]; max_tiles >= pairs / tile + min(E, pairs)
int dib_moe_sort(const int* ids, int pairs, int E, int tile, int max_tiles, int* order, cudaStream_t st) {
  if (pairs == 0) return DIB_OK;
  if (E < 1 || E > SORT_THREADS || tile < 1 || max_tiles < 1) return DIB_BAD_SIZE;
  dib_launch(moe_sort_kernel, dim3(1), dim3(SORT_THREADS), 0, st, ids, pairs, E, tile, max_tiles, order);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_moe_gate_up(const void* x, int dtype, const int* order, int max_tiles, int tile, int top, const void* w_gate_up,
                    void* hidden, int F, int W, cudaStream_t st) {
  return moe_product(x, dtype, order, max_tiles, tile, top, w_gate_up, hidden, W, F, 0, st);
}

int dib_moe_down(const void* hidden, int dtype, const int* order, int max_tiles, int tile, const void* w_down,
                 float* per_pair, int F, int W, cudaStream_t st) {
  return moe_product(hidden, dtype, order, max_tiles, tile, 1, w_down, per_pair, F, W, 1, st);
}

// shared null: no shared expert.
int dib_moe_combine(const float* per_pair, const float* weights, const void* shared, int skind, int ssplits,
                    long long sstride, const void* logits, int lkind, int lsplits, long long lstride,
                    long long logit_row, int gate_col, float* out, int T, int top, int W, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (top < 1 || W < 1) return DIB_BAD_SIZE;
  const long long n = (long long)T * W;
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  dib_launch(moe_combine_kernel, dim3(blocks), dim3(256), 0, st, per_pair, weights,
             make_source(shared, skind, ssplits, sstride), make_source(logits, lkind, lsplits, lstride), logit_row,
             gate_col, out, T, top, W);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // extern "C"
