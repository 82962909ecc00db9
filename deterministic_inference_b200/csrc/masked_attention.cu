// Softmax attention over the paged cache with a mask that is a parameter, keys and values of
// different sizes, an optional sink in the denominator and an optional sigmoid gate on the
// output; and what feeds it: the kernel that norms, rotates and stores a projection's q, k and v
// rows, the one that prepares a latent (low-rank) key/value row, and a product per head.
//
// Masks (mask_kind, mask_size): 0 causal: a query at position p sees keys 0 .. p; 1 window:
// p - size + 1 .. p, and with keep > 0 also the sequence's first keys 0 .. keep - 1 (at their true
// positions); 2 chunk: floor(p / size) * size .. p (chunks counted from position 0).
//
// A page of a cache holds its keys [Hkv, page_size, Dk] and then its values [Hkv, page_size, Dv];
// with Dv_stored == 0 nothing is stored for values and a key's first Dv elements are its value
// (a latent cache: one row per token serves as the key of every head and, in part, as the value).
//
// softcap > 0: a score s (after the scale) becomes softcap * tanh(s / softcap) before the softmax.
//
// Arithmetic: scores, the softmax, norms, angles and sums are float32 (expf, cosf, sinf; no fast
// intrinsics) in the kernels of this file's first half, which take every size; the tensor-core
// forms (masked_attention_mma.cuh) take bfloat16 sizes that are multiples of 16.  Keys are visited
// in tiles anchored at position 0, so the order of a query's sums depends on its position alone.
#include "conv_tail.cuh"
#include "masked_attention_mma.cuh"

namespace {

constexpr int WARPS = 4;
constexpr float NEG_BIG = -1e30f;

__device__ __forceinline__ int first_visible(int pos, int mask_kind, int mask_size) {
  if (mask_kind == 1) return pos - mask_size + 1 > 0 ? pos - mask_size + 1 : 0;
  if (mask_kind == 2) return pos / mask_size * mask_size;
  return 0;
}

// ---- q/k norm, rotation, cache write -------------------------------------------------------
// One warp per (token, slot): slots 0 .. Hq-1 are query heads, then Hkv key heads, then Hkv value
// heads of the projection row [q | k | v | ...] (row_width elements apart).  q and k: RMS norm
// over the head with a weight (when given), then the first `rot` elements rotated by the token's
// position: element i pairs with i + rot/2, angle = position * freq[i], all float32.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_prepare_kernel(Source proj, long long row_width, T* __restrict__ q_out, T* __restrict__ cache,
                    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                    const float* __restrict__ freq, int rot, const int* __restrict__ positions,
                    const int* __restrict__ slot_mapping, int T_tokens, int Hq, int Hkv, int D, int Dv,
                    int page_size, long long num_pages) {
  extern __shared__ float smem[];
  pdl_prologue(proj.p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = Hq + 2 * Hkv;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)T_tokens * slots) return;
  const int t = (int)(item / slots), s = (int)(item % slots);
  const long long row = (long long)t * row_width;
  const long long page_elems = (long long)Hkv * page_size * (D + Dv);
  long long cache_at = -1;
  if (s >= Hq) {
    if (cache == nullptr) return;
    const int slot = slot_mapping[t];
    if (slot < 0 || slot >= num_pages * page_size) return;
    const int page = slot / page_size, off = slot % page_size;
    if (s < Hq + Hkv) cache_at = page * page_elems + ((long long)(s - Hq) * page_size + off) * D;
    else cache_at = page * page_elems + (long long)Hkv * page_size * D + ((long long)(s - Hq - Hkv) * page_size + off) * Dv;
  }
  if (s >= Hq + Hkv) {       // a value head: stored as it is
    const long long src = row + (long long)Hq * D + (long long)Hkv * D + (long long)(s - Hq - Hkv) * Dv;
    for (int d = lane; d < Dv; d += 32) Elem<T>::store(cache + cache_at + d, source_load(proj, src + d));
    return;
  }
  float* x = smem + (size_t)warp * D;
  const long long src = row + (long long)s * D;
  const float* w = s < Hq ? q_w : k_w;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float v = round_to<T>(source_load(proj, src + d));
    x[d] = v;
    ss = __fmaf_rn(v, v, ss);
  }
  if (w != nullptr) {
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
    for (int d = lane; d < D; d += 32) x[d] = x[d] * rstd * w[d];
  }
  __syncwarp();
  T* dst = s < Hq ? q_out + ((long long)t * Hq + s) * D : cache + cache_at;
  const int half = rot / 2;
  const float pos = (float)positions[t];
  for (int d = lane; d < D; d += 32) {
    float v = x[d];
    if (d < rot) {
      const int i = d < half ? d : d - half;
      const float a = __fmul_rn(pos, freq[i]);
      const float c = cosf(a), sn = sinf(a);
      v = d < half ? __fmaf_rn(x[d], c, -__fmul_rn(x[d + half], sn)) : __fmaf_rn(x[d], c, __fmul_rn(x[d - half], sn));
    }
    Elem<T>::store(dst + d, v);
  }
}

// The same for a whole projection row at once: one block per token, which sees every head of q and k.
// A bias (float32 over [q | k | v]) joins the projection before anything else; the RMS norm of q and
// of k runs per head (whole == 0, weights of D elements) or over all heads of the projection at once
// (whole == 1, weights of Hq * D and Hkv * D elements); the rotation pairs element i with i + rot/2
// (pairs == 0) or element 2i with 2i + 1 (pairs == 1), angle = position * freq[i].
// cw given ([nq + nk + nv][taps] float32, the last tap the current token's): every channel of [q | k | v]
// first passes a causal convolution over the sequence's tokens, y_t = sum_j cw[c][j] u_(t - taps + 1 + j),
// with zeros before the sequence's start; the inputs before the step's first token come from the tail
// of the sequence's state slot ([taps - 1][channels] float32, oldest first; slot 0 has none).  The
// convolution's sums stay float32 into the norm.
constexpr int ROW_THREADS = 256;
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
attn_prepare_row_kernel(Source proj, long long row_width, const float* __restrict__ bias, T* __restrict__ q_out,
                        T* __restrict__ cache, const float* __restrict__ q_w, const float* __restrict__ k_w,
                        int whole, float eps, const float* __restrict__ freq, int rot, int pairs,
                        const int* __restrict__ positions, const int* __restrict__ slot_mapping, int Hq, int Hkv,
                        int D, int Dv, int page_size, long long num_pages, const float* __restrict__ cw, int taps,
                        const float* state, long long slot_stride, long long tail_at,
                        const int* __restrict__ token_seq, const int* __restrict__ cu_q_lens,
                        const int* __restrict__ state_slots) {
  extern __shared__ float smem[];      // the row's [q | k | v] (nq + nk + nv floats), then a factor per q and k head
  __shared__ float scratch[32];
  pdl_prologue(proj.p, state);
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = Hq * D, nk = Hkv * D, nv = Hkv * Dv;
  float* x = smem;
  float* factor = smem + nq + nk + nv;
  const long long row = (long long)t * row_width;
  if (cw != nullptr) {
    const int CH = nq + nk + nv;
    const int b = token_seq[t];
    const int local = t - cu_q_lens[b];
    const long long slot = state_slots[b];
    const float* tail = slot != 0 ? state + slot * slot_stride + tail_at : nullptr;
    for (int i = threadIdx.x; i < CH; i += ROW_THREADS) {
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) {          // tap j reads the input taps - 1 - j tokens back
        const int back = taps - 1 - j;
        float u;
        if (back <= local) {
          u = source_load(proj, (long long)(t - back) * row_width + i);
          if (bias != nullptr) u = __fadd_rn(u, bias[i]);
        } else {
          u = tail != nullptr ? tail[(long long)(taps - 1 - (back - local)) * CH + i] : 0.f;
        }
        acc = __fmaf_rn(cw[(long long)i * taps + j], u, acc);
      }
      x[i] = acc;
    }
  } else {
    for (int i = threadIdx.x; i < nq + nk + nv; i += ROW_THREADS) {
      float v = source_load(proj, row + i);
      if (bias != nullptr) v = __fadd_rn(v, bias[i]);
      x[i] = round_to<T>(v);
    }
  }
  __syncthreads();
  if (q_w != nullptr) {
    if (whole) {
      float sq = 0.f, sk = 0.f;
      for (int i = threadIdx.x; i < nq; i += ROW_THREADS) sq = __fmaf_rn(x[i], x[i], sq);
      for (int i = threadIdx.x; i < nk; i += ROW_THREADS) sk = __fmaf_rn(x[nq + i], x[nq + i], sk);
      const float rq = 1.0f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
      const float rk = 1.0f / sqrtf(block_sum(sk, scratch) / (float)nk + eps);
      for (int i = threadIdx.x; i < nq; i += ROW_THREADS) x[i] = x[i] * rq * q_w[i];
      for (int i = threadIdx.x; i < nk; i += ROW_THREADS) x[nq + i] = x[nq + i] * rk * k_w[i];
    } else {
      for (int s = warp; s < Hq + Hkv; s += ROW_THREADS / 32) {
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = __fmaf_rn(x[s * D + d], x[s * D + d], ss);
        ss = warp_sum(ss);
        if (lane == 0) factor[s] = 1.0f / sqrtf(ss / (float)D + eps);
      }
      __syncthreads();
      for (int i = threadIdx.x; i < nq + nk; i += ROW_THREADS) {
        const int s = i / D, d = i - s * D;
        x[i] = x[i] * factor[s] * (s < Hq ? q_w[d] : k_w[d]);
      }
    }
    __syncthreads();
  }
  long long page_at = -1;
  int off = 0;
  if (cache != nullptr) {
    const int slot = slot_mapping[t];
    if (slot >= 0 && slot < num_pages * page_size) {
      page_at = (long long)(slot / page_size) * Hkv * page_size * (D + Dv);
      off = slot % page_size;
    }
  }
  const float pos = (float)positions[t];
  const int half = rot / 2;
  for (int i = threadIdx.x; i < nq + nk; i += ROW_THREADS) {
    const int s = i / D, d = i - s * D;
    float v = x[i];
    if (d < rot) {
      // the element's partner, its frequency, and whether it is the pair's first element
      const bool first = pairs ? (d & 1) == 0 : d < half;
      const int other = pairs ? (d ^ 1) : (first ? d + half : d - half);
      const float a = __fmul_rn(pos, freq[pairs ? d >> 1 : (first ? d : d - half)]);
      const float c = cosf(a), sn = sinf(a), o = x[s * D + other];
      v = first ? __fmaf_rn(v, c, -__fmul_rn(o, sn)) : __fmaf_rn(v, c, __fmul_rn(o, sn));
    }
    if (s < Hq) Elem<T>::store(q_out + (long long)t * nq + i, v);
    else if (page_at >= 0) Elem<T>::store(cache + page_at + ((long long)(s - Hq) * page_size + off) * D + d, v);
  }
  if (page_at >= 0)
    for (int i = threadIdx.x; i < nv; i += ROW_THREADS) {
      const int s = i / Dv, d = i - s * Dv;
      Elem<T>::store(cache + page_at + (long long)Hkv * page_size * D + ((long long)s * page_size + off) * Dv + d,
                     x[nq + nk + i]);
    }
}

// ---- a latent key/value row ------------------------------------------------------------------
// The projection row is [q: H heads of (Dn + R) | latent: C | shared rotated key part: R].  One warp
// per (token, slot): slot 0 norms the latent (RMS, weight) into the cache row's first C elements and
// rotates the key part into its last R; slot 1 + h rotates the last R elements of query head h into
// q_out[t, h, C .. C + R) (the first C are the product of the head's other Dn elements with its
// key map, written by the per-head product).  The cache row of a token is [C + R], one key head.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
latent_prepare_kernel(Source proj, long long row_width, T* __restrict__ q_out, T* __restrict__ cache,
                      const float* __restrict__ c_w, float eps, const float* __restrict__ freq,
                      const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                      int T_tokens, int H, int Dn, int R, int C, int page_size, long long num_pages) {
  pdl_prologue(proj.p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = H + 1;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)T_tokens * slots) return;
  const int t = (int)(item / slots), s = (int)(item % slots);
  const long long row = (long long)t * row_width;
  const float pos = (float)positions[t];
  const int half = R / 2;
  long long src;       // the R elements to rotate
  T* dst;
  if (s == 0) {
    if (cache == nullptr) return;
    const int slot = slot_mapping[t];
    if (slot < 0 || slot >= num_pages * page_size) return;
    T* crow = cache + (long long)slot * (C + R);
    const long long lat = row + (long long)H * (Dn + R);
    float ss = 0.f;
    for (int d = lane; d < C; d += 32) {
      const float v = round_to<T>(source_load(proj, lat + d));
      ss = __fmaf_rn(v, v, ss);
    }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)C + eps);
    for (int d = lane; d < C; d += 32)
      Elem<T>::store(crow + d, round_to<T>(source_load(proj, lat + d)) * rstd * c_w[d]);
    src = lat + C;
    dst = crow + C;
  } else {
    src = row + (long long)(s - 1) * (Dn + R) + Dn;
    dst = q_out + ((long long)t * H + (s - 1)) * (C + R) + C;
  }
  for (int d = lane; d < R; d += 32) {
    const int i = d < half ? d : d - half;
    const float a = __fmul_rn(pos, freq[i]);
    const float c = cosf(a), sn = sinf(a);
    const float u = round_to<T>(source_load(proj, src + d));
    const float o = round_to<T>(source_load(proj, src + (d < half ? d + half : d - half)));
    Elem<T>::store(dst + d, d < half ? __fmaf_rn(u, c, -__fmul_rn(o, sn)) : __fmaf_rn(u, c, __fmul_rn(o, sn)));
  }
}

// ---- a product per head --------------------------------------------------------------------------
// out[m, h, n] = sum_k x[m, h, k] * w[h, k, n]; x and out with free row and head strides (elements),
// w contiguous [H, K, N].  float32 accumulation.  A block takes HL_ROWS rows and HL_COLS columns of one
// head; k is cut into HL_SLICES equal runs, a group of threads each (so that few rows still keep many
// loads of the weights in flight), every run added up in ascending k and the runs' sums in run order:
// a row's bits depend on K alone.
constexpr int HL_ROWS = 8, HL_COLS = 64, HL_SLICES = 4;
template <typename T>
__global__ void __launch_bounds__(HL_COLS * HL_SLICES)
heads_linear_kernel(const T* __restrict__ x, long long xs_m, long long xs_h, const T* __restrict__ w,
                    T* __restrict__ out, long long os_m, long long os_h, int M, int K, int N) {
  extern __shared__ float xs[];      // [HL_ROWS][K], then the runs' sums [HL_SLICES][HL_ROWS][HL_COLS]
  float* part = xs + (size_t)HL_ROWS * K;
  pdl_prologue(x);
  const int h = blockIdx.y, m0 = blockIdx.z * HL_ROWS;
  const int col = threadIdx.x % HL_COLS, run = threadIdx.x / HL_COLS;
  const int n = blockIdx.x * HL_COLS + col;
  const int rows = M - m0 < HL_ROWS ? M - m0 : HL_ROWS;
  for (int i = threadIdx.x; i < HL_ROWS * K; i += HL_COLS * HL_SLICES) {
    const int r = i / K, k = i % K;
    xs[i] = r < rows ? Elem<T>::load(x + (long long)(m0 + r) * xs_m + (long long)h * xs_h + k) : 0.f;
  }
  __syncthreads();
  float acc[HL_ROWS];
#pragma unroll
  for (int r = 0; r < HL_ROWS; ++r) acc[r] = 0.f;
  const int per = (K + HL_SLICES - 1) / HL_SLICES;
  const int k_begin = run * per, k_end = k_begin + per < K ? k_begin + per : K;
  if (n < N) {
    const T* wp = w + (long long)h * K * N + n;
#pragma unroll 8
    for (int k = k_begin; k < k_end; ++k) {
      const float wv = Elem<T>::load(wp + (long long)k * N);
#pragma unroll
      for (int r = 0; r < HL_ROWS; ++r) acc[r] = __fmaf_rn(xs[r * K + k], wv, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < HL_ROWS; ++r) part[(run * HL_ROWS + r) * HL_COLS + col] = acc[r];
  __syncthreads();
  if (run == 0 && n < N) {
    for (int r = 0; r < rows; ++r) {
      float v = part[r * HL_COLS + col];
#pragma unroll
      for (int s = 1; s < HL_SLICES; ++s) v = __fadd_rn(v, part[(s * HL_ROWS + r) * HL_COLS + col]);
      Elem<T>::store(out + (long long)(m0 + r) * os_m + (long long)h * os_h + n, v);
    }
  }
}

// ---- attention, float32 arithmetic ----------------------------------------------------------------
// One warp per (token, query head); key tiles of 32 anchored at position 0, a lane a key.
template <typename T, int NV>
__global__ void __launch_bounds__(WARPS * 32)
masked_attention_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ cache,
                        const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ token_seq, const int* __restrict__ positions,
                        int T_tokens, int Hq, int Hkv, int Dk, int Dv, int Dv_stored, int page_size,
                        float scale, int mask_kind, int mask_size, int keep, const float* __restrict__ sink,
                        Source gate, long long gate_row, long long gate_col, float softcap) {
  extern __shared__ float smem[];
  pdl_prologue(q, cache, block_table, token_seq, positions, gate.p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)T_tokens * Hq) return;
  const int t = (int)(item / Hq), h = (int)(item % Hq);
  const int kvh = h / (Hq / Hkv);
  const int pos = positions[t];
  const int* bt = block_table + (size_t)token_seq[t] * max_blocks;
  float* sq = smem + (size_t)warp * Dk;
  const T* qrow = q + ((size_t)t * Hq + h) * Dk;
  for (int d = lane; d < Dk; d += 32) sq[d] = Elem<T>::load(qrow + d);
  __syncwarp();

  const int first = first_visible(pos, mask_kind, mask_size);
  // the sink is a key without a value whose score is sink[h], unscaled
  float m = sink != nullptr ? sink[h] : NEG_BIG, l = sink != nullptr ? 1.f : 0.f;
  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
  const size_t page_elems = (size_t)Hkv * page_size * (Dk + Dv_stored);
  const size_t values_at = (size_t)Hkv * page_size * Dk;

  // kept first keys that the window has passed: their tiles come first, then the window's
  const int kept_end = keep < first ? keep : first;
  const int window_from = (first / 32) * 32 > (kept_end + 31) / 32 * 32 ? (first / 32) * 32 : (kept_end + 31) / 32 * 32;
  for (int k0 = kept_end > 0 ? 0 : window_from; k0 <= pos; k0 = (k0 + 32 >= kept_end && k0 + 32 < window_from) ? window_from : k0 + 32) {
    const int key = k0 + lane;
    const bool visible = (key >= first || key < kept_end) && key <= pos;
    float s = NEG_BIG;
    const T* vrow = nullptr;
    if (visible) {
      // (a key beyond the table's width, a padding sequence's, reads page 0)
      const T* page = cache + (size_t)(key / page_size < max_blocks ? bt[key / page_size] : 0) * page_elems;
      const size_t in_page = (size_t)kvh * page_size + key % page_size;
      const T* krow = page + in_page * Dk;
      vrow = Dv_stored > 0 ? page + values_at + in_page * Dv : krow;
      float dot = 0.f;
      for (int d = 0; d < Dk; ++d) dot = __fmaf_rn(sq[d], Elem<T>::load(krow + d), dot);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = visible ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] *= alpha;
    const unsigned long long vaddr = (unsigned long long)vrow;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const unsigned long long va = __shfl_sync(0xffffffffu, vaddr, j);
      if (va == 0ull) continue;   // warp-uniform
      const T* vr = (const T*)va;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) acc[i] = __fmaf_rn(pj, Elem<T>::load(vr + d), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* orow = out + ((size_t)t * Hq + h) * Dv;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = lane + 32 * i;
    if (d < Dv) {
      float o = acc[i] * inv;
      if (gate.p != nullptr)
        o = round_to<T>(o) * sigmoid_f32(round_to<T>(source_load(gate, (long long)t * gate_row + gate_col + (long long)h * Dv + d)));
      Elem<T>::store(orow + d, o);
    }
  }
}

// x[t, c] *= sigmoid(gate[t, gate_col + c]), in place; float32 arithmetic, one rounding
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, Source gate, long long gate_row, long long gate_col,
                                    int rows, int width) {
  pdl_prologue(x, gate.p);
  const long long n = (long long)rows * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / width, c = i % width;
    const float g = round_to<T>(source_load(gate, r * gate_row + gate_col + c));
    Elem<T>::store(x + i, Elem<T>::load(x + i) * sigmoid_f32(g));
  }
}

template <typename T>
int launch_masked_attention(const void* q, void* out, const void* cache, const int* block_table,
                            int max_blocks, const int* token_seq, const int* positions, int T_tokens, int Hq,
                            int Hkv, int Dk, int Dv, int Dv_stored, int page_size, float scale, int mask_kind,
                            int mask_size, int keep, const float* sink, Source gate, long long gate_row,
                            long long gate_col, float softcap, cudaStream_t st) {
  const int blocks = ceil_div_host((long long)T_tokens * Hq, WARPS);
  const size_t smem = (size_t)WARPS * Dk * sizeof(float);
#define DIB_MA(NV)                                                                                       \
  dib_launch(masked_attention_kernel<T, NV>, dim3(blocks), dim3(WARPS * 32), smem, st, (const T*)q, (T*)out, \
             (const T*)cache, block_table, max_blocks, token_seq, positions, T_tokens, Hq, Hkv, Dk, Dv,   \
             Dv_stored, page_size, scale, mask_kind, mask_size, keep, sink, gate, gate_row, gate_col, softcap)
  if (Dv <= 64) DIB_MA(2);
  else if (Dv <= 128) DIB_MA(4);
  else if (Dv <= 256) DIB_MA(8);
  else if (Dv <= 512) DIB_MA(16);
  else DIB_MA(32);
#undef DIB_MA
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // namespace

extern "C" {

// q_w / k_w null: no norm.  freq null or rot 0: no rotation.  cache null: keys and values are not stored.
int dib_attn_prepare(const void* proj, int kind, int splits, long long stride, long long row_width, void* q_out,
                     void* cache, const float* q_w, const float* k_w, float eps, const float* freq, int rot,
                     const int* positions, const int* slot_mapping, int T, int Hq, int Hkv, int D, int Dv,
                     int page_size, long long num_pages, int dtype, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (D < 1 || D > 2048 || Dv < 1 || Hq < 1 || Hkv < 1 || rot < 0 || rot > D || rot % 2 || page_size < 1)
    return DIB_BAD_SIZE;
  if (freq == nullptr) rot = 0;
  const Source src = make_source(proj, kind, splits, stride);
  const int blocks = ceil_div_host((long long)T * (Hq + 2 * Hkv), WARPS);
  const size_t smem = (size_t)WARPS * D * sizeof(float);
  if (dtype == 0)
    dib_launch(attn_prepare_kernel<float>, dim3(blocks), dim3(WARPS * 32), smem, st, src, row_width, (float*)q_out,
               (float*)cache, q_w, k_w, eps, freq, rot, positions, slot_mapping, T, Hq, Hkv, D, Dv, page_size, num_pages);
  else if (dtype == 1)
    dib_launch(attn_prepare_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), smem, st, src, row_width,
               (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, q_w, k_w, eps, freq, rot, positions, slot_mapping, T,
               Hq, Hkv, D, Dv, page_size, num_pages);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The form that takes a row at once (attn_prepare_row_kernel): a bias, a norm over the whole projection,
// interleaved rotation pairs.  bias null: none.
int dib_attn_prepare_row(const void* proj, int kind, int splits, long long stride, long long row_width,
                         const float* bias, void* q_out, void* cache, const float* q_w, const float* k_w, int whole,
                         float eps, const float* freq, int rot, int pairs, const int* positions,
                         const int* slot_mapping, int T, int Hq, int Hkv, int D, int Dv, int page_size,
                         long long num_pages, int dtype, const float* cw, int taps, float* state,
                         long long slot_stride, long long tail_at, const int* token_seq, const int* cu_q_lens,
                         const int* state_slots, int B, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (D < 1 || Dv < 1 || Hq < 1 || Hkv < 1 || rot < 0 || rot > D || rot % 2 || page_size < 1) return DIB_BAD_SIZE;
  if (cw != nullptr && (taps < 1 || taps > 64 || token_seq == nullptr || cu_q_lens == nullptr ||
                        state_slots == nullptr || (taps > 1 && state == nullptr)))
    return DIB_BAD_SIZE;
  if (freq == nullptr) rot = 0;
  const size_t smem = sizeof(float) * ((size_t)Hq * D + (size_t)Hkv * (D + Dv) + Hq + Hkv);
  if (smem > 200 * 1024) return DIB_BAD_SIZE;
  const Source src = make_source(proj, kind, splits, stride);
  static DeviceOnce once32, once16;
  if (dtype == 0) {
    if (smem > 48 * 1024 && !once32.done()) {
      if (cudaFuncSetAttribute(attn_prepare_row_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               200 * 1024) != cudaSuccess) return DIB_LAUNCH_FAILED;
      once32.mark();
    }
    dib_launch(attn_prepare_row_kernel<float>, dim3(T), dim3(ROW_THREADS), smem, st, src, row_width, bias,
               (float*)q_out, (float*)cache, q_w, k_w, whole, eps, freq, rot, pairs, positions, slot_mapping, Hq, Hkv,
               D, Dv, page_size, num_pages, cw, taps, (const float*)state, slot_stride, tail_at, token_seq, cu_q_lens,
               state_slots);
  } else if (dtype == 1) {
    if (smem > 48 * 1024 && !once16.done()) {
      if (cudaFuncSetAttribute(attn_prepare_row_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               200 * 1024) != cudaSuccess) return DIB_LAUNCH_FAILED;
      once16.mark();
    }
    dib_launch(attn_prepare_row_kernel<__nv_bfloat16>, dim3(T), dim3(ROW_THREADS), smem, st, src, row_width, bias,
               (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, q_w, k_w, whole, eps, freq, rot, pairs, positions,
               slot_mapping, Hq, Hkv, D, Dv, page_size, num_pages, cw, taps, (const float*)state, slot_stride, tail_at,
               token_seq, cu_q_lens, state_slots);
  } else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  if (cw != nullptr && taps > 1 && B > 0) {
    // the convolutions' tails move on by the step's tokens, once every row has read them
    dib_launch(conv_tail_update_kernel, dim3(B), dim3(256), 0, st, src, row_width, 0ll, bias, state, slot_stride,
               tail_at, cu_q_lens, state_slots, Hq * D + Hkv * (D + Dv), taps);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

int dib_latent_prepare(const void* proj, int kind, int splits, long long stride, long long row_width, void* q_out,
                       void* cache, const float* c_w, float eps, const float* freq, const int* positions,
                       const int* slot_mapping, int T, int H, int Dn, int R, int C, int page_size,
                       long long num_pages, int dtype, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (H < 1 || Dn < 1 || R < 2 || R % 2 || C < 1 || page_size < 1 || freq == nullptr || c_w == nullptr)
    return DIB_BAD_SIZE;
  const Source src = make_source(proj, kind, splits, stride);
  const int blocks = ceil_div_host((long long)T * (H + 1), WARPS);
  if (dtype == 0)
    dib_launch(latent_prepare_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, st, src, row_width, (float*)q_out,
               (float*)cache, c_w, eps, freq, positions, slot_mapping, T, H, Dn, R, C, page_size, num_pages);
  else if (dtype == 1)
    dib_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, st, src, row_width,
               (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, c_w, eps, freq, positions, slot_mapping, T, H, Dn, R,
               C, page_size, num_pages);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_heads_linear(const void* x, long long xs_m, long long xs_h, const void* w, void* out, long long os_m,
                     long long os_h, int M, int H, int K, int N, int dtype, cudaStream_t st) {
  if (M == 0) return DIB_OK;
  if (H < 1 || H > 65535 || K < 1 || K > 4096 || N < 1) return DIB_BAD_SIZE;
  const dim3 grid(ceil_div_host(N, HL_COLS), H, ceil_div_host(M, HL_ROWS));
  if (grid.z > 65535) return DIB_BAD_SIZE;
  const size_t smem = ((size_t)HL_ROWS * K + (size_t)HL_SLICES * HL_ROWS * HL_COLS) * sizeof(float);
  if (dtype == 0) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(heads_linear_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dib_launch(heads_linear_kernel<float>, grid, dim3(HL_COLS * HL_SLICES), smem, st, (const float*)x, xs_m, xs_h,
               (const float*)w, (float*)out, os_m, os_h, M, K, N);
  } else if (dtype == 1) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(heads_linear_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dib_launch(heads_linear_kernel<__nv_bfloat16>, grid, dim3(HL_COLS * HL_SLICES), smem, st, (const __nv_bfloat16*)x, xs_m,
               xs_h, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, os_m, os_h, M, K, N);
  } else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_sigmoid_gate_(void* x, const void* gate, int kind, int splits, long long stride, long long gate_row,
                      long long gate_col, int rows, int width, int dtype, cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (width < 1) return DIB_BAD_SIZE;
  const Source g = make_source(gate, kind, splits, stride);
  const long long n = (long long)rows * width;
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  if (dtype == 0)
    dib_launch(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, st, (float*)x, g, gate_row, gate_col, rows, width);
  else if (dtype == 1)
    dib_launch(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, (__nv_bfloat16*)x, g, gate_row,
               gate_col, rows, width);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The tensor-core form (bfloat16; Dk and Dv multiples of 16, Dv at most 256): tiles [num_tiles][3] =
// (sequence, first token among the sequence's new tokens, tokens) of at most rows / (Hq / Hkv) tokens
// each; rows 64 or 128.
// partial_o / partial_ml given (tiles of ONE token only): a token's key tiles are cut into chunks of
// chunk_tiles, a CTA each, merged by a second kernel over the step's first num_tokens tokens.
int dib_masked_attention_mma(const void* q, void* out, const void* cache, const int* block_table, int max_blocks,
                             const int* positions, const int* seq_lens, const int* cu_q_lens, const int* tiles,
                             int num_tiles, const float* sink, int Hq, int Hkv, int Dk, int Dv, int Dv_stored, int page_size,
                             float scale, int mask_kind, int mask_size, int keep, const void* gate, int gate_kind,
                             int gate_splits, long long gate_stride, long long gate_row, long long gate_col,
                             int rows, float* partial_o, float* partial_ml, int chunk_tiles, int max_chunks,
                             int num_tokens, float softcap, cudaStream_t st) {
  if (num_tiles == 0) return DIB_OK;
  if (Dk < 16 || Dk % 16 || Dv < 16 || Dv % 16 || Dv > 256 || Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > rows ||
      (rows != 64 && rows != 128) || page_size < 1 || mask_kind < 0 || mask_kind > 2 ||
      (mask_kind > 0 && mask_size < 1) || keep < 0 || (keep > 0 && mask_kind != 1) ||
      (Dv_stored != 0 && Dv_stored != Dv) || (Dv_stored == 0 && Dv > Dk) ||
      num_tiles > 1 << 30 || Hkv > 65535 || max_chunks > 65535 || (partial_o != nullptr && chunk_tiles < 1))
    return DIB_BAD_SIZE;
  const Source g = make_source(gate, gate_kind, gate_splits, gate_stride);
#define DIB_MAM(NV, ROWS)                                                                                    \
  return ma_mma::launch<NV, ROWS>(q, out, cache, block_table, max_blocks, positions, seq_lens, cu_q_lens, tiles, num_tiles, \
                                  sink, Hq, Hkv, Dk, Dv, Dv_stored, page_size, scale, mask_kind, mask_size, keep, g, \
                                  gate_row, gate_col, partial_o, partial_ml, chunk_tiles, max_chunks, num_tokens, softcap, st)
  const int nv = (Dv + 63) / 64;
  if (rows == 64) {
    if (nv == 1) DIB_MAM(4, 64);
    if (nv == 2) DIB_MAM(8, 64);
    if (nv == 3) DIB_MAM(12, 64);
    DIB_MAM(16, 64);
  }
  if (nv == 1) DIB_MAM(4, 128);
  if (nv == 2) DIB_MAM(8, 128);
  if (nv == 3) DIB_MAM(12, 128);
  DIB_MAM(16, 128);
#undef DIB_MAM
}

// sink null: a plain softmax.  gate null: no output gate; else out *= sigmoid(gate[t, gate_col + h * Dv + d])
// with rows gate_row elements apart.  Dv_stored 0: a key's first Dv elements are its value.
int dib_masked_attention(const void* q, void* out, const void* cache, const int* block_table, int max_blocks,
                         const int* token_seq, const int* positions, int T, int Hq, int Hkv, int Dk, int Dv,
                         int Dv_stored, int page_size, float scale, int mask_kind, int mask_size, int keep,
                         const float* sink, const void* gate, int gate_kind, int gate_splits,
                         long long gate_stride, long long gate_row, long long gate_col, int dtype, float softcap,
                         cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (Dk < 1 || Dk > 2048 || Dv < 1 || Dv > 1024 || Hkv < 1 || Hq % Hkv != 0 || page_size < 1 ||
      mask_kind < 0 || mask_kind > 2 || (mask_kind > 0 && mask_size < 1) || keep < 0 || (keep > 0 && mask_kind != 1) ||
      (Dv_stored != 0 && Dv_stored != Dv) || (Dv_stored == 0 && Dv > Dk))
    return DIB_BAD_SIZE;
  const Source g = make_source(gate, gate_kind, gate_splits, gate_stride);
  if (dtype == 0)
    return launch_masked_attention<float>(q, out, cache, block_table, max_blocks, token_seq, positions, T, Hq,
                                          Hkv, Dk, Dv, Dv_stored, page_size, scale, mask_kind, mask_size, keep, sink, g,
                                          gate_row, gate_col, softcap, st);
  if (dtype == 1)
    return launch_masked_attention<__nv_bfloat16>(q, out, cache, block_table, max_blocks, token_seq, positions, T,
                                                  Hq, Hkv, Dk, Dv, Dv_stored, page_size, scale, mask_kind,
                                                  mask_size, keep, sink, g, gate_row, gate_col, softcap, st);
  return DIB_BAD_DTYPE;
}

}  // extern "C"
