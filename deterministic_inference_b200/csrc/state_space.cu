// A state-space recurrence with one scalar decay per head (the recurrent form of state-space
// duality): what goes in front of the recurrence, the recurrence, and what comes behind it.
//
// proj row (row_width elements): [z: H P | x: H P | B: G N | C: G N | dt: H | ...].  The channels
// x, B and C (CH = H P + 2 G N of them, from column H P on) pass a causal convolution over time
// (cw [CH][taps], the last tap the current token's, zeros before the sequence's start), a bias and
// silu.  dt = softplus(dt + dt_bias), no clamp.  Per head h (its B and C are those of group
// h / (H / G)), with a state S [N][P] from zero:
//     S <- exp(-exp(A_log[h]) dt) S + dt B x^T;     y = S^T C + D[h] x.
// y (heads side by side) times silu(z), then RMS-normed in `parts` equal parts, each by its own
// root mean square, times a weight.
//
// A request's state slot holds the heads' states [H][N][P] and then the convolution's last
// taps - 1 inputs [taps - 1][CH] (oldest first); slot 0 is no request's: a sequence on it starts
// from zeros and stores nothing.  Everything is float32.
#include "conv_tail.cuh"

#include <cuda_pipeline.h>

namespace {

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// grid (T, ceil(CH / 256)): xbc[t][c] = silu(conv(c) + cb[c]); the blocks of the first column of
// the grid also leave dtv[t][h] = (dt, exp(-exp(A_log[h]) dt)).
__global__ void __launch_bounds__(256)
ssm_prepare_kernel(Source proj, long long row_width, const float* __restrict__ cw, const float* __restrict__ cb,
                   const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* state,
                   long long slot_stride, long long tail_at, const int* __restrict__ token_seq,
                   const int* __restrict__ cu_q_lens, const int* __restrict__ state_slots, float* __restrict__ xbc,
                   float2* __restrict__ dtv, int H, int inner, int CH, int taps) {
  pdl_prologue(proj.p, state);
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int local = t - cu_q_lens[b];
  const long long slot = state_slots[b];
  const float* tail = slot != 0 ? state + slot * slot_stride + tail_at : nullptr;
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c < CH) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {          // tap j reads the input taps - 1 - j tokens back
      const int back = taps - 1 - j;
      float u;
      if (back <= local) u = source_load(proj, (long long)(t - back) * row_width + inner + c);
      else u = tail != nullptr ? tail[(long long)(taps - 1 - (back - local)) * CH + c] : 0.f;
      acc = __fmaf_rn(cw[(long long)c * taps + j], u, acc);
    }
    if (cb != nullptr) acc = __fadd_rn(acc, cb[c]);
    xbc[(long long)t * CH + c] = acc * sigmoid_f32(acc);
  }
  if (blockIdx.y == 0)
    for (int h = threadIdx.x; h < H; h += 256) {
      const float z = __fadd_rn(source_load(proj, (long long)t * row_width + inner + CH + h), dt_bias[h]);
      const float dt = softplus_f32(z);
      dtv[(long long)t * H + h] = make_float2(dt, expf(-expf(a_log[h]) * dt));
    }
}

// grid (B, H, ceil(P / COLS)), COLS * LANES threads: COLS columns of the head's state, a column's N rows
// over LANES lanes (16 or 32; row n on lane n % LANES, so MAXR = ceil(N / LANES) rows a lane, kept in
// registers).  The
// sequence's tokens are walked in chunks of CHUNK tokens whose vectors (B and C of the head's group,
// the x of the block's columns, dt and the decay) are staged in shared memory by cp.async (16 bytes
// at a time where the sizes allow), one chunk ahead of the arithmetic.  A lane adds its rows'
// share of a column's read-out in ascending order and leaves it in shared memory; once the chunk
// is through, a thread per (token, column) adds the lanes' shares in lane order: the order
// depends on N alone (which decides LANES), not on COLS, the chunk or the step.
template <int MAXR, int CHUNK, int COLS, int LANES>
__global__ void __launch_bounds__(COLS * LANES)
ssm_recurrence_kernel(const float* __restrict__ xbc, const float2* __restrict__ dtv, const float* __restrict__ d_skip,
                      float* state, long long slot_stride, float* __restrict__ y, const int* __restrict__ cu_q_lens,
                      const int* __restrict__ state_slots, int H, int G, int N, int P, int CH, int vec) {
  extern __shared__ __align__(16) float stage[];   // [2][CHUNK][per], then part [CHUNK * COLS][LANES + 1], skip [CHUNK * COLS]
  pdl_prologue(xbc, dtv, state);
  constexpr int THREADS = COLS * LANES;
  const int b = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * COLS;
  const int g = h / (H / G);
  const int t0 = cu_q_lens[b], n_tok = cu_q_lens[b + 1] - t0;
  if (n_tok <= 0) return;
  const long long slot = state_slots[b];
  const int col = threadIdx.x / LANES, lane = threadIdx.x % LANES;
  const int p = p0 + col;
  const bool has_col = p < P;
  const int inner = H * P;
  const int per = (2 * N + COLS + 2 + 3) / 4 * 4;       // B [N], C [N], x [COLS], dt, decay; rows 16 bytes apart
  float* part = stage + (size_t)2 * CHUNK * per;
  float* skip = part + CHUNK * COLS * (LANES + 1);
  float* srow = state + slot * slot_stride + (long long)h * N * P;
  const bool full_cols = p0 + COLS <= P;

  float S[MAXR];
#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int n = lane + LANES * r;
    S[r] = (slot != 0 && has_col && n < N) ? srow[(long long)n * P + p] : 0.f;
  }

  auto load_chunk = [&](int first, int buf) {
    const int count = n_tok - first < CHUNK ? n_tok - first : CHUNK;
    float* base = stage + (size_t)buf * CHUNK * per;
    if (vec) {
      // 16-byte pieces: N / 4 of B, N / 4 of C, COLS / 4 of x (whole columns only), then dt and the decay (8 bytes)
      const int nb = N / 4, nx = full_cols ? COLS / 4 : 0, pieces = 2 * nb + nx + 1;
      for (int i = threadIdx.x; i < count * pieces; i += THREADS) {
        const int k = i / pieces, e = i - k * pieces;
        const long long t = t0 + first + k;
        float* dst = base + k * per;
        if (e < nb) __pipeline_memcpy_async(dst + 4 * e, xbc + t * CH + inner + (long long)g * N + 4 * e, 16);
        else if (e < 2 * nb)
          __pipeline_memcpy_async(dst + N + 4 * (e - nb), xbc + t * CH + inner + (long long)(G + g) * N + 4 * (e - nb), 16);
        else if (e < 2 * nb + nx)
          __pipeline_memcpy_async(dst + 2 * N + 4 * (e - 2 * nb), xbc + t * CH + (long long)h * P + p0 + 4 * (e - 2 * nb), 16);
        else __pipeline_memcpy_async(dst + 2 * N + COLS, dtv + t * H + h, 8);
      }
      if (!full_cols)
        for (int i = threadIdx.x; i < count * COLS; i += THREADS) {
          const int k = i / COLS, c = i - k * COLS;
          __pipeline_memcpy_async(base + k * per + 2 * N + c,
                                  xbc + (long long)(t0 + first + k) * CH + (long long)h * P + (p0 + c < P ? p0 + c : P - 1), 4);
        }
    } else {
      const int items = 2 * N + COLS + 2;
      for (int i = threadIdx.x; i < count * items; i += THREADS) {
        const int k = i / items, e = i - k * items;
        const long long t = t0 + first + k;
        const float* src;
        if (e < N) src = xbc + t * CH + inner + (long long)g * N + e;
        else if (e < 2 * N) src = xbc + t * CH + inner + (long long)(G + g) * N + (e - N);
        else if (e < 2 * N + COLS) src = xbc + t * CH + (long long)h * P + (p0 + e - 2 * N < P ? p0 + e - 2 * N : P - 1);
        else src = reinterpret_cast<const float*>(dtv + t * H + h) + (e - 2 * N - COLS);
        __pipeline_memcpy_async(base + k * per + e, src, 4);
      }
    }
    __pipeline_commit();
  };

  const float dh = d_skip[h];
  load_chunk(0, 0);
  int buf = 0;
  for (int first = 0; first < n_tok; first += CHUNK, buf ^= 1) {
    if (first + CHUNK < n_tok) {
      load_chunk(first + CHUNK, buf ^ 1);
      __pipeline_wait_prior(1);
    } else {
      __pipeline_wait_prior(0);
    }
    __syncthreads();
    const int count = n_tok - first < CHUNK ? n_tok - first : CHUNK;
    const float* base = stage + (size_t)buf * CHUNK * per;
    // one token: the state's rows move on, and the lane's share of the column's read-out
    auto token = [&](const float* v) {
      const float x = v[2 * N + col], dt = v[2 * N + COLS], decay = v[2 * N + COLS + 1];
      const float dtx = __fmul_rn(dt, x);
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        const int n = lane + LANES * r;
        if (n < N) {
          S[r] = __fmaf_rn(v[n], dtx, __fmul_rn(decay, S[r]));
          acc = __fmaf_rn(S[r], v[N + n], acc);
        }
      }
      return acc;
    };
    if (count == CHUNK) {
      // a whole chunk: the shares stay in registers until the chunk is through, so that no store to
      // shared memory stands between one token's loads and the next one's
      float accs[CHUNK];
#pragma unroll
      for (int k = 0; k < CHUNK; ++k) accs[k] = token(base + k * per);
#pragma unroll
      for (int k = 0; k < CHUNK; ++k) {
        part[(k * COLS + col) * (LANES + 1) + lane] = accs[k];
        if (lane == 0) skip[k * COLS + col] = __fmul_rn(dh, base[k * per + 2 * N + col]);
      }
    } else {
      for (int k = 0; k < count; ++k) {
        const float acc = token(base + k * per);
        part[(k * COLS + col) * (LANES + 1) + lane] = acc;
        if (lane == 0) skip[k * COLS + col] = __fmul_rn(dh, base[k * per + 2 * N + col]);
      }
    }
    __syncthreads();       // the shares are complete; the buffer may be written again a chunk on
    for (int i = threadIdx.x; i < count * COLS; i += THREADS) {
      const int k = i / COLS, c = i - k * COLS;
      const float* ps = part + i * (LANES + 1);
      float acc = ps[0];
#pragma unroll
      for (int l = 1; l < LANES; ++l) acc = __fadd_rn(acc, ps[l]);
      if (p0 + c < P) y[(long long)(t0 + first + k) * inner + (long long)h * P + p0 + c] = __fadd_rn(acc, skip[i]);
    }
  }
  if (slot != 0 && has_col) {
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
      const int n = lane + LANES * r;
      if (n < N) srow[(long long)n * P + p] = S[r];
    }
  }
}

// grid (T, parts): out[t, part] = u / sqrt(mean(u^2) + eps) * norm_w, u = y * silu(z) over the part's
// inner / parts channels.
__global__ void __launch_bounds__(256)
ssm_output_kernel(const float* __restrict__ y, Source proj, long long row_width, const float* __restrict__ norm_w,
                  void* out, int out_dtype, int inner, int parts, float eps) {
  __shared__ float scratch[32];
  pdl_prologue(y, proj.p);
  const int t = blockIdx.x, part = blockIdx.y;
  const int width = inner / parts, c0 = part * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += 256) {
    const float z = source_load(proj, (long long)t * row_width + c0 + c);
    const float u = y[(long long)t * inner + c0 + c] * (z * sigmoid_f32(z));
    ss = __fmaf_rn(u, u, ss);
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += 256) {
    const float z = source_load(proj, (long long)t * row_width + c0 + c);
    const float u = y[(long long)t * inner + c0 + c] * (z * sigmoid_f32(z));
    store_as(out, out_dtype, (long long)t * inner + c0 + c, u * rstd * norm_w[c0 + c]);
  }
}

template <int MAXR, int CHUNK, int COLS, int LANES>
int launch_ssm_recurrence(const float* xbc, const float2* dtv, const float* d_skip, float* state, long long slot_stride,
                          float* y, const int* cu_q_lens, const int* state_slots, int B, int H, int G, int N, int P,
                          int CH, cudaStream_t st) {
  const int per = (2 * N + COLS + 2 + 3) / 4 * 4;
  const size_t smem = sizeof(float) * (2 * (size_t)CHUNK * per + (size_t)CHUNK * COLS * (LANES + 2));
  static DeviceOnce once;
  if (smem > 48 * 1024 && !once.done()) {
    if (cudaFuncSetAttribute(ssm_recurrence_kernel<MAXR, CHUNK, COLS, LANES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             100 * 1024) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    once.mark();
  }
  // whole 16-byte pieces where every run starts on a 16-byte boundary
  const int vec = (N % 4 == 0 && P % 4 == 0 && CH % 4 == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0) ? 1 : 0;
  dib_launch(ssm_recurrence_kernel<MAXR, CHUNK, COLS, LANES>, dim3(B, H, (P + COLS - 1) / COLS), dim3(COLS * LANES), smem, st, xbc,
             dtv, d_skip, state, slot_stride, y, cu_q_lens, state_slots, H, G, N, P, CH, vec);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // namespace

extern "C" {

// xbc float32 [T][CH], dtv float32 [T][H][2]; tail_at: where the convolution's tail lies in a slot.
int dib_ssm_prepare(const void* proj, int kind, int splits, long long stride, long long row_width, const float* cw,
                    const float* cb, const float* a_log, const float* dt_bias, const float* state,
                    long long slot_stride, long long tail_at, const int* token_seq, const int* cu_q_lens,
                    const int* state_slots, float* xbc, float* dtv, int T_, int H, int G, int N, int P, int taps,
                    cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  if (H < 1 || G < 1 || H % G || N < 1 || P < 1 || taps < 1 || taps > 64) return DIB_BAD_SIZE;
  const int inner = H * P, CH = inner + 2 * G * N;
  if (row_width < (long long)inner + CH + H) return DIB_BAD_SIZE;
  const int cols = (CH + 255) / 256;
  if (cols > 65535) return DIB_BAD_SIZE;
  dib_launch(ssm_prepare_kernel, dim3(T_, cols), dim3(256), 0, st, make_source(proj, kind, splits, stride), row_width,
             cw, cb, a_log, dt_bias, state, slot_stride, tail_at, token_seq, cu_q_lens, state_slots, xbc,
             reinterpret_cast<float2*>(dtv), H, inner, CH, taps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// state: float32 rows of slot_stride elements, a slot's first H N P the heads' states [H][N][P];
// sequence b of the step owns tokens cu_q_lens[b] .. cu_q_lens[b+1]-1 and the slot state_slots[b].
int dib_ssm_recurrence(const float* xbc, const float* dtv, const float* d_skip, float* state, long long slot_stride,
                       float* y, const int* cu_q_lens, const int* state_slots, int B, int H, int G, int N, int P,
                       cudaStream_t st) {
  if (B == 0) return DIB_OK;
  if (H < 1 || H > 65535 || G < 1 || H % G || N < 1 || N > 512 || P < 1 || (P + 7) / 8 > 65535) return DIB_BAD_SIZE;
  const int CH = H * P + 2 * G * N;
  const float2* dv = reinterpret_cast<const float2*>(dtv);
  // blocks of 4 columns where blocks of 8 would leave SMs with less than two of them (the sums are the same);
  // a column's rows over 32 lanes from a state of 64 on
  const bool narrow = (long long)B * H * ((P + 7) / 8) < 2 * 148 && P > 4;
#define DIB_SSM(MAXR, CHUNK, LANES)                                                                                  \
  return narrow ? launch_ssm_recurrence<MAXR, CHUNK, 4, LANES>(xbc, dv, d_skip, state, slot_stride, y, cu_q_lens,       \
                                                               state_slots, B, H, G, N, P, CH, st)                      \
                : launch_ssm_recurrence<MAXR, CHUNK, 8, LANES>(xbc, dv, d_skip, state, slot_stride, y, cu_q_lens,       \
                                                               state_slots, B, H, G, N, P, CH, st)
  if (N <= 16) DIB_SSM(1, 16, 16);
  if (N <= 32) DIB_SSM(2, 16, 16);
  if (N <= 64) DIB_SSM(2, 16, 32);
  if (N <= 128) DIB_SSM(4, 16, 32);
  if (N <= 256) DIB_SSM(8, 8, 32);
  DIB_SSM(16, 4, 32);
#undef DIB_SSM
}

// The output rows, and then (B sequences) the convolution's tail moved on by the step's tokens.
int dib_ssm_output(const float* y, const void* proj, int kind, int splits, long long stride, long long row_width,
                   const float* norm_w, void* out, int out_dtype, float* state, long long slot_stride,
                   long long tail_at, const int* cu_q_lens, const int* state_slots, int T_, int B, int H, int G, int N,
                   int P, int parts, int taps, float eps, cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  const int inner = H * P, CH = inner + 2 * G * N;
  if (H < 1 || P < 1 || parts < 1 || parts > 65535 || inner % parts || taps < 1) return DIB_BAD_SIZE;
  if (out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  const Source src = make_source(proj, kind, splits, stride);
  dib_launch(ssm_output_kernel, dim3(T_, parts), dim3(256), 0, st, y, src, row_width, norm_w, out, out_dtype, inner,
             parts, eps);
  DIB_CHECK_LAUNCH();
  if (taps > 1 && B > 0) {
    dib_launch(conv_tail_update_kernel, dim3(B), dim3(256), 0, st, src, row_width, (long long)inner,
               (const float*)nullptr, state, slot_stride, tail_at, cu_q_lens, state_slots, CH, taps);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

}  // extern "C"
