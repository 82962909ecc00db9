// Generalised delta rule with a decay per key channel: per head a state S [D keys, D values]
// in float32, carried from token to token in the request's state slot,
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,   o_t = S_t^T r_t,
// with u = k / sqrt(sum(k^2) + key_eps) the unit key, w = exp(-decay_scale * sigmoid(lora + w0))
// the decay and a = sigmoid(. + bias) the removal rate.  Three kernels: the per-token vectors
// (all float32), the recurrence, and the output (per-head RMS norm, weight, sigmoid gate).
//
// The recurrence kernels take a state of D key rows by E value columns per head and a token's
// vectors as [w | b | u | k | r] of D elements each and v of E:
//   S_t = diag(w) S_(t-1) - b (u^T S_(t-1)) + k v^T,   o_t = S_t^T r,
// which is also the gated delta rule (S <- g S; S <- S + beta k (v - S^T k)^T) with w = g in
// every row, u = the unit key, b = g beta u and k = beta u.  Its per-token vectors (short causal
// convolutions with silu in front of q, k and v, unit vectors, rate and decay) and its output
// (RMS norm over a head, weight, silu gate) have kernels of their own below.
#include <cuda_pipeline.h>

#include "source.cuh"
#include "conv_tail.cuh"

// proj row: [r | k | v | g | a_pre | lora hidden] = 5 * H * D + R columns; w2t [R][H * D] (the
// decay map's second matrix, transposed: the threads of a block read consecutive elements).
// packed [T][H][6][D] float32: w, a * u, u, k, r, v.
__global__ void delta_prepare_kernel(Source proj, const void* w2t, int w_dtype, const float* w0,
                                     const float* a_bias, float* packed, int H, int D, int R,
                                     float decay_scale, float key_eps) {
  extern __shared__ float dp_smem[];     // [R] tanh of the lora hidden, then 32 floats of scratch
  float* th = dp_smem;
  float* scratch = dp_smem + R;
  pdl_prologue();
  const int t = blockIdx.x, h = blockIdx.y, c = threadIdx.x;
  const int HD = H * D;
  const long long row = (long long)t * (5 * HD + R);
  for (int j = threadIdx.x; j < R; j += blockDim.x) th[j] = tanhf(source_load(proj, row + 5 * HD + j));
  float k = 0.f, r = 0.f, v = 0.f, a = 0.f, w = 0.f;
  const int ch = h * D + c;
  if (c < D) {
    r = source_load(proj, row + ch);
    k = source_load(proj, row + HD + ch);
    v = source_load(proj, row + 2 * HD + ch);
    a = sigmoid_f32(__fadd_rn(source_load(proj, row + 4 * HD + ch), a_bias != nullptr ? a_bias[ch] : 0.f));
  }
  const float ss = block_sum(k * k, scratch);      // (also orders the writes of th before their reads)
  if (c < D) {
    float z = 0.f;
    for (int j = 0; j < R; ++j) z = __fmaf_rn(load_as(w2t, w_dtype, (long long)j * HD + ch), th[j], z);
    z = __fadd_rn(z, w0[ch]);
    w = expf(-decay_scale * sigmoid_f32(z));
    const float u = k / sqrtf(ss + key_eps);
    float* out = packed + ((long long)t * H + h) * 6 * D + c;
    out[0] = w;
    out[D] = a * u;
    out[2 * D] = u;
    out[3 * D] = k;
    out[4 * D] = r;
    out[5 * D] = v;
  }
}

// One warp per (sequence, head, 8 value columns); a column's D state rows are spread over
// 4 lanes (row i = 16 q + 4 s + e for lane s), each lane keeping its rows in registers over
// all tokens of the sequence in this step.  Each of the two sums over the rows (u . S and
// r . S) is taken as four chains inside a lane (rows e, e + 16, e + 32, ... for e = 0..3, in
// ascending order), added as (c0 + c1) + (c2 + c3), and then over the 4 lanes by a butterfly:
// an order that depends on D alone.  Every warp stages the token's six vectors in a ring of
// its own in shared memory by asynchronous copies, DR_STAGES tokens deep, and waits for nobody
// but itself.
template <int MAXR, int DR_STAGES>
__global__ void __launch_bounds__(128)
delta_recurrence_kernel(const float* packed, float* state, long long slot_stride, float* o_out,
                        const int* cu_q_lens, const int* state_slots, int H, int D, int E) {
  extern __shared__ __align__(16) float dr_smem[];           // [4 warps][DR_STAGES][5 Dp + Ep]
  const int Dp = (D + 15) / 16 * 16, Ep = (E + 15) / 16 * 16;
  const int SV = 5 * Dp + Ep;                  // a stage: w, b, u, k, r of Dp floats each, then v of Ep
  const int NR = Dp / 4;                       // rows per lane (<= MAXR)
  const int b = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = lane & 3;
  const int c = (blockIdx.z * 4 + warp) * 8 + (lane >> 2);
  const bool active = c < E;
  if ((blockIdx.z * 4 + warp) * 8 >= E) return;              // none of this warp's columns exists
  float* ring = dr_smem + warp * DR_STAGES * SV;
  if (Dp != D)
    for (int i = lane; i < DR_STAGES * SV; i += 32) ring[i] = 0.f;   // the padding stays 0
  pdl_wait();                        // (the kernel behind this one is not launched ahead of its end)
  const int t0 = cu_q_lens[b], t1 = cu_q_lens[b + 1];
  if (t1 <= t0) return;
  const long long slot = state_slots[b];
  const bool kept = slot != 0;       // slot 0 belongs to padding sequences: zero state, nothing stored
  float* S = state + slot * slot_stride + (long long)h * D * E;
  float st[MAXR];
#pragma unroll
  for (int ii = 0; ii < MAXR; ++ii) {
    const int i = (ii >> 2) * 16 + s * 4 + (ii & 3);
    st[ii] = (kept && ii < NR && active && i < D) ? S[(long long)i * E + c] : 0.f;
  }
  __syncwarp();
  const int PV = 5 * D + E;                    // a token's vectors of one head, as they are stored
  const bool wide = ((D | E) & 3) == 0;        // every vector starts on 16 bytes
  // this lane's 16-byte pieces of a token's vectors: where they come from and go to
  constexpr int PIECES = MAXR * 4 * 6 / 4 / 32;      // (5 D + E) / 4 pieces over 32 lanes, at most
  int src_at[PIECES], dst_at[PIECES];
#pragma unroll
  for (int k = 0; k < PIECES; ++k) {
    const int at = (lane + 32 * k) * 4;
    const int vsel = at < 5 * D ? at / D : 5, d = at - vsel * D;
    src_at[k] = (wide && at < PV) ? at : -1;
    dst_at[k] = vsel * Dp + d;
  }
  auto prefetch = [&](int t, int stage) {
    if (t < t1) {
      const float* src = packed + ((long long)t * H + h) * PV;
      float* dst = ring + stage * SV;
      if (wide) {
#pragma unroll
        for (int k = 0; k < PIECES; ++k)
          if (src_at[k] >= 0) __pipeline_memcpy_async(dst + dst_at[k], src + src_at[k], 16);
      } else {
        for (int i = lane; i < PV; i += 32) {
          const int vsel = i < 5 * D ? i / D : 5, d = i - vsel * D;
          __pipeline_memcpy_async(dst + vsel * Dp + d, src + i, 4);
        }
      }
    }
    __pipeline_commit();                       // (an empty group past the end keeps the count)
  };
#pragma unroll
  for (int k = 0; k < DR_STAGES - 1; ++k) prefetch(t0 + k, k);
  for (int t = t0; t < t1; ++t) {
    const int stage = (t - t0) % DR_STAGES;
    prefetch(t + DR_STAGES - 1, (stage + DR_STAGES - 1) % DR_STAGES);
    __pipeline_wait_prior(DR_STAGES - 1);
    __syncwarp();
    const float* vw = ring + stage * SV;
    const float* vb = vw + Dp;
    const float* vu = vb + Dp;
    const float* vk = vu + Dp;
    const float* vr = vk + Dp;
    const float v = active ? vr[Dp + c] : 0.f;
    float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
    for (int q = 0; q < MAXR / 4; ++q) {
      if (q * 4 < NR) {
        const float4 u4 = *reinterpret_cast<const float4*>(vu + q * 16 + s * 4);
        d0 = __fmaf_rn(u4.x, st[q * 4 + 0], d0);
        d1 = __fmaf_rn(u4.y, st[q * 4 + 1], d1);
        d2 = __fmaf_rn(u4.z, st[q * 4 + 2], d2);
        d3 = __fmaf_rn(u4.w, st[q * 4 + 3], d3);
      }
    }
    float dot = __fadd_rn(__fadd_rn(d0, d1), __fadd_rn(d2, d3));
    dot = __fadd_rn(dot, __shfl_xor_sync(0xffffffffu, dot, 1));
    dot = __fadd_rn(dot, __shfl_xor_sync(0xffffffffu, dot, 2));
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int q = 0; q < MAXR / 4; ++q) {
      if (q * 4 < NR) {
        const int at = q * 16 + s * 4;
        const float4 w4 = *reinterpret_cast<const float4*>(vw + at);
        const float4 b4 = *reinterpret_cast<const float4*>(vb + at);
        const float4 k4 = *reinterpret_cast<const float4*>(vk + at);
        const float4 r4 = *reinterpret_cast<const float4*>(vr + at);
        float n0 = __fmaf_rn(k4.x, v, __fmaf_rn(-b4.x, dot, __fmul_rn(w4.x, st[q * 4 + 0])));
        float n1 = __fmaf_rn(k4.y, v, __fmaf_rn(-b4.y, dot, __fmul_rn(w4.y, st[q * 4 + 1])));
        float n2 = __fmaf_rn(k4.z, v, __fmaf_rn(-b4.z, dot, __fmul_rn(w4.z, st[q * 4 + 2])));
        float n3 = __fmaf_rn(k4.w, v, __fmaf_rn(-b4.w, dot, __fmul_rn(w4.w, st[q * 4 + 3])));
        st[q * 4 + 0] = n0; st[q * 4 + 1] = n1; st[q * 4 + 2] = n2; st[q * 4 + 3] = n3;
        o0 = __fmaf_rn(r4.x, n0, o0);
        o1 = __fmaf_rn(r4.y, n1, o1);
        o2 = __fmaf_rn(r4.z, n2, o2);
        o3 = __fmaf_rn(r4.w, n3, o3);
      }
    }
    float o = __fadd_rn(__fadd_rn(o0, o1), __fadd_rn(o2, o3));
    o = __fadd_rn(o, __shfl_xor_sync(0xffffffffu, o, 1));
    o = __fadd_rn(o, __shfl_xor_sync(0xffffffffu, o, 2));
    if (active && s == 0) o_out[((long long)t * H + h) * E + c] = o;
    __syncwarp();        // the next round's copies overwrite the stage that was read one round ago
  }
#pragma unroll
  for (int ii = 0; ii < MAXR; ++ii) {
    const int i = (ii >> 2) * 16 + s * 4 + (ii & 3);
    if (kept && ii < NR && active && i < D) S[(long long)i * E + c] = st[ii];
  }
}

// The same recurrence with a column's rows over 16 lanes (row i = 64 q + 4 s + e for lane s): a
// block of four warps per (sequence, head, 8 value columns), two columns a warp, the token's
// vectors staged once per block, DR_STAGES tokens deep, one barrier a token, the block's slab of
// the state through shared memory in rows of 32 bytes.  Fewer instructions per token and warp
// (4 rows a lane at D = 64) and four times the CTAs: the form for steps with few sequences and
// many tokens (prompt portions).  Its sums are ordered differently from the form above (four
// chains by e, then a butterfly over 16 lanes), again by D alone.
template <int MAXR, int DR_STAGES>
__global__ void __launch_bounds__(128)
delta_recurrence_wide_kernel(const float* packed, float* state, long long slot_stride, float* o_out,
                             const int* cu_q_lens, const int* state_slots, int H, int D, int E) {
  extern __shared__ __align__(16) float dr_smem[];           // [DR_STAGES][5 Dp + Ep]; first also [D][8] of state
  const int Dp = (D + 63) / 64 * 64, Ep = (E + 63) / 64 * 64;
  const int SV = 5 * Dp + Ep;                  // a stage: w, b, u, k, r of Dp floats each, then v of Ep
  const int NR = Dp / 16;                      // rows per lane (<= MAXR)
  const int b = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = lane & 15;
  const int cl = warp * 2 + (lane >> 4);       // this lane's column among the block's 8
  const int c0 = blockIdx.z * 8, c = c0 + cl;
  const bool active = c < E;
  pdl_wait();                        // (launched in stream order; nothing is launched ahead of its end either)
  const int t0 = cu_q_lens[b], t1 = cu_q_lens[b + 1];
  if (t1 <= t0) return;
  const long long slot = state_slots[b];
  const bool kept = slot != 0;       // slot 0 belongs to padding sequences: zero state, nothing stored
  float* S = state + slot * slot_stride + (long long)h * D * E;
  float* slab = dr_smem;                        // [D][8]
  for (int i = threadIdx.x; i < D * 8; i += blockDim.x) {
    const int row = i >> 3, col = i & 7;
    slab[i] = (kept && c0 + col < E) ? S[(long long)row * E + c0 + col] : 0.f;
  }
  __syncthreads();
  float st[MAXR];
#pragma unroll
  for (int ii = 0; ii < MAXR; ++ii) {
    const int i = (ii >> 2) * 64 + s * 4 + (ii & 3);
    st[ii] = (ii < NR && i < D) ? slab[i * 8 + cl] : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < DR_STAGES * SV; i += blockDim.x) dr_smem[i] = 0.f;   // the padding stays 0
  __syncthreads();
  const int PV = 5 * D + E;                    // a token's vectors of one head, as they are stored
  const bool wide = ((D | E) & 3) == 0;        // every vector starts on 16 bytes
  // this thread's 16-byte pieces of a token's vectors ((5 D + E) / 4 pieces over 128 threads: at most 3)
  int src_at[3], dst_at[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int at = (threadIdx.x + 128 * k) * 4;
    const int vsel = at < 5 * D ? at / D : 5, d = at - vsel * D;
    src_at[k] = (wide && at < PV) ? at : -1;
    dst_at[k] = vsel * Dp + d;
  }
  auto prefetch = [&](int t, int stage) {
    if (t < t1) {
      const float* src = packed + ((long long)t * H + h) * PV;
      float* dst = dr_smem + stage * SV;
      if (wide) {
#pragma unroll
        for (int k = 0; k < 3; ++k)
          if (src_at[k] >= 0) __pipeline_memcpy_async(dst + dst_at[k], src + src_at[k], 16);
      } else {
        for (int i = threadIdx.x; i < PV; i += blockDim.x) {
          const int vsel = i < 5 * D ? i / D : 5, d = i - vsel * D;
          __pipeline_memcpy_async(dst + vsel * Dp + d, src + i, 4);
        }
      }
    }
    __pipeline_commit();                       // (an empty group past the end keeps the count)
  };
#pragma unroll
  for (int k = 0; k < DR_STAGES - 1; ++k) prefetch(t0 + k, k);
  float* o_at = o_out + ((long long)t0 * H + h) * E + c;
  const long long o_step = (long long)H * E;
  for (int t = t0; t < t1; ++t) {
    const int stage = (t - t0) % DR_STAGES;
    __pipeline_wait_prior(DR_STAGES - 2);      // this thread's copies of token t have landed
    __syncthreads();                           // ... and everybody's; everybody is done with token t - 1
    prefetch(t + DR_STAGES - 1, (stage + DR_STAGES - 1) % DR_STAGES);     // into the stage of token t - 1
    const float* vw = dr_smem + stage * SV;
    const float* vb = vw + Dp;
    const float* vu = vb + Dp;
    const float* vk = vu + Dp;
    const float* vr = vk + Dp;
    const float v = active ? vr[Dp + c] : 0.f;
    float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
    for (int q = 0; q < MAXR / 4; ++q) {
      if (q * 4 < NR) {
        const float4 u4 = *reinterpret_cast<const float4*>(vu + q * 64 + s * 4);
        d0 = __fmaf_rn(u4.x, st[q * 4 + 0], d0);
        d1 = __fmaf_rn(u4.y, st[q * 4 + 1], d1);
        d2 = __fmaf_rn(u4.z, st[q * 4 + 2], d2);
        d3 = __fmaf_rn(u4.w, st[q * 4 + 3], d3);
      }
    }
    float dot = __fadd_rn(__fadd_rn(d0, d1), __fadd_rn(d2, d3));
#pragma unroll
    for (int m = 1; m < 16; m <<= 1) dot = __fadd_rn(dot, __shfl_xor_sync(0xffffffffu, dot, m));
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int q = 0; q < MAXR / 4; ++q) {
      if (q * 4 < NR) {
        const int at = q * 64 + s * 4;
        const float4 w4 = *reinterpret_cast<const float4*>(vw + at);
        const float4 b4 = *reinterpret_cast<const float4*>(vb + at);
        const float4 k4 = *reinterpret_cast<const float4*>(vk + at);
        const float4 r4 = *reinterpret_cast<const float4*>(vr + at);
        float n0 = __fmaf_rn(k4.x, v, __fmaf_rn(-b4.x, dot, __fmul_rn(w4.x, st[q * 4 + 0])));
        float n1 = __fmaf_rn(k4.y, v, __fmaf_rn(-b4.y, dot, __fmul_rn(w4.y, st[q * 4 + 1])));
        float n2 = __fmaf_rn(k4.z, v, __fmaf_rn(-b4.z, dot, __fmul_rn(w4.z, st[q * 4 + 2])));
        float n3 = __fmaf_rn(k4.w, v, __fmaf_rn(-b4.w, dot, __fmul_rn(w4.w, st[q * 4 + 3])));
        st[q * 4 + 0] = n0; st[q * 4 + 1] = n1; st[q * 4 + 2] = n2; st[q * 4 + 3] = n3;
        o0 = __fmaf_rn(r4.x, n0, o0);
        o1 = __fmaf_rn(r4.y, n1, o1);
        o2 = __fmaf_rn(r4.z, n2, o2);
        o3 = __fmaf_rn(r4.w, n3, o3);
      }
    }
    float o = __fadd_rn(__fadd_rn(o0, o1), __fadd_rn(o2, o3));
#pragma unroll
    for (int m = 1; m < 16; m <<= 1) o = __fadd_rn(o, __shfl_xor_sync(0xffffffffu, o, m));
    if (active && s == 0) *o_at = o;
    o_at += o_step;
  }
  __pipeline_wait_prior(0);
  __syncthreads();                   // the ring is free: the slab goes out through it
#pragma unroll
  for (int ii = 0; ii < MAXR; ++ii) {
    const int i = (ii >> 2) * 64 + s * 4 + (ii & 3);
    if (ii < NR && i < D) slab[i * 8 + cl] = st[ii];
  }
  __syncthreads();
  if (kept)
    for (int i = threadIdx.x; i < D * 8; i += blockDim.x) {
      const int row = i >> 3, col = i & 7;
      if (c0 + col < E) S[(long long)row * E + c0 + col] = slab[i];
    }
}

// y[t, h, :] = o / sqrt(mean(o^2) + eps) * norm_w[h, :] * sigmoid(g[t, h, :])
__global__ void delta_output_kernel(const float* o, Source proj, const float* norm_w, void* out, int out_dtype,
                                    int H, int D, int R, float eps) {
  __shared__ float scratch[32];
  pdl_prologue();
  const int t = blockIdx.x, h = blockIdx.y, c = threadIdx.x;
  const int HD = H * D;
  const long long at = ((long long)t * H + h) * D + c;
  const float x = c < D ? o[at] : 0.f;
  const float ss = block_sum(x * x, scratch);
  if (c < D) {
    const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
    const float g = source_load(proj, (long long)t * (5 * HD + R) + 3 * HD + h * D + c);
    store_as(out, out_dtype, at, x * rstd * norm_w[h * D + c] * sigmoid_f32(g));
  }
}

// ---- gated delta rule: what goes in front of the recurrence and behind it ---------------------
// proj row (row_width elements): [q: G D | k: G D | v: H E | gate: H E | b: H | a: H | ...].  The
// convolutions' channels are the row's first CH = 2 G D + H E elements; cw [CH][taps] (the last
// tap is the current token's).  A sequence's inputs before the step's first token come from the
// tail of its state slot, [taps - 1][CH] floats at tail_at (oldest first); slot 0 has none (zeros).
__device__ __forceinline__ float conv_silu(const Source& proj, long long row_width, const float* cw,
                                           const float* tail, int CH, int taps, int t, int local, int ch) {
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {          // tap j reads the input taps - 1 - j tokens back
    const int back = taps - 1 - j;
    float x;
    if (back <= local) x = source_load(proj, (long long)(t - back) * row_width + ch);
    else x = tail != nullptr ? tail[(long long)(taps - 1 - (back - local)) * CH + ch] : 0.f;
    acc = __fmaf_rn(cw[(long long)ch * taps + j], x, acc);
  }
  return acc * sigmoid_f32(acc);
}

// One block per (token, value head): packed [T][H][5 D + E] = w (the decay in every row), g beta u,
// u, beta u, q (unit, times D^-1/2), v; u the unit key.
__global__ void gated_delta_prepare_kernel(Source proj, long long row_width, const float* cw, const float* a_log,
                                           const float* dt_bias, const float* state, long long slot_stride,
                                           long long tail_at, const int* token_seq, const int* cu_q_lens,
                                           const int* state_slots, float* packed, int H, int G, int D, int E,
                                           int taps, float key_eps) {
  __shared__ float scratch[32];
  pdl_prologue(proj.p);
  const int t = blockIdx.x, h = blockIdx.y, c = threadIdx.x;
  const int g = h / (H / G);
  const int CH = 2 * G * D + H * E;
  const int b = token_seq[t];
  const int local = t - cu_q_lens[b];
  const long long slot = state_slots[b];
  const float* tail = slot != 0 ? state + slot * slot_stride + tail_at : nullptr;
  float q = 0.f, k = 0.f, v = 0.f;
  if (c < D) {
    q = conv_silu(proj, row_width, cw, tail, CH, taps, t, local, g * D + c);
    k = conv_silu(proj, row_width, cw, tail, CH, taps, t, local, G * D + g * D + c);
  }
  if (c < E) v = conv_silu(proj, row_width, cw, tail, CH, taps, t, local, 2 * G * D + h * E + c);
  const float qq = block_sum(q * q, scratch);
  const float kk = block_sum(k * k, scratch);
  const long long row = (long long)t * row_width;
  const float beta = sigmoid_f32(source_load(proj, row + CH + (long long)H * E + h));
  const float z = __fadd_rn(source_load(proj, row + CH + (long long)H * E + H + h), dt_bias[h]);
  const float softplus = z > 20.f ? z : log1pf(expf(z));
  const float decay = expf(-expf(a_log[h]) * softplus);
  float* out = packed + ((long long)t * H + h) * (5 * D + E);
  if (c < D) {
    const float u = k / sqrtf(kk + key_eps);
    out[c] = decay;
    out[D + c] = decay * beta * u;
    out[2 * D + c] = u;
    out[3 * D + c] = beta * u;
    out[4 * D + c] = q / sqrtf(qq + key_eps) * rsqrtf((float)D);
  }
  if (c < E) out[5 * D + c] = v;
}

// y[t, h, :] = o / sqrt(mean(o^2) + eps) * norm_w[:] * silu(gate[t, h, :]); the weight is shared by the heads
__global__ void gated_delta_output_kernel(const float* o, Source proj, long long row_width, long long gate_col,
                                          const float* norm_w, void* out, int out_dtype, int H, int E, float eps) {
  __shared__ float scratch[32];
  pdl_prologue(o, proj.p);
  const int t = blockIdx.x, h = blockIdx.y, c = threadIdx.x;
  const long long at = ((long long)t * H + h) * E + c;
  const float x = c < E ? o[at] : 0.f;
  const float ss = block_sum(x * x, scratch);
  if (c < E) {
    const float rstd = 1.0f / sqrtf(ss / (float)E + eps);
    const float g = source_load(proj, (long long)t * row_width + gate_col + (long long)h * E + c);
    store_as(out, out_dtype, at, x * rstd * norm_w[c] * (g * sigmoid_f32(g)));
  }
}

template <int MAXR, int DR_STAGES>
static int launch_recurrence(const float* packed, float* state, long long slot_stride, float* o_out,
                             const int* cu_q_lens, const int* state_slots, int B, int H, int D, int E, cudaStream_t st) {
  const int Dp = (D + 15) / 16 * 16, Ep = (E + 15) / 16 * 16;
  const size_t smem = sizeof(float) * 4 * DR_STAGES * (5 * Dp + Ep);   // 48 KB at D = E = 64, 72 at 128, 96 at 256
  static DeviceOnce once;
  if (smem > 48 * 1024 && !once.done()) {
    if (cudaFuncSetAttribute(delta_recurrence_kernel<MAXR, DR_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             100 * 1024) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    once.mark();
  }
  dib_launch(delta_recurrence_kernel<MAXR, DR_STAGES>, dim3(B, H, (E + 31) / 32), dim3(128), smem, st, packed, state,
             slot_stride, o_out, cu_q_lens, state_slots, H, D, E);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

template <int MAXR, int DR_STAGES>
static int launch_recurrence_wide(const float* packed, float* state, long long slot_stride, float* o_out,
                                  const int* cu_q_lens, const int* state_slots, int B, int H, int D, int E,
                                  cudaStream_t st) {
  const int Dp = (D + 63) / 64 * 64, Ep = (E + 63) / 64 * 64;
  size_t smem = sizeof(float) * DR_STAGES * (5 * Dp + Ep);       // 12 KB at D = E = 64, 24 at 256
  if (smem < sizeof(float) * 8 * D) smem = sizeof(float) * 8 * D;
  // Launched in plain stream order, not ahead of its predecessor's end: blocks that are placed
  // while the kernel before still fills the GPU land several to an SM on the SMs that happen to
  // be free, and a long chain of dependent instructions then shares its scheduler for the whole
  // kernel (2,048 tokens, 16 heads of 64: 2.0 ms against 1.0 ms).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(B, H, (E + 7) / 8);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchKernelEx(&cfg, delta_recurrence_wide_kernel<MAXR, DR_STAGES>, packed, state, slot_stride, o_out,
                     cu_q_lens, state_slots, H, D, E);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

extern "C" {

int dib_delta_prepare(const void* proj, int kind, int splits, long long stride, const void* w2t, int w_dtype,
                      const float* w0, const float* a_bias, float* packed, int T_, int H, int D, int R,
                      float decay_scale, float key_eps, cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  if (H < 1 || H > 65535 || D < 1 || D > 1024 || R < 0 || R > 8192) return DIB_BAD_SIZE;
  if (w_dtype != 0 && w_dtype != 1) return DIB_BAD_DTYPE;
  dib_launch(delta_prepare_kernel, dim3(T_, H), dim3((D + 31) / 32 * 32), sizeof(float) * (R + 32), st,
             make_source(proj, kind, splits, stride), w2t, w_dtype, w0, a_bias, packed, H, D, R, decay_scale,
             key_eps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// state: float32 rows of slot_stride elements, a slot's first H * D * E the heads' states [H, D, E];
// sequence b of the step owns tokens cu_q_lens[b] .. cu_q_lens[b+1]-1 and the state slot
// state_slots[b].  Slot 0 is no request's: a sequence on it starts from a zero state and leaves none.
// packed [T][H][5 D + E].
// form 1: a column's rows over 16 lanes (for steps of few sequences with many tokens), 0: over 4.
int dib_delta_recurrence(const float* packed, float* state, long long slot_stride, float* o_out,
                         const int* cu_q_lens, const int* state_slots, int B, int H, int D, int E, int form,
                         cudaStream_t st) {
  if (B == 0) return DIB_OK;
  if (H < 1 || H > 65535 || D < 1 || D > 256 || E < 1 || E > 256) return DIB_BAD_SIZE;
  const int big = D > E ? D : E;       // (the staging's pieces are counted for the larger of the two)
#define DIB_DR(F, MAXR, STAGES) return F<MAXR, STAGES>(packed, state, slot_stride, o_out, cu_q_lens, state_slots, B, H, D, E, st)
  if (form == 1) {
    if (big <= 64) DIB_DR(launch_recurrence_wide, 4, 8);
    if (big <= 128) DIB_DR(launch_recurrence_wide, 8, 6);
    DIB_DR(launch_recurrence_wide, 16, 4);
  }
  if (big <= 64) DIB_DR(launch_recurrence, 16, 8);
  if (big <= 128) DIB_DR(launch_recurrence, 32, 6);
  DIB_DR(launch_recurrence, 64, 4);
#undef DIB_DR
}

int dib_delta_output(const float* o, const void* proj, int kind, int splits, long long stride,
                     const float* norm_w, void* out, int out_dtype, int T_, int H, int D, int R, float eps,
                     cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  if (H < 1 || H > 65535 || D < 1 || D > 1024) return DIB_BAD_SIZE;
  if (out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  dib_launch(delta_output_kernel, dim3(T_, H), dim3((D + 31) / 32 * 32), 0, st, o,
             make_source(proj, kind, splits, stride), norm_w, out, out_dtype, H, D, R, eps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_gated_delta_prepare(const void* proj, int kind, int splits, long long stride, long long row_width,
                            const float* cw, const float* a_log, const float* dt_bias, const float* state,
                            long long slot_stride, long long tail_at, const int* token_seq, const int* cu_q_lens,
                            const int* state_slots, float* packed, int T_, int H, int G, int D, int E, int taps,
                            float key_eps, cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  if (H < 1 || H > 65535 || G < 1 || H % G || D < 1 || D > 1024 || E < 1 || E > 1024 || taps < 1 || taps > 64)
    return DIB_BAD_SIZE;
  const int width = D > E ? D : E;
  dib_launch(gated_delta_prepare_kernel, dim3(T_, H), dim3((width + 31) / 32 * 32), 0, st,
             make_source(proj, kind, splits, stride), row_width, cw, a_log, dt_bias, state, slot_stride, tail_at,
             token_seq, cu_q_lens, state_slots, packed, H, G, D, E, taps, key_eps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The output rows, and then (B sequences) the convolutions' tails moved on by the step's tokens.
int dib_gated_delta_output(const float* o, const void* proj, int kind, int splits, long long stride,
                           long long row_width, const float* norm_w, void* out, int out_dtype, float* state,
                           long long slot_stride, long long tail_at, const int* cu_q_lens, const int* state_slots,
                           int T_, int B, int H, int G, int D, int E, int taps, float eps, cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  if (H < 1 || H > 65535 || G < 1 || E < 1 || E > 1024 || taps < 1) return DIB_BAD_SIZE;
  if (out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  const Source src = make_source(proj, kind, splits, stride);
  const int CH = 2 * G * D + H * E;
  dib_launch(gated_delta_output_kernel, dim3(T_, H), dim3((E + 31) / 32 * 32), 0, st, o, src, row_width,
             (long long)CH, norm_w, out, out_dtype, H, E, eps);
  DIB_CHECK_LAUNCH();
  if (taps > 1 && B > 0) {
    dib_launch(conv_tail_update_kernel, dim3(B), dim3(256), 0, st, src, row_width, 0ll, (const float*)nullptr, state,
               slot_stride, tail_at, cu_q_lens, state_slots, CH, taps);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

}  // extern "C"
