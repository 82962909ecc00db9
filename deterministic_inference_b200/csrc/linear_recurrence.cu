// A real-gated linear recurrent unit with a short causal convolution in front of it.  Per token and
// channel, all float32:
//   u = conv(x) + conv_bias,   r = sigmoid(u_b R_b + c_b),   i = sigmoid(u_b I_b + d_b)   (per block b of channels),
//   a = exp(r * neg_rate),     S_t = a S_(t-1) + sqrt(1 - a^2) * i * u,   out = S_t * gelu_tanh(y).
// The projection row is [y: C | x: C] (+ bias).  A state slot is [S: C | the convolution's last
// taps - 1 inputs: (taps - 1) C].  Three kernels: the convolution, the gates (a product per block of
// channels), and the scan over a sequence's tokens; then the convolution's tail moves on.
#include "source.cuh"
#include "conv_tail.cuh"

namespace {

__device__ __forceinline__ float gelu_tanh_f32(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// u[t, c] = sum_j cw[c, j] * x[t - (taps - 1 - j), c] + cb[c]; x = proj[., C + c] + bias[C + c]; inputs before
// the step's first token of the sequence come from its tail (slot 0: zeros).
__global__ void glr_conv_kernel(Source proj, const float* bias, const float* cw, const float* cb, const float* state,
                                const int* token_seq, const int* cu_q_lens, const int* state_slots, float* u,
                                int C, int taps) {
  pdl_prologue(proj.p);
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int local = t - cu_q_lens[b];
  const long long slot = state_slots[b];
  const float* tail = slot != 0 ? state + slot * (long long)taps * C + C : nullptr;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      float x;
      if (back <= local) x = __fadd_rn(source_load(proj, (long long)(t - back) * 2 * C + C + c), bias[C + c]);
      else x = tail != nullptr ? tail[(long long)(taps - 1 - (back - local)) * C + c] : 0.f;
      acc = __fmaf_rn(cw[(long long)c * taps + j], x, acc);
    }
    u[(long long)t * C + c] = __fadd_rn(acc, cb[c]);
  }
}

// gates [2][blocks][P in][P out]; a block of GT_TOKENS tokens x GT_COLS output columns of one block of
// channels; every sum runs over the inputs in ascending order.  out[0] = a, out[1] = sqrt(1 - a^2) i u.
constexpr int GT_TOKENS = 8, GT_COLS = 128;
__global__ void __launch_bounds__(GT_COLS)
glr_gates_kernel(const float* u, const float* gates, const float* gate_bias, const float* neg_rate, float* out,
                 int T, int C, int blocks) {
  extern __shared__ float us[];        // [GT_TOKENS][P]
  pdl_prologue(u);
  const int P = C / blocks;
  const int t0 = blockIdx.x * GT_TOKENS, blk = blockIdx.y;
  const int col = blockIdx.z * GT_COLS + threadIdx.x;
  const int rows = T - t0 < GT_TOKENS ? T - t0 : GT_TOKENS;
  for (int i = threadIdx.x; i < GT_TOKENS * P; i += GT_COLS) {
    const int r = i / P, k = i - r * P;
    us[i] = r < rows ? u[(long long)(t0 + r) * C + blk * P + k] : 0.f;
  }
  __syncthreads();
  if (col >= P) return;
  float ar[GT_TOKENS], ai[GT_TOKENS];
#pragma unroll
  for (int r = 0; r < GT_TOKENS; ++r) ar[r] = ai[r] = 0.f;
  const float* wr = gates + ((long long)blk * P) * P + col;
  const float* wi = gates + ((long long)(blocks + blk) * P) * P + col;
#pragma unroll 4
  for (int k = 0; k < P; ++k) {
    const float a = wr[(long long)k * P], b = wi[(long long)k * P];
#pragma unroll
    for (int r = 0; r < GT_TOKENS; ++r) {
      ar[r] = __fmaf_rn(us[r * P + k], a, ar[r]);
      ai[r] = __fmaf_rn(us[r * P + k], b, ai[r]);
    }
  }
  const int c = blk * P + col;
  const float br = gate_bias[c], bi = gate_bias[C + c], rate = neg_rate[c];
#pragma unroll
  for (int r = 0; r < GT_TOKENS; ++r) {
    if (r < rows) {
      const float gr = sigmoid_f32(__fadd_rn(ar[r], br)), gi = sigmoid_f32(__fadd_rn(ai[r], bi));
      const float log_a = gr * rate;
      const float a = expf(log_a);
      const float gain = sqrtf(-expm1f(2.0f * log_a));       // sqrt(1 - a^2)
      out[(long long)(t0 + r) * C + c] = a;
      out[((long long)T + t0 + r) * C + c] = gain * gi * us[r * P + col];
    }
  }
}

// One thread per (sequence, channel): S over the sequence's tokens of the step, in their order.
constexpr int SCAN_AHEAD = 8;
__global__ void glr_scan_kernel(const float* decay_in, Source proj, const float* bias, float* state,
                                const int* cu_q_lens, const int* state_slots, void* out, int out_dtype, int T,
                                int C, int taps) {
  pdl_prologue(decay_in, proj.p);
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = cu_q_lens[b], t1 = cu_q_lens[b + 1];
  if (t1 <= t0) return;
  const long long slot = state_slots[b];
  float* sp = state + slot * (long long)taps * C + c;
  float S = slot != 0 ? *sp : 0.f;
  const float by = bias[c];
  const float* pa = decay_in + c;
  const float* px = decay_in + (long long)T * C + c;
  for (int t = t0; t < t1; t += SCAN_AHEAD) {
    float a[SCAN_AHEAD], x[SCAN_AHEAD], y[SCAN_AHEAD];
#pragma unroll
    for (int j = 0; j < SCAN_AHEAD; ++j)
      if (t + j < t1) {
        a[j] = pa[(long long)(t + j) * C];
        x[j] = px[(long long)(t + j) * C];
        y[j] = source_load(proj, (long long)(t + j) * 2 * C + c);
      }
#pragma unroll
    for (int j = 0; j < SCAN_AHEAD; ++j)
      if (t + j < t1) {
        S = __fmaf_rn(a[j], S, x[j]);
        store_as(out, out_dtype, (long long)(t + j) * C + c, S * gelu_tanh_f32(__fadd_rn(y[j], by)));
      }
  }
  if (slot != 0) *sp = S;
}

}  // namespace

extern "C" {

int dib_glr_conv(const void* proj, int kind, int splits, long long stride, const float* bias, const float* cw,
                 const float* cb, const float* state, const int* token_seq, const int* cu_q_lens,
                 const int* state_slots, float* u, int T, int C, int taps, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (C < 1 || taps < 1 || taps > 64) return DIB_BAD_SIZE;
  dib_launch(glr_conv_kernel, dim3(T), dim3(C >= 1024 ? 256 : 128), 0, st, make_source(proj, kind, splits, stride),
             bias, cw, cb, state, token_seq, cu_q_lens, state_slots, u, C, taps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_glr_gates(const float* u, const float* gates, const float* gate_bias, const float* neg_rate, float* out,
                  int T, int C, int blocks, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (C < 1 || blocks < 1 || C % blocks || blocks > 65535) return DIB_BAD_SIZE;
  const int P = C / blocks;
  const size_t smem = sizeof(float) * GT_TOKENS * P;
  if (smem > 96 * 1024) return DIB_BAD_SIZE;
  static DeviceOnce once;
  if (smem > 48 * 1024 && !once.done()) {
    if (cudaFuncSetAttribute(glr_gates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    once.mark();
  }
  dib_launch(glr_gates_kernel, dim3((T + GT_TOKENS - 1) / GT_TOKENS, blocks, (P + GT_COLS - 1) / GT_COLS),
             dim3(GT_COLS), smem, st, u, gates, gate_bias, neg_rate, out, T, C, blocks);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// The scan over every sequence's tokens, and then the convolution's tail moved on by them.
int dib_glr_scan(const float* decay_in, const void* proj, int kind, int splits, long long stride, const float* bias,
                 float* state, const int* cu_q_lens, const int* state_slots, void* out, int out_dtype, int B, int T,
                 int C, int taps, cudaStream_t st) {
  if (T == 0 || B == 0) return DIB_OK;
  if (C < 1 || taps < 1 || B > 65535) return DIB_BAD_SIZE;
  if (out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  const Source src = make_source(proj, kind, splits, stride);
  dib_launch(glr_scan_kernel, dim3((C + 63) / 64, B), dim3(64), 0, st, decay_in, src, bias, state, cu_q_lens,
             state_slots, out, out_dtype, T, C, taps);
  DIB_CHECK_LAUNCH();
  if (taps > 1) {
    dib_launch(conv_tail_update_kernel, dim3(B), dim3(256), 0, st, src, (long long)2 * C, (long long)C, bias + C, state,
               (long long)taps * C, (long long)C, cu_q_lens, state_slots, C, taps);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

}  // extern "C"
