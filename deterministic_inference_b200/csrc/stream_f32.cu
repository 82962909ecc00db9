// Kernels of models whose residual stream is kept in float32 whatever the engine's
// storage type is: token + learned position embedding, RMSNorm of the float32 stream
// (alone, or after adding up to two scaled mixer outputs to it), the scaled sum as a
// tensor, the xIELU activation and the soft cap of the logits.  All arithmetic is float32;
// inputs that come from a matrix product may be its split-k partial products.
#include "source.cuh"

// out[t] = table[ids[t]] + pos_table[positions[t]], float32
__global__ void embed_pos_kernel(const void* table, const void* pos_table, int dtype, const int* ids,
                                 const int* positions, float* out, int T, int W, int V, int P) {
  pdl_prologue();
  const int t = blockIdx.x;
  int id = ids[t], p = positions[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  p = p < 0 ? 0 : (p >= P ? P - 1 : p);
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    out[(long long)t * W + c] =
        __fadd_rn(load_as(table, dtype, (long long)id * W + c), load_as(pos_table, dtype, (long long)p * W + c));
}

// out[t] = table[ids[t]] * scale, float32
__global__ void embed_scale_kernel(const void* table, int dtype, const int* ids, float scale, float* out,
                                   int T, int W, int V) {
  pdl_prologue();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    out[(long long)t * W + c] = __fmul_rn(load_as(table, dtype, (long long)id * W + c), scale);
}

// One block per row: residual[row] += x[row] / sqrt(mean(x[row]^2) + eps_x) * wx (+ bias), the
// normed output of the part before added to the stream without being rounded; then, when out is
// given, out[row] = residual[row] / sqrt(mean(residual[row]^2) + eps) * w (w null: out[row] =
// residual[row], not normed).  x null: only the bias is added.  VPT > 0: a thread keeps its VPT elements of the row in registers (W <= VPT * blockDim.x),
// so the row is read once; VPT == 0: any width, the row is read again for every pass.  Both add a
// row's squares in the same order (a thread its own elements in ascending order, then the block's sum).
template <int VPT>
__global__ void stream_normed_add_kernel(float* residual, Source x, const float* wx, float eps_x,
                                         const float* bias, const float* w, void* out, int out_dtype,
                                         int W, float eps) {
  __shared__ float scratch[32];
  pdl_prologue(x.p);
  const long long base = (long long)blockIdx.x * W;
  constexpr int N = VPT > 0 ? VPT : 1;
  float xv[N], rv[N];
  float rx = 0.f;
  if (VPT > 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      xv[i] = (x.p != nullptr && c < W) ? source_load(x, base + c) : 0.f;
      rv[i] = c < W ? residual[base + c] : 0.f;
    }
  }
  if (x.p != nullptr) {
    float sx = 0.f;
    if (VPT > 0) {
#pragma unroll
      for (int i = 0; i < N; ++i) sx = __fmaf_rn(xv[i], xv[i], sx);
    } else {
      for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = source_load(x, base + c);
        sx = __fmaf_rn(v, v, sx);
      }
    }
    rx = 1.0f / sqrtf(block_sum(sx, scratch) / (float)W + eps_x);
  }
  float ss = 0.f;
  if (VPT > 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < W) {
        float r = rv[i];
        if (x.p != nullptr) r = __fadd_rn(r, xv[i] * rx * wx[c]);
        if (bias != nullptr) r = __fadd_rn(r, bias[c]);
        residual[base + c] = r;
        rv[i] = r;
        ss = __fmaf_rn(r, r, ss);
      }
    }
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float r = residual[base + c];
      if (x.p != nullptr) r = __fadd_rn(r, source_load(x, base + c) * rx * wx[c]);
      if (bias != nullptr) r = __fadd_rn(r, bias[c]);
      residual[base + c] = r;
      ss = __fmaf_rn(r, r, ss);
    }
  }
  if (out == nullptr) return;
  if (w == nullptr) {
    // no norm: out is the updated stream itself in out's type
    if (VPT > 0) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < W) store_as(out, out_dtype, base + c, rv[i]);
      }
    } else {
      for (int c = threadIdx.x; c < W; c += blockDim.x) store_as(out, out_dtype, base + c, residual[base + c]);
    }
    return;
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)W + eps);
  if (VPT > 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < W) store_as(out, out_dtype, base + c, rv[i] * rstd * w[c]);
    }
  } else {
    for (int c = threadIdx.x; c < W; c += blockDim.x)
      store_as(out, out_dtype, base + c, residual[base + c] * rstd * w[c]);
  }
}

// [gate | up] rows of width 2I -> I: g = min(gate, limit), u = clamp(up, -limit, limit),
// y = g * sigmoid(alpha * g) * (u + 1)
__global__ void limited_gate_kernel(Source gu, float limit, float alpha, void* out, int out_dtype,
                                    int rows, int I) {
  pdl_prologue(gu.p);
  const long long n = (long long)rows * I;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / I, c = i % I;
    const float g = fminf(source_load(gu, r * 2 * I + c), limit);
    const float u = fminf(fmaxf(source_load(gu, r * 2 * I + I + c), -limit), limit);
    store_as(out, out_dtype, i, g * sigmoid_f32(alpha * g) * (u + 1.0f));
  }
}

// One block per row.  TERMS > 0: residual[row] += a0 * x0[row] (+ a1 * x1[row]) first, the
// terms added in their order; then out[row] = residual[row] / sqrt(mean(residual[row]^2) + eps)
// * w.  The sum of squares is taken by a block of a width that depends on W alone.
template <int TERMS>
__global__ void stream_norm_kernel(float* residual, Source x0, float a0, Source x1, float a1,
                                   const float* w, void* out, int out_dtype, int W, float eps) {
  __shared__ float scratch[32];
  pdl_prologue();
  const long long base = (long long)blockIdx.x * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float r = residual[base + c];
    if (TERMS >= 1) r = __fmaf_rn(a0, source_load(x0, base + c), r);
    if (TERMS >= 2) r = __fmaf_rn(a1, source_load(x1, base + c), r);
    if (TERMS >= 1) residual[base + c] = r;
    ss = __fmaf_rn(r, r, ss);
  }
  const float total = block_sum(ss, scratch);
  const float rstd = 1.0f / sqrtf(total / (float)W + eps);
  if (out == nullptr) return;
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    store_as(out, out_dtype, base + c, residual[base + c] * rstd * w[c]);
}

// One block per row, every term normed before it joins the stream:
// residual[row] += a0 * x0[row] / sqrt(mean(x0[row]^2) + e0) * w0 (+ a1 * x1[row] / sqrt(mean(x1[row]^2) + e1) * w1),
// the terms' sum taken first and then added, nothing rounded below float32; then, when out is given,
// out[row] = residual[row] / sqrt(mean(residual[row]^2) + eps) * w.  A term without a weight (w0 null)
// joins as a0 * x0.  The block's width depends on W alone.
__global__ void stream_norm_normed_terms_kernel(float* residual, int terms, Source x0, float a0, const float* w0,
                                                float e0, Source x1, float a1, const float* w1, float e1,
                                                const float* w, void* out, int out_dtype, int W, float eps) {
  __shared__ float scratch[32];
  pdl_prologue(x0.p, x1.p);
  const long long base = (long long)blockIdx.x * W;
  float r0 = 1.f, r1 = 1.f;
  if (w0 != nullptr) {
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = source_load(x0, base + c);
      s = __fmaf_rn(v, v, s);
    }
    r0 = 1.0f / sqrtf(block_sum(s, scratch) / (float)W + e0);
  }
  if (terms >= 2 && w1 != nullptr) {
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = source_load(x1, base + c);
      s = __fmaf_rn(v, v, s);
    }
    r1 = 1.0f / sqrtf(block_sum(s, scratch) / (float)W + e1);
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = source_load(x0, base + c);
    if (w0 != nullptr) v = v * r0 * w0[c];
    float sum = __fmul_rn(a0, v);
    if (terms >= 2) {
      float u = source_load(x1, base + c);
      if (w1 != nullptr) u = u * r1 * w1[c];
      sum = __fmaf_rn(a1, u, sum);
    }
    const float r = __fadd_rn(residual[base + c], sum);
    residual[base + c] = r;
    ss = __fmaf_rn(r, r, ss);
  }
  if (out == nullptr) return;
  const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    store_as(out, out_dtype, base + c, residual[base + c] * rstd * w[c]);
}

// out = a0 * x0 (+ a1 * x1), float32
__global__ void weighted_sum_kernel(Source x0, float a0, Source x1, float a1, int terms, float* out,
                                    long long n) {
  pdl_prologue();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float r = __fmul_rn(a0, source_load(x0, i));
    if (terms >= 2) r = __fmaf_rn(a1, source_load(x1, i), r);
    out[i] = r;
  }
}

// xIELU: z > 0: ap z^2 + z / 2;  z <= 0: an (exp(z) - 1 - z) + z / 2
__global__ void xielu_kernel(Source z, float ap, float an, void* out, int out_dtype, long long n) {
  pdl_prologue();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float x = source_load(z, i);
    const float y = x > 0.f ? __fmaf_rn(__fmul_rn(ap, x), x, 0.5f * x)
                            : __fmaf_rn(an, expm1f(x) - x, 0.5f * x);
    store_as(out, out_dtype, i, y);
  }
}

// x = cap * tanh(x / cap), in place
__global__ void softcap_kernel(float* x, float cap, long long n) {
  pdl_prologue();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

// x = x * a, in place
__global__ void scale_kernel(float* x, float a, long long n) {
  pdl_prologue();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    x[i] = __fmul_rn(x[i], a);
}

static inline int flat_grid(long long n, int block) {
  long long g = (n + block - 1) / block;
  return (int)(g > 148 * 16 ? 148 * 16 : (g < 1 ? 1 : g));
}

extern "C" {

int dib_embed_pos(const void* table, const void* pos_table, int dtype, const int* ids,
                  const int* positions, float* out, int T, int W, int V, int P, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (dtype != 0 && dtype != 1) return DIB_BAD_DTYPE;
  if (W < 1 || V < 1 || P < 1) return DIB_BAD_SIZE;
  dib_launch(embed_pos_kernel, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, st, table, pos_table, dtype, ids,
             positions, out, T, W, V, P);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_embed_scale(const void* table, int dtype, const int* ids, float scale, float* out, int T, int W,
                    int V, cudaStream_t st) {
  if (T == 0) return DIB_OK;
  if (dtype != 0 && dtype != 1) return DIB_BAD_DTYPE;
  if (W < 1 || V < 1) return DIB_BAD_SIZE;
  dib_launch(embed_scale_kernel, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, st, table, dtype, ids, scale, out,
             T, W, V);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// x null: no normed term; bias null: none; out null: the stream is updated and nothing is normed.
int dib_stream_normed_add(float* residual, const void* x, int kind, int splits, long long stride,
                          const float* wx, float eps_x, const float* bias, const float* w, void* out,
                          int out_dtype, int rows, int W, float eps, cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (W < 1) return DIB_BAD_SIZE;
  if (out != nullptr && out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  const dim3 grid(rows), block(W >= 2048 ? 512 : (W >= 512 ? 256 : 128));
  const Source src = make_source(x, kind, splits, stride);
  const int per_thread = (W + (int)block.x - 1) / (int)block.x;
#define DIB_SNA(VPT) \
  dib_launch(stream_normed_add_kernel<VPT>, grid, block, 0, st, residual, src, wx, eps_x, bias, w, out, out_dtype, W, eps)
  if (per_thread <= 4) DIB_SNA(4);
  else if (per_thread <= 8) DIB_SNA(8);
  else if (per_thread <= 16) DIB_SNA(16);
  else DIB_SNA(0);
#undef DIB_SNA
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_limited_gate(const void* gu, int kind, int splits, long long stride, float limit, float alpha,
                     void* out, int out_dtype, int rows, int I, cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (I < 1) return DIB_BAD_SIZE;
  if (out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  dib_launch(limited_gate_kernel, dim3(flat_grid((long long)rows * I, 256)), dim3(256), 0, st,
             make_source(gu, kind, splits, stride), limit, alpha, out, out_dtype, rows, I);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// terms 0: norm of the stream alone.  x kinds: 0 float32 (splits >= 1), 1 bfloat16.
// out may be null (terms > 0): the stream is updated and nothing is normed.
int dib_stream_norm(float* residual, int terms, const void* x0, int kind0, int splits0, long long stride0,
                    float a0, const void* x1, int kind1, int splits1, long long stride1, float a1,
                    const float* w, void* out, int out_dtype, int rows, int W, float eps,
                    cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (W < 1 || terms < 0 || terms > 2) return DIB_BAD_SIZE;
  if (out != nullptr && out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  const Source s0 = make_source(x0, kind0, splits0, stride0), s1 = make_source(x1, kind1, splits1, stride1);
  const dim3 grid(rows), block(W >= 2048 ? 512 : (W >= 512 ? 256 : 128));
  if (terms == 0) dib_launch(stream_norm_kernel<0>, grid, block, 0, st, residual, s0, a0, s1, a1, w, out, out_dtype, W, eps);
  else if (terms == 1) dib_launch(stream_norm_kernel<1>, grid, block, 0, st, residual, s0, a0, s1, a1, w, out, out_dtype, W, eps);
  else dib_launch(stream_norm_kernel<2>, grid, block, 0, st, residual, s0, a0, s1, a1, w, out, out_dtype, W, eps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

// Terms that are normed on their way into the stream (w0 / w1 null: that term joins as it is).
// out null: the stream is updated and nothing is normed.
int dib_stream_norm_normed_terms(float* residual, int terms, const void* x0, int kind0, int splits0, long long stride0,
                                 float a0, const float* w0, float e0, const void* x1, int kind1, int splits1,
                                 long long stride1, float a1, const float* w1, float e1, const float* w, void* out,
                                 int out_dtype, int rows, int W, float eps, cudaStream_t st) {
  if (rows == 0) return DIB_OK;
  if (W < 1 || terms < 1 || terms > 2) return DIB_BAD_SIZE;
  if (out != nullptr && (w == nullptr || (out_dtype != 0 && out_dtype != 1))) return DIB_BAD_DTYPE;
  const Source s0 = make_source(x0, kind0, splits0, stride0), s1 = make_source(x1, kind1, splits1, stride1);
  const dim3 grid(rows), block(W >= 2048 ? 512 : (W >= 512 ? 256 : 128));
  dib_launch(stream_norm_normed_terms_kernel, grid, block, 0, st, residual, terms, s0, a0, w0, e0, s1, a1, w1, e1, w,
             out, out_dtype, W, eps);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_weighted_sum(int terms, const void* x0, int kind0, int splits0, long long stride0, float a0,
                     const void* x1, int kind1, int splits1, long long stride1, float a1, float* out,
                     long long n, cudaStream_t st) {
  if (n == 0) return DIB_OK;
  if (terms < 1 || terms > 2) return DIB_BAD_SIZE;
  dib_launch(weighted_sum_kernel, dim3(flat_grid(n, 256)), dim3(256), 0, st,
             make_source(x0, kind0, splits0, stride0), a0, make_source(x1, kind1, splits1, stride1), a1, terms,
             out, n);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_xielu(const void* z, int kind, int splits, long long stride, float ap, float an, void* out,
              int out_dtype, long long n, cudaStream_t st) {
  if (n == 0) return DIB_OK;
  if (out_dtype != 0 && out_dtype != 1) return DIB_BAD_DTYPE;
  dib_launch(xielu_kernel, dim3(flat_grid(n, 256)), dim3(256), 0, st, make_source(z, kind, splits, stride), ap,
             an, out, out_dtype, n);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_scale(float* x, float a, long long n, cudaStream_t st) {
  if (n == 0) return DIB_OK;
  dib_launch(scale_kernel, dim3(flat_grid(n, 256)), dim3(256), 0, st, x, a, n);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_softcap(float* x, float cap, long long n, cudaStream_t st) {
  if (n == 0) return DIB_OK;
  dib_launch(softcap_kernel, dim3(flat_grid(n, 256)), dim3(256), 0, st, x, cap, n);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

}  // extern "C"
