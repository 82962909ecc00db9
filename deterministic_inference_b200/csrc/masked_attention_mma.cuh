// bfloat16 tensor-core form of the masked softmax attention of masked_attention.cu for key and
// value sizes the tcgen05 and split-KV kernels do not take (keys wider than values, one latent
// row that is the key of every head and whose first elements are its value): mma.sync m16n8k16
// with float32 accumulators.  One CTA of four or eight warps works on up to 64 or 128 (token,
// head-of-group) rows of one sequence and one key/value head, 16 rows a warp; key tiles of 64
// keys are anchored at absolute position 0, so the tiles a row walks, and their order, depend on
// the row's position alone.  Scores are float32 sums of exact bfloat16 products; the softmax runs
// on line in float32 (a row's maximum so far, its sum, its output rescaled when the maximum
// rises; 2^x on the special-function unit); the weights are rounded to bfloat16 for the product
// with the values.  Keys (and values, where they are stored) of a tile arrive by cp.async, two
// tiles deep.  values_in_keys: the value tile IS the key tile (its first VD columns), so it is
// fetched once.
//
// Decoded tokens (tiles of one token): the token's key tiles are cut into chunks of
// `chunk_tiles`, a CTA per chunk (blockIdx.z), each leaving its unnormalised sums, its maximum and
// its denominator; a second kernel merges a row's chunks in chunk order and applies the sink and
// the gate.  Where a row's sums are cut depends on its position alone.
#pragma once

#include "sigmoid_attention_mma.cuh"      // ldmatrix / mma.sync / cp.async helpers

namespace ma_mma {

using sa_mma::KT;
using sa_mma::PAD;
using sa_mma::copy16;
using sa_mma::ldsm_x4;
using sa_mma::ldsm_x4_trans;
using sa_mma::mma_bf16;
using sa_mma::pack_bf16;

constexpr float MA_NEG_BIG = -1e30f;
constexpr float MA_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ int first_seen(int pos, int mask_kind, int mask_size) {
  if (mask_kind == 1) return pos - mask_size + 1 > 0 ? pos - mask_size + 1 : 0;
  if (mask_kind == 2) return pos > 0 ? pos / mask_size * mask_size : 0;
  return 0;
}
// A window mask may keep the sequence's first `keep` keys visible too.  Their tiles come first in a
// row's walk: the key tiles 0 .. kept_tiles - 1 that lie wholly before the window's first tile, then
// the window's tiles.
__device__ __forceinline__ int kept_tiles(int keep, int first_window_tile) {
  const int n = (keep + KT - 1) / KT;
  return n < first_window_tile ? n : first_window_tile;
}

// tiles: int32 [n][3] = (sequence of the step, first token of the tile among the sequence's new tokens,
// tokens at most).  Where the sequence's tokens lie in the step and how many it really brings is read
// on the device (cu_q_lens): a list made for upper bounds (a captured graph's) names tiles past a
// sequence's real tokens, which leave at once.
// NV16: value columns in units of 16 the accumulators are sized for (VD <= 16 * NV16).
template <int NV16, int ROWS>
__global__ void __launch_bounds__(ROWS * 2)
masked_attention_mma_kernel(const __nv_bfloat16* q, __nv_bfloat16* out, const __nv_bfloat16* cache,
                            const int* block_table, int bt_width, const int* positions, const int* seq_lens,
                            const int* cu_q_lens, const int* tiles, const float* sink, int Hq, int Hkv, int D,
                            int VD, int VD_stored,
                            int page_size, float scale, int mask_kind, int mask_size, int keep, Source gate,
                            long long gate_row, long long gate_col, float* partial_o, float* partial_ml,
                            int chunk_tiles, int max_chunks, float softcap) {
  extern __shared__ __align__(16) unsigned char mam_smem[];
  const int R = Hq / Hkv;
  const bool in_keys = VD_stored == 0;
  const int qs = D + PAD, vs = in_keys ? qs : VD + PAD;   // row strides in elements
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(mam_smem);            // [ROWS][qs]
  __nv_bfloat16* Ks = Qs + ROWS * qs;                                         // [2][KT][qs]
  __nv_bfloat16* Vs = in_keys ? Ks : Ks + 2 * KT * qs;                        // [2][KT][vs]
  __shared__ long long k_off[2][KT], v_off[2][KT];
  pdl_prologue(q, cache, gate.p);
  const int tile = blockIdx.x, g = blockIdx.y;
  const int b = tiles[3 * tile], start = tiles[3 * tile + 1];
  const int q_begin = cu_q_lens[b], q_len = cu_q_lens[b + 1] - q_begin;
  if (start >= q_len) return;               // (the whole CTA: the sequence brings fewer tokens)
  const int t0 = q_begin + start;
  const int count = tiles[3 * tile + 2] < q_len - start ? tiles[3 * tile + 2] : q_len - start;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int kv_len = seq_lens[b];
  const int pos0 = positions[t0];                        // the tile's tokens are consecutive positions
  const int pos_last = pos0 + count - 1;
  const int rows_used = count * R;
  const int* bt = block_table + (long long)b * bt_width;
  const long long page_elems = (long long)Hkv * page_size * (D + VD_stored);

  const int t_first = first_seen(pos0, mask_kind, mask_size) / KT, t_last = pos_last / KT;
  const int n_kept = kept_tiles(keep, t_first);
  const int n_tiles = n_kept + t_last - t_first + 1;
  auto tile_at = [&](int it) { return it < n_kept ? it : t_first + it - n_kept; };   // walk step -> key tile
  const bool chunked = partial_o != nullptr;
  const int chunk = chunked ? blockIdx.z : 0;
  const int it_begin = chunked ? chunk * chunk_tiles : 0;
  const int it_end = (chunked && it_begin + chunk_tiles < n_tiles) ? it_begin + chunk_tiles : n_tiles;
  if (it_begin >= n_tiles) return;          // (the whole CTA: no such chunk at this position)

  const int dchunks = D / 8;
  for (int idx = threadIdx.x; idx < ROWS * dchunks; idx += blockDim.x) {
    const int r = idx / dchunks, ch = idx - r * dchunks;
    const bool ok = r < rows_used;
    const int tl = ok ? r / R : 0, hh = ok ? r % R : 0;
    copy16(Qs + r * qs + ch * 8, q + ((long long)(t0 + tl) * Hq + g * R + hh) * D + ch * 8, ok);
  }
  const int vchunks = VD / 8;
  auto find_rows = [&](int it) {          // by the first KT threads, for tile `it` (if there is one)
    if (threadIdx.x < KT && it < it_end) {
      const int j = tile_at(it) * KT + threadIdx.x;
      long long ko = -1, vo = -1;
      if (j < kv_len) {
        // (a key beyond the table's width, a padding sequence's, reads page 0)
        const long long base = (long long)(j / page_size < bt_width ? bt[j / page_size] : 0) * page_elems;
        const long long r = (long long)g * page_size + j % page_size;
        ko = base + r * D;
        vo = base + (long long)Hkv * page_size * D + r * VD;
      }
      k_off[it & 1][threadIdx.x] = ko;
      v_off[it & 1][threadIdx.x] = vo;
    }
  };
  auto load_tile = [&](int it, int stage) {
    __nv_bfloat16* kd = Ks + stage * KT * qs;
    for (int idx = threadIdx.x; idx < KT * dchunks; idx += blockDim.x) {
      const int jj = idx / dchunks, ch = idx - jj * dchunks;
      const long long off = k_off[stage][jj];
      copy16(kd + jj * qs + ch * 8, cache + (off < 0 ? 0 : off) + ch * 8, off >= 0);
    }
    if (!in_keys) {
      __nv_bfloat16* vd = Vs + stage * KT * vs;
      for (int idx = threadIdx.x; idx < KT * vchunks; idx += blockDim.x) {
        const int jj = idx / vchunks, ch = idx - jj * vchunks;
        const long long off = v_off[stage][jj];
        copy16(vd + jj * vs + ch * 8, cache + (off < 0 ? 0 : off) + ch * 8, off >= 0);
      }
    }
    __pipeline_commit();
  };

  // this thread's two rows: warp * 16 + gid and + 8
  int row_pos[2], row_lo[2];
  const int row_base = warp * 16;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_base + gid + 8 * h;
    const bool ok = r < rows_used;
    row_pos[h] = ok ? pos0 + r / R : -1;               // -1: sees nothing
    row_lo[h] = ok ? first_seen(row_pos[h], mask_kind, mask_size) : 0;
  }
  const int wr1 = row_base + 15 < rows_used - 1 ? row_base + 15 : rows_used - 1;
  const bool warp_has_rows = row_base < rows_used;
  const int wpos_first = pos0 + row_base / R, wpos_last = warp_has_rows ? pos0 + wr1 / R : -1;
  const int wlo_first = first_seen(wpos_first, mask_kind, mask_size);
  const float scale_log2 = scale * MA_LOG2E;

  float o[NV16 * 2][4];
#pragma unroll
  for (int n = 0; n < NV16 * 2; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_row[2] = {MA_NEG_BIG, MA_NEG_BIG}, l_row[2] = {0.f, 0.f};
  constexpr int NKT = KT / 8;

  find_rows(it_begin);
  find_rows(it_begin + 1);
  __syncthreads();
  load_tile(it_begin, it_begin & 1);
  for (int it = it_begin; it < it_end; ++it) {
    const int stage = it & 1;
    if (it + 1 < it_end) {
      load_tile(it + 1, stage ^ 1);
      find_rows(it + 2);        // into this tile's entries: its copies were issued a round ago
      __pipeline_wait_prior(1);
    } else {
      __pipeline_wait_prior(0);
    }
    __syncthreads();
    const int k0 = tile_at(it) * KT;
    // does any row of this warp see a key of this tile?  (a row's first key never lies before an
    // earlier row's)
    const bool needed = warp_has_rows && k0 <= wpos_last && (k0 + KT - 1 >= wlo_first || k0 < keep);
    if (needed) {
      const __nv_bfloat16* kd = Ks + stage * KT * qs;
      const __nv_bfloat16* vd = Vs + stage * KT * vs;
      float s[NKT][4];
#pragma unroll
      for (int n = 0; n < NKT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a0, a1, a2, a3;
        ldsm_x4(a0, a1, a2, a3, Qs + (row_base + (lane & 15)) * qs + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < NKT / 2; ++np) {
          unsigned b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3,
                  kd + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * qs + kk * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * np], a0, a1, a2, a3, b0, b1);
          mma_bf16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      // the softmax on line: scores in units of log 2, masked ones far below everything
      float mx[2] = {MA_NEG_BIG, MA_NEG_BIG};
#pragma unroll
      for (int n = 0; n < NKT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int j = k0 + n * 8 + tig * 2 + (e & 1);
          const bool sees = j <= row_pos[h] && (j >= row_lo[h] || j < keep);
          // (softcap > 0: the scaled score passes softcap * tanh(. / softcap), float32, before the softmax)
          const float sc = softcap > 0.f ? softcap * tanhf(s[n][e] * scale / softcap) * MA_LOG2E : s[n][e] * scale_log2;
          s[n][e] = sees ? sc : MA_NEG_BIG;
          mx[h] = fmaxf(mx[h], s[n][e]);
        }
      float alpha[2], ref[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_row[h], mx[h]);
        ref[h] = m_new <= -1e29f ? 0.f : m_new;       // nothing seen yet: every weight becomes 0
        alpha[h] = ex2(m_row[h] - ref[h]);
        m_row[h] = m_new;
      }
      float sum[2] = {0.f, 0.f};
      unsigned p[NKT][2];
#pragma unroll
      for (int n = 0; n < NKT; ++n)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float w0 = ex2(s[n][2 * h] - ref[h]), w1 = ex2(s[n][2 * h + 1] - ref[h]);
          sum[h] += w0 + w1;
          p[n][h] = pack_bf16(w0, w1);
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
        l_row[h] = l_row[h] * alpha[h] + sum[h];
      }
#pragma unroll
      for (int n = 0; n < NV16 * 2; ++n) {
        o[n][0] *= alpha[0];
        o[n][1] *= alpha[0];
        o[n][2] *= alpha[1];
        o[n][3] *= alpha[1];
      }
#pragma unroll
      for (int kk = 0; kk < NKT / 2; ++kk) {
        const unsigned a0 = p[2 * kk][0], a1 = p[2 * kk][1], a2 = p[2 * kk + 1][0], a3 = p[2 * kk + 1][1];
#pragma unroll
        for (int np = 0; np < NV16; ++np) {
          if (np * 16 < VD) {
            unsigned b0, b1, b2, b3;
            ldsm_x4_trans(b0, b1, b2, b3,
                          vd + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vs + np * 16 + (lane >> 4) * 8);
            mma_bf16(o[2 * np], a0, a1, a2, a3, b0, b1);
            mma_bf16(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
    }
    __syncthreads();       // the stage is written again two tiles on
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + gid + 8 * h;
    if (r >= rows_used) continue;
    const int t = t0 + r / R, head = g * R + r % R;
    const long long row = (long long)t * Hq + head;
    if (chunked) {
      float* po = partial_o + (row * max_chunks + chunk) * VD;
#pragma unroll
      for (int n = 0; n < NV16 * 2; ++n) {
        const int col = n * 8 + tig * 2;
        if (col < VD) *reinterpret_cast<float2*>(po + col) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
      }
      if (tig == 0) *reinterpret_cast<float2*>(partial_ml + (row * max_chunks + chunk) * 2) = make_float2(m_row[h], l_row[h]);
      continue;
    }
    float l = l_row[h];
    if (sink != nullptr) {
      // exp(sink) joins the denominator; a sink above every score becomes the reference
      const float sl = sink[head] * MA_LOG2E;
      const float ref = fmaxf(m_row[h], sl);
      const float a = ex2(m_row[h] - ref);
      l = l * a + ex2(sl - ref);
#pragma unroll
      for (int n = 0; n < NV16 * 2; ++n) {
        o[n][2 * h] *= a;
        o[n][2 * h + 1] *= a;
      }
    }
    const float inv = 1.0f / l;
    __nv_bfloat16* dst = out + row * VD;
#pragma unroll
    for (int n = 0; n < NV16 * 2; ++n) {
      const int col = n * 8 + tig * 2;
      if (col < VD) {
        float x0 = o[n][2 * h] * inv, x1 = o[n][2 * h + 1] * inv;
        if (gate.p != nullptr) {
          const long long at = (long long)t * gate_row + gate_col + (long long)head * VD + col;
          x0 = round_to<__nv_bfloat16>(x0) * sigmoid_f32(round_to<__nv_bfloat16>(source_load(gate, at)));
          x1 = round_to<__nv_bfloat16>(x1) * sigmoid_f32(round_to<__nv_bfloat16>(source_load(gate, at + 1)));
        }
        *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(x0, x1);
      }
    }
  }
}

// out[t, h, :] from the row's chunks, in chunk order: with M the largest of the chunks' maxima (and
// of the sink), out = sum_c o_c 2^(m_c - M) / (sum_c l_c 2^(m_c - M) + 2^(sink - M)), then the gate.
// A token at position p has ceil(tiles(p) / chunk_tiles) chunks, tiles(p) as the kernel above counts.
__global__ void masked_attention_merge_kernel(const float* partial_o, const float* partial_ml, __nv_bfloat16* out,
                                              const int* positions, const float* sink, int Hq, int VD,
                                              int mask_kind, int mask_size, int keep, Source gate,
                                              long long gate_row, long long gate_col, int chunk_tiles,
                                              int max_chunks) {
  pdl_prologue(partial_o, partial_ml, gate.p);
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  const int t_first = first_seen(pos, mask_kind, mask_size) / KT;
  const int n_tiles = kept_tiles(keep, t_first) + pos / KT - t_first + 1;
  int chunks = (n_tiles + chunk_tiles - 1) / chunk_tiles;
  if (chunks > max_chunks) chunks = max_chunks;
  const long long row = (long long)t * Hq + h;
  const float sl = sink != nullptr ? sink[h] * MA_LOG2E : MA_NEG_BIG;
  float M = sl;
  for (int c = 0; c < chunks; ++c) M = fmaxf(M, partial_ml[(row * max_chunks + c) * 2]);
  float L = sink != nullptr ? ex2(sl - M) : 0.f;
  for (int c = 0; c < chunks; ++c) {
    const float2 ml = *reinterpret_cast<const float2*>(partial_ml + (row * max_chunks + c) * 2);
    L += ml.y * ex2(ml.x - M);
  }
  const float inv = 1.0f / L;
  for (int col = threadIdx.x; col < VD; col += blockDim.x) {
    float v = 0.f;
    for (int c = 0; c < chunks; ++c)
      v = __fmaf_rn(partial_o[(row * max_chunks + c) * VD + col], ex2(partial_ml[(row * max_chunks + c) * 2] - M), v);
    v *= inv;
    if (gate.p != nullptr)
      v = round_to<__nv_bfloat16>(v) *
          sigmoid_f32(round_to<__nv_bfloat16>(source_load(gate, (long long)t * gate_row + gate_col + (long long)h * VD + col)));
    out[row * VD + col] = __float2bfloat16_rn(v);
  }
}

// (227 KB a block less the kernel's static arrays)
constexpr int MAX_DYNAMIC_SMEM = 224 * 1024;

static inline size_t smem_bytes(int D, int VD, int VD_stored, int rows) {
  size_t n = (size_t)rows * (D + PAD) + 2 * (size_t)KT * (D + PAD);
  if (VD_stored > 0) n += 2 * (size_t)KT * (VD + PAD);
  return sizeof(__nv_bfloat16) * n;
}

template <int NV16, int ROWS>
static int launch(const void* q, void* out, const void* cache, const int* block_table, int bt_width,
                  const int* positions, const int* seq_lens, const int* cu_q_lens, const int* tiles, int num_tiles,
                  const float* sink, int Hq, int Hkv, int D, int VD, int VD_stored, int page_size, float scale, int mask_kind,
                  int mask_size, int keep, Source gate, long long gate_row, long long gate_col, float* partial_o,
                  float* partial_ml, int chunk_tiles, int max_chunks, int num_tokens, float softcap, cudaStream_t st) {
  const size_t smem = smem_bytes(D, VD, VD_stored, ROWS);
  if (smem > MAX_DYNAMIC_SMEM) return DIB_BAD_SIZE;
  const bool chunked = partial_o != nullptr && max_chunks > 1;
  static DeviceOnce once;
  if (!once.done()) {
    if (cudaFuncSetAttribute(masked_attention_mma_kernel<NV16, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             MAX_DYNAMIC_SMEM) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    once.mark();
  }
  dib_launch(masked_attention_mma_kernel<NV16, ROWS>, dim3(num_tiles, Hkv, chunked ? max_chunks : 1), dim3(ROWS * 2),
             smem, st, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)cache, block_table,
             bt_width, positions, seq_lens, cu_q_lens, tiles, sink, Hq, Hkv, D, VD, VD_stored, page_size, scale, mask_kind,
             mask_size, keep, gate, gate_row, gate_col, chunked ? partial_o : (float*)nullptr,
             chunked ? partial_ml : (float*)nullptr, chunk_tiles, max_chunks, softcap);
  DIB_CHECK_LAUNCH();
  if (chunked) {
    dib_launch(masked_attention_merge_kernel, dim3(num_tokens, Hq), dim3(VD >= 128 ? 128 : 64), 0, st,
               (const float*)partial_o, (const float*)partial_ml, (__nv_bfloat16*)out, positions, sink, Hq, VD,
               mask_kind, mask_size, keep, gate, gate_row, gate_col, chunk_tiles, max_chunks);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

}  // namespace ma_mma
