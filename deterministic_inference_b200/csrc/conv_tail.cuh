// The state a short causal convolution over time keeps between steps: a sequence's last taps - 1
// inputs, [taps - 1][CH] float32 at tail_at inside its state slot (oldest first).
#pragma once

#include "source.cuh"

// One block per sequence: the tail moves on by the sequence's tokens of this step.  The inputs are the
// columns first_col .. first_col + CH - 1 of the projection rows (plus bias[ch], when given).  A thread
// takes a channel and walks its tail from the oldest entry: entry k takes the input n tokens later,
// which is an older entry (k + n, not yet overwritten) or one of the step's tokens.  Slot 0 keeps none.
__global__ void conv_tail_update_kernel(Source proj, long long row_width, long long first_col, const float* bias,
                                        float* state, long long slot_stride, long long tail_at,
                                        const int* cu_q_lens, const int* state_slots, int CH, int taps) {
  pdl_prologue(proj.p);
  const int b = blockIdx.x;
  const long long slot = state_slots[b];
  const int t0 = cu_q_lens[b], n = cu_q_lens[b + 1] - t0;
  if (slot == 0 || n <= 0) return;
  float* tail = state + slot * slot_stride + tail_at;
  const int keep = taps - 1;
  for (int ch = threadIdx.x; ch < CH; ch += blockDim.x)
    for (int k = 0; k < keep; ++k) {
      const int from = k + n;            // in units of tail entries; entries >= keep are the step's tokens
      float x;
      if (from < keep) {
        x = tail[(long long)from * CH + ch];
      } else {
        x = source_load(proj, (long long)(t0 + from - keep) * row_width + first_col + ch);
        if (bias != nullptr) x = __fadd_rn(x, bias[ch]);
      }
      tail[(long long)k * CH + ch] = x;
    }
}
