// Decode KV-cache update: ring insert + retained append + counters in one launch, one block per
// sequence so the ring counters are read before anything is written (no cross-block ordering).
// Reference computation: src/modeling/models/utils/decode_attention_fast.py:34-136.
#pragma once

#include "common.cuh"

namespace spsattn {

struct KvUpdateParams {
  uint32_t* nw_k;
  uint32_t* nw_v;
  int64_t* nw_len;
  int64_t* nw_pos;
  uint32_t* br_k;
  uint32_t* br_v;
  int64_t* br_len;
  const uint32_t* k_window;
  const uint32_t* v_window;
  const uint32_t* k_retained;
  const uint32_t* v_retained;
  const int8_t* active;
  int H, row_words;  // 32-bit words per [D] row
  int window_storage, retained_storage, window_tokens;
};

__global__ void __launch_bounds__(256) kv_update_kernel(const KvUpdateParams p) {
  extern __shared__ long long s_len[];  // [H] retained lengths before the update
  const int s = blockIdx.x;
  if (p.active[s] == 0) return;
  const int tid = threadIdx.x;
  long long ring_len = 0, ring_pos = 0;
  if (p.window_tokens > 0) {
    ring_len = p.nw_len[s];
    ring_pos = p.nw_pos[s];
  }
  for (int h = tid; h < p.H; h += blockDim.x) s_len[h] = p.br_len[(size_t)s * p.H + h];
  __syncthreads();
  const bool full = ring_len >= p.window_tokens;
  const long long ins = full ? ring_pos : ring_len;
  const int total = p.H * p.row_words;
  for (int idx = tid; idx < total; idx += blockDim.x) {
    const int h = idx / p.row_words, x = idx % p.row_words;
    const size_t src = ((size_t)s * p.H + h) * p.row_words + x;
    if (p.window_tokens > 0 && ins >= 0 && ins < p.window_storage) {
      const size_t dst = (((size_t)s * p.H + h) * p.window_storage + (size_t)ins) * p.row_words + x;
      p.nw_k[dst] = p.k_window[src];
      p.nw_v[dst] = p.v_window[src];
    }
    const long long ln = s_len[h];
    if (ln >= 0 && ln < p.retained_storage) {
      const size_t dst = (((size_t)s * p.H + h) * p.retained_storage + (size_t)ln) * p.row_words + x;
      p.br_k[dst] = p.k_retained[src];
      p.br_v[dst] = p.v_retained[src];
    }
  }
  for (int h = tid; h < p.H; h += blockDim.x) {
    const long long ln = s_len[h];
    if (ln < p.retained_storage) p.br_len[(size_t)s * p.H + h] = ln + 1;
  }
  if (tid == 0 && p.window_tokens > 0) {
    if (full) {
      p.nw_pos[s] = (ring_pos + 1) % p.window_tokens;
    } else {
      p.nw_len[s] = ring_len + 1;
    }
  }
}

}  // namespace spsattn
