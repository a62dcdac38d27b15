// Prefill -> decode hand-over: fill the decode caches of one layer from the prefill K/V.
// For every batch row, the tokens selected by `doc_mask` (the prompt's last document) are
// compacted: their retained-slot K/V rows go to the retained cache rows 0..doc_len-1, the
// window-slot K/V rows of the last `window_tokens` of them go to the ring rows 0..window_len-1,
// and the counters are set (ring position 0).  Rows with no selected token are left untouched.
// Reference computation (a Python loop over batch rows with host syncs):
// src/modeling/models/reverse_sps/inference.py:568-613.
#pragma once

#include "common.cuh"

namespace spsattn {

struct CacheFillParams {
  const uint16_t* k;     // [B, 2T, H, D] with strides (elements), D contiguous
  const uint16_t* v;
  int64_t stride_b, stride_n, stride_h;
  const uint8_t* doc_mask;   // [B, T], non-zero = token belongs to the last document
  uint16_t* br_k;        // [B, H, retained_storage, D]
  uint16_t* br_v;
  int64_t* br_len;       // [B, H]
  uint16_t* nw_k;        // [B, H, window_storage, D] (null when window_tokens == 0)
  uint16_t* nw_v;
  int64_t* nw_len;       // [B]
  int64_t* nw_pos;       // [B]
  int T, H, D;
  int retained_storage, window_storage, window_tokens;
  int retained_slot, window_slot;   // parity (0/1) of the row that feeds each cache
};

constexpr int kFillChunk = 64;     // tokens per block

__global__ void __launch_bounds__(256) cache_fill_kernel(const CacheFillParams p) {
  __shared__ int s_warp[8];
  __shared__ int s_rank[kFillChunk];
  __shared__ int s_before, s_total;
  const int b = blockIdx.y;
  const int t0 = blockIdx.x * kFillChunk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint8_t* mask = p.doc_mask + (size_t)b * p.T;

  // selected tokens before this chunk, and in the whole row
  int before = 0, total = 0;
  for (int t = tid; t < p.T; t += blockDim.x) {
    const int m = mask[t] != 0;
    total += m;
    before += (t < t0) ? m : 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    total += __shfl_xor_sync(0xffffffffu, total, o);
    before += __shfl_xor_sync(0xffffffffu, before, o);
  }
  if (lane == 0) s_warp[warp] = (total << 16) | before;   // T < 32768 tokens
  __syncthreads();
  if (tid == 0) {
    int tt = 0, bb = 0;
    for (int w = 0; w < 8; ++w) {
      tt += s_warp[w] >> 16;
      bb += s_warp[w] & 0xffff;
    }
    s_total = tt;
    s_before = bb;
  }
  __syncthreads();
  const int doc_len = s_total;
  if (doc_len == 0) return;

  // rank of every selected token of the chunk (warps 0 and 1 scan 64 flags)
  if (tid < kFillChunk) {
    const int t = t0 + tid;
    const int m = (t < p.T && mask[t] != 0) ? 1 : 0;
    const unsigned bal = __ballot_sync(0xffffffffu, m);
    const int in_warp = __popc(bal & ((1u << lane) - 1));
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncwarp();
    s_rank[tid] = m ? in_warp : -1;
  }
  __syncthreads();
  if (tid >= 32 && tid < kFillChunk && s_rank[tid] >= 0) s_rank[tid] += s_warp[0];
  __syncthreads();

  const int window_len = p.window_tokens > 0 ? min(p.window_tokens, doc_len) : 0;
  const int win_first = doc_len - window_len;   // rank of the first token that enters the ring
  const int vec_per_row = p.D / 8;              // 16-byte vectors per [D] row
  const int vec_per_tok = p.H * vec_per_row;
  for (int idx = tid; idx < kFillChunk * vec_per_tok; idx += blockDim.x) {
    const int lt = idx / vec_per_tok;
    const int r = s_rank[lt];
    if (r < 0) continue;
    const int rank = s_before + r;
    const int rem = idx - lt * vec_per_tok;
    const int h = rem / vec_per_row, x = rem - h * vec_per_row;
    const int t = t0 + lt;
    const size_t src_ret = (size_t)b * p.stride_b + (size_t)(2 * t + p.retained_slot) * p.stride_n +
                           (size_t)h * p.stride_h + x * 8;
    if (rank < p.retained_storage) {
      const size_t dst = (((size_t)b * p.H + h) * p.retained_storage + rank) * p.D + x * 8;
      *reinterpret_cast<uint4*>(p.br_k + dst) = *reinterpret_cast<const uint4*>(p.k + src_ret);
      *reinterpret_cast<uint4*>(p.br_v + dst) = *reinterpret_cast<const uint4*>(p.v + src_ret);
    }
    if (rank >= win_first && rank - win_first < p.window_storage) {
      const size_t src_win = (size_t)b * p.stride_b + (size_t)(2 * t + p.window_slot) * p.stride_n +
                             (size_t)h * p.stride_h + x * 8;
      const size_t dst = (((size_t)b * p.H + h) * p.window_storage + (rank - win_first)) * p.D + x * 8;
      *reinterpret_cast<uint4*>(p.nw_k + dst) = *reinterpret_cast<const uint4*>(p.k + src_win);
      *reinterpret_cast<uint4*>(p.nw_v + dst) = *reinterpret_cast<const uint4*>(p.v + src_win);
    }
  }
  if (blockIdx.x == 0) {
    for (int h = tid; h < p.H; h += blockDim.x) p.br_len[(size_t)b * p.H + h] = doc_len;
    if (tid == 0 && p.window_tokens > 0) {
      p.nw_len[b] = window_len;
      p.nw_pos[b] = 0;
    }
  }
}

}  // namespace spsattn
