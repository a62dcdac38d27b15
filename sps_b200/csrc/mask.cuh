// Visibility rule of the SPS attention family as per-row key-token intervals.
//
// The doubled sequence has N rows; in the SPS modes row = 2 * tok + parity and the keys are
// treated as two streams (parity 0 and 1), in the standard mode there is one stream with
// row = tok.  For a query row i the visible keys of stream p are exactly the tokens
// kt in [kmin, kmax]:
//   causal      2*kt+p <= i                               -> kmax = floor((i - p) / 2)
//   document    row >= lo[i] (lo = first row of i's run of equal ids, valid for non-decreasing
//               ids; for arbitrary ids lo = 0 and the ids are compared element by element)
//   window      temporary stream:  tok_i - kt <= w        -> kmin >= tok_i - w
//               persistent stream: only if a persistent window is given, with the key i == j
//               always visible (reference: triton_sps_flash_attention.py:88-108)
// Every prefill kernel and the visibility test hook call row_interval(), so the mask that is
// checked bit-exactly against the CPU oracle is the mask the tensor-core kernel applies.
#pragma once

#include <stdint.h>

namespace spsattn {

struct MaskParams {
  int n_rows;      // N
  int ks;          // rows per token: 2 (SPS modes) or 1 (standard)
  int pp;          // persistent parity 0 / 1, -1 in standard mode
  int w;           // temporary window, clamped to [-1, N] by the host
  int pw;          // persistent window, clamped to [-1, N]
  int has_pw;      // 0: persistent keys are window-exempt
  int flags;       // SPSATTN_FLAG_*
};

// [kmin, kmax] (inclusive; empty when kmax < kmin) for query row i and key stream p.
__host__ __device__ __forceinline__ void row_interval(const MaskParams& m, int i, int lo_i, int p,
                                                      int& kmin, int& kmax) {
  if (i >= m.n_rows) {
    kmin = 0;
    kmax = -1;
    return;
  }
  if (m.ks == 1) {
    kmax = i;
    kmin = lo_i;
    return;
  }
  kmax = (i - p) >> 1;        // floor, -1 when i - p == -1
  kmin = (lo_i - p + 1) >> 1; // ceil((lo - p) / 2), lo - p >= -1
  const int ti = i >> 1;
  if (p == m.pp) {
    if (m.has_pw) {
      if (m.pw >= 0) {
        const int k = ti - m.pw;
        kmin = k > kmin ? k : kmin;
      } else if ((i & 1) == p) {  // only the key i == j survives
        kmin = ti;
        kmax = ti;
      } else {
        kmin = 0;
        kmax = -1;
      }
    }
  } else {
    const int k = ti - m.w;
    kmin = k > kmin ? k : kmin;
    if ((m.flags & SPSATTN_FLAG_PERSISTENT_Q_SKIPS_TEMPORARY) && (i & 1) == m.pp) {
      kmin = 0;
      kmax = -1;
    }
  }
}

// Which rows of [i0, i1] can see stream p at all: rows of every parity (0), or only rows whose
// parity equals `only` (returned through the reference).  Used when planning key tiles.
__host__ __device__ __forceinline__ bool stream_row_filter(const MaskParams& m, int p, int& only) {
  only = -1;
  if (m.ks == 1) return false;
  if (p == m.pp) {
    if (m.has_pw && m.pw < 0) {
      only = p;
      return true;
    }
  } else if (m.flags & SPSATTN_FLAG_PERSISTENT_Q_SKIPS_TEMPORARY) {
    only = 1 - m.pp;
    return true;
  }
  return false;
}

// Key tiles one 128-row query tile has to visit in one stream: tiles of 128 key tokens, the
// first one ending at the last visible token (`top`), going down to the first visible token.
struct StreamPlan {
  int top;       // last key token of tile 0
  int ntiles;    // 0 when nothing is visible
  int kmin_hi;   // largest kmin over the tile's rows
  int kmax_lo;   // smallest kmax over the tile's rows
  int force_mask;
};

__host__ __device__ __forceinline__ StreamPlan plan_stream(const MaskParams& m, int i0, int lo_i0,
                                                           int lo_i1, int p, int tile_keys) {
  StreamPlan sp;
  sp.top = -1;
  sp.ntiles = 0;
  sp.kmin_hi = 0;
  sp.kmax_lo = -1;
  sp.force_mask = 0;
  int i1 = i0 + 127;
  if (i1 > m.n_rows - 1) {
    i1 = m.n_rows - 1;
    sp.force_mask = 1;  // rows past the end must see nothing
  }
  int only;
  int a = i0, b = i1;
  int lo_a = lo_i0, lo_b = lo_i1;
  if (stream_row_filter(m, p, only)) {
    sp.force_mask = 1;
    // lo of a neighbouring row is a valid bound here: it is only used to place tiles, the
    // per-row interval is recomputed from the row's own lo when masking
    if ((a & 1) != only) a += 1;
    if ((b & 1) != only) b -= 1;
    if (a > b) return sp;
    lo_a = lo_i0;
    lo_b = lo_i1;
  }
  int kmin_a, kmax_a, kmin_b, kmax_b;
  row_interval(m, a, lo_a, p, kmin_a, kmax_a);
  row_interval(m, b, lo_b, p, kmin_b, kmax_b);
  int kmin = kmin_a < 0 ? 0 : kmin_a;
  if (kmax_b < kmin) return sp;
  sp.top = kmax_b;
  sp.ntiles = (kmax_b - kmin) / tile_keys + 1;
  sp.kmin_hi = kmin_b;
  sp.kmax_lo = kmax_a;
  return sp;
}

}  // namespace spsattn
