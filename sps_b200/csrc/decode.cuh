// Segmented decode attention: nq (1 or 2) queries per (sequence, head) over up to three
// length-masked KV segments plus up to two single-token "current" entries.
//
// The job is bandwidth bound (every live K/V row is read exactly once, both queries share the
// load), so it is split-K: the live rows of one (sequence, head) — the segments laid end to
// end — are cut into chunks of `chunk_rows`, one block per chunk.  A block streams its rows with
// 128-bit loads (D/8 lanes per row, four row batches in flight per lane), keeps an online
// softmax per lane group in fp32, merges the groups and writes one (max, sum, acc[D]) record
// per query into the workspace; a second small kernel merges the records of each
// (sequence, head) and writes the output (fp32, or 16-bit for a caller that feeds a projection).
// Lengths are read on the device, so the grid is sized from the host-side caps and blocks past
// the live length return at once.
// The decode-step form is a single launch: every block of a (sequence, head) takes a ticket when
// it is done and the last one merges the records itself, and (when asked) also performs the step's
// cache update for its (sequence, head) — ring insert, retained append, counters.  By then every
// block of that (sequence, head) has read the counters and finished reading the rows, which is
// what makes the in-place update safe; the per-sequence ring counters are advanced by the last
// (sequence, head) of the sequence to finish, through a second ticket.  Nothing waits on a ticket.
// Reference computation: src/modeling/models/utils/decode_attention.py:191-368 and, for the
// update, src/modeling/models/utils/decode_attention_fast.py:34-136.
#pragma once

#include "common.cuh"

namespace spsattn {

constexpr int kMaxSegments = 3;
constexpr int kMaxExtras = 2;
constexpr int kDecodeThreads = 128;
constexpr int kDecodeUnroll = 4;

struct DecodeSeg {
  const void* k;
  const void* v;
  const int64_t* seq_offset;
  int64_t seq_stride, head_stride, row_stride;
  const int64_t* lengths;
  int lengths_per_head;
  int max_rows;
  uint32_t query_mask;
};

// The cache update folded into the merge kernel (all pointers null = no update).
struct DecodeAppend {
  uint16_t* nw_k;            // ring      [S, H, window_storage, D]
  uint16_t* nw_v;
  int64_t* nw_len;           // [S]
  int64_t* nw_pos;           // [S]
  uint16_t* br_k;            // retained  [S, H, retained_storage, D]
  uint16_t* br_v;
  int64_t* br_len;           // [S, H]
  const uint16_t* k_window;  // [S, H, D]
  const uint16_t* v_window;
  const uint16_t* k_retained;
  const uint16_t* v_retained;
  const int8_t* active;      // [S]
  int window_storage, retained_storage, window_tokens;
};

struct DecodeParams {
  const void* q;       // [S, nq, H, D]
  void* out;           // [S, nq, H, D] fp32, or 16-bit in the queries' format when out16 is set
  int out16;
  float* partial;      // [S*H][n_chunks][nq][D + 2]
  int* tickets;        // [S*H + S] zero before the first launch, left zero; null = separate merge launch
  // Tensor-core kernel only: records are indexed by slot = (segment, chunk inside the segment),
  // segment after segment, then one slot for the current-token entries.
  int seg_chunks[kMaxSegments];   // 0 for the short segments of small_segs
  int extras_slot;     // slot of the current-token entries and the short segments, -1 when none
  uint32_t small_segs; // bit x: segment x is short and handled with the entries, on the CUDA cores
  int* status;         // bounded-wait failures are reported here (may be null)
  DecodeAppend app;
  DecodeSeg seg[kMaxSegments];
  const void* extra_k[kMaxExtras];
  const void* extra_v[kMaxExtras];
  uint32_t extra_mask[kMaxExtras];
  int n_segments, n_extras;
  int S, H, nq;
  int chunk_rows, n_chunks;
  float scale_log2;
};

__device__ __forceinline__ int live_rows(const DecodeSeg& sg, int s, int h, int H) {
  long long len = sg.lengths_per_head ? sg.lengths[(size_t)s * H + h] : sg.lengths[s];
  if (len < 0) len = 0;
  return len < sg.max_rows ? (int)len : sg.max_rows;
}

// Merge the chunk records of one (sequence, head) and write its outputs; `nthreads` threads of
// one block cooperate.  Records are read past L1 (other blocks may have written them), eight
// chunks at a time with all their loads in flight together, so a merge costs about one round
// trip to L2 instead of one per chunk.
template <int D, int NQ, bool FP16>
__device__ __forceinline__ void merge_records(const DecodeParams& prm, int sh, int s, int h, int n_total,
                                              int tid, int nthreads) {
  constexpr int G = 8;
  int n_chunks = (n_total + prm.chunk_rows - 1) / prm.chunk_rows;
  if (n_chunks < 1) n_chunks = 1;
  for (int idx = tid; idx < NQ * D; idx += nthreads) {
    const int qi = idx / D, d = idx % D;
    const float* rec0 = prm.partial + (size_t)sh * prm.n_chunks * NQ * (D + 2) + qi * (D + 2);
    float m_run = -1.0e30f, l_run = 0.f, a_run = 0.f;
    for (int c0 = 0; c0 < n_chunks; c0 += G) {
      float m[G], l[G], a[G];
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const int c = min(c0 + j, n_chunks - 1);      // clamped: the tail repeats a valid record
        const float* rec = rec0 + (size_t)c * NQ * (D + 2);
        m[j] = __ldcg(rec);
        l[j] = __ldcg(rec + 1);
        a[j] = __ldcg(rec + 2 + d);
      }
      float mx = m_run;
#pragma unroll
      for (int j = 0; j < G; ++j) mx = fmaxf(mx, m[j]);
      const float keep = fast_exp2(m_run - mx);
      l_run *= keep;
      a_run *= keep;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const float f = c0 + j < n_chunks ? fast_exp2(m[j] - mx) : 0.f;
        l_run = fmaf(l[j], f, l_run);
        a_run = fmaf(a[j], f, a_run);
      }
      m_run = mx;
    }
    const float o = l_run > 0.f ? a_run / l_run : 0.f;
    const size_t off = (((size_t)s * NQ + qi) * prm.H + h) * D + d;
    if (prm.out16)
      reinterpret_cast<uint16_t*>(prm.out)[off] = (uint16_t)(pack2<FP16>(o, 0.f) & 0xffffu);
    else
      reinterpret_cast<float*>(prm.out)[off] = o;
  }
}

// The same merge for the slot layout of the tensor-core kernel: a slot holds a record iff its
// chunk starts below the live length of its segment (the slot of the current-token entries and
// the short segments always does).  `seg_live[x]` = live rows of segment x.
template <int D, int NQ, bool FP16>
__device__ __forceinline__ void merge_slots(const DecodeParams& prm, int sh, int s, int h,
                                            const int (&seg_live)[kMaxSegments], int tid, int nthreads) {
  constexpr int G = 8;
  const int n_slots = prm.n_chunks;
  for (int idx = tid; idx < NQ * D; idx += nthreads) {
    const int qi = idx / D, d = idx % D;
    const float* rec0 = prm.partial + (size_t)sh * prm.n_chunks * NQ * (D + 2) + qi * (D + 2);
    float m_run = -1.0e30f, l_run = 0.f, a_run = 0.f;
    for (int c0 = 0; c0 < n_slots; c0 += G) {
      float m[G], l[G], a[G];
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const int c = c0 + j;
        bool live = false;
        if (c < n_slots) {
          if (c == prm.extras_slot) {
            live = true;
          } else {
            int cc = c;
#pragma unroll
            for (int x = 0; x < kMaxSegments; ++x) {
              if (cc >= 0 && cc < prm.seg_chunks[x]) live = cc * prm.chunk_rows < seg_live[x];
              cc -= prm.seg_chunks[x];
            }
          }
        }
        const float* rec = rec0 + (size_t)(live ? c : 0) * NQ * (D + 2);
        m[j] = live ? __ldcg(rec) : -1.0e30f;
        l[j] = live ? __ldcg(rec + 1) : 0.f;
        a[j] = live ? __ldcg(rec + 2 + d) : 0.f;
      }
      float mx = m_run;
#pragma unroll
      for (int j = 0; j < G; ++j) mx = fmaxf(mx, m[j]);
      const float keep = fast_exp2(m_run - mx);
      l_run *= keep;
      a_run *= keep;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const float f = fast_exp2(m[j] - mx);
        l_run = fmaf(l[j], f, l_run);
        a_run = fmaf(a[j], f, a_run);
      }
      m_run = mx;
    }
    const float o = l_run > 0.f ? a_run / l_run : 0.f;
    const size_t off = (((size_t)s * NQ + qi) * prm.H + h) * D + d;
    if (prm.out16)
      reinterpret_cast<uint16_t*>(prm.out)[off] = (uint16_t)(pack2<FP16>(o, 0.f) & 0xffffu);
    else
      reinterpret_cast<float*>(prm.out)[off] = o;
  }
}

// End of a block of a single-launch decode: take the ticket of this (sequence, head); the last
// block to arrive merges the records, writes the output and applies the cache update.  Every
// block takes a ticket, also those past the live length, so that all of them have read the
// counters before any update.  `wrote` = this block stored a record (its stores are fenced).
// `local` (tensor-core kernel, one block per (sequence, head)): the block's two records — its
// tiles and the short segments / current entries — are in shared memory at `local`; there is
// nobody to take a ticket against, and the merge needs no trip through global memory.
template <int D, int NQ, bool FP16, bool SLOTS>
__device__ __forceinline__ void decode_finish(const DecodeParams& prm, int sh, int s, int h, int n_total,
                                              const int (&seg_live)[kMaxSegments], long long ring_len,
                                              long long ring_pos, long long ret_len, bool wrote, int tid,
                                              int nthreads, const float* local = nullptr,
                                              uint32_t local_live = 0) {
  if (local != nullptr) {
    __syncthreads();
    for (int idx = tid; idx < NQ * D; idx += nthreads) {
      const int qi = idx / D, d = idx % D;
      float m[2], l[2], a[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float* rec = local + (c * NQ + qi) * (D + 2);
        const bool live = (local_live >> c) & 1u;
        m[c] = live ? rec[0] : -1.0e30f;
        l[c] = live ? rec[1] : 0.f;
        a[c] = live ? rec[2 + d] : 0.f;
      }
      const float mx = fmaxf(m[0], m[1]);
      const float f0 = fast_exp2(m[0] - mx), f1 = fast_exp2(m[1] - mx);
      const float lsum = l[0] * f0 + l[1] * f1, asum = a[0] * f0 + a[1] * f1;
      const float o = lsum > 0.f ? asum / lsum : 0.f;
      const size_t off = (((size_t)s * NQ + qi) * prm.H + h) * D + d;
      if (prm.out16)
        reinterpret_cast<uint16_t*>(prm.out)[off] = (uint16_t)(pack2<FP16>(o, 0.f) & 0xffffu);
      else
        reinterpret_cast<float*>(prm.out)[off] = o;
    }
  } else {
    // (the barrier orders the block's record stores before thread 0's fence, which is cumulative)
    if (wrote) __syncthreads();
    __shared__ int s_last;
    if (tid == 0) {
      if (wrote) __threadfence();
      const bool last = atomicAdd(&prm.tickets[sh], 1) == (int)gridDim.y - 1;
      if (last) __threadfence();
      s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    if constexpr (SLOTS)
      merge_slots<D, NQ, FP16>(prm, sh, s, h, seg_live, tid, nthreads);
    else
      merge_records<D, NQ, FP16>(prm, sh, s, h, n_total, tid, nthreads);
  }
  const DecodeAppend& ap = prm.app;
  const bool append = ap.br_k != nullptr && ap.active[s] != 0;
  const bool full = ring_len >= ap.window_tokens;
  if (append) {
    const long long ins = full ? ring_pos : ring_len;
    for (int d = tid; d < D; d += nthreads) {
      const size_t src = (size_t)sh * D + d;
      if (ap.window_tokens > 0 && ins >= 0 && ins < ap.window_storage) {
        const size_t dst = ((size_t)sh * ap.window_storage + (size_t)ins) * D + d;
        ap.nw_k[dst] = ap.k_window[src];
        ap.nw_v[dst] = ap.v_window[src];
      }
      if (ret_len >= 0 && ret_len < ap.retained_storage) {
        const size_t dst = ((size_t)sh * ap.retained_storage + (size_t)ret_len) * D + d;
        ap.br_k[dst] = ap.k_retained[src];
        ap.br_v[dst] = ap.v_retained[src];
      }
    }
  }
  if (tid == 0) {
    if (local == nullptr) prm.tickets[sh] = 0;   // ready for the next launch
    if (append && ret_len < ap.retained_storage) ap.br_len[sh] = ret_len + 1;
    if (ap.br_k != nullptr && ap.window_tokens > 0) {
      // the ring counters belong to the sequence: the last of its heads to get here advances them
      __threadfence();
      int* seq_ticket = prm.tickets + (size_t)prm.S * prm.H + s;
      if (atomicAdd(seq_ticket, 1) == prm.H - 1) {
        *seq_ticket = 0;
        if (append) {
          if (full)
            ap.nw_pos[s] = (ring_pos + 1) % ap.window_tokens;
          else
            ap.nw_len[s] = ring_len + 1;
        }
      }
    }
  }
}

// The CUDA-core pass over rows [c_lo, c_hi) of the segments laid end to end (`seg_start` =
// running sum of their live rows), plus the current-token entries when asked, ending in one
// record per query at `rec`.  Run by the first kDecodeThreads threads of the block, all of which
// must call it (it synchronises them on named barrier 2; the other threads stay out).
template <int D, int NQ, bool FP16>
__device__ __forceinline__ void cuda_core_chunk(const DecodeParams& prm, int s, int h, int sh,
                                                const int (&seg_start)[kMaxSegments + 1], int c_lo, int c_hi,
                                                bool with_extras, float* rec, int tid) {
  constexpr int LPR = D / 8;          // lanes per row
  constexpr int RPI = 32 / LPR;       // rows per warp load instruction
  constexpr int U = kDecodeUnroll;
  constexpr int STEP = 4 * RPI * U;   // rows per block step
  static_assert(D % 8 == 0 && 32 % LPR == 0, "head_dim");
  const int warp = (tid >> 5) & 3, lane = tid & 31;
  const int g = lane / LPR;           // row inside a load instruction
  const int dl = (lane % LPR) * 8;    // first of this lane's 8 dims
  const bool worker = tid < kDecodeThreads;
  __shared__ float s_m[4][NQ], s_l[4][NQ], s_acc[4][NQ][D];
  if (worker) {
    if (with_extras && warp == 0 && lane < 2 * prm.n_extras) {
      // the single-row entries are read last, by one warp: have them in L2 by then
      const void* base = (lane & 1) ? prm.extra_v[lane >> 1] : prm.extra_k[lane >> 1];
      asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint16_t*>(base) + (size_t)sh * D));
    }
    // queries, pre-scaled so scores are in the log2 domain
    float q[NQ][8];
#pragma unroll
    for (int qi = 0; qi < NQ; ++qi) {
      const uint4 u = *reinterpret_cast<const uint4*>(
          reinterpret_cast<const uint16_t*>(prm.q) + (((size_t)s * NQ + qi) * prm.H + h) * D + dl);
      unpack2<FP16>(u.x, q[qi][0], q[qi][1]);
      unpack2<FP16>(u.y, q[qi][2], q[qi][3]);
      unpack2<FP16>(u.z, q[qi][4], q[qi][5]);
      unpack2<FP16>(u.w, q[qi][6], q[qi][7]);
#pragma unroll
      for (int x = 0; x < 8; ++x) q[qi][x] *= prm.scale_log2;
    }

    float m_run[NQ], l_run[NQ], acc[NQ][8];
#pragma unroll
    for (int qi = 0; qi < NQ; ++qi) {
      m_run[qi] = -1.0e30f;
      l_run[qi] = 0.f;
#pragma unroll
      for (int x = 0; x < 8; ++x) acc[qi][x] = 0.f;
    }

    // one batch of U rows (one per unroll slot) for this lane group
    auto process = [&](const uint16_t* kb, const uint16_t* vb, int64_t row_stride, int r0, int r_hi,
                       uint32_t qmask) {
      uint4 kr[U], vr[U];
      bool valid[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = r0 + u * (4 * RPI);
        valid[u] = r < r_hi;
        if (valid[u]) {
          kr[u] = __ldg(reinterpret_cast<const uint4*>(kb + (size_t)r * row_stride + dl));
          vr[u] = __ldg(reinterpret_cast<const uint4*>(vb + (size_t)r * row_stride + dl));
        } else {
          kr[u] = make_uint4(0, 0, 0, 0);
          vr[u] = make_uint4(0, 0, 0, 0);
        }
      }
      float sc[NQ][U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float kf[8];
        unpack2<FP16>(kr[u].x, kf[0], kf[1]);
        unpack2<FP16>(kr[u].y, kf[2], kf[3]);
        unpack2<FP16>(kr[u].z, kf[4], kf[5]);
        unpack2<FP16>(kr[u].w, kf[6], kf[7]);
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          float d = 0.f;
#pragma unroll
          for (int x = 0; x < 8; ++x) d = fmaf(q[qi][x], kf[x], d);
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          sc[qi][u] = (valid[u] && ((qmask >> qi) & 1u)) ? d : -INFINITY;
        }
      }
      float pr[NQ][U], alpha[NQ];
#pragma unroll
      for (int qi = 0; qi < NQ; ++qi) {
        float mx = m_run[qi];
#pragma unroll
        for (int u = 0; u < U; ++u) mx = fmaxf(mx, sc[qi][u]);
        alpha[qi] = fast_exp2(m_run[qi] - mx);
        float sum = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          pr[qi][u] = fast_exp2(sc[qi][u] - mx);
          sum += pr[qi][u];
        }
        l_run[qi] = l_run[qi] * alpha[qi] + sum;
        m_run[qi] = mx;
#pragma unroll
        for (int x = 0; x < 8; ++x) acc[qi][x] *= alpha[qi];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float vf[8];
        unpack2<FP16>(vr[u].x, vf[0], vf[1]);
        unpack2<FP16>(vr[u].y, vf[2], vf[3]);
        unpack2<FP16>(vr[u].z, vf[4], vf[5]);
        unpack2<FP16>(vr[u].w, vf[6], vf[7]);
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi)
#pragma unroll
          for (int x = 0; x < 8; ++x) acc[qi][x] = fmaf(pr[qi][u], vf[x], acc[qi][x]);
      }
    };

#pragma unroll
    for (int x = 0; x < kMaxSegments; ++x) {
      if (x >= prm.n_segments) break;
      const int lo = max(c_lo, seg_start[x]) - seg_start[x];
      const int hi = min(c_hi, seg_start[x + 1]) - seg_start[x];
      if (lo >= hi) continue;
      const DecodeSeg& sg = prm.seg[x];
      const int64_t base = (sg.seq_offset ? sg.seq_offset[s] : (int64_t)s * sg.seq_stride) +
                           (int64_t)h * sg.head_stride;
      const uint16_t* kb = reinterpret_cast<const uint16_t*>(sg.k) + base;
      const uint16_t* vb = reinterpret_cast<const uint16_t*>(sg.v) + base;
      for (int r = lo + warp * RPI + g; r - (warp * RPI + g) < hi; r += STEP)
        process(kb, vb, sg.row_stride, r, hi, sg.query_mask);
    }
    if (with_extras && warp == 0) {
      // the current-token entries: one row each, handled by lane group 0 of warp 0
      for (int e = 0; e < prm.n_extras; ++e) {
        const uint16_t* kb = reinterpret_cast<const uint16_t*>(prm.extra_k[e]) + (size_t)sh * D;
        const uint16_t* vb = reinterpret_cast<const uint16_t*>(prm.extra_v[e]) + (size_t)sh * D;
        process(kb, vb, 0, g, 1, prm.extra_mask[e]);
      }
    }

    // merge the lane groups of a warp, then the four warps, then write the record
#pragma unroll
    for (int qi = 0; qi < NQ; ++qi) {
#pragma unroll
      for (int o = LPR; o < 32; o <<= 1) {
        const float m_o = __shfl_xor_sync(0xffffffffu, m_run[qi], o);
        const float l_o = __shfl_xor_sync(0xffffffffu, l_run[qi], o);
        const float mx = fmaxf(m_run[qi], m_o);
        const float a = fast_exp2(m_run[qi] - mx), bsc = fast_exp2(m_o - mx);
        l_run[qi] = l_run[qi] * a + l_o * bsc;
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const float acc_o = __shfl_xor_sync(0xffffffffu, acc[qi][x], o);
          acc[qi][x] = acc[qi][x] * a + acc_o * bsc;
        }
        m_run[qi] = mx;
      }
    }
    if (g == 0) {
#pragma unroll
      for (int qi = 0; qi < NQ; ++qi) {
        if (lane == 0) {
          s_m[warp][qi] = m_run[qi];
          s_l[warp][qi] = l_run[qi];
        }
#pragma unroll
        for (int x = 0; x < 8; ++x) s_acc[warp][qi][dl + x] = acc[qi][x];
      }
    }
  }
  if (worker) asm volatile("bar.sync 2, %0;" ::"n"(kDecodeThreads) : "memory");
  if (worker) {
    for (int idx = tid; idx < NQ * D; idx += kDecodeThreads) {
      const int qi = idx / D, d = idx % D;
      float mx = s_m[0][qi];
#pragma unroll
      for (int w = 1; w < 4; ++w) mx = fmaxf(mx, s_m[w][qi]);
      float a = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = fast_exp2(s_m[w][qi] - mx);
        a += s_acc[w][qi][d] * f;
        l += s_l[w][qi] * f;
      }
      rec[qi * (D + 2) + 2 + d] = a;
      if (d == 0) {
        rec[qi * (D + 2)] = mx;
        rec[qi * (D + 2) + 1] = l;
      }
    }
  }
}

template <int D, int NQ, bool FP16>
__global__ void __launch_bounds__(kDecodeThreads, 5)
decode_split_kernel(const DecodeParams prm) {
  const int sh = blockIdx.x;
  const int s = sh / prm.H, h = sh % prm.H;
  // highest chunk first: blocks past the live length retire at once, at the start of the launch
  const int chunk = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int tid = threadIdx.x;

  int seg_start[kMaxSegments + 1];
  seg_start[0] = 0;
#pragma unroll
  for (int x = 0; x < kMaxSegments; ++x)
    seg_start[x + 1] = seg_start[x] + (x < prm.n_segments ? live_rows(prm.seg[x], s, h, prm.H) : 0);
  const int n_total = seg_start[kMaxSegments];
  const int c_lo = chunk * prm.chunk_rows;
  const bool dead = chunk > 0 && c_lo >= n_total;
  if (dead && prm.tickets == nullptr) return;
  const int c_hi = min(c_lo + prm.chunk_rows, n_total);
  // the counters as they are before this step's update (any block may be the one that applies it)
  long long ring_len = 0, ring_pos = 0, ret_len = 0;
  if (prm.app.br_len != nullptr) {
    ret_len = prm.app.br_len[(size_t)s * prm.H + h];
    if (prm.app.window_tokens > 0) {
      ring_len = prm.app.nw_len[s];
      ring_pos = prm.app.nw_pos[s];
    }
  }

  if (!dead) {   // blocks past the live length only take their ticket below
    float* rec = prm.partial + ((size_t)sh * prm.n_chunks + chunk) * NQ * (D + 2);
    cuda_core_chunk<D, NQ, FP16>(prm, s, h, sh, seg_start, c_lo, c_hi, chunk == 0, rec, tid);
  }

  if (prm.tickets == nullptr) return;     // a separate launch merges
  int seg_live[kMaxSegments];
#pragma unroll
  for (int x = 0; x < kMaxSegments; ++x) seg_live[x] = seg_start[x + 1] - seg_start[x];
  decode_finish<D, NQ, FP16, false>(prm, sh, s, h, n_total, seg_live, ring_len, ring_pos, ret_len, !dead,
                                    tid, kDecodeThreads);
}

// Separate merge launch for callers whose workspace carries no tickets: one block of D threads
// per (sequence, head).
template <int D, int NQ, bool FP16>
__global__ void __launch_bounds__(D)
decode_merge_kernel(const DecodeParams prm) {
  const int sh = blockIdx.x;
  const int s = sh / prm.H, h = sh % prm.H;
  int n_total = 0;
  for (int x = 0; x < prm.n_segments; ++x) n_total += live_rows(prm.seg[x], s, h, prm.H);
  merge_records<D, NQ, FP16>(prm, sh, s, h, n_total, threadIdx.x, D);
}

}  // namespace spsattn
