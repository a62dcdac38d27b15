// Segmented decode attention on the tensor cores: the same computation and the same records,
// tickets, merge and cache update as decode.cuh, with the streaming of K and V done by TMA and
// both products by tcgen05.mma, so that almost no instruction is spent per byte of cache.
//
// The CUDA-core kernel needs ~0.13 issued instructions per byte (unpack bf16, FMA, shuffles),
// which at the bandwidth of one SM is three quarters of its issue slots; here a tile of 128 keys
// costs a few hundred instructions whatever the head dim.
//
// One block per (sequence, head, slot); a slot is a chunk of one long segment (chunk_rows keys,
// tiles of 128), or the one slot of the current-token entries and the short segments (a ring of
// a few dozen rows), which the CUDA-core routine of decode.cuh handles.  Per tile:
//   producer warp   TMA: K tile [128 keys x D] and V tile [128 keys x D] -> shared memory, as
//                   units of [128 keys x 64 dims] through one ring (128-byte swizzle)
//   MMA warp        S^T[128 keys x 16]  = K[128 x D] . Qpad[16 x D]^T        (queries padded to 16)
//                   O[64 x D]          += P[64 x 128 keys] . V[128 keys x D]  (rows >= nq of P are 0)
//   4 softmax warps thread t owns key t of the tile: reads its nq scores from TMEM, masks rows
//                   past the live length, block-wide running max (lazy: it moves only when a score
//                   exceeds it by 2^8), p = exp2(s - m), writes p as row q / column t of P
//                   (with two P buffers the softmax of tile j+1 overlaps the product of tile j)
// then row q of O (TMEM lane q) is the accumulator of query q: warp 0 writes the (m, l, acc)
// record and the block joins decode_finish (tickets, merge, cache update).
//
// V rows past the live length may hold anything (the caller's storage, not ours): the owning
// thread zeroes its row in shared memory before the product, so that 0 * garbage cannot make NaN.
// Every wait is bounded (mbar_wait).  Reference computation: decode_attention.py:191-368.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "decode.cuh"

namespace spsattn {

constexpr int kTcThreads = 320;      // 4 softmax warps, 1 producer warp, 1 MMA warp, 4 CUDA-core warps
constexpr int kTcTile = 128;         // keys per tile
constexpr int kTcQPad = 16;          // queries padded to the smallest N of an M = 128 MMA
constexpr float kTcRescaleLog2 = 8.0f;

template <int D>
struct DecodeTcCfg {
  // K and V tiles travel as units of [128 keys x 64 dims] (16 KB, one TMA box, one 128-byte
  // swizzled block the MMA reads as is): a tile is one K unit and one V unit at head_dim 64, two
  // and two at 128, streamed in that order through one ring of units.  A unit is released as
  // soon as the MMAs that read it are done, so the ring stays full whatever the head dim.
  // Two blocks per SM either way (the start-up and the record of one overlap the streaming of
  // the other): ring of 4 units + two P buffers at head_dim 64, 5 units + one P buffer at 128.
  static constexpr int kUnit = kTcTile * 128;
  static constexpr int kUnitsPerOperand = D / 64;
  static constexpr int kUnitsPerTile = 2 * kUnitsPerOperand;
  static constexpr int kRing = D == 64 ? 4 : 5;
  static constexpr int kPBufs = D == 64 ? 2 : 1;
  static constexpr int kQSub = kTcQPad * 128;             // 16 rows x 128 B
  static constexpr int kQBytes = 4096;                    // reserved (D = 128 needs 4096)
  static constexpr int kPRows = 64;                        // M of the second product (nq rows used)
  static constexpr int kPSub = kPRows * 128;               // [64 rows x 64 keys] sub-tile
  static constexpr int kPBuf = 2 * kPSub;                  // one P tile: [64 rows x 128 keys]
  static constexpr int kPBytes = kPBufs * kPBuf;
  static constexpr int kOffQ = 0;
  static constexpr int kOffRing = kQBytes;
  static constexpr int kOffP = kOffRing + kRing * kUnit;
  static constexpr int kOffBar = kOffP + kPBytes;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;  // barriers + alignment slack
  static constexpr int kColS = 0;                          // 2 buffers of 16 columns
  static constexpr int kColO = 32;
  static constexpr uint32_t kTmemCols = D == 64 ? 128 : 256;
};

struct DecodeMaps {
  CUtensorMap k[kMaxSegments];
  CUtensorMap v[kMaxSegments];
};

template <int D, int NQ, bool FP16>
__global__ void __launch_bounds__(kTcThreads, 2)
decode_tc_kernel(const __grid_constant__ DecodeMaps maps, const DecodeParams prm) {
  using Cfg = DecodeTcCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_red[2][4][NQ];
  __shared__ float s_lsum[4][NQ];

  const int sh = blockIdx.x;
  const int s = sh / prm.H, h = sh % prm.H;
  // highest slot first: blocks past the live length retire at once, at the start of the launch
  const int slot = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  int seg_live[kMaxSegments];
  int n_total = 0;
#pragma unroll
  for (int x = 0; x < kMaxSegments; ++x) {
    seg_live[x] = x < prm.n_segments ? live_rows(prm.seg[x], s, h, prm.H) : 0;
    n_total += seg_live[x];
  }
  // the counters as they are before this step's update (any block may be the one that applies it)
  long long ring_len = 0, ring_pos = 0, ret_len = 0;
  if (prm.app.br_len != nullptr) {
    ret_len = prm.app.br_len[(size_t)s * prm.H + h];
    if (prm.app.window_tokens > 0) {
      ring_len = prm.app.nw_len[s];
      ring_pos = prm.app.nw_pos[s];
    }
  }

  // which segment and rows this slot covers
  int seg = -1, row0 = 0, rows = 0;
  {
    int cc = slot;
#pragma unroll
    for (int x = 0; x < kMaxSegments; ++x) {
      if (cc >= 0 && cc < prm.seg_chunks[x]) {
        seg = x;
        row0 = cc * prm.chunk_rows;
        rows = min(prm.chunk_rows, seg_live[x] - row0);
      }
      cc -= prm.seg_chunks[x];
    }
  }
  // one block per (sequence, head): its two records stay in shared memory (decode_finish merges
  // them there); otherwise records go to the workspace and the last block to finish merges
  const bool solo = gridDim.y == 1;
  __shared__ __align__(16) float s_rec[2][NQ][D + 2];
  float* rec = solo ? &s_rec[0][0][0] : prm.partial + ((size_t)sh * prm.n_chunks + slot) * NQ * (D + 2);
  uint32_t local_live = 0;
  bool wrote = false;

  // The current-token entries and the short segments (a ring of a few dozen rows) are not worth
  // a pipeline of their own: the block of slot 0 runs the CUDA-core routine on them with four
  // warps of its own (6..9), beside the tile pipeline, and stores their record in the last
  // record slot.
  const bool small_owner = prm.extras_slot >= 0 && slot == 0;
  auto small_work = [&]() {
    int small_start[kMaxSegments + 1];
    small_start[0] = 0;
#pragma unroll
    for (int x = 0; x < kMaxSegments; ++x)
      small_start[x + 1] = small_start[x] + (((prm.small_segs >> x) & 1u) ? seg_live[x] : 0);
    float* srec = solo ? &s_rec[1][0][0]
                       : prm.partial + ((size_t)sh * prm.n_chunks + prm.extras_slot) * NQ * (D + 2);
    cuda_core_chunk<D, NQ, FP16>(prm, s, h, sh, small_start, 0, small_start[kMaxSegments], prm.n_extras > 0,
                                 srec, tid - 192);
  };

  if (seg >= 0 && rows > 0) {
    // ------------------------------------------------------------ a chunk of one segment
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem_base + Cfg::kOffQ;
    const uint32_t sRing = smem_base + Cfg::kOffRing;
    const uint32_t sP = smem_base + Cfg::kOffP;
    const uint32_t bar0 = smem_base + Cfg::kOffBar;
    const uint32_t bar_full = bar0;            // [kRing] unit landed
    const uint32_t bar_empty = bar0 + 64;      // [kRing] unit consumed
    const uint32_t bar_s_full = bar0 + 128;    // [2]
    const uint32_t bar_s_free = bar0 + 144;    // [2]
    const uint32_t bar_p_full = bar0 + 160;    // [kPBufs]
    const uint32_t bar_pv_done = bar0 + 176;   // [kPBufs]
    const uint32_t bar_red = bar0 + 192;       // [2] block-wide maximum published (4 warp arrivals)
    const int n_tiles = (rows + kTcTile - 1) / kTcTile;
    const uint32_t qmask = prm.seg[seg].query_mask;

    if (tid == 0)
      s_abort = (prm.status != nullptr && *reinterpret_cast<volatile int*>(prm.status) != 0) ? 1 : 0;
    // The nq query rows go into the padded query tile (K-major, 128-byte swizzle: 16-byte chunk ch
    // of row r of a 64-wide sub-tile sits at r * 128 + ((ch ^ (r & 7)) << 4)).  Its other rows,
    // and rows >= nq of P, are left as they are: they only produce score columns and accumulator
    // rows that nobody reads, and an MMA row never mixes with another.
    uint8_t* gen0 = smem_raw + (smem_base - smem_u32(smem_raw));
    if (tid < NQ * (D / 8)) {
      const int r = tid / (D / 8), chunk = tid % (D / 8);
      const int c = chunk / 8, ch = chunk % 8;
      const uint4 u = *reinterpret_cast<const uint4*>(
          reinterpret_cast<const uint16_t*>(prm.q) + (((size_t)s * NQ + r) * prm.H + h) * D + chunk * 8);
      *reinterpret_cast<uint4*>(gen0 + Cfg::kOffQ + c * Cfg::kQSub + r * 128 + ((ch ^ (r & 7)) << 4)) = u;
    }
    fence_proxy_async_smem();
    const int n_units = n_tiles * Cfg::kUnitsPerTile;
    // unit g of the stream: tile g / kUnitsPerTile; first the K units of the tile, then its V units
    auto issue_unit = [&](int g) {
      const int slot = g % Cfg::kRing;
      const int j = g / Cfg::kUnitsPerTile, w = g % Cfg::kUnitsPerTile;
      const bool is_v = w >= Cfg::kUnitsPerOperand;
      const int c = w % Cfg::kUnitsPerOperand;
      if (elect_one()) {
        mbar_arrive_expect_tx(bar_full + 8 * slot, Cfg::kUnit);
        tma_load_4d(sRing + slot * Cfg::kUnit, is_v ? &maps.v[seg] : &maps.k[seg], bar_full + 8 * slot,
                    c * 64, row0 + j * kTcTile, h, s);
      }
      __syncwarp();
    };
    const int n_early = min(Cfg::kRing, n_units);
    if (warp == 4) {
      if (lane == 0) {
        for (int x = 0; x < Cfg::kRing; ++x) {
          mbar_init(bar_full + 8 * x, 1);
          mbar_init(bar_empty + 8 * x, 1);
        }
        for (int x = 0; x < 2; ++x) {
          mbar_init(bar_s_full + 8 * x, 1);
          mbar_init(bar_s_free + 8 * x, 128);
          mbar_init(bar_red + 8 * x, 4);
        }
        for (int x = 0; x < Cfg::kPBufs; ++x) {
          mbar_init(bar_p_full + 8 * x, 128);
          mbar_init(bar_pv_done + 8 * x, 1);
        }
        fence_barrier_init();
        tma_prefetch_desc(&maps.k[seg]);
        tma_prefetch_desc(&maps.v[seg]);
      }
      __syncwarp();
      // the first ring of units is requested before the rest of the block is ready: their round
      // trip to memory overlaps the tensor-memory allocation and the block barrier
      for (int g = 0; g < n_early; ++g) issue_unit(g);
    } else if (warp == 5) {
      tmem_alloc<Cfg::kTmemCols>(smem_u32(&s_tmem_base));
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    volatile int* abort_flag = &s_abort;
    const bool bail = s_abort != 0;

    if (!bail) {
      if (warp == 4) {
        // -------------------------------------------------------------- TMA producer
        for (int g = n_early; g < n_units; ++g) {
          const int slot = g % Cfg::kRing;
          if (!warp_wait(bar_empty + 8 * slot, ((g / Cfg::kRing) - 1) & 1, abort_flag, prm.status)) break;
          issue_unit(g);
        }
      } else if (warp == 5) {
        // -------------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc_s = make_idesc_f16(FP16, 128, kTcQPad, false, false);
        constexpr uint32_t idesc_o = make_idesc_f16(FP16, Cfg::kPRows, 64, false, true);
        const uint64_t dq64 = make_smem_desc_sw128(sQ, 16, 1024);
        const uint64_t dk64 = make_smem_desc_sw128(sRing, 16, 1024);          // unit as K-major A
        const uint64_t dp64 = make_smem_desc_sw128(sP, 16, 1024);
        const uint64_t dv64 = make_smem_desc_sw128(sRing, Cfg::kUnit, 1024);  // unit as MN-major B
        const uint32_t dq_lo = (uint32_t)dq64, dq_hi = (uint32_t)(dq64 >> 32);
        const uint32_t dk_lo = (uint32_t)dk64, dk_hi = (uint32_t)(dk64 >> 32);
        const uint32_t dp_lo = (uint32_t)dp64, dp_hi = (uint32_t)(dp64 >> 32);
        const uint32_t dv_lo = (uint32_t)dv64, dv_hi = (uint32_t)(dv64 >> 32);
        // scores of tile j: one group of four K steps per K unit, each unit released on its own
        auto issue_s = [&](int j) {
          const int sb = j & 1;
          if (j >= 2 && !warp_wait(bar_s_free + 8 * sb, ((j >> 1) - 1) & 1, abort_flag, prm.status))
            return false;
          const uint32_t sd = tmem + Cfg::kColS + sb * kTcQPad;
#pragma unroll
          for (int c = 0; c < Cfg::kUnitsPerOperand; ++c) {
            const int g = j * Cfg::kUnitsPerTile + c, slot = g % Cfg::kRing;
            if (!warp_wait(bar_full + 8 * slot, (g / Cfg::kRing) & 1, abort_flag, prm.status)) return false;
            tc_fence_after();
            const uint32_t ka0 = dk_lo + ((slot * Cfg::kUnit) >> 4);
            const uint32_t qb0 = dq_lo + ((c * Cfg::kQSub) >> 4);
            if (elect_one()) {
              // a K step of 16 elements is 32 bytes inside a 128-byte row
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                if (c == 0 && kk == 0)
                  umma_ss<false>(sd, ka0, dk_hi, qb0, dq_hi, idesc_s);
                else
                  umma_ss<true>(sd, ka0 + ((kk * 32) >> 4), dk_hi, qb0 + ((kk * 32) >> 4), dq_hi, idesc_s);
              }
              umma_commit(bar_empty + 8 * slot);
              if (c == Cfg::kUnitsPerOperand - 1) umma_commit(bar_s_full + 8 * sb);
            }
            __syncwarp();
          }
          return true;
        };
        bool ok = issue_s(0);
        for (int j = 0; ok && j < n_tiles; ++j) {
          if (j + 1 < n_tiles) ok = issue_s(j + 1);
          if (!ok) break;
          const int pb = j % Cfg::kPBufs;
          if (!warp_wait(bar_p_full + 8 * pb, (j / Cfg::kPBufs) & 1, abort_flag, prm.status)) break;
          // output: one 64-column half per V unit, P: K-major, two 64-key sub-tiles; a V unit is
          // MN-major, 16 key rows = 2048 bytes per K step
#pragma unroll
          for (int c = 0; c < Cfg::kUnitsPerOperand; ++c) {
            const int g = j * Cfg::kUnitsPerTile + Cfg::kUnitsPerOperand + c, slot = g % Cfg::kRing;
            if (!warp_wait(bar_full + 8 * slot, (g / Cfg::kRing) & 1, abort_flag, prm.status)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t vb0 = dv_lo + ((slot * Cfg::kUnit) >> 4);
            const uint32_t od = tmem + Cfg::kColO + c * 64;
            if (elect_one()) {
#pragma unroll
              for (int kk = 0; kk < kTcTile / 16; ++kk) {
                const uint32_t pa = (pb * Cfg::kPBuf + (kk / 4) * Cfg::kPSub + (kk % 4) * 32) >> 4;
                if (kk == 0 && j == 0)
                  umma_ss<false>(od, dp_lo + pa, dp_hi, vb0, dv_hi, idesc_o);
                else
                  umma_ss<true>(od, dp_lo + pa, dp_hi, vb0 + ((kk * 2048) >> 4), dv_hi, idesc_o);
              }
              umma_commit(bar_empty + 8 * slot);
              if (c == Cfg::kUnitsPerOperand - 1) umma_commit(bar_pv_done + 8 * pb);
            }
            __syncwarp();
          }
        }
      } else if (warp >= 6) {
        // -------------------------------------------------------------- CUDA-core warps
        if (small_owner) small_work();
      } else {
        // -------------------------------------------------------------- softmax warps
        const int t = tid;                       // key inside the tile = TMEM lane
        const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
        uint8_t* gen = smem_raw + (smem_base - smem_u32(smem_raw));
        float m_run[NQ], l_part[NQ];
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          m_run[qi] = -1.0e30f;
          l_part[qi] = 0.f;
        }
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
          const int sb = j & 1;
          if (!mbar_wait(bar_s_full + 8 * sb, (j >> 1) & 1, abort_flag, prm.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t r0, r1;
          tmem_ld2(tmem + lane_addr + Cfg::kColS + sb * kTcQPad, r0, r1);
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive(bar_s_free + 8 * sb);
          const bool valid = j * kTcTile + t < rows;
          float sc[NQ];
          sc[0] = (valid && (qmask & 1u)) ? __uint_as_float(r0) * prm.scale_log2 : -INFINITY;
          if (NQ > 1) sc[NQ - 1] = (valid && (qmask & 2u)) ? __uint_as_float(r1) * prm.scale_log2 : -INFINITY;
          // block-wide maximum of this tile's scores, per query
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi) {
            float mx = sc[qi];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (lane == 0) s_red[sb][warp][qi] = mx;
          }
          // the four warps exchange their maxima through an mbarrier (a bounded wait like every
          // other one here; a plain named barrier could strand threads after a failed wait)
          if (lane == 0) mbar_arrive(bar_red + 8 * sb);
          if (!mbar_wait(bar_red + 8 * sb, (j >> 1) & 1, abort_flag, prm.status)) {
            ok = false;
            break;
          }
          float alpha[NQ];
          bool rescale = false;
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi) {
            const float mx = fmaxf(fmaxf(s_red[sb][0][qi], s_red[sb][1][qi]),
                                   fmaxf(s_red[sb][2][qi], s_red[sb][3][qi]));
            alpha[qi] = 1.f;
            // lazy: the reference point moves only when a score exceeds it by 2^kTcRescaleLog2
            if (mx - m_run[qi] > kTcRescaleLog2) {
              alpha[qi] = fast_exp2(m_run[qi] - mx);
              m_run[qi] = mx;
              rescale = true;
            }
          }
          // p is rounded to the operand type first and the rounded value is what the row sum
          // adds, so that numerator and denominator weigh every key identically
          uint32_t pbits[NQ];
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi) {
            pbits[qi] = pack2<FP16>(fast_exp2(sc[qi] - m_run[qi]), 0.f) & 0xffffu;
            float pr, unused;
            unpack2<FP16>(pbits[qi], pr, unused);
            l_part[qi] = l_part[qi] * alpha[qi] + pr;
          }
          const int pb = j % Cfg::kPBufs;
          if (j >= Cfg::kPBufs) {   // this P buffer is free once the product that last read it is done
            if (!mbar_wait(bar_pv_done + 8 * pb, ((j / Cfg::kPBufs) - 1) & 1, abort_flag, prm.status)) {
              ok = false;
              break;
            }
          }
          if (rescale && j > 0) {
            // O must be at rest: wait for the product of tile j - 1, then lane q of warp 0 scales
            // row q (rows q < nq of O live in TMEM lanes q; the others hold zeros)
            if (!mbar_wait(bar_pv_done + 8 * ((j - 1) % Cfg::kPBufs), ((j - 1) / Cfg::kPBufs) & 1, abort_flag,
                           prm.status)) {
              ok = false;
              break;
            }
            tc_fence_after();
            if (warp == 0) {
              const float a = lane == 0 ? alpha[0] : (lane < NQ ? alpha[NQ - 1] : 1.f);
#pragma unroll
              for (int q4 = 0; q4 < D / 32; ++q4) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_addr + Cfg::kColO + q4 * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * a);
                tmem_st32(tmem + lane_addr + Cfg::kColO + q4 * 32, r);
              }
              tmem_wait_st();
            }
          }
          // p -> row q, column t of P (K-major, 128-byte swizzle, two 64-key sub-tiles)
          {
            const int c = t >> 6, ch = (t & 63) >> 3;
#pragma unroll
            for (int qi = 0; qi < NQ; ++qi) {
              const uint32_t off = Cfg::kOffP + pb * Cfg::kPBuf + c * Cfg::kPSub + qi * 128 +
                                   ((ch ^ (qi & 7)) << 4) + (t & 7) * 2;
              *reinterpret_cast<uint16_t*>(gen + off) = (uint16_t)pbits[qi];
            }
          }
          if ((j + 1) * kTcTile > rows) {
            // last tile of the chunk: rows past the live length must not reach the product
#pragma unroll
            for (int c = 0; c < Cfg::kUnitsPerOperand; ++c) {
              const int g = j * Cfg::kUnitsPerTile + Cfg::kUnitsPerOperand + c, slot = g % Cfg::kRing;
              if (!mbar_wait(bar_full + 8 * slot, (g / Cfg::kRing) & 1, abort_flag, prm.status)) ok = false;
              if (ok && !valid) {
                uint4* vrow = reinterpret_cast<uint4*>(gen + Cfg::kOffRing + slot * Cfg::kUnit + t * 128);
#pragma unroll
                for (int x = 0; x < 8; ++x) vrow[x] = make_uint4(0, 0, 0, 0);
              }
            }
            if (!ok) break;
          }
          fence_proxy_async_smem();
          tc_fence_before();
          mbar_arrive(bar_p_full + 8 * pb);
        }
        // ------------------------------------------------------------ record of this chunk
        if (ok)
          ok = mbar_wait(bar_pv_done + 8 * ((n_tiles - 1) % Cfg::kPBufs), ((n_tiles - 1) / Cfg::kPBufs) & 1,
                         abort_flag, prm.status);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi) {
            float l = l_part[qi];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            if (lane == 0) s_lsum[warp][qi] = l;
          }
          if (lane == 0) mbar_arrive(bar_red + 8 * (n_tiles & 1));
          ok = mbar_wait(bar_red + 8 * (n_tiles & 1), (n_tiles >> 1) & 1, abort_flag, prm.status);
          if (ok && warp == 0) {
#pragma unroll
            for (int q4 = 0; q4 < D / 32; ++q4) {
              uint32_t r[32];
              tmem_ld32(tmem + lane_addr + Cfg::kColO + q4 * 32, r);
              tmem_wait_ld();
              if (lane < NQ) {
                float* dst = rec + lane * (D + 2) + 2 + q4 * 32;
#pragma unroll
                for (int e = 0; e < 32; e += 2)
                  *reinterpret_cast<float2*>(dst + e) =
                      make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
              }
            }
            if (lane < NQ) {
              rec[lane * (D + 2)] = lane == 0 ? m_run[0] : m_run[NQ - 1];
              rec[lane * (D + 2) + 1] = s_lsum[0][lane] + s_lsum[1][lane] + s_lsum[2][lane] + s_lsum[3][lane];
            }
          }
        }
      }
    }
    if (bail && warp == 4) {
      // nothing will consume the units requested early: let them land before the block goes
      for (int g = 0; g < n_early; ++g)
        if (!warp_wait(bar_full + 8 * (g % Cfg::kRing), 0, abort_flag, nullptr)) break;
    }
    // common teardown: every role arrives here, also after a failed wait
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
      tc_fence_after();
      tmem_dealloc<Cfg::kTmemCols>(tmem);
    }
    wrote = true;
    if (bail && small_owner && warp >= 6) small_work();
  } else if (small_owner) {
    if (warp >= 6) small_work();
    wrote = true;
  }

  if (prm.tickets == nullptr) return;
  if (seg >= 0 && rows > 0) local_live |= 1u;
  if (small_owner) local_live |= 2u;
  decode_finish<D, NQ, FP16, true>(prm, sh, s, h, n_total, seg_live, ring_len, ring_pos, ret_len, wrote, tid,
                                   kTcThreads, solo ? &s_rec[0][0][0] : nullptr, local_live);
}

}  // namespace spsattn
