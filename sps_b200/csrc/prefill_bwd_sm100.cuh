// Backward of the SPS prefill attention for sm_100a: dQ, dK, dV from dO, with the probabilities
// recomputed from the saved log-sum-exp (no [N, N] tensor is ever stored).
//
// Three launches, like the reference's backward (src/modeling/models/attention/
// triton_sps_flash_attention.py:623-720: `_attn_bwd_preprocess`, `_sps_bwd_dkdv_kernel`,
// `_sps_bwd_dq_kernel`):
//   delta_kernel      delta[i] = sum_d dO[i,d] * O[i,d]
//   bwd kernel, kDQ   one block per 128-row query tile; streams the key tiles the forward
//                     kernel visits for that tile:  dQ += dS K
//   bwd kernel, kDKV  one block per 128-token key tile of one parity stream; streams the 64-row
//                     query tiles that can see it:  dV += P^T dO,  dK += dS^T Q
// Both modes are the same pipeline with the operands renamed.  With X the stationary pair of
// 128-row tiles and Y the streamed pair of 64-row tiles:
//   S  = X0 Y0^T   (Q K^T, or its transpose K Q^T)        tcgen05.mma 128x64xD into TMEM
//   dP = X1 Y1^T   (dO V^T, or V dO^T)                    tcgen05.mma 128x64xD into TMEM
//   P  = exp2(S * scale*log2e - lse),  dS = P * (dP - delta) * scale     softmax warps, registers
//   acc0 += dS Y0  (dQ += dS K,  or dK += dS^T Q)         tcgen05.mma 128xDx64, Y as MN-major B
//   acc1 += P  Y1  (kDKV only: dV += P^T dO)
// P and dS are written back to tensor memory (packed 16-bit pairs over the S / dP columns already
// read) and enter the accumulating MMAs as their A operand from there; shared memory only holds
// the operand tiles delivered by TMA.  Head_dim 64: four softmax warps, two blocks per SM; head_dim
// 128: two softmax warpgroups taking alternate tiles, one block per SM with all 512 columns.
// The visibility rule is the forward's: every mask bit comes from row_interval().
#pragma once

#include "common.cuh"
#include "mask.cuh"
#include "prefill_sm100.cuh"

namespace spsattn {

constexpr int kBwdDQ = 0;
constexpr int kBwdDKV = 1;
constexpr int kBwdMaxThreads = 320;
constexpr int kBwdTable = 1024;      // streamed tiles listed per block (64K rows in kDKV mode)

struct BwdParams {
  void* out0;            // kDQ: dQ, kDKV: dK   rows of D contiguous elements, strides below
  void* out1;            // kDKV: dV
  int64_t out0_stride[3], out1_stride[3];       // batch, head, row (elements)
  const float* lse;      // [B, H, N], log2 domain (as written by the forward kernel)
  const float* delta;    // [B, H, N]
  const void* docs;
  int64_t doc_stride_b, doc_stride_t;
  int doc_is_i64;
  const int* lo;
  const int* hi;         // [B, N] last row of the run of equal ids containing the row (with lo)
  const int* mono;
  int B, H, N;
  int n_xtiles;          // stationary tiles per (batch, head)
  int group_heads;       // (batch, head) pairs whose operands share L2 at a time
  MaskParams mask;
  float scale_log2;
  float sm_scale;
  int* status;
};

template <int D, int MODE>
struct BwdCfg {
  // ring of streamed tile pairs: four stages at head_dim 128 (P / dS live in tensor memory there,
  // see kPTmem), so that the loads run ahead of the two warpgroups
  static constexpr int kStages = 4;
  static constexpr int kXBytes = 128 * D * 2;
  static constexpr int kXSub = 128 * 128;
  static constexpr int kYBytes = 64 * D * 2;
  static constexpr int kYSub = 64 * 128;
  static constexpr int kPBytes = 128 * 64 * 2;
  static constexpr int kOffX0 = 0;
  static constexpr int kOffX1 = kXBytes;
  static constexpr int kOffY = 2 * kXBytes;                    // [stage][Y0 | Y1]
  static constexpr int kOffP = kOffY + kStages * 2 * kYBytes;
  // softmax warpgroups per block: one at head_dim 64 (two blocks per SM), two at head_dim 128 (one
  // block per SM), each with its own S / dP pair in TMEM and its own P / dS tiles, taking
  // alternate streamed tiles
  static constexpr int kWGs = (D == 64) ? 1 : 2;
  static constexpr int kThreads = 32 * (4 * kWGs + 2);
  static constexpr int kProducerWarp = 4 * kWGs, kMmaWarp = 4 * kWGs + 1;
  // head_dim 128: P and dS never touch shared memory.  The softmax thread of a row writes them (packed 16-bit pairs) over the S^T / dP^T columns it has just read, and the
  // accumulating MMAs take them from tensor memory as their A operand; the 64 KB this frees hold
  // two more ring stages.  It needs the two S / dP pairs: the next product into the same pair is
  // issued after this tile's accumulation, and the tensor pipe runs in issue order.
  static constexpr bool kPTmem = true;
  static constexpr int kPRegion = kPTmem ? 0 : (MODE == kBwdDQ) ? kPBytes : 2 * kPBytes;   // per warpgroup: dS [| P]
  static constexpr int kOffBar = kOffP + kWGs * kPRegion;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;
  // S / dP accumulators: one pair at head_dim 64 (two blocks share the SM's 512 columns), two
  // pairs at head_dim 128 (one block per SM: the next tile's products run under this tile's softmax)
  static constexpr int kSBufs = kWGs;
  static constexpr uint32_t kColS = 0, kColDP = 64, kSBufCols = 128;
  static constexpr uint32_t kColAcc0 = kSBufs * kSBufCols, kColAcc1 = kColAcc0 + D;
  static constexpr uint32_t kTmemCols = (D == 64) ? 256 : 512;
  static constexpr int kBlocksPerSM = (D == 64) ? 2 : 1;
  // dQ at head_dim 64 leaves 64 of the block's 256 columns unused (no second accumulator): dS gets
  // 32 of them for itself instead of lying over the dP columns, so the products of the next tile
  // are issued as soon as the softmax warps have read this tile's S / dP, not after this tile's
  // accumulation (0 restores the shared columns)
#ifndef SPSATTN_BWD_DS_OWN
#define SPSATTN_BWD_DS_OWN 1
#endif
  static constexpr bool kDsOwn = (MODE == kBwdDQ) && D == 64 && kWGs == 1 && kPTmem && (SPSATTN_BWD_DS_OWN != 0);
  static constexpr uint32_t kColDsOwn = kColAcc0 + D;
};

// delta[b, h, i] = sum_d dO * O, rows addressed with each operand's own strides: D / 8 threads
// per row, 16 bytes of each operand per thread
struct DeltaStrides {
  int64_t o[3], g[3];     // batch, head, row strides of O and dO (elements)
};
template <bool FP16, int D>
__global__ void __launch_bounds__(256)
bwd_delta_kernel(const void* __restrict__ o, const void* __restrict__ d_o, float* __restrict__ delta,
                 long long rows, int H, int N, DeltaStrides st) {
  constexpr int TPR = D / 8;                  // threads per row (8 or 16)
  const long long r = ((long long)blockIdx.x * 256 + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  float acc = 0.f;
  if (r < rows) {
    const long long bh = r / N;
    const int i = (int)(r - bh * N);
    const long long bb = bh / H, hh = bh - bb * H;
    const uint4 a = reinterpret_cast<const uint4*>(
        reinterpret_cast<const uint16_t*>(o) + bb * st.o[0] + hh * st.o[1] + (long long)i * st.o[2])[part];
    const uint4 g = reinterpret_cast<const uint4*>(
        reinterpret_cast<const uint16_t*>(d_o) + bb * st.g[0] + hh * st.g[1] + (long long)i * st.g[2])[part];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      float a0, a1, b0, b1;
      unpack2<FP16>(aw[x], a0, a1);
      unpack2<FP16>(gw[x], b0, b1);
      acc = fmaf(a0, b0, fmaf(a1, b1, acc));
    }
  }
#pragma unroll
  for (int off = TPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (part == 0 && r < rows) delta[r] = acc;
}

// hi[b][i] = last row of the run of equal document ids that contains row i, from the run starts
// lo[b][.] of the document pre-pass (a non-decreasing step function): the first later row whose
// run starts after i, minus one.
__global__ void __launch_bounds__(256)
bwd_run_end_kernel(const int* __restrict__ lo, int* __restrict__ hi, int N, long long total) {
  const long long g = (long long)blockIdx.x * 256 + threadIdx.x;
  if (g >= total) return;
  const int i = (int)(g % N);
  const int* lo_b = lo + (g - i);
  int a = i + 1, c = N;
  while (a < c) {
    const int mid = (a + c) >> 1;
    if (lo_b[mid] > i) c = mid; else a = mid + 1;
  }
  hi[g] = a - 1;
}

struct alignas(16) BwdMeta {   // per streamed query tile in kDKV mode: one entry per column
  float lse[64];     // -lse (log2 domain)
  float delta[64];   // -delta * sm_scale
  int kmin[64];
  int kmax[64];
  long long doc[64];
};

template <int D, bool FP16, int MODE>
__global__ void __launch_bounds__(BwdCfg<D, MODE>::kThreads, BwdCfg<D, MODE>::kBlocksPerSM)
prefill_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_x0, const __grid_constant__ CUtensorMap tm_x1,
                         const __grid_constant__ CUtensorMap tm_y0, const __grid_constant__ CUtensorMap tm_y1,
                         const BwdParams prm) {
  using Cfg = BwdCfg<D, MODE>;
  constexpr bool kDKV = MODE == kBwdDKV;
  extern __shared__ uint8_t smem_raw[];
  __shared__ BlockPlan s_plan;          // kDQ: the forward's key-tile plan of this query tile
  __shared__ int s_tiles[kBwdTable];    // kDQ: packed key tiles; kDKV: (query tile << 1) | masked
  __shared__ int s_ntiles;
  __shared__ int s_cand[2];             // kDKV: first candidate query tile, number of candidates
  __shared__ BwdMeta s_meta[kDKV ? 2 * BwdCfg<D, MODE>::kWGs : 1];   // [warpgroup][tile parity]
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // (batch, head) pairs go in groups whose operands fit L2 together; inside a group the heavy
  // tiles of all its heads come first, so the launch ends on light blocks
  const int gh = prm.group_heads > 0 ? prm.group_heads : 1;
  const int per_group = gh * prm.n_xtiles;
  const int grp = blockIdx.x / per_group;
  const int in_grp = blockIdx.x - grp * per_group;
  const int gsize = min(gh, prm.B * prm.H - grp * gh);
  const int bh = grp * gh + in_grp % gsize;
  const int xt_raw = in_grp / gsize;
  const int b = bh / prm.H;
  const int h = bh - b * prm.H;
  const int ks = prm.mask.ks;
  const int Tk = prm.N / ks;                       // key tokens per stream
  // kDQ: late query tiles are the heavy ones, kDKV: early key tiles are: both go first
  const int xt = kDKV ? xt_raw : prm.n_xtiles - 1 - xt_raw;
  const int stream = kDKV ? (ks == 2 ? (xt & 1) : 0) : 0;
  const int x0 = kDKV ? (xt / ks) * 128 : xt * 128;   // first key token / first query row

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sX0 = smem_base + Cfg::kOffX0;
  const uint32_t sX1 = smem_base + Cfg::kOffX1;
  const uint32_t sY = smem_base + Cfg::kOffY;
  const uint32_t sDS = smem_base + Cfg::kOffP;              // warpgroup g: + g * kPRegion
  const uint32_t sP = sDS + Cfg::kPBytes;                   // kDKV only
  const uint32_t bar0 = smem_base + Cfg::kOffBar;
  const uint32_t bar_x_full = bar0;
  const uint32_t bar_y_full = bar0 + 8;      // [kStages <= 4]
  const uint32_t bar_y_empty = bar0 + 40;    // [kStages <= 4]
  const uint32_t bar_s_full = bar0 + 72;     // [2]
  const uint32_t bar_s_free = bar0 + 88;     // [2]
  const uint32_t bar_p_full = bar0 + 104;    // [warpgroup]
  const uint32_t bar_acc_done = bar0 + 120;  // [warpgroup]
  const uint32_t bar_meta = bar0 + 136;      // [warpgroup][2]

  const bool has_docs = prm.docs != nullptr;
  const bool general = has_docs && prm.mono != nullptr && prm.mono[b] == 0;
  const int* lo_b = (has_docs && !general) ? prm.lo + (size_t)b * prm.N : nullptr;

  if (tid == 0) {
    s_abort = (prm.status != nullptr && *reinterpret_cast<volatile int*>(prm.status) != 0) ? 1 : 0;
    if constexpr (!kDKV) {
      BlockPlan bp;
      bp.general_docs = general ? 1 : 0;
      int lo0 = 0, lo1 = 0;
      if (lo_b != nullptr) {
        lo0 = lo_b[x0];
        lo1 = lo_b[min(x0 + 127, prm.N - 1)];
      }
      if (ks == 1) {
        bp.n_streams = 1;
        bp.stream_id[0] = 0;
        bp.stream_id[1] = 0;
        bp.sp[0] = plan_stream(prm.mask, x0, lo0, lo1, 0, kTileN);
        bp.sp[1] = bp.sp[0];
        bp.sp[1].ntiles = 0;
      } else {
        bp.n_streams = 2;
        bp.stream_id[0] = prm.mask.pp;
        bp.stream_id[1] = 1 - prm.mask.pp;
        bp.sp[0] = plan_stream(prm.mask, x0, lo0, lo1, bp.stream_id[0], kTileN);
        bp.sp[1] = plan_stream(prm.mask, x0, lo0, lo1, bp.stream_id[1], kTileN);
      }
      bp.n_tiles = bp.sp[0].ntiles + bp.sp[1].ntiles;
      s_plan = bp;
      s_ntiles = bp.n_tiles;
    } else {
      // query rows that can see some key of this tile: from the first key's own row up to the
      // window / document limit of the last key
      const int kl = min(x0 + 127, Tk - 1);
      const int jr_first = ks * x0 + stream;
      const int jr_last = ks * kl + stream;
      long long i_hi = prm.N - 1;
      if (ks == 2) {
        if (stream == prm.mask.pp) {
          if (prm.mask.has_pw) i_hi = min(i_hi, 2ll * (kl + max(prm.mask.pw, 0)) + 1);
        } else {
          i_hi = min(i_hi, 2ll * (kl + max(prm.mask.w, 0)) + 1);
        }
      }
      if (lo_b != nullptr) i_hi = min(i_hi, (long long)prm.hi[(size_t)b * prm.N + jr_last]);
      int first = jr_first / 64, n = 0;
      if (x0 < Tk && i_hi >= jr_first) n = min((int)(i_hi / 64) - first + 1, kBwdTable);
      s_cand[0] = first;
      s_cand[1] = n;
    }
  }
  if (warp == Cfg::kProducerWarp) {
    if (lane == 0) {
      mbar_init(bar_x_full, 1);
      for (int s = 0; s < Cfg::kStages; ++s) {
        mbar_init(bar_y_full + 8 * s, 1);
        mbar_init(bar_y_empty + 8 * s, 1);
      }
      for (int s = 0; s < 2; ++s) {
        mbar_init(bar_meta + 8 * s, 64);
        mbar_init(bar_meta + 16 + 8 * s, 64);
        mbar_init(bar_p_full + 8 * s, 128);
        mbar_init(bar_acc_done + 8 * s, 1);
        mbar_init(bar_s_full + 8 * s, 1);
        mbar_init(bar_s_free + 8 * s, 128);
      }
      fence_barrier_init();
      tma_prefetch_desc(&tm_x0);
      tma_prefetch_desc(&tm_x1);
      mbar_arrive_expect_tx(bar_x_full, 2 * Cfg::kXBytes);
      for (int c = 0; c < D / 64; ++c) {
        if constexpr (kDKV) {
          for (int half = 0; half < 2; ++half) {
            tma_load_5d(sX0 + c * Cfg::kXSub + half * 8192, &tm_x0, bar_x_full, c * 64, stream,
                        x0 + 64 * half, h, b);
            tma_load_5d(sX1 + c * Cfg::kXSub + half * 8192, &tm_x1, bar_x_full, c * 64, stream,
                        x0 + 64 * half, h, b);
          }
        } else {
          tma_load_4d(sX0 + c * Cfg::kXSub, &tm_x0, bar_x_full, c * 64, x0, h, b);
          tma_load_4d(sX1 + c * Cfg::kXSub, &tm_x1, bar_x_full, c * 64, x0, h, b);
        }
      }
      tma_prefetch_desc(&tm_y0);
      tma_prefetch_desc(&tm_y1);
    }
    __syncwarp();
    tmem_alloc<Cfg::kTmemCols>(smem_u32(&s_tmem_base));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;

  // ---- the list of streamed tiles
  if constexpr (!kDKV) {
    for (int j = tid; j < min(s_plan.n_tiles, kBwdTable); j += Cfg::kThreads)
      s_tiles[j] = pack_tile(tile_info(s_plan, j));
  } else {
    // Per candidate query tile, one thread each: can a row see a key of this tile, do all rows see
    // all keys.  Within a tile the visible interval [kmin, kmax] of a row moves up monotonically
    // with the row (causal bound, window bound and run start all do), so the first and the last
    // row decide: the tile is interior iff the last row's kmin and the first row's kmax cover the
    // key tile, and it may be skipped if the last row's kmax or the first row's kmin misses it
    // (a superset of the truly visible tiles: a tile kept in vain is fully masked and adds zeros).
    // Streams only one row parity can see are never interior.
    const int first = s_cand[0], n_cand = s_cand[1];
    int only;
    const bool filt = stream_row_filter(prm.mask, stream, only);
    for (int cnd = tid; cnd < n_cand; cnd += Cfg::kThreads) {
      const int q0 = (first + cnd) * 64;
      int ra = q0, rb = min(q0 + 63, prm.N - 1);
      const bool partial = q0 + 63 > prm.N - 1;
      if (filt) {
        if ((ra & 1) != only) ++ra;
        if ((rb & 1) != only) --rb;
      }
      int e = -1;
      if (ra <= rb) {
        int kmin_a, kmax_a, kmin_b, kmax_b;
        row_interval(prm.mask, ra, lo_b != nullptr ? lo_b[ra] : 0, stream, kmin_a, kmax_a);
        row_interval(prm.mask, rb, lo_b != nullptr ? lo_b[rb] : 0, stream, kmin_b, kmax_b);
        const bool any = kmax_b >= x0 && kmin_a <= x0 + 127;
        const bool all = !filt && !partial && !general && kmin_b <= x0 && kmax_a >= x0 + 127;
        if (any) e = ((first + cnd) << 1) | (all ? 0 : 1);
      }
      s_tiles[cnd] = e;
    }
    __syncthreads();
    if (tid == 0) {
      int n = 0;
      for (int cnd = 0; cnd < n_cand; ++cnd) {
        const int e = s_tiles[cnd];
        if (e >= 0) s_tiles[n++] = e;
      }
      s_ntiles = n;
    }
  }
  __syncthreads();
  const int n_tiles = s_ntiles;
  volatile int* abort_flag = &s_abort;
  const bool bail = s_abort != 0;

  auto dq_tile = [&](int j) {
    return j < kBwdTable ? unpack_tile(s_tiles[j]) : tile_info(s_plan, j);
  };

  if (!bail && n_tiles > 0) {
    if (warp == Cfg::kProducerWarp) {
      // ------------------------------------------------------------------ TMA producer
      bool ok = true;
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int st = j % Cfg::kStages;
        if (j >= Cfg::kStages)
          ok = warp_wait(bar_y_empty + 8 * st, ((j / Cfg::kStages) - 1) & 1, abort_flag, prm.status);
        if (!ok) break;
        if (elect_one()) {
          const uint32_t dst0 = sY + st * 2 * Cfg::kYBytes, dst1 = dst0 + Cfg::kYBytes;
          mbar_arrive_expect_tx(bar_y_full + 8 * st, 2 * Cfg::kYBytes);
          if constexpr (kDKV) {
            const int q0 = (s_tiles[j] >> 1) * 64;
            for (int c = 0; c < D / 64; ++c) {
              tma_load_4d(dst0 + c * Cfg::kYSub, &tm_y0, bar_y_full + 8 * st, c * 64, q0, h, b);
              tma_load_4d(dst1 + c * Cfg::kYSub, &tm_y1, bar_y_full + 8 * st, c * 64, q0, h, b);
            }
          } else {
            const TileInfo t = dq_tile(j);
            for (int c = 0; c < D / 64; ++c) {
              tma_load_5d(dst0 + c * Cfg::kYSub, &tm_y0, bar_y_full + 8 * st, c * 64, t.stream, t.k0, h, b);
              tma_load_5d(dst1 + c * Cfg::kYSub, &tm_y1, bar_y_full + 8 * st, c * 64, t.stream, t.k0, h, b);
            }
          }
        }
        __syncwarp();
      }
    } else if (warp == Cfg::kMmaWarp) {
      // ------------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc_s = make_idesc_f16(FP16, 128, 64, false, false);
      constexpr uint32_t idesc_acc = make_idesc_f16(FP16, 128, D, false, true);
      const uint64_t dx0 = make_smem_desc_sw128(sX0, 16, 1024);
      const uint64_t dx1 = make_smem_desc_sw128(sX1, 16, 1024);
      const uint64_t dyk = make_smem_desc_sw128(sY, 16, 1024);               // Y as K-major B
      const uint64_t dym = make_smem_desc_sw128(sY, Cfg::kYSub, 1024);       // Y as MN-major B
      const uint64_t dp = make_smem_desc_sw128(sP, 16, 1024);
      const uint64_t dds = make_smem_desc_sw128(sDS, 16, 1024);
      const uint32_t dx0_lo = (uint32_t)dx0, dx1_lo = (uint32_t)dx1, dx_hi = (uint32_t)(dx0 >> 32);
      const uint32_t dyk_lo = (uint32_t)dyk, dyk_hi = (uint32_t)(dyk >> 32);
      const uint32_t dym_lo = (uint32_t)dym, dym_hi = (uint32_t)(dym >> 32);
      const uint32_t dp_lo = (uint32_t)dp, dds_lo = (uint32_t)dds, dp_hi = (uint32_t)(dp >> 32);
      auto issue_s = [&](int j) {
        const int st = j % Cfg::kStages;
        if (!warp_wait(bar_y_full + 8 * st, (j / Cfg::kStages) & 1, abort_flag, prm.status)) return false;
        const int sb = j % Cfg::kSBufs;
        if (j >= Cfg::kSBufs) {
          if (!warp_wait(bar_s_free + 8 * sb, ((j / Cfg::kSBufs) - 1) & 1, abort_flag, prm.status)) return false;
        }
        tc_fence_after();
        const uint32_t ts = tmem + sb * Cfg::kSBufCols;
        const uint32_t y0 = dyk_lo + ((st * 2 * Cfg::kYBytes) >> 4);
        const uint32_t y1 = y0 + (Cfg::kYBytes >> 4);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t xa = ((kk / 4) * Cfg::kXSub + (kk % 4) * 32) >> 4;
            const uint32_t yb = ((kk / 4) * Cfg::kYSub + (kk % 4) * 32) >> 4;
            if (kk == 0) umma_ss<false>(ts + Cfg::kColS, dx0_lo + xa, dx_hi, y0 + yb, dyk_hi, idesc_s);
            else umma_ss<true>(ts + Cfg::kColS, dx0_lo + xa, dx_hi, y0 + yb, dyk_hi, idesc_s);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t xa = ((kk / 4) * Cfg::kXSub + (kk % 4) * 32) >> 4;
            const uint32_t yb = ((kk / 4) * Cfg::kYSub + (kk % 4) * 32) >> 4;
            if (kk == 0) umma_ss<false>(ts + Cfg::kColDP, dx1_lo + xa, dx_hi, y1 + yb, dyk_hi, idesc_s);
            else umma_ss<true>(ts + Cfg::kColDP, dx1_lo + xa, dx_hi, y1 + yb, dyk_hi, idesc_s);
          }
          umma_commit(bar_s_full + 8 * sb);
        }
        __syncwarp();
        return true;
      };
      bool ok = warp_wait(bar_x_full, 0, abort_flag, prm.status);
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        // with P / dS laid over a single S / dP pair the next products may only be issued after this
        // tile's accumulation (the tensor pipe runs in issue order)
        constexpr bool kAhead = !(Cfg::kPTmem && Cfg::kSBufs == 1) || Cfg::kDsOwn;
        if (kAhead && j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int st = j % Cfg::kStages;
        const int g = j % Cfg::kWGs;                  // the warpgroup that produced P / dS of this tile
        if (!warp_wait(bar_p_full + 8 * g, (j / Cfg::kWGs) & 1, abort_flag, prm.status)) break;
        const uint32_t pg = (uint32_t)(g * Cfg::kPRegion) >> 4;
        tc_fence_after();
        const uint32_t y0 = dym_lo + ((st * 2 * Cfg::kYBytes) >> 4);
        const uint32_t y1 = y0 + (Cfg::kYBytes >> 4);
        if (elect_one()) {
          // dS (and P): K-major A, 16 of the 64 streamed rows = 32 bytes per step; Y: MN-major B,
          // 16 rows = 2048 bytes per step
          if constexpr (Cfg::kPTmem) {
            // A from tensor memory: 16 contraction elements = 8 columns per step
            const uint32_t ta = tmem + g * Cfg::kSBufCols;
            const uint32_t a_ds = Cfg::kDsOwn ? tmem + Cfg::kColDsOwn : ta + Cfg::kColDP;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ts(tmem + Cfg::kColAcc0, a_ds + 8 * kk, y0 + ((kk * 2048) >> 4), dym_hi, idesc_acc,
                      !(j == 0 && kk == 0));
            if constexpr (kDKV) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_ts(tmem + Cfg::kColAcc1, ta + Cfg::kColS + 8 * kk, y1 + ((kk * 2048) >> 4), dym_hi, idesc_acc,
                        !(j == 0 && kk == 0));
            }
          } else {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if (j == 0 && kk == 0)
              umma_ss<false>(tmem + Cfg::kColAcc0, dds_lo + pg + ((kk * 32) >> 4), dp_hi, y0 + ((kk * 2048) >> 4), dym_hi, idesc_acc);
            else
              umma_ss<true>(tmem + Cfg::kColAcc0, dds_lo + pg + ((kk * 32) >> 4), dp_hi, y0 + ((kk * 2048) >> 4), dym_hi, idesc_acc);
          }
          if constexpr (kDKV) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              if (j == 0 && kk == 0)
                umma_ss<false>(tmem + Cfg::kColAcc1, dp_lo + pg + ((kk * 32) >> 4), dp_hi, y1 + ((kk * 2048) >> 4), dym_hi, idesc_acc);
              else
                umma_ss<true>(tmem + Cfg::kColAcc1, dp_lo + pg + ((kk * 32) >> 4), dp_hi, y1 + ((kk * 2048) >> 4), dym_hi, idesc_acc);
            }
          }
          }
          umma_commit(bar_acc_done + 8 * g);
          umma_commit(bar_y_empty + 8 * st);
        }
        __syncwarp();
        if (!kAhead && j + 1 < n_tiles) ok = issue_s(j + 1);
      }
    } else {
      // ------------------------------------------------------------------ softmax warps
      const int wg = tid >> 7;                        // softmax warpgroup: takes tiles wg, wg + kWGs, ...
      const int row = tid & 127;                      // TMEM lane, row of the stationary tile
      const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t sPg = sP + wg * Cfg::kPRegion, sDSg = sDS + wg * Cfg::kPRegion;
      const uint32_t bar_meta_g = bar_meta + 16 * wg;
      const float c = prm.scale_log2;
      const float scale = prm.sm_scale;
      const uint8_t* docs_b = nullptr;
      if (general)
        docs_b = reinterpret_cast<const uint8_t*>(prm.docs) + (size_t)b * prm.doc_stride_b * (prm.doc_is_i64 ? 8 : 4);
      auto doc_at = [&](int r) -> long long {
        const size_t off = (size_t)r * prm.doc_stride_t;
        return prm.doc_is_i64 ? reinterpret_cast<const long long*>(docs_b)[off]
                              : (long long)reinterpret_cast<const int*>(docs_b)[off];
      };
      // per-row constants
      float neg_lse = 0.f, delta_i = 0.f;             // kDQ: this query row
      int kmin_s[2] = {0, 0}, kmax_s[2] = {-1, -1};   // kDQ: visible key tokens per stream
      long long my_doc = 0;
      const int my_row = kDKV ? ks * (x0 + row) + stream : x0 + row;   // row in the sequence
      const bool my_valid = kDKV ? (x0 + row < Tk) : (my_row < prm.N);
      if constexpr (!kDKV) {
        if (my_valid) {
          neg_lse = -prm.lse[(size_t)bh * prm.N + my_row];
          delta_i = -prm.delta[(size_t)bh * prm.N + my_row] * prm.sm_scale;   // enters as an FMA addend
        }
        const int lo_i = (lo_b != nullptr && my_valid) ? lo_b[my_row] : 0;
        row_interval(prm.mask, my_row, lo_i, 0, kmin_s[0], kmax_s[0]);
        row_interval(prm.mask, my_row, lo_i, 1, kmin_s[1], kmax_s[1]);
      }
      if (general && my_valid) my_doc = doc_at(my_row);
      const int my_kt = x0 + row;                     // kDKV: this thread's key token
      bool ok = true;

      // kDKV: the per-column constants of a streamed query tile (lse, delta, visible key interval,
      // document id) are fetched one tile ahead by the first 64 threads: the loads are issued
      // when tile j starts and land in shared memory when it ends
      float pf_l = 0.f, pf_dl = 0.f;
      int pf_lo = 0;
      long long pf_doc = 0;
      auto meta_fetch = [&](int jj) {
        const int i = (s_tiles[jj] >> 1) * 64 + row;
        pf_l = 0.f, pf_dl = 0.f, pf_lo = 0, pf_doc = 0;
        if (i < prm.N) {
          pf_l = prm.lse[(size_t)bh * prm.N + i];
          pf_dl = prm.delta[(size_t)bh * prm.N + i];
          if (lo_b != nullptr) pf_lo = lo_b[i];
          if (general) pf_doc = doc_at(i);
        }
      };
      auto meta_publish = [&](int jj) {
        const int i = (s_tiles[jj] >> 1) * 64 + row;
        const int par = (jj / Cfg::kWGs) & 1;         // this warpgroup's tiles alternate buffers
        BwdMeta* mw = &s_meta[2 * wg + par];
        int kmin = 0, kmax = -1;
        if (i < prm.N) row_interval(prm.mask, i, pf_lo, stream, kmin, kmax);
        mw->lse[row] = -pf_l;
        mw->delta[row] = -pf_dl * prm.sm_scale;
        mw->kmin[row] = kmin;
        mw->kmax[row] = kmax;
        mw->doc[row] = pf_doc;
        mbar_arrive(bar_meta_g + 8 * par);
      };
      if constexpr (kDKV) {
        if (row < 64 && wg < n_tiles) {
          meta_fetch(wg);
          meta_publish(wg);
        }
      }

      for (int j = wg; j < n_tiles; j += Cfg::kWGs) {
        const int jl = j / Cfg::kWGs;                 // tiles this warpgroup has done
        bool masked;
        int y_first = 0, y_stream = 0;                // kDQ: first key token and stream of the tile
        const BwdMeta* meta = &s_meta[0];
        if constexpr (kDKV) {
          const int e = s_tiles[j];
          masked = (e & 1) != 0;
          meta = &s_meta[2 * wg + (jl & 1)];
          if (!mbar_wait(bar_meta_g + 8 * (jl & 1), (jl >> 1) & 1, abort_flag, prm.status)) {
            ok = false;
            break;
          }
        } else {
          const TileInfo t = dq_tile(j);
          masked = t.masked != 0;
          y_first = t.k0;
          y_stream = t.stream;
        }
        const int sb = j % Cfg::kSBufs;
        const uint32_t ts = tmem + lane_addr + sb * Cfg::kSBufCols;
        if (!mbar_wait(bar_s_full + 8 * sb, (j / Cfg::kSBufs) & 1, abort_flag, prm.status)) {
          ok = false;
          break;
        }
        // this warpgroup's P / dS tiles are free once its previous accumulation is done (with dS in
        // columns of its own the wait comes later, before the first dS store)
        if (!Cfg::kDsOwn && jl > 0) {
          if (!mbar_wait(bar_acc_done + 8 * wg, (jl - 1) & 1, abort_flag, prm.status)) {
            ok = false;
            break;
          }
        }
        tc_fence_after();
        if constexpr (kDKV) {
          // every thread of the warpgroup is past its previous tile here, so the other meta buffer
          // may be refilled
          if (row < 64 && j + Cfg::kWGs < n_tiles) meta_fetch(j + Cfg::kWGs);
        }

        // kDQ: the visible keys of this row form an interval of the tile's 64 columns
        uint32_t vis_w[2] = {0xffffffffu, 0xffffffffu};
        if constexpr (!kDKV) {
          if (masked) {
            const int cmin = max(kmin_s[y_stream] - y_first, 0);
            const int cmax = min(kmax_s[y_stream] - y_first, 63);
            const unsigned long long vis =
                cmin > cmax ? 0ull : ((~0ull >> (63 - cmax)) & (~0ull << cmin));
            vis_w[0] = (uint32_t)vis;
            vis_w[1] = (uint32_t)(vis >> 32);
            if (general) {
#pragma unroll
              for (int q4 = 0; q4 < 2; ++q4) {
                uint32_t bits = 0;
                for (int e = 0; e < 32; ++e) {
                  const int jrow = ks * (y_first + q4 * 32 + e) + y_stream;
                  if (jrow >= 0 && jrow < prm.N) bits |= (doc_at(jrow) == my_doc ? 1u : 0u) << e;
                }
                vis_w[q4] &= bits;
              }
            }
          }
        }

        if constexpr (kDKV) {
          // visibility of the tile's 64 query columns for this thread's key, one bit each
          if (masked) {
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {
              uint32_t bits = 0;
#pragma unroll
              for (int e = 0; e < 32; e += 4) {
                const int4 lo4 = *reinterpret_cast<const int4*>(&meta->kmin[q4 * 32 + e]);
                const int4 hi4 = *reinterpret_cast<const int4*>(&meta->kmax[q4 * 32 + e]);
                bits |= ((my_kt >= lo4.x && my_kt <= hi4.x) ? 1u : 0u) << e;
                bits |= ((my_kt >= lo4.y && my_kt <= hi4.y) ? 1u : 0u) << (e + 1);
                bits |= ((my_kt >= lo4.z && my_kt <= hi4.z) ? 1u : 0u) << (e + 2);
                bits |= ((my_kt >= lo4.w && my_kt <= hi4.w) ? 1u : 0u) << (e + 3);
              }
              if (general) {
                for (int e = 0; e < 32; ++e)
                  if (meta->doc[q4 * 32 + e] != my_doc) bits &= ~(1u << e);
              }
              vis_w[q4] = bits;
            }
          }
        }

        // columns are processed CH at a time; in kDKV mode the per-column constants of a chunk
        // are staged in registers with vector loads before the scores arrive
        constexpr int CH = kDKV ? 16 : 32;
        // the tensor-memory loads of chunk c + 1 are issued before the arithmetic of chunk c (two
        // register sets), so only the first load of a tile is waited for at full latency
#ifdef SPSATTN_BWD_NO_LD_AHEAD
        constexpr bool kLdAhead = false;
#else
        constexpr bool kLdAhead = true;
#endif
        uint32_t rsb[kLdAhead ? 2 : 1][CH], rdb[kLdAhead ? 2 : 1][CH];
        auto ld_chunk = [&](int chunk, uint32_t (&a)[CH], uint32_t (&d)[CH]) {
          if constexpr (CH == 32) {
            tmem_ld32(ts + Cfg::kColS + chunk * CH, a);
            tmem_ld32(ts + Cfg::kColDP + chunk * CH, d);
          } else {
            tmem_ld16(ts + Cfg::kColS + chunk * CH, a);
            tmem_ld16(ts + Cfg::kColDP + chunk * CH, d);
          }
        };
        if constexpr (kLdAhead) ld_chunk(0, rsb[0], rdb[0]);
#pragma unroll
        for (int chunk = 0; chunk < 64 / CH; ++chunk) {
          float nl_c[kDKV ? CH : 1], dl_c[kDKV ? CH : 1];
          if constexpr (kDKV) {
#pragma unroll
            for (int e = 0; e < CH; e += 4) {
              const float4 a4 = *reinterpret_cast<const float4*>(&meta->lse[chunk * CH + e]);
              const float4 b4 = *reinterpret_cast<const float4*>(&meta->delta[chunk * CH + e]);
              nl_c[e] = a4.x, nl_c[e + 1] = a4.y, nl_c[e + 2] = a4.z, nl_c[e + 3] = a4.w;
              dl_c[e] = b4.x, dl_c[e + 1] = b4.y, dl_c[e + 2] = b4.z, dl_c[e + 3] = b4.w;
            }
          }
          uint32_t (&rs)[CH] = rsb[kLdAhead ? (chunk & 1) : 0];
          uint32_t (&rd)[CH] = rdb[kLdAhead ? (chunk & 1) : 0];
          if constexpr (!kLdAhead) ld_chunk(chunk, rs, rd);
          tmem_wait_ld();
          if constexpr (kLdAhead) {
            if (chunk + 1 < 64 / CH) ld_chunk(chunk + 1, rsb[(chunk + 1) & 1], rdb[(chunk + 1) & 1]);
          }
          if (chunk == 64 / CH - 1) {
            tc_fence_before();
            mbar_arrive(bar_s_free + 8 * sb);
          }
          const uint32_t vbits = vis_w[(chunk * CH) >> 5] >> ((chunk * CH) & 31);
          uint32_t pk_p[CH / 2], pk_ds[CH / 2];
          // packed fp32x2 arithmetic: one FFMA2 forms two exponents, one FFMA2 + one FMUL2 two dS
          const float2 c2 = make_float2(c, c), sc2 = make_float2(scale, scale);
#pragma unroll
          for (int e = 0; e < CH; e += 2) {
            const float2 nl2 = kDKV ? make_float2(nl_c[kDKV ? e : 0], nl_c[kDKV ? e + 1 : 0])
                                    : make_float2(neg_lse, neg_lse);
            const float2 nd2 = kDKV ? make_float2(dl_c[kDKV ? e : 0], dl_c[kDKV ? e + 1 : 0])
                                    : make_float2(delta_i, delta_i);      // -delta * scale
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), c2, nl2);
            float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            p.x = ((vbits >> e) & 1u) ? p.x : 0.f;
            p.y = ((vbits >> (e + 1)) & 1u) ? p.y : 0.f;
            const float2 t = __ffma2_rn(make_float2(__uint_as_float(rd[e]), __uint_as_float(rd[e + 1])), sc2, nd2);
            const float2 ds = __fmul2_rn(p, t);
            pk_p[e / 2] = pack2<FP16>(p.x, p.y);
            pk_ds[e / 2] = pack2<FP16>(ds.x, ds.y);
          }
          if constexpr (Cfg::kPTmem) {
            if (Cfg::kDsOwn && chunk == 0 && jl > 0) {
              // on a failed wait the tile is finished anyway (its stores are harmless) and the
              // loop ends below
              if (!mbar_wait(bar_acc_done + 8 * wg, (jl - 1) & 1, abort_flag, prm.status)) ok = false;
              tc_fence_after();
            }
            // over the columns of S / dP this warp has already read: chunk c (CH columns of each)
            // leaves CH / 2 packed columns of P at S + c * CH / 2 and of dS at dP + c * CH / 2
            // (dS at its own columns in the dQ kernel of head_dim 64)
            const uint32_t ds_to = Cfg::kDsOwn ? tmem + lane_addr + Cfg::kColDsOwn : ts + Cfg::kColDP;
#pragma unroll
            for (int q8 = 0; q8 < CH / 16; ++q8) {
              if constexpr (kDKV) tmem_st8(ts + Cfg::kColS + chunk * (CH / 2) + 8 * q8, pk_p + 8 * q8);
              tmem_st8(ds_to + chunk * (CH / 2) + 8 * q8, pk_ds + 8 * q8);
            }
          }
          // K-major 128B-swizzled [128 x 64] tiles: 16-byte chunk ch of row r sits at
          // r * 128 + ((ch ^ (r & 7)) << 4)
#pragma unroll
          for (int q4 = 0; q4 < (Cfg::kPTmem ? 0 : CH / 8); ++q4) {
            const int ch = chunk * (CH / 8) + q4;
            const uint32_t off = row * 128 + ((ch ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sDSg + off), "r"(pk_ds[q4 * 4]),
                         "r"(pk_ds[q4 * 4 + 1]), "r"(pk_ds[q4 * 4 + 2]), "r"(pk_ds[q4 * 4 + 3])
                         : "memory");
            if constexpr (kDKV) {
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sPg + off), "r"(pk_p[q4 * 4]),
                           "r"(pk_p[q4 * 4 + 1]), "r"(pk_p[q4 * 4 + 2]), "r"(pk_p[q4 * 4 + 3])
                           : "memory");
            }
          }
        }
        if constexpr (Cfg::kPTmem) tmem_wait_st();
        else fence_proxy_async_smem();
        if (!ok) break;
        tc_fence_before();
        mbar_arrive(bar_p_full + 8 * wg);
        if constexpr (kDKV) {
          if (row < 64 && j + Cfg::kWGs < n_tiles) meta_publish(j + Cfg::kWGs);
        }
      }

      // ---------------------------------------------------------------- epilogue
      // The accumulations complete in order, so the last tile's barrier covers them all.  The
      // warpgroup that owns the last tile writes the result: it has consumed every earlier phase
      // of its own barrier, so this parity wait cannot be satisfied by an older phase (the other
      // warpgroup never waited on that barrier and could pass on a stale parity).
      const bool epilogue_wg = wg == (n_tiles - 1) % Cfg::kWGs;
      if (ok && epilogue_wg)
        ok = mbar_wait(bar_acc_done + 8 * wg, ((n_tiles - 1) / Cfg::kWGs) & 1, abort_flag, prm.status);
      if (ok && epilogue_wg) {
        tc_fence_after();
#pragma unroll
        for (int a = 0; a < (kDKV ? 2 : 1); ++a) {
          const int64_t* os = a == 0 ? prm.out0_stride : prm.out1_stride;
          uint8_t* o_row = reinterpret_cast<uint8_t*>(a == 0 ? prm.out0 : prm.out1) +
                           (b * os[0] + h * os[1] + (int64_t)my_row * os[2]) * 2;
#pragma unroll
          for (int q4 = 0; q4 < D / 32; ++q4) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_addr + (a == 0 ? Cfg::kColAcc0 : Cfg::kColAcc1) + q4 * 32, r);
            tmem_wait_ld();
            if (my_valid) {
#pragma unroll
              for (int e = 0; e < 32; e += 8) {
                uint4 u;
                u.x = pack2<FP16>(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
                u.y = pack2<FP16>(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
                u.z = pack2<FP16>(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
                u.w = pack2<FP16>(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
                *reinterpret_cast<uint4*>(o_row + q4 * 64 + e * 2) = u;
              }
            }
          }
        }
        tc_fence_before();
      }
    }
  } else if (!bail && warp < 4) {
    // nothing streams through this tile: its gradients are zero
    const int my_row = kDKV ? ks * (x0 + tid) + stream : x0 + tid;
    const bool my_valid = kDKV ? (x0 + tid < Tk) : (my_row < prm.N);
    if (my_valid) {
      for (int a = 0; a < (kDKV ? 2 : 1); ++a) {
        const int64_t* os = a == 0 ? prm.out0_stride : prm.out1_stride;
        uint4* o_row = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a == 0 ? prm.out0 : prm.out1) +
                                                (b * os[0] + h * os[1] + (int64_t)my_row * os[2]) * 2);
        for (int e = 0; e < D / 8; ++e) o_row[e] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  // the stationary tiles were requested before the plan was known: never leave with them in flight
  if (warp == Cfg::kProducerWarp && lane == 0) mbar_wait(bar_x_full, 0, abort_flag, prm.status);
  __syncthreads();
  if (warp == Cfg::kProducerWarp) {
    tc_fence_after();
    tmem_dealloc<Cfg::kTmemCols>(tmem);
  }
}

}  // namespace spsattn
