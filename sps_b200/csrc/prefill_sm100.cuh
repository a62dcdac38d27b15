// SPS prefill attention for sm_100a: TMA-staged Q/K/V tiles, tcgen05 MMAs accumulating in TMEM,
// online softmax in registers (one query row per thread, no shuffles), key streams
// de-interleaved by parity so that only tiles that hold visible keys are visited.
//
// One block = one 128-row query tile of one (batch, head).  Roles:
//   warps 0-3  softmax / correction / epilogue (thread r owns query row r = TMEM lane r)
//   warp 4     TMEM allocation, TMA producer (lane 0)
//   warp 5     MMA issuer (lane 0)
// Per key tile j (64 key tokens of one parity stream):
//   S = Q K_j^T        tcgen05.mma  128x64xD, operands K-major / 128B swizzle in shared memory
//   P = exp2(S*c - m*c) softmax warps: tcgen05.ld S -> registers, mask boundary tiles only,
//                       bf16/fp16 P written to shared memory in the K-major swizzled layout
//   O += P V_j         tcgen05.mma  128xDx64, V consumed as the MN-major B operand as loaded
// Tiles of 64 keys keep a block small (64 KB of shared memory, 128 TMEM columns, ~110
// registers at head_dim 64) so that three blocks share an SM: the kernel is limited by the
// special-function unit (one exp2 per score, 16 per clock per SM) and three independent blocks
// in different phases keep that unit busier than two larger ones.
// Reference computation: src/modeling/models/attention/triton_sps_flash_attention.py:26-139,
// :147-269 (and the reverse / standard variants); unlike it, tiles whose keys are all hidden
// by the document / window / parity rule are never loaded or multiplied.
#pragma once

#include "common.cuh"
#include "mask.cuh"

namespace spsattn {

struct PrefillParams {
  void* o;               // rows of D contiguous elements, addressed with the strides below
  int64_t o_stride_b, o_stride_h, o_stride_n;   // elements
  float* lse;            // [B,H,N] or null
  const void* docs;      // [B,N] ids or null
  int64_t doc_stride_b, doc_stride_t;
  int doc_is_i64;
  const int* lo;         // [B,N] run starts (pre-pass) or null
  const int* mono;       // [B] 1 when ids of the row are non-decreasing, or null
  int B, H, N;
  int n_qtiles;
  MaskParams mask;
  float scale_log2;      // sm_scale * log2(e)
  int* status;
  int* work_counter;     // persistent kernels: next work item (zero at launch), or null
  int group_heads;       // persistent kernels: (batch, head) pairs whose K/V share L2 at a time
  long long* trace;      // cycle stamps (only read by builds with -DSPSATTN_TRACE), else null
};

// Optional per-block cycle stamps for tuning: compiled out unless SPSATTN_TRACE is defined.
// Layout: [block][tile < kTraceTiles][slot < 16] of clock64().
constexpr int kTraceTiles = 40;
#ifdef SPSATTN_TRACE
#define SPS_TRACE(tile, slot)                                                                  \
  do {                                                                                         \
    if (prm.trace != nullptr && blockIdx.x < 4096 && (tile) < kTraceTiles)                     \
      prm.trace[((size_t)blockIdx.x * kTraceTiles + (tile)) * 16 + (slot)] = clock64();        \
  } while (0)
#else
#define SPS_TRACE(tile, slot) do { } while (0)
#endif

constexpr int kTileM = 128;      // query rows per block
constexpr int kTileN = 64;       // key tokens per tile
constexpr int kPrefillThreads = 192;

#ifndef SPSATTN_P_SPLIT
#define SPSATTN_P_SPLIT_DEFAULT 1
#else
#define SPSATTN_P_SPLIT_DEFAULT (SPSATTN_P_SPLIT != 0)
#endif

template <int D>
struct PrefillCfg {
  static constexpr int kStagesK = 2;
  static constexpr int kStagesV = (D == 64) ? 2 : 1;
  static constexpr int kSBufs = (D == 64) ? 1 : 2;            // S accumulators in TMEM
  static constexpr uint32_t kTmemCols = (D == 64) ? 128 : 256;
  static constexpr uint32_t kColO = kSBufs * kTileN;           // O accumulator column offset
  static constexpr int kQBytes = kTileM * D * 2;               // the Q tile
  static constexpr int kQSubBytes = kTileM * 128;              // 128 rows x 64 elements
  static constexpr int kKVBytes = kTileN * D * 2;              // one K or V tile
  static constexpr int kKVSubBytes = kTileN * 128;             // 64 rows x 64 elements
  static constexpr int kPBytes = (D == 64 && SPSATTN_P_SPLIT_DEFAULT) ? 0 : kTileM * kTileN * 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kQBytes;
  static constexpr int kOffV = kOffK + kStagesK * kKVBytes;
  static constexpr int kOffP = kOffV + kStagesV * kKVBytes;
  static constexpr int kOffBar = kOffP + kPBytes;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;      // barriers + alignment slack
  static constexpr int kBlocksPerSM = (D == 64) ? 3 : 2;
  // head_dim 128 (two S accumulators): P never touches shared memory.  The softmax thread writes
  // it, as packed 16-bit pairs, over the S columns it has just read, and the P V product takes it
  // from tensor memory as its A operand, which also halves what that product reads from shared
  // memory.  The next Q K^T into the same accumulator is issued after this tile's P V, and the
  // tensor pipe runs in issue order.  (With the single accumulator of head_dim 64 the next Q K^T
  // would have to wait for P V; measured slower there.)
  static constexpr bool kPTmem = (D == 128);
  // head_dim 64: P also lives in tensor memory, but in 32 columns of its own (a second, small
  // allocation: 128 + 32 columns per block, three blocks per SM = 480 of 512), so the next Q K^T
  // does not have to wait for this tile's P V.  No shared-memory stores, no swizzle arithmetic,
  // no proxy fence; the P tile's 16 KB of shared memory are not needed.
#ifndef SPSATTN_P_SPLIT
#define SPSATTN_P_SPLIT 1
#endif
  static constexpr bool kPSplit = (D == 64) && (SPSATTN_P_SPLIT != 0);
  static constexpr uint32_t kPCols = kTileN / 2;
};

struct TileInfo {
  int stream;   // key parity (0 in standard mode)
  int k0;       // first key token of the tile (may be negative: zero-filled, masked)
  int masked;   // element mask needed
};

struct BlockPlan {
  StreamPlan sp[2];
  int stream_id[2];
  int n_streams;
  int n_tiles;
  int general_docs;  // ids are not monotone: compare ids element by element
};

// TN = key tokens per tile (the plan's streams must have been made with the same tile size)
template <int TN = kTileN>
__device__ __forceinline__ TileInfo tile_info(const BlockPlan& bp, int j) {
  TileInfo t;
  int s = 0;
  if (j >= bp.sp[0].ntiles) {
    j -= bp.sp[0].ntiles;
    s = 1;
  }
  t.stream = bp.stream_id[s];
  t.k0 = bp.sp[s].top - (TN - 1) - TN * j;
  t.masked = bp.sp[s].force_mask || bp.general_docs ||
             !(bp.sp[s].kmin_hi <= t.k0 && bp.sp[s].kmax_lo >= t.k0 + TN - 1);
  return t;
}

// The tile sequence of a block, precomputed once into shared memory so that every role reads one
// word per tile instead of re-deriving it from the plan: (k0 << 2) | (stream << 1) | masked.
// Blocks with more tiles than the table holds fall back to tile_info for the rest.
constexpr int kTileTable = 128;

__device__ __forceinline__ int pack_tile(const TileInfo& t) {
  return (t.k0 << 2) | ((t.stream & 1) << 1) | (t.masked ? 1 : 0);
}
__device__ __forceinline__ TileInfo unpack_tile(int w) {
  TileInfo t;
  t.k0 = w >> 2;             // arithmetic shift: k0 may be negative for a top-aligned first tile
  t.stream = (w >> 1) & 1;
  t.masked = (w & 1) != 0;
  return t;
}
template <int TN = kTileN>
__device__ __forceinline__ TileInfo get_tile(const BlockPlan& bp, const int* table, int j) {
  return j < kTileTable ? unpack_tile(table[j]) : tile_info<TN>(bp, j);
}

constexpr float kRescaleLog2 = 8.0f;

// How the four softmax warps signal the MMA warp: one arrival per warp (lane 0, after the warp has
// converged, which also orders the other lanes' writes before it) instead of one per thread: 128
// arrivals on one shared-memory word serialise, twice per tile.
#ifdef SPSATTN_ARRIVE_ALL
constexpr int kSoftmaxArrivals = 128;
__device__ __forceinline__ void softmax_arrive(uint32_t bar, int) { mbar_arrive(bar); }
#else
constexpr int kSoftmaxArrivals = 4;
__device__ __forceinline__ void softmax_arrive(uint32_t bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}
#endif

template <int D, bool FP16>
__global__ void __launch_bounds__(kPrefillThreads, PrefillCfg<D>::kBlocksPerSM)
prefill_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const PrefillParams prm) {
  using Cfg = PrefillCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ BlockPlan s_plan;
  __shared__ int s_tiles[kTileTable];
  __shared__ uint32_t s_tmem_base;
  __shared__ uint32_t s_tmem_p;
  __shared__ int s_abort;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  if (tid == 0) SPS_TRACE(0, 15);

  // (batch, head) pairs go in groups whose K/V fit L2 together; inside a group the late (heavy)
  // query tiles of all its heads come first, so the launch ends on light blocks
  const int gh = prm.group_heads > 0 ? prm.group_heads : 1;
  const int per_group = gh * prm.n_qtiles;
  const int grp = blockIdx.x / per_group;
  const int in_grp = blockIdx.x - grp * per_group;
  const int gsize = min(gh, prm.B * prm.H - grp * gh);
  const int bh = grp * gh + in_grp % gsize;
  const int qt = prm.n_qtiles - 1 - in_grp / gsize;
  const int b = bh / prm.H;
  const int h = bh - b * prm.H;
  const int i0 = qt * kTileM;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base + Cfg::kOffQ;
  const uint32_t sK = smem_base + Cfg::kOffK;
  const uint32_t sV = smem_base + Cfg::kOffV;
  const uint32_t sP = smem_base + Cfg::kOffP;
  const uint32_t bar0 = smem_base + Cfg::kOffBar;
  // barrier slots (8 bytes each)
  const uint32_t bar_q_full = bar0;
  const uint32_t bar_k_full = bar0 + 8;     // [2]
  const uint32_t bar_k_empty = bar0 + 24;   // [2]
  const uint32_t bar_v_full = bar0 + 40;    // [2]
  const uint32_t bar_v_empty = bar0 + 56;   // [2]
  const uint32_t bar_s_full = bar0 + 72;    // [2]
  const uint32_t bar_s_free = bar0 + 88;    // [2]
  const uint32_t bar_p_full = bar0 + 104;
  const uint32_t bar_pv_done = bar0 + 112;

  const bool has_docs = prm.docs != nullptr;

  if (tid == 0 || tid == 32) {
    // Two planner threads, one per key stream (thread 0: the persistent stream, which holds the
    // diagonal; thread 32: the other parity).  Launched as a programmatic dependent of the document
    // pre-pass, the block has run up to here (and its producer warp sets up barriers, the Q load
    // and tensor memory) beside that kernel; its outputs are read from here on.
    grid_dependency_wait();
    const int slot = tid >> 5;
    // the global words the plan needs are asked for together (the document starts are read
    // whether or not the ids turn out monotone: the table exists whenever ids were given)
    int st_word = 0;
    if (slot == 0 && prm.status != nullptr) st_word = *reinterpret_cast<volatile int*>(prm.status);
    const int mono_b = (has_docs && prm.mono != nullptr) ? prm.mono[b] : 1;
    int lo0 = 0, lo1 = 0;
    if (has_docs && prm.lo != nullptr) {
      const int i1 = min(i0 + kTileM - 1, prm.N - 1);
      lo0 = prm.lo[(size_t)b * prm.N + i0];
      lo1 = prm.lo[(size_t)b * prm.N + i1];
    }
    SPS_TRACE(3 + 8 * slot, 15);
    if (mono_b == 0) lo0 = lo1 = 0;
    const bool two = prm.mask.ks != 1;
    const int stream = two ? (slot == 0 ? prm.mask.pp : 1 - prm.mask.pp) : 0;
    StreamPlan sp = plan_stream(prm.mask, i0, lo0, lo1, stream, kTileN);
    if (!two && slot == 1) sp.ntiles = 0;
    s_plan.sp[slot] = sp;
    s_plan.stream_id[slot] = stream;
    if (slot == 0) {
      // a failure reported by an earlier block turns every later block into a no-op
      s_abort = st_word != 0 ? 1 : 0;
      s_plan.general_docs = mono_b == 0 ? 1 : 0;
      s_plan.n_streams = two ? 2 : 1;
    }
    SPS_TRACE(4 + 8 * slot, 15);
  }
  if (warp == 4) {
    if (lane == 0) {
      mbar_init(bar_q_full, 1);
      for (int s = 0; s < 2; ++s) {
        mbar_init(bar_k_full + 8 * s, 1);
        mbar_init(bar_k_empty + 8 * s, 1);
        mbar_init(bar_v_full + 8 * s, 1);
        mbar_init(bar_v_empty + 8 * s, 1);
        mbar_init(bar_s_full + 8 * s, 1);
        mbar_init(bar_s_free + 8 * s, kSoftmaxArrivals);
      }
      mbar_init(bar_p_full, kSoftmaxArrivals);
      mbar_init(bar_pv_done, 1);
      fence_barrier_init();
      // the Q tile depends on nothing but the block index: start it before the plan is known
      tma_prefetch_desc(&tm_q);
      mbar_arrive_expect_tx(bar_q_full, Cfg::kQBytes);
      for (int c = 0; c < D / 64; ++c)
        tma_load_4d(sQ + c * Cfg::kQSubBytes, &tm_q, bar_q_full, c * 64, i0, h, b);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      SPS_TRACE(5, 15);
    }
    __syncwarp();
    tmem_alloc<Cfg::kTmemCols>(smem_u32(&s_tmem_base));
    if constexpr (Cfg::kPSplit) tmem_alloc<Cfg::kPCols>(smem_u32(&s_tmem_p));
    tmem_relinquish();
    if (lane == 0) SPS_TRACE(6, 15);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) SPS_TRACE(7, 15);
  grid_dependency_wait();   // every thread that reads the pre-pass outputs (thread 0 is past it)

  const uint32_t tmem = s_tmem_base;
  const uint32_t tmem_p = Cfg::kPSplit ? s_tmem_p : 0u;
  const int n_tiles = s_plan.sp[0].ntiles + s_plan.sp[1].ntiles;
  if (warp == 4 && n_tiles > 0 && s_abort == 0) {
    // the first K tile goes out as soon as the plan is known, before the tile table is built
    const TileInfo t = tile_info(s_plan, 0);
    if (elect_one()) {
      mbar_arrive_expect_tx(bar_k_full, Cfg::kKVBytes);
      for (int c = 0; c < D / 64; ++c)
        tma_load_5d(sK + c * Cfg::kKVSubBytes, &tm_k, bar_k_full, c * 64, t.stream, t.k0, h, b);
    }
    __syncwarp();
  }
  for (int j = tid; j < min(n_tiles, kTileTable); j += kPrefillThreads)
    s_tiles[j] = pack_tile(tile_info(s_plan, j));
  __syncthreads();
  if (tid == 0) SPS_TRACE(1, 15);
  volatile int* abort_flag = &s_abort;
  const bool bail = s_abort != 0;

  if (!bail && n_tiles > 0) {
    if (warp == 4) {
      // ------------------------------------------------------------------ TMA producer
      // converged warp, one elected lane issues the copies (tensor-map operands stay uniform)
      {
        auto load_k = [&](int j) {
          const TileInfo t = get_tile(s_plan, s_tiles, j);
          const int st = j % Cfg::kStagesK;
          if (j >= Cfg::kStagesK) {
            if (!warp_wait(bar_k_empty + 8 * st, ((j / Cfg::kStagesK) - 1) & 1, abort_flag, prm.status))
              return false;
          }
          if (elect_one()) {
            mbar_arrive_expect_tx(bar_k_full + 8 * st, Cfg::kKVBytes);
            for (int c = 0; c < D / 64; ++c)
              tma_load_5d(sK + st * Cfg::kKVBytes + c * Cfg::kKVSubBytes, &tm_k, bar_k_full + 8 * st,
                          c * 64, t.stream, t.k0, h, b);
          }
          __syncwarp();
          if (lane == 0) SPS_TRACE(j, 13);
          return true;
        };
        auto load_v = [&](int j) {
          const TileInfo t = get_tile(s_plan, s_tiles, j);
          const int st = j % Cfg::kStagesV;
          if (j >= Cfg::kStagesV) {
            if (!warp_wait(bar_v_empty + 8 * st, ((j / Cfg::kStagesV) - 1) & 1, abort_flag, prm.status))
              return false;
          }
          if (elect_one()) {
            mbar_arrive_expect_tx(bar_v_full + 8 * st, Cfg::kKVBytes);
            for (int c = 0; c < D / 64; ++c)
              tma_load_5d(sV + st * Cfg::kKVBytes + c * Cfg::kKVSubBytes, &tm_v, bar_v_full + 8 * st,
                          c * 64, t.stream, t.k0, h, b);
          }
          __syncwarp();
          if (lane == 0) SPS_TRACE(j, 14);
          return true;
        };
        bool ok = true;   // K tile 0 is on its way already
        for (int j = 0; ok && j < n_tiles; ++j) {
          if (j + 1 < n_tiles) ok = load_k(j + 1);
          if (ok) ok = load_v(j);
        }
      }
    } else if (warp == 5) {
      // ------------------------------------------------------------------ MMA issuer
      // The whole warp runs this loop converged (so descriptors and addresses stay in uniform
      // registers); one elected lane issues the tcgen05 instructions.
      {
        constexpr uint32_t idesc_qk = make_idesc_f16(FP16, kTileM, kTileN, false, false);
        constexpr uint32_t idesc_pv = make_idesc_f16(FP16, kTileM, D, false, true);
        // descriptors differ from tile to tile and K step to K step only in the start-address
        // field, which lives in the low 32 bits
        const uint64_t dq64 = make_smem_desc_sw128(sQ, 16, 1024);
        const uint64_t dk64 = make_smem_desc_sw128(sK, 16, 1024);
        const uint64_t dp64 = make_smem_desc_sw128(sP, 16, 1024);
        const uint64_t dv64 = make_smem_desc_sw128(sV, Cfg::kKVSubBytes, 1024);
        const uint32_t dq_lo = (uint32_t)dq64, dq_hi = (uint32_t)(dq64 >> 32);
        const uint32_t dk_lo = (uint32_t)dk64, dk_hi = (uint32_t)(dk64 >> 32);
        const uint32_t dp_lo = (uint32_t)dp64, dp_hi = (uint32_t)(dp64 >> 32);
        const uint32_t dv_lo = (uint32_t)dv64, dv_hi = (uint32_t)(dv64 >> 32);
        auto issue_qk = [&](int j) {
          const int st = j % Cfg::kStagesK;
          const int sb = j % Cfg::kSBufs;
          if (!warp_wait(bar_k_full + 8 * st, (j / Cfg::kStagesK) & 1, abort_flag, prm.status)) return false;
          if (j >= Cfg::kSBufs) {
            if (!warp_wait(bar_s_free + 8 * sb, ((j / Cfg::kSBufs) - 1) & 1, abort_flag, prm.status))
              return false;
          }
          tc_fence_after();
          const uint32_t kb0 = dk_lo + ((st * Cfg::kKVBytes) >> 4);
          const uint32_t sd = tmem + sb * kTileN;
          if (elect_one()) {
            // a K step of 16 elements is 32 bytes inside a 128-byte row; 64 elements per sub-tile
            umma_ss<false>(sd, dq_lo, dq_hi, kb0, dk_hi, idesc_qk);
#pragma unroll
            for (int kk = 1; kk < D / 16; ++kk) {
              const uint32_t qa = ((kk / 4) * Cfg::kQSubBytes + (kk % 4) * 32) >> 4;
              const uint32_t kb = ((kk / 4) * Cfg::kKVSubBytes + (kk % 4) * 32) >> 4;
              umma_ss<true>(sd, dq_lo + qa, dq_hi, kb0 + kb, dk_hi, idesc_qk);
            }
            umma_commit(bar_s_full + 8 * sb);
            umma_commit(bar_k_empty + 8 * st);
          }
          __syncwarp();
          if (lane == 0) SPS_TRACE(j, 9);
          return true;
        };
        bool ok = warp_wait(bar_q_full, 0, abort_flag, prm.status);
        if (ok) ok = issue_qk(0);
        for (int j = 0; ok && j < n_tiles; ++j) {
          if (j + 1 < n_tiles) ok = issue_qk(j + 1);
          if (!ok) break;
          const int st = j % Cfg::kStagesV;
          if (!warp_wait(bar_p_full, j & 1, abort_flag, prm.status)) break;
          if (lane == 0) SPS_TRACE(j, 10);
          if (!warp_wait(bar_v_full + 8 * st, (j / Cfg::kStagesV) & 1, abort_flag, prm.status)) break;
          if (lane == 0) SPS_TRACE(j, 11);
          tc_fence_after();
          const uint32_t vb0 = dv_lo + ((st * Cfg::kKVBytes) >> 4);
          const uint32_t od = tmem + Cfg::kColO;
          if (elect_one()) {
            // P: K-major, one 64-key sub-tile; V: MN-major, 16 key rows = 2048 bytes per step
            if constexpr (Cfg::kPTmem || Cfg::kPSplit) {
              // A from tensor memory: 16 keys = 8 packed columns per step
              const uint32_t pa = Cfg::kPSplit ? tmem_p : tmem + (j % Cfg::kSBufs) * kTileN;
#pragma unroll
              for (int kk = 0; kk < kTileN / 16; ++kk)
                umma_ts(od, pa + 8 * kk, vb0 + ((kk * 2048) >> 4), dv_hi, idesc_pv, j > 0 || kk > 0);
            } else {
              if (j > 0) {
                umma_ss<true>(od, dp_lo, dp_hi, vb0, dv_hi, idesc_pv);
              } else {
                umma_ss<false>(od, dp_lo, dp_hi, vb0, dv_hi, idesc_pv);
              }
#pragma unroll
              for (int kk = 1; kk < kTileN / 16; ++kk)
                umma_ss<true>(od, dp_lo + ((kk * 32) >> 4), dp_hi, vb0 + ((kk * 2048) >> 4), dv_hi, idesc_pv);
            }
            umma_commit(bar_pv_done);
            umma_commit(bar_v_empty + 8 * st);
          }
          __syncwarp();
          if (lane == 0) SPS_TRACE(j, 12);
        }
      }
    } else {
      // ------------------------------------------------------------------ softmax warps
      const int row = tid;                 // TMEM lane and query row inside the tile
      const int i = i0 + row;
      const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
      const bool general = s_plan.general_docs != 0;
      int lo_i = 0;
      if (has_docs && !general && i < prm.N) lo_i = prm.lo[(size_t)b * prm.N + i];
      int kmin_s[2], kmax_s[2];
      row_interval(prm.mask, i, lo_i, 0, kmin_s[0], kmax_s[0]);
      row_interval(prm.mask, i, lo_i, 1, kmin_s[1], kmax_s[1]);
      long long my_doc = 0;
      const uint8_t* docs_b = nullptr;
      if (general) {
        docs_b = reinterpret_cast<const uint8_t*>(prm.docs) +
                 (size_t)b * prm.doc_stride_b * (prm.doc_is_i64 ? 8 : 4);
        if (i < prm.N) {
          const size_t off = (size_t)i * prm.doc_stride_t;
          my_doc = prm.doc_is_i64 ? reinterpret_cast<const long long*>(docs_b)[off]
                                  : (long long)reinterpret_cast<const int*>(docs_b)[off];
        }
      }

      float m_run = -1.0e30f;   // running max of raw scores (finite sentinel)
      float l_run = 0.f;
      const float c = prm.scale_log2;
      bool ok = true;

      for (int j = 0; j < n_tiles; ++j) {
        const TileInfo t = get_tile(s_plan, s_tiles, j);
        const int sb = j % Cfg::kSBufs;
        if (tid == 0) SPS_TRACE(j, 0);
        if (!mbar_wait(bar_s_full + 8 * sb, (j / Cfg::kSBufs) & 1, abort_flag, prm.status)) {
          ok = false;
          break;
        }
        if (tid == 0) SPS_TRACE(j, 1);
        tc_fence_after();
        float s[kTileN];
        {
          uint32_t r0[32], r1[32];
          tmem_ld32(tmem + lane_addr + sb * kTileN, r0);
          tmem_ld32(tmem + lane_addr + sb * kTileN + 32, r1);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            s[e] = __uint_as_float(r0[e]);
            s[32 + e] = __uint_as_float(r1[e]);
          }
        }
        tc_fence_before();
        softmax_arrive(bar_s_free + 8 * sb, lane);
        if (tid == 0) SPS_TRACE(j, 2);

        if (t.masked) {
          // the visible columns of this row form an interval: build its bit mask once, then one
          // bit test per score instead of two comparisons
          const int cmin = max(kmin_s[t.stream] - t.k0, 0);
          const int cmax = min(kmax_s[t.stream] - t.k0, kTileN - 1);
          const unsigned long long vis =
              cmin > cmax ? 0ull : ((~0ull >> (63 - cmax)) & (~0ull << cmin));
          const uint32_t vis_lo = (uint32_t)vis, vis_hi = (uint32_t)(vis >> 32);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            if (!((vis_lo >> e) & 1u)) s[e] = -INFINITY;
            if (!((vis_hi >> e) & 1u)) s[32 + e] = -INFINITY;
          }
          if (general) {
            // ids are not monotone: compare this row's id with each key's id (uniform loads)
            uint32_t same[kTileN / 32];
#pragma unroll
            for (int q4 = 0; q4 < kTileN / 32; ++q4) {
              uint32_t bits = 0;
              for (int e = 0; e < 32; ++e) {
                const int jrow = prm.mask.ks * (t.k0 + q4 * 32 + e) + t.stream;
                if (jrow >= 0 && jrow < prm.N) {
                  const size_t off = (size_t)jrow * prm.doc_stride_t;
                  const long long dk = prm.doc_is_i64
                                           ? reinterpret_cast<const long long*>(docs_b)[off]
                                           : (long long)reinterpret_cast<const int*>(docs_b)[off];
                  bits |= (dk == my_doc ? 1u : 0u) << e;
                }
              }
              same[q4] = bits;
            }
#pragma unroll
            for (int e = 0; e < kTileN; ++e)
              if (!((same[e >> 5] >> (e & 31)) & 1u)) s[e] = -INFINITY;
          }
        }
        float mx;
        {
          float m4[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) m4[x] = fmax3(s[x], s[4 + x], s[8 + x]);
#pragma unroll
          for (int e = 12; e + 8 <= kTileN; e += 8) {
#pragma unroll
            for (int x = 0; x < 4; ++x) m4[x] = fmax3(m4[x], s[e + x], s[e + 4 + x]);
          }
#pragma unroll
          for (int x = 0; x < 4; ++x) m4[x] = fmaxf(m4[x], s[kTileN - 4 + x]);
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        if (tid == 0) SPS_TRACE(j, 3);
        // Lazy rescaling: the exponent offset m_run only moves when some row of the warp grew by
        // more than 2^kRescaleLog2; until then P may exceed 1 (by at most that factor), which
        // fp32 accumulation and the final division by l absorb exactly.
        float alpha = 1.0f;
        const bool grow = (mx - m_run) * c > kRescaleLog2;
        const bool rescale = __any_sync(0xffffffffu, grow);
        if (rescale) {
          const float m_new = fmaxf(m_run, mx);
          alpha = fast_exp2((m_run - m_new) * c);
          l_run *= alpha;
          m_run = m_new;
        }
        const float neg_mc = -m_run * c;
        // packed fp32x2 arithmetic (sm_100): one FFMA2 scales and offsets two scores, one FADD2
        // accumulates two probabilities; the exponentials stay one MUFU each
        const float2 c2 = make_float2(c, c), nm2 = make_float2(neg_mc, neg_mc);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
        uint32_t pk[kTileN / 2];
#ifdef SPSATTN_EXP_PAIRWISE
#pragma unroll
        for (int e = 0; e < kTileN; e += 4) {
          const float2 xa = __ffma2_rn(make_float2(s[e], s[e + 1]), c2, nm2);
          const float2 xb = __ffma2_rn(make_float2(s[e + 2], s[e + 3]), c2, nm2);
          const float2 pa = make_float2(fast_exp2(xa.x), fast_exp2(xa.y));
          const float2 pb = make_float2(fast_exp2(xb.x), fast_exp2(xb.y));
          sum_a = __fadd2_rn(sum_a, pa);
          sum_b = __fadd2_rn(sum_b, pb);
          pk[e / 2] = pack2<FP16>(pa.x, pa.y);
          pk[e / 2 + 1] = pack2<FP16>(pb.x, pb.y);
        }
#else
        // Written as a software pipeline: all exponents first, then the exponentials in groups
        // of eight issued back to back (their order is pinned), each group followed by the row
        // sum and the packing of the group before it.  No add or pack then waits for an
        // exponential that was asked for an instruction earlier, and the special-function unit
        // is fed without gaps.
#pragma unroll
        for (int e = 0; e < kTileN; e += 2) {
          const float2 xv = __ffma2_rn(make_float2(s[e], s[e + 1]), c2, nm2);
          s[e] = xv.x;
          s[e + 1] = xv.y;
        }
#pragma unroll
        for (int grp = 0; grp <= kTileN / 8; ++grp) {
          if (grp < kTileN / 8) {
#pragma unroll
            for (int e = grp * 8; e < grp * 8 + 8; ++e) s[e] = ex2_ordered(s[e]);
          }
          if (grp > 0) {
#pragma unroll
            for (int e = (grp - 1) * 8; e < grp * 8; e += 4) {
              sum_a = __fadd2_rn(sum_a, make_float2(s[e], s[e + 1]));
              sum_b = __fadd2_rn(sum_b, make_float2(s[e + 2], s[e + 3]));
              pk[e / 2] = pack2<FP16>(s[e], s[e + 1]);
              pk[e / 2 + 1] = pack2<FP16>(s[e + 2], s[e + 3]);
            }
          }
        }
#endif
        l_run += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        if (tid == 0) SPS_TRACE(j, 4);

        // The shared-memory P tile is free, and O may be rescaled, once the previous P V product is
        // done.  P in tensor memory may be written before that (the S this thread read was written
        // after the last product that read these columns, in issue order), so there the wait comes
        // after the P write; it is still made for every tile: a parity wait is only meaningful for
        // a waiter that has consumed every earlier phase of the barrier.
        if (!Cfg::kPTmem && j > 0) {      // also the columns of a P of its own (kPSplit)
          if (!mbar_wait(bar_pv_done, (j - 1) & 1, abort_flag, prm.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
        }
        if (tid == 0) SPS_TRACE(j, 5);
        if constexpr (Cfg::kPTmem) {
#pragma unroll
          for (int q8 = 0; q8 < kTileN / 16; ++q8)
            tmem_st8(tmem + lane_addr + sb * kTileN + 8 * q8, pk + 8 * q8);
        }
        if constexpr (Cfg::kPSplit) {
          tmem_st16(tmem_p + lane_addr, pk);
          tmem_st16(tmem_p + lane_addr + 16, pk + 16);
        }
        // P -> shared memory, K-major 128B-swizzled: 16-byte chunk ch of row r sits at
        // r * 128 + ((ch ^ (r & 7)) << 4) of the [128 x 64] tile
#pragma unroll
        for (int ch = 0; ch < ((Cfg::kPTmem || Cfg::kPSplit) ? 0 : 8); ++ch) {
          const uint32_t addr = sP + row * 128 + ((ch ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[ch * 4]),
                       "r"(pk[ch * 4 + 1]), "r"(pk[ch * 4 + 2]), "r"(pk[ch * 4 + 3])
                       : "memory");
        }
        if (tid == 0) SPS_TRACE(j, 6);
        if (Cfg::kPTmem && j > 0) {
          if (!mbar_wait(bar_pv_done, (j - 1) & 1, abort_flag, prm.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
        }
        if (j > 0 && rescale) {
#pragma unroll
          for (int q4 = 0; q4 < D / 32; ++q4) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_addr + Cfg::kColO + q4 * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st32(tmem + lane_addr + Cfg::kColO + q4 * 32, r);
          }
          tmem_wait_st();
        }
        if (tid == 0) SPS_TRACE(j, 7);
        if constexpr (Cfg::kPTmem || Cfg::kPSplit) tmem_wait_st();
        else fence_proxy_async_smem();
        tc_fence_before();
        softmax_arrive(bar_p_full, lane);
        if (tid == 0) SPS_TRACE(j, 8);
      }

      // ---------------------------------------------------------------- epilogue
      if (ok) ok = mbar_wait(bar_pv_done, (n_tiles - 1) & 1, abort_flag, prm.status);
      if (ok) {
        tc_fence_after();
        const float inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
        uint8_t* o_row = reinterpret_cast<uint8_t*>(prm.o) +
                         (b * prm.o_stride_b + h * prm.o_stride_h + i * prm.o_stride_n) * 2;
#pragma unroll
        for (int q4 = 0; q4 < D / 32; ++q4) {
          uint32_t r[32];
          tmem_ld32(tmem + lane_addr + Cfg::kColO + q4 * 32, r);
          tmem_wait_ld();
          if (i < prm.N) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 u;
              u.x = pack2<FP16>(__uint_as_float(r[e]) * inv_l, __uint_as_float(r[e + 1]) * inv_l);
              u.y = pack2<FP16>(__uint_as_float(r[e + 2]) * inv_l, __uint_as_float(r[e + 3]) * inv_l);
              u.z = pack2<FP16>(__uint_as_float(r[e + 4]) * inv_l, __uint_as_float(r[e + 5]) * inv_l);
              u.w = pack2<FP16>(__uint_as_float(r[e + 6]) * inv_l, __uint_as_float(r[e + 7]) * inv_l);
              *reinterpret_cast<uint4*>(o_row + q4 * 64 + e * 2) = u;
            }
          }
        }
        if (prm.lse != nullptr && i < prm.N)
          prm.lse[(size_t)bh * prm.N + i] = l_run > 0.f ? m_run * c + log2f(l_run) : -INFINITY;
        tc_fence_before();
      }
    }
  } else if (!bail && warp < 4) {
    // nothing visible for any row of this tile: outputs are zero
    const int i = i0 + tid;
    if (i < prm.N) {
      uint4* o_row = reinterpret_cast<uint4*>(
          reinterpret_cast<uint8_t*>(prm.o) +
          (b * prm.o_stride_b + h * prm.o_stride_h + i * prm.o_stride_n) * 2);
      for (int e = 0; e < D / 8; ++e) o_row[e] = make_uint4(0, 0, 0, 0);
      if (prm.lse != nullptr) prm.lse[(size_t)bh * prm.N + i] = -INFINITY;
    }
  }

  // the Q tile load was started before the plan was known: never leave with it in flight
  if (warp == 4 && lane == 0) mbar_wait(bar_q_full, 0, abort_flag, prm.status);
  __syncthreads();
  if (tid == 0) SPS_TRACE(2, 15);
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc<Cfg::kTmemCols>(tmem);
    if constexpr (Cfg::kPSplit) tmem_dealloc<Cfg::kPCols>(tmem_p);
  }
}

}  // namespace spsattn
