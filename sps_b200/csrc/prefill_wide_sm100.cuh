// SPS prefill attention at head_dim 64 for sm_100a: persistent blocks, 128-key tiles, P in
// tensor memory.
//
// Two blocks per SM stay resident and draw work items (one 128-row query tile of one (batch,
// head), heavy tiles first, tiles of a head adjacent so that its K/V stay in L2) from a counter,
// so no SM waits for a block launch between items and the last items of a launch are the light
// ones.  Roles as in prefill_sm100.cuh: warps 0-3 softmax (thread r owns query row r = TMEM lane
// r), warp 4 producer, warp 5 MMA issuer.
//
//   producer   draws the next item while the others still work on the current one: plan, tile
//              table and the rows' document starts go to one of two item slots in shared memory,
//              the Q tile to one of two Q buffers, K/V tiles (128 key tokens of one parity stream,
//              16 KB each) through one ring that runs on across items
//   MMA        S = Q K_j^T (128x128x64) into tensor-memory columns [0,128); O += P V_j as two
//              products of 64 keys each, A operand read from tensor memory (P, columns [128,192)),
//              V consumed as the MN-major B operand as TMA delivered it; O in columns [192,256)
//   softmax    32 score columns at a time: tcgen05.ld of the next chunk is in flight while the
//              current one is processed (online softmax per chunk, lazy rescaling), so a thread
//              holds 64 scores at most and the compiler has registers left to overlap the
//              exponentials; P of 64 keys is written with tcgen05.st and handed to the MMA warp,
//              whose product then runs under the exponentials of the other 64 keys
//
// On a masked tile each warp classifies its four chunks: a chunk hidden from all 32 rows costs no
// load and no exponentials (P = 0), a chunk visible to all of them no mask tests, and only mixed
// chunks test one bit per score.  The epilogue of an item (O / l, 16-byte stores) runs while the
// MMA warp already multiplies the next item's first tile.
// Reference computation: src/modeling/models/attention/triton_sps_flash_attention.py:26-139,
// :147-269 (and the reverse / standard variants).
#pragma once

#include <type_traits>

#include "prefill_sm100.cuh"

namespace spsattn {

constexpr int kWideN = 128;          // key tokens per tile
constexpr int kWideThreads = 192;
constexpr int kWideChunk = 32;       // score columns per softmax step

// Of every four packed score pairs, how many take their exponential on the FMA pipes
// (Cody-Waite range reduction + cubic) instead of the special-function unit.
// tuning builds only: shortened row-maximum scan
#ifdef SPSATTN_ABL_NOMAX
#define ABL_MAXLEN 16
#else
#define ABL_MAXLEN kWideChunk
#endif
#ifndef SPSATTN_WIDE_POLY
#define SPSATTN_WIDE_POLY 0
#endif

// Tuning builds (-DSPSATTN_TRACE): lane 0 of every warp of blocks 0 and 1 logs (event id, clock)
// pairs into shared memory and dumps them at the end; compiled out otherwise.
constexpr int kWideTraceEvents = 160;
#ifdef SPSATTN_TRACE
#define WTR(id)                                                                                    \
  do {                                                                                             \
    if (wtr_buf != nullptr && (threadIdx.x & 31) == 0 && *wtr_n < kWideTraceEvents)                \
      wtr_buf[(*wtr_n)++] = ((long long)(id) << 48) | (clock64() & 0xffffffffffffll);              \
  } while (0)
#else
#define WTR(id) do { } while (0)
#endif

struct WideCfg {
  static constexpr int kStagesK = 2;
  static constexpr int kStagesV = 2;
  static constexpr uint32_t kTmemCols = 256;
  static constexpr uint32_t kColS = 0;
  static constexpr uint32_t kColP = 128;
  static constexpr uint32_t kColO = 192;
  static constexpr int kQBytes = kTileM * 64 * 2;
  static constexpr int kKVBytes = kWideN * 64 * 2;
  static constexpr int kOffQ = 0;                                   // two Q buffers
  static constexpr int kOffK = kOffQ + 2 * kQBytes;
  static constexpr int kOffV = kOffK + kStagesK * kKVBytes;
  static constexpr int kOffBar = kOffV + kStagesV * kKVBytes;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;          // barriers + alignment slack
};

// One work item as the producer publishes it to the other roles.
struct WideItem {
  BlockPlan plan;
  int item;                 // index of the item, -1 = no more work
  int i0, b, h, bh;
  int tiles[kTileTable];
  int lo[kTileM];           // first row of each query row's document run
};

// 2^x for two scores at once on the FMA pipes: n = round(x) through the 1.5 * 2^23 trick,
// f = x - n in [-0.5, 0.5], minimax cubic for 2^f (relative error 7.5e-5, below the rounding of a
// 16-bit P), n added into the exponent field.  x is clamped so that the result stays normal.
__device__ __forceinline__ float2 poly_exp2x2(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 magic = make_float2(12582912.f, 12582912.f);
  const float2 xr = __fadd2_rn(x, magic);
  const float2 t = __fadd2_rn(xr, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(t, make_float2(-1.f, -1.f), x);
  float2 p = __ffma2_rn(make_float2(0.05517166f, 0.05517166f), f, make_float2(0.24261113f, 0.24261113f));
  p = __ffma2_rn(p, f, make_float2(0.69326097f, 0.69326097f));
  p = __ffma2_rn(p, f, make_float2(0.99992806f, 0.99992806f));
  float2 y;
  y.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(xr.x) << 23));
  y.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(xr.y) << 23));
  return y;
}

// bit e = 1 iff key row j0 + e * step exists and carries the document id my_doc
__device__ __forceinline__ uint32_t same_doc_bits(const uint8_t* docs_b, int is_i64, int64_t stride_t,
                                                  long long my_doc, int j0, int step, int n_rows) {
  uint32_t bits = 0;
  for (int e = 0; e < 32; ++e) {
    const int jrow = j0 + e * step;
    if (jrow >= 0 && jrow < n_rows) {
      const size_t off = (size_t)jrow * stride_t;
      const long long dk = is_i64 ? reinterpret_cast<const long long*>(docs_b)[off]
                                  : (long long)reinterpret_cast<const int*>(docs_b)[off];
      bits |= (dk == my_doc ? 1u : 0u) << e;
    }
  }
  return bits;
}

// What a softmax thread carries into the tile loop of an item and gets back from it.
struct WideSoftmaxCtx {
  const PrefillParams* prm;
  const WideItem* slot;
  volatile int* abort_flag;
  uint32_t tmem_row;                 // tensor-memory address of this warp's lanes, column 0
  uint32_t bar_s_full, bar_s_free, bar_p_full, bar_pv_done;   // each [2] (one per 64-key half), 8 bytes apart
  int n_tiles, lane;
  int kmin_s[2], kmax_s[2];          // visible key tokens of this row, per stream
  const uint8_t* docs_b;             // ids of this batch row (non-monotone ids only)
  long long my_doc;
  bool general;
  uint32_t g;                        // tiles this block has processed so far (barrier phases)
  float m_run, l_run;                // running maximum (raw scores) and row sum
  bool ok;
  long long* wtr_buf;                // tuning builds: event log of this warp, or null
  int* wtr_n;
};

// The tile loop of one softmax thread for one item.  For batch rows whose ids are not monotone
// (`general`) the ids are compared element by element at the start of a tile, while few
// registers are live, and kept as one word per chunk.
template <bool FP16>
__device__ __forceinline__ void wide_softmax_tiles(WideSoftmaxCtx& x) {
  using Cfg = WideCfg;
  constexpr int D = 64;
  constexpr uint32_t kNegInf = 0xff800000u;
  constexpr int kChunks = kWideN / kWideChunk;
  const PrefillParams& prm = *x.prm;
  const WideItem& slot = *x.slot;
  volatile int* abort_flag = x.abort_flag;
  const uint32_t tmem_row = x.tmem_row;
  const uint32_t bar_s_full = x.bar_s_full, bar_s_free = x.bar_s_free, bar_p_full = x.bar_p_full,
                 bar_pv_done = x.bar_pv_done;
  const int n_tiles = x.n_tiles, lane = x.lane;
  const int kmin_s[2] = {x.kmin_s[0], x.kmin_s[1]}, kmax_s[2] = {x.kmax_s[0], x.kmax_s[1]};
  const uint8_t* docs_b = x.docs_b;
  const long long my_doc = x.my_doc;
  const bool general = x.general;
  uint32_t g = x.g;
  float m_run = x.m_run, l_run = x.l_run;
  const float c = prm.scale_log2;
  bool ok = true;
  long long* wtr_buf = x.wtr_buf;
  int* wtr_n = x.wtr_n;
  (void)wtr_buf;
  (void)wtr_n;
  uint32_t ra[kWideChunk], rb[kWideChunk];      // scores of the even / odd chunk in flight
  bool ahead = false;     // chunk 0 of the coming tile was requested at the end of the last one

  for (int j = 0; j < n_tiles && ok; ++j, ++g) {
    const TileInfo t = get_tile<kWideN>(slot.plan, slot.tiles, j);
    // which chunks this warp works on (bit ch) and which of those need the per-score mask
    // (bit 4 + ch), decided for the warp as a whole; the visible columns of a row form an
    // interval, so the chunks a warp works on are consecutive
    uint32_t run = 0xfu;
    int cmin = 0, cmax = kWideN - 1;
    if (t.masked) {
      run = 0;
      cmin = max(kmin_s[t.stream] - t.k0, 0);
      cmax = min(kmax_s[t.stream] - t.k0, kWideN - 1);
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        const int lo_c = kWideChunk * ch, hi_c = kWideChunk * ch + kWideChunk - 1;
        const bool any = cmin <= cmax && cmax >= lo_c && cmin <= hi_c;
        const bool all = cmin <= lo_c && cmax >= hi_c;
        if (__any_sync(0xffffffffu, any)) {
          run |= 1u << ch;
          if (general || !__all_sync(0xffffffffu, all)) run |= 16u << ch;
        }
      }
    }
    uint32_t docw[kChunks] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
    if (general) {
      // which keys of each chunk carry this row's document id (uniform loads), while few
      // registers are live
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch)
        if ((run >> ch) & 1u)
          docw[ch] = same_doc_bits(docs_b, prm.doc_is_i64, prm.doc_stride_t, my_doc,
                                   prm.mask.ks * (t.k0 + ch * kWideChunk) + t.stream, prm.mask.ks, prm.N);
    }
    const int first = (run & 0xfu) ? __ffs(run & 0xfu) - 1 : kChunks;   // first chunk worked on
    // S arrives as two halves of 64 columns with a barrier pair each (warp-uniform outcomes: the
    // tensor-memory accesses need the whole warp).  The first chunk this warp needs is requested
    // here unless the previous tile already did; every later one while its predecessor runs.
    bool have1 = false;                                      // second half of S waited for
    if (!ahead) {
      if (!warp_wait(bar_s_full, g & 1u, abort_flag, prm.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (first >= 2 && first < kChunks) {
        if (!warp_wait(bar_s_full + 8, g & 1u, abort_flag, prm.status)) {
          ok = false;
          break;
        }
        tc_fence_after();
        have1 = true;
      }
      if (first < kChunks) {
        if (first & 1) tmem_ld32p(tmem_row + Cfg::kColS + first * kWideChunk, rb);
        else tmem_ld32p(tmem_row + Cfg::kColS + first * kWideChunk, ra);
      }
    }
    ahead = false;
    // may the first chunk of the next tile be requested from this one?  (only when that tile
    // needs no classification: all four chunks are worked on)
    const bool next_plain = j + 1 < n_tiles && !get_tile<kWideN>(slot.plan, slot.tiles, j + 1).masked;

    // Software pipeline over the four chunks, written out by hand because the exponentials are
    // what the kernel is bound by: the 32 exp2 of a chunk are issued in groups of eight, and
    // between the groups go the row sum and the packing of the group before, the mask and the
    // row maximum of the NEXT chunk (its scores arrive while this chunk's exponentials run) and
    // the hand-over of the finished half of P, so the special-function unit idles only for the
    // decision about the exponent offset and the scaling of the next chunk.
    uint32_t pk_a[kWideChunk / 2], pk_b[kWideChunk / 2];     // P of the even / odd chunk of a half
    bool handed0 = false;                                    // half 0 of P given to the MMA warp
    const float2 c2 = make_float2(c, c);
    auto give_half0 = [&]() {
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full);
      handed0 = true;
    };
    // hide the scores of chunk cn that this row must not see: one bit test per score
    auto mask_chunk = [&](int cn, uint32_t* y) {
      const int a = max(cmin - kWideChunk * cn, 0), bb = min(cmax - kWideChunk * cn, kWideChunk - 1);
      uint32_t word = (cmin <= cmax && a <= bb) ? ((0xffffffffu >> (31 - bb)) & (0xffffffffu << a)) : 0u;
      word &= docw[cn];
#pragma unroll
      for (int e = 0; e < kWideChunk; ++e)
        if (!((word >> e) & 1u)) y[e] = kNegInf;
    };
    // Exponent offset for chunk cn whose row maximum is mx, then the chunk's scores y become
    // exponents in place.  Lazy rescaling: the offset m_run only moves when some row of the warp
    // grew by more than 2^kRescaleLog2; until then P may exceed 1 (by at most that factor), which
    // fp32 accumulation and the final division by l absorb exactly.
    auto decide_and_scale = [&](int cn, float mx, uint32_t* y) -> bool {
      const bool grow = (mx - m_run) * c > kRescaleLog2;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_run, mx);
        const float alpha = fast_exp2((m_run - m_new) * c);
        l_run *= alpha;
        m_run = m_new;
        if (cn & 1) {
          // P of the other chunk of this half is still with this thread
#pragma unroll
          for (int e = 0; e < kWideChunk / 2; ++e) {
            float lo_f, hi_f;
            unpack2<FP16>(pk_a[e], lo_f, hi_f);
            pk_a[e] = pack2<FP16>(lo_f * alpha, hi_f * alpha);
          }
        }
        if (j > 0 || cn >= 2) {
          // O holds products at the old offset: the last one issued must be done (and, for that,
          // half 0 of this tile's P handed over if it is the one); every earlier phase of that
          // barrier has been waited for at its regular place
          if (cn >= 2 && !handed0) give_half0();
          const uint32_t bar = cn >= 2 ? bar_pv_done : bar_pv_done + 8;
          const uint32_t ph = cn >= 2 ? (g & 1u) : ((g - 1u) & 1u);
          if (!warp_wait(bar, ph, abort_flag, prm.status)) return false;
          tc_fence_after();
          // (rare: 16 columns at a time keeps this path's registers out of the common one's way;
          // its wait::ld also covers a score chunk in flight, which is harmless)
#pragma unroll 1
          for (int q = 0; q < D / 16; ++q) {
            uint32_t o[16];
            tmem_ld16(tmem_row + Cfg::kColO + q * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st16(tmem_row + Cfg::kColO + q * 16, o);
          }
          tmem_wait_st();
        }
      }
      const float neg_mc = -m_run * c;
      const float2 nm2 = make_float2(neg_mc, neg_mc);
#pragma unroll
      for (int e = 0; e < kWideChunk; e += 2) {
        const float2 xv = __ffma2_rn(make_float2(__uint_as_float(y[e]), __uint_as_float(y[e + 1])), c2, nm2);
        y[e] = __float_as_uint(xv.x);
        y[e + 1] = __float_as_uint(xv.y);
      }
      return true;
    };
    auto max32 = [&](const uint32_t* y) {
      float m4[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) m4[q] = fmax3(__uint_as_float(y[q]), __uint_as_float(y[4 + q]), __uint_as_float(y[8 + q]));
#pragma unroll
      for (int e = 12; e + 8 <= kWideChunk; e += 8) {
#pragma unroll
        for (int q = 0; q < 4; ++q) m4[q] = fmax3(m4[q], __uint_as_float(y[e + q]), __uint_as_float(y[e + 4 + q]));
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) m4[q] = fmaxf(m4[q], __uint_as_float(y[kWideChunk - 4 + q]));
      return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
    };

    if (run & 1u) {
      // chunk 0 has no predecessor to hide behind
      tmem_wait_ld();
      if (run & 2u) tmem_ld32p(tmem_row + Cfg::kColS + kWideChunk, rb);     // chunk 1, same half of S
      if (run & 16u) mask_chunk(0, ra);
      if (!decide_and_scale(0, max32(ra), ra)) {
        ok = false;
        break;
      }
    }

    auto step = [&](auto ch_tag) -> bool {
      constexpr int ch = decltype(ch_tag)::value;
      uint32_t* X = (ch & 1) ? rb : ra;                      // exponents of this chunk
      uint32_t* Y = (ch & 1) ? ra : rb;                      // scores of the next chunk
      uint32_t* PK = (ch & 1) ? pk_b : pk_a;
      const bool mine = (run >> ch) & 1u;
      const bool nxt = ch + 1 < kChunks && ((run >> (ch + 1)) & 1u);
      float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
      auto exp8 = [&](int base) {
#pragma unroll
        for (int e = base; e < base + 8; ++e) X[e] = __float_as_uint(ex2_ordered(__uint_as_float(X[e])));
      };
      auto consume8 = [&](int base) {
#pragma unroll
        for (int e = base; e < base + 8; e += 4) {
          sum_a = __fadd2_rn(sum_a, make_float2(__uint_as_float(X[e]), __uint_as_float(X[e + 1])));
          sum_b = __fadd2_rn(sum_b, make_float2(__uint_as_float(X[e + 2]), __uint_as_float(X[e + 3])));
          PK[e / 2] = pack2<FP16>(__uint_as_float(X[e]), __uint_as_float(X[e + 1]));
          PK[e / 2 + 1] = pack2<FP16>(__uint_as_float(X[e + 2]), __uint_as_float(X[e + 3]));
        }
      };
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (mine) {
        exp8(0);
        exp8(8);
        consume8(0);
      }
      if (ch == 2 && !handed0) give_half0();                 // its tcgen05.st were issued in step 1
      if (nxt) {
        // chunk ch + 1 is in Y (requested by the step before, or at the start of the tile)
        tmem_wait_ld();
      }
      if (ch == 0 || ch == 2) {
        // everything this warp needs of this half of S is read (chunk ch + 1 just now, or not
        // needed): the next tile's product may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_free + 8 * (ch >> 1));
      }
      if (nxt && ((run >> (5 + ch)) & 1u)) mask_chunk(ch + 1, Y);
      if (mine) {
        exp8(16);
        consume8(8);
      }
      if (nxt) {
#pragma unroll
        for (int q = 0; q < 4; ++q) m4[q] = fmax3(__uint_as_float(Y[q]), __uint_as_float(Y[4 + q]), __uint_as_float(Y[8 + q]));
#pragma unroll
        for (int q = 0; q < 4; ++q) m4[q] = fmax3(m4[q], __uint_as_float(Y[12 + q]), __uint_as_float(Y[16 + q]));
      }
      if (mine) {
        exp8(24);
        consume8(16);
      }
      if (nxt) {
#pragma unroll
        for (int q = 0; q < 4; ++q) m4[q] = fmax3(m4[q], __uint_as_float(Y[20 + q]), __uint_as_float(Y[24 + q]));
#pragma unroll
        for (int q = 0; q < 4; ++q) m4[q] = fmaxf(m4[q], __uint_as_float(Y[28 + q]));
      }
      if (mine) {
        consume8(24);
        l_run += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
      } else {
#pragma unroll
        for (int e = 0; e < kWideChunk / 2; ++e) PK[e] = 0u;
      }
      if (ch & 1) {
        // P of 64 keys is complete; its columns are free once the product that read them one
        // tile ago is done (long since, in the steady state)
        const int half = ch >> 1;
        if (g > 0) {
          if (!warp_wait(bar_pv_done + 8 * half, (g - 1u) & 1u, abort_flag, prm.status)) return false;
          tc_fence_after();
        }
        tmem_st16(tmem_row + Cfg::kColP + 32 * half, pk_a);
        tmem_st16(tmem_row + Cfg::kColP + 32 * half + 16, pk_b);
        if (ch == 3) {
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_p_full + 8);
        }
      }
      if (ch < 3) {
        if (ch == 0 && !have1) {
          // the other half of S (there long since, in the steady state)
          if (!warp_wait(bar_s_full + 8, g & 1u, abort_flag, prm.status)) return false;
          tc_fence_after();
          have1 = true;
        }
        // X is free: the chunk after next goes there, unless it is the one the tile started with
        if (ch < 2) {
          if (((run >> (ch + 2)) & 1u) && ch + 2 != first)
            tmem_ld32p(tmem_row + Cfg::kColS + (ch + 2) * kWideChunk, X);
        }
        if (nxt) {
          if (!decide_and_scale(ch + 1, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])), Y)) return false;
        }
      } else if (next_plain) {
        // first chunk of the next tile (ra is free since step 2)
        if (!warp_wait(bar_s_full, (g + 1u) & 1u, abort_flag, prm.status)) return false;
        tc_fence_after();
        tmem_ld32p(tmem_row + Cfg::kColS, ra);
        ahead = true;
      }
      return true;
    };
    ok = step(std::integral_constant<int, 0>{}) && step(std::integral_constant<int, 1>{}) &&
         step(std::integral_constant<int, 2>{}) && step(std::integral_constant<int, 3>{});
  }
  x.g = g;
  x.m_run = m_run;
  x.l_run = l_run;
  x.ok = ok;
}

template <bool FP16>
__global__ void __launch_bounds__(kWideThreads, 2)
prefill_wide_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v,
                          const __grid_constant__ PrefillParams prm) {
  using Cfg = WideCfg;
  constexpr int D = 64;
  extern __shared__ uint8_t smem_raw[];
  __shared__ WideItem s_item[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
#ifdef SPSATTN_TRACE
  __shared__ long long s_wtr[6][kWideTraceEvents];
  __shared__ int s_wtr_n[6];
#endif

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
#ifdef SPSATTN_TRACE
  long long* wtr_buf = (prm.trace != nullptr && blockIdx.x < 2) ? s_wtr[warp] : nullptr;
  int* wtr_n = &s_wtr_n[warp];
  if (lane == 0) s_wtr_n[warp] = 0;
  __syncwarp();
#else
  long long* wtr_buf = nullptr;
  int* wtr_n = nullptr;
  (void)wtr_buf;
  (void)wtr_n;
#endif

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base + Cfg::kOffQ;
  const uint32_t sK = smem_base + Cfg::kOffK;
  const uint32_t sV = smem_base + Cfg::kOffV;
  const uint32_t bar0 = smem_base + Cfg::kOffBar;
  // barrier slots (8 bytes each)
  const uint32_t bar_item_full = bar0;        // [2] producer -> MMA and softmax warps
  const uint32_t bar_item_free = bar0 + 16;   // [2] MMA warp + 4 softmax warps -> producer
  const uint32_t bar_q_full = bar0 + 32;      // [2]
  const uint32_t bar_q_free = bar0 + 48;      // [2] last Q K^T of the item done
  const uint32_t bar_k_full = bar0 + 64;      // [2]
  const uint32_t bar_k_empty = bar0 + 80;     // [2]
  const uint32_t bar_v_full = bar0 + 96;      // [2]
  const uint32_t bar_v_empty = bar0 + 112;    // [2]
  const uint32_t bar_s_full = bar0 + 128;     // [2] one per 64-key half of a tile
  const uint32_t bar_s_free = bar0 + 144;     // [2]
  const uint32_t bar_p_full = bar0 + 160;     // [2]
  const uint32_t bar_pv_done = bar0 + 176;    // [2]

  const bool has_docs = prm.docs != nullptr;
  const int total_items = prm.n_qtiles * prm.B * prm.H;

  if (tid == 0)
    // a failure reported by an earlier launch or block turns this block into a no-op
    s_abort = (prm.status != nullptr && *reinterpret_cast<volatile int*>(prm.status) != 0) ? 1 : 0;
  if (warp == 4) {
    if (lane == 0) {
      for (int s = 0; s < 2; ++s) {
        mbar_init(bar_item_full + 8 * s, 1);
        mbar_init(bar_item_free + 8 * s, 5);
        mbar_init(bar_q_full + 8 * s, 1);
        mbar_init(bar_q_free + 8 * s, 1);
        mbar_init(bar_k_full + 8 * s, 1);
        mbar_init(bar_k_empty + 8 * s, 1);
        mbar_init(bar_v_full + 8 * s, 1);
        mbar_init(bar_v_empty + 8 * s, 1);
        mbar_init(bar_s_full + 8 * s, 1);
        mbar_init(bar_s_free + 8 * s, 4);     // one arrival per softmax warp
        mbar_init(bar_p_full + 8 * s, 4);
        mbar_init(bar_pv_done + 8 * s, 1);
      }
      fence_barrier_init();
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
    }
    __syncwarp();
    tmem_alloc<Cfg::kTmemCols>(smem_u32(&s_tmem_base));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (s_abort == 0) {
    if (warp == 4) {
      // ------------------------------------------------------------------ producer
      // converged warp; one elected lane issues the copies (tensor-map operands stay uniform)
      uint32_t gk = 0, gv = 0;        // K / V tiles requested so far (ring positions)
      uint32_t q_loads0 = 0, q_loads1 = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        const int buf = n & 1u;
        WideItem& slot = s_item[buf];
        if (n >= 2) {
          if (!warp_wait(bar_item_free + 8 * buf, ((n >> 1) - 1u) & 1u, abort_flag, prm.status)) break;
        }
        // next item: from the counter when the caller gave one, else a fixed stride
        int item = 0;
        if (lane == 0)
          item = prm.work_counter != nullptr ? atomicAdd(prm.work_counter, 1)
                                             : (int)(blockIdx.x + n * gridDim.x);
        item = __shfl_sync(0xffffffffu, item, 0);
        WTR(94);
        if (item >= total_items) {
          if (lane == 0) {
            slot.item = -1;
            mbar_arrive(bar_item_full + 8 * buf);
          }
          break;
        }
        // (batch, head) pairs go in groups whose K/V fit L2 together; inside a group the late
        // (heavy) query tiles of all its heads come first, so a launch ends on light items
        const int per_group = prm.group_heads * prm.n_qtiles;
        const int grp = item / per_group;
        const int in_grp = item - grp * per_group;
        const int gsize = min(prm.group_heads, prm.B * prm.H - grp * prm.group_heads);
        const int bh = grp * prm.group_heads + in_grp % gsize;
        const int qt = prm.n_qtiles - 1 - in_grp / gsize;
        const int b = bh / prm.H;
        const int h = bh - b * prm.H;
        const int i0 = qt * kTileM;
        const int general = (has_docs && prm.mono != nullptr && prm.mono[b] == 0) ? 1 : 0;
        // document starts of the tile's rows (one row per lane and round)
        int lo_first = 0, lo_last = 0;
        if (has_docs && !general) {
          const int i1 = min(i0 + kTileM - 1, prm.N - 1);
#pragma unroll
          for (int r = 0; r < kTileM / 32; ++r) {
            const int i = min(i0 + r * 32 + lane, prm.N - 1);
            slot.lo[r * 32 + lane] = prm.lo[(size_t)b * prm.N + i];
          }
          __syncwarp();
          lo_first = slot.lo[0];
          lo_last = slot.lo[i1 - i0];
        } else {
#pragma unroll
          for (int r = 0; r < kTileM / 32; ++r) slot.lo[r * 32 + lane] = 0;
        }
        if (lane == 0) {
          BlockPlan bp;
          bp.general_docs = general;
          if (prm.mask.ks == 1) {
            bp.n_streams = 1;
            bp.stream_id[0] = 0;
            bp.stream_id[1] = 0;
            bp.sp[0] = plan_stream(prm.mask, i0, lo_first, lo_last, 0, kWideN);
            bp.sp[1] = bp.sp[0];
            bp.sp[1].ntiles = 0;
          } else {
            bp.n_streams = 2;
            bp.stream_id[0] = prm.mask.pp;       // persistent stream first: holds the diagonal
            bp.stream_id[1] = 1 - prm.mask.pp;
            bp.sp[0] = plan_stream(prm.mask, i0, lo_first, lo_last, bp.stream_id[0], kWideN);
            bp.sp[1] = plan_stream(prm.mask, i0, lo_first, lo_last, bp.stream_id[1], kWideN);
          }
          bp.n_tiles = bp.sp[0].ntiles + bp.sp[1].ntiles;
          slot.plan = bp;
          slot.item = item;
          slot.i0 = i0;
          slot.b = b;
          slot.h = h;
          slot.bh = bh;
        }
        __syncwarp();
        const int n_tiles = slot.plan.n_tiles;
        for (int j = lane; j < min(n_tiles, kTileTable); j += 32)
          slot.tiles[j] = pack_tile(tile_info<kWideN>(slot.plan, j));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_item_full + 8 * buf);   // release: the slot is published
        WTR(95);
        if (n_tiles == 0) continue;

        // Q tile into its buffer once the products of the item that used it before are done
        const uint32_t q_before = buf ? q_loads1 : q_loads0;   // loads into this buffer so far
        if (q_before >= 1) {
          if (!warp_wait(bar_q_free + 8 * buf, (q_before - 1u) & 1u, abort_flag, prm.status)) break;
        }
        if (buf) ++q_loads1;
        else ++q_loads0;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar_q_full + 8 * buf, Cfg::kQBytes);
          tma_load_4d(sQ + buf * Cfg::kQBytes, &tm_q, bar_q_full + 8 * buf, 0, i0, h, b);
        }
        __syncwarp();
        auto load_k = [&](int j) {
          const TileInfo t = get_tile<kWideN>(slot.plan, slot.tiles, j);
          const int st = gk % Cfg::kStagesK;
          if (gk >= (uint32_t)Cfg::kStagesK) {
            if (!warp_wait(bar_k_empty + 8 * st, ((gk / Cfg::kStagesK) - 1u) & 1u, abort_flag, prm.status))
              return false;
          }
          if (elect_one()) {
            mbar_arrive_expect_tx(bar_k_full + 8 * st, Cfg::kKVBytes);
            tma_load_5d(sK + st * Cfg::kKVBytes, &tm_k, bar_k_full + 8 * st, 0, t.stream, t.k0, h, b);
          }
          __syncwarp();
          ++gk;
          return true;
        };
        auto load_v = [&](int j) {
          const TileInfo t = get_tile<kWideN>(slot.plan, slot.tiles, j);
          const int st = gv % Cfg::kStagesV;
          if (gv >= (uint32_t)Cfg::kStagesV) {
            if (!warp_wait(bar_v_empty + 8 * st, ((gv / Cfg::kStagesV) - 1u) & 1u, abort_flag, prm.status))
              return false;
          }
          if (elect_one()) {
            mbar_arrive_expect_tx(bar_v_full + 8 * st, Cfg::kKVBytes);
            tma_load_5d(sV + st * Cfg::kKVBytes, &tm_v, bar_v_full + 8 * st, 0, t.stream, t.k0, h, b);
          }
          __syncwarp();
          ++gv;
          return true;
        };
        ok = load_k(0);
        for (int j = 0; ok && j < n_tiles; ++j) {
          if (j + 1 < n_tiles) ok = load_k(j + 1);
          if (ok) ok = load_v(j);
        }
      }
    } else if (warp == 5) {
      // ------------------------------------------------------------------ MMA issuer
      // The whole warp runs this loop converged (so descriptors and addresses stay in uniform
      // registers); one elected lane issues the tcgen05 instructions.
      constexpr uint32_t idesc_qk = make_idesc_f16(FP16, kTileM, kWideN / 2, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(FP16, kTileM, D, false, true);
      const uint64_t dq64 = make_smem_desc_sw128(sQ, 16, 1024);
      const uint64_t dk64 = make_smem_desc_sw128(sK, 16, 1024);
      const uint64_t dv64 = make_smem_desc_sw128(sV, Cfg::kKVBytes, 1024);
      const uint32_t dq_lo = (uint32_t)dq64, dq_hi = (uint32_t)(dq64 >> 32);
      const uint32_t dk_lo = (uint32_t)dk64, dk_hi = (uint32_t)(dk64 >> 32);
      const uint32_t dv_lo = (uint32_t)dv64, dv_hi = (uint32_t)(dv64 >> 32);
      uint32_t g = 0;                 // tiles whose Q K^T has been issued
      uint32_t gp = 0;                // tiles whose P V has been issued
      uint32_t q_uses0 = 0, q_uses1 = 0;   // items that went through each Q buffer
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        const int buf = n & 1u;
        if (!warp_wait(bar_item_full + 8 * buf, (n >> 1) & 1u, abort_flag, prm.status)) break;
        const WideItem& slot = s_item[buf];
        if (slot.item < 0) break;
        WTR(97);
        const int n_tiles = slot.plan.n_tiles;
        if (n_tiles > 0) {
          const uint32_t qa0 = dq_lo + ((buf * Cfg::kQBytes) >> 4);
          // scores of one 64-key half of tile j (the g-th tile of this block) into its S columns
          auto issue_qk = [&](int j, int half) {
            const int st = g % Cfg::kStagesK;
            if (half == 0) {
              if (!warp_wait(bar_k_full + 8 * st, (g / Cfg::kStagesK) & 1u, abort_flag, prm.status)) return false;
            }
            if (g >= 1) {
              if (!warp_wait(bar_s_free + 8 * half, (g - 1u) & 1u, abort_flag, prm.status)) return false;
            }
            tc_fence_after();
            // 64 key rows = 8192 bytes of the tile; a K step of 16 elements is 32 bytes inside a row
            const uint32_t kb0 = dk_lo + ((st * Cfg::kKVBytes + half * (Cfg::kKVBytes / 2)) >> 4);
            const uint32_t sd = tmem + Cfg::kColS + half * (kWideN / 2);
            if (elect_one()) {
              umma_ss<false>(sd, qa0, dq_hi, kb0, dk_hi, idesc_qk);
#pragma unroll
              for (int kk = 1; kk < D / 16; ++kk)
                umma_ss<true>(sd, qa0 + ((kk * 32) >> 4), dq_hi, kb0 + ((kk * 32) >> 4), dk_hi, idesc_qk);
              umma_commit(bar_s_full + 8 * half);
              if (half == 1) {
                umma_commit(bar_k_empty + 8 * st);
                if (j == n_tiles - 1) umma_commit(bar_q_free + 8 * buf);
              }
            }
            __syncwarp();
            if (half == 1) ++g;
            return true;
          };
          ok = warp_wait(bar_q_full + 8 * buf, (buf ? q_uses1 : q_uses0) & 1u, abort_flag, prm.status);
          if (buf) ++q_uses1;
          else ++q_uses0;
          if (ok) ok = issue_qk(0, 0);
          if (ok) ok = issue_qk(0, 1);
          for (int j = 0; ok && j < n_tiles; ++j, ++gp) {
            const int st = gp % Cfg::kStagesV;
            const uint32_t vb0 = dv_lo + ((st * Cfg::kKVBytes) >> 4);
            const uint32_t od = tmem + Cfg::kColO;
            const uint32_t pa = tmem + Cfg::kColP;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              // The same half of the next tile's scores first: the softmax warps hand these S
              // columns back as soon as they have read them (a quarter / three quarters through
              // the tile), long before they deliver this half of P, so the scores of the next
              // tile are ready well before the softmax warps come round to them.
              if (j + 1 < n_tiles) {
                if (!issue_qk(j + 1, half)) {
                  ok = false;
                  break;
                }
              }
              if (!warp_wait(bar_p_full + 8 * half, gp & 1u, abort_flag, prm.status)) {
                ok = false;
                break;
              }
              if (half == 0) WTR(50);
              if (half == 0) {
                if (!warp_wait(bar_v_full + 8 * st, (gp / Cfg::kStagesV) & 1u, abort_flag, prm.status)) {
                  ok = false;
                  break;
                }
              }
              tc_fence_after();
              if (elect_one()) {
                // A from tensor memory: 16 keys = 8 packed columns per step; V: 16 key rows = 2048 bytes
#pragma unroll
                for (int kk = 4 * half; kk < 4 * half + 4; ++kk)
                  umma_ts(od, pa + 8 * kk, vb0 + ((kk * 2048) >> 4), dv_hi, idesc_pv, j > 0 || kk > 0);
                umma_commit(bar_pv_done + 8 * half);
                if (half == 1) umma_commit(bar_v_empty + 8 * st);
              }
              __syncwarp();
            }
          }
        }
        if (!ok) break;
        if (lane == 0) mbar_arrive(bar_item_free + 8 * buf);
      }
    } else {
      // ------------------------------------------------------------------ softmax warps
      const int row = tid;                 // TMEM lane and query row inside the tile
      const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
      uint32_t g = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        const int buf = n & 1u;
        if (!warp_wait(bar_item_full + 8 * buf, (n >> 1) & 1u, abort_flag, prm.status)) break;
        const WideItem& slot = s_item[buf];
        if (slot.item < 0) break;
        WTR(90);
        const int n_tiles = slot.plan.n_tiles;
        const int b = slot.b, h = slot.h;
        const int i = slot.i0 + row;
        uint8_t* o_row = reinterpret_cast<uint8_t*>(prm.o) +
                         (b * prm.o_stride_b + h * prm.o_stride_h + i * prm.o_stride_n) * 2;
        if (n_tiles > 0) {
          const bool general = slot.plan.general_docs != 0;
          WideSoftmaxCtx ctx;
          row_interval(prm.mask, i, slot.lo[row], 0, ctx.kmin_s[0], ctx.kmax_s[0]);
          row_interval(prm.mask, i, slot.lo[row], 1, ctx.kmin_s[1], ctx.kmax_s[1]);
          ctx.docs_b = nullptr;
          ctx.my_doc = 0;
          if (general) {
            ctx.docs_b = reinterpret_cast<const uint8_t*>(prm.docs) +
                         (size_t)b * prm.doc_stride_b * (prm.doc_is_i64 ? 8 : 4);
            if (i < prm.N) {
              const size_t off = (size_t)i * prm.doc_stride_t;
              ctx.my_doc = prm.doc_is_i64 ? reinterpret_cast<const long long*>(ctx.docs_b)[off]
                                          : (long long)reinterpret_cast<const int*>(ctx.docs_b)[off];
            }
          }
          ctx.prm = &prm;
          ctx.slot = &slot;
          ctx.abort_flag = abort_flag;
          ctx.tmem_row = tmem + lane_addr;
          ctx.bar_s_full = bar_s_full;
          ctx.bar_s_free = bar_s_free;
          ctx.bar_p_full = bar_p_full;
          ctx.bar_pv_done = bar_pv_done;
          ctx.n_tiles = n_tiles;
          ctx.lane = lane;
          ctx.g = g;
          ctx.m_run = -1.0e30f;   // running max of raw scores (finite sentinel)
          ctx.l_run = 0.f;
          ctx.ok = true;
          ctx.wtr_buf = wtr_buf;
          ctx.wtr_n = wtr_n;
          ctx.general = general;
          wide_softmax_tiles<FP16>(ctx);
          g = ctx.g;
          ok = ctx.ok;
          WTR(91);
          // ------------------------------------------------------------ epilogue of the item
          // (the MMA warp is free to multiply the next item's first tile meanwhile: it writes S,
          // and O only after this warp has handed over the next item's first P)
          if (ok) ok = warp_wait(bar_pv_done + 8, (g - 1u) & 1u, abort_flag, prm.status);
          if (ok) {
            tc_fence_after();
            const float l_run = ctx.l_run;
            const float inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
            for (int q4 = 0; q4 < D / 32; ++q4) {
              uint32_t o[32];
              tmem_ld32(tmem + lane_addr + Cfg::kColO + q4 * 32, o);
              tmem_wait_ld();
              if (i < prm.N) {
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
                  uint4 u;
                  u.x = pack2<FP16>(__uint_as_float(o[e]) * inv_l, __uint_as_float(o[e + 1]) * inv_l);
                  u.y = pack2<FP16>(__uint_as_float(o[e + 2]) * inv_l, __uint_as_float(o[e + 3]) * inv_l);
                  u.z = pack2<FP16>(__uint_as_float(o[e + 4]) * inv_l, __uint_as_float(o[e + 5]) * inv_l);
                  u.w = pack2<FP16>(__uint_as_float(o[e + 6]) * inv_l, __uint_as_float(o[e + 7]) * inv_l);
                  *reinterpret_cast<uint4*>(o_row + q4 * 64 + e * 2) = u;
                }
              }
            }
            if (prm.lse != nullptr && i < prm.N)
              prm.lse[(size_t)slot.bh * prm.N + i] =
                  l_run > 0.f ? ctx.m_run * prm.scale_log2 + log2f(l_run) : -INFINITY;
            tc_fence_before();
          }
        } else if (i < prm.N) {
          // nothing visible for any row of this tile: outputs are zero
          uint4* o16 = reinterpret_cast<uint4*>(o_row);
          for (int e = 0; e < D / 8; ++e) o16[e] = make_uint4(0, 0, 0, 0);
          if (prm.lse != nullptr) prm.lse[(size_t)slot.bh * prm.N + i] = -INFINITY;
        }
        if (!ok) break;
        WTR(92);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_item_free + 8 * buf);
      }
    }
  }

  __syncthreads();
#ifdef SPSATTN_TRACE
  if (wtr_buf != nullptr)
    for (int e = tid; e < 6 * kWideTraceEvents; e += kWideThreads)
      prm.trace[(size_t)blockIdx.x * 6 * kWideTraceEvents + e] =
          (e % kWideTraceEvents) < s_wtr_n[e / kWideTraceEvents] ? s_wtr[e / kWideTraceEvents][e % kWideTraceEvents] : 0;
#endif
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc<Cfg::kTmemCols>(tmem);
  }
}

}  // namespace spsattn
