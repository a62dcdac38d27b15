// Host side of libspsattn.so: argument validation, tensor-map encoding, launches.
// Plain C ABI (include/spsattn.h); no torch types, no allocation, no synchronisation.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "../../include/spsattn.h"
#include "cache_fill.cuh"
#include "decode.cuh"
#include "decode_sm100.cuh"
#include "kv_update.cuh"
#include "model_glue.cuh"
#include "prefill_aux.cuh"
#include "prefill_sm100.cuh"
#include "prefill_wide_sm100.cuh"
#include "prefill_bwd_sm100.cuh"
#include "rope.cuh"

using namespace spsattn;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int clamp_window(long long w, int n) {
  if (w < 0) return -1;
  if (w > n) return n;
  return (int)w;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// workspace layout of the prefill pre-pass: [mono: B ints, work counter: 1 int, padded to 256 B]
// [lo: B*N ints]
size_t prefill_ws_mono_bytes(int B) { return align_up((size_t)(B + 1) * sizeof(int), 256); }

MaskParams make_mask(int N, int parity, int w, int pw, int flags) {
  MaskParams m;
  m.n_rows = N;
  m.ks = parity == SPSATTN_PARITY_NONE ? 1 : 2;
  m.pp = parity == SPSATTN_PARITY_NONE ? -1 : parity;
  m.w = clamp_window(w, N);
  m.has_pw = (parity != SPSATTN_PARITY_NONE && pw != SPSATTN_NO_WINDOW) ? 1 : 0;
  m.pw = m.has_pw ? clamp_window(pw, N) : 0;
  m.flags = flags;
  return m;
}

// Strides of a [B, H, N, D] operand in elements (D is contiguous).
struct Strides {
  int64_t b, h, n;
};

// Q map: [D, N, H, B] with the operand's own strides, box [64, box_rows, 1, 1]
int encode_q_map(CUtensorMap* tm, const void* ptr, int B, int H, int N, int D, Strides st, int dtype,
                 int box_rows = 128) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return SPSATTN_ERR_DRIVER;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)st.n * 2, (cuuint64_t)st.h * 2, (cuuint64_t)st.b * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, dtype == SPSATTN_DTYPE_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                   4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// K / V map with the two parity streams as a dimension: [D, ks, N/ks, H, B], box
// [64, 1, kTileN, 1, 1].  A tile is kTileN consecutive key tokens of one parity; rows of the
// other parity are skipped by the stride, out-of-range tokens read as zero and the next head
// is never touched.
int encode_kv_map(CUtensorMap* tm, const void* ptr, int B, int H, int N, int D, int ks, Strides st,
                  int dtype, int box_tokens = kTileN) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return SPSATTN_ERR_DRIVER;
  cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)ks, (cuuint64_t)(N / ks), (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[4] = {(cuuint64_t)st.n * 2, (cuuint64_t)ks * st.n * 2, (cuuint64_t)st.h * 2,
                           (cuuint64_t)st.b * 2};
  cuuint32_t box[5] = {64, 1, (cuuint32_t)box_tokens, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(tm, dtype == SPSATTN_DTYPE_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                   5, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

bool strides_ok(Strides st, int D) {
  return st.n >= D && st.h >= D && st.b >= D && (st.n % 8) == 0 && (st.h % 8) == 0 && (st.b % 8) == 0;
}

template <int D, bool FP16>
int launch_prefill_sm100(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const PrefillParams& prm, cudaStream_t st) {
  using Cfg = PrefillCfg<D>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(prefill_sm100_kernel<D, FP16>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return (int)attr_err;
  const long long blocks = (long long)prm.n_qtiles * prm.B * prm.H;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return SPSATTN_ERR_TOO_LARGE;
  // With document ids the kernel just before this one in the stream is the pre-pass (8 blocks of
  // a few microseconds): launched as its programmatic dependent, the attention blocks set up
  // their barriers, tensor memory and Q tile beside it and wait for it only before they read its
  // outputs.  Without ids the launch is an ordinary one (whatever precedes it may produce Q, K, V).
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(kPrefillThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
#ifdef SPSATTN_NO_PDL
  cfg.numAttrs = 0;         // tuning builds: ordinary launch
#else
  cfg.numAttrs = prm.lo != nullptr ? 1 : 0;
#endif
  const cudaError_t le = cudaLaunchKernelEx(&cfg, prefill_sm100_kernel<D, FP16>, tq, tk, tv, prm);
  return le != cudaSuccess ? (int)le : (int)cudaGetLastError();
}

// Persistent launch: two blocks per SM draw the (batch, head, query tile) items from
// prm.work_counter (zero at launch), or take them with a fixed stride when there is no counter.
template <bool FP16>
int launch_prefill_wide(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                        const PrefillParams& prm, cudaStream_t st) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(prefill_wide_sm100_kernel<FP16>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, WideCfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return (int)attr_err;
  const long long items = (long long)prm.n_qtiles * prm.B * prm.H;
  if (items <= 0 || items > 0x7fffffffLL) return SPSATTN_ERR_TOO_LARGE;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
#ifdef SPSATTN_ONE_CTA
  const long long per_sm = 1;      // tuning builds: one block per SM
#else
  const long long per_sm = 2;
#endif
  const long long blocks = items < per_sm * sms ? items : per_sm * sms;
  prefill_wide_sm100_kernel<FP16><<<(unsigned)blocks, kWideThreads, WideCfg::kSmemBytes, st>>>(tq, tk, tv, prm);
  return (int)cudaGetLastError();
}

// 0: automatic (the 64-key-tile kernel, the faster one as measured), 1: the same, forced,
// 2: the persistent 128-key-tile kernel (head_dim 64)
std::atomic<int> g_prefill_path{0};

template <int D, bool FP16, int MODE>
int launch_prefill_bwd(const CUtensorMap& x0, const CUtensorMap& x1, const CUtensorMap& y0,
                       const CUtensorMap& y1, const BwdParams& prm, cudaStream_t st) {
  using Cfg = BwdCfg<D, MODE>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(prefill_bwd_sm100_kernel<D, FP16, MODE>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return (int)attr_err;
  const long long blocks = (long long)prm.n_xtiles * prm.B * prm.H;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return SPSATTN_ERR_TOO_LARGE;
  prefill_bwd_sm100_kernel<D, FP16, MODE><<<(unsigned)blocks, Cfg::kThreads, Cfg::kSmemBytes, st>>>(x0, x1, y0, y1, prm);
  return (int)cudaGetLastError();
}

int run_doc_prepass(const void* doc_ids, int doc_is_i64, int64_t sb, int64_t stt, int B, int N,
                    void* workspace, size_t workspace_bytes, int** lo, int** mono, cudaStream_t st) {
  *lo = nullptr;
  *mono = nullptr;
  if (doc_ids == nullptr) return 0;
  const size_t need = prefill_ws_mono_bytes(B) + (size_t)B * N * sizeof(int);
  if (workspace == nullptr || workspace_bytes < need) return SPSATTN_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return SPSATTN_ERR_ALIGN;
  *mono = reinterpret_cast<int*>(workspace);
  *lo = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(workspace) + prefill_ws_mono_bytes(B));
  doc_prepass_kernel<<<B, 1024, 0, st>>>(doc_ids, doc_is_i64, sb, stt, N, *lo, *mono, *mono + B);
  return (int)cudaGetLastError();
}

static int decode_chunk_rows(int S, int H, long long max_rows_total) {
  // large chunks keep the record traffic small; small problems get smaller chunks so that the
  // grid still fills the 148 SMs several times over
  int chunk = 512;
  while (chunk > 128) {
    const long long blocks = (long long)S * H * ((max_rows_total + chunk - 1) / chunk);
    if (blocks >= 148LL * 16) break;
    chunk >>= 1;
  }
  return chunk;
}

static long long decode_max_rows(const spsattn_segment* segs, int n_segments) {
  long long t = 0;
  for (int x = 0; x < n_segments; ++x) t += segs[x].max_rows > 0 ? segs[x].max_rows : 0;
  return t;
}

template <int D, int NQ, bool FP16>
static int launch_decode(const DecodeParams& prm, cudaStream_t st) {
  dim3 grid((unsigned)(prm.S * prm.H), (unsigned)prm.n_chunks);
  decode_split_kernel<D, NQ, FP16><<<grid, kDecodeThreads, 0, st>>>(prm);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || prm.tickets != nullptr) return (int)e;   // with tickets the last block merges
  decode_merge_kernel<D, NQ, FP16><<<(unsigned)(prm.S * prm.H), D, 0, st>>>(prm);
  return (int)cudaGetLastError();
}

template <int D>
static int launch_decode_d(const DecodeParams& prm, int nq, bool fp16, cudaStream_t st) {
  if (nq == 1) return fp16 ? launch_decode<D, 1, true>(prm, st) : launch_decode<D, 1, false>(prm, st);
  return fp16 ? launch_decode<D, 2, true>(prm, st) : launch_decode<D, 2, false>(prm, st);
}

// ---- tensor-core decode (decode_sm100.cuh): slot layout and launch
constexpr int kTcSmallRows = 128;   // segments up to this many rows go with the current-token entries
std::atomic<int> g_decode_path{0};   // 0 auto, 1 CUDA-core kernel, 2 tensor-core kernel

int tc_chunk_rows(int S, int H, const spsattn_segment* segs, int n_segments) {
  // A block pays a fixed start-up (tensor memory, barriers, zeroed operand tiles) and a block
  // past the live length still occupies a shared-memory slot while it takes its ticket: one
  // chunk per segment when there are enough (sequence, head) pairs to fill the machine, halved
  // until there are.
  long long longest = kTcTile;
  for (int x = 0; x < n_segments; ++x)
    if (segs[x].max_rows > longest) longest = segs[x].max_rows;
  long long chunk = (longest + kTcTile - 1) / kTcTile * kTcTile;
  while (chunk > kTcTile) {
    long long blocks = 0;
    for (int x = 0; x < n_segments; ++x)
      if (segs[x].max_rows > kTcSmallRows) blocks += (segs[x].max_rows + chunk - 1) / chunk;
    if ((long long)S * H * blocks >= 148LL * 3) break;
    chunk = (chunk / 2 + kTcTile - 1) / kTcTile * kTcTile;
  }
  return (int)chunk;
}

bool tc_supported(const spsattn_segment* segs, int n_segments, int D) {
  if (D != 64 && D != 128) return false;
  for (int x = 0; x < n_segments; ++x)
    if (segs[x].seq_offset != nullptr) return false;   // packed caches have no single tensor map
  return true;
}

int tc_slots(const spsattn_segment* segs, int n_segments, int n_extras, int chunk, int* seg_chunks,
             uint32_t* small_segs) {
  int total = 0;
  uint32_t small = 0;
  for (int x = 0; x < kMaxSegments; ++x) {
    const int rows = (x < n_segments && segs[x].max_rows > 0) ? segs[x].max_rows : 0;
    int c = (rows + chunk - 1) / chunk;
    if (rows > 0 && rows <= kTcSmallRows) {
      small |= 1u << x;
      c = 0;
    }
    if (seg_chunks) seg_chunks[x] = c;
    total += c;
  }
  if (small_segs) *small_segs = small;
  if (n_extras > 0 || small != 0) ++total;
  return total > 0 ? total : 1;
}

int encode_cache_map(CUtensorMap* tm, const void* ptr, const spsattn_segment& sg, int S, int H, int D,
                            int dtype) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return SPSATTN_ERR_DRIVER;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)sg.max_rows, (cuuint64_t)H, (cuuint64_t)S};
  cuuint64_t strides[3] = {(cuuint64_t)sg.row_stride * 2, (cuuint64_t)sg.head_stride * 2,
                           (cuuint64_t)sg.seq_stride * 2};
  // a degenerate extent (one head or one sequence) may carry any stride: keep it encodable
  if (H == 1) strides[1] = strides[0] * (cuuint64_t)sg.max_rows;
  if (S == 1) strides[2] = strides[1] * (cuuint64_t)H;
  cuuint32_t box[4] = {64, (cuuint32_t)kTcTile, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, dtype == SPSATTN_DTYPE_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                   4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

template <int D, int NQ, bool FP16>
int launch_decode_tc(const DecodeMaps& maps, const DecodeParams& prm, cudaStream_t st) {
  using Cfg = DecodeTcCfg<D>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(decode_tc_kernel<D, NQ, FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return (int)attr_err;
  // one block per chunk of a long segment; the record slot of the current-token entries and short
  // segments has no block of its own (slot 0's block fills it)
  int blocks_y = 0;
  for (int x = 0; x < kMaxSegments; ++x) blocks_y += prm.seg_chunks[x];
  if (blocks_y < 1) blocks_y = 1;
  dim3 grid((unsigned)(prm.S * prm.H), (unsigned)blocks_y);
  decode_tc_kernel<D, NQ, FP16><<<grid, kTcThreads, Cfg::kSmemBytes, st>>>(maps, prm);
  return (int)cudaGetLastError();
}

template <int D>
int launch_decode_tc_d(const DecodeMaps& maps, const DecodeParams& prm, int nq, bool fp16,
                              cudaStream_t st) {
  if (nq == 1)
    return fp16 ? launch_decode_tc<D, 1, true>(maps, prm, st) : launch_decode_tc<D, 1, false>(maps, prm, st);
  return fp16 ? launch_decode_tc<D, 2, true>(maps, prm, st) : launch_decode_tc<D, 2, false>(maps, prm, st);
}

}  // namespace

#ifdef SPSATTN_TRACE
static long long* g_trace_buffer = nullptr;
// tuning builds only: where the prefill kernel writes its cycle stamps
extern "C" void spsattn_debug_set_trace(long long* device_buffer) { g_trace_buffer = device_buffer; }
#endif

extern "C" {

int spsattn_version(void) { return 1; }

const char* spsattn_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case SPSATTN_ERR_ARG: return "invalid argument (null pointer, bad enum or bad size)";
    case SPSATTN_ERR_HEAD_DIM: return "head_dim not supported by this entry point";
    case SPSATTN_ERR_ALIGN: return "pointer or stride not suitably aligned";
    case SPSATTN_ERR_WORKSPACE: return "workspace missing or too small";
    case SPSATTN_ERR_ODD_LENGTH: return "doubled sequence length must be even";
    case SPSATTN_ERR_DRIVER: return "cuTensorMapEncodeTiled is unavailable in this driver";
    case SPSATTN_ERR_TOO_LARGE: return "size beyond a documented maximum";
    case SPSATTN_ERR_SCRATCH_LIMIT:
      return "the split-K records of this call exceed the built-in 16 MiB scratch buffer "
             "(SPSATTN_NOALLOC_SCRATCH_BYTES); split the sequences over several calls or use "
             "spsattn_decode_fwd with a caller-owned workspace";
    default: break;
  }
  if (code > 0) return cudaGetErrorString((cudaError_t)code);
  return "unknown spsattn error";
}

size_t spsattn_prefill_workspace_bytes(int B, int H, int N, int D) {
  (void)H;
  (void)D;
  if (B <= 0 || N <= 0) return 256;
  return prefill_ws_mono_bytes(B) + align_up((size_t)B * N * sizeof(int), 256);
}

int spsattn_prefill_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse,
                                const int64_t* q_strides, const int64_t* k_strides,
                                const int64_t* v_strides, const int64_t* o_strides, const void* doc_ids,
                                int doc_is_i64, int64_t doc_stride_b, int64_t doc_stride_t, int B, int H,
                                int N, int D, int dtype, float sm_scale, int persistent_parity,
                                int temporary_window, int persistent_window, int mask_flags,
                                void* workspace, size_t workspace_bytes, int* device_status,
                                void* stream) {
  if (!q || !k || !v || !o || !q_strides || !k_strides || !v_strides || !o_strides) return SPSATTN_ERR_ARG;
  if (B <= 0 || H <= 0 || N <= 0) return SPSATTN_ERR_ARG;
  if (dtype != SPSATTN_DTYPE_BF16 && dtype != SPSATTN_DTYPE_FP16) return SPSATTN_ERR_ARG;
  if (persistent_parity != SPSATTN_PARITY_EVEN && persistent_parity != SPSATTN_PARITY_ODD &&
      persistent_parity != SPSATTN_PARITY_NONE)
    return SPSATTN_ERR_ARG;
  if (!(sm_scale > 0.f) || !isfinite(sm_scale)) return SPSATTN_ERR_ARG;
  if (D != 16 && D != 32 && D != 64 && D != 128 && D != 256) return SPSATTN_ERR_HEAD_DIM;
  if (persistent_parity != SPSATTN_PARITY_NONE && (N & 1)) return SPSATTN_ERR_ODD_LENGTH;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return SPSATTN_ERR_ALIGN;
  if ((long long)B * H > 0x7fffffffLL / 64) return SPSATTN_ERR_TOO_LARGE;
  const Strides sq = {q_strides[0], q_strides[1], q_strides[2]};
  const Strides sk = {k_strides[0], k_strides[1], k_strides[2]};
  const Strides sv = {v_strides[0], v_strides[1], v_strides[2]};
  const Strides so = {o_strides[0], o_strides[1], o_strides[2]};
  if (!strides_ok(sq, D) || !strides_ok(sk, D) || !strides_ok(sv, D) || !strides_ok(so, D))
    return SPSATTN_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  int *lo = nullptr, *mono = nullptr;
  int rc = run_doc_prepass(doc_ids, doc_is_i64, doc_stride_b, doc_stride_t, B, N, workspace,
                           workspace_bytes, &lo, &mono, st);
  if (rc != 0) return rc;

  const MaskParams mask = make_mask(N, persistent_parity, temporary_window, persistent_window, mask_flags);
  const float scale_log2 = sm_scale * 1.4426950408889634f;
  const bool fp16 = dtype == SPSATTN_DTYPE_FP16;

  if (D == 64 || D == 128) {
    CUtensorMap tq, tk, tv;
    if ((rc = encode_q_map(&tq, q, B, H, N, D, sq, dtype)) != 0) return rc;
    const bool wide = D == 64 && g_prefill_path.load() == 2;
    const int box_tokens = wide ? kWideN : kTileN;
    if ((rc = encode_kv_map(&tk, k, B, H, N, D, mask.ks, sk, dtype, box_tokens)) != 0) return rc;
    if ((rc = encode_kv_map(&tv, v, B, H, N, D, mask.ks, sv, dtype, box_tokens)) != 0) return rc;
    PrefillParams prm;
    memset(&prm, 0, sizeof(prm));
    prm.o = o;
    prm.o_stride_b = so.b;
    prm.o_stride_h = so.h;
    prm.o_stride_n = so.n;
    prm.lse = lse;
    prm.docs = doc_ids;
    prm.doc_stride_b = doc_stride_b;
    prm.doc_stride_t = doc_stride_t;
    prm.doc_is_i64 = doc_is_i64;
    prm.lo = lo;
    prm.mono = mono;
    prm.B = B;
    prm.H = H;
    prm.N = N;
    prm.n_qtiles = (N + kTileM - 1) / kTileM;
    prm.mask = mask;
    prm.scale_log2 = scale_log2;
    prm.status = device_status;
#ifdef SPSATTN_TRACE
    prm.trace = g_trace_buffer;
#endif
    // heads whose K and V (2 * N * D * 2 bytes each) share about 48 MB of L2 at a time
    const long long kv_bytes = 4LL * N * D;
    const long long gh = (48LL << 20) / (kv_bytes > 0 ? kv_bytes : 1);
    prm.group_heads = (int)(gh < 1 ? 1 : (gh > 32 ? 32 : gh));
#ifdef SPSATTN_NO_GROUP
    prm.group_heads = 1;      // tuning builds: one head after the other
#endif
    if (wide) {
      // the item counter lives behind the pre-pass flags: the pre-pass has zeroed it when ids were
      // given, else it is cleared here; without a workspace the blocks take items with a stride
      if (mono != nullptr) {
        prm.work_counter = mono + B;
      } else if (workspace != nullptr && workspace_bytes >= prefill_ws_mono_bytes(B) &&
                 (reinterpret_cast<uintptr_t>(workspace) & 3u) == 0) {
        prm.work_counter = reinterpret_cast<int*>(workspace) + B;
        cudaError_t me = cudaMemsetAsync(prm.work_counter, 0, sizeof(int), st);
        if (me != cudaSuccess) return (int)me;
      }
      return fp16 ? launch_prefill_wide<true>(tq, tk, tv, prm, st)
                  : launch_prefill_wide<false>(tq, tk, tv, prm, st);
    }
    if (D == 64) return fp16 ? launch_prefill_sm100<64, true>(tq, tk, tv, prm, st)
                             : launch_prefill_sm100<64, false>(tq, tk, tv, prm, st);
    return fp16 ? launch_prefill_sm100<128, true>(tq, tk, tv, prm, st)
                : launch_prefill_sm100<128, false>(tq, tk, tv, prm, st);
  }
  // the CUDA-core kernel for the other head dims reads dense [B, H, N, D] operands only
  const Strides dense = {(int64_t)H * N * D, (int64_t)N * D, (int64_t)D};
  auto is_dense = [&](Strides x) { return x.b == dense.b && x.h == dense.h && x.n == dense.n; };
  if (!is_dense(sq) || !is_dense(sk) || !is_dense(sv) || !is_dense(so)) return SPSATTN_ERR_ALIGN;
  dim3 grid((N + 3) / 4, B * H);
  const size_t smem = 4 * (size_t)D * sizeof(float);
  if (fp16)
    prefill_generic_kernel<true><<<grid, 128, smem, st>>>(q, k, v, o, lse, doc_ids, doc_is_i64, doc_stride_b,
                                                          doc_stride_t, lo, mono, H, N, D, mask, scale_log2);
  else
    prefill_generic_kernel<false><<<grid, 128, smem, st>>>(q, k, v, o, lse, doc_ids, doc_is_i64, doc_stride_b,
                                                           doc_stride_t, lo, mono, H, N, D, mask, scale_log2);
  return (int)cudaGetLastError();
}

size_t spsattn_prefill_bwd_workspace_bytes(int B, int H, int N, int D) {
  if (B <= 0 || H <= 0 || N <= 0) return 256;
  return spsattn_prefill_workspace_bytes(B, H, N, D) + align_up((size_t)B * H * N * sizeof(float), 256) +
         align_up((size_t)B * N * sizeof(int), 256);
}

int spsattn_prefill_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                const float* lse, void* dq, void* dk, void* dv, const int64_t* strides,
                                const void* doc_ids, int doc_is_i64, int64_t doc_stride_b,
                                int64_t doc_stride_t, int B, int H, int N, int D, int dtype, float sm_scale,
                                int persistent_parity, int temporary_window, int persistent_window,
                                int mask_flags, void* workspace, size_t workspace_bytes,
                                int* device_status, void* stream) {
  if (!q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv || !strides) return SPSATTN_ERR_ARG;
  if (B <= 0 || H <= 0 || N <= 0) return SPSATTN_ERR_ARG;
  if (dtype != SPSATTN_DTYPE_BF16 && dtype != SPSATTN_DTYPE_FP16) return SPSATTN_ERR_ARG;
  if (persistent_parity != SPSATTN_PARITY_EVEN && persistent_parity != SPSATTN_PARITY_ODD &&
      persistent_parity != SPSATTN_PARITY_NONE)
    return SPSATTN_ERR_ARG;
  if (!(sm_scale > 0.f) || !isfinite(sm_scale)) return SPSATTN_ERR_ARG;
  if (D != 64 && D != 128) return SPSATTN_ERR_HEAD_DIM;
  if (persistent_parity != SPSATTN_PARITY_NONE && (N & 1)) return SPSATTN_ERR_ODD_LENGTH;
  if (N > 64 * kBwdTable) return SPSATTN_ERR_TOO_LARGE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(d_o) ||
      !aligned16(dq) || !aligned16(dk) || !aligned16(dv))
    return SPSATTN_ERR_ALIGN;
  if ((long long)B * H > 0x7fffffffLL / 1024) return SPSATTN_ERR_TOO_LARGE;
  if (workspace == nullptr || workspace_bytes < spsattn_prefill_bwd_workspace_bytes(B, H, N, D))
    return SPSATTN_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return SPSATTN_ERR_ALIGN;
  // strides: eight (batch, head, row) triples in elements, in the order q, k, v, o, d_o, dq, dk, dv
  Strides sx[8];
  for (int x = 0; x < 8; ++x) {
    sx[x] = {strides[3 * x], strides[3 * x + 1], strides[3 * x + 2]};
    if (!strides_ok(sx[x], D)) return SPSATTN_ERR_ALIGN;
  }
  const Strides &sq = sx[0], &sk = sx[1], &sv = sx[2], &so = sx[3], &sg = sx[4];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool fp16 = dtype == SPSATTN_DTYPE_FP16;

  int *lo = nullptr, *mono = nullptr;
  const size_t pre_bytes = spsattn_prefill_workspace_bytes(B, H, N, D);
  int rc = run_doc_prepass(doc_ids, doc_is_i64, doc_stride_b, doc_stride_t, B, N, workspace, pre_bytes,
                           &lo, &mono, st);
  if (rc != 0) return rc;
  float* delta = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + pre_bytes);
  int* hi = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(delta) + align_up((size_t)B * H * N * sizeof(float), 256));
  if (lo != nullptr) {
    const long long total = (long long)B * N;
    bwd_run_end_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(lo, hi, N, total);
    if ((rc = (int)cudaGetLastError()) != 0) return rc;
  }
  const long long rows = (long long)B * H * N;
  const unsigned dgrid = (unsigned)((rows * (D / 8) + 255) / 256);
  const DeltaStrides ds = {{so.b, so.h, so.n}, {sg.b, sg.h, sg.n}};
  if (D == 64) {
    if (fp16) bwd_delta_kernel<true, 64><<<dgrid, 256, 0, st>>>(o, d_o, delta, rows, H, N, ds);
    else bwd_delta_kernel<false, 64><<<dgrid, 256, 0, st>>>(o, d_o, delta, rows, H, N, ds);
  } else {
    if (fp16) bwd_delta_kernel<true, 128><<<dgrid, 256, 0, st>>>(o, d_o, delta, rows, H, N, ds);
    else bwd_delta_kernel<false, 128><<<dgrid, 256, 0, st>>>(o, d_o, delta, rows, H, N, ds);
  }
  if ((rc = (int)cudaGetLastError()) != 0) return rc;

  const MaskParams mask = make_mask(N, persistent_parity, temporary_window, persistent_window, mask_flags);
  CUtensorMap q128, do128, q64, do64, ks_map, vs_map;
  if ((rc = encode_q_map(&q128, q, B, H, N, D, sq, dtype, 128)) != 0) return rc;
  if ((rc = encode_q_map(&do128, d_o, B, H, N, D, sg, dtype, 128)) != 0) return rc;
  if ((rc = encode_q_map(&q64, q, B, H, N, D, sq, dtype, 64)) != 0) return rc;
  if ((rc = encode_q_map(&do64, d_o, B, H, N, D, sg, dtype, 64)) != 0) return rc;
  if ((rc = encode_kv_map(&ks_map, k, B, H, N, D, mask.ks, sk, dtype)) != 0) return rc;
  if ((rc = encode_kv_map(&vs_map, v, B, H, N, D, mask.ks, sv, dtype)) != 0) return rc;

  BwdParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.lse = lse;
  prm.delta = delta;
  prm.docs = doc_ids;
  prm.doc_stride_b = doc_stride_b;
  prm.doc_stride_t = doc_stride_t;
  prm.doc_is_i64 = doc_is_i64;
  prm.lo = lo;
  prm.hi = hi;
  prm.mono = mono;
  prm.B = B;
  prm.H = H;
  prm.N = N;
  prm.mask = mask;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.sm_scale = sm_scale;
  prm.status = device_status;

  // dK, dV: one block per 128-token key tile of each parity stream
  auto set_out = [&](int slot, void* ptr, const Strides& s3) {
    (slot == 0 ? prm.out0 : prm.out1) = ptr;
    int64_t* dst = slot == 0 ? prm.out0_stride : prm.out1_stride;
    dst[0] = s3.b, dst[1] = s3.h, dst[2] = s3.n;
  };
  set_out(0, dk, sx[6]);
  set_out(1, dv, sx[7]);
  prm.n_xtiles = mask.ks * ((N / mask.ks + 127) / 128);
  {
    // heads whose q, k, v, dO (4 * N * D * 2 bytes each) share about 48 MB of L2 at a time
    const long long op_bytes = 8LL * N * D;
    const long long gh = (48LL << 20) / (op_bytes > 0 ? op_bytes : 1);
    prm.group_heads = (int)(gh < 1 ? 1 : (gh > 32 ? 32 : gh));
#ifdef SPSATTN_NO_GROUP
    prm.group_heads = 1;
#endif
  }
  if (D == 64)
    rc = fp16 ? launch_prefill_bwd<64, true, kBwdDKV>(ks_map, vs_map, q64, do64, prm, st)
              : launch_prefill_bwd<64, false, kBwdDKV>(ks_map, vs_map, q64, do64, prm, st);
  else
    rc = fp16 ? launch_prefill_bwd<128, true, kBwdDKV>(ks_map, vs_map, q64, do64, prm, st)
              : launch_prefill_bwd<128, false, kBwdDKV>(ks_map, vs_map, q64, do64, prm, st);
  if (rc != 0) return rc;
  // dQ: one block per 128-row query tile
  set_out(0, dq, sx[5]);
  prm.out1 = nullptr;
  prm.n_xtiles = (N + 127) / 128;
  if (D == 64)
    return fp16 ? launch_prefill_bwd<64, true, kBwdDQ>(q128, do128, ks_map, vs_map, prm, st)
                : launch_prefill_bwd<64, false, kBwdDQ>(q128, do128, ks_map, vs_map, prm, st);
  return fp16 ? launch_prefill_bwd<128, true, kBwdDQ>(q128, do128, ks_map, vs_map, prm, st)
              : launch_prefill_bwd<128, false, kBwdDQ>(q128, do128, ks_map, vs_map, prm, st);
}

int spsattn_prefill_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                        const float* lse, void* dq, void* dk, void* dv, const void* doc_ids,
                        int doc_is_i64, int64_t doc_stride_b, int64_t doc_stride_t, int B, int H, int N,
                        int D, int dtype, float sm_scale, int persistent_parity, int temporary_window,
                        int persistent_window, int mask_flags, void* workspace, size_t workspace_bytes,
                        int* device_status, void* stream) {
  int64_t dense[24];
  for (int x = 0; x < 8; ++x) {
    dense[3 * x] = (int64_t)H * N * D;
    dense[3 * x + 1] = (int64_t)N * D;
    dense[3 * x + 2] = D;
  }
  return spsattn_prefill_bwd_strided(q, k, v, o, d_o, lse, dq, dk, dv, dense, doc_ids, doc_is_i64,
                                     doc_stride_b, doc_stride_t, B, H, N, D, dtype, sm_scale,
                                     persistent_parity, temporary_window, persistent_window, mask_flags,
                                     workspace, workspace_bytes, device_status, stream);
}

int spsattn_prefill_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                        const void* doc_ids, int doc_is_i64, int64_t doc_stride_b, int64_t doc_stride_t,
                        int B, int H, int N, int D, int dtype, float sm_scale, int persistent_parity,
                        int temporary_window, int persistent_window, int mask_flags, void* workspace,
                        size_t workspace_bytes, int* device_status, void* stream) {
  const int64_t dense[3] = {(int64_t)H * N * D, (int64_t)N * D, (int64_t)D};
  return spsattn_prefill_fwd_strided(q, k, v, o, lse, dense, dense, dense, dense, doc_ids, doc_is_i64,
                                     doc_stride_b, doc_stride_t, B, H, N, D, dtype, sm_scale,
                                     persistent_parity, temporary_window, persistent_window, mask_flags,
                                     workspace, workspace_bytes, device_status, stream);
}

int spsattn_debug_visibility(uint8_t* vis, const void* doc_ids, int doc_is_i64, int64_t doc_stride_b,
                             int64_t doc_stride_t, int B, int N, int persistent_parity,
                             int temporary_window, int persistent_window, int mask_flags,
                             void* workspace, size_t workspace_bytes, void* stream) {
  if (!vis || B <= 0 || N <= 0 || N > 4096) return SPSATTN_ERR_ARG;
  if (persistent_parity != SPSATTN_PARITY_NONE && (N & 1)) return SPSATTN_ERR_ODD_LENGTH;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int *lo = nullptr, *mono = nullptr;
  int rc = run_doc_prepass(doc_ids, doc_is_i64, doc_stride_b, doc_stride_t, B, N, workspace,
                           workspace_bytes, &lo, &mono, st);
  if (rc != 0) return rc;
  const MaskParams mask = make_mask(N, persistent_parity, temporary_window, persistent_window, mask_flags);
  dim3 grid((N + 255) / 256, N, B);
  visibility_kernel<<<grid, 256, 0, st>>>(vis, doc_ids, doc_is_i64, doc_stride_b, doc_stride_t, lo, mono, N,
                                          mask);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------ decode

static size_t decode_ticket_bytes(int S, int H) {
  return align_up(((size_t)S * H + (size_t)S) * sizeof(int), 256);
}

static size_t decode_records_bytes(int S, int H, int D, int nq, const spsattn_segment* segs,
                                   int n_segments) {
  const long long rows = decode_max_rows(segs, n_segments);
  const int chunk = decode_chunk_rows(S, H, rows);
  long long n_chunks = (rows + chunk - 1) / chunk;
  if (n_chunks < 1) n_chunks = 1;
  // the tensor-core kernel indexes its records by (segment, chunk) plus one slot for the
  // current-token entries: room for whichever layout the call ends up using
  const long long slots = tc_slots(segs, n_segments, kMaxExtras, tc_chunk_rows(S, H, segs, n_segments), nullptr, nullptr);
  if (slots > n_chunks) n_chunks = slots;
  return align_up((size_t)S * H * n_chunks * nq * (D + 2) * sizeof(float), 256);
}

size_t spsattn_decode_workspace_bytes(int S, int H, int D, int nq, const spsattn_segment* segs,
                                      int n_segments) {
  if (S <= 0 || H <= 0 || D <= 0 || nq <= 0 || n_segments < 0 || (n_segments > 0 && !segs)) return 256;
  return decode_records_bytes(S, H, D, nq, segs, n_segments);
}

size_t spsattn_decode_step_workspace_bytes(int S, int H, int D, int nq, const spsattn_segment* segs,
                                           int n_segments) {
  if (S <= 0 || H <= 0 || D <= 0 || nq <= 0 || n_segments < 0 || (n_segments > 0 && !segs)) return 256;
  return decode_records_bytes(S, H, D, nq, segs, n_segments) + decode_ticket_bytes(S, H);
}

// Shared body of the decode entry points.  out_dtype: 2 = fp32, else 16-bit in the queries' format.
static int decode_impl(const void* q, int nq, void* out, int out_dtype, const spsattn_segment* segs,
                       int n_segments, const spsattn_extra* extras, int n_extras,
                       const spsattn_kv_append* append, bool single_launch, int S, int H, int D, int dtype,
                       float sm_scale, void* workspace, size_t workspace_bytes, int* device_status,
                       void* stream) {
  if (!q || !out) return SPSATTN_ERR_ARG;
  if (nq != 1 && nq != 2) return SPSATTN_ERR_ARG;
  if (S <= 0 || H <= 0) return SPSATTN_ERR_ARG;
  if (n_segments < 0 || n_segments > kMaxSegments || (n_segments > 0 && !segs)) return SPSATTN_ERR_ARG;
  if (n_extras < 0 || n_extras > kMaxExtras || (n_extras > 0 && !extras)) return SPSATTN_ERR_ARG;
  if (dtype != SPSATTN_DTYPE_BF16 && dtype != SPSATTN_DTYPE_FP16) return SPSATTN_ERR_ARG;
  if (out_dtype != SPSATTN_DTYPE_FP32 && out_dtype != dtype) return SPSATTN_ERR_ARG;
  if (!isfinite(sm_scale)) return SPSATTN_ERR_ARG;
  if (D != 8 && D != 16 && D != 32 && D != 64 && D != 128 && D != 256) return SPSATTN_ERR_HEAD_DIM;
  if (!aligned16(q) || !aligned16(out)) return SPSATTN_ERR_ALIGN;
  if ((long long)S * H > 0x7fffffffLL) return SPSATTN_ERR_TOO_LARGE;

  DecodeParams prm;
  memset(&prm, 0, sizeof(prm));
  for (int x = 0; x < n_segments; ++x) {
    const spsattn_segment& sg = segs[x];
    if (!sg.lengths) return SPSATTN_ERR_ARG;
    if (sg.max_rows > 0 && (!sg.k || !sg.v)) return SPSATTN_ERR_ARG;
    if (sg.max_rows > 0 && (!aligned16(sg.k) || !aligned16(sg.v))) return SPSATTN_ERR_ALIGN;
    if ((sg.seq_stride % 8) || (sg.head_stride % 8) || (sg.row_stride % 8) || sg.row_stride < D)
      return SPSATTN_ERR_ALIGN;
    DecodeSeg& d = prm.seg[x];
    d.k = sg.k;
    d.v = sg.v;
    d.seq_offset = sg.seq_offset;
    d.seq_stride = sg.seq_stride;
    d.head_stride = sg.head_stride;
    d.row_stride = sg.row_stride;
    d.lengths = sg.lengths;
    d.lengths_per_head = sg.lengths_per_head;
    d.max_rows = sg.max_rows > 0 ? sg.max_rows : 0;
    d.query_mask = sg.query_mask;
  }
  for (int e = 0; e < n_extras; ++e) {
    if (!extras[e].k || !extras[e].v) return SPSATTN_ERR_ARG;
    if (!aligned16(extras[e].k) || !aligned16(extras[e].v)) return SPSATTN_ERR_ALIGN;
    prm.extra_k[e] = extras[e].k;
    prm.extra_v[e] = extras[e].v;
    prm.extra_mask[e] = extras[e].query_mask;
  }
  const long long rows = decode_max_rows(segs, n_segments);
  const int path = g_decode_path.load();
  const bool tc_ok = single_launch && tc_supported(segs, n_segments, D);
  if (path == 2 && !tc_ok) return SPSATTN_ERR_ARG;
  // automatic choice: the tensor-core kernel when whole segments, one block each, already fill
  // the machine (two blocks per SM): then every block streams a long run of tiles, merges in
  // shared memory and its start-up is amortised (90 % of the copy bandwidth at 128 sequences x 16
  // heads x 64, 5.1 TB/s against 4.4 at 32 x 16 x 128).  With fewer (sequence, head) pairs the
  // segments have to be cut into short chunks and the CUDA-core kernel, with its 740 small
  // resident blocks, is the better fit.
  long long long_segments = 0;
  for (int x = 0; x < n_segments; ++x) long_segments += segs[x].max_rows > kTcSmallRows ? 1 : 0;
  const bool tc_fits = (long long)S * H * long_segments >= 148LL * 3;
  const bool use_tc = tc_ok && (path == 2 || (path == 0 && tc_fits));
  long long n_chunks;
  if (use_tc) {
    prm.chunk_rows = tc_chunk_rows(S, H, segs, n_segments);
    n_chunks = tc_slots(segs, n_segments, n_extras, prm.chunk_rows, prm.seg_chunks, &prm.small_segs);
    prm.extras_slot = (n_extras > 0 || prm.small_segs != 0) ? (int)n_chunks - 1 : -1;
  } else {
    prm.chunk_rows = decode_chunk_rows(S, H, rows);
    n_chunks = (rows + prm.chunk_rows - 1) / prm.chunk_rows;
    if (n_chunks < 1) n_chunks = 1;
    prm.extras_slot = -1;
  }
  if (n_chunks > 65535) return SPSATTN_ERR_TOO_LARGE;
  prm.n_chunks = (int)n_chunks;
  const size_t raw = (size_t)S * H * n_chunks * nq * (D + 2) * sizeof(float);
  const size_t records = single_launch ? decode_records_bytes(S, H, D, nq, segs, n_segments) : align_up(raw, 256);
  const size_t need = single_launch ? records + decode_ticket_bytes(S, H) : raw;
  if (!workspace || workspace_bytes < need) return SPSATTN_ERR_WORKSPACE;
  if (append && !single_launch) return SPSATTN_ERR_ARG;
  if (!aligned16(workspace)) return SPSATTN_ERR_ALIGN;
  if (append) {
    const spsattn_kv_append& a = *append;
    if (!a.br_k || !a.br_v || !a.br_len || !a.k_retained || !a.v_retained || !a.active)
      return SPSATTN_ERR_ARG;
    if (a.retained_storage < 0) return SPSATTN_ERR_ARG;
    if (a.window_tokens > 0) {
      if (!a.nw_k || !a.nw_v || !a.nw_len || !a.nw_pos || !a.k_window || !a.v_window)
        return SPSATTN_ERR_ARG;
      if (a.window_storage <= 0) return SPSATTN_ERR_ARG;
    }
    DecodeAppend& d = prm.app;
    d.nw_k = reinterpret_cast<uint16_t*>(a.nw_k);
    d.nw_v = reinterpret_cast<uint16_t*>(a.nw_v);
    d.nw_len = a.nw_len;
    d.nw_pos = a.nw_pos;
    d.br_k = reinterpret_cast<uint16_t*>(a.br_k);
    d.br_v = reinterpret_cast<uint16_t*>(a.br_v);
    d.br_len = a.br_len;
    d.k_window = reinterpret_cast<const uint16_t*>(a.k_window);
    d.v_window = reinterpret_cast<const uint16_t*>(a.v_window);
    d.k_retained = reinterpret_cast<const uint16_t*>(a.k_retained);
    d.v_retained = reinterpret_cast<const uint16_t*>(a.v_retained);
    d.active = a.active;
    d.window_storage = a.window_storage;
    d.retained_storage = a.retained_storage;
    d.window_tokens = a.window_tokens > 0 ? a.window_tokens : 0;
  }
  if (single_launch) prm.tickets = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(workspace) + records);
  prm.q = q;
  prm.out = out;
  prm.out16 = out_dtype != SPSATTN_DTYPE_FP32;
  prm.partial = reinterpret_cast<float*>(workspace);
  prm.n_segments = n_segments;
  prm.n_extras = n_extras;
  prm.S = S;
  prm.H = H;
  prm.nq = nq;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.status = device_status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool fp16 = dtype == SPSATTN_DTYPE_FP16;
  if (use_tc) {
    DecodeMaps maps;
    memset(&maps, 0, sizeof(maps));
    for (int x = 0; x < n_segments; ++x) {
      if (prm.seg_chunks[x] == 0) continue;
      int rc = encode_cache_map(&maps.k[x], segs[x].k, segs[x], S, H, D, dtype);
      if (rc == 0) rc = encode_cache_map(&maps.v[x], segs[x].v, segs[x], S, H, D, dtype);
      if (rc != 0) return rc;
    }
    return D == 64 ? launch_decode_tc_d<64>(maps, prm, nq, fp16, st)
                   : launch_decode_tc_d<128>(maps, prm, nq, fp16, st);
  }
  switch (D) {
    case 8: return launch_decode_d<8>(prm, nq, fp16, st);
    case 16: return launch_decode_d<16>(prm, nq, fp16, st);
    case 32: return launch_decode_d<32>(prm, nq, fp16, st);
    case 64: return launch_decode_d<64>(prm, nq, fp16, st);
    case 128: return launch_decode_d<128>(prm, nq, fp16, st);
    default: return launch_decode_d<256>(prm, nq, fp16, st);
  }
}

int spsattn_decode_fwd(const void* q, int nq, float* out, const spsattn_segment* segs, int n_segments,
                       const spsattn_extra* extras, int n_extras, int S, int H, int D, int dtype,
                       float sm_scale, void* workspace, size_t workspace_bytes, int* device_status,
                       void* stream) {
  return decode_impl(q, nq, out, SPSATTN_DTYPE_FP32, segs, n_segments, extras, n_extras, nullptr, false, S, H,
                     D, dtype, sm_scale, workspace, workspace_bytes, device_status, stream);
}

int spsattn_decode_step(const void* q, int nq, void* out, int out_dtype, const spsattn_segment* segs,
                        int n_segments, const spsattn_extra* extras, int n_extras,
                        const spsattn_kv_append* append, int S, int H, int D, int dtype, float sm_scale,
                        void* workspace, size_t workspace_bytes, int* device_status, void* stream) {
  return decode_impl(q, nq, out, out_dtype, segs, n_segments, extras, n_extras, append, true, S, H, D, dtype,
                     sm_scale, workspace, workspace_bytes, device_status, stream);
}

int spsattn_debug_wait_expiry(int* device_status, unsigned long long limit_ns, int* device_result,
                              void* stream) {
  if (device_status == nullptr) return SPSATTN_ERR_ARG;
  if (limit_ns > 1000000000ull) return SPSATTN_ERR_ARG;    // a test hook: never more than a second
  wait_expiry_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(device_status, limit_ns,
                                                                         device_result);
  return (int)cudaGetLastError();
}

int spsattn_debug_prefill_path(int path) {
  if (path < 0 || path > 2) return SPSATTN_ERR_ARG;
  g_prefill_path.store(path);
  return 0;
}

int spsattn_debug_decode_path(int path) {
  if (path < 0 || path > 2) return SPSATTN_ERR_ARG;
  g_decode_path.store(path);
  return 0;
}

// ------------------------------------------------------------------------------------ rope + cast

static int rope_impl(const void* x, int x_dtype, int64_t xs_b, int64_t xs_n, int64_t xs_h,
                     const float* freqs_cis, int64_t freqs_stride_b, const spsattn_rope_group* groups,
                     int n_groups, int out_dtype, int B, int N, int heads_per_group, int D, void* stream) {
  if (!x || !groups || n_groups < 1 || n_groups > kMaxRopeGroups) return SPSATTN_ERR_ARG;
  if (B <= 0 || N <= 0 || heads_per_group <= 0 || D <= 0) return SPSATTN_ERR_ARG;
  if (x_dtype < 0 || x_dtype > 2) return SPSATTN_ERR_ARG;
  if (out_dtype != SPSATTN_DTYPE_BF16 && out_dtype != SPSATTN_DTYPE_FP16) return SPSATTN_ERR_ARG;
  if (D % 8) return SPSATTN_ERR_HEAD_DIM;
  const int in_align = x_dtype == 2 ? 4 : 8;   // elements per 16 bytes
  if ((xs_b % in_align) || (xs_n % in_align) || (xs_h % in_align) || (freqs_stride_b % 2))
    return SPSATTN_ERR_ALIGN;
  if (!aligned16(x)) return SPSATTN_ERR_ALIGN;
  RopeParams p;
  memset(&p, 0, sizeof(p));
  bool any_rotate = false;
  for (int g = 0; g < n_groups; ++g) {
    const spsattn_rope_group& sg = groups[g];
    if (!sg.out) return SPSATTN_ERR_ARG;
    if ((sg.stride_b % 8) || (sg.stride_n % 8) || (sg.stride_h % 8) || !aligned16(sg.out))
      return SPSATTN_ERR_ALIGN;
    p.group[g].out = reinterpret_cast<uint16_t*>(sg.out);
    p.group[g].os_b = sg.stride_b;
    p.group[g].os_n = sg.stride_n;
    p.group[g].os_h = sg.stride_h;
    p.group[g].rotate = sg.rotate != 0;
    any_rotate |= sg.rotate != 0;
  }
  if (any_rotate && (!freqs_cis || !aligned16(freqs_cis))) return freqs_cis ? SPSATTN_ERR_ALIGN : SPSATTN_ERR_ARG;
  p.x = x;
  p.x_dtype = x_dtype;
  p.xs_b = xs_b;
  p.xs_n = xs_n;
  p.xs_h = xs_h;
  p.freqs = reinterpret_cast<const float2*>(freqs_cis);
  p.fs_b = freqs_stride_b;
  p.heads_per_group = heads_per_group;
  p.out_fp16 = out_dtype == SPSATTN_DTYPE_FP16;
  p.B = B;
  p.N = N;
  p.H = heads_per_group * n_groups;
  p.D = D;
  const long long total = (long long)B * N * p.H * (D / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  rope_cast_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return (int)cudaGetLastError();
}

int spsattn_rope_cast(const void* x, int x_dtype, int64_t x_stride_b, int64_t x_stride_n,
                      int64_t x_stride_h, const float* freqs_cis, int64_t freqs_stride_b, void* out,
                      int out_dtype, int64_t out_stride_b, int64_t out_stride_n, int64_t out_stride_h,
                      int B, int N, int H, int D, int rotate, void* stream) {
  spsattn_rope_group g;
  g.out = out;
  g.stride_b = out_stride_b;
  g.stride_n = out_stride_n;
  g.stride_h = out_stride_h;
  g.rotate = rotate;
  g.reserved = 0;
  return rope_impl(x, x_dtype, x_stride_b, x_stride_n, x_stride_h, freqs_cis, freqs_stride_b, &g, 1,
                   out_dtype, B, N, H, D, stream);
}

int spsattn_qkv_rope_cast(const void* x, int x_dtype, int64_t x_stride_b, int64_t x_stride_n,
                          int64_t x_stride_h, const float* freqs_cis, int64_t freqs_stride_b,
                          const spsattn_rope_group* groups, int n_groups, int out_dtype, int B, int N,
                          int heads_per_group, int D, void* stream) {
  return rope_impl(x, x_dtype, x_stride_b, x_stride_n, x_stride_h, freqs_cis, freqs_stride_b, groups,
                   n_groups, out_dtype, B, N, heads_per_group, D, stream);
}

// ------------------------------------------------------------------------------- prefill -> caches

int spsattn_fill_decode_caches(const void* k, const void* v, int64_t stride_b, int64_t stride_n,
                               int64_t stride_h, const uint8_t* doc_mask, void* br_k, void* br_v,
                               int64_t* br_len, void* nw_k, void* nw_v, int64_t* nw_len, int64_t* nw_pos,
                               int B, int T, int H, int D, int retained_storage, int window_storage,
                               int window_tokens, int retained_slot, int window_slot, void* stream) {
  if (!k || !v || !doc_mask || !br_k || !br_v || !br_len) return SPSATTN_ERR_ARG;
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0 || retained_storage < 0) return SPSATTN_ERR_ARG;
  if (T >= 32768) return SPSATTN_ERR_TOO_LARGE;
  if ((retained_slot != 0 && retained_slot != 1) || (window_slot != 0 && window_slot != 1))
    return SPSATTN_ERR_ARG;
  if (window_tokens > 0 && (!nw_k || !nw_v || !nw_len || !nw_pos || window_storage <= 0))
    return SPSATTN_ERR_ARG;
  if ((D % 8) || (stride_b % 8) || (stride_n % 8) || (stride_h % 8) || stride_h < D) return SPSATTN_ERR_ALIGN;
  if (!aligned16(k) || !aligned16(v) || !aligned16(br_k) || !aligned16(br_v)) return SPSATTN_ERR_ALIGN;
  if (window_tokens > 0 && (!aligned16(nw_k) || !aligned16(nw_v))) return SPSATTN_ERR_ALIGN;
  CacheFillParams p;
  p.k = reinterpret_cast<const uint16_t*>(k);
  p.v = reinterpret_cast<const uint16_t*>(v);
  p.stride_b = stride_b;
  p.stride_n = stride_n;
  p.stride_h = stride_h;
  p.doc_mask = doc_mask;
  p.br_k = reinterpret_cast<uint16_t*>(br_k);
  p.br_v = reinterpret_cast<uint16_t*>(br_v);
  p.br_len = br_len;
  p.nw_k = reinterpret_cast<uint16_t*>(nw_k);
  p.nw_v = reinterpret_cast<uint16_t*>(nw_v);
  p.nw_len = nw_len;
  p.nw_pos = nw_pos;
  p.T = T;
  p.H = H;
  p.D = D;
  p.retained_storage = retained_storage;
  p.window_storage = window_storage;
  p.window_tokens = window_tokens > 0 ? window_tokens : 0;
  p.retained_slot = retained_slot;
  p.window_slot = window_slot;
  dim3 grid((T + kFillChunk - 1) / kFillChunk, B);
  cache_fill_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------- allocation-free decode
// Scratch for spsattn_decode_fwd_noalloc: lives in the library image, one copy per device that
// loads it.  In host code the name below is only a handle for cudaGetSymbolAddress, never a
// device address; kernels receive the looked-up pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SPSATTN_NOALLOC_SCRATCH_BYTES];

namespace {
// Device address of the scratch buffer on the current device.  Looked up on every call: after the
// first call on a device (which loads the module there) this is a host-side table look-up, and
// an address cached across cudaDeviceReset or a new context would be stale.
int noalloc_scratch_ptr(void** out) {
  void* ptr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
  if (e != cudaSuccess) return (int)e;
  if (ptr == nullptr) return SPSATTN_ERR_ARG;
  *out = ptr;
  return 0;
}
}  // namespace

int spsattn_decode_fwd_noalloc(const void* q, int nq, float* out, const spsattn_segment* segs,
                               int n_segments, const spsattn_extra* extras, int n_extras, int S, int H,
                               int D, int dtype, float sm_scale, int* device_status, void* stream) {
  if (S <= 0 || H <= 0 || D <= 0 || (nq != 1 && nq != 2)) return SPSATTN_ERR_ARG;
  if (n_segments < 0 || n_segments > kMaxSegments || (n_segments > 0 && !segs)) return SPSATTN_ERR_ARG;
  const size_t need = spsattn_decode_workspace_bytes(S, H, D, nq, segs, n_segments);
  if (need > (size_t)SPSATTN_NOALLOC_SCRATCH_BYTES) return SPSATTN_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  const int rc = noalloc_scratch_ptr(&scratch);
  if (rc != 0) return rc;
  return spsattn_decode_fwd(q, nq, out, segs, n_segments, extras, n_extras, S, H, D, dtype, sm_scale,
                            scratch, (size_t)SPSATTN_NOALLOC_SCRATCH_BYTES, device_status, stream);
}

// --------------------------------------------------------------------------------------- kv update

int spsattn_kv_update(void* nw_k, void* nw_v, int64_t* nw_len, int64_t* nw_pos, void* br_k, void* br_v,
                      int64_t* br_len, const void* k_window, const void* v_window, const void* k_retained,
                      const void* v_retained, const int8_t* active, int S, int H, int D,
                      int window_storage, int retained_storage, int window_tokens, int elem_bytes,
                      void* stream) {
  if (!br_k || !br_v || !br_len || !k_retained || !v_retained || !active) return SPSATTN_ERR_ARG;
  if (S <= 0 || H <= 0 || D <= 0 || retained_storage < 0) return SPSATTN_ERR_ARG;
  if (elem_bytes != 2 && elem_bytes != 4) return SPSATTN_ERR_ARG;
  if ((D * elem_bytes) % 4) return SPSATTN_ERR_ALIGN;
  if (window_tokens > 0) {
    if (!nw_k || !nw_v || !nw_len || !nw_pos || !k_window || !v_window) return SPSATTN_ERR_ARG;
    if (window_storage <= 0) return SPSATTN_ERR_ARG;
  }
  KvUpdateParams p;
  p.nw_k = reinterpret_cast<uint32_t*>(nw_k);
  p.nw_v = reinterpret_cast<uint32_t*>(nw_v);
  p.nw_len = nw_len;
  p.nw_pos = nw_pos;
  p.br_k = reinterpret_cast<uint32_t*>(br_k);
  p.br_v = reinterpret_cast<uint32_t*>(br_v);
  p.br_len = br_len;
  p.k_window = reinterpret_cast<const uint32_t*>(k_window);
  p.v_window = reinterpret_cast<const uint32_t*>(v_window);
  p.k_retained = reinterpret_cast<const uint32_t*>(k_retained);
  p.v_retained = reinterpret_cast<const uint32_t*>(v_retained);
  p.active = active;
  p.H = H;
  p.row_words = D * elem_bytes / 4;
  p.window_storage = window_storage;
  p.retained_storage = retained_storage;
  p.window_tokens = window_tokens > 0 ? window_tokens : 0;
  kv_update_kernel<<<S, 256, (size_t)H * sizeof(long long), reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------ block glue (norm, gate)

int spsattn_add_rmsnorm(void* x, const void* delta, const void* weight, void* y, int dtype,
                        long long rows, int C, float eps, void* stream) {
  if (!x || !weight || (!y && !delta)) return SPSATTN_ERR_ARG;
  if (rows <= 0 || C <= 0 || !(eps >= 0.f)) return SPSATTN_ERR_ARG;
  if (dtype != SPSATTN_DTYPE_BF16 && dtype != SPSATTN_DTYPE_FP32) return SPSATTN_ERR_ARG;
  const int vec = dtype == SPSATTN_DTYPE_BF16 ? 8 : 4;
  if (C % vec) return SPSATTN_ERR_ALIGN;
  if (!aligned16(x) || !aligned16(weight) || (y && !aligned16(y)) || (delta && !aligned16(delta)))
    return SPSATTN_ERR_ALIGN;
  RmsNormParams p;
  p.x = x;
  p.delta = delta;
  p.weight = weight;
  p.y = y;
  p.rows = rows;
  p.C = C;
  p.eps = eps;
  const unsigned blocks = (unsigned)(rows < 148LL * 16 ? rows : 148LL * 16);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == SPSATTN_DTYPE_BF16)
    add_rmsnorm_kernel<true><<<blocks, 256, 0, st>>>(p);
  else
    add_rmsnorm_kernel<false><<<blocks, 256, 0, st>>>(p);
  return (int)cudaGetLastError();
}

int spsattn_swiglu(const void* gate_up, void* y, int dtype, long long rows, int I, void* stream) {
  if (!gate_up || !y) return SPSATTN_ERR_ARG;
  if (rows <= 0 || I <= 0) return SPSATTN_ERR_ARG;
  if (dtype != SPSATTN_DTYPE_BF16 && dtype != SPSATTN_DTYPE_FP32) return SPSATTN_ERR_ARG;
  const int vec = dtype == SPSATTN_DTYPE_BF16 ? 8 : 4;
  if (I % vec) return SPSATTN_ERR_ALIGN;
  if (!aligned16(gate_up) || !aligned16(y)) return SPSATTN_ERR_ALIGN;
  SwigluParams p;
  p.gate_up = gate_up;
  p.y = y;
  p.rows = rows;
  p.I = I;
  const long long total = rows * (I / vec);
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == SPSATTN_DTYPE_BF16)
    swiglu_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(p);
  else
    swiglu_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(p);
  return (int)cudaGetLastError();
}

}  // extern "C"
