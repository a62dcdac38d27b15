// Small kernels around the prefill path: the document pre-pass, a plain CUDA-core prefill for
// head dims the tensor-core kernel does not cover, and the visibility test hook.
#pragma once

#include "common.cuh"
#include "mask.cuh"

namespace spsattn {

__device__ __forceinline__ long long load_doc(const void* docs, int is_i64, size_t off) {
  return is_i64 ? reinterpret_cast<const long long*>(docs)[off]
                : (long long)reinterpret_cast<const int*>(docs)[off];
}

// One block per batch row: lo[b][i] = first row of the run of equal ids containing row i
// (inclusive max-scan of run-start positions), mono[b] = 1 iff the ids never decrease.
// Each thread scans kItems consecutive rows, so rows up to 8192 need a single pass.
__global__ void __launch_bounds__(1024)
doc_prepass_kernel(const void* docs, int is_i64, int64_t stride_b, int64_t stride_t, int N,
                   int* __restrict__ lo, int* __restrict__ mono, int* __restrict__ work_counter) {
  constexpr int kItems = 8;
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  __shared__ int s_mono;
  const int b = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  // the attention kernel behind this one may be launched as a programmatic dependent: let its
  // blocks take the free SMs now (it waits for this grid before it reads lo / mono)
  grid_launch_dependents();
  const uint8_t* base =
      reinterpret_cast<const uint8_t*>(docs) + (size_t)b * stride_b * (is_i64 ? 8 : 4);
  if (tid == 0) {
    s_carry = 0;
    s_mono = 1;
    // the attention kernel that follows in the stream draws its work items from this counter
    if (b == 0 && work_counter != nullptr) *work_counter = 0;
  }
  __syncthreads();
  bool dec = false;
  for (int c0 = 0; c0 < N; c0 += 1024 * kItems) {
    const int i0 = c0 + tid * kItems;
    int v[kItems];
    long long prev = 0;
    if (i0 > 0 && i0 - 1 < N) prev = load_doc(base, is_i64, (size_t)(i0 - 1) * stride_t);
    int run = 0;
#pragma unroll
    for (int x = 0; x < kItems; ++x) {
      const int i = i0 + x;
      if (i < N) {
        const long long d = load_doc(base, is_i64, (size_t)i * stride_t);
        if (i > 0) {
          if (d != prev) run = i;
          dec |= d < prev;
        }
        prev = d;
      }
      v[x] = run;   // inclusive max of the run starts inside this thread's span
    }
    int tot = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, tot, o);
      if (lane >= o) tot = max(tot, u);
    }
    if (lane == 31) s_warp[warp] = tot;
    __syncthreads();
    if (warp == 0) {
      int wv = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, wv, o);
        if (lane >= o) wv = max(wv, u);
      }
      s_warp[lane] = wv;
    }
    __syncthreads();
    int pre = __shfl_up_sync(0xffffffffu, tot, 1);   // everything before this thread in its warp
    if (lane == 0) pre = 0;
    pre = max(pre, max(s_carry, warp > 0 ? s_warp[warp - 1] : 0));
#pragma unroll
    for (int x = 0; x < kItems; ++x)
      if (i0 + x < N) lo[(size_t)b * N + i0 + x] = max(v[x], pre);
    __syncthreads();
    if (tid == 1023) s_carry = max(tot, pre);
    __syncthreads();
  }
  if (dec) s_mono = 0;
  __syncthreads();
  if (tid == 0) mono[b] = s_mono;
}

// Test hook for the bounded waits: one warp waits, with the given limit, on an mbarrier that
// nobody ever arrives at.  No copy or tensor-core operation is in flight; the wait gives up,
// reports SPSATTN_STATUS_WAIT_EXPIRED through the status word exactly as the attention kernels
// do, and the block ends normally.  result[0] = 1 when the wait returned "gave up".
__global__ void __launch_bounds__(32)
wait_expiry_kernel(int* status, unsigned long long limit_ns, int* result) {
  __shared__ __align__(8) unsigned long long s_bar;
  __shared__ int s_abort;
  const uint32_t bar = smem_u32(&s_bar);
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  __syncwarp();
  bool ok = mbar_try_wait(bar, 0);
  if (!ok) ok = mbar_wait_slow(bar, 0, &s_abort, status, limit_ns);
  ok = __all_sync(0xffffffffu, ok);
  if (threadIdx.x == 0 && result != nullptr) result[0] = ok ? 0 : 1;
}

// vis[b][i][j] = 1 iff key row j is visible to query row i, using the kernels' own arithmetic.
__global__ void visibility_kernel(uint8_t* __restrict__ vis, const void* docs, int is_i64,
                                  int64_t stride_b, int64_t stride_t, const int* __restrict__ lo,
                                  const int* __restrict__ mono, int N, MaskParams m) {
  const int b = blockIdx.z;
  const int i = blockIdx.y;
  const uint8_t* base = docs == nullptr ? nullptr
                                         : reinterpret_cast<const uint8_t*>(docs) +
                                               (size_t)b * stride_b * (is_i64 ? 8 : 4);
  const bool general = docs != nullptr && mono[b] == 0;
  const int lo_i = (docs != nullptr && !general) ? lo[(size_t)b * N + i] : 0;
  int kmin[2], kmax[2];
  row_interval(m, i, lo_i, 0, kmin[0], kmax[0]);
  row_interval(m, i, lo_i, 1, kmin[1], kmax[1]);
  const long long my_doc = general ? load_doc(base, is_i64, (size_t)i * stride_t) : 0;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < N; j += gridDim.x * blockDim.x) {
    const int p = m.ks == 2 ? (j & 1) : 0;
    const int kt = m.ks == 2 ? (j >> 1) : j;
    bool v = kt >= kmin[p] && kt <= kmax[p];
    if (v && general) v = load_doc(base, is_i64, (size_t)j * stride_t) == my_doc;
    vis[((size_t)b * N + i) * N + j] = v ? 1 : 0;
  }
}

// Plain CUDA-core prefill: one warp per query row, lanes stride over the visible key tokens of
// each stream, fp32 math, online softmax per lane merged across the warp at the end.  Serves
// head dims 16, 32 and 256; slow, but the same rule and the same numerics contract.
template <bool FP16>
__global__ void __launch_bounds__(128)
prefill_generic_kernel(const void* __restrict__ q, const void* __restrict__ k,
                       const void* __restrict__ v, void* __restrict__ o, float* __restrict__ lse,
                       const void* docs, int is_i64, int64_t stride_b, int64_t stride_t,
                       const int* __restrict__ lo, const int* __restrict__ mono, int H, int N, int D,
                       MaskParams m, float scale_log2) {
  extern __shared__ float s_q[];  // [4 warps][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + warp;
  const int bh = blockIdx.y;
  const int b = bh / H;
  if (i >= N) return;
  const uint16_t* qp = reinterpret_cast<const uint16_t*>(q) + ((size_t)bh * N + i) * D;
  const uint16_t* kp = reinterpret_cast<const uint16_t*>(k) + (size_t)bh * N * D;
  const uint16_t* vp = reinterpret_cast<const uint16_t*>(v) + (size_t)bh * N * D;
  float* myq = s_q + warp * D;
  for (int d = lane; d < D; d += 32) {
    float lo_f, hi_f;
    unpack2<FP16>((uint32_t)qp[d], lo_f, hi_f);
    myq[d] = lo_f;
  }
  __syncwarp();
  const uint8_t* base = docs == nullptr ? nullptr
                                         : reinterpret_cast<const uint8_t*>(docs) +
                                               (size_t)b * stride_b * (is_i64 ? 8 : 4);
  const bool general = docs != nullptr && mono[b] == 0;
  const int lo_i = (docs != nullptr && !general) ? lo[(size_t)b * N + i] : 0;
  const long long my_doc = general ? load_doc(base, is_i64, (size_t)i * stride_t) : 0;

  // per-lane online softmax state; the accumulator covers D / 32 ... handled by looping d
  float m_run = -1.0e30f, l_run = 0.f;
  float acc[8];  // lane owns dims lane, lane+32, ... (D <= 256)
#pragma unroll
  for (int x = 0; x < 8; ++x) acc[x] = 0.f;

  const int n_streams = m.ks == 2 ? 2 : 1;
  for (int p = 0; p < n_streams; ++p) {
    int kmin, kmax;
    row_interval(m, i, lo_i, p, kmin, kmax);
    if (kmin < 0) kmin = 0;
    for (int kt = kmin; kt <= kmax; ++kt) {
      const int j = m.ks * kt + p;
      if (general && load_doc(base, is_i64, (size_t)j * stride_t) != my_doc) continue;
      // whole warp cooperates on one key: lanes split D
      float part = 0.f;
      for (int d = lane; d < D; d += 32) {
        float kv, dummy;
        unpack2<FP16>((uint32_t)kp[(size_t)j * D + d], kv, dummy);
        part = fmaf(myq[d], kv, part);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
      const float sc = part;
      const float m_new = fmaxf(m_run, sc);
      const float alpha = fast_exp2((m_run - m_new) * scale_log2);
      const float pr = fast_exp2((sc - m_new) * scale_log2);
      l_run = l_run * alpha + pr;
      m_run = m_new;
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const int d = lane + 32 * x;
        if (d < D) {
          float vv, dummy;
          unpack2<FP16>((uint32_t)vp[(size_t)j * D + d], vv, dummy);
          acc[x] = acc[x] * alpha + pr * vv;
        }
      }
    }
  }
  const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
  uint16_t* op = reinterpret_cast<uint16_t*>(o) + ((size_t)bh * N + i) * D;
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const int d = lane + 32 * x;
    if (d < D) op[d] = (uint16_t)(pack2<FP16>(acc[x] * inv_l, 0.f) & 0xffffu);
  }
  if (lse != nullptr && lane == 0)
    lse[(size_t)bh * N + i] = l_run > 0.f ? m_run * scale_log2 + log2f(l_run) : -INFINITY;
}

}  // namespace spsattn
