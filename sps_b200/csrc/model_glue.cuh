// Element-wise kernels that sit between the attention calls and the projections of an SPS
// decoder block, so that a generation step is a short fixed chain of launches: residual add +
// RMSNorm in one pass, and the SwiGLU gate.  Both are bandwidth bound and keep the reference's
// rounding points for 16-bit parameters (every torch op there rounds its result to bf16).
// Reference computation: RMSNorm src/modeling/models/model.py:101-132 (normalise in fp32, cast
// back to the input type, then multiply by the weight), residual adds :324-327, MLP :304-314
// (down(silu(gate(x)) * up(x))).
#pragma once

#include "common.cuh"

namespace spsattn {

struct RmsNormParams {
  void* x;             // [rows, C] residual stream, updated in place when delta is given
  const void* delta;   // [rows, C] or null
  const void* weight;  // [C]
  void* y;             // [rows, C] normalised output
  long long rows;
  int C;
  float eps;
};

__device__ __forceinline__ float round_bf16(float f) {
  return __bfloat162float(__float2bfloat16_rn(f));
}

// One block per row.  BF16 = true: x, delta, weight, y are bf16 and results are rounded where the
// reference's bf16 tensors round; false: everything fp32.  A row of up to 256 * kRowVecs vectors
// stays in registers between the sum of squares and the scaling (one read of x); longer rows are
// read again.
constexpr int kRowVecs = 4;

template <bool BF16>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const RmsNormParams p) {
  constexpr int V = BF16 ? 8 : 4;   // elements per 16-byte access
  __shared__ float s_part[8];
  __shared__ float s_scale;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_vec = p.C / V;
  const bool in_regs = n_vec <= 256 * kRowVecs;

  auto load_row_vec = [&](size_t base, int i, float (&f)[V]) {
    if constexpr (BF16) {
      uint16_t* xp = reinterpret_cast<uint16_t*>(p.x) + base + (size_t)i * V;
      const uint4 u = *reinterpret_cast<const uint4*>(xp);
      unpack2<false>(u.x, f[0], f[1]);
      unpack2<false>(u.y, f[2], f[3]);
      unpack2<false>(u.z, f[4], f[5]);
      unpack2<false>(u.w, f[6], f[7]);
      if (p.delta != nullptr) {
        const uint4 d = *reinterpret_cast<const uint4*>(
            reinterpret_cast<const uint16_t*>(p.delta) + base + (size_t)i * V);
        float g[8];
        unpack2<false>(d.x, g[0], g[1]);
        unpack2<false>(d.y, g[2], g[3]);
        unpack2<false>(d.z, g[4], g[5]);
        unpack2<false>(d.w, g[6], g[7]);
#pragma unroll
        for (int e = 0; e < V; ++e) f[e] = round_bf16(f[e] + g[e]);
        uint4 o;
        o.x = pack2<false>(f[0], f[1]);
        o.y = pack2<false>(f[2], f[3]);
        o.z = pack2<false>(f[4], f[5]);
        o.w = pack2<false>(f[6], f[7]);
        *reinterpret_cast<uint4*>(xp) = o;
      }
    } else {
      float* xp = reinterpret_cast<float*>(p.x) + base + (size_t)i * V;
      const float4 u = *reinterpret_cast<const float4*>(xp);
      f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
      if (p.delta != nullptr) {
        const float4 d = *reinterpret_cast<const float4*>(
            reinterpret_cast<const float*>(p.delta) + base + (size_t)i * V);
        f[0] += d.x; f[1] += d.y; f[2] += d.z; f[3] += d.w;
        *reinterpret_cast<float4*>(xp) = make_float4(f[0], f[1], f[2], f[3]);
      }
    }
  };
  auto store_y_vec = [&](size_t base, int i, const float (&f)[V], float scale) {
    if constexpr (BF16) {
      const uint4 w = *reinterpret_cast<const uint4*>(
          reinterpret_cast<const uint16_t*>(p.weight) + (size_t)i * V);
      float g[8], r[8];
      unpack2<false>(w.x, g[0], g[1]); unpack2<false>(w.y, g[2], g[3]);
      unpack2<false>(w.z, g[4], g[5]); unpack2<false>(w.w, g[6], g[7]);
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = round_bf16(f[e] * scale) * g[e];
      uint4 o;
      o.x = pack2<false>(r[0], r[1]); o.y = pack2<false>(r[2], r[3]);
      o.z = pack2<false>(r[4], r[5]); o.w = pack2<false>(r[6], r[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.y) + base + (size_t)i * V) = o;
    } else {
      const float4 w = *reinterpret_cast<const float4*>(
          reinterpret_cast<const float*>(p.weight) + (size_t)i * V);
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + base + (size_t)i * V) =
          make_float4(f[0] * scale * w.x, f[1] * scale * w.y, f[2] * scale * w.z, f[3] * scale * w.w);
    }
  };

  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const size_t base = (size_t)row * p.C;
    float ss = 0.f;
    float kept[kRowVecs][V];
    if (in_regs) {
#pragma unroll
      for (int k = 0; k < kRowVecs; ++k) {
        const int i = tid + k * 256;
        if (i < n_vec) {
          load_row_vec(base, i, kept[k]);
#pragma unroll
          for (int e = 0; e < V; ++e) ss = fmaf(kept[k][e], kept[k][e], ss);
        }
      }
    } else {
      for (int i = tid; i < n_vec; i += 256) {
        float f[V];
        load_row_vec(base, i, f);
#pragma unroll
        for (int e = 0; e < V; ++e) ss = fmaf(f[e], f[e], ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_part[warp] = ss;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += s_part[w];
      s_scale = rsqrtf(t / (float)p.C + p.eps);
    }
    __syncthreads();
    const float scale = s_scale;
    if (p.y != nullptr) {
      if (in_regs) {
#pragma unroll
        for (int k = 0; k < kRowVecs; ++k) {
          const int i = tid + k * 256;
          if (i < n_vec) store_y_vec(base, i, kept[k], scale);
        }
      } else {
        // second read: x already holds the sum
        for (int i = tid; i < n_vec; i += 256) {
          float f[V];
          if constexpr (BF16) {
            const uint4 u = *reinterpret_cast<const uint4*>(
                reinterpret_cast<const uint16_t*>(p.x) + base + (size_t)i * V);
            unpack2<false>(u.x, f[0], f[1]); unpack2<false>(u.y, f[2], f[3]);
            unpack2<false>(u.z, f[4], f[5]); unpack2<false>(u.w, f[6], f[7]);
          } else {
            const float4 u = *reinterpret_cast<const float4*>(
                reinterpret_cast<const float*>(p.x) + base + (size_t)i * V);
            f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
          }
          store_y_vec(base, i, f, scale);
        }
      }
    }
    __syncthreads();   // s_part / s_scale are reused by the next row
  }
}

struct SwigluParams {
  const void* gate_up;   // [rows, 2 * I]: gate in columns [0, I), up in [I, 2I)
  void* y;               // [rows, I]
  long long rows;
  int I;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

template <bool BF16>
__global__ void __launch_bounds__(256) swiglu_kernel(const SwigluParams p) {
  constexpr int V = BF16 ? 8 : 4;
  const int n_vec = p.I / V;
  const long long total = p.rows * n_vec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / n_vec;
    const int i = (int)(idx % n_vec);
    const size_t src = (size_t)row * 2 * p.I + (size_t)i * V;
    const size_t dst = (size_t)row * p.I + (size_t)i * V;
    if constexpr (BF16) {
      const uint16_t* gp = reinterpret_cast<const uint16_t*>(p.gate_up);
      const uint4 a = *reinterpret_cast<const uint4*>(gp + src);
      const uint4 b = *reinterpret_cast<const uint4*>(gp + src + p.I);
      float g[8], u[8];
      unpack2<false>(a.x, g[0], g[1]); unpack2<false>(a.y, g[2], g[3]);
      unpack2<false>(a.z, g[4], g[5]); unpack2<false>(a.w, g[6], g[7]);
      unpack2<false>(b.x, u[0], u[1]); unpack2<false>(b.y, u[2], u[3]);
      unpack2<false>(b.z, u[4], u[5]); unpack2<false>(b.w, u[6], u[7]);
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] = round_bf16(silu_f(g[e])) * u[e];
      uint4 o;
      o.x = pack2<false>(g[0], g[1]); o.y = pack2<false>(g[2], g[3]);
      o.z = pack2<false>(g[4], g[5]); o.w = pack2<false>(g[6], g[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.y) + dst) = o;
    } else {
      const float* gp = reinterpret_cast<const float*>(p.gate_up);
      const float4 a = *reinterpret_cast<const float4*>(gp + src);
      const float4 b = *reinterpret_cast<const float4*>(gp + src + p.I);
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + dst) =
          make_float4(silu_f(a.x) * b.x, silu_f(a.y) * b.y, silu_f(a.z) * b.z, silu_f(a.w) * b.w);
    }
  }
}

}  // namespace spsattn
