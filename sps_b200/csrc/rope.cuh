// Rotary embedding + cast, the producer side of the attention operands: reads q or k as the
// projection left them ([B, N, H, D] view, bf16 / fp16 / fp32, any row strides), rotates adjacent
// element pairs by the position's complex frequency in fp32 and writes 16-bit rows in the layout
// the attention kernel reads in place.  With rotate = 0 it is a plain cast (for v).
// The H heads of the view may be split into up to six consecutive groups (the q, k and v thirds
// of a fused projection; for a decode step, those of both slots of a token pair), each with its
// own destination, strides and rotate flag, so that one launch produces all operands.
// Reference computation: src/modeling/models/model.py:201-230 (apply_rotary_emb: view pairs as
// complex, multiply by freqs_cis, back to real, cast) followed by the bf16 cast of
// src/modeling/models/sps/core.py:53-55.
#pragma once

#include "common.cuh"

namespace spsattn {

constexpr int kMaxRopeGroups = 6;

struct RopeGroup {
  uint16_t* out;
  int64_t os_b, os_n, os_h;    // elements
  int rotate;
};

struct RopeParams {
  const void* x;
  int x_dtype;                 // 0 bf16, 1 fp16, 2 fp32
  int64_t xs_b, xs_n, xs_h;    // elements
  const float2* freqs;         // [N, D/2] or [B, N, D/2] (cos, sin)
  int64_t fs_b;                // elements of float2 per batch row, 0 when shared
  RopeGroup group[kMaxRopeGroups];
  int heads_per_group;         // H = n_groups * heads_per_group
  int out_fp16;
  int B, N, H, D;
};

__global__ void __launch_bounds__(256) rope_cast_kernel(const RopeParams p) {
  const int vec_per_row = p.D / 8;
  const long long total = (long long)p.B * p.N * p.H * vec_per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int x8 = (int)(idx % vec_per_row);
    long long r = idx / vec_per_row;
    const int h = (int)(r % p.H);
    r /= p.H;
    const int n = (int)(r % p.N);
    const int b = (int)(r / p.N);
    const size_t src = (size_t)b * p.xs_b + (size_t)n * p.xs_n + (size_t)h * p.xs_h + x8 * 8;
    float f[8];
    if (p.x_dtype == 2) {
      const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + src);
      const float4 c = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + src + 4);
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
      f[4] = c.x; f[5] = c.y; f[6] = c.z; f[7] = c.w;
    } else {
      const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.x) + src);
      if (p.x_dtype == 1) {
        unpack2<true>(u.x, f[0], f[1]); unpack2<true>(u.y, f[2], f[3]);
        unpack2<true>(u.z, f[4], f[5]); unpack2<true>(u.w, f[6], f[7]);
      } else {
        unpack2<false>(u.x, f[0], f[1]); unpack2<false>(u.y, f[2], f[3]);
        unpack2<false>(u.z, f[4], f[5]); unpack2<false>(u.w, f[6], f[7]);
      }
    }
    const int gi = h / p.heads_per_group;
    RopeGroup grp = p.group[0];   // selected without indexing the parameter block dynamically
    if (gi == 1) grp = p.group[1];
    if (gi == 2) grp = p.group[2];
    if (gi == 3) grp = p.group[3];
    if (gi == 4) grp = p.group[4];
    if (gi == 5) grp = p.group[5];
    if (grp.rotate) {
      const float2* fr = p.freqs + (size_t)b * p.fs_b + (size_t)n * (p.D / 2) + x8 * 4;
      const float4 c01 = *reinterpret_cast<const float4*>(fr);
      const float4 c23 = *reinterpret_cast<const float4*>(fr + 2);
      const float cs[8] = {c01.x, c01.y, c01.z, c01.w, c23.x, c23.y, c23.z, c23.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = f[2 * i], bb = f[2 * i + 1], c = cs[2 * i], s = cs[2 * i + 1];
        // (a + bi)(c + si), products and sums rounded separately like the complex multiply
        f[2 * i] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(bb, s));
        f[2 * i + 1] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(bb, c));
      }
    }
    uint4 o;
    if (p.out_fp16) {
      o.x = pack2<true>(f[0], f[1]); o.y = pack2<true>(f[2], f[3]);
      o.z = pack2<true>(f[4], f[5]); o.w = pack2<true>(f[6], f[7]);
    } else {
      o.x = pack2<false>(f[0], f[1]); o.y = pack2<false>(f[2], f[3]);
      o.z = pack2<false>(f[4], f[5]); o.w = pack2<false>(f[6], f[7]);
    }
    const int hg = h - gi * p.heads_per_group;
    *reinterpret_cast<uint4*>(grp.out + (size_t)b * grp.os_b + (size_t)n * grp.os_n +
                              (size_t)hg * grp.os_h + x8 * 8) = o;
  }
}

}  // namespace spsattn
