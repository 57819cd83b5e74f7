// One warp reads one 512-element bf16 row (16 elements per lane) and can write it back as fp16: the building
// block of the kernels that make the fp16 operand copies and the row statistics of the backward.
#pragma once
#include "ptx.cuh"

namespace sd {

struct Row16 {
  float x[16];  // this lane's 16 of the row's 512 elements: [0,8) = elements lane*8.., [8,16) = 256 + lane*8..
};
__device__ __forceinline__ Row16 load_row(const uint16_t* r, int lane) {
  Row16 o;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 w4 = *reinterpret_cast<const uint4*>(r + i * 256 + lane * 8);
    const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[t]));
      o.x[i * 8 + 2 * t] = f.x, o.x[i * 8 + 2 * t + 1] = f.y;
    }
  }
  return o;
}
// the same 16 elements, times `mul`, to fp16 (clamped to the largest finite fp16)
__device__ __forceinline__ void store_row_half(uint16_t* r, int lane, const Row16& v, float mul) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float a = fminf(fmaxf(v.x[i * 8 + 2 * t] * mul, -65504.f), 65504.f);
      const float b = fminf(fmaxf(v.x[i * 8 + 2 * t + 1] * mul, -65504.f), 65504.f);
      w[t] = pack_half2(a, b);
    }
    *reinterpret_cast<uint4*>(r + i * 256 + lane * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

}  // namespace sd
