// Pre-kernel shared by the tensor-core forward and backward: the bias halves of the two relative
// products, which do not depend on the query.
#pragma once

#include <cuda_bf16.h>

namespace mvpa {

// Per-column constants of the two relative products, once per kv head instead of once per CTA:
//   relc[hk][j] = vt[hk] . r_time[hk][j]  (j < T),   relc[hk][128 + j] = z[hk] . r_chan[hk][j]  (j < C)
// (the bias halves of `_rel_bias`, `attentions/attn.py:1308-1313`).
static __global__ void __launch_bounds__(256) rel_const_kernel(const __nv_bfloat16* __restrict__ vt,
                                                        const __nv_bfloat16* __restrict__ z,
                                                        const __nv_bfloat16* __restrict__ rt,
                                                        const __nv_bfloat16* __restrict__ rc, float* __restrict__ relc,
                                                        int T, int C, int D) {
  const int hk = blockIdx.x, j = threadIdx.x & 127;
  const bool is_t = threadIdx.x < 128;
  const int rows = is_t ? T : C;
  float acc = 0.f;
  if (j < rows) {
    const __nv_bfloat16* key = (is_t ? rt : rc) + ((size_t)hk * rows + j) * D;
    const __nv_bfloat16* bias = (is_t ? vt : z) + (size_t)hk * D;
    for (int d = 0; d < D; d += 2) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(key + d));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bias + d));
      acc += a.x * b.x + a.y * b.y;
    }
  }
  relc[hk * 256 + threadIdx.x] = acc;
}

}  // namespace mvpa
