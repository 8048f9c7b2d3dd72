// Pre-kernel shared by the tensor-core forward and backward: the bias halves of the two relative
// products, which do not depend on the query.
#pragma once

#include <cuda_bf16.h>

namespace mvpa {

// Per-column constants of the two relative products, once per kv head instead of once per CTA:
//   relc[hk][j] = vt[hk] . r_time[hk][j]  (j < T),   relc[hk][128 + j] = z[hk] . r_chan[hk][j]  (j < C)
// (the bias halves of `_rel_bias`, `attentions/attn.py:1308-1313`).
// One thread per column: its key row comes in with 16-byte loads that are all in flight at once (D is 64
// or 128 on the tensor-core paths: 8 or 16 loads), so the kernel costs one memory round trip, not D / 2.
template <int D>
static __global__ void __launch_bounds__(256) rel_const_kernel(const __nv_bfloat16* __restrict__ vt,
                                                               const __nv_bfloat16* __restrict__ z,
                                                               const __nv_bfloat16* __restrict__ rt,
                                                               const __nv_bfloat16* __restrict__ rc,
                                                               float* __restrict__ relc, int T, int C,
                                                               int* __restrict__ status_words) {
  // (also clears the 64 status words of the kernels that follow, where the caller asks for it: one memset
  // node less in front of them)
  if (status_words != nullptr && blockIdx.x == 0 && threadIdx.x < 64) status_words[threadIdx.x] = 0;
  const int hk = blockIdx.x, j = threadIdx.x & 127;
  const bool is_t = threadIdx.x < 128;
  const int rows = is_t ? T : C;
  float acc = 0.f;
  if (j < rows) {
    const uint4* key = reinterpret_cast<const uint4*>((is_t ? rt : rc) + ((size_t)hk * rows + j) * D);
    const uint4* bias = reinterpret_cast<const uint4*>((is_t ? vt : z) + (size_t)hk * D);
    uint4 k[D / 8], b[D / 8];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      k[i] = key[i];
      b[i] = bias[i];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const uint32_t kw[4] = {k[i].x, k[i].y, k[i].z, k[i].w}, bw[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {  // the same pairs in the same order as a two-element walk over d
        const float ax = __uint_as_float(kw[e] << 16), ay = __uint_as_float(kw[e] & 0xffff0000u);
        const float bx = __uint_as_float(bw[e] << 16), by = __uint_as_float(bw[e] & 0xffff0000u);
        acc += ax * bx + ay * by;
      }
    }
  }
  relc[hk * 256 + threadIdx.x] = acc;
}

}  // namespace mvpa
