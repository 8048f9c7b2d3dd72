// HBM-bound kernels around the attention of an MVPFormer block, encoder and heads:
//
//   rmsnorm / add_rmsnorm   `ln_1`, `ln_f` and the residual sum of the parallel block
//                           (`models/mvpformer.py:132-147`: h = x + MLP(ln_1 x) + Attn(ln_1 x)),
//                           one pass over the hidden state instead of three
//   silu_mul                the SwiGLU gate of the MLP (`LlamaMLP`: down(silu(gate x) * up x)) on a
//                           strided view of a fused gate|up projection
//   wave_encode             `WaveEncoder.block` + its RMSNorm (`models/fftencoder.py:79-97`): all levels
//                           of the periodic db4 wavelet transform of one segment in shared memory,
//                           concatenated coarse-to-fine, normalised, written once in the model's dtype
//   channel_mean            the classification readout `out[:, -1].mean(dim=1)` (`models/mvpformer.py:951-953`)
//   contrastive_logits      cosine similarity of each prediction with its target and K sampled negatives
//                           (`models/mvpformer.py:574-594`) without materialising the (tokens, 1+K, E) targets
//
// Every kernel moves 16 bytes per thread per access, keeps a row in registers (one warp per row)
// or shared memory (one CTA per segment) and reduces with warp shuffles.
#include <cuda_bf16.h>

#include "mvpa_common.cuh"

namespace mvpa {
namespace {

constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
struct Vec;  // 16 bytes of T
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static void unpack(const uint4& r, float (&f)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static void store(__nv_bfloat16* p, const float (&f)[8]) { *reinterpret_cast<uint4*>(p) = pack(f); }
  __device__ static float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <>
struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&f)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
  }
  __device__ static void unpack(const uint4& r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
  __device__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  __device__ static void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __device__ static float round(float x) { return x; }
};

// y = rmsnorm(h) * w with h = x (+ a), h optionally written out.  One warp per row; the row stays in
// registers, in its storage format (NV 16-byte vectors per lane: half the registers of an fp32 copy for
// bf16, which doubles the rows in flight per multiprocessor), between the sum of squares and the scaling.
template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32) rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ a,
                                                                    const T* __restrict__ w, T* __restrict__ h_out,
                                                                    T* __restrict__ y, int64_t rows, int E, float eps) {
  constexpr int N = Vec<T>::N;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * E;
  uint4 raw[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * 32 + lane) * N;
    if (col < E) raw[i] = *reinterpret_cast<const uint4*>(xr + col);
  }
  float ss = 0.f;
  if (a != nullptr) {
    uint4 rawa[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * N;
      if (col < E) rawa[i] = *reinterpret_cast<const uint4*>(a + row * E + col);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * N;
      if (col < E) {
        float v[N], b[N];
        Vec<T>::unpack(raw[i], v);
        Vec<T>::unpack(rawa[i], b);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          v[e] = Vec<T>::round(v[e] + b[e]);  // the sum lives in T, as in eager PyTorch
          ss += v[e] * v[e];
        }
        raw[i] = Vec<T>::pack(v);
        if (h_out != nullptr) *reinterpret_cast<uint4*>(h_out + row * E + col) = raw[i];
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * N;
      if (col < E) {
        float v[N];
        Vec<T>::unpack(raw[i], v);
#pragma unroll
        for (int e = 0; e < N; ++e) ss += v[e] * v[e];
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)E + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * 32 + lane) * N;
    if (col < E) {
      float v[N], g[N];
      Vec<T>::unpack(raw[i], v);
      Vec<T>::load(w + col, g);
#pragma unroll
      for (int e = 0; e < N; ++e) g[e] = v[e] * rstd * g[e];
      Vec<T>::store(y + row * E + col, g);
    }
  }
}

// out = silu(gate) * up, elementwise, rows of `width` elements at independent leading dimensions.
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up, int64_t ld_in,
                                                       T* __restrict__ out, int64_t ld_out, int64_t rows, int width) {
  constexpr int N = Vec<T>::N;
  const int vec_per_row = width / N;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * N;
    float g[N], u[N];
    Vec<T>::load(gate + r * ld_in + c, g);
    Vec<T>::load(up + r * ld_in + c, u);
#pragma unroll
    for (int e = 0; e < N; ++e) g[e] = Vec<T>::round(g[e] / (1.f + __expf(-g[e]))) * u[e];
    Vec<T>::store(out + r * ld_out + c, g);
  }
}

constexpr int kMaxLevels = 16;
struct WaveLevels {
  int n_levels;
  int len[kMaxLevels + 1];  // len[0] = segment length, len[l+1] = coefficients of level l+1
  int out_off[kMaxLevels];  // where the detail coefficients of level l+1 start in the output row
  int total;                // sum of all detail lengths + the last approximation
};
struct WaveFilters {
  float lo[8], hi[8];  // decomposition filters (8 taps: db4)
};

// One CTA per segment: every level of the periodic wavelet transform in shared memory.
//   cA[k] = sum_m lo[m] x[(2k + 1 - m) mod n],  cD likewise with hi,  k < (n + 7) / 2
// (periodic extension of the level's own input, even or odd; n_out = floor((n + 8 - 1) / 2)).
// Output row: [cA_L, cD_L, cD_{L-1}, ..., cD_1], then RMSNorm over the whole row, times `w`.
//
// A level's input sits in shared memory with its periodic extension written out: ten samples of its end in
// front, eight of its start behind, b[10 + i] = x[i].  Output k reads x[2k-6 .. 2k+1] = b[2k+4 .. 2k+11], so
// a thread that makes outputs 2t and 2t+1 of both bands needs the ten floats b[4t+4 .. 4t+13]: two 16-byte
// loads and one 8-byte load, no index arithmetic per tap, consecutive threads on consecutive banks.  The
// approximation is written straight into the next level's padded layout.
constexpr int kWaveThreads = 128;
constexpr int kWaveFront = 10, kWaveBack = 8;
__host__ __device__ constexpr int wave_buf_floats(int n) { return (n + kWaveFront + kWaveBack + 2 + 3) & ~3; }

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(kWaveThreads) wave_encode_kernel(const Tin* __restrict__ x, int64_t ld_x,
                                                                   const WaveLevels lv, const WaveFilters flt,
                                                                   const Tout* __restrict__ w, Tout* __restrict__ out,
                                                                   int64_t ld_out, float eps) {
  extern __shared__ __align__(16) float smem[];
  float* coef = smem;                                  // [total], padded to 8
  float* buf0 = coef + ((lv.total + 7) & ~7);          // level input, extended
  float* buf1 = buf0 + wave_buf_floats(lv.len[0]);     // next level's input, extended
  __shared__ float s_red[kWaveThreads / 32];
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x;
  const Tin* xr = x + row * ld_x;
  const int n0 = lv.len[0];
  if (lv.n_levels == 0) {
    for (int i = tid; i < n0; i += kWaveThreads) coef[i] = to_f32<Tin>(xr[i]);
  } else {
    bool vec = false;
    if constexpr (sizeof(Tin) == 4) vec = (ld_x % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && (n0 % 4 == 0);
    if (vec) {
      if constexpr (sizeof(Tin) == 4) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        for (int i = tid; i < n0 / 4; i += kWaveThreads) {
          const float4 v = x4[i];
          float2* d = reinterpret_cast<float2*>(buf0 + kWaveFront + 4 * i);  // 8-byte aligned
          d[0] = make_float2(v.x, v.y);
          d[1] = make_float2(v.z, v.w);
        }
      }
    } else {
      for (int i = tid; i < n0; i += kWaveThreads) buf0[kWaveFront + i] = to_f32<Tin>(xr[i]);
    }
    if (tid < kWaveFront) buf0[tid] = to_f32<Tin>(xr[n0 - kWaveFront + tid]);
    else if (tid < kWaveFront + kWaveBack) buf0[kWaveFront + n0 + tid - kWaveFront] = to_f32<Tin>(xr[tid - kWaveFront]);
  }
  __syncthreads();
  float* src = buf0;
  float* dst = buf1;
  for (int l = 0; l < lv.n_levels; ++l) {
    const int m = lv.len[l + 1];
    const bool last = l == lv.n_levels - 1;
    float* det = coef + lv.out_off[l];
    for (int t = tid; 2 * t < m; t += kWaveThreads) {
      const float4 p0 = *reinterpret_cast<const float4*>(src + 4 * t + 4);
      const float4 p1 = *reinterpret_cast<const float4*>(src + 4 * t + 8);
      const float2 p2 = *reinterpret_cast<const float2*>(src + 4 * t + 12);
      const float v[10] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w, p2.x, p2.y};  // x[4t-6 .. 4t+3]
      float a0 = 0.f, d0 = 0.f, a1 = 0.f, d1 = 0.f;
#pragma unroll
      for (int tap = 0; tap < 8; ++tap) {
        a0 = fmaf(flt.lo[tap], v[7 - tap], a0);
        d0 = fmaf(flt.hi[tap], v[7 - tap], d0);
        a1 = fmaf(flt.lo[tap], v[9 - tap], a1);
        d1 = fmaf(flt.hi[tap], v[9 - tap], d1);
      }
      const int k0 = 2 * t, k1 = 2 * t + 1;
      const bool two = k1 < m;
      det[k0] = d0;
      if (two) det[k1] = d1;
      if (last) {
        coef[k0] = a0;
        if (two) coef[k1] = a1;
      } else {
        if (two) *reinterpret_cast<float2*>(dst + kWaveFront + k0) = make_float2(a0, a1);  // 8-byte aligned: one store
        else dst[kWaveFront + k0] = a0;
        // the next level's periodic extension: its last ten samples in front, its first eight behind
        if (k0 >= m - kWaveFront) dst[k0 - (m - kWaveFront)] = a0;
        if (two && k1 >= m - kWaveFront) dst[k1 - (m - kWaveFront)] = a1;
        if (k0 < kWaveBack) dst[kWaveFront + m + k0] = a0;
        if (two && k1 < kWaveBack) dst[kWaveFront + m + k1] = a1;
      }
    }
    __syncthreads();
    float* t = src; src = dst; dst = t;
  }
  float ss = 0.f;
  for (int i = tid; i < lv.total; i += kWaveThreads) ss += coef[i] * coef[i];
  ss = warp_sum(ss);
  if ((tid & 31) == 0) s_red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kWaveThreads / 32; ++i) tot += s_red[i];
  const float rstd = rsqrtf(tot / (float)lv.total + eps);
  Tout* orow = out + row * ld_out;
  constexpr int N = Vec<Tout>::N;
  const bool vec_out = (ld_out % N == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
  if (vec_out) {
    for (int i = tid * N; i < (int)ld_out; i += kWaveThreads * N) {
      float g[N], y[N];
      if (i + N <= lv.total) {
        Vec<Tout>::load(w + i, g);
#pragma unroll
        for (int e4 = 0; e4 < N; e4 += 4) {  // 16-byte shared-memory reads (coef is 16-byte aligned, i a multiple of 4)
          const float4 c = *reinterpret_cast<const float4*>(coef + i + e4);
          y[e4] = c.x * rstd * g[e4];
          y[e4 + 1] = c.y * rstd * g[e4 + 1];
          y[e4 + 2] = c.z * rstd * g[e4 + 2];
          y[e4 + 3] = c.w * rstd * g[e4 + 3];
        }
      } else {
#pragma unroll
        for (int e = 0; e < N; ++e) y[e] = i + e < lv.total ? coef[i + e] * rstd * to_f32<Tout>(w[i + e]) : 0.f;
      }
      Vec<Tout>::store(orow + i, y);
    }
  } else {
    for (int i = tid; i < (int)ld_out; i += kWaveThreads)
      orow[i] = i < lv.total ? from_f32<Tout>(coef[i] * rstd * to_f32<Tout>(w[i])) : from_f32<Tout>(0.f);
  }
}

// out[b, :] = mean over channels of h[b, T-1, :, :]   (h is (B, T, C, E), contiguous)
template <typename T>
__global__ void __launch_bounds__(256) channel_mean_kernel(const T* __restrict__ h, T* __restrict__ out, int Tn, int C,
                                                           int E) {
  const int b = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const T* p = h + (((int64_t)b * Tn + (Tn - 1)) * C) * E + e;
  float acc = 0.f;
  for (int c = 0; c < C; ++c) acc += to_f32<T>(p[(int64_t)c * E]);
  out[(int64_t)b * E + e] = from_f32<T>(acc / (float)C);
}

// Contrastive logits.  pred, enc: (B, T, C, E).  For every target position (b, t >= 1, c):
//   row n = (b (T-1) + (t-1)) C + c,  p = pred[b, t-1, c],  candidate 0 = enc[b, t, c],
//   candidate j = enc_flat[neg[b, t, c, j-1]];  logits[n, j] = cos(p, candidate j) / temp,
//   -inf for a negative that equals the positive (|neg - pos| < 1e-8 + 1e-5 |pos|).
// One warp per target position; p and the positive stay in registers while the negatives stream by.
template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 2) contrastive_kernel(const T* __restrict__ pred, const T* __restrict__ enc,
                                                                        const int* __restrict__ neg, float* __restrict__ logits,
                                                                        int B, int Tn, int C, int E, int K, float inv_temp) {
  constexpr int N = Vec<T>::N;
  const int64_t n = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)B * (Tn - 1) * C;
  if (n >= rows) return;
  const int c = (int)(n % C);
  const int t = (int)((n / C) % (Tn - 1)) + 1;
  const int b = (int)(n / ((int64_t)C * (Tn - 1)));
  const int64_t tok_pos = ((int64_t)b * Tn + t) * C + c, tok_pred = tok_pos - C;
  // p, the positive and the candidate rows stay in their storage format; the next candidate's row is
  // requested before the current one is reduced, so its latency hides behind the arithmetic.
  uint4 pr[NV], qr[NV], cur[NV], nxt[NV];
  float pp = 0.f, qq = 0.f, pq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * 32 + lane) * N;
    if (col < E) {
      pr[i] = *reinterpret_cast<const uint4*>(pred + tok_pred * E + col);
      qr[i] = *reinterpret_cast<const uint4*>(enc + tok_pos * E + col);
      float p[N], q[N];
      Vec<T>::unpack(pr[i], p);
      Vec<T>::unpack(qr[i], q);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        pp += p[e] * p[e];
        qq += q[e] * q[e];
        pq += p[e] * q[e];
      }
    }
  }
  auto fetch = [&](uint4 (&dst)[NV], int j) {
    const int64_t src = neg[tok_pos * K + j];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * N;
      if (col < E) dst[i] = *reinterpret_cast<const uint4*>(enc + src * E + col);
    }
  };
  if (K > 0) fetch(cur, 0);
  pp = warp_sum(pp); qq = warp_sum(qq); pq = warp_sum(pq);
  const float np_ = fmaxf(sqrtf(pp), 1e-8f), nq = sqrtf(qq);
  float* lrow = logits + n * (K + 1);
  if (lane == 0) lrow[0] = pq / (np_ * fmaxf(nq, 1e-8f)) * inv_temp;
  for (int j = 0; j < K; ++j) {
    if (j + 1 < K) fetch(nxt, j + 1);
    float rr = 0.f, prd = 0.f, dd = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * N;
      if (col < E) {
        float r[N], p[N], q[N];
        Vec<T>::unpack(cur[i], r);
        Vec<T>::unpack(pr[i], p);
        Vec<T>::unpack(qr[i], q);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          rr += r[e] * r[e];
          prd += p[e] * r[e];
          const float df = Vec<T>::round(r[e] - q[e]);
          dd += df * df;
        }
      }
    }
    rr = warp_sum(rr); prd = warp_sum(prd); dd = warp_sum(dd);
    if (lane == 0) {
      const bool same = sqrtf(dd) < 1e-8f + 1e-5f * nq;
      lrow[j + 1] = same ? -INFINITY : prd / (np_ * fmaxf(sqrtf(rr), 1e-8f)) * inv_temp;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) cur[i] = nxt[i];
  }
}

template <typename T>
int launch_rmsnorm(const void* x, const void* a, const void* w, void* h_out, void* y, int64_t rows, int E, float eps,
                   cudaStream_t s) {
  constexpr int N = Vec<T>::N;
  const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
  const int nv = (E / N + 31) / 32;
#define MVPA_RMS(NV)                                                                                             \
  rmsnorm_kernel<T, NV><<<grid, kWarpsPerCta * 32, 0, s>>>((const T*)x, (const T*)a, (const T*)w, (T*)h_out, (T*)y, \
                                                            rows, E, eps)
  if (nv <= 2) MVPA_RMS(2);
  else if (nv <= 4) MVPA_RMS(4);
  else if (nv <= 8) MVPA_RMS(8);
  else MVPA_RMS(16);
#undef MVPA_RMS
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

int check_rows(const char* what, int64_t rows, int width, int dtype, int max_vectors) {
  if (dtype != MVPA_F32 && dtype != MVPA_BF16) {
    set_error("%s: element type must be MVPA_F32 or MVPA_BF16", what);
    return MVPA_ERR_DTYPE;
  }
  const int n = dtype == MVPA_F32 ? 4 : 8;
  if (rows <= 0 || width <= 0 || width % n != 0 || (max_vectors > 0 && width / n > 32 * max_vectors)) {
    set_error("%s: %lld rows of %d elements: the width must be a positive multiple of %d%s", what, (long long)rows, width,
              n, max_vectors > 0 ? " and at most 512 sixteen-byte vectors" : "");
    return MVPA_ERR_SHAPE;
  }
  if (rows > (int64_t)1 << 31) {
    set_error("%s: too many rows (%lld)", what, (long long)rows);
    return MVPA_ERR_SHAPE;
  }
  return MVPA_OK;
}

bool aligned16(const void* p) { return p != nullptr && ((uintptr_t)p & 15) == 0; }

}  // namespace
}  // namespace mvpa

using namespace mvpa;

extern "C" {

int mvpa_rmsnorm(const void* x, const void* add, const void* weight, void* sum_out, void* y, int64_t rows,
                 int32_t width, float eps, int32_t dtype, void* cuda_stream) {
  int rc = check_rows("mvpa_rmsnorm", rows, width, dtype, 16);
  if (rc) return rc;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || (add != nullptr && !aligned16(add)) ||
      (sum_out != nullptr && !aligned16(sum_out))) {
    set_error("mvpa_rmsnorm: x, weight, y (and add, sum_out when given) must be 16-byte aligned and not NULL");
    return MVPA_ERR_ALIGNMENT;
  }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  return dtype == MVPA_F32 ? launch_rmsnorm<float>(x, add, weight, sum_out, y, rows, width, eps, s)
                           : launch_rmsnorm<__nv_bfloat16>(x, add, weight, sum_out, y, rows, width, eps, s);
}

int mvpa_silu_mul(const void* gate, const void* up, int64_t ld_in, void* out, int64_t ld_out, int64_t rows,
                  int32_t width, int32_t dtype, void* cuda_stream) {
  int rc = check_rows("mvpa_silu_mul", rows, width, dtype, 0);
  if (rc) return rc;
  const int n = dtype == MVPA_F32 ? 4 : 8;
  if (!aligned16(gate) || !aligned16(up) || !aligned16(out) || ld_in % n != 0 || ld_out % n != 0 || ld_in < width ||
      ld_out < width) {
    set_error("mvpa_silu_mul: pointers must be 16-byte aligned, leading dimensions multiples of %d and >= the width", n);
    return MVPA_ERR_ALIGNMENT;
  }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const int64_t total = rows * (width / n);
  const unsigned grid = (unsigned)((total + 255) / 256 < (int64_t)device_sm_count() * 16 ? (total + 255) / 256
                                                                                         : (int64_t)device_sm_count() * 16);
  if (dtype == MVPA_F32)
    silu_mul_kernel<float><<<grid, 256, 0, s>>>((const float*)gate, (const float*)up, ld_in, (float*)out, ld_out, rows, width);
  else
    silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, ld_in,
                                                       (__nv_bfloat16*)out, ld_out, rows, width);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

int32_t mvpa_wave_encode_size(int32_t segment_len, int32_t* level_sizes, int32_t max_levels) {
  // db4: 8 taps.  Levels while the input is at least as long as the filter support allows
  // (floor(log2(len / 7))), each producing floor((n + 7) / 2) coefficients.
  if (segment_len < 8) return 0;
  int levels = 0;
  for (int v = segment_len / 7; v > 1; v >>= 1) ++levels;
  if (levels > kMaxLevels) levels = kMaxLevels;
  int n = segment_len, total = 0;
  for (int l = 0; l < levels; ++l) {
    n = (n + 7) / 2;
    if (level_sizes != nullptr && l < max_levels) level_sizes[l] = n;
    total += n;
  }
  return total + n;  // + the last approximation
}

int mvpa_wave_encode(const void* x, int64_t ld_x, int32_t x_dtype, const float* dec_lo, const float* dec_hi,
                     const void* weight, void* out, int64_t ld_out, int32_t out_dtype, int64_t rows,
                     int32_t segment_len, float eps, void* cuda_stream) {
  const int total = mvpa_wave_encode_size(segment_len, nullptr, 0);
  if (total == 0 || rows <= 0 || rows > (int64_t)1 << 31 || segment_len > 16384) {
    set_error("mvpa_wave_encode: %lld segments of %d samples (8 .. 16384 samples per segment)", (long long)rows, segment_len);
    return MVPA_ERR_SHAPE;
  }
  if ((x_dtype != MVPA_F32 && x_dtype != MVPA_BF16) || (out_dtype != MVPA_F32 && out_dtype != MVPA_BF16)) {
    set_error("mvpa_wave_encode: element types must be MVPA_F32 or MVPA_BF16");
    return MVPA_ERR_DTYPE;
  }
  if (x == nullptr || out == nullptr || weight == nullptr || dec_lo == nullptr || dec_hi == nullptr || ld_x < segment_len ||
      ld_out < total) {
    set_error("mvpa_wave_encode: NULL pointer, or a leading dimension shorter than its row (%d in, %d out)", segment_len, total);
    return MVPA_ERR_SHAPE;
  }
  WaveLevels lv;
  WaveFilters flt;
  for (int i = 0; i < 8; ++i) { flt.lo[i] = dec_lo[i]; flt.hi[i] = dec_hi[i]; }  // host pointers: eight taps each
  lv.n_levels = 0;
  for (int v = segment_len / 7; v > 1; v >>= 1) ++lv.n_levels;
  if (lv.n_levels > kMaxLevels) lv.n_levels = kMaxLevels;
  lv.len[0] = segment_len;
  for (int l = 0; l < lv.n_levels; ++l) lv.len[l + 1] = (lv.len[l] + 7) / 2;
  lv.total = total;
  int off = total;
  for (int l = 0; l < lv.n_levels; ++l) {  // finest details last
    off -= lv.len[l + 1];
    lv.out_off[l] = off;
  }
  const size_t smem = sizeof(float) * (((total + 7) & ~7) + wave_buf_floats(lv.len[0]) +
                                       wave_buf_floats(lv.n_levels > 0 ? lv.len[1] : 0));
  cudaStream_t s = (cudaStream_t)cuda_stream;
#define MVPA_WAVE(TI, TO)                                                                                         \
  do {                                                                                                            \
    MVPA_CUDA_CHECK(cudaFuncSetAttribute(wave_encode_kernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem));                                                             \
    wave_encode_kernel<TI, TO><<<(unsigned)rows, kWaveThreads, smem, s>>>((const TI*)x, ld_x, lv, flt, (const TO*)weight, \
                                                                 (TO*)out, ld_out, eps);                          \
  } while (0)
  if (x_dtype == MVPA_F32 && out_dtype == MVPA_F32) MVPA_WAVE(float, float);
  else if (x_dtype == MVPA_F32) MVPA_WAVE(float, __nv_bfloat16);
  else if (out_dtype == MVPA_F32) MVPA_WAVE(__nv_bfloat16, float);
  else MVPA_WAVE(__nv_bfloat16, __nv_bfloat16);
#undef MVPA_WAVE
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

// ---- gather of row pieces from peers' memory (plain loads over NVLink) ----
struct GatherPieces {
  const uint4* src[MVPA_MAX_GATHER_PIECES];
  uint4* dst[MVPA_MAX_GATHER_PIECES];
  int64_t n16[MVPA_MAX_GATHER_PIECES];  // 16-byte words per piece
  int n;
};
// The pieces are cut into 64 KB chunks and the chunks dealt round-robin over the pieces, so at any time
// the CTAs read from every source at once: each source GPU then serves its readers at an even share of its
// link bandwidth (all ranks walking the pieces in the same order would all pull from one source at a time).
// Four independent 16-byte loads per thread and turn keep enough bytes in flight for the link latency.
constexpr int kGatherChunk16 = 4096;  // 16-byte words per chunk
static __global__ void __launch_bounds__(512) peer_gather_kernel(const __grid_constant__ GatherPieces g, int64_t max_chunks) {
  const int64_t n_slots = max_chunks * g.n;  // chunk c of piece p is slot c * n + p
  for (int64_t slot = blockIdx.x; slot < n_slots; slot += gridDim.x) {
    const int pc = (int)(slot % g.n);
    const int64_t base = (slot / g.n) * kGatherChunk16;
    const int64_t n = g.n16[pc] - base < kGatherChunk16 ? g.n16[pc] - base : kGatherChunk16;
    if (n <= 0) continue;
    const uint4* __restrict__ src = g.src[pc] + base;
    uint4* __restrict__ dst = g.dst[pc] + base;
    int i = threadIdx.x;
    for (; i + 3 * 512 < n; i += 4 * 512) {
      const uint4 a = __ldcg(src + i), b = __ldcg(src + i + 512), c = __ldcg(src + i + 1024), d = __ldcg(src + i + 1536);
      dst[i] = a;
      dst[i + 512] = b;
      dst[i + 1024] = c;
      dst[i + 1536] = d;
    }
    for (; i < n; i += 512) dst[i] = __ldcg(src + i);
  }
}

int mvpa_peer_gather(void* const* dst, const void* const* src, const int64_t* bytes, int32_t n_pieces,
                     void* cuda_stream) {
  if (n_pieces < 0 || n_pieces > MVPA_MAX_GATHER_PIECES || (n_pieces > 0 && (!dst || !src || !bytes))) {
    set_error("mvpa_peer_gather: between 0 and %d pieces, arrays not NULL", MVPA_MAX_GATHER_PIECES);
    return MVPA_ERR_SHAPE;
  }
  GatherPieces g;
  g.n = 0;
  for (int i = 0; i < n_pieces; ++i) {
    if (bytes[i] == 0) continue;
    if (bytes[i] < 0 || bytes[i] % 16 != 0 || ((uintptr_t)dst[i] & 15) != 0 || ((uintptr_t)src[i] & 15) != 0 ||
        !dst[i] || !src[i]) {
      set_error("mvpa_peer_gather: piece %d: pointers and size must be non-NULL multiples of 16 bytes", i);
      return MVPA_ERR_ALIGNMENT;
    }
    g.src[g.n] = (const uint4*)src[i];
    g.dst[g.n] = (uint4*)dst[i];
    g.n16[g.n] = bytes[i] / 16;
    ++g.n;
  }
  if (g.n == 0) return MVPA_OK;
  int64_t max_chunks = 0;
  for (int i = 0; i < g.n; ++i) {
    const int64_t c = (g.n16[i] + kGatherChunk16 - 1) / kGatherChunk16;
    max_chunks = c > max_chunks ? c : max_chunks;
  }
  // whole waves of CTAs (two per SM), fewer for small transfers
  const int64_t want = max_chunks * g.n, cap = 2 * (int64_t)device_sm_count();
  const unsigned grid = (unsigned)(want > cap ? cap : want);
  peer_gather_kernel<<<grid, 512, 0, (cudaStream_t)cuda_stream>>>(g, max_chunks);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

// ---- flags between GPUs ----
struct FlagSlots {
  uint32_t* slot[MVPA_MAX_GATHER_PIECES];
  int n;
};
static __global__ void peer_signal_kernel(const __grid_constant__ FlagSlots f, uint32_t value, const uint32_t* base) {
  const int i = threadIdx.x;
  if (base != nullptr) value += *base;
  if (i < f.n) {
    __threadfence_system();  // what this stream wrote before is visible before the flag is
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.slot[i]), "r"(value) : "memory");
  }
}
static __global__ void peer_wait_kernel(const __grid_constant__ FlagSlots f, uint32_t value, const uint32_t* base,
                                        uint64_t limit_ns, int* status) {
  const int i = threadIdx.x;
  if (base != nullptr) value += *base;
  if (i < f.n) {
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f.slot[i]) : "memory");
      if ((int32_t)(v - value) >= 0) break;
      uint64_t t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > limit_ns) {  // give up: report and return, the context stays usable
        if (status != nullptr) *status = 1;
        break;
      }
      __nanosleep(200);
    }
  }
  __threadfence_system();
}

static int flag_slots(FlagSlots& f, const void* const* slots, int32_t n, const char* what) {
  if (n < 0 || n > MVPA_MAX_GATHER_PIECES || (n > 0 && !slots)) {
    set_error("%s: between 0 and %d slots, array not NULL", what, MVPA_MAX_GATHER_PIECES);
    return MVPA_ERR_SHAPE;
  }
  f.n = n;
  for (int i = 0; i < n; ++i) {
    if (!slots[i] || ((uintptr_t)slots[i] & 3) != 0) {
      set_error("%s: slot %d is NULL or not 4-byte aligned", what, i);
      return MVPA_ERR_ALIGNMENT;
    }
    f.slot[i] = (uint32_t*)slots[i];
  }
  return MVPA_OK;
}

int mvpa_peer_signal(uint32_t* const* remote_slots, int32_t n, uint32_t value, const uint32_t* base,
                     void* cuda_stream) {
  FlagSlots f;
  const int rc = flag_slots(f, (const void* const*)remote_slots, n, "mvpa_peer_signal");
  if (rc != MVPA_OK || n == 0) return rc;
  peer_signal_kernel<<<1, MVPA_MAX_GATHER_PIECES, 0, (cudaStream_t)cuda_stream>>>(f, value, base);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

int mvpa_peer_wait(const uint32_t* const* local_slots, int32_t n, uint32_t value, const uint32_t* base,
                   uint32_t limit_us, int32_t* status, void* cuda_stream) {
  FlagSlots f;
  const int rc = flag_slots(f, (const void* const*)local_slots, n, "mvpa_peer_wait");
  if (rc != MVPA_OK || n == 0) return rc;
  const uint64_t limit_ns = limit_us != 0 ? (uint64_t)limit_us * 1000ull : 2000000000ull;
  peer_wait_kernel<<<1, MVPA_MAX_GATHER_PIECES, 0, (cudaStream_t)cuda_stream>>>(f, value, base, limit_ns, status);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

int mvpa_channel_mean(const void* h, void* out, int32_t B, int32_t T, int32_t C, int32_t E, int32_t dtype,
                      void* cuda_stream) {
  if (B <= 0 || T <= 0 || C <= 0 || E <= 0 || h == nullptr || out == nullptr) {
    set_error("mvpa_channel_mean: sizes must be positive and pointers not NULL");
    return MVPA_ERR_SHAPE;
  }
  if (dtype != MVPA_F32 && dtype != MVPA_BF16) {
    set_error("mvpa_channel_mean: element type must be MVPA_F32 or MVPA_BF16");
    return MVPA_ERR_DTYPE;
  }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const dim3 grid((E + 255) / 256, B);
  if (dtype == MVPA_F32) channel_mean_kernel<float><<<grid, 256, 0, s>>>((const float*)h, (float*)out, T, C, E);
  else channel_mean_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)h, (__nv_bfloat16*)out, T, C, E);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

int mvpa_contrastive_logits(const void* pred, const void* enc, const int32_t* negatives, float* logits, int32_t B,
                            int32_t T, int32_t C, int32_t E, int32_t K, float temperature, int32_t dtype,
                            void* cuda_stream) {
  if (B <= 0 || T < 2 || C <= 0 || K < 0 || temperature <= 0.f) {
    set_error("mvpa_contrastive_logits: B, C > 0, T >= 2, K >= 0 and a positive temperature are required");
    return MVPA_ERR_SHAPE;
  }
  int rc = check_rows("mvpa_contrastive_logits", (int64_t)B * (T - 1) * C, E, dtype, 8);
  if (rc) return rc;
  if (!aligned16(pred) || !aligned16(enc) || logits == nullptr || (K > 0 && negatives == nullptr)) {
    set_error("mvpa_contrastive_logits: pred and enc must be 16-byte aligned; logits (and negatives when K > 0) not NULL");
    return MVPA_ERR_ALIGNMENT;
  }
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const int64_t rows = (int64_t)B * (T - 1) * C;
  const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
  const int n = dtype == MVPA_F32 ? 4 : 8;
  const int nv = (E / n + 31) / 32;
#define MVPA_CL(TT, NV)                                                                                          \
  contrastive_kernel<TT, NV><<<grid, kWarpsPerCta * 32, 0, s>>>((const TT*)pred, (const TT*)enc, negatives, logits, B, T, \
                                                                C, E, K, 1.f / temperature)
  if (dtype == MVPA_F32) {
    if (nv <= 2) MVPA_CL(float, 2); else if (nv <= 4) MVPA_CL(float, 4); else MVPA_CL(float, 8);
  } else {
    if (nv <= 2) MVPA_CL(__nv_bfloat16, 2); else if (nv <= 4) MVPA_CL(__nv_bfloat16, 4); else MVPA_CL(__nv_bfloat16, 8);
  }
#undef MVPA_CL
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

}  // extern "C"
