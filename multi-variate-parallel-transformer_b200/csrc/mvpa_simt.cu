// fp32 CUDA-core kernels of Flash-MVPA: forward and the full backward.
//
// These serve element type fp32 (where tensor-core input rounding would break the
// 1e-4 relative tolerance) and every shape the tcgen05 kernels do not take.  They
// are tiled through shared memory (32 query rows x 64 keys per step, 256 threads)
// and deterministic: no floating-point atomics anywhere, cross-tile sums go through
// per-tile partials.
//
// Math follows the reference forward (`attentions/attn.py:232-333`: base-2 online
// softmax, window zero-fill, time-block causal mask, L = m + log2 l) and backward
// (`attentions/attn.py:561-751` plus autograd through `_rel_bias`, `:1305-1314`).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "mvpa_common.cuh"

namespace mvpa {
namespace {

constexpr int kThreads = 256;
constexpr int kBM = 32;   // rows of the register-tiled products
constexpr int kBN = 64;   // columns
constexpr int kPLd = kBN + 1;
constexpr int kDrelSplit = 32;  // split-K factor of the relative-key gradient reduction

// ---- tile helpers (256 threads: ty = tid/16 owns rows 2ty,2ty+1; tx = tid%16) ----

// acc[a][j] += sum_d A[2ty+a][d] * B[tx+16j][d]       (A: 32 x D, B: 64 x D, ld = D+4)
template <int D>
__device__ __forceinline__ void tile_nt(const float* __restrict__ As, const float* __restrict__ Bs,
                                        float (&acc)[2][4]) {
  constexpr int LD = D + 4;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const float4* a0 = reinterpret_cast<const float4*>(As + (2 * ty) * LD);
  const float4* a1 = reinterpret_cast<const float4*>(As + (2 * ty + 1) * LD);
#pragma unroll 4
  for (int d4 = 0; d4 < D / 4; ++d4) {
    const float4 x0 = a0[d4], x1 = a1[d4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 y = reinterpret_cast<const float4*>(Bs + (tx + 16 * j) * LD)[d4];
      acc[0][j] += x0.x * y.x + x0.y * y.y + x0.z * y.z + x0.w * y.w;
      acc[1][j] += x1.x * y.x + x1.y * y.y + x1.z * y.z + x1.w * y.w;
    }
  }
}

// out[a][e] += sum_c P[2ty+a][c] * B[c][tx+16e]        (P: 32 x 64, ld 65; B: 64 x D)
template <int D>
__device__ __forceinline__ void tile_nn(const float* __restrict__ Ps, const float* __restrict__ Bs,
                                        float (&out)[2][D / 16]) {
  constexpr int LD = D + 4;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const float* p0 = Ps + (2 * ty) * kPLd;
  const float* p1 = p0 + kPLd;
#pragma unroll 4
  for (int c = 0; c < kBN; ++c) {
    const float x0 = p0[c], x1 = p1[c];
#pragma unroll
    for (int e = 0; e < D / 16; ++e) {
      const float y = Bs[c * LD + tx + 16 * e];
      out[0][e] += x0 * y;
      out[1][e] += x1 * y;
    }
  }
}

// Copy `rows` rows of D elements from global (row stride `sn`, first row `row0`, rows >= n_rows
// read as zero) to shared (ld = D+4), as (x + bias[d]) * scale in fp32.
template <typename Tin, int D>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, const Tin* __restrict__ src,
                                          int64_t sn, int row0, int n_rows, int rows,
                                          const Tin* __restrict__ bias, float scale) {
  constexpr int LD = D + 4;
  for (int idx = threadIdx.x; idx < rows * D; idx += kThreads) {
    const int r = idx / D, d = idx % D;
    const int row = row0 + r;
    float x = 0.f;
    if (row < n_rows) {
      x = to_f32<Tin>(src[(int64_t)row * sn + d]);
      if (bias != nullptr) x += to_f32<Tin>(bias[d]);
      x *= scale;
    }
    dst[r * LD + d] = x;
  }
}

// Relative scores of `rows` query rows held raw in shared memory (ld = D+4):
//   out_t[r*ldt + s] = c2 * (q_r + vt) . r_time[s],  out_c[r*ldc + e] = c2 * (q_r + z) . r_chan[e]
// (`attentions/attn.py:1305-1314`, scaled like `:292,307`).  out_* may be shared or global.
template <typename Tin, int D>
__device__ __forceinline__ void rel_scores(const float* __restrict__ Qraw, int rows,
                                           const Tin* __restrict__ vt, const Tin* __restrict__ z,
                                           const Tin* __restrict__ rt, const Tin* __restrict__ rc,
                                           int T, int C, float c2, float* out_t, int64_t ldt,
                                           float* out_c, int64_t ldc, int valid_rows) {
  constexpr int LD = D + 4;
  const int total = rows * (T + C);
  for (int idx = threadIdx.x; idx < total; idx += kThreads) {
    const int r = idx % rows, s = idx / rows;
    if (r >= valid_rows) continue;
    const bool is_t = s < T;
    const Tin* key = is_t ? rt + (int64_t)s * D : rc + (int64_t)(s - T) * D;
    const Tin* bias = is_t ? vt : z;
    float acc = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; ++d)
      acc += (Qraw[r * LD + d] + to_f32<Tin>(bias[d])) * to_f32<Tin>(key[d]);
    acc *= c2;
    if (is_t) out_t[(int64_t)r * ldt + s] = acc;
    else out_c[(int64_t)r * ldc + (s - T)] = acc;
  }
}

__device__ __forceinline__ bool in_window(int ti, int tk, int T, int window) {
  const int dt = ti - tk;
  return window <= 0 || (dt <= window && dt >= -window) || ti == T - 1;
}

// ------------------------------- forward -------------------------------------

template <typename Tin, int D>
__global__ void __launch_bounds__(kThreads) simt_fwd_kernel(Args p) {
  constexpr int LD = D + 4;
  constexpr int DV = D / 16;
  extern __shared__ float smem[];
  float* Qs = smem;
  float* Ks = Qs + kBM * LD;
  float* Vs = Ks + kBN * LD;
  float* Ps = Vs + kBN * LD;
  float* TBs = Ps + kBM * kPLd;
  float* CBs = TBs + kBM * p.T;
  float* ms = CBs + kBM * p.C;
  float* ls = ms + kBM;
  float* alphas = ls + kBM;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heaviest (latest) query tiles first
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H, hk = h / p.g;
  const int m0 = qt * kBM;               // first row of the tile inside this call's q / o / lse
  const int N = p.N, T = p.T, C = p.C;
  const int Nq = p.q_tn * C;             // rows of this call (a query time range, or all of N)
  const int row0 = p.q_t0 * C;           // token index of row 0
  const Tin* q = (const Tin*)p.q + b * p.q_sb + h * p.q_sh;
  const Tin* k = (const Tin*)p.k + b * p.k_sb + hk * p.k_sh;
  const Tin* v = (const Tin*)p.v + b * p.v_sb + hk * p.v_sh;
  const int valid = min(kBM, Nq - m0);

  load_tile<Tin, D>(Qs, q, p.q_sn, m0, Nq, kBM, nullptr, 1.f);
  if (tid < kBM) { ms[tid] = -INFINITY; ls[tid] = 0.f; }
  __syncthreads();
  rel_scores<Tin, D>(Qs, kBM, (const Tin*)p.vt + hk * D, (const Tin*)p.z + hk * D,
                     (const Tin*)p.rt + (int64_t)hk * T * D, (const Tin*)p.rc + (int64_t)hk * C * D,
                     T, C, p.c2, TBs, T, CBs, C, valid);
  __syncthreads();
  {  // Qs <- (q + u) * c2   (`attentions/attn.py:180-183`)
    const Tin* u = (const Tin*)p.u + hk * D;
    for (int idx = tid; idx < kBM * D; idx += kThreads) {
      const int r = idx / D, d = idx % D;
      Qs[r * LD + d] = (Qs[r * LD + d] + to_f32<Tin>(u[d])) * p.c2;
    }
  }
  int ti[2], ci[2];
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int i = row0 + min(m0 + 2 * ty + a, Nq - 1);  // token index in the whole sequence
    ti[a] = i / C;
    ci[a] = i % C;
  }
  float oacc[2][DV];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int e = 0; e < DV; ++e) oacc[a][e] = 0.f;

  const int t_last = (row0 + m0 + valid - 1) / C;
  const int hi = min(N, (t_last + 1) * C);  // causal bound (`attentions/attn.py:102-104,125-127`)
  for (int n0 = 0; n0 < hi; n0 += kBN) {
    __syncthreads();
    load_tile<Tin, D>(Ks, k, p.k_sn, n0, N, kBN, nullptr, 1.f);
    load_tile<Tin, D>(Vs, v, p.v_sn, n0, N, kBN, nullptr, 1.f);
    __syncthreads();
    float acc[2][4] = {};
    tile_nt<D>(Qs, Ks, acc);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = tx + 16 * j, kk = n0 + col;
      const int tk = kk / C, ck = kk % C;
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const int r = 2 * ty + a;
        float s = -INFINITY;
        if (kk < N && r < valid && tk <= ti[a]) {
          s = in_window(ti[a], tk, T, p.window) ? acc[a][j] : 0.f;
          s += TBs[r * T + (T - 1 - (ti[a] - tk))] + CBs[r * C + (C - 1 - abs(ci[a] - ck))];
        }
        Ps[r * kPLd + col] = s;
      }
    }
    __syncthreads();
    {  // online softmax, one warp per 4 rows (`attentions/attn.py:309-315`)
      const int w = tid >> 5, lane = tid & 31;
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        const int r = 4 * w + rr;
        const float s0 = Ps[r * kPLd + lane], s1 = Ps[r * kPLd + lane + 32];
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_old = ms[r];
        const float m_new = fmaxf(m_old, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_old - m_use);
        const float p0 = exp2f(s0 - m_use), p1 = exp2f(s1 - m_use);
        float sum = p0 + p1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        Ps[r * kPLd + lane] = p0;
        Ps[r * kPLd + lane + 32] = p1;
        if (lane == 0) {
          ls[r] = ls[r] * alpha + sum;
          ms[r] = m_new;
          alphas[r] = alpha;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const float al = alphas[2 * ty + a];
#pragma unroll
      for (int e = 0; e < DV; ++e) oacc[a][e] *= al;
    }
    tile_nn<D>(Ps, Vs, oacc);
  }
  __syncthreads();
  Tin* o = (Tin*)p.o + b * p.o_sb + h * p.o_sh;
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int r = 2 * ty + a, i = m0 + r;
    if (r < valid) {
      const float inv = 1.f / ls[r];
#pragma unroll
      for (int e = 0; e < DV; ++e) o[(int64_t)i * p.o_sn + tx + 16 * e] = from_f32<Tin>(oacc[a][e] * inv);
      if (tx == 0 && p.lse != nullptr) p.lse[(int64_t)bh * Nq + i] = ms[r] + log2f(ls[r]);
    }
  }
}

// ------------------------------- backward ------------------------------------

// Relative scores of every query row to the workspace (the SIMT backward gathers from them).
template <typename Tin, int D>
__global__ void __launch_bounds__(kThreads) simt_rel_kernel(BwdArgs bw) {
  constexpr int LD = D + 4;
  const Args& p = bw.a;
  extern __shared__ float smem[];
  float* Qs = smem;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H, hk = h / p.g;
  const int m0 = blockIdx.x * kBM, valid = min(kBM, p.N - m0);
  const Tin* q = (const Tin*)p.q + b * p.q_sb + h * p.q_sh;
  load_tile<Tin, D>(Qs, q, p.q_sn, m0, p.N, kBM, nullptr, 1.f);
  __syncthreads();
  rel_scores<Tin, D>(Qs, kBM, (const Tin*)p.vt + hk * D, (const Tin*)p.z + hk * D,
                     (const Tin*)p.rt + (int64_t)hk * p.T * D, (const Tin*)p.rc + (int64_t)hk * p.C * D,
                     p.T, p.C, p.c2, bw.tbg + ((int64_t)bh * p.N + m0) * p.T, p.T,
                     bw.cbg + ((int64_t)bh * p.N + m0) * p.C, p.C, valid);
}

// delta[bh][i] = sum_d dO[i][d] * O[i][d]   (`attentions/attn.py:1213`).  HBM-bound: a thread reads 16
// bytes of each tensor at a time, D / VEC threads share a row (VEC = elements per 16 bytes) and
// combine with shuffles; D is a power of two >= 16, so a row never straddles warps.
template <typename Tin, int D>
__global__ void __launch_bounds__(kThreads) simt_delta_kernel(BwdArgs bw) {
  constexpr int VEC = 16 / sizeof(Tin), TPR = D / VEC;  // threads per row: 4 .. 32
  const Args& p = bw.a;
  const int gid = blockIdx.x * kThreads + threadIdx.x;
  const int rowi = gid / TPR, part = gid % TPR;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  float acc = 0.f;
  if (rowi < p.N) {
    const Tin* o = (const Tin*)p.o + b * p.o_sb + h * p.o_sh + (int64_t)rowi * p.o_sn + part * VEC;
    const Tin* g = (const Tin*)bw.d_o + b * bw.do_sb + h * bw.do_sh + (int64_t)rowi * bw.do_sn + part * VEC;
    const uint4 ov = *reinterpret_cast<const uint4*>(o), gv = *reinterpret_cast<const uint4*>(g);
    const Tin* oe = reinterpret_cast<const Tin*>(&ov);
    const Tin* ge = reinterpret_cast<const Tin*>(&gv);
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc += to_f32<Tin>(oe[e]) * to_f32<Tin>(ge[e]);
  }
#pragma unroll
  for (int s = TPR / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (part == 0 && rowi < p.N) bw.delta[(int64_t)bh * p.N + rowi] = acc;
}

// dQ side: one CTA per (32 query rows, b, h).  Walks the causal key tiles, recomputes
// P = exp2(S2 - L), forms dS, accumulates the content part of dQ and the per-row sums of dS by
// time slot / channel slot, then finishes dq = dS_w K + dTB r_time + dCB r_chan.
template <typename Tin, int D>
__global__ void __launch_bounds__(kThreads) simt_dq_kernel(BwdArgs bw) {
  constexpr int LD = D + 4;
  constexpr int DV = D / 16;
  const Args& p = bw.a;
  extern __shared__ float smem[];
  float* Qs = smem;                 // (q+u)*c2
  float* Gs = Qs + kBM * LD;        // dO rows
  float* Ks = Gs + kBM * LD;
  float* Vs = Ks + kBN * LD;
  float* Ds = Vs + kBN * LD;        // dS
  float* Dw = Ds + kBM * kPLd;      // dS * win
  float* dTBs = Dw + kBM * kPLd;    // 32 x T
  float* dCBs = dTBs + kBM * p.T;   // 32 x C
  float* lse_s = dCBs + kBM * p.C;
  float* dl_s = lse_s + kBM;
  float* red = dl_s + kBM;          // 16 x D column-sum scratch

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H, hk = h / p.g;
  const int m0 = qt * kBM;
  const int N = p.N, T = p.T, C = p.C;
  const int valid = min(kBM, N - m0);
  const Tin* q = (const Tin*)p.q + b * p.q_sb + h * p.q_sh;
  const Tin* k = (const Tin*)p.k + b * p.k_sb + hk * p.k_sh;
  const Tin* v = (const Tin*)p.v + b * p.v_sb + hk * p.v_sh;
  const Tin* g = (const Tin*)bw.d_o + b * bw.do_sb + h * bw.do_sh;
  const float* tbg = bw.tbg + (int64_t)bh * N * T;
  const float* cbg = bw.cbg + (int64_t)bh * N * C;

  load_tile<Tin, D>(Qs, q, p.q_sn, m0, N, kBM, (const Tin*)p.u + hk * D, p.c2);
  load_tile<Tin, D>(Gs, g, bw.do_sn, m0, N, kBM, nullptr, 1.f);
  for (int idx = tid; idx < kBM * (T + C); idx += kThreads) dTBs[idx] = 0.f;  // dTBs,dCBs adjacent
  if (tid < kBM) {
    const int i = min(m0 + tid, N - 1);
    lse_s[tid] = p.lse[(int64_t)bh * N + i];
    dl_s[tid] = bw.delta[(int64_t)bh * N + i];
  }
  int ti[2], ci[2];
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int i = min(m0 + 2 * ty + a, N - 1);
    ti[a] = i / C;
    ci[a] = i % C;
  }
  float qacc[2][DV];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int e = 0; e < DV; ++e) qacc[a][e] = 0.f;

  const int t_last = (m0 + valid - 1) / C;
  const int hi = min(N, (t_last + 1) * C);
  for (int n0 = 0; n0 < hi; n0 += kBN) {
    __syncthreads();
    load_tile<Tin, D>(Ks, k, p.k_sn, n0, N, kBN, nullptr, 1.f);
    load_tile<Tin, D>(Vs, v, p.v_sn, n0, N, kBN, nullptr, 1.f);
    __syncthreads();
    float sacc[2][4] = {}, pacc[2][4] = {};
    tile_nt<D>(Qs, Ks, sacc);
    tile_nt<D>(Gs, Vs, pacc);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = tx + 16 * j, kk = n0 + col;
      const int tk = kk / C, ck = kk % C;
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const int r = 2 * ty + a;
        float ds = 0.f, dsw = 0.f;
        if (kk < N && r < valid && tk <= ti[a]) {
          const bool w = in_window(ti[a], tk, T, p.window);
          const int64_t i = m0 + r;
          const float s2 = (w ? sacc[a][j] : 0.f) + tbg[i * T + (T - 1 - (ti[a] - tk))] +
                           cbg[i * C + (C - 1 - abs(ci[a] - ck))];
          const float pr = exp2f(s2 - lse_s[r]);
          ds = pr * (pacc[a][j] - dl_s[r]) * p.sm_scale;  // `attentions/attn.py:680`
          dsw = w ? ds : 0.f;                             // `attentions/attn.py:708-717`
        }
        Ds[r * kPLd + col] = ds;
        Dw[r * kPLd + col] = dsw;
      }
    }
    __syncthreads();
    {  // row sums of dS per key time step (the reference's dS x csm_time product, `:681-694`)
      const int tk0 = n0 / C, tk1 = (min(n0 + kBN, N) - 1) / C, nT = tk1 - tk0 + 1;
      for (int idx = tid; idx < kBM * nT; idx += kThreads) {
        const int r = idx / nT, tk = tk0 + idx % nT;
        const int t_i = min(m0 + r, N - 1) / C;
        if (r >= valid || tk > t_i) continue;
        const int c_lo = max(n0, tk * C) - n0, c_hi = min(min(n0 + kBN, N), (tk + 1) * C) - n0;
        float s = 0.f;
        for (int c = c_lo; c < c_hi; ++c) s += Ds[r * kPLd + c];
        dTBs[r * T + (T - 1 - (t_i - tk))] += s;
      }
      // ... and per channel distance (`:695-707`): slot e collects c_k = c_i - e and c_i + e
      for (int idx = tid; idx < kBM * C; idx += kThreads) {
        const int r = idx / C, e = idx % C;
        if (r >= valid) continue;
        const int c_i = (m0 + r) % C;
        float s = 0.f;
        for (int tk = tk0; tk <= tk1; ++tk) {
          const int base = tk * C - n0;
          const int ca = base + c_i - e, cb = base + c_i + e;
          if (c_i - e >= 0 && ca >= 0 && ca < kBN) s += Ds[r * kPLd + ca];
          if (e > 0 && c_i + e < C && cb >= 0 && cb < kBN) s += Ds[r * kPLd + cb];
        }
        dCBs[r * C + (C - 1 - e)] += s;
      }
    }
    tile_nn<D>(Dw, Ks, qacc);  // dQ += dS_w K   (`attentions/attn.py:719-730`)
  }
  __syncthreads();
  // Finish dq and the three bias partials (autograd through `_rel_bias`).
  const Tin* rt = (const Tin*)p.rt + (int64_t)hk * T * D;
  const Tin* rc = (const Tin*)p.rc + (int64_t)hk * C * D;
  float tacc[2][DV] = {}, cacc[2][DV] = {};
  for (int s = 0; s < T; ++s) {
    const float x0 = dTBs[(2 * ty) * T + s], x1 = dTBs[(2 * ty + 1) * T + s];
#pragma unroll
    for (int e = 0; e < DV; ++e) {
      const float y = to_f32<Tin>(rt[(int64_t)s * D + tx + 16 * e]);
      tacc[0][e] += x0 * y;
      tacc[1][e] += x1 * y;
    }
  }
  for (int s = 0; s < C; ++s) {
    const float x0 = dCBs[(2 * ty) * C + s], x1 = dCBs[(2 * ty + 1) * C + s];
#pragma unroll
    for (int e = 0; e < DV; ++e) {
      const float y = to_f32<Tin>(rc[(int64_t)s * D + tx + 16 * e]);
      cacc[0][e] += x0 * y;
      cacc[1][e] += x1 * y;
    }
  }
  Tin* dq = (Tin*)bw.dq + b * bw.dq_sb + h * bw.dq_sh;
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int r = 2 * ty + a;
    if (r < valid) {
#pragma unroll
      for (int e = 0; e < DV; ++e)
        dq[(int64_t)(m0 + r) * bw.dq_sn + tx + 16 * e] = from_f32<Tin>(qacc[a][e] + tacc[a][e] + cacc[a][e]);
    }
  }
  // rows >= valid contributed zeros everywhere, so plain column sums are exact.
  float* part = bw.partial + ((int64_t)bh * gridDim.x + qt) * 3 * D;
  for (int which = 0; which < 3; ++which) {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < DV; ++e) {
      const float x = which == 0 ? qacc[0][e] + qacc[1][e]
                      : which == 1 ? tacc[0][e] + tacc[1][e] : cacc[0][e] + cacc[1][e];
      red[ty * D + tx + 16 * e] = x;
    }
    __syncthreads();
    for (int d = tid; d < D; d += kThreads) {
      float s = 0.f;
      for (int y = 0; y < 16; ++y) s += red[y * D + d];
      part[which * D + d] = s;
    }
  }
  // gradients of the relative scores, kept for dr_time / dr_chan
  float* dtbg = bw.dtbg + ((int64_t)bh * N + m0) * T;
  float* dcbg = bw.dcbg + ((int64_t)bh * N + m0) * C;
  for (int idx = tid; idx < valid * T; idx += kThreads) dtbg[idx] = dTBs[idx];
  for (int idx = tid; idx < valid * C; idx += kThreads) dcbg[idx] = dCBs[idx];
}

// dK / dV side: one CTA per (32 keys, b, kv head); loops over the g query heads of the group and
// the causal query tiles (64 rows each).  Products are formed transposed (key rows x query cols).
template <typename Tin, int D>
__global__ void __launch_bounds__(kThreads) simt_dkv_kernel(BwdArgs bw) {
  constexpr int LD = D + 4;
  constexpr int DV = D / 16;
  const Args& p = bw.a;
  extern __shared__ float smem[];
  float* Ks = smem;               // 32 keys (raw)
  float* Vs = Ks + kBM * LD;
  float* Qs = Vs + kBM * LD;      // 64 queries, (q+u)*c2
  float* Gs = Qs + kBN * LD;      // 64 dO rows
  float* Ps = Gs + kBN * LD;      // P^T   (32 x 64)
  float* Dw = Ps + kBM * kPLd;    // dS_w^T
  float* lse_s = Dw + kBM * kPLd;
  float* dl_s = lse_s + kBN;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int bk = blockIdx.y, b = bk / p.Hkv, hk = bk % p.Hkv;
  const int n0 = blockIdx.x * kBM;
  const int N = p.N, T = p.T, C = p.C;
  const int valid = min(kBM, N - n0);
  const Tin* k = (const Tin*)p.k + b * p.k_sb + hk * p.k_sh;
  const Tin* v = (const Tin*)p.v + b * p.v_sb + hk * p.v_sh;
  load_tile<Tin, D>(Ks, k, p.k_sn, n0, N, kBM, nullptr, 1.f);
  load_tile<Tin, D>(Vs, v, p.v_sn, n0, N, kBM, nullptr, 1.f);
  int tk[2], ck[2];
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int kk = min(n0 + 2 * ty + a, N - 1);
    tk[a] = kk / C;
    ck[a] = kk % C;
  }
  float kacc[2][DV], vacc[2][DV];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int e = 0; e < DV; ++e) kacc[a][e] = vacc[a][e] = 0.f;

  const int m_first = ((n0 / C) * C) / kBN * kBN;  // first query tile that can see these keys
  for (int hh = 0; hh < p.g; ++hh) {
    const int h = hk * p.g + hh, bh = b * p.H + h;
    const Tin* q = (const Tin*)p.q + b * p.q_sb + h * p.q_sh;
    const Tin* g = (const Tin*)bw.d_o + b * bw.do_sb + h * bw.do_sh;
    const float* tbg = bw.tbg + (int64_t)bh * N * T;
    const float* cbg = bw.cbg + (int64_t)bh * N * C;
    for (int m0 = m_first; m0 < N; m0 += kBN) {
      __syncthreads();
      load_tile<Tin, D>(Qs, q, p.q_sn, m0, N, kBN, (const Tin*)p.u + hk * D, p.c2);
      load_tile<Tin, D>(Gs, g, bw.do_sn, m0, N, kBN, nullptr, 1.f);
      if (tid < kBN) {
        const int i = min(m0 + tid, N - 1);
        lse_s[tid] = p.lse[(int64_t)bh * N + i];
        dl_s[tid] = bw.delta[(int64_t)bh * N + i];
      }
      __syncthreads();
      float sacc[2][4] = {}, pacc[2][4] = {};
      tile_nt<D>(Ks, Qs, sacc);  // S^T in base 2 (Qs carries c2)
      tile_nt<D>(Vs, Gs, pacc);  // dP^T
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = tx + 16 * j, i = m0 + col;
        const int t_i = i / C, c_i = i % C;
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          const int r = 2 * ty + a;
          float pr = 0.f, dsw = 0.f;
          if (i < N && r < valid && tk[a] <= t_i) {
            const bool w = in_window(t_i, tk[a], T, p.window);
            const float s2 = (w ? sacc[a][j] : 0.f) + tbg[(int64_t)i * T + (T - 1 - (t_i - tk[a]))] +
                             cbg[(int64_t)i * C + (C - 1 - abs(c_i - ck[a]))];
            pr = exp2f(s2 - lse_s[col]);
            const float ds = pr * (pacc[a][j] - dl_s[col]) * p.sm_scale;
            dsw = w ? ds : 0.f;
          }
          Ps[r * kPLd + col] = pr;
          Dw[r * kPLd + col] = dsw;
        }
      }
      __syncthreads();
      tile_nn<D>(Ps, Gs, vacc);  // dV += P^T dO        (`attentions/attn.py:671-675`)
      tile_nn<D>(Dw, Qs, kacc);  // dK += dS_w^T (q+u)  (`attentions/attn.py:718`), times c2
    }
  }
  Tin* dk = (Tin*)bw.dk + b * bw.dk_sb + hk * bw.dk_sh;
  Tin* dv = (Tin*)bw.dv + b * bw.dv_sb + hk * bw.dv_sh;
  const float inv_c2 = 1.f / p.c2;
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int r = 2 * ty + a;
    if (r < valid) {
#pragma unroll
      for (int e = 0; e < DV; ++e) {
        dk[(int64_t)(n0 + r) * bw.dk_sn + tx + 16 * e] = from_f32<Tin>(kacc[a][e] * inv_c2);
        dv[(int64_t)(n0 + r) * bw.dv_sn + tx + 16 * e] = from_f32<Tin>(vacc[a][e]);
      }
    }
  }
}

// dr[hk][slot][d] = sum_{b, h in group, i} dX[b,h,i,slot] * (q[b,h,i,d] + bias[hk][d])
// One CTA per (32 slots, kv head, split); streams its share of the group's query rows in chunks of 64.
template <typename Tin, int D>
__global__ void __launch_bounds__(kThreads) simt_drel_kernel(BwdArgs bw, int which) {
  constexpr int LD = D + 4;
  constexpr int DV = D / 16;
  const Args& p = bw.a;
  extern __shared__ float smem[];
  float* Xs = smem;            // 64 rows x 33
  float* Qs = Xs + kBN * 33;   // 64 rows x LD
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int S = which == 0 ? p.T : p.C;
  const float* dx = which == 0 ? bw.dtbg : bw.dcbg;
  const Tin* bias = (const Tin*)(which == 0 ? p.vt : p.z) + blockIdx.y * D;
  // split-K over the (batch, head of the group, 64-row chunk) range: gridDim.z partial sums
  float* out = bw.drel_part + (((int64_t)blockIdx.z * p.Hkv + blockIdx.y) * (p.T + p.C) + (which == 0 ? 0 : p.T)) * D;
  const int hk = blockIdx.y, s0 = blockIdx.x * 32;
  const int chunks_per_head = (p.N + kBN - 1) / kBN;
  const int n_chunks = p.B * p.g * chunks_per_head;
  const int per_z = (n_chunks + gridDim.z - 1) / gridDim.z;
  const int c_begin = blockIdx.z * per_z, c_end = min(n_chunks, c_begin + per_z);
  float acc[2][DV] = {};
  for (int ch = c_begin; ch < c_end; ++ch) {
    {
      const int b = ch / (p.g * chunks_per_head), hh = (ch / chunks_per_head) % p.g;
      const int m0 = (ch % chunks_per_head) * kBN;
      const int h = hk * p.g + hh, bh = b * p.H + h;
      const Tin* q = (const Tin*)p.q + b * p.q_sb + h * p.q_sh;
      {
        __syncthreads();
        load_tile<Tin, D>(Qs, q, p.q_sn, m0, p.N, kBN, bias, 1.f);
        for (int idx = tid; idx < kBN * 32; idx += kThreads) {
          const int r = idx / 32, s = idx % 32;
          const int i = m0 + r;
          Xs[r * 33 + s] = (i < p.N && s0 + s < S) ? dx[((int64_t)bh * p.N + i) * S + s0 + s] : 0.f;
        }
        __syncthreads();
        // rows >= N hold bias only in Qs but zero in Xs, so they add nothing
#pragma unroll 4
        for (int r = 0; r < kBN; ++r) {
          const float x0 = Xs[r * 33 + 2 * ty], x1 = Xs[r * 33 + 2 * ty + 1];
#pragma unroll
          for (int e = 0; e < DV; ++e) {
            const float y = Qs[r * LD + tx + 16 * e];
            acc[0][e] += x0 * y;
            acc[1][e] += x1 * y;
          }
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int s = s0 + 2 * ty + a;
    if (s < S) {
#pragma unroll
      for (int e = 0; e < DV; ++e) out[(int64_t)s * D + tx + 16 * e] = acc[a][e];
    }
  }
}

// dr_time / dr_chan = sum of the split-K partials of simt_drel_kernel (fixed order: deterministic).
__global__ void simt_drel_reduce_kernel(BwdArgs bw, int n_z) {
  const Args& p = bw.a;
  const int S = p.T + p.C;
  const int64_t total = (int64_t)p.Hkv * S * p.D;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    float sum = 0.f;
    for (int zz = 0; zz < n_z; ++zz) sum += bw.drel_part[(int64_t)zz * total + idx];
    const int d = idx % p.D, sl = (idx / p.D) % S, hk = idx / ((int64_t)p.D * S);
    if (sl < p.T) bw.drt[((int64_t)hk * p.T + sl) * p.D + d] = sum;
    else bw.drc[((int64_t)hk * p.C + (sl - p.T)) * p.D + d] = sum;
  }
}

// du/dvt/dz[hk][d] = sum over (b, h in group, query tile) of the per-tile partials.
__global__ void simt_dbias_kernel(BwdArgs bw, int n_qt) {
  const Args& p = bw.a;
  const int hk = blockIdx.x, which = blockIdx.y, D = p.D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float s = 0.f;
    for (int b = 0; b < p.B; ++b)
      for (int hh = 0; hh < p.g; ++hh) {
        const int64_t bh = (int64_t)b * p.H + hk * p.g + hh;
        for (int t = 0; t < n_qt; ++t) s += bw.partial[((bh * n_qt + t) * 3 + which) * D + d];
      }
    float* out = which == 0 ? bw.du : which == 1 ? bw.dvt : bw.dz;
    out[hk * D + d] = s;
  }
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    MVPA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  }
  return MVPA_OK;
}

template <typename Tin, int D>
int launch_fwd(const Args& a, cudaStream_t s) {
  const size_t smem = sizeof(float) * ((size_t)kBM * (D + 4) + 2 * kBN * (D + 4) + kBM * kPLd +
                                       (size_t)kBM * (a.T + a.C) + 3 * kBM);
  if (smem > 227 * 1024) {
    set_error("fp32 path: T + C = %d needs %zu bytes of shared memory (max 232448)", a.T + a.C, smem);
    return MVPA_ERR_UNSUPPORTED;
  }
  int rc = set_smem(simt_fwd_kernel<Tin, D>, smem);
  if (rc) return rc;
  dim3 grid((a.q_tn * a.C + kBM - 1) / kBM, a.B * a.H);
  simt_fwd_kernel<Tin, D><<<grid, kThreads, smem, s>>>(a);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

template <typename Tin, int D>
int launch_bwd(const BwdArgs& b, cudaStream_t s) {
  const Args& a = b.a;
  constexpr int LD = D + 4;
  const int n_qt = (a.N + kBM - 1) / kBM;
  const dim3 grid_q(n_qt, a.B * a.H);
  if (b.tc_extra == nullptr) {
    const size_t smem = sizeof(float) * kBM * LD;
    simt_rel_kernel<Tin, D><<<grid_q, kThreads, smem, s>>>(b);
    count_launch();
  }
  {
    constexpr int kRowThreads = D / (16 / (int)sizeof(Tin));
    dim3 grid((a.N * kRowThreads + kThreads - 1) / kThreads, a.B * a.H);
    simt_delta_kernel<Tin, D><<<grid, kThreads, 0, s>>>(b);
    count_launch();
  }
  if (b.tc_extra != nullptr) {
    // bf16 on the tensor cores: dq, dk, dv and the relative-score gradients
    if constexpr (D >= 64) {
      int rc = tc_bwd_q(b, b.tc_extra, s);
      if (rc) return rc;
    }
  } else {
    const size_t smem = sizeof(float) * ((size_t)2 * kBM * LD + 2 * kBN * LD + 2 * kBM * kPLd +
                                         (size_t)kBM * (a.T + a.C) + 2 * kBM + 16 * D);
    if (smem > 227 * 1024) {
      set_error("fp32 backward: T + C = %d needs %zu bytes of shared memory", a.T + a.C, smem);
      return MVPA_ERR_UNSUPPORTED;
    }
    int rc = set_smem(simt_dq_kernel<Tin, D>, smem);
    if (rc) return rc;
    simt_dq_kernel<Tin, D><<<grid_q, kThreads, smem, s>>>(b);
    count_launch();
  }
  if (b.tc_extra == nullptr) {  // (the tensor-core path has produced dK / dV already)
    const size_t smem = sizeof(float) * ((size_t)2 * kBM * LD + 2 * kBN * LD + 2 * kBM * kPLd + 2 * kBN);
    int rc = set_smem(simt_dkv_kernel<Tin, D>, smem);
    if (rc) return rc;
    dim3 grid(n_qt, a.B * a.Hkv);
    simt_dkv_kernel<Tin, D><<<grid, kThreads, smem, s>>>(b);
    count_launch();
  }
  if (b.tc_extra != nullptr) {  // the tensor-core kernels have accumulated the relative-key gradients already
    MVPA_CUDA_CHECK(cudaGetLastError());
    return tc_bwd_bias(b, b.tc_extra, s);
  }
  {
    const size_t smem = sizeof(float) * ((size_t)kBN * 33 + kBN * LD);
    int rc = set_smem(simt_drel_kernel<Tin, D>, smem);
    if (rc) return rc;
    simt_drel_kernel<Tin, D><<<dim3((a.T + 31) / 32, a.Hkv, kDrelSplit), kThreads, smem, s>>>(b, 0);
    simt_drel_kernel<Tin, D><<<dim3((a.C + 31) / 32, a.Hkv, kDrelSplit), kThreads, smem, s>>>(b, 1);
    simt_drel_reduce_kernel<<<148, 256, 0, s>>>(b, kDrelSplit);
    count_launch(3);
  }
  simt_dbias_kernel<<<dim3(a.Hkv, 3), 128, 0, s>>>(b, n_qt);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

template <typename Tin>
int dispatch_fwd(const Args& a, cudaStream_t s) {
  switch (a.D) {
    case 16: return launch_fwd<Tin, 16>(a, s);
    case 32: return launch_fwd<Tin, 32>(a, s);
    case 64: return launch_fwd<Tin, 64>(a, s);
    case 128: return launch_fwd<Tin, 128>(a, s);
  }
  return MVPA_ERR_SHAPE;
}

template <typename Tin>
int dispatch_bwd(const BwdArgs& b, cudaStream_t s) {
  switch (b.a.D) {
    case 16: return launch_bwd<Tin, 16>(b, s);
    case 32: return launch_bwd<Tin, 32>(b, s);
    case 64: return launch_bwd<Tin, 64>(b, s);
    case 128: return launch_bwd<Tin, 128>(b, s);
  }
  return MVPA_ERR_SHAPE;
}

}  // namespace

int simt_fwd(const Args& a, int dtype, cudaStream_t s) {
  return dtype == MVPA_F32 ? dispatch_fwd<float>(a, s)
         : dtype == MVPA_F16 ? dispatch_fwd<__half>(a, s) : dispatch_fwd<__nv_bfloat16>(a, s);
}

int simt_bwd(const BwdArgs& b, int dtype, cudaStream_t s) {
  return dtype == MVPA_F32 ? dispatch_bwd<float>(b, s)
         : dtype == MVPA_F16 ? dispatch_bwd<__half>(b, s) : dispatch_bwd<__nv_bfloat16>(b, s);
}

namespace {
// bf16 problems the tensor-core backward takes need only delta and (when two threads own a temporal
// slot) the temporal-score gradients from this file's areas; everything else lives in tc_extra.
bool tc_path(int dtype, int D, int C, int T) {
  Args a{};
  a.D = D; a.C = C; a.T = T;
  return dtype == MVPA_BF16 && tc_bwd_q_supported(a);
}
bool tc_needs_dtb(int D, int C) { return !(D == 64 && C <= 64); }
}  // namespace

size_t simt_bwd_workspace_floats(const mvpa_problem* p) {
  const size_t BH = (size_t)p->B * p->H, N = (size_t)p->T * p->C;
  if (tc_path(p->dtype, p->D, p->C, p->T)) {
    size_t n = BH * N + (tc_needs_dtb(p->D, p->C) ? BH * N * p->T : 0);
    n = (n + 63) & ~(size_t)63;
    return n + tc_bwd_q_workspace_floats(p);
  }
  const size_t n_qt = (N + kBM - 1) / kBM;
  size_t n = 2 * BH * N * (p->T + p->C) + BH * N + BH * n_qt * 3 * p->D +
             (size_t)kDrelSplit * p->Hkv * (p->T + p->C) * p->D;
  return (n + 63) & ~(size_t)63;
}

const int* bwd_status_word(const mvpa_problem* p, const void* workspace) {
  if (!tc_path(p->dtype, p->D, p->C, p->T)) return nullptr;  // the CUDA-core kernels have no device-side waits
  const size_t BH = (size_t)p->B * p->H, N = (size_t)p->T * p->C;
  size_t used = BH * N + (tc_needs_dtb(p->D, p->C) ? BH * N * p->T : 0);
  used = (used + 63) & ~(size_t)63;
  return reinterpret_cast<const int*>(static_cast<const float*>(workspace) + used + tc_bwd_status_offset_floats(p));
}

void simt_bwd_carve(BwdArgs& b, float* ws, int dtype) {
  const Args& a = b.a;
  const size_t BH = (size_t)a.B * a.H, N = a.N;
  if (tc_path(dtype, a.D, a.C, a.T)) {
    b.tbg = b.cbg = b.dcbg = b.partial = b.drel_part = nullptr;
    b.delta = ws;
    b.dtbg = ws + BH * N;  // (B*H, T, N) scratch of the tensor-core kernels, when they need it
    size_t used = BH * N + (tc_needs_dtb(a.D, a.C) ? BH * N * a.T : 0);
    used = (used + 63) & ~(size_t)63;
    b.tc_extra = ws + used;
    return;
  }
  const size_t n_qt = (N + kBM - 1) / kBM;
  b.tbg = ws;
  b.cbg = b.tbg + BH * N * a.T;
  b.dtbg = b.cbg + BH * N * a.C;
  b.dcbg = b.dtbg + BH * N * a.T;
  b.delta = b.dcbg + BH * N * a.C;
  b.partial = b.delta + BH * N;
  b.drel_part = b.partial + BH * n_qt * 3 * a.D;
  b.tc_extra = nullptr;
}

}  // namespace mvpa
