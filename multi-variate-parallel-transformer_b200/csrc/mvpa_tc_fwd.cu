// Flash-MVPA forward for bf16 on sm_100a: TMA-staged tiles, tcgen05 MMAs, TMEM accumulators.
//
// One CTA owns 128 query rows (= TPB whole time steps of CP channel slots, CP = channels padded
// to a power of two) of one (batch, head) and walks the causal key tiles of the same shape.
//
//   warp 4   TMA producer (one lane): Q tile, relative keys, then the K/V ring
//   warp 5   MMA issuer (one lane):   S = Q'K^T and O += P V on tcgen05, plus the two small
//            products that replace the reference's `_rel_bias` matrices
//            (`attentions/attn.py:1305-1314`); allocates / frees TMEM
//   warps 0-3 softmax: one thread per query row (= one TMEM lane): adds the temporal and channel
//            relative scores, masks, online softmax in base 2 (`attentions/attn.py:309-315`),
//            writes P (bf16) back into TMEM for the PV product, rescales O only when the
//            running maximum moved by more than 2^8, epilogue O / l and L = m + log2 l.
//
// TMEM columns: [0,128) S0 / P0, [128,256) S1 / P1, [256,256+D) O, [384,512) temporal scores
// TB[row][j] = c2 (q+vt).r_time[j].  The channel scores of a row are gathered once per CTA into
// registers (fp16x2, relative to their maximum).
//
// Tiles whose every pair lies outside the content window skip the K load and the QK^T product
// (the reference zero-fills the content term there, `attentions/attn.py:261-271`, but still
// computes it); their scores are the two relative terms only.
#include <cuda_fp16.h>

#include "mvpa_common.cuh"
#include "tc_ptx.cuh"
#include "tc_tma_host.cuh"

namespace mvpa {
namespace {

using namespace ptx;

constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr uint32_t kColS = 0;      // + 128 * buf
constexpr uint32_t kColO = 256;
constexpr uint32_t kColTB = 384;
constexpr float kRescaleThreshold = 8.f;  // log2 units: P stays below 2^8

struct TcMaps {
  CUtensorMap q, k, v, rt, rc;
};

struct TcArgs {
  const __nv_bfloat16 *u, *vt, *z;
  __nv_bfloat16* o;
  float* lse;
  int64_t o_sb, o_sh, o_sn;
  int B, H, Hkv, T, C, g, window, n_qt;
  float c2;
  int* status;
};

enum BarrierIndex {
  kBarProFull = 0, kBarProReady, kBarProMma, kBarProDone,
  kBarSFull,                 // 2
  kBarPFull = kBarSFull + 2, // 2
  kBarPvDone = kBarPFull + 2,// 2
  kBarKvFull = kBarPvDone + 2,  // ST, then kv_free ST
};

template <int D>
struct Cfg {
  static constexpr int NH = D / 64;              // 64-column (128-byte) halves of a row
  static constexpr int HALF = 16384;             // 128 rows x 128 B
  static constexpr int TILE = NH * HALF;         // one 128 x D bf16 tile
  static constexpr int ST = D == 64 ? 4 : 2;     // K/V ring depth
  static constexpr int STAGE = 2 * TILE;         // K then V
  static constexpr int SMEM_Q = 0;
  static constexpr int SMEM_RING = TILE;
  static constexpr int SMEM_TAIL = SMEM_RING + ST * STAGE;
  static constexpr int TAIL_BYTES = 3 * D * 4 + (kBarKvFull + 2 * ST) * 8 + 16;
  static constexpr int SMEM_BYTES = SMEM_TAIL + TAIL_BYTES + 1024;  // + alignment slack
};

// Bounded wait whose verdict is uniform across the warp (warp-collective TMEM ops follow it).
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, status, code));
}

__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// True when no pair of (query tile I, key tile J) has a non-zero content term.
__device__ __forceinline__ bool tile_is_light(int I, int J, int TPB, int window, int n_qt) {
  if (window <= 0 || I == n_qt - 1) return false;  // last tile holds the row t = T-1 that sees all
  const int min_dt = I * TPB - (J * TPB + TPB - 1);
  return min_dt > window;
}

template <int D, int CP>
__global__ void __launch_bounds__(kThreads, 1)
tc_fwd_kernel(const __grid_constant__ TcMaps maps, const TcArgs p) {
  using C_ = Cfg<D>;
  constexpr int NH = C_::NH, HALF = C_::HALF, TILE = C_::TILE, ST = C_::ST;
  constexpr int TPB = 128 / CP;   // time steps per tile
  constexpr int KSTEPS = D / 16;
  constexpr int LDC = CP + 1;     // scratch row stride (floats)
  static_assert(CP >= 32 && CP <= 128 && (CP & (CP - 1)) == 0, "CP in {32,64,128}");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C_::SMEM_Q;
  uint8_t* ring = smem + C_::SMEM_RING;
  uint8_t* sQv = ring;                   // prologue-only buffers alias the K/V ring
  uint8_t* sQz = ring + TILE;
  uint8_t* sR = ring + 2 * TILE;         // r_time rows 0..127 (rows >= T are zero)
  uint8_t* sC = ring + 3 * TILE;         // r_chan rows 0..CP-1
  float* scratch = reinterpret_cast<float*>(ring);  // [128][LDC], after the prologue MMAs
  float* s_bias = reinterpret_cast<float*>(smem + C_::SMEM_TAIL);  // u, vt, z as fp32, times 1
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + 3 * D);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBarKvFull + 2 * ST);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
  uint64_t* kv_full = bars + kBarKvFull;
  uint64_t* kv_free = kv_full + ST;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int BH = p.B * p.H;
  const int I = p.n_qt - 1 - (int)(blockIdx.x / BH);  // latest (heaviest) query tiles first
  const int bh = blockIdx.x % BH, b = bh / p.H, h = bh % p.H, hk = h / p.g;
  const int n_tiles = I + 1;
  const int T = p.T, C = p.C;

  if (tid == 0) {
    *s_abort = *p.status;  // a previous CTA already gave up: do nothing
    mbar_init(&bars[kBarProFull], 1);
    mbar_init(&bars[kBarProReady], 128);
    mbar_init(&bars[kBarProMma], 1);
    mbar_init(&bars[kBarProDone], 128);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[kBarSFull + i], 1);
      mbar_init(&bars[kBarPFull + i], 128);
      mbar_init(&bars[kBarPvDone + i], 1);
    }
    for (int i = 0; i < ST; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_free[i], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (*s_abort != 0) return;
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&maps.q);
      prefetch_tensormap(&maps.k);
      prefetch_tensormap(&maps.v);
      prefetch_tensormap(&maps.rt);
      prefetch_tensormap(&maps.rc);
      mbar_arrive_expect_tx(&bars[kBarProFull], 2 * TILE + NH * CP * 128);
      for (int hh = 0; hh < NH; ++hh) {
        tma_load_5d(sQ + hh * HALF, &maps.q, &bars[kBarProFull], hh * 64, 0, I * TPB, h, b);
        tma_load_3d(sR + hh * HALF, &maps.rt, &bars[kBarProFull], hh * 64, 0, hk);
        tma_load_3d(sC + hh * CP * 128, &maps.rc, &bars[kBarProFull], hh * 64, 0, hk);
      }
      bool ok = mbar_wait(&bars[kBarProDone], 0, p.status, 10);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % ST;
        if (j >= ST) ok = mbar_wait(&kv_free[s], ((j / ST) - 1) & 1, p.status, 11);
        if (!ok) break;
        const bool light = tile_is_light(I, j, TPB, p.window, p.n_qt);
        uint8_t* sK = ring + s * C_::STAGE;
        uint8_t* sV = sK + TILE;
        mbar_arrive_expect_tx(&kv_full[s], (light ? 1 : 2) * TILE);
        for (int hh = 0; hh < NH; ++hh) {
          if (!light) tma_load_5d(sK + hh * HALF, &maps.k, &kv_full[s], hh * 64, 0, j * TPB, hk, b);
          tma_load_5d(sV + hh * HALF, &maps.v, &kv_full[s], hh * 64, 0, j * TPB, hk, b);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_c = make_idesc_bf16(128, CP, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 1);
      bool ok = mbar_wait(&bars[kBarProReady], 0, p.status, 20);
      if (ok) {
        tc_fence_after();
        for (int kk = 0; kk < KSTEPS; ++kk) {  // temporal scores, all T columns at once
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          mma_ss(tmem + kColTB, make_desc_sw128(smem_u32(sQv) + off, 16, 1024),
                 make_desc_sw128(smem_u32(sR) + off, 16, 1024), idesc_s, kk > 0);
        }
        for (int kk = 0; kk < KSTEPS; ++kk) {  // channel scores -> S0 columns [0, CP)
          const uint32_t offa = (kk / 4) * HALF + (kk % 4) * 32;
          const uint32_t offb = (kk / 4) * (CP * 128) + (kk % 4) * 32;
          mma_ss(tmem + kColS, make_desc_sw128(smem_u32(sQz) + offa, 16, 1024),
                 make_desc_sw128(smem_u32(sC) + offb, 16, 1024), idesc_c, kk > 0);
        }
        mma_commit(&bars[kBarProMma]);
        ok = mbar_wait(&bars[kBarProDone], 0, p.status, 21);
      }
      auto issue_qk = [&](int j) {
        if (tile_is_light(I, j, TPB, p.window, p.n_qt)) return;
        const int s = j % ST;
        ok = mbar_wait(&kv_full[s], (j / ST) & 1, p.status, 22);
        if (!ok) return;
        tc_fence_after();
        const uint32_t sK = smem_u32(ring + s * C_::STAGE);
        for (int kk = 0; kk < KSTEPS; ++kk) {
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          mma_ss(tmem + kColS + 128 * (j & 1), make_desc_sw128(smem_u32(sQ) + off, 16, 1024),
                 make_desc_sw128(sK + off, 16, 1024), idesc_s, kk > 0);
        }
        mma_commit(&bars[kBarSFull + (j & 1)]);
      };
      if (ok) issue_qk(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles) issue_qk(j + 1);
        if (!ok) break;
        const int s = j % ST;
        ok = mbar_wait(&bars[kBarPFull + (j & 1)], (j >> 1) & 1, p.status, 23);
        if (ok) ok = mbar_wait(&kv_full[s], (j / ST) & 1, p.status, 24);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sV = smem_u32(ring + s * C_::STAGE + TILE);
        for (int kk = 0; kk < 8; ++kk) {  // 128 keys, 16 per step; P read from TMEM
          mma_ts(tmem + kColO, tmem + kColS + 128 * (j & 1) + kk * 8,
                 make_desc_sw128(sV + kk * 2048, HALF, 1024), idesc_o, (j > 0 || kk > 0));
        }
        mma_commit(&kv_free[s]);
        mma_commit(&bars[kBarPvDone + (j & 1)]);
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int r = tid;                       // query row of the tile == TMEM lane
    const int ti_loc = r / CP, c_i = r % CP;
    const int ti_abs = I * TPB + ti_loc;
    const bool row_valid = c_i < C && ti_abs < T;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    for (int d = r; d < 3 * D; d += 128) {
      const __nv_bfloat16* src = d < D ? p.u : (d < 2 * D ? p.vt : p.z);
      s_bias[d] = __bfloat162float(src[hk * D + d % D]);
    }
    softmax_bar();
    bool ok = warp_wait(&bars[kBarProFull], 0, p.status, 30);
    if (ok) {
      // Q' = (q+u) c2 in place, (q+vt) c2 and (q+z) c2 beside it (`attentions/attn.py:180-183`)
      for (int hh = 0; hh < NH; ++hh) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t off = hh * HALF + r * 128 + ((c ^ (r & 7)) << 4);
          const uint4 raw = *reinterpret_cast<const uint4*>(sQ + off);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          uint32_t ou[4], ov[4], oz[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int d = hh * 64 + c * 8 + 2 * e;
            const float x0 = __uint_as_float(w[e] << 16), x1 = __uint_as_float(w[e] & 0xffff0000u);
            ou[e] = pack_bf16((x0 + s_bias[d]) * p.c2, (x1 + s_bias[d + 1]) * p.c2);
            ov[e] = pack_bf16((x0 + s_bias[D + d]) * p.c2, (x1 + s_bias[D + d + 1]) * p.c2);
            oz[e] = pack_bf16((x0 + s_bias[2 * D + d]) * p.c2, (x1 + s_bias[2 * D + d + 1]) * p.c2);
          }
          *reinterpret_cast<uint4*>(sQ + off) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
          *reinterpret_cast<uint4*>(sQv + off) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
          *reinterpret_cast<uint4*>(sQz + off) = make_uint4(oz[0], oz[1], oz[2], oz[3]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&bars[kBarProReady]);
      ok = warp_wait(&bars[kBarProMma], 0, p.status, 31);
    }
    // Channel scores of this row, gathered by |c_i - c_k|, relative to their maximum, as fp16x2.
    __half2 cbl[CP / 2];
    float mc = 0.f;
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < CP; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + kColS + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) scratch[r * LDC + c0 + j] = __uint_as_float(v[j]);
      }
      tc_fence_before();
      float mx = -INFINITY;
      if (c_i < C)
        for (int ck = 0; ck < C; ++ck) mx = fmaxf(mx, scratch[r * LDC + (C - 1 - abs(c_i - ck))]);
      mc = (mx == -INFINITY) ? 0.f : mx;
#pragma unroll
      for (int k2 = 0; k2 < CP / 2; ++k2) {
        float x[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int ck = 2 * k2 + e;
          x[e] = (c_i < C && ck < C) ? scratch[r * LDC + (C - 1 - abs(c_i - ck))] - mc : -INFINITY;
        }
        cbl[k2] = __floats2half2_rn(x[0], x[1]);
      }
    }
    mbar_arrive(&bars[kBarProDone]);  // ring and S0 may be overwritten from here on

    float m_used = -INFINITY, l_sum = 0.f;
    int dense_seen[2] = {0, 0};
    for (int j = 0; ok && j < n_tiles; ++j) {
      const int buf = j & 1;
      const bool light = tile_is_light(I, j, TPB, p.window, p.n_qt);
      const uint32_t s_addr = lane_base + kColS + 128 * buf;
      // per key time step of the tile: temporal score, validity, content on/off
      float tbv[TPB], wmul[TPB];
      bool valid[TPB];
      {
        uint32_t raw[TPB];
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt) {
          const int tk_abs = j * TPB + tt, dt = ti_abs - tk_abs;
          valid[tt] = dt >= 0 && tk_abs < T;
          wmul[tt] = (p.window > 0 && dt > p.window && ti_abs != T - 1) ? 0.f : 1.f;
          const int dtc = min(max(dt, 0), T - 1);
          tmem_ld1(lane_base + kColTB + (T - 1 - dtc), raw[tt]);
        }
        tmem_ld_wait();
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt) tbv[tt] = __uint_as_float(raw[tt]) + mc;
      }
      float gmax[TPB];
      if (!light) {
        ok = warp_wait(&bars[kBarSFull + buf], dense_seen[buf] & 1, p.status, 32);
        if (!ok) break;
        ++dense_seen[buf];
        tc_fence_after();
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt) gmax[tt] = -INFINITY;
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(s_addr + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; jj += 2) {
            const int col = c0 + jj, tt = col / CP, ck = col % CP;
            const float2 cb = __half22float2(cbl[ck / 2]);
            gmax[tt] = fmaxf(gmax[tt], fmaf(__uint_as_float(v[jj]), wmul[tt], cb.x));
            gmax[tt] = fmaxf(gmax[tt], fmaf(__uint_as_float(v[jj + 1]), wmul[tt], cb.y));
          }
        }
      } else {
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt) gmax[tt] = 0.f;  // max of (cb - mc) over the row's channels
      }
      float m_tile = -INFINITY;
#pragma unroll
      for (int tt = 0; tt < TPB; ++tt)
        if (valid[tt]) m_tile = fmaxf(m_tile, gmax[tt] + tbv[tt]);
      if (j == 0) {
        m_used = (m_tile == -INFINITY) ? 0.f : m_tile;
      } else {
        const bool need = m_tile > m_used + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // O and l follow the maximum only when it moved by more than 2^8
          ok = warp_wait(&bars[kBarPvDone + ((j - 1) & 1)], ((j - 1) >> 1) & 1, p.status, 33);
          if (!ok) break;
          tc_fence_after();
          const float alpha = need ? ex2(m_used - m_tile) : 1.f;
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(lane_base + kColO + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) * alpha);
            tmem_st32(lane_base + kColO + c0, v);
          }
          tmem_st_wait();
          l_sum *= alpha;
          if (need) m_used = m_tile;
        }
      }
      if (j >= 2) {
        // P_j reuses the columns of P_{j-2}: the PV product that reads those must have finished.
        // (For a dense tile S_full already implies it; a light tile has no other wait.)
        ok = warp_wait(&bars[kBarPvDone + buf], ((j - 2) >> 1) & 1, p.status, 35);
        if (!ok) break;
        tc_fence_after();
      }
      float negmu[TPB];
#pragma unroll
      for (int tt = 0; tt < TPB; ++tt) negmu[tt] = valid[tt] ? tbv[tt] - m_used : -INFINITY;
      float psum = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t v[32];
        if (!light) {
          tmem_ld32(s_addr + c0, v);
          tmem_ld_wait();
        }
        uint32_t pk[16];
#pragma unroll
        for (int jj = 0; jj < 32; jj += 2) {
          const int col = c0 + jj, tt = col / CP, ck = col % CP;
          const float2 cb = __half22float2(cbl[ck / 2]);
          const float s0 = light ? cb.x : fmaf(__uint_as_float(v[jj]), wmul[tt], cb.x);
          const float s1 = light ? cb.y : fmaf(__uint_as_float(v[jj + 1]), wmul[tt], cb.y);
          const float p0 = ex2(s0 + negmu[tt]), p1 = ex2(s1 + negmu[tt]);
          psum += p0 + p1;
          pk[jj / 2] = pack_bf16(p0, p1);
        }
        tmem_st16(s_addr + c0 / 2, pk);  // P (bf16) overwrites the S columns already consumed
      }
      l_sum += psum;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[kBarPFull + buf]);
    }
    // ------------------------------- epilogue ---------------------------------
    if (ok) ok = warp_wait(&bars[kBarPvDone + ((n_tiles - 1) & 1)], ((n_tiles - 1) >> 1) & 1, p.status, 34);
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l_sum;
      const int64_t n = (int64_t)ti_abs * C + c_i;
      __nv_bfloat16* orow = p.o + b * p.o_sb + h * p.o_sh + n * p.o_sn;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + kColO + c0, v);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack_bf16(__uint_as_float(v[q4 * 8 + 2 * e]) * inv, __uint_as_float(v[q4 * 8 + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (row_valid && p.lse != nullptr) p.lse[(int64_t)bh * T * C + n] = m_used + log2f(l_sum);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

int make_maps(TcMaps& m, const Args& a, int CP) {
  const int TPB = 128 / CP;
  const uint64_t es = 2;
  int rc;
  {
    const uint64_t dims[5] = {(uint64_t)a.D, (uint64_t)a.C, (uint64_t)a.T, (uint64_t)a.H, (uint64_t)a.B};
    const uint64_t str[4] = {(uint64_t)a.q_sn * es, (uint64_t)a.q_sn * a.C * es, (uint64_t)a.q_sh * es,
                             (uint64_t)a.q_sb * es};
    const uint32_t box[5] = {64, (uint32_t)CP, (uint32_t)TPB, 1, 1};
    if ((rc = encode_bf16_sw128(&m.q, a.q, 5, dims, str, box))) return rc;
  }
  {
    const uint64_t dims[5] = {(uint64_t)a.D, (uint64_t)a.C, (uint64_t)a.T, (uint64_t)a.Hkv, (uint64_t)a.B};
    const uint32_t box[5] = {64, (uint32_t)CP, (uint32_t)TPB, 1, 1};
    const uint64_t strk[4] = {(uint64_t)a.k_sn * es, (uint64_t)a.k_sn * a.C * es, (uint64_t)a.k_sh * es,
                              (uint64_t)a.k_sb * es};
    if ((rc = encode_bf16_sw128(&m.k, a.k, 5, dims, strk, box))) return rc;
    const uint64_t strv[4] = {(uint64_t)a.v_sn * es, (uint64_t)a.v_sn * a.C * es, (uint64_t)a.v_sh * es,
                              (uint64_t)a.v_sb * es};
    if ((rc = encode_bf16_sw128(&m.v, a.v, 5, dims, strv, box))) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)a.D, (uint64_t)a.T, (uint64_t)a.Hkv};
    const uint64_t str[2] = {(uint64_t)a.D * es, (uint64_t)a.T * a.D * es};
    const uint32_t box[3] = {64, 128, 1};
    if ((rc = encode_bf16_sw128(&m.rt, a.rt, 3, dims, str, box))) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)a.D, (uint64_t)a.C, (uint64_t)a.Hkv};
    const uint64_t str[2] = {(uint64_t)a.D * es, (uint64_t)a.C * a.D * es};
    const uint32_t box[3] = {64, (uint32_t)CP, 1};
    if ((rc = encode_bf16_sw128(&m.rc, a.rc, 3, dims, str, box))) return rc;
  }
  return MVPA_OK;
}

int padded_channels(int C) { return C <= 32 ? 32 : (C <= 64 ? 64 : 128); }

template <int D, int CP>
int launch(const Args& a, int* status, cudaStream_t s) {
  TcMaps maps;
  int rc = make_maps(maps, a, CP);
  if (rc) return rc;
  TcArgs t;
  t.u = (const __nv_bfloat16*)a.u; t.vt = (const __nv_bfloat16*)a.vt; t.z = (const __nv_bfloat16*)a.z;
  t.o = (__nv_bfloat16*)a.o; t.lse = a.lse;
  t.o_sb = a.o_sb; t.o_sh = a.o_sh; t.o_sn = a.o_sn;
  t.B = a.B; t.H = a.H; t.Hkv = a.Hkv; t.T = a.T; t.C = a.C; t.g = a.g; t.window = a.window;
  constexpr int TPB = 128 / CP;
  t.n_qt = (a.T + TPB - 1) / TPB;
  t.c2 = a.c2;
  t.status = status;
  constexpr int smem = Cfg<D>::SMEM_BYTES;
  static_assert(smem <= 232448, "shared memory budget");
  MVPA_CUDA_CHECK(cudaFuncSetAttribute(tc_fwd_kernel<D, CP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  MVPA_CUDA_CHECK(cudaMemsetAsync(status, 0, sizeof(int), s));
  const unsigned grid = (unsigned)t.n_qt * a.B * a.H;
  tc_fwd_kernel<D, CP><<<grid, kThreads, smem, s>>>(maps, t);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

}  // namespace

bool tc_fwd_supported(const Args& a) {
  return (a.D == 64 || a.D == 128) && a.C <= 128 && a.T <= 128;
}

size_t tc_fwd_workspace_bytes(const mvpa_problem* p) {
  const bool tc = (p->D == 64 || p->D == 128) && p->C <= 128 && p->T <= 128;
  return tc ? 256 : 0;  // the kernel status word (bounded waits report here)
}

int tc_fwd(const Args& a, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (workspace == nullptr || workspace_bytes < 256) {
    set_error("tensor-core forward needs a 256-byte workspace");
    return MVPA_ERR_WORKSPACE;
  }
  int* status = reinterpret_cast<int*>(workspace);
  const int CP = padded_channels(a.C);
  if (a.D == 64) {
    if (CP == 32) return launch<64, 32>(a, status, s);
    if (CP == 64) return launch<64, 64>(a, status, s);
    return launch<64, 128>(a, status, s);
  }
  if (CP == 32) return launch<128, 32>(a, status, s);
  if (CP == 64) return launch<128, 64>(a, status, s);
  return launch<128, 128>(a, status, s);
}

}  // namespace mvpa
