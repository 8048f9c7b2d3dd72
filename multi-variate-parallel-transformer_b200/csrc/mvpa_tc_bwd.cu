// Flash-MVPA backward for bf16 on sm_100a, query side: dQ and the gradients of the two relative
// score matrices, on tcgen05 tensor cores with TMEM accumulators and TMA-staged tiles.
//
// Replaces, for the query side, `_bwd_kernel_one_col_block` (`attentions/attn.py:561-751`):
//   P  = exp2(S2 - L)                      S2 as in the forward, L = m + log2 l saved by it
//   dP = dO V^T                            (`:677`)
//   dS = P o (dP - delta) * sm_scale       (`:680`)
//   dQ += (dS o win) K                     (`:708-730`)
//   dTB[i, T-1-(t_i-t_k)] += sum_{c_k} dS[i,k],  dCB[i, C-1-|c_i-c_k|] += sum_{t_k} dS[i,k]   (`:681-707`)
// The reference builds the two relative-score gradients with 0/1 "csm" matmuls and atomics; here a
// thread owns a query row, so they are plain register sums (per key time step / per channel slot).
//
// Same CTA shape as the forward (mvpa_tc_fwd.cu): 128 query rows of one (b,h); two softmax
// warpgroups (thread = TMEM lane = query row, 64 key columns each), one TMA producer lane, one MMA
// issuer warp (convergent code, the tcgen05 instructions guarded by the elected lane); dense tiles (inside the content window) first, then light tiles.  Per dense tile
// three products: S = Q'K^T, dP = dO V^T, dQ += dS_w K (dS_w as bf16 in TMEM, K as MN-major
// operand); a light tile needs dP only: its content term is zero-filled, so it contributes to the
// relative-score gradients but not to dQ's content part, and P is the outer product of the forward.
// After the last tile the relative-score gradients of the tile's rows go back through the tensor
// cores: dQ += dTB r_time + dCB r_chan (autograd through `_rel_bias`, `attentions/attn.py:1305-1314`),
// and dq leaves as bf16.
//
// TMEM columns: [0,128) and [128,256) S / dS (two buffers), [256,384) dP, [384,384+D) dQ: the score
// product of the next tile runs while the softmax warps work on the current one.
#include <cuda_fp16.h>

#include "mvpa_common.cuh"
#include "tc_ptx.cuh"
#include "tc_tma_host.cuh"
#include "tc_rel_const.cuh"

namespace mvpa {
namespace {

using namespace ptx;

constexpr int kSoftmaxThreads = 256;
constexpr int kThreads = 384;  // warps 10, 11 only donate their registers
constexpr int kTmemCols = 512;
constexpr uint32_t kColS = 0;
constexpr uint32_t kColDP = 128;

// The per-kv-head accumulators receive one partial from every query-side CTA through global atomics.
// Floating-point atomics would make the sums depend on the order in which CTAs finish; integer addition is
// associative, so the partials are added as 64-bit fixed-point numbers with 32 fractional bits (resolution
// 2.3e-10, range +-2.1e9: gradients of bf16 problems sit many orders inside both) and the result is the same
// bits on every run.  The reference's kernels use relaxed fp32 atomics here (`attentions/attn.py:683-707`).
constexpr float kFix = 4294967296.f;  // 2^32
__device__ __forceinline__ void fix_add(unsigned long long* acc, float x) {
  atomicAdd(acc, (unsigned long long)__float2ll_rn(x * kFix));
}
__device__ __forceinline__ float fix_read(unsigned long long v) {
  return (float)((double)(long long)v * (1.0 / 4294967296.0));
}

struct BqMaps {
  CUtensorMap q, k, v, dout, rt, rc;
  CUtensorMap qp, dq;  // stores: Q' rows for the key-side kernel, the dq output
};

struct BqArgs {
  const __nv_bfloat16* u;
  const float* relc;   // (Hkv, 256): vt.r_time[j] at [0,128), z.r_chan[j] at [128,256)
  const float* lse;    // (B*H, N) base-2 log-sum-exp of the forward
  const float* delta;  // (B*H, N) sum_d dO*O
  float* cs_dq;        // (grid, D) per-CTA column sums of dq (fp32), for du
  // Everything a thread (= query row) reads or writes per row is stored row-innermost, so that the 32
  // rows of a warp touch consecutive addresses.
  float* dtb;          // (B*H, T, N) zero-initialised; slot T-1-(t_i-t_k)
  // Accumulators over all query-side CTAs of a kv head, zero-initialised, in 64-bit fixed point (see kFix):
  unsigned long long* racc;  // (Hkv, 2, D, 128): sum over query rows of dTB^T Q' / dCB^T Q'
  unsigned long long* cacc;  // (Hkv, 2, 128):    column sums of dTB / dCB (as bf16, like racc)
  // per query row, kept for the key-side kernel (which visits every query tile many times):
  //   Q' = (q+u) c2 as (B*H, N, D) bf16, written through the `qp` tensor map
  __half* cblw;        // (B*H, CP/8, N, 8) channel scores gathered by key channel slot, relative to their max
  __nv_bfloat16* bcw;  // same layout: exp2 of them (the key-side kernel's light pairs are outer products)
  float* offw;         // (B*H, N)     that max minus L
  float* tbw;          // (B*H, T, N)  temporal scores, log2 units
  int B, H, Hkv, T, C, g, window, n_qt;
  int kv_major;  // CTA order: see kv_major_order()
  float c2, sm_scale;
  int* status;
};

enum BarrierIndex {
  kBarProFull = 0, kBarProMma, kBarProDone, kBarSFull, kBarSFull1, kBarDpFull, kBarDpFull1, kBarDsFull, kBarDsFull1, kBarAllDone,
  kBarFinFull, kBarFinLoaded, kBarFinDone, kBarRelDone,
  kBarSlotFull,  // NS, then slot_free NS
};

template <int D>
struct Cfg {
  static constexpr int NH = D / 64;
  static constexpr int HALF = 16384;
  static constexpr int TILE = NH * HALF;
  static constexpr int NS = D == 64 ? 8 : 4;       // K/V ring slots (dense tile: K and V; light: V)
  static constexpr int PRO_SLOTS = 65536 / TILE;   // borrowed by the prologue (sR + sC, then scratch)
  static constexpr int EARLY = NS - PRO_SLOTS;
  static constexpr int SMEM_Q = 0;
  static constexpr int SMEM_DO = TILE;
  static constexpr int SMEM_RING = 2 * TILE;
  static constexpr int SMEM_PRO = SMEM_RING + EARLY * TILE;
  // head_dim 64 leaves room for the tile's temporal-score gradients, [row][slot] as bf16 in the operand
  // layout, through the whole main loop (used when every (row, slot) has a single owning thread)
  static constexpr int SMEM_TBT = SMEM_RING + NS * TILE;
  static constexpr int SMEM_TAIL = SMEM_TBT + (D == 64 ? 32768 : 0);
  // tail: u (D f32), vR[128], zC[128], smax[2][128], barriers, tmem slot, abort
  static constexpr int TAIL_FLOATS = D + 128 + 128 + 256;
  static constexpr int TAIL_BYTES = TAIL_FLOATS * 4 + (kBarSlotFull + 2 * NS) * 8 + 16;
  static constexpr int SMEM_BYTES = SMEM_TAIL + TAIL_BYTES + 1024;
};

__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, status, code));
}
// All 256 softmax threads; only called outside data-dependent control flow.
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ int light_tiles(int I, int TPB, int window, int n_qt) {
  if (window <= 0 || I == n_qt - 1) return 0;
  const int x = I * TPB - TPB - window;
  return x < 0 ? 0 : x / TPB + 1;
}

template <int D, int CP>
__global__ void __launch_bounds__(kThreads, 1)
tc_bwd_q_kernel(const __grid_constant__ BqMaps maps, const BqArgs p) {
  using C_ = Cfg<D>;
  constexpr int NH = C_::NH, HALF = C_::HALF, TILE = C_::TILE, NS = C_::NS;
  constexpr int TPB = 128 / CP;
  constexpr int TPW = TPB >= 2 ? TPB / 2 : 1;
  constexpr int NCH = CP < 64 ? CP : 64;
  constexpr int KSTEPS = D / 16;
  constexpr int DW = D / 2;
  // TMEM columns: S / dS double-buffered, so that the score product of the next tile runs while the
  // softmax warps work on this one.  The raw temporal products only pass through the dQ columns during
  // the prologue (the scaled scores are re-read from the workspace, tile by tile); the dr_time
  // accumulator of the epilogue takes the second S buffer.
  constexpr uint32_t kQS = 0, kQS1 = 128, kQDP = 256, kQDQ = 384;
  // With at most 64 channel slots a key time step belongs to one warpgroup, so each (row, slot) sum of
  // dS has one owner and goes straight into a shared-memory tile; otherwise the two owners add into the
  // workspace with atomics and the tile is rebuilt from there after the loop.
  constexpr bool TBS = (D == 64) && (CP <= 64);
  // The prologue's scratch rows are padded instead of rotated when that fits (<= 64 channel slots).
  constexpr bool PAD = CP <= 64;
  constexpr int LDP = PAD ? CP + 2 : CP;
  static_assert(CP >= 32 && CP <= 128 && (CP & (CP - 1)) == 0, "CP in {32,64,128}");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C_::SMEM_Q;
  uint8_t* sDO = smem + C_::SMEM_DO;
  uint8_t* ring = smem + C_::SMEM_RING;
  uint8_t* sR = smem + C_::SMEM_PRO;
  uint8_t* sC = sR + TILE;
  float* scratch = reinterpret_cast<float*>(smem + C_::SMEM_PRO);  // [128][CP]
  uint8_t* s_tbt_main = smem + C_::SMEM_TBT;
  float* s_bias = reinterpret_cast<float*>(smem + C_::SMEM_TAIL);  // u as fp32
  float* s_vr = s_bias + D;
  float* s_zc = s_vr + 128;
  float* s_max = s_zc + 128;  // [2 wg][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_max + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBarSlotFull + 2 * NS);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
  uint64_t* slot_full = bars + kBarSlotFull;
  uint64_t* slot_free = slot_full + NS;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int BH = p.B * p.H;
  int I, bh;
  if (p.kv_major) {
    const int per = p.n_qt * p.g, grp = (int)(blockIdx.x / per), r = (int)(blockIdx.x % per);
    I = p.n_qt - 1 - r / p.g;
    bh = grp * p.g + r % p.g;  // grp = b * Hkv + hk
  } else {
    I = p.n_qt - 1 - (int)(blockIdx.x / BH);
    bh = blockIdx.x % BH;
  }
  const int b = bh / p.H, h = bh % p.H, hk = h / p.g;
  const int cta_slot = (p.n_qt - 1 - I) * BH + bh;  // index of this CTA's per-CTA outputs, whatever the order
  const int n_tiles = I + 1;
  const int n_light = light_tiles(I, TPB, p.window, p.n_qt);
  // Visit order: the light tiles 0 .. n_light-1 first, then the dense ones (natural key order).  In the
  // light phase the channel-score gradient is accumulated unscaled (see the softmax warps) and folded
  // into the ordinary accumulators at the transition, so it must come first.
  auto tile_of = [&](int s) { return s; };
  auto is_dense = [&](int s) { return s >= n_light; };
  // position of a tile's K / V in the load sequence (a light tile loads V only)
  auto q_of_k = [&](int s) { return n_light + 2 * (s - n_light); };
  auto q_of_v = [&](int s) { return s < n_light ? s : n_light + 2 * (s - n_light) + 1; };
  const int T = p.T, C = p.C;

  // One barrier at entry: thread 0 initialises the mbarriers, another warp fetches the status word (an
  // earlier CTA may have given up), warp 9 allocates the tensor memory - all at the same time.
  if (tid == 0) {
    mbar_init(&bars[kBarProFull], 1);
    mbar_init(&bars[kBarProMma], 1);
    mbar_init(&bars[kBarProDone], kSoftmaxThreads);
    mbar_init(&bars[kBarSFull], 1);
    mbar_init(&bars[kBarSFull + 1], 1);
    mbar_init(&bars[kBarDpFull], 1);
    mbar_init(&bars[kBarDpFull + 1], 1);
    mbar_init(&bars[kBarDsFull], kSoftmaxThreads);
    mbar_init(&bars[kBarDsFull + 1], kSoftmaxThreads);
    mbar_init(&bars[kBarAllDone], 1);
    mbar_init(&bars[kBarFinFull], kSoftmaxThreads);
    mbar_init(&bars[kBarFinLoaded], 1);
    mbar_init(&bars[kBarFinDone], 1);
    mbar_init(&bars[kBarRelDone], 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_free[i], 1);
    }
    mbar_fence_init();
  } else if (tid == 64) {
    *s_abort = *p.status;
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (*s_abort != 0) {  // do nothing, but give the columns back
    if (warp == 9) tmem_dealloc(tmem, kTmemCols);
    return;
  }

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&maps.q);
      prefetch_tensormap(&maps.k);
      prefetch_tensormap(&maps.v);
      prefetch_tensormap(&maps.dout);
      mbar_arrive_expect_tx(&bars[kBarProFull], 3 * TILE + NH * CP * 128);
      for (int hh = 0; hh < NH; ++hh) {
        tma_load_5d(sQ + hh * HALF, &maps.q, &bars[kBarProFull], hh * 64, 0, I * TPB, h, b);
        tma_load_5d(sDO + hh * HALF, &maps.dout, &bars[kBarProFull], hh * 64, 0, I * TPB, h, b);
        tma_load_3d(sR + hh * HALF, &maps.rt, &bars[kBarProFull], hh * 64, 0, hk);
        tma_load_3d(sC + hh * CP * 128, &maps.rc, &bars[kBarProFull], hh * 64, 0, hk);
      }
      bool ok = true;
      auto load_slot = [&](const CUtensorMap* map, int q, int J) {
        if (q == C_::EARLY) ok = mbar_wait(&bars[kBarProDone], 0, p.status, 110);
        const int sl = q % NS;
        if (ok && q >= NS) ok = mbar_wait(&slot_free[sl], ((q / NS) - 1) & 1, p.status, 111);
        if (!ok) return;
        uint8_t* dst = ring + sl * TILE;
        mbar_arrive_expect_tx(&slot_full[sl], TILE);
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) tma_load_5d(dst + hh * HALF, map, &slot_full[sl], hh * 64, 0, J * TPB, hk, b);
      };
      for (int s = 0; ok && s < n_tiles; ++s) {
        const int J = tile_of(s);
        if (is_dense(s)) load_slot(&maps.k, q_of_k(s), J);
        if (ok) load_slot(&maps.v, q_of_v(s), J);
      }
      // finish: the relative keys once more (the ring is idle once every product has completed)
      if (ok) ok = mbar_wait(&bars[kBarAllDone], 0, p.status, 112);
      if (ok) {
        uint8_t* fR = ring + 65536;
        uint8_t* fC = fR + TILE;
        mbar_arrive_expect_tx(&bars[kBarFinLoaded], TILE + NH * CP * 128);
        for (int hh = 0; hh < NH; ++hh) {
          tma_load_3d(fR + hh * HALF, &maps.rt, &bars[kBarFinLoaded], hh * 64, 0, hk);
          tma_load_3d(fC + hh * CP * 128, &maps.rc, &bars[kBarFinLoaded], hh * 64, 0, hk);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -------------------------------
    // (the whole warp, in convergent code; the tcgen05 instructions are guarded by the elected lane)
    {
      constexpr uint32_t kFull = 0xffffffffu;
      const uint32_t el = elect_one();
      const uint32_t tm = __shfl_sync(kFull, tmem, 0);
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_c = make_idesc_bf16(128, CP, 0);
      constexpr uint32_t idesc_q = make_idesc_bf16(128, D, 1);
      const DescHalves dq = make_desc_halves_sw128(smem_u32(sQ), 16, 1024);
      const DescHalves ddo = make_desc_halves_sw128(smem_u32(sDO), 16, 1024);
      const DescHalves dkm0 = make_desc_halves_sw128(smem_u32(ring), 16, 1024);    // K-major view of a slot
      const DescHalves dmn0 = make_desc_halves_sw128(smem_u32(ring), HALF, 1024);  // MN-major view of a slot
      bool ok = __all_sync(kFull, mbar_wait(&bars[kBarProFull], 0, p.status, 120));
      if (ok) {
        tc_fence_after();
        const DescHalves dr = make_desc_halves_sw128(smem_u32(sR), 16, 1024);
        const DescHalves dc = make_desc_halves_sw128(smem_u32(sC), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          mma_ss_w(el, tm + kQDQ, dq, off, dr, off, idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          const uint32_t offa = (kk / 4) * HALF + (kk % 4) * 32;
          const uint32_t offb = (kk / 4) * (CP * 128) + (kk % 4) * 32;
          mma_ss_w(el, tm + kQS, dq, offa, dc, offb, idesc_c, kk > 0);
        }
        mma_commit_w(el, smem_u32(&bars[kBarProMma]));
        ok = __all_sync(kFull, mbar_wait(&bars[kBarProDone], 0, p.status, 121));
        if (ok && lane == 0) {  // Q' (written to sQ and fenced by the softmax warps) goes out for the key-side kernel
#pragma unroll
          for (int hh = 0; hh < NH; ++hh) tma_store_5d(&maps.qp, sQ + hh * HALF, hh * 64, 0, I * TPB, h, b);
          tma_store_commit();
        }
      }
      // Order on the tensor pipe: S_{s+1} (needs nothing from the softmax warps) runs while they work on
      // tile s; once they report dS_s, dP_{s+1} goes first (their second phase waits for it), then dQ += dS_s K_s.
      auto issue_s = [&](int s) {
        const int qk = q_of_k(s), ksl = qk % NS;
        ok = __all_sync(kFull, mbar_wait(&slot_full[ksl], (qk / NS) & 1, p.status, 123));
        if (!ok) return;
        tc_fence_after();
        DescHalves dk = dkm0;
        dk.lo += (uint32_t)ksl * (TILE >> 4);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {  // S = Q' K^T
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          mma_ss_w(el, tm + kQS + 128 * (s & 1), dq, off, dk, off, idesc_s, kk > 0);
        }
        mma_commit_w(el, smem_u32(&bars[kBarSFull + (s & 1)]));
      };
      auto issue_dp = [&](int s) {
        const int qv = q_of_v(s), vsl = qv % NS;
        ok = __all_sync(kFull, mbar_wait(&slot_full[vsl], (qv / NS) & 1, p.status, 124));
        if (!ok) return;
        tc_fence_after();
        DescHalves dv = dkm0;
        dv.lo += (uint32_t)vsl * (TILE >> 4);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {  // dP = dO V^T  (V rows = keys, D contiguous: K-major operand)
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          // a light tile has no score product: its dP takes the idle S buffer, so two are in flight
          mma_ss_w(el, tm + (is_dense(s) ? kQDP : kQS + 128 * (s & 1)), ddo, off, dv, off, idesc_s, kk > 0);
        }
        mma_commit_w(el, smem_u32(&bars[kBarDpFull + (s & 1)]));
        mma_commit_w(el, smem_u32(&slot_free[vsl]));
      };
      if (ok && is_dense(0)) issue_s(0);
      if (ok) issue_dp(0);
      for (int s = 0; ok && s < n_tiles; ++s) {
        const bool next = s + 1 < n_tiles, next_dense = next && is_dense(s + 1);
        // (S buffer (s+1)&1 is free: tile s-1 left it when its dS / dP was consumed)
        if (next_dense) issue_s(s + 1);
        if (ok && next && !next_dense) issue_dp(s + 1);
        // (two barriers, by tile parity: in the light phase a fast warp may report tile s+1 before a slow
        // one has reported tile s, and arrivals of two tiles must not mix in one phase)
        if (ok) ok = __all_sync(kFull, mbar_wait(&bars[kBarDsFull + (s & 1)], (s >> 1) & 1, p.status, 122));  // dS_w in the S columns, dP read
        if (!ok) break;
        tc_fence_after();
        if (next_dense) issue_dp(s + 1);
        if (!ok) break;
        if (is_dense(s)) {  // dQ += dS_w K   (A from TMEM, K as MN-major operand)
          const int ksl = q_of_k(s) % NS;
          const uint32_t b_lo = dmn0.lo + (uint32_t)ksl * (TILE >> 4);
          const uint32_t a0 = tm + kQS + 128 * (s & 1);
          mma_ts_x4_w(el, tm + kQDQ, a0, b_lo, dmn0.hi, 2048 >> 4, idesc_q, (uint32_t)(s > n_light));
          mma_ts_x4_w(el, tm + kQDQ, a0 + 64, b_lo + 4 * (2048 >> 4), dmn0.hi, 2048 >> 4, idesc_q, 1u);
          mma_commit_w(el, smem_u32(&slot_free[ksl]));
        }
      }
      mma_commit_w(el, smem_u32(&bars[kBarAllDone]));
      // finish: dQ += dTB r_time + dCB r_chan  (autograd through `_rel_bias`, `attentions/attn.py:1305-1314`);
      // the softmax warps have put dTB / dCB of the tile's rows into TMEM as bf16
      if (ok) ok = __all_sync(kFull, mbar_wait(&bars[kBarFinFull], 0, p.status, 125));
      if (ok) ok = __all_sync(kFull, mbar_wait(&bars[kBarFinLoaded], 0, p.status, 126));
      if (ok) {
        tc_fence_after();
        const DescHalves dfr = make_desc_halves_sw128(smem_u32(ring + 65536), HALF, 1024);
        const DescHalves dfc = make_desc_halves_sw128(smem_u32(ring + 65536 + TILE), CP * 128, 1024);
        mma_ts_x4_w(el, tm + kQDQ, tm + kQS, dfr.lo, dfr.hi, 2048 >> 4, idesc_q, 1u);
        mma_ts_x4_w(el, tm + kQDQ, tm + kQS + 32, dfr.lo + 4 * (2048 >> 4), dfr.hi, 2048 >> 4, idesc_q, 1u);
#pragma unroll
        for (int kk = 0; kk < CP / 16; ++kk) mma_ts_w(el, tm + kQDQ, tm + kQDP + kk * 8, dfc, kk * 2048, idesc_q, 1u);
      }
      mma_commit_w(el, smem_u32(&bars[kBarFinDone]));
      // Relative-key gradients of this tile's rows (autograd through `_rel_bias`, `attentions/attn.py:1305-1314`):
      //   R_t[j, d] = sum_i dTB[i, j] Q'[i, d],  R_c[j, d] = sum_i dCB[i, j] Q'[i, d]   (A = the bf16 tiles the
      //   softmax warps left in shared memory, keys-of-the-sum = query rows; B = Q' as MN-major operand)
      // and the column sums of dTB / dCB as products with a tile of ones.  Accumulators: the idle S, dP
      // and temporal-score columns.
      if (ok) {
        constexpr uint32_t idesc_r = make_idesc_bf16_ab(128, D, 1, 1);
        constexpr uint32_t idesc_1 = make_idesc_bf16_ab(128, 16, 1, 0);
        const DescHalves dtbt = make_desc_halves_sw128(smem_u32(TBS ? s_tbt_main : ring), HALF, 1024);
        const DescHalves dcbt = make_desc_halves_sw128(smem_u32(D == 128 ? sDO : ring + 98304), HALF, 1024);
        const DescHalves dqm = make_desc_halves_sw128(smem_u32(sQ), HALF, 1024);
        const DescHalves dones = make_desc_halves_sw128(smem_u32(ring + 32768), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss_w(el, tm + kQS1, dtbt, kk * 2048, dqm, kk * 2048, idesc_r, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss_w(el, tm + kQS, dcbt, kk * 2048, dqm, kk * 2048, idesc_r, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offb = (kk / 4) * 2048 + (kk % 4) * 32;
          mma_ss_w(el, tm + kQDP, dtbt, kk * 2048, dones, offb, idesc_1, kk > 0);
          mma_ss_w(el, tm + kQDP + 16, dcbt, kk * 2048, dones, offb, idesc_1, kk > 0);
        }
      }
      mma_commit_w(el, smem_u32(&bars[kBarRelDone]));
      if (lane == 0) tma_store_wait_all();  // the store reads sQ: it has to finish before the CTA can go away
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ------------------------------ softmax warps ------------------------------
    const int row = tid & 127;
    const int wg = tid >> 7;
    const int ti_loc = row / CP, c_i = row % CP;
    const int ti_abs = I * TPB + ti_loc;
    const bool row_valid = c_i < C && ti_abs < T;
    const int N = T * C;
    const int n_loc = ti_abs * C + c_i;                   // row within the (b,h) slice
    const int64_t n_row = (int64_t)bh * N + n_loc;        // global row of this thread
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int tt_base = (64 * wg) / CP;
    const int ck_base = CP == 128 ? 64 * wg : 0;
    if constexpr (TBS) {  // slots no key tile reaches stay zero
#pragma unroll
      for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(s_tbt_main + tid * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int d = tid; d < D; d += kSoftmaxThreads) s_bias[d] = __bfloat162float(p.u[hk * D + d]);
    s_vr[tid] = p.relc[hk * 256 + tid];  // s_vr and s_zc are adjacent: 256 floats
    // L = +inf on rows that do not exist: their P is 0 everywhere
    const float L_i = row_valid ? p.lse[n_row] : INFINITY;
    const float delta_i = row_valid ? p.delta[n_row] : 0.f;
    softmax_bar();
    bool ok = warp_wait(&bars[kBarProMma], 0, p.status, 131);
    if (ok) {
      tc_fence_after();
      // The prologue and the epilogue run once per CTA, so their instructions come from memory rather
      // than the instruction cache: they are written as short loops, not unrolled.
      // temporal scores of the row, for the key-side kernel (each warpgroup dumps half of the columns)
      {
        float* dst = p.tbw + ((int64_t)bh * T + 64 * wg) * N + (row_valid ? n_loc : 0);
        // Only the slots of keys a row can see (t_k <= t_i: slot >= T-1-t_i) are ever read, by this
        // kernel's loop and by the key-side kernel: early query tiles skip most of the dump.
        const int j_row = T - 1 - min(ti_abs, T - 1);
        auto put8 = [&](const uint32_t (&v)[8], int c8) {
          if (row_valid) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int j = 64 * wg + c8 + e;
              if (j >= j_row && j < T) dst[(int64_t)(c8 + e) * N] = p.c2 * (__uint_as_float(v[e]) + s_vr[j]);
            }
          }
        };
        const int j_tile = max(T - 1 - (I * TPB + TPB - 1), 0) - 64 * wg;  // first slot any row of the tile can see
        const int c_first = j_tile <= 0 ? 0 : (j_tile & ~15);
        uint32_t va[8], vb[8];  // the next 8 columns are in flight while 8 are stored
        if (c_first < 64) tmem_ld8(lane_base + kQDQ + 64 * wg + c_first, va);
#pragma unroll 1
        for (int c8 = c_first; c8 < 64; c8 += 16) {
          tmem_ld_wait();
          tmem_ld8(lane_base + kQDQ + 64 * wg + c8 + 8, vb);
          put8(va, c8);
          tmem_ld_wait();
          if (c8 + 16 < 64) tmem_ld8(lane_base + kQDQ + 64 * wg + c8 + 16, va);
          put8(vb, c8 + 8);
        }
      }
      // channel scores by |c_i - c_k| slot to shared memory (8-column chunks alternate between the warpgroups)
#pragma unroll 1
      for (int c8 = 8 * wg; c8 < CP; c8 += 16) {
        uint32_t v[8];
        tmem_ld8(lane_base + kQS + c8, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float val = p.c2 * (__uint_as_float(v[e]) + s_zc[c8 + e]);
          if constexpr (PAD) scratch[row * LDP + c8 + e] = val;
          else scratch[row * CP + ((c8 + e + 2 * row) & (CP - 1))] = val;
        }
      }
      tc_fence_before();
    }
    softmax_bar();
    float mc = 0.f;
    {
      // gather by key channel slot: g_k = CB[i, C-1-|c_i - c_k|]; first the row maximum, then fp16 values
      // relative to it, staged in this thread's own row of s_cbl (16-byte chunks swizzled by the row)
      // (up to 64 channel slots: padded rows, slot C-1-|c_i - c_k| runs up through the row for c_k <= c_i
      // and down for c_k > c_i; positions of channels that do not exist may lie outside the row and
      // are dropped.  128 slots: rotated rows.)
      const float* up = scratch + row * LDP + (C - 1 - c_i);
      const float* down = scratch + row * LDP + (C - 1 + c_i);
      const int climit = c_i < C ? C : 0;
      auto gathered = [&](int k) {
        if constexpr (PAD) {
          const float val = ok ? (k <= c_i ? up[k] : down[-k]) : 0.f;
          return k < climit ? val : -INFINITY;
        } else {
          const int ck = ck_base + k;
          const int jc = min(max(C - 1 - abs(c_i - ck), 0), CP - 1);
          const float val = ok ? scratch[row * CP + ((jc + 2 * row) & (CP - 1))] : 0.f;
          return (c_i < C && ck < C) ? val : -INFINITY;
        }
      };
      float mx = -INFINITY;
#pragma unroll 4
      for (int k = 0; k < NCH; ++k) mx = fmaxf(mx, gathered(k));
      if constexpr (!PAD) {  // the row maximum spans both warpgroups' columns
        s_max[wg * 128 + row] = mx;
        softmax_bar();
        mx = fmaxf(mx, s_max[(wg ^ 1) * 128 + row]);
      }
      mc = (mx == -INFINITY) ? 0.f : mx;
      // fp16 pairs relative to the maximum, staged in this thread's lane of idle TMEM columns so that the
      // loop stays short and the values still end up in registers
#pragma unroll 1
      for (int k16 = 0; k16 < NCH; k16 += 16) {
        uint32_t pk[8], pb[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float x0 = gathered(k16 + 2 * e) - mc, x1 = gathered(k16 + 2 * e + 1) - mc;
          const __half2 hh2 = __floats2half2_rn(x0, x1);
          const __half2 eh2 = __floats2half2_rn(ex2(x0), ex2(x1));
          pk[e] = *reinterpret_cast<const uint32_t*>(&hh2);
          pb[e] = *reinterpret_cast<const uint32_t*>(&eh2);
        }
        tmem_st8(lane_base + kQDP + 32 * wg + k16 / 2, pk);
        tmem_st8(lane_base + kQDP + 64 + 32 * wg + k16 / 2, pb);
        if (ok && row_valid && (CP == 128 || wg == 0)) {  // copies for the key-side kernel (exponentials as bf16)
          const int64_t chunk = ((int64_t)bh * (CP / 8) + (ck_base + k16) / 8) * N + n_loc;
          uint4* cdst = reinterpret_cast<uint4*>(p.cblw) + chunk;
          uint4* bdst = reinterpret_cast<uint4*>(p.bcw) + chunk;
          uint32_t wb[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pb[e]));
            wb[e] = pack_bf16(f.x, f.y);
          }
          cdst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          cdst[N] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          bdst[0] = make_uint4(wb[0], wb[1], wb[2], wb[3]);
          bdst[N] = make_uint4(wb[4], wb[5], wb[6], wb[7]);
        }
      }
      tmem_st_wait();  // the staged values are read back where they are needed (light phase: bc; dense phase: cbl)
      tc_fence_before();
      const bool store_cbl = ok && row_valid && (CP == 128 || wg == 0);
      if (store_cbl && wg == 0) p.offw[n_row] = mc - L_i;
      if (ok) {
        const float4* u4 = reinterpret_cast<const float4*>(s_bias);
#pragma unroll 1
        for (int cc = 0; cc < D / 16; ++cc) {
          const int chunk = wg * (D / 16) + cc, hh = chunk / 8, c = chunk % 8;
          const uint32_t off = hh * HALF + row * 128 + ((c ^ (row & 7)) << 4);
          const uint4 raw = *reinterpret_cast<const uint4*>(sQ + off);
          const float4 b0 = u4[chunk * 2], b1 = u4[chunk * 2 + 1];
          uint4 out;
          out.x = pack_bf16((__uint_as_float(raw.x << 16) + b0.x) * p.c2, (__uint_as_float(raw.x & 0xffff0000u) + b0.y) * p.c2);
          out.y = pack_bf16((__uint_as_float(raw.y << 16) + b0.z) * p.c2, (__uint_as_float(raw.y & 0xffff0000u) + b0.w) * p.c2);
          out.z = pack_bf16((__uint_as_float(raw.z << 16) + b1.x) * p.c2, (__uint_as_float(raw.z & 0xffff0000u) + b1.y) * p.c2);
          out.w = pack_bf16((__uint_as_float(raw.w << 16) + b1.z) * p.c2, (__uint_as_float(raw.w & 0xffff0000u) + b1.w) * p.c2);
          *reinterpret_cast<uint4*>(sQ + off) = out;
        }
        fence_proxy_async_smem();
      }
    }

    // gradient of the channel scores, per channel slot of this thread's columns (summed over time)
    float dcb_acc[NCH];
#pragma unroll
    for (int k = 0; k < NCH; ++k) dcb_acc[k] = 0.f;
    const float off_row = mc - L_i;  // every exponent carries +mc (cbl is relative to it) and -L

    // Temporal scores of the row come back from the workspace (this CTA wrote them in the prologue; the
    // barriers since then order the accesses): TPW values per tile, fetched one tile ahead.
    const float* tb_src = p.tbw + (int64_t)bh * T * N + (row_valid ? n_loc : 0);
    auto tb_slot = [&](int s, int tl) {
      const int tk_abs = tile_of(s) * TPB + tt_base + tl;
      return T - 1 - min(max(ti_abs - tk_abs, 0), T - 1);
    };
    float tb_next[TPW];
#pragma unroll
    for (int tl = 0; tl < TPW; ++tl) tb_next[tl] = ok ? __ldcg(tb_src + (int64_t)tb_slot(0, tl) * N) : 0.f;

    // sm_scale is folded into the exponent: the loop works with P' = sm_scale * P, so dS = P' (dP - delta)
    const float lscale = log2f(p.sm_scale);
    // The gathered channel scores (fp16, dense tiles) and their exponentials (light tiles) wait in this
    // thread's lane of the dP columns, which no MMA touches before the first dense tile.
    __half2 cbl[NCH / 2];
    auto load_cbl = [&]() {
      uint32_t w[32];
      tmem_ld32(lane_base + kQDP + 32 * wg, w);
      tmem_ld_wait();
#pragma unroll
      for (int k2 = 0; k2 < NCH / 2; ++k2) *reinterpret_cast<uint32_t*>(&cbl[k2]) = w[k2];
    };
    // Light tiles: P'[i,k] = a[t_k] bc[c_k] with a = exp2(temporal score + max - L + log2 sm_scale), so
    //   sum_t dS = bc[c_k] (sum_t a[t] dP[t, c_k] - delta sum_t a[t])        -> two FMAs per element:
    //   sum_c dS = a[t] (sum_c bc[c] dP[t, c] - delta sum_c bc[c])
    // dcb_acc holds the inner sums until the transition below scales them.
    float bcf[NCH];
    float a_sum = 0.f, bc_sum = 0.f;
    if (n_light > 0) {
      uint32_t w[32];
      tmem_ld32(lane_base + kQDP + 64 + 32 * wg, w);
      tmem_ld_wait();
#pragma unroll
      for (int k2 = 0; k2 < NCH / 2; ++k2) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k2]));
        bcf[2 * k2] = f.x;
        bcf[2 * k2 + 1] = f.y;
        bc_sum += f.x + f.y;
      }
    } else {
#pragma unroll
      for (int k = 0; k < NCH; ++k) bcf[k] = 0.f;
      load_cbl();
    }
    tc_fence_before();
    mbar_arrive(&bars[kBarProDone]);  // only now may a dP product overwrite the staged values
    for (int s = 0; ok && s < n_tiles; ++s) {
      const bool dense = is_dense(s);
      const int J = tile_of(s);
      float offs[TPW], wmul[TPW], dtb_acc[TPW];
      int slot[TPW];
      bool valid[TPW];
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) {
        const int tk_abs = J * TPB + tt_base + tl, dt = ti_abs - tk_abs;
        valid[tl] = dt >= 0 && tk_abs < T && row_valid;
        slot[tl] = T - 1 - min(max(dt, 0), T - 1);
        wmul[tl] = (p.window > 0 && dt > p.window && ti_abs != T - 1) ? 0.f : 1.f;
        dtb_acc[tl] = 0.f;
        offs[tl] = valid[tl] ? tb_next[tl] + off_row + lscale : -INFINITY;
      }
      if (s + 1 < n_tiles) {
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl) tb_next[tl] = __ldcg(tb_src + (int64_t)tb_slot(s + 1, tl) * N);
      }
      if (dense) {
        ok = warp_wait(&bars[kBarSFull + (s & 1)], ((s - n_light) >> 1) & 1, p.status, 132);
        if (!ok) break;
      }
      ok = warp_wait(&bars[kBarDpFull + (s & 1)], (s >> 1) & 1, p.status, 133);
      if (!ok) break;
      tc_fence_after();
      if (dense) {
        // P' = exp2(S2 - L + log2 sm_scale), dS = P' (dP - delta)   (`attentions/attn.py:680`)
        const uint32_t s_addr = lane_base + kQS + 128 * (s & 1) + 64 * wg;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t sv[32], dp[32];
          tmem_ld32(s_addr + 32 * half, sv);
          tmem_ld32(lane_base + kQDP + 64 * wg + 32 * half, dp);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int jj = 0; jj < 32; jj += 2) {
            const int lc = 32 * half + jj, tl = lc / CP, k = lc % NCH;
            const float2 cb = __half22float2(cbl[k / 2]);
            const float p0 = ex2(fmaf(__uint_as_float(sv[jj]), wmul[tl], cb.x) + offs[tl]);
            const float p1 = ex2(fmaf(__uint_as_float(sv[jj + 1]), wmul[tl], cb.y) + offs[tl]);
            const float ds0 = p0 * (__uint_as_float(dp[jj]) - delta_i);
            const float ds1 = p1 * (__uint_as_float(dp[jj + 1]) - delta_i);
            dcb_acc[k] += ds0;
            dcb_acc[k + 1] += ds1;
            dtb_acc[tl] += ds0 + ds1;
            const uint32_t both = pack_bf16(ds0, ds1);
            pk[jj / 2] = wmul[tl] != 0.f ? both : 0u;  // content term only inside the window
          }
          tmem_st16(s_addr + 16 * half, pk);  // dS_w over this thread's consumed S columns
        }
        tmem_st_wait();
      } else {
        float a[TPW], w0[TPW], w1[TPW];
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl) {
          a[tl] = ex2(offs[tl]);  // 0 where the time step is not visible
          a_sum += a[tl];
          w0[tl] = 0.f;
          w1[tl] = 0.f;
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t dp[32];
          tmem_ld32(lane_base + kQS + 128 * (s & 1) + 64 * wg + 32 * half, dp);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; jj += 2) {
            const int lc = 32 * half + jj, tl = lc / CP, k = lc % NCH;
            const float d0 = __uint_as_float(dp[jj]), d1 = __uint_as_float(dp[jj + 1]);
            dcb_acc[k] = fmaf(a[tl], d0, dcb_acc[k]);
            dcb_acc[k + 1] = fmaf(a[tl], d1, dcb_acc[k + 1]);
            w0[tl] = fmaf(bcf[k], d0, w0[tl]);
            w1[tl] = fmaf(bcf[k + 1], d1, w1[tl]);
          }
        }
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl) dtb_acc[tl] = a[tl] * (w0[tl] + w1[tl] - delta_i * bc_sum);
        if (s == n_light - 1) {
          // transition: scale the light phase's inner sums, then fetch the scores the dense tiles need
          // (before the report below lets the first dense dP product overwrite where they wait)
#pragma unroll
          for (int k = 0; k < NCH; ++k) dcb_acc[k] = bcf[k] * (dcb_acc[k] - delta_i * a_sum);
          load_cbl();
        }
      }
      tc_fence_before();
      mbar_arrive(&bars[kBarDsFull + (s & 1)]);
      // row sums per key time step; both warpgroups may own part of a time step (CP = 128)
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) {
        if (valid[tl]) {
          if constexpr (TBS) {
            const int sl = slot[tl];
            *reinterpret_cast<__nv_bfloat16*>(s_tbt_main + (sl >> 6) * HALF + row * 128 +
                                              ((((sl & 63) >> 3) ^ (row & 7)) << 4) + (sl & 7) * 2) =
                __float2bfloat16_rn(dtb_acc[tl]);
          } else {
            atomicAdd(&p.dtb[((int64_t)bh * T + slot[tl]) * N + n_loc], dtb_acc[tl]);
          }
        }
      }
    }
    // ------------------------------- epilogue ---------------------------------
    if (ok) ok = warp_wait(&bars[kBarAllDone], 0, p.status, 134);
    // du = sum over rows of dq's content part (`attentions/attn.py:1305-1306`: q + q_bias feeds the content
    // term only): column sums of the accumulator before the relative terms are added to it
    // (32 rows of a warp are summed with a shuffle butterfly that halves the values per lane each round and
    // leaves column c0 + lane in lane `lane`; the four warps of a warpgroup meet in shared memory)
    float* cs = reinterpret_cast<float*>(ring);  // [2 wg][4 warps][DW]
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < DW; c0 += 32) {
        uint32_t raw[32];
        tmem_ld32(lane_base + kQDQ + wg * DW + c0, raw);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = row_valid ? __uint_as_float(raw[e]) : 0.f;
#pragma unroll
        for (int step = 16; step >= 1; step >>= 1) {
          const bool upper = (lane & step) != 0;
#pragma unroll
          for (int j = 0; j < step; ++j) {
            const float keep = upper ? v[j + step] : v[j];
            const float send = upper ? v[j] : v[j + step];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, step);
          }
        }
        cs[(wg * 4 + (warp & 3)) * DW + c0 + lane] = v[0];
      }
    }
    softmax_bar();
    if (row < DW) {  // fixed summation order: deterministic
      const float* c4 = cs + wg * 4 * DW + row;
      p.cs_dq[(size_t)cta_slot * D + wg * DW + row] = (c4[0] + c4[DW]) + (c4[2 * DW] + c4[3 * DW]);
    }
    softmax_bar();
    // channel-score gradient: from key-channel slots to |c_i - c_k| slots, through shared memory
    float* sc = reinterpret_cast<float*>(ring);  // [128][CP]; every TMA load has been consumed by now
    if (CP == 128 || wg == 0) {
#pragma unroll
      for (int k = 0; k < NCH; ++k) sc[row * CP + ((ck_base + k + 2 * row) & (CP - 1))] = dcb_acc[k];
    }
    softmax_bar();
    if (CP < 128 && wg == 1) {  // both warpgroups hold sums for the same channel slots (different time steps)
#pragma unroll
      for (int k = 0; k < NCH; ++k) sc[row * CP + ((k + 2 * row) & (CP - 1))] += dcb_acc[k];
    }
    softmax_bar();
    // dCB[i, j], j = C-1-e, e = |c_i - c_k|, as bf16 pairs: into TMEM columns kQDP + j/2 (A operand of
    // dQ += dCB r_chan) and into a shared-memory tile [row][j] (A operand, transposed, of the dr_chan product).
    // Each warpgroup takes half of the slots.
    uint8_t* s_cbt = D == 128 ? sDO : ring + 98304;  // dO is dead by now; at head_dim 64 the ring has room
    if (ok) {
      const int jb = wg * (CP / 2);
      constexpr int G = CP / 4 < 8 ? CP / 4 : 8;  // packed pairs per TMEM store (CP = 32 has 8 per warpgroup)
#pragma unroll 1
      for (int m0 = 0; m0 < CP / 4; m0 += G) {
        uint32_t pkv[8];
#pragma unroll
        for (int mi = 0; mi < G; ++mi) {
          const int m = m0 + mi;
          float vv[2];
#pragma unroll
          for (int t2 = 0; t2 < 2; ++t2) {
            const int j = jb + 2 * m + t2, e = C - 1 - j;
            // both candidates are read from wrapped (always valid) positions and masked: no divergence
            const float lo = sc[row * CP + ((c_i - e + 2 * row) & (CP - 1))];
            const float hi = sc[row * CP + ((c_i + e + 2 * row) & (CP - 1))];
            const bool on = row_valid && e >= 0;
            vv[t2] = ((on && c_i - e >= 0) ? lo : 0.f) + ((on && e > 0 && c_i + e < C) ? hi : 0.f);
          }
          pkv[mi] = pack_bf16(vv[0], vv[1]);
          const int j = jb + 2 * m;
          *reinterpret_cast<uint32_t*>(s_cbt + (j >> 6) * HALF + row * 128 + ((((j & 63) >> 3) ^ (row & 7)) << 4) +
                                       (j & 7) * 2) = pkv[mi];
        }
#pragma unroll
        for (int mi = G; mi < 8; ++mi) pkv[mi] = 0u;
        tmem_st8(lane_base + kQDP + jb / 2 + m0, pkv);
      }
    }
    if constexpr (!TBS) __threadfence();  // this CTA's atomic row sums in dtb are complete before anyone re-reads them
    softmax_bar();
    if (ok) {
      // dTB of the row (this thread's 64 of the 128 r_time rows) as bf16 pairs: A operand of dQ += dTB r_time
      // in TMEM, and the [row][j] tile in shared memory for the dr_time product
      if constexpr (TBS) {
        const uint8_t* my = s_tbt_main + wg * HALF + row * 128;
#pragma unroll
        for (int m8 = 0; m8 < 32; m8 += 8) {
          const uint4 w0 = *reinterpret_cast<const uint4*>(my + (((m8 / 4) ^ (row & 7)) << 4));
          const uint4 w1 = *reinterpret_cast<const uint4*>(my + (((m8 / 4 + 1) ^ (row & 7)) << 4));
          const uint32_t pk[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          tmem_st8(lane_base + kQS + 32 * wg + m8, pk);
        }
      } else {
        const float* src = p.dtb + ((int64_t)bh * T + 64 * wg) * N + (row_valid ? n_loc : 0);
        const float keep = row_valid ? 1.f : 0.f;
        uint8_t* s_tbt = ring + wg * HALF + row * 128;  // (the scatter area is dead)
        float a[64];  // every load in flight at once
#pragma unroll
        for (int jl = 0; jl < 64; ++jl) a[jl] = (64 * wg + jl < T) ? __ldcg(src + (int64_t)jl * N) : 0.f;
#pragma unroll
        for (int m8 = 0; m8 < 32; m8 += 8) {
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) pk[e] = pack_bf16(a[2 * (m8 + e)] * keep, a[2 * (m8 + e) + 1] * keep);
          tmem_st8(lane_base + kQS + 32 * wg + m8, pk);
          const int c0 = m8 / 4;  // 16-byte chunks c0 and c0 + 1 of this row's 128 bytes
          *reinterpret_cast<uint4*>(s_tbt + (((c0) ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(s_tbt + (((c0 + 1) ^ (row & 7)) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
      // a [16 x 128] tile of ones (K-major): column sums of dTB / dCB come out of the tensor core too
      *reinterpret_cast<uint4*>(ring + 32768 + tid * 16) = make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
      fence_proxy_async_smem();
      tmem_st_wait();
    }
    tc_fence_before();
    mbar_arrive(&bars[kBarFinFull]);
    if (ok) ok = warp_wait(&bars[kBarFinDone], 0, p.status, 135);
    uint8_t* s_out = ring + 65536;  // dq tile as bf16, laid out like a Q tile (the relative keys are dead)
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < DW; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + kQDQ + wg * DW + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w[e] = pack_bf16(__uint_as_float(v[q4 * 8 + 2 * e]), __uint_as_float(v[q4 * 8 + 2 * e + 1]));
          const int col = wg * DW + c0 + q4 * 8, hh = col / 64, c = (col % 64) / 8;
          *reinterpret_cast<uint4*>(s_out + hh * HALF + row * 128 + ((c ^ (row & 7)) << 4)) =
              make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async_smem();
    }
    softmax_bar();
    if (ok && tid == 0) {
#pragma unroll
      for (int hh = 0; hh < NH; ++hh) tma_store_5d(&maps.dq, s_out + hh * HALF, hh * 64, 0, I * TPB, h, b);
      tma_store_commit();
      tma_store_wait_all();
    }
    // relative-key gradient partials: lane = slot j now; added to the per-kv-head accumulators
    if (ok) ok = warp_wait(&bars[kBarRelDone], 0, p.status, 136);
    if (ok) {
      tc_fence_after();
      const int j = row;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const bool jv = which == 0 ? j < T : j < C;
        unsigned long long* acc = p.racc + (((size_t)hk * 2 + which) * D + wg * DW) * 128 + j;
        const uint32_t col = which == 0 ? kQS1 : kQS;
#pragma unroll 1
        for (int c8 = 0; c8 < DW; c8 += 8) {
          uint32_t v[8];
          tmem_ld8(lane_base + col + wg * DW + c8, v);
          tmem_ld_wait();
          if (jv) {
#pragma unroll
            for (int e = 0; e < 8; ++e) fix_add(acc + (size_t)(c8 + e) * 128, __uint_as_float(v[e]));
          }
        }
        if (wg == which) {  // column sums: one warpgroup each
          uint32_t cs1;
          tmem_ld1(lane_base + kQDP + 16 * which, cs1);
          tmem_ld_wait();
          if (jv) fix_add(p.cacc + ((size_t)hk * 2 + which) * 128 + j, __uint_as_float(cs1));
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}


// ---------------------------------------------------------------------------------------------
// Key side: dK, dV.  One CTA owns 128 keys (one key tile) of one (batch, kv head) and visits every
// query tile that can see them, for each of the g query heads of the group; dK and dV stay in
// TMEM for the whole CTA, so nothing is accumulated through global memory (the reference adds
// dK / dV with atomics when g > 1, `attentions/attn.py:752-773`).
//
// Per (query tile, key tile) pair, with thread = query row as everywhere else:
//   S = Q'K^T, dP = dO V^T on tcgen05;  P = exp2(S2 - L), dS = P o (dP - delta) sm_scale in registers;
//   P and dS_w go to shared memory as bf16 in the MN-major operand layout (keys contiguous), and
//   dV += P^T dO,  dK += dS_w^T Q'  (`attentions/attn.py:671-675, 718`) read them as the A operand.
// The per-row quantities of the query tile (Q', gathered channel scores, temporal scores, offsets)
// come from the workspace the query-side kernel filled.  Light pairs need neither S nor dK.
// TMEM columns: [0,128) S, [128,256) dP, [256,256+D) dV, [384,384+D) dK.
struct BkMaps {
  CUtensorMap qp, dout, k, v;
};
struct BkArgs {
  const __half* cblw;
  const __nv_bfloat16* bcw;
  const float *offw, *tbw, *delta;
  __nv_bfloat16 *dk, *dv;
  int64_t dk_sb, dk_sh, dk_sn, dv_sb, dv_sh, dv_sn;
  int B, H, Hkv, T, C, g, window, n_qt;
  int kv_major;  // CTA order: see kv_major_order()
  float c2, sm_scale;
  int* status;
};
enum BkBarrier {
  kKvFull = 0, kQdoFull, kQdoFull1, kBkSdpFull, kPdsFull, kPairDone, kBkAllDone,
  kLdoFull, kLdoFull1, kLdoFull2, kLdoFull3, kLdoFree, kLdoFree1, kLdoFree2, kLdoFree3,  // light pairs: four dO buffers
  kLpFull, kLpFull1, kLFree, kLFree1,                                                      // ... and two P buffers
  kBkBars
};

template <int D>
struct BkCfg {
  static constexpr int TILE = (D / 64) * 16384;
  static constexpr int SMEM_K = 0, SMEM_V = TILE, SMEM_Q = 2 * TILE, SMEM_DO = 3 * TILE;
  static constexpr int SMEM_P = 4 * TILE, SMEM_DS = 4 * TILE + 32768;
  // head_dim 64 has room for a second Q' / dO pair: the loads of the next dense pair and its S / dP
  // products then overlap the softmax work and the dV / dK products of the current one
  static constexpr int NSET = D == 64 ? 2 : 1;
  static constexpr int SMEM_QDO1 = 4 * TILE + 65536;
  static constexpr int SMEM_TAIL = SMEM_QDO1 + (NSET - 1) * 2 * TILE;
  static constexpr int SMEM_BYTES = SMEM_TAIL + kBkBars * 8 + 16 + 1024;
};

template <int D, int CP>
__global__ void __launch_bounds__(kThreads, 1)
tc_bwd_kv_kernel(const __grid_constant__ BkMaps maps, const BkArgs p) {
  using C_ = BkCfg<D>;
  constexpr int NH = D / 64, HALF = 16384, TILE = C_::TILE;
  constexpr int TPB = 128 / CP;
  constexpr int TPW = TPB >= 2 ? TPB / 2 : 1;
  constexpr int NCH = CP < 64 ? CP : 64;
  constexpr int KSTEPS = D / 16;
  constexpr int DW = D / 2;
  constexpr uint32_t kColDV = 256, kColDK = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + C_::SMEM_K;
  uint8_t* sV = smem + C_::SMEM_V;
  uint8_t* sQ = smem + C_::SMEM_Q;
  uint8_t* sDO = smem + C_::SMEM_DO;
  constexpr int NSET = C_::NSET;
  uint8_t* sQ1 = smem + C_::SMEM_QDO1;  // second set (head_dim 64 only)
  uint8_t* sDO1 = sQ1 + TILE;
  uint8_t* sP = smem + C_::SMEM_P;
  uint8_t* sDS = smem + C_::SMEM_DS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C_::SMEM_TAIL);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBkBars);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int BK = p.B * p.Hkv;
  // earliest key tiles (seen by the most query tiles) first, over all kv heads or inside one
  const int J = p.kv_major ? (int)(blockIdx.x % p.n_qt) : (int)(blockIdx.x / BK);
  const int bk = p.kv_major ? (int)(blockIdx.x / p.n_qt) : (int)(blockIdx.x % BK);
  const int b = bk / p.Hkv, hk = bk % p.Hkv;
  const int n_i = p.n_qt - J;            // query tiles J .. n_qt-1
  const int T = p.T, C = p.C;
  // Query tile i is "light" for this key tile when every pair lies outside the content window:
  //   (i - J) TPB - (TPB - 1) > window, except the last tile (its row t = T-1 sees everything).
  // Dense pairs of all g heads come first, then the light ones: a light pair needs neither S, dP, dS nor
  // dK (the content term is zero there), only dV += P^T dO with P = a[t_k] bc[c_k], so the light phase
  // runs with two dO / P buffers (the Q' and dS areas are idle then) and is bound by its MMAs.
  const int dl = p.window > 0 ? (p.window + TPB - 1) / TPB + 1 : n_i;  // first light offset i - J
  const int n_lead = min(dl, n_i);                                      // dense tiles J .. J+n_lead-1
  const int n_dense_i = n_lead + ((p.window > 0 && n_i > dl) ? 1 : 0);  // ... plus the last tile
  const int n_light_i = n_i - n_dense_i;
  const int n_dense = p.g * n_dense_i, n_light = p.g * n_light_i;
  auto dense_pair = [&](int s, int& h, int& i) {
    h = hk * p.g + s / n_dense_i;
    const int e = s % n_dense_i;
    i = e < n_lead ? J + e : p.n_qt - 1;
  };
  auto light_pair = [&](int l, int& h, int& i) {
    h = hk * p.g + l / n_light_i;
    i = J + dl + l % n_light_i;
  };

  // One barrier at entry: thread 0 initialises the mbarriers, another warp fetches the status word (an
  // earlier CTA may have given up), warp 9 allocates the tensor memory - all at the same time.
  if (tid == 0) {
    mbar_init(&bars[kKvFull], 1);
    mbar_init(&bars[kQdoFull], 1);
    mbar_init(&bars[kQdoFull + 1], 1);
    mbar_init(&bars[kBkSdpFull], 1);
    mbar_init(&bars[kPdsFull], kSoftmaxThreads);
    mbar_init(&bars[kPairDone], 1);
    mbar_init(&bars[kBkAllDone], 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars[kLdoFull + i], 1);
      mbar_init(&bars[kLdoFree + i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[kLpFull + i], kSoftmaxThreads);
      mbar_init(&bars[kLFree + i], 1);
    }
    mbar_fence_init();
  } else if (tid == 64) {
    *s_abort = *p.status;
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (*s_abort != 0) {  // do nothing, but give the columns back
    if (warp == 9) tmem_dealloc(tmem, kTmemCols);
    return;
  }

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 8) {
    if (lane == 0) {  // ---- TMA producer ----
      prefetch_tensormap(&maps.qp);
      prefetch_tensormap(&maps.dout);
      mbar_arrive_expect_tx(&bars[kKvFull], 2 * TILE);
      for (int hh = 0; hh < NH; ++hh) {
        tma_load_5d(sK + hh * HALF, &maps.k, &bars[kKvFull], hh * 64, 0, J * TPB, hk, b);
        tma_load_5d(sV + hh * HALF, &maps.v, &bars[kKvFull], hh * 64, 0, J * TPB, hk, b);
      }
      bool ok = true;
      for (int s = 0; ok && s < n_dense; ++s) {
        int h, i;
        dense_pair(s, h, i);
        const int set = s % NSET;
        if (s >= NSET) ok = mbar_wait(&bars[kPairDone], (s - NSET) & 1, p.status, 210);  // the set's buffers are free
        if (!ok) break;
        uint8_t* dq_ = set == 0 ? sQ : sQ1;
        uint8_t* ddo_ = set == 0 ? sDO : sDO1;
        mbar_arrive_expect_tx(&bars[kQdoFull + set], 2 * TILE);
        for (int hh = 0; hh < NH; ++hh) {
          tma_load_5d(dq_ + hh * HALF, &maps.qp, &bars[kQdoFull + set], hh * 64, 0, i * TPB, h, b);
          tma_load_5d(ddo_ + hh * HALF, &maps.dout, &bars[kQdoFull + set], hh * 64, 0, i * TPB, h, b);
        }
      }
      // light pairs: dO only, alternately into the dO and the (now idle) Q' area
      // (a parity wait can only tell the current phase from the one before it: the phases are waited for
      // one by one, none skipped)
      if (ok && n_light > 0 && NSET == 2 && n_dense >= 2)
        ok = mbar_wait(&bars[kPairDone], (n_dense - 2) & 1, p.status, 211);
      if (ok && n_light > 0) ok = mbar_wait(&bars[kPairDone], (n_dense - 1) & 1, p.status, 211);
      // Four dO buffers in the light phase: the dO, Q', K and V areas (K and V are dead once the dense pairs
      // are done).  The loads run far enough ahead to cover the TMA latency.
      for (int l = 0; ok && l < n_light; ++l) {
        int h, i;
        light_pair(l, h, i);
        const int bsel = l & 3;
        if (l >= 4) ok = mbar_wait(&bars[kLdoFree + bsel], ((l >> 2) - 1) & 1, p.status, 212);
        if (!ok) break;
        uint8_t* dst = bsel == 0 ? sDO : bsel == 1 ? sQ : bsel == 2 ? sK : sV;
        mbar_arrive_expect_tx(&bars[kLdoFull + bsel], TILE);
        for (int hh = 0; hh < NH; ++hh)
          tma_load_5d(dst + hh * HALF, &maps.dout, &bars[kLdoFull + bsel], hh * 64, 0, i * TPB, h, b);
      }
    }
  } else if (warp == 9) {
    {  // ---- MMA issuer: the whole warp, in convergent code; the tcgen05 instructions are guarded by the elected lane ----
      constexpr uint32_t kFull = 0xffffffffu;
      const uint32_t el = elect_one();
      const uint32_t tm = __shfl_sync(kFull, tmem, 0);
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_g = make_idesc_bf16_ab(128, D, 1, 1);  // A = P^T / dS^T (MN-major), B MN-major
      const DescHalves dqk = make_desc_halves_sw128(smem_u32(sQ), 16, 1024);
      const DescHalves ddok = make_desc_halves_sw128(smem_u32(sDO), 16, 1024);
      const DescHalves dk = make_desc_halves_sw128(smem_u32(sK), 16, 1024);
      const DescHalves dv = make_desc_halves_sw128(smem_u32(sV), 16, 1024);
      const DescHalves dqm = make_desc_halves_sw128(smem_u32(sQ), HALF, 1024);    // MN-major views
      const DescHalves ddom = make_desc_halves_sw128(smem_u32(sDO), HALF, 1024);
      const DescHalves dpm = make_desc_halves_sw128(smem_u32(sP), HALF, 1024);
      const DescHalves ddsm = make_desc_halves_sw128(smem_u32(sDS), HALF, 1024);
      bool ok = __all_sync(kFull, mbar_wait(&bars[kKvFull], 0, p.status, 220));
      const uint32_t set1 = (uint32_t)(C_::SMEM_QDO1 - C_::SMEM_Q) >> 4;  // descriptor distance to the second set
      auto issue_sdp = [&](int s) {  // S = Q' K^T, dP = dO V^T of dense pair s
        const int set = s % NSET;
        ok = __all_sync(kFull, mbar_wait(&bars[kQdoFull + set], (s / NSET) & 1, p.status, 221));
        if (!ok) return;
        tc_fence_after();
        DescHalves a_q = dqk, a_do = ddok;
        a_q.lo += set * set1;
        a_do.lo += set * set1;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          mma_ss_w(el, tm + kColS, a_q, off, dk, off, idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          mma_ss_w(el, tm + kColDP, a_do, off, dv, off, idesc_s, kk > 0);
        }
        mma_commit_w(el, smem_u32(&bars[kBkSdpFull]));
      };
      if (ok && n_dense > 0) issue_sdp(0);
      for (int s = 0; ok && s < n_dense; ++s) {
        const int set = s % NSET;
        ok = __all_sync(kFull, mbar_wait(&bars[kPdsFull], s & 1, p.status, 222));  // P / dS_w are in shared memory, S / dP consumed
        if (!ok) break;
        tc_fence_after();
        // with a second buffer set the next pair's S / dP go first: the softmax warps wait for them
        if (NSET == 2 && s + 1 < n_dense) issue_sdp(s + 1);
        if (!ok) break;
        DescHalves b_do = ddom, b_q = dqm;
        b_do.lo += set * set1;
        b_q.lo += set * set1;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // dV += P^T dO   (K = 128 query rows, 16 per step)
          mma_ss_w(el, tm + kColDV, dpm, kk * 2048, b_do, kk * 2048, idesc_g, (s > 0 || kk > 0));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // dK += dS_w^T Q'
          mma_ss_w(el, tm + kColDK, ddsm, kk * 2048, b_q, kk * 2048, idesc_g, (s > 0 || kk > 0));
        mma_commit_w(el, smem_u32(&bars[kPairDone]));
        if (NSET == 1 && s + 1 < n_dense) issue_sdp(s + 1);
      }
      const DescHalves dkm = make_desc_halves_sw128(smem_u32(sK), HALF, 1024);  // K / V areas as dO buffers
      const DescHalves dvm = make_desc_halves_sw128(smem_u32(sV), HALF, 1024);
      for (int l = 0; ok && l < n_light; ++l) {  // dV += P^T dO
        const int bsel = l & 1, dsel = l & 3;
        ok = __all_sync(kFull, mbar_wait(&bars[kLdoFull + dsel], (l >> 2) & 1, p.status, 223));
        if (ok) ok = __all_sync(kFull, mbar_wait(&bars[kLpFull + bsel], (l >> 1) & 1, p.status, 224));
        if (!ok) break;
        tc_fence_after();
        const DescHalves ap = bsel == 0 ? dpm : ddsm;   // P buffers: the P and the dS areas
        const DescHalves bd = dsel == 0 ? ddom : dsel == 1 ? dqm : dsel == 2 ? dkm : dvm;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss_w(el, tm + kColDV, ap, kk * 2048, bd, kk * 2048, idesc_g, 1u);
        mma_commit_w(el, smem_u32(&bars[kLFree + bsel]));
        mma_commit_w(el, smem_u32(&bars[kLdoFree + dsel]));
      }
      mma_commit_w(el, smem_u32(&bars[kBkAllDone]));
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int row = tid & 127;
    const int wg = tid >> 7;
    const int ti_loc = row / CP, c_i = row % CP;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int tt_base = (64 * wg) / CP;
    const int ck_base = CP == 128 ? 64 * wg : 0;
    bool ok = true;
    for (int s = 0; ok && s < n_dense; ++s) {
      int h, i;
      dense_pair(s, h, i);
      const int ti_abs = i * TPB + ti_loc;
      const bool row_valid = c_i < C && ti_abs < T;
      const int N = T * C, n_loc = ti_abs * C + c_i;
      const int64_t bhq = (int64_t)b * p.H + h, n_row = bhq * N + n_loc;
      // per-row quantities of this query tile, from the query-side kernel's workspace
      __half2 cbl[NCH / 2];
      float off_row = -INFINITY, delta_i = 0.f;
      if (row_valid) {
        const uint4* src = reinterpret_cast<const uint4*>(p.cblw) + (bhq * (CP / 8) + ck_base / 8) * N + n_loc;
#pragma unroll
        for (int m = 0; m < NCH / 8; ++m) {
          const uint4 w = src[(int64_t)m * N];
          *reinterpret_cast<uint32_t*>(&cbl[4 * m]) = w.x;
          *reinterpret_cast<uint32_t*>(&cbl[4 * m + 1]) = w.y;
          *reinterpret_cast<uint32_t*>(&cbl[4 * m + 2]) = w.z;
          *reinterpret_cast<uint32_t*>(&cbl[4 * m + 3]) = w.w;
        }
        off_row = p.offw[n_row];
        delta_i = p.delta[n_row];
      } else {
#pragma unroll
        for (int k2 = 0; k2 < NCH / 2; ++k2) cbl[k2] = __floats2half2_rn(0.f, 0.f);
      }
      float offs[TPW], wmul[TPW], scw[TPW];
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) {
        const int tk_abs = J * TPB + tt_base + tl, dt = ti_abs - tk_abs;
        const bool valid = dt >= 0 && tk_abs < T && row_valid;
        wmul[tl] = (p.window > 0 && dt > p.window && ti_abs != T - 1) ? 0.f : 1.f;
        scw[tl] = wmul[tl] * p.sm_scale;  // dS_w = P (dP - delta) sm_scale inside the window, 0 outside
        offs[tl] = valid ? p.tbw[(bhq * T + (T - 1 - dt)) * N + n_loc] + off_row : -INFINITY;
      }
      ok = warp_wait(&bars[kBkSdpFull], s & 1, p.status, 232);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32], dp[32];
        tmem_ld32(lane_base + kColS + 64 * wg + 32 * half, sv);
        tmem_ld32(lane_base + kColDP + 64 * wg + 32 * half, dp);
        tmem_ld_wait();
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int jj = 0; jj < 32; jj += 2) {
          const int lc = 32 * half + jj, tl = lc / CP, k = lc % NCH;
          const float2 cb = __half22float2(cbl[k / 2]);
          const float s0 = fmaf(__uint_as_float(sv[jj]), wmul[tl], cb.x);
          const float s1 = fmaf(__uint_as_float(sv[jj + 1]), wmul[tl], cb.y);
          const float p0 = ex2(s0 + offs[tl]), p1 = ex2(s1 + offs[tl]);
          const float ds0 = p0 * (__uint_as_float(dp[jj]) - delta_i) * scw[tl];
          const float ds1 = p1 * (__uint_as_float(dp[jj + 1]) - delta_i) * scw[tl];
          pp[jj / 2] = pack_bf16(p0, p1);
          pd[jj / 2] = pack_bf16(ds0, ds1);
        }
        // (with two buffer sets these warps run ahead of the previous pair's dV / dK products, which
        // still read the P / dS areas)
        if (NSET == 2 && half == 0 && s > 0) {
          ok = warp_wait(&bars[kPairDone], (s - 1) & 1, p.status, 233);
          if (!ok) break;
        }
        // MN-major operand layout: 64-key block = this warpgroup, one 128-byte row per query row,
        // 16-byte chunks swizzled by (row mod 8)
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int c = 4 * half + c4;
          const uint32_t o = wg * HALF + row * 128 + ((c ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(sP + o) = make_uint4(pp[4 * c4], pp[4 * c4 + 1], pp[4 * c4 + 2], pp[4 * c4 + 3]);
          *reinterpret_cast<uint4*>(sDS + o) = make_uint4(pd[4 * c4], pd[4 * c4 + 1], pd[4 * c4 + 2], pd[4 * c4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars[kPdsFull]);
    }
    // ---- light pairs: P[i, k] = a_i[t_k] bc_i[c_k] straight into the operand layout ----
    // The row's data of pair l+1 is requested while pair l is processed: with nothing else to wait for,
    // the latency of these loads would otherwise be the whole cost of a light pair.
    if (ok && n_light > 0) ok = warp_wait(&bars[kPairDone], (n_dense - 1) & 1, p.status, 235);  // P / dS areas are free
    // Two register stages: the row's data of pair l+2 is requested while pair l is processed (one pair
    // ahead does not cover the latency of these loads once a pair takes about a thousand cycles).
    struct RowData {
      uint4 bc[NCH / 8];
      float tb[TPW];
      float off;
    };
    // (head, query tile) of a light pair advance as running cursors: no integer division in the loop
    struct Cursor {
      int h, i;
    };
    auto advance = [&](Cursor& c, int by) {
      c.i += by;
      while (c.i >= J + dl + n_light_i) {
        c.i -= n_light_i;
        ++c.h;
      }
    };
    auto light_fetch = [&](Cursor c, RowData& r) {
      const int h = c.h, i = c.i;
      const int ti_abs = i * TPB + ti_loc;
      const bool row_valid = c_i < C && ti_abs < T;
      const int N = T * C, n_loc = row_valid ? ti_abs * C + c_i : 0;
      const int64_t bhq = (int64_t)b * p.H + h;
      const uint4* src = reinterpret_cast<const uint4*>(p.bcw) + (bhq * (CP / 8) + ck_base / 8) * N + n_loc;
#pragma unroll
      for (int m = 0; m < NCH / 8; ++m) r.bc[m] = src[(int64_t)m * N];
      r.off = p.offw[bhq * N + n_loc];
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) {
        const int dt = min(max(ti_abs - (J * TPB + tt_base + tl), 0), T - 1);
        r.tb[tl] = p.tbw[(bhq * T + (T - 1 - dt)) * N + n_loc];
      }
    };
    Cursor cur{hk * p.g, J + dl}, nxt{hk * p.g, J + dl};  // pair l, pair l + 2 (the one to fetch)
    auto light_body = [&](int l, RowData& r) {
      const int i = cur.i;
      advance(cur, 1);
      const int bsel = l & 1;
      const int ti_abs = i * TPB + ti_loc;
      const bool row_valid = c_i < C && ti_abs < T;
      uint32_t bcr[NCH / 2];  // exp2(channel score - max) of the row, bf16 pairs
      uint32_t a2[TPW];
#pragma unroll
      for (int m = 0; m < NCH / 8; ++m) {
        bcr[4 * m] = r.bc[m].x; bcr[4 * m + 1] = r.bc[m].y; bcr[4 * m + 2] = r.bc[m].z; bcr[4 * m + 3] = r.bc[m].w;
      }
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) {
        const int tk_abs = J * TPB + tt_base + tl;  // (t_i - t_k > window > 0 here)
        const float a = (row_valid && tk_abs < T) ? ex2(r.tb[tl] + r.off) : 0.f;
        a2[tl] = pack_bf16(a, a);
      }
      if (l + 2 < n_light) {  // this stage's registers are free again
        light_fetch(nxt, r);
        advance(nxt, 1);
      }
      if (l >= 2) {
        ok = warp_wait(&bars[kLFree + bsel], ((l >> 1) - 1) & 1, p.status, 236);
        if (!ok) return;
      }
      uint8_t* dstP = bsel == 0 ? sP : sDS;
#pragma unroll
      for (int c = 0; c < 8; ++c) {  // 16-byte chunk c = key columns 8c .. 8c+7 of this warpgroup's 64
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int lc = 8 * c + 2 * e, tl = lc / CP, k = lc % NCH;
          w[e] = mul_bf16x2(a2[tl], bcr[k / 2]);
        }
        *reinterpret_cast<uint4*>(dstP + wg * HALF + row * 128 + ((c ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&bars[kLpFull + bsel]);
    };
    RowData r0, r1;
    if (ok && n_light > 0) {
      light_fetch(nxt, r0);
      advance(nxt, 1);
    }
    if (ok && n_light > 1) {
      light_fetch(nxt, r1);
      advance(nxt, 1);
    }
    for (int l = 0; ok && l < n_light; l += 2) {
      light_body(l, r0);
      if (ok && l + 1 < n_light) light_body(l + 1, r1);
    }
    // ---- epilogue: lane = key row now ----
    if (ok) ok = warp_wait(&bars[kBkAllDone], 0, p.status, 234);
    if (ok) {
      tc_fence_after();
      const int tk_abs = J * TPB + ti_loc;
      const bool key_valid = c_i < C && tk_abs < T;
      const int64_t n = (int64_t)tk_abs * C + c_i;
      __nv_bfloat16* dvrow = p.dv + b * p.dv_sb + hk * p.dv_sh + n * p.dv_sn + wg * DW;
      __nv_bfloat16* dkrow = p.dk + b * p.dk_sb + hk * p.dk_sh + n * p.dk_sn + wg * DW;
      const float inv_c2 = 1.f / p.c2;  // Q' carries c2
#pragma unroll
      for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int c0 = 0; c0 < DW; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(lane_base + (which == 0 ? kColDV : kColDK) + wg * DW + c0, v);
          tmem_ld_wait();
          if (key_valid) {
            const float sc = which == 0 ? 1.f : inv_c2;
            __nv_bfloat16* dst = (which == 0 ? dvrow : dkrow) + c0;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w[e] = pack_bf16(__uint_as_float(v[q4 * 8 + 2 * e]) * sc, __uint_as_float(v[q4 * 8 + 2 * e + 1]) * sc);
              *reinterpret_cast<uint4*>(dst + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <int D, int CP>
int launch_kv(const BwdArgs& bw, const BqArgs& q, const void* qp, cudaStream_t s) {
  const Args& a = bw.a;
  constexpr int TPB = 128 / CP;
  const uint64_t es = 2;
  const uint32_t box[5] = {64, (uint32_t)CP, (uint32_t)TPB, 1, 1};
  BkMaps m;
  int rc;
  auto enc5 = [&](CUtensorMap* map, const void* ptr, int heads, int64_t sn, int64_t sh, int64_t sb) {
    const uint64_t dims[5] = {(uint64_t)a.D, (uint64_t)a.C, (uint64_t)a.T, (uint64_t)heads, (uint64_t)a.B};
    const uint64_t str[4] = {(uint64_t)sn * es, (uint64_t)sn * a.C * es, (uint64_t)sh * es, (uint64_t)sb * es};
    return encode_bf16_sw128(map, ptr, 5, dims, str, box);
  };
  if ((rc = enc5(&m.qp, qp, a.H, a.D, (int64_t)a.N * a.D, (int64_t)a.H * a.N * a.D))) return rc;
  if ((rc = enc5(&m.dout, bw.d_o, a.H, bw.do_sn, bw.do_sh, bw.do_sb))) return rc;
  if ((rc = enc5(&m.k, a.k, a.Hkv, a.k_sn, a.k_sh, a.k_sb))) return rc;
  if ((rc = enc5(&m.v, a.v, a.Hkv, a.v_sn, a.v_sh, a.v_sb))) return rc;
  BkArgs t;
  t.cblw = q.cblw; t.bcw = q.bcw; t.offw = q.offw; t.tbw = q.tbw; t.delta = bw.delta;
  t.dk = (__nv_bfloat16*)bw.dk; t.dv = (__nv_bfloat16*)bw.dv;
  t.dk_sb = bw.dk_sb; t.dk_sh = bw.dk_sh; t.dk_sn = bw.dk_sn;
  t.dv_sb = bw.dv_sb; t.dv_sh = bw.dv_sh; t.dv_sn = bw.dv_sn;
  t.B = a.B; t.H = a.H; t.Hkv = a.Hkv; t.T = a.T; t.C = a.C; t.g = a.g; t.window = a.window;
  t.n_qt = q.n_qt; t.c2 = a.c2; t.sm_scale = a.sm_scale; t.status = q.status;
  t.kv_major = kv_major_order(a.B, a.Hkv, a.g, a.N, D);
  constexpr int smem = BkCfg<D>::SMEM_BYTES;
  static_assert(smem <= 232448, "shared memory budget");
  MVPA_CUDA_CHECK(cudaFuncSetAttribute(tc_bwd_kv_kernel<D, CP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const unsigned grid = (unsigned)t.n_qt * a.B * a.Hkv;
  tc_bwd_kv_kernel<D, CP><<<grid, kThreads, smem, s>>>(m, t);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

int make_maps(BqMaps& m, const BwdArgs& bw, int CP, const void* qp) {
  const Args& a = bw.a;
  const int TPB = 128 / CP;
  const uint64_t es = 2;
  const uint32_t box[5] = {64, (uint32_t)CP, (uint32_t)TPB, 1, 1};
  int rc;
  auto enc5 = [&](CUtensorMap* map, const void* ptr, int heads, int64_t sn, int64_t sh, int64_t sb) {
    const uint64_t dims[5] = {(uint64_t)a.D, (uint64_t)a.C, (uint64_t)a.T, (uint64_t)heads, (uint64_t)a.B};
    const uint64_t str[4] = {(uint64_t)sn * es, (uint64_t)sn * a.C * es, (uint64_t)sh * es, (uint64_t)sb * es};
    return encode_bf16_sw128(map, ptr, 5, dims, str, box);
  };
  if ((rc = enc5(&m.q, a.q, a.H, a.q_sn, a.q_sh, a.q_sb))) return rc;
  if ((rc = enc5(&m.dout, bw.d_o, a.H, bw.do_sn, bw.do_sh, bw.do_sb))) return rc;
  if ((rc = enc5(&m.k, a.k, a.Hkv, a.k_sn, a.k_sh, a.k_sb))) return rc;
  if ((rc = enc5(&m.v, a.v, a.Hkv, a.v_sn, a.v_sh, a.v_sb))) return rc;
  if ((rc = enc5(&m.qp, qp, a.H, a.D, (int64_t)a.N * a.D, (int64_t)a.H * a.N * a.D))) return rc;
  if ((rc = enc5(&m.dq, bw.dq, a.H, bw.dq_sn, bw.dq_sh, bw.dq_sb))) return rc;
  {
    const uint64_t dims[3] = {(uint64_t)a.D, (uint64_t)a.T, (uint64_t)a.Hkv};
    const uint64_t str[2] = {(uint64_t)a.D * es, (uint64_t)a.T * a.D * es};
    const uint32_t b3[3] = {64, 128, 1};
    if ((rc = encode_bf16_sw128(&m.rt, a.rt, 3, dims, str, b3))) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)a.D, (uint64_t)a.C, (uint64_t)a.Hkv};
    const uint64_t str[2] = {(uint64_t)a.D * es, (uint64_t)a.C * a.D * es};
    const uint32_t b3[3] = {64, (uint32_t)CP, 1};
    if ((rc = encode_bf16_sw128(&m.rc, a.rc, 3, dims, str, b3))) return rc;
  }
  return MVPA_OK;
}

// du / dvt / dz of one kv head: du = sum of the query tiles' content column sums; dvt = (column sums
// of dTB) r_time, dz = (column sums of dCB) r_chan (`_rel_bias` adds q_btime / q_bchan to every row, so
// their gradients are the row sums of dq's temporal / channel parts).
__global__ void __launch_bounds__(1024) tc_dbias_kernel(const float* __restrict__ cs_dq,
                                                       const unsigned long long* __restrict__ cacc,
                                                       const __nv_bfloat16* __restrict__ rt,
                                                       const __nv_bfloat16* __restrict__ rc, float* __restrict__ du,
                                                       float* __restrict__ dvt, float* __restrict__ dz, int B, int H,
                                                       int g, int T, int C, int D, int n_qt) {
  __shared__ float s_cs[256];
  __shared__ float s_part[3][1024];
  const int hk = blockIdx.x;
  if (threadIdx.x < 256) s_cs[threadIdx.x] = fix_read(cacc[(size_t)hk * 256 + threadIdx.x]);
  __syncthreads();
  const int d = threadIdx.x % D, part = threadIdx.x / D, parts = blockDim.x / D;
  float su = 0.f, st = 0.f, sz = 0.f;
  const int n_items = n_qt * B * g;
#pragma unroll 8
  for (int it = part; it < n_items; it += parts) {  // (independent loads: eight in flight per thread)
    const int tq = it / (B * g), b = (it / g) % B, hh = it % g;
    su += cs_dq[((size_t)tq * B * H + (size_t)b * H + hk * g + hh) * D + d];
  }
  for (int j = part; j < T; j += parts) st += s_cs[j] * __bfloat162float(rt[((size_t)hk * T + j) * D + d]);
  for (int j = part; j < C; j += parts) sz += s_cs[128 + j] * __bfloat162float(rc[((size_t)hk * C + j) * D + d]);
  s_part[0][threadIdx.x] = su;
  s_part[1][threadIdx.x] = st;
  s_part[2][threadIdx.x] = sz;
  __syncthreads();
  if (part == 0) {
    for (int q = 1; q < parts; ++q) {
      su += s_part[0][q * D + d];
      st += s_part[1][q * D + d];
      sz += s_part[2][q * D + d];
    }
    du[hk * D + d] = su;
    dvt[hk * D + d] = st;
    dz[hk * D + d] = sz;
  }
}

// dr_time / dr_chan from the accumulators of the query-side kernel:
//   dr[j, d] = sum_i dX[i, j] (q[i, d] + bias[d]) = R'[j, d] / c2 + colsum[j] (bias[d] - u[d]),   Q' = (q + u) c2.
__global__ void __launch_bounds__(256) tc_drel_final_kernel(const unsigned long long* __restrict__ racc,
                                                            const unsigned long long* __restrict__ cacc,
                                                            const __nv_bfloat16* __restrict__ u,
                                                            const __nv_bfloat16* __restrict__ vt,
                                                            const __nv_bfloat16* __restrict__ z, float* __restrict__ drt,
                                                            float* __restrict__ drc, int T, int C, int D, float inv_c2) {
  const int hk = blockIdx.x, which = blockIdx.y, S = which == 0 ? T : C;
  const unsigned long long* acc = racc + ((size_t)hk * 2 + which) * D * 128;
  const unsigned long long* cs = cacc + ((size_t)hk * 2 + which) * 128;
  const __nv_bfloat16* bias = (which == 0 ? vt : z) + (size_t)hk * D;
  float* out = (which == 0 ? drt : drc) + (size_t)hk * S * D;
  for (int idx = threadIdx.x; idx < S * D; idx += blockDim.x) {
    const int j = idx / D, d = idx % D;
    out[idx] = fix_read(acc[(size_t)d * 128 + j]) * inv_c2 +
               fix_read(cs[j]) * (__bfloat162float(bias[d]) - __bfloat162float(u[(size_t)hk * D + d]));
  }
}

template <int D, int CP>
int launch(const BwdArgs& bw, float* cs_dq, int* status, float* relc, unsigned long long* racc, float* rows_ws,
           cudaStream_t s) {
  const Args& a = bw.a;
  BqMaps maps;
  int rc = make_maps(maps, bw, CP, rows_ws);
  if (rc) return rc;
  BqArgs t;
  t.u = (const __nv_bfloat16*)a.u;
  t.relc = relc; t.lse = a.lse; t.delta = bw.delta;
  t.cs_dq = cs_dq; t.dtb = bw.dtbg;
  t.racc = racc; t.cacc = racc + (size_t)a.Hkv * 2 * D * 128;
  {
    const size_t rows = (size_t)a.B * a.H * a.N;
    t.cblw = reinterpret_cast<__half*>(rows_ws + rows * (D / 2));
    t.bcw = reinterpret_cast<__nv_bfloat16*>(rows_ws + rows * (D / 2) + rows * (CP / 2));
    t.offw = rows_ws + rows * (D / 2) + rows * CP;
    t.tbw = t.offw + ((rows + 3) & ~(size_t)3);
  }
  t.B = a.B; t.H = a.H; t.Hkv = a.Hkv; t.T = a.T; t.C = a.C; t.g = a.g; t.window = a.window;
  constexpr int TPB = 128 / CP;
  t.n_qt = (a.T + TPB - 1) / TPB;
  t.kv_major = kv_major_order(a.B, a.Hkv, a.g, a.N, D);
  t.c2 = a.c2; t.sm_scale = a.sm_scale;
  t.status = status;
  constexpr int smem = Cfg<D>::SMEM_BYTES;
  static_assert(smem <= 232448, "shared memory budget");
  static_assert(Cfg<D>::EARLY >= 2, "the first tile's K and V load while the prologue runs");
  MVPA_CUDA_CHECK(cudaFuncSetAttribute(tc_bwd_q_kernel<D, CP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  MVPA_CUDA_CHECK(cudaMemsetAsync(status, 0, 256, s));
  MVPA_CUDA_CHECK(cudaMemsetAsync(racc, 0, sizeof(unsigned long long) * (size_t)a.Hkv * (2 * D * 128 + 256), s));
  if (!(D == 64 && CP <= 64))  // (the kernel keeps these sums in shared memory otherwise)
    MVPA_CUDA_CHECK(cudaMemsetAsync(bw.dtbg, 0, sizeof(float) * (size_t)a.B * a.H * a.N * a.T, s));
  rel_const_kernel<D><<<a.Hkv, 256, 0, s>>>((const __nv_bfloat16*)a.vt, (const __nv_bfloat16*)a.z,
                                           (const __nv_bfloat16*)a.rt, (const __nv_bfloat16*)a.rc, relc, a.T, a.C, nullptr);
  const unsigned grid = (unsigned)t.n_qt * a.B * a.H;
  tc_bwd_q_kernel<D, CP><<<grid, kThreads, smem, s>>>(maps, t);
  count_launch(2);
  MVPA_CUDA_CHECK(cudaGetLastError());
  return launch_kv<D, CP>(bw, t, rows_ws, s);
}

}  // namespace

bool tc_bwd_q_supported(const Args& a) { return (a.D == 64 || a.D == 128) && a.C <= 128 && a.T <= 128; }

namespace {
// per-CTA column sums of dq's content part: at most one query tile per time step
size_t cs_dq_floats(int B, int H, int T, int D) { return (((size_t)B * H * T * D) + 63) & ~(size_t)63; }
}  // namespace

// where, inside the tensor-core backward's extra workspace, its kernels keep their status word
size_t tc_bwd_status_offset_floats(const mvpa_problem* p) { return cs_dq_floats(p->B, p->H, p->T, p->D); }

// extra fp32 workspace elements of the tensor-core backward
size_t tc_bwd_q_workspace_floats(const mvpa_problem* p) {
  const size_t rows = (size_t)p->B * p->H * p->T * p->C;
  const size_t cp = p->C <= 32 ? 32 : (p->C <= 64 ? 64 : 128);  // channel slots per row (two 16-bit copies)
  // column sums + status + constants + per-row data for the key side (Q' bf16, channel scores fp16
  // padded to 128 slots, offset, temporal scores)
  size_t n = cs_dq_floats(p->B, p->H, p->T, p->D) + 64 + (size_t)p->Hkv * 256 +
             2 * (size_t)p->Hkv * (2 * p->D * 128 + 256) + rows * (p->D / 2) + rows * cp +
             ((rows + 3) & ~(size_t)3) + rows * p->T + 64;
  return n;
}

int tc_bwd_bias(const BwdArgs& bw, float* extra, cudaStream_t s) {
  const Args& a = bw.a;
  const int CP = a.C <= 32 ? 32 : (a.C <= 64 ? 64 : 128), TPB = 128 / CP;
  const unsigned long long* racc =
      reinterpret_cast<const unsigned long long*>(extra + cs_dq_floats(a.B, a.H, a.T, a.D) + 64 + (size_t)a.Hkv * 256);
  const unsigned long long* cacc = racc + (size_t)a.Hkv * 2 * a.D * 128;
  tc_dbias_kernel<<<a.Hkv, 1024, 0, s>>>(extra, cacc, (const __nv_bfloat16*)a.rt, (const __nv_bfloat16*)a.rc, bw.du,
                                       bw.dvt, bw.dz, a.B, a.H, a.g, a.T, a.C, a.D, (a.T + TPB - 1) / TPB);
  tc_drel_final_kernel<<<dim3(a.Hkv, 2), 256, 0, s>>>(racc, cacc, (const __nv_bfloat16*)a.u,
                                                     (const __nv_bfloat16*)a.vt, (const __nv_bfloat16*)a.z, bw.drt,
                                                     bw.drc, a.T, a.C, a.D, 1.f / a.c2);
  count_launch(2);
  MVPA_CUDA_CHECK(cudaGetLastError());
  return MVPA_OK;
}

int tc_bwd_q(const BwdArgs& bw, float* extra, cudaStream_t s) {
  const Args& a = bw.a;
  float* dqc = extra;  // column sums of dq's content part, one row of D per query-side CTA
  int* status = reinterpret_cast<int*>(extra + cs_dq_floats(a.B, a.H, a.T, a.D));
  float* relc = reinterpret_cast<float*>(status) + 64;
  unsigned long long* racc = reinterpret_cast<unsigned long long*>(relc + (size_t)a.Hkv * 256);  // 8-byte aligned
  float* rows_ws = reinterpret_cast<float*>(racc + (size_t)a.Hkv * (2 * a.D * 128 + 256));
  const int CP = a.C <= 32 ? 32 : (a.C <= 64 ? 64 : 128);
  if (a.D == 64) {
    if (CP == 32) return launch<64, 32>(bw, dqc, status, relc, racc, rows_ws, s);
    if (CP == 64) return launch<64, 64>(bw, dqc, status, relc, racc, rows_ws, s);
    return launch<64, 128>(bw, dqc, status, relc, racc, rows_ws, s);
  }
  if (CP == 32) return launch<128, 32>(bw, dqc, status, relc, racc, rows_ws, s);
  if (CP == 64) return launch<128, 64>(bw, dqc, status, relc, racc, rows_ws, s);
  return launch<128, 128>(bw, dqc, status, relc, racc, rows_ws, s);
}

}  // namespace mvpa
