// Flash-MVPA forward for bf16 on sm_100a: TMA-staged tiles, tcgen05 MMAs, TMEM accumulators.
//
// One CTA owns 128 query rows (= TPB whole time steps of CP channel slots, CP = channels padded
// to a power of two) of one (batch, head) and walks the causal key tiles of the same shape.
//
//   warps 0-3, 4-7  two softmax warpgroups.  Thread (row, wg) owns TMEM lane `row` and the key
//            columns [64 wg, 64 wg + 64) of every tile: it adds the temporal and channel
//            relative scores, masks, runs the base-2 online softmax
//            (`attentions/attn.py:309-315`) and writes P (bf16) back into TMEM for the PV
//            product.  O is rescaled only when the running maximum moved by more than 2^8.
//   warp 8   TMA producer (one lane): Q tile, relative keys, then the K/V ring
//   warp 9   MMA issuer: S = Q'K^T and O += P V on tcgen05, plus the two small products that
//            replace the reference's `_rel_bias` matrices (`attentions/attn.py:1305-1314`);
//            allocates / frees TMEM.  The whole warp runs the issue loop in convergent code and
//            the elected lane's predicate guards the tcgen05 instructions themselves.
//
// Key tiles are visited dense-first: the tiles that overlap the content window (and the
// diagonal), then the "light" tiles that lie wholly outside it.  The reference zero-fills the
// content term there (`attentions/attn.py:261-271`) but still computes it; here a light tile
// loads no K, issues no QK^T and computes no exponential per pair: its probabilities are the
// outer product  exp2(tb_i[t_k] - m) x exp2(cb_i[c_k])  of a per-time-step scalar and the row's
// channel vector, formed with packed bf16 multiplies, two tiles per turn; one maximum over the
// temporal scores of all light tiles (and at most one rescale of O) serves the whole phase.
//
// TMEM columns: [0,128) S0 / P0, [128,256) S1 / P1, [256,256+D) O, [384,512) raw temporal
// products TBraw[row][j] = q.r_time[j]  (the bias part vt.r_time[j] is a per-column constant
// kept in shared memory).
#include <cuda_fp16.h>

#include <mutex>

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
constexpr uint32_t kColS = 0;  // + 128 * buf
constexpr uint32_t kColO = 256;
constexpr uint32_t kColTB = 384;
constexpr float kRescaleThreshold = 8.f;  // log2 units: P stays below 2^8

struct TcMaps {
  CUtensorMap q, k, v, rt, rc;
  CUtensorMap o;  // store
};

struct TcArgs {
  const __nv_bfloat16 *u, *vt, *z;
  __nv_bfloat16* o;
  float* lse;
  int64_t o_sb, o_sh, o_sn;
  int B, H, Hkv, T, C, g, window, n_qt;
  int q_t0, q_tn, q_tiles;  // query time range of this call and its number of query tiles
  int kv_major;             // CTA order: see kv_major_order()
  float c2;
  int* status;
  const float* relc;  // (Hkv, 256): vt.r_time[j] at [0,128), z.r_chan[j] at [128,256)
};

enum BarrierIndex {
  kBarProFull = 0, kBarProMma, kBarProDone, kBarXchg,
  kBarSFull,                     // 2
  kBarPFull = kBarSFull + 2,     // 2
  kBarPlFull = kBarPFull + 2,    // 4: P of the light tiles (four buffers, 64 TMEM columns each)
  kBarSlotFull = kBarPlFull + 4,  // NS, then slot_free NS
};

template <int D>
struct Cfg {
  static constexpr int NH = D / 64;            // 64-column (128-byte) halves of a row
  static constexpr int HALF = 16384;           // 128 rows x 128 B
  static constexpr int TILE = NH * HALF;       // one 128 x D bf16 tile = one ring slot
  // K/V ring of NS slots.  A dense tile takes two consecutive slots (K then V), a light tile one (V).
  static constexpr int NS = D == 64 ? 10 : 5;
  static constexpr int PRO_SLOTS = 65536 / TILE;  // slots the prologue borrows (64 KB: sR + sC, then the scratch)
  static constexpr int EARLY = NS - PRO_SLOTS;    // loads that may start before the prologue ends
  static constexpr int SMEM_Q = 0;
  static constexpr int SMEM_RING = TILE;
  static constexpr int SMEM_PRO = SMEM_RING + EARLY * TILE;
  static constexpr int SMEM_TAIL = SMEM_RING + NS * TILE;
  // tail: u/vt/z (3D f32), vR[128], zC[128], smax[2][2][128], lsum[2][128], barriers, tmem slot, abort
  static constexpr int TAIL_FLOATS = 3 * D + 128 + 128 + 512 + 256 + 512;
  static constexpr int TAIL_BYTES = TAIL_FLOATS * 4 + (kBarSlotFull + 2 * NS) * 8 + 16;
  static constexpr int SMEM_BYTES = SMEM_TAIL + TAIL_BYTES + 1024;  // + alignment slack
};

// Bounded wait whose outcome is uniform across the warp (warp-collective TMEM ops follow it).
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, status, code));
}

// All 256 softmax threads.  Only ever called outside data-dependent control flow.
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Packed fp32 arithmetic (two lanes per instruction) and the three-input maximum: the dense tiles'
// softmax is bound by instruction issue next to the exponentials, and these halve its fp32 stream.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)),
        "l"(reinterpret_cast<const uint64_t&>(c)));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for two lanes on the fp32 pipe instead of the special-function unit, which the dense tiles keep
// saturated: round x to the nearest integer n with the 1.5 * 2^23 trick, a cubic for 2^(x - n) on
// [-0.5, 0.5] (relative error 8e-5, well below the bf16 resolution of P), n added into the exponent
// field.  Arguments below -126 (masked scores are -inf) give 2^-126, which vanishes in every sum.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  constexpr float kMagic = 12582912.f;
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 y = fadd2(x, make_float2(kMagic, kMagic));
  const float2 n = fadd2(y, make_float2(-kMagic, -kMagic));
  const float2 r = ffma2(n, make_float2(-1.f, -1.f), x);
  float2 q = ffma2(r, make_float2(0.05519810691f, 0.05519810691f), make_float2(0.24267712235f, 0.24267712235f));
  q = ffma2(q, r, make_float2(0.69326180220f, 0.69326180220f));
  q = ffma2(q, r, make_float2(0.99992275238f, 0.99992275238f));
  return make_float2(__int_as_float(__float_as_int(q.x) + (__float_as_int(y.x) << 23)),
                     __int_as_float(__float_as_int(q.y) + (__float_as_int(y.y) << 23)));
}
// Which column pairs of a 32-column chunk take the polynomial (kPolyOf8 of every 8 pairs) on the
// alternating path, where two warps in their exponentials share one special-function unit: 2 of 8
// measured best (3 of 8 about equal, 4 of 8 slower than none; no gain where the warpgroups split columns).
constexpr int kPolyOf8 = 2;
__device__ __forceinline__ constexpr bool poly_pair(int pair) { return ((pair % 8) * kPolyOf8) % 8 < kPolyOf8; }

__device__ __forceinline__ uint32_t hmul2_bf16(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Number of leading key tiles of query tile I that are "light": every pair outside the content
// window, i.e.  I*TPB - (J*TPB + TPB - 1) > window.  Light-ness is monotone in J.
__device__ __forceinline__ int light_tiles(int I, int TPB, int window, int n_qt) {
  if (window <= 0 || I == n_qt - 1) return 0;  // the last tile holds the row t = T-1 that sees all
  const int x = I * TPB - TPB - window;
  return x < 0 ? 0 : x / TPB + 1;
}

template <int D, int CP>
__global__ void __launch_bounds__(kThreads, 1)
tc_fwd_kernel(const __grid_constant__ TcMaps maps, const TcArgs p) {
  using C_ = Cfg<D>;
  constexpr int NH = C_::NH, HALF = C_::HALF, TILE = C_::TILE, NS = C_::NS;
  constexpr int TPB = 128 / CP;                // time steps per tile
  constexpr int TPW = TPB >= 2 ? TPB / 2 : 1;  // time steps inside one warpgroup's 64 columns
  constexpr int NCH = CP < 64 ? CP : 64;       // distinct channel slots inside those columns
  constexpr int KSTEPS = D / 16;
  constexpr int DW = D / 2;                    // O columns each warpgroup rescales / stores
  // Alternating dense tiles (head_dim 64, at most 64 channel slots): each softmax warpgroup takes every
  // other dense tile with whole rows and its own O accumulator, so the two warps that share a
  // scheduler are in different phases (one in its exponentials, the other loading or reducing)
  // and no barrier is needed inside a tile; the accumulators are merged before the light tiles.
  constexpr bool ALT = (D == 64) && (CP <= 64);
  // Split accumulators (head_dim 64 with 128 channel slots): both warpgroups work on every dense tile, each
  // on its 64 key columns with its OWN running maximum, row sum and O accumulator (O_0 / O_1, 2 x 64 TMEM
  // columns; the PV product of a tile is issued as two groups of four K-steps).  No maximum exchange and no
  // barrier inside a tile; the two accumulators are merged once before the light tiles.  (Measured against
  // the alternating path at 64 and 32 channel slots it is 1-5 % slower there, and 2.6 % faster than the
  // exchange at 128 slots; head_dim 128 has no TMEM columns for a second accumulator.)
  constexpr bool SPLIT = (D == 64) && !ALT;
  // With at most 64 channel slots the prologue's scratch rows are padded instead of rotated, and each
  // thread's columns hold every channel slot (no maximum exchange between the warpgroups).
  constexpr bool PAD = CP <= 64;
  constexpr int LDP = PAD ? CP + 2 : CP;
  static_assert(CP >= 32 && CP <= 128 && (CP & (CP - 1)) == 0, "CP in {32,64,128}");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C_::SMEM_Q;
  uint8_t* ring = smem + C_::SMEM_RING;
  uint8_t* sR = smem + C_::SMEM_PRO;            // r_time rows 0..127 (rows >= T are zero)
  uint8_t* sC = sR + TILE;                      // r_chan rows 0..CP-1
  float* scratch = reinterpret_cast<float*>(smem + C_::SMEM_PRO);  // [128][CP], once sR / sC are dead
  float* s_bias = reinterpret_cast<float*>(smem + C_::SMEM_TAIL);  // u, vt, z as fp32
  float* s_vr = s_bias + 3 * D;                 // vt . r_time[j]
  float* s_zc = s_vr + 128;                     // z  . r_chan[j]
  float* s_max = s_zc + 128;                    // [2 slots][2 wg][128 rows]
  float* s_lsum = s_max + 512;                  // [2 wg][128]
  float* s_merge = s_lsum + 256;                // [m, l][2 wg][128]: accumulator merge of the alternating path
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_merge + 512);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBarSlotFull + 2 * NS);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
  int* s_giveup = s_abort + 1;
  uint64_t* slot_full = bars + kBarSlotFull;
  uint64_t* slot_free = slot_full + NS;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int BH = p.B * p.H;
  int I_loc, bh;  // latest (heaviest) query tiles first, over all heads or inside one kv head
  if (p.kv_major) {
    const int per = p.q_tiles * p.g, grp = (int)(blockIdx.x / per), r = (int)(blockIdx.x % per);
    I_loc = p.q_tiles - 1 - r / p.g;
    bh = grp * p.g + r % p.g;  // grp = b * Hkv + hk
  } else {
    I_loc = p.q_tiles - 1 - (int)(blockIdx.x / BH);
    bh = blockIdx.x % BH;
  }
  const int I = p.q_t0 / TPB + I_loc;                         // tile index in the whole sequence
  const int b = bh / p.H, h = bh % p.H, hk = h / p.g;
  const int n_tiles = I + 1;
  const int n_light = light_tiles(I, TPB, p.window, p.n_qt);
  const int n_dense = n_tiles - n_light;
  // visit order: dense tiles n_light..I, then light tiles 0..n_light-1
  auto tile_of = [&](int s) { return s < n_dense ? n_light + s : s - n_dense; };
  // position of a tile's K / V in the load sequence; slot = q % NS, use count = q / NS
  auto q_of_k = [&](int s) { return 2 * s; };
  auto q_of_v = [&](int s) { return s < n_dense ? 2 * s + 1 : n_dense + s; };
  const int T = p.T, C = p.C;

  // One barrier at entry: thread 0 initialises the mbarriers, another warp fetches the status word (an
  // earlier CTA may have given up), warp 9 allocates the tensor memory - all at the same time.
  if (tid == 0) {
    *s_giveup = 0;
    mbar_init(&bars[kBarProFull], 1);
    mbar_init(&bars[kBarProMma], 1);
    mbar_init(&bars[kBarProDone], kSoftmaxThreads);
    mbar_init(&bars[kBarXchg], kSoftmaxThreads);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[kBarSFull + i], 1);
      mbar_init(&bars[kBarPFull + i], ALT ? kSoftmaxThreads / 2 : kSoftmaxThreads);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&bars[kBarPlFull + i], kSoftmaxThreads);
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
  // Register re-balancing between warpgroups: the producer / MMA warpgroup keeps 40 registers
  // per thread, the two softmax warpgroups grow to 232.
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&maps.q);
      prefetch_tensormap(&maps.k);
      prefetch_tensormap(&maps.v);
      prefetch_tensormap(&maps.rt);
      prefetch_tensormap(&maps.rc);
      mbar_arrive_expect_tx(&bars[kBarProFull], 2 * TILE + NH * CP * 128);
      for (int hh = 0; hh < NH; ++hh) {
        tma_load_5d(sQ + hh * HALF, &maps.q, &bars[kBarProFull], hh * 64, 0, I_loc * TPB, h, b);
        tma_load_3d(sR + hh * HALF, &maps.rt, &bars[kBarProFull], hh * 64, 0, hk);
        tma_load_3d(sC + hh * CP * 128, &maps.rc, &bars[kBarProFull], hh * 64, 0, hk);
      }
      bool ok = true;
      auto load_slot = [&](const CUtensorMap* map, int q, int J) {
        if (q == C_::EARLY) ok = mbar_wait(&bars[kBarProDone], 0, p.status, 10);  // borrowed slots are back
        const int sl = q % NS;
        if (ok && q >= NS) ok = mbar_wait(&slot_free[sl], ((q / NS) - 1) & 1, p.status, 11);
        if (!ok) return;
        uint8_t* dst = ring + sl * TILE;
        mbar_arrive_expect_tx(&slot_full[sl], TILE);
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) tma_load_5d(dst + hh * HALF, map, &slot_full[sl], hh * 64, 0, J * TPB, hk, b);
      };
      for (int s = 0; ok && s < n_tiles; ++s) {
        const int J = tile_of(s);
        if (s < n_dense) load_slot(&maps.k, q_of_k(s), J);
        if (ok) load_slot(&maps.v, q_of_v(s), J);
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp runs this stream in convergent code and only the tcgen05 instructions are
    // guarded by the elected lane: their operands then come straight from warp-uniform registers and
    // the stream issues at the tensor pipe's rate (a single-lane branch costs 80-160 cycles per MMA).
    {
      constexpr uint32_t kFull = 0xffffffffu;
      const uint32_t el = elect_one();
      const uint32_t tm = __shfl_sync(kFull, tmem, 0);
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_c = make_idesc_bf16(128, CP, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 1);
      bool ok = __all_sync(kFull, mbar_wait(&bars[kBarProFull], 0, p.status, 20));
      if (ok) {
        tc_fence_after();
        const DescHalves dq = make_desc_halves_sw128(smem_u32(sQ), 16, 1024);
        const DescHalves dr = make_desc_halves_sw128(smem_u32(sR), 16, 1024);
        const DescHalves dc = make_desc_halves_sw128(smem_u32(sC), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {  // raw temporal products, all 128 columns at once
          const uint32_t off = (kk / 4) * HALF + (kk % 4) * 32;
          mma_ss_w(el, tm + kColTB, dq, off, dr, off, idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {  // raw channel products -> S0 columns [0, CP)
          const uint32_t offa = (kk / 4) * HALF + (kk % 4) * 32;
          const uint32_t offb = (kk / 4) * (CP * 128) + (kk % 4) * 32;
          mma_ss_w(el, tm + kColS, dq, offa, dc, offb, idesc_c, kk > 0);
        }
        mma_commit_w(el, smem_u32(&bars[kBarProMma]));
        ok = __all_sync(kFull, mbar_wait(&bars[kBarProDone], 0, p.status, 21));  // Q rewritten as (q+u) c2; S0 free
      }
      const DescHalves dq = make_desc_halves_sw128(smem_u32(sQ), 16, 1024);
      const DescHalves dk0 = make_desc_halves_sw128(smem_u32(ring), 16, 1024);
      const DescHalves dv0 = make_desc_halves_sw128(smem_u32(ring), HALF, 1024);
      const uint32_t a_full = smem_u32(slot_full), a_free = smem_u32(slot_free);
      const uint32_t a_sfull = smem_u32(&bars[kBarSFull]), a_pfull = smem_u32(&bars[kBarPFull]);
      const uint32_t a_plfull = smem_u32(&bars[kBarPlFull]);
      // ring cursor of the next slot to be consumed (K and V slots are consumed in load order)
      uint32_t k_sl = 0, k_par = 0;  // slot / parity of the next K (dense tiles only)
      auto advance = [&](uint32_t& sl, uint32_t& par, int by) {
        sl += by;
        if (sl >= (uint32_t)NS) { sl -= NS; par ^= 1; }
      };
      auto issue_qk = [&](int s) {  // S_s = Q' K_s^T ; K_s sits in slot (2s) % NS
        ok = __all_sync(kFull, mbar_wait_a(a_full + 8 * k_sl, k_par, p.status, 22));
        if (!ok) return;
        tc_fence_after();
        const uint32_t d_s = tm + kColS + 128 * (s & 1);
        const uint32_t klo = dk0.lo + k_sl * (TILE >> 4);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          const uint32_t off = ((kk / 4) * HALF + (kk % 4) * 32) >> 4;
          DescHalves da = dq, db = dk0;
          da.lo = dq.lo + off;
          db.lo = klo + off;
          mma_ss_w(el, d_s, da, 0, db, 0, idesc_s, kk > 0);
        }
        mma_commit_w(el, a_sfull + 8 * (s & 1));
        mma_commit_w(el, a_free + 8 * k_sl);
        advance(k_sl, k_par, 2);
      };
      if (ok && n_dense > 0) issue_qk(0);
      // The completion of PV_s is signalled on the free-barrier of the V slot it read: the producer
      // waits there to refill the slot, the softmax warps to reuse P columns / rescale O / finish.
      uint32_t v_sl = 1 % NS, v_par = 0;  // slot / parity of V_s (V_0 is load 1)
      auto advance_v = [&](int by) {
        v_sl += by;
        if (v_sl >= (uint32_t)NS) { v_sl -= NS; v_par ^= 1; }
      };
      // ---- dense tiles ----
      for (int s = 0; ok && s < n_dense; ++s) {
        if (s + 1 < n_dense) issue_qk(s + 1);  // S of the next tile first: its softmax is the long pole
        if (ok) ok = __all_sync(kFull, mbar_wait_a(a_full + 8 * v_sl, v_par, p.status, 24));
        if (ok) ok = __all_sync(kFull, mbar_wait_a(a_pfull + 8 * (s & 1), (s >> 1) & 1, p.status, 23));
        if (!ok) break;
        tc_fence_after();
        // P_s: two 32-column halves at the start of each warpgroup's S columns (stride 64)
        const uint32_t a0 = tm + kColS + 128 * (s & 1);
        const uint32_t b_lo = dv0.lo + v_sl * (TILE >> 4);
        const bool dn = s + 1 < n_dense;
        // alternating path: P_s is one contiguous 64-column block, O of even / odd tiles are separate
        const uint32_t d_o = ALT ? tm + kColO + 64 * (s & 1) : tm + kColO;
        const uint32_t acc0 = ALT ? (uint32_t)(s > 1) : (uint32_t)(s > 0);
        mma_ts_x4_w(el, d_o, a0, b_lo, dv0.hi, 2048 >> 4, idesc_o, acc0);
        mma_ts_x4_w(el, SPLIT ? d_o + 64 : d_o, a0 + (ALT ? 32 : 64), b_lo + 4 * (2048 >> 4), dv0.hi, 2048 >> 4, idesc_o,
                    SPLIT ? acc0 : 1u);
        mma_commit_w(el, a_free + 8 * v_sl);
        advance_v(dn ? 2 : 1);  // a dense successor's V is two loads on, a light successor's one
      }
      // ---- light tiles: P in four contiguous 64-column buffers ----
      uint32_t pb = 0, pb_par = 0;
      for (int l = 0; ok && l < n_light; ++l) {
        ok = __all_sync(kFull, mbar_wait_a(a_full + 8 * v_sl, v_par, p.status, 24));
        if (ok) ok = __all_sync(kFull, mbar_wait_a(a_plfull + 8 * pb, pb_par, p.status, 23));
        if (!ok) break;
        tc_fence_after();
        const uint32_t a0 = tm + kColS + 64 * pb;
        const uint32_t b_lo = dv0.lo + v_sl * (TILE >> 4);
        pb = (pb + 1) & 3;
        if (pb == 0) pb_par ^= 1;
        mma_ts_x4_w(el, tm + kColO, a0, b_lo, dv0.hi, 2048 >> 4, idesc_o, 1u);
        mma_ts_x4_w(el, tm + kColO, a0 + 32, b_lo + 4 * (2048 >> 4), dv0.hi, 2048 >> 4, idesc_o, 1u);
        mma_commit_w(el, a_free + 8 * v_sl);
        advance_v(1);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ------------------------------ softmax warps ------------------------------
    const int row = tid & 127;               // query row of the tile == TMEM lane
    const int wg = tid >> 7;                 // column half this thread owns
    const int ti_loc = row / CP, c_i = row % CP;
    const int ti_abs = I * TPB + ti_loc;
    const bool row_valid = c_i < C && ti_abs < p.q_t0 + p.q_tn;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int tt_base = (64 * wg) / CP;      // first tile-local time step of this thread's columns
    const int ck_base = CP == 128 ? 64 * wg : 0;  // first channel slot of this thread's columns
    for (int d = tid; d < D; d += kSoftmaxThreads) s_bias[d] = __bfloat162float(p.u[hk * D + d]);
    s_vr[tid] = p.relc[hk * 256 + tid];  // s_vr and s_zc are adjacent: 256 floats
    softmax_bar();
    bool ok = warp_wait(&bars[kBarProFull], 0, p.status, 30);
    if (ok) ok = warp_wait(&bars[kBarProMma], 0, p.status, 31);
    // (the relative-key tiles sR / sC were only read by the two MMAs: the scratch may overwrite them)
    // Channel scores of the row, c2 (q.r_chan[j] + z.r_chan[j]), parked in shared memory in
    // 32-column chunks (split between the warpgroups) for the per-row gather below.
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int ci = 0; ci < CP / 32; ++ci) {
        if ((ci & 1) == wg) {
          uint32_t v[32];
          tmem_ld32(lane_base + kColS + ci * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 zc = reinterpret_cast<const float4*>(s_zc)[ci * 8 + j4];
            const float zz[4] = {zc.x, zc.y, zc.z, zc.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int jj = j4 * 4 + e;
              const float val = p.c2 * (__uint_as_float(v[jj]) + zz[e]);
              if constexpr (PAD) scratch[row * LDP + ci * 32 + jj] = val;
              else scratch[row * CP + ((ci * 32 + jj + 2 * row) & (CP - 1))] = val;
            }
          }
        }
      }
      tc_fence_before();
    }
    softmax_bar();  // scratch complete; the MMAs no longer need the raw Q tile
    // Gathered by |c_i - c_k| for this thread's columns:
    //   cbf = cb - max (fp32, log2 domain) for dense tiles; the light tiles use bc = exp2(cbf) (bf16x2),
    //   formed when their phase starts (the two never live in registers together).
    float cbf[NCH];
    float mc = 0.f;
    {
      float g[NCH];
      float mx = -INFINITY;
      if (ok) {
        if constexpr (PAD) {
          // slot C-1-|c_i - c_k| runs up through the row for c_k <= c_i and down for c_k > c_i: two base
          // pointers with constant offsets (rows padded by two floats: no bank conflicts on either diagonal;
          // positions of channels that do not exist may lie outside the row, their values are dropped)
          const float* up = scratch + row * LDP + (C - 1 - c_i);
          const float* down = scratch + row * LDP + (C - 1 + c_i);
          const int climit = c_i < C ? C : 0;
#pragma unroll
          for (int k = 0; k < NCH; ++k) {
            const float val = k <= c_i ? up[k] : down[-k];
            g[k] = k < climit ? val : -INFINITY;
            mx = fmaxf(mx, g[k]);
          }
        } else {
#pragma unroll
          for (int k = 0; k < NCH; ++k) {
            const int ck = ck_base + k;
            const int jc = min(max(C - 1 - abs(c_i - ck), 0), CP - 1);
            const float val = scratch[row * CP + ((jc + 2 * row) & (CP - 1))];  // rows rotated: no bank conflicts on the (anti)diagonal
            g[k] = (c_i < C && ck < C) ? val : -INFINITY;
            mx = fmaxf(mx, g[k]);
          }
        }
      }
      if constexpr (!PAD) {  // the row maximum spans both warpgroups' columns when CP = 128
        s_max[wg * 128 + row] = mx;
        softmax_bar();
        mx = fmaxf(mx, s_max[(wg ^ 1) * 128 + row]);
      }
      mc = (mx == -INFINITY) ? 0.f : mx;
      if (!ok) {
#pragma unroll
        for (int k = 0; k < NCH; ++k) cbf[k] = 0.f;
      }
      if (ok) {
#pragma unroll
        for (int k = 0; k < NCH; ++k) cbf[k] = g[k] - mc;
        // Q' = (q+u) c2 in place (`attentions/attn.py:180-183`); each warpgroup converts half of the chunks
        const float4* u4 = reinterpret_cast<const float4*>(s_bias);
#pragma unroll
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
    mbar_arrive(&bars[kBarProDone]);  // borrowed ring stages, S0 and the rewritten Q are ready
    float m_used = -INFINITY, l_sum = 0.f;

    // O and l follow the running maximum only when it moved by more than 2^8.  Needs every PV
    // product issued so far (tiles < s) to be complete; they execute in order, so the last one is
    // enough.  Returns false if the wait ran out.
    auto maybe_rescale = [&](int s, float m_tile) -> bool {
      const bool need = m_tile > m_used + kRescaleThreshold;
      if (!__any_sync(0xffffffffu, need)) return true;
      const int qp = q_of_v(s - 1);
      if (!warp_wait(&slot_free[qp % NS], (qp / NS) & 1, p.status, 33)) return false;
      tc_fence_after();
      const float alpha = need ? ex2(m_used - m_tile) : 1.f;
      // (split accumulators: all D columns of this warpgroup's own O; otherwise its half of the one O)
      constexpr int own0 = SPLIT ? 64 : DW, own_n = SPLIT ? D : DW;
#pragma unroll
      for (int c0 = 0; c0 < own_n; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + kColO + wg * own0 + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) * alpha);
        tmem_st32(lane_base + kColO + wg * own0 + c0, v);
      }
      tmem_st_wait();
      l_sum *= alpha;
      if (need) m_used = m_tile;
      return true;
    };
    // temporal scores of the TPB key time steps of tile J, in log2 units, plus the channel maximum.
    // Issue and use are split so that the TMEM round trip overlaps the barrier waits in between;
    // the values are valid after the next tmem_ld_wait().
    auto tb_issue = [&](int J, uint32_t (&raw)[TPB], int (&colj)[TPB], bool (&valid_all)[TPB]) {
#pragma unroll
      for (int tt = 0; tt < TPB; ++tt) {
        const int tk_abs = J * TPB + tt, dt = ti_abs - tk_abs;
        valid_all[tt] = dt >= 0 && tk_abs < T;
        colj[tt] = T - 1 - min(max(dt, 0), T - 1);
        tmem_ld1(lane_base + kColTB + colj[tt], raw[tt]);
      }
    };
    auto tb_finish = [&](const uint32_t (&raw)[TPB], const int (&colj)[TPB], float (&tb_all)[TPB]) {
#pragma unroll
      for (int tt = 0; tt < TPB; ++tt) tb_all[tt] = p.c2 * (__uint_as_float(raw[tt]) + s_vr[colj[tt]]) + mc;
    };

    // ------------------------------ dense tiles ------------------------------
    // Abort protocol: this loop contains a named barrier, which must never lose a participant.
    // A warp whose bounded wait runs out raises s_giveup, stops touching TMEM, and keeps walking
    // to the next named barrier; there every warp sees the flag and all leave together.
    if constexpr (ALT) {
      const uint32_t s_addr = lane_base + kColS + 128 * wg;  // this warpgroup's tiles use S buffer `wg`
      const uint32_t o_addr = lane_base + kColO + 64 * wg;
      for (int s = wg; ok && s < n_dense; s += 2) {
        const int J = tile_of(s);
        float tb_all[TPB], wmul[TPB];
        bool valid_all[TPB];
        {
          uint32_t tb_raw[TPB];
          int tb_col[TPB];
          tb_issue(J, tb_raw, tb_col, valid_all);
          ok = warp_wait(&bars[kBarSFull + wg], (s >> 1) & 1, p.status, 32);
          tmem_ld_wait();
          if (!ok) break;
          tc_fence_after();
          tb_finish(tb_raw, tb_col, tb_all);
        }
#pragma unroll
        for (int tt = 0; tt < TPB; ++tt) {
          const int dt = ti_abs - (J * TPB + tt);
          wmul[tt] = (p.window > 0 && dt > p.window && ti_abs != T - 1) ? 0.f : 1.f;
        }
        // pass 1: the row's maximum over the tile.  The TMEM load of the next 32 columns is always in
        // flight while the current ones are processed (two register buffers).
        float m_tile = -INFINITY;
        uint32_t va[32], vb[32];
        auto max_chunk = [&](const uint32_t (&v)[32], int c) {
          const int tt = (32 * c) / CP;
          const float2 w2 = make_float2(wmul[tt], wmul[tt]);
          float g0 = -INFINITY, g1 = -INFINITY;
#pragma unroll
          for (int jj = 0; jj < 32; jj += 4) {
            const int k = (32 * c + jj) % CP;
            const float2 t0 = ffma2(make_float2(__uint_as_float(v[jj]), __uint_as_float(v[jj + 1])), w2, make_float2(cbf[k], cbf[k + 1]));
            const float2 t1 = ffma2(make_float2(__uint_as_float(v[jj + 2]), __uint_as_float(v[jj + 3])), w2, make_float2(cbf[k + 2], cbf[k + 3]));
            g0 = fmax3(g0, t0.x, t0.y);
            g1 = fmax3(g1, t1.x, t1.y);
          }
          if (valid_all[tt]) m_tile = fmaxf(m_tile, fmaxf(g0, g1) + tb_all[tt]);
        };
        tmem_ld32(s_addr, va);
        tmem_ld_wait();
        tmem_ld32(s_addr + 32, vb);
        max_chunk(va, 0);
        tmem_ld_wait();
        tmem_ld32(s_addr + 64, va);
        max_chunk(vb, 1);
        tmem_ld_wait();
        tmem_ld32(s_addr + 96, vb);
        max_chunk(va, 2);
        tmem_ld_wait();
        tmem_ld32(s_addr, va);  // first chunk of pass 2
        max_chunk(vb, 3);
        if (s == wg) {
          m_used = (m_tile == -INFINITY) ? 0.f : m_tile;
        } else {
          const bool need = m_tile > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            const int qp = q_of_v(s - 2);  // this accumulator's previous product
            if (!warp_wait(&slot_free[qp % NS], (qp / NS) & 1, p.status, 33)) { ok = false; break; }
            tc_fence_after();
            const float alpha = need ? ex2(m_used - m_tile) : 1.f;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t v[32];
              tmem_ld32(o_addr + c0, v);
              tmem_ld_wait();
#pragma unroll
              for (int jj = 0; jj < 32; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) * alpha);
              tmem_st32(o_addr + c0, v);
            }
            tmem_st_wait();
            l_sum *= alpha;
            if (need) m_used = m_tile;
          }
        }
        // pass 2: P = exp2(S2 - m) as bf16 over the consumed S columns (chunk c lands in columns 16c..16c+15,
        // always behind the columns still to be read)
        float2 psum2 = make_float2(0.f, 0.f);
        auto exp_chunk = [&](const uint32_t (&v)[32], int c) {
          const int tt = (32 * c) / CP;
          const float negmu = valid_all[tt] ? tb_all[tt] - m_used : -INFINITY;
          const float2 w2 = make_float2(wmul[tt], wmul[tt]), n2 = make_float2(negmu, negmu);
          uint32_t pk[16];
#pragma unroll
          for (int jj = 0; jj < 32; jj += 2) {
            const int k = (32 * c + jj) % CP;
            float2 t = ffma2(make_float2(__uint_as_float(v[jj]), __uint_as_float(v[jj + 1])), w2, make_float2(cbf[k], cbf[k + 1]));
            t = fadd2(t, n2);
            const float2 e = poly_pair(jj / 2) ? ex2_poly2(t) : make_float2(ex2(t.x), ex2(t.y));
            psum2 = fadd2(psum2, e);
            pk[jj / 2] = pack_bf16(e.x, e.y);
          }
          tmem_st16(s_addr + 16 * c, pk);
        };
        tmem_ld_wait();
        tmem_ld32(s_addr + 32, vb);
        exp_chunk(va, 0);
        tmem_ld_wait();
        tmem_ld32(s_addr + 64, va);
        exp_chunk(vb, 1);
        tmem_ld_wait();
        tmem_ld32(s_addr + 96, vb);
        exp_chunk(va, 2);
        tmem_ld_wait();
        exp_chunk(vb, 3);
        l_sum += psum2.x + psum2.y;
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars[kBarPFull + wg]);
      }
      // ---- merge the two accumulators: O_even <- O_even 2^(m_e - m) + O_odd 2^(m_o - m) ----
      s_merge[wg * 128 + row] = m_used;
      s_merge[256 + wg * 128 + row] = l_sum;
      if (!ok) *s_giveup = 1;
      softmax_bar();
      if (*s_giveup != 0) ok = false;
      if (ok) {
        const float m_other = s_merge[(wg ^ 1) * 128 + row], l_other = s_merge[256 + (wg ^ 1) * 128 + row];
        if (n_dense >= 2) {
          const float m_new = fmaxf(m_used, m_other);
          const float a_self = ex2(m_used - m_new), a_oth = ex2(m_other - m_new);
          const int q1 = q_of_v(n_dense - 1), q2 = q_of_v(n_dense - 2);
          ok = warp_wait(&slot_free[q1 % NS], (q1 / NS) & 1, p.status, 36);
          if (ok) ok = warp_wait(&slot_free[q2 % NS], (q2 / NS) & 1, p.status, 36);
          if (ok) {
            tc_fence_after();
            const float a_e = wg == 0 ? a_self : a_oth, a_o = wg == 0 ? a_oth : a_self;
            uint32_t ve[32], vo[32];
            tmem_ld32(lane_base + kColO + wg * DW, ve);
            tmem_ld32(lane_base + kColO + 64 + wg * DW, vo);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              ve[jj] = __float_as_uint(__uint_as_float(ve[jj]) * a_e + __uint_as_float(vo[jj]) * a_o);
            tmem_st32(lane_base + kColO + wg * DW, ve);
            tmem_st_wait();
            tc_fence_before();
          }
          l_sum = wg == 0 ? l_sum * a_self + l_other * a_oth : 0.f;
          m_used = m_new;
        } else if (wg == 1) {  // a single dense tile: the second warpgroup adopts the first one's maximum
          m_used = m_other;
          l_sum = 0.f;
        }
      }
    } else {
    for (int s = 0; s < n_dense; ++s) {
      const int buf = s & 1;
      const int J = tile_of(s);
      const uint32_t s_addr = lane_base + kColS + 128 * buf + 64 * wg;
      float tb_all[TPB];
      bool valid_all[TPB];
      uint32_t tb_raw[TPB];
      int tb_col[TPB];
#pragma unroll
      for (int tt = 0; tt < TPB; ++tt) { tb_all[tt] = 0.f; valid_all[tt] = false; tb_raw[tt] = 0; tb_col[tt] = 0; }
      if (ok) tb_issue(J, tb_raw, tb_col, valid_all);
      float tbv[TPW], wmul[TPW];
      bool valid[TPW];
      float sreg[64];
      if (ok && !warp_wait(&bars[kBarSFull + buf], (s >> 1) & 1, p.status, 32)) ok = false;
      float m_part = -INFINITY;
      if (ok) {
        tc_fence_after();
        uint32_t v0[32], v1[32];
        tmem_ld32(s_addr, v0);
        tmem_ld32(s_addr + 32, v1);
        tmem_ld_wait();
        tb_finish(tb_raw, tb_col, tb_all);
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          sreg[jj] = __uint_as_float(v0[jj]);
          sreg[32 + jj] = __uint_as_float(v1[jj]);
        }
      }
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) {
        const int tt = tt_base + tl;
        float tsel = 0.f;
        bool vsel = false;
#pragma unroll
        for (int q = 0; q < TPB; ++q)  // compile-time indices keep tb_all in registers
          if (q == tt) { tsel = tb_all[q]; vsel = valid_all[q]; }
        tbv[tl] = tsel;
        valid[tl] = vsel;
        const int dt = ti_abs - (J * TPB + tt);
        wmul[tl] = (p.window > 0 && dt > p.window && ti_abs != T - 1) ? 0.f : 1.f;
      }
      if (ok) {
        float gmax[TPW];
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl) gmax[tl] = -INFINITY;
#pragma unroll
        for (int lc = 0; lc < 64; lc += 2) {
          const int tl = lc / CP, k = lc % NCH;
          const float2 t = ffma2(make_float2(sreg[lc], sreg[lc + 1]), make_float2(wmul[tl], wmul[tl]), make_float2(cbf[k], cbf[k + 1]));
          sreg[lc] = t.x;
          sreg[lc + 1] = t.y;
          gmax[tl] = fmax3(gmax[tl], t.x, t.y);
        }
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl)
          if (valid[tl]) m_part = fmaxf(m_part, gmax[tl] + tbv[tl]);
      }
      float m_tile = m_part;
      if constexpr (SPLIT) {
        if (!ok) break;  // (no barrier inside this loop: the flag is raised at the merge below)
      } else {
        // the two column halves of a row must agree on the tile maximum
        s_max[(buf * 2 + wg) * 128 + row] = m_part;
        if (!ok) *s_giveup = 1;
        softmax_bar();
        if (*s_giveup != 0) { ok = false; break; }  // some warp's wait ran out: everyone leaves together
        m_tile = fmaxf(m_part, s_max[(buf * 2 + (wg ^ 1)) * 128 + row]);
      }
      if (s == 0) {
        m_used = (m_tile == -INFINITY) ? 0.f : m_tile;
      } else if (!maybe_rescale(s, m_tile)) {
        ok = false;
        continue;
      }
      // (P_s reuses the columns of S_s / P_{s-2}; S_full of this tile already implies PV_{s-2} is done)
      float negmu[TPW];
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) negmu[tl] = valid[tl] ? tbv[tl] - m_used : -INFINITY;
      float2 psum2 = make_float2(0.f, 0.f);
      uint32_t lo[16], hi[16];
#pragma unroll
      for (int lc = 0; lc < 64; lc += 2) {
        const int tl = lc / CP;
        const float2 t = fadd2(make_float2(sreg[lc], sreg[lc + 1]), make_float2(negmu[tl], negmu[tl]));
        const float2 e = make_float2(ex2(t.x), ex2(t.y));
        psum2 = fadd2(psum2, e);
        if (lc < 32) lo[lc / 2] = pack_bf16(e.x, e.y);
        else hi[lc / 2 - 16] = pack_bf16(e.x, e.y);
      }
      l_sum += psum2.x + psum2.y;
      tmem_st16(s_addr, lo);  // P (bf16) over this thread's own, already consumed S columns
      tmem_st16(s_addr + 16, hi);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[kBarPFull + buf]);
    }
    if constexpr (SPLIT) {
      // ---- merge the two accumulators: O_0 <- O_0 2^(m_0 - m) + O_1 2^(m_1 - m); each warpgroup takes half
      //      of the columns; the row sum moves to the first warpgroup ----
      s_merge[wg * 128 + row] = m_used;
      s_merge[256 + wg * 128 + row] = l_sum;
      if (!ok) *s_giveup = 1;
      softmax_bar();
      if (*s_giveup != 0) ok = false;
      if (ok && n_dense > 0) {
        const float m_other = s_merge[(wg ^ 1) * 128 + row], l_other = s_merge[256 + (wg ^ 1) * 128 + row];
        const float m_new = fmaxf(m_used, m_other);
        const float a_self = ex2(m_used - m_new), a_oth = ex2(m_other - m_new);
        const int q1 = q_of_v(n_dense - 1);
        ok = warp_wait(&slot_free[q1 % NS], (q1 / NS) & 1, p.status, 36);
        if (ok) {
          tc_fence_after();
          const float a_0 = wg == 0 ? a_self : a_oth, a_1 = wg == 0 ? a_oth : a_self;
          uint32_t v0[32], v1[32];
          tmem_ld32(lane_base + kColO + wg * DW, v0);
          tmem_ld32(lane_base + kColO + 64 + wg * DW, v1);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            v0[jj] = __float_as_uint(__uint_as_float(v0[jj]) * a_0 + __uint_as_float(v1[jj]) * a_1);
          tmem_st32(lane_base + kColO + wg * DW, v0);
          tmem_st_wait();
          tc_fence_before();
        }
        l_sum = wg == 0 ? l_sum * a_self + l_other * a_oth : 0.f;
        m_used = m_new;
      }
      // (each warpgroup goes on with its own half of the merged columns; the first light PV product needs both
      // warpgroups' arrival, so it cannot start before both halves are merged)
    }

    }  // !ALT

    // ------------------------------ light tiles ------------------------------
    // P[i,k] = a_i[t_k] * bc_i[c_k]: one exponential per (row, key time step), packed bf16
    // multiplies for the rest.  Four P buffers of 64 TMEM columns (the idle S columns) let these
    // warps run ahead of the PV products.
    if (ok && n_light > 0) {
      // the buffers overlap S0 / S1: the last dense PV products must be done with them (and with O)
      const int q1 = q_of_v(n_dense - 1);
      ok = warp_wait(&slot_free[q1 % NS], (q1 / NS) & 1, p.status, 37);
      tc_fence_after();
    }
    // Every light tile's score is its temporal score alone (the channel maximum is folded into bc), and
    // the temporal scores of the row sit in TMEM: one pass finds the maximum over all light tiles, one
    // rescale of O covers the whole phase, and the loop below carries no maximum.
    // Key step tk of the light tiles (0 <= tk < n_light * TPB) is temporal column col0 + tk.
    const int col0 = T - 1 - ti_abs;
    uint32_t bc[NCH / 2];  // exp2(channel score - its maximum), bf16 pairs
    float sum_bc = 0.f;
#pragma unroll
    for (int k2 = 0; k2 < NCH / 2; ++k2) {
      bc[k2] = pack_bf16(ex2(cbf[2 * k2]), ex2(cbf[2 * k2 + 1]));
      sum_bc += __uint_as_float(bc[k2] << 16) + __uint_as_float(bc[k2] & 0xffff0000u);
    }
    if (ok && n_light > 0) {
      const int col1 = col0 + n_light * TPB;
      float m_light = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (32 * c + 32 <= col0 || 32 * c >= col1) continue;  // (warp-uniform)
        uint32_t v[32];
        tmem_ld32(lane_base + kColTB + 32 * c, v);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const int col = 32 * c + jj;
          const float tb = p.c2 * (__uint_as_float(v[jj]) + s_vr[col]) + mc;
          if (col >= col0 && col < col1) m_light = fmaxf(m_light, tb);
        }
      }
      const bool need = m_light > m_used + kRescaleThreshold;
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = need ? ex2(m_used - m_light) : 1.f;
#pragma unroll
        for (int c0 = 0; c0 < DW; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(lane_base + kColO + wg * DW + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) * alpha);
          tmem_st32(lane_base + kColO + wg * DW + c0, v);
        }
        tmem_st_wait();
        l_sum *= alpha;
        if (need) m_used = m_light;
      }
    }
    // Two tiles per turn: one round trip for the temporal scores and one look at the barriers serve both,
    // and the second tile's products are formed while the first tile's stores are in flight.  (The scores
    // of the next pair are fetched meanwhile; with an odd count the last fetch reads the column after the
    // light tiles, still inside the temporal columns, and drops it.)
    uint32_t tb_next[2 * TPB];
    auto tb_fetch = [&](int l) {
#pragma unroll
      for (int j = 0; j < 2 * TPB; ++j) tmem_ld1(lane_base + kColTB + col0 + l * TPB + j, tb_next[j]);
    };
    auto p_regs = [&](float (&a_t)[TPW], uint32_t (&lo)[16], uint32_t (&hi)[16], bool count) {
#pragma unroll
      for (int tl = 0; tl < TPW; ++tl) {
        const uint32_t a2 = pack_bf16(a_t[tl], a_t[tl]);
        if (count) l_sum += __uint_as_float(a2 << 16) * sum_bc;
#pragma unroll
        for (int k2 = 0; k2 < NCH / 2; ++k2) {
          const int idx = tl * (NCH / 2) + k2;
          if (idx < 16) lo[idx] = hmul2_bf16(a2, bc[k2]);
          else hi[idx - 16] = hmul2_bf16(a2, bc[k2]);
        }
      }
    };
    if (ok && n_light > 0) tb_fetch(0);
    for (int l = 0; ok && l < n_light; l += 2) {
      const int s = n_dense + l;
      const bool two = l + 1 < n_light;
      float a_t[2][TPW];  // exp2(temporal score - m) of this thread's key steps, both tiles
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int tl = 0; tl < TPW; ++tl) {
          const int tt = tt_base + tl;
          uint32_t raw = 0;
#pragma unroll
          for (int q = 0; q < TPB; ++q)
            if (q == tt) raw = tb_next[u * TPB + q];
          const float tb = p.c2 * (__uint_as_float(raw) + s_vr[col0 + (l + u) * TPB + tt]) + mc;
          a_t[u][tl] = ex2(tb - m_used);
        }
      }
      if (l + 2 < n_light) tb_fetch(l + 2);
      if (l >= 4) {
        // these buffers last held P of light tiles l-4 and l-3: a PV product frees the V slot it read
        const int q = q_of_v(s - 4);
        ok = warp_wait(&slot_free[q % NS], (q / NS) & 1, p.status, 35);
        if (ok && two) ok = warp_wait(&slot_free[(q + 1) % NS], ((q + 1) / NS) & 1, p.status, 35);
        if (!ok) break;
        tc_fence_after();
      }
      uint32_t lo0[16], hi0[16], lo1[16], hi1[16];
      const uint32_t p_addr0 = lane_base + kColS + 64 * (l & 3) + 32 * wg;
      const uint32_t p_addr1 = lane_base + kColS + 64 * ((l + 1) & 3) + 32 * wg;
      p_regs(a_t[0], lo0, hi0, true);
      tmem_st16(p_addr0, lo0);
      tmem_st16(p_addr0 + 16, hi0);
      p_regs(a_t[1], lo1, hi1, two);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[kBarPlFull + (l & 3)]);
      if (two) {
        tmem_st16(p_addr1, lo1);
        tmem_st16(p_addr1 + 16, hi1);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars[kBarPlFull + ((l + 1) & 3)]);
      }
    }
    // ------------------------------- epilogue ---------------------------------
    if (ok) {
      const int ql = q_of_v(n_tiles - 1);
      ok = warp_wait(&slot_free[ql % NS], (ql / NS) & 1, p.status, 34);
    }
    s_lsum[wg * 128 + row] = l_sum;
    softmax_bar();
    l_sum = s_lsum[row] + s_lsum[128 + row];
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l_sum;
      const int64_t n = (int64_t)(ti_abs - p.q_t0) * C + c_i;  // row inside this call's q / o / lse
      // O / l as bf16 into the Q tile's place (laid out like it: 128-byte swizzled rows), then one TMA
      // store per 64-column half; rows and channels outside the tensor are not written.
#pragma unroll
      for (int c0 = 0; c0 < DW; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + kColO + wg * DW + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w[e] = pack_bf16(__uint_as_float(v[q4 * 8 + 2 * e]) * inv, __uint_as_float(v[q4 * 8 + 2 * e + 1]) * inv);
          const int col = wg * DW + c0 + q4 * 8, hh = col / 64, c = (col % 64) / 8;
          *reinterpret_cast<uint4*>(sQ + hh * HALF + row * 128 + ((c ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async_smem();
      if (wg == 0 && row_valid && p.lse != nullptr) p.lse[(int64_t)bh * p.q_tn * C + n] = m_used + log2f(l_sum);
    }
    if (!ok) *s_giveup = 1;
    softmax_bar();
    if (*s_giveup == 0 && tid == 0) {
#pragma unroll
      for (int hh = 0; hh < NH; ++hh) tma_store_5d(&maps.o, sQ + hh * HALF, hh * 64, 0, I_loc * TPB, h, b);
      tma_store_commit();
      tma_store_wait_all();
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

int make_maps(TcMaps& m, const Args& a, int CP) {
  const int TPB = 128 / CP;
  const uint64_t es = 2;
  int rc;
  {
    const uint64_t dims[5] = {(uint64_t)a.D, (uint64_t)a.C, (uint64_t)a.q_tn, (uint64_t)a.H, (uint64_t)a.B};
    const uint64_t str[4] = {(uint64_t)a.q_sn * es, (uint64_t)a.q_sn * a.C * es, (uint64_t)a.q_sh * es,
                             (uint64_t)a.q_sb * es};
    const uint32_t box[5] = {64, (uint32_t)CP, (uint32_t)TPB, 1, 1};
    if ((rc = encode_bf16_sw128(&m.q, a.q, 5, dims, str, box))) return rc;
    const uint64_t stro[4] = {(uint64_t)a.o_sn * es, (uint64_t)a.o_sn * a.C * es, (uint64_t)a.o_sh * es,
                              (uint64_t)a.o_sb * es};
    if ((rc = encode_bf16_sw128(&m.o, a.o, 5, dims, stro, box))) return rc;
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
  t.q_t0 = a.q_t0; t.q_tn = a.q_tn;
  t.q_tiles = (a.q_tn + TPB - 1) / TPB;
  t.kv_major = kv_major_order(a.B, a.Hkv, a.g, a.N, D);
  if (a.q_t0 % TPB != 0) {
    set_error("query time range must start on a tile boundary: q_time_begin %d is not a multiple of %d", a.q_t0, TPB);
    return MVPA_ERR_ALIGNMENT;
  }
  t.c2 = a.c2;
  t.status = status;
  float* relc = reinterpret_cast<float*>(status) + 64;  // workspace + 256 bytes
  t.relc = relc;
  constexpr int smem = Cfg<D>::SMEM_BYTES;
  static_assert(smem <= 232448, "shared memory budget");
  static_assert(Cfg<D>::EARLY >= 2, "the first tile's K and V load while the prologue runs");
  MVPA_CUDA_CHECK(cudaFuncSetAttribute(tc_fwd_kernel<D, CP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  rel_const_kernel<D><<<a.Hkv, 256, 0, s>>>(t.vt, t.z, (const __nv_bfloat16*)a.rt, (const __nv_bfloat16*)a.rc, relc, a.T,
                                           a.C, status);  // (clears the status words too)
  count_launch();
  const unsigned grid = (unsigned)t.q_tiles * a.B * a.H;
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
  // status word (bounded waits report here) + per-kv-head constants of the relative products
  size_t bytes = 256 + (size_t)p->Hkv * 1024;
  return tc ? bytes : 0;
}

// ---- forward without caller scratch --------------------------------------------------------
// Scratch of the forward kernels (status word + per-kv-head constants of the relative products)
// for callers that cannot hand over a workspace: a fixed array in device memory, part of the
// library image, so every GPU that loads the library carries these 65 KB until the process exits.
constexpr int kStaticMaxKvHeads = 64;
constexpr size_t kStaticScratchBytes = 256 + (size_t)kStaticMaxKvHeads * 1024;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// In host code `g_static_scratch` only names the symbol; its device address has to be asked for,
// once per device, while that device is current.
constexpr int kStaticMaxDevices = 64;
void* g_static_addr[kStaticMaxDevices] = {};
std::mutex g_static_mu;
}  // namespace

int tc_fwd_static(const Args& a, cudaStream_t s) {
  if (a.Hkv > kStaticMaxKvHeads) {
    set_error("mvpa_fwd_noalloc: %d kv heads exceed the built-in scratch (at most %d); use mvpa_fwd with a workspace",
              a.Hkv, kStaticMaxKvHeads);
    return MVPA_ERR_WORKSPACE;
  }
  int dev = -1;
  MVPA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kStaticMaxDevices) {
    set_error("mvpa_fwd_noalloc: device ordinal %d out of range", dev);
    return MVPA_ERR_CUDA;
  }
  void* ptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_addr[dev] == nullptr) {
      void* got = nullptr;
      MVPA_CUDA_CHECK(cudaGetSymbolAddress(&got, g_static_scratch));
      g_static_addr[dev] = got;
    }
    ptr = g_static_addr[dev];
  }
  return tc_fwd(a, ptr, kStaticScratchBytes, s);
}

const int* tc_fwd_static_status_word() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_static_mu);
  return static_cast<const int*>(g_static_addr[dev]);
}

int tc_fwd(const Args& a, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (workspace == nullptr || workspace_bytes < 256 + (size_t)a.Hkv * 1024 || ((uintptr_t)workspace & 15) != 0) {
    set_error("tensor-core forward needs a 16-byte aligned workspace of mvpa_fwd_workspace_bytes() bytes");
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
