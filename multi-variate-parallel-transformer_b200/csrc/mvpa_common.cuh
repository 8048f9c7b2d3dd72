// Shared declarations of the Flash-MVPA library: the internal problem record
// every kernel family receives, error plumbing and the launch counter.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mvpa.h"

namespace mvpa {

constexpr float kLog2e = 1.4426950408889634f;

// Flattened view of the C-ABI arguments (include/mvpa.h) handed to kernels.
struct Args {
  const void *q, *k, *v, *u, *vt, *z, *rt, *rc;
  void* o;
  float* lse;
  int64_t q_sb, q_sh, q_sn;
  int64_t k_sb, k_sh, k_sn;
  int64_t v_sb, v_sh, v_sn;
  int64_t o_sb, o_sh, o_sn;
  int B, H, Hkv, T, C, D, N, g, window;
  int q_t0, q_tn;  // query rows cover time steps [q_t0, q_t0 + q_tn); N_q = q_tn * C
  float sm_scale;  // natural-log domain scale of the score sum
  float c2;        // sm_scale * log2(e): scores are kept in base 2
};

struct BwdArgs {
  Args a;
  const void* d_o;
  int64_t do_sb, do_sh, do_sn;
  void *dq, *dk, *dv;
  int64_t dq_sb, dq_sh, dq_sn;
  int64_t dk_sb, dk_sh, dk_sn;
  int64_t dv_sb, dv_sh, dv_sn;
  float *du, *dvt, *dz, *drt, *drc;
  // workspace carve-up (fp32 elements)
  float *tbg, *cbg;    // (B*H, N, T), (B*H, N, C) relative scores, base-2 scaled
  float *dtbg, *dcbg;  // gradients w.r.t. the unscaled relative scores, (B*H, N, slots); the tensor-core
                       // kernels use dtbg as (B*H, T, N) scratch and leave dcbg alone
  float* delta;        // (B*H, N)
  float* partial;      // (B*H*nQT, 3, D) per-tile column sums for du/dvt/dz
  float* drel_part;    // (split, Hkv, T + C, D) split-K partials of dr_time / dr_chan
  float* tc_extra;     // workspace of the tensor-core query-side kernel (bf16 problems it supports)
};

void set_error(const char* fmt, ...);
void count_launch(int n = 1);

// fp32 CUDA-core kernels (any T, C; D in {16,32,64,128}); element type float or bf16.
// Multiprocessors of the current device (cudaDevAttrMultiProcessorCount, cached per device; 148 on a B200).
int device_sm_count();

// Order in which the tensor-core kernels' CTAs take their work.  Tile-major (all batch x head pairs of the
// heaviest tile first) balances best, but the CTAs resident together (one per multiprocessor) then stream
// the K/V (or Q'/dO) of up to SMs/g different kv heads: once that set is several times the L2, every CTA reads from DRAM.  Past
// 256 MB the kernels switch to kv-head-major: the CTAs of one kv head (all its query tiles and group heads)
// are adjacent, so the operands they share stay in the L2 (tiles still heaviest first inside a head).
// Measured: at 592 MB (B 32 x 8 kv heads x 16k tokens, D 128) kv-head-major is 15 % (forward) and 32 %
// (forward + backward) faster; at 128 MB (B 8 x 16 heads x 4k tokens, D 64) tile-major is 6-13 % faster.
inline int kv_major_order(int B, int Hkv, int g, int N, int D) {
  const int64_t resident = (device_sm_count() + g - 1) / g;
  const int64_t heads = (int64_t)B * Hkv < resident ? (int64_t)B * Hkv : resident;
  return heads * 2 * N * D * 2 > (int64_t)256 * 1024 * 1024 ? 1 : 0;
}

int simt_fwd(const Args& a, int dtype, cudaStream_t s);
int simt_bwd(const BwdArgs& b, int dtype, cudaStream_t s);
size_t simt_bwd_workspace_floats(const mvpa_problem* p);
void simt_bwd_carve(BwdArgs& b, float* ws, int dtype);

// tcgen05 / TMEM / TMA forward for bf16 (mvpa_tc_fwd.cu).
bool tc_fwd_supported(const Args& a);
size_t tc_fwd_workspace_bytes(const mvpa_problem* p);
int tc_fwd(const Args& a, void* workspace, size_t workspace_bytes, cudaStream_t s);
int tc_fwd_static(const Args& a, cudaStream_t s);  // same, scratch in a built-in device array
// Status word of the built-in array on the current device (nullptr before the first tc_fwd_static call there).
const int* tc_fwd_static_status_word();

// tcgen05 backward for bf16 (mvpa_tc_bwd.cu): dq, dk, dv, and per-kv-head accumulators of the
// relative-key gradients; tc_bwd_bias turns those into dr_time / dr_chan / du / dvt / dz.
bool tc_bwd_q_supported(const Args& a);
size_t tc_bwd_q_workspace_floats(const mvpa_problem* p);
int tc_bwd_q(const BwdArgs& b, float* extra_workspace, cudaStream_t s);
int tc_bwd_bias(const BwdArgs& b, float* extra_workspace, cudaStream_t s);
size_t tc_bwd_status_offset_floats(const mvpa_problem* p);
// Status word of the backward's kernels inside the caller's workspace (nullptr: this problem runs on
// kernels without device-side waits).
const int* bwd_status_word(const mvpa_problem* p, const void* workspace);
// Wait self-test (mvpa_selftest.cu).
int selftest_wait_timeout(int* status, unsigned limit_us, cudaStream_t s);

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

}  // namespace mvpa

#define MVPA_CUDA_CHECK(expr)                                                        \
  do {                                                                               \
    cudaError_t err__ = (expr);                                                      \
    if (err__ != cudaSuccess) {                                                      \
      ::mvpa::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__),   \
                        __FILE__, __LINE__);                                         \
      return MVPA_ERR_CUDA;                                                          \
    }                                                                                \
  } while (0)
