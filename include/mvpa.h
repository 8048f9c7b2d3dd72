/*
 * mvpa.h — C ABI of the B200 multi-variate parallel attention (Flash-MVPA) library.
 *
 * The library replaces the device side of the reference operator
 * `attentions.flashmvpa` (`attentions/attn.py:1317-1366`): its Triton forward
 * kernel (`attentions/attn.py:38-347`), the materialised relative-score
 * matrices of `_rel_bias` (`attentions/attn.py:1305-1314`), its Triton backward
 * kernels (`attentions/attn.py:350-1010`) and the autograd that runs through
 * `_rel_bias` afterwards.  Every entry point takes plain device pointers, sizes
 * and a CUDA stream; the caller owns every buffer, including the workspace.
 * Nothing here allocates device memory, synchronises the device or keeps
 * state between calls (except where an entry point says otherwise).
 *
 * Token order is time-major: token n = t*C + c, N = T*C.
 *
 *   S[i,k] = sm_scale * ( win(i,k) * (q_i+u).K_k
 *                         + (q_i+vt).r_time[T-1-(t_i-t_k)]
 *                         + (q_i+z).r_chan[C-1-|c_i-c_k|] ),   -inf where t_k > t_i
 *   win    = window <= 0  or  |t_i-t_k| <= window  or  t_i == T-1
 *   O      = softmax_k(S) V ;  lse[i] = log2( sum_k 2^(S[i,k]*log2 e) )
 *
 * Return value: MVPA_OK (0) or a negative MVPA_ERR_* code; the text of the last
 * error on the calling thread is returned by mvpa_last_error_string().
 */
#ifndef MVPA_H_
#define MVPA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MVPA_OK 0
#define MVPA_ERR_SHAPE (-1)       /* a size is zero/negative, H % Hkv != 0, unsupported D */
#define MVPA_ERR_DTYPE (-2)       /* unknown element type */
#define MVPA_ERR_ALIGNMENT (-3)   /* a pointer or stride breaks the 16-byte rule */
#define MVPA_ERR_WORKSPACE (-4)   /* workspace missing or smaller than *_workspace_bytes() */
#define MVPA_ERR_CUDA (-5)        /* a CUDA runtime / driver call failed */
#define MVPA_ERR_UNSUPPORTED (-6) /* shape outside what the selected kernel handles */
#define MVPA_ERR_DEVICE (-7)      /* a kernel reported a non-zero status word (bounded wait ran out) */

/* Element type of q, k, v, u, vt, z, r_time, r_chan, o, dO, dq, dk, dv. */
#define MVPA_F32 0  /* fp32 I/O, fp32 arithmetic on CUDA cores                      */
#define MVPA_BF16 1 /* bf16 I/O, tcgen05 tensor cores with fp32 accumulation in TMEM */
#define MVPA_F16 2  /* fp16 I/O (the reference op takes it too), fp32 arithmetic on CUDA cores */

/* Problem description.  Mirrors the constexpr arguments of the reference launch
 * (`attentions/attn.py:1103-1120`: Z, H_Q, H_KV, N_CTX, TIME_CTX, CHANNEL_CTX,
 * WINDOW_SIZE, BLOCK_DMODEL) plus sm_scale. */
typedef struct mvpa_problem {
  int32_t B;      /* batch                                                        */
  int32_t H;      /* query heads                                                  */
  int32_t Hkv;    /* key/value heads, H % Hkv == 0                                */
  int32_t T;      /* time segments  (rows of r_time)                              */
  int32_t C;      /* channels       (rows of r_chan)                              */
  int32_t D;      /* head dim: 16, 32, 64 or 128 (`attentions/attn.py:1043`)      */
  int32_t window; /* content-window half width in time steps; <= 0: no window     */
  int32_t dtype;  /* MVPA_F32, MVPA_BF16, MVPA_F16                                       */
  float sm_scale; /* applied to the sum of the three score terms                  */
  int32_t flags;  /* reserved, must be 0                                          */
  /* Query time range (forward only).  q, o and lse then hold the tokens of time steps
   * [q_time_begin, q_time_begin + q_time_count) only, N_q = q_time_count*C rows, while k, v,
   * r_time, T describe the whole sequence: the time-block sharding of one long sample across
   * GPUs (each rank all-gathers K/V and computes its own query rows).  q_time_count == 0 means
   * the whole sequence.  The tensor-core forward needs q_time_begin to be a multiple of its
   * time steps per tile (128 / next_pow2(max(C,32))).  No counterpart in the reference. */
  int32_t q_time_begin;
  int32_t q_time_count;
} mvpa_problem;

/* A (batch, head, token, D) tensor with D contiguous; strides in elements.
 * The reference passes contiguous (B,H,N,D) tensors (`layers/mvpa.py:382-397`);
 * strides let a caller hand over the projection output without a permute copy. */
typedef struct mvpa_tensor {
  void* ptr;
  int64_t stride_b, stride_h, stride_n;
} mvpa_tensor;

/* Bytes of caller-owned scratch mvpa_fwd / mvpa_bwd need for this problem (may be 0). */
size_t mvpa_fwd_workspace_bytes(const mvpa_problem* p);
size_t mvpa_bwd_workspace_bytes(const mvpa_problem* p);

/*
 * Forward.  Replaces `_rel_bias` + `FlashMVPA.forward` + `_fwd_kernel`
 * (`attentions/attn.py:1305-1314, 1013-1138, 38-347`).
 *   q (B,H,N_q,D); k, v (B,Hkv,N,D); u, vt, z (Hkv,D) contiguous;
 *   r_time (Hkv,T,D), r_chan (Hkv,C,D) contiguous; o (B,H,N_q,D);
 *   lse (B*H, N_q) fp32, may be NULL when no backward will follow.  N_q = N unless the problem
 *   names a query time range.
 */
int mvpa_fwd(const mvpa_problem* p, const mvpa_tensor* q, const mvpa_tensor* k,
             const mvpa_tensor* v, const void* u, const void* vt, const void* z,
             const void* r_time, const void* r_chan, const mvpa_tensor* o, float* lse,
             void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * Backward.  Replaces `FlashMVPA.backward` + `_bwd_kernel`
 * (`attentions/attn.py:1140-1302, 776-1010, 350-773`) and the autograd through
 * `_rel_bias` that follows it (`attentions/attn.py:1305-1314`).
 *   o, lse: outputs of mvpa_fwd;  d_o (B,H,N,D) upstream gradient.
 *   dq (B,H,N,D), dk, dv (B,Hkv,N,D) in the element type of the inputs;
 *   du, dvt, dz (Hkv,D), dr_time (Hkv,T,D), dr_chan (Hkv,C,D) fp32, overwritten.
 */
int mvpa_bwd(const mvpa_problem* p, const mvpa_tensor* q, const mvpa_tensor* k,
             const mvpa_tensor* v, const void* u, const void* vt, const void* z,
             const void* r_time, const void* r_chan, const mvpa_tensor* o, const float* lse,
             const mvpa_tensor* d_o, const mvpa_tensor* dq, const mvpa_tensor* dk,
             const mvpa_tensor* dv, float* du, float* dvt, float* dz, float* dr_time,
             float* dr_chan, void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * Forward for callers that must not allocate.  (No counterpart in the reference, which allocates
 * freely through torch.)  Some hosts of this library cannot call cudaMalloc on the path that runs
 * attention: a serving process that handed all device memory to its own pool at start-up, or a
 * plugin whose host forbids allocator calls inside its execute hook.  mvpa_fwd leaves the scratch to the caller;
 * this variant of the bf16 tensor-core forward keeps its scratch (status word + per-kv-head
 * constants, 65 792 bytes) in a fixed array that is part of the library's device image, so each
 * GPU that loads the library holds those bytes until the process ends.
 *
 *   - Same arguments and results as mvpa_fwd, minus the workspace.  bf16 only, and only the
 *     shapes the tensor-core forward takes (D 64 or 128, C <= 128, T <= 128); at most 64 kv
 *     heads.  Anything else returns MVPA_ERR_UNSUPPORTED / MVPA_ERR_WORKSPACE with a message.
 *   - The first call on a device looks up the array's device address (once per device, with
 *     that device current).  Make that first call outside any stream capture.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - All calls on a device share the one array; whatever must start from zero is cleared on
 *     the stream at the start of each call.  Two calls whose kernels overlap on the GPU (two
 *     streams, two host threads) race on it: serialise them, or use mvpa_fwd with one
 *     workspace per stream.
 */
int mvpa_fwd_noalloc(const mvpa_problem* p, const mvpa_tensor* q, const mvpa_tensor* k,
                     const mvpa_tensor* v, const void* u, const void* vt, const void* z,
                     const void* r_time, const void* r_chan, const mvpa_tensor* o, float* lse,
                     void* cuda_stream);

/* Reads back the status word the kernels of the last mvpa_fwd call left at the start of
 * `workspace` (every device-side wait is bounded by a deadline on the GPU's nanosecond timer;
 * one that runs out records a code there and the kernel returns instead of hanging).  Synchronises `cuda_stream`.  Returns MVPA_OK, or
 * MVPA_ERR_DEVICE with the code in the error text.  Has no counterpart in the reference. */
int mvpa_workspace_status(const void* workspace, size_t workspace_bytes, void* cuda_stream);

/* The same for mvpa_bwd: its kernels keep their status word inside the workspace, at an offset that
 * depends on the problem.  `p`, `workspace`, `workspace_bytes` are the ones given to mvpa_bwd.
 * Problems that run on the CUDA-core kernels (no device-side waits) always return MVPA_OK.
 * Synchronises `cuda_stream`.  Has no counterpart in the reference. */
int mvpa_bwd_status(const mvpa_problem* p, const void* workspace, size_t workspace_bytes,
                    void* cuda_stream);

/* The same for mvpa_fwd_noalloc: reads the status word of the built-in array on the current
 * device (MVPA_OK if mvpa_fwd_noalloc has not run there yet).  Synchronises `cuda_stream`.
 * Allocates nothing.  Has no counterpart in the reference. */
int mvpa_noalloc_status(void* cuda_stream);

/* Self-test of the bounded waits: launches a one-warp kernel that waits, with a deadline of
 * `limit_us` microseconds (1 .. 1 000 000), on an mbarrier nothing arrives at.  The wait runs out,
 * the kernel records its code in the status word at the start of `workspace` (>= 256 bytes) and
 * returns; mvpa_workspace_status(workspace, ...) must then report MVPA_ERR_DEVICE.  Nothing
 * faults or hangs; the product kernels' own deadline (two seconds) is not changed.
 * Has no counterpart in the reference. */
int mvpa_selftest_wait_timeout(void* workspace, size_t workspace_bytes, uint32_t limit_us,
                               void* cuda_stream);

/* ---- kernels around the attention: block glue, encoder, heads (HBM-bound) -------------------
 * Rows are contiguous (`width` elements, a multiple of 16 bytes) unless a leading dimension is
 * given; element types MVPA_F32 / MVPA_BF16; arithmetic in fp32. */

/*
 * y = rmsnorm(h) * weight,  h = x (+ add, rounded to the element type as eager PyTorch does);
 * h is also written to `sum_out` when that is not NULL.  Replaces `ln_1` / `ln_f`
 * (`models/mvpformer.py:108,133,167,383`; RMSNorm: x * rsqrt(mean(x^2) + eps) * weight) and, with
 * `add`, the residual sum of the parallel block that precedes the next layer's norm
 * (`models/mvpformer.py:147`).  width <= 4096 (bf16) / 2048 (fp32).
 */
int mvpa_rmsnorm(const void* x, const void* add, const void* weight, void* sum_out, void* y,
                 int64_t rows, int32_t width, float eps, int32_t dtype, void* cuda_stream);

/*
 * out = silu(gate) * up, elementwise; gate, up share the leading dimension ld_in (two column blocks
 * of one fused projection), out has ld_out.  Replaces the activation inside `LlamaMLP`
 * (`models/mvpformer.py:114,146`: down_proj(act_fn(gate_proj(x)) * up_proj(x))).
 */
int mvpa_silu_mul(const void* gate, const void* up, int64_t ld_in, void* out, int64_t ld_out,
                  int64_t rows, int32_t width, int32_t dtype, void* cuda_stream);

/*
 * Number of coefficients `WaveEncoder` produces for a segment of `segment_len` samples with an
 * 8-tap wavelet in periodic mode (`models/fftencoder.py:69-78`: every level floor((n + 7) / 2),
 * floor(log2(len / 7)) levels, plus the last approximation); 0 if the segment is too short.
 * `level_sizes` (may be NULL) receives the per-level sizes, finest first.
 */
int32_t mvpa_wave_encode_size(int32_t segment_len, int32_t* level_sizes, int32_t max_levels);

/*
 * Encoder front end: all levels of the periodic 8-tap wavelet transform of each segment,
 * concatenated [cA_L, cD_L, ..., cD_1], RMS-normalised and scaled by `weight`, written once in
 * the output element type (columns past the coefficient count, up to ld_out, are zeroed so the
 * projection can run on a padded K).  Replaces `WaveEncoder.block` + `self.ln`
 * (`models/fftencoder.py:79-94`; `ptwt.wavedec(..., mode="periodic")` = circular padding + strided
 * convolution per level).  dec_lo / dec_hi: the eight decomposition taps, HOST pointers.
 */
int mvpa_wave_encode(const void* x, int64_t ld_x, int32_t x_dtype, const float* dec_lo,
                     const float* dec_hi, const void* weight, void* out, int64_t ld_out,
                     int32_t out_dtype, int64_t rows, int32_t segment_len, float eps,
                     void* cuda_stream);

/*
 * Gather of row pieces from other GPUs' memory into this GPU's memory with plain peer loads over
 * NVLink (no counterpart in the reference, whose only parallelism is data-parallel training,
 * `configs/*.yaml:3-6`): piece i copies bytes[i] bytes from src[i] (a device pointer that may lie in a
 * peer's memory, mapped into this process, e.g. through a CUDA IPC handle) to dst[i] (local memory).
 * src, dst and bytes are HOST arrays of n_pieces <= MVPA_MAX_GATHER_PIECES entries; every pointer and
 * size must be a multiple of 16 bytes.  One kernel launch, nothing allocated; the caller orders it
 * against the producers of the pieces (the data must be complete before the launch) and keeps the
 * sources alive and unchanged until it has finished.  Used by the time-sharded attention of one long
 * sample to bring every rank's K/V rows into local HBM.
 */
#define MVPA_MAX_GATHER_PIECES 32
int mvpa_peer_gather(void* const* dst, const void* const* src, const int64_t* bytes, int32_t n_pieces,
                     void* cuda_stream);

/*
 * Flags between GPUs for `mvpa_peer_gather` (no counterpart in the reference): 32-bit counters in device
 * memory that a peer has mapped.  The number signalled or waited for is `value`, plus `*base` when `base`
 * (device memory, read when the kernel runs) is not NULL - a step counter kept on the device lets a CUDA
 * graph replay the same launches step after step.  `mvpa_peer_signal` stores the number into each of the n
 * remote slots after a system-wide fence, so everything enqueued earlier on the stream is visible to a peer
 * that has seen the flag.  `mvpa_peer_wait` returns (on the stream) once each of the n local slots has
 * reached the number (compared as a wrapping counter); the wait is bounded: after `limit_us` microseconds
 * (0 = two seconds) the kernel stores 1 to *status (device memory, may be NULL) and returns, so a missing
 * peer surfaces as a status the host reads later, not as a hung GPU.  Both take HOST arrays of at most
 * MVPA_MAX_GATHER_PIECES device pointers.  The waiting and the signalling kernels must run on different
 * GPUs (one rank per GPU).
 */
int mvpa_peer_signal(uint32_t* const* remote_slots, int32_t n, uint32_t value, const uint32_t* base,
                     void* cuda_stream);
int mvpa_peer_wait(const uint32_t* const* local_slots, int32_t n, uint32_t value, const uint32_t* base,
                   uint32_t limit_us, int32_t* status, void* cuda_stream);

/*
 * Classification readout: out[b] = mean over channels of h[b, T-1] for h (B,T,C,E)
 * (`models/mvpformer.py:951-953`: `out[:, -1].mean(dim=1)`).
 */
int mvpa_channel_mean(const void* h, void* out, int32_t B, int32_t T, int32_t C, int32_t E,
                      int32_t dtype, void* cuda_stream);

/*
 * Contrastive next-state logits (`models/mvpformer.py:574-594, 631-660`).  pred, enc (B,T,C,E);
 * negatives (B,T,C,K) int32 row indices into enc viewed as (B*T*C, E); logits (B*(T-1)*C, 1+K) fp32:
 * row of target (b, t >= 1, c) holds cos(pred[b,t-1,c], enc[b,t,c]) / temperature, then the same
 * against each negative, -inf where a negative equals the positive.  The (rows, 1+K, E) target
 * tensor of the reference is never formed.  E <= 2048 (bf16) / 1024 (fp32).
 */
int mvpa_contrastive_logits(const void* pred, const void* enc, const int32_t* negatives,
                            float* logits, int32_t B, int32_t T, int32_t C, int32_t E, int32_t K,
                            float temperature, int32_t dtype, void* cuda_stream);

/* Text of the last error raised on this host thread ("" if none).
 * Stands where the reference raises RuntimeError / assert
 * (`attentions/attn.py:1034-1045, 1339, 1344`). */
const char* mvpa_last_error_string(void);

/* Number of kernels this library has launched on the calling process so far
 * (all threads); bench harnesses use the difference around a timed region. */
uint64_t mvpa_launch_count(void);

/* Library ABI version (bumped when a signature above changes). */
int mvpa_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MVPA_H_ */
