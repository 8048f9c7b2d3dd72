// C ABI of the Flash-MVPA library (declared in include/mvpa.h): argument checks,
// kernel-family selection, error text and the launch counter.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "mvpa_common.cuh"

namespace mvpa {

static thread_local char g_error[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int device_sm_count() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cache[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

namespace {

size_t elem_size(int dtype) { return dtype == MVPA_F32 ? 4 : 2; }

int check_problem(const mvpa_problem* p) {
  if (p == nullptr) {
    set_error("problem pointer is NULL");
    return MVPA_ERR_SHAPE;
  }
  if (p->dtype != MVPA_F32 && p->dtype != MVPA_BF16 && p->dtype != MVPA_F16) {
    set_error("unknown dtype %d (MVPA_F32=0, MVPA_BF16=1, MVPA_F16=2)", p->dtype);
    return MVPA_ERR_DTYPE;
  }
  if (p->B <= 0 || p->H <= 0 || p->Hkv <= 0 || p->T <= 0 || p->C <= 0) {
    set_error("B, H, Hkv, T, C must be positive (got %d %d %d %d %d)", p->B, p->H, p->Hkv, p->T, p->C);
    return MVPA_ERR_SHAPE;
  }
  if (p->H % p->Hkv != 0) {
    set_error("Q heads (%d) must be divisible by KV heads (%d)", p->H, p->Hkv);
    return MVPA_ERR_SHAPE;
  }
  if (p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128) {
    set_error("head dim %d not in {16, 32, 64, 128}", p->D);
    return MVPA_ERR_SHAPE;
  }
  if ((int64_t)p->T * p->C > (int64_t)1 << 30 || (int64_t)p->B * p->H > 65535) {
    set_error("problem too large: T*C = %lld tokens, B*H = %lld", (long long)p->T * p->C,
              (long long)p->B * p->H);
    return MVPA_ERR_SHAPE;
  }
  if (p->flags != 0) {
    set_error("flags must be 0");
    return MVPA_ERR_SHAPE;
  }
  if (p->q_time_begin < 0 || p->q_time_count < 0 || p->q_time_begin + p->q_time_count > p->T ||
      (p->q_time_count == 0 && p->q_time_begin != 0)) {
    set_error("query time range [%d, %d) is not inside [0, T = %d)", p->q_time_begin,
              p->q_time_begin + p->q_time_count, p->T);
    return MVPA_ERR_SHAPE;
  }
  return MVPA_OK;
}

int check_tensor(const char* name, const mvpa_tensor* t, int dtype) {
  if (t == nullptr || t->ptr == nullptr) {
    set_error("tensor %s is NULL", name);
    return MVPA_ERR_SHAPE;
  }
  const size_t es = elem_size(dtype);
  if (((uintptr_t)t->ptr & 15) != 0 || (t->stride_b * es) % 16 != 0 || (t->stride_h * es) % 16 != 0 ||
      (t->stride_n * es) % 16 != 0) {
    set_error("tensor %s: base address and byte strides must be multiples of 16", name);
    return MVPA_ERR_ALIGNMENT;
  }
  return MVPA_OK;
}

int check_ptr(const char* name, const void* ptr) {
  if (ptr == nullptr) {
    set_error("pointer %s is NULL", name);
    return MVPA_ERR_SHAPE;
  }
  if (((uintptr_t)ptr & 15) != 0) {
    set_error("pointer %s must be 16-byte aligned", name);
    return MVPA_ERR_ALIGNMENT;
  }
  return MVPA_OK;
}

int fill_args(Args& a, const mvpa_problem* p, const mvpa_tensor* q, const mvpa_tensor* k,
              const mvpa_tensor* v, const void* u, const void* vt, const void* z, const void* rt,
              const void* rc, const mvpa_tensor* o, float* lse) {
  int rcode;
  if ((rcode = check_problem(p))) return rcode;
  if ((rcode = check_tensor("q", q, p->dtype))) return rcode;
  if ((rcode = check_tensor("k", k, p->dtype))) return rcode;
  if ((rcode = check_tensor("v", v, p->dtype))) return rcode;
  if ((rcode = check_tensor("o", o, p->dtype))) return rcode;
  if ((rcode = check_ptr("u", u))) return rcode;
  if ((rcode = check_ptr("vt", vt))) return rcode;
  if ((rcode = check_ptr("z", z))) return rcode;
  if ((rcode = check_ptr("r_time", rt))) return rcode;
  if ((rcode = check_ptr("r_chan", rc))) return rcode;
  a.q = q->ptr; a.k = k->ptr; a.v = v->ptr; a.o = o->ptr;
  a.u = u; a.vt = vt; a.z = z; a.rt = rt; a.rc = rc; a.lse = lse;
  a.q_sb = q->stride_b; a.q_sh = q->stride_h; a.q_sn = q->stride_n;
  a.k_sb = k->stride_b; a.k_sh = k->stride_h; a.k_sn = k->stride_n;
  a.v_sb = v->stride_b; a.v_sh = v->stride_h; a.v_sn = v->stride_n;
  a.o_sb = o->stride_b; a.o_sh = o->stride_h; a.o_sn = o->stride_n;
  a.B = p->B; a.H = p->H; a.Hkv = p->Hkv; a.T = p->T; a.C = p->C; a.D = p->D;
  a.N = p->T * p->C; a.g = p->H / p->Hkv; a.window = p->window;
  a.sm_scale = p->sm_scale; a.c2 = p->sm_scale * kLog2e;
  a.q_t0 = p->q_time_count > 0 ? p->q_time_begin : 0;
  a.q_tn = p->q_time_count > 0 ? p->q_time_count : p->T;
  return MVPA_OK;
}

bool use_tc(const Args& a, int dtype) { return dtype == MVPA_BF16 && tc_fwd_supported(a); }

}  // namespace
}  // namespace mvpa

using namespace mvpa;

extern "C" {

size_t mvpa_fwd_workspace_bytes(const mvpa_problem* p) {
  if (check_problem(p) != MVPA_OK) return 0;
  return p->dtype == MVPA_BF16 ? tc_fwd_workspace_bytes(p) : 0;
}

size_t mvpa_bwd_workspace_bytes(const mvpa_problem* p) {
  if (check_problem(p) != MVPA_OK) return 0;
  return simt_bwd_workspace_floats(p) * sizeof(float);
}

int mvpa_fwd(const mvpa_problem* p, const mvpa_tensor* q, const mvpa_tensor* k, const mvpa_tensor* v,
             const void* u, const void* vt, const void* z, const void* r_time, const void* r_chan,
             const mvpa_tensor* o, float* lse, void* workspace, size_t workspace_bytes,
             void* cuda_stream) {
  Args a;
  int rc = fill_args(a, p, q, k, v, u, vt, z, r_time, r_chan, o, lse);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  if (use_tc(a, p->dtype)) {
    const size_t need = tc_fwd_workspace_bytes(p);
    if (need > 0 && (workspace == nullptr || workspace_bytes < need)) {
      set_error("mvpa_fwd: workspace of %zu bytes required, %zu given", need, workspace_bytes);
      return MVPA_ERR_WORKSPACE;
    }
    return tc_fwd(a, workspace, workspace_bytes, s);
  }
  return simt_fwd(a, p->dtype, s);
}

int mvpa_bwd(const mvpa_problem* p, const mvpa_tensor* q, const mvpa_tensor* k, const mvpa_tensor* v,
             const void* u, const void* vt, const void* z, const void* r_time, const void* r_chan,
             const mvpa_tensor* o, const float* lse, const mvpa_tensor* d_o, const mvpa_tensor* dq,
             const mvpa_tensor* dk, const mvpa_tensor* dv, float* du, float* dvt, float* dz,
             float* dr_time, float* dr_chan, void* workspace, size_t workspace_bytes,
             void* cuda_stream) {
  BwdArgs b;
  int rc = fill_args(b.a, p, q, k, v, u, vt, z, r_time, r_chan, o, const_cast<float*>(lse));
  if (rc) return rc;
  if (lse == nullptr) {
    set_error("mvpa_bwd: lse is NULL (run mvpa_fwd with an lse buffer first)");
    return MVPA_ERR_SHAPE;
  }
  if (b.a.q_tn != b.a.T) {
    set_error("mvpa_bwd: a query time range is a forward-only feature");
    return MVPA_ERR_UNSUPPORTED;
  }
  if ((rc = check_tensor("d_o", d_o, p->dtype))) return rc;
  if ((rc = check_tensor("dq", dq, p->dtype))) return rc;
  if ((rc = check_tensor("dk", dk, p->dtype))) return rc;
  if ((rc = check_tensor("dv", dv, p->dtype))) return rc;
  if ((rc = check_ptr("du", du))) return rc;
  if ((rc = check_ptr("dvt", dvt))) return rc;
  if ((rc = check_ptr("dz", dz))) return rc;
  if ((rc = check_ptr("dr_time", dr_time))) return rc;
  if ((rc = check_ptr("dr_chan", dr_chan))) return rc;
  const size_t need = mvpa_bwd_workspace_bytes(p);
  if (workspace == nullptr || workspace_bytes < need || ((uintptr_t)workspace & 15) != 0) {
    set_error("mvpa_bwd: 16-byte aligned workspace of %zu bytes required, %zu given", need,
              workspace_bytes);
    return MVPA_ERR_WORKSPACE;
  }
  b.d_o = d_o->ptr; b.do_sb = d_o->stride_b; b.do_sh = d_o->stride_h; b.do_sn = d_o->stride_n;
  b.dq = dq->ptr; b.dq_sb = dq->stride_b; b.dq_sh = dq->stride_h; b.dq_sn = dq->stride_n;
  b.dk = dk->ptr; b.dk_sb = dk->stride_b; b.dk_sh = dk->stride_h; b.dk_sn = dk->stride_n;
  b.dv = dv->ptr; b.dv_sb = dv->stride_b; b.dv_sh = dv->stride_h; b.dv_sn = dv->stride_n;
  b.du = du; b.dvt = dvt; b.dz = dz; b.drt = dr_time; b.drc = dr_chan;
  simt_bwd_carve(b, (float*)workspace, p->dtype);
  return simt_bwd(b, p->dtype, (cudaStream_t)cuda_stream);
}

int mvpa_fwd_noalloc(const mvpa_problem* p, const mvpa_tensor* q, const mvpa_tensor* k, const mvpa_tensor* v,
                     const void* u, const void* vt, const void* z, const void* r_time, const void* r_chan,
                     const mvpa_tensor* o, float* lse, void* cuda_stream) {
  Args a;
  int rc = fill_args(a, p, q, k, v, u, vt, z, r_time, r_chan, o, lse);
  if (rc) return rc;
  if (!use_tc(a, p->dtype)) {
    set_error("mvpa_fwd_noalloc covers the bf16 tensor-core forward only (D 64/128, C <= 128, T <= 128); "
              "other problems need no scratch at all: call mvpa_fwd");
    return MVPA_ERR_UNSUPPORTED;
  }
  return tc_fwd_static(a, (cudaStream_t)cuda_stream);
}

static int read_status_word(const int* word, cudaStream_t s) {
  if (word == nullptr) return MVPA_OK;  // nothing was recorded
  int code = 0;
  MVPA_CUDA_CHECK(cudaMemcpyAsync(&code, word, sizeof(int), cudaMemcpyDeviceToHost, s));
  MVPA_CUDA_CHECK(cudaStreamSynchronize(s));
  if (code != 0) {
    set_error("a kernel gave up a bounded wait (code %d) and returned early; outputs are invalid", code);
    return MVPA_ERR_DEVICE;
  }
  return MVPA_OK;
}

int mvpa_workspace_status(const void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (workspace == nullptr || workspace_bytes < sizeof(int)) return MVPA_OK;
  return read_status_word(static_cast<const int*>(workspace), (cudaStream_t)cuda_stream);
}

int mvpa_bwd_status(const mvpa_problem* p, const void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (check_problem(p) != MVPA_OK) return MVPA_ERR_SHAPE;
  if (workspace == nullptr || workspace_bytes < mvpa_bwd_workspace_bytes(p)) {
    set_error("mvpa_bwd_status: the workspace handed to mvpa_bwd (%zu bytes) is required",
              mvpa_bwd_workspace_bytes(p));
    return MVPA_ERR_WORKSPACE;
  }
  return read_status_word(bwd_status_word(p, workspace), (cudaStream_t)cuda_stream);
}

int mvpa_noalloc_status(void* cuda_stream) {
  return read_status_word(tc_fwd_static_status_word(), (cudaStream_t)cuda_stream);
}

int mvpa_selftest_wait_timeout(void* workspace, size_t workspace_bytes, uint32_t limit_us, void* cuda_stream) {
  if (workspace == nullptr || workspace_bytes < 256 || ((uintptr_t)workspace & 15) != 0) {
    set_error("mvpa_selftest_wait_timeout: a 16-byte aligned workspace of at least 256 bytes is required");
    return MVPA_ERR_WORKSPACE;
  }
  if (limit_us == 0 || limit_us > 1000000u) {
    set_error("mvpa_selftest_wait_timeout: limit_us must be in [1, 1000000]");
    return MVPA_ERR_SHAPE;
  }
  return selftest_wait_timeout(static_cast<int*>(workspace), limit_us, (cudaStream_t)cuda_stream);
}

const char* mvpa_last_error_string(void) { return g_error; }

uint64_t mvpa_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int mvpa_abi_version(void) { return 3; }

}  // extern "C"
