// Library state shared by all entry points: the thread-local error string,
// the per-device status word that kernels with bounded waits report into, the
// launch counter, and the GEMM dispatcher.

#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "common.cuh"

namespace mtfc {

namespace {
thread_local char g_error[512] = "";
std::atomic<long long> g_launches{0};
constexpr int kMaxDevices = 64;
int* g_status_words[kMaxDevices] = {nullptr};
int g_sm_counts[kMaxDevices] = {0};
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (!g_status_words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return nullptr;
    g_status_words[dev] = p;
  }
  return g_status_words[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (!g_sm_counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_counts[dev] = n;
  }
  return g_sm_counts[dev];
}

bool gemm_tcgen05_eligible(const mtfc_gemm_desc* d, const void* a, const void* b, const void* c);
int gemm_tcgen05_launch(const mtfc_gemm_desc* d, const void* a, const void* b, void* c,
                        cudaStream_t stream, int cta_group, void* progress);
int gemm_simt_launch(const mtfc_gemm_desc* d, const void* a, const void* b, void* c,
                     cudaStream_t stream);
int gemm_allreduce_flag_bytes();
void gemm_allreduce_set_wait_ms(int ms);
int gemm_allreduce_cooperative();
long long gemm_allreduce_stage_bytes(long long m, long long n, int nranks);
int gemm_allreduce_launch(const mtfc_gemm_desc* d, const void* a, const void* b,
                          void* const* stage, void* const* out, void* const* flags, void* ctl,
                          int rank, int nranks, int exchange, const void* mc_stage, void* mc_out,
                          cudaStream_t stream);

}  // namespace mtfc

using namespace mtfc;

extern "C" {

const char* mtfc_last_error(void) { return g_error; }

int mtfc_version(void) { return 1; }

int64_t mtfc_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int mtfc_device_status(void) {
  MTFC_CUDA(cudaDeviceSynchronize());
  int* w = device_status_word();
  if (!w) return fail(MTFC_ERR_CUDA, "no status word for the current device");
  int v = 0;
  MTFC_CUDA(cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    MTFC_CUDA(cudaMemset(w, 0, sizeof(int)));
    return fail(v, "a kernel's bounded wait ran out (status word %d)", v);
  }
  return MTFC_OK;
}

static int validate_gemm(const mtfc_gemm_desc* d, const void* a, const void* b, const void* c) {
  if (!d || !a || !b || !c) return fail(MTFC_ERR_SHAPE, "gemm: null argument");
  if (d->batch < 0 || d->m < 0 || d->n < 0 || d->k < 0)
    return fail(MTFC_ERR_SHAPE, "gemm: negative extent");
  if (dtype_size(d->in_dtype) == 0 || dtype_size(d->out_dtype) == 0)
    return fail(MTFC_ERR_UNSUPPORTED, "gemm: unknown dtype");
  return MTFC_OK;
}

int mtfc_gemm_uses_tensor_cores(const mtfc_gemm_desc* d, const void* a, const void* b,
                                const void* c) {
  int rc = validate_gemm(d, a, b, c);
  if (rc != MTFC_OK) return rc;
  if (d->force_path == 2) return 0;
  return gemm_tcgen05_eligible(d, a, b, c) ? 1 : 0;
}

int mtfc_gemm(const mtfc_gemm_desc* d, const void* a, const void* b, void* c, void* stream) {
  int rc = validate_gemm(d, a, b, c);
  if (rc != MTFC_OK) return rc;
  if (d->batch == 0 || d->m == 0 || d->n == 0) return MTFC_OK;  // empty output
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc_ok = d->k > 0 && gemm_tcgen05_eligible(d, a, b, c);
  const bool forced_tc = d->force_path == 1 || d->force_path == 3 || d->force_path == 4;
  if (forced_tc && !tc_ok)
    return fail(MTFC_ERR_SHAPE, "gemm: tensor-core path forced but the problem is not eligible");
  if (tc_ok && d->force_path != 2) {
    rc = gemm_tcgen05_launch(d, a, b, c, s,
                             d->force_path == 3 ? 1 : (d->force_path == 4 ? 2 : 0), nullptr);
  } else {
    rc = gemm_simt_launch(d, a, b, c, s);
  }
  if (rc == MTFC_OK) count_launch(1);
  return rc;
}

int mtfc_gemm_with_progress(const mtfc_gemm_desc* d, const void* a, const void* b, void* c,
                            uint32_t* progress, void* stream) {
  int rc = validate_gemm(d, a, b, c);
  if (rc != MTFC_OK) return rc;
  if (!progress) return fail(MTFC_ERR_SHAPE, "gemm_with_progress: null progress array");
  if (d->batch != 1 || d->m < 256 || d->n < 1 || d->k < 1 || !gemm_tcgen05_eligible(d, a, b, c))
    return fail(MTFC_ERR_UNSUPPORTED,
                "gemm_with_progress: needs one bf16 tensor-core GEMM of at least 256 rows");
  rc = gemm_tcgen05_launch(d, a, b, c, static_cast<cudaStream_t>(stream), 2, progress);
  if (rc == MTFC_OK) count_launch(1);
  return rc;
}

int mtfc_gemm_allreduce_flag_bytes(void) { return gemm_allreduce_flag_bytes(); }

int mtfc_gemm_allreduce_cooperative(void) { return gemm_allreduce_cooperative(); }

int mtfc_gemm_allreduce_set_wait_ms(int ms) {
  gemm_allreduce_set_wait_ms(ms);
  return MTFC_OK;
}

int64_t mtfc_gemm_allreduce_stage_bytes(int64_t m, int64_t n, int nranks) {
  return gemm_allreduce_stage_bytes(m, n, nranks);
}

int mtfc_gemm_allreduce_ex(const mtfc_gemm_desc* d, const void* a, const void* b,
                           void* const* stage_ptrs, void* const* out_ptrs, void* const* flag_ptrs,
                           void* ctl, int rank, int nranks, int exchange,
                           const void* stage_multicast, void* out_multicast, void* stream) {
  if (!d || !a || !b) return fail(MTFC_ERR_SHAPE, "gemm_allreduce: null argument");
  if (d->batch < 1 || d->m < 1 || d->n < 1 || d->k < 1)
    return fail(MTFC_ERR_SHAPE, "gemm_allreduce: empty problem");
  int rc = gemm_allreduce_launch(d, a, b, stage_ptrs, out_ptrs, flag_ptrs, ctl, rank, nranks,
                                 exchange, stage_multicast, out_multicast,
                                 static_cast<cudaStream_t>(stream));
  if (rc == MTFC_OK) count_launch(1);
  return rc;
}

int mtfc_gemm_allreduce(const mtfc_gemm_desc* d, const void* a, const void* b,
                        void* const* stage_ptrs, void* const* out_ptrs, void* const* flag_ptrs,
                        void* ctl, int rank, int nranks, void* stream) {
  return mtfc_gemm_allreduce_ex(d, a, b, stage_ptrs, out_ptrs, flag_ptrs, ctl, rank, nranks,
                                MTFC_EXCHANGE_PUSH, nullptr, nullptr, stream);
}

}  // extern "C"
