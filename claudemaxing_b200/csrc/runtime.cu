// Process-wide pieces of libsoup_b200: version, the thread-local error string, cached device facts.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"
#include "rowpipe.cuh"

namespace soup {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  // Cached per device ordinal; a wrong value only changes a grid size, never correctness.
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace rowpipe {
namespace {
__device__ int g_row_status = 0;
}
int sm_count_for_plan() { return sm_count(); }
int* status_word() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_row_status) != cudaSuccess) return nullptr;
    cached[dev] = reinterpret_cast<int*>(p);
  }
  return cached[dev];
}
}  // namespace rowpipe

}  // namespace soup

namespace soup {
namespace {
__device__ int g_selftest[2] = {0, 0};   // [0] status code, [1] 1 when the wait returned "gave up"

// A barrier that nothing ever completes: every thread's bounded wait has to run out, record its
// code and return, leaving the context healthy.
__global__ void wait_selftest_kernel(int* words, uint64_t limit_ns, int* sticky) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    umma::mbar_init(&bar, 1);
    abort_flag = 0;
  }
  umma::fence_barrier_init();
  __syncthreads();
  const bool ok = umma::mbar_wait_for(&bar, 0, &abort_flag, &words[0], 99, limit_ns);
  if (!ok && threadIdx.x == 0) {
    words[1] = 1;
    if (sticky) atomicCAS(sticky, 0, words[0]);   // as the real kernels publish a wait that gave up
  }
}
}  // namespace
}  // namespace soup

extern "C" int soup_wait_selftest(int64_t limit_ns, int* host_gave_up, int* host_status,
                                  void* stream) {
  using namespace soup;
  if (limit_ns <= 0 || limit_ns > 100000000 || !host_gave_up || !host_status)
    SOUP_FAIL(SOUP_ERR_ARG, "wait_selftest: limit must be in (0, 100 ms] and the outputs non-null");
  void* words = nullptr;
  if (cudaGetSymbolAddress(&words, g_selftest) != cudaSuccess || !words)
    SOUP_FAIL(SOUP_ERR_DEVICE, "wait_selftest: no scratch on this device");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int out[2] = {0, 0};
  if (cudaMemsetAsync(words, 0, sizeof(out), s) != cudaSuccess)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "wait_selftest: %s", cudaGetErrorString(cudaGetLastError()));
  wait_selftest_kernel<<<1, 64, 0, s>>>(reinterpret_cast<int*>(words), (uint64_t)limit_ns,
                                        rowpipe::status_word());
  SOUP_CHECK_LAUNCH("wait_selftest");
  if (cudaMemcpyAsync(out, words, sizeof(out), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "wait_selftest: %s", cudaGetErrorString(cudaGetLastError()));
  *host_status = out[0];
  *host_gave_up = out[1];
  return SOUP_OK;
}

extern "C" int soup_row_status(int* host_status, void* stream) {
  using namespace soup;
  if (!host_status) SOUP_FAIL(SOUP_ERR_ARG, "row_status: null pointer");
  int* word = rowpipe::status_word();
  if (!word) SOUP_FAIL(SOUP_ERR_DEVICE, "row_status: no status word on this device");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(host_status, word, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "row_status: %s", cudaGetErrorString(cudaGetLastError()));
  return SOUP_OK;
}

extern "C" int soup_device_status(int* host_status, int clear, void* stream) {
  using namespace soup;
  if (!host_status) SOUP_FAIL(SOUP_ERR_ARG, "device_status: null pointer");
  int* word = rowpipe::status_word();
  if (!word) SOUP_FAIL(SOUP_ERR_DEVICE, "device_status: no status word on this device");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(host_status, word, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      (clear && cudaMemsetAsync(word, 0, sizeof(int), s) != cudaSuccess) ||
      cudaStreamSynchronize(s) != cudaSuccess)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "device_status: %s", cudaGetErrorString(cudaGetLastError()));
  return SOUP_OK;
}

extern "C" int soup_version(void) { return 2; }

extern "C" const char* soup_last_error_string(void) { return soup::g_error; }
