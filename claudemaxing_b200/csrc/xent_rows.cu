// Per-row loss / entropy / argmax-accuracy from logits that were materialised anyway (the
// fallback path; solution/lm_head_loss.py:54-96,285-297 of the reference). One CTA per row: every
// thread keeps an online (max, sum exp, sum exp*z, first argmax) over its columns, then the CTA
// merges them; ties on the maximum keep the lowest column, as torch.argmax does.
#include <math.h>

#include "common.cuh"

namespace soup {
namespace {

constexpr int kThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

struct Stat { float m, s, d; int arg; };

__device__ __forceinline__ void push(Stat& a, float z, int col) {
  if (z > a.m) {
    const float r = exp2f((a.m - z) * kLog2e);  // exp(-inf) = 0 on the first element
    a.s = a.s * r + 1.0f;
    a.d = a.d * r + z;
    a.m = z;
    a.arg = col;
  } else {
    const float e = exp2f((z - a.m) * kLog2e);
    a.s += e;
    a.d = fmaf(e, z, a.d);
  }
}

__device__ __forceinline__ Stat merge(const Stat& a, const Stat& b) {
  if (b.m == -INFINITY) return a;
  if (a.m == -INFINITY) return b;
  Stat o;
  o.m = fmaxf(a.m, b.m);
  const float ra = exp2f((a.m - o.m) * kLog2e), rb = exp2f((b.m - o.m) * kLog2e);
  o.s = a.s * ra + b.s * rb;
  o.d = a.d * ra + b.d * rb;
  o.arg = a.m > b.m ? a.arg : (b.m > a.m ? b.arg : min(a.arg, b.arg));
  return o;
}

__global__ void __launch_bounds__(kThreads)
xent_rows_kernel(const void* __restrict__ logits, const int64_t* __restrict__ target,
                 float* __restrict__ loss, float* __restrict__ entropy, int* __restrict__ correct,
                 int n_cols, int64_t row_stride, int dt, int vec) {
  __shared__ Stat s_stat[kThreads / 32];
  const int64_t row = blockIdx.x;
  const int64_t base = row * row_stride;
  Stat st = {-INFINITY, 0.f, 0.f, 0};
  if (vec) {
    const int n8 = n_cols >> 3;
    for (int v = threadIdx.x; v < n8; v += kThreads) {
      float z[8];
      load8(logits, base + ((int64_t)v << 3), dt, z);
#pragma unroll
      for (int k = 0; k < 8; ++k) push(st, z[k], (v << 3) + k);
    }
    for (int c = (n8 << 3) + threadIdx.x; c < n_cols; c += kThreads) push(st, load1(logits, base + c, dt), c);
  } else {
    for (int c = threadIdx.x; c < n_cols; c += kThreads) push(st, load1(logits, base + c, dt), c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Stat other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    other.d = __shfl_xor_sync(0xffffffffu, st.d, o);
    other.arg = __shfl_xor_sync(0xffffffffu, st.arg, o);
    st = merge(st, other);
  }
  if ((threadIdx.x & 31) == 0) s_stat[threadIdx.x >> 5] = st;
  __syncthreads();
  if (threadIdx.x == 0) {
    Stat all = s_stat[0];
    for (int w = 1; w < kThreads / 32; ++w) all = merge(all, s_stat[w]);
    const float lse = all.m + logf(all.s);
    const long long tg = target[row];
    const bool labelled = tg != -100;
    const float tl = labelled ? load1(logits, base + tg, dt) : 0.f;
    loss[row] = labelled ? lse - tl : 0.f;
    entropy[row] = lse - all.d / all.s;
    correct[row] = (labelled && (long long)all.arg == tg) ? 1 : 0;
  }
}

}  // namespace
}  // namespace soup

extern "C" int soup_xent_rows(const void* logits, const int64_t* target, float* loss,
                              float* entropy, int* correct, int64_t n_rows, int64_t n_cols,
                              int64_t row_stride, int dtype, void* stream) {
  using namespace soup;
  if (n_rows == 0) return SOUP_OK;
  if (n_rows < 0 || n_cols <= 0 || n_cols > INT32_MAX) SOUP_FAIL(SOUP_ERR_ARG, "xent_rows: bad shape");
  if (!logits || !target || !loss || !entropy || !correct) SOUP_FAIL(SOUP_ERR_ARG, "xent_rows: null pointer");
  if (!is_float_dtype(dtype)) SOUP_FAIL(SOUP_ERR_ARG, "xent_rows: unsupported dtype");
  const int vec = aligned16(logits) && (row_stride % 8 == 0);
  xent_rows_kernel<<<(unsigned)n_rows, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, target, loss, entropy, correct, (int)n_cols, row_stride, dtype, vec);
  SOUP_CHECK_LAUNCH("xent_rows");
  return SOUP_OK;
}
