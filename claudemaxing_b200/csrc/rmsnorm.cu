// RMSNorm forward and backward for Qwen2 (fp32 statistics, the reference's rounding points).
//
// Layout of the work: a thread owns VPT column vectors of 8 elements and keeps them in registers;
// a CTA of TPR threads covers one row (TPR * VPT * 8 >= n_cols) and processes R rows per step so
// that two rows' worth of 128-bit loads are in flight before the first reduction. The row sums are
// reduced with warp shuffles and one shared-memory exchange. Backward reads each row twice (the
// second time from L1/L2) instead of holding it in registers, which keeps ten CTAs per SM in
// flight; it is persistent when dw is
// wanted: a thread accumulates dw of its own columns in registers across the rows of its CTA and
// writes one partial row per CTA; a second tiny kernel adds the partial rows in a fixed order, so
// dw is deterministic.
//
// Rounding (solution/rmsnorm.py:28-91 of the reference): the normalised value is rounded to the
// dtype of x before it meets the weight; in backward dy*w is rounded to that dtype too, except on
// the saved-output path, where x is fp32 and nothing is rounded.
#include "common.cuh"

namespace soup {
namespace {

constexpr int kMaxWarps = 8;  // TPR <= 256

template <int R>
__device__ __forceinline__ void block_sum(float (&v)[R], float* s_red, int n_warps) {
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = warp_sum(v[r]);
  if (n_warps == 1) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // previous use of s_red is over
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) s_red[r * kMaxWarps + warp] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float t = 0.f;
    for (int wi = 0; wi < n_warps; ++wi) t += s_red[r * kMaxWarps + wi];
    v[r] = t;
  }
}

template <int VPT, int R>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const void* __restrict__ x, const void* __restrict__ w, void* __restrict__ out,
                   float* __restrict__ rstd_out, void* __restrict__ low,
                   const int32_t* __restrict__ slot, void* __restrict__ small, int64_t n_small,
                   int64_t n_rows, int n_cols, float eps, int xdt, int wdt, int odt) {
  __shared__ float s_red[R * kMaxWarps];
  const int n_vec = n_cols >> 3, n_warps = blockDim.x >> 5;
  const int64_t row0 = (int64_t)blockIdx.x * R;
  float xv[R][VPT][8];
  float ss[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    ss[r] = 0.f;
    const int64_t row = row0 + r;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vi = threadIdx.x + j * blockDim.x;
      if (row < n_rows && vi < n_vec) {
        load8(x, row * n_cols + (vi << 3), xdt, xv[r][j]);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss[r] += xv[r][j][k] * xv[r][j][k];
      }
    }
  }
  block_sum<R>(ss, s_red, n_warps);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int vi = threadIdx.x + j * blockDim.x;
    if (vi >= n_vec) continue;
    float wv[8];
    load8(w, vi << 3, wdt, wv);
    int sl[8];
    if (low) {
      const int4 a = *reinterpret_cast<const int4*>(slot + (vi << 3));
      const int4 b = *reinterpret_cast<const int4*>(slot + (vi << 3) + 4);
      sl[0] = a.x; sl[1] = a.y; sl[2] = a.z; sl[3] = a.w;
      sl[4] = b.x; sl[5] = b.y; sl[6] = b.z; sl[7] = b.w;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = row0 + r;
      if (row >= n_rows) continue;
      const float rstd = 1.0f / sqrtf(ss[r] / (float)n_cols + eps);
      if (j == 0 && threadIdx.x == 0) rstd_out[row] = rstd;
      float o[8], nrm[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        nrm[k] = round_through(xv[r][j][k] * rstd, xdt);
        o[k] = nrm[k] * wv[k];
      }
      store8(out, row * n_cols + (vi << 3), odt, o);
      if (low) {
        store8(low, row * n_cols + (vi << 3), SOUP_F16, o);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (sl[k] >= 0) store1(small, row * n_small + sl[k], SOUP_F16, nrm[k]);
      }
    }
  }
}

// Any n_cols / alignment: one CTA per row, columns re-read from global (L1/L2) for the second pass.
__global__ void __launch_bounds__(256)
rmsnorm_fwd_scalar_kernel(const void* __restrict__ x, const void* __restrict__ w,
                          void* __restrict__ out, float* __restrict__ rstd_out,
                          void* __restrict__ low, const int32_t* __restrict__ slot,
                          void* __restrict__ small, int64_t n_small, int n_cols, float eps, int xdt,
                          int wdt, int odt) {
  __shared__ float s_red[kMaxWarps];
  const int64_t row = blockIdx.x;
  float ss[1] = {0.f};
  for (int c = threadIdx.x; c < n_cols; c += blockDim.x) {
    const float v = load1(x, row * n_cols + c, xdt);
    ss[0] += v * v;
  }
  block_sum<1>(ss, s_red, blockDim.x >> 5);
  const float rstd = 1.0f / sqrtf(ss[0] / (float)n_cols + eps);
  if (threadIdx.x == 0) rstd_out[row] = rstd;
  for (int c = threadIdx.x; c < n_cols; c += blockDim.x) {
    const float nrm = round_through(load1(x, row * n_cols + c, xdt) * rstd, xdt);
    const float o = nrm * load1(w, c, wdt);
    store1(out, row * n_cols + c, odt, o);
    if (low) {
      store1(low, row * n_cols + c, SOUP_F16, o);
      const int s = slot[c];
      if (s >= 0) store1(small, row * n_small + s, SOUP_F16, nrm);
    }
  }
}

// One row of backward for one thread's column vector. Returns the thread's part of sum(gn * n).
__device__ __forceinline__ float bwd_prepare(const float (&dy)[8], const float (&xin)[8],
                                             const float (&wv)[8], const int (&sl)[8],
                                             const void* small, int64_t small_row, float rstd,
                                             int xdt, bool saved_output, float (&gn)[8],
                                             float (&nrm)[8]) {
  float dot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (saved_output) {
      // xin holds fp16((x*rstd)*w); the tiny-|w| columns kept their normalised value aside.
      nrm[k] = sl[k] >= 0 ? load1(small, small_row + sl[k], SOUP_F16) : xin[k] / wv[k];
      gn[k] = dy[k] * wv[k];
    } else {
      nrm[k] = xin[k] * rstd;
      gn[k] = round_through(dy[k] * wv[k], xdt);
    }
    dot += gn[k] * nrm[k];
  }
  return dot;
}

template <int VPT, bool DW>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const void* __restrict__ dy, const void* __restrict__ xin,
                   const void* __restrict__ w, const float* __restrict__ rstd_in,
                   void* __restrict__ dx, float* __restrict__ dw_partial,
                   const int32_t* __restrict__ slot, const void* __restrict__ small,
                   int64_t n_small, int64_t n_rows, int n_cols, int ydt, int xdt, int wdt, int dxdt,
                   int saved_output) {
  __shared__ float s_red[kMaxWarps];
  const int n_vec = n_cols >> 3, n_warps = blockDim.x >> 5;
  float wv[VPT][8];
  int sl[VPT][8];
  float dw_acc[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int vi = threadIdx.x + j * blockDim.x;
#pragma unroll
    for (int k = 0; k < 8; ++k) { wv[j][k] = 0.f; sl[j][k] = -1; dw_acc[j][k] = 0.f; }
    if (vi < n_vec) {
      load8(w, vi << 3, wdt, wv[j]);
      if (saved_output) {
        const int4 a = *reinterpret_cast<const int4*>(slot + (vi << 3));
        const int4 b = *reinterpret_cast<const int4*>(slot + (vi << 3) + 4);
        sl[j][0] = a.x; sl[j][1] = a.y; sl[j][2] = a.z; sl[j][3] = a.w;
        sl[j][4] = b.x; sl[j][5] = b.y; sl[j][6] = b.z; sl[j][7] = b.w;
      }
    }
  }
  // Two passes per row with few live registers, so that many CTAs fit on an SM and their loads
  // overlap: pass 1 reads dy and x for the row's dot product, pass 2 reads them again (they are
  // still in L1/L2, the row is 6 KB) and writes dx.
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float dot[1] = {0.f};
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vi = threadIdx.x + j * blockDim.x;
      if (vi < n_vec) {
        float yv[8], xv[8], gn[8], nrm[8];
        load8(dy, row * n_cols + (vi << 3), ydt, yv);
        load8(xin, row * n_cols + (vi << 3), xdt, xv);
        dot[0] += bwd_prepare(yv, xv, wv[j], sl[j], small, row * n_small, rstd, xdt,
                              saved_output != 0, gn, nrm);
        if (DW) {
#pragma unroll
          for (int k = 0; k < 8; ++k) dw_acc[j][k] += yv[k] * round_through(nrm[k], xdt);
        }
      }
    }
    block_sum<1>(dot, s_red, n_warps);
    const float mean_dot = dot[0] / (float)n_cols;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vi = threadIdx.x + j * blockDim.x;
      if (vi < n_vec) {
        float yv[8], xv[8], gn[8], nrm[8], o[8];
        load8(dy, row * n_cols + (vi << 3), ydt, yv);
        load8(xin, row * n_cols + (vi << 3), xdt, xv);
        bwd_prepare(yv, xv, wv[j], sl[j], small, row * n_small, rstd, xdt, saved_output != 0, gn, nrm);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (gn[k] - nrm[k] * mean_dot) * rstd;
        store8(dx, row * n_cols + (vi << 3), dxdt, o);
      }
    }
  }
  if (DW) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int vi = threadIdx.x + j * blockDim.x;
      if (vi < n_vec) store8(dw_partial, (int64_t)blockIdx.x * n_cols + (vi << 3), SOUP_F32, dw_acc[j]);
    }
  }
}

template <bool DW>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_scalar_kernel(const void* __restrict__ dy, const void* __restrict__ xin,
                          const void* __restrict__ w, const float* __restrict__ rstd_in,
                          void* __restrict__ dx, float* __restrict__ dw_partial,
                          const int32_t* __restrict__ slot, const void* __restrict__ small,
                          int64_t n_small, int64_t n_rows, int n_cols, int ydt, int xdt, int wdt,
                          int dxdt, int saved_output) {
  // dw_partial row of this CTA is accumulated in place in global memory (zeroed first).
  __shared__ float s_red[kMaxWarps];
  if (DW)
    for (int c = threadIdx.x; c < n_cols; c += blockDim.x)
      dw_partial[(int64_t)blockIdx.x * n_cols + c] = 0.f;
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float dot[1] = {0.f};
    for (int c = threadIdx.x; c < n_cols; c += blockDim.x) {
      const float yv = load1(dy, row * n_cols + c, ydt), xv = load1(xin, row * n_cols + c, xdt);
      const float wc = load1(w, c, wdt);
      float nrm, gn;
      if (saved_output) {
        const int s = slot[c];
        nrm = s >= 0 ? load1(small, row * n_small + s, SOUP_F16) : xv / wc;
        gn = yv * wc;
      } else {
        nrm = xv * rstd;
        gn = round_through(yv * wc, xdt);
      }
      dot[0] += gn * nrm;
      if (DW) dw_partial[(int64_t)blockIdx.x * n_cols + c] += yv * round_through(nrm, xdt);
    }
    block_sum<1>(dot, s_red, blockDim.x >> 5);
    const float mean_dot = dot[0] / (float)n_cols;
    for (int c = threadIdx.x; c < n_cols; c += blockDim.x) {
      const float yv = load1(dy, row * n_cols + c, ydt), xv = load1(xin, row * n_cols + c, xdt);
      const float wc = load1(w, c, wdt);
      float nrm, gn;
      if (saved_output) {
        const int s = slot[c];
        nrm = s >= 0 ? load1(small, row * n_small + s, SOUP_F16) : xv / wc;
        gn = yv * wc;
      } else {
        nrm = xv * rstd;
        gn = round_through(yv * wc, xdt);
      }
      store1(dx, row * n_cols + c, dxdt, (gn - nrm * mean_dot) * rstd);
    }
  }
}

// dw[c] = sum over partial rows, fixed order, rounded once to the weight dtype.
__global__ void __launch_bounds__(256)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, void* __restrict__ dw, int n_partials,
                         int n_cols, int wdt) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_cols) return;
  float acc = 0.f;
  for (int p = 0; p < n_partials; ++p) acc += partial[(int64_t)p * n_cols + c];
  store1(dw, c, wdt, acc);
}

struct Shape { int vpt, tpr; };

// Smallest VPT in {1,2,4,8} whose CTA (<= 256 threads) covers the row.
inline Shape pick_shape(int n_cols) {
  const int n_vec = n_cols >> 3;
  int vpt = 1;
  while (vpt < 8 && (n_vec + vpt - 1) / vpt > 256) vpt <<= 1;
  int tpr = (n_vec + vpt - 1) / vpt;
  tpr = ((tpr + 31) / 32) * 32;
  return {vpt, tpr};
}

inline int64_t bwd_ctas(int64_t n_rows) {
  const int64_t cap = (int64_t)sm_count() * 4;
  return n_rows < cap ? (n_rows < 1 ? 1 : n_rows) : cap;
}

}  // namespace
}  // namespace soup

extern "C" int soup_rmsnorm_fwd(const void* x, const void* w, void* out, float* rstd, void* low,
                                const int32_t* slot, void* small, int64_t n_small, int64_t n_rows,
                                int64_t n_cols, float eps, int x_dtype, int w_dtype, int out_dtype,
                                void* stream) {
  using namespace soup;
  if (n_rows == 0) return SOUP_OK;
  if (n_rows < 0 || n_cols <= 0 || n_cols > 16384)
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_fwd: need 0 < n_cols <= 16384 (got %lld)", (long long)n_cols);
  if (!x || !w || !out || !rstd) SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_fwd: null pointer");
  if (!is_float_dtype(x_dtype) || !is_float_dtype(w_dtype) || !is_float_dtype(out_dtype))
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_fwd: unsupported dtype");
  if (low && (!slot || !small || n_small < 1))
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_fwd: low copy needs slot map and side buffer");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool vec = (n_cols % 8 == 0) && aligned16(x) && aligned16(w) && aligned16(out) &&
                   (!low || (aligned16(low) && aligned16(slot)));
  if (!vec) {
    rmsnorm_fwd_scalar_kernel<<<(unsigned)n_rows, 256, 0, s>>>(x, w, out, rstd, low, slot, small,
                                                               n_small, (int)n_cols, eps, x_dtype,
                                                               w_dtype, out_dtype);
  } else {
    const Shape sh = pick_shape((int)n_cols);
    constexpr int R = 2;  // rows per CTA step (4 measured slower: fewer CTAs fit on an SM)
    const unsigned grid = (unsigned)((n_rows + R - 1) / R);
#define SOUP_RMS_FWD(V_)                                                                       \
  rmsnorm_fwd_kernel<V_, R><<<grid, sh.tpr, 0, s>>>(x, w, out, rstd, low, slot, small, n_small, \
                                                    n_rows, (int)n_cols, eps, x_dtype, w_dtype, \
                                                    out_dtype)
    switch (sh.vpt) {
      case 1: SOUP_RMS_FWD(1); break;
      case 2: SOUP_RMS_FWD(2); break;
      case 4: SOUP_RMS_FWD(4); break;
      default: SOUP_RMS_FWD(8); break;
    }
#undef SOUP_RMS_FWD
  }
  SOUP_CHECK_LAUNCH("rmsnorm_fwd");
  return SOUP_OK;
}

extern "C" int64_t soup_rmsnorm_bwd_partials(int64_t n_rows, int64_t n_cols) {
  (void)n_cols;
  return soup::bwd_ctas(n_rows);
}

extern "C" int soup_rmsnorm_bwd(const void* dy, const void* xin, const void* w, const float* rstd,
                                void* dx, float* dw_partial, void* dw, const int32_t* slot,
                                const void* small, int64_t n_small, int64_t n_rows, int64_t n_cols,
                                int dy_dtype, int xin_dtype, int w_dtype, int dx_dtype,
                                int saved_output, void* stream) {
  using namespace soup;
  if (n_rows < 0 || n_cols <= 0 || n_cols > 16384)
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd: need 0 < n_cols <= 16384 (got %lld)", (long long)n_cols);
  const bool want_dw = dw != nullptr;
  if (want_dw && !dw_partial) SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd: dw needs the partial workspace");
  if (want_dw && saved_output)
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd: the saved-output path is for a frozen weight (no dw)");
  if (!is_float_dtype(dy_dtype) || !is_float_dtype(xin_dtype) || !is_float_dtype(w_dtype) ||
      !is_float_dtype(dx_dtype))
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd: unsupported dtype");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n_rows == 0) {
    if (want_dw) cudaMemsetAsync(dw, 0, (size_t)n_cols * dtype_size(w_dtype), s);
    return SOUP_OK;
  }
  if (!dy || !xin || !w || !rstd || !dx) SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd: null pointer");
  if (saved_output && (!slot || !small || n_small < 1))
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd: saved-output path needs slot map and side buffer");
  // one row per CTA, or a persistent grid (more CTAs than fit at once) when dw is accumulated
  const unsigned grid = (unsigned)(want_dw ? bwd_ctas(n_rows) : n_rows);
  const bool vec = (n_cols % 8 == 0) && aligned16(dy) && aligned16(xin) && aligned16(w) &&
                   aligned16(dx) && (!saved_output || aligned16(slot)) &&
                   (!want_dw || aligned16(dw_partial));
  if (!vec) {
    if (want_dw)
      rmsnorm_bwd_scalar_kernel<true><<<grid, 256, 0, s>>>(dy, xin, w, rstd, dx, dw_partial, slot,
                                                           small, n_small, n_rows, (int)n_cols,
                                                           dy_dtype, xin_dtype, w_dtype, dx_dtype,
                                                           saved_output);
    else
      rmsnorm_bwd_scalar_kernel<false><<<grid, 256, 0, s>>>(dy, xin, w, rstd, dx, dw_partial, slot,
                                                            small, n_small, n_rows, (int)n_cols,
                                                            dy_dtype, xin_dtype, w_dtype, dx_dtype,
                                                            saved_output);
  } else {
    const Shape sh = pick_shape((int)n_cols);
#define SOUP_RMS_BWD(V_, D_)                                                                     \
  rmsnorm_bwd_kernel<V_, D_><<<grid, sh.tpr, 0, s>>>(dy, xin, w, rstd, dx, dw_partial, slot, small, \
                                                     n_small, n_rows, (int)n_cols, dy_dtype,      \
                                                     xin_dtype, w_dtype, dx_dtype, saved_output)
    if (want_dw) {
      switch (sh.vpt) {
        case 1: SOUP_RMS_BWD(1, true); break;
        case 2: SOUP_RMS_BWD(2, true); break;
        case 4: SOUP_RMS_BWD(4, true); break;
        default: SOUP_RMS_BWD(8, true); break;
      }
    } else {
      switch (sh.vpt) {
        case 1: SOUP_RMS_BWD(1, false); break;
        case 2: SOUP_RMS_BWD(2, false); break;
        case 4: SOUP_RMS_BWD(4, false); break;
        default: SOUP_RMS_BWD(8, false); break;
      }
    }
#undef SOUP_RMS_BWD
  }
  SOUP_CHECK_LAUNCH("rmsnorm_bwd");
  if (want_dw) {
    rmsnorm_dw_reduce_kernel<<<(unsigned)((n_cols + 255) / 256), 256, 0, s>>>(
        dw_partial, dw, (int)grid, (int)n_cols, w_dtype);
    SOUP_CHECK_LAUNCH("rmsnorm_dw_reduce");
  }
  return SOUP_OK;
}


// ------------------------------------------------------------------------------------------
// Backward with the dw workspace inside the library, for callers that cannot allocate.
// ------------------------------------------------------------------------------------------
namespace soup {
namespace {

constexpr int kStaticPartialRows = 640;   // >= 4 CTAs per SM on a 148-SM part (592)
constexpr int kStaticMaxCols = 4096;

// 640 x 4096 fp32 = 10 MiB of device memory per GPU that loads the library, held until exit.
static __device__ __align__(256) float g_dw_scratch[kStaticPartialRows * kStaticMaxCols];

// In host code `g_dw_scratch` is only a handle for the runtime, not a device address; the address
// a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
float* g_dw_scratch_addr[64] = {nullptr};

int static_scratch(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!g_dw_scratch_addr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_dw_scratch);
    if (e != cudaSuccess || !p) {
      set_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return -2;
    }
    g_dw_scratch_addr[dev] = reinterpret_cast<float*>(p);
  }
  *out = g_dw_scratch_addr[dev];
  return 0;
}

}  // namespace
}  // namespace soup

extern "C" int soup_rmsnorm_bwd_noalloc(const void* dy, const void* xin, const void* w,
                                        const float* rstd, void* dx, void* dw, const int32_t* slot,
                                        const void* small, int64_t n_small, int64_t n_rows,
                                        int64_t n_cols, int dy_dtype, int xin_dtype, int w_dtype,
                                        int dx_dtype, int saved_output, void* stream) {
  using namespace soup;
  if (n_cols > kStaticMaxCols)
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd_noalloc: n_cols %lld exceeds the built-in workspace (max %d); "
              "use soup_rmsnorm_bwd with a caller-provided workspace", (long long)n_cols, kStaticMaxCols);
  if (soup_rmsnorm_bwd_partials(n_rows, n_cols) > kStaticPartialRows)
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd_noalloc: this device needs %lld partial rows, the built-in "
              "workspace has %d", (long long)soup_rmsnorm_bwd_partials(n_rows, n_cols), kStaticPartialRows);
  float* scratch = nullptr;
  if (dw) {
    const int rc = static_scratch(&scratch);
    if (rc == -1) SOUP_FAIL(SOUP_ERR_DEVICE, "rmsnorm_bwd_noalloc: no current CUDA device");
    if (rc != 0) return SOUP_ERR_DEVICE;
  }
  // Every partial row the reduce reads is fully rewritten by its CTA first, so nothing in the
  // workspace has to start at zero even though it keeps the previous call's contents.
  return soup_rmsnorm_bwd(dy, xin, w, rstd, dx, scratch, dw, slot, small, n_small, n_rows, n_cols,
                          dy_dtype, xin_dtype, w_dtype, dx_dtype, saved_output, stream);
}
