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
#include "rowpipe.cuh"

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

// ------------------------------------------------------------------------------------------
// Warp-per-row kernels (rows of at most 16 vectors per lane: 2048 fp32 or 4096 16-bit columns).
//
// A warp owns a row: every lane issues all of its 16-byte loads of the row at once, keeps the raw
// bits in registers (4 registers per vector whatever the dtype), reduces with shuffles only (no
// shared memory, no CTA barrier) and streams the results out; then it takes its next row. A lane's
// vector is 16 bytes of the widest streamed input, so every load instruction of the warp covers
// 512 contiguous bytes. With ~50-80 registers per thread 24-36 warps are resident per SM, each
// with a whole row (3-6 KB) in flight, which is what HBM latency x bandwidth asks for.
// ------------------------------------------------------------------------------------------
constexpr int kWarpsPerCta = 8;

template <int EPV>
__device__ __forceinline__ void load_slots(const int32_t* slot, int i, int (&sl)[EPV]) {
#pragma unroll
  for (int q = 0; q < EPV / 4; ++q) {
    const int4 a = *reinterpret_cast<const int4*>(slot + i + 4 * q);
    sl[4 * q] = a.x; sl[4 * q + 1] = a.y; sl[4 * q + 2] = a.z; sl[4 * q + 3] = a.w;
  }
}

// Bit j of the result: vector j of this lane contains a column with a side-buffer slot.
template <int NV, int EPV>
__device__ __forceinline__ uint32_t lane_slot_mask(const int32_t* slot, int n_vec, int lane) {
  uint32_t mask = 0;
  if (!slot) return 0;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int vi = j * 32 + lane;
    if (vi < n_vec) {
      int sl[EPV];
      load_slots<EPV>(slot, vi * EPV, sl);
#pragma unroll
      for (int k = 0; k < EPV; ++k) if (sl[k] >= 0) mask |= 1u << j;
    }
  }
  return mask;
}

// ------------------------------------------------------------------------------------------
// Pipelined warp-per-row kernels: rows arrive in the warp's shared-memory ring (rowpipe.cuh), both
// passes over a row read it from there, results go straight to global memory. Any n_cols whose
// row slot fits the ring; vectors are 16 bytes of the widest streamed input.
// ------------------------------------------------------------------------------------------
template <int EPV, int B>
__device__ __forceinline__ void unpack_smem(const char* row, int vi, int dt, float (&v)[EPV]) {
  unpack<EPV, B>(ld_raw<EPV * B>(row, (int64_t)vi * EPV * B), dt, v);
}

// A dtype that is a template constant (>= 0) is folded by the compiler; -1 takes the run-time code.
template <int C> __device__ __forceinline__ int dt_sel(int rt) { return C >= 0 ? C : rt; }

// XDT / WDT / ODT: compile-time dtype codes of the hot combinations, or -1 for "read the argument".
template <int XB, int XDT, int WDT, int ODT>
__global__ void __launch_bounds__(rowpipe::kMaxWarps * 32, 2)
rmsnorm_fwd_pipe_kernel(const void* __restrict__ x, const void* __restrict__ w,
                        void* __restrict__ out, float* __restrict__ rstd_out,
                        void* __restrict__ low, const int32_t* __restrict__ slot,
                        void* __restrict__ small, int64_t n_small, int64_t n_rows, int n_cols,
                        float eps, int xdt_rt, int wdt_rt, int odt_rt, int stages, int team, int* status) {
  constexpr int EPV = 16 / XB;
  const int xdt = dt_sel<XDT>(xdt_rt), wdt = dt_sel<WDT>(wdt_rt), odt = dt_sel<ODT>(odt_rt);
  extern __shared__ __align__(128) char smem[];
  __shared__ int s_abort;
  __shared__ float s_part[2 * rowpipe::kMaxWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  // a team of `team` (1 or 2) warps shares a row: member m owns vectors [v0, v0 + n_vec)
  const int member = team == 2 ? (warp & 1) : 0;
  const int n_vec = n_cols / EPV / team, v0 = member * n_vec;
  const uint32_t row_bytes = (uint32_t)n_cols * XB / team;   // this member's share of a row
  if (threadIdx.x == 0) s_abort = 0;
  rowpipe::Ring ring;
  ring.init(smem, row_bytes, stages, warp, lane);
  __syncthreads();
  const int64_t row0 = (int64_t)blockIdx.x * (warps / team) + warp / team;
  const int64_t stride = (int64_t)gridDim.x * (warps / team);
  const char* xb = reinterpret_cast<const char*>(x) + (size_t)member * row_bytes;
  const int64_t row_pitch = (int64_t)n_cols * XB;
  int64_t next = row0;   // next row to request
  if (lane == 0) {
    for (int s = 0; s < stages && next < n_rows; ++s, next += stride) {
      umma::mbar_expect_tx(&ring.bars[s], row_bytes);
      rowpipe::bulk_load(ring.slot_ptr(s), xb + next * row_pitch, row_bytes, &ring.bars[s]);
    }
  }
  next = __shfl_sync(0xffffffffu, next, 0);
  // bit v of slot_mask: this lane's v-th vector holds a column with a side-buffer slot
  uint64_t slot_mask = 0;
  if (low) {
    for (int vi = lane, v = 0; vi < n_vec; vi += 32, ++v) {
      int sl[EPV];
      load_slots<EPV>(slot, (v0 + vi) * EPV, sl);
#pragma unroll
      for (int k = 0; k < EPV; ++k) if (sl[k] >= 0) slot_mask |= 1ull << v;
    }
  }
  const float inv_cols = 1.0f / (float)n_cols;
  int iter = 0;
  for (int64_t row = row0; row < n_rows; row += stride, ++iter) {
    if (!ring.wait(&s_abort, status, 11)) {
      ring.drain((int)((next - row) / stride));   // the copies still travelling to this warp's slots
      // a partner already waiting at this row's team barrier is released (it gives up at its next wait)
      if (team == 2) asm volatile("bar.arrive %0, 64;" ::"r"((warp >> 1) + 1) : "memory");
      return;
    }
    const char* src = ring.slot_ptr(ring.slot);
    float ss = 0.f;
#pragma unroll 4
    for (int vi = lane; vi < n_vec; vi += 32) {
      float xv[EPV];
      unpack_smem<EPV, XB>(src, vi, xdt, xv);
#pragma unroll
      for (int k = 0; k < EPV; ++k) ss += xv[k] * xv[k];
    }
    ss = warp_sum(ss);
    if (team == 2) ss = rowpipe::team_sum2(ss, s_part, warp, lane, iter);
    const float rstd = 1.0f / sqrtf(ss * inv_cols + eps);
    if (lane == 0 && member == 0) rstd_out[row] = rstd;
    int v = 0;
#pragma unroll 2
    for (int vi = lane; vi < n_vec; vi += 32, ++v) {
      float xv[EPV], wv[EPV], o[EPV], nrm[EPV];
      unpack_smem<EPV, XB>(src, vi, xdt, xv);
      const int col = (v0 + vi) * EPV;
      loadv<EPV>(w, col, wdt, wv);   // a few KB of weights: L1-resident after the first row
#pragma unroll
      for (int k = 0; k < EPV; ++k) {
        nrm[k] = round_through(xv[k] * rstd, xdt);
        o[k] = nrm[k] * wv[k];
      }
      storev<EPV>(out, row * n_cols + col, odt, o);
      if (low) {
        storev<EPV>(low, row * n_cols + col, SOUP_F16, o);
        if (slot_mask >> v & 1ull) {
          int sl[EPV];
          load_slots<EPV>(slot, col, sl);
#pragma unroll
          for (int k = 0; k < EPV; ++k)
            if (sl[k] >= 0) store1(small, row * n_small + sl[k], SOUP_F16, nrm[k]);
        }
      }
    }
    __syncwarp();
    if (next < n_rows) {
      if (lane == 0) {
        umma::fence_proxy_async_smem();   // the slot's reads are done before the copy overwrites it
        umma::mbar_expect_tx(&ring.bars[ring.slot], row_bytes);
        rowpipe::bulk_load(ring.slot_ptr(ring.slot), xb + next * row_pitch, row_bytes,
                           &ring.bars[ring.slot]);
      }
      next += stride;
    }
    ring.advance();
  }
}

// Backward without dw: a slot holds the dy row followed by the saved row (x, or the fp16 copy of
// the output). YDT .. SAVED: compile-time values of the hot combinations, or -1 for the argument.
template <int YB, int XB, int YDT, int XDT, int WDT, int DXDT, int SAVED>
__global__ void __launch_bounds__(rowpipe::kMaxWarps * 32, 2)
rmsnorm_bwd_pipe_kernel(const void* __restrict__ dy, const void* __restrict__ xin,
                        const void* __restrict__ w, const float* __restrict__ rstd_in,
                        void* __restrict__ dx, const int32_t* __restrict__ slot,
                        const void* __restrict__ small, int64_t n_small, int64_t n_rows, int n_cols,
                        int ydt_rt, int xdt_rt, int wdt_rt, int dxdt_rt, int saved_rt, int stages,
                        int team, int* status) {
  constexpr int EPV = 16 / (YB > XB ? YB : XB);
  const int ydt = dt_sel<YDT>(ydt_rt), xdt = dt_sel<XDT>(xdt_rt), wdt = dt_sel<WDT>(wdt_rt);
  const int dxdt = dt_sel<DXDT>(dxdt_rt), saved_output = dt_sel<SAVED>(saved_rt);
  extern __shared__ __align__(128) char smem[];
  __shared__ int s_abort;
  __shared__ float s_part[2 * rowpipe::kMaxWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int member = team == 2 ? (warp & 1) : 0;
  const int n_vec = n_cols / EPV / team, v0 = member * n_vec;
  // this member's share of a dy row and of a saved row
  const uint32_t y_bytes = (uint32_t)n_cols * YB / team, x_bytes = (uint32_t)n_cols * XB / team;
  const int64_t y_pitch = (int64_t)n_cols * YB, x_pitch = (int64_t)n_cols * XB;
  if (threadIdx.x == 0) s_abort = 0;
  rowpipe::Ring ring;
  ring.init(smem, y_bytes + x_bytes, stages, warp, lane);
  __syncthreads();
  const int64_t row0 = (int64_t)blockIdx.x * (warps / team) + warp / team;
  const int64_t stride = (int64_t)gridDim.x * (warps / team);
  const char* yb = reinterpret_cast<const char*>(dy) + (size_t)member * y_bytes;
  const char* xb = reinterpret_cast<const char*>(xin) + (size_t)member * x_bytes;
  int64_t next = row0;
  if (lane == 0) {
    for (int s = 0; s < stages && next < n_rows; ++s, next += stride) {
      umma::mbar_expect_tx(&ring.bars[s], y_bytes + x_bytes);
      rowpipe::bulk_load(ring.slot_ptr(s), yb + next * y_pitch, y_bytes, &ring.bars[s]);
      rowpipe::bulk_load(ring.slot_ptr(s) + y_bytes, xb + next * x_pitch, x_bytes, &ring.bars[s]);
    }
  }
  next = __shfl_sync(0xffffffffu, next, 0);
  uint64_t slot_mask = 0;
  if (saved_output) {
    for (int vi = lane, v = 0; vi < n_vec; vi += 32, ++v) {
      int sl[EPV];
      load_slots<EPV>(slot, (v0 + vi) * EPV, sl);
#pragma unroll
      for (int k = 0; k < EPV; ++k) if (sl[k] >= 0) slot_mask |= 1ull << v;
    }
  }
  const float inv_cols = 1.0f / (float)n_cols;
  int iter = 0;
  for (int64_t row = row0; row < n_rows; row += stride, ++iter) {
    if (!ring.wait(&s_abort, status, 12)) {
      ring.drain((int)((next - row) / stride));
      if (team == 2) asm volatile("bar.arrive %0, 64;" ::"r"((warp >> 1) + 1) : "memory");
      return;
    }
    const char* ysrc = ring.slot_ptr(ring.slot);
    const char* xsrc = ysrc + y_bytes;
    const float rstd = rstd_in[row];
    float dot = 0.f;
    int v = 0;
#pragma unroll 2
    for (int vi = lane; vi < n_vec; vi += 32, ++v) {
      float yv[EPV], xv[EPV], wv[EPV];
      unpack_smem<EPV, YB>(ysrc, vi, ydt, yv);
      unpack_smem<EPV, XB>(xsrc, vi, xdt, xv);
      const int col = (v0 + vi) * EPV;
      loadv<EPV>(w, col, wdt, wv);
      int sl[EPV];
#pragma unroll
      for (int k = 0; k < EPV; ++k) sl[k] = -1;
      if (slot_mask >> v & 1ull) load_slots<EPV>(slot, col, sl);
#pragma unroll
      for (int k = 0; k < EPV; ++k) {
        float nrm, gn;
        if (saved_output) {
          nrm = sl[k] >= 0 ? load1(small, row * n_small + sl[k], SOUP_F16) : xv[k] / wv[k];
          gn = yv[k] * wv[k];
        } else {
          nrm = xv[k] * rstd;
          gn = round_through(yv[k] * wv[k], xdt);
        }
        dot += gn * nrm;
      }
    }
    dot = warp_sum(dot);
    if (team == 2) dot = rowpipe::team_sum2(dot, s_part, warp, lane, iter);
    const float mean_dot = dot * inv_cols;
    v = 0;
#pragma unroll 2
    for (int vi = lane; vi < n_vec; vi += 32, ++v) {
      float yv[EPV], xv[EPV], wv[EPV], o[EPV];
      unpack_smem<EPV, YB>(ysrc, vi, ydt, yv);
      unpack_smem<EPV, XB>(xsrc, vi, xdt, xv);
      const int col = (v0 + vi) * EPV;
      loadv<EPV>(w, col, wdt, wv);
      int sl[EPV];
#pragma unroll
      for (int k = 0; k < EPV; ++k) sl[k] = -1;
      if (slot_mask >> v & 1ull) load_slots<EPV>(slot, col, sl);
#pragma unroll
      for (int k = 0; k < EPV; ++k) {
        float nrm, gn;
        if (saved_output) {
          nrm = sl[k] >= 0 ? load1(small, row * n_small + sl[k], SOUP_F16) : xv[k] / wv[k];
          gn = yv[k] * wv[k];
        } else {
          nrm = xv[k] * rstd;
          gn = round_through(yv[k] * wv[k], xdt);
        }
        o[k] = (gn - nrm * mean_dot) * rstd;
      }
      storev<EPV>(dx, row * n_cols + col, dxdt, o);
    }
    __syncwarp();
    if (next < n_rows) {
      if (lane == 0) {
        umma::fence_proxy_async_smem();
        umma::mbar_expect_tx(&ring.bars[ring.slot], y_bytes + x_bytes);
        rowpipe::bulk_load(ring.slot_ptr(ring.slot), yb + next * y_pitch, y_bytes,
                           &ring.bars[ring.slot]);
        rowpipe::bulk_load(ring.slot_ptr(ring.slot) + y_bytes, xb + next * x_pitch, x_bytes,
                           &ring.bars[ring.slot]);
      }
      next += stride;
    }
    ring.advance();
  }
}

// The 4-bit model's backward: fp32 dy, the fp16 copy of the forward's output as the saved tensor,
// fp32 weight and dx. Only dy travels through the warp's ring; the saved row, half as many bytes,
// comes through plain 8-byte loads into registers one row ahead (as RoPE's cos/sin rows do). That
// halves the bulk copies per row (the copy engine has a cost per copy) and leaves the ring two
// stages where a slot of dy + saved row had room for one. NVX: 4-element vectors per lane.
template <int NVX>
__global__ void __launch_bounds__(rowpipe::kMaxWarps * 32, 2)
rmsnorm_bwd_saved_kernel(const float* __restrict__ dy, const __half* __restrict__ saved,
                         const float* __restrict__ w, const float* __restrict__ rstd_in,
                         const float* __restrict__ add, float* __restrict__ dx,
                         __half* __restrict__ dx16, const int32_t* __restrict__ slot,
                         const __half* __restrict__ small, int64_t n_small, int64_t n_rows,
                         int n_cols, int stages, int team, int w_offset, int* status) {
  constexpr int EPV = 4;
  extern __shared__ __align__(128) char smem[];
  __shared__ int s_abort;
  __shared__ float s_part[2 * rowpipe::kMaxWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int member = team == 2 ? (warp & 1) : 0;
  const int n_vec = n_cols / EPV / team, v0 = member * n_vec;
  const uint32_t y_bytes = (uint32_t)n_cols * 4 / team;
  const int64_t y_pitch = (int64_t)n_cols * 4;
  if (threadIdx.x == 0) s_abort = 0;
  rowpipe::Ring ring;
  ring.init(smem, y_bytes, stages, warp, lane);
  __syncthreads();
  const int64_t row0 = (int64_t)blockIdx.x * (warps / team) + warp / team;
  const int64_t stride = (int64_t)gridDim.x * (warps / team);
  const char* yb = reinterpret_cast<const char*>(dy) + (size_t)member * y_bytes;
  const __half* xb = saved + (size_t)v0 * EPV;
  int64_t next = row0;
  if (lane == 0) {
    for (int s = 0; s < stages && next < n_rows; ++s, next += stride) {
      umma::mbar_expect_tx(&ring.bars[s], y_bytes);
      rowpipe::bulk_load(ring.slot_ptr(s), yb + next * y_pitch, y_bytes, &ring.bars[s]);
    }
  }
  next = __shfl_sync(0xffffffffu, next, 0);
  // The weight and its reciprocal, needed by every row, sit in shared memory behind the ring
  // (registers are taken by the two saved rows in flight and the normalised values).
  float* s_w = reinterpret_cast<float*>(smem + w_offset);
  float* s_winv = s_w + n_cols;
  for (int c = threadIdx.x; c < n_cols; c += blockDim.x) {
    const float wc = w[c];
    s_w[c] = wc;
    s_winv[c] = 1.0f / wc;
  }
  __syncthreads();
  uint32_t slot_mask = 0;
#pragma unroll
  for (int v = 0; v < NVX; ++v) {
    const int vi = lane + 32 * v;
    if (vi < n_vec) {
      int sl[EPV];
      load_slots<EPV>(slot, (v0 + vi) * EPV, sl);
#pragma unroll
      for (int k = 0; k < EPV; ++k)
        if (sl[k] >= 0) slot_mask |= 1u << v;
    }
  }
  Raw<8> xcur[NVX], xnxt[NVX];
  auto fetch_saved = [&](int64_t row, Raw<8> (&dst)[NVX]) {
#pragma unroll
    for (int v = 0; v < NVX; ++v) {
      const int vi = lane + 32 * v;
      if (vi < n_vec) dst[v] = ld_raw<8>(xb, (row * n_cols + (int64_t)vi * EPV) * 2);
    }
  };
  if (row0 < n_rows) fetch_saved(row0, xcur);
  const float inv_cols = 1.0f / (float)n_cols;
  int iter = 0;
  for (int64_t row = row0; row < n_rows; row += stride, ++iter) {
    if (row + stride < n_rows) fetch_saved(row + stride, xnxt);
    if (!ring.wait(&s_abort, status, 12)) {
      ring.drain((int)((next - row) / stride));
      if (team == 2) asm volatile("bar.arrive %0, 64;" ::"r"((warp >> 1) + 1) : "memory");
      return;
    }
    const char* ysrc = ring.slot_ptr(ring.slot);
    const float rstd = rstd_in[row];
    // the normalised value: saved / w, except in the side-buffer columns (|w| tiny)
    float nrm[NVX][EPV];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < NVX; ++v) {
      const int vi = lane + 32 * v;
      if (vi < n_vec) {
        float yv[EPV], xv[EPV];
        unpack_smem<EPV, 4>(ysrc, vi, SOUP_F32, yv);
        unpack<EPV, 2>(xcur[v], SOUP_F16, xv);
        const float4 wq = *reinterpret_cast<const float4*>(s_w + (v0 + vi) * EPV);
        const float4 iq = *reinterpret_cast<const float4*>(s_winv + (v0 + vi) * EPV);
        const float wv[EPV] = {wq.x, wq.y, wq.z, wq.w}, winv[EPV] = {iq.x, iq.y, iq.z, iq.w};
        int sl[EPV];
#pragma unroll
        for (int k = 0; k < EPV; ++k) sl[k] = -1;
        if (slot_mask >> v & 1u) load_slots<EPV>(slot, (v0 + vi) * EPV, sl);
#pragma unroll
        for (int k = 0; k < EPV; ++k) {
          nrm[v][k] = sl[k] >= 0 ? __half2float(small[row * n_small + sl[k]]) : xv[k] * winv[k];
          dot += yv[k] * wv[k] * nrm[v][k];
        }
      }
    }
    dot = warp_sum(dot);
    if (team == 2) dot = rowpipe::team_sum2(dot, s_part, warp, lane, iter);
    const float mean_dot = dot * inv_cols;
#pragma unroll
    for (int v = 0; v < NVX; ++v) {
      const int vi = lane + 32 * v;
      if (vi < n_vec) {
        float yv[EPV];
        unpack_smem<EPV, 4>(ysrc, vi, SOUP_F32, yv);
        const float4 wq = *reinterpret_cast<const float4*>(s_w + (v0 + vi) * EPV);
        float4 o;
        o.x = (yv[0] * wq.x - nrm[v][0] * mean_dot) * rstd;
        o.y = (yv[1] * wq.y - nrm[v][1] * mean_dot) * rstd;
        o.z = (yv[2] * wq.z - nrm[v][2] * mean_dot) * rstd;
        o.w = (yv[3] * wq.w - nrm[v][3] * mean_dot) * rstd;
        const int64_t at = row * n_cols + (int64_t)(v0 + vi) * EPV;
        if (add) {   // the gradient that reaches the same tensor along the residual connection
          const float4 r = *reinterpret_cast<const float4*>(add + at);
          o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
        }
        *reinterpret_cast<float4*>(dx + at) = o;
        if (dx16) {  // and its fp16 copy, for the projection backward that receives it next
          __half2 lo = __floats2half2_rn(o.x, o.y), hi = __floats2half2_rn(o.z, o.w);
          uint2 packed;
          packed.x = *reinterpret_cast<uint32_t*>(&lo);
          packed.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(dx16 + at) = packed;
        }
      }
    }
    __syncwarp();
    if (next < n_rows) {
      if (lane == 0) {
        umma::fence_proxy_async_smem();
        umma::mbar_expect_tx(&ring.bars[ring.slot], y_bytes);
        rowpipe::bulk_load(ring.slot_ptr(ring.slot), yb + next * y_pitch, y_bytes, &ring.bars[ring.slot]);
      }
      next += stride;
    }
    ring.advance();
#pragma unroll
    for (int v = 0; v < NVX; ++v) xcur[v] = xnxt[v];
  }
}

// YB / XB: bytes per element of dy and of the saved tensor (x, or the fp16 copy of the output).
template <int NV, int YB, int XB, bool DW>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
rmsnorm_bwd_warp_kernel(const void* __restrict__ dy, const void* __restrict__ xin,
                        const void* __restrict__ w, const float* __restrict__ rstd_in,
                        void* __restrict__ dx, float* __restrict__ dw_partial,
                        const int32_t* __restrict__ slot, const void* __restrict__ small,
                        int64_t n_small, int64_t n_rows, int n_cols, int ydt, int xdt, int wdt,
                        int dxdt, int saved_output) {
  constexpr int EPV = 16 / (YB > XB ? YB : XB);
  extern __shared__ float s_dw[];   // DW only: n_cols floats
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_vec = n_cols / EPV;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerCta + warp;
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerCta;
  const uint32_t slot_mask = saved_output ? lane_slot_mask<NV, EPV>(slot, n_vec, lane) : 0u;
  const float inv_cols = 1.0f / (float)n_cols;
  float dw_acc[DW ? NV : 1][EPV];
  if (DW) {
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int k = 0; k < EPV; ++k) dw_acc[j][k] = 0.f;
  }
  for (int64_t row = warp0; row < n_rows; row += stride) {
    Raw<EPV * YB> yraw[NV];
    Raw<EPV * XB> xraw[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vi = j * 32 + lane;
      if (vi < n_vec) {
        const int64_t e = row * n_cols + (int64_t)vi * EPV;
        yraw[j] = ld_raw<EPV * YB>(dy, e * YB);
        xraw[j] = ld_raw<EPV * XB>(xin, e * XB);
      }
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vi = j * 32 + lane;
      if (vi < n_vec) {
        float yv[EPV], xv[EPV], wv[EPV];
        unpack<EPV, YB>(yraw[j], ydt, yv);
        unpack<EPV, XB>(xraw[j], xdt, xv);
        loadv<EPV>(w, vi * EPV, wdt, wv);
        int sl[EPV];
#pragma unroll
        for (int k = 0; k < EPV; ++k) sl[k] = -1;
        if (slot_mask >> j & 1u) load_slots<EPV>(slot, vi * EPV, sl);
#pragma unroll
        for (int k = 0; k < EPV; ++k) {
          float nrm, gn;
          if (saved_output) {
            nrm = sl[k] >= 0 ? load1(small, row * n_small + sl[k], SOUP_F16) : xv[k] / wv[k];
            gn = yv[k] * wv[k];
          } else {
            nrm = xv[k] * rstd;
            gn = round_through(yv[k] * wv[k], xdt);
          }
          dot += gn * nrm;
          if (DW) dw_acc[j][k] += yv[k] * round_through(nrm, xdt);
        }
      }
    }
    dot = warp_sum(dot);
    const float mean_dot = dot * inv_cols;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vi = j * 32 + lane;
      if (vi < n_vec) {
        float yv[EPV], xv[EPV], wv[EPV], o[EPV];
        unpack<EPV, YB>(yraw[j], ydt, yv);
        unpack<EPV, XB>(xraw[j], xdt, xv);
        loadv<EPV>(w, vi * EPV, wdt, wv);
        int sl[EPV];
#pragma unroll
        for (int k = 0; k < EPV; ++k) sl[k] = -1;
        if (slot_mask >> j & 1u) load_slots<EPV>(slot, vi * EPV, sl);
#pragma unroll
        for (int k = 0; k < EPV; ++k) {
          float nrm, gn;
          if (saved_output) {
            nrm = sl[k] >= 0 ? load1(small, row * n_small + sl[k], SOUP_F16) : xv[k] / wv[k];
            gn = yv[k] * wv[k];
          } else {
            nrm = xv[k] * rstd;
            gn = round_through(yv[k] * wv[k], xdt);
          }
          o[k] = (gn - nrm * mean_dot) * rstd;
        }
        storev<EPV>(dx, row * n_cols + (int64_t)vi * EPV, dxdt, o);
      }
    }
  }
  if (DW) {
    // The CTA's warps add their column sums in warp order (deterministic), one partial row per CTA.
    for (int turn = 0; turn < kWarpsPerCta; ++turn) {
      if (warp == turn) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int vi = j * 32 + lane;
          if (vi < n_vec) {
#pragma unroll
            for (int k = 0; k < EPV; ++k) {
              const int c = vi * EPV + k;
              s_dw[c] = turn == 0 ? dw_acc[j][k] : s_dw[c] + dw_acc[j][k];
            }
          }
        }
      }
      __syncthreads();
    }
    for (int c = threadIdx.x; c < n_cols; c += blockDim.x)
      dw_partial[(int64_t)blockIdx.x * n_cols + c] = s_dw[c];
  }
}

// Vectors per lane the warp kernels are built for; 0: the row is too wide for them.
inline int pick_nv(int n_cols, int epv) {
  const int need = (n_cols / epv + 31) / 32;
  const int options[] = {2, 4, 6, 8, 12, 16};
  for (int o : options) if (need <= o) return o;
  return 0;
}

inline unsigned warp_grid(int64_t n_rows, int ctas_per_sm) {
  const int64_t need = (n_rows + kWarpsPerCta - 1) / kWarpsPerCta;
  const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
  return (unsigned)(need < cap ? (need < 1 ? 1 : need) : cap);
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
  const int xb = dtype_size(x_dtype);
  // a team of two can split a row whose halves are whole 16-byte vectors
  const rowpipe::Plan plan = vec ? rowpipe::make_plan((size_t)n_cols * xb, 0, (n_cols * xb) % 32 == 0, n_rows)
                                 : rowpipe::Plan{8, 0, 1, 1, 0, 0};
  int* status = plan.stages ? rowpipe::status_word() : nullptr;
  if (!vec) {
    rmsnorm_fwd_scalar_kernel<<<(unsigned)n_rows, 256, 0, s>>>(x, w, out, rstd, low, slot, small,
                                                               n_small, (int)n_cols, eps, x_dtype,
                                                               w_dtype, out_dtype);
  } else if (plan.stages && status) {
#define SOUP_RMS_FWD_P(XB_, X_, W_, O_)                                                          \
  do {                                                                                            \
    auto kernel = rmsnorm_fwd_pipe_kernel<XB_, X_, W_, O_>;                                       \
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);    \
    kernel<<<plan.grid, plan.warps * 32, plan.smem, s>>>(x, w, out, rstd, low, slot, small,       \
                                                         n_small, n_rows, (int)n_cols, eps,       \
                                                         x_dtype, w_dtype, out_dtype, plan.stages, \
                                                         plan.team, status);                      \
  } while (0)
    const bool same = x_dtype == w_dtype && x_dtype == out_dtype;
    if (same && x_dtype == SOUP_F32) SOUP_RMS_FWD_P(4, SOUP_F32, SOUP_F32, SOUP_F32);
    else if (same && x_dtype == SOUP_F16) SOUP_RMS_FWD_P(2, SOUP_F16, SOUP_F16, SOUP_F16);
    else if (same && x_dtype == SOUP_BF16) SOUP_RMS_FWD_P(2, SOUP_BF16, SOUP_BF16, SOUP_BF16);
    else if (xb == 4) SOUP_RMS_FWD_P(4, SOUP_F32, -1, -1);
    else SOUP_RMS_FWD_P(2, -1, -1, -1);
#undef SOUP_RMS_FWD_P
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

namespace soup {
namespace {
int rmsnorm_bwd_any(const void* dy, const void* xin, const void* w, const float* rstd, void* dx,
                    float* dw_partial, void* dw, const int32_t* slot, const void* small,
                    int64_t n_small, int64_t n_rows, int64_t n_cols, int dy_dtype, int xin_dtype,
                    int w_dtype, int dx_dtype, int saved_output, const float* add, __half* dx16,
                    void* stream);
}  // namespace
}  // namespace soup

extern "C" int soup_rmsnorm_bwd(const void* dy, const void* xin, const void* w, const float* rstd,
                                void* dx, float* dw_partial, void* dw, const int32_t* slot,
                                const void* small, int64_t n_small, int64_t n_rows, int64_t n_cols,
                                int dy_dtype, int xin_dtype, int w_dtype, int dx_dtype,
                                int saved_output, void* stream) {
  return soup::rmsnorm_bwd_any(dy, xin, w, rstd, dx, dw_partial, dw, slot, small, n_small, n_rows,
                               n_cols, dy_dtype, xin_dtype, w_dtype, dx_dtype, saved_output, nullptr,
                               nullptr, stream);
}

extern "C" int soup_rmsnorm_bwd_residual(const float* dy, const void* low, const float* w,
                                         const float* rstd, const float* add, float* dx, void* dx16,
                                         const int32_t* slot, const void* small, int64_t n_small,
                                         int64_t n_rows, int64_t n_cols, void* stream) {
  if (add && (reinterpret_cast<uintptr_t>(add) & 15u))
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd_residual: the residual gradient must be 16-byte aligned");
  if (dx16 && (reinterpret_cast<uintptr_t>(dx16) & 7u))
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd_residual: the fp16 copy must be 8-byte aligned");
  return soup::rmsnorm_bwd_any(dy, low, w, rstd, dx, nullptr, nullptr, slot, small, n_small, n_rows,
                               n_cols, SOUP_F32, SOUP_F16, SOUP_F32, SOUP_F32, 1, add,
                               reinterpret_cast<__half*>(dx16), stream);
}

namespace soup {
namespace {
int rmsnorm_bwd_any(const void* dy, const void* xin, const void* w, const float* rstd, void* dx,
                    float* dw_partial, void* dw, const int32_t* slot, const void* small,
                    int64_t n_small, int64_t n_rows, int64_t n_cols, int dy_dtype, int xin_dtype,
                    int w_dtype, int dx_dtype, int saved_output, const float* add, __half* dx16,
                    void* stream) {
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
  // Rows of moderate width go to the warp-per-row kernel; wider ones to one CTA per row (a
  // persistent grid when dw is accumulated). A 16-bit dy with a 32-bit saved tensor does not occur
  // on the training path and takes the CTA kernel.
  const bool vec = (n_cols % 8 == 0) && aligned16(dy) && aligned16(xin) && aligned16(w) &&
                   aligned16(dx) && (!saved_output || aligned16(slot)) &&
                   (!want_dw || aligned16(dw_partial));
  const int yb = dtype_size(dy_dtype), xb = dtype_size(xin_dtype);
  const int nv = (vec && want_dw && yb >= xb) ? pick_nv((int)n_cols, 16 / yb) : 0;
  const rowpipe::Plan plan = (vec && !want_dw && yb >= xb)
                                 ? rowpipe::make_plan((size_t)n_cols * (yb + xb), 0,
                                                      (n_cols * xb) % 32 == 0, n_rows)
                                 : rowpipe::Plan{8, 0, 1, 1, 0, 0};
  int* status = plan.stages ? rowpipe::status_word() : nullptr;
  unsigned grid = (unsigned)(want_dw ? bwd_ctas(n_rows) : n_rows);
  if ((add || dx16) && !(vec && plan.stages && status))
    SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd_residual: this shape does not take the residual form");
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
  } else if (plan.stages && status) {
    grid = plan.grid;
#define SOUP_RMS_BWD_P(YB_, XB_, Y_, X_, W_, DX_, SV_)                                           \
  do {                                                                                            \
    auto kernel = rmsnorm_bwd_pipe_kernel<YB_, XB_, Y_, X_, W_, DX_, SV_>;                        \
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);    \
    kernel<<<plan.grid, plan.warps * 32, plan.smem, s>>>(dy, xin, w, rstd, dx, slot, small,       \
                                                         n_small, n_rows, (int)n_cols, dy_dtype,  \
                                                         xin_dtype, w_dtype, dx_dtype,            \
                                                         saved_output, plan.stages, plan.team,    \
                                                         status);                                 \
  } while (0)
    const bool same = dy_dtype == xin_dtype && dy_dtype == w_dtype && dy_dtype == dx_dtype;
    const bool four_bit = saved_output && dy_dtype == SOUP_F32 && xin_dtype == SOUP_F16 &&
                          w_dtype == SOUP_F32 && dx_dtype == SOUP_F32;
    // the 4-bit model's path with the saved row through registers: the ring carries dy only
    const rowpipe::Plan plan_y = four_bit ? rowpipe::make_plan((size_t)n_cols * 4, 0, (n_cols * 2) % 32 == 0, n_rows)
                                          : rowpipe::Plan{8, 0, 1, 1, 0, 0};
    const int per_lane = plan_y.stages ? (int)((n_cols / 4 / plan_y.team + 31) / 32) : 0;
    // weight and reciprocal behind the ring; two CTAs of this size must still fit an SM
    const size_t w_off = (plan_y.smem + 15) / 16 * 16;
    const size_t smem_y = w_off + 2 * (size_t)n_cols * sizeof(float);
    const bool saved_kernel = four_bit && plan_y.stages >= 1 && per_lane >= 1 && per_lane <= 8 &&
                              smem_y <= 112 * 1024;
    if ((add || dx16) && !saved_kernel)
      SOUP_FAIL(SOUP_ERR_ARG, "rmsnorm_bwd_residual: this shape does not take the residual form");
    if (saved_kernel) {
      grid = plan_y.grid;
#define SOUP_RMS_BWD_S(NVX_)                                                                     \
  do {                                                                                            \
    auto kernel = rmsnorm_bwd_saved_kernel<NVX_>;                                                 \
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_y);       \
    kernel<<<plan_y.grid, plan_y.warps * 32, smem_y, s>>>(                                        \
        reinterpret_cast<const float*>(dy), reinterpret_cast<const __half*>(xin),                 \
        reinterpret_cast<const float*>(w), rstd, add, reinterpret_cast<float*>(dx), dx16, slot,   \
        reinterpret_cast<const __half*>(small), n_small, n_rows, (int)n_cols, plan_y.stages,      \
        plan_y.team, (int)w_off, status);                                                         \
  } while (0)
      if (per_lane <= 2) SOUP_RMS_BWD_S(2);
      else if (per_lane <= 4) SOUP_RMS_BWD_S(4);
      else if (per_lane <= 6) SOUP_RMS_BWD_S(6);
      else SOUP_RMS_BWD_S(8);
#undef SOUP_RMS_BWD_S
    } else if (four_bit)
      SOUP_RMS_BWD_P(4, 2, SOUP_F32, SOUP_F16, SOUP_F32, SOUP_F32, 1);
    else if (!saved_output && same && dy_dtype == SOUP_F16)
      SOUP_RMS_BWD_P(2, 2, SOUP_F16, SOUP_F16, SOUP_F16, SOUP_F16, 0);
    else if (!saved_output && same && dy_dtype == SOUP_BF16)
      SOUP_RMS_BWD_P(2, 2, SOUP_BF16, SOUP_BF16, SOUP_BF16, SOUP_BF16, 0);
    else if (!saved_output && same && dy_dtype == SOUP_F32)
      SOUP_RMS_BWD_P(4, 4, SOUP_F32, SOUP_F32, SOUP_F32, SOUP_F32, 0);
    else if (yb == 4 && xb == 4) SOUP_RMS_BWD_P(4, 4, SOUP_F32, SOUP_F32, -1, -1, -1);
    else if (yb == 4) SOUP_RMS_BWD_P(4, 2, SOUP_F32, -1, -1, -1, -1);
    else SOUP_RMS_BWD_P(2, 2, -1, -1, -1, -1, -1);
#undef SOUP_RMS_BWD_P
  } else if (nv) {
    grid = warp_grid(n_rows, 2);
    const size_t smem = (size_t)n_cols * sizeof(float);
#define SOUP_RMS_BWD_W(NV_, YB_, XB_)                                                            \
  rmsnorm_bwd_warp_kernel<NV_, YB_, XB_, true><<<grid, kWarpsPerCta * 32, smem, s>>>(             \
      dy, xin, w, rstd, dx, dw_partial, slot, small, n_small, n_rows, (int)n_cols, dy_dtype,      \
      xin_dtype, w_dtype, dx_dtype, saved_output)
#define SOUP_RMS_BWD_NV(YB_, XB_)                                                                \
  switch (nv) {                                                                                   \
    case 2: SOUP_RMS_BWD_W(2, YB_, XB_); break;                                                   \
    case 4: SOUP_RMS_BWD_W(4, YB_, XB_); break;                                                   \
    case 6: SOUP_RMS_BWD_W(6, YB_, XB_); break;                                                   \
    case 8: SOUP_RMS_BWD_W(8, YB_, XB_); break;                                                   \
    case 12: SOUP_RMS_BWD_W(12, YB_, XB_); break;                                                 \
    default: SOUP_RMS_BWD_W(16, YB_, XB_); break;                                                 \
  }
    if (yb == 4 && xb == 4) { SOUP_RMS_BWD_NV(4, 4) }
    else if (yb == 4) { SOUP_RMS_BWD_NV(4, 2) }
    else { SOUP_RMS_BWD_NV(2, 2) }
#undef SOUP_RMS_BWD_NV
#undef SOUP_RMS_BWD_W
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
}  // namespace
}  // namespace soup


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
