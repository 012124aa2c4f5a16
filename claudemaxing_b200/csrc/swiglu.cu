// SwiGLU activation of the MLP: silu(gate) * up forward, and the recomputing backward that keeps
// nothing but gate and up and may write its two gradients over them.
//
// Both kernels stream: each thread owns 8 consecutive elements per step (128-bit accesses for
// 16-bit dtypes, two for fp32) and takes two steps so that enough loads are in flight to cover
// HBM latency. The rounding points follow solution/swiglu_recompute.py:36-79 of the reference:
// silu is computed in fp32 as g / (1 + 2^(-g*log2 e)), rounded to the gate dtype when round_silu,
// and only then multiplied by up; dy*up is rounded the same way before it meets silu'.
#include "common.cuh"
#include "rowpipe.cuh"

namespace soup {
namespace {

constexpr int kThreads = 256;
constexpr int kSteps = 2;      // forward: vectors per thread
constexpr int kStepsBwd = 2;   // backward: same depth (4 vectors per thread measured slower: fewer CTAs fit)
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float silu_denom(float g) { return 1.0f + exp2f(g * -kLog2e); }

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
silu_mul_fwd_kernel(const void* __restrict__ gate, const void* __restrict__ up,
                    void* __restrict__ out, int64_t n, int gdt, int udt, int odt, int round_silu) {
  if (VEC) {
    const int64_t n8 = n >> 3;
    const int64_t v0 = (int64_t)blockIdx.x * (kThreads * kSteps) + threadIdx.x;
    float g[kSteps][8], u[kSteps][8];
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      const int64_t v = v0 + (int64_t)s * kThreads;
      if (v < n8) { load8(gate, v << 3, gdt, g[s]); load8(up, v << 3, udt, u[s]); }
    }
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      const int64_t v = v0 + (int64_t)s * kThreads;
      if (v >= n8) continue;
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float silu = __fdividef(g[s][k], silu_denom(g[s][k]));
        if (round_silu) silu = round_through(silu, gdt);
        o[k] = silu * u[s][k];
      }
      store8(out, v << 3, odt, o);
    }
    if (blockIdx.x == 0) {  // ragged tail, at most 7 elements
      for (int64_t i = (n8 << 3) + threadIdx.x; i < n; i += kThreads) {
        const float gv = load1(gate, i, gdt);
        float silu = __fdividef(gv, silu_denom(gv));
        if (round_silu) silu = round_through(silu, gdt);
        store1(out, i, odt, silu * load1(up, i, udt));
      }
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * kThreads) {
      const float gv = load1(gate, i, gdt);
      float silu = __fdividef(gv, silu_denom(gv));
      if (round_silu) silu = round_through(silu, gdt);
      store1(out, i, odt, silu * load1(up, i, udt));
    }
  }
}

__device__ __forceinline__ void bwd_elem(float dy, float g, float u, int gdt, int round_silu,
                                         float& d_gate, float& d_up) {
  const float sig = __fdividef(1.0f, silu_denom(g));
  float silu = g * sig;
  float d_silu = dy * u;
  if (round_silu) {
    silu = round_through(silu, gdt);
    d_silu = round_through(d_silu, gdt);
  }
  d_up = dy * silu;
  d_gate = d_silu * sig * (1.0f + g * (1.0f - sig));
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
silu_mul_bwd_kernel(const void* __restrict__ dy, const void* gate, const void* up, void* dgate,
                    void* dup, int64_t n, int ydt, int gdt, int udt, int round_silu) {
  // gate/up are not __restrict__: dgate may be gate and dup may be up. Every element is loaded
  // into registers before the thread stores to the same positions, and no other thread touches
  // them, so the aliasing is safe.
  if (VEC) {
    const int64_t n8 = n >> 3;
    const int64_t v0 = (int64_t)blockIdx.x * (kThreads * kStepsBwd) + threadIdx.x;
    float y[kStepsBwd][8], g[kStepsBwd][8], u[kStepsBwd][8];
#pragma unroll
    for (int s = 0; s < kStepsBwd; ++s) {
      const int64_t v = v0 + (int64_t)s * kThreads;
      if (v < n8) {
        load8(dy, v << 3, ydt, y[s]);
        load8(gate, v << 3, gdt, g[s]);
        load8(up, v << 3, udt, u[s]);
      }
    }
#pragma unroll
    for (int s = 0; s < kStepsBwd; ++s) {
      const int64_t v = v0 + (int64_t)s * kThreads;
      if (v >= n8) continue;
      float dg[8], du[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) bwd_elem(y[s][k], g[s][k], u[s][k], gdt, round_silu, dg[k], du[k]);
      if (dgate) store8(dgate, v << 3, gdt, dg);
      if (dup) store8(dup, v << 3, udt, du);
    }
    if (blockIdx.x == 0) {
      for (int64_t i = (n8 << 3) + threadIdx.x; i < n; i += kThreads) {
        float dg, du;
        bwd_elem(load1(dy, i, ydt), load1(gate, i, gdt), load1(up, i, udt), gdt, round_silu, dg, du);
        if (dgate) store1(dgate, i, gdt, dg);
        if (dup) store1(dup, i, udt, du);
      }
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * kThreads) {
      float dg, du;
      bwd_elem(load1(dy, i, ydt), load1(gate, i, gdt), load1(up, i, udt), gdt, round_silu, dg, du);
      if (dgate) store1(dgate, i, gdt, dg);
      if (dup) store1(dup, i, udt, du);
    }
  }
}

// Backward for 16-bit tensors of one dtype on the warp-private shared-memory pipeline
// (rowpipe.cuh): the flat arrays are cut into chunks of kChunk elements; a warp's slot holds the
// dy, gate and up pieces of a chunk (three bulk async copies of 2 KB), so 32 warps per SM keep
// ~190 KB in flight whatever the register pressure of the arithmetic. The two gradients are
// written from registers, over gate and up when the caller asks for that: a chunk is read by
// exactly one warp, and completely (all three copies have landed) before that warp stores to it.
constexpr int kChunk = 1024;

template <int DT>
__global__ void __launch_bounds__(rowpipe::kMaxWarps * 32, 2)
silu_mul_bwd_pipe_kernel(const void* __restrict__ dy, const void* gate, const void* up, void* dgate,
                         void* dup, int64_t n_chunks, int round_silu, int stages, int* status) {
  constexpr uint32_t kPiece = kChunk * 2;   // bytes of one array's piece
  extern __shared__ __align__(128) char smem[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  if (threadIdx.x == 0) s_abort = 0;
  rowpipe::Ring ring;
  ring.init(smem, 3 * kPiece, stages, warp, lane);
  __syncthreads();
  const int64_t c0 = (int64_t)blockIdx.x * warps + warp, stride = (int64_t)gridDim.x * warps;
  auto request = [&](int s, int64_t chunk) {   // lane 0 only
    char* dst = ring.slot_ptr(s);
    const int64_t off = chunk * kPiece;
    umma::mbar_expect_tx(&ring.bars[s], 3 * kPiece);
    rowpipe::bulk_load(dst, reinterpret_cast<const char*>(dy) + off, kPiece, &ring.bars[s]);
    rowpipe::bulk_load(dst + kPiece, reinterpret_cast<const char*>(gate) + off, kPiece, &ring.bars[s]);
    rowpipe::bulk_load(dst + 2 * kPiece, reinterpret_cast<const char*>(up) + off, kPiece, &ring.bars[s]);
  };
  int64_t next = c0;
  if (lane == 0)
    for (int s = 0; s < stages && next < n_chunks; ++s, next += stride) request(s, next);
  next = __shfl_sync(0xffffffffu, next, 0);
  for (int64_t chunk = c0; chunk < n_chunks; chunk += stride) {
    if (!ring.wait(&s_abort, status, 14)) {
      ring.drain((int)((next - chunk) / stride));
      return;
    }
    const char* src = ring.slot_ptr(ring.slot);
#pragma unroll 2
    for (int vi = lane; vi < kChunk / 8; vi += 32) {
      float y[8], g[8], u[8], dg[8], du[8];
      unpack<8, 2>(ld_raw<16>(src, vi * 16), DT, y);
      unpack<8, 2>(ld_raw<16>(src + kPiece, vi * 16), DT, g);
      unpack<8, 2>(ld_raw<16>(src + 2 * kPiece, vi * 16), DT, u);
#pragma unroll
      for (int k = 0; k < 8; ++k) bwd_elem(y[k], g[k], u[k], DT, round_silu, dg[k], du[k]);
      const int64_t e = chunk * kChunk + vi * 8;
      if (dgate) store8(dgate, e, DT, dg);
      if (dup) store8(dup, e, DT, du);
    }
    __syncwarp();
    if (next < n_chunks) {
      if (lane == 0) {
        umma::fence_proxy_async_smem();
        request(ring.slot, next);
      }
      next += stride;
    }
    ring.advance();
  }
}

inline unsigned vec_blocks(int64_t n, int steps = kSteps) {
  const int64_t n8 = n >> 3, per = kThreads * steps;
  int64_t b = (n8 + per - 1) / per;
  return (unsigned)(b < 1 ? 1 : b);
}

inline unsigned scalar_blocks(int64_t n) {
  int64_t b = (n + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace
}  // namespace soup

extern "C" int soup_silu_mul_fwd(const void* gate, const void* up, void* out, int64_t n,
                                 int gate_dtype, int up_dtype, int out_dtype, int round_silu,
                                 void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || !gate || !up || !out) SOUP_FAIL(SOUP_ERR_ARG, "silu_mul_fwd: bad argument");
  if (!is_float_dtype(gate_dtype) || !is_float_dtype(up_dtype) || !is_float_dtype(out_dtype))
    SOUP_FAIL(SOUP_ERR_ARG, "silu_mul_fwd: unsupported dtype");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (aligned16(gate) && aligned16(up) && aligned16(out))
    silu_mul_fwd_kernel<true><<<vec_blocks(n), kThreads, 0, s>>>(gate, up, out, n, gate_dtype,
                                                                 up_dtype, out_dtype, round_silu);
  else
    silu_mul_fwd_kernel<false><<<scalar_blocks(n), kThreads, 0, s>>>(gate, up, out, n, gate_dtype,
                                                                     up_dtype, out_dtype, round_silu);
  SOUP_CHECK_LAUNCH("silu_mul_fwd");
  return SOUP_OK;
}

extern "C" int soup_silu_mul_bwd(const void* dy, const void* gate, const void* up, void* dgate,
                                 void* dup, int64_t n, int dy_dtype, int gate_dtype, int up_dtype,
                                 int round_silu, void* stream) {
  using namespace soup;
  if (n == 0 || (!dgate && !dup)) return SOUP_OK;
  if (n < 0 || !dy || !gate || !up) SOUP_FAIL(SOUP_ERR_ARG, "silu_mul_bwd: bad argument");
  if (!is_float_dtype(dy_dtype) || !is_float_dtype(gate_dtype) || !is_float_dtype(up_dtype))
    SOUP_FAIL(SOUP_ERR_ARG, "silu_mul_bwd: unsupported dtype");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool vec = aligned16(dy) && aligned16(gate) && aligned16(up) &&
                   (!dgate || aligned16(dgate)) && (!dup || aligned16(dup));
  // whole chunks of 16-bit tensors of one dtype go through the pipelined kernel, the rest (a tail
  // shorter than a chunk, or other dtypes) through the streaming kernel below
  const bool one_16bit = dy_dtype == gate_dtype && dy_dtype == up_dtype && dy_dtype != SOUP_F32;
  const int64_t n_chunks = (vec && one_16bit) ? n / kChunk : 0;
  if (n_chunks > 0) {
    const rowpipe::Plan plan = rowpipe::make_plan(3 * kChunk * 2, 0, false, n_chunks);
    int* status = rowpipe::status_word();
    if (plan.stages && status) {
      if (dy_dtype == SOUP_F16) {
        cudaFuncSetAttribute(silu_mul_bwd_pipe_kernel<SOUP_F16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
        silu_mul_bwd_pipe_kernel<SOUP_F16><<<plan.grid, plan.warps * 32, plan.smem, s>>>(
            dy, gate, up, dgate, dup, n_chunks, round_silu, plan.stages, status);
      } else {
        cudaFuncSetAttribute(silu_mul_bwd_pipe_kernel<SOUP_BF16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
        silu_mul_bwd_pipe_kernel<SOUP_BF16><<<plan.grid, plan.warps * 32, plan.smem, s>>>(
            dy, gate, up, dgate, dup, n_chunks, round_silu, plan.stages, status);
      }
      SOUP_CHECK_LAUNCH("silu_mul_bwd");
      const int64_t done = n_chunks * kChunk;
      if (done == n) return SOUP_OK;
      const int es = 2;
      dy = reinterpret_cast<const char*>(dy) + done * es;
      gate = reinterpret_cast<const char*>(gate) + done * es;
      up = reinterpret_cast<const char*>(up) + done * es;
      if (dgate) dgate = reinterpret_cast<char*>(dgate) + done * es;
      if (dup) dup = reinterpret_cast<char*>(dup) + done * es;
      n -= done;
    }
  }
  if (vec)
    silu_mul_bwd_kernel<true><<<vec_blocks(n, kStepsBwd), kThreads, 0, s>>>(dy, gate, up, dgate, dup, n,
                                                                 dy_dtype, gate_dtype, up_dtype,
                                                                 round_silu);
  else
    silu_mul_bwd_kernel<false><<<scalar_blocks(n), kThreads, 0, s>>>(dy, gate, up, dgate, dup, n,
                                                                     dy_dtype, gate_dtype, up_dtype,
                                                                     round_silu);
  SOUP_CHECK_LAUNCH("silu_mul_bwd");
  return SOUP_OK;
}
