// SwiGLU activation of the MLP: silu(gate) * up forward, and the recomputing backward that keeps
// nothing but gate and up and may write its two gradients over them.
//
// Both kernels stream: each thread owns 8 consecutive elements per step (128-bit accesses for
// 16-bit dtypes, two for fp32) and takes two steps so that enough loads are in flight to cover
// HBM latency. The rounding points follow solution/swiglu_recompute.py:36-79 of the reference:
// silu is computed in fp32 as g / (1 + 2^(-g*log2 e)), rounded to the gate dtype when round_silu,
// and only then multiplied by up; dy*up is rounded the same way before it meets silu'.
#include "common.cuh"

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
  const float denom = silu_denom(g);
  const float sig = __fdividef(1.0f, denom);
  float silu = __fdividef(g, denom);
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
