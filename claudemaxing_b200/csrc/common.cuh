// Shared helpers for every kernel family of libsoup_b200: dtype codes, the thread-local error
// string behind soup_last_error_string(), launch checks, and 128-bit typed vector access.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/soup_b200.h"

namespace soup {

void set_error(const char* fmt, ...);
int sm_count();

#define SOUP_FAIL(code, ...)          \
  do {                                \
    ::soup::set_error(__VA_ARGS__);   \
    return (code);                    \
  } while (0)

#define SOUP_CHECK_LAUNCH(name)                                                      \
  do {                                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess) SOUP_FAIL(SOUP_ERR_LAUNCH, "%s: %s", name, cudaGetErrorString(e__)); \
  } while (0)

inline bool is_float_dtype(int dt) { return dt == SOUP_F32 || dt == SOUP_F16 || dt == SOUP_BF16; }
inline int dtype_size(int dt) { return dt == SOUP_F32 ? 4 : 2; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- scalar typed access (dt is uniform across the grid, so the branches do not diverge) ----
__device__ __forceinline__ float load1(const void* base, int64_t i, int dt) {
  if (dt == SOUP_F16) return __half2float(reinterpret_cast<const __half*>(base)[i]);
  if (dt == SOUP_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  return reinterpret_cast<const float*>(base)[i];
}

__device__ __forceinline__ void store1(void* base, int64_t i, int dt, float v) {
  if (dt == SOUP_F16) reinterpret_cast<__half*>(base)[i] = __float2half_rn(v);
  else if (dt == SOUP_BF16) reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(base)[i] = v;
}

// Round an fp32 value through a storage dtype (round-to-nearest-even), back to fp32.
__device__ __forceinline__ float round_through(float v, int dt) {
  if (dt == SOUP_F16) return __half2float(__float2half_rn(v));
  if (dt == SOUP_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

// ---- 8-element vector access; element index must be a multiple of 8 and the address 16B aligned ----
__device__ __forceinline__ void load8(const void* base, int64_t i, int dt, float (&v)[8]) {
  if (dt == SOUP_F32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + i);
    float4 a = p[0], b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + i);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (dt == SOUP_F16) {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
        v[2 * k] = f.x; v[2 * k + 1] = f.y;
      } else {
        float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
        v[2 * k] = f.x; v[2 * k + 1] = f.y;
      }
    }
  }
}

__device__ __forceinline__ void store8(void* base, int64_t i, int dt, const float (&v)[8]) {
  if (dt == SOUP_F32) {
    float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + i);
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (dt == SOUP_F16) {
        __half2 h = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
        w[k] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
        w[k] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + i) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---- 16-byte (or 8-byte) raw vectors: EPV elements of B bytes kept as bits until they are used ----
template <int NB> struct Raw;
template <> struct Raw<16> { uint4 v; };
template <> struct Raw<8> { uint2 v; };

template <int NB>
__device__ __forceinline__ Raw<NB> ld_raw(const void* base, int64_t byte_off) {
  Raw<NB> r;
  const char* p = reinterpret_cast<const char*>(base) + byte_off;
  if constexpr (NB == 16) r.v = *reinterpret_cast<const uint4*>(p);
  else r.v = *reinterpret_cast<const uint2*>(p);
  return r;
}

__device__ __forceinline__ float2 unpack2(uint32_t w, int dt) {
  if (dt == SOUP_F16) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}

// EPV elements of B bytes each from their raw bits.
template <int EPV, int B>
__device__ __forceinline__ void unpack(const Raw<EPV * B>& r, int dt, float (&v)[EPV]) {
  if constexpr (B == 4) {
    static_assert(EPV == 4, "fp32 vectors hold four elements");
    v[0] = __uint_as_float(r.v.x); v[1] = __uint_as_float(r.v.y);
    v[2] = __uint_as_float(r.v.z); v[3] = __uint_as_float(r.v.w);
  } else if constexpr (EPV == 8) {
    const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 f = unpack2(w[k], dt); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
  } else {
    const float2 a = unpack2(r.v.x, dt), b = unpack2(r.v.y, dt);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}

// EPV (4 or 8) consecutive elements of a runtime dtype; element index a multiple of EPV.
template <int EPV>
__device__ __forceinline__ void loadv(const void* base, int64_t i, int dt, float (&v)[EPV]) {
  if constexpr (EPV == 8) {
    load8(base, i, dt, v);
  } else {
    if (dt == SOUP_F32) {
      const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + i);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    } else {
      const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + i);
      const float2 a = unpack2(r.x, dt), b = unpack2(r.y, dt);
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
  }
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int dt) {
  if (dt == SOUP_F16) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int EPV>
__device__ __forceinline__ void storev(void* base, int64_t i, int dt, const float (&v)[EPV]) {
  if constexpr (EPV == 8) {
    store8(base, i, dt, v);
  } else {
    if (dt == SOUP_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + i) =
          make_uint2(pack2(v[0], v[1], dt), pack2(v[2], v[3], dt));
    }
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace soup
