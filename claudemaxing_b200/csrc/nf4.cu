// NF4 dequantisation with the nested 8-bit absmax fused in: an HBM-streaming kernel.
//
// One thread turns 16 packed bytes (one 128-bit load) into 32 outputs (four 128-bit fp16 stores,
// or eight for fp32). The 32 outputs of a thread share one absmax block because every supported
// blocksize is a multiple of 32, so the scale is computed once per load. The arithmetic is the
// reference's, operation for operation, with explicitly unfused fp32 intrinsics:
//   scale = code2[absmax8[b]] * absmax2[b / blocksize2]   (__fmul_rn)
//   scale = scale + offset                                 (__fadd_rn)
//   out   = round(code[nibble] * scale)                    (__fmul_rn, then RN to the out dtype)
// which is what makes the result bit-identical (solution/nf4.py:31-46 of the reference).
#include "common.cuh"

namespace soup {
namespace {

constexpr int kThreads = 256;
constexpr int kVecPerThread = 2;  // independent 128-bit loads in flight per thread

template <bool NESTED>
__device__ __forceinline__ float block_scale(const void* absmax, const float* s_code2,
                                             const float* absmax2, float offset, int64_t blk,
                                             int shift2) {
  if (NESTED) {
    const uint32_t q8 = reinterpret_cast<const uint8_t*>(absmax)[blk];
    const float a2 = __ldg(absmax2 + (blk >> shift2));
    return __fadd_rn(__fmul_rn(s_code2[q8], a2), offset);
  }
  return __ldg(reinterpret_cast<const float*>(absmax) + blk);
}

// One CTA's share of one tensor: blocks [0, n_blocks) of the tensor, this CTA being `block`.
template <bool NESTED, bool OUT_F16>
__device__ __forceinline__ void
nf4_dequant_body(const uint8_t* __restrict__ packed, const void* __restrict__ absmax,
                 const float* __restrict__ code, const float* __restrict__ code2,
                 const float* __restrict__ absmax2, const float* __restrict__ offset_ptr,
                 void* __restrict__ out, int64_t n_bytes, int shift, int shift2, int64_t block,
                 int64_t n_blocks) {
  __shared__ float s_code[16];
  __shared__ float s_code2[256];
  if (threadIdx.x < 16) s_code[threadIdx.x] = code[threadIdx.x];
  if (NESTED) s_code2[threadIdx.x] = code2[threadIdx.x];  // kThreads == 256
  __syncthreads();
  const float offset = NESTED ? __ldg(offset_ptr) : 0.f;

  const int64_t n_vec = n_bytes >> 4;  // whole 16-byte groups
  const int64_t v_base = block * (kThreads * kVecPerThread) + threadIdx.x;

  uint4 raw[kVecPerThread];
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const int64_t v = v_base + (int64_t)u * kThreads;
    if (v < n_vec) raw[u] = __ldcs(reinterpret_cast<const uint4*>(packed) + v);
  }
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const int64_t v = v_base + (int64_t)u * kThreads;
    if (v >= n_vec) continue;
    const int64_t e0 = v << 5;  // first output element of this group
    const float scale = block_scale<NESTED>(absmax, s_code2, absmax2, offset, e0 >> shift, shift2);
    const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
    if (OUT_F16) {
      uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(out) + e0);
#pragma unroll
      for (int k = 0; k < 4; ++k) {  // one 32-bit word = 4 bytes = 8 outputs = one 128-bit store
        uint32_t h[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t byte = (w[k] >> (8 * b)) & 0xffu;
          const float hi = __fmul_rn(s_code[byte >> 4], scale);
          const float lo = __fmul_rn(s_code[byte & 15u], scale);
          __half2 p = __floats2half2_rn(hi, lo);
          h[b] = *reinterpret_cast<uint32_t*>(&p);
        }
        __stcs(o + k, make_uint4(h[0], h[1], h[2], h[3]));
      }
    } else {
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + e0);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
#pragma unroll
        for (int b = 0; b < 4; b += 2) {
          const uint32_t b0 = (w[k] >> (8 * b)) & 0xffu, b1 = (w[k] >> (8 * b + 8)) & 0xffu;
          __stcs(o + k * 2 + (b >> 1),
                 make_float4(__fmul_rn(s_code[b0 >> 4], scale), __fmul_rn(s_code[b0 & 15u], scale),
                             __fmul_rn(s_code[b1 >> 4], scale), __fmul_rn(s_code[b1 & 15u], scale)));
        }
      }
    }
  }

  // Ragged tail (n_bytes not a multiple of 16): the last block's first threads go byte by byte.
  if (block == n_blocks - 1) {
    const int64_t tail0 = n_vec << 4;
    for (int64_t i = tail0 + threadIdx.x; i < n_bytes; i += kThreads) {
      const uint32_t byte = packed[i];
      const int64_t e = i << 1;
      const float scale = block_scale<NESTED>(absmax, s_code2, absmax2, offset, e >> shift, shift2);
      const float hi = __fmul_rn(s_code[byte >> 4], scale);
      const float lo = __fmul_rn(s_code[byte & 15u], scale);
      if (OUT_F16) {
        reinterpret_cast<__half*>(out)[e] = __float2half_rn(hi);
        reinterpret_cast<__half*>(out)[e + 1] = __float2half_rn(lo);
      } else {
        reinterpret_cast<float*>(out)[e] = hi;
        reinterpret_cast<float*>(out)[e + 1] = lo;
      }
    }
  }
}

template <bool NESTED, bool OUT_F16>
__global__ void __launch_bounds__(kThreads)
nf4_dequant_kernel(const uint8_t* __restrict__ packed, const void* __restrict__ absmax,
                   const float* __restrict__ code, const float* __restrict__ code2,
                   const float* __restrict__ absmax2, const float* __restrict__ offset_ptr,
                   void* __restrict__ out, int64_t n_bytes, int shift, int shift2) {
  nf4_dequant_body<NESTED, OUT_F16>(packed, absmax, code, code2, absmax2, offset_ptr, out, n_bytes,
                                    shift, shift2, blockIdx.x, gridDim.x);
}

// Several tensors in one launch (blockIdx.y = tensor): removes the per-launch latency that
// dominates the small projection weights (k/v of Qwen2.5-1.5B are 0.4 M elements each).
constexpr int kMaxBatch = 8;
struct Nf4Batch {
  soup_nf4_item item[kMaxBatch];
  int64_t n_blocks[kMaxBatch];
};

template <bool NESTED, bool OUT_F16>
__global__ void __launch_bounds__(kThreads)
nf4_dequant_batch_kernel(const Nf4Batch b, const float* __restrict__ code, int shift, int shift2) {
  const soup_nf4_item& it = b.item[blockIdx.y];
  const int64_t n_blocks = b.n_blocks[blockIdx.y];
  if ((int64_t)blockIdx.x >= n_blocks) return;
  nf4_dequant_body<NESTED, OUT_F16>(reinterpret_cast<const uint8_t*>(it.packed), it.absmax, code,
                                    it.code2, it.absmax2, it.offset, it.out, it.n_elems >> 1, shift,
                                    shift2, blockIdx.x, n_blocks);
}

inline int log2_exact(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return (1 << s) == v ? s : -1;
}

}  // namespace
}  // namespace soup

extern "C" int soup_nf4_dequant(const void* packed, const void* absmax, const float* code,
                                const float* code2, const float* absmax2, const float* offset,
                                void* out, int64_t n_elems, int blocksize, int blocksize2,
                                int nested, int out_dtype, void* stream) {
  using namespace soup;
  if (n_elems == 0) return SOUP_OK;
  if (!packed || !absmax || !code || !out) SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant: null pointer");
  if (n_elems < 0 || (n_elems & 1)) SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant: n_elems must be even");
  const int shift = log2_exact(blocksize);
  if (shift < 5 || shift > 12)
    SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant: blocksize %d not a power of two in [32,4096]", blocksize);
  int shift2 = 0;
  if (nested) {
    if (!code2 || !absmax2 || !offset) SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant: nested tables missing");
    shift2 = log2_exact(blocksize2);
    if (shift2 < 0) SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant: blocksize2 %d not a power of two", blocksize2);
  }
  if (out_dtype != SOUP_F16 && out_dtype != SOUP_F32)
    SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant: out dtype must be fp16 or fp32");
  if (!aligned16(packed) || !aligned16(out))
    SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant: packed and out must be 16-byte aligned");
  const int64_t n_bytes = n_elems >> 1;
  const int64_t n_vec = n_bytes >> 4;
  const int64_t per_block = kThreads * kVecPerThread;
  int64_t blocks = (n_vec + per_block - 1) / per_block;
  if (blocks < 1) blocks = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define SOUP_NF4_LAUNCH(N_, F_)                                                              \
  nf4_dequant_kernel<N_, F_><<<(unsigned)blocks, kThreads, 0, s>>>(                          \
      reinterpret_cast<const uint8_t*>(packed), absmax, code, code2, absmax2, offset, out,   \
      n_bytes, shift, shift2)
  if (nested) {
    if (out_dtype == SOUP_F16) SOUP_NF4_LAUNCH(true, true); else SOUP_NF4_LAUNCH(true, false);
  } else {
    if (out_dtype == SOUP_F16) SOUP_NF4_LAUNCH(false, true); else SOUP_NF4_LAUNCH(false, false);
  }
#undef SOUP_NF4_LAUNCH
  SOUP_CHECK_LAUNCH("nf4_dequant");
  return SOUP_OK;
}


extern "C" int soup_nf4_dequant_batch(const soup_nf4_item* items, int count, const float* code,
                                      int blocksize, int blocksize2, int nested, int out_dtype,
                                      void* stream) {
  using namespace soup;
  if (count == 0) return SOUP_OK;
  if (count < 0 || !items || !code) SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant_batch: bad argument");
  const int shift = log2_exact(blocksize);
  if (shift < 5 || shift > 12)
    SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant_batch: blocksize %d not a power of two in [32,4096]", blocksize);
  int shift2 = 0;
  if (nested) {
    shift2 = log2_exact(blocksize2);
    if (shift2 < 0) SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant_batch: blocksize2 %d not a power of two", blocksize2);
  }
  if (out_dtype != SOUP_F16 && out_dtype != SOUP_F32)
    SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant_batch: out dtype must be fp16 or fp32");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int64_t per_block = kThreads * kVecPerThread;
  for (int i0 = 0; i0 < count; i0 += kMaxBatch) {
    Nf4Batch b;
    int m = 0;
    int64_t max_blocks = 1;
    for (int i = i0; i < count && m < kMaxBatch; ++i) {
      const soup_nf4_item& it = items[i];
      if (it.n_elems == 0) continue;
      if (!it.packed || !it.absmax || !it.out || it.n_elems < 0 || (it.n_elems & 1) ||
          (nested && (!it.code2 || !it.absmax2 || !it.offset)) || !aligned16(it.packed) ||
          !aligned16(it.out))
        SOUP_FAIL(SOUP_ERR_ARG, "nf4_dequant_batch: item %d is malformed", i);
      b.item[m] = it;
      int64_t blocks = (((it.n_elems >> 1) >> 4) + per_block - 1) / per_block;
      if (blocks < 1) blocks = 1;
      b.n_blocks[m] = blocks;
      if (blocks > max_blocks) max_blocks = blocks;
      ++m;
    }
    if (m == 0) continue;
    dim3 grid((unsigned)max_blocks, (unsigned)m);
    if (nested) {
      if (out_dtype == SOUP_F16) nf4_dequant_batch_kernel<true, true><<<grid, kThreads, 0, s>>>(b, code, shift, shift2);
      else nf4_dequant_batch_kernel<true, false><<<grid, kThreads, 0, s>>>(b, code, shift, shift2);
    } else {
      if (out_dtype == SOUP_F16) nf4_dequant_batch_kernel<false, true><<<grid, kThreads, 0, s>>>(b, code, shift, shift2);
      else nf4_dequant_batch_kernel<false, false><<<grid, kThreads, 0, s>>>(b, code, shift, shift2);
    }
    SOUP_CHECK_LAUNCH("nf4_dequant_batch");
  }
  return SOUP_OK;
}
