// LoRA dropout with a bit-packed mask: pack (forward) and unpack (backward).
//
// A thread owns 16 consecutive elements = two mask bytes of output bits (one 16-bit store), so
// that x (fp32: four 128-bit loads), the boolean mask (one 128-bit load) and the fp16 output (two
// 128-bit stores) are all moved with full-width accesses. Bit l of byte r is element 8r+l (least
// significant bit = lowest index), as lora_dropout_pack_kernel of the reference writes it
// (solution/lora.py:30-57). The products are single fp32 multiplies rounded to fp16 (RN), so the
// fp16 values, and of course the bits, are bit-identical to the reference's.
#include "common.cuh"

namespace soup {
namespace {

constexpr int kThreads = 256;

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
dropout_pack_kernel(const void* __restrict__ x, const uint8_t* __restrict__ mask,
                    void* __restrict__ xd, uint8_t* __restrict__ bits, int64_t n_bytes, float scale,
                    int xdt) {
  const int64_t n_pairs = n_bytes >> 1;  // 16-element groups
  const int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (VEC && p < n_pairs) {
    const int64_t e0 = p << 4;
    float a[8], b[8];
    load8(x, e0, xdt, a);
    load8(x, e0 + 8, xdt, b);
    const uint4 m = *reinterpret_cast<const uint4*>(mask + e0);
    const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
    uint32_t bitword = 0;
    float oa[8], ob[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool ka = ((mw[k >> 2] >> (8 * (k & 3))) & 0xffu) != 0;
      const bool kb = ((mw[2 + (k >> 2)] >> (8 * (k & 3))) & 0xffu) != 0;
      bitword |= (ka ? 1u : 0u) << k;
      bitword |= (kb ? 1u : 0u) << (8 + k);
      oa[k] = ka ? __fmul_rn(a[k], scale) : 0.0f;
      ob[k] = kb ? __fmul_rn(b[k], scale) : 0.0f;
    }
    store8(xd, e0, SOUP_F16, oa);
    store8(xd, e0 + 8, SOUP_F16, ob);
    *reinterpret_cast<uint16_t*>(bits + (p << 1)) = (uint16_t)bitword;
  }
  // Bytes the vector path does not cover: an odd last byte, or everything when unaligned.
  const int64_t first = VEC ? (n_pairs << 1) : 0;
  for (int64_t r = first + p; r < n_bytes; r += (int64_t)gridDim.x * kThreads) {
    uint32_t byte = 0;
    for (int l = 0; l < 8; ++l) {
      const int64_t e = (r << 3) + l;
      const bool keep = mask[e] != 0;
      byte |= (keep ? 1u : 0u) << l;
      store1(xd, e, SOUP_F16, keep ? __fmul_rn(load1(x, e, xdt), scale) : 0.0f);
    }
    bits[r] = (uint8_t)byte;
  }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
dropout_unpack_kernel(const void* __restrict__ x16, const uint8_t* __restrict__ bits,
                      const void* __restrict__ g16, void* __restrict__ xd, void* __restrict__ dx,
                      int64_t n_bytes, float scale, int dxdt) {
  const int64_t n_pairs = n_bytes >> 1;
  const int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (VEC && p < n_pairs) {
    const int64_t e0 = p << 4;
    float xa[8], xb[8], ga[8], gb[8];
    load8(x16, e0, SOUP_F16, xa);
    load8(x16, e0 + 8, SOUP_F16, xb);
    load8(g16, e0, SOUP_F16, ga);
    load8(g16, e0 + 8, SOUP_F16, gb);
    const uint32_t bitword = *reinterpret_cast<const uint16_t*>(bits + (p << 1));
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool ka = (bitword >> k) & 1u, kb = (bitword >> (8 + k)) & 1u;
      xa[k] = ka ? __fmul_rn(xa[k], scale) : 0.0f;
      xb[k] = kb ? __fmul_rn(xb[k], scale) : 0.0f;
      ga[k] = ka ? __fmul_rn(ga[k], scale) : 0.0f;
      gb[k] = kb ? __fmul_rn(gb[k], scale) : 0.0f;
    }
    store8(xd, e0, SOUP_F16, xa);
    store8(xd, e0 + 8, SOUP_F16, xb);
    store8(dx, e0, dxdt, ga);
    store8(dx, e0 + 8, dxdt, gb);
  }
  const int64_t first = VEC ? (n_pairs << 1) : 0;
  for (int64_t r = first + p; r < n_bytes; r += (int64_t)gridDim.x * kThreads) {
    const uint32_t byte = bits[r];
    for (int l = 0; l < 8; ++l) {
      const int64_t e = (r << 3) + l;
      const bool keep = (byte >> l) & 1u;
      store1(xd, e, SOUP_F16, keep ? __fmul_rn(load1(x16, e, SOUP_F16), scale) : 0.0f);
      store1(dx, e, dxdt, keep ? __fmul_rn(load1(g16, e, SOUP_F16), scale) : 0.0f);
    }
  }
}

// The two adapters of a block (q_proj's and v_proj's) see the same x with different masks: one
// launch packs both (x read once) and one launch unpacks both, summing the two input gradients
// (dx = keep_a * g_a * scale_a + keep_b * g_b * scale_b, fp32). Same 16-element groups and the same
// roundings per adapter as the single kernels; vector accesses only (the host checks alignment).
__global__ void __launch_bounds__(kThreads)
dropout_pack2_kernel(const void* __restrict__ x, const uint8_t* __restrict__ mask_a,
                     const uint8_t* __restrict__ mask_b, void* __restrict__ xd_a,
                     void* __restrict__ xd_b, uint8_t* __restrict__ bits_a,
                     uint8_t* __restrict__ bits_b, int64_t n_pairs, float scale_a, float scale_b,
                     int xdt) {
  const int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (p >= n_pairs) return;
  const int64_t e0 = p << 4;
  float a[8], b[8];
  load8(x, e0, xdt, a);
  load8(x, e0 + 8, xdt, b);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const uint4 m = *reinterpret_cast<const uint4*>((which ? mask_b : mask_a) + e0);
    const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
    const float scale = which ? scale_b : scale_a;
    uint32_t bitword = 0;
    float oa[8], ob[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool ka = ((mw[k >> 2] >> (8 * (k & 3))) & 0xffu) != 0;
      const bool kb = ((mw[2 + (k >> 2)] >> (8 * (k & 3))) & 0xffu) != 0;
      bitword |= (ka ? 1u : 0u) << k;
      bitword |= (kb ? 1u : 0u) << (8 + k);
      oa[k] = ka ? __fmul_rn(a[k], scale) : 0.0f;
      ob[k] = kb ? __fmul_rn(b[k], scale) : 0.0f;
    }
    void* xd = which ? xd_b : xd_a;
    store8(xd, e0, SOUP_F16, oa);
    store8(xd, e0 + 8, SOUP_F16, ob);
    *reinterpret_cast<uint16_t*>((which ? bits_b : bits_a) + (p << 1)) = (uint16_t)bitword;
  }
}

__global__ void __launch_bounds__(kThreads)
dropout_unpack2_kernel(const void* __restrict__ x16, const uint8_t* __restrict__ bits_a,
                       const uint8_t* __restrict__ bits_b, const void* __restrict__ g_a,
                       const void* __restrict__ g_b, void* __restrict__ xd_a,
                       void* __restrict__ xd_b, float* __restrict__ dx, int64_t n_pairs,
                       float scale_a, float scale_b) {
  const int64_t p = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (p >= n_pairs) return;
  const int64_t e0 = p << 4;
  float xa[8], xb[8], sum_a[8], sum_b[8];
  load8(x16, e0, SOUP_F16, xa);
  load8(x16, e0 + 8, SOUP_F16, xb);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    float ga[8], gb[8], oa[8], ob[8];
    const void* g = which ? g_b : g_a;
    load8(g, e0, SOUP_F16, ga);
    load8(g, e0 + 8, SOUP_F16, gb);
    const uint32_t bitword = *reinterpret_cast<const uint16_t*>((which ? bits_b : bits_a) + (p << 1));
    const float scale = which ? scale_b : scale_a;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool ka = (bitword >> k) & 1u, kb = (bitword >> (8 + k)) & 1u;
      oa[k] = ka ? __fmul_rn(xa[k], scale) : 0.0f;
      ob[k] = kb ? __fmul_rn(xb[k], scale) : 0.0f;
      const float da = ka ? __fmul_rn(ga[k], scale) : 0.0f, db = kb ? __fmul_rn(gb[k], scale) : 0.0f;
      sum_a[k] = which ? __fadd_rn(sum_a[k], da) : da;
      sum_b[k] = which ? __fadd_rn(sum_b[k], db) : db;
    }
    void* xd = which ? xd_b : xd_a;
    store8(xd, e0, SOUP_F16, oa);
    store8(xd, e0 + 8, SOUP_F16, ob);
  }
  store8(dx, e0, SOUP_F32, sum_a);
  store8(dx, e0 + 8, SOUP_F32, sum_b);
}

inline unsigned blocks_for(int64_t n_bytes) {
  const int64_t n_pairs = (n_bytes + 1) >> 1;
  int64_t b = (n_pairs + kThreads - 1) / kThreads;
  return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace
}  // namespace soup

extern "C" int soup_dropout_pack(const void* x, const uint8_t* mask, void* xd, uint8_t* bits,
                                 int64_t n, float scale, int x_dtype, void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || (n & 7)) SOUP_FAIL(SOUP_ERR_ARG, "dropout_pack: n must be a multiple of 8");
  if (!x || !mask || !xd || !bits) SOUP_FAIL(SOUP_ERR_ARG, "dropout_pack: null pointer");
  if (!is_float_dtype(x_dtype)) SOUP_FAIL(SOUP_ERR_ARG, "dropout_pack: unsupported dtype");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n_bytes = n >> 3;
  const bool vec = aligned16(x) && aligned16(mask) && aligned16(xd) &&
                   (reinterpret_cast<uintptr_t>(bits) & 1u) == 0;
  if (vec)
    dropout_pack_kernel<true><<<blocks_for(n_bytes), kThreads, 0, s>>>(x, mask, xd, bits, n_bytes,
                                                                       scale, x_dtype);
  else
    dropout_pack_kernel<false><<<blocks_for(n_bytes), kThreads, 0, s>>>(x, mask, xd, bits, n_bytes,
                                                                        scale, x_dtype);
  SOUP_CHECK_LAUNCH("dropout_pack");
  return SOUP_OK;
}

extern "C" int soup_dropout_unpack(const void* x16, const uint8_t* bits, const void* g16, void* xd,
                                   void* dx, int64_t n, float scale, int dx_dtype, void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || (n & 7)) SOUP_FAIL(SOUP_ERR_ARG, "dropout_unpack: n must be a multiple of 8");
  if (!x16 || !bits || !g16 || !xd || !dx) SOUP_FAIL(SOUP_ERR_ARG, "dropout_unpack: null pointer");
  if (!is_float_dtype(dx_dtype)) SOUP_FAIL(SOUP_ERR_ARG, "dropout_unpack: unsupported dtype");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n_bytes = n >> 3;
  const bool vec = aligned16(x16) && aligned16(g16) && aligned16(xd) && aligned16(dx) &&
                   (reinterpret_cast<uintptr_t>(bits) & 1u) == 0;
  if (vec)
    dropout_unpack_kernel<true><<<blocks_for(n_bytes), kThreads, 0, s>>>(x16, bits, g16, xd, dx,
                                                                         n_bytes, scale, dx_dtype);
  else
    dropout_unpack_kernel<false><<<blocks_for(n_bytes), kThreads, 0, s>>>(x16, bits, g16, xd, dx,
                                                                          n_bytes, scale, dx_dtype);
  SOUP_CHECK_LAUNCH("dropout_unpack");
  return SOUP_OK;
}

extern "C" int soup_dropout_pack2(const void* x, const uint8_t* mask_a, const uint8_t* mask_b,
                                  void* xd_a, void* xd_b, uint8_t* bits_a, uint8_t* bits_b, int64_t n,
                                  float scale_a, float scale_b, int x_dtype, void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || (n & 15)) SOUP_FAIL(SOUP_ERR_ARG, "dropout_pack2: n must be a multiple of 16");
  if (!x || !mask_a || !mask_b || !xd_a || !xd_b || !bits_a || !bits_b)
    SOUP_FAIL(SOUP_ERR_ARG, "dropout_pack2: null pointer");
  if (!is_float_dtype(x_dtype)) SOUP_FAIL(SOUP_ERR_ARG, "dropout_pack2: unsupported dtype");
  if (!aligned16(x) || !aligned16(mask_a) || !aligned16(mask_b) || !aligned16(xd_a) || !aligned16(xd_b) ||
      ((reinterpret_cast<uintptr_t>(bits_a) | reinterpret_cast<uintptr_t>(bits_b)) & 1u))
    SOUP_FAIL(SOUP_ERR_ARG, "dropout_pack2: pointers must be 16-byte aligned (bits: 2-byte)");
  const int64_t n_pairs = n >> 4;
  dropout_pack2_kernel<<<(unsigned)((n_pairs + kThreads - 1) / kThreads), kThreads, 0,
                         reinterpret_cast<cudaStream_t>(stream)>>>(
      x, mask_a, mask_b, xd_a, xd_b, bits_a, bits_b, n_pairs, scale_a, scale_b, x_dtype);
  SOUP_CHECK_LAUNCH("dropout_pack2");
  return SOUP_OK;
}

extern "C" int soup_dropout_unpack2(const void* x16, const uint8_t* bits_a, const uint8_t* bits_b,
                                    const void* g_a, const void* g_b, void* xd_a, void* xd_b,
                                    float* dx, int64_t n, float scale_a, float scale_b,
                                    void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || (n & 15)) SOUP_FAIL(SOUP_ERR_ARG, "dropout_unpack2: n must be a multiple of 16");
  if (!x16 || !bits_a || !bits_b || !g_a || !g_b || !xd_a || !xd_b || !dx)
    SOUP_FAIL(SOUP_ERR_ARG, "dropout_unpack2: null pointer");
  if (!aligned16(x16) || !aligned16(g_a) || !aligned16(g_b) || !aligned16(xd_a) || !aligned16(xd_b) ||
      !aligned16(dx) || ((reinterpret_cast<uintptr_t>(bits_a) | reinterpret_cast<uintptr_t>(bits_b)) & 1u))
    SOUP_FAIL(SOUP_ERR_ARG, "dropout_unpack2: pointers must be 16-byte aligned (bits: 2-byte)");
  const int64_t n_pairs = n >> 4;
  dropout_unpack2_kernel<<<(unsigned)((n_pairs + kThreads - 1) / kThreads), kThreads, 0,
                           reinterpret_cast<cudaStream_t>(stream)>>>(
      x16, bits_a, bits_b, g_a, g_b, xd_a, xd_b, dx, n_pairs, scale_a, scale_b);
  SOUP_CHECK_LAUNCH("dropout_unpack2");
  return SOUP_OK;
}
