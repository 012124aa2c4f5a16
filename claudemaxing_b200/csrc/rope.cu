// Rotary position embedding of q and k in one launch, forward or the transposed rotation.
//
// A thread owns 8 elements of the first half of a head row and the matching 8 of the second half
// (two 128-bit loads and two 128-bit stores per head). It loads its cos/sin vectors once and walks
// its share of the heads with them, kHeadsPerThread at a time, q heads first, then k heads, so
// cos/sin traffic is amortised over the heads and q and k need a single launch. Inputs are read
// through their strides (q and k arrive as transposed views of the projection outputs) and the
// outputs are written through theirs ([b, h, t, d] contiguous for the plain entry point). q may
// come as a sum of two tensors (the frozen projection's output and the adapter's), added in fp32
// before the rotation. Arithmetic is fp32, as in qwen_rope_kernel of the reference
// (solution/rope.py:17-43).
#include "common.cuh"
#include "rowpipe.cuh"

namespace soup {
namespace {

constexpr int kThreads = 256;
constexpr int kHeadsPerThread = 4;   // heads whose loads are in flight together

struct RopeArgs {
  const void* x[2];   // q, k
  const void* add;    // optional second term of q, with strides of its own
  int64_t asb, ash, ast;
  void* out[2];
  int64_t sb[2], sh[2], st[2];
  int64_t osb[2], osh[2], ost[2];
  int heads[2];
  int xdt[2], odt[2], adt;
  const void* cos;
  const void* sin;
  int64_t cs_b, cs_t;
  int csdt;
  int64_t b, t;
  int d;
  int backward;
};

__device__ __forceinline__ void rotate(float x1, float x2, float c1, float c2, float s1, float s2,
                                       int backward, float& o1, float& o2) {
  if (backward) {  // g*cos + rotate_half^T(g*sin)
    o1 = x1 * c1 + x2 * s2;
    o2 = x2 * c2 - x1 * s1;
  } else {  // x*cos + [-x2, x1]*sin
    o1 = x1 * c1 - x2 * s1;
    o2 = x2 * c2 + x1 * s2;
  }
}

__global__ void __launch_bounds__(kThreads) rope_vec_kernel(RopeArgs a) {
  const int half = a.d >> 1, group = half >> 3;
  const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (tid >= a.b * a.t * group) return;
  const int gi = (int)(tid % group);
  const int64_t bt = tid / group;
  const int64_t ti = bt % a.t, bi = bt / a.t;
  const int64_t cs_row = bi * a.cs_b + ti * a.cs_t + (gi << 3);
  float c1[8], c2[8], s1[8], s2[8];
  load8(a.cos, cs_row, a.csdt, c1);
  load8(a.cos, cs_row + half, a.csdt, c2);
  load8(a.sin, cs_row, a.csdt, s1);
  load8(a.sin, cs_row + half, a.csdt, s2);
  // This thread's share of the heads (q heads first, then k heads); a position's heads are
  // adjacent in memory, so the threads of a position read whole contiguous rows.
  const int total_heads = a.heads[0] + a.heads[1];
  const int per = (total_heads + gridDim.y - 1) / gridDim.y;
  const int h_begin = blockIdx.y * per;
  const int h_end = min(total_heads, h_begin + per);
  for (int h0 = h_begin; h0 < h_end; h0 += kHeadsPerThread) {
    float x1[kHeadsPerThread][8], x2[kHeadsPerThread][8];
#pragma unroll
    for (int u = 0; u < kHeadsPerThread; ++u) {
      const int h = h0 + u;
      if (h < h_end) {
        const int which = h < a.heads[0] ? 0 : 1;
        const int hh = which ? h - a.heads[0] : h;
        const int64_t off = bi * a.sb[which] + hh * a.sh[which] + ti * a.st[which] + (gi << 3);
        load8(a.x[which], off, a.xdt[which], x1[u]);
        load8(a.x[which], off + half, a.xdt[which], x2[u]);
        if (which == 0 && a.add) {
          float y1[8], y2[8];
          const int64_t aoff = bi * a.asb + hh * a.ash + ti * a.ast + (gi << 3);
          load8(a.add, aoff, a.adt, y1);
          load8(a.add, aoff + half, a.adt, y2);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            x1[u][k] += y1[k];
            x2[u][k] += y2[k];
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kHeadsPerThread; ++u) {
      const int h = h0 + u;
      if (h < h_end) {
        const int which = h < a.heads[0] ? 0 : 1;
        const int hh = which ? h - a.heads[0] : h;
        float o1[8], o2[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          rotate(x1[u][k], x2[u][k], c1[k], c2[k], s1[k], s2[k], a.backward, o1[k], o2[k]);
        const int64_t orow = bi * a.osb[which] + hh * a.osh[which] + ti * a.ost[which] + (gi << 3);
        store8(a.out[which], orow, a.odt[which], o1);
        store8(a.out[which], orow + half, a.odt[which], o2);
      }
    }
  }
}

// Pipelined variant for the model's layout (the heads of a position adjacent in memory, as in a
// transposed view of the projection output): a warp owns a position; its q row, k row, cos row and
// sin row arrive in the warp's shared-memory ring by bulk async copies (rowpipe.cuh) while it
// rotates the previous position, so the bytes in flight are bounded by shared memory, not by
// registers. Lanes walk the (head, 16-byte chunk) pairs of the position; stores go straight to
// the [b, h, t, d] outputs, 128 contiguous bytes per quarter warp.
// DT: the one dtype code of q, k, cos, sin and both outputs when they all agree (the hot cases:
// all fp16, all bf16, all fp32), -2 for fp16 rows with fp32 tables, or -1 to read the codes from
// the arguments.
template <int XB, int DT>
__global__ void __launch_bounds__(rowpipe::kMaxWarps * 32, 2)
rope_pipe_kernel(RopeArgs a, int stages, int* status) {
  constexpr int EPV = 4;   // elements per lane and half: 8- or 16-byte vectors, 16 cos/sin registers
  // DT == -2: fp16 rows (q, k, q's second term, both outputs) with fp32 tables, the fused block's case
  constexpr bool kHalfRows = DT == -2;
  const int xdt_q = DT >= 0 ? DT : kHalfRows ? SOUP_F16 : a.xdt[0];
  const int xdt_k = DT >= 0 ? DT : kHalfRows ? SOUP_F16 : a.xdt[1];
  const int odt_q = DT >= 0 ? DT : kHalfRows ? SOUP_F16 : a.odt[0];
  const int odt_k = DT >= 0 ? DT : kHalfRows ? SOUP_F16 : a.odt[1];
  const int csdt = DT >= 0 ? DT : kHalfRows ? SOUP_F32 : a.csdt;
  extern __shared__ __align__(128) char smem[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int half = a.d >> 1, chunks = half / EPV;   // chunks divides 32 (checked by the host)
  const uint32_t q_bytes = (uint32_t)(a.heads[0] * a.d) * XB, k_bytes = (uint32_t)(a.heads[1] * a.d) * XB;
  const uint32_t add_bytes = a.add ? q_bytes : 0;   // the addend has q's element size (host check)
  const int adt = DT >= 0 ? DT : kHalfRows ? SOUP_F16 : a.adt;
  if (threadIdx.x == 0) s_abort = 0;
  rowpipe::Ring ring;
  ring.init(smem, q_bytes + k_bytes + add_bytes, stages, warp, lane);
  __syncthreads();
  const int64_t n_rows = a.b * a.t;
  const int64_t row0 = (int64_t)blockIdx.x * warps + warp;
  const int64_t stride = (int64_t)gridDim.x * warps;
  // Two bulk copies per position (its q heads, its k heads; a third for q's second term). The copy engine has a cost per copy,
  // so the 256-byte cos and sin rows do not go through it: every lane keeps the cos/sin values of
  // its own chunk in registers (its chunk is the same for all heads, as chunks divides 32) and
  // fetches the next position's with plain loads while it rotates the current one.
  auto request = [&](int s, int64_t row) {   // lane 0 only
    const int64_t bi = row / a.t, ti = row % a.t;
    char* dst = ring.slot_ptr(s);
    umma::mbar_expect_tx(&ring.bars[s], q_bytes + k_bytes + add_bytes);
    if (add_bytes)
      rowpipe::bulk_load(dst + q_bytes + k_bytes,
                         reinterpret_cast<const char*>(a.add) + (bi * a.asb + ti * a.ast) * XB,
                         add_bytes, &ring.bars[s]);
    if (q_bytes)
      rowpipe::bulk_load(dst, reinterpret_cast<const char*>(a.x[0]) + (bi * a.sb[0] + ti * a.st[0]) * XB,
                         q_bytes, &ring.bars[s]);
    if (k_bytes)
      rowpipe::bulk_load(dst + q_bytes,
                         reinterpret_cast<const char*>(a.x[1]) + (bi * a.sb[1] + ti * a.st[1]) * XB,
                         k_bytes, &ring.bars[s]);
  };
  int64_t next = row0;
  if (lane == 0)
    for (int s = 0; s < stages && next < n_rows; ++s, next += stride) request(s, next);
  next = __shfl_sync(0xffffffffu, next, 0);
  const int total_pairs = (a.heads[0] + a.heads[1]) * chunks;
  const int dh = 32 / chunks;
  const int h_first = lane / chunks, c = lane - h_first * chunks;
  float c1[EPV], c2[EPV], s1[EPV], s2[EPV];
  auto fetch_cs = [&](int64_t row) {
    const int64_t cs_row = (row / a.t) * a.cs_b + (row % a.t) * a.cs_t + c * EPV;
    loadv<EPV>(a.cos, cs_row, csdt, c1);
    loadv<EPV>(a.cos, cs_row + half, csdt, c2);
    loadv<EPV>(a.sin, cs_row, csdt, s1);
    loadv<EPV>(a.sin, cs_row + half, csdt, s2);
  };
  if (row0 < n_rows) fetch_cs(row0);
  for (int64_t row = row0; row < n_rows; row += stride) {
    if (!ring.wait(&s_abort, status, 13)) {
      ring.drain((int)((next - row) / stride));
      return;
    }
    const int64_t bi = row / a.t, ti = row % a.t;
    const char* src = ring.slot_ptr(ring.slot);
    int h = h_first;
#pragma unroll 2
    for (int p = lane; p < total_pairs; p += 32, h += dh) {
      const int which = h < a.heads[0] ? 0 : 1;
      const int hh = which ? h - a.heads[0] : h;
      float x1[EPV], x2[EPV], o1[EPV], o2[EPV];
      const int e = h * a.d + c * EPV;   // q heads and then k heads are adjacent in the slot as well
      unpack<EPV, XB>(ld_raw<EPV * XB>(src, (int64_t)e * XB), which ? xdt_k : xdt_q, x1);
      unpack<EPV, XB>(ld_raw<EPV * XB>(src, (int64_t)(e + half) * XB), which ? xdt_k : xdt_q, x2);
      if (add_bytes && !which) {   // q heads come first in the slot: the addend's element index is e
        float y1[EPV], y2[EPV];
        const char* more = src + q_bytes + k_bytes;
        unpack<EPV, XB>(ld_raw<EPV * XB>(more, (int64_t)e * XB), adt, y1);
        unpack<EPV, XB>(ld_raw<EPV * XB>(more, (int64_t)(e + half) * XB), adt, y2);
#pragma unroll
        for (int k = 0; k < EPV; ++k) {
          x1[k] += y1[k];
          x2[k] += y2[k];
        }
      }
#pragma unroll
      for (int k = 0; k < EPV; ++k)
        rotate(x1[k], x2[k], c1[k], c2[k], s1[k], s2[k], a.backward, o1[k], o2[k]);
      const int64_t orow = bi * a.osb[which] + hh * a.osh[which] + ti * a.ost[which] + c * EPV;
      void* dst = which ? a.out[1] : a.out[0];
      storev<EPV>(dst, orow, which ? odt_k : odt_q, o1);
      storev<EPV>(dst, orow + half, which ? odt_k : odt_q, o2);
    }
    if (row + stride < n_rows) fetch_cs(row + stride);   // in flight during the next wait
    __syncwarp();
    if (next < n_rows) {
      if (lane == 0) {
        umma::fence_proxy_async_smem();
        request(ring.slot, next);
      }
      next += stride;
    }
    ring.advance();
  }
}

// Any head_dim / strides / alignment: one thread per (b, head, t, i < half).
__global__ void __launch_bounds__(kThreads) rope_scalar_kernel(RopeArgs a) {
  const int half = a.d >> 1;
  const int total_heads = a.heads[0] + a.heads[1];
  const int64_t n = a.b * total_heads * a.t * half;
  for (int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x; idx < n;
       idx += (int64_t)gridDim.x * kThreads) {
    const int i = (int)(idx % half);
    int64_t r = idx / half;
    const int64_t ti = r % a.t; r /= a.t;
    const int h = (int)(r % total_heads);
    const int64_t bi = r / total_heads;
    const int which = h < a.heads[0] ? 0 : 1;
    const int hh = which ? h - a.heads[0] : h;
    const int64_t off = bi * a.sb[which] + hh * a.sh[which] + ti * a.st[which] + i;
    const int64_t cs_row = bi * a.cs_b + ti * a.cs_t + i;
    float o1, o2;
    float v1 = load1(a.x[which], off, a.xdt[which]), v2 = load1(a.x[which], off + half, a.xdt[which]);
    if (which == 0 && a.add) {
      const int64_t aoff = bi * a.asb + hh * a.ash + ti * a.ast + i;
      v1 += load1(a.add, aoff, a.adt);
      v2 += load1(a.add, aoff + half, a.adt);
    }
    rotate(v1, v2,
           load1(a.cos, cs_row, a.csdt), load1(a.cos, cs_row + half, a.csdt),
           load1(a.sin, cs_row, a.csdt), load1(a.sin, cs_row + half, a.csdt), a.backward, o1, o2);
    const int64_t orow = bi * a.osb[which] + hh * a.osh[which] + ti * a.ost[which] + i;
    store1(a.out[which], orow, a.odt[which], o1);
    store1(a.out[which], orow + half, a.odt[which], o2);
  }
}

inline bool mult8(int64_t v) { return (v & 7) == 0; }

}  // namespace
}  // namespace soup

extern "C" int soup_rope_sum(const void* q, const void* q_add, const void* k, const void* cos,
                             const void* sin, void* q_out, void* k_out, int64_t b, int64_t hq,
                             int64_t hk, int64_t t, int64_t d, int64_t q_sb, int64_t q_sh,
                             int64_t q_st, int64_t k_sb, int64_t k_sh, int64_t k_st, int64_t cs_b,
                             int64_t cs_t, int64_t qa_sb, int64_t qa_sh, int64_t qa_st,
                             int64_t qo_sb, int64_t qo_sh, int64_t qo_st,
                             int64_t ko_sb, int64_t ko_sh, int64_t ko_st, int q_dtype,
                             int q_add_dtype, int k_dtype, int cs_dtype, int q_out_dtype,
                             int k_out_dtype, int backward, void* stream) {
  using namespace soup;
  if (!q) hq = 0;
  if (!k) hk = 0;
  if (!hq) q_add = nullptr;
  if (b == 0 || t == 0 || hq + hk == 0) return SOUP_OK;
  if (b < 0 || t < 0 || hq < 0 || hk < 0 || d <= 0 || (d & 1))
    SOUP_FAIL(SOUP_ERR_ARG, "rope: bad shape (head_dim must be even)");
  if (!cos || !sin || (hq && !q_out) || (hk && !k_out)) SOUP_FAIL(SOUP_ERR_ARG, "rope: null pointer");
  if (!is_float_dtype(cs_dtype) || (hq && !(is_float_dtype(q_dtype) && is_float_dtype(q_out_dtype))) ||
      (hk && !(is_float_dtype(k_dtype) && is_float_dtype(k_out_dtype))))
    SOUP_FAIL(SOUP_ERR_ARG, "rope: unsupported dtype");
  if (q_add && !is_float_dtype(q_add_dtype)) SOUP_FAIL(SOUP_ERR_ARG, "rope: unsupported dtype of q's second term");
  RopeArgs a;
  a.x[0] = q; a.x[1] = k; a.out[0] = q_out; a.out[1] = k_out;
  a.add = q_add; a.adt = q_add ? q_add_dtype : q_dtype;
  a.asb = qa_sb; a.ash = qa_sh; a.ast = qa_st;
  a.sb[0] = q_sb; a.sh[0] = q_sh; a.st[0] = q_st;
  a.sb[1] = k_sb; a.sh[1] = k_sh; a.st[1] = k_st;
  a.osb[0] = qo_sb; a.osh[0] = qo_sh; a.ost[0] = qo_st;
  a.osb[1] = ko_sb; a.osh[1] = ko_sh; a.ost[1] = ko_st;
  a.heads[0] = (int)hq; a.heads[1] = (int)hk;
  a.xdt[0] = q_dtype; a.xdt[1] = k_dtype; a.odt[0] = q_out_dtype; a.odt[1] = k_out_dtype;
  a.cos = cos; a.sin = sin; a.cs_b = cs_b; a.cs_t = cs_t; a.csdt = cs_dtype;
  a.b = b; a.t = t; a.d = (int)d; a.backward = backward;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  bool vec = (d % 16 == 0) && aligned16(cos) && aligned16(sin) && mult8(cs_b) && mult8(cs_t);
  if (hq) vec = vec && aligned16(q) && aligned16(q_out) && mult8(q_sb) && mult8(q_sh) && mult8(q_st) &&
              mult8(qo_sb) && mult8(qo_sh) && mult8(qo_st) &&
              (!q_add || (aligned16(q_add) && mult8(qa_sb) && mult8(qa_sh) && mult8(qa_st)));
  if (hk) vec = vec && aligned16(k) && aligned16(k_out) && mult8(k_sb) && mult8(k_sh) && mult8(k_st) &&
              mult8(ko_sb) && mult8(ko_sh) && mult8(ko_st);
  // The pipelined kernel: both tensors with a position's heads adjacent (stride d between heads),
  // one element size for q and k, a slot that fits the ring.
  const int xb = dtype_size(hq ? q_dtype : k_dtype);
  const bool adjacent = vec && (!hq || q_sh == d) && (!hk || k_sh == d) &&
                        (!hq || !hk || dtype_size(q_dtype) == dtype_size(k_dtype)) &&
                        (!q_add || (dtype_size(q_add_dtype) == dtype_size(q_dtype) && qa_sh == d));
  rowpipe::Plan plan = {8, 0, 1, 1, 0, 0};
  const int chunks = (int)(d / 2) / 4;
  if (adjacent && chunks > 0 && 32 % chunks == 0)
    plan = rowpipe::make_plan((size_t)(hq + hk + (q_add ? hq : 0)) * d * xb, 0, false, b * t);
  int* status = plan.stages ? rowpipe::status_word() : nullptr;
  if (plan.stages && status) {
    const int dt0 = hq ? q_dtype : k_dtype;
    const bool same = (!hq || (q_dtype == dt0 && q_out_dtype == dt0)) &&
                      (!hk || (k_dtype == dt0 && k_out_dtype == dt0)) && cs_dtype == dt0 &&
                      (!q_add || q_add_dtype == dt0);
#define SOUP_ROPE_P(XB_, DT_)                                                                    \
  do {                                                                                            \
    auto kernel = rope_pipe_kernel<XB_, DT_>;                                                     \
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);    \
    kernel<<<plan.grid, plan.warps * 32, plan.smem, s>>>(a, plan.stages, status);                 \
  } while (0)
    const bool half_rows = cs_dtype == SOUP_F32 &&
                           (!hq || (q_dtype == SOUP_F16 && q_out_dtype == SOUP_F16)) &&
                           (!hk || (k_dtype == SOUP_F16 && k_out_dtype == SOUP_F16)) &&
                           (!q_add || q_add_dtype == SOUP_F16);
    if (same && dt0 == SOUP_F16) SOUP_ROPE_P(2, SOUP_F16);
    else if (half_rows) SOUP_ROPE_P(2, -2);
    else if (same && dt0 == SOUP_BF16) SOUP_ROPE_P(2, SOUP_BF16);
    else if (same && dt0 == SOUP_F32) SOUP_ROPE_P(4, SOUP_F32);
    else if (xb == 4) SOUP_ROPE_P(4, -1);
    else SOUP_ROPE_P(2, -1);
#undef SOUP_ROPE_P
  } else if (vec) {
    const int64_t threads = b * t * (d >> 4);
    // One thread walks all heads of its position when there are enough positions to fill the
    // GPU; otherwise the heads are split over grid.y so that about 2^17 threads exist.
    int64_t hsplit = (131072 + threads - 1) / threads;
    const int64_t max_split = (hq + hk + kHeadsPerThread - 1) / kHeadsPerThread;
    if (hsplit > max_split) hsplit = max_split;
    if (hsplit < 1) hsplit = 1;
    dim3 grid((unsigned)((threads + kThreads - 1) / kThreads), (unsigned)hsplit);
    rope_vec_kernel<<<grid, kThreads, 0, s>>>(a);
  } else {
    const int64_t n = b * (hq + hk) * t * (d >> 1);
    int64_t blocks = (n + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    rope_scalar_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(a);
  }
  SOUP_CHECK_LAUNCH("rope");
  return SOUP_OK;
}

extern "C" int soup_rope(const void* q, const void* k, const void* cos, const void* sin,
                         void* q_out, void* k_out, int64_t b, int64_t hq, int64_t hk, int64_t t,
                         int64_t d, int64_t q_sb, int64_t q_sh, int64_t q_st, int64_t k_sb,
                         int64_t k_sh, int64_t k_st, int64_t cs_b, int64_t cs_t, int q_dtype,
                         int k_dtype, int cs_dtype, int q_out_dtype, int k_out_dtype, int backward,
                         void* stream) {
  // contiguous [b, h, t, d] outputs, no second term
  return soup_rope_sum(q, nullptr, k, cos, sin, q_out, k_out, b, hq, hk, t, d, q_sb, q_sh, q_st,
                       k_sb, k_sh, k_st, cs_b, cs_t, 0, 0, 0, hq * t * d, t * d, d, hk * t * d, t * d, d,
                       q_dtype, q_dtype, k_dtype, cs_dtype, q_out_dtype, k_out_dtype, backward,
                       stream);
}
