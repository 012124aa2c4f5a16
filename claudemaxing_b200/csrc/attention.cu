// Causal attention inside the segments of one packed row (the batch rows of a packed training
// batch), forward and backward, for head_dim 128 and fp16 q/k/v with grouped-query heads.
//
// Forward. One CTA owns 128 consecutive query tokens of one segment and one query head. The keys
// and values it may see (its segment, up to its last token) arrive in tiles of 128 tokens by TMA
// (keys through a two-stage ring). S = Q K^T of a tile is one tcgen05 product (M 128, N 128,
// K 128) into a 128-column accumulator in tensor memory; the four softmax warps read it (thread =
// query row). The softmax is done in two passes over the key tiles, so that the output
// accumulator never has to be rescaled: the first pass only reduces the row maximum; the second
// sums the exponentials, writes P = exp(S - max) as fp16 into a 128-byte-swizzled shared-memory
// tile (the A operand) and accumulates O += P V in tensor memory (V as MN-major B operand). A
// walk of up to three key tiles keeps all its score tiles in tensor memory between the passes
// (S is formed once); a longer walk alternates two accumulators and forms every tile twice,
// which at these sizes is cheap next to the latency of a rescale round trip through tensor
// memory. The epilogue divides by the sum and writes fp16 rows and the log-sum-exp (natural log,
// of the scaled scores) per row and head. The backward kernel is described where it starts.
//
// One CTA per SM (160 KB of shared memory, 512 columns of tensor memory): a CTA's walk is a chain
// of dependent steps, so few large steps beat many small ones; CTAs take the tiles with the
// longest walks first. Every wait is bounded (umma::mbar_wait).
//
// The reference calls torch SDPA here (solution/attention.py:332-343) on a [1, 1, N, N] mask
// built by its packing (solution/lm_head_loss.py:300-337); this kernel takes the segment offsets.
#include <cuda.h>

#include "common.cuh"
#include "rowpipe.cuh"
#include "umma.cuh"

namespace soup {
namespace {

using namespace umma;

constexpr int kD = 128;          // head dimension
constexpr int kBQ = 128;         // query rows per CTA
constexpr int kBKV = 128;        // key/value rows per tile
constexpr int kStages = 2;       // key tiles in flight (the value tile has one buffer)
constexpr int kTileBytes = 128 * kD * 2;       // 32 KB: a [128 x 128] fp16 tile, two swizzled boxes
constexpr int kQBytes = kBQ * kD * 2;          // 32 KB: two boxes of [128 rows x 64 cols]
constexpr int kQBox = kBQ * 128;               // 16 KB
constexpr int kKBytes = kBKV * kD * 2;         // 32 KB: two boxes of [128 rows x 64 cols]
constexpr int kKVBox = kBKV * 128;             // 16 KB
constexpr int kPBytes = kBQ * kBKV * 2;        // 32 KB: two boxes of [128 rows x 64 cols]
constexpr int kThreads = 224;                  // warps 0-3 softmax, 4 key TMA, 5 MMA, 6 value TMA
constexpr uint32_t kTmemCols = 512;            // score tiles from column 0, O behind them

struct __align__(1024) Smem {
  uint8_t q[kQBytes];
  uint8_t k[kStages][kKBytes];
  uint8_t v[kKBytes];
  uint8_t p[kPBytes];
  uint64_t q_full, k_full[kStages], k_empty[kStages], v_full, v_empty, s_full[3], s_empty[2], p_full,
      p_empty, o_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct AttnArgs {
  const int32_t* cu;     // [segments + 1]
  __half* out;           // [n, hq, 128]
  float* lse;            // [hq, n]
  int n, segments, hq, group;
  float scale_log2;      // softmax scale * log2(e)
  float scale;
  int* status;
};

// Which (segment, first query token) a tile slot is: slots enumerate the 128-row tiles of the
// segments in order. Returns false for a slot past the last tile.
__device__ __forceinline__ bool locate(const int32_t* cu, int segments, int slot, int& seg_begin,
                                       int& seg_end, int& q0) {
  int base = 0;
  for (int s = 0; s < segments; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int tiles = (e - b + kBQ - 1) / kBQ;
    if (slot < base + tiles) {
      seg_begin = b;
      seg_end = e;
      q0 = b + (slot - base) * kBQ;
      return true;
    }
    base += tiles;
  }
  return false;
}


// Four 16-byte chunks (32 fp16 columns starting at column `col0`, a multiple of 32) of row r of a
// [128 x 128] fp16 tile stored as two 128-byte-swizzled boxes of 64 columns.
__device__ __forceinline__ void write_tile_chunks(uint8_t* tile, int r, int col0, const uint32_t (&w)[16]) {
  uint8_t* row = tile + (col0 >> 6) * (kTileBytes / 2) + r * 128;
  const int j0 = (col0 & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(row + (((j0 + j) ^ (r & 7)) << 4)) =
        make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}

// Like `locate`, but the slots go through the tiles in the order of their walks' lengths: the
// last tile of every segment first, then the ones before them, and so on.
__device__ __forceinline__ bool locate_heavy_first(const int32_t* cu, int segments, int slot,
                                                   int& seg_begin, int& seg_end, int& q0) {
  if (segments > 64) return locate(cu, segments, slot, seg_begin, seg_end, q0);
  int deepest = 0;
  for (int s = 0; s < segments; ++s) deepest = max(deepest, (cu[s + 1] - cu[s] + kBQ - 1) / kBQ);
  int base = 0;
  for (int level = deepest - 1; level >= 0; --level)
    for (int s = 0; s < segments; ++s) {
      const int b = cu[s], e = cu[s + 1];
      if ((e - b + kBQ - 1) / kBQ > level) {
        if (slot == base) {
          seg_begin = b;
          seg_end = e;
          q0 = b + level * kBQ;
          return true;
        }
        ++base;
      }
    }
  return false;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, AttnArgs a) {
  extern __shared__ uint8_t raw[];
  int seg_begin, seg_end, q0;
  if (!locate_heavy_first(a.cu, a.segments, blockIdx.x, seg_begin, seg_end, q0)) return;   // the whole CTA leaves
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, hk = h / a.group;
  const int q_end = min(seg_end, q0 + kBQ);                      // one past this tile's last token
  const int n_kv = (q_end - seg_begin + kBKV - 1) / kBKV;        // key tiles it may see (>= 1)
  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.k_full[i], 1);
      mbar_init(&s.k_empty[i], 1);
    }
    mbar_init(&s.v_full, 1);
    mbar_init(&s.v_empty, 1);
    for (int i = 0; i < 3; ++i) mbar_init(&s.s_full[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&s.s_empty[i], 4);
    mbar_init(&s.p_full, 4);
    mbar_init(&s.p_empty, 1);
    mbar_init(&s.o_full, 1);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(&s.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;
  // Up to three key tiles (segments of up to 384 tokens): all score tiles stay in tensor memory
  // (columns 0-383, O in 384-511), so the second pass reads them again instead of forming them
  // again and the keys are loaded once. Longer walks alternate two score accumulators and form
  // every tile twice (O in columns 256-383).
  const bool resident = n_kv <= 3;
  const uint32_t o_col = resident ? 3 * kBKV : 2 * kBKV;

  if (warp == 4) {
    // ---------------------------------------------------------------- Q and the key tiles
    if (lane == 0) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      mbar_expect_tx(&s.q_full, kQBytes);
      tma_load_2d(s.q, &map_q, h * kD, q0, &s.q_full);
      tma_load_2d(s.q + kQBox, &map_q, h * kD + 64, q0, &s.q_full);
      for (int g = 0; g < (resident ? n_kv : 2 * n_kv); ++g) {
        const int st = g % kStages;
        if (g >= kStages &&
            !mbar_wait(&s.k_empty[st], ((g / kStages) & 1) ^ 1, abort_flag, a.status, 41))
          break;
        const int row = seg_begin + (g < n_kv ? g : g - n_kv) * kBKV;
        mbar_expect_tx(&s.k_full[st], kKBytes);
        tma_load_2d(s.k[st], &map_k, hk * kD, row, &s.k_full[st]);
        tma_load_2d(s.k[st] + kKVBox, &map_k, hk * kD + 64, row, &s.k_full[st]);
      }
    }
  } else if (warp == 6) {
    // ---------------------------------------------------------------- the value tiles (pass 2)
    if (lane == 0) {
      prefetch_tensormap(&map_v);
      for (int t = 0; t < n_kv; ++t) {
        if (t > 0 && !mbar_wait(&s.v_empty, (t - 1) & 1, abort_flag, a.status, 42)) break;
        const int row = seg_begin + t * kBKV;
        mbar_expect_tx(&s.v_full, kKBytes);
        tma_load_2d(s.v, &map_v, hk * kD, row, &s.v_full);
        tma_load_2d(s.v + kKVBox, &map_v, hk * kD + 64, row, &s.v_full);
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(kBQ, kBKV, kFmtF16, kFmtF16, false, false);
      constexpr uint32_t idesc_o = make_idesc_f16(kBQ, kD, kFmtF16, kFmtF16, false, true);
      const uint64_t dq = make_smem_desc(smem_u32(s.q), 16, 1024);
      bool ok = mbar_wait(&s.q_full, 0, abort_flag, a.status, 43);
      const uint64_t dp = make_smem_desc(smem_u32(s.p), 16, 1024);
      const uint64_t dv = make_smem_desc(smem_u32(s.v), kKVBox, 1024);   // MN-major: boxes kKVBox apart
      // S = Q K^T of the key tile in stage `st` into the accumulator at column `col`: 8 steps of
      // 16 along the head dimension
      auto mma_s = [&](int st, uint32_t col) {
        const uint64_t dk = make_smem_desc(smem_u32(s.k[st]), 16, 1024);
#pragma unroll
        for (int k8 = 0; k8 < kD / 16; ++k8) {
          const uint32_t qa = (uint32_t)(k8 >> 2) * (kQBox >> 4) + (uint32_t)(k8 & 3) * 2;
          const uint32_t kb = (uint32_t)(k8 >> 2) * (kKVBox >> 4) + (uint32_t)(k8 & 3) * 2;
          mma_f16_ss(tmem + col, dq + qa, dk + kb, idesc_s, k8 != 0);
        }
      };
      // O (+)= P V along the key rows of the tile: P K-major, V MN-major
      auto mma_pv = [&](int t) {
#pragma unroll
        for (int k8 = 0; k8 < kBKV / 16; ++k8) {
          const uint32_t pa = (uint32_t)(k8 >> 2) * (kQBox >> 4) + (uint32_t)(k8 & 3) * 2;
          mma_f16_ss(tmem + o_col, dp + pa, dv + k8 * (2048 >> 4), idesc_o, (t | k8) != 0);
        }
      };
      auto issue_s = [&](int g) -> bool {   // the two-accumulator walk: tile g into accumulator g & 1
        const int st = g % kStages, sb = g & 1;
        if (!mbar_wait(&s.k_full[st], (g / kStages) & 1, abort_flag, a.status, 44)) return false;
        if (g >= 2 && !mbar_wait(&s.s_empty[sb], ((g >> 1) & 1) ^ 1, abort_flag, a.status, 45))
          return false;
        tc_fence_after_sync();
        mma_s(st, sb * kBKV);
        tc_commit(&s.s_full[sb]);
        return true;
      };
      if (resident) {
        for (int t = 0; t < n_kv && ok; ++t) {
          ok = mbar_wait(&s.k_full[t % kStages], (t / kStages) & 1, abort_flag, a.status, 44);
          if (!ok) break;
          tc_fence_after_sync();
          mma_s(t % kStages, t * kBKV);
          tc_commit(&s.s_full[t]);
          tc_commit(&s.k_empty[t % kStages]);
        }
        for (int t = 0; t < n_kv && ok; ++t) {
          ok = mbar_wait(&s.v_full, t & 1, abort_flag, a.status, 46);
          if (ok) ok = mbar_wait(&s.p_full, t & 1, abort_flag, a.status, 47);
          if (!ok) break;
          tc_fence_after_sync();
          mma_pv(t);
          tc_commit(&s.v_empty);
          tc_commit(&s.p_empty);
        }
      } else {
        for (int g = 0; g < n_kv && ok; ++g) {   // pass 1: scores only
          ok = issue_s(g);
          if (ok) tc_commit(&s.k_empty[g % kStages]);
        }
        if (ok) ok = issue_s(n_kv);
        for (int t = 0; t < n_kv && ok; ++t) {   // pass 2: scores of the next tile, then O += P V
          const int g = n_kv + t;
          if (t + 1 < n_kv) ok = issue_s(g + 1);
          if (ok) ok = mbar_wait(&s.v_full, t & 1, abort_flag, a.status, 46);
          if (ok) ok = mbar_wait(&s.p_full, t & 1, abort_flag, a.status, 47);
          if (!ok) break;
          tc_fence_after_sync();
          mma_pv(t);
          tc_commit(&s.k_empty[g % kStages]);
          tc_commit(&s.v_empty);
          tc_commit(&s.p_empty);
        }
      }
      if (ok) tc_commit(&s.o_full);
    }
  } else {
    // ---------------------------------------------------------------- softmax: thread = query row
    const int r = threadIdx.x;
    const int q_idx = q0 + r;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const float sl = a.scale_log2;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int g = 0; g < 2 * n_kv && ok; ++g) {
      const int sb = g & 1;
      const int tile = g < n_kv ? g : g - n_kv;
      const uint32_t s_col = resident ? tile * kBKV : sb * kBKV;
      if (!resident || g < n_kv) {   // resident tiles are complete once pass 1 has seen them
        ok = resident ? mbar_wait(&s.s_full[tile], 0, abort_flag, a.status, 48)
                      : mbar_wait(&s.s_full[sb], (g >> 1) & 1, abort_flag, a.status, 48);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      tc_fence_after_sync();
      const int t = g < n_kv ? g : g - n_kv;
      const int limit = q_idx - (seg_begin + t * kBKV);   // columns 0..limit are visible
      if (g < n_kv) {   // pass 1: the row maximum only
#pragma unroll 1
        for (int c0 = 0; c0 < kBKV; c0 += 32) {
          uint32_t x[32];
          tmem_ld_32x32(lane_base + s_col + c0, x);
          tmem_ld_wait_on(x);
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (c0 + c <= limit) m = fmaxf(m, __uint_as_float(x[c]));
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0 && !resident) mbar_arrive(&s.s_empty[sb]);
      } else {          // pass 2: P = exp(S - max) as the fp16 A operand of O += P V
        if (t > 0) {
          ok = mbar_wait(&s.p_empty, (t - 1) & 1, abort_flag, a.status, 49);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < kBKV; c0 += 32) {
          uint32_t x[32], packed[16];
          tmem_ld_32x32(lane_base + s_col + c0, x);
          tmem_ld_wait_on(x);
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float p0 = c0 + c <= limit ? exp2f((__uint_as_float(x[c]) - m) * sl) : 0.f;
            const float p1 = c0 + c + 1 <= limit ? exp2f((__uint_as_float(x[c + 1]) - m) * sl) : 0.f;
            l += p0 + p1;       // the sum of exponentials, from the values before rounding
            __half2 hh = __floats2half2_rn(p0, p1);
            packed[c >> 1] = *reinterpret_cast<uint32_t*>(&hh);
          }
          write_tile_chunks(s.p, r, c0, packed);
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (!resident) mbar_arrive(&s.s_empty[sb]);
          mbar_arrive(&s.p_full);
        }
      }
    }
    if (ok) {
      ok = mbar_wait(&s.o_full, 0, abort_flag, a.status, 50);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.f / l;
      const bool valid = q_idx < seg_end;
      __half* dst = a.out + ((size_t)q_idx * a.hq + h) * kD;
#pragma unroll
      for (int c0 = 0; c0 < kD; c0 += 32) {
        uint32_t o[32];
        tmem_ld_32x32(lane_base + o_col + c0, o);
        tmem_ld_wait_on(o);
        if (valid) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __half2 hh = __floats2half2_rn(__uint_as_float(o[8 * j + 2 * e]) * inv,
                                             __uint_as_float(o[8 * j + 2 * e + 1]) * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(dst + c0 + 8 * j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (valid) a.lse[(size_t)h * a.n + q_idx] = m * a.scale + logf(l);
      tc_fence_before_sync();
    }
  }
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace
}  // namespace soup

namespace soup {
namespace {

// ------------------------------------------------------------------------------------------
// Backward. Same decomposition as forward (a CTA owns 128 query tokens of one segment and one
// query head and walks the key tiles it may see), but with key tiles of 128 tokens and one CTA
// per SM: the walk is a chain of dependent steps, so fewer and larger steps are what shorten it.
// Per key tile:
//   S = Q K^T and dP = dO V^T            (two products into tensor-memory columns 0-127 / 128-255)
//   P = exp(scale S - lse), dS = P (dP - D)   by the four row warps (D = rowsum(dO o O), formed
//                                         by the same threads when the kernel starts)
//   dV^T = dO^T P, dK^T = Q^T dS          (A and B both MN-major; into the columns S and dP left)
//   dQ  += dS K                            (accumulates over the key tiles in columns 256-383)
// dV^T and dK^T come out with the head dimension on the tensor-memory lanes; the row warps stage
// them in shared memory as [key row][head dim] fp32 (over the V, P, dS and K tiles, all dead by
// then) and bulk reductions (cp.reduce.async.bulk) add each key row to the fp32 dK / dV buffers:
// the query heads of a group and the query tiles of a segment all add into the same rows. dQ
// needs no atomics; it is scaled, rounded to fp16 and stored when the walk ends. CTAs take the
// tiles with the longest walks first (`locate_heavy_first`), so that the few CTAs beyond one per
// SM are short ones.
constexpr int kBKVb = 128;                     // key rows per tile in backward
constexpr uint32_t kTmemColsBwd = 512;         // S/dV^T [0,128) dP/dK^T [128,256) dQ [256,384)

struct BwdSmem {
  uint8_t q[kTileBytes];
  uint8_t d_o[kTileBytes];
  uint8_t v[kTileBytes];     // V_t; with p: the fp32 staging tile of dV
  uint8_t p[kTileBytes];
  uint8_t ds[kTileBytes];    // dS_t; with k: the fp32 staging tile of dK
  uint8_t k[kTileBytes];
  uint64_t q_full, k_full, k_empty, v_full, v_empty, sdp_full, pds_full, grads_full, acc_free;
  uint32_t tmem_base;
  int abort_flag;
};

struct AttnBwdArgs {
  const int32_t* cu;
  const __half* out;     // [n, hq, 128]
  const __half* d_out;   // [n, hq, 128]
  const float* lse;      // [hq, n]
  __half* dq;            // [n, hq, 128]
  float* dk;             // [n, hk, 128] fp32, zero on entry
  float* dv;             // [n, hk, 128] fp32, zero on entry
  int n, segments, hq, hk, group;
  float scale_log2, scale;
  int* status;
};

// Adds `bytes` of fp32 values in shared memory to global memory (both 16-byte aligned, bytes a
// multiple of 16) by one bulk asynchronous reduction; part of the thread's current bulk group.
__device__ __forceinline__ void bulk_red_add_f32(float* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void row_warps_sync() {   // the four row warps, named barrier 1
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                AttnBwdArgs a) {
  extern __shared__ uint8_t raw[];
  int seg_begin, seg_end, q0;
  if (!locate_heavy_first(a.cu, a.segments, blockIdx.x, seg_begin, seg_end, q0)) return;
  BwdSmem& s = *reinterpret_cast<BwdSmem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, hk = h / a.group;
  const int q_end = min(seg_end, q0 + kBQ);
  const int n_kv = (q_end - seg_begin + kBKVb - 1) / kBKVb;
  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    mbar_init(&s.k_full, 1);
    mbar_init(&s.k_empty, 1);
    mbar_init(&s.v_full, 1);
    mbar_init(&s.v_empty, 1);
    mbar_init(&s.sdp_full, 1);
    mbar_init(&s.pds_full, 4);
    mbar_init(&s.grads_full, 1);
    mbar_init(&s.acc_free, 4);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(&s.tmem_base, kTmemColsBwd);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;
  constexpr int kBox = kTileBytes / 2;   // one [128 rows x 64 cols] box

  if (warp == 4) {
    if (lane == 0) {   // Q, dO, then the key tiles
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_do);
      prefetch_tensormap(&map_k);
      mbar_expect_tx(&s.q_full, 2 * kTileBytes);
      tma_load_2d(s.q, &map_q, h * kD, q0, &s.q_full);
      tma_load_2d(s.q + kBox, &map_q, h * kD + 64, q0, &s.q_full);
      tma_load_2d(s.d_o, &map_do, h * kD, q0, &s.q_full);
      tma_load_2d(s.d_o + kBox, &map_do, h * kD + 64, q0, &s.q_full);
      for (int t = 0; t < n_kv; ++t) {
        if (t > 0 && !mbar_wait(&s.k_empty, (t - 1) & 1, abort_flag, a.status, 51)) break;
        const int row = seg_begin + t * kBKVb;
        mbar_expect_tx(&s.k_full, kTileBytes);
        tma_load_2d(s.k, &map_k, hk * kD, row, &s.k_full);
        tma_load_2d(s.k + kBox, &map_k, hk * kD + 64, row, &s.k_full);
      }
    }
  } else if (warp == 6) {
    if (lane == 0) {   // the value tiles
      prefetch_tensormap(&map_v);
      for (int t = 0; t < n_kv; ++t) {
        if (t > 0 && !mbar_wait(&s.v_empty, (t - 1) & 1, abort_flag, a.status, 52)) break;
        const int row = seg_begin + t * kBKVb;
        mbar_expect_tx(&s.v_full, kTileBytes);
        tma_load_2d(s.v, &map_v, hk * kD, row, &s.v_full);
        tma_load_2d(s.v + kBox, &map_v, hk * kD + 64, row, &s.v_full);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // every operand is a [128 x 128] fp16 tile of two swizzled boxes: K-major steps of 16
      // columns advance 32 bytes inside a box (4 per box); MN-major steps of 16 rows advance
      // 2048 bytes, the two boxes being the leading-dimension offset apart
      constexpr uint32_t idesc_s = make_idesc_f16(kBQ, kBKVb, kFmtF16, kFmtF16, false, false);
      constexpr uint32_t idesc_t = make_idesc_f16(kD, kBKVb, kFmtF16, kFmtF16, true, true);
      constexpr uint32_t idesc_q = make_idesc_f16(kBQ, kD, kFmtF16, kFmtF16, false, true);
      const uint64_t q_k = make_smem_desc(smem_u32(s.q), 16, 1024);
      const uint64_t do_k = make_smem_desc(smem_u32(s.d_o), 16, 1024);
      const uint64_t k_k = make_smem_desc(smem_u32(s.k), 16, 1024);
      const uint64_t v_k = make_smem_desc(smem_u32(s.v), 16, 1024);
      const uint64_t ds_k = make_smem_desc(smem_u32(s.ds), 16, 1024);
      const uint64_t q_mn = make_smem_desc(smem_u32(s.q), kBox, 1024);
      const uint64_t do_mn = make_smem_desc(smem_u32(s.d_o), kBox, 1024);
      const uint64_t k_mn = make_smem_desc(smem_u32(s.k), kBox, 1024);
      const uint64_t p_mn = make_smem_desc(smem_u32(s.p), kBox, 1024);
      const uint64_t ds_mn = make_smem_desc(smem_u32(s.ds), kBox, 1024);
      auto kstep = [](int k8) { return (uint32_t)(k8 >> 2) * (uint32_t)(kBox >> 4) + (uint32_t)(k8 & 3) * 2u; };
      bool ok = mbar_wait(&s.q_full, 0, abort_flag, a.status, 53);
      for (int t = 0; t < n_kv && ok; ++t) {
        ok = mbar_wait(&s.k_full, t & 1, abort_flag, a.status, 54);
        if (ok && t > 0) ok = mbar_wait(&s.acc_free, (t - 1) & 1, abort_flag, a.status, 56);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k8 = 0; k8 < kD / 16; ++k8)
          mma_f16_ss(tmem, q_k + kstep(k8), k_k + kstep(k8), idesc_s, k8 != 0);
        ok = mbar_wait(&s.v_full, t & 1, abort_flag, a.status, 55);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k8 = 0; k8 < kD / 16; ++k8)
          mma_f16_ss(tmem + 128, do_k + kstep(k8), v_k + kstep(k8), idesc_s, k8 != 0);
        tc_commit(&s.sdp_full);
        ok = mbar_wait(&s.pds_full, t & 1, abort_flag, a.status, 57);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k8 = 0; k8 < kBQ / 16; ++k8)   // along the query rows
          mma_f16_ss(tmem, do_mn + k8 * (2048 >> 4), p_mn + k8 * (2048 >> 4), idesc_t, k8 != 0);
#pragma unroll
        for (int k8 = 0; k8 < kBQ / 16; ++k8)
          mma_f16_ss(tmem + 128, q_mn + k8 * (2048 >> 4), ds_mn + k8 * (2048 >> 4), idesc_t, k8 != 0);
#pragma unroll
        for (int k8 = 0; k8 < kBKVb / 16; ++k8)  // along the key rows of the tile
          mma_f16_ss(tmem + 256, ds_k + kstep(k8), k_mn + k8 * (2048 >> 4), idesc_q, (t | k8) != 0);
        tc_commit(&s.grads_full);
      }
    }
  } else {
    const int r = threadIdx.x;
    const int q_idx = q0 + r;
    const bool valid = q_idx < seg_end;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    // D = rowsum(dO o O) and the row's log-sum-exp (in log2 units)
    float delta = 0.f, lse2 = 0.f;
    if (valid) {
      const uint4* po = reinterpret_cast<const uint4*>(a.out + ((size_t)q_idx * a.hq + h) * kD);
      const uint4* pg = reinterpret_cast<const uint4*>(a.d_out + ((size_t)q_idx * a.hq + h) * kD);
#pragma unroll
      for (int i = 0; i < kD / 8; ++i) {
        const uint4 x = po[i], y = pg[i];
        const __half2* xh = reinterpret_cast<const __half2*>(&x);
        const __half2* yh = reinterpret_cast<const __half2*>(&y);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 xf = __half22float2(xh[e]), yf = __half22float2(yh[e]);
          delta = fmaf(xf.x, yf.x, fmaf(xf.y, yf.y, delta));
        }
      }
      lse2 = a.lse[(size_t)h * a.n + q_idx] * 1.4426950408889634f;
    }
    const float sl = a.scale_log2;
    const int d_idx = warp * 32 + lane;          // this thread's row of dV^T / dK^T
    bool ok = true;
    for (int t = 0; t < n_kv && ok; ++t) {
      const int kv0 = seg_begin + t * kBKVb;
      ok = mbar_wait(&s.sdp_full, t & 1, abort_flag, a.status, 58);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int limit = valid ? q_idx - kv0 : -1;    // columns 0..limit are visible
#pragma unroll 1
      for (int c0 = 0; c0 < kBKVb; c0 += 32) {
        uint32_t x[32], y[32], pp[16], ds[16];
        tmem_ld_32x32(lane_base + c0, x);
        tmem_ld_32x32(lane_base + 128 + c0, y);
        tmem_ld_wait_on(x);
        tmem_ld_wait_on(y);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float p0 = 0.f, p1 = 0.f;
          if (c0 + c <= limit) p0 = exp2f(fmaf(__uint_as_float(x[c]), sl, -lse2));
          if (c0 + c + 1 <= limit) p1 = exp2f(fmaf(__uint_as_float(x[c + 1]), sl, -lse2));
          const float g0 = p0 * (__uint_as_float(y[c]) - delta);
          const float g1 = p1 * (__uint_as_float(y[c + 1]) - delta);
          __half2 ph = __floats2half2_rn(p0, p1), gh = __floats2half2_rn(g0, g1);
          pp[c >> 1] = *reinterpret_cast<uint32_t*>(&ph);
          ds[c >> 1] = *reinterpret_cast<uint32_t*>(&gh);
        }
        write_tile_chunks(s.p, r, c0, pp);
        write_tile_chunks(s.ds, r, c0, ds);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.pds_full);
      ok = mbar_wait(&s.grads_full, t & 1, abort_flag, a.status, 59);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      // dV^T and dK^T leave through shared memory: thread d writes its values as column d of a
      // [128 key rows x 128] fp32 tile (dV over the V and P tiles, dK over the dS and K tiles, all
      // four dead now), and thread r adds key row r of both to global memory with two bulk
      // reductions: the copy engine does the atomic adds.
      float* stage_v = reinterpret_cast<float*>(s.v);
      float* stage_k = reinterpret_cast<float*>(s.ds);
#pragma unroll 1
      for (int c0 = 0; c0 < kBKVb; c0 += 32) {
        uint32_t x[32], y[32];
        tmem_ld_32x32(lane_base + c0, x);
        tmem_ld_32x32(lane_base + 128 + c0, y);
        tmem_ld_wait_on(x);
        tmem_ld_wait_on(y);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          stage_v[(c0 + c) * kD + d_idx] = __uint_as_float(x[c]);
          stage_k[(c0 + c) * kD + d_idx] = __uint_as_float(y[c]) * a.scale;
        }
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      row_warps_sync();
      if (lane == 0) mbar_arrive(&s.acc_free);        // the accumulators have been read
      if (kv0 + r < q_end) {                          // key row r of this tile exists for this CTA
        const size_t row = ((size_t)(kv0 + r) * a.hk + hk) * kD;
        bulk_red_add_f32(a.dv + row, stage_v + r * kD, kD * sizeof(float));
        bulk_red_add_f32(a.dk + row, stage_k + r * kD, kD * sizeof(float));
      }
      tma_store_commit();
      tma_store_wait_read<0>();    // the staged rows have been read: the tiles can be reloaded
      row_warps_sync();
      if (r == 0) {
        mbar_arrive(&s.k_empty);
        mbar_arrive(&s.v_empty);
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // this thread's reductions have landed
    if (ok) {   // dQ: complete once the last tile's products are (grads_full of the last step)
      __half* dst = a.dq + ((size_t)q_idx * a.hq + h) * kD;
#pragma unroll
      for (int c0 = 0; c0 < kD; c0 += 32) {
        uint32_t o[32];
        tmem_ld_32x32(lane_base + 256 + c0, o);
        tmem_ld_wait_on(o);
        if (valid) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __half2 hh = __floats2half2_rn(__uint_as_float(o[8 * j + 2 * e]) * a.scale,
                                             __uint_as_float(o[8 * j + 2 * e + 1]) * a.scale);
              w[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(dst + c0 + 8 * j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      tc_fence_before_sync();
    }
  }
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemColsBwd);
  }
}
}  // namespace
}  // namespace soup

extern "C" int soup_attn_fwd(const void* q, const void* k, const void* v, const int32_t* cu_rows,
                             void* out, float* lse, int64_t n_tokens, int64_t n_segments,
                             int64_t hq, int64_t hk, int64_t head_dim, int64_t q_pitch,
                             int64_t k_pitch, int64_t v_pitch, float scale, void* stream) {
  using namespace soup;
  if (n_tokens == 0 || n_segments == 0) return SOUP_OK;
  if (!q || !k || !v || !cu_rows || !out || !lse) SOUP_FAIL(SOUP_ERR_ARG, "attn_fwd: null pointer");
  if (head_dim != kD) SOUP_FAIL(SOUP_ERR_ARG, "attn_fwd: head_dim must be 128");
  if (n_tokens < 0 || n_segments < 0 || hq <= 0 || hk <= 0 || hq % hk)
    SOUP_FAIL(SOUP_ERR_ARG, "attn_fwd: bad sizes (query heads must be a multiple of key heads)");
  if (n_tokens > (1 << 30) || n_segments > 65535 || hq > 65535)
    SOUP_FAIL(SOUP_ERR_ARG, "attn_fwd: too many tokens, segments or heads");
  if (q_pitch < hq * kD || k_pitch < hk * kD || v_pitch < hk * kD || (q_pitch | k_pitch | v_pitch) & 7)
    SOUP_FAIL(SOUP_ERR_ARG, "attn_fwd: row pitches must cover the heads and be multiples of 8 elements");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
    SOUP_FAIL(SOUP_ERR_ARG, "attn_fwd: pointers must be 16-byte aligned");
  // a runtime call first: it makes the device's context current on this thread (autograd runs
  // backward on threads of its own), which the driver's tensor-map encoder needs
  const size_t smem = sizeof(Smem) + 1024;
  if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "attn_fwd: shared memory attribute");
  CUtensorMap mq, mk, mv;
  if (umma::encode_map_2d_16bit(&mq, q, (uint64_t)n_tokens, (uint64_t)(hq * kD), (uint64_t)q_pitch, kBQ, 64, false) ||
      umma::encode_map_2d_16bit(&mk, k, (uint64_t)n_tokens, (uint64_t)(hk * kD), (uint64_t)k_pitch, kBKV, 64, false) ||
      umma::encode_map_2d_16bit(&mv, v, (uint64_t)n_tokens, (uint64_t)(hk * kD), (uint64_t)v_pitch, kBKV, 64, false))
    SOUP_FAIL(SOUP_ERR_LAUNCH, "attn_fwd: cuTensorMapEncodeTiled failed");
  AttnArgs a;
  a.cu = cu_rows;
  a.out = reinterpret_cast<__half*>(out);
  a.lse = lse;
  a.n = (int)n_tokens;
  a.segments = (int)n_segments;
  a.hq = (int)hq;
  a.group = (int)(hq / hk);
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = rowpipe::status_word();
  // every segment adds at most one partial tile to the tiles of the packed row
  const unsigned slots = (unsigned)((n_tokens + kBQ - 1) / kBQ + n_segments);
  dim3 grid(slots, (unsigned)hq);
  attn_fwd_kernel<<<grid, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(mq, mk, mv, a);
  SOUP_CHECK_LAUNCH("attn_fwd");
  return SOUP_OK;
}

extern "C" int soup_attn_bwd(const void* q, const void* k, const void* v, const void* out,
                             const void* d_out, const float* lse, const int32_t* cu_rows, void* dq,
                             float* dk, float* dv, int64_t n_tokens, int64_t n_segments, int64_t hq,
                             int64_t hk, int64_t head_dim, int64_t q_pitch, int64_t k_pitch,
                             int64_t v_pitch, float scale, void* stream) {
  using namespace soup;
  if (n_tokens == 0 || n_segments == 0) return SOUP_OK;
  if (!q || !k || !v || !out || !d_out || !lse || !cu_rows || !dq || !dk || !dv)
    SOUP_FAIL(SOUP_ERR_ARG, "attn_bwd: null pointer");
  if (head_dim != kD) SOUP_FAIL(SOUP_ERR_ARG, "attn_bwd: head_dim must be 128");
  if (n_tokens < 0 || n_segments < 0 || hq <= 0 || hk <= 0 || hq % hk)
    SOUP_FAIL(SOUP_ERR_ARG, "attn_bwd: bad sizes (query heads must be a multiple of key heads)");
  if (n_tokens > (1 << 30) || n_segments > 65535 || hq > 65535)
    SOUP_FAIL(SOUP_ERR_ARG, "attn_bwd: too many tokens, segments or heads");
  if (q_pitch < hq * kD || k_pitch < hk * kD || v_pitch < hk * kD || (q_pitch | k_pitch | v_pitch) & 7)
    SOUP_FAIL(SOUP_ERR_ARG, "attn_bwd: row pitches must cover the heads and be multiples of 8 elements");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(d_out) || !aligned16(dq))
    SOUP_FAIL(SOUP_ERR_ARG, "attn_bwd: pointers must be 16-byte aligned");
  // a runtime call first (see soup_attn_fwd): backward usually runs on an autograd thread
  const size_t smem = sizeof(BwdSmem) + 1024;
  if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "attn_bwd: shared memory attribute");
  CUtensorMap mq, mdo, mk, mv;
  const int e_q = umma::encode_map_2d_16bit(&mq, q, (uint64_t)n_tokens, (uint64_t)(hq * kD), (uint64_t)q_pitch, kBQ, 64, false);
  const int e_do = umma::encode_map_2d_16bit(&mdo, d_out, (uint64_t)n_tokens, (uint64_t)(hq * kD), (uint64_t)(hq * kD), kBQ, 64, false);
  const int e_k = umma::encode_map_2d_16bit(&mk, k, (uint64_t)n_tokens, (uint64_t)(hk * kD), (uint64_t)k_pitch, kBKVb, 64, false);
  const int e_v = umma::encode_map_2d_16bit(&mv, v, (uint64_t)n_tokens, (uint64_t)(hk * kD), (uint64_t)v_pitch, kBKVb, 64, false);
  if (e_q || e_do || e_k || e_v)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "attn_bwd: cuTensorMapEncodeTiled failed (q %d, d_out %d, k %d, v %d)", e_q, e_do, e_k, e_v);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t kv_bytes = (size_t)n_tokens * hk * kD * sizeof(float);
  const bool adjacent = reinterpret_cast<char*>(dk) + kv_bytes == reinterpret_cast<char*>(dv);
  if (cudaMemsetAsync(dk, 0, adjacent ? 2 * kv_bytes : kv_bytes, st) != cudaSuccess ||
      (!adjacent && cudaMemsetAsync(dv, 0, kv_bytes, st) != cudaSuccess))
    SOUP_FAIL(SOUP_ERR_LAUNCH, "attn_bwd: clearing dk / dv failed");
  AttnBwdArgs a;
  a.cu = cu_rows;
  a.out = reinterpret_cast<const __half*>(out);
  a.d_out = reinterpret_cast<const __half*>(d_out);
  a.lse = lse;
  a.dq = reinterpret_cast<__half*>(dq);
  a.dk = dk;
  a.dv = dv;
  a.n = (int)n_tokens;
  a.segments = (int)n_segments;
  a.hq = (int)hq;
  a.hk = (int)hk;
  a.group = (int)(hq / hk);
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = rowpipe::status_word();
  const unsigned slots = (unsigned)((n_tokens + kBQ - 1) / kBQ + n_segments);
  dim3 grid(slots, (unsigned)hq);
  attn_bwd_kernel<<<grid, kThreads, smem, st>>>(mq, mdo, mk, mv, a);
  SOUP_CHECK_LAUNCH("attn_bwd");
  return SOUP_OK;
}
