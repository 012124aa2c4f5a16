// Fused LM head + cross-entropy, forward and hidden-state gradient, without the logits in HBM.
//
// The vocabulary is walked in chunks of column tiles (256 columns each): a first chunk of one
// wave of CTA pairs, then chunks of eight waves. Per chunk three kernels run back to back on the
// caller's stream; a chunk's probabilities pass from the first to the third through a bf16 buffer
// in HBM (the GEMMs leave more than 80 % of the memory bandwidth unused):
//
//   logits kernel  tcgen05 GEMM  S = H[rows,K] * W[cols,K]^T on CTA pairs (cta_group::2): a pair
//                  owns a 256 x 256 tile, each CTA 128 rows of it and half of the W columns, fp32
//                  accumulators double-buffered in TMEM, TMA-fed 6-stage ring. The epilogue never
//                  writes S. In one sweep over the accumulator it forms, against the row's running
//                  log-sum-exp `ref` of all earlier chunks, e = exp(z - ref), the tile's sum e and
//                  sum e*z, the tile maximum with its first index, the label's logit, and stores
//                  P = bf16(e) (label column and unlabelled rows zeroed) through a swizzled staging
//                  box and a TMA store. bf16 keeps fp32's exponent range, so a logit far above
//                  everything seen so far cannot overflow P.
//   row kernel     one warp per row: adds the tile sums to the running state (the state is kept
//                  normalised: run_max = lse so far, run_sum = 1), and sets the row's multiplier
//                  exp(ref - base) for this chunk's gradient contribution.
//   grad kernel    tcgen05 GEMM  dH += mult * P[rows,cols] * W[cols,K] on CTA pairs, 256 x 256
//                  tiles with the vocabulary (K) dimension split so that all SMs have work; W is
//                  the MN-major operand straight from its row-major storage. kind::f16 wants the
//                  same element format for both operands, so this GEMM reads a bf16 copy of W
//                  (made once per frozen weight by the caller). Partial sums are added with
//                  fire-and-forget reductions; dH is kept relative to `base`, the lse after the
//                  first chunk.
//
// The first chunk has no earlier lse: its statistics and its P are taken against each tile's own
// maximum (two sweeps over the accumulator), the row kernel merges the tiles, and a small kernel
// rescales the chunk's P in place to the merged lse. A last kernel
// turns the state into loss / entropy / correct, rescales dH from `base` to the final lse and
// adds (p_label - 1) * W[label] in fp32.
//
// Relation to the reference (_FusedHeadLoss.forward, solution/lm_head_loss.py:192-245 with the
// kernel of :108-160): same single pass over W in column chunks, same carried statistics (max, sum
// exp, sum exp*z, first argmax, label logit), same GRAD_SCALE convention for the returned
// gradient. The reference rescales the accumulated gradient by exp(lse_before - lse_after) every
// chunk and writes softmax against the *new* lse in fp16; here each chunk is written against the
// lse *before* it (known when its tiles are computed) and the per-chunk multiplier is applied to
// the chunk's contribution instead, which removes the second pass over the chunk buffer.
//
// Vocabulary-parallel use: a rank passes its shard of W and the global index of its first column
// and gets its state and dH relative to its own `base` (returned in grad_ref);
// soup_lmhead_merge combines the ranks' states and soup_lmhead_finish rescales by
// exp(grad_ref - lse_global) before the caller sums dH across ranks.
#include <math.h>
#include <stdlib.h>

#include <vector>

#include "common.cuh"
#include "rowpipe.cuh"
#include "umma.cuh"

namespace soup {
namespace {

using namespace umma;

constexpr int kBM = 128;          // rows per CTA (TMEM lanes); a pair owns 2 * kBM rows
constexpr int kBN = 256;          // columns per tile (vocabulary for logits, hidden for gradient)
constexpr int kBK = 64;           // 64 16-bit elements = one 128-byte swizzle row
constexpr int kABytes = kBM * kBK * 2;            // 16 KB: this CTA's rows of the A operand
constexpr int kBHalfBytes = (kBN / 2) * kBK * 2;  // 16 KB: this CTA's half of the B operand
constexpr int kStageBytes = kABytes + kBHalfBytes;
constexpr int kStages = 6;
constexpr int kThreadsGemm = 192;  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kGradScale = 1024.0f;  // as GRAD_SCALE of the reference
constexpr float kRebase = 30.0f;       // rebase dH when the multiplier would exceed e^30
constexpr float kHot = 30.0f;          // a tile whose maximum is this far above the running lse is
                                       // written against its own maximum instead (see is_hot)
constexpr int kIgnore = -100;
constexpr int kEW = 16;                // accumulator columns per tcgen05.ld in the epilogues

constexpr int kStageP = 4 * 2 * 4096;          // logits: per epilogue warp two 32 x 64 bf16 boxes
constexpr int kStageT = 4 * 32 * 33 * 4;       // gradient: per epilogue warp a padded 32 x 32 fp32 block
constexpr int kSmemLogits = kStages * kStageBytes + kStageP + 1024 + 256;
constexpr int kSmemGrad = kStages * kStageBytes + kStageT + 1024 + 256;

// Waits until all of this thread's bulk stores have completed (written, not only read).
__device__ __forceinline__ void tma_store_wait_done() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

enum LogitsMode {
  kModeTileMax = 0,  // statistics (and P, when wanted) against the tile maximum: the first chunk
  kModePOnly = 1,    // P against ref, no statistics (kept for callers that recompute a chunk)
  kModeCombined = 2  // statistics and P against ref (all later chunks)
};

// Later chunks exponentiate against `ref`, the row's log-sum-exp over the earlier chunks. A tile
// whose maximum lies more than kHot above it ("hot": a logit far larger than anything the row has
// seen, legal for fp16 inputs) would overflow exp(z - ref); such a (row, tile) is written against
// the tile's own maximum instead. The logits epilogue and the row kernel both decide with this one
// predicate on the same two stored fp32 values, so they always agree.
__device__ __forceinline__ bool is_hot(float tile_max, float ref) {
  return tile_max > __fadd_rn(ref, kHot);
}

struct PipeState {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance() {
    if (++stage == kStages) { stage = 0; phase ^= 1u; }
  }
};

struct GemmSmem {
  uint8_t* tiles;        // 1024-byte aligned
  uint8_t* extra;        // kernel-specific staging area behind the stages
  uint64_t* full;        // [kStages]  (used in the leader CTA)
  uint64_t* empty;       // [kStages]
  uint64_t* acc_full;    // [2]
  uint64_t* acc_empty;   // [2]        (used in the leader CTA)
  uint32_t* tmem_base;
  int* abort_flag;
};

template <int EXTRA_BYTES>
__device__ __forceinline__ GemmSmem carve_smem(uint8_t* raw) {
  GemmSmem s;
  const uintptr_t base = (reinterpret_cast<uintptr_t>(raw) + 1023u) & ~static_cast<uintptr_t>(1023u);
  s.tiles = reinterpret_cast<uint8_t*>(base);
  s.extra = s.tiles + kStages * kStageBytes;  // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(s.extra + EXTRA_BYTES);
  s.full = bars;
  s.empty = bars + kStages;
  s.acc_full = bars + 2 * kStages;
  s.acc_empty = bars + 2 * kStages + 2;
  s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  s.abort_flag = reinterpret_cast<int*>(s.tmem_base + 1);
  return s;
}

// ------------------------------------------------------------------------------------------
// CTA pairs (cta_group::2): each CTA brings its own 128 rows of A and half of the B columns, so a
// shared-memory stage holds half the B bytes a single CTA would need; the leader (cluster rank 0)
// issues the MMAs and each CTA receives its 128 rows of the accumulator in its own tensor memory.
// ------------------------------------------------------------------------------------------
struct PairInit {
  uint32_t tmem;
  uint32_t rank;
  bool run;
};

// Barrier set-up, tensor-memory allocation and the agreement of both CTAs on whether to run at all
// (an earlier kernel of the call may have given up). Every thread of both CTAs calls this.
__device__ __forceinline__ PairInit init_pair(const GemmSmem& s, int warp, int lane, const int* status) {
  PairInit r;
  r.rank = cluster_ctarank();
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s.acc_full[i], 1); mbar_init(&s.acc_empty[i], 8); }
    *s.abort_flag = *reinterpret_cast<const volatile int*>(status) != 0;
    fence_barrier_init();
  }
  __syncthreads();
  cluster_sync_all();
  // the leader's view decides for the pair
  r.run = ld_shared_cluster_s32(mapa_u32(smem_u32(s.abort_flag), 0)) == 0;
  cluster_sync_all();  // nobody leaves (or rewrites the flag) while the peer may still read it
  if (!r.run) { r.tmem = 0; return r; }
  if (warp == 0 && lane == 0) *s.abort_flag = 0;
  if (warp == 1) {
    tmem_alloc_pair(s.tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  r.tmem = *s.tmem_base;
  return r;
}

__device__ __forceinline__ void finish_pair(const GemmSmem& s, int warp, uint32_t tmem) {
  tc_fence_before_sync();
  __syncthreads();
  if (*s.abort_flag) {
    // A wait was abandoned: give copies that may still be in flight time to land before the
    // shared memory is released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  // The leader's MMAs read the peer's shared memory and both CTAs signal each other's barriers:
  // neither may exit before the other is done.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem, 512);
  }
}

__device__ __forceinline__ void release_accumulator(const GemmSmem& s, int ab, uint32_t rank, int lane) {
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) {
    if (rank == 0) mbar_arrive(&s.acc_empty[ab]);
    else mbar_arrive_remote(mapa_u32(smem_u32(&s.acc_empty[ab]), 0));
  }
}

// ------------------------------------------------------------------------------------------
// Logits kernel
// ------------------------------------------------------------------------------------------
struct LogitsArgs {
  const int64_t* target;   // [n_rows] of this row block
  const float* ref;        // [n_rows] running lse of the earlier chunks (modes POnly / Combined)
  float4* tile_stats;      // [n_rows, ct_stride]
                           //   TileMax : (tile max, sum exp(z - max), sum exp(z - max) z, argmax bits)
                           //   Combined: (tile max, sum exp(z - ref), sum exp(z - ref) z, argmax bits)
  float* label_logit;      // [n_rows]
  int n_rows;              // rows in this row block
  int row0;                // first row of the block inside the hidden matrix (TMA coordinate)
  int k_dim;               // hidden size
  int col0;                // first column of the chunk inside the weight shard
  int v_shard;             // columns of the weight shard
  int col_offset;          // global vocabulary index of shard column 0
  int ct;                  // column tiles in this chunk
  int ct_stride;           // row pitch of tile_stats
  int mode;                // LogitsMode
  int store_p;             // write P (gradient wanted)
  int* status;
};

// First chunk, first launch: statistics of one 128 x 256 tile for one thread (= one row) against
// the tile's own maximum. Two sweeps over the accumulator, 16 columns per tcgen05.ld with the next
// load in flight while the current columns are consumed; loop bodies stay small enough for the
// instruction cache.
template <bool FULL>
__device__ __noinline__ void tile_stats_tilemax(uint32_t taddr, int n_valid, int label_local,
                                                float& m_out, float& sum_out, float& dot_out,
                                                float& lab_out, int& arg_out) {
  constexpr int kLoads = kBN / kEW;
  uint32_t ra[kEW], rb[kEW];
  float m = -INFINITY;
  int arg = 0;
  auto sweep_max = [&](const uint32_t (&r)[kEW], int col0) {
#pragma unroll
    for (int j = 0; j < kEW; ++j) {
      const float z = __uint_as_float(r[j]);
      const int col = col0 + j;
      if ((FULL || col < n_valid) && z > m) { m = z; arg = col; }
    }
  };
  tmem_ld_32x16(taddr, ra);
#pragma unroll 1
  for (int i = 0; i < kLoads; i += 2) {
    tmem_ld_wait_on(ra);
    tmem_ld_32x16(taddr + (i + 1) * kEW, rb);
    sweep_max(ra, i * kEW);
    tmem_ld_wait_on(rb);
    if (i + 2 < kLoads) tmem_ld_32x16(taddr + (i + 2) * kEW, ra);
    sweep_max(rb, (i + 1) * kEW);
  }
  const float bias = -m * kLog2e;
  float s0 = 0.f, s1 = 0.f, d0 = 0.f, d1 = 0.f, lab = 0.f;
  auto sweep_exp = [&](const uint32_t (&r)[kEW], int col0) {
#pragma unroll
    for (int j = 0; j < kEW; j += 2) {
      const float z0 = __uint_as_float(r[j]), z1 = __uint_as_float(r[j + 1]);
      const int col = col0 + j;
      float e0 = exp2f(fmaf(z0, kLog2e, bias)), e1 = exp2f(fmaf(z1, kLog2e, bias));
      if (!FULL) {
        if (col >= n_valid) e0 = 0.f;
        if (col + 1 >= n_valid) e1 = 0.f;
      }
      s0 += e0;
      s1 += e1;
      d0 = fmaf(e0, (FULL || col < n_valid) ? z0 : 0.f, d0);
      d1 = fmaf(e1, (FULL || col + 1 < n_valid) ? z1 : 0.f, d1);
    }
    if (label_local >= col0 && label_local < col0 + kEW) {  // rare
#pragma unroll
      for (int j = 0; j < kEW; ++j)
        if (col0 + j == label_local) lab = __uint_as_float(r[j]);
    }
  };
  tmem_ld_32x16(taddr, ra);
#pragma unroll 1
  for (int i = 0; i < kLoads; i += 2) {
    tmem_ld_wait_on(ra);
    tmem_ld_32x16(taddr + (i + 1) * kEW, rb);
    sweep_exp(ra, i * kEW);
    tmem_ld_wait_on(rb);
    if (i + 2 < kLoads) tmem_ld_32x16(taddr + (i + 2) * kEW, ra);
    sweep_exp(rb, (i + 1) * kEW);
  }
  m_out = m;
  sum_out = s0 + s1;
  dot_out = d0 + d1;
  lab_out = lab;
  arg_out = arg;
}

// The tile's maximum over its valid columns (one sweep over the accumulator).
template <bool FULL>
__device__ __noinline__ float tile_max_sweep(uint32_t taddr, int n_valid) {
  constexpr int kLoads = kBN / kEW;
  uint32_t ra[kEW], rb[kEW];
  float m = -INFINITY;
  auto sweep = [&](const uint32_t (&r)[kEW], int col0) {
#pragma unroll
    for (int j = 0; j < kEW; ++j)
      if (FULL || col0 + j < n_valid) m = fmaxf(m, __uint_as_float(r[j]));
  };
  tmem_ld_32x16(taddr, ra);
#pragma unroll 1
  for (int i = 0; i < kLoads; i += 2) {
    tmem_ld_wait_on(ra);
    tmem_ld_32x16(taddr + (i + 1) * kEW, rb);
    sweep(ra, i * kEW);
    tmem_ld_wait_on(rb);
    if (i + 2 < kLoads) tmem_ld_32x16(taddr + (i + 2) * kEW, ra);
    sweep(rb, (i + 1) * kEW);
  }
  return m;
}

// All other launches: one sweep against `ref`, the row's log-sum-exp over the earlier chunks.
// e = exp(z - ref); with STATS the tile's sum e, sum e*z, maximum and first argmax; with store_p
// P = bf16(e) leaves through the warp's swizzled staging boxes (32 rows x 64 columns, 16-byte piece
// k of row r at piece k ^ (r & 7)) and one TMA store per box. `keep_mask` is 0 for rows without a
// label (their gradient is zero) and the label's own column is zeroed: its term is added exactly,
// in fp32, by the finish kernel.
template <bool FULL, bool STATS>
__device__ __noinline__ void tile_ref_pass(uint32_t taddr, int n_valid, int label_local, float ref,
                                           uint32_t keep_mask, bool store_p, const CUtensorMap* map_p,
                                           uint8_t* stage_warp, int p_col0, int p_row0, float& m_out,
                                           float& sum_out, float& dot_out, float& lab_out,
                                           int& arg_out) {
  constexpr int kLoads = kBN / kEW;       // 16
  constexpr int kPerBox = 64 / kEW;       // loads per 64-column staging box
  const int lane = threadIdx.x & 31;
  const int row_swz = lane & 7;
  uint32_t ra[kEW], rb[kEW];
  float m = -INFINITY, lab = 0.f;
  int arg = 0;
  float s0 = 0.f, s1 = 0.f, d0 = 0.f, d1 = 0.f;
  const float bias = -ref * kLog2e;
  auto sweep = [&](uint32_t (&r)[kEW], int col0, uint8_t* stage_row, int piece0) {
    uint32_t packed[kEW / 2];
    const bool has_label = label_local >= col0 && label_local < col0 + kEW;  // rare
    if (has_label) {
#pragma unroll
      for (int j = 0; j < kEW; ++j)
        if (col0 + j == label_local) lab = __uint_as_float(r[j]);
    }
#pragma unroll
    for (int j = 0; j < kEW; j += 2) {
      const float z0 = __uint_as_float(r[j]), z1 = __uint_as_float(r[j + 1]);
      const int col = col0 + j;
      float e0 = exp2f(fmaf(z0, kLog2e, bias)), e1 = exp2f(fmaf(z1, kLog2e, bias));
      if (!FULL) {
        if (col >= n_valid) e0 = 0.f;
        if (col + 1 >= n_valid) e1 = 0.f;
      }
      if (STATS) {
        if ((FULL || col < n_valid) && z0 > m) { m = z0; arg = col; }
        if ((FULL || col + 1 < n_valid) && z1 > m) { m = z1; arg = col + 1; }
        s0 += e0;
        s1 += e1;
        d0 = fmaf(e0, (FULL || col < n_valid) ? z0 : 0.f, d0);
        d1 = fmaf(e1, (FULL || col + 1 < n_valid) ? z1 : 0.f, d1);
      }
      __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
      packed[j >> 1] = *reinterpret_cast<uint32_t*>(&h) & keep_mask;
    }
    if (has_label) {  // the label's own column carries no P
#pragma unroll
      for (int j = 0; j < kEW; ++j)
        if (col0 + j == label_local) packed[j >> 1] &= (j & 1) ? 0x0000FFFFu : 0xFFFF0000u;
    }
    if (store_p) {
#pragma unroll
      for (int v = 0; v < kEW / 8; ++v) {
        const int piece = (piece0 + v) ^ row_swz;
        *reinterpret_cast<uint4*>(stage_row + piece * 16) =
            make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
      }
    }
  };
  tmem_ld_32x16(taddr, ra);
#pragma unroll 1
  for (int i = 0; i < kLoads; i += 2) {
    // 64-column boxes alternate between the warp's two staging areas; the area used two boxes ago
    // must have been read by its TMA store before it is overwritten.
    const int box_id = i / kPerBox;
    uint8_t* box = stage_warp + (box_id & 1) * 4096;
    if (store_p && (i % kPerBox) == 0) {
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
    }
    uint8_t* stage_row = box + lane * 128;
    tmem_ld_wait_on(ra);
    tmem_ld_32x16(taddr + (i + 1) * kEW, rb);
    sweep(ra, i * kEW, stage_row, (i % kPerBox) * (kEW / 8));
    tmem_ld_wait_on(rb);
    if (i + 2 < kLoads) tmem_ld_32x16(taddr + (i + 2) * kEW, ra);
    sweep(rb, (i + 1) * kEW, stage_row, ((i + 1) % kPerBox) * (kEW / 8));
    if (store_p && ((i + 2) % kPerBox) == 0) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map_p, box, p_col0 + box_id * 64, p_row0);
        tma_store_commit();
      }
    }
  }
  m_out = m;
  sum_out = s0 + s1;
  dot_out = d0 + d1;
  lab_out = lab;
  arg_out = arg;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsGemm, 1)
lmhead_logits_kernel(const __grid_constant__ CUtensorMap map_h,
                     const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_p, const LogitsArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const GemmSmem s = carve_smem<kStageP>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&map_h);
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_p);
  }
  const PairInit pi = init_pair(s, warp, lane, a.status);
  if (!pi.run) return;
  const uint32_t tmem = pi.tmem, rank = pi.rank;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  // Tiles are ordered row-tile-fastest: the row tiles that share a weight tile run together, so
  // the weight streams from HBM once.
  const int rt = (a.n_rows + 2 * kBM - 1) / (2 * kBM);   // 256-row tiles
  const int n_tiles = rt * a.ct;
  const int n_kb = (a.k_dim + kBK - 1) / kBK;

  if (warp == 0) {
    if (lane == 0) {
      PipeState p;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        const int tr = tile % rt, tc = tile / rt;
        const int row0 = a.row0 + tr * 2 * kBM + (int)rank * kBM;
        const int col0 = a.col0 + tc * kBN + (int)rank * (kBN / 2);
        for (int kb = 0; kb < n_kb; ++kb) {
          ok = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 11);
          if (!ok) break;
          uint8_t* st = s.tiles + p.stage * kStageBytes;
          // both CTAs' bytes are counted on the leader's barrier
          const uint32_t full_leader = mapa_u32(smem_u32(&s.full[p.stage]), 0);
          if (rank == 0) mbar_expect_tx(&s.full[p.stage], 2 * kStageBytes);
          tma_load_2d_pair(st, &map_h, kb * kBK, row0, full_leader);
          tma_load_2d_pair(st + kABytes, &map_w, kb * kBK, col0, full_leader);
          p.advance();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * kBM, kBN, kFmtF16, kFmtF16, false, false);
      PipeState p;
      bool ok = true;
      int it = 0;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait(&s.acc_empty[ab], acc_phase ^ 1u, s.abort_flag, a.status, 12);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + ab * kBN;
        for (int kb = 0; kb < n_kb; ++kb) {
          ok = mbar_wait(&s.full[p.stage], p.phase, s.abort_flag, a.status, 13);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.tiles + p.stage * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr, 16, 1024);
          const uint64_t db = make_smem_desc(a_addr + kABytes, 16, 1024);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            mma_f16_ss_pair(d_tmem, da + k4 * 2, db + k4 * 2, idesc, (kb | k4) != 0);
          tc_commit_pair(&s.empty[p.stage], 3);   // frees the stage in both CTAs
          p.advance();
        }
        if (ok) tc_commit_pair(&s.acc_full[ab], 3);
      }
    }
  } else {
    // Epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32).
    const int q = warp & 3;
    uint8_t* stage_warp = s.extra + (warp - 2) * 8192;
    bool ok = true;
    int it = 0;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
      const int tr = tile % rt, tc = tile / rt;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&s.acc_full[ab], acc_phase, s.abort_flag, a.status, 14));
      if (!ok) break;
      tc_fence_after_sync();
      const int p_row0 = tr * 2 * kBM + (int)rank * kBM + q * 32;   // row inside the row block
      const int row = p_row0 + lane;
      const bool row_ok = row < a.n_rows;
      const int tile_col0 = a.col0 + tc * kBN;                      // column inside the shard
      const int n_valid = min(kBN, a.v_shard - tile_col0);          // >= 1 by construction
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + ab * kBN;
      int label_local = -1;
      bool labelled = false;
      float ref = 0.f;
      if (row_ok) {
        const long long tg = a.target[row];
        labelled = tg != kIgnore;
        const long long loc = tg - a.col_offset - tile_col0;
        if (labelled && loc >= 0 && loc < n_valid) label_local = (int)loc;
        if (a.mode != kModeTileMax) ref = a.ref[row];
      }
      const uint32_t keep_mask = labelled ? 0xFFFFFFFFu : 0u;
      float m, sum, dot, lab;
      int arg;
      const bool full = n_valid == kBN;
      if (a.mode == kModeTileMax && a.store_p) {
        // first chunk with a gradient wanted: P is written against the tile's own maximum (the
        // row's lse is not known yet) and rescaled in place once the row kernel has merged the tiles
        if (full) {
          const float tm = tile_max_sweep<true>(taddr, n_valid);
          tile_ref_pass<true, true>(taddr, n_valid, label_local, tm, keep_mask, true, &map_p,
                                    stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
        } else {
          const float tm = tile_max_sweep<false>(taddr, n_valid);
          tile_ref_pass<false, true>(taddr, n_valid, label_local, tm, keep_mask, true, &map_p,
                                     stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
        }
      } else if (a.mode == kModeTileMax) {
        if (full) tile_stats_tilemax<true>(taddr, n_valid, label_local, m, sum, dot, lab, arg);
        else tile_stats_tilemax<false>(taddr, n_valid, label_local, m, sum, dot, lab, arg);
      } else if (a.mode == kModeCombined) {
        if (full)
          tile_ref_pass<true, true>(taddr, n_valid, label_local, ref, keep_mask, a.store_p != 0,
                                    &map_p, stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
        else
          tile_ref_pass<false, true>(taddr, n_valid, label_local, ref, keep_mask, a.store_p != 0,
                                     &map_p, stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
        // Rare: some row of this warp met a logit far above its running lse. The pass is repeated
        // (tcgen05.ld is warp-wide) with the hot rows exponentiated against their tile maximum;
        // the other rows get the values they had. The first pass's stores must have landed
        // before the same boxes are stored again. The row kernel sees the same predicate and
        // brings the row's tiles to one reference.
        const bool hot = row_ok && is_hot(m, ref);
        if (__any_sync(0xffffffffu, hot)) {
          if (a.store_p) {
            if (lane == 0) tma_store_wait_done();
            __syncwarp();
          }
          const float rho = hot ? m : ref;
          if (full)
            tile_ref_pass<true, true>(taddr, n_valid, label_local, rho, keep_mask, a.store_p != 0,
                                      &map_p, stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
          else
            tile_ref_pass<false, true>(taddr, n_valid, label_local, rho, keep_mask, a.store_p != 0,
                                       &map_p, stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
        }
      } else {
        if (full)
          tile_ref_pass<true, false>(taddr, n_valid, label_local, ref, keep_mask, true, &map_p,
                                     stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
        else
          tile_ref_pass<false, false>(taddr, n_valid, label_local, ref, keep_mask, true, &map_p,
                                      stage_warp, tc * kBN, p_row0, m, sum, dot, lab, arg);
      }
      release_accumulator(s, ab, rank, lane);
      if (row_ok && a.mode != kModePOnly) {
        a.tile_stats[(size_t)row * a.ct_stride + tc] =
            make_float4(m, sum, dot, __int_as_float(tile_col0 + arg + a.col_offset));
        if (label_local >= 0) a.label_logit[row] = lab;
      }
    }
    if (lane == 0) tma_store_wait_read<0>();  // staging boxes fully read before shared memory goes away
  }
  finish_pair(s, warp, tmem);
}

// ------------------------------------------------------------------------------------------
// Row kernel: one warp per row merges the chunk's tile statistics into the running state.
// The state is kept normalised: run_max = log-sum-exp so far, run_sum = 1, run_dot = sum of
// softmax-so-far * z. For the gradient it also maintains `base` (the lse dH is relative to) and
// writes the row's multiplier for this chunk's contribution.
// ------------------------------------------------------------------------------------------
struct RowArgs {
  const float4* tile_stats;
  float* run_max;
  float* run_sum;
  float* run_dot;
  int* best;
  float* best_val;  // [n_rows] largest logit so far (the state itself carries the lse, not the max)
  float* base;      // [n_rows] lse that dH is relative to (set by the first chunk)
  float* mult;      // [n_rows] out: exp(ref - base) for the gradient kernel of this chunk
  float* dh;        // nullable: [n_rows, k_dim], touched only when a row is rebased
  __nv_bfloat16* p; // nullable: the chunk's probabilities [n_rows, ld_p], touched only for hot rows
  int ld_p;
  int n_rows;
  int k_dim;
  int ct;
  int ct_stride;
  int mode;         // kModeTileMax (first chunk) or kModeCombined
  int want_grad;
  int* status;
};

__global__ void __launch_bounds__(256) lmhead_row_kernel(const RowArgs a) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= a.n_rows) return;
  const float ref = a.run_max[row];   // lse so far (-inf before the first chunk)
  float run_dot = a.run_dot[row];
  int best = a.best[row];
  float best_val = a.mode == kModeTileMax ? -INFINITY : a.best_val[row];
  float new_lse, new_dot;
  bool hot_row = false;
  if (a.mode == kModeTileMax) {
    // statistics relative to each tile's own maximum: log-sum-exp merge
    float run_max = -INFINITY, run_sum = 0.f;
    run_dot = 0.f;
    for (int t0 = 0; t0 < a.ct; t0 += 32) {
      const int t = t0 + lane;
      float4 st = make_float4(-INFINITY, 0.f, 0.f, 0.f);
      if (t < a.ct) st = a.tile_stats[(size_t)row * a.ct_stride + t];
      float gmax = st.x;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
      const unsigned holders = __ballot_sync(0xffffffffu, st.x == gmax);
      const int first = __ffs(holders) - 1;  // lowest tile that holds the maximum
      const int cand = __shfl_sync(0xffffffffu, __float_as_int(st.w), first);
      if (gmax > best_val) { best_val = gmax; best = cand; }
      const float new_max = fmaxf(run_max, gmax);
      const float w = t < a.ct ? exp2f((st.x - new_max) * kLog2e) : 0.f;
      const float part_sum = warp_sum(st.y * w);
      const float part_dot = warp_sum(st.z * w);
      const float rescale = exp2f((run_max - new_max) * kLog2e);  // exp(-inf) = 0 at the start
      run_sum = run_sum * rescale + part_sum;
      run_dot = run_dot * rescale + part_dot;
      run_max = new_max;
    }
    new_lse = run_max + logf(run_sum);
    new_dot = run_dot / run_sum;
  } else {
    // statistics relative to ref: the mass so far is exp(ref) * 1
    float add_sum = 0.f, add_dot = 0.f;
    for (int t0 = 0; t0 < a.ct; t0 += 32) {
      const int t = t0 + lane;
      float4 st = make_float4(-INFINITY, 0.f, 0.f, 0.f);
      if (t < a.ct) st = a.tile_stats[(size_t)row * a.ct_stride + t];
      float gmax = st.x;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
      const unsigned holders = __ballot_sync(0xffffffffu, st.x == gmax);
      const int first = __ffs(holders) - 1;
      const int cand = __shfl_sync(0xffffffffu, __float_as_int(st.w), first);
      if (gmax > best_val) { best_val = gmax; best = cand; }  // later tiles win only if larger
      add_sum += warp_sum(st.y);
      add_dot += warp_sum(st.z);
    }
    const float total = 1.0f + add_sum;
    new_lse = ref + logf(total);
    new_dot = (run_dot + add_dot) / total;
    // Hot tiles (is_hot: written against their own maximum, not against ref) make the sums above
    // meaningless for this row; best_val is then the largest of them. Redo the merge with every
    // tile's own reference, relative to rho = best_val.
    hot_row = is_hot(best_val, ref);
    if (hot_row) {
      const float rho = best_val;
      const float w_ref = exp2f((ref - rho) * kLog2e);   // < e^-30
      float sum = 0.f, dot = 0.f;
      for (int t0 = 0; t0 < a.ct; t0 += 32) {
        const int t = t0 + lane;
        float4 st = make_float4(-INFINITY, 0.f, 0.f, 0.f);
        if (t < a.ct) st = a.tile_stats[(size_t)row * a.ct_stride + t];
        const float w = t < a.ct ? (is_hot(st.x, ref) ? exp2f((st.x - rho) * kLog2e) : w_ref) : 0.f;
        sum += warp_sum(st.y * w);
        dot += warp_sum(st.z * w);
      }
      const float total_hot = w_ref + sum;
      new_lse = rho + logf(total_hot);
      new_dot = (run_dot * w_ref + dot) / total_hot;
    } else if (!(total < INFINITY) && lane == 0) {
      atomicCAS(a.status, 0, 90);  // cannot happen: every non-hot tile sum is below 256 e^30
    }
  }
  float mult = 1.0f;
  if (a.want_grad) {
    if (a.mode == kModeTileMax) {
      if (lane == 0) a.base[row] = new_lse;   // the first chunk's P is written against this lse
    } else if (hot_row) {
      // The chunk's P of this row mixes references (ref for ordinary tiles, the tile maximum for
      // hot ones). Bring all of it to rho = best_val, move dH of the row to the same reference and
      // let the gradient kernel add the chunk with multiplier 1. Everything that was relative to
      // ref shrinks by more than e^-30.
      const float rho = best_val;
      const float w_ref = exp2f((ref - rho) * kLog2e);
      uint4* prow = reinterpret_cast<uint4*>(a.p + (size_t)row * a.ld_p);
      for (int t = 0; t < a.ct; ++t) {
        const float tm = a.tile_stats[(size_t)row * a.ct_stride + t].x;
        const float f = is_hot(tm, ref) ? exp2f((tm - rho) * kLog2e) : w_ref;
        if (f == 1.0f) continue;
        uint4 v = prow[t * (kBN / 8) + lane];
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 e = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
          __nv_bfloat162 h = __floats2bfloat162_rn(e.x * f, e.y * f);
          w[k] = *reinterpret_cast<uint32_t*>(&h);
        }
        prow[t * (kBN / 8) + lane] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      const float down = expf(a.base[row] - rho);
      for (int i = lane; i < a.k_dim; i += 32) a.dh[(size_t)row * a.k_dim + i] *= down;
      __syncwarp();
      if (lane == 0) a.base[row] = rho;
      mult = 1.0f;
    } else {
      float base = a.base[row];
      if (ref - base > kRebase) {
        // rare: the multiplier exp(ref - base) is getting large; bring dH of this row to ref
        const float down = expf(base - ref);
        for (int i = lane; i < a.k_dim; i += 32) a.dh[(size_t)row * a.k_dim + i] *= down;
        base = ref;
        __syncwarp();
        if (lane == 0) a.base[row] = base;
      }
      mult = expf(ref - base);
    }
  }
  if (lane == 0) {
    a.run_max[row] = new_lse;
    a.run_sum[row] = 1.0f;
    a.run_dot[row] = new_dot;
    a.best[row] = best;
    a.best_val[row] = best_val;
    if (a.want_grad) a.mult[row] = mult;
  }
}

// First chunk only: P was written as exp(z - tile maximum); bring it to exp(z - lse) in place, one
// warp per row, one 16-byte vector (8 bf16) per lane and tile. A memory-bound pass over a chunk
// that is still in L2, instead of a second GEMM pass over the chunk's logits.
__global__ void __launch_bounds__(256)
lmhead_rescale_first_kernel(__nv_bfloat16* __restrict__ p, int ld_p,
                            const float4* __restrict__ tile_stats, int ct_stride,
                            const float* __restrict__ lse, int n_rows, int ct) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const float row_lse = lse[row];
  uint4* prow = reinterpret_cast<uint4*>(p + (size_t)row * ld_p);
#pragma unroll 2
  for (int t = 0; t < ct; ++t) {
    const float f = exp2f((tile_stats[(size_t)row * ct_stride + t].x - row_lse) * kLog2e);
    uint4 v = prow[t * (kBN / 8) + lane];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 e = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
      __nv_bfloat162 h = __floats2bfloat162_rn(e.x * f, e.y * f);
      w[k] = *reinterpret_cast<uint32_t*>(&h);
    }
    prow[t * (kBN / 8) + lane] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ------------------------------------------------------------------------------------------
// Gradient kernel: dH[rows, K] += mult[row] * P[rows, cols] * W[cols, K] for one chunk. A pair owns
// a 256-row x 256-hidden-column output tile; a work unit is (tile, K split). The epilogue transposes
// each 32 x 32 block of the accumulator through shared memory so that dH is touched in full
// 128-byte rows.
// ------------------------------------------------------------------------------------------
struct GradArgs {
  float* dh;            // [n_rows, k_dim] fp32 of this row block, zeroed before the first chunk
  const float* mult;    // [n_rows]
  int n_rows;
  int k_dim;            // hidden size (output columns)
  int col0;             // first shard column of the chunk (TMA row coordinate into W)
  int n_kb;             // 64-column blocks of the chunk
  int ksplit;           // K (vocabulary) splits per output tile
  int* status;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsGemm, 1)
lmhead_grad_kernel(const __grid_constant__ CUtensorMap map_p,
                   const __grid_constant__ CUtensorMap map_w, const GradArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const GemmSmem s = carve_smem<kStageT>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) { prefetch_tensormap(&map_p); prefetch_tensormap(&map_w); }
  const PairInit pi = init_pair(s, warp, lane, a.status);
  if (!pi.run) return;
  const uint32_t tmem = pi.tmem, rank = pi.rank;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  const int rt = (a.n_rows + 2 * kBM - 1) / (2 * kBM);
  const int nt = (a.k_dim + kBN - 1) / kBN;
  const int n_tiles = rt * nt;
  const int n_units = n_tiles * a.ksplit;
  constexpr int kBoxBytes = kBK * 128;   // one 64-column x 64-k box of W

  if (warp == 0) {
    if (lane == 0) {
      PipeState p;
      bool ok = true;
      for (int unit = pair; unit < n_units && ok; unit += n_pairs) {
        const int tile = unit % n_tiles, ks = unit / n_tiles;
        const int tr = tile % rt, tn = tile / rt;
        const int row0 = tr * 2 * kBM + (int)rank * kBM;
        const int hcol0 = tn * kBN + (int)rank * (kBN / 2);
        const int kb_end = (a.n_kb * (ks + 1)) / a.ksplit;
        for (int kb = (a.n_kb * ks) / a.ksplit; kb < kb_end; ++kb) {
          ok = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 21);
          if (!ok) break;
          uint8_t* st = s.tiles + p.stage * kStageBytes;
          const uint32_t full_leader = mapa_u32(smem_u32(&s.full[p.stage]), 0);
          if (rank == 0) mbar_expect_tx(&s.full[p.stage], 2 * kStageBytes);
          tma_load_2d_pair(st, &map_p, kb * kBK, row0, full_leader);
#pragma unroll
          for (int j = 0; j < kBN / 2 / 64; ++j)
            tma_load_2d_pair(st + kABytes + j * kBoxBytes, &map_w, hcol0 + j * 64, a.col0 + kb * kBK,
                             full_leader);
          p.advance();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // A = P (K-major) and B = W (MN-major), both bf16: kind::f16 wants one element format for
      // both operands (a bf16 A with an fp16 B raises an illegal-instruction fault).
      constexpr uint32_t idesc = make_idesc_f16(2 * kBM, kBN, kFmtBF16, kFmtBF16, false, true);
      PipeState p;
      bool ok = true;
      int it = 0;
      for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++it) {
        const int ks = unit / n_tiles;
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait(&s.acc_empty[ab], acc_phase ^ 1u, s.abort_flag, a.status, 22);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + ab * kBN;
        const int kb_begin = (a.n_kb * ks) / a.ksplit, kb_end = (a.n_kb * (ks + 1)) / a.ksplit;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(&s.full[p.stage], p.phase, s.abort_flag, a.status, 23);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.tiles + p.stage * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr, 16, 1024);
          // MN-major B: the two 64-column boxes are kBoxBytes apart (leading offset), 8-k groups
          // 1024 bytes apart (stride offset); one MMA consumes 16 k = 2048 bytes.
          const uint64_t db = make_smem_desc(a_addr + kABytes, kBoxBytes, 1024);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            mma_f16_ss_pair(d_tmem, da + k4 * 2, db + k4 * (2048 >> 4), idesc,
                            (kb != kb_begin) || k4 != 0);
          tc_commit_pair(&s.empty[p.stage], 3);
          p.advance();
        }
        if (ok) tc_commit_pair(&s.acc_full[ab], 3);
      }
    }
  } else {
    const int q = warp & 3;
    float* tpose = reinterpret_cast<float*>(s.extra) + (warp - 2) * (32 * 33);
    bool ok = true;
    int it = 0;
    for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++it) {
      const int tile = unit % n_tiles;
      const int tr = tile % rt, tn = tile / rt;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&s.acc_full[ab], acc_phase, s.abort_flag, a.status, 24));
      if (!ok) break;
      tc_fence_after_sync();
      const int row_base = tr * 2 * kBM + (int)rank * kBM + q * 32;   // first of this warp's 32 rows
      const float my_mult = (row_base + lane < a.n_rows) ? a.mult[row_base + lane] : 0.f;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + ab * kBN;
      const int col_base = tn * kBN;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait_on(r);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; ++j) tpose[lane * 33 + j] = __uint_as_float(r[j]) * my_mult;
        __syncwarp();
        // Fire-and-forget reductions: with one K split exactly one CTA adds to an element per
        // chunk and the result is deterministic; with several the order of the adds is not.
        const int col = col_base + c * 32 + lane;
        const bool col_ok = col < a.k_dim;
#pragma unroll 8
        for (int rr = 0; rr < 32; ++rr) {
          const int row = row_base + rr;
          if (col_ok && row < a.n_rows)
            atomicAdd(a.dh + (size_t)row * a.k_dim + col, tpose[rr * 33 + lane]);
        }
      }
      release_accumulator(s, ab, rank, lane);
    }
  }
  finish_pair(s, warp, tmem);
}

// ------------------------------------------------------------------------------------------
// Small kernels: state initialisation, merge across ranks, finish, backward scale.
// ------------------------------------------------------------------------------------------
__global__ void lmhead_init_state_kernel(float* run_max, float* run_sum, float* run_dot, int* best,
                                         float* best_val, float* label_logit, float* grad_ref,
                                         int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  run_max[i] = -INFINITY;
  run_sum[i] = 0.f;
  run_dot[i] = 0.f;
  best[i] = 0;
  best_val[i] = -INFINITY;
  label_logit[i] = 0.f;
  grad_ref[i] = 0.f;
}

// states: [n_ranks, n] each; out: [n]. Ranks are in ascending vocabulary order, so a later rank
// wins the argmax only if strictly larger. Each rank's (max, sum, dot) means: mass = sum * e^max,
// dot mass = dot * e^max.
__global__ void lmhead_merge_kernel(const float* g_max, const float* g_sum, const float* g_dot,
                                    const int* g_best, const float* g_best_val,
                                    const float* g_label_logit, const int64_t* target,
                                    const int64_t* shard_begin, float* o_max, float* o_sum,
                                    float* o_dot, int* o_best, float* o_best_val,
                                    float* o_label_logit, float* o_lse, int n, int n_ranks) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float m = -INFINITY, bv = -INFINITY;
  int best = 0;
  for (int r = 0; r < n_ranks; ++r) {
    m = fmaxf(m, g_max[(size_t)r * n + i]);
    const float v = g_best_val[(size_t)r * n + i];
    if (v > bv) { bv = v; best = g_best[(size_t)r * n + i]; }
  }
  float sum = 0.f, dot = 0.f;
  for (int r = 0; r < n_ranks; ++r) {
    const float w = exp2f((g_max[(size_t)r * n + i] - m) * kLog2e);
    sum += g_sum[(size_t)r * n + i] * w;
    dot += g_dot[(size_t)r * n + i] * w;
  }
  float ll = 0.f;
  const long long tg = target[i];
  if (tg != kIgnore) {
    for (int r = 0; r < n_ranks; ++r)
      if (tg >= shard_begin[r] && tg < shard_begin[r + 1]) ll = g_label_logit[(size_t)r * n + i];
  }
  o_max[i] = m; o_sum[i] = sum; o_dot[i] = dot; o_best[i] = best; o_best_val[i] = bv;
  o_label_logit[i] = ll;
  o_lse[i] = m + logf(sum);
}

struct FinishArgs {
  const float* run_max;     // final (merged) state
  const float* run_sum;
  const float* run_dot;
  const int* best;
  const float* label_logit;
  const float* grad_ref;    // lse this rank's dH is relative to (needed when dh is given)
  const int64_t* target;
  const __half* weight;     // this rank's shard [v_shard, k_dim]
  float* token_loss;        // nullable (only the rank that reports writes them)
  float* entropy;
  int* correct;
  float* dh;                // nullable
  int n_rows, k_dim, v_shard, col_offset;
  void* dh_out;             // nullable: the finished gradient goes here (dh_out_dtype), dh stays as it is
  int dh_out_dtype;
};

__global__ void __launch_bounds__(256) lmhead_finish_kernel(const FinishArgs a) {
  const int row = blockIdx.x;
  const float lse = a.run_max[row] + logf(a.run_sum[row]);
  const long long tg = a.target[row];
  const bool labelled = tg != kIgnore;
  if (threadIdx.x == 0 && a.token_loss) {
    a.token_loss[row] = labelled ? lse - a.label_logit[row] : 0.f;
    a.entropy[row] = lse - a.run_dot[row] / a.run_sum[row];
    a.correct[row] = (labelled && (long long)a.best[row] == tg) ? 1 : 0;
  }
  if (!a.dh) return;
  float* dh_row = a.dh + (size_t)row * a.k_dim;
  // dH holds sum_v exp(z_v - grad_ref) W_v over the shard's columns except the label's.
  const float scale = kGradScale * expf(a.grad_ref[row] - lse);
  const long long local = tg - a.col_offset;
  const bool mine = labelled && local >= 0 && local < a.v_shard;
  // the label's term, (p_label - 1) W[label], in fp32 (expm1 keeps it exact when p_label ~ 1)
  const float label_term = mine ? expm1f(a.label_logit[row] - lse) * kGradScale : 0.f;
  const __half* w_row = a.weight + (size_t)(mine ? local : 0) * a.k_dim;
  for (int c = threadIdx.x; c < a.k_dim; c += blockDim.x) {
    float v = labelled ? dh_row[c] * scale : 0.f;
    if (mine) v = fmaf(__half2float(w_row[c]), label_term, v);
    if (a.dh_out) store1(a.dh_out, (int64_t)row * a.k_dim + c, a.dh_out_dtype, v);
    else dh_row[c] = v;
  }
}

// grad = dh * scale, cast to the hidden dtype (the backward of the loss).
__global__ void lmhead_scale_cast_kernel(const float* __restrict__ dh, void* __restrict__ out,
                                         const float* __restrict__ scale_ptr, int64_t n, int odt) {
  const float scale = *scale_ptr;
  const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t n8 = n >> 3;
  if (v < n8) {
    float x[8];
    load8(dh, v << 3, SOUP_F32, x);
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] *= scale;
    store8(out, v << 3, odt, x);
  }
  if (v == 0)
    for (int64_t i = n8 << 3; i < n; ++i) store1(out, i, odt, dh[i] * scale);
}

// Copies a non-zero status of the call into the device's sticky status word (read and cleared by
// soup_device_status), so that a failure outlives the call's workspace.
__global__ void lmhead_publish_status_kernel(const int* call_status, int* sticky) {
  const int code = *call_status;
  if (code != 0) atomicCAS(sticky, 0, code);
}

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// K splits per gradient tile that minimise the makespan of `tiles` output tiles on `pairs` CTA
// pairs (each pair runs its units one after another). 1 keeps the result deterministic.
inline int pick_ksplit(int tiles, int pairs, int n_kb, bool deterministic) {
  if (deterministic || tiles <= 0) return 1;
  int best = 1;
  long best_span = (long)((tiles + pairs - 1) / pairs) * n_kb;
  for (int ks = 2; ks <= 4; ++ks) {
    if (n_kb / ks < 8) break;  // too little work per unit to amortise its epilogue
    const long span = (long)((tiles * ks + pairs - 1) / pairs) * ((n_kb + ks - 1) / ks);
    if (span * 10 < best_span * 9) { best = ks; best_span = span; }  // needs a 10 % gain
  }
  return best;
}

struct Plan {
  int row_block;   // rows per row block
  int ct_first;    // column tiles of the first chunk
  int ct;          // column tiles of every later chunk (>= ct_first)
};

// Rows per block and column tiles per chunk. The first chunk is the one whose logits are computed
// twice (once for its row statistics, once for its probabilities against them), so it is one wave
// of CTA pairs wide and no wider. Every later chunk is written against the running statistics in
// a single pass and can be large: eight waves (SOUP_LMHEAD_WAVES overrides), which cuts the
// launches of a step, and the ramp and drain each one pays, from 55 to 13 at 2048 x 151936 (1.80 ->
// 1.50 ms measured; four waves 1.56, sixteen 1.52). Its probabilities (bf16, 310 MB at 2048 rows)
// then go through HBM instead of staying in L2, which these compute-bound kernels have bandwidth
// to spare for. row_tiles * ct fills whole waves of CTA pairs. An override applies to all chunks.
inline Plan make_plan(int64_t n, int64_t v_shard, int sms, int ct_override) {
  Plan p;
  const int pairs = sms / 2 > 0 ? sms / 2 : 1;
  const int total_ct = (int)((v_shard + kBN - 1) / kBN);
  int waves = 8;
  if (const char* e = getenv("SOUP_LMHEAD_WAVES")) { const int v = atoi(e); if (v >= 1 && v <= 64) waves = v; }
  // A chunk is `wave` column tiles per wave of CTA pairs at eight row tiles (2048 rows).
  int wave = 37;
  for (int c = 40; c >= 8; --c)
    if ((8 * c) % pairs == 0) { wave = c; break; }
  p.ct_first = ct_override > 0 ? ct_override : wave;
  p.ct = ct_override > 0 ? ct_override : waves * wave;
  if (p.ct_first > total_ct) p.ct_first = total_ct;
  if (p.ct_first < 1) p.ct_first = 1;
  if (p.ct > total_ct) p.ct = total_ct;
  if (p.ct < p.ct_first) p.ct = p.ct_first;
  // Rows per block: 2048 for a full-width chunk; more when the shard is narrow (a rank of a
  // vocabulary-parallel group), so that a launch still has a dozen tiles per CTA pair and the
  // probability buffer stays around 600 MB. Whole multiples of 2048, at most 8192.
  int64_t rb = 2048;
  if (ct_override <= 0) {
    rb = 2048 * (int64_t)((2 * waves * wave) / p.ct);
    if (rb < 2048) rb = 2048;
    if (rb > 8192) rb = 8192;
  }
  p.row_block = (int)(n < rb ? (n < 1 ? 1 : n) : rb);
  return p;
}

struct Workspace {
  __nv_bfloat16* p_buf;   // [row_block, ct * 256]
  float4* tile_stats;     // [row_block, ct]
  float* mult;            // [row_block]
  int* status;
  int64_t bytes;
};

inline Workspace carve_workspace(void* base, const Plan& p) {
  Workspace w;
  uint8_t* b = reinterpret_cast<uint8_t*>(base);
  int64_t off = 0;
  const int64_t ld_p = (int64_t)p.ct * kBN;
  w.p_buf = reinterpret_cast<__nv_bfloat16*>(b + off);
  off += round_up((int64_t)p.row_block * ld_p * 2, 1024);
  w.tile_stats = reinterpret_cast<float4*>(b + off);
  off += round_up((int64_t)p.row_block * p.ct * 16, 1024);
  w.mult = reinterpret_cast<float*>(b + off);
  off += round_up((int64_t)p.row_block * 4, 1024);
  w.status = reinterpret_cast<int*>(b + off);
  off += 1024;
  w.bytes = off;
  return w;
}

bool g_attr_set[64] = {false};

// Optional per-kernel-class timing for benchmarks: when a sink is set, soup_lmhead_ce brackets each
// launch with events, synchronises the stream at the end and adds the elapsed milliseconds of the
// logits / row / grad kernels to sink[0..2] and their launch counts to sink[3..5].
float* g_timing_sink = nullptr;

struct LaunchTimer {
  cudaStream_t s;
  bool on;
  std::vector<cudaEvent_t> ev[3];
  explicit LaunchTimer(cudaStream_t stream) : s(stream), on(g_timing_sink != nullptr) {}
  void mark(int k) {
    if (!on) return;
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, s);
    ev[k].push_back(e);
  }
  void finish() {
    if (!on) return;
    cudaStreamSynchronize(s);
    for (int k = 0; k < 3; ++k) {
      for (size_t i = 0; i + 1 < ev[k].size(); i += 2) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev[k][i], ev[k][i + 1]);
        g_timing_sink[k] += ms;
        g_timing_sink[3 + k] += 1.f;
      }
      for (cudaEvent_t e : ev[k]) cudaEventDestroy(e);
    }
  }
};

int ensure_smem_attr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (g_attr_set[dev]) return 0;
  int major = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) return -2;
  if (cudaFuncSetAttribute(lmhead_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kSmemLogits) != cudaSuccess)
    return -1;
  if (cudaFuncSetAttribute(lmhead_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kSmemGrad) != cudaSuccess)
    return -1;
  g_attr_set[dev] = true;
  return 0;
}

}  // namespace

namespace umma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

int encode_map_2d_16bit(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t pitch_elems, uint32_t box_rows, uint32_t box_cols, bool bf16) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_elems * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

int encode_map_2d_bytes(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

}  // namespace umma
}  // namespace soup

extern "C" int64_t soup_lmhead_workspace_bytes(int64_t n, int64_t h, int64_t v_shard,
                                               int64_t chunk_tiles) {
  using namespace soup;
  (void)h;
  const Plan p = make_plan(n, v_shard, sm_count(), (int)chunk_tiles);
  return carve_workspace(nullptr, p).bytes;
}

extern "C" int soup_lmhead_ce(const void* hidden, const void* weight, const void* weight_bf16,
                              const int64_t* target, float* run_max, float* run_sum, float* run_dot, int* best,
                              float* best_val, float* label_logit, float* grad_ref, float* dh,
                              void* workspace, int64_t workspace_bytes, int64_t n, int64_t h,
                              int64_t v_shard, int64_t col_offset, int64_t chunk_tiles,
                              int want_grad, void* stream) {
  using namespace soup;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n < 0 || h <= 0 || v_shard <= 0) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: bad shape");
  if (n == 0) return SOUP_OK;
  if (!hidden || !weight || !target || !run_max || !run_sum || !run_dot || !best || !best_val ||
      !label_logit || !grad_ref || !workspace || (want_grad && (!dh || !weight_bf16)))
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: null pointer");
  if (h % 8 != 0) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: hidden size must be a multiple of 8 (TMA pitch)");
  if (!aligned16(hidden) || !aligned16(weight) || !aligned16(workspace) || (dh && !aligned16(dh)) ||
      (weight_bf16 && !aligned16(weight_bf16)))
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: pointers must be 16-byte aligned");
  if (n > INT32_MAX / 2 || v_shard > INT32_MAX / 2 || col_offset + v_shard > INT32_MAX)
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: shape exceeds 32-bit tile coordinates");
  const int attr = ensure_smem_attr();
  if (attr == -2) SOUP_FAIL(SOUP_ERR_DEVICE, "lmhead_ce: needs a compute capability 10.x device");
  if (attr != 0) SOUP_FAIL(SOUP_ERR_DEVICE, "lmhead_ce: cannot raise the shared-memory limit");
  const int sms = sm_count();
  const int max_pairs = sms / 2;
  if (max_pairs < 1) SOUP_FAIL(SOUP_ERR_DEVICE, "lmhead_ce: needs at least two SMs");
  const Plan plan = make_plan(n, v_shard, sms, (int)chunk_tiles);
  const Workspace ws = carve_workspace(workspace, plan);
  if (workspace_bytes < ws.bytes)
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: workspace too small (%lld < %lld)",
              (long long)workspace_bytes, (long long)ws.bytes);
  const int ld_p = plan.ct * kBN;
  const int total_ct = (int)((v_shard + kBN - 1) / kBN);
  const char* det_env = getenv("SOUP_LMHEAD_DETERMINISTIC");
  const bool deterministic = det_env && atoi(det_env) != 0;

  CUtensorMap map_h, map_w_k, map_w_mn, map_p_ld, map_p_st;
  if (umma::encode_map_2d_16bit(&map_h, hidden, (uint64_t)n, (uint64_t)h, (uint64_t)h, kBM, kBK, false) ||
      umma::encode_map_2d_16bit(&map_w_k, weight, (uint64_t)v_shard, (uint64_t)h, (uint64_t)h, kBN / 2, kBK, false) ||
      (want_grad &&
       umma::encode_map_2d_16bit(&map_w_mn, weight_bf16, (uint64_t)v_shard, (uint64_t)h, (uint64_t)h, kBK, 64, true)) ||
      umma::encode_map_2d_16bit(&map_p_ld, ws.p_buf, (uint64_t)plan.row_block, (uint64_t)ld_p,
                                (uint64_t)ld_p, kBM, kBK, true) ||
      umma::encode_map_2d_16bit(&map_p_st, ws.p_buf, (uint64_t)plan.row_block, (uint64_t)ld_p,
                                (uint64_t)ld_p, 32, 64, true))
    SOUP_FAIL(SOUP_ERR_DEVICE, "lmhead_ce: cuTensorMapEncodeTiled failed");

  cudaMemsetAsync(ws.status, 0, 4, s);
  if (want_grad) cudaMemsetAsync(dh, 0, (size_t)n * h * sizeof(float), s);
  lmhead_init_state_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(
      run_max, run_sum, run_dot, best, best_val, label_logit, grad_ref, (int)n);
  SOUP_CHECK_LAUNCH("lmhead_init_state");

  LaunchTimer timer(s);
  for (int64_t r0 = 0; r0 < n; r0 += plan.row_block) {
    const int rows = (int)((n - r0) < plan.row_block ? (n - r0) : plan.row_block);
    const int rt = (rows + 2 * kBM - 1) / (2 * kBM);
    for (int t0 = 0; t0 < total_ct;) {
      const bool first = t0 == 0;
      const int want_ct = first ? plan.ct_first : plan.ct;
      const int ct = (total_ct - t0) < want_ct ? (total_ct - t0) : want_ct;
      LogitsArgs la;
      la.target = target + r0;
      la.ref = run_max + r0;
      la.tile_stats = ws.tile_stats;
      la.label_logit = label_logit + r0;
      la.n_rows = rows;
      la.row0 = (int)r0;
      la.k_dim = (int)h;
      la.col0 = t0 * kBN;
      la.v_shard = (int)v_shard;
      la.col_offset = (int)col_offset;
      la.ct = ct;
      la.ct_stride = plan.ct;
      la.store_p = want_grad;
      la.status = ws.status;
      const int tiles1 = rt * ct;
      const unsigned grid1 = 2u * (unsigned)(tiles1 < max_pairs ? tiles1 : max_pairs);

      la.mode = first ? kModeTileMax : kModeCombined;
      timer.mark(0);
      lmhead_logits_kernel<<<grid1, kThreadsGemm, kSmemLogits, s>>>(map_h, map_w_k, map_p_st, la);
      timer.mark(0);
      SOUP_CHECK_LAUNCH("lmhead_logits");

      RowArgs ra;
      ra.tile_stats = ws.tile_stats;
      ra.run_max = run_max + r0;
      ra.run_sum = run_sum + r0;
      ra.run_dot = run_dot + r0;
      ra.best = best + r0;
      ra.best_val = best_val + r0;
      ra.base = grad_ref + r0;
      ra.mult = ws.mult;
      ra.dh = want_grad ? dh + r0 * h : nullptr;
      ra.p = want_grad ? ws.p_buf : nullptr;
      ra.ld_p = ld_p;
      ra.n_rows = rows;
      ra.k_dim = (int)h;
      ra.ct = ct;
      ra.ct_stride = plan.ct;
      ra.mode = la.mode;
      ra.want_grad = want_grad;
      ra.status = ws.status;
      timer.mark(1);
      lmhead_row_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(ra);
      timer.mark(1);
      SOUP_CHECK_LAUNCH("lmhead_row");

      if (want_grad) {
        if (first) {  // the first chunk's P from "against its tile maximum" to "against the lse"
          timer.mark(1);
          lmhead_rescale_first_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(
              ws.p_buf, ld_p, ws.tile_stats, plan.ct, run_max + r0, rows, ct);
          timer.mark(1);
          SOUP_CHECK_LAUNCH("lmhead_rescale_first");
        }
        GradArgs ga;
        ga.dh = dh + r0 * h;
        ga.mult = ws.mult;
        ga.n_rows = rows;
        ga.k_dim = (int)h;
        ga.col0 = t0 * kBN;
        ga.n_kb = ct * (kBN / kBK);
        ga.status = ws.status;
        const int tiles2 = rt * (int)((h + kBN - 1) / kBN);
        ga.ksplit = pick_ksplit(tiles2, max_pairs, ga.n_kb, deterministic);
        const int units = tiles2 * ga.ksplit;
        const unsigned grid2 = 2u * (unsigned)(units < max_pairs ? units : max_pairs);
        timer.mark(2);
        lmhead_grad_kernel<<<grid2, kThreadsGemm, kSmemGrad, s>>>(map_p_ld, map_w_mn, ga);
        timer.mark(2);
        SOUP_CHECK_LAUNCH("lmhead_grad");
      }
      t0 += ct;
    }
  }
  if (int* sticky = rowpipe::status_word()) {
    lmhead_publish_status_kernel<<<1, 1, 0, s>>>(ws.status, sticky);
    SOUP_CHECK_LAUNCH("lmhead_publish_status");
  }
  timer.finish();
  return SOUP_OK;
}

extern "C" int soup_lmhead_set_timing(float* host_sink6) {
  soup::g_timing_sink = host_sink6;
  return SOUP_OK;
}

extern "C" int soup_lmhead_plan(int64_t n, int64_t v_shard, int64_t chunk_tiles, int64_t* row_block,
                                int64_t* first_chunk_tiles, int64_t* tiles_per_chunk) {
  using namespace soup;
  const Plan p = make_plan(n, v_shard, sm_count(), (int)chunk_tiles);
  if (row_block) *row_block = p.row_block;
  if (first_chunk_tiles) *first_chunk_tiles = p.ct_first;
  if (tiles_per_chunk) *tiles_per_chunk = p.ct;
  return SOUP_OK;
}

extern "C" int soup_lmhead_status(const void* workspace, int64_t n, int64_t v_shard,
                                  int64_t chunk_tiles, int* host_status, void* stream) {
  using namespace soup;
  const Plan plan = make_plan(n, v_shard, sm_count(), (int)chunk_tiles);
  const Workspace ws = carve_workspace(const_cast<void*>(workspace), plan);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(host_status, ws.status, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    SOUP_FAIL(SOUP_ERR_LAUNCH, "lmhead_status: %s", cudaGetErrorString(cudaGetLastError()));
  return SOUP_OK;
}

extern "C" int soup_lmhead_merge(const float* g_max, const float* g_sum, const float* g_dot,
                                 const int* g_best, const float* g_best_val,
                                 const float* g_label_logit, const int64_t* target,
                                 const int64_t* shard_begin, float* o_max, float* o_sum,
                                 float* o_dot, int* o_best, float* o_best_val,
                                 float* o_label_logit, float* o_lse, int64_t n, int n_ranks,
                                 void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || n_ranks < 1) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_merge: bad shape");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  lmhead_merge_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(
      g_max, g_sum, g_dot, g_best, g_best_val, g_label_logit, target, shard_begin, o_max, o_sum,
      o_dot, o_best, o_best_val, o_label_logit, o_lse, (int)n, n_ranks);
  SOUP_CHECK_LAUNCH("lmhead_merge");
  return SOUP_OK;
}

extern "C" int soup_lmhead_finish_to(const float* run_max, const float* run_sum, const float* run_dot,
                                     const int* best, const float* label_logit, const float* grad_ref,
                                     const int64_t* target, const void* weight, float* token_loss,
                                     float* entropy, int* correct, float* dh, void* dh_out,
                                     int dh_out_dtype, int64_t n, int64_t h, int64_t v_shard,
                                     int64_t col_offset, void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || h <= 0) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: bad shape");
  if (!run_max || !run_sum || !run_dot || !best || !label_logit || !target)
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: null pointer");
  if (dh && (!weight || !grad_ref))
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: dH needs the weight shard and grad_ref");
  if (token_loss && (!entropy || !correct)) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: null output");
  if (dh_out && (!dh || !is_float_dtype(dh_out_dtype)))
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: a separate output needs dh and a floating dtype");
  FinishArgs a;
  a.run_max = run_max; a.run_sum = run_sum; a.run_dot = run_dot; a.best = best;
  a.label_logit = label_logit; a.grad_ref = grad_ref;
  a.target = target; a.weight = reinterpret_cast<const __half*>(weight);
  a.token_loss = token_loss; a.entropy = entropy; a.correct = correct; a.dh = dh;
  a.dh_out = dh_out; a.dh_out_dtype = dh_out_dtype;
  a.n_rows = (int)n; a.k_dim = (int)h; a.v_shard = (int)v_shard; a.col_offset = (int)col_offset;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  lmhead_finish_kernel<<<(unsigned)n, 256, 0, s>>>(a);
  SOUP_CHECK_LAUNCH("lmhead_finish");
  return SOUP_OK;
}

extern "C" int soup_lmhead_finish(const float* run_max, const float* run_sum, const float* run_dot,
                                  const int* best, const float* label_logit, const float* grad_ref,
                                  const int64_t* target, const void* weight, float* token_loss,
                                  float* entropy, int* correct, float* dh, int64_t n, int64_t h,
                                  int64_t v_shard, int64_t col_offset, void* stream) {
  return soup_lmhead_finish_to(run_max, run_sum, run_dot, best, label_logit, grad_ref, target, weight,
                               token_loss, entropy, correct, dh, nullptr, SOUP_F32, n, h, v_shard,
                               col_offset, stream);
}

extern "C" int soup_lmhead_grad_scale(const float* dh, void* out, const float* scale, int64_t n,
                                      int out_dtype, void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (!dh || !out || !scale || n < 0) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_grad_scale: bad argument");
  if (!is_float_dtype(out_dtype)) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_grad_scale: unsupported dtype");
  if (!aligned16(dh) || !aligned16(out)) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_grad_scale: unaligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n8 = (n >> 3) + 1;
  lmhead_scale_cast_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, s>>>(dh, out, scale, n, out_dtype);
  SOUP_CHECK_LAUNCH("lmhead_grad_scale");
  return SOUP_OK;
}
