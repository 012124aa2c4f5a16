// Fused LM head + cross-entropy, forward and hidden-state gradient, without the logits in HBM.
//
// The vocabulary is walked in chunks of `ct` column tiles (256 columns each). Per chunk, three
// kernels run back to back on the caller's stream; what they exchange stays in the 126 MB L2:
//
//   logits kernel  tcgen05 GEMM  S = H[rows,K] * W[cols,K]^T, 128x256 tiles, fp32 in TMEM, TMA-fed
//                  4-stage pipeline, double-buffered accumulator. The epilogue never writes S: per
//                  row and tile it keeps (max, sum exp, sum exp*z, first argmax, label logit) and
//                  writes E = 2^14 * exp(z - tile_max) as fp16 (always a normal number at the top
//                  of the tile, so nothing a 152K vocabulary needs flushes to zero).
//   row kernel     merges the tile statistics into the running per-row state (max, sum, dot,
//                  argmax, label logit), forms the running log-sum-exp, and rescales E in place to
//                  P = 1024 * softmax against that running lse (the label's entry gets p - 1,
//                  computed in fp32). Emits factor = exp(lse_before - lse_after).
//   grad kernel    tcgen05 GEMM  dH = factor * dH + P[rows,cols] * W[cols,K], with W as the
//                  MN-major operand straight from its row-major storage, 128x192 tiles.
//
// A last kernel turns the state into loss / entropy / correct and restores the part of the
// label's -1 that later rescaling removed. The algorithm (running lse, factor, label fix-up,
// GRAD_SCALE 1024) is the one of _FusedHeadLoss.forward, solution/lm_head_loss.py:192-245 of the
// reference; only the tiling, the on-chip statistics and the exp-relative-to-tile-max storage
// are new.
//
// Vocabulary-parallel use: a rank passes its shard of W, the global index of its first column,
// and gets state and dH relative to its own lse; soup_lmhead_merge combines the ranks' states and
// soup_lmhead_finish applies exp(lse_rank - lse_global) before the caller sums dH across ranks.
#include <math.h>
#include <stdlib.h>

#include <vector>

#include "common.cuh"
#include "umma.cuh"

namespace soup {
namespace {

using namespace umma;

constexpr int kBM = 128;         // rows per tile (TMEM lanes)
constexpr int kBN1 = 256;        // vocabulary columns per logits tile
constexpr int kBN2 = 192;        // hidden columns per gradient tile
constexpr int kBK = 64;          // 64 fp16 = one 128-byte swizzle row
constexpr int kStages1 = 4;
constexpr int kStages2 = 5;
constexpr int kABytes = kBM * kBK * 2;      // 16 KB
constexpr int kB1Bytes = kBN1 * kBK * 2;    // 32 KB
constexpr int kB2Bytes = kBN2 * kBK * 2;    // 24 KB, three 64-column boxes of 8 KB
constexpr int kThreadsGemm = 192;           // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kEScale = 16384.0f;         // 2^14, E = kEScale * exp(z - tile_max)
constexpr float kGradScale = 1024.0f;       // as GRAD_SCALE of the reference
constexpr int kIgnore = -100;

constexpr int kStageE = 4 * 2 * 4096;        // per epilogue warp two 32-row x 64-column fp16 boxes
constexpr int kSmem1 = kStages1 * (kABytes + kB1Bytes) + kStageE + 1024 + 256;
constexpr int kSmem2 = kStages2 * (kABytes + kB2Bytes) + 1024 + 256;

struct PipeState {
  int stage = 0;
  uint32_t phase = 0;
  template <int STAGES>
  __device__ __forceinline__ void advance() {
    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
  }
};

struct GemmSmem {
  uint8_t* tiles;        // 1024-byte aligned
  uint8_t* extra;        // kernel-specific staging area behind the stages
  uint64_t* full;        // [STAGES]
  uint64_t* empty;       // [STAGES]
  uint64_t* acc_full;    // [2]
  uint64_t* acc_empty;   // [2]
  uint32_t* tmem_base;
  int* abort_flag;
};

template <int STAGES, int STAGE_BYTES, int EXTRA_BYTES = 0>
__device__ __forceinline__ GemmSmem carve_smem(uint8_t* raw) {
  GemmSmem s;
  const uintptr_t base = (reinterpret_cast<uintptr_t>(raw) + 1023u) & ~static_cast<uintptr_t>(1023u);
  s.tiles = reinterpret_cast<uint8_t*>(base);
  s.extra = s.tiles + STAGES * STAGE_BYTES;  // 1024-byte aligned (stage sizes are multiples of 1024)
  uint64_t* bars = reinterpret_cast<uint64_t*>(s.tiles + STAGES * STAGE_BYTES + EXTRA_BYTES);
  s.full = bars;
  s.empty = bars + STAGES;
  s.acc_full = bars + 2 * STAGES;
  s.acc_empty = bars + 2 * STAGES + 2;
  s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  s.abort_flag = reinterpret_cast<int*>(s.tmem_base + 1);
  return s;
}

template <int STAGES>
__device__ __forceinline__ void init_pipeline(const GemmSmem& s, int warp, int lane) {
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s.acc_full[i], 1); mbar_init(&s.acc_empty[i], 4); }
    *s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {  // one warp owns the tensor-memory allocation (all 512 columns)
    tmem_alloc(s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
}

__device__ __forceinline__ void finish_pipeline(const GemmSmem& s, int warp, uint32_t tmem) {
  tc_fence_before_sync();
  __syncthreads();
  if (*s.abort_flag) {
    // A wait was abandoned: give copies that may still be in flight time to land before the
    // shared memory is released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// Statistics epilogue of one 128 x 256 logits tile for one thread (= one row). Two sweeps over the
// accumulator in TMEM, 32 columns at a time, with the load of the next 32 columns issued before the
// current ones are consumed: sweep 1 finds the row maximum of the tile and its first index, sweep 2
// forms E = 2^14 * exp(z - max) (the scale folded into the exponent), its sum, the sum of E*z, and
// writes E as fp16. FULL tiles (all 256 columns inside the vocabulary) skip every validity select.
constexpr int kEW = 16;  // accumulator columns per tcgen05.ld in the statistics epilogue

template <bool FULL>
__device__ __forceinline__ void sweep_max(const uint32_t (&r)[kEW], int col0, int n_valid, float& m,
                                          int& arg) {
#pragma unroll
  for (int j = 0; j < kEW; ++j) {
    const float z = __uint_as_float(r[j]);
    const int col = col0 + j;
    if ((FULL || col < n_valid) && z > m) { m = z; arg = col; }
  }
}

// `stage_row` points at this thread's 128-byte row of a 32-row x 64-column staging box laid out with
// the 128-byte swizzle (16-byte piece k of row r lives at piece k ^ (r & 7)); `piece0` is the first
// of the two 16-byte pieces these 16 columns fill.
template <bool FULL>
__device__ __forceinline__ void sweep_exp(const uint32_t (&r)[kEW], int col0, int n_valid,
                                          bool store_e, uint8_t* stage_row, int row_swz, int piece0,
                                          float bias, float (&acc)[4]) {
  uint32_t packed[kEW / 2];
#pragma unroll
  for (int j = 0; j < kEW; j += 2) {
    const float z0 = __uint_as_float(r[j]), z1 = __uint_as_float(r[j + 1]);
    const int col = col0 + j;
    float e0 = exp2f(fmaf(z0, kLog2e, bias));
    float e1 = exp2f(fmaf(z1, kLog2e, bias));
    if (!FULL) {
      if (col >= n_valid) e0 = 0.f;
      if (col + 1 >= n_valid) e1 = 0.f;
    }
    acc[0] += e0;
    acc[1] += e1;
    acc[2] = fmaf(e0, (FULL || col < n_valid) ? z0 : 0.f, acc[2]);
    acc[3] = fmaf(e1, (FULL || col + 1 < n_valid) ? z1 : 0.f, acc[3]);
    __half2 h = __floats2half2_rn(e0, e1);
    packed[j >> 1] = *reinterpret_cast<uint32_t*>(&h);
  }
  if (store_e) {
#pragma unroll
    for (int v = 0; v < kEW / 8; ++v) {
      const int piece = (piece0 + v) ^ row_swz;
      *reinterpret_cast<uint4*>(stage_row + piece * 16) =
          make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
    }
  }
}

// Statistics epilogue of one 128 x 256 logits tile for one thread (= one row). Two sweeps over the
// accumulator in TMEM, 16 columns per tcgen05.ld, the next load in flight while the current columns
// are consumed; the loop bodies are kept small enough to stay in the instruction cache. Sweep 1:
// row maximum of the tile and its first index. Sweep 2: E = 2^14 * exp(z - max) (scale folded into
// the exponent), its sum and the sum of E*z; E leaves as fp16 through a swizzled staging box and a
// TMA store per 64 columns. FULL tiles (all 256 columns inside the vocabulary) skip the validity
// selects. The label's logit, needed by very few rows of a tile, is fetched in a third, rare sweep.
template <bool FULL>
__device__ __noinline__ void tile_statistics(uint32_t taddr, int n_valid, int label_local,
                                             bool store_e, const CUtensorMap* map_e,
                                             uint8_t* stage_warp, int e_col0, int e_row0,
                                             float& m_out, float& sum_out, float& dot_out,
                                             float& lab_out, int& arg_out, int debug) {
  constexpr int kLoads = kBN1 / kEW;      // 16
  constexpr int kPerBox = 64 / kEW;       // loads per 64-column staging box
  const int lane = threadIdx.x & 31;
  uint32_t ra[kEW], rb[kEW];
  float m = -INFINITY;
  int arg = 0;
  if (debug & 2) m = 0.f;
  if (!(debug & 2)) tmem_ld_32x16(taddr, ra);
#pragma unroll 1
  for (int i = 0; i < ((debug & 2) ? 0 : kLoads); i += 2) {
    tmem_ld_wait_on(ra);
    tmem_ld_32x16(taddr + (i + 1) * kEW, rb);
    sweep_max<FULL>(ra, i * kEW, n_valid, m, arg);
    tmem_ld_wait_on(rb);
    if (i + 2 < kLoads) tmem_ld_32x16(taddr + (i + 2) * kEW, ra);
    sweep_max<FULL>(rb, (i + 1) * kEW, n_valid, m, arg);
  }
  // exp2(z*log2e - m*log2e + 14) = 2^14 * exp(z - m)
  const float bias = 14.0f - m * kLog2e;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  uint8_t* stage_row = stage_warp + lane * 128;
  if (!(debug & 4)) tmem_ld_32x16(taddr, ra);
#pragma unroll 1
  for (int i = 0; i < ((debug & 4) ? 0 : kLoads); i += 2) {
    // 64-column boxes alternate between the warp's two staging areas; the area used two boxes ago
    // must have been read by its TMA store before it is overwritten.
    const int box_id = i / kPerBox;
    uint8_t* box = stage_warp + (box_id & 1) * 4096;
    if (store_e && (i % kPerBox) == 0) {
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
    }
    tmem_ld_wait_on(ra);
    tmem_ld_32x16(taddr + (i + 1) * kEW, rb);
    sweep_exp<FULL>(ra, i * kEW, n_valid, store_e, stage_row + (box_id & 1) * 4096, lane & 7,
                    (i % kPerBox) * (kEW / 8), bias, acc);
    tmem_ld_wait_on(rb);
    if (i + 2 < kLoads) tmem_ld_32x16(taddr + (i + 2) * kEW, ra);
    sweep_exp<FULL>(rb, (i + 1) * kEW, n_valid, store_e, stage_row + (box_id & 1) * 4096, lane & 7,
                    ((i + 1) % kPerBox) * (kEW / 8), bias, acc);
    if (store_e && ((i + 2) % kPerBox) == 0) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map_e, box, e_col0 + box_id * 64, e_row0);
        tma_store_commit();
      }
    }
  }
  float lab = 0.f;
  if (__any_sync(0xffffffffu, label_local >= 0)) {  // rare: some row's label falls in this tile
#pragma unroll 1
    for (int i = 0; i < kLoads; ++i) {
      tmem_ld_32x16(taddr + i * kEW, ra);
      tmem_ld_wait_on(ra);
#pragma unroll
      for (int j = 0; j < kEW; ++j)
        if (i * kEW + j == label_local) lab = __uint_as_float(ra[j]);
    }
  }
  m_out = m;
  sum_out = (acc[0] + acc[1]) * (1.0f / kEScale);
  dot_out = (acc[2] + acc[3]) * (1.0f / kEScale);
  lab_out = lab;
  arg_out = arg;
}

// ------------------------------------------------------------------------------------------
// Logits kernel: tile statistics + E for one chunk of column tiles of one row block.
// ------------------------------------------------------------------------------------------
struct LogitsArgs {
  const int64_t* target;   // [n_rows] of this row block
  __half* e_buf;           // [n_rows, ld_e]
  float4* tile_stats;      // [n_rows, ct_stride]  (max, sum, dot, argmax bits)
  float* label_logit;      // [n_rows]
  int n_rows;              // rows in this row block
  int row0;                // first row of the block inside the hidden matrix (TMA coordinate)
  int k_dim;               // hidden size
  int col0;                // first column of the chunk inside the weight shard
  int v_shard;             // columns of the weight shard
  int col_offset;          // global vocabulary index of shard column 0
  int ct;                  // column tiles in this chunk
  int ct_stride;           // row pitch of tile_stats
  int ld_e;                // row pitch of e_buf in elements
  int write_e;
  int debug;               // bit 0: skip the statistics sweeps (timing experiments only)
  int* status;
};

__global__ void __launch_bounds__(kThreadsGemm, 1)
lmhead_logits_kernel(const __grid_constant__ CUtensorMap map_h,
                     const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_e, const LogitsArgs a) {
  extern __shared__ uint8_t smem_raw[];
  if (*reinterpret_cast<volatile int*>(a.status) != 0) return;  // an earlier kernel gave up
  constexpr int kStageBytes = kABytes + kB1Bytes;
  const GemmSmem s = carve_smem<kStages1, kStageBytes, kStageE>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&map_h);
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_e);
  }
  init_pipeline<kStages1>(s, warp, lane);
  const uint32_t tmem = *s.tmem_base;

  const int rt = (a.n_rows + kBM - 1) / kBM;
  const int n_tiles = rt * a.ct;
  const int n_kb = (a.k_dim + kBK - 1) / kBK;

  if (warp == 0) {
    if (lane == 0) {
      PipeState p;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int tr = tile % rt, tc = tile / rt;
        for (int kb = 0; kb < n_kb; ++kb) {
          ok = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 11);
          if (!ok) break;
          uint8_t* st = s.tiles + p.stage * kStageBytes;
          mbar_expect_tx(&s.full[p.stage], kStageBytes);
          tma_load_2d(st, &map_h, kb * kBK, a.row0 + tr * kBM, &s.full[p.stage]);
          tma_load_2d(st + kABytes, &map_w, kb * kBK, a.col0 + tc * kBN1, &s.full[p.stage]);
          p.advance<kStages1>();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBM, kBN1, false, false);
      PipeState p;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait(&s.acc_empty[ab], acc_phase ^ 1u, s.abort_flag, a.status, 12);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + ab * kBN1;
        for (int kb = 0; kb < n_kb; ++kb) {
          ok = mbar_wait(&s.full[p.stage], p.phase, s.abort_flag, a.status, 13);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.tiles + p.stage * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr, 16, 1024);
          const uint64_t db = make_smem_desc(a_addr + kABytes, 16, 1024);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            mma_f16_ss(d_tmem, da + k4 * 2, db + k4 * 2, idesc, (kb | k4) != 0);
          tc_commit(&s.empty[p.stage]);
          p.advance<kStages1>();
        }
        if (ok) tc_commit(&s.acc_full[ab]);
      }
    }
  } else {
    // Epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32).
    const int q = warp & 3;
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
      const int tr = tile % rt, tc = tile / rt;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&s.acc_full[ab], acc_phase, s.abort_flag, a.status, 14));
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tr * kBM + q * 32 + lane;       // row inside the row block
      const bool row_ok = row < a.n_rows;
      const int tile_col0 = a.col0 + tc * kBN1;       // column inside the shard
      const int n_valid = min(kBN1, a.v_shard - tile_col0);  // >= 1 by construction
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + ab * kBN1;
      int label_local = -1;
      if (row_ok) {
        const long long tg = a.target[row];
        const long long loc = tg - a.col_offset - tile_col0;
        if (tg != kIgnore && loc >= 0 && loc < n_valid) label_local = (int)loc;
      }
      float m, sum, dot, lab;
      int arg;
      // E leaves through a per-warp staging box and a TMA store (rows past the buffer are clipped).
      uint8_t* stage_warp = s.extra + (warp - 2) * 8192;
      const int e_row0 = tr * kBM + q * 32;
      if (a.debug & 1) {
        m = 0.f; sum = 1.f; dot = 0.f; lab = 0.f; arg = 0;
      } else if (n_valid == kBN1)
        tile_statistics<true>(taddr, n_valid, label_local, a.write_e != 0, &map_e, stage_warp,
                              tc * kBN1, e_row0, m, sum, dot, lab, arg, a.debug);
      else
        tile_statistics<false>(taddr, n_valid, label_local, a.write_e != 0, &map_e, stage_warp,
                               tc * kBN1, e_row0, m, sum, dot, lab, arg, a.debug);
      // the accumulator buffer is free again
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[ab]);
      if (row_ok) {
        a.tile_stats[(size_t)row * a.ct_stride + tc] =
            make_float4(m, sum, dot, __int_as_float(tile_col0 + arg + a.col_offset));
        if (label_local >= 0) a.label_logit[row] = lab;
      }
    }
    if (lane == 0) tma_store_wait_read<0>();  // staging boxes fully read before shared memory goes away
  }
  finish_pipeline(s, warp, tmem);
}

// ------------------------------------------------------------------------------------------
// CTA-pair variants (cta_group::2): the pair owns a 256-row tile, each CTA 128 rows of it, and the
// B operand is split between the two CTAs, so every shared-memory stage holds half the B bytes of
// the single-CTA kernel and the operand traffic through the crossbar per flop drops by a third.
// ------------------------------------------------------------------------------------------
constexpr int kBHalf1Bytes = (kBN1 / 2) * kBK * 2;   // 16 KB: this CTA's 128 vocabulary columns
constexpr int kStagesP1 = 6;
constexpr int kSmemP1 = kStagesP1 * (kABytes + kBHalf1Bytes) + kStageE + 1024 + 256;

struct PairInit {
  uint32_t tmem;
  uint32_t rank;
  bool run;
};

// Barrier set-up, tensor-memory allocation and the agreement of both CTAs on whether to run at all
// (an earlier kernel of the call may have given up). Every thread of both CTAs calls this.
template <int STAGES>
__device__ __forceinline__ PairInit init_pair(const GemmSmem& s, int warp, int lane, const int* status) {
  PairInit r;
  r.rank = cluster_ctarank();
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
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

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsGemm, 1)
lmhead_logits_pair_kernel(const __grid_constant__ CUtensorMap map_h,
                          const __grid_constant__ CUtensorMap map_w,
                          const __grid_constant__ CUtensorMap map_e, const LogitsArgs a) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int kStageBytes = kABytes + kBHalf1Bytes;
  const GemmSmem s = carve_smem<kStagesP1, kStageBytes, kStageE>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&map_h);
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_e);
  }
  const PairInit pi = init_pair<kStagesP1>(s, warp, lane, a.status);
  if (!pi.run) return;
  const uint32_t tmem = pi.tmem, rank = pi.rank;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

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
        const int col0 = a.col0 + tc * kBN1 + (int)rank * (kBN1 / 2);
        for (int kb = 0; kb < n_kb; ++kb) {
          ok = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 31);
          if (!ok) break;
          uint8_t* st = s.tiles + p.stage * kStageBytes;
          // both CTAs' bytes are counted on the leader's barrier
          const uint32_t full_leader = mapa_u32(smem_u32(&s.full[p.stage]), 0);
          if (rank == 0) mbar_expect_tx(&s.full[p.stage], 2 * kStageBytes);
          tma_load_2d_pair(st, &map_h, kb * kBK, row0, full_leader);
          tma_load_2d_pair(st + kABytes, &map_w, kb * kBK, col0, full_leader);
          p.advance<kStagesP1>();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * kBM, kBN1, false, false);
      PipeState p;
      bool ok = true;
      int it = 0;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait(&s.acc_empty[ab], acc_phase ^ 1u, s.abort_flag, a.status, 32);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + ab * kBN1;
        for (int kb = 0; kb < n_kb; ++kb) {
          ok = mbar_wait(&s.full[p.stage], p.phase, s.abort_flag, a.status, 33);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.tiles + p.stage * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr, 16, 1024);
          const uint64_t db = make_smem_desc(a_addr + kABytes, 16, 1024);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            mma_f16_ss_pair(d_tmem, da + k4 * 2, db + k4 * 2, idesc, (kb | k4) != 0);
          tc_commit_pair(&s.empty[p.stage], 3);   // frees the stage in both CTAs
          p.advance<kStagesP1>();
        }
        if (ok) tc_commit_pair(&s.acc_full[ab], 3);
      }
    }
  } else {
    const int q = warp & 3;
    bool ok = true;
    int it = 0;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
      const int tr = tile % rt, tc = tile / rt;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&s.acc_full[ab], acc_phase, s.abort_flag, a.status, 34));
      if (!ok) break;
      tc_fence_after_sync();
      const int e_row0 = tr * 2 * kBM + (int)rank * kBM + q * 32;
      const int row = e_row0 + lane;
      const bool row_ok = row < a.n_rows;
      const int tile_col0 = a.col0 + tc * kBN1;
      const int n_valid = min(kBN1, a.v_shard - tile_col0);
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + ab * kBN1;
      int label_local = -1;
      if (row_ok) {
        const long long tg = a.target[row];
        const long long loc = tg - a.col_offset - tile_col0;
        if (tg != kIgnore && loc >= 0 && loc < n_valid) label_local = (int)loc;
      }
      float m, sum, dot, lab;
      int arg;
      uint8_t* stage_warp = s.extra + (warp - 2) * 8192;
      if (a.debug & 1) {
        m = 0.f; sum = 1.f; dot = 0.f; lab = 0.f; arg = 0;
      } else if (n_valid == kBN1)
        tile_statistics<true>(taddr, n_valid, label_local, a.write_e != 0, &map_e, stage_warp,
                              tc * kBN1, e_row0, m, sum, dot, lab, arg, a.debug);
      else
        tile_statistics<false>(taddr, n_valid, label_local, a.write_e != 0, &map_e, stage_warp,
                               tc * kBN1, e_row0, m, sum, dot, lab, arg, a.debug);
      // the accumulator buffer of this CTA is free again: tell the leader's MMA thread
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&s.acc_empty[ab]);
        else mbar_arrive_cluster(mapa_u32(smem_u32(&s.acc_empty[ab]), 0));
      }
      if (row_ok) {
        a.tile_stats[(size_t)row * a.ct_stride + tc] =
            make_float4(m, sum, dot, __int_as_float(tile_col0 + arg + a.col_offset));
        if (label_local >= 0) a.label_logit[row] = lab;
      }
    }
    if (lane == 0) tma_store_wait_read<0>();
  }
  finish_pair(s, warp, tmem);
}

// ------------------------------------------------------------------------------------------
// Row kernel: one warp per row. Merges the chunk's tile statistics into the running state and
// rescales E to P in place.
// ------------------------------------------------------------------------------------------
struct RowArgs {
  const int64_t* target;
  __half* e_buf;
  const float4* tile_stats;
  float* run_max;
  float* run_sum;
  float* run_dot;
  int* best;
  const float* label_logit;
  float* label_lse;
  float* factor;
  int n_rows;
  int col0;         // first shard column of the chunk
  int v_shard;
  int col_offset;
  int ct;
  int ct_stride;
  int ld_e;
  int write_p;
  float* dh;        // nullable: [n_rows, k_dim] gradient to rescale by this chunk's factor
  int k_dim;
  int first;        // first chunk: nothing accumulated yet
};

constexpr int kRowWarps = 4;          // warps per row in the row kernel
constexpr int kRowTilesPerWarp = 16;  // register-resident tiles per warp per pass

__global__ void __launch_bounds__(kRowWarps * 32) lmhead_row_kernel(const RowArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x;
  // Every warp merges the (at most a few dozen) tile statistics itself: cheaper than a block-wide
  // exchange, and all warps then hold the same running state and log-sum-exp.
  const float prev_max = a.run_max[row], prev_sum = a.run_sum[row];
  float run_max = prev_max, run_sum = prev_sum, run_dot = a.run_dot[row];
  int best = a.best[row];
  // Tiles in ascending column order, so a later tile wins the argmax only if strictly larger.
  for (int t0 = 0; t0 < a.ct; t0 += 32) {
    const int t = t0 + lane;
    float4 st = make_float4(-INFINITY, 0.f, 0.f, 0.f);
    if (t < a.ct) st = a.tile_stats[(size_t)row * a.ct_stride + t];
    float gmax = st.x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
    const unsigned holders = __ballot_sync(0xffffffffu, st.x == gmax);
    const int first = __ffs(holders) - 1;  // first lane (lowest tile) that holds the maximum
    const int cand = __shfl_sync(0xffffffffu, __float_as_int(st.w), first);
    if (gmax > run_max) best = cand;
    const float new_max = fmaxf(run_max, gmax);
    const float w = t < a.ct ? exp2f((st.x - new_max) * kLog2e) : 0.f;
    const float part_sum = warp_sum(st.y * w);
    const float part_dot = warp_sum(st.z * w);
    const float rescale = exp2f((run_max - new_max) * kLog2e);  // exp(-inf) = 0 on the first chunk
    run_sum = run_sum * rescale + part_sum;
    run_dot = run_dot * rescale + part_dot;
    run_max = new_max;
  }
  const float lse = run_max + logf(run_sum);
  const float fac = expf(prev_max + logf(prev_sum) - lse);  // exp(-inf) = 0 on the first chunk
  const long long tg = a.target[row];
  const bool labelled = tg != kIgnore;
  const long long local = tg - a.col_offset - a.col0;  // column inside this chunk
  const bool hit = labelled && local >= 0 && local < (long long)a.ct * kBN1 &&
                   a.col0 + local < a.v_shard;
  // All state of the previous chunk has been read by every warp before anyone overwrites it.
  __syncthreads();
  if (threadIdx.x == 0) {
    a.run_max[row] = run_max;
    a.run_sum[row] = run_sum;
    a.run_dot[row] = run_dot;
    a.best[row] = best;
    if (a.write_p) {
      a.factor[row] = fac;
      if (hit) a.label_lse[row] = lse;
    }
  }
  if (!a.write_p) return;
  if (a.dh && !a.first) {  // rescale what is accumulated to the new log-sum-exp
    float4* g = reinterpret_cast<float4*>(a.dh + (size_t)row * a.k_dim);
    const int n4 = a.k_dim >> 2;
    for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * blockDim.x < n4) v[u] = g[i0 + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * blockDim.x < n4) {
          v[u].x *= fac; v[u].y *= fac; v[u].z *= fac; v[u].w *= fac;
          g[i0 + u * blockDim.x] = v[u];
        }
    }
    for (int i = (a.k_dim & ~3) + threadIdx.x; i < a.k_dim; i += blockDim.x)
      a.dh[(size_t)row * a.k_dim + i] *= fac;
  }
  // P = 1024 * exp(z - lse) = E * 2^-14 * 1024 * exp(tile_max - lse); zero for unlabelled rows.
  // Warp w owns tiles w, w + 4, ...; their loads are all issued before the first store.
  __half* e_row = a.e_buf + (size_t)row * a.ld_e;
  for (int tb = warp; tb < a.ct; tb += kRowWarps * kRowTilesPerWarp) {
    uint4 v[kRowTilesPerWarp];
    float scale[kRowTilesPerWarp];
#pragma unroll
    for (int u = 0; u < kRowTilesPerWarp; ++u) {
      const int t = tb + u * kRowWarps;
      if (t < a.ct) {
        v[u] = *(reinterpret_cast<const uint4*>(e_row + t * kBN1) + lane);
        const float tmax = a.tile_stats[(size_t)row * a.ct_stride + t].x;
        scale[u] = labelled ? (kGradScale / kEScale) * exp2f((tmax - lse) * kLog2e) : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kRowTilesPerWarp; ++u) {
      const int t = tb + u * kRowWarps;
      if (t < a.ct) {
        uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 f = __half22float2(*reinterpret_cast<__half2*>(&w[k]));
          __half2 h = __floats2half2_rn(f.x * scale[u], f.y * scale[u]);
          w[k] = *reinterpret_cast<uint32_t*>(&h);
        }
        *(reinterpret_cast<uint4*>(e_row + t * kBN1) + lane) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  if (hit) {  // uniform over the CTA (one row per CTA)
    __syncthreads();
    if (threadIdx.x == 0) {
      // The label's entry carries p - 1, formed in fp32 and rounded once.
      const float p = expf(a.label_logit[row] - lse);
      e_row[local] = __float2half_rn((p - 1.0f) * kGradScale);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Gradient kernel: dH[rows, K] = factor * dH + P[rows, cols] * W[cols, K] for one chunk.
// ------------------------------------------------------------------------------------------
struct GradArgs {
  float* dh;            // [n_rows, k_dim] fp32 of this row block
  const float* factor;  // [n_rows]
  int n_rows;
  int k_dim;            // hidden size (output columns)
  int col0;             // first shard column of the chunk (TMA row coordinate into W)
  int n_kb;             // 64-column blocks of the chunk
  int first;            // first chunk: overwrite instead of accumulate
  int ksplit;           // pair kernel: K (vocabulary) splits per output tile, partial sums added with RED
  int debug;            // bit 5: skip the epilogue's global traffic (timing experiments only)
  int* status;
};

__global__ void __launch_bounds__(kThreadsGemm, 1)
lmhead_grad_kernel(const __grid_constant__ CUtensorMap map_p,
                   const __grid_constant__ CUtensorMap map_w, const GradArgs a) {
  extern __shared__ uint8_t smem_raw[];
  if (*reinterpret_cast<volatile int*>(a.status) != 0) return;  // an earlier kernel gave up
  constexpr int kStageBytes = kABytes + kB2Bytes;
  const GemmSmem s = carve_smem<kStages2, kStageBytes>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) { prefetch_tensormap(&map_p); prefetch_tensormap(&map_w); }
  init_pipeline<kStages2>(s, warp, lane);
  const uint32_t tmem = *s.tmem_base;

  const int rt = (a.n_rows + kBM - 1) / kBM;
  const int nt = (a.k_dim + kBN2 - 1) / kBN2;
  const int n_tiles = rt * nt;

  if (warp == 0) {
    if (lane == 0) {
      PipeState p;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int tr = tile % rt, tn = tile / rt;
        for (int kb = 0; kb < a.n_kb; ++kb) {
          ok = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 21);
          if (!ok) break;
          uint8_t* st = s.tiles + p.stage * kStageBytes;
          mbar_expect_tx(&s.full[p.stage], kStageBytes);
          tma_load_2d(st, &map_p, kb * kBK, tr * kBM, &s.full[p.stage]);
#pragma unroll
          for (int j = 0; j < kBN2 / 64; ++j)
            tma_load_2d(st + kABytes + j * (kBK * 128), &map_w, tn * kBN2 + j * 64,
                        a.col0 + kb * kBK, &s.full[p.stage]);
          p.advance<kStages2>();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBM, kBN2, false, true);
      PipeState p;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait(&s.acc_empty[ab], acc_phase ^ 1u, s.abort_flag, a.status, 22);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + ab * 256;
        for (int kb = 0; kb < a.n_kb; ++kb) {
          ok = mbar_wait(&s.full[p.stage], p.phase, s.abort_flag, a.status, 23);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.tiles + p.stage * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr, 16, 1024);
          // MN-major B: 64-column groups are kBK*128 bytes apart (leading offset), 8-k groups
          // 1024 bytes apart (stride offset); one MMA consumes 16 k = 2048 bytes.
          const uint64_t db = make_smem_desc(a_addr + kABytes, kBK * 128, 1024);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            mma_f16_ss(d_tmem, da + k4 * 2, db + k4 * (2048 >> 4), idesc, (kb | k4) != 0);
          tc_commit(&s.empty[p.stage]);
          p.advance<kStages2>();
        }
        if (ok) tc_commit(&s.acc_full[ab]);
      }
    }
  } else {
    const int q = warp & 3;
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
      const int tr = tile % rt, tn = tile / rt;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&s.acc_full[ab], acc_phase, s.abort_flag, a.status, 24));
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tr * kBM + q * 32 + lane;
      const bool row_ok = row < a.n_rows;
      const float fac = (row_ok && !a.first) ? a.factor[row] : 0.f;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + ab * 256;
      float* out_row = a.dh + (size_t)row * a.k_dim + tn * kBN2;
      const int n_valid = min(kBN2, a.k_dim - tn * kBN2);
#pragma unroll 1
      for (int c = 0; c < kBN2 / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row_ok && !(a.debug & 32)) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int col = c * 32 + j;
            if (col + 3 < n_valid) {
              float4* dst = reinterpret_cast<float4*>(out_row + col);
              float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                     __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              if (!a.first) {
                const float4 old = *dst;
                o.x = fmaf(old.x, fac, o.x); o.y = fmaf(old.y, fac, o.y);
                o.z = fmaf(old.z, fac, o.z); o.w = fmaf(old.w, fac, o.w);
              }
              *dst = o;
            } else {
              for (int u = 0; u < 4; ++u)
                if (col + u < n_valid) {
                  const float acc = __uint_as_float(r[j + u]);
                  out_row[col + u] = a.first ? acc : fmaf(out_row[col + u], fac, acc);
                }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[ab]);
    }
  }
  finish_pipeline(s, warp, tmem);
}

// ------------------------------------------------------------------------------------------
// Gradient kernel, CTA pairs: the pair owns 256 rows x 192 hidden columns; each CTA loads its 128
// rows of P and 96 of the 192 weight columns (three 32-column boxes, 64-byte swizzle, MN-major).
// 8 x 8 = 64 pair tiles cover [2048, 1536]. The epilogue transposes each 32 x 32 block of the
// accumulator through shared memory so that dH is read and written in full 128-byte rows.
// ------------------------------------------------------------------------------------------
constexpr int kStageT = 4 * 32 * 33 * 4;             // per epilogue warp a padded 32 x 32 fp32 block

// BN = hidden columns per pair tile, SWZ = swizzle width in bytes of the B boxes (64 or 128; the
// half of BN one CTA holds must be a whole number of SWZ/2-column boxes).
template <int BN, int SWZ>
struct GradPairCfg {
  static constexpr int kBoxCols = SWZ / 2;
  static constexpr int kBoxes = BN / 2 / kBoxCols;
  static constexpr int kBoxBytes = kBK * SWZ;
  static constexpr int kBHalfBytes = kBoxes * kBoxBytes;
  static constexpr int kStageBytes = kABytes + kBHalfBytes;
  static constexpr int kStages = (200 * 1024) / kStageBytes;
  static constexpr int kSmem = kStages * kStageBytes + kStageT + 1024 + 256;
  static_assert(kBoxes * kBoxCols * 2 == BN, "half tile must be whole boxes");
  static_assert(kStageBytes % 1024 == 0, "stages must keep 1024-byte alignment");
};

template <int BN, int SWZ>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsGemm, 1)
lmhead_grad_pair_kernel(const __grid_constant__ CUtensorMap map_p,
                        const __grid_constant__ CUtensorMap map_w, const GradArgs a) {
  using Cfg = GradPairCfg<BN, SWZ>;
  extern __shared__ uint8_t smem_raw[];
  constexpr int kStageBytes = Cfg::kStageBytes;
  constexpr int kStages = Cfg::kStages;
  const GemmSmem s = carve_smem<kStages, kStageBytes, kStageT>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) { prefetch_tensormap(&map_p); prefetch_tensormap(&map_w); }
  const PairInit pi = init_pair<kStages>(s, warp, lane, a.status);
  if (!pi.run) return;
  const uint32_t tmem = pi.tmem, rank = pi.rank;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  const int rt = (a.n_rows + 2 * kBM - 1) / (2 * kBM);
  const int nt = (a.k_dim + BN - 1) / BN;
  const int n_tiles = rt * nt;
  const int n_units = n_tiles * a.ksplit;   // unit = (output tile, K split)

  if (warp == 0) {
    if (lane == 0) {
      PipeState p;
      bool ok = true;
      for (int unit = pair; unit < n_units && ok; unit += n_pairs) {
        const int tile = unit % n_tiles, ks = unit / n_tiles;
        const int tr = tile % rt, tn = tile / rt;
        const int row0 = tr * 2 * kBM + (int)rank * kBM;
        const int hcol0 = tn * BN + (int)rank * (BN / 2);
        const int kb_end = (a.n_kb * (ks + 1)) / a.ksplit;
        for (int kb = (a.n_kb * ks) / a.ksplit; kb < kb_end; ++kb) {
          ok = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 41);
          if (!ok) break;
          uint8_t* st = s.tiles + p.stage * kStageBytes;
          const uint32_t full_leader = mapa_u32(smem_u32(&s.full[p.stage]), 0);
          if (rank == 0) mbar_expect_tx(&s.full[p.stage], 2 * kStageBytes);
          tma_load_2d_pair(st, &map_p, kb * kBK, row0, full_leader);
#pragma unroll
          for (int j = 0; j < Cfg::kBoxes; ++j)
            tma_load_2d_pair(st + kABytes + j * Cfg::kBoxBytes, &map_w, hcol0 + j * Cfg::kBoxCols,
                             a.col0 + kb * kBK, full_leader);
          p.template advance<kStages>();
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * kBM, BN, false, true);
      PipeState p;
      bool ok = true;
      int it = 0;
      for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++it) {
        const int ks = unit / n_tiles;
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait(&s.acc_empty[ab], acc_phase ^ 1u, s.abort_flag, a.status, 42);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem + ab * 256;
        const int kb_begin = (a.n_kb * ks) / a.ksplit, kb_end = (a.n_kb * (ks + 1)) / a.ksplit;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ok = mbar_wait(&s.full[p.stage], p.phase, s.abort_flag, a.status, 43);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.tiles + p.stage * kStageBytes);
          const uint64_t da = make_smem_desc(a_addr, 16, 1024);
          // MN-major B: column groups of one box are kBoxBytes apart (leading offset), 8-k groups
          // 8*SWZ bytes apart (stride offset); one MMA consumes 16 k = 16*SWZ bytes.
          const uint64_t db = make_smem_desc(a_addr + kABytes, Cfg::kBoxBytes, 8 * SWZ,
                                             SWZ == 128 ? 2 : 4);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            mma_f16_ss_pair(d_tmem, da + k4 * 2, db + k4 * ((16 * SWZ) >> 4), idesc,
                            (kb != kb_begin) || k4 != 0);
          tc_commit_pair(&s.empty[p.stage], 3);
          p.template advance<kStages>();
        }
        if (ok) tc_commit_pair(&s.acc_full[ab], 3);
      }
    }
  } else {
    const int q = warp & 3;
    float* tpose = reinterpret_cast<float*>(s.extra) + (warp - 2) * (32 * 33);
    bool ok = true;
    int it = 0;
    const bool plain_store = a.first && a.ksplit == 1;   // else dH was zeroed / rescaled before
    for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++it) {
      const int tile = unit % n_tiles;
      const int tr = tile % rt, tn = tile / rt;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&s.acc_full[ab], acc_phase, s.abort_flag, a.status, 44));
      if (!ok) break;
      tc_fence_after_sync();
      const int row_base = tr * 2 * kBM + (int)rank * kBM + q * 32;   // first of this warp's 32 rows
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + ab * 256;
      const int col_base = tn * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait_on(r);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; ++j) tpose[lane * 33 + j] = __uint_as_float(r[j]);
        __syncwarp();
        // dH was already multiplied by this chunk's factor (row kernel), so partial sums are added
        // with fire-and-forget reductions. With ksplit == 1 one CTA adds to an element per chunk
        // and the result is deterministic; with K splits the order of the adds is not.
        const int col = col_base + c * 32 + lane;
        const bool col_ok = col < a.k_dim && !(a.debug & 32);
#pragma unroll 8
        for (int rr = 0; rr < 32; ++rr) {
          const int row = row_base + rr;
          if (col_ok && row < a.n_rows) {
            float* dst = a.dh + (size_t)row * a.k_dim + col;
            const float acc = tpose[rr * 33 + lane];
            if (plain_store) *dst = acc;
            else atomicAdd(dst, acc);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&s.acc_empty[ab]);
        else mbar_arrive_cluster(mapa_u32(smem_u32(&s.acc_empty[ab]), 0));
      }
    }
  }
  finish_pair(s, warp, tmem);
}

// ------------------------------------------------------------------------------------------
// Small kernels: state initialisation, merge across ranks, finish.
// ------------------------------------------------------------------------------------------
__global__ void lmhead_init_state_kernel(float* run_max, float* run_sum, float* run_dot, int* best,
                                         float* label_logit, float* label_lse, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  run_max[i] = -INFINITY;
  run_sum[i] = 0.f;
  run_dot[i] = 0.f;
  best[i] = 0;
  label_logit[i] = 0.f;
  label_lse[i] = 0.f;
}

// states: [n_ranks, n] each; out: [n]. Ranks are in ascending vocabulary order, so a later rank
// wins the argmax only if strictly larger.
__global__ void lmhead_merge_kernel(const float* g_max, const float* g_sum, const float* g_dot,
                                    const int* g_best, const float* g_label_logit,
                                    const float* g_label_lse, const int64_t* target,
                                    const int64_t* shard_begin, float* o_max, float* o_sum,
                                    float* o_dot, int* o_best, float* o_label_logit,
                                    float* o_label_lse, float* o_lse, int n, int n_ranks) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float m = -INFINITY;
  int best = 0;
  for (int r = 0; r < n_ranks; ++r) {
    const float v = g_max[(size_t)r * n + i];
    if (v > m) { m = v; best = g_best[(size_t)r * n + i]; }
  }
  float sum = 0.f, dot = 0.f;
  for (int r = 0; r < n_ranks; ++r) {
    const float w = exp2f((g_max[(size_t)r * n + i] - m) * kLog2e);
    sum += g_sum[(size_t)r * n + i] * w;
    dot += g_dot[(size_t)r * n + i] * w;
  }
  float ll = 0.f, lls = 0.f;
  const long long tg = target[i];
  if (tg != kIgnore) {
    for (int r = 0; r < n_ranks; ++r)
      if (tg >= shard_begin[r] && tg < shard_begin[r + 1]) {
        ll = g_label_logit[(size_t)r * n + i];
        lls = g_label_lse[(size_t)r * n + i];
      }
  }
  o_max[i] = m; o_sum[i] = sum; o_dot[i] = dot; o_best[i] = best;
  o_label_logit[i] = ll; o_label_lse[i] = lls;
  o_lse[i] = m + logf(sum);
}

struct FinishArgs {
  const float* run_max;     // final (merged) state
  const float* run_sum;
  const float* run_dot;
  const int* best;
  const float* label_logit;
  const float* label_lse;
  const float* local_lse;   // nullable: lse of this rank's own shard, for the dH rescale
  const int64_t* target;
  const __half* weight;     // this rank's shard [v_shard, k_dim]
  float* token_loss;        // nullable (only the rank that reports writes them)
  float* entropy;
  int* correct;
  float* dh;                // nullable
  int n_rows, k_dim, v_shard, col_offset;
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
  const float scale = a.local_lse ? expf(a.local_lse[row] - lse) : 1.0f;
  const long long local = tg - a.col_offset;
  const bool mine = labelled && local >= 0 && local < a.v_shard;
  // The label's -1 entered the sum in its chunk and was rescaled with it by
  // exp(lse_at_label_chunk - lse); put the missing part of -W[label] back.
  const float missing = mine ? (1.0f - expf(a.label_lse[row] - lse)) * kGradScale : 0.f;
  const __half* w_row = a.weight + (size_t)(mine ? local : 0) * a.k_dim;
  if (scale == 1.0f && !mine) return;
  for (int c = threadIdx.x; c < a.k_dim; c += blockDim.x) {
    float v = dh_row[c] * scale;
    if (mine) v -= __half2float(w_row[c]) * missing;
    dh_row[c] = v;
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
  int ct;          // column tiles per chunk
};

// Rows per block and column tiles per chunk: the E buffer of one chunk must stay L2 resident
// (about 40 MB) and rows_tiles * ct should fill whole waves of SMs.
inline Plan make_plan(int64_t n, int64_t v_shard, int sms, int ct_override) {
  Plan p;
  p.row_block = (int)(n < 2048 ? (n < 1 ? 1 : n) : 2048);
  const int rt = (p.row_block + kBM - 1) / kBM;
  const int total_ct = (int)((v_shard + kBN1 - 1) / kBN1);
  int ct = 37;
  if (ct_override > 0) {
    ct = ct_override;
  } else {
    // largest ct <= 40 with rt*ct a multiple of the SM count, else 37
    int best = -1;
    for (int c = 40; c >= 8; --c)
      if ((rt * c) % sms == 0) { best = c; break; }
    if (best > 0) ct = best;
  }
  if (ct > total_ct) ct = total_ct;
  if (ct < 1) ct = 1;
  p.ct = ct;
  return p;
}

struct Workspace {
  __half* e_buf;
  float4* tile_stats;
  float* factor;
  int* status;
  int64_t bytes;
};

inline Workspace carve_workspace(void* base, const Plan& p) {
  Workspace w;
  uint8_t* b = reinterpret_cast<uint8_t*>(base);
  int64_t off = 0;
  const int64_t ld_e = (int64_t)p.ct * kBN1;
  w.e_buf = reinterpret_cast<__half*>(b + off);
  off += round_up((int64_t)p.row_block * ld_e * 2, 1024);
  w.tile_stats = reinterpret_cast<float4*>(b + off);
  off += round_up((int64_t)p.row_block * p.ct * 16, 1024);
  w.factor = reinterpret_cast<float*>(b + off);
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
  void begin(int k) { if (on) { cudaEvent_t e; cudaEventCreate(&e); cudaEventRecord(e, s); ev[k].push_back(e); } }
  void end(int k) { begin(k); }
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
                           kSmem1) != cudaSuccess)
    return -1;
  if (cudaFuncSetAttribute(lmhead_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kSmem2) != cudaSuccess)
    return -1;
  if (cudaFuncSetAttribute(lmhead_logits_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kSmemP1) != cudaSuccess)
    return -1;
  if (cudaFuncSetAttribute(lmhead_grad_pair_kernel<256, 128>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                           GradPairCfg<256, 128>::kSmem) != cudaSuccess)
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

int encode_map_2d_f16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                      uint64_t pitch_elems, uint32_t box_rows, uint32_t box_cols, int swizzle_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_elems * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
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

extern "C" int soup_lmhead_ce(const void* hidden, const void* weight, const int64_t* target,
                              float* run_max, float* run_sum, float* run_dot, int* best,
                              float* label_logit, float* label_lse, float* dh, void* workspace,
                              int64_t workspace_bytes, int64_t n, int64_t h, int64_t v_shard,
                              int64_t col_offset, int64_t chunk_tiles, int want_grad,
                              void* stream) {
  using namespace soup;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n < 0 || h <= 0 || v_shard <= 0) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: bad shape");
  if (n == 0) return SOUP_OK;
  if (!hidden || !weight || !target || !run_max || !run_sum || !run_dot || !best || !label_logit ||
      !label_lse || !workspace || (want_grad && !dh))
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: null pointer");
  if (h % 8 != 0) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: hidden size must be a multiple of 8 (TMA pitch)");
  if (!aligned16(hidden) || !aligned16(weight) || !aligned16(workspace) || (dh && !aligned16(dh)))
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: pointers must be 16-byte aligned");
  if (n > INT32_MAX / 2 || v_shard > INT32_MAX / 2 || col_offset + v_shard > INT32_MAX)
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: shape exceeds 32-bit tile coordinates");
  const int attr = ensure_smem_attr();
  if (attr == -2) SOUP_FAIL(SOUP_ERR_DEVICE, "lmhead_ce: needs a compute capability 10.x device");
  if (attr != 0) SOUP_FAIL(SOUP_ERR_DEVICE, "lmhead_ce: cannot raise the shared-memory limit");
  const int sms = sm_count();
  const Plan plan = make_plan(n, v_shard, sms, (int)chunk_tiles);
  const Workspace ws = carve_workspace(workspace, plan);
  if (workspace_bytes < ws.bytes)
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_ce: workspace too small (%lld < %lld)",
              (long long)workspace_bytes, (long long)ws.bytes);
  const int ld_e = plan.ct * kBN1;
  const int total_ct = (int)((v_shard + kBN1 - 1) / kBN1);

  CUtensorMap map_h, map_w1, map_w1h, map_w2, map_w2h, map_p, map_e;
  const char* single_env = getenv("SOUP_LMHEAD_SINGLE_CTA");
  const bool use_pairs = !(single_env && atoi(single_env) != 0) && (sms % 2 == 0);
  const char* det_env = getenv("SOUP_LMHEAD_DETERMINISTIC");
  const bool deterministic = det_env && atoi(det_env) != 0;
  if (umma::encode_map_2d_f16(&map_h, hidden, (uint64_t)n, (uint64_t)h, (uint64_t)h, kBM, kBK) ||
      umma::encode_map_2d_f16(&map_w1, weight, (uint64_t)v_shard, (uint64_t)h, (uint64_t)h, kBN1, kBK) ||
      umma::encode_map_2d_f16(&map_w1h, weight, (uint64_t)v_shard, (uint64_t)h, (uint64_t)h, kBN1 / 2, kBK) ||
      umma::encode_map_2d_f16(&map_w2, weight, (uint64_t)v_shard, (uint64_t)h, (uint64_t)h, kBK, 64) ||
      umma::encode_map_2d_f16(&map_w2h, weight, (uint64_t)v_shard, (uint64_t)h, (uint64_t)h, kBK, 32, 64) ||
      umma::encode_map_2d_f16(&map_p, ws.e_buf, (uint64_t)plan.row_block, (uint64_t)ld_e,
                              (uint64_t)ld_e, kBM, kBK) ||
      umma::encode_map_2d_f16(&map_e, ws.e_buf, (uint64_t)plan.row_block, (uint64_t)ld_e,
                              (uint64_t)ld_e, 32, 64))
    SOUP_FAIL(SOUP_ERR_DEVICE, "lmhead_ce: cuTensorMapEncodeTiled failed");

  cudaMemsetAsync(ws.status, 0, 4, s);
  if (use_pairs && want_grad && !deterministic)   // K-split partial sums are added into dH
    cudaMemsetAsync(dh, 0, (size_t)n * h * sizeof(float), s);
  lmhead_init_state_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(
      run_max, run_sum, run_dot, best, label_logit, label_lse, (int)n);
  SOUP_CHECK_LAUNCH("lmhead_init_state");

  LaunchTimer timer(s);
  for (int64_t r0 = 0; r0 < n; r0 += plan.row_block) {
    const int rows = (int)((n - r0) < plan.row_block ? (n - r0) : plan.row_block);
    const int rt = (rows + kBM - 1) / kBM;
    for (int t0 = 0; t0 < total_ct; t0 += plan.ct) {
      const int ct = (total_ct - t0) < plan.ct ? (total_ct - t0) : plan.ct;
      LogitsArgs la;
      la.target = target + r0;
      la.e_buf = ws.e_buf;
      la.tile_stats = ws.tile_stats;
      la.label_logit = label_logit + r0;
      la.n_rows = rows;
      la.row0 = (int)r0;
      la.k_dim = (int)h;
      la.col0 = t0 * kBN1;
      la.v_shard = (int)v_shard;
      la.col_offset = (int)col_offset;
      la.ct = ct;
      la.ct_stride = plan.ct;
      la.ld_e = ld_e;
      la.write_e = want_grad;
      {
        const char* dbg = getenv("SOUP_LMHEAD_DEBUG");
        la.debug = dbg ? atoi(dbg) : 0;
      }
      la.status = ws.status;
      const int tiles1 = rt * ct;
      timer.begin(0);
      if (use_pairs) {
        const int tiles_p = ((rows + 2 * kBM - 1) / (2 * kBM)) * ct;
        const int pairs = tiles_p < sms / 2 ? tiles_p : sms / 2;
        lmhead_logits_pair_kernel<<<(unsigned)(2 * pairs), kThreadsGemm, kSmemP1, s>>>(
            map_h, map_w1h, map_e, la);
      } else {
        lmhead_logits_kernel<<<(unsigned)(tiles1 < sms ? tiles1 : sms), kThreadsGemm, kSmem1, s>>>(
            map_h, map_w1, map_e, la);
      }
      timer.end(0);
      SOUP_CHECK_LAUNCH("lmhead_logits");

      RowArgs ra;
      ra.target = target + r0;
      ra.e_buf = ws.e_buf;
      ra.tile_stats = ws.tile_stats;
      ra.run_max = run_max + r0;
      ra.run_sum = run_sum + r0;
      ra.run_dot = run_dot + r0;
      ra.best = best + r0;
      ra.label_logit = label_logit + r0;
      ra.label_lse = label_lse + r0;
      ra.factor = ws.factor;
      ra.n_rows = rows;
      ra.col0 = t0 * kBN1;
      ra.v_shard = (int)v_shard;
      ra.col_offset = (int)col_offset;
      ra.ct = ct;
      ra.ct_stride = plan.ct;
      ra.ld_e = ld_e;
      ra.write_p = want_grad;
      ra.dh = (use_pairs && want_grad) ? dh + r0 * h : nullptr;
      ra.k_dim = (int)h;
      ra.first = t0 == 0;
      timer.begin(1);
      lmhead_row_kernel<<<(unsigned)rows, kRowWarps * 32, 0, s>>>(ra);
      timer.end(1);
      SOUP_CHECK_LAUNCH("lmhead_row");

      if (want_grad) {
        GradArgs ga;
        ga.dh = dh + r0 * h;
        ga.factor = ws.factor;
        ga.n_rows = rows;
        ga.k_dim = (int)h;
        ga.col0 = t0 * kBN1;
        ga.n_kb = ct * (kBN1 / kBK);
        ga.first = t0 == 0;
        ga.ksplit = 1;
        ga.debug = la.debug;
        ga.status = ws.status;
        const int tiles2 = rt * (int)((h + kBN2 - 1) / kBN2);
        timer.begin(2);
        if (use_pairs) {
          const int tiles_p = ((rows + 2 * kBM - 1) / (2 * kBM)) * (int)((h + 255) / 256);
          ga.ksplit = pick_ksplit(tiles_p, sms / 2, ga.n_kb, deterministic);
          const int units = tiles_p * ga.ksplit;
          const int pairs = units < sms / 2 ? units : sms / 2;
          lmhead_grad_pair_kernel<256, 128><<<(unsigned)(2 * pairs), kThreadsGemm,
                                               GradPairCfg<256, 128>::kSmem, s>>>(map_p, map_w2, ga);
        } else {
          lmhead_grad_kernel<<<(unsigned)(tiles2 < sms ? tiles2 : sms), kThreadsGemm, kSmem2, s>>>(
              map_p, map_w2, ga);
        }
        timer.end(2);
        SOUP_CHECK_LAUNCH("lmhead_grad");
      }
    }
  }
  timer.finish();
  return SOUP_OK;
}

extern "C" int soup_lmhead_set_timing(float* host_sink6) {
  soup::g_timing_sink = host_sink6;
  return SOUP_OK;
}

extern "C" int soup_lmhead_plan(int64_t n, int64_t v_shard, int64_t chunk_tiles, int64_t* row_block,
                                int64_t* tiles_per_chunk) {
  using namespace soup;
  const Plan p = make_plan(n, v_shard, sm_count(), (int)chunk_tiles);
  if (row_block) *row_block = p.row_block;
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
                                 const int* g_best, const float* g_label_logit,
                                 const float* g_label_lse, const int64_t* target,
                                 const int64_t* shard_begin, float* o_max, float* o_sum,
                                 float* o_dot, int* o_best, float* o_label_logit,
                                 float* o_label_lse, float* o_lse, int64_t n, int n_ranks,
                                 void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || n_ranks < 1) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_merge: bad shape");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  lmhead_merge_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(
      g_max, g_sum, g_dot, g_best, g_label_logit, g_label_lse, target, shard_begin, o_max, o_sum,
      o_dot, o_best, o_label_logit, o_label_lse, o_lse, (int)n, n_ranks);
  SOUP_CHECK_LAUNCH("lmhead_merge");
  return SOUP_OK;
}

extern "C" int soup_lmhead_finish(const float* run_max, const float* run_sum, const float* run_dot,
                                  const int* best, const float* label_logit, const float* label_lse,
                                  const float* local_lse, const int64_t* target, const void* weight,
                                  float* token_loss, float* entropy, int* correct, float* dh,
                                  int64_t n, int64_t h, int64_t v_shard, int64_t col_offset,
                                  void* stream) {
  using namespace soup;
  if (n == 0) return SOUP_OK;
  if (n < 0 || h <= 0) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: bad shape");
  if (!run_max || !run_sum || !run_dot || !best || !label_logit || !label_lse || !target)
    SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: null pointer");
  if (dh && !weight) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: dH needs the weight shard");
  if (token_loss && (!entropy || !correct)) SOUP_FAIL(SOUP_ERR_ARG, "lmhead_finish: null output");
  FinishArgs a;
  a.run_max = run_max; a.run_sum = run_sum; a.run_dot = run_dot; a.best = best;
  a.label_logit = label_logit; a.label_lse = label_lse; a.local_lse = local_lse;
  a.target = target; a.weight = reinterpret_cast<const __half*>(weight);
  a.token_loss = token_loss; a.entropy = entropy; a.correct = correct; a.dh = dh;
  a.n_rows = (int)n; a.k_dim = (int)h; a.v_shard = (int)v_shard; a.col_offset = (int)col_offset;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  lmhead_finish_kernel<<<(unsigned)n, 256, 0, s>>>(a);
  SOUP_CHECK_LAUNCH("lmhead_finish");
  return SOUP_OK;
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
