// Warp-private shared-memory row pipeline for the row-wise memory-bound kernels (RMSNorm, RoPE).
//
// A row kernel has a dependency inside each row (load the row, reduce, then write), so the bytes
// it keeps in flight are what decides its HBM throughput. Holding rows in registers caps that at
// what the register file allows (~100 KB per SM, measured 50-65 % of copy bandwidth). Here every
// warp owns a ring of `stages` row slots in shared memory and one lane feeds it with 1-D bulk
// async copies (cp.async.bulk, completion counted on an mbarrier per slot), so the warp's next
// rows are already travelling while it works on the current one; in-flight bytes are bounded by
// shared memory (up to ~190 KB per SM) instead of registers. No CTA-wide barrier is involved after
// set-up: each warp runs its own pipeline over its own rows.
//
// Bulk copies need 16-byte aligned source/destination and a size that is a multiple of 16 bytes.
// Every wait is bounded (umma::mbar_wait); a warp that gives up waits, bounded again, for the
// copies it still has in flight before it leaves, so no copy can land in a dead CTA's memory.
#pragma once

#include "umma.cuh"

namespace soup {
namespace rowpipe {

constexpr int kMaxWarps = 16;      // warps per CTA (8 or 16), each with its own ring
constexpr int kMaxStages = 8;
constexpr int kRingBytesPerCta = 100 * 1024;  // two CTAs per SM

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(umma::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(umma::smem_u32(bar))
      : "memory");
}

// Launch shape of a pipelined row kernel. These kernels spend a good part of their issue slots on
// unpacking and rounding, so they want 32 warps per SM (two CTAs of 16) as well as bytes in
// flight. A row whose slot would leave a warp fewer than two stages is split over a team of two
// warps, each with its own half-row slots (`team_divisible` says the kernel can split this shape;
// `team_extra` is what every member's slot carries in addition to its share, e.g. RoPE's cos/sin
// rows). `stages` is 0 when nothing fits (the caller falls back to another kernel).
struct Plan {
  int warps, stages, team;
  unsigned grid;
  size_t smem, slot_bytes;   // slot_bytes: per warp
};

int sm_count_for_plan();

inline Plan make_plan(size_t split_bytes, size_t team_extra, bool team_divisible, int64_t n_rows) {
  Plan p = {16, 0, 1, 1, 0, 0};
  if (split_bytes == 0 || n_rows <= 0) return p;
  auto stages_at = [&](int warps, int team) {
    const size_t slot = split_bytes / team + team_extra;
    return (int)(kRingBytesPerCta / (warps * slot));
  };
  if (stages_at(16, 1) >= 2 || !team_divisible) {
    p.team = 1;
    p.warps = stages_at(16, 1) >= 1 ? 16 : 8;
  } else if (stages_at(16, 2) >= 1) {
    p.team = 2;
  } else {
    p.team = 1;
    p.warps = 8;
  }
  p.stages = stages_at(p.warps, p.team);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (p.stages == 0) return p;
  p.slot_bytes = split_bytes / p.team + team_extra;
  const int64_t rows_per_cta = p.warps / p.team;
  const int64_t need = (n_rows + rows_per_cta - 1) / rows_per_cta;
  const int64_t cap = (int64_t)sm_count_for_plan() * 2;
  const int64_t grid = need < cap ? need : cap;
  const int64_t per_team = (n_rows + grid * rows_per_cta - 1) / (grid * rows_per_cta);
  if (p.stages > per_team) p.stages = (int)per_team;
  p.grid = (unsigned)grid;
  p.smem = (size_t)p.warps * p.stages * p.slot_bytes + kMaxWarps * kMaxStages * sizeof(uint64_t);
  return p;
}

// Sum over the two warps of a team (every lane of both warps gets the total). `part` is a
// [2][kMaxWarps] float array in shared memory, `iter` the team's row counter (the two halves of
// `part` alternate so that a fast warp cannot overwrite a value its partner has not read yet).
__device__ __forceinline__ float team_sum2(float warp_total, float* part, int warp, int lane,
                                           int iter) {
  float* mine = part + (iter & 1) * kMaxWarps;
  if (lane == 0) mine[warp] = warp_total;
  // named barrier of this team: ids 1..8, 64 threads
  asm volatile("bar.sync %0, 64;" ::"r"((warp >> 1) + 1) : "memory");
  return mine[warp] + mine[warp ^ 1];
}

// Device status word shared by the row kernels: 0, or the code of the first wait that timed out.
int* status_word();   // host: device address for the current device (nullptr on failure)

struct Ring {
  char* buf;            // this warp's slots
  uint64_t* bars;       // this warp's barriers
  uint32_t slot_bytes;
  int stages;
  uint32_t phases;      // parity bit per slot
  int slot;             // slot of the row being consumed

  __device__ __forceinline__ void init(char* smem, uint32_t slot_bytes_, int stages_, int warp,
                                       int lane) {
    slot_bytes = slot_bytes_;
    stages = stages_;
    const int warps = blockDim.x >> 5;
    buf = smem + (size_t)warp * stages * slot_bytes;
    bars = reinterpret_cast<uint64_t*>(smem + (size_t)warps * stages * slot_bytes) +
           warp * kMaxStages;
    phases = 0;
    slot = 0;
    if (lane == 0)
      for (int s = 0; s < stages; ++s) umma::mbar_init(&bars[s], 1);
    umma::fence_barrier_init();
  }
  __device__ __forceinline__ char* slot_ptr(int s) const { return buf + (size_t)s * slot_bytes; }
  __device__ __forceinline__ bool wait(volatile int* abort_flag, int* status, int code) {
    const bool ok = umma::mbar_wait(&bars[slot], (phases >> slot) & 1u, abort_flag, status, code);
    if (ok) phases ^= 1u << slot;
    return ok;
  }
  __device__ __forceinline__ void advance() { slot = slot + 1 == stages ? 0 : slot + 1; }
  // Bounded wait for `pending` more slots starting at the current one (used when giving up).
  __device__ __forceinline__ void drain(int pending) {
    for (int i = 0; i < pending; ++i) {
      const uint64_t t0 = umma::global_timer_ns();
      while (!umma::mbar_try_wait(&bars[slot], (phases >> slot) & 1u)) {
        if (umma::global_timer_ns() - t0 > umma::kWaitLimitNs) break;
      }
      phases ^= 1u << slot;
      advance();
    }
  }
};

}  // namespace rowpipe
}  // namespace soup
