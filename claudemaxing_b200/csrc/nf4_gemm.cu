// Linear layers on NF4 weights without the fp16 weight in HBM: tcgen05 GEMMs whose B operand is
// dequantised from the packed 4-bit codes straight into the shared-memory tile the tensor core
// reads.
//
//   forward   y[m, n]  = x[m, k] * W[n, k]^T (+ bias)     W is the K-major operand
//   backward  dx[m, k] = sum_i dy_i[m, n_i] * W_i[n_i, k]  W is the MN-major operand (no transpose)
//
// Both run on CTA pairs (cta_group::2): a pair owns 256 output columns and 256 or 512 rows (one or
// two accumulators of 256 TMEM columns per CTA, so that a dequantised weight tile is used by up to
// four 128-row A tiles), each CTA bringing its 128 rows of A by TMA and dequantising its half of
// the weight tile.
//
// Warp roles per CTA (16 warps): 0 TMA loads of A into the operand ring; 1 MMA issue (leader CTA
// only); 2 TMA loads of the packed codes into the raw ring; 3 block scales into the raw ring;
// 4-7 epilogue; 8-15 conversion, in two groups of four warps that take alternate pipeline steps.
//
// Dequantisation. One NF4 block of 64 elements along K (32 packed bytes, one absmax) is exactly
// one 128-byte row of the 128-byte-swizzled operand tile in either direction: in the forward
// tile a row is one weight row's 64 k-values, in the backward (MN-major) tile a row is one
// weight row's 64 output columns. Per pipeline step a CTA needs 128 such blocks. Their packed
// bytes arrive by TMA (two boxes of 64 rows x 32 bytes) in a slot of the raw ring; warp 3 writes
// the 128 block scales beside them,
//   scale = code2[absmax8[b]] * absmax2[b / blocksize2] + offset      (__fmul_rn, __fadd_rn)
// from statistics it loads several steps ahead. A conversion thread owns one block of its
// group's step: it forms the block's sixteen possible values once,
//   t[i]  = fp16_rn(code[i] * scale)                                  (__fmul_rn)
// the same unfused fp32 operations, in the same order, as the stand-alone dequantisation kernel,
// so the operand is bit-identical to dequantize_nf4's output; splits them into a low-byte and a
// high-byte plane (four registers each); and looks four nibbles at a time up with byte permutes
// (prmt: a 4-bit index is a 3-bit select in either half of a plane plus a mask on its top bit).
// No shared-memory table look-ups: the tensor core's operand reads need that bandwidth. The eight
// 16-byte pieces of the row go to their swizzled places of the operand slot (piece p of row r at
// p ^ (r & 7)); a proxy fence makes the writes visible to the tensor core and one lane per warp
// arrives on the leader CTA's "full" barrier of the slot, next to the byte count of the A loads.
//
// What was learned on the way (cycle stamps written by every role, B200):
//  * conversion threads must not have global loads in flight at the proxy fence (a first version
//    fetched the codes into registers): hence the TMA-fed raw ring and the separate scale warp;
//  * mbarrier waits with .acquire.cluster and arrivals with .release.cluster cost the issuing
//    thread on the order of a thousand cycles each; the per-step hand-over uses the default
//    scope on both sides (the data is already visible to the tensor core's proxy);
//  * a conversion step has ~900 cycles of fixed latency (two barrier waits, fence, two arrivals)
//    beside ~700 of arithmetic, so two groups alternate steps;
//  * with all SMs busy the conversion of a CTA's 128 blocks takes ~1400 cycles per step, more
//    than one accumulator's MMAs (512): two accumulators per CTA halve the conversion per flop, at
//    the price of an epilogue (~8000 cycles per accumulator) that cannot overlap the next unit.
//
// Relation to the reference: its 4-bit projections are bitsandbytes' dequantise-then-F.linear
// (solution/nf4.py:122) and bnb.matmul_4bit in the MLP forward and recompute
// (solution/swiglu_recompute.py:165-166, 198-199), whose backward multiplies the incoming gradient
// with the dequantised weight. Here the dequantised weight exists only as shared-memory tiles.
#include <math.h>

#include "common.cuh"
#include "rowpipe.cuh"
#include "umma.cuh"

namespace soup {
namespace {

using namespace umma;

constexpr int kBM = 128;                 // rows per CTA and accumulator (TMEM lanes)
constexpr int kBN = 256;                 // output columns per CTA pair
constexpr int kBK = 64;                  // contraction elements per pipeline step = one NF4 block
constexpr int kSub = kBM * kBK * 2;      // 16 KB: one 128 x 64 fp16 tile (an A tile; this CTA's half of B)
constexpr int kCvGroups = 2;              // conversion groups; group g converts the steps g, g + kCvGroups, ...
constexpr int kCvGroupWarps = 4;          // 128 threads: one block of a step per thread
constexpr int kCvWarps = kCvGroups * kCvGroupWarps;
constexpr int kFirstCvWarp = 8;
constexpr int kThreads = (kFirstCvWarp + kCvWarps) * 32;
constexpr int kFullCount = 1 + 2 * kCvGroupWarps;   // the A loads' arrive + the converting group's warps of both CTAs
constexpr int kMaxItems = 4;
constexpr int kLutFloats = 16 + kMaxItems * 256 + kMaxItems;   // code, code2 per weight, offset per weight
constexpr int kLutBytes = (kLutFloats * 4 + 15) / 16 * 16;
constexpr int kRawStages = 4;             // slots of the raw ring
constexpr int kOutRow = 80;               // bytes per staged output row: 64 + 16 of padding (bank spread)
constexpr int kOutStage = 4 * 32 * kOutRow;   // per epilogue warp 32 rows of 64 bytes
constexpr int kRawBytes = 128 * 32;       // packed bytes of 128 blocks
constexpr int kRawSlot = kRawBytes + 128 * 4;   // + their 128 fp32 scales
constexpr int kStatAhead = 4;             // steps the statistics loads run ahead

template <int ACCS> struct Cfg {
  static constexpr int kStages = ACCS == 1 ? 6 : 4;
  static constexpr int kStageBytes = kSub * (ACCS + 1);
  static constexpr int kBufs = ACCS == 1 ? 2 : 1;       // accumulator sets in TMEM (512 columns)
  static constexpr int kSmem = kStages * kStageBytes + kRawStages * kRawSlot + kOutStage + kLutBytes + 1024 + 512;
};

struct Maps {
  CUtensorMap a[2];            // forward: x; backward: dy of each weight
  CUtensorMap p[kMaxItems];    // packed codes of each weight as bytes [n_out, k / 2]
};

struct Item {
  const uint8_t* packed;   // [n_out * k / 2]
  const void* absmax;      // nested: uint8 [n_out * k / 64]; else float
  const float* code2;      // [256]   (nested)
  const float* absmax2;    // [...]   (nested)
  const float* offset;     // [1]     (nested)
  const __half* bias;      // forward: [n_out] or null
  void* out;               // forward: fp16 [m, n_out]
  int n_out;
  int first;               // forward: first 256-column tile of this weight; backward: first 64-row block
};

struct Args {
  Item item[kMaxItems];
  int n_items;
  const float* code;       // [16]
  int m, k;
  int nested;
  int shift2;              // log2 of the nested blocksize
  int n_tiles;             // 256-column output tiles (forward: over all items; backward: over k)
  int n_rb;                // contraction blocks of 64 (forward: k / 64; backward: sum n_out / 64)
  int ksplit;
  float* acc;              // fp32 [m, ld_acc]: partial sums are added here when set
  int ld_acc;
  void* out;               // backward direct mode: dx [m, k]
  int out_f32;             // backward direct mode: dx dtype
  int* status;
};

struct Unit {
  int nt, m0, accs, kb_begin, kb_end;
};

template <int ACCS>
__device__ __forceinline__ int unit_count(const Args& a) {
  const int rows = 256 * ACCS;
  const int m_full = a.m / rows;
  const int tail = a.m - m_full * rows;
  return a.n_tiles * a.ksplit * (m_full + (tail > 0 ? 1 : 0));
}

// Units with all accumulators in use come first, the tail units (fewer rows) last, so that the
// round-robin over CTA pairs ends with the cheap ones.
template <int ACCS>
__device__ __forceinline__ Unit decode_unit(const Args& a, int u) {
  const int rows = 256 * ACCS;
  const int m_full = a.m / rows;
  const int n_full = a.n_tiles * a.ksplit * m_full;
  Unit t;
  int ks;
  if (u < n_full) {
    ks = u % a.ksplit;
    const int r = u / a.ksplit;
    t.nt = r / m_full;
    t.m0 = (r % m_full) * rows;
    t.accs = ACCS;
  } else {
    const int v = u - n_full;
    ks = v % a.ksplit;
    t.nt = v / a.ksplit;
    t.m0 = m_full * rows;
    t.accs = (a.m - t.m0 + 255) / 256;
  }
  t.kb_begin = (int)(((long long)a.n_rb * ks) / a.ksplit);
  t.kb_end = (int)(((long long)a.n_rb * (ks + 1)) / a.ksplit);
  return t;
}

__device__ __forceinline__ int item_of(const Args& a, int index) {
  int i = 0;
#pragma unroll
  for (int j = 1; j < kMaxItems; ++j)
    if (j < a.n_items && index >= a.item[j].first) i = j;
  return i;
}

struct Smem {
  uint8_t* tiles;
  uint8_t* raw;          // [kRawStages][kRawSlot]
  uint8_t* out_stage;    // [4 epilogue warps][32][kOutRow]
  float* lut;            // [16] code, [items][256] code2, [items] offset
  uint64_t* full;        // [stages] (leader)
  uint64_t* empty;       // [stages]
  uint64_t* raw_full;    // [kRawStages]
  uint64_t* raw_empty;   // [kRawStages]
  uint64_t* acc_full;    // [2]
  uint64_t* acc_empty;   // [2] (leader)
  uint32_t* tmem_base;
  int* abort_flag;
};

template <int ACCS>
__device__ __forceinline__ Smem carve(uint8_t* raw) {
  using C = Cfg<ACCS>;
  Smem s;
  const uintptr_t base = (reinterpret_cast<uintptr_t>(raw) + 1023u) & ~static_cast<uintptr_t>(1023u);
  s.tiles = reinterpret_cast<uint8_t*>(base);
  s.raw = s.tiles + C::kStages * C::kStageBytes;          // 1024-byte aligned, slots 128-byte aligned
  s.out_stage = s.raw + kRawStages * kRawSlot;
  s.lut = reinterpret_cast<float*>(s.out_stage + kOutStage);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s.lut) + kLutBytes);
  s.full = bars;
  s.empty = bars + C::kStages;
  s.raw_full = bars + 2 * C::kStages;
  s.raw_empty = s.raw_full + kRawStages;
  s.acc_full = s.raw_empty + kRawStages;
  s.acc_empty = s.acc_full + 2;
  s.tmem_base = reinterpret_cast<uint32_t*>(s.acc_empty + 2);
  s.abort_flag = reinterpret_cast<int*>(s.tmem_base + 1);
  return s;
}

struct Pipe {
  int stage = 0;
  uint32_t phase = 0;
  template <int STAGES>
  __device__ __forceinline__ void advance() {
    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
  }
};

// The walk of one CTA over its (unit, contraction block) steps. Every role walks the same list.
template <int ACCS>
struct Walk {
  int unit, kb;
  Unit u;
  __device__ __forceinline__ void start(const Args& a, int pair, int n_units) {
    unit = pair;
    if (unit < n_units) { u = decode_unit<ACCS>(a, unit); kb = u.kb_begin; }
  }
  __device__ __forceinline__ bool valid(int n_units) const { return unit < n_units; }
  __device__ __forceinline__ void next(const Args& a, int n_pairs, int n_units) {
    if (++kb >= u.kb_end) {
      unit += n_pairs;
      if (unit < n_units) { u = decode_unit<ACCS>(a, unit); kb = u.kb_begin; }
    }
  }
};

// Which weight, which of its rows and which of its 64-element blocks the 128 block rows of a step
// start at. Block row b of the step is
//   forward : weight row n0 + b, block kb                      (b = 0..127)
//   backward: weight row n0 + (b & 63), block cb0 + (b >> 6)
struct StepSrc {
  int item, n0, c0;
};

template <bool BWD>
__device__ __forceinline__ StepSrc step_src(const Args& a, const Unit& u, int kb, uint32_t rank) {
  StepSrc r;
  if (!BWD) {
    r.item = item_of(a, u.nt);
    r.n0 = (u.nt - a.item[r.item].first) * kBN + (int)rank * (kBN / 2);
    r.c0 = kb;
  } else {
    r.item = item_of(a, kb);
    r.n0 = (kb - a.item[r.item].first) * kBK;
    r.c0 = u.nt * (kBN / 64) + (int)rank * 2;
  }
  return r;
}

struct Stat {
  uint32_t q8;   // nested: the block's 8-bit absmax code
  float a;       // nested: absmax2 of the block's group; else the block's fp32 absmax
};

template <bool BWD>
__device__ __forceinline__ void load_stats(const Args& a, const StepSrc& src, int lane, Stat (&st)[4]) {
  const Item& w = a.item[src.item];
  const int kblocks = a.k >> 6;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int b = lane + 32 * e;
    int n, c;
    if (!BWD) { n = src.n0 + b; c = src.c0; }
    else { n = src.n0 + (b & 63); c = src.c0 + (b >> 6); }
    n = n < w.n_out ? n : w.n_out - 1;
    c = c < kblocks ? c : kblocks - 1;
    const long long blk = (long long)n * kblocks + c;
    if (a.nested) {
      st[e].q8 = __ldg(reinterpret_cast<const uint8_t*>(w.absmax) + blk);
      st[e].a = __ldg(w.absmax2 + (blk >> a.shift2));
    } else {
      st[e].q8 = 0;
      st[e].a = __ldg(reinterpret_cast<const float*>(w.absmax) + blk);
    }
  }
}

// prmt.b32 in its generic form: result byte i is byte (sel nibble i & 7) of {a, b}, or, when bit 3 of
// the nibble is set, that byte's sign bit replicated over the byte.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ void red_add_v4(float* addr, float x, float y, float z, float w) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x), "f"(y), "f"(z), "f"(w)
               : "memory");
}

template <int ACCS, bool BWD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
nf4_gemm_kernel(const __grid_constant__ Maps maps, const __grid_constant__ Args a) {
  using C = Cfg<ACCS>;
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve<ACCS>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&maps.a[0]);
    if (BWD && a.n_items > 1) prefetch_tensormap(&maps.a[1]);
    for (int i = 0; i < a.n_items; ++i) prefetch_tensormap(&maps.p[i]);
    for (int i = 0; i < C::kStages; ++i) { mbar_init(&s.full[i], kFullCount); mbar_init(&s.empty[i], 1); }
    for (int i = 0; i < kRawStages; ++i) { mbar_init(&s.raw_full[i], 2); mbar_init(&s.raw_empty[i], kCvGroupWarps); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s.acc_full[i], 1); mbar_init(&s.acc_empty[i], 8); }
    *s.abort_flag = *reinterpret_cast<const volatile int*>(a.status) != 0;
    fence_barrier_init();
  }
  if (warp >= kFirstCvWarp) {
    const int t = threadIdx.x - kFirstCvWarp * 32;
    if (t < 16) s.lut[t] = a.code[t];
    if (a.nested) {
      for (int i = 0; i < a.n_items; ++i)
        for (int e = t; e < 256; e += kCvWarps * 32) s.lut[16 + i * 256 + e] = a.item[i].code2[e];
      if (t < a.n_items) s.lut[16 + kMaxItems * 256 + t] = a.item[t].offset[0];
    }
  }
  __syncthreads();
  cluster_sync_all();
  const bool run = ld_shared_cluster_s32(mapa_u32(smem_u32(s.abort_flag), 0)) == 0;
  cluster_sync_all();
  if (!run) return;
  if (warp == 0 && lane == 0) *s.abort_flag = 0;
  if (warp == 1) {
    tmem_alloc_pair(s.tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *s.tmem_base;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int n_units = unit_count<ACCS>(a);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA: the A tiles
    if (lane == 0) {
      Pipe p;
      bool ok = true;
      for (int unit = pair; unit < n_units && ok; unit += n_pairs) {
        const Unit u = decode_unit<ACCS>(a, unit);
        for (int kb = u.kb_begin; kb < u.kb_end; ++kb) {
          ok = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 31);
          if (!ok) break;
          uint8_t* st = s.tiles + p.stage * C::kStageBytes;
          const uint32_t full_leader = mapa_u32(smem_u32(&s.full[p.stage]), 0);
          if (rank == 0) mbar_expect_tx(&s.full[p.stage], 2 * u.accs * kSub);
          const CUtensorMap* map = &maps.a[0];
          int c0 = kb * kBK;
          if (BWD) {
            const int it = item_of(a, kb);
            map = &maps.a[it];
            c0 = (kb - a.item[it].first) * kBK;
          }
          for (int acc = 0; acc < u.accs; ++acc)
            tma_load_2d_pair(st + acc * kSub, map, c0, u.m0 + acc * 256 + (int)rank * kBM, full_leader);
          p.advance<C::kStages>();
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue (leader CTA)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * kBM, kBN, kFmtF16, kFmtF16, false, BWD);
      Pipe p;
      bool ok = true;
      int it = 0;
      for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++it) {
        const Unit u = decode_unit<ACCS>(a, unit);
        const int ab = it % C::kBufs;
        const uint32_t acc_phase = (it / C::kBufs) & 1u;
        ok = mbar_wait(&s.acc_empty[ab], acc_phase ^ 1u, s.abort_flag, a.status, 32);
        if (!ok) break;
        tc_fence_after_sync();
        for (int kb = u.kb_begin; kb < u.kb_end; ++kb) {
          ok = mbar_wait(&s.full[p.stage], p.phase, s.abort_flag, a.status, 33);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t st = smem_u32(s.tiles + p.stage * C::kStageBytes);
          const uint32_t b_addr = st + ACCS * kSub;
          // forward: B is K-major (rows = output columns, 128-byte rows of 64 k);
          // backward: B is MN-major: two 64-column boxes 8 KB apart, 8-row groups 1 KB apart,
          // one MMA consumes 16 contraction rows = 2 KB
          const uint64_t db = BWD ? make_smem_desc(b_addr, kBK * 128, 1024) : make_smem_desc(b_addr, 16, 1024);
          for (int acc = 0; acc < u.accs; ++acc) {
            const uint64_t da = make_smem_desc(st + acc * kSub, 16, 1024);
            const uint32_t d_tmem = tmem + (ab * ACCS + acc) * kBN;
#pragma unroll
            for (int k4 = 0; k4 < kBK / 16; ++k4)
              mma_f16_ss_pair(d_tmem, da + k4 * 2, db + (BWD ? k4 * (2048 >> 4) : k4 * 2), idesc,
                              (kb != u.kb_begin) || k4 != 0);
          }
          tc_commit_pair(&s.empty[p.stage], 3);
          p.advance<C::kStages>();
        }
        if (ok) tc_commit_pair(&s.acc_full[ab], 3);
      }
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------------- TMA: the packed codes
    if (lane == 0) {
      Walk<ACCS> w;
      w.start(a, pair, n_units);
      int r = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (w.valid(n_units) && ok) {
        ok = mbar_wait(&s.raw_empty[r], phase ^ 1u, s.abort_flag, a.status, 36);
        if (!ok) break;
        const StepSrc src = step_src<BWD>(a, w.u, w.kb, rank);
        uint8_t* dst = s.raw + r * kRawSlot;
        mbar_expect_tx(&s.raw_full[r], kRawBytes);
        // two boxes of 64 block rows x 32 bytes; coordinates (byte column, weight row)
        if (!BWD) {
          tma_load_2d(dst, &maps.p[src.item], src.c0 * 32, src.n0, &s.raw_full[r]);
          tma_load_2d(dst + 2048, &maps.p[src.item], src.c0 * 32, src.n0 + 64, &s.raw_full[r]);
        } else {
          tma_load_2d(dst, &maps.p[src.item], src.c0 * 32, src.n0, &s.raw_full[r]);
          tma_load_2d(dst + 2048, &maps.p[src.item], (src.c0 + 1) * 32, src.n0, &s.raw_full[r]);
        }
        w.next(a, n_pairs, n_units);
        if (++r == kRawStages) { r = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 3) {
    // ---------------------------------------------------------------- block scales
    Walk<ACCS> cur, ahead;
    cur.start(a, pair, n_units);
    ahead.start(a, pair, n_units);
    Stat ring[kStatAhead][4];
    int ring_item[kStatAhead];
#pragma unroll
    for (int i = 0; i < kStatAhead; ++i) {
      if (ahead.valid(n_units)) {
        const StepSrc src = step_src<BWD>(a, ahead.u, ahead.kb, rank);
        load_stats<BWD>(a, src, lane, ring[i]);
        ring_item[i] = src.item;
        ahead.next(a, n_pairs, n_units);
      }
    }
    int r = 0;
    uint32_t phase = 0;
    bool ok = true;
    while (cur.valid(n_units) && ok) {
#pragma unroll
      for (int i = 0; i < kStatAhead; ++i) {
        if (!cur.valid(n_units) || !ok) break;
        int won = 1;
        if (lane == 0) won = mbar_wait(&s.raw_empty[r], phase ^ 1u, s.abort_flag, a.status, 37) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, won, 0) != 0;
        if (!ok) break;
        float* scales = reinterpret_cast<float*>(s.raw + r * kRawSlot + kRawBytes);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float scale = ring[i][e].a;
          if (a.nested)
            scale = __fadd_rn(__fmul_rn(s.lut[16 + ring_item[i] * 256 + ring[i][e].q8], ring[i][e].a),
                              s.lut[16 + kMaxItems * 256 + ring_item[i]]);
          scales[lane + 32 * e] = scale;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.raw_full[r]);
        if (ahead.valid(n_units)) {
          const StepSrc src = step_src<BWD>(a, ahead.u, ahead.kb, rank);
          load_stats<BWD>(a, src, lane, ring[i]);
          ring_item[i] = src.item;
          ahead.next(a, n_pairs, n_units);
        }
        cur.next(a, n_pairs, n_units);
        if (++r == kRawStages) { r = 0; phase ^= 1u; }
      }
    }
  } else if (warp < kFirstCvWarp) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    bool ok = true;
    int it = 0;
    for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++it) {
      const Unit u = decode_unit<ACCS>(a, unit);
      const int ab = it % C::kBufs;
      const uint32_t acc_phase = (it / C::kBufs) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&s.acc_full[ab], acc_phase, s.abort_flag, a.status, 34));
      if (!ok) break;
      tc_fence_after_sync();
      // where this tile's columns go
      int ld, col_base, n_cols;
      const __half* bias = nullptr;
      void* direct = nullptr;
      int direct_f32 = 0;
      if (!BWD) {
        const Item& w = a.item[item_of(a, u.nt)];
        col_base = (u.nt - w.first) * kBN;
        n_cols = w.n_out;
        ld = w.n_out;
        bias = w.bias;
        direct = w.out;
      } else {
        col_base = u.nt * kBN;
        n_cols = a.k;
        ld = a.k;
        direct = a.out;
        direct_f32 = a.out_f32;
      }
      // A thread holds 32 consecutive columns of one row. Written from there, every store
      // instruction of a warp would touch 32 different lines; the values go through a small
      // staging area instead (64 bytes per row and pass, rows 80 bytes apart), from which four
      // lanes write the 64 bytes of one row, so that an instruction covers eight rows.
      uint8_t* stage_out = s.out_stage + (warp - 4) * (32 * kOutRow);
      const int part = lane & 3, sub = lane >> 2;
      for (int acc = 0; acc < u.accs; ++acc) {
        const int row_base = u.m0 + acc * 256 + (int)rank * kBM + q * 32;
        const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + (ab * ACCS + acc) * kBN;
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
         {
          if (col_base + c * 32 >= n_cols) break;     // uniform over the warp
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait_on(r);
          const int col0 = col_base + c * 32;
          if (a.acc == nullptr && !direct_f32) {
            // fp16 result (+ bias): one pass of 32 columns
            uint32_t h[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              float x0 = __uint_as_float(r[2 * e]), x1 = __uint_as_float(r[2 * e + 1]);
              if (bias && col0 + 2 * e < n_cols) {
                x0 += __half2float(bias[col0 + 2 * e]);
                x1 += __half2float(bias[col0 + 2 * e + 1]);
              }
              __half2 pk = __floats2half2_rn(x0, x1);
              h[e] = *reinterpret_cast<uint32_t*>(&pk);
            }
            __syncwarp();
#pragma unroll
            for (int v = 0; v < 4; ++v)
              *reinterpret_cast<uint4*>(stage_out + lane * kOutRow + v * 16) =
                  make_uint4(h[4 * v], h[4 * v + 1], h[4 * v + 2], h[4 * v + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rr = sub + 8 * i;
              const int row = row_base + rr;
              const uint4 v = *reinterpret_cast<const uint4*>(stage_out + rr * kOutRow + part * 16);
              if (row < a.m && col0 + part * 8 < n_cols)
                *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(direct) + (size_t)row * ld + col0 + part * 8) = v;
            }
          } else {
            // fp32 result or partial sums of a contraction split: two passes of 16 columns
#pragma unroll
            for (int hpass = 0; hpass < 2; ++hpass) {
              __syncwarp();
#pragma unroll
              for (int v = 0; v < 4; ++v)
                *reinterpret_cast<uint4*>(stage_out + lane * kOutRow + v * 16) =
                    make_uint4(r[hpass * 16 + 4 * v], r[hpass * 16 + 4 * v + 1], r[hpass * 16 + 4 * v + 2],
                               r[hpass * 16 + 4 * v + 3]);
              __syncwarp();
              const int colh = col0 + hpass * 16 + part * 4;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = sub + 8 * i;
                const int row = row_base + rr;
                const float4 v = *reinterpret_cast<const float4*>(stage_out + rr * kOutRow + part * 16);
                if (row < a.m && colh < n_cols) {
                  if (a.acc != nullptr) red_add_v4(a.acc + (size_t)row * a.ld_acc + colh, v.x, v.y, v.z, v.w);
                  else *reinterpret_cast<float4*>(reinterpret_cast<float*>(direct) + (size_t)row * ld + colh) = v;
                }
              }
            }
          }
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
  } else {
    // ---------------------------------------------------------------- conversion
    // Group g converts the steps g, g + kCvGroups, ... of this CTA's walk: the fixed cost of a step
    // (two barrier waits, the proxy fence, two arrivals: several hundred cycles of latency) is
    // paid per group, so the groups' steps overlap.
    const int group = (warp - kFirstCvWarp) / kCvGroupWarps;
    const int b0 = (warp - kFirstCvWarp) % kCvGroupWarps * 32 + lane;   // first block row of the step
    constexpr int kPerThread = 128 / (kCvGroupWarps * 32);               // block rows per thread
    Walk<ACCS> w;
    w.start(a, pair, n_units);
    int stage = 0, r = 0;
    uint32_t phase = 0, raw_phase = 0;
    auto skip = [&](int n) {
      for (int i = 0; i < n && w.valid(n_units); ++i) {
        w.next(a, n_pairs, n_units);
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        if (++r == kRawStages) { r = 0; raw_phase ^= 1u; }
      }
    };
    skip(group);
    float code[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) code[i] = s.lut[i];
    bool ok = true;
    while (w.valid(n_units) && ok) {
      int won = 1;
      if (lane == 0) won = mbar_wait(&s.raw_full[r], raw_phase, s.abort_flag, a.status, 38) ? 1 : 0;
      else if (lane == 1) won = mbar_wait(&s.empty[stage], phase ^ 1u, s.abort_flag, a.status, 35) ? 1 : 0;
      ok = __all_sync(0xffffffffu, won != 0);
      if (!ok) break;
      const uint8_t* raw = s.raw + r * kRawSlot;
#pragma unroll 1
      for (int bi = 0; bi < kPerThread; ++bi) {
      const int b = b0 + bi * (kCvGroupWarps * 32);
      const int row_swz = b & 7;
      const uint4 c0 = *reinterpret_cast<const uint4*>(raw + b * 32);
      const uint4 c1 = *reinterpret_cast<const uint4*>(raw + b * 32 + 16);
      const float scale = *reinterpret_cast<const float*>(raw + kRawBytes + b * 4);
      uint8_t* row_base = s.tiles + stage * C::kStageBytes + ACCS * kSub + b * 128;
      const uint32_t wds[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      // The block's 16 possible values, fp16_rn(code[i] * scale), once per block ...
      uint32_t tab[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        __half2 pk = __floats2half2_rn(__fmul_rn(code[2 * j], scale), __fmul_rn(code[2 * j + 1], scale));
        tab[j] = *reinterpret_cast<uint32_t*>(&pk);
      }
      // ... as byte planes: lo[q] / hi[q] hold the low / high bytes of entries 4q .. 4q+3
      uint32_t lo[4], hi[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        lo[q] = prmt(tab[2 * q], tab[2 * q + 1], 0x6420);
        hi[q] = prmt(tab[2 * q], tab[2 * q + 1], 0x7531);
      }
      // Four nibbles at a time select their bytes from the planes with byte permutes (a 4-bit
      // index is a 3-bit select in either half of a plane plus a mask on its top bit): no
      // shared-memory look-ups, which the tensor core's operand reads compete with.
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        uint32_t h[4];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          // two packed bytes: nibbles n0..n3 = elements 1, 0, 3, 2 of the four
          const uint32_t two = c == 0 ? wds[k] : wds[k] >> 16;
          const uint32_t sel = two & 0x7777u;
          const uint32_t top = prmt(two, two << 4, 0x9D8C);   // 0xFF where the nibble is >= 8
          const uint32_t xl = prmt(lo[0], lo[1], sel), xh = prmt(lo[2], lo[3], sel);
          const uint32_t yl = prmt(hi[0], hi[1], sel), yh = prmt(hi[2], hi[3], sel);
          const uint32_t x = (xl & ~top) | (xh & top);   // low bytes of elements 1, 0, 3, 2
          const uint32_t y = (yl & ~top) | (yh & top);   // high bytes
          h[2 * c] = prmt(x, y, 0x4051);           // elements 0, 1
          h[2 * c + 1] = prmt(x, y, 0x6273);       // elements 2, 3
        }
        *reinterpret_cast<uint4*>(row_base + ((k ^ row_swz) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
      }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&s.full[stage]);
        else mbar_arrive_remote(mapa_u32(smem_u32(&s.full[stage]), 0));
      } else if (lane == 1) {
        mbar_arrive(&s.raw_empty[r]);
      }
      skip(kCvGroups);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*s.abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem, 512);
  }
}

// out = fp16/fp32(acc (+ bias)): the last step of a contraction split.
__global__ void nf4_gemm_finalize_kernel(const float* __restrict__ acc, void* __restrict__ out,
                                         const __half* __restrict__ bias, int64_t m, int n, int out_f32) {
  const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one 8-column group
  const int groups = n >> 3;
  if (v >= m * groups) return;
  const int64_t row = v / groups;
  const int col = (int)(v % groups) << 3;
  float x[8];
  load8(acc, row * n + col, SOUP_F32, x);
  if (bias) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += __half2float(bias[col + j]);
  }
  store8(out, row * n + col, out_f32 ? SOUP_F32 : SOUP_F16, x);
}

bool g_attr[64][4] = {};

template <int ACCS, bool BWD>
int set_attr(int dev, int slot) {
  if (g_attr[dev][slot]) return 0;
  if (cudaFuncSetAttribute(nf4_gemm_kernel<ACCS, BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           Cfg<ACCS>::kSmem) != cudaSuccess)
    return -1;
  g_attr[dev][slot] = true;
  return 0;
}

// Accumulators per unit and contraction split that minimise the estimated makespan over `pairs`
// CTA pairs, from what was measured on B200 with all SMs busy: a pipeline step takes the longer of
// the tensor core's ~512 cycles per accumulator and the conversion's ~1400 cycles for a CTA's 128
// blocks; with two accumulators the epilogue (~8000 cycles per accumulator) is not overlapped with
// the next unit's MMAs (one accumulator set fills tensor memory), with one it is. A split needs
// the fp32 buffer.
void pick_shape(int m, int n_tiles, int n_rb, int pairs, bool can_split, int* accs_out, int* ksplit_out) {
  double best = 1e30;
  *accs_out = 1;
  *ksplit_out = 1;
  for (int accs = 1; accs <= 2; ++accs) {
    const int rows = 256 * accs;
    const int m_units = (m + rows - 1) / rows;
    for (int ks = 1; ks <= 8; ++ks) {
      if (ks > 1 && (!can_split || n_rb / ks < 12)) break;
      const long units = (long)n_tiles * m_units * ks;
      const long waves = (units + pairs - 1) / pairs;
      const double step = accs * 512.0 > 1400.0 ? accs * 512.0 : 1400.0;
      const double unit_cost = ((n_rb + ks - 1) / ks) * step + (accs == 2 ? 16000.0 : 1000.0) + 2000.0;
      const double span = waves * unit_cost;
      if (span < best * 0.97) { best = span; *accs_out = accs; *ksplit_out = ks; }
    }
  }
}

int fill_items(const soup_nf4_gemm_item* items, int n_items, bool bwd, int64_t k, Args* a) {
  int index = 0;
  for (int i = 0; i < n_items; ++i) {
    const soup_nf4_gemm_item& src = items[i];
    if (!src.packed || !src.absmax || src.n_out <= 0) return -1;
    if (src.n_out > INT32_MAX / 2) return -2;
    Item& d = a->item[i];
    d.packed = reinterpret_cast<const uint8_t*>(src.packed);
    d.absmax = src.absmax;
    d.code2 = src.code2;
    d.absmax2 = src.absmax2;
    d.offset = src.offset;
    d.bias = reinterpret_cast<const __half*>(src.bias);
    d.out = src.out;
    d.n_out = (int)src.n_out;
    d.first = index;
    index += bwd ? (int)(src.n_out / kBK) : (int)((src.n_out + kBN - 1) / kBN);
  }
  a->n_items = n_items;
  return index;
}

template <bool BWD>
int launch(const Maps& maps, const Args& a, int accs, int pairs, cudaStream_t s) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  const int rows = 256 * accs;
  const long units = (long)a.n_tiles * a.ksplit * ((a.m + rows - 1) / rows);
  const unsigned grid = 2u * (unsigned)(units < pairs ? units : pairs);
  if (accs == 1) {
    if (set_attr<1, BWD>(dev, BWD ? 1 : 0)) return -1;
    nf4_gemm_kernel<1, BWD><<<grid, kThreads, Cfg<1>::kSmem, s>>>(maps, a);
  } else {
    if (set_attr<2, BWD>(dev, BWD ? 3 : 2)) return -1;
    nf4_gemm_kernel<2, BWD><<<grid, kThreads, Cfg<2>::kSmem, s>>>(maps, a);
  }
  return 0;
}

// The packed codes of every weight as a byte matrix [n_out, k / 2], fetched in boxes of 64 rows x
// 32 bytes (64 NF4 blocks).
int encode_packed_maps(const soup_nf4_gemm_item* items, int n_items, int64_t k, Maps* maps) {
  for (int i = 0; i < kMaxItems; ++i) {
    const soup_nf4_gemm_item& it = items[i < n_items ? i : 0];
    if (umma::encode_map_2d_bytes(&maps->p[i], it.packed, (uint64_t)it.n_out, (uint64_t)(k / 2),
                                  (uint64_t)(k / 2), 64, 32))
      return -1;
  }
  return 0;
}

int common_checks(const char* who, const soup_nf4_gemm_item* items, int n_items, const float* code,
                  int64_t m, int64_t k, int nested, int blocksize, int blocksize2) {
  if (!items || n_items < 1 || n_items > kMaxItems) SOUP_FAIL(SOUP_ERR_ARG, "%s: 1 to %d weights per call", who, kMaxItems);
  if (!code || m < 0 || k <= 0) SOUP_FAIL(SOUP_ERR_ARG, "%s: bad argument", who);
  if (blocksize != 64) SOUP_FAIL(SOUP_ERR_ARG, "%s: the NF4 blocksize must be 64 (one block per 128-byte tile row)", who);
  if (k % 64 != 0) SOUP_FAIL(SOUP_ERR_ARG, "%s: in_features must be a multiple of 64", who);
  if (nested && (blocksize2 <= 0 || (blocksize2 & (blocksize2 - 1)) != 0))
    SOUP_FAIL(SOUP_ERR_ARG, "%s: the nested blocksize must be a power of two", who);
  if (m > INT32_MAX / 2 || k > INT32_MAX / 2) SOUP_FAIL(SOUP_ERR_ARG, "%s: shape exceeds 32-bit tile coordinates", who);
  for (int i = 0; i < n_items; ++i) {
    if (nested && (!items[i].code2 || !items[i].absmax2 || !items[i].offset))
      SOUP_FAIL(SOUP_ERR_ARG, "%s: nested statistics missing for weight %d", who, i);
    if (!aligned16(items[i].packed)) SOUP_FAIL(SOUP_ERR_ARG, "%s: packed weights must be 16-byte aligned", who);
  }
  int major = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) SOUP_FAIL(SOUP_ERR_DEVICE, "%s: needs a compute capability 10.x device", who);
  return SOUP_OK;
}

int ilog2(int v) {
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

}  // namespace
}  // namespace soup

extern "C" int64_t soup_nf4_gemm_workspace_bytes(int64_t m, int64_t cols) {
  return m <= 0 || cols <= 0 ? 0 : m * cols * (int64_t)sizeof(float);
}

extern "C" int soup_nf4_linear_fwd(const void* x, const soup_nf4_gemm_item* items, int n_items,
                                   const float* code, int64_t m, int64_t k, int nested, int blocksize,
                                   int blocksize2, void* workspace, int64_t workspace_bytes,
                                   void* stream) {
  using namespace soup;
  const int rc = common_checks("nf4_linear_fwd", items, n_items, code, m, k, nested, blocksize, blocksize2);
  if (rc != SOUP_OK) return rc;
  if (m == 0) return SOUP_OK;
  if (!x || !aligned16(x)) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_fwd: x must be a 16-byte aligned device pointer");
  for (int i = 0; i < n_items; ++i) {
    if (!items[i].out || !aligned16(items[i].out)) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_fwd: output %d missing or unaligned", i);
    if (items[i].n_out % 8 != 0) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_fwd: out_features must be a multiple of 8");
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  Args a = {};
  const int n_tiles = fill_items(items, n_items, false, k, &a);
  if (n_tiles < 0) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_fwd: bad weight description");
  a.code = code;
  a.m = (int)m;
  a.k = (int)k;
  a.nested = nested != 0;
  a.shift2 = nested ? ilog2(blocksize2) : 0;
  a.n_tiles = n_tiles;
  a.n_rb = (int)(k / kBK);
  a.status = rowpipe::status_word();
  if (!a.status) SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_fwd: no status word on this device");
  const int pairs = sm_count() / 2;
  if (pairs < 1) SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_fwd: needs at least two SMs");
  // a contraction split needs the fp32 buffer and a single weight (one buffer, one finalize pass)
  const int64_t need = m * items[0].n_out * (int64_t)sizeof(float);
  const bool can_split = n_items == 1 && workspace && workspace_bytes >= need && aligned16(workspace);
  int accs = 1, ksplit = 1;
  pick_shape((int)m, n_tiles, a.n_rb, pairs, can_split, &accs, &ksplit);
  a.ksplit = ksplit;
  if (ksplit > 1) {
    a.acc = reinterpret_cast<float*>(workspace);
    a.ld_acc = (int)items[0].n_out;
    if (cudaMemsetAsync(workspace, 0, (size_t)need, s) != cudaSuccess)
      SOUP_FAIL(SOUP_ERR_LAUNCH, "nf4_linear_fwd: %s", cudaGetErrorString(cudaGetLastError()));
  }
  Maps maps;
  if (umma::encode_map_2d_16bit(&maps.a[0], x, (uint64_t)m, (uint64_t)k, (uint64_t)k, kBM, kBK, false) ||
      encode_packed_maps(items, n_items, k, &maps))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_fwd: cuTensorMapEncodeTiled failed");
  maps.a[1] = maps.a[0];
  if (launch<false>(maps, a, accs, pairs, s))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_fwd: cannot raise the shared-memory limit");
  SOUP_CHECK_LAUNCH("nf4_linear_fwd");
  if (ksplit > 1) {
    const int64_t groups = m * (items[0].n_out / 8);
    nf4_gemm_finalize_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>(
        a.acc, items[0].out, reinterpret_cast<const __half*>(items[0].bias), m, (int)items[0].n_out, 0);
    SOUP_CHECK_LAUNCH("nf4_gemm_finalize");
  }
  return SOUP_OK;
}

extern "C" int soup_nf4_linear_dx(const soup_nf4_gemm_item* items, int n_items, const float* code,
                                  void* dx, int dx_dtype, int64_t m, int64_t k, int nested,
                                  int blocksize, int blocksize2, void* workspace,
                                  int64_t workspace_bytes, void* stream) {
  using namespace soup;
  const int rc = common_checks("nf4_linear_dx", items, n_items, code, m, k, nested, blocksize, blocksize2);
  if (rc != SOUP_OK) return rc;
  if (m == 0) return SOUP_OK;
  if (n_items > 2) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_dx: at most two weights per call");
  if (!dx || !aligned16(dx)) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_dx: dx must be a 16-byte aligned device pointer");
  if (dx_dtype != SOUP_F16 && dx_dtype != SOUP_F32) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_dx: dx must be fp16 or fp32");
  if (k % 8 != 0) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_dx: in_features must be a multiple of 8");
  for (int i = 0; i < n_items; ++i) {
    if (!items[i].dy || !aligned16(items[i].dy)) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_dx: dy %d missing or unaligned", i);
    if (items[i].n_out % 64 != 0) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_dx: out_features must be a multiple of 64");
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  Args a = {};
  const int n_rb = fill_items(items, n_items, true, k, &a);
  if (n_rb < 0) SOUP_FAIL(SOUP_ERR_ARG, "nf4_linear_dx: bad weight description");
  a.code = code;
  a.m = (int)m;
  a.k = (int)k;
  a.nested = nested != 0;
  a.shift2 = nested ? ilog2(blocksize2) : 0;
  a.n_tiles = (int)((k + kBN - 1) / kBN);
  a.n_rb = n_rb;
  a.status = rowpipe::status_word();
  if (!a.status) SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: no status word on this device");
  const int pairs = sm_count() / 2;
  if (pairs < 1) SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: needs at least two SMs");
  // partial sums go to dx itself when it is fp32, else to the caller's fp32 buffer
  const int64_t need = m * k * (int64_t)sizeof(float);
  float* acc = dx_dtype == SOUP_F32 ? reinterpret_cast<float*>(dx)
               : (workspace && workspace_bytes >= need && aligned16(workspace) ? reinterpret_cast<float*>(workspace) : nullptr);
  int accs = 1, ksplit = 1;
  pick_shape((int)m, a.n_tiles, a.n_rb, pairs, acc != nullptr, &accs, &ksplit);
  a.ksplit = ksplit;
  a.out = dx;
  a.out_f32 = dx_dtype == SOUP_F32;
  if (ksplit > 1) {
    a.acc = acc;
    a.ld_acc = (int)k;
    if (cudaMemsetAsync(acc, 0, (size_t)need, s) != cudaSuccess)
      SOUP_FAIL(SOUP_ERR_LAUNCH, "nf4_linear_dx: %s", cudaGetErrorString(cudaGetLastError()));
  }
  Maps maps;
  if (umma::encode_map_2d_16bit(&maps.a[0], items[0].dy, (uint64_t)m, (uint64_t)items[0].n_out,
                                (uint64_t)items[0].n_out, kBM, kBK, false) ||
      encode_packed_maps(items, n_items, k, &maps))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: cuTensorMapEncodeTiled failed");
  maps.a[1] = maps.a[0];
  if (n_items > 1 &&
      umma::encode_map_2d_16bit(&maps.a[1], items[1].dy, (uint64_t)m, (uint64_t)items[1].n_out,
                                (uint64_t)items[1].n_out, kBM, kBK, false))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: cuTensorMapEncodeTiled failed");
  if (launch<true>(maps, a, accs, pairs, s))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: cannot raise the shared-memory limit");
  SOUP_CHECK_LAUNCH("nf4_linear_dx");
  if (ksplit > 1 && dx_dtype != SOUP_F32) {
    const int64_t groups = m * (k / 8);
    nf4_gemm_finalize_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>(acc, dx, nullptr, m, (int)k, 0);
    SOUP_CHECK_LAUNCH("nf4_gemm_finalize");
  }
  return SOUP_OK;
}
