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
// the weight tile. Warp roles per CTA: warp 0 issues the TMA loads of A, warp 1 the MMAs (leader
// CTA only), warps 2-5 the epilogue, warps 6-13 (256 threads) dequantise.
//
// Dequantisation. One NF4 block of 64 elements along K (32 packed bytes, one absmax) is exactly
// one 128-byte row of the 128-byte-swizzled operand tile in either direction: in the forward
// tile a row is one weight row's 64 k-values, in the backward (MN-major) tile a row is one
// weight row's 64 output columns. A thread owns half a block: it loads 16 packed bytes and the
// block's statistics from global memory two pipeline steps ahead, forms
//   scale = code2[absmax8[b]] * absmax2[b / blocksize2] + offset      (__fmul_rn, __fadd_rn)
//   w     = fp16_rn(code[nibble] * scale)                             (__fmul_rn)
// the same unfused fp32 operations, in the same order, as the stand-alone dequantisation kernel,
// so the operand is bit-identical to dequantize_nf4's output, and writes four 16-byte pieces to
// their swizzled places (piece p of row r at p ^ (r & 7)). A fence makes the writes visible to the
// tensor core's proxy and one lane per warp arrives on the leader CTA's "full" barrier of the
// stage, next to the byte count of the TMA loads.
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
constexpr int kDqWarps = 8;
constexpr int kDqThreads = kDqWarps * 32;
constexpr int kFirstDqWarp = 6;
constexpr int kThreads = (kFirstDqWarp + kDqWarps) * 32;   // 448
constexpr int kFullCount = 1 + 2 * kDqWarps;   // the TMA's arrive + every dequant warp of both CTAs
constexpr int kMaxItems = 4;
constexpr int kStageT = 4 * 32 * 33 * 4;      // per epilogue warp a padded 32 x 32 fp32 block
constexpr int kLutFloats = 16 + kMaxItems * 256 + kMaxItems;   // code, code2 per weight, offset per weight
constexpr int kLutBytes = (kLutFloats * 4 + 15) / 16 * 16;
constexpr int kAhead = 2;                      // pipeline steps the dequant loads run ahead

template <int ACCS> struct Cfg {
  static constexpr int kStages = ACCS == 1 ? 6 : 4;
  static constexpr int kStageBytes = kSub * (ACCS + 1);
  static constexpr int kBufs = ACCS == 1 ? 2 : 1;       // accumulator sets in TMEM (512 columns)
  static constexpr int kSmem = kStages * kStageBytes + kStageT + kLutBytes + 1024 + 256;
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
  float* tpose;
  float* lut;            // [16] code, [items][256] code2, [items] offset
  uint64_t* full;        // [stages] (leader)
  uint64_t* empty;       // [stages]
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
  s.tpose = reinterpret_cast<float*>(s.tiles + C::kStages * C::kStageBytes);
  s.lut = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s.tpose) + kStageT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s.lut) + kLutBytes);
  s.full = bars;
  s.empty = bars + C::kStages;
  s.acc_full = bars + 2 * C::kStages;
  s.acc_empty = bars + 2 * C::kStages + 2;
  s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
  s.abort_flag = reinterpret_cast<int*>(s.tmem_base + 1);
  return s;
}

// try_wait with acquire semantics at cluster scope: the barrier is also completed by arrivals of
// the peer CTA's dequant warps, whose shared-memory writes the waiter's MMAs then read.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) break;
    }
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}

struct Pipe {
  int stage = 0;
  uint32_t phase = 0;
  template <int STAGES>
  __device__ __forceinline__ void advance() {
    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
  }
};

// What a dequant thread fetches ahead for one pipeline step: its 16 packed bytes and the raw
// statistics of their block.
struct Fetch {
  uint4 raw;
  uint32_t q8;     // nested: the block's 8-bit absmax code
  float a;         // nested: absmax2 of the block's group; else the block's fp32 absmax
  int item;        // which weight of the launch (selects its code2 table and offset)
};

// The walk of one CTA over its (unit, contraction block) steps; the dequant warps keep a second
// copy running kAhead steps in front of the one they consume.
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

template <bool BWD>
__device__ __forceinline__ Fetch fetch_step(const Args& a, const Unit& u, int kb, uint32_t rank, int t) {
  // forward: t -> weight row (t >> 1) of this CTA's 128, half-block (t & 1)
  // backward: t -> 64-column box (t >> 7), weight row ((t >> 1) & 63) of the contraction block
  const int half = t & 1;
  const int kblocks = a.k >> 6;
  int it;
  long long blk;
  if (!BWD) {
    it = item_of(a, u.nt);
    const Item& w = a.item[it];
    int n = (u.nt - w.first) * kBN + (int)rank * (kBN / 2) + (t >> 1);
    n = n < w.n_out ? n : w.n_out - 1;
    blk = (long long)n * kblocks + kb;
  } else {
    it = item_of(a, kb);
    const Item& w = a.item[it];
    const int n = (kb - w.first) * kBK + ((t >> 1) & 63);
    int cb = u.nt * (kBN / 64) + (int)rank * 2 + (t >> 7);
    cb = cb < kblocks ? cb : kblocks - 1;
    blk = (long long)n * kblocks + cb;
  }
  const Item& w = a.item[it];
  Fetch f;
  f.raw = __ldg(reinterpret_cast<const uint4*>(w.packed + blk * 32 + half * 16));
  f.item = it;
  if (a.nested) {
    f.q8 = __ldg(reinterpret_cast<const uint8_t*>(w.absmax) + blk);
    f.a = __ldg(w.absmax2 + (blk >> a.shift2));
  } else {
    f.q8 = 0;
    f.a = __ldg(reinterpret_cast<const float*>(w.absmax) + blk);
  }
  return f;
}

// 16 packed bytes -> 32 fp16 values at their swizzled places of one 128-byte tile row.
__device__ __forceinline__ void dequant_store(const Fetch& f, bool nested, const float* lut,
                                              uint8_t* row_base, int row_swz, int half) {
  float scale = f.a;
  if (nested)
    scale = __fadd_rn(__fmul_rn(lut[16 + f.item * 256 + f.q8], f.a), lut[16 + kMaxItems * 256 + f.item]);
  const uint32_t w[4] = {f.raw.x, f.raw.y, f.raw.z, f.raw.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint32_t h[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (w[k] >> (8 * b)) & 0xffu;
      const float hi = __fmul_rn(lut[byte >> 4], scale);
      const float lo = __fmul_rn(lut[byte & 15u], scale);
      __half2 p = __floats2half2_rn(hi, lo);
      h[b] = *reinterpret_cast<uint32_t*>(&p);
    }
    const int piece = (half * 4 + k) ^ row_swz;
    *reinterpret_cast<uint4*>(row_base + piece * 16) = make_uint4(h[0], h[1], h[2], h[3]);
  }
}

template <int ACCS, bool BWD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
nf4_gemm_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                const __grid_constant__ Args a) {
  using C = Cfg<ACCS>;
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve<ACCS>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&map_a0);
    if (BWD) prefetch_tensormap(&map_a1);
    for (int i = 0; i < C::kStages; ++i) { mbar_init(&s.full[i], kFullCount); mbar_init(&s.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s.acc_full[i], 1); mbar_init(&s.acc_empty[i], 8); }
    *s.abort_flag = *reinterpret_cast<const volatile int*>(a.status) != 0;
    fence_barrier_init();
  }
  if (warp >= kFirstDqWarp) {
    const int t = threadIdx.x - kFirstDqWarp * 32;
    if (t < 16) s.lut[t] = a.code[t];
    if (a.nested) {
      for (int i = 0; i < a.n_items; ++i) s.lut[16 + i * 256 + t] = a.item[i].code2[t];
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
          const CUtensorMap* map = &map_a0;
          int c0 = kb * kBK;
          if (BWD) {
            const int it = item_of(a, kb);
            if (it != 0) map = &map_a1;
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
          ok = mbar_wait_cluster(&s.full[p.stage], p.phase, s.abort_flag, a.status, 33);
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
  } else if (warp < kFirstDqWarp) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    float* tpose = s.tpose + (warp - 2) * (32 * 33);
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
      for (int acc = 0; acc < u.accs; ++acc) {
        const int row_base = u.m0 + acc * 256 + (int)rank * kBM + q * 32;
        const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + (ab * ACCS + acc) * kBN;
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          const int col0 = col_base + c * 32;
          if (col0 >= n_cols) break;     // uniform over the warp
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait_on(r);
          if (a.acc != nullptr) {
            // partial sums of a contraction split: transposed through shared memory so that the
            // reductions touch full 128-byte rows
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j) tpose[lane * 33 + j] = __uint_as_float(r[j]);
            __syncwarp();
            const int col = col0 + lane;
            const bool col_ok = col < n_cols;
#pragma unroll 8
            for (int rr = 0; rr < 32; ++rr) {
              const int row = row_base + rr;
              if (col_ok && row < a.m) atomicAdd(a.acc + (size_t)row * a.ld_acc + col, tpose[rr * 33 + lane]);
            }
          } else {
            const int row = row_base + lane;
            if (row < a.m) {
              if (direct_f32) {
                float* o = reinterpret_cast<float*>(direct) + (size_t)row * ld + col0;
#pragma unroll
                for (int v = 0; v < 8; ++v)
                  if (col0 + v * 4 < n_cols)
                    *reinterpret_cast<float4*>(o + v * 4) =
                        make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                    __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
              } else {
                __half* o = reinterpret_cast<__half*>(direct) + (size_t)row * ld + col0;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  if (col0 + v * 8 >= n_cols) break;
                  uint32_t h[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float x0 = __uint_as_float(r[v * 8 + 2 * e]), x1 = __uint_as_float(r[v * 8 + 2 * e + 1]);
                    if (bias) {
                      x0 += __half2float(bias[col0 + v * 8 + 2 * e]);
                      x1 += __half2float(bias[col0 + v * 8 + 2 * e + 1]);
                    }
                    __half2 p = __floats2half2_rn(x0, x1);
                    h[e] = *reinterpret_cast<uint32_t*>(&p);
                  }
                  *reinterpret_cast<uint4*>(o + v * 8) = make_uint4(h[0], h[1], h[2], h[3]);
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
    // ---------------------------------------------------------------- dequantisation
    const int t = threadIdx.x - kFirstDqWarp * 32;
    const int half = t & 1;
    int row_off, row_swz;
    if (!BWD) {
      const int row = t >> 1;
      row_off = row * 128;
      row_swz = row & 7;
    } else {
      const int r = (t >> 1) & 63;
      row_off = (t >> 7) * (kBK * 128) + r * 128;
      row_swz = r & 7;
    }
    Walk<ACCS> cur, ahead;
    cur.start(a, pair, n_units);
    ahead.start(a, pair, n_units);
    Fetch ring[kAhead];
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      if (ahead.valid(n_units)) {
        ring[i] = fetch_step<BWD>(a, ahead.u, ahead.kb, rank, t);
        ahead.next(a, n_pairs, n_units);
      }
    }
    Pipe p;
    bool ok = true;
    while (cur.valid(n_units) && ok) {
#pragma unroll
      for (int i = 0; i < kAhead; ++i) {
        if (!cur.valid(n_units) || !ok) break;
        int won = 1;
        if (lane == 0) won = mbar_wait(&s.empty[p.stage], p.phase ^ 1u, s.abort_flag, a.status, 35) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, won, 0) != 0;
        if (!ok) break;
        uint8_t* b_tile = s.tiles + p.stage * C::kStageBytes + ACCS * kSub;
        dequant_store(ring[i], a.nested != 0, s.lut, b_tile + row_off, row_swz, half);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) mbar_arrive(&s.full[p.stage]);
          else mbar_arrive_cluster(mapa_u32(smem_u32(&s.full[p.stage]), 0));
        }
        if (ahead.valid(n_units)) {
          ring[i] = fetch_step<BWD>(a, ahead.u, ahead.kb, rank, t);
          ahead.next(a, n_pairs, n_units);
        }
        cur.next(a, n_pairs, n_units);
        p.advance<C::kStages>();
      }
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
// CTA pairs. Per pipeline step the tensor core needs ~512 cycles per accumulator and the 256
// dequantising threads ~600 for their half tile, whichever is longer; a unit ends with an
// epilogue of ~1500 cycles per accumulator. A split needs the fp32 buffer.
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
      const double step = accs * 512.0 > 600.0 ? accs * 512.0 : 600.0;
      const double unit_cost = ((n_rb + ks - 1) / ks) * step + accs * (ks > 1 ? 3000.0 : 1500.0) + 2000.0;
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
int launch(const CUtensorMap& m0, const CUtensorMap& m1, const Args& a, int accs, int pairs, cudaStream_t s) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  const int rows = 256 * accs;
  const long units = (long)a.n_tiles * a.ksplit * ((a.m + rows - 1) / rows);
  const unsigned grid = 2u * (unsigned)(units < pairs ? units : pairs);
  if (accs == 1) {
    if (set_attr<1, BWD>(dev, BWD ? 1 : 0)) return -1;
    nf4_gemm_kernel<1, BWD><<<grid, kThreads, Cfg<1>::kSmem, s>>>(m0, m1, a);
  } else {
    if (set_attr<2, BWD>(dev, BWD ? 3 : 2)) return -1;
    nf4_gemm_kernel<2, BWD><<<grid, kThreads, Cfg<2>::kSmem, s>>>(m0, m1, a);
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
  CUtensorMap map_x;
  if (umma::encode_map_2d_16bit(&map_x, x, (uint64_t)m, (uint64_t)k, (uint64_t)k, kBM, kBK, false))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_fwd: cuTensorMapEncodeTiled failed");
  if (launch<false>(map_x, map_x, a, accs, pairs, s))
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
  CUtensorMap map0, map1;
  if (umma::encode_map_2d_16bit(&map0, items[0].dy, (uint64_t)m, (uint64_t)items[0].n_out,
                                (uint64_t)items[0].n_out, kBM, kBK, false))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: cuTensorMapEncodeTiled failed");
  map1 = map0;
  if (n_items > 1 &&
      umma::encode_map_2d_16bit(&map1, items[1].dy, (uint64_t)m, (uint64_t)items[1].n_out,
                                (uint64_t)items[1].n_out, kBM, kBK, false))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: cuTensorMapEncodeTiled failed");
  if (launch<true>(map0, map1, a, accs, pairs, s))
    SOUP_FAIL(SOUP_ERR_DEVICE, "nf4_linear_dx: cannot raise the shared-memory limit");
  SOUP_CHECK_LAUNCH("nf4_linear_dx");
  if (ksplit > 1 && dx_dtype != SOUP_F32) {
    const int64_t groups = m * (k / 8);
    nf4_gemm_finalize_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>(acc, dx, nullptr, m, (int)k, 0);
    SOUP_CHECK_LAUNCH("nf4_gemm_finalize");
  }
  return SOUP_OK;
}
