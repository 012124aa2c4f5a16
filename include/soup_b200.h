/* libsoup_b200 — C ABI of the B200 (sm_100a) kernels behind the QLoRA training hot path.
 *
 * The reference project (arturbaimuratov1-sys/claudemaxing) has no native layer: every entry here
 * stands where the reference launches one of its Triton kernels from Python, and the comment on
 * each entry names that launch site (path inside the reference project : line).
 *
 * Conventions
 *  - Every pointer is a device pointer owned by the caller; the library allocates nothing, frees
 *    nothing and never synchronises the device. Work is enqueued on `stream`.
 *  - `stream` is a cudaStream_t passed as void* (0 = the legacy default stream).
 *  - Return value: 0 = enqueued; negative = SOUP_ERR_*; the message is in soup_last_error_string()
 *    (thread local). Nothing aborts or traps.
 *  - dtype codes: SOUP_F32, SOUP_F16, SOUP_BF16.
 *  - The compute entries keep no state between calls and use no scratch of their own, so autograd
 *    worker threads may call them concurrently on different streams. Exceptions, each said again
 *    in its own comment: soup_rmsnorm_bwd_noalloc (built-in workspace, calls must not overlap);
 *    soup_lmhead_set_timing (a benchmark aid, off by default, that installs a process-wide host
 *    pointer which every soup_lmhead_ce then writes to and synchronises on: never set it while
 *    other threads call the library); the sticky per-device status word behind
 *    soup_device_status (written with atomics, safe from any number of calls). soup_lmhead_ce
 *    reads the environment (SOUP_LMHEAD_WAVES, SOUP_LMHEAD_DETERMINISTIC) on every call.
 *  - Accumulation order: soup_lmhead_ce splits the vocabulary dimension of the gradient GEMM
 *    across CTA pairs that add into dH with atomics, so dH can differ in the last fp32 bits from
 *    run to run; SOUP_LMHEAD_DETERMINISTIC=1 switches the split off (one adder per element, fixed
 *    order). The RMSNorm dw reduction is always in a fixed order.
 */
#ifndef SOUP_B200_H
#define SOUP_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SOUP_F32 0
#define SOUP_F16 1
#define SOUP_BF16 2

#define SOUP_OK 0
#define SOUP_ERR_ARG (-1)     /* bad shape / dtype / alignment / null pointer */
#define SOUP_ERR_LAUNCH (-2)  /* the CUDA runtime refused the launch */
#define SOUP_ERR_DEVICE (-3)  /* wrong device (not sm_100) or driver entry point missing */

/* Library ABI version; bumped when a signature changes. */
int soup_version(void);
/* Message of the last failing call on this thread ("" if none). */
const char* soup_last_error_string(void);
/* Status word of the pipelined row kernels (RMSNorm, RoPE) on the current device: 0, or the code
 * of the first bounded wait that ran out (11 RMSNorm forward, 12 RMSNorm backward, 13 RoPE). The
 * word is sticky. Synchronises `stream`. No counterpart in the reference (its Triton kernels have
 * no waits). */
int soup_row_status(int* host_status, void* stream);
/* The same sticky word, for every kernel family: besides the row-kernel codes it receives the
 * code of a soup_lmhead_ce call whose bounded waits gave up (11-14 logits kernel, 21-24 gradient
 * kernel: producer, accumulator, operand and epilogue waits) or whose row merge met a non-finite
 * sum (90), copied from the call's workspace by the call's last launch, and 99 from
 * soup_wait_selftest. `clear` != 0 resets the word after reading it. Synchronises `stream`; meant
 * to be called where the host waits for the step's loss anyway. A non-zero word means outputs
 * since the last clear may be unwritten. No counterpart in the reference (its kernels cannot
 * time out; its failures are Python exceptions). */
int soup_device_status(int* host_status, int clear, void* stream);
/* Self-test of the bounded waits every kernel of the library uses: launches one small CTA that
 * waits, with a limit of `limit_ns` (at most 100 ms), on a barrier nothing ever completes. The
 * wait has to run out: *host_gave_up becomes 1 and *host_status the code 99, and the context stays
 * usable. Synchronises `stream`. No counterpart in the reference. */
int soup_wait_selftest(int64_t limit_ns, int* host_gave_up, int* host_status, void* stream);

/* NF4 -> fp16/fp32 weight, nested (double-quantised) absmax fused, bit-exact unfused fp32 math.
 * Replaces nf4_dequant_kernel[grid](...) at solution/nf4.py:78-81 (kernel :26-46).
 *   packed   uint8 [n_elems/2]; element 2i = high nibble of byte i, 2i+1 = low nibble
 *   absmax   nested: uint8 [n_elems/blocksize]; else float [n_elems/blocksize]
 *   code     float [16]   4-bit code table
 *   code2    float [256]  8-bit map of the nested absmax          (nested only)
 *   absmax2  float [ceil(n_elems/blocksize/blocksize2)]            (nested only)
 *   offset   float [1]                                             (nested only)
 *   out      out_dtype [n_elems]
 * scale = nested ? code2[absmax[b]] * absmax2[b / blocksize2] + offset : absmax[b]   (mul, then add)
 * out[j] = round_out_dtype(code[nibble_j] * scale)
 * Requires: n_elems even, blocksize in {32..4096} power of two, out_dtype F16 or F32. */
int soup_nf4_dequant(const void* packed, const void* absmax, const float* code, const float* code2,
                     const float* absmax2, const float* offset, void* out, int64_t n_elems,
                     int blocksize, int blocksize2, int nested, int out_dtype, void* stream);

/* The same for several weights in one launch per 8 tensors (e.g. the seven projections of a
 * decoder layer): one element of `items` (a host array) per tensor, fields as the arguments of
 * soup_nf4_dequant; blocksize, blocksize2, nested and out_dtype are common to the batch. The
 * reference dequantises one weight per launch (solution/nf4.py:78-81); on B200 the launch latency
 * is longer than the data movement of the small projections. */
typedef struct {
  const void* packed;
  const void* absmax;
  const float* code2;
  const float* absmax2;
  const float* offset;
  void* out;
  int64_t n_elems;
} soup_nf4_item;
int soup_nf4_dequant_batch(const soup_nf4_item* items, int count, const float* code, int blocksize,
                           int blocksize2, int nested, int out_dtype, void* stream);

/* RMSNorm forward: rstd = 1/sqrt(mean(x^2)+eps); normed = round_x_dtype(x*rstd);
 * out = round_out_dtype(normed*w). Replaces qwen_rmsnorm_fwd_kernel at solution/rmsnorm.py:180-184
 * (kernel :28-47).
 *   low   (nullable) fp16 copy of out [n_rows,n_cols]; when given, slot/small are used too:
 *   slot  int32 [n_cols], index among the tiny-|w| columns or -1
 *   small fp16 [n_rows,n_small], normalised value of the tiny-|w| columns */
int soup_rmsnorm_fwd(const void* x, const void* w, void* out, float* rstd, void* low,
                     const int32_t* slot, void* small, int64_t n_small, int64_t n_rows,
                     int64_t n_cols, float eps, int x_dtype, int w_dtype, int out_dtype,
                     void* stream);

/* Number of fp32 rows of the dw workspace soup_rmsnorm_bwd needs for this shape. */
int64_t soup_rmsnorm_bwd_partials(int64_t n_rows, int64_t n_cols);

/* RMSNorm backward: dx = (gn - n*mean(gn*n))*rstd with gn = dy*w (rounded to xin dtype unless
 * saved_output), n = xin*rstd, or (saved_output) n = low/w with the tiny-|w| columns taken from
 * `small`. Optional dw = sum_rows dy*round_x_dtype(n): needs dw_partial (fp32
 * [soup_rmsnorm_bwd_partials(), n_cols]) and dw (w_dtype [n_cols]); pass both NULL to skip.
 * Replaces qwen_rmsnorm_bwd_kernel at solution/rmsnorm.py:205-212 (kernel :51-91) and the
 * partial.sum(0) that follows it (:213-214). */
int soup_rmsnorm_bwd(const void* dy, const void* xin, const void* w, const float* rstd, void* dx,
                     float* dw_partial, void* dw, const int32_t* slot, const void* small,
                     int64_t n_small, int64_t n_rows, int64_t n_cols, int dy_dtype, int xin_dtype,
                     int w_dtype, int dx_dtype, int saved_output, void* stream);

/* soup_rmsnorm_bwd for callers that cannot allocate device memory. It has no counterpart in the
 * reference. Same arguments and results as soup_rmsnorm_bwd, minus dw_partial: the fp32 partial
 * rows of dw live in a 10 MiB array built into the library (640 rows x 4096 columns, resident on
 * every GPU that loads the library until the process exits). Meant for hosts that bind this
 * library without a framework allocator behind them (a plain C or C++ trainer that sized all of its
 * device memory up front), or that cannot afford cudaMalloc's device-wide synchronisation in
 * the middle of a step. The call allocates and frees nothing.
 *  - Limits: n_cols <= 4096 and at most 640 partial rows (4 CTAs per SM, 148 SMs need 592);
 *    anything larger is refused with SOUP_ERR_ARG and the caller should use soup_rmsnorm_bwd.
 *  - The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
 *    that device current); make that first call outside any stream capture.
 *  - All calls on a device share the one array, which keeps the previous call's contents (each call
 *    rewrites every row it later reads, so nothing needs clearing). Two calls with dw != NULL that
 *    overlap on the GPU (different streams, no ordering between them) race on it: serialise them. */
int soup_rmsnorm_bwd_noalloc(const void* dy, const void* xin, const void* w, const float* rstd,
                             void* dx, void* dw, const int32_t* slot, const void* small,
                             int64_t n_small, int64_t n_rows, int64_t n_cols, int dy_dtype,
                             int xin_dtype, int w_dtype, int dx_dtype, int saved_output,
                             void* stream);

/* The 4-bit model's RMSNorm backward (fp32 dy, the forward's fp16 copy `low` as the saved tensor,
 * fp32 weight and dx; the saved-output form of soup_rmsnorm_bwd) with the residual connection
 * folded in: dx = rmsnorm_backward(dy) + add, where `add` (nullable, fp32 [n_rows, n_cols]) is the
 * gradient that reaches the norm's input along the residual branch, and dx16 (nullable) receives
 * the fp16 copy of dx that the projection backward one block earlier wants. Two elementwise
 * kernels (an add and a cast over [tokens, hidden]) per norm disappear. Returns SOUP_ERR_ARG for
 * shapes the saved-output kernel does not take; the caller then adds and casts itself. No
 * counterpart of its own in the reference (its block leaves both to autograd). */
int soup_rmsnorm_bwd_residual(const float* dy, const void* low, const float* w, const float* rstd,
                              const float* add, float* dx, void* dx16, const int32_t* slot,
                              const void* small, int64_t n_small, int64_t n_rows, int64_t n_cols,
                              void* stream);

/* Rotary embedding of q and k in one launch (forward, or the transposed rotation for backward).
 * Replaces the two qwen_rope_kernel launches of RoPE.forward / RoPE.backward at
 * solution/rope.py:54-56 (kernel :17-43). Either of q / k may be NULL (skipped).
 *   q      [b, hq, t, d] with strides (q_sb, q_sh, q_st, 1) in elements; k likewise with hk
 *   cos,sin [cb, t, d] contiguous in t,d; batch stride cs_b elements (0 to broadcast)
 *   q_out  [b, hq, t, d] contiguous, k_out [b, hk, t, d] contiguous
 * fwd: o1 = x1*c1 - x2*s1, o2 = x2*c2 + x1*s2;  bwd: o1 = x1*c1 + x2*s2, o2 = x2*c2 - x1*s1. */
int soup_rope(const void* q, const void* k, const void* cos, const void* sin, void* q_out,
              void* k_out, int64_t b, int64_t hq, int64_t hk, int64_t t, int64_t d, int64_t q_sb,
              int64_t q_sh, int64_t q_st, int64_t k_sb, int64_t k_sh, int64_t k_st, int64_t cs_b,
              int64_t cs_t, int q_dtype, int k_dtype, int cs_dtype, int q_out_dtype,
              int k_out_dtype, int backward, void* stream);

/* The same rotation with q given as a sum of two tensors and with strided outputs, for a decoder
 * block that keeps q, k and v in half precision between the projections and the attention:
 *   q_add  NULL, or q's second term (the adapter branch's output), read through
 *          (qa_sb, qa_sh, qa_st, 1) and added in fp32 before the rotation, so the result equals rotating the fp32 sum the reference's
 *          layer forms (base output + adapter output, then solution/rope.py:54-56 on the sum)
 *   q_out, k_out  written through (qo_sb, qo_sh, qo_st, 1) / (ko_sb, ko_sh, ko_st, 1): any layout
 *          with a contiguous head row, e.g. [b, t, h, d] for a variable-length attention kernel,
 *          or a column block of a wider [b*t, n] gradient buffer in backward
 * No counterpart of its own in the reference (its RoPE.apply takes and returns whole tensors). */
int soup_rope_sum(const void* q, const void* q_add, const void* k, const void* cos,
                  const void* sin, void* q_out, void* k_out, int64_t b, int64_t hq, int64_t hk,
                  int64_t t, int64_t d, int64_t q_sb, int64_t q_sh, int64_t q_st, int64_t k_sb,
                  int64_t k_sh, int64_t k_st, int64_t cs_b, int64_t cs_t, int64_t qa_sb,
                  int64_t qa_sh, int64_t qa_st, int64_t qo_sb, int64_t qo_sh, int64_t qo_st,
                  int64_t ko_sb, int64_t ko_sh, int64_t ko_st,
                  int q_dtype, int q_add_dtype, int k_dtype, int cs_dtype, int q_out_dtype,
                  int k_out_dtype, int backward, void* stream);

/* Causal attention inside the segments of one packed row, forward: for every token i of segment s,
 * out[i, h] = softmax_j(scale * q[i, h] . k[j, h / (hq/hk)]) v[j, h / (hq/hk)] over the tokens j <= i
 * of the same segment. Stands where the reference calls torch SDPA on the [1, 1, N, N] mask of its
 * packed batch (solution/attention.py:332-343, mask from solution/lm_head_loss.py:300-337); the
 * segments are given as offsets instead of a mask.
 *   q [n_tokens, hq, 128] fp16, row pitch q_pitch elements (heads adjacent); k, v [n_tokens, hk, 128]
 *   cu_rows int32 [n_segments + 1] on the device: segment s is tokens cu_rows[s] .. cu_rows[s+1]-1
 *   out [n_tokens, hq, 128] fp16 contiguous; lse fp32 [hq, n_tokens]: log(sum_j exp(scale * s_ij))
 * head_dim must be 128; pointers 16-byte aligned, pitches multiples of 8. tcgen05 / TMEM / TMA. */
int soup_attn_fwd(const void* q, const void* k, const void* v, const int32_t* cu_rows, void* out,
                  float* lse, int64_t n_tokens, int64_t n_segments, int64_t hq, int64_t hk,
                  int64_t head_dim, int64_t q_pitch, int64_t k_pitch, int64_t v_pitch, float scale,
                  void* stream);

/* Backward of soup_attn_fwd: from q, k, v, the forward's out and lse, and d_out, the gradients
 *   dq [n_tokens, hq, 128] fp16 contiguous (every token inside a segment is written),
 *   dk, dv [n_tokens, hk, 128] fp32 contiguous: cleared here, then accumulated with atomic adds over
 *   the query heads of a group and the query tiles of a segment (their last bits can differ
 *   between runs).
 * out and d_out are [n_tokens, hq, 128] fp16 contiguous; the rest as in soup_attn_fwd. In the
 * reference this is the backward of torch SDPA (solution/attention.py:332-343). */
int soup_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                  const float* lse, const int32_t* cu_rows, void* dq, float* dk, float* dv,
                  int64_t n_tokens, int64_t n_segments, int64_t hq, int64_t hk, int64_t head_dim,
                  int64_t q_pitch, int64_t k_pitch, int64_t v_pitch, float scale, void* stream);

/* out = round_out(round_gate?(silu(gate)) * up). Replaces silu_mul_fwd_persistent at
 * solution/swiglu_recompute.py:98-100 and :176-178 (kernel :36-48). */
int soup_silu_mul_fwd(const void* gate, const void* up, void* out, int64_t n, int gate_dtype,
                      int up_dtype, int out_dtype, int round_silu, void* stream);

/* Recompute backward of silu(gate)*up: dup = dy*silu, dgate = round?(dy*up)*sig*(1+g*(1-sig)).
 * dgate may alias gate and dup may alias up (each element is read before it is written).
 * Either output may be NULL (not wanted). Replaces silu_mul_bwd_recompute at
 * solution/swiglu_recompute.py:122-124 and :203-205 (kernel :51-79). */
int soup_silu_mul_bwd(const void* dy, const void* gate, const void* up, void* dgate, void* dup,
                      int64_t n, int dy_dtype, int gate_dtype, int up_dtype, int round_silu,
                      void* stream);

/* LoRA dropout pack: xd = fp16(keep ? x*scale : 0); bits[r] = sum_l keep[8r+l] << l.
 * Replaces lora_dropout_pack_kernel at solution/lora.py:64-65 (kernel :30-42).
 *   x [n] x_dtype, mask bool/uint8 [n], xd fp16 [n], bits uint8 [n/8]; n % 8 == 0 */
int soup_dropout_pack(const void* x, const uint8_t* mask, void* xd, uint8_t* bits, int64_t n,
                      float scale, int x_dtype, void* stream);

/* LoRA dropout unpack: xd = fp16(keep ? x16*scale : 0), dx = dx_dtype(keep ? g16*scale : 0).
 * Replaces lora_dropout_unpack_kernel at solution/lora.py:73-74 (kernel :45-57). */
int soup_dropout_unpack(const void* x16, const uint8_t* bits, const void* g16, void* xd, void* dx,
                        int64_t n, float scale, int dx_dtype, void* stream);

/* The two adapters of a block (same x, two masks) in one launch each: soup_dropout_pack and
 * soup_dropout_unpack for both, x read once, and the two input gradients summed:
 * dx = keep_a*g_a*scale_a + keep_b*g_b*scale_b (fp32). n a multiple of 16; 16-byte aligned
 * pointers. Per adapter the values and bits are those of the single entries (which replace the
 * launches of solution/lora.py:64-65 and :73-74). */
int soup_dropout_pack2(const void* x, const uint8_t* mask_a, const uint8_t* mask_b, void* xd_a,
                       void* xd_b, uint8_t* bits_a, uint8_t* bits_b, int64_t n, float scale_a,
                       float scale_b, int x_dtype, void* stream);
int soup_dropout_unpack2(const void* x16, const uint8_t* bits_a, const uint8_t* bits_b,
                         const void* g_a, const void* g_b, void* xd_a, void* xd_b, float* dx,
                         int64_t n, float scale_a, float scale_b, void* stream);

/* ---- linear layers on NF4 weights: tcgen05 GEMM with the dequantisation in its operand prologue --
 * One weight of a launch. `packed`, `absmax`, `code2`, `absmax2`, `offset` as in soup_nf4_dequant
 * (blocksize 64 only: one block is one 128-byte row of the operand tile). Forward reads `bias`
 * (fp16 [n_out] or NULL) and writes `out` (fp16 [m, n_out] row-major); backward reads `dy`
 * (fp16 [m, n_out] row-major). The dequantised operand is bit-identical to soup_nf4_dequant's
 * fp16 output (same unfused fp32 operations in the same order). */
typedef struct {
  const void* packed;
  const void* absmax;
  const float* code2;
  const float* absmax2;
  const float* offset;
  const void* bias;
  void* out;
  const void* dy;
  int64_t n_out;
} soup_nf4_gemm_item;

/* Bytes of the optional fp32 buffer of the two entries below for an [m, cols] result. */
int64_t soup_nf4_gemm_workspace_bytes(int64_t m, int64_t cols);

/* out_i[m, n_i] = x[m, k] * dequant(W_i)[n_i, k]^T (+ bias_i) for up to four weights that share x
 * (one launch: gate_proj and up_proj, or q/k/v). fp16 operands, fp32 accumulation, fp16 result.
 * Replaces the dequantise + F.linear pair of solution/nf4.py:122 and bnb.matmul_4bit at
 * solution/swiglu_recompute.py:165-166 (forward) and :198-199 (recompute in backward); the fp16
 * weight never exists in HBM. x fp16 [m, k] row-major, k % 64 == 0, n_i % 8 == 0, blocksize 64.
 * `workspace` (nullable, fp32 [m, n_0]): with a single weight and a long k the contraction is
 * split over CTA pairs that add into it (the result is then not bit-reproducible from run to
 * run); without it nothing is split. A failed bounded wait reports through soup_device_status
 * (codes 31-38). */
int soup_nf4_linear_fwd(const void* x, const soup_nf4_gemm_item* items, int n_items,
                        const float* code, int64_t m, int64_t k, int nested, int blocksize,
                        int blocksize2, void* workspace, int64_t workspace_bytes, void* stream);

/* dx[m, k] = sum_i dy_i[m, n_i] * dequant(W_i)[n_i, k] for one or two weights (the input gradient
 * of the projections above; two weights: gate_proj and up_proj of one MLP, summed in the
 * accumulator). Replaces the dequantise + matmul of bitsandbytes' MatMul4Bit.backward, reached
 * from solution/nf4.py:127-132 and solution/swiglu_recompute.py:210-213. dx fp16 or fp32
 * (dx_dtype), n_i % 64 == 0. A long contraction is split over CTA pairs that add partial sums
 * into dx itself when it is fp32, else into `workspace` (nullable, fp32 [m, k]). */
int soup_nf4_linear_dx(const soup_nf4_gemm_item* items, int n_items, const float* code, void* dx,
                       int dx_dtype, int64_t m, int64_t k, int nested, int blocksize,
                       int blocksize2, void* workspace, int64_t workspace_bytes, void* stream);

/* ---- fused LM head + cross-entropy (tcgen05 / TMEM / TMA) -------------------------------------
 * Replaces the chunk loop of _FusedHeadLoss.forward, solution/lm_head_loss.py:213-224 (torch.mm,
 * lm_head_vocab_chunk_kernel :108-160, torch.mm, mul_/add_), over the columns of one weight shard.
 * State arrays are fp32/int32 [n] and are initialised by the call; (run_max, run_sum, run_dot)
 * mean: mass = run_sum * e^run_max, dot mass = run_dot * e^run_max (the call leaves them
 * normalised, run_max = log-sum-exp of the shard, run_sum = 1):
 *   run_max, run_sum  log-sum-exp bookkeeping over the shard's columns
 *   run_dot           sum of softmax_shard(z) * z                               (entropy)
 *   best, best_val    global vocabulary index and value of the first maximum    (accuracy)
 *   label_logit       the label's logit, where the label falls in this shard    (loss)
 *   grad_ref          the log-sum-exp dh is relative to
 *   dh                fp32 [n,h]: sum over the shard's columns except the label's of
 *                     exp(z_v - grad_ref) * W[v], zero for unlabelled rows; soup_lmhead_finish
 *                     completes it. NULL when want_grad == 0
 * hidden fp16 [n,h] and weight fp16 [v_shard,h] row-major, 16-byte aligned, h % 8 == 0.
 * weight_bf16: the same weight rounded to bf16 (needed when want_grad != 0; the gradient GEMM
 * multiplies bf16 probabilities with it, and the tensor core takes one format for both operands).
 * col_offset = global index of the shard's first column. chunk_tiles = 256-column tiles per
 * chunk (0 = library default). workspace: soup_lmhead_workspace_bytes() bytes, 16-byte aligned.
 * With SOUP_LMHEAD_DETERMINISTIC=1 in the environment the gradient GEMM does not split its
 * reduction dimension and dh is bit-reproducible (at a lower SM occupancy). */
int64_t soup_lmhead_workspace_bytes(int64_t n, int64_t h, int64_t v_shard, int64_t chunk_tiles);
int soup_lmhead_ce(const void* hidden, const void* weight, const void* weight_bf16,
                   const int64_t* target, float* run_max, float* run_sum, float* run_dot, int* best,
                   float* best_val, float* label_logit, float* grad_ref, float* dh, void* workspace,
                   int64_t workspace_bytes, int64_t n, int64_t h, int64_t v_shard,
                   int64_t col_offset, int64_t chunk_tiles, int want_grad, void* stream);

/* Benchmark aid: while a host array of 6 floats is set, every soup_lmhead_ce call brackets its
 * launches with events, synchronises its stream before returning, and adds the milliseconds of the
 * logits / row / grad kernels to sink[0..2] and their launch counts to sink[3..5]. NULL switches it
 * off (the default). Not for use from concurrent threads. No counterpart in the reference (its
 * harness times kernels from Python, harness/_train.py:44-83). */
int soup_lmhead_set_timing(float* host_sink6);

/* The tiling soup_lmhead_ce uses for a shape: rows per row block, 256-column tiles of the first
 * chunk (whose logits are computed twice) and of every later chunk. */
int soup_lmhead_plan(int64_t n, int64_t v_shard, int64_t chunk_tiles, int64_t* row_block,
                     int64_t* first_chunk_tiles, int64_t* tiles_per_chunk);

/* Reads back the device status word of the last soup_lmhead_ce on this workspace (synchronises
 * `stream`): 0 = every bounded wait completed; otherwise the code of the wait that gave up. */
int soup_lmhead_status(const void* workspace, int64_t n, int64_t v_shard, int64_t chunk_tiles,
                       int* host_status, void* stream);

/* Vocabulary-parallel merge of per-rank states gathered as [n_ranks, n] arrays (rank order =
 * ascending vocabulary order; shard_begin int64 [n_ranks + 1] on the device). o_lse = merged
 * log-sum-exp. No counterpart in the reference, which is single-GPU (solution/lm_head_loss.py:
 * 426-428 refuses n_gpu > 1); the merge rule is the chunk-to-chunk carry of :119-145. */
int soup_lmhead_merge(const float* g_max, const float* g_sum, const float* g_dot,
                      const int* g_best, const float* g_best_val, const float* g_label_logit,
                      const int64_t* target, const int64_t* shard_begin, float* o_max,
                      float* o_sum, float* o_dot, int* o_best, float* o_best_val,
                      float* o_label_logit, float* o_lse, int64_t n, int n_ranks, void* stream);

/* Finalisation, solution/lm_head_loss.py:225-237: token_loss = lse - label_logit (0 if ignored),
 * entropy = lse - run_dot/run_sum, correct = labelled && best == target (all nullable together);
 * dh (nullable, in place): dh = 1024 * (exp(grad_ref - lse) * dh + (p_label - 1) * W[label]) with
 * the label term only where the label falls in this shard; grad_ref is the array the same
 * rank's soup_lmhead_ce returned (not a merged one). */
int soup_lmhead_finish(const float* run_max, const float* run_sum, const float* run_dot,
                       const int* best, const float* label_logit, const float* grad_ref,
                       const int64_t* target, const void* weight, float* token_loss,
                       float* entropy, int* correct, float* dh, int64_t n, int64_t h,
                       int64_t v_shard, int64_t col_offset, void* stream);

/* The same finalisation with the finished gradient written to a buffer of its own in
 * `dh_out_dtype` (dh is then only read): the vocabulary-parallel head sends fp16 partial
 * gradients over NVLink, and writing them here saves rewriting the fp32 buffer and a separate
 * rounding pass over [rows, hidden]. dh_out NULL: exactly soup_lmhead_finish. */
int soup_lmhead_finish_to(const float* run_max, const float* run_sum, const float* run_dot,
                          const int* best, const float* label_logit, const float* grad_ref,
                          const int64_t* target, const void* weight, float* token_loss,
                          float* entropy, int* correct, float* dh, void* dh_out, int dh_out_dtype,
                          int64_t n, int64_t h, int64_t v_shard, int64_t col_offset, void* stream);

/* out = out_dtype(dh * scale[0]) — _FusedHeadLoss.backward, solution/lm_head_loss.py:248-254. */
int soup_lmhead_grad_scale(const float* dh, void* out, const float* scale, int64_t n,
                           int out_dtype, void* stream);

/* Loss / entropy / correct per row from materialised logits [n_rows, n_cols] (row pitch
 * row_stride elements). Replaces lm_head_xent_rows_kernel, solution/lm_head_loss.py:168-172
 * (kernel :54-96) in its WRITE_GRAD = False use. */
int soup_xent_rows(const void* logits, const int64_t* target, float* loss, float* entropy,
                   int* correct, int64_t n_rows, int64_t n_cols, int64_t row_stride, int dtype,
                   void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SOUP_B200_H */
