/* strixite_b200 - the C ABI of the sm_100a quantized-MoE FFN library (libstrixite_b200.so).
 *
 * One entry point per kernel function of strixite's MoE hot path; each comment names the reference interface it
 * replaces (paths relative to the strixite tree). Conventions, the same for every function:
 *   - plain pointers and sizes only; device pointers unless the name says host;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - everything is enqueued asynchronously; nothing allocates, synchronizes or keeps state between calls, except
 *     the check_*_error readers (which copy 3 words back, so they synchronize), the strix_moe_layer_* session object
 *     and the function whose comment says otherwise;
 *   - return value: 0 = enqueued; 1 = an argument check failed; 2 = a CUDA call failed. strix_last_error() gives
 *     the message of the calling thread's last failure ("func (file:line): check `cond` failed: ...");
 *   - `act`: 0 = FP32 activations, 1 = BF16 activations as raw bits (strixite kernels/norm.hpp:20 enum Act);
 *   - `err`: >= 3 zeroed uint32 on the device. Data errors never fail a call: the kernel sets err = {1, a, b}
 *     (the first flag wins, kernels never clear it) and writes NaN to the affected outputs.
 */
#ifndef STRIXITE_B200_H
#define STRIXITE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STRIX_ACT_F32 0
#define STRIX_ACT_BF16 1

/* strixite kernels/moe_grouped.hpp:30-35 enum class MoeMath. F32: FP32 FMA on the CUDA cores. WMMA_BF16 / WMMA_F16:
 * both select the tensor-core path here: activations and dequantized weights as F16 operands in shared memory (one
 * F16 rounding of code * s + m, the precision of the reference's WmmaF16; BF16 activations convert exactly inside
 * F16's normal range, |x| < 65504, the assumption of strixite kernels/wmma_gemm.hpp:371-372), FP32 accumulation in
 * tensor memory, FP32 combine partials. */
#define STRIX_MATH_F32 0
#define STRIX_MATH_WMMA_BF16 1
#define STRIX_MATH_WMMA_F16 2

/* A quantized matrix [N, K] resident on the device - field for field strixite runtime/q4_device.hpp:13-18
 * (Q4DeviceView; q5_device.hpp, q6_device.hpp, q8_device.hpp have the same fields). q: N * row_bytes code bytes,
 * 16-byte aligned; scale, minv: [N, K / G] BF16 bits. Row layouts: strixite formats/q4.hpp:3-6, q5.hpp:5-10,
 * q6.hpp:5-10, q8.hpp:5-8. */
typedef struct strix_qview {
    const uint8_t *q;
    const uint16_t *scale;
    const uint16_t *minv;
    int64_t N, K, G;
} strix_qview;

/* E experts stacked [E * N, K] with a format PER EXPERT (4, 5, 6 or 8 bits). No counterpart in the reference, whose
 * expert stacks have one format (runtime/qweight.hpp:75-125 accepts 4 or 5 bits only): it exists for stacks that mix
 * q4/q5/q6/q8 experts. bits [E] and q_off [E] (byte offset of expert e's first row in q, a multiple of 16) are device
 * arrays; scale/minv are [E * N, K / G] as for a uniform stack. N = rows per expert. */
typedef struct strix_qmix_view {
    const uint8_t *q;
    const uint16_t *scale;
    const uint16_t *minv;
    const uint8_t *bits;
    const int64_t *q_off;
    int64_t E, N, K, G;
} strix_qmix_view;

const char *strix_last_error(void);
/* Library identity: "strixite_b200 <version> sm_100a". */
const char *strix_version(void);

/* ---- formats (host side) ------------------------------------------------------------------------------------- */

/* strixite formats/q4.hpp:27-29 quantize_q4, q5.hpp:39-40, q6.hpp:39-40, q8.hpp:27-28. Host arrays. Per group:
 * s = bf16((max - min) / (2^bits - 1)), m = bf16(min), code = clamp(rne((w - m) / s), 0, 2^bits - 1), 0 when s == 0.
 * Fails (1) on a bad shape, G not in {32, 64, 128}, K % G != 0, q5 K % 128 != 0, q6 K % 64 != 0, a non-finite weight,
 * or a rounding mode other than nearest-even - the cases where the reference throws. */
int strix_quantize(int bits, const float *w, int64_t N, int64_t K, int64_t G, uint8_t *q, uint16_t *scale,
                   uint16_t *minv);
/* strixite formats/q4.hpp:40-41 dequantize_q4 (and q5/q6/q8): w = code * s + m, two roundings. Host arrays. */
int strix_dequantize(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K,
                     int64_t G, float *w);
/* strixite formats/q4.hpp:31-32 check_q4 (and q5/q6/q8) on array sizes given in bytes / entries. */
int strix_check_qweight(int bits, int64_t N, int64_t K, int64_t G, size_t q_bytes, size_t n_scale, size_t n_min);
/* strixite formats/strixw.hpp:59 strix_hash64: the 64-bit hash of a byte range that strixw weight files carry for their
 * header, index and every tensor component. Host memory. */
uint64_t strix_hash64(const void *data, size_t n);
/* strixite formats/q4.hpp:22-23, q5.hpp:31, q6.hpp:31: packed bytes of one row. */
int64_t strix_row_bytes(int bits, int64_t K);
/* The same quantizer on the device (w, q, scale, minv device arrays): bit-identical to strix_quantize. A non-finite
 * weight sets err = {1, row, column}. No counterpart in the reference (its quantizers are host-only). */
int strix_quantize_device(int bits, const float *w, int64_t N, int64_t K, int64_t G, uint8_t *q, uint16_t *scale,
                          uint16_t *minv, uint32_t *err, void *stream);

/* ---- router and the shared expert's gate ------------------------------------------------------------------- */

/* strixite kernels/moe_router.hpp:38-40 moe_router. */
int strix_moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit,
                     int64_t shared_ld, int32_t shared_id, int32_t *ids, float *coef, int act, uint32_t *err,
                     void *stream);
/* strixite kernels/moe_router.hpp:41-43 check_router_error / report_router_error. */
int strix_check_router_error(const uint32_t *err, const char *what);
int strix_report_router_error(const uint32_t e[3], const char *what);
/* strixite kernels/moe_router.hpp:53-54 moe_shared_add. */
int strix_moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                         uint32_t gate_index, int act, uint32_t *err, void *stream);
/* strixite kernels/moe_router.hpp:61-63 moe_shared_add_inject. */
int strix_moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M,
                                int64_t N, uint32_t gate_index, void *x, const float *w_in, int64_t H, int act,
                                uint32_t *err, void *stream);

/* ---- dense projections ----------------------------------------------------------------------------------------- */

/* strixite kernels/linear_q4.hpp:26-30 linear_q4 (with out_act), linear_q5.hpp:14-15, linear_q6.hpp:14-15,
 * linear_q8.hpp:13-14: y[M, N] = x[M, K] * dequant(W)^T. out_act == act, or BF16 x -> F32 y (unrounded). */
int strix_linear_q4(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
int strix_linear_q5(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
int strix_linear_q6(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
int strix_linear_q8(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
/* strixite kernels/linear.hpp:20-26 linear_bf16w: W [N, K] raw BF16 bits (the router projection). */
int strix_linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, int act,
                       int out_act, void *stream);
/* strixite kernels/linear_wmma.hpp:21-24 linear_q{4,5,6,8}_wmma: the same projections on the tensor cores (tcgen05, FP32
 * accumulation; activations and dequantized weights as F16 operands, see STRIX_MATH_*). K % 64 == 0. */
int strix_linear_q4_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
int strix_linear_q5_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
int strix_linear_q6_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
int strix_linear_q8_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream);
/* strixite kernels/linear_wmma.hpp:27-29 linear_bf16w_wmma: BF16 tokens, BF16 weights, FP32 outputs on the tensor cores
 * (both operands by TMA; products exact, only the summation order differs from linear_bf16w). K % 64 == 0. */
int strix_linear_bf16w_wmma(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, int act,
                            int out_act, void *stream);
/* The same with FP32 weights [N, K] (a router kept in FP32). No counterpart in the reference. */
int strix_linear_f32w(const void *x, const float *w, void *y, int64_t M, int64_t N, int64_t K, int act, int out_act,
                      void *stream);

/* ---- elementwise ----------------------------------------------------------------------------------------------- */

/* strixite kernels/swiglu.hpp:21 swiglu. */
int strix_swiglu(const void *gu, void *h, int64_t rows, int64_t I, int act, void *stream);
/* strixite kernels/residual.hpp:17 residual_add. */
int strix_residual_add(void *x, const void *y, int64_t n, int act, void *stream);
/* strixite kernels/hc.hpp:52-55 hc_inject: x[t, s*N + n] = fma(w_in[t, s], y[t, n], x[t, s*N + n]), x [M, H*N]. */
int strix_hc_inject(void *x, const void *y, const float *w_in, int64_t M, int64_t N, int64_t H, int act, void *stream);

/* ---- the hyper-connection bracket around the MoE sublayer ------------------------------------------------------ */

/* strixite kernels/hc.hpp:36-39 hc_mix_down (the Q4 and Q8 overloads; `bits` 4 or 8): X [T, H*d] -> h [T, r] =
 * silu(a / H) for the first r rows of the folded weights w [r (+ H), H*d], w_in [T, H] = 2 sigmoid(a / H) for the next H rows
 * (when inject; w_in NULL otherwise), inv [T, H] = the per-stream inverse RMS. H == 4, d % 32 == 0, x 16-byte aligned. */
int strix_hc_mix_down(const void *x, const strix_qview *w, int bits, int64_t T, int64_t H, int64_t d, int64_t r, int inject,
                      float eps, float *h, float *w_in, float *inv, int act, void *stream);
/* strixite kernels/hc.hpp:47-50 hc_mix_up: u[t, j] = (1/H) sum_s sigmoid(W_up[s*d + j] . h[t]) * X[t, s*d + j] * inv[t, s] *
 * (1 + norm_w[s*d + j]). w_up [H*d, r] is CHUNK-major (strixite formats/q4.hpp:41-55: 32-code chunk c of row n at
 * q[(c*N + n) * chunk bytes], group g's scale / min at [g*N + n]); r % 32 == 0, r <= 1024. u [T, d] in the activation dtype. */
int strix_hc_mix_up(const float *h, const strix_qview *w_up, int bits, const void *x, const float *norm_w, const float *inv,
                    int64_t T, int64_t H, int64_t d, void *u, int act, void *stream);
/* strixite kernels/hc_wmma.hpp:38-42 hc_inject_inv: hc_inject (X[t, s*d + j] += w_in[t, s] * y[t, j], one rounding) and the
 * inverse RMS of the updated, stored streams into inv [T, H], in one pass. X is bit-identical to strix_hc_inject's. */
int strix_hc_inject_inv(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, float eps, float *inv,
                        int act, void *stream);
/* strixite formats/q4.hpp:55 to_chunk_major (and the Q8 twin): host arrays, row-major -> chunk-major. */
int strix_to_chunk_major(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K,
                         int64_t G, uint8_t *q_out, uint16_t *scale_out, uint16_t *min_out);

/* ---- experts, per slot (decode / verify) ---------------------------------------------------------------------- */

/* strixite kernels/linear_q4.hpp:42-58: linear_q4_experts_gather / _combine / _gather_swiglu and the q5 twins.
 * w: E experts stacked [E * N, K]. */
int strix_linear_q4_experts_gather(const void *x, const strix_qview *w, int64_t E, const int32_t *ids, int64_t M,
                                   int64_t A, void *y, int act, uint32_t *err, void *stream);
int strix_linear_q4_experts_combine(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                    const float *coef, int64_t M, int64_t A, void *y, int act, uint32_t *err,
                                    void *stream);
int strix_linear_q4_experts_gather_swiglu(const void *x, const strix_qview *w, int64_t E, const int32_t *ids,
                                          int64_t M, int64_t A, void *h, int act, uint32_t *err, void *stream);
int strix_linear_q5_experts_gather(const void *x, const strix_qview *w, int64_t E, const int32_t *ids, int64_t M,
                                   int64_t A, void *y, int act, uint32_t *err, void *stream);
int strix_linear_q5_experts_combine(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                    const float *coef, int64_t M, int64_t A, void *y, int act, uint32_t *err,
                                    void *stream);
int strix_linear_q5_experts_gather_swiglu(const void *x, const strix_qview *w, int64_t E, const int32_t *ids,
                                          int64_t M, int64_t A, void *h, int act, uint32_t *err, void *stream);
/* The same three over a stack with a format per expert (strix_qmix_view). No counterpart in the reference. */
int strix_linear_qmix_experts_gather(const void *x, const strix_qmix_view *w, const int32_t *ids, int64_t M,
                                     int64_t A, void *y, int act, uint32_t *err, void *stream);
int strix_linear_qmix_experts_combine(const void *h, const strix_qmix_view *w, const int32_t *ids, const float *coef,
                                      int64_t M, int64_t A, void *y, int act, uint32_t *err, void *stream);
int strix_linear_qmix_experts_gather_swiglu(const void *x, const strix_qmix_view *w, const int32_t *ids, int64_t M,
                                            int64_t A, void *h, int act, uint32_t *err, void *stream);
/* strixite kernels/linear_q4.hpp:59-61 check_expert_error / report_expert_error. */
int strix_check_expert_error(const uint32_t *err, const char *what);
int strix_report_expert_error(const uint32_t e[3], const char *what);

/* ---- experts, grouped by expert (prefill, verify) ------------------------------------------------------------- */

/* strixite kernels/moe_grouped.hpp:43 moe_route_workspace_bytes. Returns 0 when M, A, E are out of range
 * (E <= 1023, A <= 64, M * A <= 2^20) and sets the error message. */
size_t strix_moe_route_workspace_bytes(int64_t M, int64_t A, int64_t E);
/* strixite kernels/moe_grouped.hpp:48-49 moe_group_routes. The workspace keeps the reference's layout
 * (moe_grouped.hip:63-81); inside a bucket the slots are in ascending order (a stable counting sort), so the
 * permutation is the same on every run. */
int strix_moe_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, void *ws, size_t ws_bytes,
                           uint32_t *err, void *stream);
/* strixite kernels/moe_grouped.hpp:53-55 / :65-67 linear_q{4,5}_experts_gather_grouped. */
int strix_linear_q4_experts_gather_grouped(const void *x, const strix_qview *w, int64_t E, const void *ws,
                                           size_t ws_bytes, int64_t M, int64_t A, void *y, int act, int math,
                                           void *stream);
int strix_linear_q5_experts_gather_grouped(const void *x, const strix_qview *w, int64_t E, const void *ws,
                                           size_t ws_bytes, int64_t M, int64_t A, void *y, int act, int math,
                                           void *stream);
/* strixite kernels/moe_grouped.hpp:60-62 / :68-70 linear_q{4,5}_experts_combine_grouped. partial: M * A * N floats. */
int strix_linear_q4_experts_combine_grouped(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                            const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                            int64_t M, int64_t A, void *y, int act, int math, void *stream);
int strix_linear_q5_experts_combine_grouped(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                            const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                            int64_t M, int64_t A, void *y, int act, int math, void *stream);
/* linear_q4_experts_combine_grouped without the `partial` argument: the M * A * N partial sums go to a fixed array of
 * STRIX_FIXED_PARTIAL_FLOATS floats (4 MiB) that is part of the library's device image. No counterpart in the
 * reference. It is for callers that have no buffer to give and may not allocate one at the call site: a host that has
 * handed all device memory to its own pool, or a latency-critical loop in which cudaMalloc (which can synchronize the
 * whole device) is ruled out. The call itself allocates nothing, on the host or the device.
 *   - Limit: M * A * N <= STRIX_FIXED_PARTIAL_FLOATS, else the call fails (1) before anything is enqueued; larger
 *     shapes use the variant above with a caller-provided buffer.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and caches it; make that first call outside any stream capture.
 *   - Every call on a device uses the same array. Nothing in it has to be zero beforehand (each partial sum that is
 *     read is written first by the same call), but two calls whose kernels can overlap in time - different streams,
 *     or different host threads without ordering - race on it; calls on one stream are safe. The array's address is looked up
 * once per device and cached: after cudaDeviceReset() the cached address is stale - do not call this entry again in a process
 * that reset the device. */
#define STRIX_FIXED_PARTIAL_FLOATS (1 << 20)
int strix_linear_q4_experts_combine_grouped_fixed(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                                  const float *coef, const void *ws, size_t ws_bytes, int64_t M,
                                                  int64_t A, void *y, int act, int math, void *stream);
/* Number of thread blocks of the tensor-core grouped GEMM that abandoned a bounded wait since the library was loaded:
 * 0 in a healthy run (their outputs are undefined otherwise). No counterpart in the reference. Synchronizes. */
unsigned int strix_umma_abort_count(void);
/* Launches of the grouped kernels that stored nothing because the workspace they were given had been grouped for another
 * (M * A, E) than the call stated (same byte size, other contents): the caller's outputs are untouched. 0 in a healthy run.
 * No counterpart in the reference (its kernels trust the workspace header). Synchronizes. */
unsigned int strix_workspace_refusal_count(void);
/* Diagnostics of the many-token tensor-core kernels: clock cycles their warp roles spent waiting on each other, summed
 * over thread blocks since the last reset; out32 = 2 kernels x 16 counters (index list in csrc/prefill_umma.cu).
 * No counterpart in the reference. Synchronizes. */
void strix_umma_wait_cycles(unsigned long long *out32, int reset);
/* The grouped pair over a stack with a format per expert. No counterpart in the reference. */
int strix_linear_qmix_experts_gather_grouped(const void *x, const strix_qmix_view *w, const void *ws, size_t ws_bytes,
                                             int64_t M, int64_t A, void *y, int act, int math, void *stream);
int strix_linear_qmix_experts_combine_grouped(const void *h, const strix_qmix_view *w, const int32_t *ids,
                                              const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                              int64_t M, int64_t A, void *y, int act, int math, void *stream);

/* ---- the MoE sublayer as one object ----------------------------------------------------------------------------
 * The per-layer driver of strixite runtime/qwen4exp.cpp:1126-1186 (Qwen4ExpSession::forward's MoE block, and
 * :1523-1542 for the draft head) with the session buffers it uses (:297-380): router projection -> moe_router ->
 * experts (per slot below grouped_min_tokens, grouped from there on) -> the shared expert -> gated add. The weights
 * stay the caller's (views); the layer owns only its workspaces. create/destroy allocate and free device memory;
 * forward is asynchronous on `stream` and allocates nothing. */

#define STRIX_SHARED_NONE 0      /* no shared expert */
#define STRIX_SHARED_STACKED 1   /* the shared expert is expert #E of the stacks (formats/merge_plan.cpp:29-42) */
#define STRIX_SHARED_SEPARATE 2  /* dense projections sh_gate_up / sh_down (runtime/qwen4exp.cpp:1167-1172) */
#define STRIX_SHARED_COEF_SIGMOID 0 /* the reference: sigmoid of the gate logit = router row E */
#define STRIX_SHARED_COEF_ONE 1     /* always-on shared expert: coefficient 1, no gate row in the router */
#define STRIX_ROUTER_F32 0
#define STRIX_ROUTER_BF16 1
#define STRIX_ROUTER_Q 2

typedef struct strix_moe_layer_desc {
    int64_t d, I, E, k;
    int act;               /* dtype of x and y */
    int shared_mode, shared_coef_mode;
    int router_kind;       /* rows: E + 1 when the shared expert is gated (sigmoid mode), else E */
    const void *router_w;  /* F32 / BF16 [rows, d], or NULL for STRIX_ROUTER_Q */
    int router_bits;       /* STRIX_ROUTER_Q: 4, 5, 6 or 8 */
    strix_qview router_q;
    const float *router_bias; /* optional [E]: added to the routed logits before selection */
    int experts_mixed;     /* 0: gate_up / down are uniform stacks in gate_up_bits / down_bits (4 or 5); 1: *_mix */
    int gate_up_bits, down_bits;
    strix_qview gate_up, down;          /* [Estack * 2I, d], [Estack * d, I]; Estack = E (+1 when stacked) */
    strix_qmix_view gate_up_mix, down_mix;
    int sh_gate_up_bits, sh_down_bits;  /* STRIX_SHARED_SEPARATE */
    strix_qview sh_gate_up, sh_down;    /* [2I, d], [d, I] */
    int64_t max_tokens;
    int64_t grouped_min_tokens; /* the grouped path runs from this many tokens (reference: 6, runtime/qwen4exp.hpp:266) */
    int math;                   /* STRIX_MATH_* of the grouped path */
    int64_t tensor_min_tokens;  /* math != STRIX_MATH_F32: forwards of at least this many tokens run the tensor-core path
                                 * (0 = the default, 64); below it the FP32 kernels run */
    int decode_impl;            /* forwards of <= 8 tokens: 0 = the single streaming kernel where the shapes allow it (d and I
                                 * multiples of 128, 4/5/6-bit projections in groups of 128, 8-bit ones in groups of 64 or
                                 * 128; activations are F16 operands there, |x| and |h| up to 65504), 1 = the
                                 * per-function kernels in the reference's sequence */
} strix_moe_layer_desc;

typedef struct strix_moe_layer strix_moe_layer;

int strix_moe_layer_create(const strix_moe_layer_desc *desc, strix_moe_layer **out);
void strix_moe_layer_destroy(strix_moe_layer *layer);
/* y[M, d] = MoE(x[M, d]) on device buffers. */
int strix_moe_layer_forward(strix_moe_layer *layer, const void *x, int64_t M, void *y, void *stream);
/* The same through HOST buffers: x is copied in, y and the six error words are copied back behind the kernels, one
 * synchronization at the end (the reference's read_back, runtime/qwen4exp.cpp:810-846). Page-locked caller buffers
 * (cudaHostAlloc / cudaHostRegister) are copied from and to directly; pageable ones pass through the layer's own page-locked
 * staging area with a host memcpy each way. A raised error word fails the call like report_router_error / report_expert_error. */
int strix_moe_layer_forward_host(strix_moe_layer *layer, const void *x_host, int64_t M, void *y_host, void *stream);
/* x[M, d] += MoE_l(x) for l = 0 .. n_layers - 1 (residual_add between layers); tmp [M, d] is scratch. */
int strix_moe_stack_forward(strix_moe_layer *const *layers, int64_t n_layers, void *x, int64_t M, void *tmp, void *stream);
/* The expert half of the layer for expert-parallel runs, one call per batch of routed slots that arrived on this
 * device: ids[n] is each slot's expert in THIS layer's stacks (0 .. Estack - 1) and its activation row is
 * rows[row_index[i], :] (the layer's activation dtype), or rows[i, :] when row_index is NULL - with row_index a token
 * routed to several local experts is sent once. partial[i, :] = W_down[ids[i]] * SwiGLU(W_gate_up[ids[i]] * row), FP32
 * [n, d] or (partial_f16 != 0) F16 [n, d] - one rounding of each FP32 sum, half the bytes - without the routing coefficient.
 * Groups the slots by expert and runs the tensor-core kernels; needs a layer created with math != STRIX_MATH_F32 over
 * uniform 4-bit stacks, and n <= max_tokens * (k + shared). Slots with an invalid id
 * raise the expert error words and are left unwritten; an id of -2 marks an absent slot (padding of a fixed-capacity list):
 * skipped without an error. No counterpart in the reference (which has no expert parallelism). */
int strix_moe_layer_experts_partial(strix_moe_layer *layer, const void *rows, const int32_t *row_index, const int32_t *ids,
                                    int64_t n, void *partial, int partial_f16, void *stream);
/* The ordered weighted sum of the reference's combine (kernels/moe_grouped.hpp:60-62, second half): y[m, :] = sum over a
 * ascending of coef[m, a] * partial[m * A + a, :], one rounding; a token with an id outside [0, E) gets a NaN row.
 * pos (optional, [M * A]): slot (m, a) is row pos[m * A + a] of partial instead of row m * A + a - partial rows that
 * came back from other devices in another order are summed where they lie. */
int strix_moe_combine_reduce(const float *partial, const int64_t *pos, const int32_t *ids, const float *coef, int64_t M,
                             int64_t A, int64_t E, int64_t N, void *y, int act, void *stream);
/* ---- expert parallelism: the device side of the token exchange. No counterpart in the reference (one device). -------------
 * A rank sends every token once to each rank that owns one of its experts, in FIXED-capacity blocks per (source, destination)
 * pair so that no size goes through the host: C rows [C, d] and strix_ep_meta_ints(C, Cs) int32 of metadata -
 * {n_rows, n_slots, 0, 0}, per row {first slot, slots}, per slot {local expert id, row, coefficient bits} - all in token
 * order. P <= 8 ranks. */
int64_t strix_ep_meta_ints(int64_t C, int64_t Cs);
/* Home rank, after moe_router: ids / coef [T, A] (id E = the stacked shared expert, kept home; an invalid id stays home with
 * local id -1 and poisons the token), owner / local_of [E + 1] (rank and local index of every routed expert) ->
 * rowtok [P, C] (the token behind every row to send), meta [P, MW], pos [T, P] (row of token t in destination r's block, or
 * -1). flags[0] / flags[1] receive the largest row / slot count that exceeded C / Cs (0 = the step fitted). scratch:
 * strix_ep_plan_scratch_ints(T) int32 of device memory the call may overwrite (per-segment counts of its three launches). */
int64_t strix_ep_plan_scratch_ints(int64_t T);
int strix_ep_plan(const int32_t *ids, const float *coef, int64_t T, int64_t A, int64_t E, const int32_t *owner,
                  const int32_t *local_of, int P, int rank, int64_t C, int64_t Cs, int32_t *rowtok, int32_t *meta, int32_t *pos,
                  uint32_t *flags, int32_t *scratch, void *stream);
/* rows_send[r, i, :] = x[rowtok[r, i], :] for the rows the plan counted. */
int strix_ep_gather_rows(const void *x, int64_t d, int act, const int32_t *rowtok, const int32_t *meta, int P, int64_t C,
                         int64_t Cs, void *rows_send, void *stream);
/* Expert rank: the received metadata [P, MW] as one slot list of P * Cs entries for strix_moe_layer_experts_partial -
 * slot_ids (-2 = absent, beyond a pair's count) and slot_row (the slot's row among the P * C received rows). */
int strix_ep_unpack(const int32_t *meta_recv, int P, int64_t C, int64_t Cs, int32_t *slot_ids, int32_t *slot_row,
                    void *stream);
/* Expert rank: summed[s, i, :] = sum over row (s, i)'s slots, in slot order, of coef * partial[slot, :] (FP32 sums of FP32 or,
 * with partial_f16, F16 partials - what strix_moe_layer_experts_partial wrote). */
int strix_ep_row_sum(const void *partial, int partial_f16, const int32_t *meta_recv, int P, int64_t C, int64_t Cs, int64_t d,
                     float *summed, void *stream);
/* Home rank: y[t, :] = the returned rows back[r, pos[t, r], :] (FP32, or F16 with back_f16) added in ascending r, rounded once to
 * `act`; NaN for a token with an id outside [0, E]. */
int strix_ep_home_sum(const void *back, int back_f16, const int32_t *pos, const int32_t *ids, int64_t T, int64_t A, int64_t E,
                      int P, int64_t C, int64_t d, void *y, int act, void *stream);
/* The exchange done by the kernels themselves, over memory the peers have mapped (NVLink peer stores) - no library all-to-all,
 * no staging copy. `*_ptrs` are device arrays of P addresses: rank r's receive buffer as this GPU sees it ([P, C, d] rows,
 * [P, MW] metadata, [P, C, d] returned sums; a rank's own entry is its local buffer). The ranks must meet at a barrier between
 * a push and the kernels that read what was pushed.
 *   strix_ep_push_rows     strix_ep_gather_rows with destination r's rows and the used part of its metadata block written into
 *                          block [rank] of r's buffers
 *   strix_ep_row_sum_push  strix_ep_row_sum with source s's sums written into block [rank] of s's `back` buffer, FP32 or
 *                          (back_f16) F16 - one rounding of each FP32 sum, half the bytes on the links */
int strix_ep_push_rows(const void *x, int64_t d, int act, const int32_t *rowtok, const int32_t *meta, int P, int rank, int64_t C,
                       int64_t Cs, const uint64_t *rows_ptrs, const uint64_t *meta_ptrs, void *stream);
int strix_ep_row_sum_push(const void *partial, int partial_f16, const int32_t *meta_recv, int P, int rank, int64_t C, int64_t Cs,
                          int64_t d, const uint64_t *back_ptrs, int back_f16, void *stream);

/* Device pointer of a named intermediate of the last forward - the reference's probes (runtime/qwen4exp.hpp:179-188):
 * "router_logits" f32 [M, E(+1)], "router_ids" i32 [M, A], "router_coef" f32 [M, A], "experts_h" [M, A, I],
 * "shared_h" [M, I], "shared_y" [M, d], "err" u32 [6] (router words 0..2, expert words 3..5), "group_ws", and
 * "decode_sync": the streaming decode kernel's barrier words, NULL when forwards of <= 8 tokens run the per-function
 * kernels instead (shapes or group sizes it does not take). */
const void *strix_moe_layer_probe(strix_moe_layer *layer, const char *name);
/* Zeroes the layer's error words. */
int strix_moe_layer_reset_errors(strix_moe_layer *layer, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* STRIXITE_B200_H */
