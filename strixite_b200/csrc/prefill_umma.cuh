// The many-token expert FFN on tcgen05 tensor cores (prefill_umma.cu), as the layer object drives it.
#pragma once

#include "common.cuh"
#include "grouped.cuh"
#include "strixite_b200.h"

namespace sb {

struct PrefillPlan;  // tensor maps of the weight stacks, the bucket-ordered activation buffers and the tile table

// Uniform 4-bit stacks with d % 256 == 0 and I % 128 == 0.
bool prefill_supported(const strix_moe_layer_desc &d);
int prefill_create(const strix_moe_layer_desc &d, int64_t A, int64_t Estack, int64_t router_rows, PrefillPlan **out);
void prefill_destroy(PrefillPlan *p);
// BF16 activations with a BF16 router: the router projection runs on the tensor cores too.
bool prefill_has_dense_router(const PrefillPlan *p);
// bias (optional, n_bias entries) is added to rows r < n_bias.
int prefill_router_logits(PrefillPlan *p, const void *x, int64_t M, float *logits, const float *bias, int64_t n_bias, cudaStream_t st);
// Tiles -> bucket-ordered F16 activations -> gate/up + SwiGLU -> down: FP32 partial[slot, d] for every slot with a
// valid expert. `ws` is the grouping workspace of moe_group_routes for (M, A, Estack).
// Slot s reads activation row row_index[s], or s / A (one row per token) when row_index is null.
// half_partial: partial is F16 [slots, d] (one rounding of each FP32 sum; half the bytes to write and to combine) instead of FP32.
int prefill_experts(PrefillPlan *p, const void *x, const int32_t *row_index, int act, const int32_t *ws, int64_t M, int64_t A, void *partial,
                    bool half_partial, cudaStream_t st);
// y[M, N] (FP32) = x[M, K] (BF16) * w[N, K]^T (BF16) + bias[n < n_bias] on the tensor cores; dense_bf16_ok says whether the
// shape and alignment qualify (M >= 64, K % 64 == 0, 16-byte aligned pointers).
bool dense_bf16_ok(const void *x, const void *w, int64_t M, int64_t N, int64_t K);
int dense_bf16(const char *fn, const void *x, const uint16_t *w, float *y, int64_t M, int64_t N, int64_t K, const float *bias, int64_t n_bias,
               cudaStream_t st);
// CTAs of these kernels that gave up on a bounded wait since the library was loaded.
unsigned int prefill_aborts();
// Forwards refused because the grouping workspace was built for other sizes than the call stated.
unsigned int prefill_ws_refusals();
// Wait-cycle counters of the FFN kernels' roles, 2 x 16 words (diagnostics; see prefill_umma.cu). Synchronizes.
void prefill_cycles(unsigned long long *out, bool reset);

// y[m, :] = sum_a coef[m, a] * partial[m * A + a, :] in ascending a; NaN rows for tokens with an invalid id (grouped.cu).
// pos: slot (m, a) is row pos[m * A + a] of partial; half_partial: the partial sums are F16 (prefill_experts with half_partial).
int combine_reduce(const char *fn, const void *partial, const int32_t *ids, const float *coef, int64_t M, int64_t A, int64_t E, int64_t N,
                   void *y, int act, cudaStream_t st, const int64_t *pos = nullptr, bool half_partial = false);

}  // namespace sb
