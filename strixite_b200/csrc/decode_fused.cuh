// Parameters of the fused decode kernel (decode_fused.cu), filled by the layer object.
#pragma once

#include "common.cuh"

#include "strixite_b200.h"

namespace sb {

struct DecodeParams {
    int M, d, I, E, k, A, R, Estack;
    int act, shared_mode, gated;
    const void *x;   // [M, d]
    void *y;         // [M, d]
    int router_kind, router_bits;
    const void *router_w;
    strix_qview router_q;
    const float *router_bias;
    StackView gate_up, down;  // N = 2I and d rows per expert
    int sh_gate_up_bits, sh_down_bits;
    strix_qview sh_gate_up, sh_down;
    float *logits;   // [M, R]
    int32_t *ids;    // [M, A]
    float *coef;     // [M, A]
    void *hh;        // [M, A, I] the routed experts' hidden, activation dtype
    void *sh_h;      // [M, I] the separate shared expert's hidden, or null
    uint8_t *hrec;   // (M * A + M) records of hrec_bytes: per BF16 plane, h in the tensor-core k order, then per plane I / 8 partial sums
    int hrec_bytes;
    uint32_t *err;   // router words 0..2, expert words 3..5
    uint32_t *sync;  // 16 words, zero before the first launch: two barrier counters, CTAs done, abort; [8..15] phase timestamps
    // shared-memory plan, computed on the host (decode_fused_plan)
    int smem_bytes;
    int fmask;  // expert formats present (bit 0: 4 bits, 1: 5, 2: 6, 3: 8), set by the caller: selects the kernel variant
    int g128_4bit;  // every 4-bit projection (experts, separate shared expert) uses groups of 128 codes, set by the caller
    int gu_nk;  // K slices (= warps) per gate/up tile
    int gu_row_stride, gu_scale_bytes, gu_stage_bytes, gu_stages;
    int gu_active, gu_depth;  // consumer warps in use and stages per warp (gu_stages = gu_active * gu_depth)
    int dn_row_stride, dn_scale_bytes, dn_stage_bytes_fixed;  // + col_max * hrec_bytes at run time
};

// 1 if the shapes fit the kernel (and its shared-memory plan has at least two stages); fills the plan.
int decode_fused_plan(DecodeParams &p, int max_bits_gate_up, int max_bits_down, int min_G);
int decode_fused_launch(const char *fn, const DecodeParams &p, cudaStream_t stream);

}  // namespace sb
