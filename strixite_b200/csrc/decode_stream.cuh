// Parameters of the streaming decode kernel (decode_stream.cu), filled by the layer object.
#pragma once

#include "common.cuh"

#include "strixite_b200.h"

namespace sb {

struct StreamParams {
    int M, d, I, E, k, A, R, Estack;
    int act, shared_mode, gated;
    int planes;      // F16 planes per activation value: 2 (value = hi + lo) for at most two_plane_tokens FP32 tokens, else 1
    int two_plane_tokens;  // 0..4, set by the plan (what shared memory allows)
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
    uint8_t *hrec;   // hidden records for the down projection: (M * A + M) * planes records of rec_bytes
    uint32_t *err;   // router words 0..2, expert words 3..5
    uint32_t *sync;  // 4 words, zero before the first launch: two barrier counters, CTAs done, abort
    int rec_bytes;   // I * 2 + 64
    int n_rec;       // records in use for M tokens
    int n_rec_max;   // records hrec holds (the most any token count of the plan needs)
    int smem_bytes;
    int format_set;  // set by the caller, picks the kernel variant: 0 = every projection 4-bit; 1 = 4-bit experts and an 8-bit
                     // separate shared expert in groups of 64; 2 = anything else the plan accepts
};

// 1 if the kernel takes the shapes and formats for up to `tokens` tokens (fills rec_bytes, n_rec_max, smem_bytes).
// min_nibble_G / min_q8_G: the smallest group size among the 4/5/6-bit and the 8-bit projections it will stream.
int decode_stream_plan(StreamParams &p, int tokens, int min_nibble_G, int min_q8_G);
// Sets M and what follows from it (planes, n_rec) for one forward of M <= the plan's tokens.
void decode_stream_set_tokens(StreamParams &p, int M);
int decode_stream_launch(const char *fn, const StreamParams &p, cudaStream_t stream);

}  // namespace sb
