// The routed experts for a handful of tokens (decode, speculative verify), one launch per projection:
//   gather          y[m, a, :] = x[m, :] * W[ids[m, a]]^T
//   gather_swiglu   h[m, a, j] = silu(g_j) * u_j with g, u the gate and up rows of the merged [gate | up] projection
//   combine         y[m, :]    = sum_a coef[m, a] * (h[m, a, :] * W[ids[m, a]]^T)
// over E experts stacked [E * N, K] in one format or a format per expert. One warp per output row; an expert id
// outside [0, E) sets err {1, id, slot} and turns the slot's outputs (combine: the token's row) into NaN instead of
// reading out of bounds.
#include "common.cuh"

#include "strixite_b200.h"

namespace {

using namespace sb;

constexpr int kWarps = 8;

template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(kWarps * 32)
    experts_gather_kernel(const T *x, StackView w, int64_t E, const int32_t *ids, int64_t A, T *y, uint32_t *err) {
    const int lane = threadIdx.x & 31;
    const int64_t out_rows = SWIGLU ? w.N / 2 : w.N;
    // SWIGLU: two outputs per warp = four weight rows (gate j, j + 1, up j, j + 1) against one pass over the activations
    const int64_t j = ((int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5)) * (SWIGLU ? 2 : 1);
    if (j >= out_rows) return;
    const int64_t j1 = SWIGLU && j + 1 < out_rows ? j + 1 : j;  // an odd last output is computed twice and stored once
    const int64_t m = blockIdx.z, slot = m * A + blockIdx.y;
    const int32_t id = ids[slot];
    if (id < 0 || id >= E) {
        if (j == 0 && lane == 0) raise_err(err, (uint32_t)id, (uint32_t)slot);
        if (lane == 0) {
            st_act(y, slot * out_rows + j, qnan());
            if (j1 != j) st_act(y, slot * out_rows + j1, qnan());
        }
        return;
    }
    const int bits = w.bits_of(id);
    const int64_t gpr = w.K / w.G;
    const T *xr = x + m * w.K;
    by_bits(bits, [&](auto bc) {
        constexpr int BITS = decltype(bc)::value;
        const uint8_t *rows = w.rows(id, BITS);
        const int64_t rb = row_bytes(BITS, w.K), r0 = (int64_t)id * w.N;
        if constexpr (SWIGLU) {
            const int64_t rr[4] = {j, j1, j + out_rows, j1 + out_rows};
            const uint8_t *const row[4] = {rows + rr[0] * rb, rows + rr[1] * rb, rows + rr[2] * rb, rows + rr[3] * rb};
            const uint16_t *const sr[4] = {w.scale + (r0 + rr[0]) * gpr, w.scale + (r0 + rr[1]) * gpr, w.scale + (r0 + rr[2]) * gpr, w.scale + (r0 + rr[3]) * gpr};
            const uint16_t *const mr[4] = {w.minv + (r0 + rr[0]) * gpr, w.minv + (r0 + rr[1]) * gpr, w.minv + (r0 + rr[2]) * gpr, w.minv + (r0 + rr[3]) * gpr};
            float a[4];
            row_partial_n<BITS, 4>(row, sr, mr, xr, w.K, (int)w.G, lane, 32, a);
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = warp_sum(a[i]);
            // g and u as their store and reload would give them, h formed as the swiglu kernel forms it.
            if (lane == 0) {
                st_act(y, slot * out_rows + j, as_stored(silu_f(as_stored(a[0], y)), y) * as_stored(a[2], y));
                if (j1 != j) st_act(y, slot * out_rows + j1, as_stored(silu_f(as_stored(a[1], y)), y) * as_stored(a[3], y));
            }
        } else {
            float g = row_partial<BITS>(rows + j * rb, w.scale + (r0 + j) * gpr, w.minv + (r0 + j) * gpr, xr, w.K, (int)w.G, lane, 32);
            g = warp_sum(g);
            if (lane == 0) st_act(y, slot * out_rows + j, g);
        }
    });
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
    experts_combine_kernel(const T *h, StackView w, int64_t E, const int32_t *ids, const float *coef, int64_t A, T *y,
                           uint32_t *err) {
    const int lane = threadIdx.x & 31;
    // four output rows per warp: all read the same h chunks, which are the L1 traffic that bounds this kernel
    constexpr int NR = 4;
    const int64_t n = ((int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5)) * NR;
    if (n >= w.N) return;
    int64_t nn[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) nn[r] = n + r < w.N ? n + r : n;  // rows past the end repeat row n and are not stored
    const int64_t m = blockIdx.y;
    int64_t first_bad = -1;
    for (int64_t a = 0; a < A; ++a) {
        const int32_t id = ids[m * A + a];
        if ((id < 0 || id >= E) && first_bad < 0) first_bad = a;
    }
    if (first_bad >= 0) {
        if (n == 0 && lane == 0) raise_err(err, (uint32_t)ids[m * A + first_bad], (uint32_t)(m * A + first_bad));
        if (lane == 0)
            for (int r = 0; r < NR; ++r)
                if (r == 0 || nn[r] != n) st_act(y, m * w.N + nn[r], qnan());
        return;
    }
    const int64_t gpr = w.K / w.G;
    float acc[NR] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t a = 0; a < A; ++a) {
        const int32_t id = ids[m * A + a];
        const int bits = w.bits_of(id);
        by_bits(bits, [&](auto bc) {
            constexpr int BITS = decltype(bc)::value;
            const uint8_t *rows = w.rows(id, BITS);
            const int64_t rb = row_bytes(BITS, w.K), r0 = (int64_t)id * w.N;
            const uint8_t *const row[NR] = {rows + nn[0] * rb, rows + nn[1] * rb, rows + nn[2] * rb, rows + nn[3] * rb};
            const uint16_t *const sr[NR] = {w.scale + (r0 + nn[0]) * gpr, w.scale + (r0 + nn[1]) * gpr, w.scale + (r0 + nn[2]) * gpr, w.scale + (r0 + nn[3]) * gpr};
            const uint16_t *const mr[NR] = {w.minv + (r0 + nn[0]) * gpr, w.minv + (r0 + nn[1]) * gpr, w.minv + (r0 + nn[2]) * gpr, w.minv + (r0 + nn[3]) * gpr};
            float p[NR];
            row_partial_n<BITS, NR>(row, sr, mr, h + (m * A + a) * w.K, w.K, (int)w.G, lane, 32, p);
#pragma unroll
            for (int r = 0; r < NR; ++r) acc[r] = fmaf(coef[m * A + a], p[r], acc[r]);
        });
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = warp_sum(acc[r]);
    if (lane == 0)
        for (int r = 0; r < NR; ++r)
            if (r == 0 || nn[r] != n) st_act(y, m * w.N + nn[r], acc[r]);
}

enum Op { kGather, kGatherSwiglu, kCombine };

int experts(const char *fn, Op op, const void *x, const StackView &w, int64_t E, const int32_t *ids, const float *coef,
            int64_t M, int64_t A, void *y, int act, uint32_t *err, void *stream) {
    SB_CHECK(x != nullptr && y != nullptr && ids != nullptr && err != nullptr, fn, ": null pointer (x=", x, ", y=", y, ", ids=",
             (const void *)ids, ", err=", (const void *)err, ")");
    SB_CHECK(op != kCombine || coef != nullptr, fn, ": null coef");
    SB_CHECK(w.q != nullptr && w.scale != nullptr && w.minv != nullptr, fn, ": null weight pointer (q=", (const void *)w.q,
             ", scale=", (const void *)w.scale, ", min=", (const void *)w.minv, ")");
    SB_CHECK(group_ok(w.G), fn, ": group size ", w.G, " unsupported (32, 64 or 128)");
    SB_CHECK(w.N >= 1 && w.N <= 0x7fffffff, fn, ": N = ", w.N, " rows per expert, expected 1..2^31-1");
    SB_CHECK(w.K >= w.G && w.K <= (1 << 24) && w.K % w.G == 0, fn, ": K = ", w.K, " must be a positive multiple of group size ",
             w.G, " and <= 2^24");
    if (w.bits_tab == nullptr) {
        SB_CHECK(bits_ok(w.bits), fn, ": ", w.bits, " bits, expected 4, 5, 6 or 8");
        SB_CHECK(w.bits != 5 || w.K % 128 == 0, fn, ": Q5 K = ", w.K, " is not a multiple of 128 (the layout's)");
        SB_CHECK(w.bits != 6 || w.K % 64 == 0, fn, ": Q6 K = ", w.K, " is not a multiple of 64 (the layout's)");
    } else {
        SB_CHECK(w.q_off != nullptr, fn, ": per-expert formats need the q_off table");
        SB_CHECK(w.K % 128 == 0, fn, ": mixed-format experts need K % 128 == 0 (Q5 rows), got ", w.K);
    }
    SB_CHECK(aligned16(w.q) && aligned16(x), fn, ": code array ", (const void *)w.q, " and input ", x, " must be 16-byte aligned");
    SB_CHECK(E >= 1, fn, ": E = ", E, " experts");
    SB_CHECK(M >= 1 && M <= 65535, fn, ": M (tokens) = ", M, ", expected 1..65535");
    SB_CHECK(A >= 1 && A <= 64 && A <= E, fn, ": A (active experts per token) = ", A, ", expected 1..min(64, E=", E, ")");
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SB_CHECK(op != kGatherSwiglu || w.N % 2 == 0, fn, ": SwiGLU gather needs an even row count per expert ([gate | up]), got ", w.N);
    const int64_t es = act_size(act), out_rows = op == kGatherSwiglu ? w.N / 2 : w.N;
    const int64_t in_bytes = (op == kCombine ? M * A : M) * w.K * es, out_bytes = (op == kCombine ? M : M * A) * out_rows * es;
    SB_CHECK(apart(y, out_bytes, x, in_bytes), fn, ": output [", y, ", +", out_bytes, " B) overlaps input [", x, ", +", in_bytes, " B)");
    auto st = static_cast<cudaStream_t>(stream);
    const unsigned bx = (unsigned)((out_rows + kWarps - 1) / kWarps);
    const dim3 block(kWarps * 32);
    auto go = [&](auto tag) {
        using T = decltype(tag);
        if (op == kCombine)  // four output rows per warp
            experts_combine_kernel<T><<<dim3((unsigned)((out_rows + 4 * kWarps - 1) / (4 * kWarps)), (unsigned)M), block, 0, st>>>((const T *)x, w, E, ids, coef, A, (T *)y, err);
        else if (op == kGatherSwiglu)  // two outputs per warp
            experts_gather_kernel<T, true><<<dim3((unsigned)((out_rows + 2 * kWarps - 1) / (2 * kWarps)), (unsigned)A, (unsigned)M), block, 0, st>>>((const T *)x, w, E, ids, A, (T *)y, err);
        else
            experts_gather_kernel<T, false><<<dim3(bx, (unsigned)A, (unsigned)M), block, 0, st>>>((const T *)x, w, E, ids, A, (T *)y, err);
    };
    if (act == kF32) go(float{});
    else go(uint16_t{});
    SB_LAUNCH_OK(fn, " ", act_name(act), " M=", M, " A=", A, " E=", E, " N=", w.N, " K=", w.K, " G=", w.G);
    return 0;
}

int uniform(const char *fn, int bits, Op op, const void *x, const strix_qview *w, int64_t E, const int32_t *ids,
            const float *coef, int64_t M, int64_t A, void *y, int act, uint32_t *err, void *stream) {
    SB_CHECK(w != nullptr, fn, ": null weight view");
    SB_CHECK(E >= 1 && w->N % E == 0, fn, ": weight has ", w->N, " rows, not a multiple of E = ", E, " experts");
    const StackView sv{w->q, w->scale, w->minv, nullptr, nullptr, bits, w->N / E, w->K, w->G};
    return experts(fn, op, x, sv, E, ids, coef, M, A, y, act, err, stream);
}

int mixed(const char *fn, Op op, const void *x, const strix_qmix_view *w, const int32_t *ids, const float *coef, int64_t M,
          int64_t A, void *y, int act, uint32_t *err, void *stream) {
    SB_CHECK(w != nullptr && w->bits != nullptr && w->q_off != nullptr, fn, ": null view, format table or offset table");
    const StackView sv{w->q, w->scale, w->minv, w->bits, w->q_off, 0, w->N, w->K, w->G};
    return experts(fn, op, x, sv, w->E, ids, coef, M, A, y, act, err, stream);
}

}  // namespace

extern "C" {

int strix_linear_q4_experts_gather(const void *x, const strix_qview *w, int64_t E, const int32_t *ids, int64_t M,
                                   int64_t A, void *y, int act, uint32_t *err, void *stream) {
    return uniform("linear_q4_experts_gather", 4, kGather, x, w, E, ids, nullptr, M, A, y, act, err, stream);
}
int strix_linear_q4_experts_combine(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                    const float *coef, int64_t M, int64_t A, void *y, int act, uint32_t *err,
                                    void *stream) {
    return uniform("linear_q4_experts_combine", 4, kCombine, h, w, E, ids, coef, M, A, y, act, err, stream);
}
int strix_linear_q4_experts_gather_swiglu(const void *x, const strix_qview *w, int64_t E, const int32_t *ids,
                                          int64_t M, int64_t A, void *h, int act, uint32_t *err, void *stream) {
    return uniform("linear_q4_experts_gather_swiglu", 4, kGatherSwiglu, x, w, E, ids, nullptr, M, A, h, act, err, stream);
}
int strix_linear_q5_experts_gather(const void *x, const strix_qview *w, int64_t E, const int32_t *ids, int64_t M,
                                   int64_t A, void *y, int act, uint32_t *err, void *stream) {
    return uniform("linear_q5_experts_gather", 5, kGather, x, w, E, ids, nullptr, M, A, y, act, err, stream);
}
int strix_linear_q5_experts_combine(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                    const float *coef, int64_t M, int64_t A, void *y, int act, uint32_t *err,
                                    void *stream) {
    return uniform("linear_q5_experts_combine", 5, kCombine, h, w, E, ids, coef, M, A, y, act, err, stream);
}
int strix_linear_q5_experts_gather_swiglu(const void *x, const strix_qview *w, int64_t E, const int32_t *ids,
                                          int64_t M, int64_t A, void *h, int act, uint32_t *err, void *stream) {
    return uniform("linear_q5_experts_gather_swiglu", 5, kGatherSwiglu, x, w, E, ids, nullptr, M, A, h, act, err, stream);
}
int strix_linear_qmix_experts_gather(const void *x, const strix_qmix_view *w, const int32_t *ids, int64_t M,
                                     int64_t A, void *y, int act, uint32_t *err, void *stream) {
    return mixed("linear_qmix_experts_gather", kGather, x, w, ids, nullptr, M, A, y, act, err, stream);
}
int strix_linear_qmix_experts_combine(const void *h, const strix_qmix_view *w, const int32_t *ids, const float *coef,
                                      int64_t M, int64_t A, void *y, int act, uint32_t *err, void *stream) {
    return mixed("linear_qmix_experts_combine", kCombine, h, w, ids, coef, M, A, y, act, err, stream);
}
int strix_linear_qmix_experts_gather_swiglu(const void *x, const strix_qmix_view *w, const int32_t *ids, int64_t M,
                                            int64_t A, void *h, int act, uint32_t *err, void *stream) {
    return mixed("linear_qmix_experts_gather_swiglu", kGatherSwiglu, x, w, ids, nullptr, M, A, h, act, err, stream);
}

}  // extern "C"
