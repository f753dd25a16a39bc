// TEST INFRASTRUCTURE - NOT PRODUCT CODE.
//
// The timed CPU baseline: the same arithmetic as moe_oracle.cpp, multi-threaded (OpenMP) and dequantizing on the
// fly in the form the reference kernels use, acc = fma(s, sum x*q, fma(m, sum x, acc)) per 32-code chunk
// (kernels/linear_q4.hip:88-94), FP32 accumulation. Built with -O3 -march=native; only the bench's cpu_baseline /
// reference arm and the tests that compare it with the double-accumulating oracle call it.
//
// Threads: output rows for the dense and per-slot (decode) forms; experts for the grouped (prefill) form, where an
// expert's row is decoded once and applied to every slot routed to it - the reference's moe_grouped.hpp:3-11 idea.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#include <omp.h>

namespace {

inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0x007fffffu) ? 0x0040u : 0u));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float act_load(const void *p, int64_t i, int act) {
    return act == 0 ? static_cast<const float *>(p)[i] : bf16_to_f32(static_cast<const uint16_t *>(p)[i]);
}
inline void act_store(void *p, int64_t i, float v, int act) {
    if (act == 0) static_cast<float *>(p)[i] = v;
    else static_cast<uint16_t *>(p)[i] = f32_to_bf16(v);
}
inline float as_stored(float v, int act) { return act == 0 ? v : bf16_to_f32(f32_to_bf16(v)); }
inline float silu(float v) { return v / (1.0f + expf(-v)); }
inline int64_t row_bytes(int bits, int64_t K) {
    return bits == 4 ? K / 2 : bits == 5 ? K / 2 + K / 8 : bits == 6 ? K / 2 + K / 4 : K;
}

// The 32 codes of chunk c (codes 32c .. 32c+31) of a row, as floats.
inline void chunk_codes(int bits, const uint8_t *row, int64_t K, int64_t c, float *out) {
    if (bits == 8) {
        for (int i = 0; i < 32; ++i) out[i] = (float)row[c * 32 + i];
        return;
    }
    const uint8_t *lo = row + c * 16;
    for (int i = 0; i < 16; ++i) out[2 * i] = (float)(lo[i] & 0xF), out[2 * i + 1] = (float)(lo[i] >> 4);
    if (bits == 5) {
        uint32_t hb;
        std::memcpy(&hb, row + K / 2 + c * 4, 4);
        for (int i = 0; i < 32; ++i) out[i] += (float)(((hb >> i) & 1u) << 4);
    } else if (bits == 6) {
        uint64_t hb;
        std::memcpy(&hb, row + K / 2 + c * 8, 8);
        for (int i = 0; i < 32; ++i) out[i] += (float)(((hb >> (2 * i)) & 3u) << 4);
    }
}

// x rows as FP32, converted once.
std::vector<float> widen(const void *x, int64_t n, int act) {
    std::vector<float> v((size_t)n);
    for (int64_t i = 0; i < n; ++i) v[i] = act_load(x, i, act);
    return v;
}

// dot of one quantized row with R activation rows (xs[r] + K floats each), the kernels' per-chunk form.
inline void row_dots(int bits, const uint8_t *row, const uint16_t *srow, const uint16_t *mrow, int64_t K, int64_t G,
                     const float *const *xs, int R, float *out) {
    for (int r = 0; r < R; ++r) out[r] = 0.f;
    float codes[32];
    for (int64_t c = 0; c < K / 32; ++c) {
        chunk_codes(bits, row, K, c, codes);
        const float s = bf16_to_f32(srow[c * 32 / G]), m = bf16_to_f32(mrow[c * 32 / G]);
        for (int r = 0; r < R; ++r) {
            const float *x = xs[r] + c * 32;
            float dot = 0.f, xsum = 0.f;
            for (int i = 0; i < 32; ++i) dot += x[i] * codes[i], xsum += x[i];
            out[r] += s * dot + m * xsum;
        }
    }
}

struct Stack {
    const uint8_t *q;
    const uint16_t *scale, *minv;
    const uint8_t *bits_tab;
    const int64_t *q_off;
    int bits;
    int64_t N, K, G;
    int bits_of(int64_t e) const { return bits_tab ? bits_tab[e] : bits; }
    const uint8_t *row(int64_t e, int64_t n) const {
        const int b = bits_of(e);
        return q + (q_off ? q_off[e] : e * N * row_bytes(b, K)) + n * row_bytes(b, K);
    }
    const uint16_t *srow(int64_t e, int64_t n) const { return scale + (e * N + n) * (K / G); }
    const uint16_t *mrow(int64_t e, int64_t n) const { return minv + (e * N + n) * (K / G); }
};

// Slots grouped by expert (stable): experts[] with their slot lists. Invalid ids are skipped (the callers NaN them).
struct Groups {
    std::vector<int32_t> expert;
    std::vector<std::vector<int64_t>> slots;
};
Groups group_slots(const int32_t *ids, int64_t S, int64_t E) {
    std::vector<int32_t> where((size_t)E, -1);
    Groups g;
    for (int64_t s = 0; s < S; ++s) {
        const int32_t id = ids[s];
        if (id < 0 || id >= E) continue;
        if (where[id] < 0) where[id] = (int32_t)g.expert.size(), g.expert.push_back(id), g.slots.emplace_back();
        g.slots[where[id]].push_back(s);
    }
    return g;
}

}  // namespace

extern "C" {

int orc_fast_threads() { return omp_get_max_threads(); }

void orc_fast_linear_q(int bits, const void *x, int act, const uint8_t *q, const uint16_t *scale, const uint16_t *minv,
                       int64_t N, int64_t K, int64_t G, void *y, int out_act, int64_t M) {
    const std::vector<float> xf = widen(x, M * K, act);
    const int64_t rb = row_bytes(bits, K);
    constexpr int RB = 16;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m0 = 0; m0 < M; m0 += RB) {
            const int R = (int)(M - m0 < RB ? M - m0 : RB);
            const float *xs[RB];
            float out[RB];
            for (int r = 0; r < R; ++r) xs[r] = xf.data() + (m0 + r) * K;
            row_dots(bits, q + n * rb, scale + n * (K / G), minv + n * (K / G), K, G, xs, R, out);
            for (int r = 0; r < R; ++r) act_store(y, (m0 + r) * N + n, out[r], out_act);
        }
    }
}

void orc_fast_linear_w(const void *x, int act, const void *w, int wtype, void *y, int out_act, int64_t M, int64_t N,
                       int64_t K) {
    const std::vector<float> xf = widen(x, M * K, act);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        std::vector<float> wr((size_t)K);
        for (int64_t k = 0; k < K; ++k) wr[k] = act_load(w, n * K + k, wtype);
        for (int64_t m = 0; m < M; ++m) {
            const float *xr = xf.data() + m * K;
            float acc = 0.f;
            for (int64_t k = 0; k < K; ++k) acc += xr[k] * wr[k];
            act_store(y, m * N + n, acc, out_act);
        }
    }
}

// Gather with the SwiGLU epilogue (kernels/linear_q4.hip:205-233): h [M, A, I], N = 2I rows per expert.
void orc_fast_experts_gather_swiglu(int bits, const uint8_t *bits_tab, const int64_t *q_off, const void *x,
                                    const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t E,
                                    int64_t N, int64_t K, int64_t G, const int32_t *ids, int64_t M, int64_t A,
                                    void *h, int act) {
    const Stack st{q, scale, minv, bits_tab, q_off, bits, N, K, G};
    const std::vector<float> xf = widen(x, M * K, act);
    const int64_t I = N / 2, S = M * A;
    for (int64_t s = 0; s < S; ++s)
        if (ids[s] < 0 || ids[s] >= E)
            for (int64_t j = 0; j < I; ++j) act_store(h, s * I + j, std::numeric_limits<float>::quiet_NaN(), act);
    const Groups g = group_slots(ids, S, E);
    const int64_t n_groups = (int64_t)g.expert.size();
    // (expert, row) pairs are the parallel units: plenty of them even at one token.
#pragma omp parallel for schedule(dynamic, 16) collapse(2)
    for (int64_t gi = 0; gi < n_groups; ++gi)
        for (int64_t j = 0; j < I; ++j) {
            const int32_t e = g.expert[gi];
            const std::vector<int64_t> &sl = g.slots[gi];
            constexpr int RB = 16;
            for (size_t s0 = 0; s0 < sl.size(); s0 += RB) {
                const int R = (int)(sl.size() - s0 < RB ? sl.size() - s0 : RB);
                const float *xs[RB];
                float gv[RB], uv[RB];
                for (int r = 0; r < R; ++r) xs[r] = xf.data() + (sl[s0 + r] / A) * K;
                row_dots(st.bits_of(e), st.row(e, j), st.srow(e, j), st.mrow(e, j), K, G, xs, R, gv);
                row_dots(st.bits_of(e), st.row(e, j + I), st.srow(e, j + I), st.mrow(e, j + I), K, G, xs, R, uv);
                for (int r = 0; r < R; ++r) {
                    const float gs = as_stored(gv[r], act), us = as_stored(uv[r], act);
                    act_store(h, sl[s0 + r] * I + j, as_stored(silu(gs), act) * us, act);
                }
            }
        }
}

// Combine (kernels/moe_grouped.hip:456-472): per-slot dots, then y[m, n] = sum_a fma(coef, dot, v) in slot order.
void orc_fast_experts_combine(int bits, const uint8_t *bits_tab, const int64_t *q_off, const void *h, const uint8_t *q,
                              const uint16_t *scale, const uint16_t *minv, int64_t E, int64_t N, int64_t K, int64_t G,
                              const int32_t *ids, const float *coef, int64_t M, int64_t A, void *y, int act) {
    const Stack st{q, scale, minv, bits_tab, q_off, bits, N, K, G};
    const int64_t S = M * A;
    const std::vector<float> hf = widen(h, S * K, act);
    std::vector<float> partial((size_t)(S * N), 0.f);
    const Groups g = group_slots(ids, S, E);
    const int64_t n_groups = (int64_t)g.expert.size();
#pragma omp parallel for schedule(dynamic, 16) collapse(2)
    for (int64_t gi = 0; gi < n_groups; ++gi)
        for (int64_t n = 0; n < N; ++n) {
            const int32_t e = g.expert[gi];
            const std::vector<int64_t> &sl = g.slots[gi];
            constexpr int RB = 16;
            for (size_t s0 = 0; s0 < sl.size(); s0 += RB) {
                const int R = (int)(sl.size() - s0 < RB ? sl.size() - s0 : RB);
                const float *xs[RB];
                float out[RB];
                for (int r = 0; r < R; ++r) xs[r] = hf.data() + sl[s0 + r] * K;
                row_dots(st.bits_of(e), st.row(e, n), st.srow(e, n), st.mrow(e, n), K, G, xs, R, out);
                for (int r = 0; r < R; ++r) partial[(size_t)(sl[s0 + r] * N + n)] = out[r];
            }
        }
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        bool ok = true;
        for (int64_t a = 0; a < A; ++a) ok = ok && ids[m * A + a] >= 0 && ids[m * A + a] < E;
        for (int64_t n = 0; n < N; ++n) {
            float v = 0.f;
            for (int64_t a = 0; a < A; ++a) v = std::fmaf(coef[m * A + a], partial[(size_t)((m * A + a) * N + n)], v);
            act_store(y, m * N + n, ok ? v : std::numeric_limits<float>::quiet_NaN(), act);
        }
    }
}

}  // extern "C"
