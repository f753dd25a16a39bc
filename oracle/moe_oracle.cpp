// TEST INFRASTRUCTURE - NOT PRODUCT CODE.
//
// CPU restatement of strixite's quantized-MoE FFN arithmetic, used only as the checker for the CUDA path
// (tests, the smoke check, and the bench's cpu_baseline leg). Nothing in the product package may call it.
//
// Every function cites the reference file:line it follows (paths relative to the strixite tree). The
// quantizer part is pinned against the reference's own formats/q{4,5,6,8}.cpp compiled unchanged (see
// ref_shim.cpp and the committed golden vectors); the layer part has no golden vectors upstream (the
// reference ships no tests/ or reference/ directory), so for those functions parity is UNPINNED beyond the
// in-tree invariants the tests assert (fused == unfused, sum(coef) == 1, NaN rows + err words on bad ids).
//
// Numerics: dots are accumulated in double over the dequantized FP32 weights (the values
// formats/q4.cpp:121-134 defines as "the exact values the kernel must use"), then rounded once to FP32.
// The reference kernels accumulate in FP32 in a lane-dependent order, so layer parity is a tolerance
// (2e-3 of the row maximum), never bitwise; integer outputs (ids, permutations, codes) are bit-exact.

#include <cfenv>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

namespace {

// formats/q4.cpp:14-27 - RNE with NaN quieting (sign kept).
inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0x007fffffu) ? 0x0040u : 0u));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline float qnan() { return std::numeric_limits<float>::quiet_NaN(); }

// Act: 0 = F32, 1 = BF16 bits (kernels/norm.hpp:20).
inline float act_load(const void *p, int64_t i, int act) {
    return act == 0 ? static_cast<const float *>(p)[i] : bf16_to_f32(static_cast<const uint16_t *>(p)[i]);
}
inline void act_store(void *p, int64_t i, float v, int act) {
    if (act == 0) static_cast<float *>(p)[i] = v;
    else static_cast<uint16_t *>(p)[i] = f32_to_bf16(v);
}
inline float as_stored(float v, int act) { return act == 0 ? v : bf16_to_f32(f32_to_bf16(v)); }

inline int qmax_of(int bits) { return (1 << bits) - 1; }

// Row bytes: formats/q4.hpp:5, q5.hpp:31, q6.hpp:31, q8.hpp:6.
inline int64_t row_bytes(int bits, int64_t K) {
    switch (bits) {
        case 4: return K / 2;
        case 5: return K / 2 + K / 8;
        case 6: return K / 2 + K / 4;
        default: return K;
    }
}

// formats/q5.hpp:33-36, q6.hpp:33-36, q4.cpp:130, q8.cpp (one byte per code).
inline int code_at(int bits, const uint8_t *row, int64_t K, int64_t k) {
    if (bits == 8) return row[k];
    const int lo = (row[k / 2] >> (4 * (k % 2))) & 0xF;
    if (bits == 4) return lo;
    if (bits == 5) return lo | (((row[K / 2 + k / 8] >> (k % 8)) & 0x1) << 4);
    return lo | (((row[K / 2 + k / 4] >> (2 * (k % 4))) & 0x3) << 4);
}

inline void put_code(int bits, uint8_t *row, int64_t K, int64_t k, int code) {
    if (bits == 8) {
        row[k] = (uint8_t)code;
        return;
    }
    row[k / 2] |= (uint8_t)((code & 0xF) << (4 * (k % 2)));
    if (bits == 5) row[K / 2 + k / 8] |= (uint8_t)(((code >> 4) & 0x1) << (k % 8));
    if (bits == 6) row[K / 2 + k / 4] |= (uint8_t)(((code >> 4) & 0x3) << (2 * (k % 4)));
}

// Dequantized row into w[K]: code * s then + m, two roundings (formats/q4.cpp:121-133: no FMA contraction;
// this translation unit is compiled with -ffp-contract=off).
inline void dequant_row(int bits, const uint8_t *row, const uint16_t *srow, const uint16_t *mrow, int64_t K, int64_t G,
                        float *w) {
    for (int64_t k = 0; k < K; ++k) {
        const float s = bf16_to_f32(srow[k / G]), m = bf16_to_f32(mrow[k / G]);
        const float p = (float)code_at(bits, row, K, k) * s;
        w[k] = p + m;
    }
}

inline double dot_row(const float *w, const void *x, int64_t xoff, int64_t K, int act) {
    double acc = 0.0;
    for (int64_t k = 0; k < K; ++k) acc += (double)act_load(x, xoff + k, act) * (double)w[k];
    return acc;
}

inline float silu(float v) { return v / (1.0f + std::exp(-v)); }  // kernels/swiglu.hip:22 (expf)

struct Stack {  // E experts stacked; uniform (bits_tab == null) or per-expert formats
    const uint8_t *q;
    const uint16_t *scale, *minv;
    const uint8_t *bits_tab;   // [E] or null
    const int64_t *q_off;      // [E] byte offset of expert e's first row, or null (uniform: e * N * row_bytes)
    int bits;
    int64_t N, K, G;           // N rows per expert
    int bits_of(int64_t e) const { return bits_tab ? bits_tab[e] : bits; }
    const uint8_t *row(int64_t e, int64_t n) const {
        const int b = bits_of(e);
        const int64_t base = q_off ? q_off[e] : e * N * row_bytes(b, K);
        return q + base + n * row_bytes(b, K);
    }
    const uint16_t *srow(int64_t e, int64_t n) const { return scale + (e * N + n) * (K / G); }
    const uint16_t *mrow(int64_t e, int64_t n) const { return minv + (e * N + n) * (K / G); }
};

void set_err(uint32_t *err, uint32_t a, uint32_t b) {  // first flag wins (kernels/moe_router.hip:58-61)
    if (err && err[0] == 0) err[0] = 1, err[1] = a, err[2] = b;
}

}  // namespace

extern "C" {

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t b) { return bf16_to_f32(b); }
int64_t orc_row_bytes(int bits, int64_t K) { return row_bytes(bits, K); }

// formats/q4.cpp:39-83, q5.cpp:58-98, q6.cpp:44-86, q8.cpp:43-78. Returns 0, or a negative code where the
// reference throws: -1 shape, -2 group size, -3 K % G, -4 plane alignment (q5 K%128, q6 K%64), -5 non-finite
// input, -6 rounding mode.
int orc_quantize(int bits, const float *w, int64_t N, int64_t K, int64_t G, uint8_t *q, uint16_t *scale,
                 uint16_t *minv) {
    if (w == nullptr || N < 1 || K < 1) return -1;
    if (!(G == 32 || G == 64 || G == 128)) return -2;
    if (K % G != 0) return -3;
    if ((bits == 5 && K % 128 != 0) || (bits == 6 && K % 64 != 0)) return -4;
    if (std::fegetround() != FE_TONEAREST) return -6;
    const int64_t rb = row_bytes(bits, K);
    const float qmax = (float)qmax_of(bits);
    std::memset(q, 0, (size_t)(N * rb));
    for (int64_t n = 0; n < N; ++n) {
        uint8_t *row = q + n * rb;
        for (int64_t g = 0; g < K / G; ++g) {
            const float *grp = w + n * K + g * G;
            float lo = grp[0], hi = grp[0];
            for (int64_t i = 0; i < G; ++i) {
                if (!std::isfinite(grp[i])) return -5;
                lo = std::fmin(lo, grp[i]);
                hi = std::fmax(hi, grp[i]);
            }
            const uint16_t s_bits = f32_to_bf16((hi - lo) / qmax), m_bits = f32_to_bf16(lo);
            const float s = bf16_to_f32(s_bits), m = bf16_to_f32(m_bits);
            scale[n * (K / G) + g] = s_bits;
            minv[n * (K / G) + g] = m_bits;
            for (int64_t i = 0; i < G; ++i) {
                int code = 0;
                if (s > 0.0f) {
                    const float r = std::nearbyint((grp[i] - m) / s);
                    code = (int)std::fmin(std::fmax(r, 0.0f), qmax);
                }
                put_code(bits, row, K, g * G + i, code);
            }
        }
    }
    return 0;
}

// formats/q4.cpp:119-134 and its q5/q6/q8 twins.
void orc_dequantize(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K,
                    int64_t G, float *w) {
    const int64_t rb = row_bytes(bits, K);
    for (int64_t n = 0; n < N; ++n) dequant_row(bits, q + n * rb, scale + n * (K / G), minv + n * (K / G), K, G, w + n * K);
}

// Dense projections: kernels/linear_q4.hpp:3-4,26-30 (and q5/q6/q8): y[M,N] = x[M,K] * dequant(W)^T, FP32
// accumulate, output in out_act (F32 output stored unrounded).
void orc_linear_q(int bits, const void *x, int act, const uint8_t *q, const uint16_t *scale, const uint16_t *minv,
                  int64_t N, int64_t K, int64_t G, void *y, int out_act, int64_t M) {
    std::vector<float> w((size_t)K);
    const int64_t rb = row_bytes(bits, K);
    for (int64_t n = 0; n < N; ++n) {
        dequant_row(bits, q + n * rb, scale + n * (K / G), minv + n * (K / G), K, G, w.data());
        for (int64_t m = 0; m < M; ++m) act_store(y, m * N + n, (float)dot_row(w.data(), x, m * K, K, act), out_act);
    }
}

// kernels/linear.hpp:3-5,20-26: unquantized weights [N, K]; wtype 0 = F32, 1 = BF16 bits.
void orc_linear_w(const void *x, int act, const void *w, int wtype, void *y, int out_act, int64_t M, int64_t N,
                  int64_t K) {
    std::vector<float> wr((size_t)K);
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) wr[k] = act_load(w, n * K + k, wtype);
        for (int64_t m = 0; m < M; ++m) act_store(y, m * N + n, (float)dot_row(wr.data(), x, m * K, K, act), out_act);
    }
}

// kernels/moe_router.hpp:11-23, moe_router.hip:32-112. Selection: k rounds of arg-max, larger logit first, a tie
// to the lower index. coef_j = expf(l_j - top) / sum, the sum taken over 32 lanes (lanes >= k hold 0) in the
// xor-butterfly order of moe_router.hip:101-103. Shared slot: id shared_id, coef 1 / (1 + expf(-sl)).
// A non-finite logit fails the token: ids -1, coef NaN, err = {1, token, smallest bad expert index (E = shared)}.
void orc_moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit,
                    int64_t shared_ld, int32_t shared_id, int32_t *ids, float *coef, int act, uint32_t *err) {
    const int64_t A = k + (shared_logit ? 1 : 0);
    std::vector<float> v((size_t)E);
    for (int64_t m = 0; m < M; ++m) {
        int64_t bad = -1;
        for (int64_t e = 0; e < E; ++e) {
            v[e] = act_load(logits, m * ld + e, act);
            if (!std::isfinite(v[e]) && bad < 0) bad = e;
        }
        float sl = 0.f;
        if (shared_logit) {
            sl = act_load(shared_logit, m * shared_ld, act);
            if (!std::isfinite(sl) && bad < 0) bad = E;
        }
        if (bad >= 0) {
            set_err(err, (uint32_t)m, (uint32_t)bad);
            for (int64_t a = 0; a < A; ++a) ids[m * A + a] = -1, coef[m * A + a] = qnan();
            continue;
        }
        float pick_v[32];
        int32_t pick_i[32];
        for (int64_t r = 0; r < k; ++r) {
            int64_t bi = -1;
            float bv = -INFINITY;
            for (int64_t e = 0; e < E; ++e)
                if (v[e] > bv) bv = v[e], bi = e;  // strict > keeps the lower index on a tie
            pick_v[r] = bv, pick_i[r] = (int32_t)bi;
            v[bi] = -INFINITY;
        }
        float lane[32];
        for (int l = 0; l < 32; ++l) lane[l] = l < k ? expf(pick_v[l] - pick_v[0]) : 0.f;
        float ex[32];
        std::memcpy(ex, lane, sizeof(ex));
        for (int off = 16; off > 0; off >>= 1) {
            float nx[32];
            for (int l = 0; l < 32; ++l) nx[l] = lane[l] + lane[l ^ off];
            std::memcpy(lane, nx, sizeof(nx));
        }
        for (int64_t r = 0; r < k; ++r) ids[m * A + r] = pick_i[r], coef[m * A + r] = ex[r] / lane[r];
        if (shared_logit) ids[m * A + k] = shared_id, coef[m * A + k] = 1.0f / (1.0f + expf(-sl));
    }
}

// kernels/swiglu.hip:24-37: F32 h = silu(g) * u; BF16 h = bf16(bf16(silu(g)) * u).
void orc_swiglu(const void *gu, void *h, int64_t rows, int64_t I, int act) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < I; ++j) {
            const float g = act_load(gu, r * 2 * I + j, act), u = act_load(gu, r * 2 * I + I + j, act);
            act_store(h, r * I + j, as_stored(silu(g), act) * u, act);
        }
}

// kernels/linear_q4.hpp:32-41, linear_q4.hip:172-194 (gather) and :205-233 (gather + SwiGLU epilogue: g and u
// rounded as their store would, h formed as swiglu does). bits_tab / q_off null = one format for all experts.
// swiglu != 0: N = 2I rows per expert [gate | up], y [M, A, I]; else y [M, A, N].
void orc_experts_gather(int bits, const uint8_t *bits_tab, const int64_t *q_off, const void *x, const uint8_t *q,
                        const uint16_t *scale, const uint16_t *minv, int64_t E, int64_t N, int64_t K, int64_t G,
                        const int32_t *ids, int64_t M, int64_t A, void *y, int act, uint32_t *err, int swiglu) {
    const Stack st{q, scale, minv, bits_tab, q_off, bits, N, K, G};
    std::vector<float> w((size_t)K), wu((size_t)K);
    const int64_t I = N / 2, out = swiglu ? I : N;
    for (int64_t m = 0; m < M; ++m)
        for (int64_t a = 0; a < A; ++a) {
            const int64_t slot = m * A + a;
            const int32_t id = ids[slot];
            if (id < 0 || id >= E) {
                set_err(err, (uint32_t)id, (uint32_t)slot);
                for (int64_t n = 0; n < out; ++n) act_store(y, slot * out + n, qnan(), act);
                continue;
            }
            const int b = st.bits_of(id);
            for (int64_t n = 0; n < out; ++n) {
                dequant_row(b, st.row(id, n), st.srow(id, n), st.mrow(id, n), K, G, w.data());
                const float g = (float)dot_row(w.data(), x, m * K, K, act);
                if (!swiglu) {
                    act_store(y, slot * out + n, g, act);
                    continue;
                }
                dequant_row(b, st.row(id, n + I), st.srow(id, n + I), st.mrow(id, n + I), K, G, wu.data());
                const float u = (float)dot_row(wu.data(), x, m * K, K, act);
                const float gs = as_stored(g, act), us = as_stored(u, act);
                act_store(y, slot * out + n, as_stored(silu(gs), act) * us, act);
            }
        }
}

// kernels/linear_q4.hip:238-279 and moe_grouped.hip:456-472: y[m,:] = sum_a coef[m,a] * (h[m,a,:] * W[ids[m,a]]^T),
// a in order, one rounding; any invalid id of token m makes its whole row NaN and sets err {1, id, slot}.
void orc_experts_combine(int bits, const uint8_t *bits_tab, const int64_t *q_off, const void *h, const uint8_t *q,
                         const uint16_t *scale, const uint16_t *minv, int64_t E, int64_t N, int64_t K, int64_t G,
                         const int32_t *ids, const float *coef, int64_t M, int64_t A, void *y, int act,
                         uint32_t *err) {
    const Stack st{q, scale, minv, bits_tab, q_off, bits, N, K, G};
    std::vector<float> w((size_t)K);
    for (int64_t m = 0; m < M; ++m) {
        bool ok = true;
        for (int64_t a = 0; a < A; ++a) {
            const int32_t id = ids[m * A + a];
            if (id < 0 || id >= E) {
                if (ok) set_err(err, (uint32_t)id, (uint32_t)(m * A + a));
                ok = false;
            }
        }
        for (int64_t n = 0; n < N; ++n) {
            if (!ok) {
                act_store(y, m * N + n, qnan(), act);
                continue;
            }
            double v = 0.0;
            for (int64_t a = 0; a < A; ++a) {
                const int32_t id = ids[m * A + a];
                dequant_row(st.bits_of(id), st.row(id, n), st.srow(id, n), st.mrow(id, n), K, G, w.data());
                v += (double)coef[m * A + a] * dot_row(w.data(), h, (m * A + a) * K, K, act);
            }
            act_store(y, m * N + n, (float)v, act);
        }
    }
}

// kernels/moe_grouped.hpp:39-49 and moe_grouped.hip:63-81,106-151: counting sort of the S = M*A slots by bucket
// (expert id, or E for an invalid id). Workspace (int32): [n_tiles, S, E, n_wtiles], offsets[E+2], slots[S],
// tile_bucket[Tmax], tile_start[Tmax], wtile_bucket[WTmax], wtile_start[WTmax]; Tmax = S/16 + E + 2,
// WTmax = S/64 + E + 2. The reference leaves the order inside a bucket to atomics; here it is slot-ascending
// (a stable sort), which is one of the orders the reference can produce.
int64_t orc_route_workspace_ints(int64_t M, int64_t A, int64_t E) {
    const int64_t S = M * A;
    return 4 + (E + 2) + S + 2 * (S / 16 + E + 2) + 2 * (S / 64 + E + 2);
}
void orc_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, int32_t *ws, uint32_t *err) {
    const int64_t S = M * A, Tmax = S / 16 + E + 2, WTmax = S / 64 + E + 2;
    int32_t *offsets = ws + 4, *slots = offsets + E + 2, *tile_bucket = slots + S, *tile_start = tile_bucket + Tmax;
    int32_t *wtile_bucket = tile_start + Tmax, *wtile_start = wtile_bucket + WTmax;
    std::vector<int32_t> cnt((size_t)E + 1, 0);
    for (int64_t s = 0; s < S; ++s) {
        const bool bad = ids[s] < 0 || ids[s] >= E;
        if (bad) set_err(err, (uint32_t)ids[s], (uint32_t)s);
        ++cnt[bad ? E : ids[s]];
    }
    int32_t start = 0, nt = 0, nwt = 0;
    std::vector<int32_t> cursor((size_t)E + 1);
    for (int64_t b = 0; b <= E; ++b) {
        offsets[b] = start, cursor[b] = start;
        for (int32_t i = 0; i < (cnt[b] + 15) / 16; ++i) tile_bucket[nt] = (int32_t)b, tile_start[nt] = start + i * 16, ++nt;
        for (int32_t i = 0; i < (cnt[b] + 63) / 64; ++i) wtile_bucket[nwt] = (int32_t)b, wtile_start[nwt] = start + i * 64, ++nwt;
        start += cnt[b];
    }
    offsets[E + 1] = start;
    ws[0] = nt, ws[1] = (int32_t)S, ws[2] = (int32_t)E, ws[3] = nwt;
    for (int64_t s = 0; s < S; ++s) slots[cursor[(ids[s] < 0 || ids[s] >= E) ? E : ids[s]]++] = (int32_t)s;
}

// kernels/moe_router.hip:129-145: y[m,:] += sigmoid(gate_logit[m*gate_ld]) * s[m,:]; a non-finite gate logit makes
// the row NaN and sets err {1, token, gate_index}.
void orc_moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                        uint32_t gate_index, int act, uint32_t *err) {
    for (int64_t m = 0; m < M; ++m) {
        const float gl = gate_logit[m * gate_ld];
        const bool ok = std::isfinite(gl);
        if (!ok) set_err(err, (uint32_t)m, gate_index);
        const float g = ok ? 1.f / (1.f + expf(-gl)) : qnan();
        for (int64_t n = 0; n < N; ++n) {
            const float p = g * act_load(s, m * N + n, act);
            act_store(y, m * N + n, act_load(y, m * N + n, act) + p, act);
        }
    }
}

// kernels/hc.hip:244-252: x[t, s*N + n] = fma(w_in[t, s], y[t, n], x) for the H streams of x [M, H*N].
void orc_hc_inject(void *x, const void *y, const float *w_in, int64_t M, int64_t N, int64_t H, int act) {
    for (int64_t m = 0; m < M; ++m)
        for (int64_t st = 0; st < H; ++st)
            for (int64_t n = 0; n < N; ++n) {
                const int64_t i = (m * H + st) * N + n;
                act_store(x, i, std::fmaf(w_in[m * H + st], act_load(y, m * N + n, act), act_load(x, i, act)), act);
            }
}

// kernels/hc.hip:77-165 hc_mix_down (interface kernels/hc.hpp:29-39). X [T, H*d]; W [r (+ H), H*d] with the hc_norm weight
// folded in. Per stream s: inv_s = 1 / sqrt(mean(X_s^2) + eps); per row n: a_n = sum_s inv_s * (W_n,s . X_s);
// h[n] = silu(a_n / H) for n < r, w_in[n - r] = 2 sigmoid(a_n / H) behind them. The dots and the sums of squares are
// accumulated in double (the kernel: FP32 fma chains over 32-code chunks, s * dot + m * xsum per chunk); the steps after
// them are the kernel's own FP32 operations in its order.
void orc_hc_mix_down(const void *x, int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t G,
                     int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h, float *w_in, float *inv,
                     int act) {
    const int64_t K = H * d, R = r + (inject ? H : 0), rb = row_bytes(bits, K);
    std::vector<float> wrow((size_t)K);
    for (int64_t t = 0; t < T; ++t) {
        std::vector<float> iv((size_t)H);
        for (int64_t s = 0; s < H; ++s) {
            double sq = 0.0;
            for (int64_t j = 0; j < d; ++j) {
                const double v = act_load(x, t * K + s * d + j, act);
                sq += v * v;
            }
            iv[(size_t)s] = 1.0f / std::sqrt((float)sq / (float)d + eps);
            inv[t * H + s] = iv[(size_t)s];
        }
        for (int64_t n = 0; n < R; ++n) {
            dequant_row(bits, q + n * rb, scale + n * (K / G), minv + n * (K / G), K, G, wrow.data());
            float a = 0.f;
            for (int64_t s = 0; s < H; ++s)
                a = std::fmaf(iv[(size_t)s], (float)dot_row(wrow.data() + s * d, x, t * K + s * d, d, act), a);
            const float z = a / (float)H;
            if (n < r) h[t * r + n] = z / (1.0f + std::exp(-z));
            else w_in[t * H + (n - r)] = 2.0f / (1.0f + std::exp(-z));
        }
    }
}

// formats/q4.cpp:101-119 to_chunk_major (formats/q8.hpp:37-46 for one code per byte): 32-code chunk c of row n moves to
// [(c * N + n) * chunk bytes], group g's scale / min to [g * N + n]. 4- and 8-bit codes only.
void orc_to_chunk_major(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K,
                        int64_t G, uint8_t *q_out, uint16_t *scale_out, uint16_t *min_out) {
    const int64_t cb = 32 * bits / 8, chunks = K / 32, groups = K / G;
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t c = 0; c < chunks; ++c)
            for (int64_t b = 0; b < cb; ++b) q_out[(c * N + n) * cb + b] = q[(n * chunks + c) * cb + b];
        for (int64_t g = 0; g < groups; ++g) {
            scale_out[g * N + n] = scale[n * groups + g];
            min_out[g * N + n] = minv[n * groups + g];
        }
    }
}

// kernels/hc.hip:176-242 hc_mix_up (interface kernels/hc.hpp:41-50). W_up [H*d, r] CHUNK-major, 4- or 8-bit:
// u[t, j] = (1/H) sum_s sigmoid(W_up[s*d + j] . h[t]) * (X[t, s*d + j] * inv[t, s] * (1 + norm_w[s*d + j])), rounded once
// to the activation dtype. The dot accumulates in double; the gate and the combine are the kernel's FP32 steps in order.
void orc_hc_mix_up(const float *h, int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t G,
                   int64_t r, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d, void *u,
                   int act) {
    const int64_t N = H * d, cb = 32 * bits / 8;
    for (int64_t t = 0; t < T; ++t)
        for (int64_t j = 0; j < d; ++j) {
            float sum = 0.f;
            for (int64_t s = 0; s < H; ++s) {
                const int64_t row = s * d + j;
                double acc = 0.0;
                for (int64_t k = 0; k < r; ++k) {
                    const uint8_t *chunk = q + ((k / 32) * N + row) * cb;
                    const int kk = (int)(k % 32);
                    const int code = bits == 8 ? chunk[kk] : (chunk[kk / 2] >> ((kk & 1) ? 4 : 0)) & 0xF;
                    const int64_t gi = (k / G) * N + row;
                    const float w = (float)code * bf16_to_f32(scale[gi]) + bf16_to_f32(minv[gi]);
                    acc += (double)w * (double)h[t * r + k];
                }
                const float z = 1.0f / (1.0f + std::exp(-(float)acc));
                sum += z * (act_load(x, t * N + row, act) * inv[t * H + s] * (1.0f + norm_w[row]));
            }
            act_store(u, t * d + j, sum / (float)H, act);
        }
}

// kernels/moe_router.hip:154-180 - defined as moe_shared_add then hc_inject on the stored y.
void orc_moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                               uint32_t gate_index, void *x, const float *w_in, int64_t H, int act, uint32_t *err) {
    orc_moe_shared_add(y, s, gate_logit, gate_ld, M, N, gate_index, act, err);
    orc_hc_inject(x, y, w_in, M, N, H, act);
}

// kernels/residual.hip:22-30: x = x + y, one rounding.
void orc_residual_add(void *x, const void *y, int64_t n, int act) {
    for (int64_t i = 0; i < n; ++i) act_store(x, i, act_load(x, i, act) + act_load(y, i, act), act);
}

}  // extern "C"
