// The hyper-connection bracket around the MoE sublayer (strixite kernels/hc.hpp:29-55): hc_mix_down produces the low-rank
// mixer state and the injection weights from the H = 4 residual streams, hc_mix_up the sublayer's input u. (hc_inject, the
// step after the sublayer, lives with the other elementwise kernels.)
//
//   hc_mix_down  X [T, H d] and folded weights W [r (+ H), H d] (Q4 or Q8, row-major): per stream s the inverse RMS
//                inv_s = 1 / sqrt(mean(X_s^2) + eps); per row n the per-stream partial dots p_ns = W_n,s . X_s;
//                a_n = sum_s inv_s p_ns; rows n < r give h[n] = silu(a_n / H), the H rows behind them
//                w_in[n - r] = 2 sigmoid(a_n / H).
//   hc_mix_up    h [T, r], W_up [H d, r] (Q4 or Q8, CHUNK-major: 32-code chunk c of row n at q[(c N + n) * chunk bytes],
//                group g's scale / min at [g N + n]; strixite formats/q4.hpp:41-55): per row (s, j)
//                z = sigmoid(W_up[s d + j] . h), u[j] = (1 / H) sum_s z * X[s d + j] * inv_s * (1 + norm_w[s d + j]).
// Both are small weight-streaming kernels (a 324 x 10240 Q4 matrix is 1.9 MB): a block per weight row with a warp per stream
// (down), or a lane per weight row with the chunk-major layout making a warp's loads one contiguous run (up).
#include "common.cuh"

#include "strixite_b200.h"

#include <cmath>
#include <type_traits>
#include <cstring>

namespace {

using namespace sb;

constexpr int kH = 4;          // streams
constexpr int kMaxR = 1024;    // low rank, kept in shared memory by hc_mix_up

// ---- hc_mix_down: one block per weight row and batch of up to kDownTokens tokens, a warp per stream (its quarter of K). The
//      row's codes are decoded once per chunk and applied to every token of the batch; a token's arithmetic does not depend on
//      the batch it is in. A handful of tokens (decode, verify) run one token per block: these launches are latency-bound, and
//      more blocks beat fewer decodes (T = 5: 10 us either way for down, 8 vs 14 us for up); from kBatchFrom tokens on the
//      batches win (T = 64: 88 -> 71 us down, 53 -> 34 us up). --------------------------------------------------------------------
constexpr int kBatchFrom = 16, kDownBatch = 8, kUpBatch = 4;
template <typename T, int BITS, int kDownTokens>
__global__ void __launch_bounds__(32 * kH)
    hc_down_kernel(const T *x, strix_qview w, int64_t Tn, int64_t d, int r, float eps, float *h, float *w_in, float *inv) {
    __shared__ float ps[kDownTokens][kH], sqs[kDownTokens][kH];
    const int lane = threadIdx.x & 31, s = threadIdx.x >> 5;  // s: the stream this warp covers
    const int64_t n = blockIdx.x, t0 = (int64_t)blockIdx.y * kDownTokens, K = w.K;
    const int nt = (int)(Tn - t0 < kDownTokens ? Tn - t0 : kDownTokens);
    const uint8_t *row = w.q + n * row_bytes(BITS, K);
    const uint16_t *srow = w.scale + n * (K / w.G), *mrow = w.minv + n * (K / w.G);
    float p[kDownTokens], sq[kDownTokens];
#pragma unroll
    for (int tt = 0; tt < kDownTokens; ++tt) p[tt] = 0.f, sq[tt] = 0.f;
    const int64_t c0 = (int64_t)s * (d / 32), c1 = c0 + d / 32;  // a 32-code chunk lies inside one stream: d % 32 == 0
    for (int64_t c = c0 + lane; c < c1; c += 32) {
        float code[32];
        load_codes32<BITS>(row, K, c, code);
        const float sc = bf16_bits_to_f32(srow[c * 32 / w.G]), mn = bf16_bits_to_f32(mrow[c * 32 / w.G]);
#pragma unroll
        for (int tt = 0; tt < kDownTokens; ++tt) {
            if (tt >= nt) break;
            float xv[32];
            load_x32(x + (t0 + tt) * K, c * 32, xv);
            float dot = 0.f, xsum = 0.f, s2 = sq[tt];
#pragma unroll
            for (int i = 0; i < 32; ++i) dot = fmaf(xv[i], code[i], dot), xsum += xv[i], s2 = fmaf(xv[i], xv[i], s2);
            sq[tt] = s2;
            p[tt] += fmaf(sc, dot, mn * xsum);
        }
    }
#pragma unroll
    for (int tt = 0; tt < kDownTokens; ++tt) {
        if (tt >= nt) break;
        const float pv = warp_sum(p[tt]), sv = warp_sum(sq[tt]);
        if (lane == 0) ps[tt][s] = pv, sqs[tt][s] = sv;
    }
    __syncthreads();
    const int tt = threadIdx.x;  // thread tt finishes token tt of the batch
    if (tt >= nt) return;
    const int64_t t = t0 + tt;
    float a = 0.f, iv[kH];
#pragma unroll
    for (int q = 0; q < kH; ++q) {
        iv[q] = 1.0f / sqrtf(sqs[tt][q] / (float)d + eps);
        a = fmaf(iv[q], ps[tt][q], a);
    }
    const float z = a / (float)kH;
    if (n < r) h[t * r + n] = z / (1.0f + expf(-z));
    else w_in[t * kH + (n - r)] = 2.0f / (1.0f + expf(-z));
    if (n == 0)
#pragma unroll
        for (int q = 0; q < kH; ++q) inv[t * kH + q] = iv[q];
}

// ---- hc_mix_up: block = 32 outputs j x the 4 streams (a warp per stream, a lane per weight row), grid.y = token --------------
template <int BITS>
__device__ __forceinline__ void load_chunk_cm(const uint8_t *q, int64_t N, int64_t row, int c, float (&code)[32]) {
    constexpr int CB = BITS == 8 ? 32 : 16;  // bytes of one 32-code chunk
    const uint4 *p = reinterpret_cast<const uint4 *>(q + ((int64_t)c * N + row) * CB);
    if constexpr (BITS == 8) {
        const uint4 a = __ldg(p), b = __ldg(p + 1);
        const uint32_t wd[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 32; ++i) code[i] = code_f((wd[i / 4] >> (8 * (i % 4))) & 0xFFu);
    } else {
        const uint4 a = __ldg(p);
        const uint32_t wd[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 32; ++i) code[i] = code_f((wd[i / 8] >> (4 * (i % 8))) & 0xFu);
    }
}

// A block also takes up to kUpTokens tokens: a weight chunk is decoded once and dotted with every token's h.
template <typename T, int BITS, int kUpTokens>
__global__ void __launch_bounds__(128)
    hc_up_kernel(const float *h, strix_qview w, const T *x, const float *norm_w, const float *inv, int64_t Tn, int64_t d, T *u) {
    __shared__ float hs[kUpTokens][kMaxR], hsum[kUpTokens][kMaxR / 32], contrib[kUpTokens][kH][32];
    const int lane = threadIdx.x & 31, s = threadIdx.x >> 5, r = (int)w.K;
    const int64_t t0 = (int64_t)blockIdx.y * kUpTokens, j = (int64_t)blockIdx.x * 32 + lane, N = w.N;
    const int nt = (int)(Tn - t0 < kUpTokens ? Tn - t0 : kUpTokens);
    for (int tt = 0; tt < nt; ++tt)
        for (int i = threadIdx.x; i < r; i += 128) hs[tt][i] = h[(t0 + tt) * r + i];
    __syncthreads();
    for (int i = threadIdx.x; i < nt * (r / 32); i += 128) {
        const int tt = i / (r / 32), c = i % (r / 32);
        float a = 0.f;
        for (int k = 0; k < 32; ++k) a += hs[tt][c * 32 + k];
        hsum[tt][c] = a;
    }
    __syncthreads();
    if (j < d) {
        const int64_t row = (int64_t)s * d + j;
        float acc[kUpTokens];
#pragma unroll
        for (int tt = 0; tt < kUpTokens; ++tt) acc[tt] = 0.f;
        for (int c = 0; c < r / 32; ++c) {
            float code[32];
            load_chunk_cm<BITS>(w.q, N, row, c, code);
            const int64_t gi = (int64_t)(c * 32 / w.G) * N + row;
            const float sc = bf16_bits_to_f32(__ldg(w.scale + gi)), mn = bf16_bits_to_f32(__ldg(w.minv + gi));
#pragma unroll
            for (int tt = 0; tt < kUpTokens; ++tt) {
                if (tt >= nt) break;
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < 32; ++i) dot = fmaf(hs[tt][c * 32 + i], code[i], dot);
                acc[tt] = fmaf(sc, dot, fmaf(mn, hsum[tt][c], acc[tt]));
            }
        }
        const float nw = 1.0f + norm_w[row];
#pragma unroll
        for (int tt = 0; tt < kUpTokens; ++tt) {
            if (tt >= nt) break;
            const int64_t t = t0 + tt;
            const float z = 1.0f / (1.0f + expf(-acc[tt]));
            contrib[tt][s][lane] = z * (ld_act(x, t * N + row) * inv[t * kH + s] * nw);
        }
    }
    __syncthreads();
    if (s == 0 && j < d)
        for (int tt = 0; tt < nt; ++tt) {
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < kH; ++q) sum += contrib[tt][q][lane];
            st_act(u, (t0 + tt) * d + j, sum / (float)kH);
        }
}

// ---- hc_inject_inv: the injection and the next mix's inverse RMS of the updated streams in one pass; block = token -----------------
template <typename T>
__global__ void __launch_bounds__(256) hc_inject_inv_kernel(T *x, const float *w_in, const T *y, int64_t d, float eps, float *inv) {
    __shared__ float red[8];
    const int64_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int s = 0; s < kH; ++s) {
        T *xs = x + (t * kH + s) * d;
        const float w = w_in[t * kH + s];
        float ss = 0.f;
        for (int64_t j = threadIdx.x; j < d; j += 256) {
            st_act(xs, j, fmaf(w, ld_act(y, t * d + j), ld_act(xs, j)));
            const float v = ld_act(xs, j);  // the stored (rounded) value: what the next mix reads
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) tot += red[i];
            inv[t * kH + s] = 1.0f / sqrtf(tot / (float)d + eps);
        }
        __syncthreads();
    }
}

int check_view(const char *fn, const strix_qview *wp, int bits) {
    SB_CHECK(wp != nullptr && wp->q != nullptr && wp->scale != nullptr && wp->minv != nullptr, fn, ": null weight view");
    SB_CHECK(bits == 4 || bits == 8, fn, ": ", bits, "-bit weights, expected 4 or 8 (strixite kernels/hc.hpp:13-14)");
    SB_CHECK(group_ok(wp->G) && wp->K % wp->G == 0 && wp->K % 32 == 0 && aligned16(wp->q), fn, ": K = ", wp->K, ", G = ", wp->G,
             ": K must be a multiple of 32 and of the group size, the codes 16-byte aligned");
    return 0;
}

}  // namespace

extern "C" {

int strix_hc_mix_down(const void *x, const strix_qview *w, int bits, int64_t T, int64_t H, int64_t d, int64_t r, int inject, float eps, float *h,
                      float *w_in, float *inv, int act, void *stream) {
    const char *fn = "hc_mix_down";
    SB_TRY(check_view(fn, w, bits));
    SB_CHECK(x != nullptr && h != nullptr && inv != nullptr, fn, ": null pointer (x=", x, ", h=", (const void *)h, ", inv=", (const void *)inv, ")");
    SB_CHECK((inject != 0) == (w_in != nullptr), fn, ": w_in must be given exactly when inject (inject=", inject, ", w_in=", (const void *)w_in, ")");
    SB_CHECK(H == kH, fn, ": H = ", H, ", expected ", kH);
    SB_CHECK(T >= 1 && T <= 65535 && d >= 32 && d % 32 == 0, fn, ": T = ", T, ", d = ", d, " (d a multiple of 32: a 32-code load never straddles two streams)");
    SB_CHECK(r >= 1 && r <= kMaxR, fn, ": r = ", r, ", expected 1..", kMaxR);
    const int64_t R = r + (inject ? H : 0);
    SB_CHECK(w->K == H * d && w->N == R, fn, ": weight [", w->N, ", ", w->K, "], expected [", R, ", ", H * d, "]");
    SB_CHECK(aligned16(x) && act_ok(act), fn, ": x ", x, " must be 16-byte aligned; activation dtype ", act);
    SB_CHECK(std::isfinite(eps) && eps > 0.f, fn, ": eps must be finite and > 0, got ", eps);
    auto st = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto tag, auto bits_tag, auto mt_tag) {
        using X = decltype(tag);
        constexpr int B = decltype(bits_tag)::value, MT = decltype(mt_tag)::value;
        const dim3 grid((unsigned)R, (unsigned)((T + MT - 1) / MT));
        hc_down_kernel<X, B, MT><<<grid, 32 * kH, 0, st>>>((const X *)x, *w, T, d, (int)r, eps, h, w_in, inv);
    };
    auto by_batch = [&](auto tag, auto bits_tag) {
        if (T < kBatchFrom) launch(tag, bits_tag, std::integral_constant<int, 1>{});
        else launch(tag, bits_tag, std::integral_constant<int, kDownBatch>{});
    };
    auto by_bits = [&](auto tag) {
        if (bits == 4) by_batch(tag, std::integral_constant<int, 4>{});
        else by_batch(tag, std::integral_constant<int, 8>{});
    };
    if (act == kF32) by_bits(float{});
    else by_bits(uint16_t{});
    SB_LAUNCH_OK(fn, " T=", T, " d=", d, " r=", r);
    return 0;
}

int strix_hc_mix_up(const float *h, const strix_qview *w_up, int bits, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d,
                    void *u, int act, void *stream) {
    const char *fn = "hc_mix_up";
    SB_TRY(check_view(fn, w_up, bits));
    SB_CHECK(h != nullptr && x != nullptr && norm_w != nullptr && inv != nullptr && u != nullptr, fn, ": null pointer");
    SB_CHECK(H == kH, fn, ": H = ", H, ", expected ", kH);
    SB_CHECK(T >= 1 && T <= 65535 && d >= 1 && w_up->N == H * d, fn, ": T = ", T, ", W_up has ", w_up->N, " rows, expected H*d = ", H * d);
    SB_CHECK(w_up->K >= 32 && w_up->K <= kMaxR, fn, ": r = ", w_up->K, ", expected 32..", kMaxR, " in steps of 32");
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    auto st = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto tag, auto bits_tag, auto mt_tag) {
        using X = decltype(tag);
        constexpr int B = decltype(bits_tag)::value, MT = decltype(mt_tag)::value;
        const dim3 grid((unsigned)((d + 31) / 32), (unsigned)((T + MT - 1) / MT));
        hc_up_kernel<X, B, MT><<<grid, 128, 0, st>>>(h, *w_up, (const X *)x, norm_w, inv, T, d, (X *)u);
    };
    auto by_batch = [&](auto tag, auto bits_tag) {
        if (T < kBatchFrom) launch(tag, bits_tag, std::integral_constant<int, 1>{});
        else launch(tag, bits_tag, std::integral_constant<int, kUpBatch>{});
    };
    auto by_bits = [&](auto tag) {
        if (bits == 4) by_batch(tag, std::integral_constant<int, 4>{});
        else by_batch(tag, std::integral_constant<int, 8>{});
    };
    if (act == kF32) by_bits(float{});
    else by_bits(uint16_t{});
    SB_LAUNCH_OK(fn, " T=", T, " d=", d, " r=", w_up->K);
    return 0;
}

int strix_hc_inject_inv(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, float eps, float *inv, int act, void *stream) {
    const char *fn = "hc_inject_inv";
    SB_CHECK(H == kH, fn, ": H = ", H, " streams, only ", kH, " is supported");
    SB_CHECK(T >= 1 && T <= 0x7fffffff && d >= 1 && d <= (1 << 20), fn, ": T = ", T, ", d = ", d);
    SB_CHECK(x != nullptr && w_in != nullptr && y != nullptr && inv != nullptr, fn, ": null pointer (x=", x, ", w_in=", (const void *)w_in, ", y=", y,
             ", inv=", (const void *)inv, ")");
    SB_CHECK(std::isfinite(eps) && eps > 0.f, fn, ": eps must be finite and > 0, got ", eps);
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    const size_t es = act == kF32 ? 4 : 2;
    const auto xb = reinterpret_cast<uintptr_t>(x), yb = reinterpret_cast<uintptr_t>(y);
    SB_CHECK(yb + (uintptr_t)(T * d) * es <= xb || xb + (uintptr_t)(T * H * d) * es <= yb, fn, ": y overlaps the streams x");
    auto st = static_cast<cudaStream_t>(stream);
    if (act == kF32) hc_inject_inv_kernel<float><<<(unsigned)T, 256, 0, st>>>((float *)x, w_in, (const float *)y, d, eps, inv);
    else hc_inject_inv_kernel<uint16_t><<<(unsigned)T, 256, 0, st>>>((uint16_t *)x, w_in, (const uint16_t *)y, d, eps, inv);
    SB_LAUNCH_OK(fn, " T=", T, " d=", d);
    return 0;
}

int strix_to_chunk_major(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K, int64_t G, uint8_t *q_out,
                         uint16_t *scale_out, uint16_t *min_out) {
    const char *fn = "to_chunk_major";
    SB_CHECK(q && scale && minv && q_out && scale_out && min_out, fn, ": null pointer");
    SB_CHECK((bits == 4 || bits == 8) && N >= 1 && K >= 32 && K % 32 == 0 && group_ok(G) && K % G == 0, fn, ": ", bits, " bits, [", N, ", ", K, "], G = ", G,
             ": chunk-major needs 4- or 8-bit codes and K % 32 == 0 (32-code chunks)");
    const int64_t cb = bits == 8 ? 32 : 16, chunks = K / 32, groups = K / G;
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t c = 0; c < chunks; ++c) std::memcpy(q_out + (c * N + n) * cb, q + n * chunks * cb + c * cb, (size_t)cb);
        for (int64_t g = 0; g < groups; ++g) scale_out[g * N + n] = scale[n * groups + g], min_out[g * N + n] = minv[n * groups + g];
    }
    return 0;
}

}  // extern "C"
