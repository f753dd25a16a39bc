// Dense projections y[M, N] = x[M, K] * W^T for small M (decode, verify): W quantized (q4/q5/q6/q8) or plain
// BF16 / FP32 rows. One warp per output row: lanes stride over the row's 16-byte chunks, so a warp's loads are one
// contiguous 512-byte run; up to 8 activation rows share each weight pass; a shuffle reduction ends the row.
// FP32 accumulation; the output is rounded once (BF16) or stored as accumulated (F32).
#include "common.cuh"
#include "prefill_umma.cuh"

#include "grouped.cuh"
#include "strixite_b200.h"

namespace {

using namespace sb;

constexpr int kWarps = 8;  // output rows per block at most

// Few output rows (a router projection: ~500 rows of a long K) would fill fewer blocks of 8 rows than the GPU has SMs: two
// rows per block then.
inline int rows_per_block(int64_t N) { return N >= 8 * 2 * sm_count() ? kWarps : 2; }

template <int BITS, typename TX, typename TY, int MR>
__global__ void __launch_bounds__(kWarps * 32)
    linear_q_kernel(const TX *x, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, TY *y, int64_t M,
                    int64_t N, int64_t K, int G) {
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    const int64_t m0 = (int64_t)blockIdx.y * MR;
    const int rows = (int)(M - m0 < MR ? M - m0 : MR);
    const uint8_t *row = q + n * row_bytes(BITS, K);
    const uint16_t *srow = scale + n * (K / G), *mrow = minv + n * (K / G);
    float acc[MR];
#pragma unroll
    for (int r = 0; r < MR; ++r) acc[r] = 0.f;
    for (int64_t c = lane; c < K / 32; c += 32) {
        float code[32];
        load_codes32<BITS>(row, K, c, code);
        const float s = bf16_bits_to_f32(srow[c * 32 / G]), mn = bf16_bits_to_f32(mrow[c * 32 / G]);
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            if (r < rows) {
                float xv[32];
                load_x32(x, (m0 + r) * K + c * 32, xv);
                float dot = 0.f, xs = 0.f;
#pragma unroll
                for (int i = 0; i < 32; ++i) dot = fmaf(xv[i], code[i], dot), xs += xv[i];
                acc[r] = fmaf(s, dot, fmaf(mn, xs, acc[r]));
            }
        }
    }
#pragma unroll
    for (int r = 0; r < MR; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && r < rows) st_act(y, (m0 + r) * N + n, v);
    }
}

// Unquantized weights: TW = float (4 per 16-byte load) or uint16_t BF16 bits (8 per load). K % 8 == 0.
template <typename TW, typename TX, typename TY, int MR>
__global__ void __launch_bounds__(kWarps * 32)
    linear_w_kernel(const TX *x, const TW *w, TY *y, int64_t M, int64_t N, int64_t K) {
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    const int64_t m0 = (int64_t)blockIdx.y * MR;
    const int rows = (int)(M - m0 < MR ? M - m0 : MR);
    const TW *wr = w + n * K;
    float acc[MR];
#pragma unroll
    for (int r = 0; r < MR; ++r) acc[r] = 0.f;
    for (int64_t k = (int64_t)lane * 8; k < K; k += 256) {
        float wv[8];
        if constexpr (sizeof(TW) == 4) {
            const float4 a = *reinterpret_cast<const float4 *>(wr + k), b = *reinterpret_cast<const float4 *>(wr + k + 4);
            wv[0] = a.x, wv[1] = a.y, wv[2] = a.z, wv[3] = a.w, wv[4] = b.x, wv[5] = b.y, wv[6] = b.z, wv[7] = b.w;
        } else {
            const uint4 u = *reinterpret_cast<const uint4 *>(wr + k);
            const uint32_t p[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[2 * j] = __uint_as_float(p[j] << 16), wv[2 * j + 1] = __uint_as_float(p[j] & 0xffff0000u);
        }
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            if (r < rows) {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[r] = fmaf(ld_act(x, (m0 + r) * K + k + j), wv[j], acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < MR; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && r < rows) st_act(y, (m0 + r) * N + n, v);
    }
}

int pick_mr(int64_t M) { return M == 1 ? 1 : M == 2 ? 2 : M <= 4 ? 4 : 8; }

template <int BITS, typename TX, typename TY>
void launch_q(const TX *x, const strix_qview &w, TY *y, int64_t M, cudaStream_t st) {
    const int mr = pick_mr(M);
    const int rpb = rows_per_block(w.N);
    const dim3 grid((unsigned)((w.N + rpb - 1) / rpb), (unsigned)((M + mr - 1) / mr)), block(rpb * 32);
    switch (mr) {
        case 1: linear_q_kernel<BITS, TX, TY, 1><<<grid, block, 0, st>>>(x, w.q, w.scale, w.minv, y, M, w.N, w.K, (int)w.G); break;
        case 2: linear_q_kernel<BITS, TX, TY, 2><<<grid, block, 0, st>>>(x, w.q, w.scale, w.minv, y, M, w.N, w.K, (int)w.G); break;
        case 4: linear_q_kernel<BITS, TX, TY, 4><<<grid, block, 0, st>>>(x, w.q, w.scale, w.minv, y, M, w.N, w.K, (int)w.G); break;
        default: linear_q_kernel<BITS, TX, TY, 8><<<grid, block, 0, st>>>(x, w.q, w.scale, w.minv, y, M, w.N, w.K, (int)w.G); break;
    }
}

template <int BITS>
int linear_q(const char *fn, const void *x, const strix_qview *wp, void *y, int64_t M, int act, int out_act, void *stream) {
    SB_CHECK(wp != nullptr, fn, ": null weight view");
    const strix_qview &w = *wp;
    SB_CHECK(x != nullptr && y != nullptr && w.q != nullptr && w.scale != nullptr && w.minv != nullptr, fn, ": null pointer (x=", x,
             ", y=", y, ", q=", (const void *)w.q, ", scale=", (const void *)w.scale, ", min=", (const void *)w.minv, ")");
    SB_CHECK(group_ok(w.G), fn, ": group size ", w.G, " unsupported (32, 64 or 128)");
    SB_CHECK(M >= 1 && M <= 65535ll * 8, fn, ": M (rows of x) = ", M, ", expected 1..", 65535ll * 8);
    SB_CHECK(w.N >= 1 && w.N <= 0x7fffffff, fn, ": N = ", w.N, ", expected 1..2^31-1");
    SB_CHECK(w.K >= w.G && w.K <= (1 << 24) && w.K % w.G == 0, fn, ": K = ", w.K, " must be a positive multiple of group size ", w.G,
             " and <= 2^24");
    SB_CHECK(BITS != 5 || w.K % 128 == 0, fn, ": Q5 K = ", w.K, " is not a multiple of 128");
    SB_CHECK(BITS != 6 || w.K % 64 == 0, fn, ": Q6 K = ", w.K, " is not a multiple of 64");
    SB_CHECK(aligned16(w.q), fn, ": code array ", (const void *)w.q, " must be 16-byte aligned for vector loads");
    SB_CHECK(aligned16(x), fn, ": x ", x, " must be 16-byte aligned for vector loads");
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SB_CHECK(out_act == act || (act == kBF16 && out_act == kF32), fn, ": output dtype ", act_name(out_act), " with input ",
             act_name(act), " unsupported (same dtype, or BF16 -> F32)");
    SB_CHECK(apart(y, M * w.N * act_size(out_act), x, M * w.K * act_size(act)), fn, ": output y [", y, ", +",
             M * w.N * act_size(out_act), " B) overlaps input x [", x, ", +", M * w.K * act_size(act), " B)");
    auto st = static_cast<cudaStream_t>(stream);
    if (act == kF32) launch_q<BITS>((const float *)x, w, (float *)y, M, st);
    else if (out_act == kF32) launch_q<BITS>((const uint16_t *)x, w, (float *)y, M, st);
    else launch_q<BITS>((const uint16_t *)x, w, (uint16_t *)y, M, st);
    SB_LAUNCH_OK(fn, " ", act_name(act), "->", act_name(out_act), " M=", M, " N=", w.N, " K=", w.K, " G=", w.G);
    return 0;
}

template <typename TW, typename TX, typename TY>
void launch_w(const TX *x, const TW *w, TY *y, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    const int mr = pick_mr(M);
    const int rpb = rows_per_block(N);
    const dim3 grid((unsigned)((N + rpb - 1) / rpb), (unsigned)((M + mr - 1) / mr)), block(rpb * 32);
    switch (mr) {
        case 1: linear_w_kernel<TW, TX, TY, 1><<<grid, block, 0, st>>>(x, w, y, M, N, K); break;
        case 2: linear_w_kernel<TW, TX, TY, 2><<<grid, block, 0, st>>>(x, w, y, M, N, K); break;
        case 4: linear_w_kernel<TW, TX, TY, 4><<<grid, block, 0, st>>>(x, w, y, M, N, K); break;
        default: linear_w_kernel<TW, TX, TY, 8><<<grid, block, 0, st>>>(x, w, y, M, N, K); break;
    }
}

template <typename TW>
int linear_w(const char *fn, const void *x, const TW *w, void *y, int64_t M, int64_t N, int64_t K, int act, int out_act,
             void *stream) {
    SB_CHECK(x != nullptr && w != nullptr && y != nullptr, fn, ": null pointer (x=", x, ", w=", (const void *)w, ", y=", y, ")");
    SB_CHECK(M >= 1 && M <= 65535ll * 8, fn, ": M = ", M, ", expected 1..", 65535ll * 8);
    SB_CHECK(N >= 1 && N <= 0x7fffffff, fn, ": N = ", N, ", expected 1..2^31-1");
    SB_CHECK(K >= 8 && K <= (1 << 24) && K % 8 == 0, fn, ": K = ", K, " must be a positive multiple of 8 and <= 2^24");
    SB_CHECK(aligned16(w) && aligned16(x), fn, ": w ", (const void *)w, " and x ", x, " must be 16-byte aligned");
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SB_CHECK(out_act == act || (act == kBF16 && out_act == kF32), fn, ": output dtype ", act_name(out_act), " with input ",
             act_name(act), " unsupported (same dtype, or BF16 -> F32)");
    SB_CHECK(apart(y, M * N * act_size(out_act), x, M * K * act_size(act)), fn, ": output y overlaps input x");
    auto st = static_cast<cudaStream_t>(stream);
    if (act == kF32) launch_w(static_cast<const float *>(x), w, static_cast<float *>(y), M, N, K, st);
    else if (out_act == kF32) launch_w(static_cast<const uint16_t *>(x), w, static_cast<float *>(y), M, N, K, st);
    else launch_w(static_cast<const uint16_t *>(x), w, static_cast<uint16_t *>(y), M, N, K, st);
    SB_LAUNCH_OK(fn, " ", act_name(act), "->", act_name(out_act), " M=", M, " N=", N, " K=", K);
    return 0;
}

}  // namespace

extern "C" {

int strix_linear_q4(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q<4>("linear_q4", x, w, y, M, act, out_act, stream);
}
int strix_linear_q5(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q<5>("linear_q5", x, w, y, M, act, out_act, stream);
}
int strix_linear_q6(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q<6>("linear_q6", x, w, y, M, act, out_act, stream);
}
int strix_linear_q8(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q<8>("linear_q8", x, w, y, M, act, out_act, stream);
}
int strix_linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, int act,
                       int out_act, void *stream) {
    // many BF16 tokens with FP32 outputs (the router projection of a prefill chunk): the tensor-core kernel. Products of two
    // BF16 values are exact in FP32, so only the summation order differs from the FMA kernel.
    if (x != nullptr && w != nullptr && y != nullptr && act == STRIX_ACT_BF16 && out_act == STRIX_ACT_F32 && N >= 1 &&
        sb::dense_bf16_ok(x, w, M, N, K) && reinterpret_cast<uintptr_t>(y) % 4 == 0)
        return sb::dense_bf16("linear_bf16w", x, w, static_cast<float *>(y), M, N, K, nullptr, 0, static_cast<cudaStream_t>(stream));
    return linear_w<uint16_t>("linear_bf16w", x, w, y, M, N, K, act, out_act, stream);
}
int strix_linear_f32w(const void *x, const float *w, void *y, int64_t M, int64_t N, int64_t K, int act, int out_act,
                      void *stream) {
    return linear_w<float>("linear_f32w", x, w, y, M, N, K, act, out_act, stream);
}

// ---- the same projections on the tensor cores (strixite kernels/linear_wmma.hpp:21-29) ---------------------------------
static int linear_q_wmma(const char *fn, int bits, const void *x, const strix_qview *wp, void *y, int64_t M, int act, int out_act, void *stream) {
    SB_CHECK(wp != nullptr, fn, ": null weight view");
    const strix_qview &w = *wp;
    SB_CHECK(x != nullptr && y != nullptr && w.q != nullptr && w.scale != nullptr && w.minv != nullptr, fn, ": null pointer (x=", x, ", y=", y, ", q=",
             (const void *)w.q, ")");
    SB_CHECK(group_ok(w.G), fn, ": group size ", w.G, " unsupported (32, 64 or 128)");
    SB_CHECK(w.N >= 1 && w.N <= 0x7fffffff && w.K >= w.G && w.K <= (1 << 24) && w.K % w.G == 0 && w.K % 64 == 0, fn, ": [", w.N, ", ", w.K,
             "]: K must be a multiple of the group size ", w.G, " and of 64 (strixite kernels/linear_wmma.hpp:7)");
    SB_CHECK(bits != 5 || w.K % 128 == 0, fn, ": Q5 K = ", w.K, " is not a multiple of 128");
    SB_CHECK(aligned16(w.q) && aligned16(x), fn, ": code array ", (const void *)w.q, " and x ", x, " must be 16-byte aligned");
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    SB_CHECK(out_act == act || (act == kBF16 && out_act == kF32), fn, ": output dtype ", act_name(out_act), " with input ", act_name(act),
             " unsupported (same dtype, or BF16 -> F32)");
    SB_CHECK(apart(y, M * w.N * act_size(out_act), x, M * w.K * act_size(act)), fn, ": output y overlaps input x");
    const sb::StackView sv{w.q, w.scale, w.minv, nullptr, nullptr, bits, w.N, w.K, w.G};
    return sb::dense_umma(fn, x, sv, M, y, act, out_act, static_cast<cudaStream_t>(stream));
}
int strix_linear_q4_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q_wmma("linear_q4_wmma", 4, x, w, y, M, act, out_act, stream);
}
int strix_linear_q5_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q_wmma("linear_q5_wmma", 5, x, w, y, M, act, out_act, stream);
}
int strix_linear_q6_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q_wmma("linear_q6_wmma", 6, x, w, y, M, act, out_act, stream);
}
int strix_linear_q8_wmma(const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    return linear_q_wmma("linear_q8_wmma", 8, x, w, y, M, act, out_act, stream);
}
int strix_linear_bf16w_wmma(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, int act, int out_act, void *stream) {
    const char *fn = "linear_bf16w_wmma";
    SB_CHECK(x != nullptr && w != nullptr && y != nullptr, fn, ": null pointer");
    SB_CHECK(act == STRIX_ACT_BF16 && out_act == STRIX_ACT_F32, fn, ": BF16 tokens with FP32 outputs only (the router projection), got ",
             act_name(act), " -> ", act_name(out_act));
    SB_CHECK(N >= 1 && sb::dense_bf16_ok(x, w, M, N, K) && reinterpret_cast<uintptr_t>(y) % 4 == 0, fn, ": M = ", M, ", N = ", N, ", K = ", K,
             ": needs K % 64 == 0 and 16-byte aligned x and W");
    return sb::dense_bf16(fn, x, w, static_cast<float *>(y), M, N, K, nullptr, 0, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
