// Shared host + device helpers of the sm_100a MoE-FFN library.
//
// Error convention (mirrors strixite common/check.hpp:43-61 across a C ABI): every entry point validates its
// arguments first; a failed check stores "func (file:line): check `cond` failed: message" in a thread-local string
// (strix_last_error) and returns STRIX_ERR_CHECK; CUDA launch failures return STRIX_ERR_CUDA the same way. Data
// errors found on the device (bad expert ids, non-finite logits) never fail a call: they set the caller's err
// words {1, a, b} (first flag wins) and poison the affected outputs with NaN.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <sstream>
#include <string>
#include <type_traits>

#define STRIX_OK 0
#define STRIX_ERR_CHECK 1
#define STRIX_ERR_CUDA 2

namespace sb {

std::string &last_error();  // thread-local (api.cu)

template <typename... Args>
inline std::string cat(Args &&...args) {
    std::ostringstream os;
    (os << ... << args);
    return os.str();
}

inline int fail_check(const char *file, int line, const char *func, const char *cond, const std::string &msg) {
    const char *base = file;
    for (const char *p = file; *p; ++p)
        if (*p == '/') base = p + 1;
    last_error() = cat(func, " (", base, ":", line, "): check `", cond, "` failed: ", msg);
    return STRIX_ERR_CHECK;
}

inline int fail_cuda(const char *file, int line, const char *func, cudaError_t e, const std::string &msg) {
    const char *base = file;
    for (const char *p = file; *p; ++p)
        if (*p == '/') base = p + 1;
    last_error() = cat(func, " (", base, ":", line, "): CUDA error ", cudaGetErrorName(e), " (", cudaGetErrorString(e), "): ", msg);
    return STRIX_ERR_CUDA;
}

}  // namespace sb

#define SB_CHECK(cond, ...)                                                                             \
    do {                                                                                                \
        if (!(cond)) return ::sb::fail_check(__FILE__, __LINE__, __func__, #cond, ::sb::cat(__VA_ARGS__)); \
    } while (0)

#define SB_CUDA(expr, ...)                                                                              \
    do {                                                                                                \
        cudaError_t sb_e_ = (expr);                                                                     \
        if (sb_e_ != cudaSuccess) return ::sb::fail_cuda(__FILE__, __LINE__, __func__, sb_e_, ::sb::cat(__VA_ARGS__)); \
    } while (0)

// After a kernel launch: launch-configuration errors only (no synchronization).
#define SB_LAUNCH_OK(...) SB_CUDA(cudaGetLastError(), __VA_ARGS__)

// Propagate a nonzero status from a helper.
#define SB_TRY(expr)                 \
    do {                             \
        int sb_rc_ = (expr);         \
        if (sb_rc_ != 0) return sb_rc_; \
    } while (0)

namespace sb {

enum Act : int { kF32 = 0, kBF16 = 1 };  // strixite kernels/norm.hpp:20
inline const char *act_name(int a) { return a == kF32 ? "f32" : a == kBF16 ? "bf16" : "?"; }
inline bool act_ok(int a) { return a == kF32 || a == kBF16; }
inline int64_t act_size(int a) { return a == kF32 ? 4 : 2; }

inline bool apart(const void *a, int64_t an, const void *b, int64_t bn) {
    const auto ab = reinterpret_cast<uintptr_t>(a), bb = reinterpret_cast<uintptr_t>(b);
    return ab + (uintptr_t)an <= bb || bb + (uintptr_t)bn <= ab;
}
inline bool aligned16(const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// Packed row bytes of the four formats (strixite formats/q4.hpp:5, q5.hpp:31, q6.hpp:31, q8.hpp:6).
__host__ __device__ inline int64_t row_bytes(int bits, int64_t K) {
    return bits == 4 ? K / 2 : bits == 5 ? K / 2 + K / 8 : bits == 6 ? K / 2 + K / 4 : K;
}
inline bool bits_ok(int b) { return b == 4 || b == 5 || b == 6 || b == 8; }
inline bool group_ok(int64_t G) { return G == 32 || G == 64 || G == 128; }

int sm_count();  // of the current device, cached (api.cu)

// ---- device helpers --------------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
// Round to nearest even; NaN stays a quiet NaN with its sign (strixite formats/q4.cpp:14-20).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0x007fffffu) ? 0x0040u : 0u));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float qnan() { return __int_as_float(0x7fc00000); }

__device__ __forceinline__ float ld_act(const float *p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ld_act(const uint16_t *p, int64_t i) { return bf16_bits_to_f32(p[i]); }
__device__ __forceinline__ void st_act(float *p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st_act(uint16_t *p, int64_t i, float v) { p[i] = f32_to_bf16_bits(v); }
// The value a store in T followed by a load gives back.
__device__ __forceinline__ float as_stored(float v, const float *) { return v; }
__device__ __forceinline__ float as_stored(float v, const uint16_t *) { return bf16_bits_to_f32(f32_to_bf16_bits(v)); }

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

// First flag wins; the kernels never clear it (strixite kernels/moe_router.hpp:19-23).
__device__ __forceinline__ void raise_err(uint32_t *err, uint32_t a, uint32_t b) {
    if (atomicCAS(&err[0], 0u, 1u) == 0u) {
        err[1] = a;
        err[2] = b;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// 32 consecutive activations starting at element `off` (a multiple of 8), widened to FP32.
__device__ __forceinline__ void load_x32(const float *x, int64_t off, float (&v)[32]) {
    const float4 *p = reinterpret_cast<const float4 *>(x + off);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 f = p[i];
        v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
    }
}
__device__ __forceinline__ void load_x32(const uint16_t *x, int64_t off, float (&v)[32]) {
    const uint4 *p = reinterpret_cast<const uint4 *>(x + off);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 u = p[i];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

// The 32 codes of chunk c (codes 32c .. 32c + 31) of one packed row, as floats. BITS 4: 16 bytes of nibbles (low
// nibble = even k). 5: + one u32 of 5th bits (code i at bit i). 6: + two u32 of bits 4..5 (code i at bits 2(i%16) of
// word i/16). 8: 32 bytes. Row starts are 16-byte aligned for every format the entry points accept.
// A code (< 2^23) as a float without the quarter-rate integer conversion: 2^23 + code has the code in its low mantissa
// bits, and subtracting 2^23 is exact.
__device__ __forceinline__ float code_f(uint32_t code) { return __uint_as_float(0x4B000000u | code) - 8388608.0f; }

template <int BITS>
__device__ __forceinline__ void load_codes32(const uint8_t *row, int64_t K, int64_t c, float (&q)[32]) {
    if constexpr (BITS == 8) {
        const uint4 *p = reinterpret_cast<const uint4 *>(row + c * 32);
        const uint4 a = p[0], b = p[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 32; ++i) q[i] = code_f((w[i / 4] >> (8 * (i % 4))) & 0xFFu);
    } else {
        const uint4 a = *reinterpret_cast<const uint4 *>(row + c * 16);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
        if constexpr (BITS == 4) {
#pragma unroll
            for (int i = 0; i < 32; ++i) q[i] = code_f((w[i / 8] >> (4 * (i % 8))) & 0xFu);
        } else if constexpr (BITS == 5) {
            const uint32_t hb = *reinterpret_cast<const uint32_t *>(row + K / 2 + c * 4);
#pragma unroll
            for (int i = 0; i < 32; ++i) q[i] = code_f(((w[i / 8] >> (4 * (i % 8))) & 0xFu) | (((hb >> i) & 1u) << 4));
        } else {
            const uint2 hb = *reinterpret_cast<const uint2 *>(row + K / 2 + c * 8);
            const uint32_t h[2] = {hb.x, hb.y};
#pragma unroll
            for (int i = 0; i < 32; ++i)
                q[i] = code_f(((w[i / 8] >> (4 * (i % 8))) & 0xFu) | (((h[i / 16] >> (2 * (i % 16))) & 3u) << 4));
        }
    }
}

// One lane's share of dot(dequant(row), x): chunks c = first, first + stride, .. < chunks; per chunk
// acc = fma(s, sum x*q, fma(m, sum x, acc)) - one FMA per weight, scale and min applied once per chunk
// (the arithmetic form of strixite kernels/linear_q4.hip:88-94).
template <int BITS, typename T>
__device__ __forceinline__ float row_partial(const uint8_t *row, const uint16_t *srow, const uint16_t *mrow, const T *x,
                                             int64_t K, int G, int64_t first, int64_t stride) {
    float acc = 0.f;
    for (int64_t c = first; c < K / 32; c += stride) {
        float q[32], xv[32];
        load_codes32<BITS>(row, K, c, q);
        load_x32(x, c * 32, xv);
        const float s = bf16_bits_to_f32(srow[c * 32 / G]), m = bf16_bits_to_f32(mrow[c * 32 / G]);
        float dot = 0.f, xs = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) dot = fmaf(xv[i], q[i], dot), xs += xv[i];
        acc = fmaf(s, dot, fmaf(m, xs, acc));
    }
    return acc;
}

// The same for NR rows against the same activations: x is loaded once per chunk and used for every row (these kernels are
// bound by the L1 traffic of the activation loads, 128 bytes per 16 bytes of 4-bit codes). Each row's arithmetic is
// exactly row_partial's. row[r], srow[r], mrow[r]: the rows' code bytes, scales and minimums.
template <int BITS, int NR, typename T>
__device__ __forceinline__ void row_partial_n(const uint8_t *const (&row)[NR], const uint16_t *const (&srow)[NR], const uint16_t *const (&mrow)[NR],
                                              const T *x, int64_t K, int G, int64_t first, int64_t stride, float (&acc)[NR]) {
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.f;
    for (int64_t c = first; c < K / 32; c += stride) {
        float xv[32];
        load_x32(x, c * 32, xv);
        float xs = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) xs += xv[i];
        const int64_t g = c * 32 / G;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            float q[32];
            load_codes32<BITS>(row[r], K, c, q);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) dot = fmaf(xv[i], q[i], dot);
            acc[r] = fmaf(bf16_bits_to_f32(srow[r][g]), dot, fmaf(bf16_bits_to_f32(mrow[r][g]), xs, acc[r]));
        }
    }
}

// Per-expert formats: a stack of E experts, N rows each. bits_tab / q_off null = one format (bits) for all, expert e's
// rows at q + e * N * row_bytes; else expert e's format is bits_tab[e] and its rows start at q + q_off[e].
struct StackView {
    const uint8_t *q;
    const uint16_t *scale, *minv;
    const uint8_t *bits_tab;
    const int64_t *q_off;
    int bits;
    int64_t N, K, G;
    __device__ __forceinline__ int bits_of(int64_t e) const { return bits_tab ? (int)bits_tab[e] : bits; }
    __device__ __forceinline__ const uint8_t *rows(int64_t e, int b) const {
        return q + (q_off ? q_off[e] : e * N * row_bytes(b, K));
    }
};

// Calls f(std::integral_constant<int, BITS>) for a runtime format.
template <typename F>
__device__ __forceinline__ void by_bits(int bits, F &&f) {
    switch (bits) {
        case 4: f(std::integral_constant<int, 4>{}); break;
        case 5: f(std::integral_constant<int, 5>{}); break;
        case 6: f(std::integral_constant<int, 6>{}); break;
        default: f(std::integral_constant<int, 8>{}); break;
    }
}

#endif  // __CUDACC__

}  // namespace sb
