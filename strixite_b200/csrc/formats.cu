// The q4 / q5 / q6 / q8 weight formats: host quantizer and dequantizer (the reference's are host code too:
// strixite formats/q4.cpp:39-83, q5.cpp:58-98, q6.cpp, q8.cpp:43-78) and a device quantizer that produces the same
// bytes, so that large synthetic or converted weights can be packed where they already live.
//
// One group (G consecutive weights of a row): s = bf16((max - min) / qmax), m = bf16(min),
// code = clamp(rne((w - m) / s), 0, qmax), 0 when s == 0. IEEE division and rintf on both sides: no fast-math.
#include "common.cuh"

#include "strixite_b200.h"

#include <cfenv>
#include <cmath>
#include <cstring>

namespace {

using namespace sb;

inline uint16_t h_f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0x007fffffu) ? 0x0040u : 0u));
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float h_bf16_to_f32(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// Where code k of a row lives: low nibble plane for 4/5/6 bits, plus the high plane (1 or 2 bits) behind it.
__host__ __device__ inline void store_code(int bits, uint8_t *row, int64_t K, int64_t k, int code) {
    if (bits == 8) {
        row[k] = (uint8_t)code;
        return;
    }
    row[k >> 1] |= (uint8_t)((code & 0xF) << ((k & 1) * 4));
    if (bits == 5) row[K / 2 + (k >> 3)] |= (uint8_t)(((code >> 4) & 1) << (k & 7));
    else if (bits == 6) row[K / 2 + (k >> 2)] |= (uint8_t)(((code >> 4) & 3) << ((k & 3) * 2));
}
inline int fetch_code(int bits, const uint8_t *row, int64_t K, int64_t k) {
    if (bits == 8) return row[k];
    const int lo = (row[k >> 1] >> ((k & 1) * 4)) & 0xF;
    if (bits == 4) return lo;
    if (bits == 5) return lo | (((row[K / 2 + (k >> 3)] >> (k & 7)) & 1) << 4);
    return lo | (((row[K / 2 + (k >> 2)] >> ((k & 3) * 2)) & 3) << 4);
}

int check_shape(const char *fn, int bits, int64_t N, int64_t K, int64_t G) {
    SB_CHECK(bits_ok(bits), fn, ": ", bits, " bits, expected 4, 5, 6 or 8");
    SB_CHECK(N >= 1 && K >= 1, fn, ": shape [", N, ", ", K, "] must be positive");
    SB_CHECK(group_ok(G), fn, ": group size ", G, " unsupported (32, 64 or 128)");
    SB_CHECK(K % G == 0, fn, ": K = ", K, " is not a multiple of group size ", G);
    SB_CHECK(bits != 5 || K % 128 == 0, fn, ": Q5 K = ", K, " is not a multiple of 128 (16-byte aligned code planes)");
    SB_CHECK(bits != 6 || K % 64 == 0, fn, ": Q6 K = ", K, " is not a multiple of 64 (16-byte aligned code planes)");
    return 0;
}

// One warp per group; lanes stride over the group's G weights. Codes are assembled per byte by the lane that owns
// the byte's first weight, so no two lanes write the same byte: a lane handles the weights of whole bytes.
// Layout of work: a lane owns 8 consecutive weights (4 nibble bytes, 1 byte of 5th bits, 2 bytes of 6-bit highs,
// 8 bytes of q8), G / 8 lanes active per group.
template <int BITS>
__global__ void __launch_bounds__(256) quantize_kernel(const float *w, int64_t N, int64_t K, int G, uint8_t *q,
                                                       uint16_t *scale, uint16_t *minv, uint32_t *err) {
    const int64_t groups = N * (K / G);
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    constexpr float qmax = (float)((1 << BITS) - 1);
    const int64_t rb = row_bytes(BITS, K);
    for (int64_t gi = warp; gi < groups; gi += n_warps) {
        const int64_t n = gi / (K / G), g = gi % (K / G);
        const float *grp = w + n * K + g * G;
        const bool active = lane * 8 < G;
        float v[8];
        float lo = grp[0], hi = lo;
        bool bad = false;
        int bad_col = 0x7fffffff;
        if (active) {
            const float4 a = reinterpret_cast<const float4 *>(grp)[lane * 2], b = reinterpret_cast<const float4 *>(grp)[lane * 2 + 1];
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (!isfinite(v[i]) && !bad) bad = true, bad_col = (int)(g * G) + lane * 8 + i;
                lo = fminf(lo, v[i]);
                hi = fmaxf(hi, v[i]);
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
            bad_col = min(bad_col, __shfl_xor_sync(0xffffffffu, bad_col, off));
        }
        if (bad_col != 0x7fffffff && lane == 0) raise_err(err, (uint32_t)n, (uint32_t)bad_col);
        const uint16_t s_bits = f32_to_bf16_bits((hi - lo) / qmax), m_bits = f32_to_bf16_bits(lo);
        const float s = bf16_bits_to_f32(s_bits), m = bf16_bits_to_f32(m_bits);
        if (lane == 0) scale[gi] = s_bits, minv[gi] = m_bits;
        if (!active) continue;
        uint32_t code[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float r = 0.f;
            if (s > 0.0f) r = fminf(fmaxf(rintf((v[i] - m) / s), 0.0f), qmax);
            code[i] = (uint32_t)(int)r;
        }
        uint8_t *row = q + n * rb;
        const int64_t k0 = g * G + lane * 8;
        if constexpr (BITS == 8) {
            uint2 o;
            o.x = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
            o.y = code[4] | (code[5] << 8) | (code[6] << 16) | (code[7] << 24);
            *reinterpret_cast<uint2 *>(row + k0) = o;
        } else {
            uint32_t lo4 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) lo4 |= (code[i] & 0xFu) << (4 * i);
            *reinterpret_cast<uint32_t *>(row + k0 / 2) = lo4;
            if constexpr (BITS == 5) {
                uint32_t h = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) h |= ((code[i] >> 4) & 1u) << i;
                row[K / 2 + k0 / 8] = (uint8_t)h;
            } else if constexpr (BITS == 6) {
                uint32_t h = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) h |= ((code[i] >> 4) & 3u) << (2 * i);
                *reinterpret_cast<uint16_t *>(row + K / 2 + k0 / 4) = (uint16_t)h;
            }
        }
    }
}

}  // namespace

extern "C" {

// strixite formats/strixw.hpp:59 strix_hash64 (formats/strixw.cpp:197-221): four interleaved multiply-xorshift lanes over
// 8-byte little-endian words, 32 bytes per step; leftover whole words go to lanes 0, 1, 2; a last partial word is tagged
// with its length; the lanes fold into one word with a final avalanche. Not a standard hash: the file format defines it.
uint64_t strix_hash64(const void *data, size_t n) {
    constexpr uint64_t k1 = 0x9e3779b97f4a7c15ull, k2 = 0xd6e8feb86659fd93ull;
    auto mix = [](uint64_t h, uint64_t w) {
        h ^= w * k1;
        return (h ^ (h >> 31)) * k2;
    };
    const auto *p = static_cast<const uint8_t *>(data);
    uint64_t lanes[4] = {n ^ k1, n ^ k2, ~(uint64_t)n ^ k1, ~(uint64_t)n ^ k2};
    size_t i = 0;
    for (; i + 32 <= n; i += 32)
        for (int l = 0; l < 4; ++l) {
            uint64_t w;
            std::memcpy(&w, p + i + 8 * l, 8);
            lanes[l] = mix(lanes[l], w);
        }
    for (int l = 0; i + 8 <= n; i += 8, ++l) {
        uint64_t w;
        std::memcpy(&w, p + i, 8);
        lanes[l] = mix(lanes[l], w);
    }
    if (i < n) {
        uint64_t w = 0;
        std::memcpy(&w, p + i, n - i);
        lanes[0] = mix(lanes[0], w ^ ((uint64_t)(n - i) << 56));
    }
    uint64_t r = mix(mix(mix(lanes[0], lanes[1]), lanes[2]), lanes[3]);
    r ^= r >> 33;
    r *= k1;
    return r ^ (r >> 29);
}

int64_t strix_row_bytes(int bits, int64_t K) { return sb::row_bytes(bits, K); }

int strix_check_qweight(int bits, int64_t N, int64_t K, int64_t G, size_t q_bytes, size_t n_scale, size_t n_min) {
    SB_TRY(check_shape("check_qweight", bits, N, K, G));
    SB_CHECK(q_bytes == (size_t)(N * row_bytes(bits, K)), "check_qweight: code array has ", q_bytes,
             " bytes, expected N * row_bytes = ", N * row_bytes(bits, K));
    const size_t n_groups = (size_t)(N * (K / G));
    SB_CHECK(n_scale == n_groups && n_min == n_groups, "check_qweight: scale/min arrays have ", n_scale, "/", n_min,
             " entries, expected N*K/G = ", n_groups);
    return 0;
}

int strix_quantize(int bits, const float *w, int64_t N, int64_t K, int64_t G, uint8_t *q, uint16_t *scale,
                   uint16_t *minv) {
    SB_CHECK(w != nullptr && q != nullptr && scale != nullptr && minv != nullptr, "quantize: null pointer");
    SB_TRY(check_shape("quantize", bits, N, K, G));
    SB_CHECK(std::fegetround() == FE_TONEAREST, "quantize: FP rounding mode isn't round-to-nearest-even");
    const int64_t rb = row_bytes(bits, K), gpr = K / G;
    const float qmax = (float)((1 << bits) - 1);
    std::memset(q, 0, (size_t)(N * rb));
    for (int64_t n = 0; n < N; ++n)
        for (int64_t g = 0; g < gpr; ++g) {
            const float *grp = w + n * K + g * G;
            float lo = grp[0], hi = grp[0];
            for (int64_t i = 0; i < G; ++i) {
                SB_CHECK(std::isfinite(grp[i]), "quantize: non-finite weight ", grp[i], " at [", n, ", ", g * G + i, "]");
                lo = std::fmin(lo, grp[i]), hi = std::fmax(hi, grp[i]);
            }
            const uint16_t sb_ = h_f32_to_bf16((hi - lo) / qmax), mb = h_f32_to_bf16(lo);
            scale[n * gpr + g] = sb_, minv[n * gpr + g] = mb;
            const float s = h_bf16_to_f32(sb_), m = h_bf16_to_f32(mb);
            if (!(s > 0.0f)) continue;  // a constant group: every code 0
            for (int64_t i = 0; i < G; ++i) {
                const float r = std::fmin(std::fmax(std::nearbyint((grp[i] - m) / s), 0.0f), qmax);
                store_code(bits, q + n * rb, K, g * G + i, (int)r);
            }
        }
    return 0;
}

int strix_dequantize(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K,
                     int64_t G, float *w) {
    SB_CHECK(w != nullptr && q != nullptr && scale != nullptr && minv != nullptr, "dequantize: null pointer");
    SB_TRY(check_shape("dequantize", bits, N, K, G));
    const int64_t rb = row_bytes(bits, K), gpr = K / G;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) {
            // Two roundings (product, then sum): volatile keeps the compiler from fusing them.
            volatile float p = (float)fetch_code(bits, q + n * rb, K, k) * h_bf16_to_f32(scale[n * gpr + k / G]);
            w[n * K + k] = p + h_bf16_to_f32(minv[n * gpr + k / G]);
        }
    return 0;
}

int strix_quantize_device(int bits, const float *w, int64_t N, int64_t K, int64_t G, uint8_t *q, uint16_t *scale,
                          uint16_t *minv, uint32_t *err, void *stream) {
    SB_CHECK(w != nullptr && q != nullptr && scale != nullptr && minv != nullptr && err != nullptr,
             "quantize_device: null pointer");
    SB_TRY(check_shape("quantize_device", bits, N, K, G));
    SB_CHECK(aligned16(w) && reinterpret_cast<uintptr_t>(q) % 8 == 0, "quantize_device: w must be 16-byte and q 8-byte aligned");
    const int64_t groups = N * (K / G);
    const int64_t want = (groups + 7) / 8;
    const int blocks = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
    auto st = static_cast<cudaStream_t>(stream);
    switch (bits) {
        case 4: quantize_kernel<4><<<blocks, 256, 0, st>>>(w, N, K, (int)G, q, scale, minv, err); break;
        case 5: quantize_kernel<5><<<blocks, 256, 0, st>>>(w, N, K, (int)G, q, scale, minv, err); break;
        case 6: quantize_kernel<6><<<blocks, 256, 0, st>>>(w, N, K, (int)G, q, scale, minv, err); break;
        default: quantize_kernel<8><<<blocks, 256, 0, st>>>(w, N, K, (int)G, q, scale, minv, err); break;
    }
    SB_LAUNCH_OK("quantize_device q", bits, " N=", N, " K=", K, " G=", G);
    return 0;
}

}  // extern "C"
