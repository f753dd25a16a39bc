// TEST INFRASTRUCTURE - NOT PRODUCT CODE.
//
// C-ABI doors onto the REFERENCE's own host quantizers (strixite formats/q4.cpp, q5.cpp, q6.cpp, q8.cpp,
// q4_from_q8.cpp), which build.py compiles unchanged from the mounted reference tree, where they lie, into
// oracle/_ref/libstrix_formats_ref.so. This file holds no arithmetic: it only copies between the reference's
// std::vector-based structs and flat arrays, and turns strix::Error into a return code + message.
// Used to pin moe_oracle.cpp's quantizer restatement and to generate tests/golden/.

#include "formats/q4.hpp"
#include "formats/q4_from_q8.hpp"
#include "formats/q5.hpp"
#include "formats/q6.hpp"
#include "formats/q8.hpp"

#include <cstdint>
#include <cstring>
#include <exception>
#include <string>

namespace {
thread_local std::string g_msg;

template <typename W>
void copy_out(const W &w, uint8_t *q, uint16_t *scale, uint16_t *minv) {
    std::memcpy(q, w.q.data(), w.q.size());
    std::memcpy(scale, w.scale.data(), w.scale.size() * 2);
    std::memcpy(minv, w.minv.data(), w.minv.size() * 2);
}
template <typename W>
W make(const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K, int64_t G, int64_t rb) {
    W w;
    w.N = N, w.K = K, w.G = G;
    w.q.assign(q, q + N * rb);
    w.scale.assign(scale, scale + N * (K / G));
    w.minv.assign(minv, minv + N * (K / G));
    return w;
}
}  // namespace

extern "C" {

const char *ref_last_error() { return g_msg.c_str(); }

int ref_quantize(int bits, const float *w, int64_t N, int64_t K, int64_t G, uint8_t *q, uint16_t *scale,
                 uint16_t *minv) {
    try {
        switch (bits) {
            case 4: copy_out(strix::quantize_q4(w, N, K, G), q, scale, minv); return 0;
            case 5: copy_out(strix::quantize_q5(w, N, K, G), q, scale, minv); return 0;
            case 6: copy_out(strix::quantize_q6(w, N, K, G), q, scale, minv); return 0;
            case 8: copy_out(strix::quantize_q8(w, N, K, G), q, scale, minv); return 0;
            default: g_msg = "ref_quantize: bits must be 4, 5, 6 or 8"; return 2;
        }
    } catch (const std::exception &e) {
        g_msg = e.what();
        return 1;
    }
}

int ref_dequantize(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K,
                   int64_t G, float *out) {
    try {
        std::vector<float> v;
        switch (bits) {
            case 4: v = strix::dequantize_q4(make<strix::Q4Weight>(q, scale, minv, N, K, G, K / 2)); break;
            case 5: v = strix::dequantize_q5(make<strix::Q5Weight>(q, scale, minv, N, K, G, strix::q5_row_bytes(K))); break;
            case 6: v = strix::dequantize_q6(make<strix::Q6Weight>(q, scale, minv, N, K, G, strix::q6_row_bytes(K))); break;
            case 8: v = strix::dequantize_q8(make<strix::Q8Weight>(q, scale, minv, N, K, G, K)); break;
            default: g_msg = "ref_dequantize: bits must be 4, 5, 6 or 8"; return 2;
        }
        std::memcpy(out, v.data(), v.size() * 4);
        return 0;
    } catch (const std::exception &e) {
        g_msg = e.what();
        return 1;
    }
}

// formats/q4_from_q8.hpp: Q8 rows -> the Q4 nearest to what the engine serves.
int ref_q4_from_q8(const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K, int64_t G8,
                   int64_t G4, int threads, uint8_t *q4, uint16_t *scale4, uint16_t *minv4) {
    try {
        copy_out(strix::quantize_q4_from_q8(make<strix::Q8Weight>(q, scale, minv, N, K, G8, K), G4, threads), q4,
                 scale4, minv4);
        return 0;
    } catch (const std::exception &e) {
        g_msg = e.what();
        return 1;
    }
}

// formats/q4.hpp:55 / formats/q8.hpp:46 to_chunk_major: the reference's own row-major -> chunk-major conversion.
int ref_to_chunk_major(int bits, const uint8_t *q, const uint16_t *scale, const uint16_t *minv, int64_t N, int64_t K,
                       int64_t G, uint8_t *q_out, uint16_t *scale_out, uint16_t *min_out) {
    try {
        if (bits == 4) copy_out(strix::to_chunk_major(make<strix::Q4Weight>(q, scale, minv, N, K, G, K / 2), "ref_to_chunk_major"), q_out, scale_out, min_out);
        else if (bits == 8) copy_out(strix::to_chunk_major(make<strix::Q8Weight>(q, scale, minv, N, K, G, K), "ref_to_chunk_major"), q_out, scale_out, min_out);
        else {
            g_msg = "ref_to_chunk_major: bits must be 4 or 8";
            return 2;
        }
        return 0;
    } catch (const std::exception &e) {
        g_msg = e.what();
        return 1;
    }
}

}  // extern "C"
