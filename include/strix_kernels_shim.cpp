// Drop-in definitions of strixite's MoE-path kernel functions (namespace strix::kernels) over the C ABI of
// libstrixite_b200.so: compile this file into the reference's strix_kernels target INSTEAD of the .hip files that define the
// same functions (kernels/moe_router.hip, moe_grouped.hip, linear_q4.hip, linear_q56.hip, linear_q8.hip, linear.hip,
// linear_wmma.hip, swiglu.hip, residual.hip, hc.hip and hc_wmma.hip), link libstrixite_b200.so, and runtime/qwen4exp.cpp builds
// unchanged. The stream handle is passed through as an opaque pointer (a cudaStream_t on the B200 side).
//
// One function per declaration of the reference headers it includes; argument order and meaning are the reference's. A nonzero
// status of the library becomes the strix::Error the reference's own functions throw (common/check.hpp:21-24), carrying the
// library's "func (file:line): check ... failed: ..." message.
#include "kernels/hc.hpp"
#include "kernels/hc_wmma.hpp"
#include "kernels/linear.hpp"
#include "kernels/linear_q4.hpp"
#include "kernels/linear_q5.hpp"
#include "kernels/linear_q6.hpp"
#include "kernels/linear_q8.hpp"
#include "kernels/linear_wmma.hpp"
#include "kernels/moe_grouped.hpp"
#include "kernels/moe_router.hpp"
#include "kernels/residual.hpp"
#include "kernels/swiglu.hpp"

#include "common/check.hpp"

#include "strixite_b200.h"

namespace strix::kernels {

namespace {

inline void ok(int rc) {
    if (rc != 0) throw Error(strix_last_error());
}
template <typename View>  // Q4DeviceView, Q5DeviceView, Q6DeviceView, Q8DeviceView: the same six fields (runtime/q4_device.hpp:13-18)
inline strix_qview qv(const View &w) {
    return strix_qview{w.q, w.scale, w.minv, w.N, w.K, w.G};
}
inline int a(Act act) { return act == Act::F32 ? STRIX_ACT_F32 : STRIX_ACT_BF16; }
inline int m(MoeMath math) { return math == MoeMath::F32 ? STRIX_MATH_F32 : math == MoeMath::WmmaBf16 ? STRIX_MATH_WMMA_BF16 : STRIX_MATH_WMMA_F16; }

}  // namespace

// ---- kernels/moe_router.hpp:38-63 ----------------------------------------------------------------------------------------------
void moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit, int64_t shared_ld, int32_t shared_id,
                int32_t *ids, float *coef, Act act, uint32_t *err, hipStream_t stream) {
    ok(strix_moe_router(logits, ld, M, E, k, shared_logit, shared_ld, shared_id, ids, coef, a(act), err, stream));
}
void check_router_error(const uint32_t *err, const char *what) { ok(strix_check_router_error(err, what)); }
void report_router_error(const uint32_t e[3], const char *what) { ok(strix_report_router_error(e, what)); }
void moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N, uint32_t gate_index, Act act, uint32_t *err,
                    hipStream_t stream) {
    ok(strix_moe_shared_add(y, s, gate_logit, gate_ld, M, N, gate_index, a(act), err, stream));
}
void moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N, uint32_t gate_index, void *x,
                           const float *w_in, int64_t H, Act act, uint32_t *err, hipStream_t stream) {
    ok(strix_moe_shared_add_inject(y, s, gate_logit, gate_ld, M, N, gate_index, x, w_in, H, a(act), err, stream));
}

// ---- kernels/moe_grouped.hpp:43-70 ---------------------------------------------------------------------------------------------
size_t moe_route_workspace_bytes(int64_t M, int64_t A, int64_t E) {
    const size_t n = strix_moe_route_workspace_bytes(M, A, E);
    if (n == 0) throw Error(strix_last_error());
    return n;
}
void moe_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, void *ws, size_t ws_bytes, uint32_t *err, hipStream_t stream) {
    ok(strix_moe_group_routes(ids, M, A, E, ws, ws_bytes, err, stream));
}
void linear_q4_experts_gather_grouped(const void *x, const Q4DeviceView &w, int64_t E, const void *ws, size_t ws_bytes, int64_t M, int64_t A, void *y, Act act,
                                      MoeMath math, hipStream_t stream) {
    const strix_qview v = qv(w);
    ok(strix_linear_q4_experts_gather_grouped(x, &v, E, ws, ws_bytes, M, A, y, a(act), m(math), stream));
}
void linear_q4_experts_combine_grouped(const void *h, const Q4DeviceView &w, int64_t E, const int32_t *ids, const float *coef, const void *ws, size_t ws_bytes,
                                       float *partial, int64_t M, int64_t A, void *y, Act act, MoeMath math, hipStream_t stream) {
    const strix_qview v = qv(w);
    ok(strix_linear_q4_experts_combine_grouped(h, &v, E, ids, coef, ws, ws_bytes, partial, M, A, y, a(act), m(math), stream));
}
void linear_q5_experts_gather_grouped(const void *x, const Q5DeviceView &w, int64_t E, const void *ws, size_t ws_bytes, int64_t M, int64_t A, void *y, Act act,
                                      MoeMath math, hipStream_t stream) {
    const strix_qview v = qv(w);
    ok(strix_linear_q5_experts_gather_grouped(x, &v, E, ws, ws_bytes, M, A, y, a(act), m(math), stream));
}
void linear_q5_experts_combine_grouped(const void *h, const Q5DeviceView &w, int64_t E, const int32_t *ids, const float *coef, const void *ws, size_t ws_bytes,
                                       float *partial, int64_t M, int64_t A, void *y, Act act, MoeMath math, hipStream_t stream) {
    const strix_qview v = qv(w);
    ok(strix_linear_q5_experts_combine_grouped(h, &v, E, ids, coef, ws, ws_bytes, partial, M, A, y, a(act), m(math), stream));
}

// ---- kernels/linear_q4.hpp:26-61 (per-slot experts, dense q4), linear_q5.hpp, linear_q6.hpp, linear_q8.hpp ------------------------
#define STRIX_SHIM_DENSE(NAME, VIEW)                                                                                              \
    void NAME(const void *x, const VIEW &w, void *y, int64_t M, Act act, Act out_act, hipStream_t stream) {                      \
        const strix_qview v = qv(w);                                                                                             \
        ok(strix_##NAME(x, &v, y, M, a(act), a(out_act), stream));                                                               \
    }
#define STRIX_SHIM_DENSE2(NAME, VIEW)                                                                                             \
    STRIX_SHIM_DENSE(NAME, VIEW)                                                                                                  \
    void NAME(const void *x, const VIEW &w, void *y, int64_t M, Act act, hipStream_t stream) { NAME(x, w, y, M, act, act, stream); }
STRIX_SHIM_DENSE2(linear_q4, Q4DeviceView)
STRIX_SHIM_DENSE2(linear_q5, Q5DeviceView)
STRIX_SHIM_DENSE2(linear_q6, Q6DeviceView)
STRIX_SHIM_DENSE2(linear_q8, Q8DeviceView)
// kernels/linear_wmma.hpp:21-29
STRIX_SHIM_DENSE(linear_q4_wmma, Q4DeviceView)
STRIX_SHIM_DENSE(linear_q5_wmma, Q5DeviceView)
STRIX_SHIM_DENSE(linear_q6_wmma, Q6DeviceView)
STRIX_SHIM_DENSE(linear_q8_wmma, Q8DeviceView)
void linear_bf16w_wmma(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, Act act, Act out_act, hipStream_t stream) {
    ok(strix_linear_bf16w_wmma(x, w, y, M, N, K, a(act), a(out_act), stream));
}

#define STRIX_SHIM_EXPERTS(BITS, VIEW)                                                                                                        \
    void linear_q##BITS##_experts_gather(const void *x, const VIEW &w, int64_t E, const int32_t *ids, int64_t M, int64_t A, void *y, Act act,  \
                                         uint32_t *err, hipStream_t stream) {                                                                \
        const strix_qview v = qv(w);                                                                                                         \
        ok(strix_linear_q##BITS##_experts_gather(x, &v, E, ids, M, A, y, a(act), err, stream));                                              \
    }                                                                                                                                        \
    void linear_q##BITS##_experts_gather_swiglu(const void *x, const VIEW &w, int64_t E, const int32_t *ids, int64_t M, int64_t A, void *h,    \
                                                Act act, uint32_t *err, hipStream_t stream) {                                                \
        const strix_qview v = qv(w);                                                                                                         \
        ok(strix_linear_q##BITS##_experts_gather_swiglu(x, &v, E, ids, M, A, h, a(act), err, stream));                                       \
    }                                                                                                                                        \
    void linear_q##BITS##_experts_combine(const void *h, const VIEW &w, int64_t E, const int32_t *ids, const float *coef, int64_t M,           \
                                          int64_t A, void *y, Act act, uint32_t *err, hipStream_t stream) {                                  \
        const strix_qview v = qv(w);                                                                                                         \
        ok(strix_linear_q##BITS##_experts_combine(h, &v, E, ids, coef, M, A, y, a(act), err, stream));                                       \
    }
STRIX_SHIM_EXPERTS(4, Q4DeviceView)
STRIX_SHIM_EXPERTS(5, Q5DeviceView)
void check_expert_error(const uint32_t *err, const char *what) { ok(strix_check_expert_error(err, what)); }
void report_expert_error(const uint32_t e[3], const char *what) { ok(strix_report_expert_error(e, what)); }

// ---- kernels/linear.hpp:20-26, swiglu.hpp:21, residual.hpp:17, hc.hpp:52-55 -----------------------------------------------------
void linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, Act act, Act out_act, hipStream_t stream) {
    ok(strix_linear_bf16w(x, w, y, M, N, K, a(act), a(out_act), stream));
}
void linear_bf16w(const void *x, const uint16_t *w, void *y, int64_t M, int64_t N, int64_t K, Act act, hipStream_t stream) {
    linear_bf16w(x, w, y, M, N, K, act, act, stream);
}
void swiglu(const void *gu, void *h, int64_t rows, int64_t I, Act act, hipStream_t stream) { ok(strix_swiglu(gu, h, rows, I, a(act), stream)); }
void residual_add(void *x, const void *y, int64_t n, Act act, hipStream_t stream) { ok(strix_residual_add(x, y, n, a(act), stream)); }
void hc_inject(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, Act act, hipStream_t stream) {
    ok(strix_hc_inject(x, y, w_in, T, d, H, a(act), stream));
}
// ---- kernels/hc.hpp:36-50: the Q4 / Q8 overloads of the two mixes (the chunk-major views have the same six fields) -----------------
void hc_mix_down(const void *x, const Q4DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps, float *h, float *w_in, float *inv,
                 Act act, hipStream_t stream) {
    const strix_qview v = qv(w);
    ok(strix_hc_mix_down(x, &v, 4, T, H, d, r, inject ? 1 : 0, eps, h, w_in, inv, a(act), stream));
}
void hc_mix_down(const void *x, const Q8DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps, float *h, float *w_in, float *inv,
                 Act act, hipStream_t stream) {
    const strix_qview v = qv(w);
    ok(strix_hc_mix_down(x, &v, 8, T, H, d, r, inject ? 1 : 0, eps, h, w_in, inv, a(act), stream));
}
void hc_mix_up(const float *h, const Q4ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d, void *u,
               Act act, hipStream_t stream) {
    const strix_qview v = qv(w_up);
    ok(strix_hc_mix_up(h, &v, 4, x, norm_w, inv, T, H, d, u, a(act), stream));
}
void hc_mix_up(const float *h, const Q8ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d, void *u,
               Act act, hipStream_t stream) {
    const strix_qview v = qv(w_up);
    ok(strix_hc_mix_up(h, &v, 8, x, norm_w, inv, T, H, d, u, a(act), stream));
}
// kernels/hc_wmma.hpp:26-47. hc_inject_inv has its own entry. The many-token forms of the two mixes run the same entries as
// hc_mix_down / hc_mix_up (from 16 tokens on those decode a weight chunk once per batch of tokens): the same math with FP32
// instead of F16 operands, so the partials workspace is not used and inv is always recomputed from X (inv_ready only lets
// the reference skip that pass; after hc_inject_inv it would hold the same values up to summation order).
size_t hc_wmma_workspace_bytes(int64_t T, int64_t H, int64_t R) {
    if (!(T >= 1 && H >= 1 && R >= 1)) throw Error("hc_wmma_workspace_bytes: T, H and R must be positive");
    return (size_t)(H * T * R) * 4;  // the reference's size (kernels/hc_wmma.hip:368-371): callers allocate it either way
}
void hc_mix_down_wmma(const void *x, const Q4DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps, float *h, float *w_in,
                      float *inv, float *, size_t, Act act, hipStream_t stream, bool) {
    hc_mix_down(x, w, T, H, d, r, inject, eps, h, w_in, inv, act, stream);
}
void hc_mix_down_wmma(const void *x, const Q8DeviceView &w, int64_t T, int64_t H, int64_t d, int64_t r, bool inject, float eps, float *h, float *w_in,
                      float *inv, float *, size_t, Act act, hipStream_t stream, bool) {
    hc_mix_down(x, w, T, H, d, r, inject, eps, h, w_in, inv, act, stream);
}
void hc_mix_up_wmma(const float *h, const Q4ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d,
                    void *u, Act act, hipStream_t stream) {
    hc_mix_up(h, w_up, x, norm_w, inv, T, H, d, u, act, stream);
}
void hc_mix_up_wmma(const float *h, const Q8ChunkMajorView &w_up, const void *x, const float *norm_w, const float *inv, int64_t T, int64_t H, int64_t d,
                    void *u, Act act, hipStream_t stream) {
    hc_mix_up(h, w_up, x, norm_w, inv, T, H, d, u, act, stream);
}
void hc_inject_inv(void *x, const float *w_in, const void *y, int64_t T, int64_t H, int64_t d, float eps, float *inv, Act act, hipStream_t stream) {
    ok(strix_hc_inject_inv(x, w_in, y, T, H, d, eps, inv, a(act), stream));
}

}  // namespace strix::kernels
