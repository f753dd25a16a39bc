// Router top-k + renormalized softmax, the shared expert's gated add (with and without the residual injection),
// SwiGLU, residual add and hc_inject: the small kernels around the expert GEMMs.
#include "common.cuh"

#include "strixite_b200.h"

#include <climits>

namespace {

using namespace sb;

constexpr int kRouterWarps = 8;
constexpr int64_t kMaxExperts = 1024, kMaxTopK = 32, kMaxTokens = 0x7fffffff;

// Order-preserving map float -> uint32 for finite values and -inf; -0 and +0 share a key, as they compare equal.
__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// One warp per token. Lane l keeps logits l, l + 32, .. in registers with its own best (value, lowest index).
// A selection round is two warp reductions in hardware (redux.sync): the maximum key, then the minimum index among
// the lanes holding it - larger logit first, a tie to the lower expert index (strixite kernels/moe_router.hpp:11-15).
// Only the lane that owned the pick rescans its registers. The k picks' weights are exp(l - l_top) / sum, the sum
// taken by a 32-lane xor butterfly with lanes >= k holding 0.
template <typename T, int NV>
__global__ void __launch_bounds__(kRouterWarps * 32)
    router_kernel(const T *logits, int64_t ld, int64_t M, int E, int k, const T *shared, int64_t shared_ld,
                  int32_t shared_id, int32_t *ids, float *coef, int A, uint32_t *err) {
    const int lane = threadIdx.x & 31;
    const int64_t m = (int64_t)blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
    if (m >= M) return;  // whole warps leave together; no block-level barrier below
    const T *row = logits + m * ld;
    float v[NV];
    unsigned bad = UINT_MAX;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? ld_act(row, e) : -INFINITY;
        if (e < E && !isfinite(v[j]) && (unsigned)e < bad) bad = (unsigned)e;
    }
    float sl = 0.f;
    if (shared != nullptr) {
        sl = ld_act(shared, m * shared_ld);
        if (!isfinite(sl) && (unsigned)E < bad) bad = (unsigned)E;
    }
    bad = __reduce_min_sync(0xffffffffu, bad);
    int32_t *id_row = ids + m * A;
    float *coef_row = coef + m * A;
    if (bad != UINT_MAX) {  // a non-finite logit fails the token: ids -1, coefficients NaN
        if (lane == 0) raise_err(err, (uint32_t)m, bad);
        for (int a = lane; a < A; a += 32) id_row[a] = -1, coef_row[a] = qnan();
        return;
    }
    float lv;
    int li;
    auto rescan = [&]() {
        lv = -INFINITY, li = INT_MAX;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (v[j] > lv) lv = v[j], li = lane + 32 * j;  // ascending with strict >: the lower index survives a tie
    };
    rescan();
    float my_v = -INFINITY, top = 0.f;
    int my_i = -1;
    for (int r = 0; r < k; ++r) {
        const uint32_t key = order_key(lv);
        const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
        const unsigned pick = __reduce_min_sync(0xffffffffu, key == kmax ? (unsigned)li : UINT_MAX);
        const float bv = key_value(kmax);
        if (r == 0) top = bv;
        if (lane == r) my_v = bv, my_i = (int)pick;
        if ((unsigned)li == pick) {
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (lane + 32 * j == (int)pick) v[j] = -INFINITY;
            rescan();
        }
    }
    const float ex = lane < k ? expf(my_v - top) : 0.f;
    const float sum = warp_sum(ex);
    if (lane < k) id_row[lane] = my_i, coef_row[lane] = ex / sum;
    if (shared != nullptr && lane == 0) id_row[k] = shared_id, coef_row[k] = sigmoid_f(sl);
}

// y += sigmoid(gate) * s, optionally followed by x[m, st*N + n] = fma(w_in[m, st], y, x) on the stored y for H
// streams (H = 0: no injection). One thread per column; rows on grid.y.
template <typename T, int H>
__global__ void __launch_bounds__(256)
    shared_add_kernel(T *y, const T *s, const float *gate_logit, int64_t gate_ld, int64_t N, uint32_t gate_index, T *x,
                      const float *w_in, uint32_t *err) {
    const int64_t m = blockIdx.y;
    const float gl = gate_logit[m * gate_ld];
    const bool ok = isfinite(gl);
    if (!ok && blockIdx.x == 0 && threadIdx.x == 0) raise_err(err, (uint32_t)m, gate_index);
    const float g = ok ? sigmoid_f(gl) : qnan();
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const float v = as_stored(ld_act(y, m * N + n) + g * ld_act(s, m * N + n), y);
    st_act(y, m * N + n, v);
    if constexpr (H > 0) {
#pragma unroll
        for (int st = 0; st < H; ++st) {
            const int64_t i = (m * H + st) * N + n;
            st_act(x, i, fmaf(w_in[m * H + st], v, ld_act(x, i)));
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T *gu, T *h, int64_t n, int64_t I) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / I, j = i - r * I;
        const float g = ld_act(gu, r * 2 * I + j), u = ld_act(gu, r * 2 * I + I + j);
        st_act(h, i, as_stored(silu_f(g), h) * u);  // BF16: bf16(bf16(silu(g)) * u)
    }
}

template <typename T>
__global__ void __launch_bounds__(256) add_kernel(T *x, const T *y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        st_act(x, i, ld_act(x, i) + ld_act(y, i));
}

template <typename T>
__global__ void __launch_bounds__(256) inject_kernel(T *x, const T *y, const float *w_in, int64_t M, int64_t N, int64_t H) {
    const int64_t total = M * H * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / N, n = i - row * N, m = row / H;
        st_act(x, i, fmaf(w_in[row], ld_act(y, m * N + n), ld_act(x, i)));
    }
}

int elementwise_blocks(int64_t n) {
    const int64_t want = (n + 255) / 256, cap = (int64_t)sm_count() * 32;
    return (int)(want < cap ? want : cap);
}

int shared_add_common(const char *fn, void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M,
                      int64_t N, uint32_t gate_index, void *x, const float *w_in, int64_t H, int act, uint32_t *err,
                      cudaStream_t stream) {
    SB_CHECK(y != nullptr && s != nullptr && gate_logit != nullptr && err != nullptr, fn, ": null pointer (y=", y, ", s=", s,
             ", gate_logit=", (const void *)gate_logit, ", err=", (const void *)err, ")");
    SB_CHECK(M >= 1 && M <= 65535, fn, ": M = ", M, " tokens, expected 1..65535 (grid.y)");
    SB_CHECK(N >= 1 && N <= (1ll << 24), fn, ": N = ", N, ", expected 1..2^24");
    SB_CHECK(gate_ld >= 1, fn, ": gate_ld = ", gate_ld, ", expected >= 1");
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    const int64_t yb = M * N * act_size(act);
    SB_CHECK(apart(y, yb, s, yb), fn, ": s [", s, ", +", yb, " B) overlaps y [", y, ", +", yb, " B)");
    if (x != nullptr) {
        SB_CHECK(w_in != nullptr, fn, ": null w_in");
        SB_CHECK(H == 4, fn, ": H = ", H, " streams, expected 4");
        const int64_t xb = M * H * N * act_size(act);
        SB_CHECK(apart(x, xb, y, yb) && apart(x, xb, s, yb), fn, ": x [", x, ", +", xb, " B) overlaps y [", y, "] or s [", s,
                 "] (", yb, " B each)");
    }
    const dim3 grid((unsigned)((N + 255) / 256), (unsigned)M), block(256);
    if (act == kF32) {
        if (x) shared_add_kernel<float, 4><<<grid, block, 0, stream>>>((float *)y, (const float *)s, gate_logit, gate_ld, N, gate_index, (float *)x, w_in, err);
        else shared_add_kernel<float, 0><<<grid, block, 0, stream>>>((float *)y, (const float *)s, gate_logit, gate_ld, N, gate_index, nullptr, nullptr, err);
    } else {
        if (x) shared_add_kernel<uint16_t, 4><<<grid, block, 0, stream>>>((uint16_t *)y, (const uint16_t *)s, gate_logit, gate_ld, N, gate_index, (uint16_t *)x, w_in, err);
        else shared_add_kernel<uint16_t, 0><<<grid, block, 0, stream>>>((uint16_t *)y, (const uint16_t *)s, gate_logit, gate_ld, N, gate_index, nullptr, nullptr, err);
    }
    SB_LAUNCH_OK(fn, " ", act_name(act), " M=", M, " N=", N);
    return 0;
}

int read_err(const char *fn, const uint32_t *err, const char *what, uint32_t e[3]) {
    SB_CHECK(err != nullptr, fn, "(", what ? what : "", "): null err");
    SB_CUDA(cudaMemcpy(e, err, 12, cudaMemcpyDeviceToHost), "reading the error words for ", what ? what : "");
    return 0;
}

}  // namespace

extern "C" {

int strix_moe_router(const void *logits, int64_t ld, int64_t M, int64_t E, int64_t k, const void *shared_logit,
                     int64_t shared_ld, int32_t shared_id, int32_t *ids, float *coef, int act, uint32_t *err,
                     void *stream) {
    SB_CHECK(logits != nullptr && ids != nullptr && coef != nullptr && err != nullptr, "moe_router: null pointer (logits=",
             logits, ", ids=", (const void *)ids, ", coef=", (const void *)coef, ", err=", (const void *)err, ")");
    SB_CHECK(M >= 1 && M <= kMaxTokens, "moe_router: M = ", M, " tokens, expected 1..", kMaxTokens);
    SB_CHECK(E >= 1 && E <= kMaxExperts, "moe_router: E = ", E, " experts, expected 1..", kMaxExperts);
    SB_CHECK(k >= 1 && k <= E && k <= kMaxTopK, "moe_router: k = ", k, ", expected 1..min(E = ", E, ", ", kMaxTopK, ")");
    SB_CHECK(ld >= E, "moe_router: logits row stride ld = ", ld, " < E = ", E);
    if (shared_logit != nullptr) {
        SB_CHECK(shared_ld >= 1, "moe_router: shared_ld = ", shared_ld, ", expected >= 1");
        SB_CHECK(shared_id >= 0, "moe_router: shared_id = ", shared_id, ", expected >= 0 (its expert row block)");
    }
    SB_CHECK((const void *)ids != (const void *)coef, "moe_router: ids and coef are the same buffer");
    SB_CHECK(act_ok(act), "moe_router: unsupported activation dtype ", act);
    const int A = (int)k + (shared_logit != nullptr ? 1 : 0);
    const unsigned blocks = (unsigned)((M + kRouterWarps - 1) / kRouterWarps);
    auto st = static_cast<cudaStream_t>(stream);
#define SB_ROUTER(T, NV)                                                                                            \
    router_kernel<T, NV><<<blocks, kRouterWarps * 32, 0, st>>>((const T *)logits, ld, M, (int)E, (int)k,              \
                                                               (const T *)shared_logit, shared_ld, shared_id, ids, coef, A, err)
#define SB_ROUTER_NV(T)                          \
    do {                                         \
        if (E <= 128) SB_ROUTER(T, 4);           \
        else if (E <= 256) SB_ROUTER(T, 8);      \
        else if (E <= 512) SB_ROUTER(T, 16);     \
        else SB_ROUTER(T, 32);                   \
    } while (0)
    if (act == kF32) SB_ROUTER_NV(float);
    else SB_ROUTER_NV(uint16_t);
#undef SB_ROUTER_NV
#undef SB_ROUTER
    SB_LAUNCH_OK("moe_router ", act_name(act), " M=", M, " E=", E, " k=", k, shared_logit ? " +shared" : "");
    return 0;
}

int strix_report_router_error(const uint32_t e[3], const char *what) {
    SB_CHECK(e[0] == 0, what ? what : "", ": non-finite router logit at token ", e[1], ", expert ", e[2],
             " (E = the shared-expert gate); that token's ids are -1 and its coefficients NaN");
    return 0;
}
int strix_check_router_error(const uint32_t *err, const char *what) {
    uint32_t e[3];
    SB_TRY(read_err("check_router_error", err, what, e));
    return strix_report_router_error(e, what);
}

int strix_report_expert_error(const uint32_t e[3], const char *what) {
    // {2, 0xdec000 | code, block}: a bounded wait of the single-kernel decode path ran out (0x105 / 0x200: a grid barrier, here /
    // elsewhere in the grid; 0x107: the copy of the hidden records); the layer's outputs of that forward are not valid
    SB_CHECK(!(e[0] == 2 && (e[1] & 0xfff000u) == 0xdec000u), what ? what : "", ": the decode kernel gave up a bounded wait (code 0x",
             std::hex, (e[1] & 0xfffu), std::dec, ", block ", e[2], "); outputs of that forward are not valid - reset the layer's error words "
             "(strix_moe_layer_reset_errors) before the next forward");
    SB_CHECK(e[0] == 0, what ? what : "", ": expert id ", (int32_t)e[1], " at slot ", e[2],
             " (token * A + a) is out of range; outputs for that token are NaN");
    return 0;
}
int strix_check_expert_error(const uint32_t *err, const char *what) {
    uint32_t e[3];
    SB_TRY(read_err("check_expert_error", err, what, e));
    return strix_report_expert_error(e, what);
}

int strix_moe_shared_add(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M, int64_t N,
                         uint32_t gate_index, int act, uint32_t *err, void *stream) {
    return shared_add_common("moe_shared_add", y, s, gate_logit, gate_ld, M, N, gate_index, nullptr, nullptr, 0, act, err,
                             static_cast<cudaStream_t>(stream));
}

int strix_moe_shared_add_inject(void *y, const void *s, const float *gate_logit, int64_t gate_ld, int64_t M,
                                int64_t N, uint32_t gate_index, void *x, const float *w_in, int64_t H, int act,
                                uint32_t *err, void *stream) {
    SB_CHECK(x != nullptr && w_in != nullptr, "moe_shared_add_inject: null pointer (x=", x, ", w_in=", (const void *)w_in, ")");
    return shared_add_common("moe_shared_add_inject", y, s, gate_logit, gate_ld, M, N, gate_index, x, w_in, H, act, err,
                             static_cast<cudaStream_t>(stream));
}

int strix_swiglu(const void *gu, void *h, int64_t rows, int64_t I, int act, void *stream) {
    SB_CHECK(gu != nullptr && h != nullptr, "swiglu: null pointer (gu=", gu, ", h=", h, ")");
    SB_CHECK(rows >= 1 && I >= 1, "swiglu: rows = ", rows, ", I = ", I, ", both must be >= 1");
    SB_CHECK(rows <= (1ll << 40) / I / 2, "swiglu: rows * 2I = ", rows, " * ", 2 * I, " is too large (rows/I swapped?)");
    SB_CHECK(act_ok(act), "swiglu: unsupported activation dtype ", act);
    const int64_t n = rows * I, es = act_size(act);
    SB_CHECK(apart(h, n * es, gu, 2 * n * es), "swiglu: output h [", h, ", +", n * es, " B) overlaps input gu [", gu, ", +",
             2 * n * es, " B)");
    auto st = static_cast<cudaStream_t>(stream);
    if (act == kF32) swiglu_kernel<float><<<elementwise_blocks(n), 256, 0, st>>>((const float *)gu, (float *)h, n, I);
    else swiglu_kernel<uint16_t><<<elementwise_blocks(n), 256, 0, st>>>((const uint16_t *)gu, (uint16_t *)h, n, I);
    SB_LAUNCH_OK("swiglu ", act_name(act), " rows=", rows, " I=", I);
    return 0;
}

int strix_residual_add(void *x, const void *y, int64_t n, int act, void *stream) {
    SB_CHECK(x != nullptr && y != nullptr, "residual_add: null pointer (x=", x, ", y=", y, ")");
    SB_CHECK(n >= 1 && n <= (1ll << 40), "residual_add: n = ", n, ", expected 1..2^40");
    SB_CHECK(act_ok(act), "residual_add: unsupported activation dtype ", act);
    const int64_t es = act_size(act);
    SB_CHECK(reinterpret_cast<uintptr_t>(x) % es == 0 && reinterpret_cast<uintptr_t>(y) % es == 0, "residual_add: x = ", x,
             ", y = ", y, " not aligned to ", es, " bytes");
    SB_CHECK(x == y || apart(x, n * es, y, n * es), "residual_add: y [", y, ", +", n * es, " B) partly overlaps x [", x, ")");
    auto st = static_cast<cudaStream_t>(stream);
    if (act == kF32) add_kernel<float><<<elementwise_blocks(n), 256, 0, st>>>((float *)x, (const float *)y, n);
    else add_kernel<uint16_t><<<elementwise_blocks(n), 256, 0, st>>>((uint16_t *)x, (const uint16_t *)y, n);
    SB_LAUNCH_OK("residual_add ", act_name(act), " n=", n);
    return 0;
}

int strix_hc_inject(void *x, const void *y, const float *w_in, int64_t M, int64_t N, int64_t H, int act, void *stream) {
    SB_CHECK(x != nullptr && y != nullptr && w_in != nullptr, "hc_inject: null pointer");
    SB_CHECK(M >= 1 && N >= 1 && H >= 1 && H <= 16, "hc_inject: M = ", M, ", N = ", N, ", H = ", H, " (H 1..16)");
    SB_CHECK(act_ok(act), "hc_inject: unsupported activation dtype ", act);
    const int64_t es = act_size(act);
    SB_CHECK(apart(x, M * H * N * es, y, M * N * es), "hc_inject: x overlaps y");
    auto st = static_cast<cudaStream_t>(stream);
    const int blocks = elementwise_blocks(M * H * N);
    if (act == kF32) inject_kernel<float><<<blocks, 256, 0, st>>>((float *)x, (const float *)y, w_in, M, N, H);
    else inject_kernel<uint16_t><<<blocks, 256, 0, st>>>((uint16_t *)x, (const uint16_t *)y, w_in, M, N, H);
    SB_LAUNCH_OK("hc_inject ", act_name(act), " M=", M, " N=", N, " H=", H);
    return 0;
}

}  // extern "C"
