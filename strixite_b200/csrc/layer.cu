// The MoE sublayer as one object: the sequence strixite's Qwen4ExpSession::forward runs per layer
// (runtime/qwen4exp.cpp:1126-1186) over the library's own entry points, with the session buffers it needs.
// Nothing here computes: it validates, owns workspaces, picks the per-slot or grouped experts path and enqueues.
#include "common.cuh"

#include "decode_stream.cuh"
#include "grouped.cuh"
#include "prefill_umma.cuh"
#include "strixite_b200.h"

#include <cstring>
#include <new>

// Built with -DSTRIX_NVTX only: named host ranges around the phases a forward enqueues, for a timeline profiler.
#ifdef STRIX_NVTX
#include <nvtx3/nvToolsExt.h>
namespace {
struct NvtxRange {
    explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
};
}  // namespace
#define STRIX_RANGE(var, name) NvtxRange var(name)
#else
#define STRIX_RANGE(var, name) \
    do {                       \
    } while (0)
#endif

namespace {

using namespace sb;

// logits[m, e] += bias[e] for e < E (a harness-side routing skew; not part of the reference's layer).
__global__ void __launch_bounds__(256) add_bias_kernel(float *logits, int64_t ld, int64_t M, int64_t E, const float *bias) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * E) return;
    const int64_t m = i / E, e = i - m * E;
    logits[m * ld + e] += bias[e];
}

// The stacked shared slot with a constant coefficient: ids[m, k] = shared_id, coef[m, k] = 1 after the router wrote
// the k routed slots with row stride A = k + 1.
__global__ void __launch_bounds__(256) fill_shared_slot_kernel(int32_t *ids, float *coef, int64_t M, int64_t A, int32_t shared_id) {
    const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    const bool failed = ids[m * A] < 0;  // a token the router failed keeps -1 / NaN in every slot
    ids[m * A + A - 1] = failed ? -1 : shared_id;
    coef[m * A + A - 1] = failed ? qnan() : 1.0f;
}

// The router writes rows of k entries; re-spread them to stride A = k + 1 (back to front, one block per token row would
// race across rows, so one thread walks a token: k <= 32 entries).
__global__ void __launch_bounds__(256) widen_rows_kernel(const int32_t *ids_in, const float *coef_in, int32_t *ids, float *coef,
                                                         int64_t M, int64_t k) {
    const int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    for (int64_t a = 0; a < k; ++a) ids[m * (k + 1) + a] = ids_in[m * k + a], coef[m * (k + 1) + a] = coef_in[m * k + a];
}

template <typename T>
int dev_alloc(T **p, size_t n, const char *what) {
    SB_CUDA(cudaMalloc(reinterpret_cast<void **>(p), n * sizeof(T) > 0 ? n * sizeof(T) : 16), "allocating ", what, " (", n * sizeof(T), " B)");
    return 0;
}

}  // namespace

struct strix_moe_layer {
    strix_moe_layer_desc d;
    int64_t A, Estack, router_rows;
    bool gated;
    // session buffers (strixite runtime/qwen4exp.cpp:297-380)
    float *logits = nullptr;       // [max_tokens, router_rows]
    int32_t *ids = nullptr, *ids_k = nullptr;  // [max_tokens, A], router output when it must be widened
    float *coef = nullptr, *coef_k = nullptr;
    void *gu = nullptr, *hh = nullptr, *sh_h = nullptr, *sh_y = nullptr;  // act dtype
    float *partial = nullptr;
    void *group_ws = nullptr;
    size_t group_ws_bytes = 0;
    int32_t *route_scratch = nullptr;  // per-segment counts of the multi-block grouping
    uint32_t *err = nullptr;       // [8]: router words 0..2, expert words 3..5
    // host staging
    void *pin_x = nullptr, *pin_y = nullptr;
    uint32_t *pin_err = nullptr;
    void *dev_x = nullptr, *dev_y = nullptr;
    int64_t last_M = 0;
    // the streaming decode kernel's scratch and plan
    uint8_t *hrec = nullptr;
    uint32_t *sync = nullptr;
    bool fused_ok = false;
    sb::StreamParams plan{};
    // the tensor-core path for many tokens (math != F32, uniform 4-bit stacks)
    sb::PrefillPlan *prefill = nullptr;
    int64_t tensor_min = 64;
};

namespace {

constexpr int64_t kPrefillMinTokens = 64;  // below this the FP32 grouped kernels do less padded work

int check_desc(const strix_moe_layer_desc &d) {
    const char *fn = "moe_layer_create";
    SB_CHECK(d.d >= 32 && d.I >= 32 && d.E >= 1 && d.E <= 1023 && d.k >= 1 && d.k <= 32 && d.k <= d.E, fn, ": d = ", d.d, ", I = ", d.I,
             ", E = ", d.E, ", k = ", d.k, " (E 1..1023, k 1..min(32, E))");
    SB_CHECK(act_ok(d.act), fn, ": unsupported activation dtype ", d.act);
    SB_CHECK(d.shared_mode >= 0 && d.shared_mode <= 2 && d.shared_coef_mode >= 0 && d.shared_coef_mode <= 1, fn, ": shared_mode ",
             d.shared_mode, " / shared_coef_mode ", d.shared_coef_mode);
    SB_CHECK(d.max_tokens >= 1 && d.max_tokens * (d.k + 1) <= (1 << 20), fn, ": max_tokens = ", d.max_tokens);
    SB_CHECK(d.grouped_min_tokens >= 1, fn, ": grouped_min_tokens = ", d.grouped_min_tokens);
    const bool gated = d.shared_mode != STRIX_SHARED_NONE && d.shared_coef_mode == STRIX_SHARED_COEF_SIGMOID;
    const int64_t rows = d.E + (gated ? 1 : 0), Estack = d.E + (d.shared_mode == STRIX_SHARED_STACKED ? 1 : 0);
    if (d.router_kind == STRIX_ROUTER_Q) {
        SB_CHECK(bits_ok(d.router_bits) && d.router_q.q != nullptr && d.router_q.N == rows && d.router_q.K == d.d, fn,
                 ": quantized router must be [", rows, ", ", d.d, "], got [", d.router_q.N, ", ", d.router_q.K, "] in ", d.router_bits, " bits");
    } else {
        SB_CHECK((d.router_kind == STRIX_ROUTER_F32 || d.router_kind == STRIX_ROUTER_BF16) && d.router_w != nullptr, fn,
                 ": router_kind ", d.router_kind, " needs router_w");
    }
    if (d.experts_mixed) {
        SB_CHECK(d.gate_up_mix.E == Estack && d.gate_up_mix.N == 2 * d.I && d.gate_up_mix.K == d.d, fn, ": gate_up_mix must be ", Estack,
                 " experts of [", 2 * d.I, ", ", d.d, "]");
        SB_CHECK(d.down_mix.E == Estack && d.down_mix.N == d.d && d.down_mix.K == d.I, fn, ": down_mix must be ", Estack, " experts of [",
                 d.d, ", ", d.I, "]");
    } else {
        // strixite runtime/qweight.hpp:75-125: expert stacks are 4 or 5 bits.
        SB_CHECK((d.gate_up_bits == 4 || d.gate_up_bits == 5) && (d.down_bits == 4 || d.down_bits == 5), fn, ": experts have ",
                 d.gate_up_bits, "/", d.down_bits, " bits, expected 4 or 5 (or a per-expert format table)");
        SB_CHECK(d.gate_up.N == Estack * 2 * d.I && d.gate_up.K == d.d, fn, ": gate_up must be [", Estack * 2 * d.I, ", ", d.d, "], got [",
                 d.gate_up.N, ", ", d.gate_up.K, "]");
        SB_CHECK(d.down.N == Estack * d.d && d.down.K == d.I, fn, ": down must be [", Estack * d.d, ", ", d.I, "], got [", d.down.N, ", ",
                 d.down.K, "]");
    }
    if (d.shared_mode == STRIX_SHARED_SEPARATE) {
        SB_CHECK(bits_ok(d.sh_gate_up_bits) && bits_ok(d.sh_down_bits), fn, ": shared expert bits ", d.sh_gate_up_bits, "/", d.sh_down_bits);
        SB_CHECK(d.sh_gate_up.N == 2 * d.I && d.sh_gate_up.K == d.d && d.sh_down.N == d.d && d.sh_down.K == d.I, fn,
                 ": shared expert must be [", 2 * d.I, ", ", d.d, "] and [", d.d, ", ", d.I, "]");
    }
    return 0;
}

int linear_any(int bits, const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    switch (bits) {
        case 4: return strix_linear_q4(x, w, y, M, act, out_act, stream);
        case 5: return strix_linear_q5(x, w, y, M, act, out_act, stream);
        case 6: return strix_linear_q6(x, w, y, M, act, out_act, stream);
        default: return strix_linear_q8(x, w, y, M, act, out_act, stream);
    }
}

int linear_wmma_any(int bits, const void *x, const strix_qview *w, void *y, int64_t M, int act, int out_act, void *stream) {
    switch (bits) {
        case 4: return strix_linear_q4_wmma(x, w, y, M, act, out_act, stream);
        case 5: return strix_linear_q5_wmma(x, w, y, M, act, out_act, stream);
        case 6: return strix_linear_q6_wmma(x, w, y, M, act, out_act, stream);
        default: return strix_linear_q8_wmma(x, w, y, M, act, out_act, stream);
    }
}

}  // namespace

extern "C" {

int strix_moe_layer_create(const strix_moe_layer_desc *desc, strix_moe_layer **out) {
    SB_CHECK(desc != nullptr && out != nullptr, "moe_layer_create: null pointer");
    SB_TRY(check_desc(*desc));
    auto *L = new (std::nothrow) strix_moe_layer();
    SB_CHECK(L != nullptr, "moe_layer_create: out of host memory");
    L->d = *desc;
    const auto &d = L->d;
    L->gated = d.shared_mode != STRIX_SHARED_NONE && d.shared_coef_mode == STRIX_SHARED_COEF_SIGMOID;
    L->router_rows = d.E + (L->gated ? 1 : 0);
    L->Estack = d.E + (d.shared_mode == STRIX_SHARED_STACKED ? 1 : 0);
    L->A = d.k + (d.shared_mode == STRIX_SHARED_STACKED ? 1 : 0);
    const int64_t T = d.max_tokens, es = act_size(d.act);
    int rc = 0;
    auto a = [&](int r) { if (rc == 0) rc = r; };
    a(dev_alloc(&L->logits, (size_t)(T * L->router_rows), "router logits"));
    a(dev_alloc(&L->ids, (size_t)(T * L->A), "route ids"));
    a(dev_alloc(&L->coef, (size_t)(T * L->A), "route coefficients"));
    a(dev_alloc(&L->ids_k, (size_t)(T * d.k), "route ids (k)"));
    a(dev_alloc(&L->coef_k, (size_t)(T * d.k), "route coefficients (k)"));
    a(dev_alloc((char **)&L->gu, (size_t)(T * L->A * 2 * d.I * es), "gate_up outputs"));
    a(dev_alloc((char **)&L->hh, (size_t)(T * L->A * d.I * es), "expert hidden"));
    a(dev_alloc((char **)&L->sh_h, (size_t)(T * d.I * es), "shared hidden"));
    a(dev_alloc((char **)&L->sh_y, (size_t)(T * d.d * es), "shared output"));
    a(dev_alloc(&L->partial, (size_t)(T * L->A * d.d), "combine partials"));
    L->group_ws_bytes = strix_moe_route_workspace_bytes(T, L->A, L->Estack);
    a(L->group_ws_bytes == 0 ? STRIX_ERR_CHECK : 0);
    a(dev_alloc((char **)&L->group_ws, L->group_ws_bytes, "grouping workspace"));
    a(dev_alloc((char **)&L->route_scratch, sb::route_scratch_bytes(L->Estack), "grouping scratch"));
    if (rc == 0) rc = sb::route_scratch_init(L->route_scratch, L->Estack, nullptr);
    a(dev_alloc(&L->err, 8, "error words"));
    a(dev_alloc((char **)&L->dev_x, (size_t)(T * d.d * es), "x staging"));
    a(dev_alloc((char **)&L->dev_y, (size_t)(T * d.d * es), "y staging"));
    {
        // Streaming decode kernel: its shared-memory plan for up to 8 tokens, the h records and the barrier words.
        sb::StreamParams &p = L->plan;
        const int64_t Mf = T < 8 ? T : 8;
        p.M = (int)Mf, p.d = (int)d.d, p.I = (int)d.I, p.E = (int)d.E, p.k = (int)d.k, p.A = (int)L->A, p.R = (int)L->router_rows,
        p.Estack = (int)L->Estack, p.act = d.act, p.shared_mode = d.shared_mode, p.gated = L->gated ? 1 : 0;
        // the smallest group size among the 4/5/6-bit projections and among the 8-bit ones the kernel will stream
        int64_t g_nib = 128, g_q8 = 128;
        bool aligned = true;
        auto al = [&](const void *q) { aligned = aligned && sb::aligned16(q); };
        auto seen = [&](int bits, int64_t G) {
            int64_t &g = bits == 8 ? g_q8 : g_nib;
            g = G < g ? G : g;
        };
        if (d.experts_mixed) {
            al(d.gate_up_mix.scale), al(d.gate_up_mix.minv), al(d.down_mix.scale), al(d.down_mix.minv), al(d.gate_up_mix.q), al(d.down_mix.q);
            seen(4, d.gate_up_mix.G), seen(8, d.gate_up_mix.G), seen(4, d.down_mix.G), seen(8, d.down_mix.G);
        } else {
            al(d.gate_up.scale), al(d.gate_up.minv), al(d.down.scale), al(d.down.minv), al(d.gate_up.q), al(d.down.q);
            seen(d.gate_up_bits, d.gate_up.G), seen(d.down_bits, d.down.G);
        }
        if (d.shared_mode == STRIX_SHARED_SEPARATE) {
            al(d.sh_gate_up.scale), al(d.sh_gate_up.minv), al(d.sh_down.scale), al(d.sh_down.minv), al(d.sh_gate_up.q), al(d.sh_down.q);
            seen(d.sh_gate_up_bits, d.sh_gate_up.G), seen(d.sh_down_bits, d.sh_down.G);
        }
        if (d.router_kind != STRIX_ROUTER_Q) al(d.router_w);
        else al(d.router_q.q), aligned = aligned && d.router_bits == 8;  // quantized routers: 8-bit rows only
        {
            const bool experts_q4 = !d.experts_mixed && d.gate_up_bits == 4 && d.down_bits == 4;
            const bool sep = d.shared_mode == STRIX_SHARED_SEPARATE;
            if (experts_q4 && (!sep || (d.sh_gate_up_bits == 4 && d.sh_down_bits == 4))) p.format_set = 0;
            else if (experts_q4 && sep && d.sh_gate_up_bits == 8 && d.sh_down_bits == 8 && d.sh_gate_up.G == 64 && d.sh_down.G == 64) p.format_set = 1;
            else p.format_set = 2;
        }
        L->fused_ok = rc == 0 && aligned && d.decode_impl == 0 && sb::decode_stream_plan(p, (int)Mf, (int)g_nib, (int)g_q8) != 0;
        if (L->fused_ok) {
            const size_t hbytes = (size_t)p.n_rec_max * (size_t)p.rec_bytes;
            a(dev_alloc(&L->hrec, hbytes, "decode h records"));
            a(dev_alloc(&L->sync, 128, "decode barrier words"));
            if (rc == 0 && (cudaMemset(L->sync, 0, 512) != cudaSuccess || cudaMemset(L->hrec, 0, hbytes) != cudaSuccess)) rc = STRIX_ERR_CUDA;
        }
    }
    L->tensor_min = d.tensor_min_tokens > 0 ? d.tensor_min_tokens : kPrefillMinTokens;
    if (rc == 0 && d.math != STRIX_MATH_F32 && sb::prefill_supported(d) && T >= L->tensor_min)
        rc = sb::prefill_create(d, L->A, L->Estack, L->router_rows, &L->prefill);
    if (rc == 0 && cudaMemset(L->err, 0, 32) != cudaSuccess) rc = STRIX_ERR_CUDA;
    if (rc == 0 && cudaMallocHost(&L->pin_x, (size_t)(T * d.d * es)) != cudaSuccess) rc = STRIX_ERR_CUDA;
    if (rc == 0 && cudaMallocHost(&L->pin_y, (size_t)(T * d.d * es)) != cudaSuccess) rc = STRIX_ERR_CUDA;
    if (rc == 0 && cudaMallocHost(reinterpret_cast<void **>(&L->pin_err), 32) != cudaSuccess) rc = STRIX_ERR_CUDA;
    if (rc != 0) {
        if (rc == STRIX_ERR_CUDA && sb::last_error().empty()) sb::last_error() = "moe_layer_create: CUDA allocation failed";
        strix_moe_layer_destroy(L);
        return rc;
    }
    *out = L;
    return 0;
}

void strix_moe_layer_destroy(strix_moe_layer *L) {
    if (L == nullptr) return;
    void *dev[] = {L->logits, L->ids, L->coef, L->ids_k, L->coef_k, L->gu, L->hh, L->sh_h, L->sh_y, L->partial, L->group_ws, L->err, L->dev_x, L->dev_y, L->hrec, L->sync, L->route_scratch};
    for (void *p : dev)
        if (p) cudaFree(p);
    sb::prefill_destroy(L->prefill);
    if (L->pin_x) cudaFreeHost(L->pin_x);
    if (L->pin_y) cudaFreeHost(L->pin_y);
    if (L->pin_err) cudaFreeHost(L->pin_err);
    delete L;
}

int strix_moe_layer_reset_errors(strix_moe_layer *L, void *stream) {
    SB_CHECK(L != nullptr, "moe_layer_reset_errors: null layer");
    SB_CUDA(cudaMemsetAsync(L->err, 0, 32, static_cast<cudaStream_t>(stream)), "clearing the error words");
    if (L->sync != nullptr) SB_CUDA(cudaMemsetAsync(L->sync, 0, 16, static_cast<cudaStream_t>(stream)), "clearing the barrier words");
    return 0;
}

int strix_moe_layer_forward(strix_moe_layer *L, const void *x, int64_t M, void *y, void *stream) {
    const char *fn = "moe_layer_forward";
    SB_CHECK(L != nullptr && x != nullptr && y != nullptr, fn, ": null pointer");
    const auto &d = L->d;
    SB_CHECK(M >= 1 && M <= d.max_tokens, fn, ": ", M, " tokens, expected 1..", d.max_tokens);
    auto st = static_cast<cudaStream_t>(stream);
    const int act = d.act;
    const int64_t E = d.E, A = L->A, R = L->router_rows;
    uint32_t *router_err = L->err, *expert_err = L->err + 3;
    L->last_M = M;

    if (L->fused_ok && M <= 8 && !(L->prefill != nullptr && M >= L->tensor_min)) {
        // Decode / verify: the whole sublayer in one persistent kernel.
        sb::StreamParams p = L->plan;
        sb::decode_stream_set_tokens(p, (int)M);
        p.x = x, p.y = y;
        p.router_kind = d.router_kind, p.router_bits = d.router_bits, p.router_w = d.router_w, p.router_q = d.router_q, p.router_bias = d.router_bias;
        if (d.experts_mixed) {
            p.gate_up = sb::StackView{d.gate_up_mix.q, d.gate_up_mix.scale, d.gate_up_mix.minv, d.gate_up_mix.bits, d.gate_up_mix.q_off, 0, d.gate_up_mix.N, d.gate_up_mix.K, d.gate_up_mix.G};
            p.down = sb::StackView{d.down_mix.q, d.down_mix.scale, d.down_mix.minv, d.down_mix.bits, d.down_mix.q_off, 0, d.down_mix.N, d.down_mix.K, d.down_mix.G};
        } else {
            p.gate_up = sb::StackView{d.gate_up.q, d.gate_up.scale, d.gate_up.minv, nullptr, nullptr, d.gate_up_bits, 2 * d.I, d.d, d.gate_up.G};
            p.down = sb::StackView{d.down.q, d.down.scale, d.down.minv, nullptr, nullptr, d.down_bits, d.d, d.I, d.down.G};
        }
        p.sh_gate_up_bits = d.sh_gate_up_bits, p.sh_down_bits = d.sh_down_bits, p.sh_gate_up = d.sh_gate_up, p.sh_down = d.sh_down;
        p.logits = L->logits, p.ids = L->ids, p.coef = L->coef, p.hh = L->hh, p.sh_h = L->sh_h, p.hrec = L->hrec, p.err = L->err, p.sync = L->sync;
        // the plan was made for min(max_tokens, 8) tokens; fewer tokens only leave more room
        STRIX_RANGE(r_decode, "strix moe decode (one kernel)");
        SB_TRY(sb::decode_stream_launch(fn, p, st));
        return 0;
    }
    STRIX_RANGE(r_layer, "strix moe layer forward");
    // 1. Router logits, FP32 [M, R]; row E (when gated) is the shared expert's gate.
    const bool tensor_path = L->prefill != nullptr && M >= L->tensor_min;
    const bool dense_router = tensor_path && sb::prefill_has_dense_router(L->prefill);
    if (dense_router) SB_TRY(sb::prefill_router_logits(L->prefill, x, M, L->logits, d.router_bias, E, st));  // bias added in its epilogue
    else if (d.router_kind == STRIX_ROUTER_Q) SB_TRY(linear_any(d.router_bits, x, &d.router_q, L->logits, M, act, STRIX_ACT_F32, stream));
    else if (d.router_kind == STRIX_ROUTER_BF16)
        SB_TRY(strix_linear_bf16w(x, static_cast<const uint16_t *>(d.router_w), L->logits, M, R, d.d, act, STRIX_ACT_F32, stream));
    else SB_TRY(strix_linear_f32w(x, static_cast<const float *>(d.router_w), L->logits, M, R, d.d, act, STRIX_ACT_F32, stream));
    if (d.router_bias != nullptr && !dense_router) {
        add_bias_kernel<<<(unsigned)((M * E + 255) / 256), 256, 0, st>>>(L->logits, R, M, E, d.router_bias);
        SB_LAUNCH_OK(fn, ": router bias");
    }
    // 2. Top-k + weights. The stacked shared expert takes slot k: gated through the router (the reference), or with
    //    coefficient 1 written behind the router's k slots.
    const bool stacked = d.shared_mode == STRIX_SHARED_STACKED;
    if (stacked && !L->gated) {
        SB_TRY(strix_moe_router(L->logits, R, M, E, d.k, nullptr, 0, 0, L->ids_k, L->coef_k, STRIX_ACT_F32, router_err, stream));
        widen_rows_kernel<<<(unsigned)((M + 255) / 256), 256, 0, st>>>(L->ids_k, L->coef_k, L->ids, L->coef, M, d.k);
        fill_shared_slot_kernel<<<(unsigned)((M + 255) / 256), 256, 0, st>>>(L->ids, L->coef, M, A, (int32_t)E);
        SB_LAUNCH_OK(fn, ": shared slot");
    } else {
        SB_TRY(strix_moe_router(L->logits, R, M, E, d.k, stacked ? L->logits + E : nullptr, R, (int32_t)E, L->ids, L->coef, STRIX_ACT_F32,
                                router_err, stream));
    }
    // 3. Routed experts: grouped from grouped_min_tokens on, per slot below.
    if (tensor_path) {
        STRIX_RANGE(r_experts, "strix moe experts (tensor cores)");
        // many tokens on the tensor cores: bucket-ordered F16 activations, gate/up with SwiGLU in its epilogue, down into
        // FP32 partials, then the ordered reduction of the reference's combine
        SB_TRY(sb::group_routes_multi(fn, L->ids, M * A, L->Estack, static_cast<int32_t *>(L->group_ws), L->route_scratch, expert_err, false, st));
        // the per-slot sums between the down projection and the combine are F16 here: one more rounding of 2^-11 on values the
        // contract allows 2e-3 on, for half the bytes written and read back (the buffer is the FP32-sized one of the grouped path)
        SB_TRY(sb::prefill_experts(L->prefill, x, nullptr, act, static_cast<const int32_t *>(L->group_ws), M, A, L->partial, true, st));
        SB_TRY(sb::combine_reduce(fn, L->partial, L->ids, L->coef, M, A, L->Estack, d.d, y, act, st, nullptr, true));
    } else if (M >= d.grouped_min_tokens) {
        SB_TRY(strix_moe_group_routes(L->ids, M, A, L->Estack, L->group_ws, L->group_ws_bytes, expert_err, stream));
        if (d.experts_mixed) {
            SB_TRY(strix_linear_qmix_experts_gather_grouped(x, &d.gate_up_mix, L->group_ws, L->group_ws_bytes, M, A, L->gu, act, d.math, stream));
            SB_TRY(strix_swiglu(L->gu, L->hh, M * A, d.I, act, stream));
            SB_TRY(strix_linear_qmix_experts_combine_grouped(L->hh, &d.down_mix, L->ids, L->coef, L->group_ws, L->group_ws_bytes, L->partial, M,
                                                             A, y, act, d.math, stream));
        } else {
            auto gather = d.gate_up_bits == 4 ? strix_linear_q4_experts_gather_grouped : strix_linear_q5_experts_gather_grouped;
            auto combine = d.down_bits == 4 ? strix_linear_q4_experts_combine_grouped : strix_linear_q5_experts_combine_grouped;
            SB_TRY(gather(x, &d.gate_up, L->Estack, L->group_ws, L->group_ws_bytes, M, A, L->gu, act, d.math, stream));
            SB_TRY(strix_swiglu(L->gu, L->hh, M * A, d.I, act, stream));
            SB_TRY(combine(L->hh, &d.down, L->Estack, L->ids, L->coef, L->group_ws, L->group_ws_bytes, L->partial, M, A, y, act, d.math, stream));
        }
    } else if (d.experts_mixed) {
        SB_TRY(strix_linear_qmix_experts_gather_swiglu(x, &d.gate_up_mix, L->ids, M, A, L->hh, act, expert_err, stream));
        SB_TRY(strix_linear_qmix_experts_combine(L->hh, &d.down_mix, L->ids, L->coef, M, A, y, act, expert_err, stream));
    } else {
        auto gather = d.gate_up_bits == 4 ? strix_linear_q4_experts_gather_swiglu : strix_linear_q5_experts_gather_swiglu;
        auto combine = d.down_bits == 4 ? strix_linear_q4_experts_combine : strix_linear_q5_experts_combine;
        SB_TRY(gather(x, &d.gate_up, L->Estack, L->ids, M, A, L->hh, act, expert_err, stream));
        SB_TRY(combine(L->hh, &d.down, L->Estack, L->ids, L->coef, M, A, y, act, expert_err, stream));
    }
    // 4. The shared expert as dense projections, then y += sigmoid(gate) * s (or y += s when always on).
    if (d.shared_mode == STRIX_SHARED_SEPARATE) {
        STRIX_RANGE(r_shared, "strix moe shared expert");
        // many tokens with a tensor-core math mode: the dense tensor-core projections (strixite runtime/qweight.hpp:63-72)
        const bool sh_tc = d.math != STRIX_MATH_F32 && M >= L->tensor_min && d.d % 64 == 0 && d.I % 64 == 0;
        auto lin = sh_tc ? linear_wmma_any : linear_any;
        SB_TRY(lin(d.sh_gate_up_bits, x, &d.sh_gate_up, L->gu, M, act, act, stream));
        SB_TRY(strix_swiglu(L->gu, L->sh_h, M, d.I, act, stream));
        SB_TRY(lin(d.sh_down_bits, L->sh_h, &d.sh_down, L->sh_y, M, act, act, stream));
        if (L->gated) SB_TRY(strix_moe_shared_add(y, L->sh_y, L->logits + E, R, M, d.d, (uint32_t)E, act, router_err, stream));
        else SB_TRY(strix_residual_add(y, L->sh_y, M * d.d, act, stream));
    }
    return 0;
}

int strix_moe_layer_experts_partial(strix_moe_layer *L, const void *rows, const int32_t *row_index, const int32_t *ids, int64_t n, void *partial,
                                    int partial_f16, void *stream) {
    const char *fn = "moe_layer_experts_partial";
    SB_CHECK(L != nullptr && rows != nullptr && ids != nullptr && partial != nullptr, fn, ": null pointer");
    SB_CHECK(L->prefill != nullptr, fn, ": the layer has no tensor-core plan (needs math != F32, uniform 4-bit stacks, d % 256 == 0, I % 128 == 0 and max_tokens >= tensor_min_tokens)");
    SB_CHECK(n >= 1 && n <= L->d.max_tokens * L->A, fn, ": ", n, " rows, expected 1..", L->d.max_tokens * L->A);
    auto st = static_cast<cudaStream_t>(stream);
    // ids of -2 are absent slots (the padding of a fixed-capacity slot list): no error, never computed
    SB_TRY(sb::group_routes_multi(fn, ids, n, L->Estack, static_cast<int32_t *>(L->group_ws), L->route_scratch, L->err + 3, true, st));
    SB_TRY(sb::prefill_experts(L->prefill, rows, row_index, L->d.act, static_cast<const int32_t *>(L->group_ws), n, 1, partial, partial_f16 != 0, st));
    return 0;
}

int strix_moe_combine_reduce(const float *partial, const int64_t *pos, const int32_t *ids, const float *coef, int64_t M, int64_t A, int64_t E,
                             int64_t N, void *y, int act, void *stream) {
    const char *fn = "moe_combine_reduce";
    SB_CHECK(partial != nullptr && ids != nullptr && coef != nullptr && y != nullptr, fn, ": null pointer");
    SB_CHECK(M >= 1 && A >= 1 && A <= 64 && N >= 1 && E >= 1 && M * A <= (1 << 20), fn, ": M = ", M, ", A = ", A, ", N = ", N, ", E = ", E);
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    return sb::combine_reduce(fn, partial, ids, coef, M, A, E, N, y, act, static_cast<cudaStream_t>(stream), pos);
}

int strix_moe_layer_forward_host(strix_moe_layer *L, const void *x_host, int64_t M, void *y_host, void *stream) {
    const char *fn = "moe_layer_forward_host";
    SB_CHECK(L != nullptr && x_host != nullptr && y_host != nullptr, fn, ": null pointer");
    SB_CHECK(M >= 1 && M <= L->d.max_tokens, fn, ": ", M, " tokens, expected 1..", L->d.max_tokens);
    auto st = static_cast<cudaStream_t>(stream);
    const size_t bytes = (size_t)(M * L->d.d * act_size(L->d.act));
    // Page-locked caller buffers are copied from and to directly; pageable ones go through the layer's own page-locked staging
    // (a host memcpy each way: ~10 GB/s on one core, which at thousands of tokens costs more than the layer itself).
    auto page_locked = [](const void *p) {
        cudaPointerAttributes a;
        if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        return a.type == cudaMemoryTypeHost;
    };
    const bool x_direct = page_locked(x_host), y_direct = page_locked(y_host);
    if (!x_direct) std::memcpy(L->pin_x, x_host, bytes);
    SB_CUDA(cudaMemcpyAsync(L->dev_x, x_direct ? x_host : L->pin_x, bytes, cudaMemcpyHostToDevice, st), fn, ": x to the device");
    SB_TRY(strix_moe_layer_forward(L, L->dev_x, M, L->dev_y, stream));
    SB_CUDA(cudaMemcpyAsync(y_direct ? y_host : L->pin_y, L->dev_y, bytes, cudaMemcpyDeviceToHost, st), fn, ": y to the host");
    SB_CUDA(cudaMemcpyAsync(L->pin_err, L->err, 24, cudaMemcpyDeviceToHost, st), fn, ": error words to the host");
    SB_CUDA(cudaStreamSynchronize(st), fn, ": waiting for the layer");
    if (!y_direct) std::memcpy(y_host, L->pin_y, bytes);
    SB_TRY(strix_report_router_error(L->pin_err, "moe layer router"));
    SB_TRY(strix_report_expert_error(L->pin_err + 3, "moe layer experts"));
    return 0;
}

int strix_moe_stack_forward(strix_moe_layer *const *layers, int64_t n_layers, void *x, int64_t M, void *tmp, void *stream) {
    SB_CHECK(layers != nullptr && x != nullptr && tmp != nullptr && n_layers >= 1, "moe_stack_forward: null pointer or no layers");
    for (int64_t l = 0; l < n_layers; ++l) {
        SB_CHECK(layers[l] != nullptr && layers[l]->d.d == layers[0]->d.d && layers[l]->d.act == layers[0]->d.act,
                 "moe_stack_forward: layer ", l, " is null or differs in hidden size / dtype");
        SB_TRY(strix_moe_layer_forward(layers[l], x, M, tmp, stream));
        SB_TRY(strix_residual_add(x, tmp, M * layers[l]->d.d, layers[l]->d.act, stream));
    }
    return 0;
}

const void *strix_moe_layer_probe(strix_moe_layer *L, const char *name) {
    if (L == nullptr || name == nullptr) return nullptr;
    if (!std::strcmp(name, "router_logits")) return L->logits;
    if (!std::strcmp(name, "router_ids")) return L->ids;
    if (!std::strcmp(name, "router_coef")) return L->coef;
    if (!std::strcmp(name, "experts_h")) return L->hh;
    if (!std::strcmp(name, "shared_h")) return L->sh_h;
    if (!std::strcmp(name, "shared_y")) return L->sh_y;
    if (!std::strcmp(name, "err")) return L->err;
    if (!std::strcmp(name, "group_ws")) return L->group_ws;
    if (!std::strcmp(name, "decode_sync")) return L->sync;  // null when forwards of <= 8 tokens run the per-function kernels
    return nullptr;
}

}  // extern "C"
