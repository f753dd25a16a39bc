// Expert parallelism: the device side of the token exchange. The routed experts of a layer are spread over P ranks; a rank
// routes its own tokens, sends every token ONCE to each rank that owns one of its experts, the expert rank runs the experts
// and adds coef * partial over the token's slots it served, and the home rank adds the returned rows in rank order.
// strixite runs one device (runtime/qwen4exp.cpp:1126-1186), so none of this has a counterpart there.
//
// The exchange uses FIXED capacities so that no size ever goes through the host: per (source, destination) pair C rows and Cs
// slots. A pair's message is one block of rows [C, d] and one block of MW = 4 + 2 C + 3 Cs int32 of metadata:
//   [0..3]              n_rows, n_slots, 0, 0
//   [4 + 2 i ..]        row i: first slot, number of slots          (slots of a row are consecutive, in slot order)
//   [4 + 2 C + 3 j ..]  slot j: local expert id on the destination, row (inside the pair's block), coefficient bits
// Everything is in token order per destination, so the layout is a pure function of the routing.
#include "common.cuh"

#include <cuda_fp16.h>

#include "strixite_b200.h"

namespace {

using namespace sb;

constexpr int kMaxRanks = 8;
constexpr int kPlanThreads = 256;  // tokens per block of the plan kernels: a thread per token

// The destination of slot id: its owner; the stacked shared expert (id == E) and invalid ids stay on the home rank (an
// invalid id keeps local id -1 there, which poisons the token like on one device).
__device__ __forceinline__ void slot_dest(int32_t id, int E, const int32_t *owner, const int32_t *local_of, int rank, int &r, int &loc) {
    if (id >= 0 && id <= E) r = id == E ? rank : owner[id], loc = local_of[id];
    else r = rank, loc = -1;
}

// A token's slots per destination: cnt[r] (0 = the token sends no row there).
__device__ __forceinline__ void token_counts(const int32_t *ids, int t, int A, int E, const int32_t *owner, const int32_t *local_of, int rank, int (&cnt)[kMaxRanks]) {
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) cnt[q] = 0;
    for (int a = 0; a < A; ++a) {
        int r, loc;
        slot_dest(ids[(int64_t)t * A + a], E, owner, local_of, rank, r, loc);
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q) cnt[q] += q == r;
    }
}

// The plan in three launches, deterministic and in token order per destination:
//   count  block b = tokens [256 b, 256 b + 256): seg[b][r] = {rows, slots} the segment sends to destination r
//   scan   one block, a warp per destination: seg[b][r] becomes the segment's first row / first slot; message headers, overflow flags
//   place  block b again: a block-wide exclusive scan over its tokens gives each token its row and first slot; it writes them
__global__ void __launch_bounds__(kPlanThreads)
    ep_plan_count_kernel(const int32_t *ids, int T, int A, int E, const int32_t *owner, const int32_t *local_of, int P, int rank, int32_t *seg) {
    __shared__ int wrows[kPlanThreads / 32][kMaxRanks], wslots[kPlanThreads / 32][kMaxRanks];
    const int t = blockIdx.x * kPlanThreads + threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int cnt[kMaxRanks];
    if (t < T) token_counts(ids, t, A, E, owner, local_of, rank, cnt);
    else
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q) cnt[q] = 0;
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
        const int rows = __popc(__ballot_sync(0xffffffffu, cnt[q] > 0)), slots = __reduce_add_sync(0xffffffffu, cnt[q]);
        if (lane == 0) wrows[warp][q] = rows, wslots[warp][q] = slots;
    }
    __syncthreads();
    if (threadIdx.x < kMaxRanks) {
        int rows = 0, slots = 0;
        for (int w = 0; w < kPlanThreads / 32; ++w) rows += wrows[w][threadIdx.x], slots += wslots[w][threadIdx.x];
        seg[((int64_t)blockIdx.x * kMaxRanks + threadIdx.x) * 2] = rows;
        seg[((int64_t)blockIdx.x * kMaxRanks + threadIdx.x) * 2 + 1] = slots;
    }
}

__global__ void __launch_bounds__(32 * kMaxRanks) ep_plan_scan_kernel(int32_t *seg, int nseg, int P, int C, int Cs, int32_t *meta, uint32_t *flags) {
    const int r = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (r >= P) return;
    int row_base = 0, slot_base = 0;
    for (int b0 = 0; b0 < nseg; b0 += 32) {
        const int b = b0 + lane;
        int32_t *e = seg + ((int64_t)b * kMaxRanks + r) * 2;
        const int rows = b < nseg ? e[0] : 0, slots = b < nseg ? e[1] : 0;
        int ri = rows, si = slots;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, ri, off), o2 = __shfl_up_sync(0xffffffffu, si, off);
            if (lane >= off) ri += o, si += o2;
        }
        if (b < nseg) e[0] = row_base + ri - rows, e[1] = slot_base + si - slots;
        row_base += __shfl_sync(0xffffffffu, ri, 31), slot_base += __shfl_sync(0xffffffffu, si, 31);
    }
    if (lane == 0) {
        if (row_base > C) atomicMax(&flags[0], (uint32_t)row_base);
        if (slot_base > Cs) atomicMax(&flags[1], (uint32_t)slot_base);
        int32_t *m = meta + (int64_t)r * (4 + 2 * C + 3 * Cs);
        m[0] = min(row_base, C), m[1] = min(slot_base, Cs), m[2] = 0, m[3] = 0;
    }
}

__global__ void __launch_bounds__(kPlanThreads)
    ep_plan_place_kernel(const int32_t *ids, const float *coef, int T, int A, int E, const int32_t *owner, const int32_t *local_of, int P, int rank, int C, int Cs,
                         const int32_t *seg, int32_t *rowtok, int32_t *meta, int32_t *pos) {
    __shared__ int wrows[kPlanThreads / 32][kMaxRanks], wslots[kPlanThreads / 32][kMaxRanks];
    const int t = blockIdx.x * kPlanThreads + threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, MW = 4 + 2 * C + 3 * Cs;
    int cnt[kMaxRanks], row[kMaxRanks], slot[kMaxRanks];
    if (t < T) token_counts(ids, t, A, E, owner, local_of, rank, cnt);
    else
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q) cnt[q] = 0;
    // exclusive prefix inside the warp, then the warps before this one
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
        const unsigned has = __ballot_sync(0xffffffffu, cnt[q] > 0);
        int si = cnt[q];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, si, off);
            if (lane >= off) si += o;
        }
        row[q] = __popc(has & ((1u << lane) - 1u)), slot[q] = si - cnt[q];
        if (lane == 31) wrows[warp][q] = __popc(has), wslots[warp][q] = si;
    }
    __syncthreads();
    if (t >= T) return;
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q) {
        if (q >= P) continue;
        int rb = seg[((int64_t)blockIdx.x * kMaxRanks + q) * 2], sb_ = seg[((int64_t)blockIdx.x * kMaxRanks + q) * 2 + 1];
        for (int w = 0; w < warp; ++w) rb += wrows[w][q], sb_ += wslots[w][q];
        row[q] += rb, slot[q] += sb_;
        const bool sends = cnt[q] > 0 && row[q] < C;
        pos[(int64_t)t * P + q] = sends ? row[q] : -1;
        if (sends) {
            int32_t *m = meta + (int64_t)q * MW;
            rowtok[(int64_t)q * C + row[q]] = t;
            m[4 + 2 * row[q]] = slot[q];
            m[4 + 2 * row[q] + 1] = max(0, min(cnt[q], Cs - slot[q]));  // slots past the capacity are dropped (the overflow flag is up)
        }
    }
    // the slots, in slot order per destination
    for (int a = 0; a < A; ++a) {
        int r, loc;
        slot_dest(ids[(int64_t)t * A + a], E, owner, local_of, rank, r, loc);
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q) {
            if (q != r) continue;
            const int j = slot[q]++;
            if (j < Cs && row[q] < C) {
                int32_t *sm = meta + (int64_t)q * MW + 4 + 2 * C + 3 * j;
                sm[0] = loc, sm[1] = row[q], sm[2] = __float_as_int(coef[(int64_t)t * A + a]);
            }
        }
    }
}

// Row i of the block for destination r <- x[rowtok[r][i]]; one block per row, 16 bytes per thread and step.
__global__ void __launch_bounds__(256) ep_gather_rows_kernel(const uint4 *x, int row16, const int32_t *rowtok, const int32_t *meta, int C, int MW, uint4 *rows_send) {
    const int r = blockIdx.y, i = blockIdx.x;
    if (i >= meta[(int64_t)r * MW]) return;
    const uint4 *src = x + (int64_t)rowtok[(int64_t)r * C + i] * row16;
    uint4 *dst = rows_send + ((int64_t)r * C + i) * row16;
    for (int j = threadIdx.x; j < row16; j += 256) dst[j] = src[j];
}

// The received slot lists as one list of P * Cs entries for the experts: local expert id (-2 = absent: beyond the pair's count)
// and the slot's activation row among all received rows.
__global__ void __launch_bounds__(256) ep_unpack_kernel(const int32_t *meta, int P, int C, int Cs, int32_t *slot_ids, int32_t *slot_row) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= (int64_t)P * Cs) return;
    const int s = (int)(i / Cs), j = (int)(i - (int64_t)s * Cs);
    const int32_t *m = meta + (int64_t)s * (4 + 2 * C + 3 * Cs);
    if (j < m[1]) {
        const int32_t *sm = m + 4 + 2 * C + 3 * j;
        slot_ids[i] = sm[0], slot_row[i] = s * C + sm[1];
    } else {
        slot_ids[i] = -2, slot_row[i] = 0;
    }
}

// Expert side: summed[s][i][:] = sum over the row's slots, in slot order, of coef * partial[slot][:] (FP32, fmaf as the
// reference's combine, strixite kernels/moe_grouped.hip:456-472). One block per received row.
template <bool H>  // H: the partial sums are F16 (strix_moe_layer_experts_partial with partial_f16), else FP32
__global__ void __launch_bounds__(256) ep_row_sum_kernel(const void *partial, const int32_t *meta, int C, int Cs, int d4, float4 *summed) {
    const int s = blockIdx.y, i = blockIdx.x;
    const int32_t *m = meta + (int64_t)s * (4 + 2 * C + 3 * Cs);
    if (i >= m[0]) return;
    const int first = m[4 + 2 * i], n = m[4 + 2 * i + 1];
    const int32_t *sm = m + 4 + 2 * C + 3 * first;
    for (int j = threadIdx.x; j < d4; j += 256) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < n; ++q) {
            const float c = __int_as_float(sm[3 * q + 2]);
            const int64_t e = ((int64_t)s * Cs + first + q) * d4 + j;
            float4 p;
            if constexpr (H) {
                const uint2 u = static_cast<const uint2 *>(partial)[e];
                const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&u.x)), hi = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
                p = make_float4(lo.x, lo.y, hi.x, hi.y);
            } else {
                p = static_cast<const float4 *>(partial)[e];
            }
            v.x = fmaf(c, p.x, v.x), v.y = fmaf(c, p.y, v.y), v.z = fmaf(c, p.z, v.z), v.w = fmaf(c, p.w, v.w);
        }
        summed[((int64_t)s * C + i) * d4 + j] = v;
    }
}

// ---- the exchange inside the kernels: peer stores over NVLink instead of a library all-to-all --------------------------------------
// Every rank holds its receive buffers in memory its peers have mapped (symmetric allocation); `*_ptrs[r]` is rank r's buffer as
// seen from this GPU. A source writes its block [rank] of the destination's buffer directly, so the transfer is the kernel's own
// store stream and needs no staging copy; the ranks meet at a barrier (a host-enqueued collective) before anyone reads.

// Token rows and the metadata block to every destination. grid = (C + kMetaBlocks, P): blocks i < C copy row i of destination
// blockIdx.y (when the plan counted it), the others stream the used part of the metadata block.
constexpr int kMetaBlocks = 8;
__global__ void __launch_bounds__(256)
    ep_push_rows_kernel(const uint4 *x, int row16, const int32_t *rowtok, const int32_t *meta, int rank, int C, int Cs, const uint64_t *rows_ptrs,
                        const uint64_t *meta_ptrs) {
    const int r = blockIdx.y, i = blockIdx.x, MW = 4 + 2 * C + 3 * Cs;
    const int32_t *m = meta + (int64_t)r * MW;
    if (i < C) {
        if (i >= m[0]) return;
        const uint4 *src = x + (int64_t)rowtok[(int64_t)r * C + i] * row16;
        uint4 *dst = reinterpret_cast<uint4 *>(rows_ptrs[r]) + ((int64_t)rank * C + i) * row16;
        for (int j = threadIdx.x; j < row16; j += 256) dst[j] = src[j];
        return;
    }
    // metadata: the header and the row table up to n_rows, the slot table up to n_slots (the rest of the block is never read)
    int32_t *dm = reinterpret_cast<int32_t *>(meta_ptrs[r]) + (int64_t)rank * MW;
    const int n_head = 4 + 2 * m[0], n_slot_ints = 3 * m[1];
    const int t = (i - C) * 256 + threadIdx.x, stride = kMetaBlocks * 256;
    for (int j = t; j < n_head; j += stride) dm[j] = m[j];
    for (int j = t; j < n_slot_ints; j += stride) dm[4 + 2 * C + j] = m[4 + 2 * C + j];
}

// Expert side: the row sums of ep_row_sum, each written straight into the home rank's `back` buffer (block [rank] of it), FP32 or
// F16 (OH: one rounding of the FP32 sum; halves the bytes that cross the links). One block per received row.
template <bool H, bool OH>
__global__ void __launch_bounds__(256)
    ep_row_sum_push_kernel(const void *partial, const int32_t *meta, int rank, int C, int Cs, int d4, const uint64_t *back_ptrs) {
    const int s = blockIdx.y, i = blockIdx.x;
    const int32_t *m = meta + (int64_t)s * (4 + 2 * C + 3 * Cs);
    if (i >= m[0]) return;
    const int first = m[4 + 2 * i], n = m[4 + 2 * i + 1];
    const int32_t *sm = m + 4 + 2 * C + 3 * first;
    const int64_t out_row = ((int64_t)rank * C + i) * d4;
    for (int j = threadIdx.x; j < d4; j += 256) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < n; ++q) {
            const float c = __int_as_float(sm[3 * q + 2]);
            const int64_t e = ((int64_t)s * Cs + first + q) * d4 + j;
            float4 p;
            if constexpr (H) {
                const uint2 u = static_cast<const uint2 *>(partial)[e];
                const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&u.x)), hi = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
                p = make_float4(lo.x, lo.y, hi.x, hi.y);
            } else {
                p = static_cast<const float4 *>(partial)[e];
            }
            v.x = fmaf(c, p.x, v.x), v.y = fmaf(c, p.y, v.y), v.z = fmaf(c, p.z, v.z), v.w = fmaf(c, p.w, v.w);
        }
        if constexpr (OH) {
            const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
            uint2 u;
            u.x = *reinterpret_cast<const uint32_t *>(&lo), u.y = *reinterpret_cast<const uint32_t *>(&hi);
            reinterpret_cast<uint2 *>(back_ptrs[s])[out_row + j] = u;
        } else {
            reinterpret_cast<float4 *>(back_ptrs[s])[out_row + j] = v;
        }
    }
}

// Home side: y[t][:] = the rows that came back for token t, added in ascending rank order, rounded once to the activation
// dtype. A token the router failed (ids -1) or with an invalid id gets a NaN row, as on one device.
template <typename T, bool BH>  // BH: the returned rows are F16 (ep_row_sum_push with F16 output)
__global__ void __launch_bounds__(256) ep_home_sum_kernel(const void *back, const int32_t *pos, const int32_t *ids, int A, int E, int P, int C, int d4, T *y) {
    const int t = blockIdx.x;
    bool bad = false;
    for (int a = 0; a < A; ++a) {
        const int32_t id = ids[(int64_t)t * A + a];
        bad |= id < 0 || id > E;
    }
    for (int j = threadIdx.x; j < d4; j += 256) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < P; ++r) {
            const int p = pos[(int64_t)t * P + r];
            if (p < 0) continue;
            const int64_t e = ((int64_t)r * C + p) * d4 + j;
            float4 b;
            if constexpr (BH) {
                const uint2 u = static_cast<const uint2 *>(back)[e];
                const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&u.x)), hi = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
                b = make_float4(lo.x, lo.y, hi.x, hi.y);
            } else {
                b = static_cast<const float4 *>(back)[e];
            }
            v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
        }
        if (bad) v = make_float4(qnan(), qnan(), qnan(), qnan());
        const int64_t o = ((int64_t)t * d4 + j) * 4;
        st_act(y, o, v.x), st_act(y, o + 1, v.y), st_act(y, o + 2, v.z), st_act(y, o + 3, v.w);
    }
}

}  // namespace

extern "C" {

int64_t strix_ep_meta_ints(int64_t C, int64_t Cs) { return 4 + 2 * C + 3 * Cs; }

int64_t strix_ep_plan_scratch_ints(int64_t T) { return (T + kPlanThreads - 1) / kPlanThreads * kMaxRanks * 2; }

int strix_ep_plan(const int32_t *ids, const float *coef, int64_t T, int64_t A, int64_t E, const int32_t *owner, const int32_t *local_of, int P, int rank,
                  int64_t C, int64_t Cs, int32_t *rowtok, int32_t *meta, int32_t *pos, uint32_t *flags, int32_t *scratch, void *stream) {
    const char *fn = "ep_plan";
    SB_CHECK(ids && coef && owner && local_of && rowtok && meta && pos && flags && scratch, fn, ": null pointer");
    SB_CHECK(P >= 1 && P <= kMaxRanks && rank >= 0 && rank < P, fn, ": ", P, " ranks (1..", kMaxRanks, "), rank ", rank);
    SB_CHECK(T >= 1 && A >= 1 && A <= 64 && E >= 1 && T * A <= (1 << 22) && C >= 1 && Cs >= 1 && C <= (1 << 22) && Cs <= (1 << 24), fn, ": T = ", T, ", A = ", A,
             ", E = ", E, ", C = ", C, ", Cs = ", Cs);
    auto st = static_cast<cudaStream_t>(stream);
    const int nseg = (int)((T + kPlanThreads - 1) / kPlanThreads);
    ep_plan_count_kernel<<<nseg, kPlanThreads, 0, st>>>(ids, (int)T, (int)A, (int)E, owner, local_of, P, rank, scratch);
    ep_plan_scan_kernel<<<1, 32 * kMaxRanks, 0, st>>>(scratch, nseg, P, (int)C, (int)Cs, meta, flags);
    ep_plan_place_kernel<<<nseg, kPlanThreads, 0, st>>>(ids, coef, (int)T, (int)A, (int)E, owner, local_of, P, rank, (int)C, (int)Cs, scratch, rowtok, meta, pos);
    SB_LAUNCH_OK(fn);
    return 0;
}

int strix_ep_gather_rows(const void *x, int64_t d, int act, const int32_t *rowtok, const int32_t *meta, int P, int64_t C, int64_t Cs, void *rows_send, void *stream) {
    const char *fn = "ep_gather_rows";
    SB_CHECK(x && rowtok && meta && rows_send, fn, ": null pointer");
    SB_CHECK(act_ok(act) && d >= 8 && (d * act_size(act)) % 16 == 0 && aligned16(x) && aligned16(rows_send), fn, ": rows of ", d, " ", act_name(act),
             " values must be whole 16-byte pieces, 16-byte aligned");
    SB_CHECK(P >= 1 && P <= kMaxRanks && C >= 1 && C <= 0x7fffffff, fn, ": P = ", P, ", C = ", C);
    ep_gather_rows_kernel<<<dim3((unsigned)C, (unsigned)P), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(x), (int)(d * act_size(act) / 16), rowtok, meta, (int)C, (int)strix_ep_meta_ints(C, Cs), static_cast<uint4 *>(rows_send));
    SB_LAUNCH_OK(fn);
    return 0;
}

int strix_ep_unpack(const int32_t *meta_recv, int P, int64_t C, int64_t Cs, int32_t *slot_ids, int32_t *slot_row, void *stream) {
    const char *fn = "ep_unpack";
    SB_CHECK(meta_recv && slot_ids && slot_row, fn, ": null pointer");
    SB_CHECK(P >= 1 && P <= kMaxRanks && C >= 1 && Cs >= 1 && (int64_t)P * Cs <= (1 << 26), fn, ": P = ", P, ", C = ", C, ", Cs = ", Cs);
    const int64_t n = (int64_t)P * Cs;
    ep_unpack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(meta_recv, P, (int)C, (int)Cs, slot_ids, slot_row);
    SB_LAUNCH_OK(fn);
    return 0;
}

int strix_ep_row_sum(const void *partial, int partial_f16, const int32_t *meta_recv, int P, int64_t C, int64_t Cs, int64_t d, float *summed, void *stream) {
    const char *fn = "ep_row_sum";
    SB_CHECK(partial && meta_recv && summed, fn, ": null pointer");
    SB_CHECK(P >= 1 && P <= kMaxRanks && C >= 1 && Cs >= 1 && d >= 4 && d % 4 == 0 && aligned16(partial) && aligned16(summed), fn, ": P = ", P, ", C = ", C, ", d = ", d);
    const dim3 grid((unsigned)C, (unsigned)P);
    auto st = static_cast<cudaStream_t>(stream);
    if (partial_f16) ep_row_sum_kernel<true><<<grid, 256, 0, st>>>(partial, meta_recv, (int)C, (int)Cs, (int)(d / 4), reinterpret_cast<float4 *>(summed));
    else ep_row_sum_kernel<false><<<grid, 256, 0, st>>>(partial, meta_recv, (int)C, (int)Cs, (int)(d / 4), reinterpret_cast<float4 *>(summed));
    SB_LAUNCH_OK(fn);
    return 0;
}

int strix_ep_home_sum(const void *back, int back_f16, const int32_t *pos, const int32_t *ids, int64_t T, int64_t A, int64_t E, int P, int64_t C, int64_t d, void *y,
                      int act, void *stream) {
    const char *fn = "ep_home_sum";
    SB_CHECK(back && pos && ids && y, fn, ": null pointer");
    SB_CHECK(P >= 1 && P <= kMaxRanks && T >= 1 && T <= 0x7fffffff && d >= 4 && d % 4 == 0 && act_ok(act) && aligned16(back), fn, ": P = ", P, ", T = ", T, ", d = ", d);
    auto st = static_cast<cudaStream_t>(stream);
    const int Ai = (int)A, Ei = (int)E, Ci = (int)C, d4 = (int)(d / 4);
    if (act == kF32) {
        if (back_f16) ep_home_sum_kernel<float, true><<<(unsigned)T, 256, 0, st>>>(back, pos, ids, Ai, Ei, P, Ci, d4, static_cast<float *>(y));
        else ep_home_sum_kernel<float, false><<<(unsigned)T, 256, 0, st>>>(back, pos, ids, Ai, Ei, P, Ci, d4, static_cast<float *>(y));
    } else {
        if (back_f16) ep_home_sum_kernel<uint16_t, true><<<(unsigned)T, 256, 0, st>>>(back, pos, ids, Ai, Ei, P, Ci, d4, static_cast<uint16_t *>(y));
        else ep_home_sum_kernel<uint16_t, false><<<(unsigned)T, 256, 0, st>>>(back, pos, ids, Ai, Ei, P, Ci, d4, static_cast<uint16_t *>(y));
    }
    SB_LAUNCH_OK(fn);
    return 0;
}

int strix_ep_push_rows(const void *x, int64_t d, int act, const int32_t *rowtok, const int32_t *meta, int P, int rank, int64_t C, int64_t Cs, const uint64_t *rows_ptrs,
                       const uint64_t *meta_ptrs, void *stream) {
    const char *fn = "ep_push_rows";
    SB_CHECK(x && rowtok && meta && rows_ptrs && meta_ptrs, fn, ": null pointer");
    SB_CHECK(act_ok(act) && d >= 8 && (d * act_size(act)) % 16 == 0 && aligned16(x), fn, ": rows of ", d, " ", act_name(act), " values must be whole 16-byte pieces, 16-byte aligned");
    SB_CHECK(P >= 1 && P <= kMaxRanks && rank >= 0 && rank < P && C >= 1 && C <= 0x7ffffff0 && Cs >= 1, fn, ": P = ", P, ", rank = ", rank, ", C = ", C, ", Cs = ", Cs);
    ep_push_rows_kernel<<<dim3((unsigned)C + kMetaBlocks, (unsigned)P), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(x), (int)(d * act_size(act) / 16), rowtok, meta, rank, (int)C, (int)Cs, rows_ptrs, meta_ptrs);
    SB_LAUNCH_OK(fn);
    return 0;
}

int strix_ep_row_sum_push(const void *partial, int partial_f16, const int32_t *meta_recv, int P, int rank, int64_t C, int64_t Cs, int64_t d, const uint64_t *back_ptrs,
                          int back_f16, void *stream) {
    const char *fn = "ep_row_sum_push";
    SB_CHECK(partial && meta_recv && back_ptrs, fn, ": null pointer");
    SB_CHECK(P >= 1 && P <= kMaxRanks && rank >= 0 && rank < P && C >= 1 && Cs >= 1 && d >= 4 && d % 4 == 0 && aligned16(partial), fn, ": P = ", P, ", C = ", C, ", d = ", d);
    const dim3 grid((unsigned)C, (unsigned)P);
    auto st = static_cast<cudaStream_t>(stream);
    const int Ci = (int)C, Csi = (int)Cs, d4 = (int)(d / 4);
    if (partial_f16) {
        if (back_f16) ep_row_sum_push_kernel<true, true><<<grid, 256, 0, st>>>(partial, meta_recv, rank, Ci, Csi, d4, back_ptrs);
        else ep_row_sum_push_kernel<true, false><<<grid, 256, 0, st>>>(partial, meta_recv, rank, Ci, Csi, d4, back_ptrs);
    } else {
        if (back_f16) ep_row_sum_push_kernel<false, true><<<grid, 256, 0, st>>>(partial, meta_recv, rank, Ci, Csi, d4, back_ptrs);
        else ep_row_sum_push_kernel<false, false><<<grid, 256, 0, st>>>(partial, meta_recv, rank, Ci, Csi, d4, back_ptrs);
    }
    SB_LAUNCH_OK(fn);
    return 0;
}

}  // extern "C"
