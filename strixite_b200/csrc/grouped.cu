// Experts grouped by expert, for many-token forwards: the deterministic route grouping (a stable counting sort of
// the M * A slots by expert id) and the FP32 CUDA-core grouped projections over its tiles (MoeMath F32). The
// tensor-core grouped GEMM lives in its own file and reads the same workspace.
//
// Workspace (int32; the layout of strixite kernels/moe_grouped.hip:63-81):
//   [0..3]  n_tiles, S, E, n_wtiles
//   offsets[E + 2]   bucket b's slots are slots[offsets[b] .. offsets[b + 1]); bucket E collects invalid ids
//   slots[S]         slot numbers (m * A + a) ordered by bucket, ascending inside a bucket
//   tile_bucket[Tmax], tile_start[Tmax]      tiles of up to 16 slots of one bucket;  Tmax  = S / 16 + E + 2
//   wtile_bucket[WTmax], wtile_start[WTmax]  tiles of up to 64 slots of one bucket;  WTmax = S / 64 + E + 2
#include <mutex>
#include "common.cuh"

#include <cuda_fp16.h>

#include "grouped.cuh"
#include "prefill_umma.cuh"
#include "strixite_b200.h"

namespace {

using namespace sb;

constexpr int kRouteThreads = 1024, kRouteWarps = 32;

// Exclusive scan of one int per thread over the 1024-thread block: warp shuffles, then the 32 warp totals.
__device__ int block_exclusive_scan(int v, int *warp_tot, int *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += o;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int t = warp_tot[lane], ti = t;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, ti, off);
            if (lane >= off) ti += o;
        }
        warp_tot[lane] = ti - t;
        if (lane == 31) *total = ti;
    }
    __syncthreads();
    const int res = warp_tot[warp] + incl - v;
    __syncthreads();  // warp_tot / total are reused by the next scan
    return res;
}

// The bucket whose tile range [prefix[b], prefix[b + 1]) holds tile i (prefix ascending, B + 1 entries).
__device__ int bucket_of_tile(const int *prefix, int B, int i) {
    int lo = 0, hi = B;  // invariant: prefix[lo] <= i < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= i) lo = mid;
        else hi = mid;
    }
    return lo;
}

// One block. Warp w owns the contiguous slot segment [w * seg, (w + 1) * seg): it counts its slots per bucket in its own
// row of `cnt`, the per-bucket prefix over the warps turns the counts into the warp's first position in each bucket,
// and the warp then places its slots in slot order (ranks inside a 32-slot step by __match_any_sync). So a bucket
// lists its slots ascending, whatever the scheduling: the permutation is a pure function of ids.
__global__ void __launch_bounds__(kRouteThreads)
    route_kernel(const int32_t *ids, int S, int E, int Tmax, int WTmax, int32_t *ws, uint32_t *err) {
    extern __shared__ int smem[];
    const int B = E + 1;
    int *cnt = smem;                      // [kRouteWarps][B]
    int *start = cnt + kRouteWarps * B;   // [B + 1] first slot position of each bucket
    int *tile0 = start + B + 1;           // [B + 1] first 16-slot tile of each bucket
    int *wtile0 = tile0 + B + 1;          // [B + 1] first 64-slot tile
    int *warp_tot = wtile0 + B + 1;       // [32]
    __shared__ int first_bad, total_a, total_b, total_c;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    for (int i = t; i < kRouteWarps * B; i += kRouteThreads) cnt[i] = 0;
    if (t == 0) first_bad = 0x7fffffff;
    __syncthreads();
    const int seg = ((S + kRouteWarps - 1) / kRouteWarps + 31) & ~31;
    const int s_begin = min(S, warp * seg), s_end = min(S, s_begin + seg);
    for (int s = s_begin + lane; s < s_end; s += 32) {
        const int32_t id = ids[s];
        const bool bad = id < 0 || id >= E;
        atomicAdd(&cnt[warp * B + (bad ? E : id)], 1);
        if (bad) atomicMin(&first_bad, s);
    }
    __syncthreads();
    if (t == 0 && first_bad != 0x7fffffff) raise_err(err, (uint32_t)ids[first_bad], (uint32_t)first_bad);
    int count = 0;
    if (t < B) {
        for (int w = 0; w < kRouteWarps; ++w) {
            const int c = cnt[w * B + t];
            cnt[w * B + t] = count;  // this warp's first rank inside the bucket
            count += c;
        }
    }
    const int st = block_exclusive_scan(count, warp_tot, &total_a);
    const int tl = block_exclusive_scan((count + 15) / 16, warp_tot, &total_b);
    const int wt = block_exclusive_scan((count + 63) / 64, warp_tot, &total_c);
    int32_t *offsets = ws + 4, *slots = offsets + E + 2, *tile_bucket = slots + S, *tile_start = tile_bucket + Tmax;
    int32_t *wtile_bucket = tile_start + Tmax, *wtile_start = wtile_bucket + WTmax;
    if (t < B) start[t] = st, tile0[t] = tl, wtile0[t] = wt, offsets[t] = st;
    if (t == 0) {
        start[B] = total_a, tile0[B] = total_b, wtile0[B] = total_c;
        ws[0] = total_b, ws[1] = S, ws[2] = E, ws[3] = total_c;
        offsets[E + 1] = total_a;
    }
    __syncthreads();
    for (int i = t; i < total_b; i += kRouteThreads) {
        const int b = bucket_of_tile(tile0, B, i);
        tile_bucket[i] = b, tile_start[i] = start[b] + (i - tile0[b]) * 16;
    }
    for (int i = t; i < total_c; i += kRouteThreads) {
        const int b = bucket_of_tile(wtile0, B, i);
        wtile_bucket[i] = b, wtile_start[i] = start[b] + (i - wtile0[b]) * 64;
    }
    for (int s0 = s_begin; s0 < s_end; s0 += 32) {
        const int s = s0 + lane;
        const bool live = s < s_end;
        int b = 0x40000000 | lane;  // idle lanes: a bucket of their own
        if (live) {
            const int32_t id = ids[s];
            b = (id < 0 || id >= E) ? E : id;
        }
        const unsigned same = __match_any_sync(0xffffffffu, b);
        const int rank = __popc(same & ((1u << lane) - 1u));
        if (live) {
            slots[start[b] + cnt[warp * B + b] + rank] = s;
        }
        __syncwarp();
        if (live && rank == 0) cnt[warp * B + b] += __popc(same);
        __syncwarp();
    }
}

// ---- the same grouping over many blocks (the layer object's path; it owns the scratch) -------------------------------
// The slots are cut into kSegs contiguous segments, a warp each. Pass 1 counts every segment's slots per bucket into
// scratch[seg][bucket]; pass 2 (one block) turns each bucket's column into the segments' first ranks, scans the bucket
// totals and writes the header, the offsets and the tile tables; pass 3 places every segment's slots in slot order. The
// result is the single-block kernel's, bit for bit. quiet: an id of -2 marks an absent slot (padding of a fixed-capacity
// slot list): it lands in the invalid bucket like any bad id but raises no error.
constexpr int kSegBlocks = 16, kSegWarps = 8, kSegs = kSegBlocks * kSegWarps;
constexpr int kNoBad = 0x7f7f7f7f;  // "no invalid id seen": what a byte-wise memset can write

__device__ __forceinline__ int seg_len(int S) { return ((S + kSegs - 1) / kSegs + 31) & ~31; }

__global__ void __launch_bounds__(kSegWarps * 32) route_count_kernel(const int32_t *ids, int S, int E, int32_t *scratch, int quiet) {
    extern __shared__ int smem[];
    const int B = E + 1, t = threadIdx.x, lane = t & 31, warp = t >> 5, g = blockIdx.x * kSegWarps + warp;
    int *cnt = smem + warp * B;
    for (int i = lane; i < B; i += 32) cnt[i] = 0;
    __syncwarp();
    const int seg = seg_len(S), s_begin = min(S, g * seg), s_end = min(S, s_begin + seg);
    int first_bad = 0x7fffffff;
    for (int s = s_begin + lane; s < s_end; s += 32) {
        const int32_t id = ids[s];
        const bool bad = id < 0 || id >= E;
        atomicAdd(&cnt[bad ? E : id], 1);
        if (bad && !(quiet && id == -2) && s < first_bad) first_bad = s;
    }
    __syncwarp();
    for (int i = lane; i < B; i += 32) scratch[g * B + i] = cnt[i];
    first_bad = __reduce_min_sync(0xffffffffu, first_bad);
    if (lane == 0 && first_bad != 0x7fffffff) atomicMin(&scratch[kSegs * B], first_bad);
}

__global__ void __launch_bounds__(kRouteThreads)
    route_scan_kernel(const int32_t *ids, int S, int E, int Tmax, int WTmax, int32_t *ws, int32_t *scratch, uint32_t *err) {
    extern __shared__ int smem[];
    const int B = E + 1;
    int *start = smem;               // [B + 1]
    int *tile0 = start + B + 1;      // [B + 1]
    int *wtile0 = tile0 + B + 1;     // [B + 1]
    int *warp_tot = wtile0 + B + 1;  // [32]
    __shared__ int total_a, total_b, total_c;
    const int t = threadIdx.x;
    if (t == 0) {
        const int first_bad = scratch[kSegs * B];
        if (first_bad != kNoBad) raise_err(err, (uint32_t)ids[first_bad], (uint32_t)first_bad);
        scratch[kSegs * B] = kNoBad;  // ready for the next grouping
    }
    int count = 0;
    if (t < B) {
        // sixteen counts in flight per round trip (a load after a store to the same array would otherwise wait for it)
        static_assert(kSegs % 16 == 0, "the bucket's column is read in batches of 16");
        for (int g0 = 0; g0 < kSegs; g0 += 16) {
            int c[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) c[j] = scratch[(g0 + j) * B + t];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                scratch[(g0 + j) * B + t] = count;  // this segment's first rank inside the bucket
                count += c[j];
            }
        }
    }
    const int st = block_exclusive_scan(count, warp_tot, &total_a);
    const int tl = block_exclusive_scan((count + 15) / 16, warp_tot, &total_b);
    const int wt = block_exclusive_scan((count + 63) / 64, warp_tot, &total_c);
    int32_t *offsets = ws + 4, *slots = offsets + E + 2, *tile_bucket = slots + S, *tile_start = tile_bucket + Tmax;
    int32_t *wtile_bucket = tile_start + Tmax, *wtile_start = wtile_bucket + WTmax;
    if (t < B) start[t] = st, tile0[t] = tl, wtile0[t] = wt, offsets[t] = st;
    if (t == 0) {
        start[B] = total_a, tile0[B] = total_b, wtile0[B] = total_c;
        ws[0] = total_b, ws[1] = S, ws[2] = E, ws[3] = total_c;
        offsets[E + 1] = total_a;
    }
    __syncthreads();
    for (int i = t; i < total_b; i += kRouteThreads) {
        const int b = bucket_of_tile(tile0, B, i);
        tile_bucket[i] = b, tile_start[i] = start[b] + (i - tile0[b]) * 16;
    }
    for (int i = t; i < total_c; i += kRouteThreads) {
        const int b = bucket_of_tile(wtile0, B, i);
        wtile_bucket[i] = b, wtile_start[i] = start[b] + (i - wtile0[b]) * 64;
    }
}

__global__ void __launch_bounds__(kSegWarps * 32) route_place_kernel(const int32_t *ids, int S, int E, int32_t *ws, const int32_t *scratch) {
    extern __shared__ int smem[];
    const int B = E + 1, t = threadIdx.x, lane = t & 31, warp = t >> 5, g = blockIdx.x * kSegWarps + warp;
    int *pos = smem + warp * B;  // next position of each bucket for this segment
    const int32_t *offsets = ws + 4;
    int32_t *slots = ws + 4 + E + 2;
    for (int i = lane; i < B; i += 32) pos[i] = offsets[i] + scratch[g * B + i];
    __syncwarp();
    const int seg = seg_len(S), s_begin = min(S, g * seg), s_end = min(S, s_begin + seg);
    int32_t next_id = s_begin + lane < s_end ? ids[s_begin + lane] : 0;  // the next step's id is loaded under this step's work
    for (int s0 = s_begin; s0 < s_end; s0 += 32) {
        const int s = s0 + lane;
        const bool live = s < s_end;
        const int32_t id = next_id;
        if (s + 32 < s_end) next_id = ids[s + 32];
        int b = 0x40000000 | lane;  // idle lanes: a bucket of their own
        if (live) b = (id < 0 || id >= E) ? E : id;
        const unsigned same = __match_any_sync(0xffffffffu, b);
        const int rank = __popc(same & ((1u << lane) - 1u));
        if (live) slots[pos[b] + rank] = s;
        __syncwarp();
        if (live && rank == 0) pos[b] += __popc(same);
        __syncwarp();
    }
}

__device__ unsigned int g_ws_refusals = 0;  // launches refused over a workspace grouped for other sizes (strix_workspace_refusal_count)

// FP32 path: one tile (up to 16 slots of one expert) x 8 output rows per block, a warp per row. The row's codes are
// decoded once per 32-code chunk and applied to every slot of the tile. COMBINE: inputs h[slot], outputs the per-slot
// dots into `partial` (FP32); else inputs x[slot / A], outputs y[slot] in the activation dtype.
template <typename T, bool COMBINE>
__global__ void __launch_bounds__(256)
    grouped_f32_kernel(const T *x, StackView w, const int32_t *ws, int64_t A, T *y, float *partial, int32_t S, int32_t E) {
    constexpr int R = 16;
    if (!sb::ws_is_for(ws, S, E, &g_ws_refusals)) return;
    const int32_t n_tiles = ws[0];
    const int tile = blockIdx.y;
    if (tile >= n_tiles) return;
    const sb::RouteTables rt = sb::route_tables(ws, S, E);
    const int32_t bucket = rt.tile_bucket[tile], st = rt.tile_start[tile];
    const int rows = min(R, rt.offsets[bucket + 1] - st);
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= w.N) return;
    const int32_t *tile_slots = rt.slots + st;
    if (bucket == E) {  // invalid ids: NaN outputs (the grouping raised err)
        if (lane < rows) {
            const int64_t slot = tile_slots[lane];
            if (COMBINE) partial[slot * w.N + n] = qnan();
            else st_act(y, slot * w.N + n, qnan());
        }
        return;
    }
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    const int64_t gpr = w.K / w.G, wr = (int64_t)bucket * w.N + n;
    const uint16_t *srow = w.scale + wr * gpr, *mrow = w.minv + wr * gpr;
    by_bits(w.bits_of(bucket), [&](auto bc) {
        constexpr int BITS = decltype(bc)::value;
        const uint8_t *row = w.rows(bucket, BITS) + n * row_bytes(BITS, w.K);
        for (int64_t c = lane; c < w.K / 32; c += 32) {
            float code[32];
            load_codes32<BITS>(row, w.K, c, code);
            const float s = bf16_bits_to_f32(srow[c * 32 / w.G]), mn = bf16_bits_to_f32(mrow[c * 32 / w.G]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (r < rows) {
                    const int64_t slot = tile_slots[r];
                    float xv[32];
                    load_x32(x, (COMBINE ? slot : slot / A) * w.K + c * 32, xv);
                    float dot = 0.f, xs = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) dot = fmaf(xv[i], code[i], dot), xs += xv[i];
                    acc[r] = fmaf(s, dot, fmaf(mn, xs, acc[r]));
                }
            }
        }
    });
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (r < rows) {  // warp-uniform: a tile of one or two slots pays for one or two reductions, not sixteen
            const float v = warp_sum(acc[r]);
            if (lane == 0) {
                const int64_t slot = tile_slots[r];
                if (COMBINE) partial[slot * w.N + n] = v;
                else st_act(y, slot * w.N + n, v);
            }
        }
    }
}

// y[m, n] = sum_a fma(coef[m, a], partial[m * A + a, n], v), a ascending, one rounding; a token with any invalid id
// gets a NaN row whatever its partials hold.
template <typename T>
__global__ void __launch_bounds__(256)
    combine_reduce_kernel(const float *partial, const int32_t *ids, const float *coef, int64_t M, int64_t A, int64_t E,
                          int64_t N, T *y) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * N) return;
    const int64_t m = i / N, n = i - m * N;
    bool ok = true;
    float v = 0.f;
    for (int64_t a = 0; a < A; ++a) {
        const int32_t id = ids[m * A + a];
        ok = ok && id >= 0 && id < E;
        v = fmaf(coef[m * A + a], partial[(m * A + a) * N + n], v);
    }
    st_act(y, i, ok ? v : qnan());
}

// The same on four consecutive outputs per thread: 16-byte loads of the partial rows, four of them in flight per step.
// Four consecutive partial sums from element `elem` on: FP32, or F16 (the layer's own tensor-core path stores its per-slot
// sums as F16 - half the traffic of the combine; the public grouped entries keep the caller's FP32 buffer).
template <bool H>
__device__ __forceinline__ float4 ld_partial4(const void *partial, int64_t elem) {
    if constexpr (H) {
        const uint2 u = __ldcs(reinterpret_cast<const uint2 *>(static_cast<const __half *>(partial) + elem));
        const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&u.x)), hi = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    } else {
        return __ldcs(reinterpret_cast<const float4 *>(static_cast<const float *>(partial) + elem));
    }
}

template <typename T, bool H>
__global__ void __launch_bounds__(256)
    combine_reduce4_kernel(const void *partial, const int64_t *pos, const int32_t *ids, const float *coef, int64_t M, int64_t A, int64_t E,
                           int64_t N, T *y) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, N4 = N / 4;
    if (i >= M * N4) return;
    const int64_t m = i / N4, n = (i - m * N4) * 4;
    bool ok = true;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (pos != nullptr) {  // slot (m, a) lives in row pos[m * A + a] of partial
        for (int64_t a = 0; a < A; ++a) {
            const float4 p = ld_partial4<H>(partial, pos[m * A + a] * N + n);
            const float c = coef[m * A + a];
            const int32_t id = ids[m * A + a];
            ok = ok && id >= 0 && id < E;
            v.x = fmaf(c, p.x, v.x), v.y = fmaf(c, p.y, v.y), v.z = fmaf(c, p.z, v.z), v.w = fmaf(c, p.w, v.w);
        }
        const float q = qnan();
        st_act(y, m * N + n, ok ? v.x : q), st_act(y, m * N + n + 1, ok ? v.y : q), st_act(y, m * N + n + 2, ok ? v.z : q), st_act(y, m * N + n + 3, ok ? v.w : q);
        return;
    }
    const int64_t row = m * A * N + n;
    int64_t a = 0;
    for (; a + 4 <= A; a += 4) {
        float4 p[4];
        float c[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            p[j] = ld_partial4<H>(partial, row + (a + j) * N);
            c[j] = coef[m * A + a + j];
            const int32_t id = ids[m * A + a + j];
            ok = ok && id >= 0 && id < E;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) v.x = fmaf(c[j], p[j].x, v.x), v.y = fmaf(c[j], p[j].y, v.y), v.z = fmaf(c[j], p[j].z, v.z), v.w = fmaf(c[j], p[j].w, v.w);
    }
    for (; a < A; ++a) {
        const float4 p = ld_partial4<H>(partial, row + a * N);
        const float c = coef[m * A + a];
        const int32_t id = ids[m * A + a];
        ok = ok && id >= 0 && id < E;
        v.x = fmaf(c, p.x, v.x), v.y = fmaf(c, p.y, v.y), v.z = fmaf(c, p.z, v.z), v.w = fmaf(c, p.w, v.w);
    }
    const float q = qnan();
    st_act(y, m * N + n, ok ? v.x : q), st_act(y, m * N + n + 1, ok ? v.y : q), st_act(y, m * N + n + 2, ok ? v.z : q), st_act(y, m * N + n + 3, ok ? v.w : q);
}

}  // namespace

namespace sb {

int route_ints(int64_t M, int64_t A, int64_t E, int64_t *out) {
    SB_CHECK(M >= 1 && A >= 1 && A <= 64 && E >= 1 && E <= 1023 && M * A <= (1 << 20), "moe route workspace: M = ", M, ", A = ", A,
             ", E = ", E, " (A 1..64, E 1..1023, M*A <= 2^20)");
    const int64_t S = M * A;
    *out = 4 + (E + 2) + S + 2 * (S / 16 + E + 2) + 2 * (S / 64 + E + 2);
    return 0;
}

int check_grouped_common(const char *fn, const void *x, const StackView &w, int64_t E, int64_t M, int64_t A, const void *ws,
                         size_t ws_bytes, const void *y, int act) {
    SB_CHECK(x != nullptr && y != nullptr && ws != nullptr, fn, ": null pointer (x=", x, ", y=", y, ", ws=", ws, ")");
    SB_CHECK(w.q != nullptr && w.scale != nullptr && w.minv != nullptr, fn, ": null weight pointer (q=", (const void *)w.q, ", scale=",
             (const void *)w.scale, ", min=", (const void *)w.minv, ")");
    SB_CHECK(group_ok(w.G), fn, ": group size ", w.G, " unsupported (32, 64 or 128)");
    SB_CHECK(w.K >= w.G && w.K % w.G == 0 && w.K <= (1 << 24), fn, ": K = ", w.K, " must be a positive multiple of group size ", w.G,
             " and <= 2^24");
    SB_CHECK(w.N >= 1 && w.N <= 0x7fffffff, fn, ": N = ", w.N, " rows per expert");
    if (w.bits_tab == nullptr) {
        SB_CHECK(bits_ok(w.bits), fn, ": ", w.bits, " bits, expected 4, 5, 6 or 8");
        SB_CHECK(w.bits != 5 || w.K % 128 == 0, fn, ": Q5 K = ", w.K, " is not a multiple of 128 (the layout's)");
        SB_CHECK(w.bits != 6 || w.K % 64 == 0, fn, ": Q6 K = ", w.K, " is not a multiple of 64 (the layout's)");
    } else {
        SB_CHECK(w.q_off != nullptr, fn, ": per-expert formats need the q_off table");
        SB_CHECK(w.K % 128 == 0, fn, ": mixed-format experts need K % 128 == 0 (Q5 rows), got ", w.K);
    }
    int64_t ints = 0;
    SB_TRY(route_ints(M, A, E, &ints));
    SB_CHECK(A <= E, fn, ": A = ", A, " slots per token exceed E = ", E, " experts");
    SB_CHECK(ws_bytes >= (size_t)ints * 4, fn, ": workspace of ", ws_bytes, " bytes, needs ", ints * 4, " for M = ", M, ", A = ", A,
             ", E = ", E);
    SB_CHECK(aligned16(w.q) && aligned16(x), fn, ": code array ", (const void *)w.q, " and input ", x, " must be 16-byte aligned");
    SB_CHECK(act_ok(act), fn, ": unsupported activation dtype ", act);
    return 0;
}

int gather_grouped(const char *fn, const void *x, const StackView &w, int64_t E, const void *ws, size_t ws_bytes, int64_t M,
                   int64_t A, void *y, int act, int math, void *stream) {
    SB_TRY(check_grouped_common(fn, x, w, E, M, A, ws, ws_bytes, y, act));
    const int64_t es = act_size(act);
    SB_CHECK(apart(y, M * A * w.N * es, x, M * w.K * es), fn, ": y [", y, ", +", M * A * w.N * es, " B) overlaps x [", x, ", +",
             M * w.K * es, " B)");
    SB_CHECK(math == STRIX_MATH_F32 || math == STRIX_MATH_WMMA_BF16 || math == STRIX_MATH_WMMA_F16, fn, ": unknown math ", math);
    auto st = static_cast<cudaStream_t>(stream);
    const auto *wsi = static_cast<const int32_t *>(ws);
    if (math != STRIX_MATH_F32) {
        SB_TRY(grouped_umma(fn, x, w, wsi, M, A, E, y, nullptr, act, /*combine=*/false, st));
        return 0;
    }
    // tiles that can exist: S / 16 full ones + one ragged tile per non-empty bucket (at most S buckets, E + 1 with the invalid one)
    const int64_t Tmax = M * A / 16 + (E + 1 < M * A ? E + 1 : M * A) + 1;
    SB_CHECK(Tmax <= 65535, fn, ": ", Tmax, " tile slots exceed the grid");
    const dim3 grid((unsigned)((w.N + 7) / 8), (unsigned)Tmax), block(256);
    if (act == kF32) grouped_f32_kernel<float, false><<<grid, block, 0, st>>>((const float *)x, w, wsi, A, (float *)y, nullptr, (int32_t)(M * A), (int32_t)E);
    else grouped_f32_kernel<uint16_t, false><<<grid, block, 0, st>>>((const uint16_t *)x, w, wsi, A, (uint16_t *)y, nullptr, (int32_t)(M * A), (int32_t)E);
    SB_LAUNCH_OK(fn, " ", act_name(act), " M=", M, " A=", A, " E=", E, " N=", w.N, " K=", w.K, " G=", w.G);
    return 0;
}

int combine_grouped(const char *fn, const void *h, const StackView &w, int64_t E, const int32_t *ids, const float *coef,
                    const void *ws, size_t ws_bytes, float *partial, int64_t M, int64_t A, void *y, int act, int math,
                    void *stream) {
    SB_TRY(check_grouped_common(fn, h, w, E, M, A, ws, ws_bytes, y, act));
    SB_CHECK(ids != nullptr && coef != nullptr && partial != nullptr, fn, ": null pointer (ids=", (const void *)ids, ", coef=",
             (const void *)coef, ", partial=", (const void *)partial, ")");
    const int64_t es = act_size(act);
    SB_CHECK(apart(y, M * w.N * es, h, M * A * w.K * es), fn, ": y overlaps h");
    SB_CHECK(apart(y, M * w.N * es, partial, M * A * w.N * 4), fn, ": y overlaps partial");
    SB_CHECK(apart(partial, M * A * w.N * 4, h, M * A * w.K * es), fn, ": partial overlaps h");
    SB_CHECK(math == STRIX_MATH_F32 || math == STRIX_MATH_WMMA_BF16 || math == STRIX_MATH_WMMA_F16, fn, ": unknown math ", math);
    auto st = static_cast<cudaStream_t>(stream);
    const auto *wsi = static_cast<const int32_t *>(ws);
    if (math != STRIX_MATH_F32) {
        SB_TRY(grouped_umma(fn, h, w, wsi, M, A, E, nullptr, partial, act, /*combine=*/true, st));
    } else {
        const int64_t Tmax = M * A / 16 + (E + 1 < M * A ? E + 1 : M * A) + 1;  // as in gather_grouped
        SB_CHECK(Tmax <= 65535, fn, ": ", Tmax, " tile slots exceed the grid");
        const dim3 grid((unsigned)((w.N + 7) / 8), (unsigned)Tmax), block(256);
        if (act == kF32) grouped_f32_kernel<float, true><<<grid, block, 0, st>>>((const float *)h, w, wsi, A, nullptr, partial, (int32_t)(M * A), (int32_t)E);
        else grouped_f32_kernel<uint16_t, true><<<grid, block, 0, st>>>((const uint16_t *)h, w, wsi, A, nullptr, partial, (int32_t)(M * A), (int32_t)E);
        SB_LAUNCH_OK(fn, " ", act_name(act), " M=", M, " A=", A, " E=", E, " N=", w.N, " K=", w.K, " G=", w.G);
    }
    const unsigned blocks = (unsigned)((M * w.N + 255) / 256);
    if (act == kF32) combine_reduce_kernel<float><<<blocks, 256, 0, st>>>(partial, ids, coef, M, A, E, w.N, (float *)y);
    else combine_reduce_kernel<uint16_t><<<blocks, 256, 0, st>>>(partial, ids, coef, M, A, E, w.N, (uint16_t *)y);
    SB_LAUNCH_OK(fn, " reduce ", act_name(act), " M=", M, " A=", A, " N=", w.N);
    return 0;
}

int combine_reduce(const char *fn, const void *partial, const int32_t *ids, const float *coef, int64_t M, int64_t A, int64_t E, int64_t N,
                   void *y, int act, cudaStream_t st, const int64_t *pos, bool half_partial) {
    const bool vec = N % 4 == 0 && reinterpret_cast<uintptr_t>(partial) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
    SB_CHECK((pos == nullptr && !half_partial) || vec, fn, ": the indexed combine and F16 partial sums need N % 4 == 0 and 16-byte aligned buffers");
    if (vec) {
        const unsigned blocks = (unsigned)((M * (N / 4) + 255) / 256);
        if (half_partial) {
            if (act == kF32) combine_reduce4_kernel<float, true><<<blocks, 256, 0, st>>>(partial, pos, ids, coef, M, A, E, N, (float *)y);
            else combine_reduce4_kernel<uint16_t, true><<<blocks, 256, 0, st>>>(partial, pos, ids, coef, M, A, E, N, (uint16_t *)y);
        } else {
            if (act == kF32) combine_reduce4_kernel<float, false><<<blocks, 256, 0, st>>>(partial, pos, ids, coef, M, A, E, N, (float *)y);
            else combine_reduce4_kernel<uint16_t, false><<<blocks, 256, 0, st>>>(partial, pos, ids, coef, M, A, E, N, (uint16_t *)y);
        }
    } else {
        const unsigned blocks = (unsigned)((M * N + 255) / 256);
        const float *pf = static_cast<const float *>(partial);
        if (act == kF32) combine_reduce_kernel<float><<<blocks, 256, 0, st>>>(pf, ids, coef, M, A, E, N, (float *)y);
        else combine_reduce_kernel<uint16_t><<<blocks, 256, 0, st>>>(pf, ids, coef, M, A, E, N, (uint16_t *)y);
    }
    SB_LAUNCH_OK(fn, " reduce ", act_name(act), " M=", M, " A=", A, " N=", N);
    return 0;
}

}  // namespace sb

namespace {

int uniform_view(const char *fn, int bits, const strix_qview *w, int64_t E, StackView *out) {
    SB_CHECK(w != nullptr, fn, ": null weight view");
    SB_CHECK(E >= 1 && E <= 1023 && w->N % E == 0, fn, ": weight has ", w->N, " rows for E = ", E,
             " experts (E must be 1..1023 and divide the rows)");
    *out = StackView{w->q, w->scale, w->minv, nullptr, nullptr, bits, w->N / E, w->K, w->G};
    return 0;
}
int mixed_view(const char *fn, const strix_qmix_view *w, StackView *out) {
    SB_CHECK(w != nullptr && w->bits != nullptr && w->q_off != nullptr, fn, ": null view, format table or offset table");
    *out = StackView{w->q, w->scale, w->minv, w->bits, w->q_off, 0, w->N, w->K, w->G};
    return 0;
}

}  // namespace

namespace sb {

size_t route_scratch_bytes(int64_t E) { return (size_t)(kSegs * (E + 1) + 1) * 4; }

int route_scratch_init(void *scratch, int64_t E, cudaStream_t stream) {
    // the counts are rewritten by every grouping; only the first-bad word has to start at "none"
    SB_CUDA(cudaMemsetAsync(static_cast<int32_t *>(scratch) + kSegs * (E + 1), 0x7f, 4, stream), "route scratch");
    return 0;
}

int group_routes_multi(const char *fn, const int32_t *ids, int64_t S, int64_t E, int32_t *ws, int32_t *scratch, uint32_t *err, bool quiet,
                       cudaStream_t stream) {
    const size_t seg_smem = (size_t)kSegWarps * (E + 1) * sizeof(int);
    const size_t scan_smem = (size_t)(3 * (E + 2) + 32) * sizeof(int);
    route_count_kernel<<<kSegBlocks, kSegWarps * 32, seg_smem, stream>>>(ids, (int)S, (int)E, scratch, quiet ? 1 : 0);
    route_scan_kernel<<<1, kRouteThreads, scan_smem, stream>>>(ids, (int)S, (int)E, (int)(S / 16 + E + 2), (int)(S / 64 + E + 2), ws, scratch, err);
    route_place_kernel<<<kSegBlocks, kSegWarps * 32, seg_smem, stream>>>(ids, (int)S, (int)E, ws, scratch);
    SB_LAUNCH_OK(fn, ": grouping S=", S, " E=", E);
    return 0;
}

}  // namespace sb

extern "C" {

unsigned int strix_workspace_refusal_count(void) {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_ws_refusals, sizeof(v));
    return v + sb::grouped_umma_ws_refusals() + sb::prefill_ws_refusals();
}
unsigned int strix_umma_abort_count(void) { return sb::grouped_umma_aborts() + sb::prefill_aborts(); }
void strix_umma_wait_cycles(unsigned long long *out32, int reset) { sb::prefill_cycles(out32, reset != 0); }

size_t strix_moe_route_workspace_bytes(int64_t M, int64_t A, int64_t E) {
    int64_t ints = 0;
    if (sb::route_ints(M, A, E, &ints) != 0) return 0;
    return (size_t)ints * 4;
}

int strix_moe_group_routes(const int32_t *ids, int64_t M, int64_t A, int64_t E, void *ws, size_t ws_bytes,
                           uint32_t *err, void *stream) {
    const char *fn = "moe_group_routes";
    SB_CHECK(ids != nullptr && ws != nullptr && err != nullptr, fn, ": null pointer (ids=", (const void *)ids, ", ws=", ws, ", err=",
             (const void *)err, ")");
    int64_t ints = 0;
    SB_TRY(sb::route_ints(M, A, E, &ints));
    SB_CHECK(ws_bytes >= (size_t)ints * 4, fn, ": workspace of ", ws_bytes, " bytes, needs ", ints * 4);
    const int64_t S = M * A;
    const size_t smem = (size_t)(kRouteWarps * (E + 1) + 3 * (E + 2) + 32) * sizeof(int);
    static thread_local int attr_dev = -1;
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev), fn);
    if (attr_dev != dev) {
        SB_CUDA(cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024), fn,
                ": raising the shared-memory limit");
        attr_dev = dev;
    }
    route_kernel<<<1, kRouteThreads, smem, static_cast<cudaStream_t>(stream)>>>(ids, (int)S, (int)E, (int)(S / 16 + E + 2),
                                                                               (int)(S / 64 + E + 2), static_cast<int32_t *>(ws), err);
    SB_LAUNCH_OK(fn, " M=", M, " A=", A, " E=", E);
    return 0;
}

int strix_linear_q4_experts_gather_grouped(const void *x, const strix_qview *w, int64_t E, const void *ws,
                                           size_t ws_bytes, int64_t M, int64_t A, void *y, int act, int math,
                                           void *stream) {
    StackView sv;
    SB_TRY(uniform_view("linear_q4_experts_gather_grouped", 4, w, E, &sv));
    return sb::gather_grouped("linear_q4_experts_gather_grouped", x, sv, E, ws, ws_bytes, M, A, y, act, math, stream);
}
int strix_linear_q5_experts_gather_grouped(const void *x, const strix_qview *w, int64_t E, const void *ws,
                                           size_t ws_bytes, int64_t M, int64_t A, void *y, int act, int math,
                                           void *stream) {
    StackView sv;
    SB_TRY(uniform_view("linear_q5_experts_gather_grouped", 5, w, E, &sv));
    return sb::gather_grouped("linear_q5_experts_gather_grouped", x, sv, E, ws, ws_bytes, M, A, y, act, math, stream);
}
int strix_linear_q4_experts_combine_grouped(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                            const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                            int64_t M, int64_t A, void *y, int act, int math, void *stream) {
    StackView sv;
    SB_TRY(uniform_view("linear_q4_experts_combine_grouped", 4, w, E, &sv));
    return sb::combine_grouped("linear_q4_experts_combine_grouped", h, sv, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math,
                               stream);
}
int strix_linear_q5_experts_combine_grouped(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                            const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                            int64_t M, int64_t A, void *y, int act, int math, void *stream) {
    StackView sv;
    SB_TRY(uniform_view("linear_q5_experts_combine_grouped", 5, w, E, &sv));
    return sb::combine_grouped("linear_q5_experts_combine_grouped", h, sv, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math,
                               stream);
}
// ---- the combine with its partial sums in the library's own fixed device array -------------------------------------
// The array lives in the library's device image, so it exists on every device the library runs on without any
// allocation. Its name is a host-side handle, not a device address: the address comes from cudaGetSymbolAddress, asked
// once per device with that device current, and cached.
static __device__ __align__(256) float g_fixed_partial[STRIX_FIXED_PARTIAL_FLOATS];

namespace {
int fixed_partial(const char *fn, float **out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static float *addr[kMaxDevices] = {};
    int dev = -1;
    SB_CUDA(cudaGetDevice(&dev), fn);
    SB_CHECK(dev >= 0 && dev < kMaxDevices, fn, ": device ordinal ", dev, " outside 0..", kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        float *p = nullptr;
        SB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_fixed_partial), fn);
        SB_CHECK(p != nullptr, fn, ": the fixed scratch array has no address on device ", dev);
        addr[dev] = p;
    }
    *out = addr[dev];
    return 0;
}
}  // namespace

int strix_linear_q4_experts_combine_grouped_fixed(const void *h, const strix_qview *w, int64_t E, const int32_t *ids,
                                                  const float *coef, const void *ws, size_t ws_bytes, int64_t M, int64_t A,
                                                  void *y, int act, int math, void *stream) {
    const char *fn = "linear_q4_experts_combine_grouped_fixed";
    StackView sv;
    SB_TRY(uniform_view(fn, 4, w, E, &sv));
    SB_CHECK(M >= 1 && A >= 1 && sv.N >= 1 && M * A <= STRIX_FIXED_PARTIAL_FLOATS && M * A * sv.N <= STRIX_FIXED_PARTIAL_FLOATS, fn,
             ": M * A * N = ", M, " * ", A, " * ", sv.N, " partial sums exceed the fixed scratch array of ", (int64_t)STRIX_FIXED_PARTIAL_FLOATS,
             " floats; use linear_q4_experts_combine_grouped with a caller-provided buffer");
    float *partial = nullptr;
    SB_TRY(fixed_partial(fn, &partial));
    return sb::combine_grouped(fn, h, sv, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math, stream);
}

int strix_linear_qmix_experts_gather_grouped(const void *x, const strix_qmix_view *w, const void *ws, size_t ws_bytes,
                                             int64_t M, int64_t A, void *y, int act, int math, void *stream) {
    StackView sv;
    SB_TRY(mixed_view("linear_qmix_experts_gather_grouped", w, &sv));
    return sb::gather_grouped("linear_qmix_experts_gather_grouped", x, sv, w->E, ws, ws_bytes, M, A, y, act, math, stream);
}
int strix_linear_qmix_experts_combine_grouped(const void *h, const strix_qmix_view *w, const int32_t *ids,
                                              const float *coef, const void *ws, size_t ws_bytes, float *partial,
                                              int64_t M, int64_t A, void *y, int act, int math, void *stream) {
    StackView sv;
    SB_TRY(mixed_view("linear_qmix_experts_combine_grouped", w, &sv));
    return sb::combine_grouped("linear_qmix_experts_combine_grouped", h, sv, w->E, ids, coef, ws, ws_bytes, partial, M, A, y, act,
                               math, stream);
}

}  // extern "C"
