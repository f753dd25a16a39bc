// The many-token expert FFN on the 5th-generation tensor cores: persistent, warp-specialised tcgen05 kernels fed by TMA.
//
//   dense_umma_kernel   router logits[M, R] = x[M, d] * Wr[R, d]^T for BF16 activations and a BF16 router (products of
//                       two BF16 values are exact in FP32, so this equals the FP32-FMA projection up to summation
//                       order). Both operands arrive by TMA with the 128-byte swizzle; no thread touches them.
//   tiles_kernel        the per-expert buckets of the grouping workspace cut into tiles of at most 96 routed slots (32 in
//                       the small shape).
//   pregather_kernel    xg[p, :] = F16(x[row of sorted slot p, :]): the activations in bucket order, so that a tile's
//                       tokens are consecutive rows one TMA box can fetch.
//   ffn_umma_kernel<0>  hs[p, i] = SwiGLU(gate, up) with gate/up = W_gate_up[e] * xg[p]: one work item = one tile x 128
//                       intermediate columns = two row halves (128 gate rows and the matching 128 up rows), so that a
//                       thread of the epilogue holds gate and up of the same output.
//   ffn_umma_kernel<1>  partial[slot, n] = W_down[e] * hs[p]: one work item = one tile x 256 output rows.
//
// One CTA per SM walks its work items. Roles (wide shape; the small shape has 4 epilogue and 4 issuing warps):
//   warps 0-15  dequantizers: thread = 64 codes of one weight row per raw stage -> F16 code * s + m (lop3 "1024 + code",
//               exact subtract, one F16 FMA), stored with tcgen05.st into an A stage in TENSOR MEMORY (lane = weight row,
//               32 columns = 64 F16): the MMA takes A from tensor memory and only B from shared memory. Both operands keep
//               each 8 K elements in the order 0,4,1,5,2,6,3,7 (what the nibble unpack produces); xg and hs are written
//               in that order.
//   warps 16-23 epilogue: tcgen05.ld (lane = weight row, column = routed slot) of one accumulator buffer while the next
//               work item accumulates in the other.
//   warp 24     TMA producer: packed 4-bit codes (boxes of 128 rows x 64 bytes, 64-byte swizzle) into a 6-deep ring of raw
//               stages, token tiles (96 rows x 64 F16, 128-byte swizzle) into a 6-deep ring.
//   warps 25-26 one per accumulator: issue tcgen05.mma (cta_group::1, kind::f16, FP32 accumulation) and one tcgen05.commit
//               per K block, under which the probe of the next K block's barrier is issued. Warp 25 allocates all 512
//               tensor-memory columns (two buffers of two 96-column accumulators + two A stages of 64 columns).
// Every mbarrier wait is bounded: on expiry the CTA raises the abort counter, frees its tensor memory and returns.
// What bounds it (measured): a tcgen05.mma occupies its issuing thread ~100 cycles for any N <= 128 and the tensor-memory
// instruction path takes about one tcgen05 operation (mma, commit, st, ld) per ~45 cycles per SM; with ~80 slots per
// expert a K block of 256 rows is 8 MMAs + 2 commits + 8 stores ~ 1000 cycles for ~300 cycles of tensor work.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <mutex>

#include "prefill_umma.cuh"
#include "umma.cuh"

#include <cstdlib>

namespace {

using namespace sb;
using namespace sb::umma;

__device__ unsigned int g_prefill_aborts = 0;
__device__ unsigned int g_ws_refusals = 0;
// Built with -DSTRIX_PROFILE only: cycles the roles of the FFN kernels spent in their waits, summed over CTAs since the last
// reset: [mode * 16 + i], i = 0 kernel total, 1 producer raw_empty, 2 producer consumed, 3 mma acc_empty, 4 mma full, 5 unused,
// 6 dequant raw_full, 7 dequant consumed, 8 dequant total, 9 epilogue acc_full, 10 epilogue total, 11 work items.
// The product build has no clock reads and no counters in its kernels (strix_umma_wait_cycles then reports zeros).
#ifdef STRIX_PROFILE
__device__ unsigned long long g_prefill_cycles[32];
#define TIMED_WAIT(slot, expr)                 \
    do {                                       \
        const long long t0_ = clock64();       \
        ok = (expr);                           \
        waited[slot] += clock64() - t0_;       \
    } while (0)
#define PROFILE_ADD(i, v) atomicAdd(&g_prefill_cycles[MODE * 16 + (i)], (unsigned long long)(v))
#define PROFILE_CLOCK() clock64()
#else
#define TIMED_WAIT(slot, expr) \
    do {                       \
        ok = (expr);           \
    } while (0)
#define PROFILE_ADD(i, v) \
    do {                  \
    } while (0)
#define PROFILE_CLOCK() 0ll
#endif

constexpr int kBK = 64;                 // K per stage: 64 F16 = one 128-byte swizzle row
constexpr int kTile = kTileM * kBK * 2;  // 16 KB: 128 rows x 64 F16 (the dense projection's operand tiles)
constexpr int kRS = 6;                  // raw stages: 2 x (128 rows x 64 bytes) = 128 codes of 256 rows
constexpr int kRawTile = kTileM * 64;
constexpr int kRawStage = 2 * kRawTile;
constexpr int kAStageCols = 64;         // an A stage in tensor memory: 2 row halves x 32 columns (64 F16 per row)
constexpr int kDequantWarps = 16;
constexpr int64_t kSmallSlots = 1024;    // forwards with at most this many routed slots use the small-tile kernels

// Three shapes of the FFN kernel. WIDE (many tokens): tiles of up to 96 slots, two accumulators (the work item's two row
// halves), one MMA-issuing warp each, accumulators double-buffered against the epilogue. SMALL (a handful of tokens: decode,
// verify): tiles of up to 32 slots, and each row half's K block split between two accumulators and two issuing warps (an
// instruction occupies its issuing thread ~100 cycles whatever N is, so with N = 16 the issue rate is all that matters; the
// epilogue adds the two halves in a fixed order), a deeper A ring in the tensor-memory columns the narrow accumulators leave
// free. XWIDE (hundreds of slots per expert): tiles of up to 192 slots - half the instructions, dequantized weight stages and
// barrier rounds per slot; the two 192-column accumulators fill tensor memory, so they are single-buffered (the epilogue of a
// work item runs before the next item's first MMA; the item's main loop is twice as long as WIDE's).
constexpr int kWide = 0, kSmall = 1, kXWide = 2;
template <int SHAPE>
struct FC {
    static constexpr bool SMALL = SHAPE == kSmall, XW = SHAPE == kXWide;
    static constexpr int TileSlots = SMALL ? 32 : XW ? 192 : 96;  // routed slots per tile = MMA N at most
    static constexpr int BTile = TileSlots * kBK * 2;         // the token tile of one K block
    static constexpr int BS = SMALL ? 8 : XW ? 5 : 6;         // token-tile stages (= ready / consumed barriers)
    static constexpr int KSplit = SMALL ? 2 : 1;              // accumulators (and issuing warps) per row half
    static constexpr int NAcc = 2 * KSplit;
    static constexpr int AccBufs = XW ? 1 : 2;                // accumulator sets: 2 = the epilogue overlaps the next item's MMAs
    static constexpr int AccCols = TileSlots, BufCols = NAcc * AccCols, AColBase = AccBufs * BufCols;
    static constexpr int AS = SMALL ? 4 : 2;                  // A stages in tensor memory
    static constexpr int EpiWarps = SMALL ? 4 : 8;
    // XWIDE: nothing else can run while the single accumulator set drains, so the dequantizer warps take their share of it
    static constexpr bool CoopEpi = XW;
    static constexpr int DrainWarps = EpiWarps + (CoopEpi ? kDequantWarps : 0);  // warps that arrive on acc_empty
    static constexpr int ProducerWarp = kDequantWarps + EpiWarps, MmaWarp = ProducerWarp + 1;  // NAcc issuing warps from MmaWarp on
    static constexpr int Threads = (MmaWarp + NAcc) * 32;
    static_assert(AColBase + AS * kAStageCols <= 512, "tensor memory has 512 columns");
    static_assert(AS <= BS, "an A stage is freed through the barrier of the K block that used it");
};

template <int SHAPE>
struct Ctl {
    uint64_t raw_full[kRS], raw_empty[kRS], full[FC<SHAPE>::BS], consumed[FC<SHAPE>::BS], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// ---------------------------------------------------------------------------------------------------------------
// tiles[0] = number of tiles, then (bucket, first sorted position, slots) per tile; buckets in ascending order.
__global__ void __launch_bounds__(1024) tiles_kernel(const int32_t *ws, int32_t *tiles, int tile_slots, int32_t S, int32_t E) {
    __shared__ int32_t scan[1024];
    if (!ws_is_for(ws, S, E, &g_ws_refusals)) {  // no tiles: the projections that follow have no work and store nothing
        if (threadIdx.x == 0) tiles[0] = 0;
        return;
    }
    const RouteTables rt = route_tables(ws, S, E);
    const int e = threadIdx.x;
    const int32_t cnt = e < E ? rt.offsets[e + 1] - rt.offsets[e] : 0;
    const int32_t nt = (cnt + tile_slots - 1) / tile_slots;
    scan[e] = nt;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
        const int32_t v = e >= off ? scan[e - off] : 0;
        __syncthreads();
        scan[e] += v;
        __syncthreads();
    }
    const int32_t first = scan[e] - nt;
    for (int t = 0; t < nt; ++t) {
        int32_t *o = tiles + 1 + 3 * (first + t);
        o[0] = e, o[1] = rt.offsets[e] + t * tile_slots, o[2] = min(tile_slots, cnt - t * tile_slots);
    }
    if (e == 1023) tiles[0] = scan[1023];
}

// One warp per sorted position p < offsets[E] (the slots with a valid expert).
template <typename T>
__global__ void __launch_bounds__(256) pregather_kernel(const T *x, const int32_t *row_index, const int32_t *ws, int64_t A, int64_t K, uint16_t *xg, int32_t S,
                                                        int32_t E) {
    if (ws[1] != S || ws[2] != E) return;  // counted by tiles_kernel
    const RouteTables rt = route_tables(ws, S, E);
    const int32_t total = rt.offsets[E];
    const int lane = threadIdx.x & 31;
    for (int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); p < total; p += (int64_t)gridDim.x * 8) {
        const int32_t slot = rt.slots[p];
        const T *src = x + (int64_t)(row_index != nullptr ? row_index[slot] : slot / A) * K;  // row_index: slot -> activation row
        uint4 *dst = reinterpret_cast<uint4 *>(xg + p * K);
        for (int c = lane; c < K / 8; c += 32) dst[c] = act_chunk(src + c * 8);
    }
}

// ---------------------------------------------------------------------------------------------------------------
struct FfnArgs {
    const int32_t *ws, *tiles;
    const uint16_t *scale, *minv;  // [stack rows, K / G]
    int K, rows_per_expert, I, RB;
    uint16_t *hs;    // MODE 0 output: [S, I] F16, 8-groups in the order 0,4,1,5,2,6,3,7
    void *partial;   // MODE 1 output: [S, N] by slot, FP32 or (partial_f16) F16
    int partial_f16;
    int N;
    int bf16_act;    // MODE 0: round gate, up and the product as a BF16 activation pipeline does
};

__device__ __forceinline__ float bf16_rn(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// SwiGLU of one output; a BF16 activation pipeline rounds gate, up, silu(gate) and the product (strixite kernels/swiglu.hpp:21).
// exp and the divide are the hardware approximations (__expf: 2 ulp + the range reduction's error; __fdividef: 2 ulp; the
// reference uses expf and an IEEE divide, kernels/swiglu.hip:22): the result is rounded to F16 (2^-11) or BF16 (2^-8) right
// after, far coarser than the 4 ulp of FP32, and in the 192-slot tile shape the epilogue is on the critical path (it drains
// the only accumulator set), where the exact forms cost 3x the instructions. |g| > 87 (where __fdividef's range limit on the
// denominator could matter) gives silu = g or -0 in both forms.
__device__ __forceinline__ float swiglu_rounded(float g, float u, bool bf16) {
    if (bf16) {
        g = bf16_rn(g), u = bf16_rn(u);
        return bf16_rn(bf16_rn(__fdividef(g, 1.0f + __expf(-g))) * u);
    }
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}

template <int MODE, int G, int SHAPE>
__global__ void __launch_bounds__(FC<SHAPE>::Threads, 1)
    ffn_umma_kernel(const __grid_constant__ CUtensorMap raw_map, const __grid_constant__ CUtensorMap b_map, const FfnArgs a) {
    using C = FC<SHAPE>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *b_stages = base, *raws = b_stages + C::BS * C::BTile;
    Ctl<SHAPE> &ctl = *reinterpret_cast<Ctl<SHAPE> *>(raws + kRS * kRawStage);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    [[maybe_unused]] const long long t_kernel = PROFILE_CLOCK();
    if (tid == 0) {
        for (int i = 0; i < kRS; ++i) mbar_init(&ctl.raw_full[i], 1), mbar_init(&ctl.raw_empty[i], kDequantWarps);
        // full[kc % BS]: K block kc is ready = its token tile has landed (the producer's arrival + bytes) and the 8 dequantizer
        // warps of its half have stored the A stage; consumed[kc % BS]: every issuing warp has committed its MMAs of K block kc
        for (int i = 0; i < C::BS; ++i) mbar_init(&ctl.full[i], 1 + kDequantWarps / 2), mbar_init(&ctl.consumed[i], C::NAcc);
        for (int i = 0; i < 2; ++i) mbar_init(&ctl.acc_full[i], C::NAcc), mbar_init(&ctl.acc_empty[i], C::DrainWarps);
        ctl.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == C::MmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl.tmem_base;
    const int n_work = a.tiles[0] * a.RB;
    const int nkb = a.K / kBK;
    volatile int *abort_flag = &ctl.abort_flag;

    // stack row of row half `acc`, row 0, of a work item
    auto first_row = [&](int bucket, int rb, int acc) {
        return MODE == 0 ? bucket * a.rows_per_expert + acc * a.I + rb * kTileM : bucket * a.rows_per_expert + rb * 2 * kTileM + acc * kTileM;
    };

    // The epilogue of work item w (the it-th of this CTA) for one warp: its lane quadrant q (= warp % 4, the tensor-memory
    // lanes a warp may read) and every per_q-th 16-column chunk from chunk j on. Returns false when a wait was abandoned.
    const RouteTables rtab = route_tables(a.ws, a.ws[1], a.ws[2]);
    auto drain_item = [&](int w, uint32_t it, int q, int j, int per_q, long long *waited) -> bool {
        const int r = q * 32 + lane;
        const int32_t *t = a.tiles + 1 + 3 * (w / a.RB);
        const int rb = w % a.RB, start = t[1], n_valid = t[2];
        const uint32_t buf = it % C::AccBufs;
        bool ok = true;
        TIMED_WAIT(0, mbar_wait(&ctl.acc_full[buf], (it / C::AccBufs) & 1u, abort_flag));
        if (!ok) return false;
        tc_fence_after();
        const uint32_t tbase = tmem + ((uint32_t)(q * 32) << 16) + buf * C::BufCols;
        for (int c0 = j * 16; c0 < n_valid; c0 += per_q * 16) {
            uint32_t v0[16], v1[16];
            tmem_ld16(tbase + c0, v0);
            tmem_ld16(tbase + C::KSplit * C::AccCols + c0, v1);
            tmem_ld_wait();
            if constexpr (C::KSplit == 2) {  // the second K part of each row half, added in a fixed order
                uint32_t w0[16], w1[16];
                tmem_ld16(tbase + C::AccCols + c0, w0);
                tmem_ld16(tbase + 3 * C::AccCols + c0, w1);
                tmem_ld_wait();
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) {
                    v0[jj] = __float_as_uint(__uint_as_float(v0[jj]) + __uint_as_float(w0[jj]));
                    v1[jj] = __float_as_uint(__uint_as_float(v1[jj]) + __uint_as_float(w1[jj]));
                }
            }
            if (MODE == 0) {
                const int i = rb * kTileM + r;  // intermediate column
                const int pos = (i & ~7) + ((i & 3) << 1) + ((i >> 2) & 1);
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) {
                    if (c0 + jj < n_valid) {
                        const float h = swiglu_rounded(__uint_as_float(v0[jj]), __uint_as_float(v1[jj]), a.bf16_act != 0);
                        a.hs[(int64_t)(start + c0 + jj) * a.I + pos] = __half_as_ushort(__float2half_rn(h));
                    }
                }
            } else {
                const int n = rb * 2 * kTileM + r;
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) {
                    if (c0 + jj < n_valid) {
                        const int64_t o = (int64_t)rtab.slots[start + c0 + jj] * a.N + n;
                        if (a.partial_f16) {
                            __half *dst = static_cast<__half *>(a.partial) + o;
                            dst[0] = __float2half_rn(__uint_as_float(v0[jj]));
                            dst[kTileM] = __float2half_rn(__uint_as_float(v1[jj]));
                        } else {
                            float *dst = static_cast<float *>(a.partial) + o;
                            dst[0] = __uint_as_float(v0[jj]);
                            dst[kTileM] = __uint_as_float(v1[jj]);
                        }
                    }
                }
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.acc_empty[buf]);
        return true;
    };

    if (warp == C::ProducerWarp) {
        // ---- TMA producer ----
        if (lane == 0) {
            uint32_t rawc = 0, bc = 0;
            bool ok = true;
            [[maybe_unused]] long long waited[2] = {0, 0};
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
                const int32_t *t = a.tiles + 1 + 3 * (w / a.RB);
                const int rb = w % a.RB, bucket = t[0], start = t[1];
                const int r0 = first_row(bucket, rb, 0), r1 = first_row(bucket, rb, 1);
                for (int kb = 0; kb < nkb && ok; ++kb) {
                    if ((kb & 1) == 0) {
                        const int rs = rawc % kRS;
                        TIMED_WAIT(0, mbar_wait(&ctl.raw_empty[rs], ((rawc / kRS) & 1u) ^ 1u, abort_flag));
                        if (!ok) break;
                        mbar_expect_tx(&ctl.raw_full[rs], kRawStage);
                        tma_load_2d(raws + rs * kRawStage, &raw_map, (kb >> 1) * 64, r0, &ctl.raw_full[rs]);
                        tma_load_2d(raws + rs * kRawStage + kRawTile, &raw_map, (kb >> 1) * 64, r1, &ctl.raw_full[rs]);
                        ++rawc;
                    }
                    const int s = bc % C::BS;
                    TIMED_WAIT(1, mbar_wait(&ctl.consumed[s], ((bc / C::BS) & 1u) ^ 1u, abort_flag));  // K block bc - BS is done
                    if (!ok) break;
                    mbar_expect_tx(&ctl.full[s], C::BTile);
                    tma_load_2d(b_stages + s * C::BTile, &b_map, kb * kBK, start, &ctl.full[s]);
                    ++bc;
                }
            }
            PROFILE_ADD(1, waited[0]);
            PROFILE_ADD(2, waited[1]);
        }
    } else if (warp >= C::MmaWarp) {
        // ---- MMA issuers: one warp per accumulator = (row half, K part). A tcgen05.mma occupies its issuing thread ~100 cycles
        //      whatever N <= 128 is; threads issuing into different accumulators run in parallel. ----
        const int ai = warp - C::MmaWarp, acc = ai / C::KSplit, kpart = ai % C::KSplit;
        constexpr int KSteps = (kBK / 16) / C::KSplit;  // 16-element K steps of a K block per issuer
        uint32_t kc = 0, it = 0;
        bool ok = true, peeked = false;
        [[maybe_unused]] long long waited[3] = {0, 0, 0};
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++it) {
            const int32_t *t = a.tiles + 1 + 3 * (w / a.RB);
            const int n_mma = (t[2] + 15) & ~15;
            const uint32_t idesc = umma_idesc(n_mma);
            const uint32_t buf = it % C::AccBufs;
            if (lane == 0) TIMED_WAIT(0, mbar_wait(&ctl.acc_empty[buf], ((it / C::AccBufs) & 1u) ^ 1u, abort_flag));
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            for (int kb = 0; kb < nkb && ok; ++kb, ++kc) {
                const int sa = kc % C::AS, sb_ = kc % C::BS;
                if (lane == 0 && !peeked) TIMED_WAIT(1, mbar_wait(&ctl.full[sb_], (kc / C::BS) & 1u, abort_flag));
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a0 = tmem + C::AColBase + sa * kAStageCols + acc * 32, b0 = smem_u32(b_stages + sb_ * C::BTile);
                    const uint32_t d0 = tmem + buf * C::BufCols + ai * C::AccCols;
#pragma unroll
                    for (int j = 0; j < KSteps; ++j) {  // 16 K elements = 8 packed columns of A, 32 bytes of a B row
                        const int k = kpart * KSteps + j;
                        umma_f16_ts(d0, a0 + k * 8, umma_desc(b0 + k * 32), idesc, (kb | j) ? 1u : 0u);
                    }
                    // one commit per K block and issuer (together they free the token stage and the A stage), and a first look at
                    // the next K block's barrier
                    peeked = umma_commit_and_peek(&ctl.consumed[sb_], &ctl.full[(kc + 1) % C::BS], ((kc + 1) / C::BS) & 1u);
                }
                __syncwarp();
            }
            if (lane == 0 && ok) umma_commit(&ctl.acc_full[buf]);
            __syncwarp();
        }
        if (lane == 0 && ai == 0)
            for (int i = 0; i < 3; ++i) PROFILE_ADD(3 + i, waited[i]);
        tc_fence_before();
    } else if (warp < kDequantWarps) {
        // ---- dequantizers: thread = (K block half kbl, row half acc, row r): 64 codes of one row per raw stage ----
        const int r = tid & 127, acc = (tid >> 7) & 1, kbl = tid >> 8;
        const int gpr = a.K / G;
        constexpr int NG = G >= 64 ? 1 : 64 / G;  // groups in a thread's 64 codes
        uint32_t rawc = 0;
        [[maybe_unused]] uint32_t item = 0;
        bool ok = true;
        [[maybe_unused]] long long waited[2] = {0, 0};
        [[maybe_unused]] const long long t_start = PROFILE_CLOCK();
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
            const int32_t *t = a.tiles + 1 + 3 * (w / a.RB);
            const int64_t row = (int64_t)first_row(t[0], w % a.RB, acc) + r;
            const uint16_t *srow = a.scale + row * gpr, *mrow = a.minv + row * gpr;
            for (int kb2 = 0; kb2 < nkb / 2 && ok; ++kb2, ++rawc) {
                uint32_t s2[NG], m2[NG];
                const int g0 = (kb2 * 128 + kbl * 64) / G;
#pragma unroll
                for (int g = 0; g < NG; ++g) s2[g] = bf16_to_h2(__ldg(srow + g0 + g)), m2[g] = bf16_to_h2(__ldg(mrow + g0 + g));
                const int rs = rawc % kRS;
                TIMED_WAIT(0, mbar_wait(&ctl.raw_full[rs], (rawc / kRS) & 1u, abort_flag));
                if (!ok) break;
                const uint8_t *rt = raws + rs * kRawStage + acc * kRawTile + r * 64;
                uint4 c[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) c[j] = *reinterpret_cast<const uint4 *>(rt + (((kbl * 2 + j) ^ ((r >> 1) & 3)) << 4));
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl.raw_empty[rs]);  // the codes are in registers
                uint32_t av[32];  // 64 F16 of this row: tensor-memory columns 0..31 of the stage's row half
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const uint4 q = c[u >> 2];
                    const uint32_t wv = (u & 3) == 0 ? q.x : (u & 3) == 1 ? q.y : (u & 3) == 2 ? q.z : q.w;
                    const int g = NG == 1 ? 0 : (u * 8) / G;
                    const uint4 o = dequant_word4(wv, s2[g], m2[g]);
                    av[4 * u] = o.x, av[4 * u + 1] = o.y, av[4 * u + 2] = o.z, av[4 * u + 3] = o.w;
                }
                // converted first: only the store into tensor memory waits for the stage
                const uint32_t kc = rawc * 2 + kbl;  // the K block this thread feeds
                const int s = kc % C::AS;
                if (kc >= (uint32_t)C::AS) {  // the stage is free once K block kc - AS has been consumed
                    const uint32_t pc = kc - C::AS;
                    TIMED_WAIT(1, mbar_wait(&ctl.consumed[pc % C::BS], (pc / C::BS) & 1u, abort_flag));
                    if (!ok) break;
                }
                tmem_st32(tmem + ((uint32_t)(r & ~31) << 16) + C::AColBase + s * kAStageCols + acc * 32, av);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl.full[kc % C::BS]);
            }
            if constexpr (C::CoopEpi) {  // this item's weights are all stored: help drain its accumulators
                [[maybe_unused]] long long w_epi[1] = {0};
                if (ok) ok = drain_item(w, item, warp & 3, C::EpiWarps / 4 + (warp >> 2), C::DrainWarps / 4, w_epi);
                ++item;
            }
        }
        if (tid == 0) {
            PROFILE_ADD(6, waited[0]);
            PROFILE_ADD(7, waited[1]);
            PROFILE_ADD(8, (PROFILE_CLOCK() - t_start));
        }
    } else {
        // ---- epilogue warps: lane quadrant q = warp % 4; the warps of a quadrant take alternate 16-column chunks ----
        const int ew = warp - kDequantWarps;
        constexpr int PerQ = C::DrainWarps / 4;
        uint32_t it = 0;
        bool ok = true;
        [[maybe_unused]] long long waited[1] = {0};
        [[maybe_unused]] const long long t_start = PROFILE_CLOCK();
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++it) ok = drain_item(w, it, ew & 3, ew >> 2, PerQ, waited);
        if (tid == kDequantWarps * 32) {
            PROFILE_ADD(9, waited[0]);
            PROFILE_ADD(10, (PROFILE_CLOCK() - t_start));
            PROFILE_ADD(11, it);
        }
    }
    __syncthreads();
    if (tid == 0) PROFILE_ADD(0, (PROFILE_CLOCK() - t_kernel));
    if (tid == 0 && ctl.abort_flag) atomicAdd(&g_prefill_aborts, 1u);
    if (warp == C::MmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// logits[m, r] = sum_k x[m, k] * w[r, k], BF16 operands straight from global memory. Grid (row tiles, token tiles).
constexpr int kDS = 4;  // stages of [A 16 KB | B 16 KB]
struct DenseCtl {
    uint64_t full[kDS], empty[kDS], acc_full;
    uint32_t tmem_base;
    int abort_flag;
};

__global__ void __launch_bounds__(192, 1)
    dense_umma_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map, int K, int R, int M, float *logits,
                      const float *bias, int n_bias) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *stages = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    DenseCtl &ctl = *reinterpret_cast<DenseCtl *>(stages + kDS * 2 * kTile);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < kDS; ++i) mbar_init(&ctl.full[i], 1), mbar_init(&ctl.empty[i], 1);
        mbar_init(&ctl.acc_full, 1);
        ctl.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_base)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl.tmem_base;
    const int r0 = blockIdx.x * kTileM, m0 = blockIdx.y * 128;
    const int nkb = K / kBK;
    volatile int *abort_flag = &ctl.abort_flag;
    if (warp == 4) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % kDS;
                if (!mbar_wait(&ctl.empty[s], ((kb / kDS) & 1u) ^ 1u, abort_flag)) break;
                mbar_expect_tx(&ctl.full[s], 2 * kTile);
                tma_load_2d(stages + s * 2 * kTile, &w_map, kb * kBK, r0, &ctl.full[s]);
                tma_load_2d(stages + s * 2 * kTile + kTile, &x_map, kb * kBK, m0, &ctl.full[s]);
            }
        }
    } else if (warp == 5) {
        const uint32_t idesc = umma_idesc(128, /*bf16=*/true);
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % kDS;
            if (lane == 0) ok = mbar_wait(&ctl.full[s], (kb / kDS) & 1u, abort_flag);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a0 = smem_u32(stages + s * 2 * kTile), b0 = a0 + kTile;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) umma_f16(tmem, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), idesc, (kb | k) ? 1u : 0u);
                umma_commit(&ctl.empty[s]);
            }
            __syncwarp();
        }
        if (lane == 0 && ok) umma_commit(&ctl.acc_full);
        tc_fence_before();
    } else {
        if (mbar_wait(&ctl.acc_full, 0, abort_flag)) {
            tc_fence_after();
            const int r = r0 + warp * 32 + lane;
            const float b = bias != nullptr && r < n_bias ? bias[r] : 0.f;  // the same FP32 add a separate pass would do
            for (int c0 = 0; c0 < 128 && m0 + c0 < M; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (r < R && m0 + c0 + j < M) logits[(int64_t)(m0 + c0 + j) * R + r] = __uint_as_float(v[j]) + b;
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (tid == 0 && ctl.abort_flag) atomicAdd(&g_prefill_aborts, 1u);
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encoder(const char *fn, EncodeFn *out) {
    static std::mutex mu;
    static EncodeFn cached = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (cached == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        SB_CUDA(cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q), fn, ": looking up the tensor-map encoder");
        SB_CHECK(q == cudaDriverEntryPointSuccess && p != nullptr, fn, ": the driver has no tensor-map encoder");
        cached = reinterpret_cast<EncodeFn>(p);
    }
    *out = cached;
    return 0;
}

// rows x cols elements of `es` bytes, row pitch = cols * es, box = box_rows x box_cols.
int make_map(const char *fn, CUtensorMap *m, CUtensorMapDataType dt, int es, const void *ptr, int64_t rows, int64_t cols, int box_cols,
             CUtensorMapSwizzle sw, int box_rows = 128) {
    EncodeFn enc;
    SB_TRY(encoder(fn, &enc));
    SB_CHECK(reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && (cols * es) % 16 == 0, fn, ": tensor ", ptr, " with a row pitch of ", cols * es,
             " bytes is not 16-byte aligned");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows}, strides[1] = {(cuuint64_t)(cols * es)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows}, estr[2] = {1, 1};
    const CUresult rc = enc(m, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SB_CHECK(rc == CUDA_SUCCESS, fn, ": cuTensorMapEncodeTiled failed with ", (int)rc, " for a [", rows, ", ", cols, "] tensor");
    return 0;
}

template <int SHAPE>
constexpr size_t ffn_smem() {
    return (size_t)FC<SHAPE>::BS * FC<SHAPE>::BTile + (size_t)kRS * kRawStage + sizeof(Ctl<SHAPE>) + 1024;
}
constexpr size_t kDenseSmem = (size_t)kDS * 2 * kTile + sizeof(DenseCtl) + 1024;

template <int MODE, int SHAPE>
int launch_ffn(const char *fn, int G, const CUtensorMap &raw, const CUtensorMap &b, const FfnArgs &a, int ctas, cudaStream_t st) {
    static thread_local int prepared = -1;  // one per (MODE, SMALL) and host thread
    constexpr size_t smem = ffn_smem<SHAPE>();
    constexpr int threads = FC<SHAPE>::Threads;
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev), fn);
    if (prepared != dev) {
        SB_CUDA(cudaFuncSetAttribute(ffn_umma_kernel<MODE, 32, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(ffn_umma_kernel<MODE, 64, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(ffn_umma_kernel<MODE, 128, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        prepared = dev;
    }
    if (G == 32) ffn_umma_kernel<MODE, 32, SHAPE><<<ctas, threads, smem, st>>>(raw, b, a);
    else if (G == 64) ffn_umma_kernel<MODE, 64, SHAPE><<<ctas, threads, smem, st>>>(raw, b, a);
    else ffn_umma_kernel<MODE, 128, SHAPE><<<ctas, threads, smem, st>>>(raw, b, a);
    SB_LAUNCH_OK(fn, " (tcgen05 FFN stage ", MODE, SHAPE == kSmall ? ", small tiles" : SHAPE == kXWide ? ", 192-slot tiles" : "", ") K=", a.K, " G=", G);
    return 0;
}

}  // namespace

namespace sb {

struct PrefillPlan {
    CUtensorMap gu_raw, dn_raw, xg_map, hs_map, xg_map_s, hs_map_s, xg_map_x, hs_map_x, rw_map;  // _s / _x: boxes of 32 / 192 rows (small / 192-slot tiles)
    bool dense_router = false;
    int64_t d, I, Estack, max_tokens, A, router_rows;
    int G_gu, G_dn;
    const uint16_t *gu_scale, *gu_min, *dn_scale, *dn_min;
    uint16_t *xg = nullptr, *hs = nullptr;
    int32_t *tiles = nullptr;
    int sms = 0;
};

bool prefill_supported(const strix_moe_layer_desc &d) {
    return !d.experts_mixed && d.gate_up_bits == 4 && d.down_bits == 4 && d.d % 256 == 0 && d.I % 128 == 0 && d.d <= (1 << 20) && d.I <= (1 << 20);
}

int prefill_create(const strix_moe_layer_desc &d, int64_t A, int64_t Estack, int64_t router_rows, PrefillPlan **out) {
    const char *fn = "moe_layer_create (tensor-core path)";
    auto *p = new PrefillPlan();
    p->d = d.d, p->I = d.I, p->Estack = Estack, p->max_tokens = d.max_tokens, p->A = A, p->router_rows = router_rows;
    p->G_gu = (int)d.gate_up.G, p->G_dn = (int)d.down.G;
    p->gu_scale = d.gate_up.scale, p->gu_min = d.gate_up.minv, p->dn_scale = d.down.scale, p->dn_min = d.down.minv;
    p->sms = sm_count();
    const int64_t S = d.max_tokens * A;
    int rc = 0;
    auto alloc = [&](void **q, size_t bytes) {
        if (rc == 0 && cudaMalloc(q, bytes) != cudaSuccess) {
            last_error() = std::string(fn) + ": cudaMalloc failed";
            rc = STRIX_ERR_CUDA;
        }
    };
    alloc(reinterpret_cast<void **>(&p->xg), (size_t)S * d.d * 2);
    alloc(reinterpret_cast<void **>(&p->hs), (size_t)S * d.I * 2);
    alloc(reinterpret_cast<void **>(&p->tiles), (size_t)(1 + 3 * (S / FC<kSmall>::TileSlots + Estack + 2)) * 4);
    if (rc == 0) rc = make_map(fn, &p->gu_raw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d.gate_up.q, Estack * 2 * d.I, d.d / 2, 64, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc == 0) rc = make_map(fn, &p->dn_raw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d.down.q, Estack * d.d, d.I / 2, 64, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc == 0) rc = make_map(fn, &p->xg_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->xg, S, d.d, kBK, CU_TENSOR_MAP_SWIZZLE_128B, FC<kWide>::TileSlots);
    if (rc == 0) rc = make_map(fn, &p->hs_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->hs, S, d.I, kBK, CU_TENSOR_MAP_SWIZZLE_128B, FC<kWide>::TileSlots);
    if (rc == 0) rc = make_map(fn, &p->xg_map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->xg, S, d.d, kBK, CU_TENSOR_MAP_SWIZZLE_128B, FC<kSmall>::TileSlots);
    if (rc == 0) rc = make_map(fn, &p->hs_map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->hs, S, d.I, kBK, CU_TENSOR_MAP_SWIZZLE_128B, FC<kSmall>::TileSlots);
    if (rc == 0) rc = make_map(fn, &p->xg_map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->xg, S, d.d, kBK, CU_TENSOR_MAP_SWIZZLE_128B, FC<kXWide>::TileSlots);
    if (rc == 0) rc = make_map(fn, &p->hs_map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p->hs, S, d.I, kBK, CU_TENSOR_MAP_SWIZZLE_128B, FC<kXWide>::TileSlots);
    p->dense_router = d.act == kBF16 && d.router_kind == STRIX_ROUTER_BF16 && d.d % kBK == 0;
    if (rc == 0 && p->dense_router)
        rc = make_map(fn, &p->rw_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d.router_w, router_rows, d.d, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) {
        prefill_destroy(p);
        return rc;
    }
    *out = p;
    return 0;
}

void prefill_destroy(PrefillPlan *p) {
    if (p == nullptr) return;
    if (p->xg) cudaFree(p->xg);
    if (p->hs) cudaFree(p->hs);
    if (p->tiles) cudaFree(p->tiles);
    delete p;
}

bool prefill_has_dense_router(const PrefillPlan *p) { return p->dense_router; }

int prefill_router_logits(PrefillPlan *p, const void *x, int64_t M, float *logits, const float *bias, int64_t n_bias, cudaStream_t st) {
    const char *fn = "moe_layer_forward (tensor-core router)";
    CUtensorMap xm;
    SB_TRY(make_map(fn, &xm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, p->d, kBK, CU_TENSOR_MAP_SWIZZLE_128B));
    static thread_local int prepared = -1;
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev), fn);
    if (prepared != dev) {
        SB_CUDA(cudaFuncSetAttribute(dense_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDenseSmem), fn);
        prepared = dev;
    }
    const dim3 grid((unsigned)((p->router_rows + kTileM - 1) / kTileM), (unsigned)((M + 127) / 128));
    dense_umma_kernel<<<grid, 192, kDenseSmem, st>>>(p->rw_map, xm, (int)p->d, (int)p->router_rows, (int)M, logits, bias, (int)n_bias);
    SB_LAUNCH_OK(fn, " M=", M, " R=", p->router_rows, " K=", p->d);
    return 0;
}

int dense_bf16(const char *fn, const void *x, const uint16_t *w, float *y, int64_t M, int64_t N, int64_t K, const float *bias, int64_t n_bias,
               cudaStream_t st) {
    CUtensorMap xm, wm;
    SB_TRY(make_map(fn, &xm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, M, K, kBK, CU_TENSOR_MAP_SWIZZLE_128B));
    SB_TRY(make_map(fn, &wm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, N, K, kBK, CU_TENSOR_MAP_SWIZZLE_128B));
    static thread_local int prepared = -1;
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev), fn);
    if (prepared != dev) {
        SB_CUDA(cudaFuncSetAttribute(dense_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDenseSmem), fn);
        prepared = dev;
    }
    const dim3 grid((unsigned)((N + kTileM - 1) / kTileM), (unsigned)((M + 127) / 128));
    dense_umma_kernel<<<grid, 192, kDenseSmem, st>>>(wm, xm, (int)K, (int)N, (int)M, y, bias, (int)n_bias);
    SB_LAUNCH_OK(fn, " (tensor cores) M=", M, " N=", N, " K=", K);
    return 0;
}

bool dense_bf16_ok(const void *x, const void *w, int64_t M, int64_t N, int64_t K) {
    return M >= 64 && K % kBK == 0 && K <= (1 << 24) && N <= (1 << 24) && M <= (1 << 24) && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(w) % 16 == 0;
}

int prefill_experts(PrefillPlan *p, const void *x, const int32_t *row_index, int act, const int32_t *ws, int64_t M, int64_t A, void *partial,
                    bool half_partial, cudaStream_t st) {
    const char *fn = "moe_layer_forward (tensor-core experts)";
    // a handful of tokens (decode, verify): tiles of 32 slots and four issuing warps; many tokens: tiles of 96 slots; an average
    // of more than a 96-slot tile per expert: tiles of 192 slots
    int shape = M * A <= kSmallSlots ? kSmall : M * A > (int64_t)FC<kWide>::TileSlots * p->Estack ? kXWide : kWide;
#ifdef STRIX_PROFILE
    if (const char *force = std::getenv("STRIX_FFN_SHAPE")) shape = std::atoi(force);  // diagnostic build: A/B of the tile shapes
#endif
    SB_CHECK(M * A <= p->max_tokens * p->A, fn, ": ", M * A, " slots exceed the layer's ", p->max_tokens * p->A);
    const int32_t S = (int32_t)(M * A), E = (int32_t)p->Estack;
    tiles_kernel<<<1, 1024, 0, st>>>(ws, p->tiles, shape == kSmall ? FC<kSmall>::TileSlots : shape == kXWide ? FC<kXWide>::TileSlots : FC<kWide>::TileSlots, S, E);
    SB_LAUNCH_OK(fn, ": tiles");
    const unsigned gblocks = (unsigned)std::min<int64_t>((M * A + 7) / 8, 148 * 16);
    if (act == kF32) pregather_kernel<float><<<gblocks, 256, 0, st>>>((const float *)x, row_index, ws, A, p->d, p->xg, S, E);
    else pregather_kernel<uint16_t><<<gblocks, 256, 0, st>>>((const uint16_t *)x, row_index, ws, A, p->d, p->xg, S, E);
    SB_LAUNCH_OK(fn, ": gather");
    FfnArgs a{};
    a.ws = ws, a.tiles = p->tiles;
    a.scale = p->gu_scale, a.minv = p->gu_min, a.K = (int)p->d, a.rows_per_expert = (int)(2 * p->I), a.I = (int)p->I, a.RB = (int)(p->I / kTileM);
    a.hs = p->hs, a.partial = nullptr, a.partial_f16 = 0, a.N = 0, a.bf16_act = act == kBF16;
    if (shape == kSmall) SB_TRY((launch_ffn<0, kSmall>(fn, p->G_gu, p->gu_raw, p->xg_map_s, a, p->sms, st)));
    else if (shape == kXWide) SB_TRY((launch_ffn<0, kXWide>(fn, p->G_gu, p->gu_raw, p->xg_map_x, a, p->sms, st)));
    else SB_TRY((launch_ffn<0, kWide>(fn, p->G_gu, p->gu_raw, p->xg_map, a, p->sms, st)));
    a.scale = p->dn_scale, a.minv = p->dn_min, a.K = (int)p->I, a.rows_per_expert = (int)p->d, a.RB = (int)(p->d / (2 * kTileM));
    a.hs = nullptr, a.partial = partial, a.partial_f16 = half_partial ? 1 : 0, a.N = (int)p->d;
    if (shape == kSmall) SB_TRY((launch_ffn<1, kSmall>(fn, p->G_dn, p->dn_raw, p->hs_map_s, a, p->sms, st)));
    else if (shape == kXWide) SB_TRY((launch_ffn<1, kXWide>(fn, p->G_dn, p->dn_raw, p->hs_map_x, a, p->sms, st)));
    else SB_TRY((launch_ffn<1, kWide>(fn, p->G_dn, p->dn_raw, p->hs_map, a, p->sms, st)));
    return 0;
}

void prefill_cycles(unsigned long long *out, bool reset) {
#ifdef STRIX_PROFILE
    cudaMemcpyFromSymbol(out, g_prefill_cycles, sizeof(unsigned long long) * 32);
    if (reset) {
        unsigned long long z[32] = {};
        cudaMemcpyToSymbol(g_prefill_cycles, z, sizeof(z));
    }
#else
    (void)reset;
    for (int i = 0; i < 32; ++i) out[i] = 0;
#endif
}

unsigned int prefill_ws_refusals() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_ws_refusals, sizeof(v));
    return v;
}

unsigned int prefill_aborts() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_prefill_aborts, sizeof(v));
    return v;
}

}  // namespace sb
