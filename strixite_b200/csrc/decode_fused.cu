// The whole MoE sublayer for a handful of tokens (decode, speculative verify: M <= 8) as ONE persistent kernel.
//
// A decode layer moves ~20-100 MB of packed expert weights exactly once and does almost no arithmetic, so the design
// is a weight-streaming machine: one CTA per SM, twelve warps, each running its own software pipeline of asynchronous
// 16-byte copies (cp.async.cg, L2 -> shared memory, no registers) into a private ring of padded shared-memory stages,
// and turning the staged nibbles into dot products. (Bulk-copy engines were measured first: one cp.async.bulk per row
// slice costs ~100 cycles of issue time whatever its size, which capped a CTA near 5 B/clk; rows need padding for
// conflict-free reads, so they cannot be fetched as one large contiguous bulk copy either.)
// The dots run on the tensor cores as a data-movement trick, not as a GEMM: mma.sync m16n8k16 takes 16 weight rows x
// 16 codes against 8 columns, so one unpack of a weight word (lop3 into BF16 "128 + code", exact) serves every token
// and the CUDA cores only unpack. FP32 activations are split into two BF16 planes (x = hi + lo, products exact, FP32
// accumulate) that sit side by side in the 8 MMA columns (4 tokens x 2 planes per pass); the "+128" offset and the
// group minimum fold into one FMA per quantization group: s * acc + (m - 128 s) * sum(plane). Each distinct active
// expert is streamed once however many tokens chose it.
//
// Phases (two grid barriers; the CTAs are co-resident by a cooperative launch):
//   0  x -> FP32 copy and permuted BF16 planes in shared memory, per-plane chunk sums
//   1  router logits [M, R]: two warps per router row, FP32 FMA, weights straight from global memory
//   -- barrier --
//   2  every CTA: top-k + weights for the M tokens and the distinct-expert groups; then gate/up tiles: 8 gate + 8 up
//      rows of one expert as one 16-row MMA tile, K split over a team of nk warps (a stage per warp), the SwiGLU
//      lane-local in the team leader's epilogue -> h (plain, and as pre-split BF16 planes + partial sums for phase 3)
//   -- barrier --
//   3  down projection + weighted combine: a CTA owns 16 output rows and walks every active expert (a stage per
//      expert, a warp per stage), accumulating coef * (W h) in registers; one ordered cross-warp sum -> y.
// The separate (dense) shared expert is one more group whose tokens are all M; its part is rounded and added as the
// reference's moe_shared_add does. Summation orders are fixed: the output is bit-reproducible.
//
// The only waits that depend on other CTAs are the two grid barriers; they are bounded: on expiry the CTA raises the
// abort word, all CTAs leave and the host sees the expert error words {2, 0xdec000 | code, block}.
#include "common.cuh"

#include "decode_fused.cuh"
#include "strixite_b200.h"

namespace {

using namespace sb;

constexpr int CW = 12;                     // warps; every warp streams and consumes its own stages
constexpr int kThreads = 32 * CW;
constexpr int kMaxTok = 8;
constexpr int kMaxGroups = 96;
constexpr int kMaxSlots = kMaxGroups - 1;
constexpr int kDnCols = 2;                               // tokens per down-projection stage at most
constexpr int kMaxDnItems = kMaxGroups + kMaxSlots / 2;  // sum over groups of ceil(tokens / kDnCols)
constexpr int kMaxDepth = 4;               // stages per warp
constexpr uint32_t kSpinLimit = 1u << 22;  // polls before a wait gives up (each poll is tens of ns)

// ---- PTX wrappers ----------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte asynchronous copy global -> shared through L2 (both addresses 16-byte aligned).
__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most `pending` of this thread's committed copy groups are still in flight.
__device__ __forceinline__ void cp_async_wait(int pending) {
    switch (pending) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    }
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void named_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}
// Phase timestamps of block 0 for profiling: sync[8 + i] = ns (low 32 bits of %globaltimer), sync[16 + i] = SM cycles.
__device__ __forceinline__ void stamp(uint32_t *sync, int i) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        uint64_t t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        sync[8 + i] = (uint32_t)t;
        sync[16 + i] = (uint32_t)clock64();
    }
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ---- shared-memory plan ------------------------------------------------------------------------------------------

struct Group {  // one distinct active expert with both projections resolved
    const uint8_t *rows[2];      // [0] gate_up, [1] down
    const uint16_t *scale[2], *minv[2];
    int32_t expert;              // row block of the stacks, or -2 = the separate shared expert
    uint32_t mask;               // tokens routed to it
    int16_t G[2];
    uint8_t bits[2];
    int8_t slot_a[kMaxTok];      // token m's slot index a (ids[m, a] == expert), -1 if not routed
};

struct Smem {
    Group groups[kMaxGroups];
    int32_t ids[kMaxSlots + 1];
    float coef[kMaxSlots + 1];
    int16_t slot_group[kMaxSlots + 1];  // scratch of the group build
    float gate[kMaxTok];         // the separate shared expert's coefficient per token
    float red[2][CW][32][8];     // team exchange (phase 2) / cross-warp partial tiles (phase 3): [pass][4] per lane
    float red_sh[2][32][8];      // phase 3: the separate shared expert's tile, kept apart for its own rounding
    float rpart[CW][kMaxTok];  // phase 1: half-row partial logits
    int leaders_before[CW + 2];
    int n_groups, col_max, abort_flag;
    // phase 3 work list: a group's tokens in runs of at most kDnCols, so that a stage holds few h records and every warp
    // gets a stage (a wide group's weights are fetched once per run)
    uint8_t dn_group[kMaxDnItems], dn_mask[kMaxDnItems];
    int n_dn;
    uint32_t failed_mask;        // tokens the router failed (non-finite logits): NaN rows
};

__device__ __forceinline__ void resolve_group(const DecodeParams &p, Group &g) {
#pragma unroll
    for (int down = 0; down < 2; ++down) {
        if (g.expert == -2) {
            const strix_qview &v = down ? p.sh_down : p.sh_gate_up;
            g.rows[down] = v.q, g.scale[down] = v.scale, g.minv[down] = v.minv;
            g.bits[down] = (uint8_t)(down ? p.sh_down_bits : p.sh_gate_up_bits), g.G[down] = (int16_t)v.G;
        } else {
            const StackView &s = down ? p.down : p.gate_up;
            const int b = s.bits_of(g.expert);
            g.bits[down] = (uint8_t)b;
            g.rows[down] = s.rows(g.expert, b);
            const int64_t off = (int64_t)g.expert * s.N * (s.K / s.G);
            g.scale[down] = s.scale + off, g.minv[down] = s.minv + off, g.G[down] = (int16_t)s.G;
        }
    }
}

// Bytes of the slice [h * K / nk, (h + 1) * K / nk) of a packed row: the low plane's part and the high plane's part.
__host__ __device__ inline int slice_lo_bytes(int bits, int Ks) { return bits == 8 ? Ks : Ks / 2; }
__host__ __device__ inline int slice_hi_bytes(int bits, int Ks) { return bits == 5 ? Ks / 8 : bits == 6 ? Ks / 4 : 0; }

// ---- the unpack: one 8-code unit of a staged row slice -> BF16 pairs (128 + code) for two MMAs ---------------------
// lo[j] = {code j (low half), code j + 4 (high half)} for j = 0..3, each as BF16 bits 0x4300 | code (= 128 + code,
// exact for code < 128). Q8 yields the low and the high nibble of each code separately (lo[], hi[]).
constexpr uint32_t kMagic = 0x43004300u, kNib = 0x000F000Fu;

template <int BITS>
struct Unit {
    uint32_t lo[4];
    uint32_t hi[BITS == 8 ? 4 : 1];
    // row: the staged slice (low plane part, then the high plane part); unit u = its codes 8u .. 8u+7; Ks = codes in the slice
    __device__ __forceinline__ void load(const uint8_t *row, int Ks, int u) {
        if constexpr (BITS == 8) {
            const uint2 w = *reinterpret_cast<const uint2 *>(row + u * 8);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t pair = __byte_perm(w.x, w.y, 0x4040 | j | ((4 + j) << 8)) & 0x00FF00FFu;  // [b_j(w.x), 0, b_j(w.y), 0]
                lo[j] = lop3_and_or(pair, kNib, kMagic);
                hi[j] = lop3_and_or(pair >> 4, kNib, kMagic);
            }
        } else {
            const uint32_t w = *reinterpret_cast<const uint32_t *>(row + u * 4);
            if constexpr (BITS == 4) {
#pragma unroll
                for (int j = 0; j < 4; ++j) lo[j] = lop3_and_or(w >> (4 * j), kNib, kMagic);
            } else if constexpr (BITS == 5) {  // 5th bits: one byte per unit behind the low plane part
                const uint32_t t = row[Ks / 2 + u];
                const uint32_t v = ((t & 0x0Fu) | ((t & 0xF0u) << 12)) << 4;  // bits 4..7 = t0..t3, bits 20..23 = t4..t7
#pragma unroll
                for (int j = 0; j < 4; ++j) lo[j] = lop3_and_or(w >> (4 * j), kNib, kMagic) | ((v >> j) & 0x00100010u);
            } else {  // bits 4..5: two bytes per unit
                const uint32_t t = *reinterpret_cast<const uint16_t *>(row + Ks / 2 + u * 2);
                const uint32_t v = ((t & 0xFFu) | ((t & 0xFF00u) << 8)) << 4;  // bits 4..11 = pairs 0..3, bits 20..27 = pairs 4..7
#pragma unroll
                for (int j = 0; j < 4; ++j) lo[j] = lop3_and_or(w >> (4 * j), kNib, kMagic) | ((v >> (2 * j)) & 0x00300030u);
            }
        }
    }
};

// One quantization group (G codes from unit u0 of the slice) of a 16-row tile against the lane's token columns; adds to
// tot[pass][] the lane's 2 rows x 2 columns of s * sum(x * code) + m * sum(x).
//   rowA / rowB: the staged slices of MMA rows g and g + 8
//   xb[pass]: the lane's column (a token's plane) for that pass, null = zeros
//   xs[pass][e]: sum of that plane over the group for the lane's accumulator column 2c + e
// Columns: BF16 activations use one pass, column n = token n. FP32 activations pack a token's two BF16 planes side by
// side - column n = token (n & 3) + 4 * pass, plane n >> 2 - so that one MMA covers both planes of up to 4 tokens.
// Independent accumulators per MMA of a unit keep the tensor pipe from waiting on its own results.
template <int BITS, int NP, int NCH>  // NCH: 32-code chunks per group when known at compile time (4 = groups of 128), 0 = n_chunks
__device__ __forceinline__ void group_dot(const uint8_t *rowA, const uint8_t *rowB, int Ks, const uint8_t *const (&xb)[NP], int u0, int n_chunks,
                                          int c, float sA, float mA, float sB, float mB, const float (&xs)[NP][2], float (&tot)[NP][4]) {
    float a0[NP][4], a1[NP][4], h0[BITS == 8 ? NP : 1][4], h1[BITS == 8 ? NP : 1][4];
#pragma unroll
    for (int p = 0; p < NP; ++p)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            a0[p][i] = 0.f, a1[p][i] = 0.f;
            if (BITS == 8) h0[p][i] = 0.f, h1[p][i] = 0.f;
        }
#pragma unroll
    for (int q = 0; q < (NCH ? NCH : n_chunks); ++q) {
        const int u = u0 + 4 * q + c;  // a 32-code chunk is 4 units, one per lane of the quad
        Unit<BITS> a, b;
        a.load(rowA, Ks, u);
        b.load(rowB, Ks, u);
        const uint32_t f0[4] = {a.lo[0], b.lo[0], a.lo[1], b.lo[1]}, f1[4] = {a.lo[2], b.lo[2], a.lo[3], b.lo[3]};
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            uint4 x = make_uint4(0, 0, 0, 0);
            if (xb[p] != nullptr) x = *reinterpret_cast<const uint4 *>(xb[p] + u * 16);
            mma_bf16(a0[p], f0, x.x, x.y);
            mma_bf16(a1[p], f1, x.z, x.w);
            if constexpr (BITS == 8) {
                const uint32_t e0[4] = {a.hi[0], b.hi[0], a.hi[1], b.hi[1]}, e1[4] = {a.hi[2], b.hi[2], a.hi[3], b.hi[3]};
                mma_bf16(h0[p], e0, x.x, x.y);
                mma_bf16(h1[p], e1, x.z, x.w);
            }
        }
    }
    // staged codes carry +128 (x 17 for Q8's two nibble planes): s * acc + (m - off * s) * xsum
    constexpr float off = BITS == 8 ? 128.f * 17.f : 128.f;
    const float mA2 = fmaf(-off, sA, mA), mB2 = fmaf(-off, sB, mB);
#pragma unroll
    for (int p = 0; p < NP; ++p) {
        float a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = BITS == 8 ? fmaf(16.f, h0[p][i] + h1[p][i], a0[p][i] + a1[p][i]) : a0[p][i] + a1[p][i];
        tot[p][0] += fmaf(sA, a[0], mA2 * xs[p][0]);
        tot[p][1] += fmaf(sA, a[1], mA2 * xs[p][1]);
        tot[p][2] += fmaf(sB, a[2], mB2 * xs[p][0]);
        tot[p][3] += fmaf(sB, a[3], mB2 * xs[p][1]);
    }
}

// The token and plane behind MMA column n of a pass (see group_dot).
template <int PLANES>
__device__ __forceinline__ void column_of(int n, int pass, int &token, int &plane) {
    if (PLANES == 2) token = (n & 3) + 4 * pass, plane = n >> 2;
    else token = n, plane = 0;
}

// ---- grid barrier ------------------------------------------------------------------------------------------------
// counters[i] counts arrivals of barrier i; the last CTA to leave the kernel zeroes them, so a launch (or a graph
// replay) always starts from zero. Bounded: false = gave up.
__device__ __forceinline__ void grid_arrive(uint32_t *counter) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
    }
}
__device__ __forceinline__ bool grid_wait(const uint32_t *counter, uint32_t *abort_word, Smem &sm) {
    if (threadIdx.x == 0) {
        bool ok = false;
        for (uint32_t i = 0; i < kSpinLimit; ++i) {
            if (ld_acquire(counter) >= gridDim.x) {
                ok = true;
                break;
            }
            if ((i & 63u) == 63u && ld_acquire(abort_word) != 0u) break;
        }
        if (!ok && sm.abort_flag == 0) sm.abort_flag = ld_acquire(abort_word) != 0u ? 0x200 : 0x105;
    }
    __syncthreads();
    return sm.abort_flag == 0;
}

// The FP32 copy of x in shared memory keeps each 32-value chunk's eight 16-byte pieces XOR-rotated by the chunk index, so
// that lanes reading the same piece of 32 consecutive chunks (the quantized router rows: one chunk per lane) spread over
// all banks instead of colliding on four. Only with a quantized router: the unquantized rows read consecutive pieces per
// lane and keep the plain layout. k: a multiple of 4.
__device__ __forceinline__ int xf_index(int k) { return (k & ~31) + ((((k >> 2) ^ (k >> 5)) & 7) << 2); }

// ---- phase 1: router logits ----------------------------------------------------------------------------------------
// Two warps per router row (each half of K), all M tokens at once; x as FP32 from shared memory. The halves meet in
// shared memory after a block barrier.
__device__ __forceinline__ void router_half_row(const DecodeParams &p, const float *xf, int r, int half, int lane, float (&acc)[kMaxTok]) {
    const int K = p.d, Kh = K / 2, k_lo = half * Kh, M = p.M;
#pragma unroll
    for (int m = 0; m < kMaxTok; ++m) acc[m] = 0.f;
    if (p.router_kind == STRIX_ROUTER_Q) {
        const strix_qview &v = p.router_q;
        const int gpr = (int)(v.K / v.G);
        by_bits(p.router_bits, [&](auto bc) {
            constexpr int BITS = decltype(bc)::value;
            const uint8_t *row = v.q + (int64_t)r * row_bytes(BITS, K);
            for (int c = k_lo / 32 + lane; c < (k_lo + Kh) / 32; c += 32) {
                float code[32];
                load_codes32<BITS>(row, K, c, code);
                const float s = bf16_bits_to_f32(v.scale[(int64_t)r * gpr + c * 32 / v.G]);
                const float mn = bf16_bits_to_f32(v.minv[(int64_t)r * gpr + c * 32 / v.G]);
#pragma unroll
                for (int m = 0; m < kMaxTok; ++m) {
                    if (m < M) {
                        float dot = 0.f, xs = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 f = *reinterpret_cast<const float4 *>(xf + m * K + xf_index(c * 32 + 4 * i));
                            dot = fmaf(f.x, code[4 * i], dot), dot = fmaf(f.y, code[4 * i + 1], dot);
                            dot = fmaf(f.z, code[4 * i + 2], dot), dot = fmaf(f.w, code[4 * i + 3], dot);
                            xs += (f.x + f.y) + (f.z + f.w);
                        }
                        acc[m] = fmaf(s, dot, fmaf(mn, xs, acc[m]));
                    }
                }
            }
        });
        return;
    }
    // Unquantized rows: every 16-byte load of the half row is issued before the first is used.
    constexpr int U = 8;  // 8 weights per lane per load; a half row of up to 8 * 256 = 2048 weights per pass
    for (int k0 = k_lo + lane * 8; k0 < k_lo + Kh; k0 += 256 * U) {
        float wv[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * 256;
            if (k < k_lo + Kh) {
                if (p.router_kind == STRIX_ROUTER_F32) {
                    const float *wr = static_cast<const float *>(p.router_w) + (int64_t)r * K + k;
                    const float4 a = __ldg(reinterpret_cast<const float4 *>(wr)), b = __ldg(reinterpret_cast<const float4 *>(wr + 4));
                    wv[u][0] = a.x, wv[u][1] = a.y, wv[u][2] = a.z, wv[u][3] = a.w, wv[u][4] = b.x, wv[u][5] = b.y, wv[u][6] = b.z, wv[u][7] = b.w;
                } else {
                    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.router_w) + (int64_t)r * K + k));
                    const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) wv[u][2 * j] = __uint_as_float(w4[j] << 16), wv[u][2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * 256;
            if (k < k_lo + Kh) {
#pragma unroll
                for (int m = 0; m < kMaxTok; ++m) {
                    if (m < M) {
                        const float4 a = *reinterpret_cast<const float4 *>(xf + m * K + k), b = *reinterpret_cast<const float4 *>(xf + m * K + k + 4);
                        float t = acc[m];
                        t = fmaf(a.x, wv[u][0], t), t = fmaf(a.y, wv[u][1], t), t = fmaf(a.z, wv[u][2], t), t = fmaf(a.w, wv[u][3], t);
                        t = fmaf(b.x, wv[u][4], t), t = fmaf(b.y, wv[u][5], t), t = fmaf(b.z, wv[u][6], t), t = fmaf(b.w, wv[u][7], t);
                        acc[m] = t;
                    }
                }
            }
        }
    }
}

// ---- phase 2a: routing and the distinct-expert groups, computed by every CTA ---------------------------------------

__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

// One warp routes token m (the router kernel's algorithm: two hardware warp reductions per pick).
template <int NV>
__device__ void route_token(const DecodeParams &p, Smem &sm, int m, int lane, bool write_global) {
    const float *row = p.logits + (int64_t)m * p.R;
    const int E = p.E, k = p.k, A = p.A;
    float v[NV];
    unsigned bad = 0xffffffffu;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? __ldcg(row + e) : -INFINITY;
        if (e < E && !isfinite(v[j]) && (unsigned)e < bad) bad = (unsigned)e;
    }
    float sl = 0.f;
    if (p.gated) {
        sl = __ldcg(row + E);
        if (!isfinite(sl) && (unsigned)E < bad) bad = (unsigned)E;
    }
    bad = __reduce_min_sync(0xffffffffu, bad);
    if (bad != 0xffffffffu) {
        if (lane == 0) {
            atomicOr(&sm.failed_mask, 1u << m);
            if (write_global) raise_err(p.err, (uint32_t)m, bad);
        }
        for (int a = lane; a < A; a += 32) {
            sm.ids[m * A + a] = -1, sm.coef[m * A + a] = qnan();
            if (write_global) p.ids[m * A + a] = -1, p.coef[m * A + a] = qnan();
        }
        if (lane == 0) sm.gate[m] = qnan();
        return;
    }
    float lv;
    int li;
    auto rescan = [&]() {
        lv = -INFINITY, li = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (v[j] > lv) lv = v[j], li = lane + 32 * j;
    };
    rescan();
    float my_v = -INFINITY, top = 0.f;
    int my_i = -1;
    for (int r = 0; r < k; ++r) {
        const uint32_t key = order_key(lv);
        const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
        const unsigned pick = __reduce_min_sync(0xffffffffu, key == kmax ? (unsigned)li : 0xffffffffu);
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
    if (lane < k) {
        const float c = ex / sum;
        sm.ids[m * A + lane] = my_i, sm.coef[m * A + lane] = c;
        if (write_global) p.ids[m * A + lane] = my_i, p.coef[m * A + lane] = c;
    }
    if (lane == 0) {
        const float g = p.gated ? sigmoid_f(sl) : 1.0f;
        sm.gate[m] = g;
        if (p.shared_mode == STRIX_SHARED_STACKED) {
            sm.ids[m * A + k] = E, sm.coef[m * A + k] = g;
            if (write_global) p.ids[m * A + k] = E, p.coef[m * A + k] = g;
        }
    }
}

// Distinct-expert groups, by the whole block. A slot leads a group when no earlier slot has the same expert id and the
// same occurrence number inside its token (so an id repeated inside one token gets a group of its own); leaders are
// numbered in slot order by ballots; every slot then joins its leader's group. Ends with a block barrier.
__device__ void build_groups(const DecodeParams &p, Smem &sm, int tid) {
    const int S = p.M * p.A, A = p.A, lane = tid & 31, warp = tid >> 5;
    const int base = p.shared_mode == STRIX_SHARED_SEPARATE ? 1 : 0;
    int leader = -1;
    bool is_leader = false;
    if (tid < S) {
        const int32_t id = sm.ids[tid];
        if (id >= 0 && id < p.Estack) {
            const int m = tid / A;
            int occ = 0;
            for (int s2 = m * A; s2 < tid; ++s2) occ += sm.ids[s2] == id;
            leader = tid;
            for (int m2 = 0; m2 < m && leader == tid; ++m2) {
                int seen = 0;
                for (int a2 = 0; a2 < A; ++a2)
                    if (sm.ids[m2 * A + a2] == id) {
                        if (seen == occ) {
                            leader = m2 * A + a2;
                            break;
                        }
                        ++seen;
                    }
            }
            is_leader = leader == tid;
        }
    }
    const unsigned bal = __ballot_sync(0xffffffffu, is_leader);
    if (lane == 0) sm.leaders_before[warp] = __popc(bal);
    __syncthreads();
    if (tid == 0) {
        int run = base;
        for (int w = 0; w < kThreads / 32; ++w) {
            const int c = sm.leaders_before[w];
            sm.leaders_before[w] = run;
            run += c;
        }
        sm.n_groups = run;
        if (base) {
            Group &g = sm.groups[0];
            g.expert = -2, g.mask = ((1u << p.M) - 1u) & ~sm.failed_mask;
            for (int m = 0; m < kMaxTok; ++m) g.slot_a[m] = m < p.M ? 0 : -1;
        }
    }
    __syncthreads();
    if (is_leader) {
        const int gi = sm.leaders_before[warp] + __popc(bal & ((1u << lane) - 1u));
        sm.slot_group[tid] = (int16_t)gi;
        Group &g = sm.groups[gi];
        g.expert = sm.ids[tid], g.mask = 0;
        for (int m = 0; m < kMaxTok; ++m) g.slot_a[m] = -1;
    }
    __syncthreads();
    if (tid < S && leader >= 0) {
        Group &g = sm.groups[sm.slot_group[leader]];
        atomicOr(&g.mask, 1u << (tid / A));
        g.slot_a[tid / A] = (int8_t)(tid % A);
    }
    __syncthreads();
    if (tid < sm.n_groups) resolve_group(p, sm.groups[tid]);
    if (tid < sm.n_groups) {  // the widest stage of phase 3 (col_max starts at 1)
        const int c = __popc(sm.groups[tid].mask);
        atomicMax(&sm.col_max, c < kDnCols ? c : kDnCols);
    }
    // phase 3 work list, in group order: thread gi owns group gi's runs; positions by a scan over the first 96 threads
    {
        static_assert(kMaxGroups <= 96, "the run scan covers three warps");
        const uint32_t mk0 = tid < sm.n_groups ? sm.groups[tid].mask : 0u;
        const int runs = (__popc(mk0) + kDnCols - 1) / kDnCols;
        int incl = runs;
        if (tid < 96) {
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (lane == 31) sm.leaders_before[warp] = incl;
        }
        __syncthreads();
        if (tid < 96) {
            int first = incl - runs;
            for (int w = 0; w < warp; ++w) first += sm.leaders_before[w];
            uint32_t mk = mk0;
            for (int n = first; mk; ++n) {
                uint32_t sub = 0;
                for (int c = 0; c < kDnCols && mk; ++c) sub |= mk & (0u - mk), mk &= mk - 1;
                sm.dn_group[n] = (uint8_t)tid, sm.dn_mask[n] = (uint8_t)sub;
            }
            if (tid == 95) sm.n_dn = first + runs;
        }
    }
    __syncthreads();
}

// ---- the fused kernel ------------------------------------------------------------------------------------------------

// The copies of one gate/up stage: K slice h of the tile's 16 rows (8 gate rows, then the matching 8 up rows) into padded
// rows of the stage, and the tile's four scale / min runs (8 rows x all groups each). A half warp walks a row.
__device__ __forceinline__ void gu_issue(const DecodeParams &p, const Group &grp, int jb, int h, int nk, uint8_t *st, int rs, int sc_off,
                                         int sc_bytes, int lane) {
    const int d = p.d, I = p.I, Ks = d / nk;
    const int bits = grp.bits[0], gpr = d / grp.G[0];
    const int rb = (int)row_bytes(bits, d), lo_b = slice_lo_bytes(bits, Ks), hi_b = slice_hi_bytes(bits, Ks);
    const int lo_p = lo_b / 16, ppr = lo_p + hi_b / 16;  // 16-byte pieces per row slice
    // a half warp walks a row: rows (lane >> 4), + 2, ..; gate rows 0..7 then up rows 8..15 (I rows further)
    const uint8_t *src = grp.rows[0] + ((int64_t)jb * 8 + (lane >> 4)) * rb;
    uint8_t *dst = st + (lane >> 4) * rs;
    const int pc0 = lane & 15, hi_src = slice_lo_bytes(bits, d) + h * hi_b - lo_b;  // high-plane pieces: offset from pc * 16
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            for (int pc = pc0; pc < ppr; pc += 16) cp_async16(dst + pc * 16, src + (pc < lo_p ? h * lo_b : hi_src) + pc * 16);
            src += 2 * rb, dst += 2 * rs;
        }
        src += (int64_t)(I - 8) * rb;
    }
    const int rp = gpr;  // 16-byte pieces per run of 8 rows x gpr groups x 2 bytes
    for (int i = lane; i < 4 * rp; i += 32) {
        const int which = i / rp, pc = i - which * rp;  // 0 gate scale, 1 gate min, 2 up scale, 3 up min
        const int r0 = (which & 2) ? I + jb * 8 : jb * 8;
        const uint8_t *src = reinterpret_cast<const uint8_t *>(((which & 1) ? grp.minv[0] : grp.scale[0]) + (int64_t)r0 * gpr);
        cp_async16(st + sc_off + which * sc_bytes + pc * 16, src + pc * 16);
    }
}

// The copies of one down stage: 16 consecutive output rows of the group's expert, their scale / min runs, and the h records
// of the tokens routed to it (ascending token order).
__device__ __forceinline__ void dn_issue(const DecodeParams &p, const Group &grp, uint32_t tokens, int nb, uint8_t *st, int rs, int sc_off,
                                         int sc_bytes, int col_off, int lane) {
    const int I = p.I, M = p.M, A = p.A;
    const int bits = grp.bits[1], gpr = I / grp.G[1];
    const int rb = (int)row_bytes(bits, I), ppr = rb / 16;
    for (int r = lane >> 4; r < 16; r += 2) {
        const uint8_t *src = grp.rows[1] + ((int64_t)nb * 16 + r) * rb;
        for (int pc = lane & 15; pc < ppr; pc += 16) cp_async16(st + r * rs + pc * 16, src + pc * 16);
    }
    const int rp = 2 * gpr;  // 16 rows x gpr groups x 2 bytes
    for (int i = lane; i < 2 * rp; i += 32) {
        const int which = i / rp, pc = i - which * rp;
        const uint8_t *src = reinterpret_cast<const uint8_t *>((which ? grp.minv[1] : grp.scale[1]) + (int64_t)nb * 16 * gpr);
        cp_async16(st + sc_off + which * sc_bytes + pc * 16, src + pc * 16);
    }
    const int cp_n = p.hrec_bytes / 16;
    int ci = 0;
    for (uint32_t mk = tokens; mk; mk &= mk - 1, ++ci) {
        const int m = __ffs(mk) - 1;
        const int slot_i = grp.expert == -2 ? M * A + m : m * A + grp.slot_a[m];
        const uint8_t *src = p.hrec + (int64_t)slot_i * p.hrec_bytes;
        for (int pc = lane; pc < cp_n; pc += 32) cp_async16(st + col_off + ci * p.hrec_bytes + pc * 16, src + pc * 16);
    }
}

// by_bits over the formats a kernel variant was compiled for (bit 0: 4 bits, 1: 5, 2: 6, 3: 8): the variants for uniform
// 4-bit experts carry a quarter of the code of the general one, which the instruction cache rewards.
template <int FMASK, typename F>
__device__ __forceinline__ void by_bits_in(int bits, F &&f) {
    if constexpr (FMASK == 0x1) {
        f(std::integral_constant<int, 4>{});
    } else if constexpr (FMASK == 0x9) {
        if (bits == 4) f(std::integral_constant<int, 4>{});
        else f(std::integral_constant<int, 8>{});
    } else {
        by_bits(bits, f);
    }
}

// G128: every 4-bit projection has groups of 128 codes (its unrolled group loop is the only one compiled for 4 bits; other
// formats run the general loop).
// ONEPASS: the MMA columns hold every token in one pass (BF16 activations, or at most 4 FP32 tokens).
template <typename T, int FMASK, bool G128, bool ONEPASS>
__global__ void __launch_bounds__(kThreads, 1) decode_fused_kernel(const __grid_constant__ DecodeParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int planes = sizeof(T) == 4 ? 2 : 1;
    const int M = p.M, d = p.d, I = p.I, A = p.A;
    const T *x = static_cast<const T *>(p.x);
    uint32_t *counters = p.sync;  // [0], [1]: the two barriers; [2]: CTAs done; [3]: abort

    // Permuted BF16 planes of x: token m at xp + m * tok_stride, plane 1 behind plane 0; unit u (8 values) = 16 bytes holding
    // the pairs (0,4) (1,5) (2,6) (3,7) - the k order the unpacked weight words have.
    const int plane_bytes_x = d * 2, tok_stride = planes * plane_bytes_x + 64;
    uint8_t *xp = smem_raw + ((sizeof(Smem) + 127) & ~127);
    // plane sums of x over aligned runs of 32, 64 and 128 values: [M][planes][d/32 | d/64 | d/128] (a quantization group's sum is one load)
    float *xsum = reinterpret_cast<float *>(xp + M * tok_stride);
    const int nchunk_x = d / 32, xs_row = nchunk_x + nchunk_x / 2 + nchunk_x / 4;
    uint8_t *stage_base = smem_raw + ((((uint8_t *)(xsum + M * planes * xs_row) - smem_raw) + 127) & ~127);
    float *xf = reinterpret_cast<float *>(stage_base);  // phases 0-1: x as FP32 [M][d], where the stages will be

    if (tid == 0) sm.abort_flag = 0, sm.failed_mask = 0, sm.n_groups = 0, sm.col_max = 1;
    stamp(p.sync, 0);

    // Phase 0: x -> FP32 copy, permuted planes, per-plane chunk sums.
    for (int base = warp * 32; base < M * (d / 8); base += kThreads) {  // warp-uniform trips: the shuffles need whole warps
        const int i = base + lane;
        const bool valid = i < M * (d / 8);
        const int m = valid ? i / (d / 8) : 0, u = valid ? i % (d / 8) : 0;
        float v[8];
        if (valid) {
            if constexpr (sizeof(T) == 4) {
                const float4 a = *reinterpret_cast<const float4 *>(x + (int64_t)m * d + u * 8), b = *reinterpret_cast<const float4 *>(x + (int64_t)m * d + u * 8 + 4);
                v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
            } else {
                const uint4 q = *reinterpret_cast<const uint4 *>(x + (int64_t)m * d + u * 8);
                const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) v[2 * j] = __uint_as_float(w4[j] << 16), v[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
        }
        uint16_t hi[8], lo[8];
        float s_hi = 0.f, s_lo = 0.f;  // sums of what the tensor cores will see, so that the "+128" offset cancels exactly
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            hi[j] = f32_to_bf16_bits(v[j]);
            lo[j] = planes == 2 ? f32_to_bf16_bits(v[j] - bf16_bits_to_f32(hi[j])) : (uint16_t)0;
            s_hi += bf16_bits_to_f32(hi[j]), s_lo += bf16_bits_to_f32(lo[j]);
        }
        if (valid) {
            const bool rot = p.router_kind == STRIX_ROUTER_Q;
            *reinterpret_cast<float4 *>(xf + m * d + (rot ? xf_index(u * 8) : u * 8)) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(xf + m * d + (rot ? xf_index(u * 8 + 4) : u * 8 + 4)) = make_float4(v[4], v[5], v[6], v[7]);
            uint4 h4;
            h4.x = hi[0] | ((uint32_t)hi[4] << 16), h4.y = hi[1] | ((uint32_t)hi[5] << 16), h4.z = hi[2] | ((uint32_t)hi[6] << 16), h4.w = hi[3] | ((uint32_t)hi[7] << 16);
            *reinterpret_cast<uint4 *>(xp + m * tok_stride + u * 16) = h4;
            if (planes == 2) {
                uint4 l4;
                l4.x = lo[0] | ((uint32_t)lo[4] << 16), l4.y = lo[1] | ((uint32_t)lo[5] << 16), l4.z = lo[2] | ((uint32_t)lo[6] << 16), l4.w = lo[3] | ((uint32_t)lo[7] << 16);
                *reinterpret_cast<uint4 *>(xp + m * tok_stride + plane_bytes_x + u * 16) = l4;
            }
        }
        // the 32-code chunk = 4 consecutive units = 4 consecutive lanes
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1), s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1);
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2), s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
        if (valid && (u & 3) == 0) {
            xsum[(m * planes) * xs_row + u / 4] = s_hi;
            if (planes == 2) xsum[(m * planes + 1) * xs_row + u / 4] = s_lo;
        }
    }
    __syncthreads();
    for (int i = tid; i < M * planes * (nchunk_x / 2); i += kThreads) {  // runs of 64
        float *row = xsum + (i / (nchunk_x / 2)) * xs_row;
        const int j = i % (nchunk_x / 2);
        row[nchunk_x + j] = row[2 * j] + row[2 * j + 1];
    }
    __syncthreads();
    for (int i = tid; i < M * planes * (nchunk_x / 4); i += kThreads) {  // runs of 128
        float *row = xsum + (i / (nchunk_x / 4)) * xs_row;
        const int j = i % (nchunk_x / 4);
        row[nchunk_x + nchunk_x / 2 + j] = row[nchunk_x + 2 * j] + row[nchunk_x + 2 * j + 1];
    }
    __syncthreads();
    stamp(p.sync, 1);

    // Phase 1: router logits; warps 2i, 2i+1 share row (block * pairs + i).
    {
        constexpr int pairs = CW / 2;
        for (int r0 = blockIdx.x * pairs; r0 < p.R; r0 += gridDim.x * pairs) {
            const int r = r0 + (warp >> 1);
            float acc[kMaxTok];
            const bool mine = warp < 2 * pairs && r < p.R;
            if (mine) {
                router_half_row(p, xf, r, warp & 1, lane, acc);
#pragma unroll
                for (int m = 0; m < kMaxTok; ++m) {
                    if (m < M) {
                        const float v = warp_sum(acc[m]);
                        if (lane == 0) sm.rpart[warp][m] = v;
                    }
                }
            }
            __syncthreads();
            if (mine && (warp & 1) == 0 && lane < M) {
                float v = sm.rpart[warp][lane] + sm.rpart[warp + 1][lane];
                if (p.router_bias != nullptr && r < p.E) v += p.router_bias[r];
                p.logits[(int64_t)lane * p.R + r] = v;
            }
            __syncthreads();
        }
    }
    stamp(p.sync, 2);
    grid_arrive(&counters[0]);
    if (!grid_wait(&counters[0], &counters[3], sm)) goto abort;
    stamp(p.sync, 3);

    // Phase 2a: routing (one warp per token), groups.
    if (warp < M) {
        if (p.E <= 512) route_token<16>(p, sm, warp, lane, blockIdx.x == 0);
        else route_token<32>(p, sm, warp, lane, blockIdx.x == 0);
    }
    __syncthreads();
    build_groups(p, sm, tid);
    stamp(p.sync, 4);

    {
        // ---- phase 2b: gate/up tiles. Tile t = (group, block of 8 row pairs); its K is cut in nk slices, a stage each,
        //      consumed by the nk warps of a team: stage it = tile_local * nk + h goes to consumer warp it % active. ----
        const int NG = sm.n_groups;
        const int nk = p.gu_nk, Ks = d / nk;
        const int tiles_per_group = I / 8, n_tiles = NG * tiles_per_group;
        const int rs = p.gu_row_stride, sc_off = 16 * rs, sc_bytes = p.gu_scale_bytes, stage_bytes = p.gu_stage_bytes;
        const int D = p.gu_depth;  // stages per warp
        int n_local = 0;  // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ..
        if ((int)blockIdx.x < n_tiles) n_local = (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1;
        {
            const int cw = warp, g = lane >> 2, c = lane & 3;
            const int h = cw % nk, team = cw / nk, n_teams = CW / nk;
            uint8_t *my_stages = stage_base + (size_t)cw * D * stage_bytes;
            // the warp's n-th stage is slice h of tile team + n * n_teams; copies run D stages ahead of the math
            auto issue = [&](int n) {
                const int tl = team + n * n_teams;
                if (tl < n_local) {
                    const int t = (int)blockIdx.x + tl * (int)gridDim.x;
                    const int gi = t / tiles_per_group;
                    gu_issue(p, sm.groups[gi], t - gi * tiles_per_group, h, nk, my_stages + (size_t)(n % D) * stage_bytes, rs, sc_off, sc_bytes, lane);
                }
                cp_async_commit();  // one group per stage, empty past the end: the wait below counts groups
            };
            for (int n = 0; n < D; ++n) issue(n);
            int n = 0;
            for (int tl = team; tl < n_local; tl += n_teams, ++n) {
                cp_async_wait(D - 1);
                __syncwarp();
                const int t = (int)blockIdx.x + tl * (int)gridDim.x;
                const int gi = t / tiles_per_group, jb = t - gi * tiles_per_group;
                const Group &grp = sm.groups[gi];
                const int np = (!ONEPASS && planes == 2 && (grp.mask >> 4)) ? 2 : 1;  // token passes
                float tot[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                {
                    const int G = grp.G[0], gpr = d / G, gl = gpr / nk;  // groups per row, per slice
                    const uint8_t *st = my_stages + (size_t)(n % D) * stage_bytes;
                    const uint8_t *rowA = st + g * rs, *rowB = st + (g + 8) * rs;  // gate row g, up row g
                    const uint16_t *scA = reinterpret_cast<const uint16_t *>(st + sc_off) + g * gpr + h * gl;
                    const uint16_t *mnA = reinterpret_cast<const uint16_t *>(st + sc_off + sc_bytes) + g * gpr + h * gl;
                    const uint16_t *scB = reinterpret_cast<const uint16_t *>(st + sc_off + 2 * sc_bytes) + g * gpr + h * gl;
                    const uint16_t *mnB = reinterpret_cast<const uint16_t *>(st + sc_off + 3 * sc_bytes) + g * gpr + h * gl;
                    // this lane's B column (MMA column g) and the chunk sums of its two accumulator columns (2c, 2c + 1), per pass
                    const uint8_t *xb[2] = {nullptr, nullptr};
                    const float *xsp[2][2] = {{nullptr, nullptr}, {nullptr, nullptr}};
#pragma unroll
                    for (int ps = 0; ps < 2; ++ps) {
                        int tk, pl;
                        column_of<planes>(g, ps, tk, pl);
                        if (ps < np && tk < M && (grp.mask >> tk & 1u)) xb[ps] = xp + tk * tok_stride + pl * plane_bytes_x + h * (Ks / 8) * 16;
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            column_of<planes>(2 * c + e, ps, tk, pl);
                            if (ps < np && tk < M) xsp[ps][e] = xsum + (tk * planes + pl) * xs_row + (G == 32 ? 0 : G == 64 ? nchunk_x : nchunk_x + nchunk_x / 2) + h * gl;
                        }
                    }
                    by_bits_in<FMASK>(grp.bits[0], [&](auto bc) {
                        constexpr int BITS = decltype(bc)::value;
                        for (int qg = 0; qg < gl; ++qg) {
                            float xs[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
                            for (int ps = 0; ps < 2; ++ps)
#pragma unroll
                                for (int e = 0; e < 2; ++e)
                                    if (xsp[ps][e]) xs[ps][e] = xsp[ps][e][qg];
                            const float sA = bf16_bits_to_f32(scA[qg]), mA = bf16_bits_to_f32(mnA[qg]), sB = bf16_bits_to_f32(scB[qg]), mB = bf16_bits_to_f32(mnB[qg]);
                            if (ONEPASS || np == 1) {
                                const uint8_t *const xb1[1] = {xb[0]};
                                const float xs1[1][2] = {{xs[0][0], xs[0][1]}};
                                float t1[1][4] = {{0.f, 0.f, 0.f, 0.f}};
                                if constexpr (G128 && BITS == 4) group_dot<BITS, 1, 4>(rowA, rowB, Ks, xb1, qg * 16, 4, c, sA, mA, sB, mB, xs1, t1);
                                else if constexpr (G128) group_dot<BITS, 1, 0>(rowA, rowB, Ks, xb1, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs1, t1);
                                else if (G == 128) group_dot<BITS, 1, 4>(rowA, rowB, Ks, xb1, qg * 16, 4, c, sA, mA, sB, mB, xs1, t1);
                                else group_dot<BITS, 1, 0>(rowA, rowB, Ks, xb1, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs1, t1);
#pragma unroll
                                for (int i = 0; i < 4; ++i) tot[0][i] += t1[0][i];
                            } else if constexpr (!ONEPASS) {
                                const uint8_t *const xb2[2] = {xb[0], xb[1]};
                                if constexpr (G128 && BITS == 4) group_dot<BITS, 2, 4>(rowA, rowB, Ks, xb2, qg * 16, 4, c, sA, mA, sB, mB, xs, tot);
                                else if constexpr (G128) group_dot<BITS, 2, 0>(rowA, rowB, Ks, xb2, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs, tot);
                                else if (G == 128) group_dot<BITS, 2, 4>(rowA, rowB, Ks, xb2, qg * 16, 4, c, sA, mA, sB, mB, xs, tot);
                                else group_dot<BITS, 2, 0>(rowA, rowB, Ks, xb2, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs, tot);
                            }
                        }
                    });
                    __syncwarp();      // every lane is done with the stage
                    issue(n + D);      // refill it while the tile is finished
                }
                // the team's slices meet in its leader (h == 0): ordered sum, then the SwiGLU, lane-local
                const int par = n & 1;
                if (nk > 1) {
                    if (h != 0) {
                        float4 *dst = reinterpret_cast<float4 *>(&sm.red[par][cw][lane][0]);
                        dst[0] = make_float4(tot[0][0], tot[0][1], tot[0][2], tot[0][3]);
                        if (np == 2) dst[1] = make_float4(tot[1][0], tot[1][1], tot[1][2], tot[1][3]);
                    }
                    named_sync(1 + team, nk * 32);
                    if (h == 0) {
                        for (int w = 1; w < nk; ++w) {
                            const float4 *o = reinterpret_cast<const float4 *>(&sm.red[par][cw + w][lane][0]);
                            const float4 o0 = o[0];
                            tot[0][0] += o0.x, tot[0][1] += o0.y, tot[0][2] += o0.z, tot[0][3] += o0.w;
                            if (np == 2) {
                                const float4 o1 = o[1];
                                tot[1][0] += o1.x, tot[1][1] += o1.y, tot[1][2] += o1.z, tot[1][3] += o1.w;
                            }
                        }
                    }
                }
                if (h == 0 && !sm.abort_flag) {
                    T *hh = static_cast<T *>(p.hh);
                    for (int ps = 0; ps < np; ++ps) {
                        // FP32 activations: the two planes of a token sit in lanes c and c ^ 2
                        if (planes == 2) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) tot[ps][i] += __shfl_xor_sync(0xffffffffu, tot[ps][i], 2);
                        }
                        // tot[ps][e]: gate row jb*8+g, tot[ps][2+e]: the up row, for the token of column 2c + e
                        float part_hi[2], part_lo[2];
                        int slot_of[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            int tok, pl;
                            column_of<planes>(2 * c + e, ps, tok, pl);
                            const bool live = pl == 0 && tok < M && (grp.mask >> tok & 1u);
                            const float gs = as_stored(tot[ps][e], hh), us = as_stored(tot[ps][2 + e], hh);
                            const float hv = as_stored(as_stored(__fdividef(gs, 1.0f + __expf(-gs)), hh) * us, hh);
                            const uint16_t hb = f32_to_bf16_bits(hv);
                            const uint16_t hl = planes == 2 ? f32_to_bf16_bits(hv - bf16_bits_to_f32(hb)) : (uint16_t)0;
                            part_hi[e] = live ? bf16_bits_to_f32(hb) : 0.f, part_lo[e] = live ? bf16_bits_to_f32(hl) : 0.f;
                            slot_of[e] = -1;
                            if (live) {
                                const int slot_i = grp.expert == -2 ? M * A + tok : tok * A + grp.slot_a[tok];
                                slot_of[e] = slot_i;
                                if (grp.expert != -2) st_act(hh, (int64_t)slot_i * I + jb * 8 + g, hv);
                                else if (p.sh_h != nullptr) st_act(static_cast<T *>(p.sh_h), (int64_t)tok * I + jb * 8 + g, hv);
                                // the record phase 3 streams: planes of permuted BF16 pairs, then per plane I / 8 partial sums
                                uint8_t *rec = p.hrec + (int64_t)slot_i * p.hrec_bytes;
                                const int off = jb * 16 + (g & 3) * 4 + (g >> 2) * 2;
                                *reinterpret_cast<uint16_t *>(rec + off) = hb;
                                if (planes == 2) *reinterpret_cast<uint16_t *>(rec + I * 2 + off) = hl;
                            }
                        }
                        // sums over the tile's 8 rows (lanes with equal c): what the down projection's min term needs
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
#pragma unroll
                            for (int o = 4; o <= 16; o <<= 1) {
                                part_hi[e] += __shfl_xor_sync(0xffffffffu, part_hi[e], o);
                                if (planes == 2) part_lo[e] += __shfl_xor_sync(0xffffffffu, part_lo[e], o);
                            }
                            if (g == 0 && slot_of[e] >= 0) {
                                float *pp = reinterpret_cast<float *>(p.hrec + (int64_t)slot_of[e] * p.hrec_bytes + planes * I * 2);
                                pp[jb] = part_hi[e];
                                if (planes == 2) pp[I / 8 + jb] = part_lo[e];
                            }
                        }
                    }
                }
            }
        }
    }
    cp_async_wait(0);
    stamp(p.sync, 5);
    // the h records written above are read by other CTAs after the barrier
    grid_arrive(&counters[1]);
    if (!grid_wait(&counters[1], &counters[3], sm)) goto abort;
    stamp(p.sync, 6);

    {
        // ---- phase 3: down projection + combine. The x planes are dead: stages take the whole dynamic area. ----
        const int NG = sm.n_dn;  // work items: (group, run of its tokens)
        uint8_t *st3 = xp;
        const int avail3 = p.smem_bytes - (int)(xp - smem_raw);
        const int rs = p.dn_row_stride, sc_off = 16 * rs, sc_bytes = p.dn_scale_bytes;
        const int col_off = p.dn_stage_bytes_fixed;
        const int stage_bytes = (col_off + sm.col_max * p.hrec_bytes + 127) & ~127;
        // warps in use and stages per warp: all CW warps when a stage each fits, fewer (deeper is never needed then) otherwise
        int ACT = avail3 / stage_bytes;
        ACT = ACT > CW ? CW : ACT;
        if (ACT < 1) {
            if (tid == 0) sm.abort_flag = 0x106;
            __syncthreads();
            goto abort;
        }
        int D = avail3 / (stage_bytes * ACT);
        D = D > kMaxDepth ? kMaxDepth : D;
        const int n_blocks = d / 16;
        int nb_local = 0;
        if ((int)blockIdx.x < n_blocks) nb_local = (n_blocks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1;
        const int part_off = planes * I * 2;  // the partial sums inside an h record
        for (int i = tid; i < 2 * 32 * 8; i += kThreads) (&sm.red_sh[0][0][0])[i] = 0.f;  // the shared expert's tile is summed by atomic adds
        __syncthreads();
        {
            const int cw = warp, g = lane >> 2, c = lane & 3;
            uint8_t *my_stages = st3 + (size_t)cw * D * stage_bytes;
            // stages are numbered it = nbi * NG + gi over this CTA's row blocks; the warp takes it = cw, cw + ACT, ..
            const int n_total = cw < ACT ? nb_local * NG : 0;
            auto issue = [&](int n) {
                const int it = cw + n * ACT;
                if (it < n_total) {
                    const int nbi = it / NG;
                    const int ii = it - nbi * NG;
                    dn_issue(p, sm.groups[sm.dn_group[ii]], sm.dn_mask[ii], (int)blockIdx.x + nbi * (int)gridDim.x,
                             my_stages + (size_t)(n % D) * stage_bytes, rs, sc_off, sc_bytes, col_off, lane);
                }
                cp_async_commit();
            };
            for (int n = 0; n < D; ++n) issue(n);
            int n = 0;
            for (int nbi = 0; nbi < nb_local; ++nbi) {
                const int nb = (int)blockIdx.x + nbi * (int)gridDim.x;
                float tot[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                for (int it = cw + n * ACT; cw < ACT && it < (nbi + 1) * NG; it += ACT, ++n) {
                    cp_async_wait(D - 1);
                    __syncwarp();
                    const int slot = n % D;
                    const Group &grp = sm.groups[sm.dn_group[it - nbi * NG]];
                    const uint32_t gmask = sm.dn_mask[it - nbi * NG];  // the tokens of this stage
                    const int G = grp.G[1], gpr = I / G;
                    const uint8_t *st = my_stages + (size_t)slot * stage_bytes;
                    const uint8_t *rowA = st + g * rs, *rowB = st + (g + 8) * rs;
                    const uint16_t *sc = reinterpret_cast<const uint16_t *>(st + sc_off), *mn = reinterpret_cast<const uint16_t *>(st + sc_off + sc_bytes);
                    const int np = (!ONEPASS && planes == 2 && (gmask >> 4)) ? 2 : 1;
                    const bool is_sh = grp.expert == -2;
                    float sh_stage[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    const uint8_t *xb[2] = {nullptr, nullptr};
                    const float *hp[2][2] = {{nullptr, nullptr}, {nullptr, nullptr}};
                    float cf[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
                    for (int ps = 0; ps < 2; ++ps) {
                        int tk, pl;
                        column_of<planes>(g, ps, tk, pl);
                        if (ps < np && tk < M && (gmask >> tk & 1u))
                            xb[ps] = st + col_off + __popc(gmask & ((1u << tk) - 1u)) * p.hrec_bytes + pl * I * 2;
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            column_of<planes>(2 * c + e, ps, tk, pl);
                            if (ps < np && tk < M && (gmask >> tk & 1u)) {
                                hp[ps][e] = reinterpret_cast<const float *>(st + col_off + __popc(gmask & ((1u << tk) - 1u)) * p.hrec_bytes + part_off) + pl * (I / 8);
                                cf[ps][e] = is_sh ? 1.f : sm.coef[tk * A + grp.slot_a[tk]];  // the shared expert's gate comes after its own rounding
                            }
                        }
                    }
                    by_bits_in<FMASK>(grp.bits[1], [&](auto bc) {
                        constexpr int BITS = decltype(bc)::value;
                        for (int qg = 0; qg < gpr; ++qg) {
                            float xs[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
                            for (int ps = 0; ps < 2; ++ps)
#pragma unroll
                                for (int e = 0; e < 2; ++e)
                                    if (hp[ps][e]) {
                                        const float4 *v4 = reinterpret_cast<const float4 *>(hp[ps][e] + qg * (G / 8));
                                        float a = 0.f;
                                        for (int u = 0; u < G / 32; ++u) {
                                            const float4 f = v4[u];
                                            a += (f.x + f.y) + (f.z + f.w);
                                        }
                                        xs[ps][e] = a;
                                    }
                            const float sA = bf16_bits_to_f32(sc[g * gpr + qg]), mA = bf16_bits_to_f32(mn[g * gpr + qg]);
                            const float sB = bf16_bits_to_f32(sc[(g + 8) * gpr + qg]), mB = bf16_bits_to_f32(mn[(g + 8) * gpr + qg]);
                            float v[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                            if (ONEPASS || np == 1) {
                                const uint8_t *const xb1[1] = {xb[0]};
                                const float xs1[1][2] = {{xs[0][0], xs[0][1]}};
                                float t1[1][4] = {{0.f, 0.f, 0.f, 0.f}};
                                if constexpr (G128 && BITS == 4) group_dot<BITS, 1, 4>(rowA, rowB, I, xb1, qg * 16, 4, c, sA, mA, sB, mB, xs1, t1);
                                else if constexpr (G128) group_dot<BITS, 1, 0>(rowA, rowB, I, xb1, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs1, t1);
                                else if (G == 128) group_dot<BITS, 1, 4>(rowA, rowB, I, xb1, qg * 16, 4, c, sA, mA, sB, mB, xs1, t1);
                                else group_dot<BITS, 1, 0>(rowA, rowB, I, xb1, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs1, t1);
#pragma unroll
                                for (int i = 0; i < 4; ++i) v[0][i] = t1[0][i];
                            } else if constexpr (!ONEPASS) {
                                const uint8_t *const xb2[2] = {xb[0], xb[1]};
                                if constexpr (G128 && BITS == 4) group_dot<BITS, 2, 4>(rowA, rowB, I, xb2, qg * 16, 4, c, sA, mA, sB, mB, xs, v);
                                else if constexpr (G128) group_dot<BITS, 2, 0>(rowA, rowB, I, xb2, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs, v);
                                else if (G == 128) group_dot<BITS, 2, 4>(rowA, rowB, I, xb2, qg * 16, 4, c, sA, mA, sB, mB, xs, v);
                                else group_dot<BITS, 2, 0>(rowA, rowB, I, xb2, qg * (G / 8), G / 32, c, sA, mA, sB, mB, xs, v);
                            }
#pragma unroll
                            for (int ps = 0; ps < 2; ++ps) {
                                if (is_sh) {
                                    sh_stage[ps][0] += v[ps][0], sh_stage[ps][1] += v[ps][1], sh_stage[ps][2] += v[ps][2], sh_stage[ps][3] += v[ps][3];
                                } else {
                                    tot[ps][0] = fmaf(cf[ps][0], v[ps][0], tot[ps][0]), tot[ps][1] = fmaf(cf[ps][1], v[ps][1], tot[ps][1]);
                                    tot[ps][2] = fmaf(cf[ps][0], v[ps][2], tot[ps][2]), tot[ps][3] = fmaf(cf[ps][1], v[ps][3], tot[ps][3]);
                                }
                            }
                        }
                    });
                    __syncwarp();
                    issue(n + D);
                    if (is_sh) {
                        // the shared expert's runs cover disjoint tokens = disjoint accumulator columns: every word of the tile gets
                        // one non-zero addend (the others add 0), so the sum does not depend on the order of the adds
                        float *dst = &sm.red_sh[nbi & 1][lane][0];
#pragma unroll
                        for (int i = 0; i < 4; ++i) atomicAdd(dst + i, sh_stage[0][i]), atomicAdd(dst + 4 + i, sh_stage[1][i]);
                    }
                }
                const int par = nbi & 1;
                {
                    float4 *dst = reinterpret_cast<float4 *>(&sm.red[par][cw][lane][0]);
                    dst[0] = make_float4(tot[0][0], tot[0][1], tot[0][2], tot[0][3]);
                    dst[1] = make_float4(tot[1][0], tot[1][1], tot[1][2], tot[1][3]);
                }
                named_sync(1, CW * 32);
                const int ct = tid;
                if (ct < 128 && !sm.abort_flag) {
                    const int r = ct >> 3, tok = ct & 7;  // output row nb * 16 + r, token tok
                    if (tok < M) {
                        // the token's column(s): FP32 - column tok & 3 (high plane) and + 4 (low plane) of pass tok >> 2
                        const int ps = planes == 2 ? tok >> 2 : 0, col = planes == 2 ? tok & 3 : tok;
                        const int ln = 4 * (r & 7) + (col >> 1), rg = ps * 4 + (r >> 3) * 2 + (col & 1);
                        float v = 0.f;
#pragma unroll
                        for (int w = 0; w < CW; ++w) {
                            v += sm.red[par][w][ln][rg];
                            if (planes == 2) v += sm.red[par][w][ln + 2][rg];
                        }
                        T *y = static_cast<T *>(p.y);
                        if (p.shared_mode == STRIX_SHARED_SEPARATE) {  // y = stored(routed) + gate * stored(shared), as moe_shared_add
                            float sv = sm.red_sh[par][ln][rg];
                            sm.red_sh[par][ln][rg] = 0.f;  // read by this thread only: clean for the row block after next
                            if (planes == 2) sv += sm.red_sh[par][ln + 2][rg], sm.red_sh[par][ln + 2][rg] = 0.f;
                            v = as_stored(v, y) + sm.gate[tok] * as_stored(sv, y);
                        }
                        if (sm.failed_mask >> tok & 1u) v = qnan();
                        st_act(y, (int64_t)tok * d + nb * 16 + r, v);
                    }
                }
            }
        }
    }

    // The last CTA out zeroes the barrier words for the next launch.
    cp_async_wait(0);
    __syncthreads();
    stamp(p.sync, 7);
    if (sm.abort_flag) goto abort;
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&counters[2], 1u) == gridDim.x - 1) {
            counters[0] = 0, counters[1] = 0, counters[2] = 0;
            __threadfence();
        }
    }
    return;

abort:
    // A wait ran out somewhere in the grid. Tell the others, report once, and leave; outstanding bulk copies target this
    // CTA's own shared memory only: sleep (bounded) until any copy issued has certainly landed before the block retires.
    __syncthreads();
    if (tid == 0) {
        atomicExch(&counters[3], 1u);
        if (sm.abort_flag != 0x200 && atomicCAS(&p.err[3], 0u, 2u) == 0u) p.err[4] = 0xdec000u | (uint32_t)sm.abort_flag, p.err[5] = blockIdx.x;
        for (uint32_t i = 0; i < (1u << 14); ++i) __nanosleep(200);
    }
    __syncthreads();
}

}  // namespace

namespace sb {

int decode_fused_plan(DecodeParams &p, int max_bits_gate_up, int max_bits_down, int min_G) {
    if (p.M < 1 || p.M > kMaxTok) return 0;
    if (p.d % 256 != 0 || p.I % 128 != 0 || p.d > 16384 || p.I > 16384) return 0;
    if (p.E > 1024 || p.k > 32 || p.A > 64 || p.M * p.A > kMaxSlots) return 0;
    int dev = 0, max_smem = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    const int planes = p.act == kF32 ? 2 : 1;
    p.smem_bytes = max_smem;
    p.hrec_bytes = planes * (p.I * 2 + (p.I / 8) * 4);
    const int fixed = (int)((sizeof(Smem) + 127) & ~127) + p.M * (planes * p.d * 2 + 64) + p.M * planes * (p.d / 32 + p.d / 64 + p.d / 128) * 4 + 256;
    if (fixed + p.M * p.d * 4 > max_smem) return 0;  // the FP32 copy of x lives where the stages will be
    // K slices per gate/up tile (1, 2 or 4: a divisor of the warp count): the fewest that give every warp two stages of its
    // own, else the deepest; slices stay multiples of 128 codes (16-byte pieces of both code planes).
    p.gu_scale_bytes = 8 * (p.d / min_G) * 2;
    int best_nk = 0, best_depth = 0;
    for (int nk = 1; nk <= 4; nk *= 2) {
        const int Ks = p.d / nk;
        if (Ks % 128 != 0) break;
        const int stride = slice_lo_bytes(max_bits_gate_up, Ks) + slice_hi_bytes(max_bits_gate_up, Ks) + 16;
        const int stage = (16 * stride + 4 * p.gu_scale_bytes + 127) & ~127;
        int depth = (max_smem - fixed) / (stage * CW);
        if (depth > kMaxDepth) depth = kMaxDepth;
        if (depth > best_depth) best_depth = depth, best_nk = nk;
        if (depth >= 2) break;
    }
    if (best_nk == 0 || best_depth < 1) return 0;
    p.gu_nk = best_nk;
    const int Ks = p.d / best_nk;
    p.gu_row_stride = slice_lo_bytes(max_bits_gate_up, Ks) + slice_hi_bytes(max_bits_gate_up, Ks) + 16;
    p.gu_stage_bytes = (16 * p.gu_row_stride + 4 * p.gu_scale_bytes + 127) & ~127;
    p.gu_active = CW, p.gu_depth = best_depth, p.gu_stages = CW * best_depth;
    p.dn_row_stride = (int)row_bytes(max_bits_down, p.I) + 16;
    p.dn_scale_bytes = (16 * (p.I / min_G) * 2 + 15) & ~15;
    p.dn_stage_bytes_fixed = 16 * p.dn_row_stride + 2 * p.dn_scale_bytes;
    const int dn_stage_worst = (p.dn_stage_bytes_fixed + p.M * p.hrec_bytes + 127) & ~127;
    const int dn_avail = max_smem - (int)((sizeof(Smem) + 127) & ~127) - 128;
    return dn_avail / dn_stage_worst >= 1;
}

int decode_fused_launch(const char *fn, const DecodeParams &p, cudaStream_t stream) {
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev), fn);
    // the expert formats present (fmask), whether every group has 128 codes, and whether one MMA pass covers the tokens pick the
    // smallest kernel variant that covers the call: a quarter of the general kernel's code for uniform 4-bit G = 128 experts
    const bool one_pass = p.act != kF32 || p.M <= 4;
    const int fm = !p.g128_4bit ? 2 : (p.fmask & ~0x1) == 0 ? 0 : (p.fmask & ~0x9) == 0 ? 1 : 2;
    const int variant = fm == 2 ? 4 : fm * 2 + (one_pass ? 0 : 1);
    using KernelFn = void (*)(const DecodeParams);
    static const KernelFn kernels[2][5] = {
        {decode_fused_kernel<float, 0x1, true, true>, decode_fused_kernel<float, 0x1, true, false>, decode_fused_kernel<float, 0x9, true, true>,
         decode_fused_kernel<float, 0x9, true, false>, decode_fused_kernel<float, 0xF, false, false>},
        {decode_fused_kernel<uint16_t, 0x1, true, true>, decode_fused_kernel<uint16_t, 0x1, true, true>, decode_fused_kernel<uint16_t, 0x9, true, true>,
         decode_fused_kernel<uint16_t, 0x9, true, true>, decode_fused_kernel<uint16_t, 0xF, false, false>}};
    static thread_local int prepared_dev = -1;
    if (prepared_dev != dev) {
        for (int a = 0; a < 2; ++a)
            for (int v = 0; v < 5; ++v) SB_CUDA(cudaFuncSetAttribute(kernels[a][v], cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes), fn);
        prepared_dev = dev;
    }
    const int grid = sm_count();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = (size_t)p.smem_bytes, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    SB_CUDA(cudaLaunchKernelEx(&cfg, kernels[p.act == kF32 ? 0 : 1][variant], p), fn, ": launching the fused decode kernel");
    return 0;
}

}  // namespace sb
