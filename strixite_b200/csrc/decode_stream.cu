// The whole MoE sublayer for a handful of tokens (decode, speculative verify: M <= 8) as ONE persistent kernel that
// streams every distinct active expert's packed weights exactly once, straight from HBM into registers.
//
// Design (one CTA per SM, 16 warps of up to 128 registers, no shared-memory staging of weights):
//   * A warp owns a 16-row tile of one expert over a range of 128-code chunks of K. Each lane issues 128-bit loads of the
//     packed codes of "its" two rows (MMA rows g and g + 8) several chunks ahead of the arithmetic, so a CTA keeps ~64 KB of
//     loads in flight with nothing but registers; the loads bypass L1.
//   * The dot products run on the tensor cores as a data-movement device: mma.sync m16n8k16 F16 takes 16 weight rows x 16
//     codes against 8 columns (the tokens), so one unpack of a weight word serves every token. Codes become EXACT F16
//     values with one AND each: an integer below 1024 in the low bits of an F16 is the subnormal code * 2^-24, which the
//     tensor cores take at full precision (odd nibbles stay four bits up: code * 2^-20, in an accumulator of their own);
//     the accumulators hold sum(x * code) in FP32, and the group's scale (carrying the power of two) and minimum are
//     applied once per 128 codes: s * sum(x * code) + m * sum(x) - the reference's arithmetic form (strixite
//     kernels/linear_q4.hip:88-94).
//   * K inside an MMA may be permuted freely as long as both operands agree, so a lane's 32 consecutive codes feed its own
//     fragments with no shuffles; activations are staged once per CTA in shared memory in exactly that order (F16; at most
//     four FP32 tokens carry a second F16 plane with the rounding remainder in the spare MMA columns).
//   * Work is cut into contiguous ranges of (tile, chunk) units: CTAs get tile ranges of equal byte cost, the 16 warps of a
//     CTA split its units evenly; pieces of a tile computed by different warps meet in shared memory in a fixed order, so
//     the output is bit-reproducible.
//
// Phases (two grid barriers; the CTAs are co-resident by a cooperative launch):
//   0  x -> F16 fragment-order records + group sums, and a bank-swizzled FP32 copy for the router
//   1  router logits [M, R] in FP32 FMA: four rows per CTA and pass, four warps (interleaved over K) per row
//   -- barrier --
//   2  every CTA: top-k + weights for the M tokens (a candidate bound from the lanes' maxima, then an all-pairs ranking of the
//      few candidates, one warp per token), the distinct-expert groups, the
//      cost partition; then gate/up tiles (8 gate rows + the 8 matching up rows = one MMA tile, SwiGLU lane-local) -> h,
//      written plainly (the probe) and as F16 records in fragment order for phase 3
//   -- barrier --
//   3  the h records arrive in shared memory by bulk copies (cp.async.bulk on an mbarrier); down projection + weighted
//      combine: a CTA owns 16 output rows and walks every active expert; one ordered cross-warp sum -> y.
// The separate (dense) shared expert is one more group whose tokens are all M; its part is rounded and added as the
// reference's moe_shared_add does (strixite kernels/moe_router.hip:140-144).
//
// Every wait on another CTA or on the copy engine is bounded: on expiry the CTA raises the abort word, all CTAs leave
// and the host sees the expert error words {2, 0xdec000 | code, block}.
#include "common.cuh"

#include "decode_stream.cuh"
#include "strixite_b200.h"

#include <cuda_fp16.h>

namespace {

using namespace sb;

#ifndef STRIX_DS_WARPS
#define STRIX_DS_WARPS 16
#endif
constexpr int kWarps = STRIX_DS_WARPS;      // 16 warps of up to 128 registers measured best (12: 168 registers, 24: 80); a diagnostic build may override
constexpr int kRouterRows = 4;              // router rows a CTA computes per pass, kRouterSlices warps (interleaved over K) per row
constexpr int kRouterSlices = kWarps / kRouterRows;
constexpr int kThreads = 32 * kWarps;
constexpr int kMaxTok = 8;
constexpr int kMaxGroups = 96;
constexpr int kMaxSlots = 96;
constexpr int kMaxExperts = 1032;          // Estack <= 1025
constexpr uint32_t kSpinLimit = 1u << 22;  // polls before a wait gives up (each poll is tens of ns)
constexpr int kCand = 32;                  // top-k candidates a token's list holds

// ---- PTX wrappers ----------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 ldg_stream16(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const uint8_t *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream4(const uint8_t *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
// The dynamic shared memory of the CTA. B operands and activation sums are addressed by 32-bit offsets from its start and
// read with ordinary loads, so the compiler orders them against barriers and schedules them freely among the MMAs.
extern __shared__ __align__(128) uint8_t smem_raw[];
__device__ __forceinline__ uint32_t smem_off(const void *p) { return (uint32_t)(static_cast<const uint8_t *>(p) - smem_raw); }
__device__ __forceinline__ uint4 lds16(uint32_t off) { return *reinterpret_cast<const uint4 *>(smem_raw + off); }
__device__ __forceinline__ float lds_f32(uint32_t off) { return *reinterpret_cast<const float *>(smem_raw + off); }
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same with a zero accumulator coming in: a fresh sum without clearing registers first.
__device__ __forceinline__ void mma_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// F32 -> F16 bits, round to nearest even, saturating to +-65504 instead of overflowing to infinity.
__device__ __forceinline__ uint16_t f32_to_f16_sat(float f) {
    uint16_t h;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
    return h;
}
__device__ __forceinline__ float f16_to_f32(uint16_t h) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bulk copy global -> shared (both 16-byte aligned, bytes a multiple of 16), completion counted on the mbarrier.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes),
                 "r"(smem_u32(bar))
                 : "memory");
}

// Phase timestamps of block 0, compiled in only with -DSTRIX_PROFILE (a diagnostic build): sync[8 + i] = ns.
#ifdef STRIX_PROFILE
__device__ __forceinline__ void stamp(uint32_t *sync, int i) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        uint64_t t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        sync[8 + i] = (uint32_t)t;
    }
}
#else
__device__ __forceinline__ void stamp(uint32_t *, int) {}
#endif

// ---- shared-memory control block -----------------------------------------------------------------------------------

struct Group {  // one distinct active expert with both projections resolved
    const uint8_t *rows[2];      // [0] gate_up, [1] down
    const uint16_t *scale[2], *minv[2];
    int32_t expert;              // row block of the stacks, or -2 = the separate shared expert
    uint32_t mask;               // tokens routed to it
    int16_t G[2];
    uint8_t bits[2];
    int8_t slot_a[kMaxTok];      // token m's slot index a (ids[m, a] == expert), -1 if not routed
};

struct Ctl {
    Group groups[kMaxGroups];
    uint32_t gmask[kMaxExperts];   // token mask per expert of the stacks
    uint8_t gindex[kMaxExperts];   // group number per expert
    int32_t ids[kMaxSlots];
    float coef[kMaxSlots];
    float gate[kMaxTok];           // the separate shared expert's coefficient per token
    uint32_t cumw[kMaxGroups + 1]; // byte cost of the groups before group i (gate/up partition)
    float rpart[kWarps][kMaxTok];  // phase 1: quarter-row partial logits
    uint32_t sel_key[kMaxTok][32]; // top-k scratch: the selected (key, index) pairs of a token, then in output order
    int32_t sel_idx[kMaxTok][32];
    uint32_t ord_key[kMaxTok][32];
    int32_t ord_idx[kMaxTok][32];
    int32_t lead_id[kMaxSlots];    // the distinct experts, in the order they were announced
    int32_t wtile[kWarps][2];      // the tile (phase 2) or row block (phase 3) behind each warp's two partial pieces, -1 = none
    uint64_t bar;                  // phase 3: the h records' bulk copies
    int n_groups, abort_flag, n_lead;
    uint32_t failed_mask;          // tokens the router failed (non-finite logits): NaN rows
    int gu_lo, gu_hi;              // this CTA's gate/up tiles
};

__device__ __forceinline__ void resolve_group(const StreamParams &p, Group &g) {
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

// Relative byte cost of one 128-code chunk of a row (codes + scale and minimum), for the partition.
__device__ __forceinline__ uint32_t chunk_cost(int bits) { return bits == 4 ? 17u : bits == 5 ? 21u : bits == 6 ? 25u : 33u; }

// ---- the unpack: one 32-bit word of nibbles (8 codes c0..c7) -> exact F16 code pairs -------------------------------
// lo[0] = {c0, c4}, lo[1] = {c2, c6}, hi[0] = {c1, c5}, hi[1] = {c3, c7} (low half, high half). An integer v < 1024 left in
// the low bits of an F16 IS the subnormal v * 2^-24, exactly, and the tensor cores take subnormal inputs at full precision:
// so an even nibble needs one AND to become code * 2^-24, and an odd nibble, left in place four bits up, is
// 16 code * 2^-24 = code * 2^-20; the two kinds go to separate accumulators and the powers of two fold into the group's
// scale. hx: the codes' high bits - Q5: 8 bits (bit j = code j), Q6: 16 bits (bits 2j..2j+1 = code j) - merged in.
template <int BITS>
__device__ __forceinline__ void unpack_word(uint32_t w, uint32_t hx, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
    const uint32_t w8 = w >> 8;
    lo[0] = w & 0x000F000Fu, lo[1] = w8 & 0x000F000Fu;
    hi[0] = w & 0x00F000F0u, hi[1] = w8 & 0x00F000F0u;
    if constexpr (BITS == 5) {
        const uint32_t m0 = hx * 0x10010u;  // bit j at 4 + j and at 16 + j
        lo[0] |= m0 & 0x00100010u, lo[1] |= (m0 >> 2) & 0x00100010u;
        hi[0] |= (m0 << 3) & 0x01000100u, hi[1] |= (m0 << 1) & 0x01000100u;
    } else if constexpr (BITS == 6) {
        const uint32_t t = hx << 4, m0 = t | (t << 8);  // field j at 4 + 2j and at 12 + 2j
        lo[0] |= m0 & 0x00300030u, lo[1] |= (m0 >> 4) & 0x00300030u;
        hi[0] |= (m0 << 2) & 0x03000300u, hi[1] |= (m0 >> 2) & 0x03000300u;
    }
}
constexpr float kTwo20 = 1048576.f, kTwo24 = 16777216.f;

// ---- one 128-code chunk of the two rows of a lane, in registers ------------------------------------------------------
// Nibble formats: lane (g, t) holds codes 32t .. 32t + 31 of the chunk (one 16-byte load per row; Q5 / Q6 add 4 / 8 bytes
// of high bits), so the four lanes of a quad cover the chunk = one quantization group of 128.
// Q8: per 64-code half h, lane t holds codes 64h + 16t .. + 15, so the quad covers one group of 64.
template <int BITS>
struct Chunk {
    static constexpr int NW = BITS == 8 ? 8 : 4;
    static constexpr int NH = BITS == 5 ? 1 : BITS == 6 ? 2 : 1;
    uint32_t a[NW], b[NW];
    uint32_t ha[NH], hb[NH];
    uint32_t sc[4];  // raw BF16 bits of scale A, min A, scale B, min B (two groups packed when a chunk spans two)
};

// What a lane needs to stream chunks [c0, c1) of its two rows (MMA rows g and g + 8) of a 16-row tile.
struct Seg {
    const uint8_t *pa;        // row A's codes at the lane's offset inside a chunk (+ 16 t)
    uint32_t dB;              // row B - row A, bytes
    uint32_t hoff;            // Q5 / Q6: from pa to the lane's high bits of chunk 0
    const uint16_t *sc, *mn;  // the projection's scale / minimum arrays
    uint32_t oA, oB;          // the rows' first group in them
    uint32_t bq;              // shared-memory offset of the lane's B record of chunk 0, word 0 (the lane's t part folded in)
    uint32_t q0, q1;          // shared-memory offsets of the activation sums of accumulator columns 2t, 2t + 1
    int c0, c1;
};

// Shared-memory strides of the B operand, bytes. Records are 16 bytes = 8 activations k0 .. k0 + 7 in the order
// 0,4,2,6,1,5,3,7 (k0 = 128 c + 32 t' + 8 w). Gate/up reads x: record (c, w, column g, t') at ((c * 4 + w) * 32 + 4 g + t') * 16;
// down reads a token's own h record: (c, w, t') at ((c * 4 + w) * 4 + t') * 16. Sums: one float per (chunk, 64-code half, column)
// for x, per (record, chunk, half) for h.
template <bool DOWN>
struct Lay {
    static constexpr uint32_t cs = DOWN ? 256 : 2048, ws = DOWN ? 64 : 512, qc = DOWN ? 8 : 64, qh = DOWN ? 4 : 32;
};

template <int BITS, int GH>
__device__ __forceinline__ void load_chunk(Chunk<BITS> &q, const Seg &sg, int c) {
    if constexpr (BITS == 8) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 va = ldg_stream16(sg.pa + c * 128 + h * 64), vb = ldg_stream16(sg.pa + sg.dB + c * 128 + h * 64);
            q.a[4 * h] = va.x, q.a[4 * h + 1] = va.y, q.a[4 * h + 2] = va.z, q.a[4 * h + 3] = va.w;
            q.b[4 * h] = vb.x, q.b[4 * h + 1] = vb.y, q.b[4 * h + 2] = vb.z, q.b[4 * h + 3] = vb.w;
        }
    } else {
        const uint4 va = ldg_stream16(sg.pa + c * 64), vb = ldg_stream16(sg.pa + sg.dB + c * 64);
        q.a[0] = va.x, q.a[1] = va.y, q.a[2] = va.z, q.a[3] = va.w;
        q.b[0] = vb.x, q.b[1] = vb.y, q.b[2] = vb.z, q.b[3] = vb.w;
        if constexpr (BITS == 5) {
            q.ha[0] = ldg_stream4(sg.pa + sg.hoff + c * 16), q.hb[0] = ldg_stream4(sg.pa + sg.dB + sg.hoff + c * 16);
        } else if constexpr (BITS == 6) {
            const uint2 xa = ldg_stream8(sg.pa + sg.hoff + c * 32), xb = ldg_stream8(sg.pa + sg.dB + sg.hoff + c * 32);
            q.ha[0] = xa.x, q.ha[1] = xa.y, q.hb[0] = xb.x, q.hb[1] = xb.y;
        }
    }
    if constexpr (GH == 2) {  // groups of 64: the chunk's two groups are one aligned 32-bit load
        q.sc[0] = __ldg(reinterpret_cast<const uint32_t *>(sg.sc + sg.oA) + c), q.sc[1] = __ldg(reinterpret_cast<const uint32_t *>(sg.mn + sg.oA) + c);
        q.sc[2] = __ldg(reinterpret_cast<const uint32_t *>(sg.sc + sg.oB) + c), q.sc[3] = __ldg(reinterpret_cast<const uint32_t *>(sg.mn + sg.oB) + c);
    } else {
        q.sc[0] = __ldg(sg.sc + sg.oA + c), q.sc[1] = __ldg(sg.mn + sg.oA + c), q.sc[2] = __ldg(sg.sc + sg.oB + c), q.sc[3] = __ldg(sg.mn + sg.oB + c);
    }
}

template <int BITS, int GH, bool DOWN>
__device__ __forceinline__ void consume_chunk(const Chunk<BITS> &q, int c, const Seg &sg, float (&tot)[4]) {
    using L = Lay<DOWN>;
    if constexpr (BITS == 8) {
        // the lane's 16 codes of a half sit in records (w' = 2 (t & 1) + wp, t' = 2 h + (t >> 1)): bq carries the lane's part
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // a code byte b between two zero bytes is the subnormal b * 2^-24
            float acc0[4], acc1[4];
#pragma unroll
            for (int wp = 0; wp < 2; ++wp) {
                const uint4 B = lds16(sg.bq + c * L::cs + wp * L::ws + h * 32);
#pragma unroll
                for (int odd = 0; odd < 2; ++odd) {
                    const uint32_t wa = q.a[4 * h + 2 * wp + odd], wb = q.b[4 * h + 2 * wp + odd];
                    const uint32_t a0 = __byte_perm(wa, 0u, 0x4140), a2 = __byte_perm(wa, 0u, 0x4342);
                    const uint32_t a1 = __byte_perm(wb, 0u, 0x4140), a3 = __byte_perm(wb, 0u, 0x4342);
                    const uint32_t sel = odd ? 0x7632u : 0x5410u;
                    if (wp == 0) mma_f16_zero(odd ? acc1 : acc0, a0, a1, a2, a3, __byte_perm(B.x, B.z, sel), __byte_perm(B.y, B.w, sel));
                    else mma_f16(odd ? acc1 : acc0, a0, a1, a2, a3, __byte_perm(B.x, B.z, sel), __byte_perm(B.y, B.w, sel));
                }
            }
            const uint32_t sh = GH == 2 ? 16u * h : 0u;
            const float sA = __uint_as_float((q.sc[0] >> sh) << 16) * kTwo24, mA = __uint_as_float((q.sc[1] >> sh) << 16);
            const float sB = __uint_as_float((q.sc[2] >> sh) << 16) * kTwo24, mB = __uint_as_float((q.sc[3] >> sh) << 16);
            const float Q0 = lds_f32(sg.q0 + c * L::qc + h * L::qh), Q1 = lds_f32(sg.q1 + c * L::qc + h * L::qh);
            tot[0] = fmaf(sA, acc0[0] + acc1[0], fmaf(mA, Q0, tot[0])), tot[1] = fmaf(sA, acc0[1] + acc1[1], fmaf(mA, Q1, tot[1]));
            tot[2] = fmaf(sB, acc0[2] + acc1[2], fmaf(mB, Q0, tot[2])), tot[3] = fmaf(sB, acc0[3] + acc1[3], fmaf(mB, Q1, tot[3]));
        }
    } else {
        float acc0[4], acc1[4];  // even nibbles (x 2^-24), odd nibbles (x 2^-20)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t hxa = 0, hxb = 0;
            if constexpr (BITS == 5) hxa = (q.ha[0] >> (8 * w)) & 0xFFu, hxb = (q.hb[0] >> (8 * w)) & 0xFFu;
            if constexpr (BITS == 6) hxa = (q.ha[w >> 1] >> (16 * (w & 1))) & 0xFFFFu, hxb = (q.hb[w >> 1] >> (16 * (w & 1))) & 0xFFFFu;
            uint32_t la[2], ua[2], lb[2], ub[2];
            unpack_word<BITS>(q.a[w], hxa, la, ua);
            unpack_word<BITS>(q.b[w], hxb, lb, ub);
            const uint4 B = lds16(sg.bq + c * L::cs + w * L::ws);
            if (w == 0) {
                mma_f16_zero(acc0, la[0], lb[0], la[1], lb[1], B.x, B.y);
                mma_f16_zero(acc1, ua[0], ub[0], ua[1], ub[1], B.z, B.w);
            } else {
                mma_f16(acc0, la[0], lb[0], la[1], lb[1], B.x, B.y);
                mma_f16(acc1, ua[0], ub[0], ua[1], ub[1], B.z, B.w);
            }
        }
        // sum(x code) = (16 acc0 + acc1) * 2^20: the power of two rides on the scale
        const float sA = __uint_as_float(q.sc[0] << 16) * kTwo20, mA = __uint_as_float(q.sc[1] << 16);
        const float sB = __uint_as_float(q.sc[2] << 16) * kTwo20, mB = __uint_as_float(q.sc[3] << 16);
        const float Q0 = lds_f32(sg.q0 + c * L::qc) + lds_f32(sg.q0 + c * L::qc + L::qh);
        const float Q1 = lds_f32(sg.q1 + c * L::qc) + lds_f32(sg.q1 + c * L::qc + L::qh);
        tot[0] = fmaf(sA, fmaf(acc0[0], 16.f, acc1[0]), fmaf(mA, Q0, tot[0])), tot[1] = fmaf(sA, fmaf(acc0[1], 16.f, acc1[1]), fmaf(mA, Q1, tot[1]));
        tot[2] = fmaf(sB, fmaf(acc0[2], 16.f, acc1[2]), fmaf(mB, Q0, tot[2])), tot[3] = fmaf(sB, fmaf(acc0[3], 16.f, acc1[3]), fmaf(mB, Q1, tot[3]));
    }
}

// Chunks [c0, c1) of a 16-row tile. Loads run PD chunks ahead of the arithmetic. Returns the lane's 2 rows x 2 columns of
// s * sum(x code) + m * sum(x).
template <int BITS, int GH, bool DOWN>
__device__ __forceinline__ float4 run_segment(const Seg &sg) {
    constexpr int PD = kWarps >= 24 ? (BITS == 8 ? 1 : 2) : kWarps >= 16 ? (BITS == 8 ? 1 : BITS == 6 ? 2 : 3) : (BITS == 8 ? 2 : BITS == 6 ? 3 : 4);
    Chunk<BITS> q[PD];
    float tot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < PD; ++i)
        if (sg.c0 + i < sg.c1) load_chunk<BITS, GH>(q[i], sg, sg.c0 + i);
    for (int c = sg.c0; c < sg.c1; c += PD) {
#pragma unroll
        for (int i = 0; i < PD; ++i) {
            if (c + i < sg.c1) {
                consume_chunk<BITS, GH, DOWN>(q[i], c + i, sg, tot);
                if (c + i + PD < sg.c1) load_chunk<BITS, GH>(q[i], sg, c + i + PD);
            }
        }
    }
    return make_float4(tot[0], tot[1], tot[2], tot[3]);
}
// Out-of-line twin, for the kernel variant that has to carry every format: each loop keeps its registers to itself there.
template <int BITS, int GH, bool DOWN>
__device__ __noinline__ float4 run_segment_call(Seg sg) {
    return run_segment<BITS, GH, DOWN>(sg);
}

// Formats a kernel variant was compiled for: bit 0 = 4 bits, 1 = 5 bits, 2 = 6 bits, 3 = 8 bits in groups of 128, 4 = 8 bits in
// groups of 64. kFmQ4: every projection 4-bit; kFmQ4Q8: 4-bit experts with an 8-bit (groups of 64) shared expert, the reference's
// served layout (strixite docs/weights.md:19-26); both inline their loops. kFmAll carries all five, the rarer ones out of line.
constexpr int kFmQ4 = 0x01, kFmQ4Q8 = 0x11, kFmAll = 0x1F;

// Fills the lane-dependent parts of a segment for rows rA, rB of a projection [*, K] and runs it. bg: shared-memory offset of the
// lane's column's records; q0 / q1: of its two accumulator columns' sums.
template <bool DOWN, int FM>
__device__ __forceinline__ float4 run_tile(const Group &grp, int rA, int rB, int K, int c0, int c1, int t, uint32_t bg, uint32_t q0, uint32_t q1) {
    constexpr int pj = DOWN ? 1 : 0;
    using L = Lay<DOWN>;
    const int bits = FM == kFmQ4 ? 4 : grp.bits[pj], G = grp.G[pj], gpr = K / G;
    const int64_t rb = row_bytes(bits, K);
    Seg sg;
    sg.pa = grp.rows[pj] + rA * rb + t * 16;
    sg.dB = (uint32_t)((rB - rA) * rb);
    sg.hoff = (uint32_t)(K / 2 - t * 16 + (bits == 5 ? t * 4 : t * 8));
    sg.sc = grp.scale[pj], sg.mn = grp.minv[pj];
    sg.oA = (uint32_t)(rA * gpr), sg.oB = (uint32_t)(rB * gpr);
    sg.bq = bits == 8 ? bg + 2 * (t & 1) * L::ws + (t >> 1) * 16 : bg + t * 16;
    sg.q0 = q0, sg.q1 = q1, sg.c0 = c0, sg.c1 = c1;
    if constexpr (FM == kFmQ4) {
        return run_segment<4, 1, DOWN>(sg);
    } else if constexpr (FM == kFmQ4Q8) {
        return bits == 4 ? run_segment<4, 1, DOWN>(sg) : run_segment<8, 2, DOWN>(sg);
    } else {
        switch (bits) {
            case 4: return run_segment<4, 1, DOWN>(sg);
            case 5: return run_segment_call<5, 1, DOWN>(sg);
            case 6: return run_segment_call<6, 1, DOWN>(sg);
            default: return G == 64 ? run_segment_call<8, 2, DOWN>(sg) : run_segment_call<8, 1, DOWN>(sg);
        }
    }
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
__device__ __forceinline__ bool grid_wait(const uint32_t *counter, uint32_t *abort_word, Ctl &ctl) {
    if (threadIdx.x == 0) {
        bool ok = false;
        for (uint32_t i = 0; i < kSpinLimit; ++i) {
            if (ld_acquire(counter) >= gridDim.x) {
                ok = true;
                break;
            }
            if ((i & 63u) == 63u && ld_acquire(abort_word) != 0u) break;
        }
        if (!ok && ctl.abort_flag == 0) ctl.abort_flag = ld_acquire(abort_word) != 0u ? 0x200 : 0x105;
    }
    __syncthreads();
    return ctl.abort_flag == 0;
}

// ---- phase 0: activations -> fragment-order F16 records ----------------------------------------------------------------
// The FP32 copy for the router keeps float4 f of a token at f ^ ((f >> 3) & 7): lanes reading consecutive float4s, float4s
// 8 apart (one 32-code chunk per lane) or 4 apart all spread over the banks.
__device__ __forceinline__ int swz4(int f) { return f ^ ((f >> 3) & 7); }

// 8 consecutive activations -> one record in the order 0,4,2,6,1,5,3,7 (plane 1: the F16 rounding remainders).
__device__ __forceinline__ uint4 make_record(const float (&v)[8], int plane, float &sum) {
    uint16_t h[8];
    sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        h[j] = f32_to_f16_sat(v[j]);
        if (plane == 1) h[j] = f32_to_f16_sat(v[j] - f16_to_f32(h[j]));
        sum += f16_to_f32(h[j]);  // the sum of what the tensor cores will see
    }
    uint4 r;
    r.x = h[0] | ((uint32_t)h[4] << 16), r.y = h[2] | ((uint32_t)h[6] << 16), r.z = h[1] | ((uint32_t)h[5] << 16), r.w = h[3] | ((uint32_t)h[7] << 16);
    return r;
}

template <typename T>
__device__ __forceinline__ void stage_x(const StreamParams &p, uint8_t *xs, float *xq, float4 *xf4, int tid) {
    const int d = p.d, M = p.M;
    const T *x = static_cast<const T *>(p.x);
    for (int e = tid; e < d; e += kThreads) {  // d records of 16 bytes: (d / 128) chunks x 8 columns x 16; warp-uniform trip count
        const int t = e & 3, w = (e >> 2) & 3, g = (e >> 4) & 7, c = e >> 7;
        const int tok = p.planes == 2 ? (g & 3) : g, pl = p.planes == 2 ? (g >> 2) : 0;
        const int k0 = c * 128 + t * 32 + w * 8;
        float v[8];
        if (tok < M) {
            if constexpr (sizeof(T) == 4) {
                const float4 a = *reinterpret_cast<const float4 *>(x + (int64_t)tok * d + k0), b = *reinterpret_cast<const float4 *>(x + (int64_t)tok * d + k0 + 4);
                v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
            } else {
                const uint4 q = *reinterpret_cast<const uint4 *>(x + (int64_t)tok * d + k0);
                const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) v[2 * j] = __uint_as_float(w4[j] << 16), v[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
            }
            if (pl == 0) {
                const int f = k0 >> 2;
                xf4[tok * (d / 4) + swz4(f)] = make_float4(v[0], v[1], v[2], v[3]);
                xf4[tok * (d / 4) + swz4(f + 1)] = make_float4(v[4], v[5], v[6], v[7]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
        }
        float sum;
        const uint4 rec = make_record(v, pl, sum);
        *reinterpret_cast<uint4 *>(xs + ((c * 4 + w) * 32 + g * 4 + t) * 16) = rec;
        // the 64-code half (t >> 1) of the chunk: lanes with equal t >> 1 and any w
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);
        if ((t & 1) == 0 && w == 0) xq[(c * 2 + (t >> 1)) * 8 + g] = sum;
    }
}

// ---- phase 1: a slice of one router row against all tokens -------------------------------------------------------------
// The warps of a CTA form kRouterRows teams of kRouterSlices; a team takes one router row per pass and its warps interleave
// over K in steps of 32 lanes x 8 weights. Quantized rows (8-bit) are dequantized to code * s + m first - the reference's
// own values (strixite formats/q8.hpp:33-35) - so the three kinds share the FP32 multiply-add loop.
__device__ __forceinline__ void router_slice(const StreamParams &p, const float4 *xf4, int r, int slice, int lane, float (&acc)[kMaxTok]) {
    const int d = p.d, M = p.M, d4 = d / 4, n8 = d / 8;
#pragma unroll
    for (int m = 0; m < kMaxTok; ++m) acc[m] = 0.f;
    for (int e = slice * 32 + lane; e < n8; e += 32 * kRouterSlices) {  // 8 weights k = 8 e .. 8 e + 7
        float wf[8];
        if (p.router_kind == STRIX_ROUTER_F32) {
            const float4 *wr = static_cast<const float4 *>(p.router_w) + (int64_t)r * d4 + 2 * e;
            const float4 a = __ldg(wr), b = __ldg(wr + 1);
            wf[0] = a.x, wf[1] = a.y, wf[2] = a.z, wf[3] = a.w, wf[4] = b.x, wf[5] = b.y, wf[6] = b.z, wf[7] = b.w;
        } else if (p.router_kind == STRIX_ROUTER_BF16) {
            const uint4 q = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.router_w) + (int64_t)r * d) + e);
            const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) wf[2 * j] = __uint_as_float(w4[j] << 16), wf[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
        } else {
            const strix_qview &v = p.router_q;
            const int gpr = (int)(v.K / v.G);
            const uint2 q = __ldg(reinterpret_cast<const uint2 *>(v.q + (int64_t)r * d) + e);
            const float sc = bf16_bits_to_f32(__ldg(v.scale + (int64_t)r * gpr + 8 * e / (int)v.G));
            const float mn = bf16_bits_to_f32(__ldg(v.minv + (int64_t)r * gpr + 8 * e / (int)v.G));
#pragma unroll
            for (int j = 0; j < 8; ++j) wf[j] = __fadd_rn(__fmul_rn(code_f(((j < 4 ? q.x : q.y) >> (8 * (j & 3))) & 0xFFu), sc), mn);
        }
#pragma unroll
        for (int m = 0; m < kMaxTok; ++m) {
            if (m < M) {
                const float4 a = xf4[m * d4 + swz4(2 * e)], b = xf4[m * d4 + swz4(2 * e + 1)];
                float tt = acc[m];
                tt = fmaf(a.x, wf[0], tt), tt = fmaf(a.y, wf[1], tt), tt = fmaf(a.z, wf[2], tt), tt = fmaf(a.w, wf[3], tt);
                tt = fmaf(b.x, wf[4], tt), tt = fmaf(b.y, wf[5], tt), tt = fmaf(b.z, wf[6], tt), tt = fmaf(b.w, wf[7], tt);
                acc[m] = tt;
            }
        }
    }
}

// ---- phase 2a: routing, computed by every CTA --------------------------------------------------------------------------
// An order-preserving map of a float to an unsigned key (-0 = +0).
__device__ __forceinline__ uint32_t order_key(float f) {
    uint32_t u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

// One warp selects token m's k largest logits without a selection loop over k. Lane l holds experts l, l + 32, .. as
// order-preserving keys (absent experts carry key 0, below every finite float's key).
//   1. every lane's largest key; the k-th largest of those 32 maxima is a lower bound L of the k-th largest key overall
//      (k distinct elements are at least L), found by ranking the 32 maxima against each other;
//   2. the candidates, every key >= L (k of them at least, rarely many more), are compacted into shared memory;
//   3. each candidate's rank among the candidates in the order the reference emits picks - descending value, ties by
//      ascending index (strixite kernels/moe_router.hpp:11-23) - is its output slot; ranks >= k drop out.
template <int NV>
__device__ __noinline__ void route_token(const StreamParams &p, Ctl &ctl, int m, int lane, bool write_global) {
    const float *row = p.logits + (int64_t)m * p.R;
    const int E = p.E, k = p.k, A = p.A;
    uint32_t key[NV];
    bool nonfinite = false;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int e = lane + 32 * j;
        const float v = e < E ? __ldcg(row + e) : 0.f;
        key[j] = e < E ? order_key(v) : 0u;
        nonfinite |= (__float_as_uint(v) & 0x7f800000u) == 0x7f800000u;
    }
    float sl = 0.f;
    if (p.gated) {
        sl = __ldcg(row + E);
        nonfinite |= (__float_as_uint(sl) & 0x7f800000u) == 0x7f800000u;
    }
    if (m == 0) stamp(p.sync, 14);
    if (__any_sync(0xffffffffu, nonfinite)) {  // a non-finite logit fails the token: ids -1, weights NaN, err = {1, token, first such expert}
        unsigned bad = 0xffffffffu;
#pragma unroll 1
        for (int e = lane; e <= E; e += 32)
            if ((e < E || p.gated) && !isfinite(__ldcg(row + e)) && (unsigned)e < bad) bad = (unsigned)e;
        bad = __reduce_min_sync(0xffffffffu, bad);
        if (lane == 0) {
            atomicOr(&ctl.failed_mask, 1u << m);
            if (write_global) raise_err(p.err, (uint32_t)m, bad);
            ctl.gate[m] = qnan();
        }
        for (int a = lane; a < A; a += 32) {
            ctl.ids[m * A + a] = -1, ctl.coef[m * A + a] = qnan();
            if (write_global) p.ids[m * A + a] = -1, p.coef[m * A + a] = qnan();
        }
        return;
    }
    uint32_t mx[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) mx[j] = key[j];
#pragma unroll
    for (int w = NV / 2; w >= 1; w >>= 1)
#pragma unroll
        for (int j = 0; j < w; ++j) mx[j] = mx[j] > mx[j + w] ? mx[j] : mx[j + w];
    const uint32_t mine = mx[0];
    int rank = 0;
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
        const uint32_t other = __shfl_sync(0xffffffffu, mine, i);
        rank += (other > mine) || (other == mine && i < lane);
    }
    const unsigned holder = __ballot_sync(0xffffffffu, rank == k - 1);
    const uint32_t L = __shfl_sync(0xffffffffu, mine, __ffs(holder) - 1);
    if (m == 0) stamp(p.sync, 15);
    // candidates: a lane's keys >= L go to consecutive places of the list, lanes in order (an exclusive scan of the counts)
    int mine_n = 0;
#pragma unroll
    for (int j = 0; j < NV; ++j) mine_n += key[j] >= L;
    int incl = mine_n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    int n_cand = __shfl_sync(0xffffffffu, incl, 31);
    if (n_cand <= kCand) {
        int pos = incl - mine_n;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (key[j] >= L) ctl.sel_key[m][pos] = key[j], ctl.sel_idx[m][pos] = lane + 32 * j, ++pos;
    } else {
        // more candidates than the list holds (the bound is tied many times over): the exact k-th largest key T by a bitwise
        // binary search over counts; then everything above T in any order and ties at T in ascending index, as many as needed
        uint32_t T = 0;
#pragma unroll 1
        for (int b = 31; b >= 0; --b) {
            const uint32_t cand = T | (1u << b);
            int cnt = 0;
#pragma unroll
            for (int j = 0; j < NV; ++j) cnt += key[j] >= cand;
            if ((int)__reduce_add_sync(0xffffffffu, cnt) >= k) T = cand;
        }
        int above = 0;
#pragma unroll
        for (int j = 0; j < NV; ++j) above += key[j] > T;
        above = (int)__reduce_add_sync(0xffffffffu, above);
        const unsigned lt = (1u << lane) - 1u;
        int base_gt = 0, base_eq = 0;
#pragma unroll 1
        for (int j = 0; j < NV; ++j) {
            uint32_t kj = 0;  // key[j] without a dynamic register index
#pragma unroll
            for (int j2 = 0; j2 < NV; ++j2) kj = j2 == j ? key[j2] : kj;
            const bool is_gt = kj > T, is_eq = kj == T;
            const unsigned bgt = __ballot_sync(0xffffffffu, is_gt), beq = __ballot_sync(0xffffffffu, is_eq);
            const int eq_rank = base_eq + __popc(beq & lt);
            int pos = -1;
            if (is_gt) pos = base_gt + __popc(bgt & lt);
            else if (is_eq && eq_rank < k - above) pos = above + eq_rank;
            if (pos >= 0) ctl.sel_key[m][pos] = kj, ctl.sel_idx[m][pos] = lane + 32 * j;
            base_gt += __popc(bgt), base_eq += __popc(beq);
        }
        n_cand = k;
    }
    __syncwarp();
    if (m == 0) stamp(p.sync, 16);
    if (lane < n_cand) {
        const uint32_t ki = ctl.sel_key[m][lane];
        const int ii = ctl.sel_idx[m][lane];
        int r = 0;
        for (int j = 0; j < n_cand; ++j) {
            const uint32_t kj = ctl.sel_key[m][j];
            r += (kj > ki) || (kj == ki && ctl.sel_idx[m][j] < ii);
        }
        if (r < k) ctl.ord_key[m][r] = ki, ctl.ord_idx[m][r] = ii;
    }
    __syncwarp();
    if (m == 0) stamp(p.sync, 17);
    const float top = key_value(ctl.ord_key[m][0]);
    const float ex = lane < k ? expf(key_value(ctl.ord_key[m][lane]) - top) : 0.f;
    const float sum = warp_sum(ex);
    if (lane < k) {
        const float c = ex / sum;
        const int id = ctl.ord_idx[m][lane];
        ctl.ids[m * A + lane] = id, ctl.coef[m * A + lane] = c;
        if (write_global) p.ids[m * A + lane] = id, p.coef[m * A + lane] = c;
    }
    if (lane == 0) {
        const float g = p.gated ? sigmoid_f(sl) : 1.0f;
        ctl.gate[m] = g;
        if (p.shared_mode == STRIX_SHARED_STACKED) {
            ctl.ids[m * A + k] = E, ctl.coef[m * A + k] = g;
            if (write_global) p.ids[m * A + k] = E, p.coef[m * A + k] = g;
        }
    }
    if (m == 0) stamp(p.sync, 18);
}

// Distinct-expert groups in ascending expert order (the separate shared expert first), by the whole block: the first slot to
// mark an expert's token mask announces the expert; each announced expert's rank among the announced is its group. Then the
// gate/up tile range of this CTA: tiles are (group, block of 8 row pairs) in group order, a tile costs its format's bytes, and
// CTA b takes the tiles whose start cost lies in [b W / n, (b + 1) W / n).
__device__ void build_groups(const StreamParams &p, Ctl &ctl, int tid) {
    const int S = p.M * p.A, A = p.A, lane = tid & 31, warp = tid >> 5;
    const int base = p.shared_mode == STRIX_SHARED_SEPARATE ? 1 : 0;
    int32_t my_id = -1;
    if (tid < S) {
        my_id = ctl.ids[tid];
        if (my_id >= 0 && my_id < p.Estack) {
            if (atomicOr(&ctl.gmask[my_id], 1u << (tid / A)) == 0u) ctl.lead_id[atomicAdd(&ctl.n_lead, 1)] = my_id;
        } else {
            my_id = -1;
        }
    }
    __syncthreads();
    const int n_lead = ctl.n_lead;
    if (tid < n_lead) {
        const int32_t e = ctl.lead_id[tid];
        int gi = base;
        for (int j = 0; j < n_lead; ++j) gi += ctl.lead_id[j] < e;
        Group &g = ctl.groups[gi];
        g.expert = e, g.mask = ctl.gmask[e];
#pragma unroll
        for (int m = 0; m < kMaxTok; ++m) g.slot_a[m] = -1;
        ctl.gindex[e] = (uint8_t)gi;
    }
    if (tid == kThreads - 1) {
        ctl.n_groups = base + n_lead;
        if (base) {
            Group &g = ctl.groups[0];
            g.expert = -2, g.mask = ((1u << p.M) - 1u) & ~ctl.failed_mask;
#pragma unroll
            for (int m = 0; m < kMaxTok; ++m) g.slot_a[m] = m < p.M ? 0 : -1;
            if (g.mask == 0u) ctl.n_groups = 0;  // every token failed: nothing to compute
        }
    }
    __syncthreads();
    if (my_id >= 0) ctl.groups[ctl.gindex[my_id]].slot_a[tid / A] = (int8_t)(tid % A);
    if (tid < ctl.n_groups) resolve_group(p, ctl.groups[tid]);
    __syncthreads();
    const int NG = ctl.n_groups, T = p.I / 8;
    if (warp == 0) {  // inclusive scan of the groups' costs, three groups per lane
        uint32_t c[3], run = 0;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int gi = lane * 3 + i;
            c[i] = gi < NG ? chunk_cost(ctl.groups[gi].bits[0]) * (uint32_t)T : 0u;
            run += c[i];
        }
        uint32_t incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        uint32_t upto = incl - run;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int gi = lane * 3 + i;
            upto += c[i];
            if (gi < NG) ctl.cumw[gi + 1] = upto;
        }
        if (lane == 0) ctl.cumw[0] = 0u, ctl.gu_lo = 0, ctl.gu_hi = 0;
    }
    __syncthreads();
    if (tid < 2 * kMaxGroups && NG > 0) {
        const int which = tid >= kMaxGroups, gi = tid - which * kMaxGroups;
        const uint32_t W = ctl.cumw[NG];  // < 2^32 / gridDim.x: at most 96 groups x 33 x 2048 tiles
        const uint32_t L = W * (uint32_t)(blockIdx.x + which) / gridDim.x;
        if (gi < NG) {
            const uint32_t lo = ctl.cumw[gi], hi = ctl.cumw[gi + 1];
            if (L >= lo && L < hi) {
                const uint32_t w = chunk_cost(ctl.groups[gi].bits[0]);
                const int jb = (int)((L - lo + w - 1) / w);
                (which ? ctl.gu_hi : ctl.gu_lo) = gi * T + jb;
            }
        }
        if (gi == 0 && L >= W) (which ? ctl.gu_hi : ctl.gu_lo) = NG * T;
    }
    __syncthreads();
}

// ---- phase 2b epilogue: one finished gate/up tile -> h --------------------------------------------------------------------
// tot[e]: gate row jb * 8 + g, tot[2 + e]: the matching up row, for accumulator column 2t + e.
template <typename T>
__device__ __noinline__ void finish_gate_up(const StreamParams &p, const Group &grp, int jb, float4 tot4, int lane) {
    const int g = lane >> 2, t = lane & 3, M = p.M, A = p.A, I = p.I;
    float tot[4] = {tot4.x, tot4.y, tot4.z, tot4.w};
    if (p.planes == 2) {  // the remainder plane's columns sit two lanes up
#pragma unroll
        for (int i = 0; i < 4; ++i) tot[i] += __shfl_xor_sync(0xffffffffu, tot[i], 2);
    }
    T *hh = static_cast<T *>(p.hh);
    const int j = jb * 8 + g;  // the h element
    // its place in a record: chunk j / 128, lane quarter (j / 32) % 4, word (j / 8) % 4, position = bits of j % 8 reversed
    const int pos = ((g & 1) << 2) | (g & 2) | ((g & 4) >> 2);
    const int rec_off = ((((j >> 7) * 4 + ((j >> 3) & 3)) * 4 + ((j >> 5) & 3)) * 8 + pos) * 2;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int tok = 2 * t + e;
        const bool live = (p.planes == 2 ? t < 2 : true) && tok < M && (grp.mask >> tok & 1u);
        if (!live) continue;
        const float gs = as_stored(tot[e], hh), us = as_stored(tot[2 + e], hh);
        const float hv = as_stored(as_stored(silu_f(gs), hh) * us, hh);
        const int slot = grp.expert == -2 ? M * A + tok : tok * A + grp.slot_a[tok];
        if (grp.expert != -2) st_act(hh, (int64_t)slot * I + j, hv);
        else if (p.sh_h != nullptr) st_act(static_cast<T *>(p.sh_h), (int64_t)tok * I + j, hv);
        const uint16_t hb = f32_to_f16_sat(hv);
        uint8_t *rec = p.hrec + (int64_t)slot * p.planes * p.rec_bytes + rec_off;
        *reinterpret_cast<uint16_t *>(rec) = hb;
        if (p.planes == 2) *reinterpret_cast<uint16_t *>(rec + p.rec_bytes) = f32_to_f16_sat(hv - f16_to_f32(hb));
    }
}

// ---- the kernel ----------------------------------------------------------------------------------------------------------

template <typename T, int FM, int NV>
__global__ void __launch_bounds__(kThreads, 1) decode_stream_kernel(const __grid_constant__ StreamParams p) {
    Ctl &ctl = *reinterpret_cast<Ctl *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int M = p.M, d = p.d, I = p.I, A = p.A;
    uint32_t *counters = p.sync;  // [0], [1]: the two barriers; [2]: CTAs done; [3]: abort

    // shared-memory plan (decode_stream_plan computes the same sizes)
    // floats per lane of a partial tile: 4, + 4 for the separate shared expert's part (kept apart for its own rounding)
    const int kPartFloats = p.shared_mode == STRIX_SHARED_SEPARATE ? 8 : 4;
    float *part = reinterpret_cast<float *>(smem_raw + ((sizeof(Ctl) + 127) & ~(size_t)127));  // [kWarps][2][32][kPartFloats]
    float *xq = part + kWarps * 2 * 32 * kPartFloats;                                           // [d / 128][2][8]
    uint8_t *uni = reinterpret_cast<uint8_t *>(xq + (d / 128) * 16);                            // phases 0-2: xs, xf; phase 3: h records, sums
    uint8_t *xs = uni;                                                                          // d records of 16 bytes
    float4 *xf4 = reinterpret_cast<float4 *>(uni + (size_t)d * 16);                             // [M][d / 4], swizzled
    uint8_t *hs = uni;                                                                          // (n_rec + 1) records of rec_bytes
    float *hq = reinterpret_cast<float *>(uni + (size_t)(p.n_rec + 1) * p.rec_bytes);           // [n_rec + 1][I / 128][2]

    if (tid == 0) {
        ctl.abort_flag = 0, ctl.failed_mask = 0, ctl.n_groups = 0, ctl.n_lead = 0;
        mbar_init(&ctl.bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < kMaxExperts; i += kThreads) ctl.gmask[i] = 0u;

    // Phase 0
    stamp(p.sync, 0);
    stage_x<T>(p, xs, xq, xf4, tid);
    __syncthreads();
    stamp(p.sync, 1);

    // Phase 1: router logits; warp w works on row r0 + w % kRouterRows, K slice w / kRouterRows.
    for (int r0 = blockIdx.x * kRouterRows; r0 < p.R; r0 += gridDim.x * kRouterRows) {
        const int r = r0 + warp % kRouterRows;
        float acc[kMaxTok];
        if (r < p.R) {
            router_slice(p, xf4, r, warp / kRouterRows, lane, acc);
#pragma unroll
            for (int m = 0; m < kMaxTok; ++m) {
                if (m < M) {
                    const float v = warp_sum(acc[m]);
                    if (lane == 0) ctl.rpart[warp][m] = v;
                }
            }
        }
        __syncthreads();
        if (tid < kRouterRows * kMaxTok) {
            const int rr = tid >> 3, m = tid & 7;
            if (r0 + rr < p.R && m < M) {
                float v = 0.f;
#pragma unroll
                for (int sl = 0; sl < kRouterSlices; ++sl) v += ctl.rpart[rr + sl * kRouterRows][m];
                if (p.router_bias != nullptr && r0 + rr < p.E) v += p.router_bias[r0 + rr];
                p.logits[(int64_t)m * p.R + r0 + rr] = v;
            }
        }
        __syncthreads();
    }
    stamp(p.sync, 2);
    grid_arrive(&counters[0]);
    if (!grid_wait(&counters[0], &counters[3], ctl)) goto abort;
    stamp(p.sync, 3);

    // Phase 2a: routing (one warp per token), groups, partition.
    if (warp < M) route_token<NV>(p, ctl, warp, lane, blockIdx.x == 0);  // NV * 32 >= E
    __syncthreads();
    stamp(p.sync, 4);
    build_groups(p, ctl, tid);
    stamp(p.sync, 5);

    {
        // ---- phase 2b: gate/up. Units = (tile, chunk) over this CTA's tiles, split evenly over the warps. ----
        const int C = d / 128, TPG = I / 8;
        const int t_lo = ctl.gu_lo, nt = ctl.gu_hi - ctl.gu_lo, U = nt * C;
        const int u_lo = (warp * U) / kWarps, u_hi = ((warp + 1) * U) / kWarps;
        const uint32_t bg = smem_off(xs) + g * 64, q0 = smem_off(xq) + (2 * t) * 4;
        int n_part = 0;  // a warp's range has at most two pieces of tiles it does not own whole: its first and its last
        if (lane == 0) ctl.wtile[warp][0] = -1, ctl.wtile[warp][1] = -1;
        for (int u = u_lo; u < u_hi;) {
            const int tl = u / C, c0 = u - tl * C;
            const int c1 = (u_hi - u) < (C - c0) ? c0 + (u_hi - u) : C;
            const int tile = t_lo + tl, gi = tile / TPG, jb = tile - gi * TPG;
            const Group &grp = ctl.groups[gi];
            const float4 tot = run_tile<false, FM>(grp, jb * 8 + g, I + jb * 8 + g, d, c0, c1, t, bg, q0, q0 + 4);
            if (c0 == 0 && c1 == C) {
                finish_gate_up<T>(p, grp, jb, tot, lane);
            } else {
                *reinterpret_cast<float4 *>(part + ((warp * 2 + n_part) * 32 + lane) * kPartFloats) = tot;
                if (lane == 0) ctl.wtile[warp][n_part] = tl;
                ++n_part;
            }
            u += c1 - c0;
        }
        __syncthreads();
        // tiles computed in pieces: the pieces (in warp order = ascending K) meet in the warp the tile number picks
        {
            const int32_t *wt = &ctl.wtile[0][0];
            int prev = -1;
            for (int e = 0; e < 2 * kWarps; ++e) {
                const int tl = wt[e];
                if (tl < 0 || tl == prev) continue;
                prev = tl;
                if (tl % kWarps != warp) continue;
                float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int e2 = e; e2 < 2 * kWarps; ++e2) {
                    if (wt[e2] < 0) continue;
                    if (wt[e2] != tl) break;
                    const float4 v = *reinterpret_cast<const float4 *>(part + (e2 * 32 + lane) * kPartFloats);
                    tot.x += v.x, tot.y += v.y, tot.z += v.z, tot.w += v.w;
                }
                const int tile = t_lo + tl, gi = tile / TPG;
                finish_gate_up<T>(p, ctl.groups[gi], tile - gi * TPG, tot, lane);
            }
        }
    }
    // the h records written above are read by other CTAs (through the copy engine) after the barrier
    asm volatile("fence.proxy.async;" ::: "memory");
    stamp(p.sync, 6);
    grid_arrive(&counters[1]);
    if (!grid_wait(&counters[1], &counters[3], ctl)) goto abort;
    stamp(p.sync, 7);

    {
        // ---- phase 3: down projection + combine. The x records are dead: the h records take their place. ----
        const int NG = ctl.n_groups, Cd = I / 128;
        const uint32_t h_bytes = (uint32_t)p.n_rec * (uint32_t)p.rec_bytes;
        if (tid == 0) {
            asm volatile("fence.proxy.async;" ::: "memory");
            mbar_expect_tx(&ctl.bar, h_bytes);
            for (uint32_t off = 0; off < h_bytes; off += 32768u) {
                const uint32_t n = h_bytes - off < 32768u ? h_bytes - off : 32768u;
                bulk_g2s(hs + off, p.hrec + off, n, &ctl.bar);
            }
        }
        for (int i = tid; i < p.rec_bytes / 16; i += kThreads)  // the all-zero record behind the real ones: columns with no token
            *reinterpret_cast<uint4 *>(hs + (size_t)p.n_rec * p.rec_bytes + i * 16) = make_uint4(0, 0, 0, 0);
        if (tid == 0) {
            bool ok = false;
            for (uint32_t i = 0; i < kSpinLimit; ++i)
                if (mbar_try_wait(&ctl.bar, 0)) {
                    ok = true;
                    break;
                }
            if (!ok) ctl.abort_flag = 0x107;
        }
        __syncthreads();
        if (ctl.abort_flag) goto abort;
        // sums of every record over each 64-code half of every chunk: what the minimum term needs
        for (int i = tid; i < (p.n_rec + 1) * Cd * 2; i += kThreads) {
            const int rec = i / (Cd * 2), rem = i - rec * (Cd * 2), c = rem >> 1, half = rem & 1;
            const uint8_t *rp = hs + (size_t)rec * p.rec_bytes;
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w)
#pragma unroll
                for (int tt = 0; tt < 2; ++tt) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(rp + ((c * 4 + w) * 4 + 2 * half + tt) * 16);
                    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) s += f16_to_f32((uint16_t)(w4[j] & 0xffffu)) + f16_to_f32((uint16_t)(w4[j] >> 16));
                }
            hq[i] = s;
        }
        __syncthreads();
        stamp(p.sync, 8);

        const int n_blocks = d / 16;
        int nb_local = 0;
        if ((int)blockIdx.x < n_blocks) nb_local = (n_blocks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1;
        const int per_block = NG * Cd, U = nb_local * per_block;
        const int u_lo = (warp * U) / kWarps, u_hi = ((warp + 1) * U) / kWarps;
        float yr[4] = {0.f, 0.f, 0.f, 0.f}, ysh[4] = {0.f, 0.f, 0.f, 0.f};
        int cur = per_block > 0 ? u_lo / per_block : 0, n_part = 0;
        if (lane == 0) ctl.wtile[warp][0] = -1, ctl.wtile[warp][1] = -1;
        auto store_part = [&](int nbi) {
            float4 *dst = reinterpret_cast<float4 *>(part + ((warp * 2 + n_part) * 32 + lane) * kPartFloats);
            dst[0] = make_float4(yr[0], yr[1], yr[2], yr[3]);
            if (kPartFloats == 8) dst[1] = make_float4(ysh[0], ysh[1], ysh[2], ysh[3]);
            if (lane == 0) ctl.wtile[warp][n_part] = nbi;
            ++n_part;
        };
        for (int u = u_lo; u < u_hi;) {
            const int nbi = u / per_block, rem = u - nbi * per_block;
            const int gi = rem / Cd, c0 = rem - gi * Cd;
            const int c1 = (u_hi - u) < (Cd - c0) ? c0 + (u_hi - u) : Cd;
            if (nbi != cur) {
                store_part(cur);
#pragma unroll
                for (int i = 0; i < 4; ++i) yr[i] = 0.f, ysh[i] = 0.f;
                cur = nbi;
            }
            const Group &grp = ctl.groups[gi];
            const bool is_sh = grp.expert == -2;
            // the record behind MMA column n: the token's (and plane's) h for this group, or the zero record
            auto rec_of = [&](int n) {
                const int tok = p.planes == 2 ? (n & 3) : n, pl = p.planes == 2 ? (n >> 2) : 0;
                if (tok >= M || !(grp.mask >> tok & 1u)) return p.n_rec;
                return (is_sh ? M * A + tok : tok * A + grp.slot_a[tok]) * p.planes + pl;
            };
            auto coef_of = [&](int n) {
                const int tok = p.planes == 2 ? (n & 3) : n;
                if (tok >= M || !(grp.mask >> tok & 1u)) return 0.f;
                return is_sh ? 1.f : ctl.coef[tok * A + grp.slot_a[tok]];  // the shared expert's gate comes after its own rounding
            };
            const int rA = ((int)blockIdx.x + nbi * (int)gridDim.x) * 16 + g;
            const float4 v = run_tile<true, FM>(grp, rA, rA + 8, I, c0, c1, t, smem_off(hs) + rec_of(g) * p.rec_bytes, smem_off(hq) + rec_of(2 * t) * Cd * 8,
                                            smem_off(hq) + rec_of(2 * t + 1) * Cd * 8);
            if (is_sh) {
                ysh[0] += v.x, ysh[1] += v.y, ysh[2] += v.z, ysh[3] += v.w;
            } else {
                const float cf0 = coef_of(2 * t), cf1 = coef_of(2 * t + 1);
                yr[0] = fmaf(cf0, v.x, yr[0]), yr[1] = fmaf(cf1, v.y, yr[1]), yr[2] = fmaf(cf0, v.z, yr[2]), yr[3] = fmaf(cf1, v.w, yr[3]);
            }
            u += c1 - c0;
        }
        if (u_hi > u_lo) store_part(cur);
        __syncthreads();
        stamp(p.sync, 9);
        // output: thread (row r, token) sums the warps' pieces of its row block in warp order
        if (tid < 128) {
            const int r = tid >> 3, tok = tid & 7;
            if (tok < M) {
                const int ln = 4 * (r & 7) + (tok >> 1), rg = (r >> 3) * 2 + (tok & 1);
                T *y = static_cast<T *>(p.y);
                for (int nbi = 0; nbi < nb_local; ++nbi) {
                    float v = 0.f, sv = 0.f;
                    const int32_t *wt = &ctl.wtile[0][0];
                    for (int e = 0; e < 2 * kWarps; ++e) {
                        if (wt[e] != nbi) continue;
                        const float *pp = part + (e * 32 + ln) * kPartFloats;
                        v += pp[rg];
                        if (p.planes == 2) v += pp[2 * kPartFloats + rg];  // the remainder plane: two lanes up
                        if (kPartFloats == 8) {
                            sv += pp[4 + rg];
                            if (p.planes == 2) sv += pp[2 * kPartFloats + 4 + rg];
                        }
                    }
                    if (p.shared_mode == STRIX_SHARED_SEPARATE) v = as_stored(v, y) + ctl.gate[tok] * as_stored(sv, y);  // as moe_shared_add
                    if (ctl.failed_mask >> tok & 1u) v = qnan();
                    st_act(y, (int64_t)tok * d + ((int)blockIdx.x + nbi * (int)gridDim.x) * 16 + r, v);
                }
            }
        }
    }

    // The last CTA out zeroes the barrier words for the next launch.
    __syncthreads();
    stamp(p.sync, 10);
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&counters[2], 1u) == gridDim.x - 1) {
            counters[0] = 0, counters[1] = 0, counters[2] = 0;
            __threadfence();
        }
    }
    return;

abort:
    // A wait ran out somewhere in the grid. Tell the others, report once, and leave; bulk copies in flight target this
    // CTA's own shared memory: sleep (bounded) until any copy issued has certainly landed before the block retires.
    __syncthreads();
    if (tid == 0) {
        atomicExch(&counters[3], 1u);
        if (atomicCAS(&p.err[3], 0u, 2u) == 0u) p.err[4] = 0xdec000u | (uint32_t)ctl.abort_flag, p.err[5] = blockIdx.x;
#pragma unroll 1
        for (uint32_t i = 0; i < (1u << 14); ++i) __nanosleep(200);
    }
    __syncthreads();
}

size_t ctl_bytes() { return (sizeof(Ctl) + 127) & ~(size_t)127; }

}  // namespace

namespace sb {

void decode_stream_set_tokens(StreamParams &p, int M) {
    p.M = M;
    p.planes = (p.act == kF32 && M <= p.two_plane_tokens) ? 2 : 1;
    p.n_rec = (M * p.A + (p.shared_mode == STRIX_SHARED_SEPARATE ? M : 0)) * p.planes;
}

int decode_stream_plan(StreamParams &p, int tokens, int min_nibble_G, int min_q8_G) {
    if (tokens < 1 || tokens > kMaxTok) return 0;
    if (p.d % 128 != 0 || p.I % 128 != 0 || p.d > 16384 || p.I > 16384) return 0;
    if (p.E > 1024 || p.k > 32 || p.A > 33 || tokens * p.A + 1 > kMaxGroups) return 0;
    if (min_nibble_G != 128) return 0;              // a quad of lanes covers 128 codes of a 4/5/6-bit row: one group
    if (min_q8_G != 64 && min_q8_G != 128) return 0;  // and 64 codes of an 8-bit row
    int dev = 0, max_smem = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (p.d / 16 > kWarps * sms) return 0;  // a warp's units span at most two row blocks
    p.rec_bytes = p.I * 2 + 64;  // 64 bytes of padding: records of different tokens start in different bank halves
    const size_t fixed = ctl_bytes() + (size_t)kWarps * 2 * 32 * (p.shared_mode == STRIX_SHARED_SEPARATE ? 8 : 4) * 4 + (size_t)(p.d / 128) * 16 * 4;
    const size_t front = (size_t)p.d * 16 + (size_t)tokens * p.d * 4;
    // FP32 activations of up to four tokens carry a second F16 plane (the rounding remainder) in the spare MMA columns, as
    // far as the h records of the widest such batch still fit in shared memory
    for (p.two_plane_tokens = p.act == kF32 ? 4 : 0; p.two_plane_tokens >= 0; --p.two_plane_tokens) {
        p.n_rec_max = 0;
        for (int m = 1; m <= tokens; ++m) {
            decode_stream_set_tokens(p, m);
            if (p.n_rec > p.n_rec_max) p.n_rec_max = p.n_rec;
        }
        const size_t back = (size_t)(p.n_rec_max + 1) * p.rec_bytes + (size_t)(p.n_rec_max + 1) * (p.I / 128) * 2 * 4;
        const size_t total = fixed + (front > back ? front : back) + 128;
        if (total <= (size_t)max_smem) {
            p.smem_bytes = (int)total;
            decode_stream_set_tokens(p, tokens);
            return 1;
        }
    }
    return 0;
}

int decode_stream_launch(const char *fn, const StreamParams &p, cudaStream_t stream) {
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev), fn);
    using KernelFn = void (*)(const StreamParams);
    // variants: activation dtype x format set x (up to 512 | up to 1024 experts)
    static const KernelFn kernels[12] = {
        decode_stream_kernel<float, kFmQ4, 16>,   decode_stream_kernel<uint16_t, kFmQ4, 16>,   decode_stream_kernel<float, kFmQ4, 32>,   decode_stream_kernel<uint16_t, kFmQ4, 32>,
        decode_stream_kernel<float, kFmQ4Q8, 16>, decode_stream_kernel<uint16_t, kFmQ4Q8, 16>, decode_stream_kernel<float, kFmQ4Q8, 32>, decode_stream_kernel<uint16_t, kFmQ4Q8, 32>,
        decode_stream_kernel<float, kFmAll, 16>,  decode_stream_kernel<uint16_t, kFmAll, 16>,  decode_stream_kernel<float, kFmAll, 32>,  decode_stream_kernel<uint16_t, kFmAll, 32>};
    static thread_local int prepared_dev = -1;
    static thread_local int prepared_bytes = 0;
    if (prepared_dev != dev || prepared_bytes < p.smem_bytes) {
        for (int a = 0; a < 12; ++a) SB_CUDA(cudaFuncSetAttribute(kernels[a], cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes), fn);
        prepared_dev = dev, prepared_bytes = p.smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count()), cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = (size_t)p.smem_bytes, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    SB_CUDA(cudaLaunchKernelEx(&cfg, kernels[p.format_set * 4 + (p.E > 512 ? 2 : 0) + (p.act == kF32 ? 0 : 1)], p), fn, ": launching the streaming decode kernel");
    return 0;
}

}  // namespace sb
