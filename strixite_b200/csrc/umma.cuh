// Device helpers shared by the tcgen05 kernels: mbarriers with bounded waits, shared-memory operand descriptors,
// the MMA / commit / fence wrappers, TMA tile loads, and the packed-code -> F16 conversions.
#pragma once

#include "common.cuh"

namespace sb {
namespace umma {

constexpr int kTileM = 128;               // MMA M: rows of one accumulator
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 0u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups of 1024 bytes; SBO = 1024 >> 4, LBO unused
// (1), descriptor version 1, layout type 2 (SWIZZLE_128B). The tile base is 1024-byte aligned.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: D = F32 (bits 4-5 = 1), A and B both F16 (format 0) or both BF16 (format 1, bits 7
// and 10), both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n, bool bf16 = false) {
    return (1u << 4) | (bf16 ? ((1u << 7) | (1u << 10)) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// The same with the A operand in tensor memory: lane = row, each 32-bit column = two consecutive K elements.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// tcgen05.commit to `bar`, with one probe of another barrier's phase started first: the probe's ~175-cycle latency runs
// under the commit's issue time instead of in front of the next wait. Returns whether `peek` had completed `parity`.
__device__ __forceinline__ bool umma_commit_and_peek(uint64_t *bar, uint64_t *peek, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%2], %3;\n\t"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(smem_u32(peek)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// (a & mask) | orv
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// A BF16 value (scale or minimum) twice, as F16 pairs.
__device__ __forceinline__ uint32_t bf16_to_h2(uint32_t b) {
    const float f = __uint_as_float(b << 16);
    return pack_h2(f, f);
}

// One 16-byte chunk (8 K elements in the order 0,4,1,5,2,6,3,7) of row r goes to chunk (j ^ (r & 7)) of the row.
__device__ __forceinline__ void st_chunk(uint8_t *tile, int r, int j, uint4 v) {
    *reinterpret_cast<uint4 *>(tile + (r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4)) = v;
}

// The 8 codes of one unit (codes 8u .. 8u + 7 of a row) as F16 pairs (0,4) (1,5) (2,6) (3,7) of code * s + m: one F16
// rounding of the exact value (the precision of the reference's served path, strixite kernels/wmma_gemm.hpp:121-128).
template <int BITS>
__device__ __forceinline__ uint4 dequant_unit(const uint8_t *row, int64_t K, int u, uint32_t s2, uint32_t m2) {
    uint32_t pr[4];
    if constexpr (BITS == 4) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(row) + u);
#pragma unroll
        for (int j = 0; j < 4; ++j) pr[j] = lop3_and_or(w >> (4 * j), 0x000F000Fu, 0x64006400u);  // F16 1024 + code
    } else {
        // codes up to 255: through FP32 (exact in F16 too), then the same F16 FMA
        int code[8];
        if constexpr (BITS == 8) {
            const uint2 w = __ldg(reinterpret_cast<const uint2 *>(row) + u);
#pragma unroll
            for (int i = 0; i < 8; ++i) code[i] = ((i < 4 ? w.x : w.y) >> (8 * (i & 3))) & 0xFF;
        } else {
            const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(row) + u);
            uint32_t hb;
            if constexpr (BITS == 5) hb = row[K / 2 + u];
            else hb = *reinterpret_cast<const uint16_t *>(row + K / 2 + 2 * u);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int hi = BITS == 5 ? ((hb >> i) & 1) : ((hb >> (2 * i)) & 3);
                code[i] = ((w >> (4 * i)) & 0xF) | (hi << 4);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) pr[j] = pack_h2((float)code[j], (float)code[j + 4]);
        uint4 o;
        o.x = h2_fma(pr[0], s2, m2), o.y = h2_fma(pr[1], s2, m2), o.z = h2_fma(pr[2], s2, m2), o.w = h2_fma(pr[3], s2, m2);
        return o;
    }
    uint4 o;
    o.x = h2_fma(h2_sub(pr[0], 0x64006400u), s2, m2);
    o.y = h2_fma(h2_sub(pr[1], 0x64006400u), s2, m2);
    o.z = h2_fma(h2_sub(pr[2], 0x64006400u), s2, m2);
    o.w = h2_fma(h2_sub(pr[3], 0x64006400u), s2, m2);
    return o;
}

// 8 consecutive activations -> F16 pairs in the order (0,4) (1,5) (2,6) (3,7). BF16 inputs convert exactly inside F16's
// normal range (the reference's served path makes the same assumption, strixite kernels/wmma_gemm.hpp:371-372).
__device__ __forceinline__ uint4 act_chunk(const uint16_t *p) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));  // (0,1) (2,3) (4,5) (6,7)
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[2 * i] = __uint_as_float(w[i] << 16), f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    uint4 o;
    o.x = pack_h2(f[0], f[4]), o.y = pack_h2(f[1], f[5]), o.z = pack_h2(f[2], f[6]), o.w = pack_h2(f[3], f[7]);
    return o;
}
__device__ __forceinline__ uint4 act_chunk(const float *p) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    uint4 o;
    o.x = pack_h2(a.x, b.x), o.y = pack_h2(a.y, b.y), o.z = pack_h2(a.z, b.z), o.w = pack_h2(a.w, b.w);
    return o;
}


__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One box of a 2-D tensor map into shared memory; completion is counted in bytes on `bar`. x = innermost coordinate.
__device__ __forceinline__ void tma_load_2d(void *dst, const void *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// The 8 codes of one 4-bit unit (a 32-bit word: nibble i = code i) as F16 pairs (0,4) (1,5) (2,6) (3,7) of code * s + m.
__device__ __forceinline__ uint4 dequant_word4(uint32_t w, uint32_t s2, uint32_t m2) {
    uint4 o;
    o.x = h2_fma(h2_sub(lop3_and_or(w, 0x000F000Fu, 0x64006400u), 0x64006400u), s2, m2);
    o.y = h2_fma(h2_sub(lop3_and_or(w >> 4, 0x000F000Fu, 0x64006400u), 0x64006400u), s2, m2);
    o.z = h2_fma(h2_sub(lop3_and_or(w >> 8, 0x000F000Fu, 0x64006400u), 0x64006400u), s2, m2);
    o.w = h2_fma(h2_sub(lop3_and_or(w >> 12, 0x000F000Fu, 0x64006400u), 0x64006400u), s2, m2);
    return o;
}
// 32 lanes x 32 consecutive FP32 columns of tensor memory: thread i of the warp gets lane (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
// 32 registers of each thread to 32 consecutive columns of its lane.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, "
        "%21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
          "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
          "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// The same for 16 columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace umma
}  // namespace sb
