// Grouped expert projections on the 5th-generation tensor cores (tcgen05 + tensor memory), for many-token forwards.
//
// One CTA computes D[128 weight rows, up to 128 tokens] = W_e[rows, :] * X_tile^T for one expert tile: "swap-AB" - the
// expert's output rows ride the MMA M = 128 axis and the tokens routed to the expert the N axis (a multiple of 16, so a
// ragged tile pays for at most 15 padding columns instead of rounding up to 128 rows).
//
//   warps 0-3  producers, then the epilogue. Per K block of 64: thread t dequantizes weight row t (packed codes ->
//              F16 via lop3 "1024 + code", an exact F16 subtract and one F16 FMA code * s + m: a single rounding of
//              the exact dequantized value) into the A stage, and gathers token row t of the tile (x[slot / A] or
//              h[slot]) into the B stage, both in the canonical K-major layout with the 128-byte swizzle that
//              tcgen05.mma reads. Global loads of block kb + 1 are in flight while block kb is converted.
//   warp 4     allocates 128 tensor-memory columns, then one elected lane issues tcgen05.mma (cta_group::1, kind::f16,
//              F16 x F16 -> FP32 in tensor memory) for each K block as its stage fills, and releases the stage with
//              tcgen05.commit. One CTA per tile, no cluster.
//   epilogue   tcgen05.ld 32 lanes x 32 columns per warp: lane = weight row, column = token, so for each token the 32
//              lanes store 32 consecutive output values (coalesced) to y[slot, n0 + row] or partial[slot, n0 + row].
//
// Inside every 8-element (16-byte) chunk of K both operands are stored in the order 0,4,1,5,2,6,3,7 - the order the
// nibble unpack produces - which a dot product does not care about as long as A and B agree.
// Three stages of 32 KB: two CTAs share an SM (192 KB shared memory, 2 x 128 tensor-memory columns), so one CTA's
// epilogue overlaps the other's main loop.
//
// Every mbarrier wait is bounded; on expiry the CTA raises a global abort word (strix_umma_abort_count), frees its
// tensor memory and returns.
#include "grouped.cuh"
#include "umma.cuh"

namespace {

using namespace sb;
using namespace sb::umma;

constexpr int kStages = 3;
constexpr int kBK = 64;                   // K per stage: 64 F16 = one 128-byte swizzle row
constexpr int kTileN = 128;               // token rows per CTA at most (MMA N)
constexpr int kStageBytesA = kTileM * kBK * 2, kStageBytesB = kTileN * kBK * 2;
constexpr int kThreads = 160;

__device__ unsigned int g_umma_aborts = 0;
__device__ unsigned int g_ws_refusals = 0;

struct Shared {
    uint64_t full[kStages], empty[kStages], acc_full;
    uint32_t tmem_base;
    int abort_flag;
    int32_t slots[kTileN];
};

// DENSE: no grouping workspace - one weight matrix (bucket 0) against all A = M token rows; tile blockIdx.y holds rows
// 128 * blockIdx.y .. of x, row m is "slot" m, outputs y[m, :] (COMBINE selects the FP32 output array).
template <typename T, bool COMBINE, bool DENSE>
__global__ void __launch_bounds__(kThreads, 2)
    grouped_umma_kernel(const T *x, StackView w, const int32_t *ws, int64_t A, T *y, float *partial, int32_t S_call, int32_t E_call) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    int32_t E = 1, bucket = 0, st = 0;
    int rows = 0;
    RouteTables rt{};
    if constexpr (DENSE) {
        st = (int32_t)blockIdx.y * kTileN;
        rows = (int)min((int64_t)kTileN, A - st);
    } else {
        if (!ws_is_for(ws, S_call, E_call, &g_ws_refusals)) return;
        const int32_t S = S_call, n_wtiles = ws[3];
        E = E_call;
        const int wt = blockIdx.y;
        if (wt >= n_wtiles) return;
        rt = route_tables(ws, S, E);
        bucket = rt.wtile_bucket[wt], st = rt.wtile_start[wt];
        const int32_t b0 = rt.offsets[bucket], b1 = rt.offsets[bucket + 1];
        if ((st - b0) % kTileN != 0) return;  // the 64-slot tile tables: every other tile of a bucket starts a 128-slot tile
        rows = min(kTileN, b1 - st);
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t N = w.N, K = w.K;
    const int64_t n0 = (int64_t)blockIdx.x * kTileM;
    const int rows_w = (int)(N - n0 < kTileM ? N - n0 : kTileM);

    if (!DENSE && bucket == E) {  // invalid ids: NaN outputs (the grouping raised err)
        for (int i = tid; i < rows * rows_w; i += kThreads) {
            const int r = i / rows_w, c = i - r * rows_w;
            const int64_t slot = rt.slots[st + r];
            if (COMBINE) partial[slot * N + n0 + c] = qnan();
            else st_act(y, slot * N + n0 + c, qnan());
        }
        return;
    }

    // shared memory: [stages][A 16 KB | B 16 KB] on a 1024-byte boundary, then the control block
    uint8_t *tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Shared &sh = *reinterpret_cast<Shared *>(tiles + kStages * (kStageBytesA + kStageBytesB));
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&sh.full[s], 128), mbar_init(&sh.empty[s], 1);
        mbar_init(&sh.acc_full, 1);
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < kTileN) sh.slots[tid] = tid < rows ? (DENSE ? st + tid : rt.slots[st + tid]) : -1;
    if (warp == 4) {  // tensor memory: 128 FP32 accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    const int nkb = (int)(K / kBK);
    const int n_mma = (rows + 15) & ~15;  // MMA N: the tile's tokens rounded up to 16

    if (warp < 4) {
        // ---- producers ----
        const int t = tid;  // weight row and token row of this thread
        const int bits = w.bits_of(bucket);
        const int64_t gpr = K / w.G;
        const bool row_ok = t < rows_w;
        const int64_t wrow = (int64_t)bucket * N + n0 + (row_ok ? t : 0);
        const uint8_t *qrow = w.rows(bucket, bits) + (n0 + (row_ok ? t : 0)) * row_bytes(bits, K);
        const uint16_t *srow = w.scale + wrow * gpr, *mrow = w.minv + wrow * gpr;
        const int32_t slot = sh.slots[t];
        const T *xrow = slot >= 0 ? x + ((COMBINE || DENSE) ? (int64_t)slot : (int64_t)slot / A) * K : nullptr;
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % kStages;
            const uint32_t ph = (uint32_t)(kb / kStages) & 1u;
            if (!mbar_wait(&sh.empty[s], ph ^ 1u, &sh.abort_flag)) break;
            uint8_t *ta = tiles + s * (kStageBytesA + kStageBytesB), *tb = ta + kStageBytesA;
            // A: weight row t, codes kb*64 .. +63 = 8 units
            if (row_ok) {
                by_bits(bits, [&](auto bc) {
                    constexpr int BITS = decltype(bc)::value;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int u = kb * 8 + j;
                        const int gi = (u * 8) / (int)w.G;
                        const uint32_t sb = __ldg(srow + gi), mb = __ldg(mrow + gi);
                        st_chunk(ta, t, j, dequant_unit<BITS>(qrow, K, u, bf16_to_h2(sb), bf16_to_h2(mb)));
                    }
                });
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) st_chunk(ta, t, j, make_uint4(0, 0, 0, 0));
            }
            // B: token row t of the tile
            if (t < n_mma) {
#pragma unroll
                for (int j = 0; j < 8; ++j) st_chunk(tb, t, j, xrow ? act_chunk(xrow + (int64_t)kb * kBK + j * 8) : make_uint4(0, 0, 0, 0));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core's reads
            mbar_arrive(&sh.full[s]);
        }
        // ---- epilogue: lane = weight row 32 * warp + lane, columns = tokens ----
        if (mbar_wait(&sh.acc_full, 0, &sh.abort_flag)) {
            tc_fence_after();
            const int r = warp * 32 + lane;
            for (int c0 = 0; c0 < n_mma; c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
                    "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int32_t sl = c0 + j < rows ? sh.slots[c0 + j] : -1;
                    if (sl >= 0 && r < rows_w) {
                        if (COMBINE) partial[(int64_t)sl * N + n0 + r] = __uint_as_float(v[j]);
                        else st_act(y, (int64_t)sl * N + n0 + r, __uint_as_float(v[j]));
                    }
                }
            }
        }
        tc_fence_before();
    } else {
        // ---- MMA issuer ----
        const uint32_t idesc = umma_idesc(n_mma);
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % kStages;
            const uint32_t ph = (uint32_t)(kb / kStages) & 1u;
            if (lane == 0) ok = mbar_wait(&sh.full[s], ph, &sh.abort_flag);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a0 = smem_u32(tiles + s * (kStageBytesA + kStageBytesB)), b0a = a0 + kStageBytesA;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)  // 16 K elements = 32 bytes further inside the swizzled row
                    umma_f16(tmem, umma_desc(a0 + k * 32), umma_desc(b0a + k * 32), idesc, (kb | k) ? 1u : 0u);
                umma_commit(&sh.empty[s]);  // the stage is free once these MMAs have read it
            }
            __syncwarp();
        }
        if (lane == 0 && ok) umma_commit(&sh.acc_full);
        tc_fence_before();
    }
    __syncthreads();
    if (tid == 0 && sh.abort_flag) atomicAdd(&g_umma_aborts, 1u);
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

constexpr size_t kSmem = (size_t)kStages * (kStageBytesA + kStageBytesB) + sizeof(Shared) + 1024;
int prepare(const char *fn, size_t smem) {
    static thread_local int prepared_dev = -1;
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev), fn);
    if (prepared_dev != dev) {
        SB_CUDA(cudaFuncSetAttribute(grouped_umma_kernel<float, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(grouped_umma_kernel<float, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(grouped_umma_kernel<uint16_t, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(grouped_umma_kernel<uint16_t, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(grouped_umma_kernel<float, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(grouped_umma_kernel<uint16_t, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        SB_CUDA(cudaFuncSetAttribute(grouped_umma_kernel<uint16_t, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), fn);
        prepared_dev = dev;
    }
    return 0;
}
}  // namespace

namespace sb {

// y[M, N] = x[M, K] * dequant(W)^T for one quantized matrix on the tensor cores (the dense twin of the grouped projection:
// strixite kernels/linear_wmma.hpp:21-24). out_act == act, or BF16 x -> F32 y.
int dense_umma(const char *fn, const void *x, const StackView &w, int64_t M, void *y, int act, int out_act, cudaStream_t stream) {
    SB_CHECK(w.K % kBK == 0, fn, ": K = ", w.K, ", expected a multiple of ", kBK);
    SB_CHECK(out_act == act || (act == kBF16 && out_act == kF32), fn, ": out_act ", act_name(out_act), " for ", act_name(act), " inputs (same, or BF16 -> F32)");
    const int64_t tiles = (M + kTileN - 1) / kTileN;
    SB_CHECK(M >= 1 && tiles <= 65535, fn, ": M = ", M);
    SB_TRY(prepare(fn, kSmem));
    const dim3 grid((unsigned)((w.N + kTileM - 1) / kTileM), (unsigned)tiles), block(kThreads);
    if (act == kF32) grouped_umma_kernel<float, false, true><<<grid, block, kSmem, stream>>>((const float *)x, w, nullptr, M, (float *)y, nullptr, 0, 0);
    else if (out_act == kF32) grouped_umma_kernel<uint16_t, true, true><<<grid, block, kSmem, stream>>>((const uint16_t *)x, w, nullptr, M, nullptr, (float *)y, 0, 0);
    else grouped_umma_kernel<uint16_t, false, true><<<grid, block, kSmem, stream>>>((const uint16_t *)x, w, nullptr, M, (uint16_t *)y, nullptr, 0, 0);
    SB_LAUNCH_OK(fn, " M=", M, " N=", w.N, " K=", w.K, " G=", w.G);
    return 0;
}

int grouped_umma(const char *fn, const void *x, const StackView &w, const int32_t *ws, int64_t M, int64_t A, int64_t E, void *y, float *partial,
                 int act, bool combine, cudaStream_t stream) {
    SB_CHECK(w.K % kBK == 0, fn, " (tensor cores): K = ", w.K, ", expected a multiple of ", kBK);
    const int64_t S = M * A;
    const size_t smem = kSmem;
    SB_TRY(prepare(fn, smem));
    // grid.y covers the 64-slot tile table's capacity (S / 64 + E + 2 with E <= 1023); CTAs past the live tiles return at once
    const int64_t wtmax = S / 64 + 1023 + 2;
    SB_CHECK(wtmax <= 65535, fn, " (tensor cores): ", wtmax, " tile slots exceed the grid");
    const dim3 grid((unsigned)((w.N + kTileM - 1) / kTileM), (unsigned)wtmax), block(kThreads);
    if (act == kF32) {
        if (combine) grouped_umma_kernel<float, true, false><<<grid, block, smem, stream>>>((const float *)x, w, ws, A, nullptr, partial, (int32_t)(M * A), (int32_t)E);
        else grouped_umma_kernel<float, false, false><<<grid, block, smem, stream>>>((const float *)x, w, ws, A, (float *)y, nullptr, (int32_t)(M * A), (int32_t)E);
    } else {
        if (combine) grouped_umma_kernel<uint16_t, true, false><<<grid, block, smem, stream>>>((const uint16_t *)x, w, ws, A, nullptr, partial, (int32_t)(M * A), (int32_t)E);
        else grouped_umma_kernel<uint16_t, false, false><<<grid, block, smem, stream>>>((const uint16_t *)x, w, ws, A, (uint16_t *)y, nullptr, (int32_t)(M * A), (int32_t)E);
    }
    SB_LAUNCH_OK(fn, " (tensor cores) M=", M, " A=", A, " N=", w.N, " K=", w.K, " G=", w.G);
    return 0;
}

unsigned int grouped_umma_ws_refusals() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_ws_refusals, sizeof(v));
    return v;
}

unsigned int grouped_umma_aborts() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_umma_aborts, sizeof(v));
    return v;
}

}  // namespace sb
