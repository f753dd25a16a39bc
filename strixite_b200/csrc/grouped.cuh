// Shared between the grouping, the FP32 grouped kernels and the tensor-core grouped GEMM: the workspace tables and
// the tensor-core entry.
#pragma once

#include "common.cuh"

namespace sb {

struct RouteTables {
    const int32_t *offsets, *slots, *tile_bucket, *tile_start, *wtile_bucket, *wtile_start;
};
// The tables inside a grouping workspace for S slots over E experts.
__host__ __device__ inline RouteTables route_tables(const int32_t *ws, int64_t S, int64_t E) {
    const int64_t Tmax = S / 16 + E + 2, WTmax = S / 64 + E + 2;
    RouteTables t;
    t.offsets = ws + 4;
    t.slots = t.offsets + E + 2;
    t.tile_bucket = t.slots + S;
    t.tile_start = t.tile_bucket + Tmax;
    t.wtile_bucket = t.tile_start + Tmax;
    t.wtile_start = t.wtile_bucket + WTmax;
    return t;
}

// A workspace grouped for another (slots, experts) than the caller states must not drive a single store: its tables would index
// past the caller's buffers. Kernels that read a workspace call this first and return when it fails; one thread counts the refusal.
__device__ __forceinline__ bool ws_is_for(const int32_t *ws, int64_t S, int64_t E, unsigned int *refusals) {
    if (ws[1] == S && ws[2] == E) return true;
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) atomicAdd(refusals, 1u);
    return false;
}

// The grouping of moe_group_routes over many blocks, for callers that own a scratch buffer of route_scratch_bytes(E) bytes
// (initialized once with route_scratch_init; one buffer per stream that groups): same workspace contents as the public
// single-block entry, bit for bit. quiet: ids of -2 are absent slots - invalid bucket, no error.
size_t route_scratch_bytes(int64_t E);
int route_scratch_init(void *scratch, int64_t E, cudaStream_t stream);
int group_routes_multi(const char *fn, const int32_t *ids, int64_t S, int64_t E, int32_t *ws, int32_t *scratch, uint32_t *err, bool quiet,
                       cudaStream_t stream);

// Tensor-core grouped projection over a grouping workspace (grouped_umma.cu). combine = false: inputs x[slot / A],
// outputs y[slot, :] in the activation dtype. combine = true: inputs h[slot], outputs FP32 partial[slot, :].
int grouped_umma(const char *fn, const void *x, const StackView &w, const int32_t *ws, int64_t M, int64_t A, int64_t E, void *y,
                 float *partial, int act, bool combine, cudaStream_t stream);

// One quantized matrix [N, K] against M token rows on the same kernel: y[M, N] in `out_act` (act, or F32 for BF16 inputs).
int dense_umma(const char *fn, const void *x, const StackView &w, int64_t M, void *y, int act, int out_act, cudaStream_t stream);

// Launches refused because the workspace was grouped for other sizes than the call states (0 in a healthy run).
unsigned int grouped_umma_ws_refusals();

// CTAs of the tensor-core grouped GEMM that gave up on a bounded wait since the library was loaded (0 in a healthy run).
unsigned int grouped_umma_aborts();

}  // namespace sb
