// Placeholder until the tcgen05 grouped GEMM lands: the tensor-core math modes are refused loudly.
#include "grouped.cuh"

namespace sb {

int grouped_umma(const char *fn, const void *, const StackView &, const int32_t *, int64_t, int64_t, void *, float *, int, bool,
                 cudaStream_t) {
    SB_CHECK(false, fn, ": the tensor-core grouped GEMM is not built in this library yet; use math = F32");
    return 0;
}

}  // namespace sb
