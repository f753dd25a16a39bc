// Library-wide state: the thread-local error message, the version string, the cached SM count.
#include "common.cuh"

#include "strixite_b200.h"

namespace sb {

std::string &last_error() {
    thread_local std::string msg;
    return msg;
}

int sm_count() {
    // Per device: a process may drive several GPUs (one per rank is the usual case).
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace sb

extern "C" {

const char *strix_last_error(void) { return sb::last_error().c_str(); }
const char *strix_version(void) { return "strixite_b200 0.1 sm_100a"; }

}  // extern "C"
