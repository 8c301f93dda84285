// Process-wide switches of the kernel library.
#include "common.cuh"

int gesso_pdl_enabled = 1;

// Programmatic dependent launch for the kernels of decoding steps (on by default).
GESSO_API int gesso_set_pdl(int enabled) {
    const int before = gesso_pdl_enabled;
    gesso_pdl_enabled = enabled ? 1 : 0;
    return before;
}

// Streaming multiprocessors of the current device (asked once per device; 148 on a B200).  Grids of
// persistent kernels are sized from it.
GESSO_API int gesso_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = n;
    }
    return cached[dev];
}
