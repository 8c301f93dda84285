// Process-wide switches of the kernel library.
#include "common.cuh"

int gesso_pdl_enabled = 1;

// Programmatic dependent launch for the kernels of decoding steps (on by default).
GESSO_API int gesso_set_pdl(int enabled) {
    const int before = gesso_pdl_enabled;
    gesso_pdl_enabled = enabled ? 1 : 0;
    return before;
}
