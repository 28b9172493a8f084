// Host-side launch interface between the C ABI (dmm_api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dmm {

struct StreamParams {
    const void *x;          // [M, K] int8 or fp16, row-major
    const void *codes;      // tiled codes
    const void *cb;         // cb64 or cb16
    void *out;              // [M, N] int32 or fp32
    void *partials;         // workspace: [grid][2][S*MB*128] accumulator values
    unsigned *tickets;      // workspace: one counter per super-strip, zero between launches
    long long M, N, K;
    float scale;            // fp16 family only (already includes the 1/4 of quarter units)
    int accumulate;
    int sign_convention;
    int cb_is_f16;
    unsigned dyn_smem_bytes;
};

// Largest number of accumulator values per CTA partial, for workspace sizing.
constexpr int kPartialValues = 512;

}  // namespace dmm
