// Shared helpers of libtiny_llm_b200_blocks.so (see include/tiny_llm_b200_blocks.h).
#pragma once

#include "../common.cuh"
#include "../../../include/tiny_llm_b200_blocks.h"

namespace tlb {

using tl::as_stream;
using tl::ceil_div;
using tl::from_f;
using tl::to_f;
using tl::warp_max;
using tl::warp_sum;

typedef __nv_bfloat16 bf16;

// Sum over a CTA of `blockDim.x` threads (a multiple of 32, at most 1024); every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float *scratch /* [33] */) {
    v = warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// cos / sin of position * base^(-2 i / dims), evaluated in double so that the angle is exact at any position.
__device__ __forceinline__ void rope_angle(int pos, int i, int dims, double log2_base, float &c, float &s) {
    double freq = exp2(-2.0 * (double)i / (double)dims * log2_base);
    double sn, cs;
    sincos((double)pos * freq, &sn, &cs);
    c = (float)cs;
    s = (float)sn;
}

}  // namespace tlb

#define TLB_DISPATCH(dtype, name, ...)                                               \
    do {                                                                             \
        if ((dtype) == TL_F32) { using T = float; __VA_ARGS__; }                     \
        else if ((dtype) == TL_BF16) { using T = ::tlb::bf16; __VA_ARGS__; }         \
        else return ::tl::fail(TL_EDTYPE, "%s: dtype must be float32 or bfloat16", name); \
    } while (0)
