// Activation quantizer: fp32 rows -> int8 codes per 32-value group, an f16-rounded
// fp32 scale and the two 16-value code sums.
//
// Reproduces the reference's host quantizer cpu_xq bit for bit
// (src/backend/cpu/kernels/xq.cpp:10-50 of the reference):
//   mx = max|v|; inv = 127/mx (0 for an all-zero group); q = clamp(round_half_away(v*inv), +-127)
//   scale = h2f(f2h_truncate(mx/127)) (0 for an all-zero group)
// Every fp32 operation is a single correctly rounded IEEE operation in the same order
// (no contraction, no approximate division).  With `up` the value is silu(x)*up with
// silu(x) = x / (1 + exp(-x)); exp is evaluated in double and rounded once, which equals
// a correctly rounded expf.
#include <cstdlib>

#include "launch.h"
#include "xq.cuh"

namespace b200q {

// One warp per (token, group); lane i owns element i.
__global__ void __launch_bounds__(256) xq_kernel(const float * __restrict__ x, const float * __restrict__ up,
                                                 int x_stride, int up_stride, int8_t * __restrict__ x8,
                                                 float * __restrict__ xmeta, int32_t * __restrict__ xsumq, int TB,
                                                 int G) {
    // Let a dependent GEMV launch start its prologue; it still waits for this grid to
    // finish (griddepcontrol.wait) before it reads what is written here.
    asm volatile("griddepcontrol.launch_dependents;");
    // ... and wait for the producer of x when this launch was itself chained programmatically
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= (long long)TB * G) {
        return;
    }
    const int t = (int)(w / G), g = (int)(w % G);
    float a = x[(size_t)t * x_stride + g * 32 + lane];
    if (up) {
        a = __fmul_rn(silu_exact(a), up[(size_t)t * up_stride + g * 32 + lane]);
    }
    float scale;
    int s0, s1;
    const int q = xq_group(a, lane, scale, s0, s1);
    const size_t gi = (size_t)g * TB + t;
    x8[gi * 32 + lane] = (int8_t)q;
    if (lane == 0) {
        xmeta[gi * 2] = scale;
        xmeta[gi * 2 + 1] = 0.0f;
        xsumq[gi * 2] = s0;
        xsumq[gi * 2 + 1] = s1;
    }
}

cudaError_t launch_xq(cudaStream_t s, const float * x, const float * up, int x_stride, int up_stride, int8_t * x8,
                      float * xmeta, int32_t * xsumq, int TB, int K, bool pdl_primary) {
    (void)pdl_primary;
    const int G = K / 32;
    const long long warps = (long long)TB * G;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((warps + 7) / 8));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, xq_kernel, x, up, x_stride, up_stride, x8, xmeta, xsumq, TB, G);
}

} // namespace b200q
