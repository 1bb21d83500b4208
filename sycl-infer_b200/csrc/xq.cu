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
#include <cstring>

#include "async.cuh"
#include "launch.h"
#include "xq.cuh"

namespace b200q {

__device__ int g_xq_status = 0;

// One warp per (token, group); lane i owns element i.
__global__ void __launch_bounds__(256) xq_kernel(const float * __restrict__ x, const float * __restrict__ up,
                                                 int x_stride, int up_stride, int8_t * __restrict__ x8,
                                                 float * __restrict__ xmeta, int32_t * __restrict__ xsumq, int TB,
                                                 int G, const __grid_constant__ PeerSync sync) {
    // Let a dependent GEMV launch start its prologue; it still waits for this grid to
    // finish (griddepcontrol.wait) before it reads what is written here.
    asm volatile("griddepcontrol.launch_dependents;");
    // ... and wait for the producer of x when this launch was itself chained programmatically
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (sync.wait) {
        // row-sharded calls: x holds rows the peers stored; wait (bounded) until every peer has
        // signalled as often as this rank has
        if (threadIdx.x < (unsigned)sync.world && (int)threadIdx.x != sync.rank) {
            const uint32_t * own = sync.flag[sync.rank];
            uint32_t expected;
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(expected) : "l"(own + 32) : "memory");
            const long long t0 = clock64();
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(own + threadIdx.x) : "memory");
                if ((int32_t)(v - expected) >= 0) {
                    break;
                }
                if (clock64() - t0 > kSpinCycles) {
                    atomicExch(&g_xq_status, B200Q_ETIMEOUT);
                    break;
                }
            }
        }
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= (long long)TB * G) {
        return;
    }
    const int t = (int)(w / G), g = (int)(w % G);
    float a = __ldcg(x + (size_t)t * x_stride + g * 32 + lane); // through L2: peers may have stored it
    if (up) {
        a = __fmul_rn(silu_exact(a), __ldcg(up + (size_t)t * up_stride + g * 32 + lane));
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
                      float * xmeta, int32_t * xsumq, int TB, int K, bool pdl_primary, const PeerSync * wait_for) {
    (void)pdl_primary;
    PeerSync sync;
    memset(&sync, 0, sizeof(sync));
    if (wait_for) {
        sync = *wait_for;
        sync.signal = 0;
    }
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
    return cudaLaunchKernelEx(&cfg, xq_kernel, x, up, x_stride, up_stride, x8, xmeta, xsumq, TB, G, sync);
}

cudaError_t read_xq_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_xq_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_xq_status, &zero, sizeof(int));
    }
    return e;
}

} // namespace b200q
