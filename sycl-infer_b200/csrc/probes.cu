// Measurement instruments: the two ceilings the benchmark reports its kernels against and that a
// copy benchmark and a bf16 GEMM do not give - what one pass of 16-byte loads over a large buffer
// reaches (a GEMV reads, it does not copy), and what the int8 tensor-core path reaches with its
// operands resident in shared memory and nothing but MMAs in flight.  No reference counterpart.
#include "launch.h"
#include "decode.cuh"
#include "async.cuh"

namespace b200q {

__device__ int g_probe_status = 0;

// ---- read-only stream -----------------------------------------------------------------------------
__global__ void __launch_bounds__(512) probe_read_kernel(const uint4 * __restrict__ buf, size_t n16, uint32_t * sink) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    uint32_t acc = 0;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n16; i += 4 * stride) { // four independent loads in flight per thread
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[k].x), "=r"(v[k].y), "=r"(v[k].z), "=r"(v[k].w)
                         : "l"(buf + i + k * stride));
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            acc ^= v[k].x ^ v[k].y ^ v[k].z ^ v[k].w;
        }
    }
    for (; i < n16; i += stride) {
        const uint4 v = __ldg(buf + i);
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9E3779B9u) { // keeps the loads alive; practically never taken
        atomicAdd(sink, 1u);
    }
}

// ---- int8 tensor-core issue rate -------------------------------------------------------------------
// One CTA per SM.  A (128 x 32 bytes) and B (256 x 32 bytes) sit in shared memory in the K-major
// core-matrix layout; one thread issues `iters` MMAs of 128 x 256 x 32 into two accumulators of
// 256 tensor-memory columns, in batches of 32 with at most two batches in flight.
constexpr int kProbeBatch = 32;
__global__ void __launch_bounds__(128, 1) probe_i8_mma_kernel(int iters, uint32_t * sink) {
    __shared__ __align__(1024) uint8_t opA[128 * 32];
    __shared__ __align__(1024) uint8_t opB[256 * 32];
    __shared__ __align__(8) uint64_t bar[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 128 * 32 / 4; i += blockDim.x) {
        reinterpret_cast<uint32_t *>(opA)[i] = 0x01020304u * (uint32_t)(i + 1);
    }
    for (int i = threadIdx.x; i < 256 * 32 / 4; i += blockDim.x) {
        reinterpret_cast<uint32_t *>(opB)[i] = 0x04030201u * (uint32_t)(i + 7);
    }
    const uint32_t b0 = smem_u32(&bar[0]), b1 = smem_u32(&bar[1]);
    if (threadIdx.x == 0) {
        mbar_init(b0, 1);
        mbar_init(b1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async(); // the operands were written through the generic proxy
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        const uint64_t ad = smem_desc_kmajor(smem_u32(opA), 128, 256), bd = smem_desc_kmajor(smem_u32(opB), 128, 256);
        const uint32_t idesc = idesc_i8(1, 1, 128, 256);
        bool ok = true;
        int batch = 0;
        for (int it = 0; it < iters && ok; it += kProbeBatch, batch++) {
            if (batch >= 2) { // the batch that used this barrier two rounds ago has completed
                ok = mbar_wait((batch & 1) ? b1 : b0, (uint32_t)((batch >> 1) - 1) & 1u, &g_probe_status);
            }
            for (int k = 0; k < kProbeBatch; k++) {
                mma_i8(tmem + (uint32_t)((k & 1) * 256), ad, bd, idesc, k >= 2 ? 1u : 0u);
            }
            mma_commit((batch & 1) ? b1 : b0);
        }
        // everything issued has to finish before tensor memory is given back
        for (int b = batch - 2 < 0 ? 0 : batch - 2; b < batch && ok; b++) {
            ok = mbar_wait((b & 1) ? b1 : b0, (uint32_t)(b >> 1) & 1u, &g_probe_status);
        }
        if (!ok) {
            atomicAdd(sink, 1u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tmem_dealloc(tmem, 512);
    }
}

cudaError_t launch_probe_read(cudaStream_t s, const void * buf, size_t bytes, uint32_t * sink) {
    probe_read_kernel<<<kSMs * 8, 512, 0, s>>>(static_cast<const uint4 *>(buf), bytes / 16, sink);
    return cudaGetLastError();
}

cudaError_t launch_probe_i8_mma(cudaStream_t s, int iters, uint32_t * sink) {
    probe_i8_mma_kernel<<<kSMs, 128, 0, s>>>(iters, sink);
    return cudaGetLastError();
}

cudaError_t read_probe_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_probe_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_probe_status, &zero, sizeof(int));
    }
    return e;
}

} // namespace b200q
