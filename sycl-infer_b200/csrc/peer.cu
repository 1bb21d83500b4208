// Cross-GPU barrier for row-sharded calls: one warp, lane p talks to rank p.
//
// Signal: after a system-scope fence (the GEMV that ran before this kernel in the stream has
// stored its rows into the peers' buffers), store `seq` into word `rank` of every peer's flag
// array.  Wait: poll the local flag words until every peer's word has reached `seq`.  The poll
// is bounded by a clock budget; when it runs out the status word is set and the kernel returns,
// so a peer that died or never launched cannot hang this GPU.  Plain ld/st with .sys scope over
// NVLink peer mappings; no multimem, no multicast.
#include "async.cuh"
#include "launch.h"

namespace b200q {

__device__ int g_peer_status = 0;

struct PeerFlags {
    uint32_t * p[B200Q_MAX_PEERS + 1];
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const __grid_constant__ PeerFlags f, int world, int rank,
                                                          uint32_t seq) {
    const int p = threadIdx.x;
    if (seq == 0) { // count the barriers on the device: word 32 of this rank's own flag array
        uint32_t v = 0;
        if (p == 0) {
            v = atomicAdd(f.p[rank] + 32, 1u) + 1u;
        }
        seq = __shfl_sync(0xFFFFFFFFu, v, 0);
    }
    __threadfence_system();
    if (p < world && p != rank) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.p[p] + rank), "r"(seq) : "memory");
    }
    if (p < world && p != rank) {
        const uint32_t * mine = f.p[rank] + p;
        const long long t0 = clock64();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - seq) >= 0) {
                break;
            }
            if (clock64() - t0 > kSpinCycles) {
                atomicExch(&g_peer_status, B200Q_ETIMEOUT);
                break;
            }
        }
    }
    __threadfence_system();
}

cudaError_t launch_peer_barrier(cudaStream_t s, uint32_t * const * flags, int world, int rank, uint32_t seq) {
    PeerFlags f = {};
    for (int i = 0; i < world; i++) {
        f.p[i] = flags[i];
    }
    peer_barrier_kernel<<<1, 32, 0, s>>>(f, world, rank, seq);
    return cudaGetLastError();
}

cudaError_t read_peer_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_peer_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int));
    }
    return e;
}

} // namespace b200q
