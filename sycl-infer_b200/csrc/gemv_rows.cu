// Warp-per-row GEMV/GEMM straight from raw GGUF blocks in global memory.
//
// The general-shape kernel of the library: any supported type per segment, any row
// count, any token count (tokens are processed TT at a time with the weights of a row
// re-read from L1/L2 for every further token tile).  Each lane owns one 32-weight part
// of a superblock, four superblocks per warp step; the per-lane fp32 partial terms are
// summed across the warp at the end of the row.
#include "decode.cuh"
#include "launch.h"

namespace b200q {

template <int TYPE, int TT>
__device__ __forceinline__ void row_tile(const uint8_t * wrow, int nb, const ActView & a, int t0, float (&acc)[TT]) {
    const int lane = threadIdx.x & 31;
    const int j = lane & 7;
#pragma unroll 2
    for (int b = lane >> 3; b < nb; b += 4) {
        Part<TYPE, GmemW> p;
        p.load(wrow + (size_t)b * Fmt<TYPE>::SB, j);
#pragma unroll
        for (int i = 0; i < TT; i++) {
            const int t = min(t0 + i, a.TB - 1);
            acc[i] += p.term(a, 8 * b, t);
        }
    }
}

template <int TT> __global__ void __launch_bounds__(256) gemv_rows_kernel(const __grid_constant__ CallDev c) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    // wait for the activation quantizer when this launch was programmatically chained to it
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (warp >= c.total_rows) {
        return;
    }
    int si = 0;
    while (si + 1 < c.n_segs && warp >= c.seg[si].row_end) {
        si++;
    }
    const SegDev & sg = c.seg[si];
    const int row = warp - (sg.row_end - sg.n_rows);
    const int nb = c.K >> 8;
    const uint8_t * wrow = sg.w + (size_t)row * nb * sb_bytes(sg.type);
    const ActView a{c.x8, c.xmeta, c.xsumq, c.TB};
    for (int t0 = 0; t0 < c.TB; t0 += TT) {
        float acc[TT];
#pragma unroll
        for (int i = 0; i < TT; i++) {
            acc[i] = 0.f;
        }
        switch (sg.type) {
        case kQ4_K: row_tile<kQ4_K, TT>(wrow, nb, a, t0, acc); break;
        case kQ5_K: row_tile<kQ5_K, TT>(wrow, nb, a, t0, acc); break;
        case kQ6_K: row_tile<kQ6_K, TT>(wrow, nb, a, t0, acc); break;
        case kIQ4_XS: row_tile<kIQ4_XS, TT>(wrow, nb, a, t0, acc); break;
        default: row_tile<kQ8_0, TT>(wrow, nb, a, t0, acc); break;
        }
#pragma unroll
        for (int i = 0; i < TT; i++) {
            acc[i] = warp_sum(acc[i]);
        }
        float mine = 0.f;
#pragma unroll
        for (int i = 0; i < TT; i++) {
            mine = lane == i ? acc[i] : mine;
        }
        if (lane < TT && t0 + lane < c.TB) {
            const size_t o = (size_t)(t0 + lane) * sg.out_stride + row;
            float v = sg.alpha * mine;
            if (sg.residual) {
                v += sg.residual[o];
            }
            store_out(c, &sg.out[o], v);
        }
    }
}

template <int TT> static cudaError_t launch_tt(cudaStream_t s, const CallDev & call, bool pdl_secondary) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((call.total_rows + 7) / 8));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_secondary ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_rows_kernel<TT>, call);
}

cudaError_t launch_gemv_rows(cudaStream_t s, const CallDev & call, bool pdl_secondary) {
    if (call.TB <= 1) {
        return launch_tt<1>(s, call, pdl_secondary);
    }
    if (call.TB <= 2) {
        return launch_tt<2>(s, call, pdl_secondary);
    }
    if (call.TB <= 4) {
        return launch_tt<4>(s, call, pdl_secondary);
    }
    return launch_tt<8>(s, call, pdl_secondary);
}

// ---- parity instrument: exact int32 per-group dots of one token -----------------------
template <int TYPE>
__device__ __forceinline__ void row_dots(const uint8_t * wrow, int nb, const ActView & a, int t, int32_t * wd) {
    const int lane = threadIdx.x & 31;
    for (int b = lane >> 3; b < nb; b += 4) {
        Part<TYPE, GmemW> p;
        p.load(wrow + (size_t)b * Fmt<TYPE>::SB, lane & 7);
        int v[Part<TYPE, GmemW>::NP], idx[Part<TYPE, GmemW>::NP];
        p.raw_dots(a, 8 * b, t, v, idx);
#pragma unroll
        for (int i = 0; i < Part<TYPE, GmemW>::NP; i++) {
            atomicAdd(wd + idx[i], v[i]); // integer adds: exact in any order
        }
    }
}

__global__ void __launch_bounds__(256) block_dots_kernel(const uint8_t * w, int type, int K, int n_rows,
                                                         const int8_t * x8, int TB, int t, int32_t * wd) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= n_rows) {
        return;
    }
    const int nb = K >> 8;
    const int D = type == kQ6_K ? K / 16 : K / 32;
    const uint8_t * wrow = w + (size_t)row * nb * sb_bytes(type);
    const ActView a{x8, nullptr, nullptr, TB};
    int32_t * o = wd + (size_t)row * D;
    switch (type) {
    case kQ4_K: row_dots<kQ4_K>(wrow, nb, a, t, o); break;
    case kQ5_K: row_dots<kQ5_K>(wrow, nb, a, t, o); break;
    case kQ6_K: row_dots<kQ6_K>(wrow, nb, a, t, o); break;
    case kIQ4_XS: row_dots<kIQ4_XS>(wrow, nb, a, t, o); break;
    default: row_dots<kQ8_0>(wrow, nb, a, t, o); break;
    }
}

cudaError_t launch_block_dots(cudaStream_t s, const uint8_t * w, int type, int K, int n_rows, const int8_t * x8,
                              int TB, int t, int32_t * wd) {
    const int D = type == kQ6_K ? K / 16 : K / 32;
    cudaError_t e = cudaMemsetAsync(wd, 0, sizeof(int32_t) * (size_t)n_rows * D, s);
    if (e != cudaSuccess) {
        return e;
    }
    block_dots_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, s>>>(w, type, K, n_rows, x8, TB, t, wd);
    return cudaGetLastError();
}

} // namespace b200q
