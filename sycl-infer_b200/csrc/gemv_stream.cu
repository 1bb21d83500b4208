// Streaming decode GEMV for 1..8 tokens: the HBM-bound kernel of the library.
//
// Data movement.  The raw GGUF block stream of 8 consecutive weight rows x KB superblocks
// is brought into shared memory by bulk asynchronous copies (cp.async.bulk, the 1-D TMA
// path, no multicast) that complete on an mbarrier; a ring of STAGES such tiles keeps
// ~100 KB per CTA in flight so the copy engine, not the warps, hides HBM latency.  A copy
// must start on a 16-byte boundary and be a multiple of 16 bytes long: a row segment that
// starts at address A is fetched from A & ~15 and decoded from offset A & 15 inside its
// slot (Q6_K rows are only 2-byte aligned, IQ4_XS 8); the bytes read beyond either end lie
// in the same 16-byte line as valid bytes, so they are always mapped.
//
// Roles.  Warp 8 is the producer: lane r issues the copy of row r of the tile.  Warps 0..7
// are consumers: warp w owns row w of the tile for the whole K loop, so a row's partial
// sums stay in registers and no cross-warp reduction exists.  Inside a tile lane l owns
// part (l & 7) of superblocks (l >> 3), (l >> 3) + 4, ...  The quantized activation of a
// single-token call is staged once per CTA in shared memory; for 2..8 tokens it is read
// through L1.
//
// Every wait on an mbarrier is bounded; a wait that runs out records an error status the
// host can read (b200q_device_status) and the CTA leaves its loop.
#include <type_traits>

#include "decode.cuh"
#include "launch.h"

namespace b200q {

constexpr int kRowsPerTile = 8;
constexpr int kConsumerWarps = 8;
constexpr int kStreamThreads = 32 * (kConsumerWarps + 1);
constexpr long long kSpinCycles = 2000000000LL; // about one second of SM clocks

__device__ int g_device_status = 0;

struct StreamArgs {
    CallDev c;
    int32_t grp_end[B200Q_MAX_SEGS]; // exclusive prefix of 8-row groups per segment
    int32_t n_groups;
    int32_t kb_max;     // superblocks per tile along K
    int32_t slot_bytes; // shared bytes reserved per row of a tile
    int32_t stages;
};

// ---- mbarrier / bulk-copy primitives (PTX) --------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) {
            return true;
        }
        if (clock64() - t0 > kSpinCycles) {
            break;
        }
    }
    atomicExch(&g_device_status, B200Q_ETIMEOUT);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared-memory layout: barriers | ring of tiles | staged activation (single token only)
struct Smem {
    uint32_t full, empty, tiles, x8, xmeta, xsumq;
};
__device__ __forceinline__ Smem smem_layout(const StreamArgs & a, uint32_t base, bool stage_x) {
    Smem m;
    m.full = base;
    m.empty = base + 64;
    m.tiles = base + 128;
    m.x8 = m.tiles + (uint32_t)(a.stages * kRowsPerTile * a.slot_bytes);
    m.xmeta = m.x8 + (stage_x ? (uint32_t)a.c.K : 0u);
    m.xsumq = m.xmeta + (stage_x ? (uint32_t)(a.c.K / 32 * 8) : 0u);
    return m;
}

// One warp, one row, one tile: every lane walks its parts and adds the fp32 terms.
template <int TYPE, int TT, class AM>
__device__ __forceinline__ void consume_tile(const uint8_t * seg, int kb, int sb0, const ActView & act,
                                             float (&acc)[TT]) {
    const int lane = threadIdx.x & 31;
    const int j = lane & 7;
    for (int b = lane >> 3; b < kb; b += 4) {
        Part<TYPE, SmemW> p;
        p.load(seg + b * Fmt<TYPE>::SB, j);
#pragma unroll
        for (int i = 0; i < TT; i++) {
            const int t = TT == 1 ? 0 : min(i, act.TB - 1);
            acc[i] += p.template term<AM>(act, 8 * (sb0 + b), t);
        }
    }
}

template <int TT>
__global__ void __launch_bounds__(kStreamThreads, 2) gemv_stream_kernel(const __grid_constant__ StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr bool kStageX = (TT == 1);
    using AM = typename std::conditional<kStageX, SmemA, GmemA>::type;
    const uint32_t base = smem_u32(smem_raw);
    const Smem sm = smem_layout(a, base, kStageX);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = a.c.K >> 8;
    const int n_chunks = (nb + a.kb_max - 1) / a.kb_max;
    const int S = a.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(sm.full + 8 * s, 1);
            mbar_init(sm.empty + 8 * s, kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer
        uint32_t it = 0;
        bool alive = true;
        for (int g = blockIdx.x; g < a.n_groups && alive; g += gridDim.x) {
            int si = 0;
            while (si + 1 < a.c.n_segs && g >= a.grp_end[si]) {
                si++;
            }
            const SegDev & sg = a.c.seg[si];
            const int row0 = (g - (si ? a.grp_end[si - 1] : 0)) * kRowsPerTile;
            const int rows = min(kRowsPerTile, sg.n_rows - row0);
            const int sbb = sb_bytes(sg.type);
            const size_t row_bytes = (size_t)nb * sbb;
            for (int ch = 0; ch < n_chunks && alive; ch++, it++) {
                const int stage = it % S;
                const uint32_t par = ((it / S) & 1) ^ 1;
                const int sb0 = ch * a.kb_max;
                const int kb = min(a.kb_max, nb - sb0);
                uint32_t len = 0;
                const uint8_t * src = nullptr;
                if (lane < rows) {
                    const uint8_t * p = sg.w + (size_t)(row0 + lane) * row_bytes + (size_t)sb0 * sbb;
                    const uintptr_t A = reinterpret_cast<uintptr_t>(p);
                    const uintptr_t A0 = A & ~uintptr_t(15);
                    len = (uint32_t)(((A + (size_t)kb * sbb + 15) & ~uintptr_t(15)) - A0);
                    src = reinterpret_cast<const uint8_t *>(A0);
                }
                uint32_t total = len;
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) {
                    total += __shfl_xor_sync(0xFFFFFFFFu, total, o);
                }
                alive = mbar_wait(sm.empty + 8 * stage, par);
                alive = __all_sync(0xFFFFFFFFu, alive);
                if (!alive) {
                    break;
                }
                if (lane == 0) {
                    mbar_expect_tx(sm.full + 8 * stage, total);
                }
                __syncwarp();
                if (lane < rows) {
                    bulk_g2s(sm.tiles + (uint32_t)((stage * kRowsPerTile + lane) * a.slot_bytes), src, len,
                             sm.full + 8 * stage);
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    // The weights above do not depend on the activation quantizer; everything below does.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    ActView act{a.c.x8, a.c.xmeta, a.c.xsumq, a.c.TB};
    if (kStageX) {
        const int tid = threadIdx.x, nthr = 32 * kConsumerWarps;
        const uint4 * gx = reinterpret_cast<const uint4 *>(a.c.x8);
        for (int i = tid; i < a.c.K / 16; i += nthr) {
            const uint4 v = __ldg(gx + i);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sm.x8 + 16 * i), "r"(v.x), "r"(v.y), "r"(v.z),
                         "r"(v.w));
        }
        const uint2 * gm = reinterpret_cast<const uint2 *>(a.c.xmeta);
        const uint2 * gs = reinterpret_cast<const uint2 *>(a.c.xsumq);
        for (int i = tid; i < a.c.K / 32; i += nthr) {
            const uint2 m = __ldg(gm + i), s = __ldg(gs + i);
            asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(sm.xmeta + 8 * i), "r"(m.x), "r"(m.y));
            asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(sm.xsumq + 8 * i), "r"(s.x), "r"(s.y));
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps) : "memory");
        act.x8 = reinterpret_cast<const int8_t *>(smem_raw + (sm.x8 - base));
        act.xmeta = reinterpret_cast<const float *>(smem_raw + (sm.xmeta - base));
        act.xsumq = reinterpret_cast<const int32_t *>(smem_raw + (sm.xsumq - base));
    }

    uint32_t it = 0;
    for (int g = blockIdx.x; g < a.n_groups; g += gridDim.x) {
        int si = 0;
        while (si + 1 < a.c.n_segs && g >= a.grp_end[si]) {
            si++;
        }
        const SegDev & sg = a.c.seg[si];
        const int row = (g - (si ? a.grp_end[si - 1] : 0)) * kRowsPerTile + warp;
        const bool valid = row < sg.n_rows;
        const int sbb = sb_bytes(sg.type);
        const uint32_t mis =
            (uint32_t)(reinterpret_cast<uintptr_t>(sg.w + (size_t)row * nb * sbb) & 15); // chunk sizes keep it
        float acc[TT];
#pragma unroll
        for (int i = 0; i < TT; i++) {
            acc[i] = 0.f;
        }
        for (int ch = 0; ch < n_chunks; ch++, it++) {
            const int stage = it % S;
            if (!mbar_wait(sm.full + 8 * stage, (it / S) & 1)) {
                return;
            }
            const int sb0 = ch * a.kb_max;
            const int kb = min(a.kb_max, nb - sb0);
            if (valid) {
                const uint32_t off = (uint32_t)((stage * kRowsPerTile + warp) * a.slot_bytes) +
                                     ((mis + (uint32_t)sb0 * sbb) & 15);
                const uint8_t * seg = smem_raw + (sm.tiles - base) + off;
                switch (sg.type) {
                case kQ4_K: consume_tile<kQ4_K, TT, AM>(seg, kb, sb0, act, acc); break;
                case kQ5_K: consume_tile<kQ5_K, TT, AM>(seg, kb, sb0, act, acc); break;
                case kQ6_K: consume_tile<kQ6_K, TT, AM>(seg, kb, sb0, act, acc); break;
                case kIQ4_XS: consume_tile<kIQ4_XS, TT, AM>(seg, kb, sb0, act, acc); break;
                default: consume_tile<kQ8_0, TT, AM>(seg, kb, sb0, act, acc); break;
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(sm.empty + 8 * stage);
            }
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
        if (valid && lane < TT && lane < a.c.TB) {
            const size_t o = (size_t)lane * sg.out_stride + row;
            float v = sg.alpha * mine;
            if (sg.residual) {
                v += sg.residual[o];
            }
            sg.out[o] = v;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------
static int kb_cap(int type) { // superblocks per tile: 8 rows x kb x SB stays near 24-27 KB
    switch (type) {
    case kQ4_K: return 20;
    case kQ5_K: return 16;
    case kQ6_K: return 16;
    case kIQ4_XS: return 24;
    default: return 12;
    }
}

template <int TT> static cudaError_t launch_stream_tt(cudaStream_t s, const StreamArgs & a, size_t smem, int grid,
                                                      bool pdl_secondary) {
    static bool configured = false; // per instantiation; setting the attribute twice is harmless
    if (!configured) {
        cudaError_t e =
            cudaFuncSetAttribute(gemv_stream_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
        if (e != cudaSuccess) {
            return e;
        }
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_secondary ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<TT>, a);
}

bool stream_supported(const CallDev & c) {
    return c.TB >= 1 && c.TB <= 8 && c.K <= 32768;
}

cudaError_t launch_gemv_stream(cudaStream_t s, const CallDev & c, bool pdl_secondary) {
    StreamArgs a;
    a.c = c;
    const int nb = c.K >> 8;
    int groups = 0, kb = 1 << 30, max_sbb = 0;
    for (int i = 0; i < c.n_segs; i++) {
        groups += (c.seg[i].n_rows + kRowsPerTile - 1) / kRowsPerTile;
        a.grp_end[i] = groups;
        kb = kb < kb_cap(c.seg[i].type) ? kb : kb_cap(c.seg[i].type);
        max_sbb = max_sbb > sb_bytes(c.seg[i].type) ? max_sbb : sb_bytes(c.seg[i].type);
    }
    a.n_groups = groups;
    if (kb < nb) { // split K into equal chunks of a multiple of 4 superblocks (all lanes busy)
        const int n_chunks = (nb + kb - 1) / kb;
        kb = (((nb + n_chunks - 1) / n_chunks + 3) / 4) * 4;
    }
    a.kb_max = kb < nb ? kb : nb;
    a.slot_bytes = ((a.kb_max * max_sbb + 32 + 15) / 16) * 16;
    const bool stage_x = c.TB == 1;
    const size_t xbytes = stage_x ? (size_t)c.K + (size_t)c.K / 2 : 0;
    const size_t budget = 110 * 1024 - 128 - xbytes;
    int stages = (int)(budget / ((size_t)kRowsPerTile * a.slot_bytes));
    stages = stages > 8 ? 8 : stages;
    if (stages < 2) {
        return cudaErrorInvalidConfiguration;
    }
    a.stages = stages;
    const size_t smem = 128 + (size_t)stages * kRowsPerTile * a.slot_bytes + xbytes;
    const int grid = groups < 2 * kSMs ? groups : 2 * kSMs;
    if (c.TB == 1) {
        return launch_stream_tt<1>(s, a, smem, grid, pdl_secondary);
    }
    if (c.TB == 2) {
        return launch_stream_tt<2>(s, a, smem, grid, pdl_secondary);
    }
    if (c.TB <= 4) {
        return launch_stream_tt<4>(s, a, smem, grid, pdl_secondary);
    }
    return launch_stream_tt<8>(s, a, smem, grid, pdl_secondary);
}

cudaError_t read_device_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_device_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    }
    return e;
}

} // namespace b200q
