// Batched-decode / prefill GEMM on the 5th-generation tensor cores (tcgen05, kind::i8).
//
// out[t, n] = alpha * sum over 32-value groups g of
//                 sx[t,g] * ( rowA[n,g] * (wd[t,n,g] - tokC[t,g]) ) - rowB[n,g] * tokB[t,g]
// with wd the exact int32 dot of the group.  Because every group carries its own fp32 scales
// on BOTH sides, integer accumulation cannot run past K = 32: one tcgen05.mma (M = 128 weight
// rows, N = NT tokens, K = 32) per group writes a fresh int32 accumulator into tensor memory,
// and the epilogue warps read it back (tcgen05.ld) and fold it into fp32 registers.  The
// design is therefore epilogue-bound by construction; the tensor core only has to stay ahead.
//
// Roles in a CTA (416 threads, one CTA per SM, persistent over (row tile, token tile)):
//   warps 0-7   epilogue: warp w reads TMEM lanes 32*(w%4).. (its weight rows) and the token
//               columns of half w/4; accumulators stay in registers for the whole K loop
//   warps 8-11  producers: thread = weight row; unpack the group's 32 codes from the raw GGUF
//               block into the K-major core-matrix layout the MMA reads, copy the tokens'
//               int8 group the same way, publish the per-row / per-token fp32 factors
//   warp 12     one thread issues the MMAs and commits them to mbarriers; it owns TMEM
// A four-deep ring (shared tiles + factor arrays + TMEM accumulator) links the roles with
// three mbarrier arrays: full (producers -> MMA), acc_full (MMA -> epilogue), acc_empty
// (epilogue -> producers).  All waits are bounded; TMEM is always released before exit.
#include <cstdlib>

#include "async.cuh"
#include "decode.cuh"
#include "launch.h"

namespace b200q {

__device__ int g_mma_status = 0;

constexpr int kTileM = 128;
constexpr int kRing = 4;
constexpr int kEpiWarps = 8, kProdWarps = 4;
constexpr int kMmaThreads = 32 * (kEpiWarps + kProdWarps + 1);

struct MmaArgs {
    CallDev c;
    int32_t tiles_m[B200Q_MAX_SEGS]; // exclusive prefix of 128-row tiles per segment
    int32_t n_tiles_m, n_tiles_t;
    int32_t lbo, sbo; // operand descriptor strides (bytes): K-adjacent core matrices, 8-row groups
};

template <int TYPE> struct StepFmt { // steps (MMAs) per superblock, operand signedness
    static constexpr int NS = TYPE == kQ6_K ? 16 : 8;
    static constexpr int A_SIGNED = (TYPE == kQ8_0 || TYPE == kIQ4_XS) ? 1 : 0;
    static constexpr bool HAS_MIN = TYPE == kQ4_K || TYPE == kQ5_K;
    static constexpr bool HAS_C = TYPE == kQ6_K;
};

// The 32 operand bytes of step s of one superblock of one row, plus the row's fp32 factors.
template <int TYPE>
__device__ __forceinline__ void unpack_step(const uint8_t * sb, int s, uint32_t (&o)[8], float & rowA, float & rowB) {
    rowB = 0.f;
    if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        const uint4 hdr = GmemW::ld128(sb);
        const uint8_t * qs = sb + (TYPE == kQ4_K ? 16 : 48) + (s >> 1) * 32;
        const uint4 q0 = GmemW::ld128(qs), q1 = GmemW::ld128(qs + 16);
        const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) {
            o[k] = (s & 1) ? (q[k] >> 4) & 0x0F0F0F0Fu : q[k] & 0x0F0F0F0Fu;
        }
        if constexpr (TYPE == kQ5_K) {
            const uint4 h0 = GmemW::ld128(sb + 16), h1 = GmemW::ld128(sb + 32);
            const uint32_t h[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
            for (int k = 0; k < 8; k++) {
                o[k] |= ((h[k] >> s) & 0x01010101u) << 4;
            }
        }
        int sc, mn;
        k4_scale_min(s, hdr.y, hdr.z, hdr.w, sc, mn);
        rowA = h2f((uint16_t)(hdr.x & 0xFFFF)) * (float)sc;
        rowB = h2f((uint16_t)(hdr.x >> 16)) * (float)mn;
    } else if constexpr (TYPE == kQ6_K) {
        const int blk2 = s >> 3, plane = (s & 7) >> 1, hs = s & 1;
        uint32_t ql[4], qh[4];
        GmemW::ld_a2<4>(sb + 64 * blk2 + ((plane & 1) ? 32 : 0) + 16 * hs, ql);
        GmemW::ld_a2<4>(sb + 128 + 32 * blk2 + 16 * hs, qh);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t lo = plane >= 2 ? (ql[k] >> 4) & 0x0F0F0F0Fu : ql[k] & 0x0F0F0F0Fu;
            const uint32_t v = lo | (((qh[k] >> (2 * plane)) & 0x03030303u) << 4);
            o[4 * hs + k] = v;       // the half this 16-value scale group covers ...
            o[4 * (1 - hs) + k] = 0; // ... the other half contributes nothing to this step
        }
        const int s8 = (int)(int8_t)__ldg(reinterpret_cast<const int8_t *>(sb + 192 + s));
        rowA = h2f((uint16_t)GmemW::ld16(sb + 208)) * (float)s8;
    } else if constexpr (TYPE == kQ8_0) {
        const uint8_t * blk = sb + 34 * s;
        rowA = h2f((uint16_t)GmemW::ld16(blk));
        GmemW::ld_a2<8>(blk + 2, o);
    } else { // IQ4_XS
        const uint2 hdr = GmemW::ld64(sb);
        const int ls = (int)((hdr.y >> (8 * (s >> 1) + 4 * (s & 1))) & 0xF) | (int)((((hdr.x >> 16) >> (2 * s)) & 3) << 4);
        rowA = h2f((uint16_t)(hdr.x & 0xFFFF)) * (float)(ls - 32);
        const uint2 q0 = GmemW::ld64(sb + 8 + 16 * s), q1 = GmemW::ld64(sb + 16 + 16 * s);
        const uint32_t q[4] = {q0.x, q0.y, q1.x, q1.y};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            o[k] = iq4nl_lookup4(q[k] & 0x0F0F0F0Fu);
            o[4 + k] = iq4nl_lookup4((q[k] >> 4) & 0x0F0F0F0Fu);
        }
    }
}

// Shared-memory ring slot: A [128 rows][32 B] and B [NT tokens][32 B] as core matrices
// (8 rows x 16 B = 128 B contiguous; the two K halves 128 B apart, 8-row groups 256 B apart),
// then rowA[128], rowB[128], tokA[NT], tokB[NT], tokC[NT] as fp32.
template <int NT> struct Slot {
    static constexpr int A = 0, B = kTileM * 32, ROWA = B + NT * 32, ROWB = ROWA + kTileM * 4,
                         TOKA = ROWB + kTileM * 4, TOKB = TOKA + NT * 4, TOKC = TOKB + NT * 4,
                         BYTES = TOKC + NT * 4;
};
__device__ __forceinline__ uint32_t core_off(int row, int khalf) {
    return (uint32_t)((row >> 3) * 256 + khalf * 128 + (row & 7) * 16);
}

struct Bars {
    uint32_t full, acc_full, acc_empty;
};

// ---- one tile, one role each ---------------------------------------------------------------
template <int TYPE, int NT>
__device__ __forceinline__ bool produce_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, uint32_t ring,
                                             const Bars & bars, uint32_t & git) {
    using F = StepFmt<TYPE>;
    const int r = threadIdx.x - 32 * kEpiWarps; // 0..127: the weight row this thread unpacks
    const int nb = a.c.K >> 8, TB = a.c.TB;
    const bool row_ok = row0 + r < sg.n_rows;
    const uint8_t * wrow = sg.w + (size_t)(row0 + r) * nb * Fmt<TYPE>::SB;
    for (int b = 0; b < nb; b++) {
        for (int s = 0; s < F::NS; s++, git++) {
            const int slot = git % kRing;
            if (!mbar_wait(bars.acc_empty + 8 * slot, ((git / kRing) & 1) ^ 1, &g_mma_status)) {
                return false;
            }
            const uint32_t base = ring + slot * Slot<NT>::BYTES;
            uint32_t o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            float rowA = 0.f, rowB = 0.f;
            if (row_ok) {
                unpack_step<TYPE>(wrow + (size_t)b * Fmt<TYPE>::SB, s, o, rowA, rowB);
            }
            sts128(base + Slot<NT>::A + core_off(r, 0), o[0], o[1], o[2], o[3]);
            sts128(base + Slot<NT>::A + core_off(r, 1), o[4], o[5], o[6], o[7]);
            sts32(base + Slot<NT>::ROWA + 4 * r, __float_as_uint(rowA));
            sts32(base + Slot<NT>::ROWB + 4 * r, __float_as_uint(rowB));
            // the tokens' int8 group: 2*NT chunks of 16 bytes over 128 threads
            const int G = 8 * b + (F::NS == 16 ? s >> 1 : s);
            for (int c = r; c < 2 * NT; c += 32 * kProdWarps) {
                const int t = c >> 1, h = c & 1;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (t0 + t < TB) {
                    v = __ldg(reinterpret_cast<const uint4 *>(a.c.x8 + ((size_t)G * TB + t0 + t) * 32 + 16 * h));
                }
                sts128(base + Slot<NT>::B + core_off(t, h), v.x, v.y, v.z, v.w);
            }
            if (r < NT) {
                float tokA = 0.f, tokB = 0.f, tokC = 0.f;
                if (t0 + r < TB) {
                    const size_t gi = (size_t)G * TB + t0 + r;
                    tokA = __ldg(a.c.xmeta + 2 * gi);
                    const int2 xs = __ldg(reinterpret_cast<const int2 *>(a.c.xsumq) + gi);
                    tokB = tokA * (float)(xs.x + xs.y);
                    tokC = (float)(32 * ((s & 1) ? xs.y : xs.x));
                }
                sts32(base + Slot<NT>::TOKA + 4 * r, __float_as_uint(tokA));
                sts32(base + Slot<NT>::TOKB + 4 * r, __float_as_uint(tokB));
                sts32(base + Slot<NT>::TOKC + 4 * r, __float_as_uint(tokC));
            }
            fence_proxy_async(); // the tensor core reads A and B through the async proxy
            mbar_arrive(bars.full + 8 * slot);
        }
    }
    return true;
}

template <int TYPE, int NT>
__device__ __forceinline__ bool mma_tile(const MmaArgs & a, uint32_t ring, uint32_t tmem, const Bars & bars,
                                         uint32_t & git) {
    using F = StepFmt<TYPE>;
    const uint32_t idesc = idesc_i8(F::A_SIGNED, 1, kTileM, NT);
    const int steps = (a.c.K >> 8) * F::NS;
    for (int i = 0; i < steps; i++, git++) {
        const int slot = git % kRing;
        if (!mbar_wait(bars.full + 8 * slot, (git / kRing) & 1, &g_mma_status)) {
            return false;
        }
        tc_fence_after();
        const uint32_t base = ring + slot * Slot<NT>::BYTES;
        const uint64_t ad = smem_desc_kmajor(base + Slot<NT>::A, a.lbo, a.sbo);
        const uint64_t bd = smem_desc_kmajor(base + Slot<NT>::B, a.lbo, a.sbo);
        mma_i8(tmem + (uint32_t)(slot * NT), ad, bd, idesc, 0);
        mma_commit(bars.acc_full + 8 * slot);
    }
    return true;
}

// Epilogue: this thread owns weight row `row0 + 32*(warp%4) + lane` and NT/2 tokens.
template <int TYPE, int NT>
__device__ __forceinline__ bool epilogue_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, uint32_t ring,
                                              uint32_t tmem, const Bars & bars, uint32_t & git) {
    using F = StepFmt<TYPE>;
    constexpr int NC = NT / 2; // token columns per thread
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rl = 32 * (warp & 3) + lane, c0 = (warp >> 2) * NC;
    const int steps = (a.c.K >> 8) * F::NS;
    float acc[NC];
#pragma unroll
    for (int i = 0; i < NC; i++) {
        acc[i] = 0.f;
    }
    bool ok = true;
    for (int i = 0; i < steps; i++, git++) {
        const int slot = git % kRing;
        if (!mbar_wait(bars.acc_full + 8 * slot, (git / kRing) & 1, &g_mma_status)) {
            ok = false;
            break;
        }
        tc_fence_after();
        const uint32_t base = ring + slot * Slot<NT>::BYTES;
        const float rowA = __uint_as_float(lds32(base + Slot<NT>::ROWA + 4 * rl));
        const float rowB = F::HAS_MIN ? __uint_as_float(lds32(base + Slot<NT>::ROWB + 4 * rl)) : 0.f;
        const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(slot * NT + c0);
#pragma unroll
        for (int j = 0; j < NC; j += 16) {
            uint32_t v[16];
            tmem_ld16(taddr + j, v);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 16; q += 4) {
                const uint4 ta = lds128(base + Slot<NT>::TOKA + 4 * (c0 + j + q));
                const float sx[4] = {__uint_as_float(ta.x), __uint_as_float(ta.y), __uint_as_float(ta.z),
                                     __uint_as_float(ta.w)};
                float tc[4] = {0.f, 0.f, 0.f, 0.f}, tb[4] = {0.f, 0.f, 0.f, 0.f};
                if (F::HAS_C) {
                    const uint4 x = lds128(base + Slot<NT>::TOKC + 4 * (c0 + j + q));
                    tc[0] = __uint_as_float(x.x), tc[1] = __uint_as_float(x.y), tc[2] = __uint_as_float(x.z),
                    tc[3] = __uint_as_float(x.w);
                }
                if (F::HAS_MIN) {
                    const uint4 x = lds128(base + Slot<NT>::TOKB + 4 * (c0 + j + q));
                    tb[0] = __uint_as_float(x.x), tb[1] = __uint_as_float(x.y), tb[2] = __uint_as_float(x.z),
                    tb[3] = __uint_as_float(x.w);
                }
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    // exact int -> float without the conversion unit: |wd| < 2^22
                    float wdf = __uint_as_float(v[q + e] + 0x4B400000u) - 12582912.0f;
                    if (F::HAS_C) {
                        wdf -= tc[e];
                    }
                    float r = fmaf(rowA, sx[e] * wdf, acc[j + q + e]);
                    if (F::HAS_MIN) {
                        r = fmaf(-rowB, tb[e], r);
                    }
                    acc[j + q + e] = r;
                }
            }
        }
        tc_fence_before();
        mbar_arrive(bars.acc_empty + 8 * slot);
    }
    if (ok) {
        const int row = row0 + rl;
        if (row < sg.n_rows) {
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const int t = t0 + c0 + i;
                if (t < a.c.TB) {
                    const size_t o = (size_t)t * sg.out_stride + row;
                    float v = sg.alpha * acc[i];
                    if (sg.residual) {
                        v += sg.residual[o];
                    }
                    sg.out[o] = v;
                }
            }
        }
    }
    return ok;
}

template <int TYPE, int NT>
__device__ __forceinline__ bool run_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, uint32_t ring,
                                         uint32_t tmem, const Bars & bars, uint32_t & git) {
    const int warp = threadIdx.x >> 5;
    if (warp < kEpiWarps) {
        return epilogue_tile<TYPE, NT>(a, sg, row0, t0, ring, tmem, bars, git);
    }
    if (warp < kEpiWarps + kProdWarps) {
        return produce_tile<TYPE, NT>(a, sg, row0, t0, ring, bars, git);
    }
    if (threadIdx.x == 32 * (kEpiWarps + kProdWarps)) {
        return mma_tile<TYPE, NT>(a, ring, tmem, bars, git);
    }
    git += (uint32_t)((a.c.K >> 8) * StepFmt<TYPE>::NS); // idle lanes of the MMA warp keep the count
    return true;
}

template <int NT> __global__ void __launch_bounds__(kMmaThreads, 1) gemm_mma_kernel(const __grid_constant__ MmaArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const Bars bars{sbase, sbase + 64, sbase + 128};
    const uint32_t tmem_slot = sbase + 192, ring = sbase + 256;
    constexpr uint32_t kCols = kRing * NT < 32 ? 32 : kRing * NT; // power of two >= 32
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kRing; s++) {
            mbar_init(bars.full + 8 * s, 32 * kProdWarps);
            mbar_init(bars.acc_full + 8 * s, 1);
            mbar_init(bars.acc_empty + 8 * s, 32 * kEpiWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kEpiWarps + kProdWarps) {
        tmem_alloc(tmem_slot, kCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds32(tmem_slot);
    asm volatile("griddepcontrol.wait;" ::: "memory"); // the activation quantizer's output is read below

    uint32_t git = 0;
    bool ok = true;
    const int n_tiles = a.n_tiles_m * a.n_tiles_t;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int tm = tile / a.n_tiles_t, tt = tile - tm * a.n_tiles_t; // token tiles innermost: weights stay in L2
        int si = 0;
        while (si + 1 < a.c.n_segs && tm >= a.tiles_m[si]) {
            si++;
        }
        const SegDev & sg = a.c.seg[si];
        const int row0 = (tm - (si ? a.tiles_m[si - 1] : 0)) * kTileM, t0 = tt * NT;
        switch (sg.type) {
        case kQ4_K: ok = run_tile<kQ4_K, NT>(a, sg, row0, t0, ring, tmem, bars, git); break;
        case kQ5_K: ok = run_tile<kQ5_K, NT>(a, sg, row0, t0, ring, tmem, bars, git); break;
        case kQ6_K: ok = run_tile<kQ6_K, NT>(a, sg, row0, t0, ring, tmem, bars, git); break;
        case kIQ4_XS: ok = run_tile<kIQ4_XS, NT>(a, sg, row0, t0, ring, tmem, bars, git); break;
        default: ok = run_tile<kQ8_0, NT>(a, sg, row0, t0, ring, tmem, bars, git); break;
        }
    }
    // every role falls through to here, also after a wait that ran out: release tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == kEpiWarps + kProdWarps) {
        tmem_dealloc(tmem, kCols);
    }
}

// ---- host side ----------------------------------------------------------------------------------
template <int NT> static cudaError_t launch_nt(cudaStream_t s, MmaArgs & a, bool pdl_secondary) {
    const size_t smem = 256 + (size_t)kRing * Slot<NT>::BYTES;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            return e;
        }
        configured = true;
    }
    a.n_tiles_t = (a.c.TB + NT - 1) / NT;
    const int tiles = a.n_tiles_m * a.n_tiles_t;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles < kSMs ? tiles : kSMs));
    cfg.blockDim = dim3(kMmaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_secondary ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemm_mma_kernel<NT>, a);
}

cudaError_t launch_gemm_mma(cudaStream_t s, const CallDev & c, bool pdl_secondary) {
    MmaArgs a;
    a.c = c;
    int tiles = 0;
    for (int i = 0; i < c.n_segs; i++) {
        tiles += (c.seg[i].n_rows + kTileM - 1) / kTileM;
        a.tiles_m[i] = tiles;
    }
    a.n_tiles_m = tiles;
    a.lbo = 128;
    a.sbo = 256;
    if (c.TB <= 32) {
        return launch_nt<32>(s, a, pdl_secondary);
    }
    return launch_nt<128>(s, a, pdl_secondary);
}

cudaError_t read_mma_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_mma_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_mma_status, &zero, sizeof(int));
    }
    return e;
}

} // namespace b200q
