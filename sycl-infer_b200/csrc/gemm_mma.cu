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
constexpr int kRing = 4;   // tensor-memory accumulators in flight
constexpr int kHdr = 512;  // bytes of mbarriers + the TMEM address at the start of shared memory
// Role mix per instantiation <NT, EW, PG>: EW epilogue warpgroups (each covers all 128 TMEM
// lanes and NT/EW token columns), PG producer groups of 128 threads that take the steps in
// turn (step i belongs to group i % PG) so their global/shared round trips overlap.
template <int NT, int EW, int PG> struct Roles {
    // operand/factor slots in shared memory: deeper than the accumulator ring so producers run
    // many steps ahead of the epilogue and a step never waits on a global-memory round trip
    static constexpr int kDepth = 8;
    static constexpr int kEpiWarps = 4 * EW, kProdWarps = 4 * PG;
    static constexpr int kThreads = 32 * (kEpiWarps + kProdWarps + 1);
};

struct MmaArgs {
    CallDev c;
    int32_t tiles_m[B200Q_MAX_SEGS]; // exclusive prefix of 128-row tiles per segment
    int32_t n_tiles_m, n_tiles_t;
    int32_t raw_bytes; // per-thread staging bytes for one raw superblock (16-byte units)
    int32_t lbo, sbo; // operand descriptor strides (bytes): K-adjacent core matrices, 8-row groups
};

template <int TYPE> struct StepFmt { // steps (MMAs) per superblock, operand signedness
    static constexpr int NS = TYPE == kQ6_K ? 16 : 8;
    static constexpr int A_SIGNED = (TYPE == kQ8_0 || TYPE == kIQ4_XS) ? 1 : 0;
    static constexpr bool HAS_MIN = TYPE == kQ4_K || TYPE == kQ5_K;
    static constexpr bool HAS_C = TYPE == kQ6_K;
};

// The 32 operand bytes of step s of one superblock of one row, plus the row's fp32 factors.
template <int TYPE, class WM>
__device__ __forceinline__ void unpack_step(const uint8_t * sb, int s, uint32_t (&o)[8], float & rowA, float & rowB) {
    rowB = 0.f;
    if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        const uint4 hdr = WM::ld128(sb);
        const uint8_t * qs = sb + (TYPE == kQ4_K ? 16 : 48) + (s >> 1) * 32;
        const uint4 q0 = WM::ld128(qs), q1 = WM::ld128(qs + 16);
        const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) {
            o[k] = (s & 1) ? (q[k] >> 4) & 0x0F0F0F0Fu : q[k] & 0x0F0F0F0Fu;
        }
        if constexpr (TYPE == kQ5_K) {
            const uint4 h0 = WM::ld128(sb + 16), h1 = WM::ld128(sb + 32);
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
        WM::template ld_a2<4>(sb + 64 * blk2 + ((plane & 1) ? 32 : 0) + 16 * hs, ql);
        WM::template ld_a2<4>(sb + 128 + 32 * blk2 + 16 * hs, qh);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t lo = plane >= 2 ? (ql[k] >> 4) & 0x0F0F0F0Fu : ql[k] & 0x0F0F0F0Fu;
            const uint32_t v = lo | (((qh[k] >> (2 * plane)) & 0x03030303u) << 4);
            o[4 * hs + k] = v;       // the half this 16-value scale group covers ...
            o[4 * (1 - hs) + k] = 0; // ... the other half contributes nothing to this step
        }
        const int s8 = WM::ld8s(sb + 192 + s);
        rowA = h2f((uint16_t)WM::ld16(sb + 208)) * (float)s8;
    } else if constexpr (TYPE == kQ8_0) {
        const uint8_t * blk = sb + 34 * s;
        rowA = h2f((uint16_t)WM::ld16(blk));
        WM::template ld_a2<8>(blk + 2, o);
    } else { // IQ4_XS
        const uint2 hdr = WM::ld64(sb);
        const int ls = (int)((hdr.y >> (8 * (s >> 1) + 4 * (s & 1))) & 0xF) | (int)((((hdr.x >> 16) >> (2 * s)) & 3) << 4);
        rowA = h2f((uint16_t)(hdr.x & 0xFFFF)) * (float)(ls - 32);
        const uint2 q0 = WM::ld64(sb + 8 + 16 * s), q1 = WM::ld64(sb + 16 + 16 * s);
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
    uint32_t full, done, acc_full, acc_empty; // [depth] producers->MMA, [depth] epilogue->producers, [4], [4]
    int depth;
};

// ---- one tile, one role each ---------------------------------------------------------------
// Producer: software-pipelined so that no step waits on a global-memory round trip.
//   * the thread's own weight row is staged superblock by superblock into a private region of
//     shared memory with 16-byte cp.async copies (double buffered: superblock b+1 is in flight
//     while the steps of b are unpacked from shared memory);
//   * the tokens' int8 chunks of step s+1 are cp.async'ed straight into the operand slot of
//     step s+1 while step s is unpacked; the per-token factors of step s+1 sit in registers.

struct TokPrefetch {
    float sx;
    int2 xs;
};

template <int TYPE, int NT>
__device__ __forceinline__ void issue_tokens(const MmaArgs & a, int b, int s, int t0, int r, uint32_t base,
                                             TokPrefetch & tp) {
    using F = StepFmt<TYPE>;
    const int TB = a.c.TB, G = 8 * b + (F::NS == 16 ? s >> 1 : s);
    for (int c = r; c < 2 * NT; c += 128) {
        const int t = c >> 1, h = c & 1;
        const uint32_t dst = base + Slot<NT>::B + core_off(t, h);
        if (t0 + t < TB) {
            cp_async16(dst, a.c.x8 + ((size_t)G * TB + t0 + t) * 32 + 16 * h);
        } else {
            sts128(dst, 0, 0, 0, 0);
        }
    }
    tp.sx = 0.f;
    tp.xs = make_int2(0, 0);
    if (r < NT && t0 + r < TB) {
        const size_t gi = (size_t)G * TB + t0 + r;
        tp.sx = __ldg(a.c.xmeta + 2 * gi);
        tp.xs = __ldg(reinterpret_cast<const int2 *>(a.c.xsumq) + gi);
    }
}

template <int TYPE, int NT, int PG>
__device__ __forceinline__ bool produce_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, uint32_t ring,
                                             uint32_t raw_all, int pt, const Bars & bars, uint32_t & git) {
    using F = StepFmt<TYPE>;
    constexpr int SB = Fmt<TYPE>::SB;
    const int grp = pt >> 7, r = pt & 127; // producer group, weight row this thread unpacks
    const int nb = a.c.K >> 8, RB = a.raw_bytes;
    const uint32_t D = (uint32_t)bars.depth;
    const bool row_ok = row0 + r < sg.n_rows;
    const uint8_t * wrow = sg.w + (size_t)(row0 + r) * nb * SB;
    const uint32_t raw = raw_all + (uint32_t)(pt * 2 * RB);
    uint8_t * raw_gen = nullptr; // generic pointer to the same bytes, for the decode helpers
    {
        extern __shared__ __align__(128) uint8_t smem_raw[];
        raw_gen = smem_raw + (raw - smem_u32(smem_raw));
    }
    auto stage_sb = [&](int b) { // this row's superblock b -> raw[b & 1], 16-byte aligned chunks
        if (row_ok && b < nb) {
            const uintptr_t A = reinterpret_cast<uintptr_t>(wrow + (size_t)b * SB);
            const uintptr_t A0 = A & ~uintptr_t(15);
            const int n = (int)((A + SB + 15 - A0) >> 4);
            for (int i = 0; i < n; i++) {
                cp_async16(raw + (uint32_t)((b & 1) * RB + 16 * i), reinterpret_cast<const void *>(A0 + 16 * i));
            }
        }
        cp_async_commit();
    };
    const int steps = nb * F::NS;
    const uint32_t git0 = git;
    git += (uint32_t)steps; // every role advances the shared step counter by the tile's steps
    // this group's steps: i = first, first + PG, ...  (first chosen so that (git0 + i) % PG == grp)
    int i = (int)((grp + PG - (git0 % PG)) % PG);
    if (i >= steps) {
        return true;
    }
    int staged = i / F::NS; // highest superblock staged so far
    stage_sb(staged);
    {
        const uint32_t g = git0 + i;
        if (!mbar_wait(bars.done + 8 * (g % D), ((g / D) & 1) ^ 1, &g_mma_status)) {
            cp_async_wait<0>();
            return false;
        }
    }
    TokPrefetch tp;
    issue_tokens<TYPE, NT>(a, i / F::NS, i % F::NS, t0, r, ring + ((git0 + i) % D) * Slot<NT>::BYTES, tp);
    cp_async_commit();
    for (; i < steps; i += PG) {
        const int b = i / F::NS, s = i - b * F::NS;
        const uint32_t g = git0 + i;
        const uint32_t base = ring + (g % D) * Slot<NT>::BYTES;
        const TokPrefetch cur = tp;
        // keep the superblock after the one in use in flight (one commit group per step, maybe empty)
        if (staged < b + 1) {
            staged = b + 1;
            stage_sb(staged);
        } else {
            cp_async_commit();
        }
        const int i1 = i + PG;
        if (i1 < steps) { // this group's next step: its tokens go into its slot once that is released
            const uint32_t g1 = git0 + i1;
            if (!mbar_wait(bars.done + 8 * (g1 % D), ((g1 / D) & 1) ^ 1, &g_mma_status)) {
                cp_async_wait<0>();
                return false;
            }
            issue_tokens<TYPE, NT>(a, i1 / F::NS, i1 % F::NS, t0, r, ring + (g1 % D) * Slot<NT>::BYTES, tp);
        }
        cp_async_commit();
        // groups in flight, oldest first: ... [superblock b] [tokens i] | [superblock b+1 or empty] [tokens i+PG]
        cp_async_wait<2>();
        uint32_t o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        float rowA = 0.f, rowB = 0.f;
        if (row_ok) {
            const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(wrow + (size_t)b * SB) & 15);
            unpack_step<TYPE, SmemW>(raw_gen + (b & 1) * RB + mis, s, o, rowA, rowB);
        }
        sts128(base + Slot<NT>::A + core_off(r, 0), o[0], o[1], o[2], o[3]);
        sts128(base + Slot<NT>::A + core_off(r, 1), o[4], o[5], o[6], o[7]);
        sts32(base + Slot<NT>::ROWA + 4 * r, __float_as_uint(rowA));
        sts32(base + Slot<NT>::ROWB + 4 * r, __float_as_uint(rowB));
        if (r < NT) {
            sts32(base + Slot<NT>::TOKA + 4 * r, __float_as_uint(cur.sx));
            sts32(base + Slot<NT>::TOKB + 4 * r, __float_as_uint(cur.sx * (float)(cur.xs.x + cur.xs.y)));
            sts32(base + Slot<NT>::TOKC + 4 * r, __float_as_uint((float)(32 * ((s & 1) ? cur.xs.y : cur.xs.x))));
        }
        fence_proxy_async(); // the tensor core reads A and B through the async proxy
        mbar_arrive(bars.full + 8 * (g % D));
    }
    cp_async_wait<0>();
    return true;
}

template <int TYPE, int NT>
__device__ __forceinline__ bool mma_tile(const MmaArgs & a, uint32_t ring, uint32_t tmem, const Bars & bars,
                                         uint32_t & git) {
    using F = StepFmt<TYPE>;
    const uint32_t idesc = idesc_i8(F::A_SIGNED, 1, kTileM, NT);
    const int steps = (a.c.K >> 8) * F::NS;
    const uint32_t D = (uint32_t)bars.depth;
    for (int i = 0; i < steps; i++, git++) {
        const uint32_t slot = git % D, acc = git % kRing;
        // operands of this step written, and the accumulator it overwrites drained by the epilogue
        if (!mbar_wait(bars.full + 8 * slot, (git / D) & 1, &g_mma_status) ||
            !mbar_wait(bars.acc_empty + 8 * acc, ((git / kRing) & 1) ^ 1, &g_mma_status)) {
            return false;
        }
        tc_fence_after();
        const uint32_t base = ring + slot * Slot<NT>::BYTES;
        const uint64_t ad = smem_desc_kmajor(base + Slot<NT>::A, a.lbo, a.sbo);
        const uint64_t bd = smem_desc_kmajor(base + Slot<NT>::B, a.lbo, a.sbo);
        mma_i8(tmem + (uint32_t)(acc * NT), ad, bd, idesc, 0);
        mma_commit(bars.acc_full + 8 * acc);
    }
    return true;
}

// ---- packed fp32 pairs: two FMAs per instruction on this architecture ------------------------
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    return (uint64_t)__float_as_uint(lo) | ((uint64_t)__float_as_uint(hi) << 32);
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Epilogue: this thread owns weight row `row0 + 32*(warp%4) + lane` and NT/EW token columns.
template <int TYPE, int NT, int EW>
__device__ __forceinline__ bool epilogue_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, uint32_t ring,
                                              uint32_t tmem, const Bars & bars, uint32_t & git) {
    using F = StepFmt<TYPE>;
    constexpr int NC = NT / EW; // token columns per thread
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rl = 32 * (warp & 3) + lane, c0 = (warp >> 2) * NC;
    const int steps = (a.c.K >> 8) * F::NS;
    uint64_t acc[NC / 2];
#pragma unroll
    for (int i = 0; i < NC / 2; i++) {
        acc[i] = 0ull;
    }
    const uint64_t kNegMagic = pack2(-12582912.0f, -12582912.0f);
    bool ok = true;
    for (int i = 0; i < steps; i++, git++) {
        const uint32_t slot = git % (uint32_t)bars.depth, accb = git % kRing;
        if (!mbar_wait(bars.acc_full + 8 * accb, (git / kRing) & 1, &g_mma_status)) {
            ok = false;
            break;
        }
        tc_fence_after();
        const uint32_t base = ring + slot * Slot<NT>::BYTES;
        const float ra = __uint_as_float(lds32(base + Slot<NT>::ROWA + 4 * rl));
        const uint64_t rowA = pack2(ra, ra);
        uint64_t nrowB = 0ull;
        if (F::HAS_MIN) {
            const float rb = -__uint_as_float(lds32(base + Slot<NT>::ROWB + 4 * rl));
            nrowB = pack2(rb, rb);
        }
        const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(accb * NT + c0);
#pragma unroll
        for (int j = 0; j < NC; j += 16) {
            uint32_t v[16];
            tmem_ld16(taddr + j, v);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 16; q += 4) {
                const uint4 ta = lds128(base + Slot<NT>::TOKA + 4 * (c0 + j + q));
                const uint64_t sx[2] = {(uint64_t)ta.x | ((uint64_t)ta.y << 32), (uint64_t)ta.z | ((uint64_t)ta.w << 32)};
                uint64_t tc[2] = {0ull, 0ull}, tb[2] = {0ull, 0ull};
                if (F::HAS_C) {
                    const uint4 x = lds128(base + Slot<NT>::TOKC + 4 * (c0 + j + q));
                    tc[0] = pack2(-__uint_as_float(x.x), -__uint_as_float(x.y));
                    tc[1] = pack2(-__uint_as_float(x.z), -__uint_as_float(x.w));
                }
                if (F::HAS_MIN) {
                    const uint4 x = lds128(base + Slot<NT>::TOKB + 4 * (c0 + j + q));
                    tb[0] = (uint64_t)x.x | ((uint64_t)x.y << 32);
                    tb[1] = (uint64_t)x.z | ((uint64_t)x.w << 32);
                }
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    // exact int -> float without the conversion unit: |wd| < 2^22
                    uint64_t w = (uint64_t)(v[q + 2 * e] + 0x4B400000u) | ((uint64_t)(v[q + 2 * e + 1] + 0x4B400000u) << 32);
                    w = add2(w, kNegMagic);
                    if (F::HAS_C) {
                        w = add2(w, tc[e]);
                    }
                    uint64_t r = fma2(rowA, mul2(sx[e], w), acc[(j + q) / 2 + e]);
                    if (F::HAS_MIN) {
                        r = fma2(nrowB, tb[e], r);
                    }
                    acc[(j + q) / 2 + e] = r;
                }
            }
        }
        tc_fence_before();
        mbar_arrive(bars.acc_empty + 8 * accb); // the accumulator may be overwritten
        mbar_arrive(bars.done + 8 * slot);      // the operand slot and its factors may be refilled
    }
    if (ok) {
        const int row = row0 + rl;
        if (row < sg.n_rows) {
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const int t = t0 + c0 + i;
                if (t < a.c.TB) {
                    const size_t o = (size_t)t * sg.out_stride + row;
                    const uint64_t pr = acc[i / 2];
                    float v = sg.alpha * __uint_as_float((uint32_t)((i & 1) ? pr >> 32 : pr));
                    if (sg.residual) {
                        v += sg.residual[o];
                    }
                    store_out(a.c, &sg.out[o], v);
                }
            }
        }
    }
    return ok;
}

template <int TYPE, int NT, int EW, int PG>
__device__ __forceinline__ bool run_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, uint32_t ring,
                                         uint32_t tmem, const Bars & bars, uint32_t & git) {
    using R = Roles<NT, EW, PG>;
    const int warp = threadIdx.x >> 5;
    if (warp < R::kEpiWarps) {
        return epilogue_tile<TYPE, NT, EW>(a, sg, row0, t0, ring, tmem, bars, git);
    }
    if (warp < R::kEpiWarps + R::kProdWarps) {
        return produce_tile<TYPE, NT, PG>(a, sg, row0, t0, ring, ring + R::kDepth * Slot<NT>::BYTES,
                                          (int)threadIdx.x - 32 * R::kEpiWarps, bars, git);
    }
    if (threadIdx.x == 32 * (R::kEpiWarps + R::kProdWarps)) {
        return mma_tile<TYPE, NT>(a, ring, tmem, bars, git);
    }
    git += (uint32_t)((a.c.K >> 8) * StepFmt<TYPE>::NS); // idle lanes of the MMA warp keep the count
    return true;
}

template <int NT, int EW, int PG>
__global__ void __launch_bounds__(Roles<NT, EW, PG>::kThreads, 1) gemm_mma_kernel(const __grid_constant__ MmaArgs a) {
    using R = Roles<NT, EW, PG>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const Bars bars{sbase, sbase + 128, sbase + 256, sbase + 320, R::kDepth};
    const uint32_t tmem_slot = sbase + 384, ring = sbase + kHdr;
    constexpr uint32_t kCols = kRing * NT < 32 ? 32 : kRing * NT; // power of two >= 32
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < R::kDepth; s++) {
            mbar_init(bars.full + 8 * s, 128); // the one producer group that owns the step
            mbar_init(bars.done + 8 * s, 32 * R::kEpiWarps);
        }
        for (int s = 0; s < kRing; s++) {
            mbar_init(bars.acc_full + 8 * s, 1);
            mbar_init(bars.acc_empty + 8 * s, 32 * R::kEpiWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == R::kEpiWarps + R::kProdWarps) {
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
        case kQ4_K: ok = run_tile<kQ4_K, NT, EW, PG>(a, sg, row0, t0, ring, tmem, bars, git); break;
        case kQ5_K: ok = run_tile<kQ5_K, NT, EW, PG>(a, sg, row0, t0, ring, tmem, bars, git); break;
        case kQ6_K: ok = run_tile<kQ6_K, NT, EW, PG>(a, sg, row0, t0, ring, tmem, bars, git); break;
        case kIQ4_XS: ok = run_tile<kIQ4_XS, NT, EW, PG>(a, sg, row0, t0, ring, tmem, bars, git); break;
        default: ok = run_tile<kQ8_0, NT, EW, PG>(a, sg, row0, t0, ring, tmem, bars, git); break;
        }
    }
    // every role falls through to here, also after a wait that ran out: release tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == R::kEpiWarps + R::kProdWarps) {
        tmem_dealloc(tmem, kCols);
    }
}

// ---- host side ----------------------------------------------------------------------------------
template <int NT, int EW, int PG> static cudaError_t launch_nt(cudaStream_t s, MmaArgs & a, bool pdl_secondary) {
    using R = Roles<NT, EW, PG>;
    const size_t smem = kHdr + (size_t)R::kDepth * Slot<NT>::BYTES + (size_t)32 * R::kProdWarps * 2 * a.raw_bytes;
    if (smem > 227 * 1024) {
        return cudaErrorInvalidConfiguration;
    }
    static size_t configured = 0;
    if (configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mma_kernel<NT, EW, PG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) {
            return e;
        }
        configured = smem;
    }
    a.n_tiles_t = (a.c.TB + NT - 1) / NT;
    const int tiles = a.n_tiles_m * a.n_tiles_t;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles < kSMs ? tiles : kSMs));
    cfg.blockDim = dim3(R::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_secondary ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemm_mma_kernel<NT, EW, PG>, a);
}

cudaError_t launch_gemm_mma(cudaStream_t s, const CallDev & c, bool pdl_secondary) {
    MmaArgs a;
    a.c = c;
    int tiles = 0, max_sbb = 0;
    for (int i = 0; i < c.n_segs; i++) {
        tiles += (c.seg[i].n_rows + kTileM - 1) / kTileM;
        a.tiles_m[i] = tiles;
        max_sbb = max_sbb > sb_bytes(c.seg[i].type) ? max_sbb : sb_bytes(c.seg[i].type);
    }
    a.n_tiles_m = tiles;
    a.raw_bytes = ((max_sbb + 15 + 15) / 16) * 16 + 16; // superblock + misalignment, whole 16-byte chunks
    a.lbo = 128;
    a.sbo = 256;
    if (c.TB <= 32) { // batched decode: unpacking dominates; one epilogue warpgroup
        return launch_nt<32, 1, 2>(s, a, pdl_secondary);
    }
    // prefill: the fp32 epilogue dominates; a second producer group only where its staging fits
    return a.raw_bytes <= 256 ? launch_nt<128, 2, 2>(s, a, pdl_secondary) : launch_nt<128, 2, 1>(s, a, pdl_secondary);
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
