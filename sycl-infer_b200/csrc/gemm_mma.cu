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
// Roles in a CTA (one CTA per SM, persistent over (row tile, token tile)); the mix <NT, EW, PG>
// follows the token count:
//   4*EW epilogue warps   warp w reads TMEM lanes 32*(w%4).. (its weight rows) and the NT/EW token
//                         columns of group w/4; its fp32 sums stay in registers for the whole K loop
//   4*PG producer warps   thread = weight row; unpack a superblock's codes from the raw GGUF
//                         block into the K-major core-matrix layout the MMA reads, copy the tokens'
//                         int8 groups the same way, publish the per-row / per-token fp32 factors
//   1 MMA warp            one thread issues the MMAs and commits them to mbarriers; it owns TMEM
// Operands travel in slots of eight steps (one superblock): one producer/consumer handshake per
// slot.  mbarrier arrays: full (producers -> MMA) and done (epilogue -> producers) per slot,
// acc_full (MMA -> epilogue) and acc_empty (epilogue -> MMA) per tensor-memory accumulator, of
// which up to 16 form a ring.  All waits are bounded; TMEM is always released.
#include <cstdlib>
#include <cstring>

#include "async.cuh"
#include "decode.cuh"
#include "launch.h"

namespace b200q {

__device__ int g_mma_status = 0;

constexpr int kTileM = 128;
// tensor-memory accumulators in flight: all 512 columns, at most 16 (the MMA -> epilogue -> MMA
// round trip is latency-bound, so the deeper the ring the more steps overlap)
__host__ __device__ constexpr int acc_ring(int NT) {
    return 512 / NT < 16 ? 512 / NT : 16;
}
// MMA steps handled together by the epilogue and signalled by ONE barrier pair (the sums of a
// batch live in registers: NC columns x batch <= 64): per-step handshakes are mostly latency
__host__ __device__ constexpr int epi_batch(int NC) {
    return NC <= 8 ? 8 : (NC <= 16 ? 4 : 1);
}
constexpr int kHdr = 512;  // bytes of mbarriers + the TMEM address at the start of shared memory
// Role mix per instantiation <NT, EW, PG>: EW epilogue warpgroups (each covers all 128 TMEM
// lanes and NT/EW token columns), PG producer groups of 128 threads that take the steps in
// turn (step i belongs to group i % PG) so their global/shared round trips overlap.
constexpr int kMaxDepth = 4; // operand slots of eight steps each; as many as shared memory holds
template <int NT, int EW, int PG> struct Roles {
    static constexpr int kEpiWarps = 4 * EW, kProdWarps = 4 * PG;
    static constexpr int kThreads = 32 * (kEpiWarps + kProdWarps + 1);
};

// Grouped form (routed MoE, more than a few tokens per expert): the row tiles of every active
// expert's plane, each against the tokens routed to that expert (CSR lists), in one launch.  A tile
// of the fused gate|up form interleaves 64 gate rows (even tensor-memory lanes) with the 64 up rows
// of the same indices (odd lanes): the two values of h = silu(gate) * up meet in neighbouring lanes.
struct GroupDev {
    const uint8_t * bank_a, * bank_b; // expert planes (bank_b: the up planes of the fused form)
    size_t plane_a, plane_b;          // bytes from one expert's plane to the next
    const int32_t * off, * pair, * active, * n_active; // CSR lists of the routed pairs
    int32_t max_active, n_pairs, top_k, fuse, n_rows, n_vec, tiles_per_expert, type;
    float * out; // out[pair * out_stride + row]
    int32_t out_stride;
};
struct TileG { // one grouped tile's tokens: CSR positions q0 .. q0 + ntok - 1 of expert e
    int e, q0, ntok;
};

struct MmaArgs {
    CallDev c;
    GroupDev g;
    int32_t tiles_m[B200Q_MAX_SEGS]; // exclusive prefix of 128-row tiles per segment
    int32_t n_tiles_m, n_tiles_t;
    int32_t raw_bytes; // per-thread staging bytes for one raw superblock (16-byte units)
    int32_t depth;     // operand slots in the shared-memory ring
    int32_t lbo, sbo; // operand descriptor strides (bytes): K-adjacent core matrices, 8-row groups
    // parity instrument: when set, the epilogue stores the raw int32 accumulators of token dump_t
    // (dump[row * D + step], D steps per row) exactly as tcgen05.ld returned them, and folds nothing
    int32_t * dump;
    int32_t dump_t;
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

// Shared-memory ring slot = kSlotSteps consecutive MMA steps (one superblock; half a Q6_K
// superblock).  Per step s: A[s] = [128 rows][32 B]; per activation group a B buffer = [NT
// tokens][32 B]; both as core matrices (8 rows x 16 B = 128 B contiguous; the two K halves 128 B
// apart, 8-row groups 256 B apart).  Then per step the fp32 factors rowA[128], rowB[128],
// tokA[NT], tokB[NT], tokC[NT].
constexpr int kSlotSteps = 8;
template <int NT> struct Slot {
    static constexpr int A = 0, B = kSlotSteps * kTileM * 32, ROWA = B + kSlotSteps * NT * 32,
                         ROWB = ROWA + kSlotSteps * kTileM * 4, TOKA = ROWB + kSlotSteps * kTileM * 4,
                         TOKB = TOKA + kSlotSteps * NT * 4, TOKC = TOKB + kSlotSteps * NT * 4,
                         BYTES = TOKC + kSlotSteps * NT * 4;
};
__device__ __forceinline__ uint32_t core_off(int row, int khalf) {
    return (uint32_t)((row >> 3) * 256 + khalf * 128 + (row & 7) * 16);
}

struct Bars {
    uint32_t full, done, acc_full, acc_empty; // [slots] producers->MMA, [slots] epilogue->producers, [acc], [acc]
    int depth;
};

// Q6_K has 16 steps per superblock over 8 activation groups: slot h (0/1) of a superblock holds
// steps 8h..8h+7; step s there is scale group 8h+s, activation group 4h + (s>>1), half s&1.
template <int TYPE> __device__ __forceinline__ int step_group(int slot_in_sb, int s) {
    return StepFmt<TYPE>::NS == 16 ? 4 * slot_in_sb + (s >> 1) : s;
}
template <int TYPE> __device__ __forceinline__ int step_bbuf(int s) { // B buffer of step s inside its slot
    return StepFmt<TYPE>::NS == 16 ? s >> 1 : s;
}

// One row's eight steps into the slot.  Q4_K/Q5_K take a whole-superblock path: the header is
// decoded once (the eight 6-bit scale/min pairs with 32-bit operations) and every 32 bytes of qs
// yield two steps (low and high nibbles); other types go step by step.
template <int TYPE, int NT>
__device__ __forceinline__ void unpack_slot(const uint8_t * sb, int h, int r, bool row_ok, uint32_t base) {
    using F = StepFmt<TYPE>;
    const uint32_t a0 = base + Slot<NT>::A, ra = base + Slot<NT>::ROWA + 4 * r, rb = base + Slot<NT>::ROWB + 4 * r;
    if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        uint4 hdr = make_uint4(0, 0, 0, 0);
        if (row_ok) {
            hdr = SmemW::ld128(sb);
        }
        const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
        // (scale, min) bytes of groups 0-3 and 4-7 (get_scale_min_k4, src/common/quant.h:136-144 of the reference)
        const uint32_t sc[2] = {hdr.y & 0x3F3F3F3Fu, (hdr.w & 0x0F0F0F0Fu) | ((hdr.y & 0xC0C0C0C0u) >> 2)};
        const uint32_t mn[2] = {hdr.z & 0x3F3F3F3Fu, ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z & 0xC0C0C0C0u) >> 2)};
        uint32_t hq[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (TYPE == kQ5_K && row_ok) {
            const uint4 h0 = SmemW::ld128(sb + 16), h1 = SmemW::ld128(sb + 32);
            hq[0] = h0.x, hq[1] = h0.y, hq[2] = h0.z, hq[3] = h0.w, hq[4] = h1.x, hq[5] = h1.y, hq[6] = h1.z, hq[7] = h1.w;
        }
#pragma unroll
        for (int pr = 0; pr < 4; pr++) { // pair pr: steps 2pr (low nibbles) and 2pr+1 (high nibbles)
            uint4 q0 = make_uint4(0, 0, 0, 0), q1 = q0;
            if (row_ok) {
                const uint8_t * qs = sb + (TYPE == kQ4_K ? 16 : 48) + 32 * pr;
                q0 = SmemW::ld128(qs);
                q1 = SmemW::ld128(qs + 16);
            }
            const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            uint32_t lo[8], hi[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                lo[k] = q[k] & 0x0F0F0F0Fu;
                hi[k] = (q[k] >> 4) & 0x0F0F0F0Fu;
                if (TYPE == kQ5_K) { // bit g of qh[i] is the fifth bit of element i of group g
                    lo[k] |= ((hq[k] >> (2 * pr)) & 0x01010101u) << 4;
                    hi[k] |= ((hq[k] >> (2 * pr + 1)) & 0x01010101u) << 4;
                }
            }
            const uint32_t al = a0 + (uint32_t)((2 * pr) * kTileM * 32), ah = al + kTileM * 32;
            sts128(al + core_off(r, 0), lo[0], lo[1], lo[2], lo[3]);
            sts128(al + core_off(r, 1), lo[4], lo[5], lo[6], lo[7]);
            sts128(ah + core_off(r, 0), hi[0], hi[1], hi[2], hi[3]);
            sts128(ah + core_off(r, 1), hi[4], hi[5], hi[6], hi[7]);
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int g = 2 * pr + e;
                const float scf = (float)((sc[g >> 2] >> (8 * (g & 3))) & 0xFF);
                const float mnf = (float)((mn[g >> 2] >> (8 * (g & 3))) & 0xFF);
                sts32(ra + 4 * g * kTileM, __float_as_uint(d * scf));
                sts32(rb + 4 * g * kTileM, __float_as_uint(dmin * mnf));
            }
        }
    } else if constexpr (TYPE == kQ6_K) {
        // half h of the superblock: ql[64h..], qh[32h..], scales[8h..]; step 2*plane + hs holds
        // the 16 codes of plane `plane`, elements 16hs..16hs+15, in its half of the operand
        // row and zeros in the other half (the block is 2-byte aligned: aligned words, funnel shift)
        const uint32_t sa = smem_u32(sb);
        const uint32_t sh = (sa & 2u) * 8, q = (sa & ~3u) + 64u * h, qhp = (sa & ~3u) + 128u + 32u * h;
#pragma unroll
        for (int hs = 0; hs < 2; hs++) {
            uint32_t v[4][4] = {};
            if (row_ok) {
                uint32_t wa[5], wb[5], wh[5];
#pragma unroll
                for (int k = 0; k < 5; k++) {
                    wa[k] = lds32(q + 16 * hs + 4 * k);
                    wb[k] = lds32(q + 32 + 16 * hs + 4 * k);
                    wh[k] = lds32(qhp + 16 * hs + 4 * k);
                }
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const uint32_t qa = __funnelshift_r(wa[k], wa[k + 1], sh), qb = __funnelshift_r(wb[k], wb[k + 1], sh);
                    const uint32_t hh = __funnelshift_r(wh[k], wh[k + 1], sh);
                    v[0][k] = (qa & 0x0F0F0F0Fu) | ((hh << 4) & 0x30303030u);
                    v[1][k] = (qb & 0x0F0F0F0Fu) | ((hh << 2) & 0x30303030u);
                    v[2][k] = ((qa >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u);
                    v[3][k] = ((qb >> 4) & 0x0F0F0F0Fu) | ((hh >> 2) & 0x30303030u);
                }
            }
#pragma unroll
            for (int pl = 0; pl < 4; pl++) {
                const uint32_t as = a0 + (uint32_t)((2 * pl + hs) * kTileM * 32);
                sts128(as + core_off(r, hs), v[pl][0], v[pl][1], v[pl][2], v[pl][3]);
                sts128(as + core_off(r, 1 - hs), 0, 0, 0, 0);
            }
        }
        float d = 0.f;
        uint32_t sc[2] = {0, 0};
        if (row_ok) {
            const uint32_t sp = (sa & ~3u) + 192u + 8u * h;
            const uint32_t c0 = lds32(sp), c1 = lds32(sp + 4), c2 = lds32(sp + 8);
            sc[0] = __funnelshift_r(c0, c1, sh);
            sc[1] = __funnelshift_r(c1, c2, sh);
            d = h2f((uint16_t)lds16(sa + 208));
        }
#pragma unroll
        for (int st = 0; st < kSlotSteps; st++) { // scales[8h + st] belongs to step st
            const int s8 = (int)(int8_t)(sc[st >> 2] >> (8 * (st & 3)));
            sts32(ra + 4 * st * kTileM, __float_as_uint(d * (float)s8));
        }
    } else {
#pragma unroll 1
        for (int st = 0; st < kSlotSteps; st++) {
            uint32_t o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            float rowA = 0.f, rowB = 0.f;
            if (row_ok) {
                unpack_step<TYPE, SmemW>(sb, h * kSlotSteps + st, o, rowA, rowB);
            }
            const uint32_t as = a0 + (uint32_t)(st * kTileM * 32);
            sts128(as + core_off(r, 0), o[0], o[1], o[2], o[3]);
            sts128(as + core_off(r, 1), o[4], o[5], o[6], o[7]);
            sts32(ra + 4 * st * kTileM, __float_as_uint(rowA));
        }
    }
    (void)F::NS;
}

// ---- one tile, one role each ---------------------------------------------------------------
// Producer group: 128 threads, thread r = weight row r of the tile.  For every slot it owns
// (slots are dealt to the PG groups in turn) it
//   * has the row's raw superblock in a private shared-memory buffer (16-byte cp.async copies,
//     double buffered: the next superblock it needs is in flight while this one is unpacked),
//   * copies the tokens' int8 groups straight into the slot's B buffers with cp.async,
//   * unpacks the eight steps' codes into A and publishes the per-row and per-token factors.
template <int TYPE, int NT, int PG, bool G>
__device__ __forceinline__ bool produce_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, const TileG & tg,
                                             uint32_t ring, uint32_t raw_all, int pt, const Bars & bars, uint32_t & gslot) {
    using F = StepFmt<TYPE>;
    constexpr int SB = Fmt<TYPE>::SB, SPS = F::NS / kSlotSteps; // slots per superblock
    constexpr int NB = F::NS == 16 ? 4 : 8;                     // activation groups per slot
    const int grp = pt >> 7, r = pt & 127;
    const int nb = a.c.K >> 8, RB = a.raw_bytes;
    const uint32_t D = (uint32_t)bars.depth;
    bool row_ok;
    const uint8_t * wrow;
    // The token column this thread serves is the same in every round of the loops below (NT and 2*NT
    // divide 128): column r % NT of the factor arrays, column (r % 2NT) / 2 of the int8 copies.  vf / vc:
    // the activation vectors behind those columns (-1: beyond the tile's tokens); TB: vectors per group.
    int vf, vc, TB;
    if constexpr (G) {
        const int rr = a.g.fuse ? row0 + (r >> 1) : row0 + r;
        row_ok = rr < a.g.n_rows;
        const uint8_t * plane = (a.g.fuse && (r & 1)) ? a.g.bank_b + (size_t)tg.e * a.g.plane_b : a.g.bank_a + (size_t)tg.e * a.g.plane_a;
        wrow = plane + (size_t)rr * nb * SB;
        const int tf = r & (NT - 1), tc = (r & (2 * NT - 1)) >> 1;
        const int pf = tf < tg.ntok ? __ldg(a.g.pair + tg.q0 + tf) : -1, pc = tc < tg.ntok ? __ldg(a.g.pair + tg.q0 + tc) : -1;
        vf = (pf >= 0 && a.g.top_k > 0) ? pf / a.g.top_k : pf;
        vc = (pc >= 0 && a.g.top_k > 0) ? pc / a.g.top_k : pc;
        TB = a.g.n_vec;
    } else {
        row_ok = row0 + r < sg.n_rows;
        wrow = sg.w + (size_t)(row0 + r) * nb * SB;
        TB = a.c.TB;
        const int tf = t0 + (r & (NT - 1)), tc = t0 + ((r & (2 * NT - 1)) >> 1);
        vf = tf < TB ? tf : -1;
        vc = tc < TB ? tc : -1;
    }
    // staging is buffer-major: thread pt's buffer `buf` sits at (buf * threads + pt) * RB, so the
    // threads of a warp are RB bytes apart (an odd number of 16-byte chunks: no bank conflicts)
    const int BS = 128 * PG * RB;
    const uint32_t raw = raw_all + (uint32_t)(pt * RB);
    uint8_t * raw_gen = nullptr; // generic pointer to the same bytes, for the decode helpers
    {
        extern __shared__ __align__(128) uint8_t smem_raw[];
        raw_gen = smem_raw + (raw - smem_u32(smem_raw));
    }
    auto stage_sb = [&](int b, int buf) { // this row's superblock b -> raw[buf], 16-byte aligned chunks
        if (row_ok && b < nb) {
            const uintptr_t A = reinterpret_cast<uintptr_t>(wrow + (size_t)b * SB);
            const uintptr_t A0 = A & ~uintptr_t(15);
            const int n = (int)((A + SB + 15 - A0) >> 4);
            for (int i = 0; i < n; i++) {
                cp_async16(raw + (uint32_t)(buf * BS + 16 * i), reinterpret_cast<const void *>(A0 + 16 * i));
            }
        }
        cp_async_commit();
    };
    const int slots = nb * SPS;
    const uint32_t g0 = gslot;
    gslot += (uint32_t)slots; // every role advances the shared slot counter by the tile's slots
    int i = (int)((grp + PG - (g0 % PG)) % PG); // this group's first slot of the tile
    if (i >= slots) {
        return true;
    }
    int have = i / SPS, buf = 0; // superblock held in raw[buf]
    stage_sb(have, buf);
    for (; i < slots; i += PG) {
        const int b = i / SPS, h = i - b * SPS; // superblock, slot within it
        const uint32_t g = g0 + i;
        const uint32_t base = ring + (g % D) * Slot<NT>::BYTES;
        if (b != have) { // prefetched while the previous slot of this group was unpacked
            have = b;
            buf ^= 1;
        }
        // the per-token factors of the eight steps come from global memory: start those loads
        // before waiting for the slot, they do not depend on it
        // (wide token tiles keep the loads after the wait: their registers are needed elsewhere)
        constexpr int NI = (kSlotSteps * NT + 127) / 128;
        constexpr bool kHoist = NT <= 32;
        float f_sx[NI];
        int2 f_xs[NI];
#pragma unroll
        for (int k = 0; k < NI; k++) {
            const int c = r + 128 * k, st = c / NT;
            f_sx[k] = 0.f;
            f_xs[k] = make_int2(0, 0);
            if (kHoist && c < kSlotSteps * NT && vf >= 0) {
                const size_t gi = (size_t)(8 * b + step_group<TYPE>(h, st)) * TB + vf;
                f_sx[k] = __ldg(a.c.xmeta + 2 * gi);
                f_xs[k] = __ldg(reinterpret_cast<const int2 *>(a.c.xsumq) + gi);
            }
        }
        if (!mbar_wait(bars.done + 8 * (g % D), ((g / D) & 1) ^ 1, &g_mma_status)) {
            cp_async_wait<0>();
            return false;
        }
        // tokens: the int8 groups this slot's steps meet, straight into the B buffers
        for (int c = r; c < NB * NT * 2; c += 128) {
            const int gi = c / (2 * NT), rem = c - gi * 2 * NT, t = rem >> 1, hh = rem & 1;
            const int grp8 = 8 * b + (F::NS == 16 ? 4 * h + gi : gi);
            const uint32_t dst = base + Slot<NT>::B + (uint32_t)(gi * NT * 32) + core_off(t, hh);
            if (vc >= 0) {
                cp_async16(dst, a.c.x8 + ((size_t)grp8 * TB + vc) * 32 + 16 * hh);
            } else {
                sts128(dst, 0, 0, 0, 0);
            }
        }
        cp_async_commit();
        // prefetch the superblock of this group's next slot (one commit group either way)
        const int inext = i + PG, bnext = inext / SPS;
        if (inext < slots && bnext != b) {
            stage_sb(bnext, buf ^ 1);
        } else {
            cp_async_commit();
        }
#pragma unroll
        for (int k = 0; k < NI; k++) {
            const int c = r + 128 * k, st = c / NT;
            if (!kHoist && c < kSlotSteps * NT && vf >= 0) {
                const size_t gi = (size_t)(8 * b + step_group<TYPE>(h, st)) * TB + vf;
                f_sx[k] = __ldg(a.c.xmeta + 2 * gi);
                f_xs[k] = __ldg(reinterpret_cast<const int2 *>(a.c.xsumq) + gi);
            }
            if (c < kSlotSteps * NT) {
                sts32(base + Slot<NT>::TOKA + 4 * c, __float_as_uint(f_sx[k]));
                if (F::HAS_MIN) {
                    sts32(base + Slot<NT>::TOKB + 4 * c, __float_as_uint(f_sx[k] * (float)(f_xs[k].x + f_xs[k].y)));
                }
                if (F::HAS_C) {
                    sts32(base + Slot<NT>::TOKC + 4 * c, __float_as_uint((float)(32 * ((st & 1) ? f_xs[k].y : f_xs[k].x))));
                }
            }
        }
        // groups in flight, oldest first: [superblock b] | [tokens] [next superblock or empty]
        cp_async_wait<2>();
        const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(wrow + (size_t)b * SB) & 15);
        unpack_slot<TYPE, NT>(raw_gen + buf * BS + mis, h, r, row_ok, base);
        cp_async_wait<1>();  // the tokens have landed; the prefetched superblock may still be in flight
        fence_proxy_async(); // the tensor core reads A and B through the async proxy
        mbar_arrive(bars.full + 8 * (g % D));
    }
    cp_async_wait<0>();
    return true;
}

template <int TYPE, int NT, int EW>
__device__ __forceinline__ bool mma_tile(const MmaArgs & a, uint32_t ring, uint32_t tmem, const Bars & bars,
                                         uint32_t & gslot, uint32_t & git) {
    using F = StepFmt<TYPE>;
    constexpr int GB = epi_batch(NT / EW), AR = acc_ring(NT), NG = AR / GB; // steps per barrier group, groups in the ring
    const uint32_t idesc = idesc_i8(F::A_SIGNED, 1, kTileM, NT);
    const int slots = (a.c.K >> 8) * (F::NS / kSlotSteps);
    const uint32_t D = (uint32_t)bars.depth;
    for (int i = 0; i < slots; i++, gslot++) {
        const uint32_t slot = gslot % D;
        if (!mbar_wait(bars.full + 8 * slot, (gslot / D) & 1, &g_mma_status)) {
            return false;
        }
        const uint32_t base = ring + slot * Slot<NT>::BYTES;
        const uint64_t ad0 = smem_desc_kmajor(base + Slot<NT>::A, a.lbo, a.sbo);
        const uint64_t bd0 = smem_desc_kmajor(base + Slot<NT>::B, a.lbo, a.sbo);
        for (int st0 = 0; st0 < kSlotSteps; st0 += GB, git += GB) {
            const uint32_t grp = (git / GB) % NG;
            // the accumulators this group overwrites must have been drained by the epilogue
            if (!mbar_wait(bars.acc_empty + 8 * grp, (((git / GB) / NG) & 1) ^ 1, &g_mma_status)) {
                return false;
            }
            tc_fence_after();
            // the issuing thread is a serial resource (one MMA per 32-value group): descriptors of
            // a slot differ only in their address field, so a step costs two additions and the MMA
#pragma unroll
            for (int b = 0; b < GB; b++) {
                const int st = st0 + b;
                const uint32_t acc = (git + b) % AR;
                const uint64_t ad = ad0 + (uint64_t)((st * kTileM * 32) >> 4);
                const uint64_t bd = bd0 + (uint64_t)((step_bbuf<TYPE>(st) * NT * 32) >> 4);
                mma_i8(tmem + (uint32_t)(acc * NT), ad, bd, idesc, 0);
            }
            mma_commit(bars.acc_full + 8 * grp); // arrives when every MMA issued so far has completed
        }
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
template <int TYPE, int NT, int EW, bool G>
__device__ __forceinline__ bool epilogue_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, const TileG & tg,
                                              uint32_t ring, uint32_t tmem, const Bars & bars, uint32_t & gslot,
                                              uint32_t & git) {
    using F = StepFmt<TYPE>;
    constexpr int NC = NT / EW; // token columns per thread
    constexpr uint32_t AR = acc_ring(NT);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rl = 32 * (warp & 3) + lane, c0 = (warp >> 2) * NC;
    const int slots = (a.c.K >> 8) * (F::NS / kSlotSteps);
    const uint32_t D = (uint32_t)bars.depth;
    uint64_t acc[NC / 2];
#pragma unroll
    for (int i = 0; i < NC / 2; i++) {
        acc[i] = 0ull;
    }
    const uint64_t kNegMagic = pack2(-12582912.0f, -12582912.0f);
    // (grouped form: token columns beyond a tile's tokens are folded like the rest - leaving them out
    // by a branch per group of four columns made the fold slower, 451 against 349 microseconds)
    bool ok = true;
    // Steps are taken in batches: wait for the batch's MMAs, start all their tensor-memory reads,
    // wait once, hand the accumulators back, then fold.  The wait -> read -> fold -> release chain
    // of a single step is almost pure latency (mbarrier wake-up + tensor-memory read), so with few
    // token columns per thread a whole batch costs little more than one step.
    constexpr int CH = NC >= 16 ? 16 : 8;                        // columns per tensor-memory read
    constexpr int BATCH = epi_batch(NC), NG = (int)AR / BATCH;   // steps per batch, barrier groups in the ring
    for (int i = 0; i < slots && ok; i++, gslot++) {
        const uint32_t slot = gslot % D;
        const uint32_t base = ring + slot * Slot<NT>::BYTES;
#pragma unroll 1
        for (int st0 = 0; st0 < kSlotSteps; st0 += BATCH, git += BATCH) {
            uint32_t v[BATCH][NC];
            const uint32_t grp = (git / BATCH) % NG;
            if (!mbar_wait(bars.acc_full + 8 * grp, ((git / BATCH) / NG) & 1, &g_mma_status)) {
                ok = false;
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(((git + b) % AR) * NT + c0);
#pragma unroll
                for (int j = 0; j < NC; j += CH) {
                    if constexpr (CH == 16) {
                        tmem_ld16(taddr + j, *reinterpret_cast<uint32_t(*)[16]>(&v[b][j]));
                    } else {
                        tmem_ld8(taddr + j, *reinterpret_cast<uint32_t(*)[8]>(&v[b][j]));
                    }
                }
            }
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(bars.acc_empty + 8 * grp); // the batch's accumulators may be overwritten
            if (a.dump) { // parity instrument: the tensor core's int32 sums as they are
                const int tcol = a.dump_t - t0 - c0;
                if (tcol >= 0 && tcol < NC && row0 + rl < sg.n_rows) {
                    const size_t D = (size_t)slots * kSlotSteps;
#pragma unroll
                    for (int b = 0; b < BATCH; b++) {
#pragma unroll
                        for (int j = 0; j < NC; j++) {
                            if (j == tcol) {
                                a.dump[(size_t)(row0 + rl) * D + (size_t)(kSlotSteps * i + st0 + b)] = (int32_t)v[b][j];
                            }
                        }
                    }
                }
                continue;
            }
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                const int st = st0 + b;
                const float ra = __uint_as_float(lds32(base + Slot<NT>::ROWA + 4 * (st * kTileM + rl)));
                const uint64_t rowA = pack2(ra, ra);
                uint64_t nrowB = 0ull;
                if (F::HAS_MIN) {
                    const float rb = -__uint_as_float(lds32(base + Slot<NT>::ROWB + 4 * (st * kTileM + rl)));
                    nrowB = pack2(rb, rb);
                }
                const uint32_t tok = base + 4 * (st * NT + c0);
#pragma unroll
                for (int q = 0; q < NC; q += 4) {
                    const uint4 ta = lds128(tok + Slot<NT>::TOKA + 4 * q);
                    const uint64_t sx[2] = {(uint64_t)ta.x | ((uint64_t)ta.y << 32), (uint64_t)ta.z | ((uint64_t)ta.w << 32)};
                    uint64_t tc[2] = {0ull, 0ull}, tb[2] = {0ull, 0ull};
                    if (F::HAS_C) {
                        const uint4 x = lds128(tok + Slot<NT>::TOKC + 4 * q);
                        tc[0] = pack2(-__uint_as_float(x.x), -__uint_as_float(x.y));
                        tc[1] = pack2(-__uint_as_float(x.z), -__uint_as_float(x.w));
                    }
                    if (F::HAS_MIN) {
                        const uint4 x = lds128(tok + Slot<NT>::TOKB + 4 * q);
                        tb[0] = (uint64_t)x.x | ((uint64_t)x.y << 32);
                        tb[1] = (uint64_t)x.z | ((uint64_t)x.w << 32);
                    }
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        // exact int -> float without the conversion unit: |wd| < 2^22
                        uint64_t w = (uint64_t)(v[b][q + 2 * e] + 0x4B400000u) | ((uint64_t)(v[b][q + 2 * e + 1] + 0x4B400000u) << 32);
                        w = add2(w, kNegMagic);
                        if (F::HAS_C) {
                            w = add2(w, tc[e]);
                        }
                        uint64_t r = fma2(rowA, mul2(sx[e], w), acc[q / 2 + e]);
                        if (F::HAS_MIN) {
                            r = fma2(nrowB, tb[e], r);
                        }
                        acc[q / 2 + e] = r;
                    }
                }
            }
        }
        if (ok) {
            mbar_arrive(bars.done + 8 * slot); // the operand slot and its factors may be refilled
        }
    }
    if constexpr (G) {
        // out[pair, row]: the tile's token column t is CSR position q0 + t.  Fused form: even lanes hold
        // gate rows, odd lanes the up rows of the same index; the even lane stores silu(gate) * up.
        if (__all_sync(0xFFFFFFFFu, ok)) {
            const int rr = a.g.fuse ? row0 + (rl >> 1) : row0 + rl;
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const int t = c0 + i;
                const uint64_t pr2 = acc[i / 2];
                const float v = __uint_as_float((uint32_t)((i & 1) ? pr2 >> 32 : pr2));
                const float other = __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                // both lanes of a pair now hold gate and up: the even lane finishes the even columns, the odd one the odd
                if (t < tg.ntok && rr < a.g.n_rows && (!a.g.fuse || (i & 1) == (lane & 1))) {
                    const int pi = __ldg(a.g.pair + tg.q0 + t);
                    float h = v;
                    if (a.g.fuse) { // x / (1 + expf(-x)) * up, as the single-token expert kernel forms it
                        const float gv = (lane & 1) ? other : v, uv = (lane & 1) ? v : other;
                        h = __fmul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))), uv);
                    }
                    a.g.out[(size_t)pi * a.g.out_stride + rr] = h;
                }
            }
        }
        return ok;
    }
    if (ok && !a.dump) {
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

template <int TYPE, int NT, int EW, int PG, bool G>
__device__ __forceinline__ bool run_tile(const MmaArgs & a, const SegDev & sg, int row0, int t0, const TileG & tg,
                                         uint32_t ring, uint32_t tmem, const Bars & bars, uint32_t & gslot, uint32_t & git) {
    using R = Roles<NT, EW, PG>;
    const int warp = threadIdx.x >> 5;
    if (warp < R::kEpiWarps) {
        return epilogue_tile<TYPE, NT, EW, G>(a, sg, row0, t0, tg, ring, tmem, bars, gslot, git);
    }
    if (warp < R::kEpiWarps + R::kProdWarps) {
        return produce_tile<TYPE, NT, PG, G>(a, sg, row0, t0, tg, ring, ring + (uint32_t)bars.depth * Slot<NT>::BYTES,
                                             (int)threadIdx.x - 32 * R::kEpiWarps, bars, gslot);
    }
    if (threadIdx.x == 32 * (R::kEpiWarps + R::kProdWarps)) {
        return mma_tile<TYPE, NT, EW>(a, ring, tmem, bars, gslot, git);
    }
    return true; // idle lanes of the MMA warp
}

template <int NT, int EW, int PG, bool G>
__device__ __forceinline__ bool run_tile_any(int type, const MmaArgs & a, const SegDev & sg, int row0, int t0,
                                             const TileG & tg, uint32_t ring, uint32_t tmem, const Bars & bars,
                                             uint32_t & gslot, uint32_t & git) {
    switch (type) {
    case kQ4_K: return run_tile<kQ4_K, NT, EW, PG, G>(a, sg, row0, t0, tg, ring, tmem, bars, gslot, git);
    case kQ5_K: return run_tile<kQ5_K, NT, EW, PG, G>(a, sg, row0, t0, tg, ring, tmem, bars, gslot, git);
    case kQ6_K: return run_tile<kQ6_K, NT, EW, PG, G>(a, sg, row0, t0, tg, ring, tmem, bars, gslot, git);
    case kIQ4_XS: return run_tile<kIQ4_XS, NT, EW, PG, G>(a, sg, row0, t0, tg, ring, tmem, bars, gslot, git);
    default: return run_tile<kQ8_0, NT, EW, PG, G>(a, sg, row0, t0, tg, ring, tmem, bars, gslot, git);
    }
}

template <int NT, int EW, int PG, bool G>
__global__ void __launch_bounds__(Roles<NT, EW, PG>::kThreads, 1) gemm_mma_kernel(const __grid_constant__ MmaArgs a) {
    using R = Roles<NT, EW, PG>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    // mbarriers: full[8] @0, done[8] @64, acc_full[16] @128, acc_empty[16] @256, TMEM address @384
    static_assert(kMaxDepth <= 8 && acc_ring(NT) <= 16 && kHdr >= 400, "barrier header layout");
    const Bars bars{sbase, sbase + 64, sbase + 128, sbase + 256, a.depth};
    const uint32_t tmem_slot = sbase + 384, ring = sbase + kHdr;
    constexpr uint32_t kCols = acc_ring(NT) * NT; // 512: a power of two >= 32
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.depth; s++) {
            mbar_init(bars.full + 8 * s, 128); // the one producer group that owns the slot
            mbar_init(bars.done + 8 * s, 32 * R::kEpiWarps);
        }
        for (int s = 0; s < acc_ring(NT); s++) {
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

    uint32_t gslot = 0, git = 0;
    bool ok = true;
    if constexpr (G) {
        // every role walks the same list: (active expert, row tile) dealt to the CTAs in turn, row tiles of
        // an expert on neighbouring CTAs (its tokens stay in L2); the expert's tokens NT at a time
        const int tpe = a.g.tiles_per_expert, rows_per_tile = a.g.fuse ? kTileM / 2 : kTileM;
        const int n_act = min(__ldg(a.g.n_active), a.g.max_active);
        for (int tile = blockIdx.x; tile < n_act * tpe && ok; tile += gridDim.x) {
            const int s = tile / tpe, tm = tile - s * tpe;
            const int e = __ldg(a.g.active + s);
            const int q0 = max(__ldg(a.g.off + e), 0), q1 = min(__ldg(a.g.off + e + 1), a.g.n_pairs);
            for (int q = q0; q < q1 && ok; q += NT) {
                const TileG tg{e, q, min(NT, q1 - q)};
                ok = run_tile_any<NT, EW, PG, true>(a.g.type, a, a.c.seg[0], tm * rows_per_tile, 0, tg, ring, tmem, bars, gslot, git);
            }
        }
    } else {
        const int n_tiles = a.n_tiles_m * a.n_tiles_t;
        const TileG none{0, 0, 0};
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int tm = tile / a.n_tiles_t, tt = tile - tm * a.n_tiles_t; // token tiles innermost: weights stay in L2
            int si = 0;
            while (si + 1 < a.c.n_segs && tm >= a.tiles_m[si]) {
                si++;
            }
            const SegDev & sg = a.c.seg[si];
            const int row0 = (tm - (si ? a.tiles_m[si - 1] : 0)) * kTileM, t0 = tt * NT;
            ok = run_tile_any<NT, EW, PG, false>(sg.type, a, sg, row0, t0, none, ring, tmem, bars, gslot, git);
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
template <int NT, int EW, int PG, bool G = false> static cudaError_t launch_nt(cudaStream_t s, MmaArgs & a, bool pdl_secondary) {
    using R = Roles<NT, EW, PG>;
    const size_t raw = (size_t)32 * R::kProdWarps * 2 * a.raw_bytes, budget = 227 * 1024;
    if (kHdr + 2 * (size_t)Slot<NT>::BYTES + raw > budget) {
        return cudaErrorInvalidConfiguration;
    }
    int depth = (int)((budget - kHdr - raw) / Slot<NT>::BYTES);
    depth = depth > kMaxDepth ? kMaxDepth : depth;
    a.depth = depth;
    const size_t smem = kHdr + (size_t)depth * Slot<NT>::BYTES + raw;
    {
        cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(gemm_mma_kernel<NT, EW, PG, G>), (int)smem);
        if (e != cudaSuccess) {
            return e;
        }
    }
    a.n_tiles_t = (a.c.TB + NT - 1) / NT;
    const long long tiles = G ? (long long)a.g.max_active * a.g.tiles_per_expert : (long long)a.n_tiles_m * a.n_tiles_t;
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
    return cudaLaunchKernelEx(&cfg, gemm_mma_kernel<NT, EW, PG, G>, a);
}

// Per-thread staging bytes for one raw superblock of `type`: the superblock plus its misalignment in
// whole 16-byte chunks (none when the size is a multiple of 16: tensor bases, planes and rows then keep
// the 16-byte alignment), made an odd number of chunks so that the threads' 16-byte reads hit distinct banks.
static int mma_raw_bytes(int type) {
    const int sbb = sb_bytes((uint32_t)type);
    int n = sbb % 16 == 0 ? sbb : ((sbb + 30) / 16) * 16;
    if (type == kQ8_0) {
        n += 16; // the funnel-shifted 2-byte-aligned reads touch one word past the last block
    }
    return (n / 16) % 2 ? n : n + 16;
}

cudaError_t launch_gemm_mma(cudaStream_t s, const CallDev & c, bool pdl_secondary, int32_t * dump, int dump_t) {
    MmaArgs a;
    memset(&a.g, 0, sizeof(a.g));
    a.c = c;
    a.dump = dump;
    a.dump_t = dump_t;
    int tiles = 0, need = 0;
    for (int i = 0; i < c.n_segs; i++) {
        tiles += (c.seg[i].n_rows + kTileM - 1) / kTileM;
        a.tiles_m[i] = tiles;
        const int n = mma_raw_bytes((int)c.seg[i].type);
        need = need > n ? need : n;
    }
    a.n_tiles_m = tiles;
    a.raw_bytes = need;
    a.lbo = 128;
    a.sbo = 256;
    bool pg2 = a.raw_bytes <= 240; // up to 32 tokens unpacking dominates: a second producer group where its staging fits
#ifdef B200Q_TUNING
    if (const char * e = getenv("B200Q_MMA_PG")) { // A/B builds only
        pg2 = pg2 && atoi(e) == 2;
    }
#endif
    // token tile: the fp32 epilogue costs in proportion to its width, so it is as narrow as the call allows
    if (c.TB <= 8) {
        return pg2 ? launch_nt<8, 1, 2>(s, a, pdl_secondary) : launch_nt<8, 1, 1>(s, a, pdl_secondary);
    }
    if (c.TB <= 16) {
        return pg2 ? launch_nt<16, 1, 2>(s, a, pdl_secondary) : launch_nt<16, 1, 1>(s, a, pdl_secondary);
    }
    if (c.TB <= 32) { // batched decode: unpacking dominates
        return pg2 ? launch_nt<32, 2, 2>(s, a, pdl_secondary) : launch_nt<32, 2, 1>(s, a, pdl_secondary);
    }
    // prefill: the fp32 epilogue dominates; two epilogue warpgroups share the token columns
    // One producer group: the epilogue is the bound, a second group only costs registers (A/B on
    // 17408 x 5120 Q4_K: 741 -> 716 us at 512 tokens, 2717 -> 2653 us at 2048).  Four epilogue warpgroups
    // instead of two (21 warps: 80 registers, spills) were slower: 761 us.
    return launch_nt<64, 2, 1>(s, a, pdl_secondary);
}

// ---- grouped form: the expert GEMMs of a routed-MoE call --------------------------------------------
bool moe_mma_supported(int type_a, int type_b, int K, int n_rows, int fuse) {
    return K >= 256 && (K & 255) == 0 && n_rows >= 1 && (!fuse || type_a == type_b);
}

cudaError_t launch_moe_mma(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                           size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                           const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                           const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                           float * out, int out_stride, int fuse) {
    if (!moe_mma_supported(type_a, type_b, K, n_rows, fuse) || n_act_max < 1 || TB < 1 ||
        (top_k > 0 ? (long long)TB * top_k : (long long)TB) > 0x7FFFFFFFLL) {
        return cudaErrorInvalidConfiguration;
    }
    MmaArgs a;
    memset(&a, 0, sizeof(a));
    a.c.K = K;
    a.c.TB = TB;
    a.c.x8 = x8;
    a.c.xmeta = xmeta;
    a.c.xsumq = xsumq;
    a.g.bank_a = static_cast<const uint8_t *>(bank_a);
    a.g.bank_b = static_cast<const uint8_t *>(fuse ? bank_b : bank_a);
    a.g.plane_a = plane_a;
    a.g.plane_b = fuse ? plane_b : plane_a;
    a.g.off = off;
    a.g.pair = pair;
    a.g.active = active;
    a.g.n_active = n_active;
    a.g.max_active = n_act_max;
    const long long n_pairs = top_k > 0 ? (long long)TB * top_k : TB;
    a.g.n_pairs = (int32_t)n_pairs;
    a.g.top_k = top_k;
    a.g.fuse = fuse;
    a.g.n_rows = n_rows;
    a.g.n_vec = TB;
    const int rows_per_tile = fuse ? kTileM / 2 : kTileM;
    a.g.tiles_per_expert = (n_rows + rows_per_tile - 1) / rows_per_tile;
    a.g.type = type_a;
    a.g.out = out;
    a.g.out_stride = out_stride;
    a.raw_bytes = mma_raw_bytes(type_a);
    a.lbo = 128;
    a.sbo = 256;
    // one producer group: the second one's 96-register limit makes this form spill (A/B at 512 tokens of
    // 256 experts top-8: 828 against 952 microseconds per call)
    bool pg2 = false;
    // token tile from the mean number of tokens per expert: an expert with more takes several tiles
    long long mean = (n_pairs + n_act_max - 1) / n_act_max;
#ifdef B200Q_TUNING
    if (const char * e = getenv("B200Q_MOE_NT")) { // A/B builds only: force the token tile and the producer groups
        mean = atoi(e) <= 16 ? 1 : (atoi(e) <= 32 ? 20 : 100);
    }
    if (const char * e = getenv("B200Q_MOE_PG")) {
        pg2 = a.raw_bytes <= 240 && atoi(e) == 2;
    }
#endif
    if (mean <= 10) {
        return pg2 ? launch_nt<16, 1, 2, true>(s, a, true) : launch_nt<16, 1, 1, true>(s, a, true);
    }
    if (mean <= 40) {
        return pg2 ? launch_nt<32, 2, 2, true>(s, a, true) : launch_nt<32, 2, 1, true>(s, a, true);
    }
    return (pg2 && a.raw_bytes <= 192) ? launch_nt<64, 2, 2, true>(s, a, true) : launch_nt<64, 2, 1, true>(s, a, true);
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
