// Batched decode GEMM (2..32 tokens) on register fragments: int8 mma.sync per 32-value group.
//
// At a handful of tokens the work is still the weight stream (HBM-bound), but every 32-value
// group carries its own fp32 scale on both sides, so each group's int32 dot must be folded
// into fp32 separately.  Here the dots come from warp-level int8 MMAs whose A operand is built
// in registers straight from the raw GGUF bytes in shared memory (a thread's share of a row's
// group is 8 bytes: two mask operations per nibble plane) and the fold runs in the same warp
// on the accumulator fragment - no operand staging in a tensor-core layout, no tensor-memory
// round trip, which is what bounds the tcgen05 kernel at few tokens.
//
// Tiling.  One CTA per SM, persistent over (segment, tile of M = 16*RG rows).  A stage of the
// shared-memory ring holds KB superblocks of all M rows - fetched as 2-D TMA tiles, one per
// alignment class of rows - plus the int8 codes, scales and sums of all tokens for those
// superblocks (three contiguous bulk copies: the activation layout is group-major).  The 16
// warps split as RG row groups x KS slices of the stage's superblocks x WT token
// halves; a warp owns 16 rows x NTW tokens of fp32 accumulators for the whole K loop, K slices
// are summed through shared memory at the end of a tile.  M adapts to the row count so that
// the tiles fill the SMs (5120 rows: M = 32 and four K slices; 17408 rows: M = 128).
//
// Rows whose byte pitch is not a multiple of 16 (Q6_K, IQ4_XS with an odd superblock count)
// cannot be described by one tensor map (TMA strides are multiples of 16 bytes): rows r with
// the same r mod P share their misalignment, so each of the P classes gets its own map with
// pitch P*row_bytes, and a warp's 16 rows all come from one class.
//
// MMA shapes: m16n8k32 (u8 x s8 for Q4_K / Q5_K, s8 x s8 for Q8_0 / IQ4_XS), m16n8k16 for
// Q6_K, whose scale groups are 16 values.  The k index of a fragment may be any permutation of
// the group's elements as long as A and B use the same one: a thread takes 8 consecutive
// elements, which is one 64-bit shared-memory load per row and per token.
//
// Every mbarrier wait is bounded; a wait that runs out records B200Q_ETIMEOUT and the role returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstring>

#include "async.cuh"
#include "decode.cuh"
#include "launch.h"

namespace b200q {

__device__ int g_frag_status = 0;

constexpr int kFragWarps = 16;
constexpr int kFragThreads = 32 * (kFragWarps + 1); // + the producer warp
constexpr int kFragSmem = 227 * 1024;
constexpr int kFragMaxMaps = 16;
constexpr int kFragHdr = 1024; // mbarriers; the ring behind it stays 1024-byte aligned

struct FragSeg {
    int32_t map0;      // first tensor map of the segment
    int32_t P;         // alignment classes: rows r with the same r % P share a map
    int32_t tile0;     // first tile of the segment in the call's tile list
    int32_t BW;        // box width = shared-memory row pitch, bytes
    int32_t mis[8];    // (w + j * row_bytes) & 15 per class
};

struct alignas(64) FragArgs {
    CUtensorMap maps[kFragMaxMaps];
    CallDev c;
    FragSeg seg[B200Q_MAX_SEGS];
    int32_t n_tiles;
    int32_t RG, KS, WT; // row groups (M = 16*RG), K slices, token halves; RG*KS*WT == 16
    int32_t SBW;        // superblocks per warp per stage; a stage covers KB = KS*SBW superblocks
    int32_t NTP;        // token columns (WT * NTW)
    int32_t stages, stage_bytes;
    int32_t off_x8, off_meta, off_sum, off_fac; // inside a stage
    int32_t off_red;                            // K-slice reduction buffer
    // parity instrument: the raw int32 group sums of token dump_t (dump[row * D + index]) instead of outputs
    int32_t * dump;
    int32_t dump_t;
};

// ---- warp-level int8 MMAs -------------------------------------------------------------------
template <bool A_SIGNED>
__device__ __forceinline__ void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    if (A_SIGNED) {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    } else {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    }
}
__device__ __forceinline__ void mma_k16_us(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// 32 bits from a 2-byte-aligned shared address
__device__ __forceinline__ uint32_t lds32_a2(uint32_t a) {
    const uint32_t q = a & ~3u, sh = (a & 2u) * 8;
    return __funnelshift_r(lds32(q), lds32(q + 4), sh);
}

// What a warp knows about its place: rows rowp[0] / rowp[1] (fragment rows gid and gid + 8) of
// the current superblock, the stage's activation arrays, its token window.
struct FragCtx {
    uint32_t rowp[2]; // shared address of the superblock in the two rows of this thread
    uint32_t x8s;     // int8 codes [group][TB][32]
    uint32_t facs;    // token factors [group][NTP] (8 or 16 bytes each)
    int gl0;          // index of the superblock's first group inside the stage
    int TB, NTP, tw0; // tokens, token columns, first token column of this warp
    int gid, tq;      // lane >> 2, lane & 3
    // parity instrument (dump != nullptr): where the sums of this thread's two rows go
    int32_t * dump;
    int dump_t, sbg;  // token, global superblock index
    long long drow[2]; // row * D, or -1 for a row beyond the segment
};

// store the fragment's sums of token x.dump_t: c[2e + j] is row e, token column tcol + j
__device__ __forceinline__ void frag_dump(const FragCtx & x, const int (&c)[4], int tcol, int index) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (tcol + (i & 1) == x.dump_t && x.drow[i >> 1] >= 0) {
            x.dump[x.drow[i >> 1] + index] = c[i];
        }
    }
}


template <int NTW> struct FragAcc {
    float v[NTW / 8][4];
};

// ---- Q4_K / Q5_K: one superblock, 16 rows x NTW tokens -------------------------------------------
template <int TYPE, int NTW> __device__ __forceinline__ void frag_sb_k45(const FragCtx & x, FragAcc<NTW> & acc) {
    constexpr uint32_t QOFF = TYPE == kQ4_K ? 16u : 48u;
    float d[2], dmin[2];
    uint32_t sc[2][2], mn[2][2], qh[2][2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const uint4 hdr = lds128(x.rowp[e]);
        d[e] = h2f((uint16_t)(hdr.x & 0xFFFF));
        dmin[e] = h2f((uint16_t)(hdr.x >> 16));
        // (scale, min) bytes of groups 0-3 and 4-7 (get_scale_min_k4, src/common/quant.h:136-144 of the reference)
        sc[e][0] = hdr.y & 0x3F3F3F3Fu;
        sc[e][1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y & 0xC0C0C0C0u) >> 2);
        mn[e][0] = hdr.z & 0x3F3F3F3Fu;
        mn[e][1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z & 0xC0C0C0C0u) >> 2);
        qh[e][0] = qh[e][1] = 0;
        if (TYPE == kQ5_K) { // bit g of qh[i] is the fifth bit of element i of group g
            const uint2 h = lds64(x.rowp[e] + 16 + 8 * x.tq);
            qh[e][0] = h.x;
            qh[e][1] = h.y;
        }
    }
    float ve[NTW / 8][4], ms[NTW / 8][4];
#pragma unroll
    for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            ve[nt][i] = 0.f;
            ms[nt][i] = 0.f;
        }
    }
#pragma unroll
    for (int pr = 0; pr < 4; pr++) {
        uint2 q[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            q[e] = lds64(x.rowp[e] + QOFF + 32 * pr + 8 * x.tq);
        }
#pragma unroll
        for (int half = 0; half < 2; half++) { // low nibbles = group 2pr, high nibbles = group 2pr+1
            const int G = 2 * pr + half;
            uint32_t a[4]; // a0: row gid, first four elements; a1: row gid+8; a2, a3: next four elements
#pragma unroll
            for (int e = 0; e < 2; e++) {
                uint32_t w0 = half ? (q[e].x >> 4) & 0x0F0F0F0Fu : q[e].x & 0x0F0F0F0Fu;
                uint32_t w1 = half ? (q[e].y >> 4) & 0x0F0F0F0Fu : q[e].y & 0x0F0F0F0Fu;
                if (TYPE == kQ5_K) {
                    w0 |= ((qh[e][0] >> G) & 0x01010101u) << 4;
                    w1 |= ((qh[e][1] >> G) & 0x01010101u) << 4;
                }
                a[e] = w0;
                a[2 + e] = w1;
            }
            int sci[2];
            float mnf[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                sci[e] = (int)((sc[e][G >> 2] >> (8 * (G & 3))) & 0xFF);
                mnf[e] = (float)((mn[e][G >> 2] >> (8 * (G & 3))) & 0xFF);
            }
            const int gl = x.gl0 + G;
#pragma unroll
            for (int nt = 0; nt < NTW / 8; nt++) {
                const int tok = min(x.tw0 + 8 * nt + x.gid, x.TB - 1);
                const uint2 b = lds64(x.x8s + (uint32_t)((gl * x.TB + tok) * 32 + 8 * x.tq));
                int c[4];
                mma_k32<false>(c, a[0], a[1], a[2], a[3], b.x, b.y);
                if (x.dump) {
                    frag_dump(x, c, x.tw0 + 8 * nt + 2 * x.tq, 8 * x.sbg + G);
                }
                // token columns 2*tq, 2*tq+1 of this n-tile: (sx, sx*xsum) each
                const uint4 f = lds128(x.facs + (uint32_t)((gl * x.NTP + x.tw0 + 8 * nt + 2 * x.tq) * 8));
                const float sx0 = __uint_as_float(f.x), c0 = __uint_as_float(f.y);
                const float sx1 = __uint_as_float(f.z), c1 = __uint_as_float(f.w);
#pragma unroll
                for (int e = 0; e < 2; e++) { // sc * wd is an exact integer below 2^24
                    ve[nt][2 * e] = fmaf(sx0, (float)(sci[e] * c[2 * e]), ve[nt][2 * e]);
                    ve[nt][2 * e + 1] = fmaf(sx1, (float)(sci[e] * c[2 * e + 1]), ve[nt][2 * e + 1]);
                    ms[nt][2 * e] = fmaf(mnf[e], c0, ms[nt][2 * e]);
                    ms[nt][2 * e + 1] = fmaf(mnf[e], c1, ms[nt][2 * e + 1]);
                }
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = i >> 1;
            acc.v[nt][i] += d[e] * ve[nt][i] - dmin[e] * ms[nt][i];
        }
    }
}

// ---- Q6_K: 16 scale groups of 16 values, m16n8k16 ----------------------------------------------
template <int NTW> __device__ __forceinline__ void frag_sb_q6(const FragCtx & x, FragAcc<NTW> & acc) {
    float ve[NTW / 8][4];
#pragma unroll
    for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            ve[nt][i] = 0.f;
        }
    }
    uint32_t sc8[2][4]; // the 16 int8 scales of each row
    float d[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
#pragma unroll
        for (int k = 0; k < 4; k++) {
            sc8[e][k] = lds32_a2(x.rowp[e] + 192 + 4 * k);
        }
        d[e] = h2f((uint16_t)lds16(x.rowp[e] + 208));
    }
#pragma unroll
    for (int blk2 = 0; blk2 < 2; blk2++) {
        uint32_t code[2][2][4]; // [row][half][plane]: four raw 6-bit codes each
#pragma unroll
        for (int e = 0; e < 2; e++) {
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const uint32_t qa = lds32_a2(x.rowp[e] + 64 * blk2 + 16 * half + 4 * x.tq);
                const uint32_t qb = lds32_a2(x.rowp[e] + 64 * blk2 + 32 + 16 * half + 4 * x.tq);
                const uint32_t hh = lds32_a2(x.rowp[e] + 128 + 32 * blk2 + 16 * half + 4 * x.tq);
                code[e][half][0] = (qa & 0x0F0F0F0Fu) | ((hh << 4) & 0x30303030u);
                code[e][half][1] = (qb & 0x0F0F0F0Fu) | ((hh << 2) & 0x30303030u);
                code[e][half][2] = ((qa >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u);
                code[e][half][3] = ((qb >> 4) & 0x0F0F0F0Fu) | ((hh >> 2) & 0x30303030u);
            }
        }
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const int gl = x.gl0 + 4 * blk2 + p; // activation group
#pragma unroll
            for (int nt = 0; nt < NTW / 8; nt++) {
                const int tok = min(x.tw0 + 8 * nt + x.gid, x.TB - 1);
                const uint32_t fa = x.facs + (uint32_t)((gl * x.NTP + x.tw0 + 8 * nt + 2 * x.tq) * 16);
                const uint4 f0 = lds128(fa), f1 = lds128(fa + 16); // (sx, 32*xs0, 32*xs1, -) of the two token columns
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const int s = 8 * blk2 + 2 * p + half; // scale group
                    const uint32_t b = lds32(x.x8s + (uint32_t)((gl * x.TB + tok) * 32 + 16 * half + 4 * x.tq));
                    int c[4];
                    mma_k16_us(c, code[0][half][p], code[1][half][p], b);
                    if (x.dump) {
                        frag_dump(x, c, x.tw0 + 8 * nt + 2 * x.tq, 16 * x.sbg + s);
                    }
                    const int off0 = half ? (int)f0.z : (int)f0.y, off1 = half ? (int)f1.z : (int)f1.y;
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int s8 = (int)(int8_t)(sc8[e][s >> 2] >> (8 * (s & 3)));
                        ve[nt][2 * e] = fmaf(__uint_as_float(f0.x), (float)(s8 * (c[2 * e] - off0)), ve[nt][2 * e]);
                        ve[nt][2 * e + 1] = fmaf(__uint_as_float(f1.x), (float)(s8 * (c[2 * e + 1] - off1)), ve[nt][2 * e + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            acc.v[nt][i] = fmaf(d[i >> 1], ve[nt][i], acc.v[nt][i]);
        }
    }
}

// ---- Q8_0 and IQ4_XS: one fp32 scale per (row, group), no offsets ----------------------------------
template <int TYPE, int NTW> __device__ __forceinline__ void frag_sb_signed(const FragCtx & x, FragAcc<NTW> & acc) {
    uint2 hdr[2] = {make_uint2(0, 0), make_uint2(0, 0)};
    if (TYPE == kIQ4_XS) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            hdr[e] = lds64(x.rowp[e]); // d | scales_h << 16, scales_l[4]
        }
    }
#pragma unroll
    for (int G = 0; G < 8; G++) {
        uint32_t a[4];
        float dl[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            if (TYPE == kQ8_0) { // 34-byte blocks: f16 d, 32 codes; this thread's eight codes start at 2 + 8*tq
                const uint32_t blk = x.rowp[e] + 34 * G;
                dl[e] = h2f((uint16_t)lds16(blk));
                a[e] = lds32_a2(blk + 2 + 8 * x.tq);
                a[2 + e] = lds32_a2(blk + 6 + 8 * x.tq);
            } else { // byte i of a group's 16: low nibble = element i, high nibble = element 16 + i
                const uint32_t w = lds32(x.rowp[e] + 8 + 16 * G + 4 * x.tq);
                a[e] = iq4nl_lookup4(w & 0x0F0F0F0Fu);
                a[2 + e] = iq4nl_lookup4((w >> 4) & 0x0F0F0F0Fu);
                const int ls = (int)((hdr[e].y >> (8 * (G >> 1) + 4 * (G & 1))) & 0xF) | (int)((((hdr[e].x >> 16) >> (2 * G)) & 3) << 4);
                dl[e] = h2f((uint16_t)(hdr[e].x & 0xFFFF)) * (float)(ls - 32);
            }
        }
        const int gl = x.gl0 + G;
#pragma unroll
        for (int nt = 0; nt < NTW / 8; nt++) {
            const int tok = min(x.tw0 + 8 * nt + x.gid, x.TB - 1);
            const uint32_t xa = x.x8s + (uint32_t)((gl * x.TB + tok) * 32);
            uint32_t b0, b1;
            if (TYPE == kQ8_0) { // elements 8*tq .. 8*tq+7
                const uint2 b = lds64(xa + 8 * x.tq);
                b0 = b.x, b1 = b.y;
            } else { // elements 4*tq .. and 16 + 4*tq ..
                b0 = lds32(xa + 4 * x.tq);
                b1 = lds32(xa + 16 + 4 * x.tq);
            }
            int c[4];
            mma_k32<true>(c, a[0], a[1], a[2], a[3], b0, b1);
            if (x.dump) {
                frag_dump(x, c, x.tw0 + 8 * nt + 2 * x.tq, 8 * x.sbg + G);
            }
            const uint4 f = lds128(x.facs + (uint32_t)((gl * x.NTP + x.tw0 + 8 * nt + 2 * x.tq) * 8));
            const float sx0 = __uint_as_float(f.x), sx1 = __uint_as_float(f.z);
#pragma unroll
            for (int e = 0; e < 2; e++) {
                acc.v[nt][2 * e] = fmaf(sx0 * dl[e], (float)c[2 * e], acc.v[nt][2 * e]);
                acc.v[nt][2 * e + 1] = fmaf(sx1 * dl[e], (float)c[2 * e + 1], acc.v[nt][2 * e + 1]);
            }
        }
    }
}

template <int TYPE, int NTW> __device__ __forceinline__ void frag_sb(const FragCtx & x, FragAcc<NTW> & acc) {
    if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        frag_sb_k45<TYPE, NTW>(x, acc);
    } else if constexpr (TYPE == kQ6_K) {
        frag_sb_q6<NTW>(x, acc);
    } else {
        frag_sb_signed<TYPE, NTW>(x, acc);
    }
}

struct FragBars {
    uint32_t full, empty;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap * map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}

// The copy side of the ring (one thread of the producer warp): the position of the next
// (tile, K chunk) to request.
struct FragProd {
    int tile, sb0, stage;
    uint32_t par;
};

// Request the next chunk, if there is one: wait (bounded) until all 16 warps have released the
// stage, then one TMA tile per alignment class of rows and three bulk copies for the activation.
__device__ __forceinline__ bool frag_produce(const FragArgs & a, uint32_t ring, const FragBars & bars, FragProd & p) {
    if (p.tile >= a.n_tiles) {
        return true;
    }
    const int nb = a.c.K >> 8, KB = a.KS * a.SBW, M = 16 * a.RG, TB = a.c.TB;
    int si = 0;
    while (si + 1 < a.c.n_segs && p.tile >= a.seg[si + 1].tile0) {
        si++;
    }
    const FragSeg & fs = a.seg[si];
    const int row0 = (p.tile - fs.tile0) * M, P = fs.P;
    const int sbb = sb_bytes(a.c.seg[si].type);
    const uint32_t box_bytes = (uint32_t)((M / P) * fs.BW);
    const int nsb = min(KB, nb - p.sb0);
    if (!mbar_wait(bars.empty + 8 * p.stage, p.par, &g_frag_status)) {
        return false;
    }
    const uint32_t st = ring + (uint32_t)(p.stage * a.stage_bytes), fb = bars.full + 8 * p.stage;
    const uint32_t ng = (uint32_t)(8 * nsb * TB);
    mbar_expect_tx(fb, (uint32_t)P * box_bytes + ng * 48u);
    for (int j = 0; j < P; j++) {
        const int xoff = ((fs.mis[j] + p.sb0 * sbb) & ~15) >> 2; // 32-bit elements; 16-byte aligned start
        tma_load_2d(st + (uint32_t)j * box_bytes, &a.maps[fs.map0 + j], xoff, row0 / P, fb);
    }
    const size_t g0 = (size_t)8 * p.sb0 * TB;
    bulk_g2s(st + a.off_x8, a.c.x8 + g0 * 32, ng * 32u, fb);
    bulk_g2s(st + a.off_meta, a.c.xmeta + g0 * 2, ng * 8u, fb);
    bulk_g2s(st + a.off_sum, a.c.xsumq + g0 * 2, ng * 8u, fb);
    if (++p.stage == a.stages) {
        p.stage = 0;
        p.par ^= 1;
    }
    p.sb0 += KB;
    if (p.sb0 >= nb) {
        p.sb0 = 0;
        p.tile += gridDim.x;
    }
    return true;
}

// One tile (M rows of one segment, all K): the 16 warps.
template <int TYPE, int NTW>
__device__ __forceinline__ bool frag_tile(const FragArgs & a, int si, int row0, uint32_t ring, uint32_t red,
                                          const FragBars & bars, int & stage, uint32_t & phase) {
    constexpr int SB = Fmt<TYPE>::SB;
    constexpr int FB = TYPE == kQ6_K ? 16 : 8; // bytes per token factor
    const SegDev & sg = a.c.seg[si];
    const FragSeg & fs = a.seg[si];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wt = warp % a.WT, ks = (warp / a.WT) % a.KS, rg = warp / (a.WT * a.KS);
    const int nb = a.c.K >> 8, TB = a.c.TB, NTP = a.NTP, KB = a.KS * a.SBW;
    const int M = 16 * a.RG, P = fs.P;
    // this warp's 16 rows: class j of the tile, rows j + P*(16*(rg/P) + i)
    const int cls = rg % P, first = 16 * (rg / P);
    FragCtx x;
    x.gid = lane >> 2;
    x.tq = lane & 3;
    x.TB = TB;
    x.NTP = NTP;
    x.tw0 = wt * NTW;
    x.dump = a.dump;
    x.dump_t = a.dump_t;
    {
        const long long D = (long long)(TYPE == kQ6_K ? 16 : 8) * nb;
        for (int e = 0; e < 2; e++) {
            const int row = row0 + cls + P * (first + x.gid + 8 * e);
            x.drow[e] = row < sg.n_rows ? (long long)row * D : -1;
        }
    }
    FragAcc<NTW> acc;
#pragma unroll
    for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            acc.v[nt][i] = 0.f;
        }
    }
    const uint32_t region = (uint32_t)(cls * (M / P) * fs.BW);
    for (int sb0 = 0; sb0 < nb; sb0 += KB) {
        if (!mbar_wait(bars.full + 8 * stage, phase, &g_frag_status)) {
            return false;
        }
        const uint32_t st = ring + (uint32_t)(stage * a.stage_bytes);
        const int nsb = min(KB, nb - sb0);
        // token factors of the stage's groups, zero beyond the last token
        for (int e = threadIdx.x; e < 8 * nsb * NTP; e += 32 * kFragWarps) {
            const int g = e / NTP, t = e - g * NTP;
            float sx = 0.f;
            int s0 = 0, s1 = 0;
            if (t < TB) {
                sx = __uint_as_float(lds32(st + a.off_meta + (uint32_t)((g * TB + t) * 8)));
                const uint2 s = lds64(st + a.off_sum + (uint32_t)((g * TB + t) * 8));
                s0 = (int)s.x;
                s1 = (int)s.y;
            }
            if (FB == 16) {
                sts128(st + a.off_fac + (uint32_t)e * 16, __float_as_uint(sx), (uint32_t)(32 * s0), (uint32_t)(32 * s1), 0u);
            } else {
                asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(st + a.off_fac + (uint32_t)e * 8), "r"(__float_as_uint(sx)),
                             "r"(__float_as_uint(sx * (float)(s0 + s1)))
                             : "memory");
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kFragWarps) : "memory");
        x.x8s = st + a.off_x8;
        x.facs = st + a.off_fac;
        const uint32_t mis = (uint32_t)(fs.mis[cls] + sb0 * SB) & 15u;
        for (int s = 0; s < a.SBW; s++) {
            const int sl = ks * a.SBW + s; // superblock inside the stage
            if (sl < nsb) {
                x.gl0 = 8 * sl;
                x.sbg = sb0 + sl;
                const uint32_t base = st + region + mis + (uint32_t)(sl * SB);
                x.rowp[0] = base + (uint32_t)((first + x.gid) * fs.BW);
                x.rowp[1] = base + (uint32_t)((first + x.gid + 8) * fs.BW);
                frag_sb<TYPE, NTW>(x, acc);
            }
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(bars.empty + 8 * stage);
        }
        if (++stage == a.stages) {
            stage = 0;
            phase ^= 1;
        }
    }
    // K slices: partial sums through shared memory, added in slice order by slice 0
    if (a.KS > 1) {
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kFragWarps) : "memory"); // the buffer is free (previous tile's readers are done)
#pragma unroll
        for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = 16 * rg + x.gid + 8 * (i >> 1), t = x.tw0 + 8 * nt + 2 * x.tq + (i & 1);
                sts32(red + (uint32_t)(((ks * M + r) * NTP + t) * 4), __float_as_uint(acc.v[nt][i]));
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kFragWarps) : "memory");
        if (ks == 0) {
#pragma unroll
            for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = 16 * rg + x.gid + 8 * (i >> 1), t = x.tw0 + 8 * nt + 2 * x.tq + (i & 1);
                    float v = 0.f;
                    for (int k = 0; k < a.KS; k++) {
                        v += __uint_as_float(lds32(red + (uint32_t)(((k * M + r) * NTP + t) * 4)));
                    }
                    acc.v[nt][i] = v;
                }
            }
        }
    }
    if (ks == 0 && !a.dump) {
#pragma unroll
        for (int nt = 0; nt < NTW / 8; nt++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = row0 + cls + P * (first + x.gid + 8 * (i >> 1));
                const int t = x.tw0 + 8 * nt + 2 * x.tq + (i & 1);
                if (row < sg.n_rows && t < TB) {
                    const size_t o = (size_t)t * sg.out_stride + row;
                    float v = sg.alpha * acc.v[nt][i];
                    if (sg.residual) {
                        v += sg.residual[o];
                    }
                    store_out(a.c, &sg.out[o], v);
                }
            }
        }
    }
    return true;
}

template <int NTW> __global__ void __launch_bounds__(kFragThreads, 1) gemm_frag_kernel(const __grid_constant__ FragArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const FragBars bars{base, base + 64};
    const uint32_t ring = base + kFragHdr, red = base + (uint32_t)a.off_red;
    const int M = 16 * a.RG;

    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; s++) {
            mbar_init(bars.full + 8 * s, 1);
            mbar_init(bars.empty + 8 * s, kFragWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // the activation views are read by the copies below: wait for the kernel that wrote them
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if ((threadIdx.x >> 5) == kFragWarps) {
        // ------------------------------------------------------------------ producer (one thread)
        if ((threadIdx.x & 31) == 0) {
            FragProd prod{(int)blockIdx.x, 0, 0, 1u};
            while (prod.tile < a.n_tiles) {
                if (!frag_produce(a, ring, bars, prod)) {
                    return;
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    int stage = 0;
    uint32_t phase = 0;
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
        int si = 0;
        while (si + 1 < a.c.n_segs && tile >= a.seg[si + 1].tile0) {
            si++;
        }
        const int row0 = (tile - a.seg[si].tile0) * M;
        bool ok;
        switch (a.c.seg[si].type) {
        case kQ4_K: ok = frag_tile<kQ4_K, NTW>(a, si, row0, ring, red, bars, stage, phase); break;
        case kQ5_K: ok = frag_tile<kQ5_K, NTW>(a, si, row0, ring, red, bars, stage, phase); break;
        case kQ6_K: ok = frag_tile<kQ6_K, NTW>(a, si, row0, ring, red, bars, stage, phase); break;
        case kIQ4_XS: ok = frag_tile<kIQ4_XS, NTW>(a, si, row0, ring, red, bars, stage, phase); break;
        default: ok = frag_tile<kQ8_0, NTW>(a, si, row0, ring, red, bars, stage, phase); break;
        }
        if (!ok) {
            return;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled fn = [] {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            p = nullptr;
        }
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    }();
    return fn;
}

static int align_classes(int row_bytes) { // rows r, r + P, ... start at the same offset inside a 16-byte line
    int P = 1;
    while ((row_bytes * P) & 15) {
        P *= 2;
    }
    return P;
}

static bool frag_plan(const CallDev & c, FragArgs & a, int & NTW) {
    if (c.TB < 2 || c.TB > 32 || (c.K & 255)) {
        return false;
    }
    if (((reinterpret_cast<uintptr_t>(c.x8) | reinterpret_cast<uintptr_t>(c.xmeta) | reinterpret_cast<uintptr_t>(c.xsumq)) & 15) != 0) {
        return false; // the activation chunks travel as bulk copies
    }
    const int nb = c.K >> 8;
    NTW = c.TB <= 16 ? 8 : 16;
    a.WT = c.TB <= 8 ? 1 : 2;
    a.NTP = NTW * a.WT;
    int Pmax = 1, max_sbb = 0;
    for (int i = 0; i < c.n_segs; i++) {
        const int sbb = sb_bytes(c.seg[i].type), P = align_classes(nb * sbb);
        Pmax = Pmax > P ? Pmax : P;
        max_sbb = max_sbb > sbb ? max_sbb : sbb;
    }
    // K slices share a stage, and a stage's K extent is one TMA box of at most 1024 bytes per row
    const int ks_max = (1024 - 30) / max_sbb;
    // rows per tile: the largest M = 16*RG whose tiles still fill the SMs within 10 % of the best
    // fill (large tiles share a stage's activation among more rows; measured: M = 128 with 90 KB
    // stages beats M = 64 with 50 KB stages by a third on 17408 x 5120)
    const int rk = kFragWarps / a.WT; // RG * KS
    double best = -1.0;
    int best_rg = 0;
    for (int pass = 0; pass < 2 && !best_rg; pass++) {
        for (int rg = rk; rg >= 1; rg /= 2) {
            if (rg < Pmax || rk / rg > ks_max) {
                break;
            }
            long tiles = 0;
            for (int i = 0; i < c.n_segs; i++) {
                tiles += (c.seg[i].n_rows + 16 * rg - 1) / (16 * rg);
            }
            const long waves = (tiles + kSMs - 1) / kSMs;
            const double fill = (double)c.total_rows / ((double)waves * kSMs * 16 * rg); // useful rows per row slot
            if (pass == 0) {
                best = fill > best ? fill : best;
            } else if (fill >= best - 0.10) {
                best_rg = rg;
                break;
            }
        }
    }
    if (!best_rg) {
        return false;
    }
    a.RG = best_rg;
    a.KS = rk / best_rg;
    const int M = 16 * a.RG;
    // superblocks per stage: two per warp when two stages of that fit, else one
    a.SBW = 0;
    for (int sbw = 2; sbw >= 1 && !a.SBW; sbw--) {
        const int KB = a.KS * sbw;
        size_t wbytes = 0;
        bool ok = true;
        for (int i = 0; i < c.n_segs; i++) {
            const int sbb = sb_bytes(c.seg[i].type), P = align_classes(nb * sbb);
            const int BW = (P > 1 || (sbb & 15)) ? ((KB * sbb + 15 + 15) / 16) * 16 : KB * sbb;
            ok = ok && BW <= 1024;
            a.seg[i].BW = BW;
            a.seg[i].P = P;
            const size_t wb = (size_t)M * BW;
            wbytes = wbytes > wb ? wbytes : wb;
        }
        const size_t ng = (size_t)8 * KB * c.TB;
        const size_t off_x8 = (wbytes + 127) / 128 * 128;
        const size_t off_meta = off_x8 + ng * 32, off_sum = off_meta + ng * 8;
        const size_t off_fac = (off_sum + ng * 8 + 15) / 16 * 16;
        const size_t stage = (off_fac + (size_t)8 * KB * a.NTP * 16 + 1023) / 1024 * 1024;
        const size_t red_bytes = a.KS > 1 ? (size_t)a.KS * M * a.NTP * 4 : 0;
        const size_t room = (size_t)kFragSmem - kFragHdr - red_bytes;
        if (!ok || 2 * stage > room || wbytes + ng * 48 >= (1u << 20)) {
            continue;
        }
        const int stages = (int)(room / stage);
        a.SBW = sbw;
        a.stages = stages > 8 ? 8 : stages;
        a.stage_bytes = (int32_t)stage;
        a.off_x8 = (int32_t)off_x8;
        a.off_meta = (int32_t)off_meta;
        a.off_sum = (int32_t)off_sum;
        a.off_fac = (int32_t)off_fac;
        a.off_red = (int32_t)(kFragHdr + (size_t)a.stages * stage);
    }
    if (!a.SBW) {
        return false;
    }
    int tiles = 0, maps = 0;
    for (int i = 0; i < c.n_segs; i++) {
        a.seg[i].tile0 = tiles;
        a.seg[i].map0 = maps;
        tiles += (c.seg[i].n_rows + M - 1) / M;
        maps += a.seg[i].P;
        if (a.RG % a.seg[i].P) {
            return false;
        }
    }
    a.n_tiles = tiles;
    return maps <= kFragMaxMaps;
}

bool frag_supported(const CallDev & c) {
    FragArgs a;
    int NTW;
    return tensor_map_encoder() != nullptr && frag_plan(c, a, NTW);
}

cudaError_t launch_gemm_frag(cudaStream_t s, const CallDev & c, int32_t * dump, int dump_t) {
    FragArgs a;
    memset(&a, 0, sizeof(a));
    a.c = c;
    a.dump = dump;
    a.dump_t = dump_t;
    int NTW = 8;
    if (!frag_plan(c, a, NTW)) {
        return cudaErrorInvalidConfiguration;
    }
    PFN_cuTensorMapEncodeTiled encode = tensor_map_encoder();
    if (!encode) {
        return cudaErrorNotSupported;
    }
    const int nb = c.K >> 8, M = 16 * a.RG;
    for (int i = 0; i < c.n_segs; i++) {
        FragSeg & fs = a.seg[i];
        const size_t row_bytes = (size_t)nb * sb_bytes(c.seg[i].type);
        for (int j = 0; j < fs.P; j++) {
            const uintptr_t A = reinterpret_cast<uintptr_t>(c.seg[i].w) + (size_t)j * row_bytes;
            fs.mis[j] = (int32_t)(A & 15);
            const long rows_j = (c.seg[i].n_rows - j + fs.P - 1) / fs.P;
            if (rows_j <= 0) { // fewer rows than classes: the map is never read from a valid row; keep it legal
                fs.mis[j] = 0;
            }
            // bytes of a row counted from the 16-byte boundary below its start, up to the end of the
            // 16-byte line that holds its last byte; reads past that are zero-filled by the copy engine
            const cuuint64_t dims[2] = {(cuuint64_t)(((A & 15) + row_bytes + 15) / 16 * 4), (cuuint64_t)(rows_j > 0 ? rows_j : 1)};
            const cuuint64_t strides[1] = {(cuuint64_t)(row_bytes * fs.P)};
            const cuuint32_t box[2] = {(cuuint32_t)(fs.BW / 4), (cuuint32_t)(M / fs.P)};
            const cuuint32_t estr[2] = {1, 1};
            const CUresult r = encode(&a.maps[fs.map0 + j], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2,
                                      reinterpret_cast<void *>(rows_j > 0 ? (A & ~uintptr_t(15)) : (reinterpret_cast<uintptr_t>(c.seg[i].w))),
                                      dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) {
                return cudaErrorInvalidValue;
            }
        }
    }
    const size_t smem = (size_t)a.off_red + (a.KS > 1 ? (size_t)a.KS * M * a.NTP * 4 : 0);
    const void * fn = NTW == 8 ? reinterpret_cast<const void *>(gemm_frag_kernel<8>) : reinterpret_cast<const void *>(gemm_frag_kernel<16>);
    cudaError_t e = ensure_dynamic_smem(fn, kFragSmem);
    if (e != cudaSuccess) {
        return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.n_tiles < kSMs ? a.n_tiles : kSMs));
    cfg.blockDim = dim3(kFragThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return NTW == 8 ? cudaLaunchKernelEx(&cfg, gemm_frag_kernel<8>, a) : cudaLaunchKernelEx(&cfg, gemm_frag_kernel<16>, a);
}

cudaError_t read_frag_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_frag_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_frag_status, &zero, sizeof(int));
    }
    return e;
}

} // namespace b200q
