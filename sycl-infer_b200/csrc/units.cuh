// Lean per-type decode for the streaming kernel.
//
// Work unit: a quarter of a 256-value superblock (64 weights); four lanes cover a
// superblock.  Which weights unit u holds:
//   Q4_K / Q5_K     groups 2u (low nibbles of qs[32u..32u+31]) and 2u+1 (high nibbles)
//   Q6_K            blk2 = u>>1, hs = u&1: elements 16hs..16hs+15 of the four groups
//                   4*blk2 + plane (plane 0..3)
//   Q8_0 / IQ4_XS   groups 2u and 2u+1
// The activation a unit meets is loaded separately (ActG2 / ActG6) so that it is read
// from shared memory once and reused by every weight row a warp owns.
//
// Integer sums are exact; two shortcuts keep them exact while saving instructions:
//   * a high nibble is used in place ((q & 0xF0) = 16*hi), its scale carries the 1/16;
//     Q5_K's high group uses 8*(hi + 16*bit) <= 248 with a 1/8 in the scale.  Scaling an
//     fp32 by a power of two is exact, so the products are the reference's, bit for bit.
//   * Q6_K keeps the raw 0..63 codes and subtracts 32*sum(x) as an integer, the form the
//     reference uses (src/backend/cpu/kernels/i8.cpp:150-152 of the reference).
// fp32 composition per group follows the reference's association
// (src/backend/cpu/kernels/i8.cpp:59): sx * ((d*sc)*wd - (dmin*m)*xsum).
#pragma once
#include "decode.cuh"

namespace b200q {

// ---- activation pack in shared memory (single-token calls) ----------------------------
// Per 32-value group 48 bytes: int8 codes [32] | sx (f32) | xs0 (i32) | xs1 (i32) | sx*(float)(xs0+xs1);
// eight groups (one superblock) are followed by 16 bytes of padding so that the eight
// lanes of a quarter-warp hit distinct banks.
constexpr int kPackGroup = 48;
constexpr int kPackSB = 8 * kPackGroup + 16;

__device__ __forceinline__ uint32_t pack_addr(uint32_t pack, int g) {
    return pack + (uint32_t)((g >> 3) * kPackSB + (g & 7) * kPackGroup);
}

// four consecutive groups with both 16-value sums each, for a Q6_K half unit
struct ActG6H {
    uint32_t x[4][8];
    float sx[4];
    int xs[4][2];
};

struct GroupMeta {
    float sx;
    int xs0, xs1;
    float xsf; // (float)(xs0 + xs1)
};

// four consecutive groups (half a superblock), all 32 codes each, for a Q4_K/Q5_K half unit;
// c = sx * (float)(xs0 + xs1) is the activation side of the min term
struct ActG4 {
    uint32_t x[4][8];
    float sx[4], c[4];
};

// The same four groups with everything any weight type needs (scales, min-term factors and
// both 16-value sums): the activation of one 128-value unit as a thread keeps it in
// registers for a whole launch (gemv_pinned.cu)
struct ActPin {
    uint32_t x[4][8];
    float sx[4], c[4];
    int xs[4][2];
};

// two consecutive groups, all 32 codes each
struct ActG2 {
    uint32_t xa[8], xb[8];
    GroupMeta ma, mb;
};

// four groups, 16 codes each (one half), for a Q6_K unit
struct ActG6 {
    uint32_t x[4][4];
    float sx[4];
    int xs[4];
};

__device__ __forceinline__ void meta_from(const uint4 & v, GroupMeta & m) {
    m.sx = __uint_as_float(v.x);
    m.xs0 = (int)v.y;
    m.xs1 = (int)v.z;
    m.xsf = (float)(m.xs0 + m.xs1);
}

struct PackA { // staged pack, token 0
    uint32_t pack;
    __device__ __forceinline__ void g2(int g, int, ActG2 & a) const {
        const uint32_t p = pack_addr(pack, g); // g even: both groups in the same superblock
        const uint4 a0 = lds128(p), a1 = lds128(p + 16), am = lds128(p + 32);
        const uint4 b0 = lds128(p + 48), b1 = lds128(p + 64), bm = lds128(p + 80);
        a.xa[0] = a0.x, a.xa[1] = a0.y, a.xa[2] = a0.z, a.xa[3] = a0.w;
        a.xa[4] = a1.x, a.xa[5] = a1.y, a.xa[6] = a1.z, a.xa[7] = a1.w;
        a.xb[0] = b0.x, a.xb[1] = b0.y, a.xb[2] = b0.z, a.xb[3] = b0.w;
        a.xb[4] = b1.x, a.xb[5] = b1.y, a.xb[6] = b1.z, a.xb[7] = b1.w;
        meta_from(am, a.ma);
        meta_from(bm, a.mb);
    }
    __device__ __forceinline__ void g4(int g, ActG4 & a) const { // g a multiple of 4
        const uint32_t p0 = pack_addr(pack, g);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t p = p0 + i * kPackGroup;
            const uint4 x0 = lds128(p), x1 = lds128(p + 16), m = lds128(p + 32);
            a.x[i][0] = x0.x, a.x[i][1] = x0.y, a.x[i][2] = x0.z, a.x[i][3] = x0.w;
            a.x[i][4] = x1.x, a.x[i][5] = x1.y, a.x[i][6] = x1.z, a.x[i][7] = x1.w;
            a.sx[i] = __uint_as_float(m.x);
            a.c[i] = __uint_as_float(m.w);
        }
    }
    __device__ __forceinline__ void g6h(int g, ActG6H & a) const { // g a multiple of 4
        const uint32_t p0 = pack_addr(pack, g);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t p = p0 + i * kPackGroup;
            const uint4 x0 = lds128(p), x1 = lds128(p + 16), m = lds128(p + 32);
            a.x[i][0] = x0.x, a.x[i][1] = x0.y, a.x[i][2] = x0.z, a.x[i][3] = x0.w;
            a.x[i][4] = x1.x, a.x[i][5] = x1.y, a.x[i][6] = x1.z, a.x[i][7] = x1.w;
            a.sx[i] = __uint_as_float(m.x);
            a.xs[i][0] = (int)m.y;
            a.xs[i][1] = (int)m.z;
        }
    }
    __device__ __forceinline__ void g6(int g, int hs, int, ActG6 & a) const {
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const uint32_t q = pack_addr(pack, g + p);
            const uint4 x = lds128(q + 16 * hs), m = lds128(q + 32);
            a.x[p][0] = x.x, a.x[p][1] = x.y, a.x[p][2] = x.z, a.x[p][3] = x.w;
            a.sx[p] = __uint_as_float(m.x);
            a.xs[p] = hs ? (int)m.z : (int)m.y;
        }
    }
};

struct PackT { // staged packs of several tokens, `stride` bytes apart
    uint32_t pack, stride;
    int TB;
    __device__ __forceinline__ void g2(int g, int t, ActG2 & a) const {
        PackA{pack + (uint32_t)t * stride}.g2(g, 0, a);
    }
    __device__ __forceinline__ void g6(int g, int hs, int t, ActG6 & a) const {
        PackA{pack + (uint32_t)t * stride}.g6(g, hs, 0, a);
    }
};

// 16 bytes from a 2-byte-aligned shared address: five aligned words, funnel-shifted
__device__ __forceinline__ void lds128_a2(uint32_t a, uint32_t (&o)[4]) {
    const uint32_t sh = (a & 2u) * 8, q = a & ~3u;
    uint32_t w0 = lds32(q), w1 = lds32(q + 4), w2 = lds32(q + 8), w3 = lds32(q + 12), w4 = lds32(q + 16);
    o[0] = __funnelshift_r(w0, w1, sh);
    o[1] = __funnelshift_r(w1, w2, sh);
    o[2] = __funnelshift_r(w2, w3, sh);
    o[3] = __funnelshift_r(w3, w4, sh);
}

template <int TYPE> struct WUnit;

// ------------------------------------------------------------------------ Q4_K / Q5_K
template <int TYPE> struct WUnitK45 {
    using Act = ActG2;
    static constexpr int kHiShift = TYPE == kQ4_K ? 4 : 3; // high group is scaled by 16 (Q4_K) or 8 (Q5_K)
    uint32_t lo[8], hi[8];
    float dscA, dscB, dmmA, dmmB;

    __device__ __forceinline__ void load(uint32_t sb, int u) {
        const uint4 hdr = lds128(sb);
        const uint32_t qoff = TYPE == kQ4_K ? 16u : 48u;
        const uint4 q0 = lds128(sb + qoff + 32 * u), q1 = lds128(sb + qoff + 32 * u + 16);
        const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        if (TYPE == kQ4_K) {
#pragma unroll
            for (int k = 0; k < 8; k++) {
                lo[k] = q[k] & 0x0F0F0F0Fu;
                hi[k] = q[k] & 0xF0F0F0F0u;
            }
        } else { // bit 2u / 2u+1 of qh[i] is the fifth bit of element i of the low / high group
            const uint4 h0 = lds128(sb + 16), h1 = lds128(sb + 32);
            const uint32_t h[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const uint32_t t = h[k] >> (2 * u);
                lo[k] = (q[k] & 0x0F0F0F0Fu) | ((t & 0x01010101u) << 4);
                hi[k] = ((q[k] >> 1) & 0x78787878u) | ((t & 0x02020202u) << 6);
            }
        }
        // 6-bit (scale, min) of groups 2u, 2u+1 (get_scale_min_k4, src/common/quant.h:136-144
        // of the reference), two at a time in 16-bit lanes
        const uint32_t sh = 16 * (u & 1);
        const uint32_t y = (hdr.y >> sh) & 0xFFFF, z = (hdr.z >> sh) & 0xFFFF, w = (hdr.w >> sh) & 0xFFFF;
        uint32_t sc, mn;
        if (u < 2) {
            sc = y & 0x3F3F;
            mn = z & 0x3F3F;
        } else {
            const uint32_t y0 = hdr.y >> sh, z0 = hdr.z >> sh; // groups 4..7 borrow the top bits of 0..3
            sc = (w & 0x0F0F) | ((y0 & 0xC0C0) >> 2);
            mn = ((w >> 4) & 0x0F0F) | ((z0 & 0xC0C0) >> 2);
        }
        const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
        dscA = d * (float)(sc & 0xFF);
        dscB = (d * (TYPE == kQ4_K ? 0.0625f : 0.125f)) * (float)(sc >> 8);
        dmmA = dmin * (float)(mn & 0xFF);
        dmmB = dmin * (float)(mn >> 8);
    }
    // exact int32 sums of the two groups (the high group's sum is returned unscaled)
    __device__ __forceinline__ void dots(const ActG2 & a, int & wa, int & wb) const {
        int sa = 0, sb = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            sa = dp4a_us(lo[k], a.xa[k], sa);
            sb = dp4a_us(hi[k], a.xb[k], sb);
        }
        wa = sa;
        wb = sb;
    }
    __device__ __forceinline__ float term(const ActG2 & a) const {
        int wa, wb;
        dots(a, wa, wb);
        const float ta = dscA * (float)wa - dmmA * a.ma.xsf;
        const float tb = dscB * (float)wb - dmmB * a.mb.xsf;
        return a.ma.sx * ta + a.mb.sx * tb;
    }
    __device__ __forceinline__ void exact(const ActG2 & a, int G, int32_t * wd) const {
        int wa, wb;
        dots(a, wa, wb);
        wd[G] = wa;
        wd[G + 1] = wb >> kHiShift;
    }
};
template <> struct WUnit<kQ4_K> : WUnitK45<kQ4_K> {};
template <> struct WUnit<kQ5_K> : WUnitK45<kQ5_K> {};

// Half a Q4_K/Q5_K superblock (groups 4h..4h+3, 128 weights) for single-token calls: the
// four 6-bit (scale, min) pairs of a half unpack with a handful of 32-bit operations
// (bytes 0-3 / 4-7 hold groups 0-3 directly; groups 4-7 take four bits from bytes 8-11 and
// two from the top of bytes 0-7), and the fp32 work is factored as
//   d * sum_g sx_g * float(sc_g * wd_g)  -  dmin * sum_g m_g * (sx_g * xsum_g)
// (sc_g * wd_g is an exact integer) so only two multiplies per superblock half touch d and dmin.
template <int TYPE> struct HalfK45 {
    static constexpr int kHiShift = TYPE == kQ4_K ? 4 : 3;
    static constexpr float kHiScale = TYPE == kQ4_K ? 0.0625f : 0.125f;

    // exact sums of the four groups; odd groups come scaled by 1 << kHiShift
    template <class A> static __device__ __forceinline__ void dots(uint32_t sb, int h, const A & a, int (&w)[4]) {
        const uint32_t qs = sb + (TYPE == kQ4_K ? 16u : 48u) + 64u * h;
        uint32_t hq[8];
        if (TYPE == kQ5_K) {
            const uint4 h0 = lds128(sb + 16), h1 = lds128(sb + 32);
            hq[0] = h0.x, hq[1] = h0.y, hq[2] = h0.z, hq[3] = h0.w;
            hq[4] = h1.x, hq[5] = h1.y, hq[6] = h1.z, hq[7] = h1.w;
        }
#pragma unroll
        for (int pr = 0; pr < 2; pr++) { // pair pr: groups 4h+2pr (low nibbles), 4h+2pr+1 (high)
            const uint4 q0 = lds128(qs + 32 * pr), q1 = lds128(qs + 32 * pr + 16);
            const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            int sa0 = 0, sa1 = 0, sb0 = 0, sb1 = 0;
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                uint32_t lo0, hi0, lo1, hi1;
                if (TYPE == kQ4_K) {
                    lo0 = q[k] & 0x0F0F0F0Fu, hi0 = q[k] & 0xF0F0F0F0u;
                    lo1 = q[k + 1] & 0x0F0F0F0Fu, hi1 = q[k + 1] & 0xF0F0F0F0u;
                } else { // bit g of qh[i] is the fifth bit of element i of group g
                    const uint32_t t0 = hq[k] >> (4 * h + 2 * pr), t1 = hq[k + 1] >> (4 * h + 2 * pr);
                    lo0 = (q[k] & 0x0F0F0F0Fu) | ((t0 & 0x01010101u) << 4);
                    hi0 = ((q[k] >> 1) & 0x78787878u) | ((t0 & 0x02020202u) << 6);
                    lo1 = (q[k + 1] & 0x0F0F0F0Fu) | ((t1 & 0x01010101u) << 4);
                    hi1 = ((q[k + 1] >> 1) & 0x78787878u) | ((t1 & 0x02020202u) << 6);
                }
                sa0 = dp4a_us(lo0, a.x[2 * pr][k], sa0);
                sb0 = dp4a_us(hi0, a.x[2 * pr + 1][k], sb0);
                sa1 = dp4a_us(lo1, a.x[2 * pr][k + 1], sa1);
                sb1 = dp4a_us(hi1, a.x[2 * pr + 1][k + 1], sb1);
            }
            w[2 * pr] = sa0 + sa1;
            w[2 * pr + 1] = sb0 + sb1;
        }
    }
    template <class A> static __device__ __forceinline__ float term(uint32_t sb, int h, const A & a) {
        const uint4 hdr = lds128(sb);
        int w[4];
        dots(sb, h, a, w);
        // (scale, min) of groups 4h..4h+3 (get_scale_min_k4, src/common/quant.h:136-144 of the reference)
        const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, mn_lo = hdr.z & 0x3F3F3F3Fu;
        const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y & 0xC0C0C0C0u) >> 2);
        const uint32_t mn_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z & 0xC0C0C0C0u) >> 2);
        const uint32_t sc = h ? sc_hi : sc_lo, mn = h ? mn_hi : mn_lo;
        float ve = 0.f, vo = 0.f, ms = 0.f;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            // the 6-bit scale times the group's sum as an integer (below 2^22, times 16 for odd
            // groups: exactly representable), so one conversion and one FMA apply the scale
            const int scg = (int)__byte_perm(sc, 0, 0x4440 + g), mng = (int)__byte_perm(mn, 0, 0x4440 + g);
            const float t = (float)(scg * w[g]);
            if (g & 1) {
                vo = fmaf(a.sx[g], t, vo);
            } else {
                ve = fmaf(a.sx[g], t, ve);
            }
            ms = fmaf((float)mng, a.c[g], ms);
        }
        const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
        return d * fmaf(vo, kHiScale, ve) - dmin * ms;
    }
    template <class A> static __device__ __forceinline__ void exact(uint32_t sb, int h, const A & a, int G, int32_t * wd) {
        int w[4];
        dots(sb, h, a, w);
        wd[G] = w[0];
        wd[G + 1] = w[1] >> kHiShift;
        wd[G + 2] = w[2];
        wd[G + 3] = w[3] >> kHiShift;
    }
};

// ------------------------------------------------------------------------------- Q6_K
template <> struct WUnit<kQ6_K> {
    using Act = ActG6;
    uint32_t v[4][4]; // raw codes 0..63, plane p, 16 elements
    float ds[4];

    __device__ __forceinline__ void load(uint32_t sb, int u) {
        const int blk2 = u >> 1, hs = u & 1;
        uint32_t qa[4], qb[4], qh[4];
        lds128_a2(sb + 64 * blk2 + 16 * hs, qa);
        lds128_a2(sb + 64 * blk2 + 32 + 16 * hs, qb);
        lds128_a2(sb + 128 + 32 * blk2 + 16 * hs, qh);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t a = qa[k], b = qb[k], h = qh[k];
            v[0][k] = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
            v[1][k] = (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
            v[2][k] = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
            v[3][k] = ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
        }
        const float d = h2f((uint16_t)lds16(sb + 208));
#pragma unroll
        for (int p = 0; p < 4; p++) {
            int s8;
            asm volatile("ld.shared.s8 %0, [%1];" : "=r"(s8) : "r"(sb + 192 + 8 * blk2 + 2 * p + hs));
            ds[p] = d * (float)s8;
        }
    }
    __device__ __forceinline__ void dots(const ActG6 & a, int (&w)[4]) const {
#pragma unroll
        for (int p = 0; p < 4; p++) {
            int s = 0;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                s = dp4a_us(v[p][k], a.x[p][k], s);
            }
            w[p] = s;
        }
    }
    // raw-code sums per 16-value scale group: index 2*group + half
    __device__ __forceinline__ void exact(const ActG6 & a, int G, int hs, int32_t * wd) const {
        int w[4];
        dots(a, w);
#pragma unroll
        for (int p = 0; p < 4; p++) {
            wd[2 * (G + p) + hs] = w[p];
        }
    }
    __device__ __forceinline__ float term(const ActG6 & a) const {
        int w[4];
        dots(a, w);
        float r = 0.f;
#pragma unroll
        for (int p = 0; p < 4; p++) {
            r += (a.sx[p] * ds[p]) * (float)(w[p] - 32 * a.xs[p]);
        }
        return r;
    }
};

// Half a Q6_K superblock (groups 4h..4h+3, 128 weights) for single-token calls.  Against the
// quarter unit above it reads every activation group whole (both 16-value halves), so a unit
// moves 176 bytes of activation for 96 bytes of weights instead of 2 x 128 for 2 x 48: the
// quarter unit is bound by shared-memory bandwidth, not by HBM.  The int8 block scale is
// folded in as an integer, sum_half s8 * (wd - 32 * xsum) (below 2^24, so its conversion to
// fp32 is exact), leaving one conversion and one FMA per group and a single multiply by d.
struct HalfQ6 {
    // raw-code sums per 16-value scale group: w[plane][half]
    template <class A> static __device__ __forceinline__ void dots(uint32_t sb, int h, const A & a, int (&w)[4][2]) {
        const uint32_t sh = (sb & 2u) * 8, q = (sb & ~3u) + 64u * h, qhp = (sb & ~3u) + 128u + 32u * h;
#pragma unroll
        for (int hs = 0; hs < 2; hs++) {
            uint32_t wa[5], wb[5], wh[5];
#pragma unroll
            for (int k = 0; k < 5; k++) { // aligned words; the block is only 2-byte aligned
                wa[k] = lds32(q + 16 * hs + 4 * k);
                wb[k] = lds32(q + 32 + 16 * hs + 4 * k);
                wh[k] = lds32(qhp + 16 * hs + 4 * k);
            }
            int s0 = 0, s1 = 0, s2 = 0, s3 = 0;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t qa = __funnelshift_r(wa[k], wa[k + 1], sh), qb = __funnelshift_r(wb[k], wb[k + 1], sh);
                const uint32_t hh = __funnelshift_r(wh[k], wh[k + 1], sh);
                s0 = dp4a_us((qa & 0x0F0F0F0Fu) | ((hh << 4) & 0x30303030u), a.x[0][4 * hs + k], s0);
                s1 = dp4a_us((qb & 0x0F0F0F0Fu) | ((hh << 2) & 0x30303030u), a.x[1][4 * hs + k], s1);
                s2 = dp4a_us(((qa >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u), a.x[2][4 * hs + k], s2);
                s3 = dp4a_us(((qb >> 4) & 0x0F0F0F0Fu) | ((hh >> 2) & 0x30303030u), a.x[3][4 * hs + k], s3);
            }
            w[0][hs] = s0, w[1][hs] = s1, w[2][hs] = s2, w[3][hs] = s3;
        }
    }
    template <class A> static __device__ __forceinline__ float term(uint32_t sb, int h, const A & a) {
        int w[4][2];
        dots(sb, h, a, w);
        // the half's eight int8 scales: scales[8h + 2*plane + half]
        const uint32_t sh = (sb & 2u) * 8, sp = (sb & ~3u) + 192u + 8u * h;
        const uint32_t c0 = lds32(sp), c1 = lds32(sp + 4), c2 = lds32(sp + 8);
        const uint32_t sc[2] = {__funnelshift_r(c0, c1, sh), __funnelshift_r(c1, c2, sh)};
        float r = 0.f;
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const int sa = (int)(int8_t)(sc[p >> 1] >> (16 * (p & 1))), sb8 = (int)(int8_t)(sc[p >> 1] >> (16 * (p & 1) + 8));
            const int t = sa * (w[p][0] - 32 * a.xs[p][0]) + sb8 * (w[p][1] - 32 * a.xs[p][1]);
            r = fmaf(a.sx[p], (float)t, r);
        }
        return h2f((uint16_t)lds16(sb + 208)) * r;
    }
    template <class A> static __device__ __forceinline__ void exact(uint32_t sb, int h, const A & a, int G, int32_t * wd) {
        int w[4][2];
        dots(sb, h, a, w);
#pragma unroll
        for (int p = 0; p < 4; p++) {
            wd[2 * (G + p)] = w[p][0];
            wd[2 * (G + p) + 1] = w[p][1];
        }
    }
};

// ----------------------------------------------------------------------------- IQ4_XS
// Codebook kvalues_iq4nl (src/common/quant.h:417 of the reference) as four little-endian words.
// A 32-bit word of eight 4-bit indices n0..n7 is looked up with byte permutes whose
// selectors are the indices themselves: result word 0 holds kv[n0],kv[n1],kv[n2],kv[n3].
// Since n0,n2 are low nibbles (elements i, i+1) and n1,n3 high nibbles (elements 16+i, 17+i),
// the activation bytes are interleaved the same way before the dp4a.
// prmt.b32 in its default mode: a selector nibble with bit 3 set replicates the sign bit of
// the selected byte (the __byte_perm intrinsic only defines the low three bits)
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ void iq4_lookup8(uint32_t q, uint32_t & r0, uint32_t & r1) {
    constexpr uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;
    const uint32_t s = q & 0x77777777u;
    const uint32_t l0 = prmt(T0, T1, s), l1 = prmt(T0, T1, s >> 16);
    const uint32_t h0 = prmt(T2, T3, s), h1 = prmt(T2, T3, s >> 16);
    // byte masks from bit 3 of every nibble: sign-replicating permutes of q (odd nibbles)
    // and q << 4 (even nibbles), interleaved in nibble order
    const uint32_t e = q << 4;
    const uint32_t m0 = prmt(e, q, 0xD9C8), m1 = prmt(e, q, 0xFBEA);
    r0 = (l0 & ~m0) | (h0 & m0);
    r1 = (l1 & ~m1) | (h1 & m1);
}

template <> struct WUnit<kIQ4_XS> {
    using Act = ActG2;
    uint32_t v[16]; // codebook values; word pairs in interleaved element order
    float dlA, dlB;

    __device__ __forceinline__ void load(uint32_t sb, int u) {
        const uint2 hdr = lds64(sb); // d | scales_h << 16, scales_l[4]
        const uint32_t sl = (hdr.y >> (8 * u)) & 0xFF, shh = (hdr.x >> (16 + 4 * u)) & 0xF;
        const int lsA = (int)((sl & 0xF) | ((shh & 3) << 4)), lsB = (int)((sl >> 4) | ((shh >> 2) << 4));
        const float d = h2f((uint16_t)(hdr.x & 0xFFFF));
        dlA = d * (float)(lsA - 32);
        dlB = d * (float)(lsB - 32);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint2 q = lds64(sb + 8 + 32 * u + 8 * k);
            iq4_lookup8(q.x, v[4 * k], v[4 * k + 1]);
            iq4_lookup8(q.y, v[4 * k + 2], v[4 * k + 3]);
        }
    }
    // group g of the unit occupies v[8g..8g+7]; word pair (2j, 2j+1) covers index word j:
    // elements 4j..4j+3 (low nibbles) and 16+4j..19+4j (high nibbles), interleaved
    static __device__ __forceinline__ int group_dot(const uint32_t * vv, const uint32_t * x) {
        int s = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t xl = x[j], xh = x[4 + j];
            s = dp4a_ss(vv[2 * j], __byte_perm(xl, xh, 0x5140), s);
            s = dp4a_ss(vv[2 * j + 1], __byte_perm(xl, xh, 0x7362), s);
        }
        return s;
    }
    __device__ __forceinline__ void dots(const ActG2 & a, int & wa, int & wb) const {
        wa = group_dot(v, a.xa);
        wb = group_dot(v + 8, a.xb);
    }
    __device__ __forceinline__ float term(const ActG2 & a) const {
        int wa, wb;
        dots(a, wa, wb);
        return (a.ma.sx * dlA) * (float)wa + (a.mb.sx * dlB) * (float)wb;
    }
    __device__ __forceinline__ void exact(const ActG2 & a, int G, int32_t * wd) const {
        dots(a, wd[G], wd[G + 1]);
    }
};

// ------------------------------------------------------------------------------- Q8_0
template <> struct WUnit<kQ8_0> {
    using Act = ActG2;
    uint32_t va[8], vb[8];
    float dA, dB;

    __device__ __forceinline__ void load(uint32_t sb, int u) {
        const uint32_t ba = sb + 68 * u, bb = ba + 34;
        dA = h2f((uint16_t)lds16(ba));
        dB = h2f((uint16_t)lds16(bb));
        uint32_t t[4];
        lds128_a2(ba + 2, t);
        va[0] = t[0], va[1] = t[1], va[2] = t[2], va[3] = t[3];
        lds128_a2(ba + 18, t);
        va[4] = t[0], va[5] = t[1], va[6] = t[2], va[7] = t[3];
        lds128_a2(bb + 2, t);
        vb[0] = t[0], vb[1] = t[1], vb[2] = t[2], vb[3] = t[3];
        lds128_a2(bb + 18, t);
        vb[4] = t[0], vb[5] = t[1], vb[6] = t[2], vb[7] = t[3];
    }
    __device__ __forceinline__ void dots(const ActG2 & a, int & wa, int & wb) const {
        int sa = 0, sb = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            sa = dp4a_ss(va[k], a.xa[k], sa);
            sb = dp4a_ss(vb[k], a.xb[k], sb);
        }
        wa = sa;
        wb = sb;
    }
    __device__ __forceinline__ float term(const ActG2 & a) const {
        int wa, wb;
        dots(a, wa, wb);
        return (a.ma.sx * dA) * (float)wa + (a.mb.sx * dB) * (float)wb;
    }
    __device__ __forceinline__ void exact(const ActG2 & a, int G, int32_t * wd) const {
        dots(a, wd[G], wd[G + 1]);
    }
};

// load the activation of unit u of superblock `sbi` (token t) for any weight type
template <int TYPE, class AS>
__device__ __forceinline__ void load_act(const AS & as, int sbi, int u, int t, typename WUnit<TYPE>::Act & a) {
    if constexpr (TYPE == kQ6_K) {
        as.g6(8 * sbi + 4 * (u >> 1), u & 1, t, a);
    } else {
        as.g2(8 * sbi + 2 * u, t, a);
    }
}

// exact int32 sums of unit u of superblock sbi into the row's dot array
template <int TYPE>
__device__ __forceinline__ void unit_exact(const WUnit<TYPE> & w, const typename WUnit<TYPE>::Act & a, int sbi, int u,
                                           int32_t * wd) {
    if constexpr (TYPE == kQ6_K) {
        w.exact(a, 8 * sbi + 4 * (u >> 1), u & 1, wd);
    } else {
        w.exact(a, 8 * sbi + 2 * u, wd);
    }
}

// ---- the unit a single-token call works in -----------------------------------------------
// H units per superblock; the activation of a unit is loaded once (from the pack) and met
// by every row the warp owns.
template <int TYPE> struct Unit1 {
    static constexpr int H = 4;
    using Act = typename WUnit<TYPE>::Act;
    static __device__ __forceinline__ void load_act(const PackA & as, int sbi, int u, Act & a) {
        b200q::load_act<TYPE>(as, sbi, u, 0, a);
    }
    static __device__ __forceinline__ float term(uint32_t sb, int u, const Act & a) {
        WUnit<TYPE> w;
        w.load(sb, u);
        return w.term(a);
    }
    static __device__ __forceinline__ void exact(uint32_t sb, int sbi, int u, const Act & a, int32_t * wd) {
        WUnit<TYPE> w;
        w.load(sb, u);
        unit_exact<TYPE>(w, a, sbi, u, wd);
    }
};
template <int TYPE> struct Unit1K45 {
    static constexpr int H = 2;
    using Act = ActG4;
    static __device__ __forceinline__ void load_act(const PackA & as, int sbi, int u, Act & a) {
        as.g4(8 * sbi + 4 * u, a);
    }
    static __device__ __forceinline__ float term(uint32_t sb, int u, const Act & a) {
        return HalfK45<TYPE>::term(sb, u, a);
    }
    static __device__ __forceinline__ void exact(uint32_t sb, int sbi, int u, const Act & a, int32_t * wd) {
        HalfK45<TYPE>::exact(sb, u, a, 8 * sbi + 4 * u, wd);
    }
};
template <> struct Unit1<kQ6_K> {
    static constexpr int H = 2;
    using Act = ActG6H;
    static __device__ __forceinline__ void load_act(const PackA & as, int sbi, int u, Act & a) {
        as.g6h(8 * sbi + 4 * u, a);
    }
    static __device__ __forceinline__ float term(uint32_t sb, int u, const Act & a) { return HalfQ6::term(sb, u, a); }
    static __device__ __forceinline__ void exact(uint32_t sb, int sbi, int u, const Act & a, int32_t * wd) {
        HalfQ6::exact(sb, u, a, 8 * sbi + 4 * u, wd);
    }
};
template <> struct Unit1<kQ4_K> : Unit1K45<kQ4_K> {};
template <> struct Unit1<kQ5_K> : Unit1K45<kQ5_K> {};

} // namespace b200q
