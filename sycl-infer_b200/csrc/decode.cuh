// In-register decode of raw GGUF blocks + dp4a against int8 activation groups.
//
// A 256-value superblock is split into 8 "parts" of 32 weights; one lane owns one
// part.  `Part<TYPE, WM>::load` reads and unpacks the part's weights once (they are
// reused for every token of the call); `dots` forms the exact int32 sums against one
// token's int8 codes; `term` applies the fp32 scales exactly as the reference's CPU
// path composes them (src/backend/cpu/kernels/i8.cpp:40-155 of the reference):
//   Q4_K/Q5_K  sx * (d*sc * wd - dmin*m * xsum)
//   Q6_K       sx * d*sc_s * (wd - 32*xsum)      (formed here as the dot of q-32)
//   Q8_0       sx * d * wd                        (src/backend/cpu/kernels/q4exp.cpp:442-470)
//   IQ4_XS     sx * d*(ls-32) * wd                (block layout src/common/quant.h:978-991)
// Which 32 weights a part holds, and which activation bytes they meet:
//   Q4_K/Q5_K  part j: bytes 16j..16j+15 of qs -> elements 16*(j&1).. of groups 2*(j>>1)
//              (low nibbles) and 2*(j>>1)+1 (high nibbles)
//   Q6_K       part j: blk2 = j>>2, l0 = 8*(j&3): 8 elements at offset l0 of each of the
//              groups 4*blk2 + plane, plane 0..3
//   Q8_0 / IQ4_XS  part j = group j, all 32 elements
#pragma once
#include "common.cuh"

namespace b200q {

struct ActView {
    const int8_t * x8;
    const float * xmeta;
    const int32_t * xsumq;
    int TB;
};

// ---- weight memory policies ------------------------------------------------------
// Global memory through the read-only path.  Alignment-2 reads are assembled from
// aligned 32-bit words with a funnel shift and never touch a word past the last byte
// requested.
struct GmemW {
    static __device__ __forceinline__ uint4 ld128(const uint8_t * p) {
        return __ldg(reinterpret_cast<const uint4 *>(p));
    }
    static __device__ __forceinline__ uint2 ld64(const uint8_t * p) {
        return __ldg(reinterpret_cast<const uint2 *>(p));
    }
    static __device__ __forceinline__ uint32_t ld16(const uint8_t * p) {
        return __ldg(reinterpret_cast<const uint16_t *>(p));
    }
    static __device__ __forceinline__ int ld8s(const uint8_t * p) {
        return (int)__ldg(reinterpret_cast<const int8_t *>(p));
    }
    template <int N> static __device__ __forceinline__ void ld_a2(const uint8_t * p, uint32_t (&out)[N]) {
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        const uint32_t * q = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
        const uint32_t sh = (uint32_t)(a & 2) * 8;
        uint32_t prev = __ldg(q);
#pragma unroll
        for (int k = 0; k < N; k++) {
            const uint32_t next = (k + 1 < N || sh) ? __ldg(q + k + 1) : 0u;
            out[k] = __funnelshift_r(prev, next, sh);
            prev = next;
        }
    }
};

// Shared memory (a staged tile), explicit ld.shared.  The tile buffer carries slack after
// the last byte, so the trailing word of a misaligned read may be fetched unconditionally.
__device__ __forceinline__ uint32_t smem_u32(const void * p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

struct SmemW {
    static __device__ __forceinline__ uint4 ld128(const uint8_t * p) { return lds128(smem_u32(p)); }
    static __device__ __forceinline__ uint2 ld64(const uint8_t * p) { return lds64(smem_u32(p)); }
    static __device__ __forceinline__ uint32_t ld16(const uint8_t * p) { return lds16(smem_u32(p)); }
    static __device__ __forceinline__ int ld8s(const uint8_t * p) {
        int v;
        asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)));
        return v;
    }
    template <int N> static __device__ __forceinline__ void ld_a2(const uint8_t * p, uint32_t (&out)[N]) {
        const uint32_t a = smem_u32(p);
        const uint32_t sh = (a & 2u) * 8;
        const uint32_t q = a & ~3u;
        uint32_t prev = lds32(q);
#pragma unroll
        for (int k = 0; k < N; k++) {
            const uint32_t next = lds32(q + 4 * (k + 1));
            out[k] = __funnelshift_r(prev, next, sh);
            prev = next;
        }
    }
};

// ---- activation memory policies (same group-major layout in either space) ---------
struct GmemA {
    static __device__ __forceinline__ uint4 ld128(const int8_t * p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
    static __device__ __forceinline__ uint2 ld64(const int8_t * p) { return __ldg(reinterpret_cast<const uint2 *>(p)); }
    static __device__ __forceinline__ float ldf(const float * p) { return __ldg(p); }
    static __device__ __forceinline__ int ldi(const int32_t * p) { return __ldg(p); }
};
struct SmemA {
    static __device__ __forceinline__ uint4 ld128(const int8_t * p) { return lds128(smem_u32(p)); }
    static __device__ __forceinline__ uint2 ld64(const int8_t * p) { return lds64(smem_u32(p)); }
    static __device__ __forceinline__ float ldf(const float * p) { return __uint_as_float(lds32(smem_u32(p))); }
    static __device__ __forceinline__ int ldi(const int32_t * p) { return (int)lds32(smem_u32(p)); }
};

__device__ __forceinline__ int dp4a_us(uint32_t w, uint32_t x, int acc) { // unsigned weights x signed codes
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(x), "r"(acc));
    return r;
}
__device__ __forceinline__ int dp4a_ss(uint32_t w, uint32_t x, int acc) {
    int r;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(x), "r"(acc));
    return r;
}

// (scale, min) 6-bit pair g of a Q4_K/Q5_K superblock from its 12 packed bytes
// (get_scale_min_k4, src/common/quant.h:136-144 of the reference); s0,s1,s2 = bytes 0-3, 4-7, 8-11.
__device__ __forceinline__ void k4_scale_min(int g, uint32_t s0, uint32_t s1, uint32_t s2, int & sc, int & mn) {
    const int sh = 8 * (g & 3);
    const uint32_t b0 = (s0 >> sh) & 0xFF, b1 = (s1 >> sh) & 0xFF, b2 = (s2 >> sh) & 0xFF;
    if (g < 4) {
        sc = b0 & 63;
        mn = b1 & 63;
    } else {
        sc = (b2 & 0xF) | ((b0 >> 6) << 4);
        mn = (b2 >> 4) | ((b1 >> 6) << 4);
    }
}

template <int TYPE, class WM> struct Part;

// ------------------------------------------------------------------------- Q4_K / Q5_K
template <int TYPE, class WM> struct PartK45 {
    static constexpr int NP = 2;
    uint32_t lo[4], hi[4];
    float dsc[2], dmm[2];
    int g0, half;

    __device__ __forceinline__ void load(const uint8_t * sb, int j) {
        const uint4 hdr = WM::ld128(sb);
        half = j & 1;
        g0 = j & ~1; // groups g0 (low nibbles) and g0+1 (high nibbles)
        uint4 q;
        if (TYPE == kQ4_K) {
            q = WM::ld128(sb + 16 + 16 * j);
        } else {
            q = WM::ld128(sb + 48 + 16 * j);
        }
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            lo[k] = qw[k] & 0x0F0F0F0Fu;
            hi[k] = (qw[k] >> 4) & 0x0F0F0F0Fu;
        }
        if (TYPE == kQ5_K) { // bit g of qh[i] is the fifth bit of element i of group g
            const uint4 h = WM::ld128(sb + 16 + 16 * half);
            const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                lo[k] |= ((hw[k] >> g0) & 0x01010101u) << 4;
                hi[k] |= ((hw[k] >> (g0 + 1)) & 0x01010101u) << 4;
            }
        }
        const float d = h2f((uint16_t)(hdr.x & 0xFFFF)), dmin = h2f((uint16_t)(hdr.x >> 16));
#pragma unroll
        for (int i = 0; i < 2; i++) {
            int sc, mn;
            k4_scale_min(g0 + i, hdr.y, hdr.z, hdr.w, sc, mn);
            dsc[i] = d * (float)sc;
            dmm[i] = dmin * (float)mn;
        }
    }
    // exact int32 sums of this part against token t; idx[] = position in the row's dot array
    template <class AM = GmemA>
    __device__ __forceinline__ void dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const size_t gi = (size_t)(G0 + g0 + i) * a.TB + t;
            const uint4 x = AM::ld128(a.x8 + gi * 32 + 16 * half);
            const uint32_t * w = i ? hi : lo;
            wd[i] = dp4a_us(w[0], x.x, dp4a_us(w[1], x.y, dp4a_us(w[2], x.z, dp4a_us(w[3], x.w, 0))));
            idx[i] = G0 + g0 + i;
        }
    }
    __device__ __forceinline__ void raw_dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
        dots(a, G0, t, wd, idx);
    }
    template <class AM = GmemA>
    __device__ __forceinline__ float term(const ActView & a, int G0, int t) const {
        int wd[NP], idx[NP];
        dots<AM>(a, G0, t, wd, idx);
        float r = 0.f;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const size_t gi = (size_t)idx[i] * a.TB + t;
            const float sx = AM::ldf(a.xmeta + 2 * gi);
            const int xs = AM::ldi(a.xsumq + 2 * gi + half);
            r += sx * (dsc[i] * (float)wd[i] - dmm[i] * (float)xs);
        }
        return r;
    }
};
template <class WM> struct Part<kQ4_K, WM> : PartK45<kQ4_K, WM> {};
template <class WM> struct Part<kQ5_K, WM> : PartK45<kQ5_K, WM> {};

// ------------------------------------------------------------------------------- Q6_K
template <class WM> struct Part<kQ6_K, WM> {
    static constexpr int NP = 4;
    uint32_t v[4][2]; // (q - 32) as signed bytes, plane p, 8 elements
    float ds[4];
    int gb, l0; // first group (4*blk2), element offset

    __device__ __forceinline__ void load(const uint8_t * sb, int j) {
        const int blk2 = j >> 2;
        l0 = 8 * (j & 3);
        gb = 4 * blk2;
        uint32_t qa[2], qb[2], qh[2], sc[2];
        WM::template ld_a2<2>(sb + 64 * blk2 + l0, qa);
        WM::template ld_a2<2>(sb + 64 * blk2 + 32 + l0, qb);
        WM::template ld_a2<2>(sb + 128 + 32 * blk2 + l0, qh);
        WM::template ld_a2<2>(sb + 192 + 8 * blk2, sc);
        const float d = h2f((uint16_t)WM::ld16(sb + 208));
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const uint32_t a = qa[k], b = qb[k], h = qh[k];
            v[0][k] = __vsub4((a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u), 0x20202020u);
            v[1][k] = __vsub4((b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u), 0x20202020u);
            v[2][k] = __vsub4(((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u), 0x20202020u);
            v[3][k] = __vsub4(((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u), 0x20202020u);
        }
        const int hs = l0 >> 4; // which 16-value half of the group -> which of its two scales
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const int bi = hs + 2 * p; // byte 0..7 of the 8 scales of this 128-value half
            const uint32_t word = bi < 4 ? sc[0] : sc[1];
            const int s8 = (int)(int8_t)((word >> (8 * (bi & 3))) & 0xFF);
            ds[p] = d * (float)s8;
        }
    }
    // wd[] here are the dots of (q-32): what `term` needs.  raw_dots adds the 32*sum(x)
    // back so the parity instrument reports the reference's raw-code sums.
    template <class AM = GmemA>
    __device__ __forceinline__ void dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const size_t gi = (size_t)(G0 + gb + p) * a.TB + t;
            const uint2 x = AM::ld64(a.x8 + gi * 32 + l0);
            wd[p] = dp4a_ss(v[p][0], x.x, dp4a_ss(v[p][1], x.y, 0));
            idx[p] = G0 + gb + p;
        }
    }
    // raw-code sums per 16-value scale group: idx = 2*group + half
    __device__ __forceinline__ void raw_dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
        dots(a, G0, t, wd, idx);
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const size_t gi = (size_t)idx[p] * a.TB + t;
            const uint2 x = __ldg(reinterpret_cast<const uint2 *>(a.x8 + gi * 32 + l0));
            wd[p] += 32 * dp4a_ss(0x01010101u, x.x, dp4a_ss(0x01010101u, x.y, 0));
            idx[p] = 2 * idx[p] + (l0 >> 4);
        }
    }
    template <class AM = GmemA>
    __device__ __forceinline__ float term(const ActView & a, int G0, int t) const {
        int wd[NP], idx[NP];
        dots<AM>(a, G0, t, wd, idx);
        float r = 0.f;
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const float sx = AM::ldf(a.xmeta + 2 * ((size_t)idx[p] * a.TB + t));
            r += (sx * ds[p]) * (float)wd[p];
        }
        return r;
    }
};

// ----------------------------------------------------------------------------- IQ4_XS
// 16-entry signed codebook kvalues_iq4nl (src/common/quant.h:417 of the reference),
// packed little-endian four entries per word for byte-permute lookups.
__device__ __forceinline__ uint32_t iq4nl_lookup4(uint32_t idx /* four indices 0..15, one per byte */) {
    constexpr uint32_t T0 = 0xBFAD9881u; // -127 -104 -83 -65
    constexpr uint32_t T1 = 0xF6EADDCFu; //  -49  -35 -22 -10
    constexpr uint32_t T2 = 0x26190D01u; //    1   13  25  38
    constexpr uint32_t T3 = 0x71594535u; //   53   69  89 113
    const uint32_t s = idx & 0x07070707u;
    const uint32_t t = s | (s >> 4);
    const uint32_t sel = __byte_perm(t, 0, 0x0020); // four 3-bit selectors packed as nibbles
    const uint32_t lo = __byte_perm(T0, T1, sel);
    const uint32_t hi = __byte_perm(T2, T3, sel);
    const uint32_t m = ((idx >> 3) & 0x01010101u) * 0xFFu; // bytes whose index is >= 8
    return (lo & ~m) | (hi & m);
}

template <class WM> struct Part<kIQ4_XS, WM> {
    static constexpr int NP = 1;
    uint32_t v[8]; // codebook values, elements 0..31
    float dl;
    int g;

    __device__ __forceinline__ void load(const uint8_t * sb, int j) {
        g = j;
        const uint2 hdr = WM::ld64(sb); // d | scales_h << 16, scales_l[4]
        const int ls = (int)((hdr.y >> (8 * (j >> 1) + 4 * (j & 1))) & 0xF) | (int)((((hdr.x >> 16) >> (2 * j)) & 3) << 4);
        dl = h2f((uint16_t)(hdr.x & 0xFFFF)) * (float)(ls - 32);
        const uint2 q0 = WM::ld64(sb + 8 + 16 * j), q1 = WM::ld64(sb + 16 + 16 * j);
        const uint32_t qw[4] = {q0.x, q0.y, q1.x, q1.y};
#pragma unroll
        for (int k = 0; k < 4; k++) { // byte i: low nibble = element i, high nibble = element 16+i
            v[k] = iq4nl_lookup4(qw[k] & 0x0F0F0F0Fu);
            v[4 + k] = iq4nl_lookup4((qw[k] >> 4) & 0x0F0F0F0Fu);
        }
    }
    template <class AM = GmemA>
    __device__ __forceinline__ void dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
        const size_t gi = (size_t)(G0 + g) * a.TB + t;
        const uint4 x0 = AM::ld128(a.x8 + gi * 32);
        const uint4 x1 = AM::ld128(a.x8 + gi * 32 + 16);
        int s = dp4a_ss(v[0], x0.x, dp4a_ss(v[1], x0.y, dp4a_ss(v[2], x0.z, dp4a_ss(v[3], x0.w, 0))));
        s = dp4a_ss(v[4], x1.x, dp4a_ss(v[5], x1.y, dp4a_ss(v[6], x1.z, dp4a_ss(v[7], x1.w, s))));
        wd[0] = s;
        idx[0] = G0 + g;
    }
    __device__ __forceinline__ void raw_dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
        dots(a, G0, t, wd, idx);
    }
    template <class AM = GmemA>
    __device__ __forceinline__ float term(const ActView & a, int G0, int t) const {
        int wd[NP], idx[NP];
        dots<AM>(a, G0, t, wd, idx);
        const float sx = AM::ldf(a.xmeta + 2 * ((size_t)idx[0] * a.TB + t));
        return (sx * dl) * (float)wd[0];
    }
};

// ------------------------------------------------------------------------------- Q8_0
template <class WM> struct Part<kQ8_0, WM> {
    static constexpr int NP = 1;
    uint32_t v[8];
    float d;
    int g;

    __device__ __forceinline__ void load(const uint8_t * sb, int j) {
        g = j;
        const uint8_t * blk = sb + 34 * j;
        d = h2f((uint16_t)WM::ld16(blk));
        WM::template ld_a2<8>(blk + 2, v);
    }
    template <class AM = GmemA>
    __device__ __forceinline__ void dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
        const size_t gi = (size_t)(G0 + g) * a.TB + t;
        const uint4 x0 = AM::ld128(a.x8 + gi * 32);
        const uint4 x1 = AM::ld128(a.x8 + gi * 32 + 16);
        int s = dp4a_ss(v[0], x0.x, dp4a_ss(v[1], x0.y, dp4a_ss(v[2], x0.z, dp4a_ss(v[3], x0.w, 0))));
        s = dp4a_ss(v[4], x1.x, dp4a_ss(v[5], x1.y, dp4a_ss(v[6], x1.z, dp4a_ss(v[7], x1.w, s))));
        wd[0] = s;
        idx[0] = G0 + g;
    }
    __device__ __forceinline__ void raw_dots(const ActView & a, int G0, int t, int (&wd)[NP], int (&idx)[NP]) const {
        dots(a, G0, t, wd, idx);
    }
    template <class AM = GmemA>
    __device__ __forceinline__ float term(const ActView & a, int G0, int t) const {
        int wd[NP], idx[NP];
        dots<AM>(a, G0, t, wd, idx);
        const float sx = AM::ldf(a.xmeta + 2 * ((size_t)idx[0] * a.TB + t));
        return (sx * d) * (float)wd[0];
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    }
    return v;
}

} // namespace b200q
