// Device code shared by the streaming GEMV kernels: the activation pack, one warp's work on one
// tile, and the byte-balanced split of a call's rows.
#pragma once
#include "async.cuh"
#include "units.cuh"
#include "xq.cuh"

namespace b200q {

constexpr int kConsumerWarps = 8; // consumer warps of one ring: a tile is kConsumerWarps x RW rows

// Pack of token `tok` of a TB-token activation (group-major views).
__device__ __forceinline__ void stage_pack_token(uint32_t pack, const CallDev & c, int tok, int n_sb, int tid, int nthr) {
    for (int g = tid; g < 8 * n_sb; g += nthr) {
        const size_t gi = (size_t)g * c.TB + tok;
        const uint4 * gx = reinterpret_cast<const uint4 *>(c.x8 + gi * 32);
        const uint4 x0 = __ldg(gx), x1 = __ldg(gx + 1);
        const float sx = __ldg(c.xmeta + 2 * gi);
        const int2 xs = __ldg(reinterpret_cast<const int2 *>(c.xsumq) + gi);
        const uint32_t p = pack_addr(pack, g);
        sts128(p, x0.x, x0.y, x0.z, x0.w);
        sts128(p + 16, x1.x, x1.y, x1.z, x1.w);
        sts128(p + 32, __float_as_uint(sx), (uint32_t)xs.x, (uint32_t)xs.y, __float_as_uint(sx * (float)(xs.x + xs.y)));
    }
}

// One warp, RW rows, one tile, one token.  A superblock is H units (Unit1<TYPE>::H); lane l
// owns unit l % H of superblocks l / H, + 32/H, ...  The superblocks left over after the
// full passes are handled with the lanes split between the rows when that fills more lanes.
template <int TYPE, int RW>
__device__ __forceinline__ void consume_tile1(uint32_t slot0, uint32_t slot_stride, const uint32_t (&mis)[RW], int kb,
                                              int sb0, const PackA & as, float (&acc)[RW][1]) {
    using U = Unit1<TYPE>;
    constexpr int H = U::H, SPI = 32 / H, SB = Fmt<TYPE>::SB;
    const int lane = threadIdx.x & 31;
    const int bl = lane / H, u = lane % H;
    const int full = kb / SPI, rem = kb - full * SPI;
    for (int it = 0; it < full; it++) {
        const int b = it * SPI + bl;
        typename U::Act a;
        U::load_act(as, sb0 + b, u, a);
#pragma unroll
        for (int r = 0; r < RW; r++) {
            acc[r][0] += U::term(slot0 + r * slot_stride + mis[r] + (uint32_t)(b * SB), u, a);
        }
    }
    if (rem == 0) {
        return;
    }
    const int m = rem * H; // units per row in the tail, < 32
    if (RW > 1 && 2 * m <= 32) {
        const int rpp = min(RW, 32 / m); // rows per pass
        for (int r0 = 0; r0 < RW; r0 += rpp) {
            const int rr = (lane >= m ? 1 : 0) + (lane >= 2 * m ? 1 : 0); // lane / m, or 2 = beyond the pass
            const int item = lane - rr * m, row = r0 + rr;
            const bool valid = rr < rpp && rr < 2 && row < RW;
            float t = 0.f;
            if (valid) {
                const int b = full * SPI + item / H, uu = item % H;
                uint32_t mr = mis[0];
#pragma unroll
                for (int r = 1; r < RW; r++) {
                    mr = row == r ? mis[r] : mr;
                }
                typename U::Act a;
                U::load_act(as, sb0 + b, uu, a);
                t = U::term(slot0 + row * slot_stride + mr + (uint32_t)(b * SB), uu, a);
            }
#pragma unroll
            for (int r = 0; r < RW; r++) {
                acc[r][0] += row == r ? t : 0.f;
            }
        }
    } else if (bl < rem) {
        const int b = full * SPI + bl;
        typename U::Act a;
        U::load_act(as, sb0 + b, u, a);
#pragma unroll
        for (int r = 0; r < RW; r++) {
            acc[r][0] += U::term(slot0 + r * slot_stride + mis[r] + (uint32_t)(b * SB), u, a);
        }
    }
}

// 2..4 tokens: quarter-superblock units whose unpacked weights stay in registers for all tokens
template <int TYPE, int RW, int TT, class AS>
__device__ __forceinline__ void consume_tile(uint32_t slot0, uint32_t slot_stride, const uint32_t (&mis)[RW], int kb,
                                             int sb0, const AS & as, float (&acc)[RW][TT]) {
    const int lane = threadIdx.x & 31;
    const int u = lane & 3;
    for (int b = lane >> 2; b < kb; b += 8) {
#pragma unroll
        for (int r = 0; r < RW; r++) {
            WUnit<TYPE> w;
            w.load(slot0 + r * slot_stride + mis[r] + (uint32_t)(b * Fmt<TYPE>::SB), u);
#pragma unroll
            for (int t = 0; t < TT; t++) {
                typename WUnit<TYPE>::Act a;
                load_act<TYPE>(as, sb0 + b, u, min(t, as.TB - 1), a);
                acc[r][t] += w.term(a);
            }
        }
    }
}
// The rows of a call are split among the G parts (CTAs, or consumer groups) in proportion to
// their bytes: part p owns the flattened cost range [total*p/G, total*(p+1)/G), cost = rows x
// bytes per superblock.  All in 32-bit arithmetic (64-bit division is a long software routine
// every warp would run before its first copy): with total = q*G + r computed by the host,
// total*p/G = q*p + r*p/G exactly.
struct RowRange {
    int lo, hi;
};
struct CostSplit {
    uint32_t q, r; // total / G, total % G
};
inline bool cost_split(const CallDev & c, uint32_t G, CostSplit & cs) { // host; false when the cost overflows 31 bits
    unsigned long long total = 0;
    for (int i = 0; i < c.n_segs; i++) {
        total += (unsigned long long)c.seg[i].n_rows * sb_bytes(c.seg[i].type);
    }
    cs.q = (uint32_t)(total / G);
    cs.r = (uint32_t)(total % G);
    return total < (1ull << 31) && G < 65536;
}
__device__ __forceinline__ uint32_t cost_at(const CostSplit & cs, uint32_t p, uint32_t G) {
    return cs.q * p + (cs.r * p) / G;
}
__device__ __forceinline__ RowRange cta_rows(const CallDev & c, int si, uint32_t lo, uint32_t hi) {
    uint32_t c0 = 0;
    for (int i = 0; i < si; i++) {
        c0 += (uint32_t)c.seg[i].n_rows * (uint32_t)sb_bytes(c.seg[i].type);
    }
    const uint32_t w = (uint32_t)sb_bytes(c.seg[si].type);
    const uint32_t c1 = c0 + (uint32_t)c.seg[si].n_rows * w;
    const uint32_t a = lo > c0 ? lo : c0, b = hi < c1 ? hi : c1;
    RowRange r{0, 0};
    if (a < b) {
        r.lo = (int)((a - c0 + w - 1) / w);
        r.hi = (int)((b - c0 + w - 1) / w);
    }
    return r;
}

} // namespace b200q
