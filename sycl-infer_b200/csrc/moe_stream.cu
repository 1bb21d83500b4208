// Grouped expert GEMV for routed MoE decode, streaming form.
//
// The work of one launch is the flattened list (active expert, row tile) - the number of active
// experts is read on the device, so the launch is graph-replayable - dealt to persistent CTAs in
// contiguous runs.  As in the dense streaming kernel a producer warp moves each tile's raw GGUF
// rows into a shared-memory ring with bulk asynchronous copies (1-D TMA, no multicast) and eight
// consumer warps decode them with dp4a against an activation pack in shared memory.  What is
// particular to MoE:
//   * gate and up rows travel together: a tile is rows r0.. of the expert's gate plane AND of its
//     up plane, warp w owns the pair (gate[r0+w], up[r0+w]), so both meet every activation load
//     and h = silu(g) * u is formed in registers;
//   * the activation pack belongs to an expert's routed tokens, not to the call: it is restaged
//     (up to kMoeTok tokens at a time) whenever the CTA moves to another expert;
//   * the down projection has a short K (the expert's FFN width): lanes then cover
//     (row, unit) pairs - several rows per pass - instead of one row's units.
// Rows must be 16-byte multiples (the copies then need no realignment); other shapes stay on the
// warp-per-row kernel, the prefill regime (many tokens per expert) runs as grouped tensor-core tiles
// (gemm_mma.cu).
#include <cstdlib>
#include <cstring>

#include "launch.h"
#include "stream_core.cuh"

namespace b200q {

constexpr int kMoeThreads = 32 * (kConsumerWarps + 1);
constexpr int kMoeSmem = 110 * 1024; // two CTAs per SM
constexpr int kMoeHdr = 128;
constexpr int kMoeTok = 4; // activation packs staged at a time

__device__ int g_moe_status = 0;

struct MoeStreamArgs {
    const uint8_t *bank_a, *bank_b; // gate and up planes, or the down plane in bank_a
    size_t plane_a, plane_b;
    const int32_t *off, *pair, *active, *n_active;
    const int8_t * x8;
    const float * xmeta;
    const int32_t * xsumq;
    float * out;
    int32_t type_a, type_b;
    int32_t TB, top_k;      // tokens (gate|up: token of pair p is p / top_k) or pairs (down: top_k = 0)
    int32_t nb, n_rows;     // superblocks per row, rows per expert plane
    int32_t out_stride;
    int32_t row_bytes_a, row_bytes_b;
    int32_t rows_per_tile, tiles_per_expert;
    int32_t half_bytes;     // shared bytes of one plane's part of a tile
    int32_t tile_bytes, stages;
    int32_t max_active;     // bound on the active experts (sizes the shared prefix array)
    int32_t units_per_row;  // down, short K: lanes cover (row, unit); 0 = two rows per warp over all of K
};

// Pack of token `tok` of a TB-token activation (group-major views) for superblocks [0, nb).
__device__ __forceinline__ void stage_pack_tok(uint32_t pack, const MoeStreamArgs & a, int tok, int tid, int nthr) {
    for (int g = tid; g < 8 * a.nb; g += nthr) {
        const size_t gi = (size_t)g * a.TB + tok;
        const uint4 * gx = reinterpret_cast<const uint4 *>(a.x8 + gi * 32);
        const uint4 x0 = __ldg(gx), x1 = __ldg(gx + 1);
        const float sx = __ldg(a.xmeta + 2 * gi);
        const int2 xs = __ldg(reinterpret_cast<const int2 *>(a.xsumq) + gi);
        const uint32_t p = pack_addr(pack, g);
        sts128(p, x0.x, x0.y, x0.z, x0.w);
        sts128(p + 16, x1.x, x1.y, x1.z, x1.w);
        sts128(p + 32, __float_as_uint(sx), (uint32_t)xs.x, (uint32_t)xs.y, __float_as_uint(sx * (float)(xs.x + xs.y)));
    }
}

__device__ __forceinline__ float moe_silu(float g) { // x / (1 + expf(-x)); expf is within an ulp of the host's
    return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
}

// one row over all of K against the pack (any type)
__device__ __forceinline__ float row_dot(int type, uint32_t row_addr, int nb, const PackA & as) {
    float acc[1][1] = {{0.f}};
    const uint32_t mis[1] = {0};
    switch (type) {
    case kQ4_K: consume_tile1<kQ4_K, 1>(row_addr, 0, mis, nb, 0, as, acc); break;
    case kQ5_K: consume_tile1<kQ5_K, 1>(row_addr, 0, mis, nb, 0, as, acc); break;
    case kQ6_K: consume_tile1<kQ6_K, 1>(row_addr, 0, mis, nb, 0, as, acc); break;
    case kIQ4_XS: consume_tile1<kIQ4_XS, 1>(row_addr, 0, mis, nb, 0, as, acc); break;
    default: consume_tile1<kQ8_0, 1>(row_addr, 0, mis, nb, 0, as, acc); break;
    }
    return acc[0][0];
}
// two rows `stride` bytes apart sharing every activation load (same type)
__device__ __forceinline__ void row_dot2(int type, uint32_t row_addr, uint32_t stride, int nb, const PackA & as, float & r0,
                                         float & r1) {
    float acc[2][1] = {{0.f}, {0.f}};
    const uint32_t mis[2] = {0, 0};
    switch (type) {
    case kQ4_K: consume_tile1<kQ4_K, 2>(row_addr, stride, mis, nb, 0, as, acc); break;
    case kQ5_K: consume_tile1<kQ5_K, 2>(row_addr, stride, mis, nb, 0, as, acc); break;
    case kQ6_K: consume_tile1<kQ6_K, 2>(row_addr, stride, mis, nb, 0, as, acc); break;
    case kIQ4_XS: consume_tile1<kIQ4_XS, 2>(row_addr, stride, mis, nb, 0, as, acc); break;
    default: consume_tile1<kQ8_0, 2>(row_addr, stride, mis, nb, 0, as, acc); break;
    }
    r0 = acc[0][0];
    r1 = acc[1][0];
}
// short K: this lane's unit of its row
template <int TYPE> __device__ __forceinline__ float unit_term(uint32_t row_addr, int u, const PackA & as) {
    using U = Unit1<TYPE>;
    typename U::Act act;
    U::load_act(as, u / U::H, u % U::H, act);
    return U::term(row_addr + (uint32_t)((u / U::H) * Fmt<TYPE>::SB), u % U::H, act);
}
__device__ __forceinline__ float unit_term_any(int type, uint32_t row_addr, int u, const PackA & as) {
    switch (type) {
    case kQ4_K: return unit_term<kQ4_K>(row_addr, u, as);
    case kQ5_K: return unit_term<kQ5_K>(row_addr, u, as);
    case kQ6_K: return unit_term<kQ6_K>(row_addr, u, as);
    case kIQ4_XS: return unit_term<kIQ4_XS>(row_addr, u, as);
    default: return unit_term<kQ8_0>(row_addr, u, as);
    }
}

template <int FUSE>
__global__ void __launch_bounds__(kMoeThreads, 2) moe_stream_kernel(const __grid_constant__ MoeStreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t bar_full = base, bar_empty = base + 64, tiles = base + kMoeHdr;
    const uint32_t packs = tiles + (uint32_t)(a.stages * a.tile_bytes);
    const uint32_t pack_bytes = (uint32_t)(a.nb * kPackSB);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = a.stages;
    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // the expert lists come from the CSR kernel, the activation from the quantizer
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Work split.  A tile costs as many decode passes as its expert has routed tokens, so the
    // CTAs take equal shares of cost = sum over tiles of (pairs of the tile's expert), not of tiles.
    // pre[s] = pairs of active experts 0..s-1 (built by every CTA; a few hundred entries).
    const int n_act = min(*a.n_active, a.max_active);
    int32_t * pre = reinterpret_cast<int32_t *>(smem_raw + (packs - base) + kMoeTok * pack_bytes);
    if (warp == 0) {
        int carry = 0;
        for (int s0 = 0; s0 < n_act; s0 += 32) {
            const int sl = s0 + lane;
            int v = 0;
            if (sl < n_act) {
                const int e = a.active[sl];
                v = a.off[e + 1] - a.off[e];
            }
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xFFFFFFFFu, v, o);
                if (lane >= o) {
                    v += u;
                }
            }
            if (sl < n_act) {
                pre[sl + 1] = carry + v;
            }
            carry += __shfl_sync(0xFFFFFFFFu, v, 31);
        }
        if (lane == 0) {
            pre[0] = 0;
        }
    }
    __syncthreads();
    const int tpe = a.tiles_per_expert;
    const unsigned long long C = (unsigned long long)pre[n_act] * tpe;
    const uint32_t c_lo = (uint32_t)(C * blockIdx.x / gridDim.x), c_hi = (uint32_t)(C * (blockIdx.x + 1) / gridDim.x);
    // first tile whose starting cost is >= c_lo: expert slot by bisection, tile by division
    int slot0 = 0, tile0 = 0;
    {
        int lo = 0, hi = n_act; // largest s with pre[s] * tpe <= c_lo
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((uint32_t)pre[mid] * (uint32_t)tpe <= c_lo) {
                lo = mid;
            } else {
                hi = mid;
            }
        }
        slot0 = lo;
        if (n_act > 0) {
            const uint32_t cnt = (uint32_t)(pre[lo + 1] - pre[lo]), rel = c_lo - (uint32_t)pre[lo] * (uint32_t)tpe;
            tile0 = (int)((rel + cnt - 1) / cnt);
            if (tile0 >= tpe) {
                slot0++;
                tile0 = 0;
            }
        }
    }
    // walks the CTA's tiles: (slot, j) with starting cost c, until c >= c_hi
    struct Walk {
        int slot, j;
        uint32_t c;
    };
    auto walk_begin = [&]() {
        Walk w{slot0, tile0, 0};
        if (slot0 < n_act) {
            w.c = (uint32_t)pre[slot0] * (uint32_t)tpe + (uint32_t)tile0 * (uint32_t)(pre[slot0 + 1] - pre[slot0]);
        }
        return w;
    };
    auto walk_valid = [&](const Walk & w) { return w.slot < n_act && w.c < c_hi; };
    auto walk_next = [&](Walk & w) {
        w.c += (uint32_t)(pre[w.slot + 1] - pre[w.slot]);
        if (++w.j == tpe) {
            w.j = 0;
            w.slot++;
        }
    };
    int stage = 0;
    uint32_t phase = 0;

    if (warp == kConsumerWarps) { // ------------------------------------------------------ producer
        for (Walk w = walk_begin(); walk_valid(w); walk_next(w)) {
            const int slot = w.slot, j = w.j;
            const int e = a.active[slot];
            const int r0 = j * a.rows_per_tile, rows = min(a.rows_per_tile, a.n_rows - r0);
            bool alive = mbar_wait(bar_empty + 8 * stage, phase ^ 1, &g_moe_status);
            alive = __all_sync(0xFFFFFFFFu, alive);
            if (!alive) {
                return;
            }
            if (lane == 0) {
                const uint32_t ba = (uint32_t)(rows * a.row_bytes_a), bb = FUSE ? (uint32_t)(rows * a.row_bytes_b) : 0u;
                const uint32_t dst = tiles + (uint32_t)(stage * a.tile_bytes);
                mbar_expect_tx(bar_full + 8 * stage, ba + bb);
                bulk_g2s(dst, a.bank_a + (size_t)e * a.plane_a + (size_t)r0 * a.row_bytes_a, ba, bar_full + 8 * stage);
                if (FUSE) {
                    bulk_g2s(dst + (uint32_t)a.half_bytes, a.bank_b + (size_t)e * a.plane_b + (size_t)r0 * a.row_bytes_b, bb,
                             bar_full + 8 * stage);
                }
            }
            __syncwarp();
            if (++stage == S) {
                stage = 0;
                phase ^= 1;
            }
        }
        return;
    }

    // ---------------------------------------------------------------------------------- consumers
    int staged_e = -1, staged_q = -1;
    for (Walk w = walk_begin(); walk_valid(w); walk_next(w)) {
        const int slot = w.slot, j = w.j;
        const int e = a.active[slot];
        const int r0 = j * a.rows_per_tile, rows = min(a.rows_per_tile, a.n_rows - r0);
        const int p0 = a.off[e], p1 = a.off[e + 1];
        if (!mbar_wait(bar_full + 8 * stage, phase, &g_moe_status)) {
            return;
        }
        const uint32_t tile = tiles + (uint32_t)(stage * a.tile_bytes);
        for (int q0 = p0; q0 < p1; q0 += kMoeTok) {
            const int nq = min(kMoeTok, p1 - q0);
            if (staged_e != e || staged_q != q0) { // uniform over the CTA: all warps walk the same tiles
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps) : "memory"); // the old packs are no longer read
                for (int i = 0; i < nq; i++) {
                    const int pr = a.pair[q0 + i];
                    stage_pack_tok(packs + (uint32_t)i * pack_bytes, a, FUSE ? pr / a.top_k : pr, threadIdx.x,
                                   32 * kConsumerWarps);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps) : "memory");
                staged_e = e;
                staged_q = q0;
            }
            for (int i = 0; i < nq; i++) {
                PackA as;
                as.pack = packs + (uint32_t)i * pack_bytes;
                const size_t orow = (size_t)a.pair[q0 + i] * a.out_stride;
                if (FUSE) {
                    float hv = 0.f; // lane k keeps the k-th result of this warp: one parallel silu at the end
                    int n = 0;
                    for (int r = warp; r < rows; r += kConsumerWarps, n++) { // gate row r0+r and up row r0+r
                        float g, u;
                        if (a.type_a == a.type_b) {
                            row_dot2(a.type_a, tile + (uint32_t)(r * a.row_bytes_a), (uint32_t)a.half_bytes, a.nb, as, g, u);
                        } else {
                            g = row_dot(a.type_a, tile + (uint32_t)(r * a.row_bytes_a), a.nb, as);
                            u = row_dot(a.type_b, tile + (uint32_t)(a.half_bytes + r * a.row_bytes_b), a.nb, as);
                        }
                        g = warp_sum(g);
                        u = warp_sum(u);
                        // lanes n (gate) and 16 + n (up) take the sums
                        hv = lane == n ? g : (lane == 16 + n ? u : hv);
                    }
                    const float uu = __shfl_down_sync(0xFFFFFFFFu, hv, 16);
                    if (lane < n) {
                        a.out[orow + r0 + warp + lane * kConsumerWarps] = __fmul_rn(moe_silu(hv), uu);
                    }
                } else if (a.units_per_row > 0) { // short K: lane = (row, unit), several rows per pass
                    const int U = a.units_per_row, rp = 32 / U;
                    const int jr = lane / U, u = lane - jr * U;
                    for (int rb = warp * rp; rb < rows; rb += kConsumerWarps * rp) {
                        const int r = rb + jr;
                        float v = r < rows ? unit_term_any(a.type_a, tile + (uint32_t)(r * a.row_bytes_a), u, as) : 0.f;
                        for (int o = U >> 1; o > 0; o >>= 1) { // the U lanes of a row
                            v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                        }
                        if (u == 0 && r < rows) {
                            a.out[orow + r0 + r] = v;
                        }
                    }
                } else { // two rows per warp over all of K
                    const int r = 2 * warp;
                    if (r < rows) {
                        float v0, v1;
                        row_dot2(a.type_a, tile + (uint32_t)(r * a.row_bytes_a), (uint32_t)a.row_bytes_a, a.nb, as, v0, v1);
                        v0 = warp_sum(v0);
                        v1 = warp_sum(v1);
                        if (lane == 0) {
                            a.out[orow + r0 + r] = v0;
                            if (r + 1 < rows) {
                                a.out[orow + r0 + r + 1] = v1;
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(bar_empty + 8 * stage);
        }
        if (++stage == S) {
            stage = 0;
            phase ^= 1;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------
bool moe_stream_supported(int type_a, int type_b, int K, int n_rows, int fuse_silu) {
#ifdef B200Q_TUNING
    static const bool off = [] {
        const char * e = getenv("B200Q_MOE_KERNEL");
        return e && strcmp(e, "rows") == 0;
    }();
#else
    const bool off = false;
#endif
    const int nb = K >> 8;
    const int ra = nb * sb_bytes((uint32_t)type_a), rb = nb * sb_bytes((uint32_t)type_b);
    if (off || (ra & 15) || (fuse_silu && (rb & 15)) || n_rows < 1) {
        return false;
    }
    // two stages of at least eight row pairs (gate|up) / sixteen rows, plus kMoeTok packs, must fit
    const size_t packs = (size_t)kMoeTok * nb * kPackSB + 4096; // + the cost prefix of up to 1023 active experts
    const size_t tile = fuse_silu ? (size_t)8 * (ra + rb) + 64 : (size_t)16 * ra + 32;
    return kMoeHdr + packs + 2 * tile <= (size_t)kMoeSmem;
}

cudaError_t launch_moe_stream(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                              size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                              const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                              const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                              float * out, int out_stride, int fuse_silu) {
    MoeStreamArgs a;
    a.max_active = n_act_max;
    a.bank_a = static_cast<const uint8_t *>(bank_a);
    a.bank_b = static_cast<const uint8_t *>(bank_b);
    a.plane_a = plane_a;
    a.plane_b = plane_b;
    a.off = off;
    a.pair = pair;
    a.active = active;
    a.n_active = n_active;
    a.x8 = x8;
    a.xmeta = xmeta;
    a.xsumq = xsumq;
    a.out = out;
    a.type_a = type_a;
    a.type_b = type_b;
    a.TB = TB;
    a.top_k = top_k;
    a.nb = K >> 8;
    a.n_rows = n_rows;
    a.out_stride = out_stride;
    a.row_bytes_a = a.nb * sb_bytes((uint32_t)type_a);
    a.row_bytes_b = fuse_silu ? a.nb * sb_bytes((uint32_t)type_b) : 0;
    a.units_per_row = 0;
    if (fuse_silu) {
        // (gate, up) row pairs per tile: two per warp when two such tiles fit, to spread a tile's fixed cost
        const size_t packs_b = (size_t)kMoeTok * a.nb * kPackSB + 4096;
        const size_t pair16 = (size_t)2 * (2 * kConsumerWarps * (a.row_bytes_a > a.row_bytes_b ? a.row_bytes_a : a.row_bytes_b) + 32);
        a.rows_per_tile = (kMoeHdr + packs_b + 2 * pair16 <= (size_t)kMoeSmem && n_rows >= 2 * kConsumerWarps) ? 2 * kConsumerWarps
                                                                                                       : kConsumerWarps;
        const int big = a.row_bytes_a > a.row_bytes_b ? a.row_bytes_a : a.row_bytes_b;
        a.half_bytes = ((a.rows_per_tile * big + 15) / 16) * 16 + 16;
        a.tile_bytes = 2 * a.half_bytes;
    } else {
        const bool half_units = type_a == kQ4_K || type_a == kQ5_K || type_a == kQ6_K;
        const int U = a.nb * (half_units ? 2 : 4);
        if (U <= 32 && (U & (U - 1)) == 0) {
            a.units_per_row = U;
            a.rows_per_tile = kConsumerWarps * (32 / U);
            // short rows make small tiles: take several passes per tile while the copy stays below 32 KB
            while (a.rows_per_tile * 2 * a.row_bytes_a <= 44 * 1024 && a.rows_per_tile * 2 <= n_rows) {
                a.rows_per_tile *= 2;
            }
        } else {
            a.rows_per_tile = 2 * kConsumerWarps;
        }
        a.half_bytes = ((a.rows_per_tile * a.row_bytes_a + 15) / 16) * 16 + 16;
        a.tile_bytes = a.half_bytes;
    }
    a.tiles_per_expert = (n_rows + a.rows_per_tile - 1) / a.rows_per_tile;
    const size_t packs = (size_t)kMoeTok * a.nb * kPackSB + ((size_t)(n_act_max + 1) * 4 + 15) / 16 * 16; // + the cost prefix
    int stages = (int)((kMoeSmem - kMoeHdr - packs) / (size_t)a.tile_bytes);
    if (stages < 2) {
        return cudaErrorInvalidConfiguration;
    }
    a.stages = stages > 8 ? 8 : stages;
    const size_t smem = kMoeHdr + (size_t)a.stages * a.tile_bytes + packs;
    {
        const void * fn = fuse_silu ? reinterpret_cast<const void *>(moe_stream_kernel<1>)
                                    : reinterpret_cast<const void *>(moe_stream_kernel<0>);
        cudaError_t e = ensure_dynamic_smem(fn, kMoeSmem);
        if (e != cudaSuccess) {
            return e;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * kSMs));
    cfg.blockDim = dim3(kMoeThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return fuse_silu ? cudaLaunchKernelEx(&cfg, moe_stream_kernel<1>, a) : cudaLaunchKernelEx(&cfg, moe_stream_kernel<0>, a);
}

cudaError_t read_moe_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_moe_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_moe_status, &zero, sizeof(int));
    }
    return e;
}

} // namespace b200q
