// Streaming GEMV for two to four tokens (one token runs in gemv_pinned.cu).
//
// Data movement.  A tile is the raw GGUF block stream of `rows_per_tile` consecutive weight
// rows x kb superblocks.  It is brought into shared memory by bulk asynchronous copies
// (cp.async.bulk, the 1-D TMA path, no multicast), one per row, that complete on an
// mbarrier; a ring of tiles keeps ~75 KB per CTA in flight so the copy engine, not the
// warps, hides HBM latency.  A copy must start on a 16-byte boundary and be a multiple of 16
// bytes long: a row segment that starts at address A is fetched from A & ~15 and decoded
// from offset A & 15 inside its slot (Q6_K rows are only 2-byte aligned, IQ4_XS 8); the
// bytes read beyond either end lie in the same 16-byte line as valid bytes, so they are
// always mapped.
//
// Roles.  Warp 8 is the producer: lane r issues the copy of row r of the tile.  Warps 0..7
// are consumers: warp w owns rows RW*w .. RW*w+RW-1 of the tile for the whole K loop, so a
// row's partial sums stay in registers and no cross-warp reduction exists.  Four lanes
// cover a superblock (64 weights each, see units.cuh); the unpacked weights of a unit stay in
// registers for all tokens.  Every token's quantized activation is staged once per CTA in
// shared memory as a pack (units.cuh).
//
// Every wait on an mbarrier is bounded by a clock budget; a wait that runs out records an
// error status the host can read (b200q_device_status) and the CTA leaves its loop.

#include "launch.h"
#include "stream_core.cuh"

namespace b200q {

constexpr int kStreamThreads = 32 * (kConsumerWarps + 1);
constexpr int kSmemBudget = 110 * 1024;         // two CTAs per SM

__device__ int g_device_status = 0;

struct SegTile {
    int16_t kb_max;     // superblocks per tile along K
    int16_t contig;     // tiles hold whole rows: one bulk copy per tile, rows packed back to back
    int32_t slot_bytes; // shared bytes reserved per row of a tile (when not contiguous)
};

struct StreamArgs {
    CallDev c;
    SegTile seg_tile[B200Q_MAX_SEGS]; // tile shape per segment (a tile never spans segments)
    int32_t stages;
    int32_t tile_bytes; // shared bytes reserved per tile (the largest segment's)
    CostSplit cost; // the call's cost over the grid, for the row split
};

// Position in the shared-memory ring: slot and the parity of its full barrier.
struct RingPos {
    int stage;
    uint32_t phase;
};

// One consumer warp's share of one segment: rows RW*warp.. of every tile of the CTA's row range.
template <int TYPE, int TT, int RW, class AS>
__device__ __forceinline__ bool consume_segment(const StreamArgs & a, int si, const RowRange rr, uint32_t tiles,
                                                uint32_t bar_full, uint32_t bar_empty, const AS & as, RingPos & pos) {
    constexpr int kRows = kConsumerWarps * RW, SB = Fmt<TYPE>::SB;
    const SegDev & sg = a.c.seg[si];
    const SegTile st = a.seg_tile[si];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = a.c.K >> 8, S = a.stages;
    // bytes between consecutive rows of a tile: rows back to back, or one slot per row segment
    const uint32_t stride = st.contig ? (uint32_t)(nb * SB) : (uint32_t)st.slot_bytes;
    const uint32_t wbase = (uint32_t)(reinterpret_cast<uintptr_t>(sg.w) & 15);
    const uint32_t warp_off = (uint32_t)(warp * RW) * stride;
    for (int tile_row0 = rr.lo; tile_row0 < rr.hi; tile_row0 += kRows) {
        const int row0 = tile_row0 + warp * RW;
        // where a row's bytes start inside its slot: its own misalignment, or in contiguous
        // mode the misalignment of the tile's first row (only the low four address bits matter)
        uint32_t mis0[RW];
#pragma unroll
        for (int r = 0; r < RW; r++) {
            const uint32_t rx = (uint32_t)(st.contig ? tile_row0 : row0 + r);
            mis0[r] = wbase + rx * (uint32_t)(nb * SB);
        }
        float acc[RW][TT];
#pragma unroll
        for (int r = 0; r < RW; r++) {
#pragma unroll
            for (int t = 0; t < TT; t++) {
                acc[r][t] = 0.f;
            }
        }
        for (int sb0 = 0; sb0 < nb; sb0 += st.kb_max) {
            if (!mbar_wait(bar_full + 8 * pos.stage, pos.phase, &g_device_status)) {
                return false;
            }
            if (row0 < rr.hi) { // rows past the range hold stale bytes: their results are dropped
                const int kb = min((int)st.kb_max, nb - sb0);
                const uint32_t slot0 = tiles + (uint32_t)(pos.stage * a.tile_bytes) + warp_off;
                uint32_t mis[RW];
#pragma unroll
                for (int r = 0; r < RW; r++) {
                    mis[r] = (mis0[r] + (uint32_t)(sb0 * SB)) & 15;
                }
                consume_tile<TYPE, RW, TT>(slot0, stride, mis, kb, sb0, as, acc);
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_empty + 8 * pos.stage);
            }
            if (++pos.stage == S) {
                pos.stage = 0;
                pos.phase ^= 1;
            }
        }
#pragma unroll
        for (int r = 0; r < RW; r++) {
#pragma unroll
            for (int t = 0; t < TT; t++) {
                acc[r][t] = warp_sum(acc[r][t]);
            }
        }
        // lane (r*TT + t) stores row r, token t
        float mine = 0.f;
#pragma unroll
        for (int r = 0; r < RW; r++) {
#pragma unroll
            for (int t = 0; t < TT; t++) {
                mine = lane == r * TT + t ? acc[r][t] : mine;
            }
        }
        const int r = lane / TT, t = lane % TT;
        if (lane < RW * TT && row0 + r < rr.hi && t < a.c.TB) {
            const size_t o = (size_t)t * sg.out_stride + row0 + r;
            float v = sg.alpha * mine;
            if (sg.residual) {
                v += sg.residual[o];
            }
            store_out(a.c, &sg.out[o], v);
        }
    }
    return true;
}

template <int TT, int RW>
__global__ void __launch_bounds__(kStreamThreads, 2) gemv_stream_kernel(const __grid_constant__ StreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int kRows = kConsumerWarps * RW; // rows per tile
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t bar_full = base, bar_empty = base + 64, tiles = base + 128;
    const uint32_t pack = tiles + (uint32_t)(a.stages * a.tile_bytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = a.c.K >> 8;
    const int S = a.stages;
    const uint32_t cost_lo = cost_at(a.cost, blockIdx.x, gridDim.x), cost_hi = cost_at(a.cost, blockIdx.x + 1, gridDim.x);

    // Let the next kernel in the stream be scheduled as soon as this grid is resident: its
    // CTAs start on SMs this grid's tail frees, and prefetch weights while it still waits
    // (griddepcontrol.wait) for this grid to complete.
    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer
        int stage = 0;
        uint32_t par = 1; // parity of the empty barrier: a fresh slot is free
        bool alive = true;
        for (int si = 0; si < a.c.n_segs && alive; si++) {
            const SegDev & sg = a.c.seg[si];
            const SegTile st = a.seg_tile[si];
            const RowRange rr = cta_rows(a.c, si, cost_lo, cost_hi);
            const int sbb = sb_bytes(sg.type);
            const size_t row_bytes = (size_t)nb * sbb;
            for (int row0 = rr.lo; row0 < rr.hi && alive; row0 += kRows) {
                const int rows = min(kRows, rr.hi - row0);
                for (int sb0 = 0; sb0 < nb && alive; sb0 += st.kb_max) {
                    const int kb = min((int)st.kb_max, nb - sb0);
                    uint32_t len = 0;
                    const uint8_t * src = nullptr;
                    if (st.contig) {
                        if (lane == 0) { // the tile's rows are one contiguous byte range
                            const uintptr_t A = reinterpret_cast<uintptr_t>(sg.w + (size_t)row0 * row_bytes);
                            const uintptr_t A0 = A & ~uintptr_t(15);
                            len = (uint32_t)(((A + (size_t)rows * row_bytes + 15) & ~uintptr_t(15)) - A0);
                            src = reinterpret_cast<const uint8_t *>(A0);
                        }
                    } else if (lane < rows) {
                        const uint8_t * p = sg.w + (size_t)(row0 + lane) * row_bytes + (size_t)sb0 * sbb;
                        const uintptr_t A = reinterpret_cast<uintptr_t>(p);
                        const uintptr_t A0 = A & ~uintptr_t(15);
                        len = (uint32_t)(((A + (size_t)kb * sbb + 15) & ~uintptr_t(15)) - A0);
                        src = reinterpret_cast<const uint8_t *>(A0);
                    }
                    uint32_t total = len;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        total += __shfl_xor_sync(0xFFFFFFFFu, total, o);
                    }
                    alive = mbar_wait(bar_empty + 8 * stage, par, &g_device_status);
                    alive = __all_sync(0xFFFFFFFFu, alive);
                    if (!alive) {
                        break;
                    }
                    if (lane == 0) {
                        mbar_expect_tx(bar_full + 8 * stage, total);
                    }
                    __syncwarp();
                    if (len) {
                        bulk_g2s(tiles + (uint32_t)(stage * a.tile_bytes + (st.contig ? 0 : lane * st.slot_bytes)), src,
                                 len, bar_full + 8 * stage);
                    }
                    if (++stage == S) {
                        stage = 0;
                        par ^= 1;
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    // The weight copies above do not depend on the activation quantizer; all below does.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    PackT as; // a pack per token in shared memory
    {
        const uint32_t stride = (uint32_t)(nb * kPackSB);
        for (int t = 0; t < a.c.TB; t++) {
            stage_pack_token(pack + (uint32_t)t * stride, a.c, t, nb, threadIdx.x, 32 * kConsumerWarps);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps) : "memory");
        as.pack = pack;
        as.stride = stride;
        as.TB = a.c.TB;
    }

    RingPos pos{0, 0};
    for (int si = 0; si < a.c.n_segs; si++) {
        const RowRange rr = cta_rows(a.c, si, cost_lo, cost_hi);
        bool ok;
        switch (a.c.seg[si].type) { // one decoder per segment: the tile and chunk loops are specialised
        case kQ4_K: ok = consume_segment<kQ4_K, TT, RW>(a, si, rr, tiles, bar_full, bar_empty, as, pos); break;
        case kQ5_K: ok = consume_segment<kQ5_K, TT, RW>(a, si, rr, tiles, bar_full, bar_empty, as, pos); break;
        case kQ6_K: ok = consume_segment<kQ6_K, TT, RW>(a, si, rr, tiles, bar_full, bar_empty, as, pos); break;
        case kIQ4_XS: ok = consume_segment<kIQ4_XS, TT, RW>(a, si, rr, tiles, bar_full, bar_empty, as, pos); break;
        default: ok = consume_segment<kQ8_0, TT, RW>(a, si, rr, tiles, bar_full, bar_empty, as, pos); break;
        }
        if (!ok) {
            return;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------
template <int TT, int RW>
static cudaError_t launch_stream_tt(cudaStream_t s, StreamArgs & a, bool pdl_secondary) {
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(gemv_stream_kernel<TT, RW>), kSmemBudget);
    if (e != cudaSuccess) {
        return e;
    }
    const CallDev & c = a.c;
    constexpr int kRows = kConsumerWarps * RW;
    const int nb = c.K >> 8;
    int groups = 0;
    for (int i = 0; i < c.n_segs; i++) {
        groups += (c.seg[i].n_rows + kRows - 1) / kRows;
    }
    // Superblocks per tile along K, per segment.  Copies are efficient when large (the copy
    // engine spends about as long on a copy's fixed cost as on 750 bytes), so take whole rows
    // - one copy per tile - when two tiles of whole rows fit, else per row the largest run of
    // superblocks that leaves room for two tiles, in multiples of eight.
    const size_t pack_probe = (size_t)TT * nb * kPackSB;
    const size_t room = (kSmemBudget - 128 - pack_probe) / 2; // bytes per tile with two stages
    a.tile_bytes = 0;
    for (int i = 0; i < c.n_segs; i++) {
        const int type = c.seg[i].type, sbb = sb_bytes((uint32_t)type);
        SegTile & st = a.seg_tile[i];
        int kb;
        if ((size_t)kRows * nb * sbb + 48 <= room) {
            kb = nb;
        } else {
            const int fit = (int)((room / kRows - 48) / sbb);
            kb = fit / 8 * 8;
            kb = kb < 8 ? 8 : kb;
            const int n_chunks = (nb + kb - 1) / kb; // equal chunks, rounded up to a multiple of eight
            kb = (((nb + n_chunks - 1) / n_chunks + 7) / 8) * 8;
        }
        st.kb_max = (int16_t)(kb < nb ? kb : nb);
        st.contig = st.kb_max == nb ? 1 : 0;
        st.slot_bytes = ((st.kb_max * sbb + 32 + 15) / 16) * 16;
        const int tile = st.contig ? ((kRows * nb * sbb + 32 + 15) / 16) * 16 : kRows * st.slot_bytes;
        a.tile_bytes = a.tile_bytes > tile ? a.tile_bytes : tile;
    }
    const size_t pack_bytes = (size_t)TT * nb * kPackSB;
    const size_t fixed = 128 + pack_bytes;
    if (fixed + 2 * (size_t)a.tile_bytes > (size_t)kSmemBudget) {
        return cudaErrorInvalidConfiguration;
    }
    int stages = (int)((kSmemBudget - fixed) / (size_t)a.tile_bytes);
    a.stages = stages > 8 ? 8 : stages;
    const size_t smem = 128 + (size_t)a.stages * a.tile_bytes + pack_bytes;
    int grid = 2 * kSMs;
    grid = groups < grid ? groups : grid;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1; // see the note on launch chaining in b200q.h
    (void)pdl_secondary;
    if (!cost_split(c, (uint32_t)grid, a.cost)) {
        return cudaErrorInvalidConfiguration;
    }
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<TT, RW>, a);
}

bool stream_supported(const CallDev & c) {
    // the activation packs (400 B per superblock and token) must leave room for two tiles of
    // at least eight superblocks per row ...
    const int nb = c.K >> 8, tt = c.TB;
    int max_sbb = 0;
    for (int i = 0; i < c.n_segs; i++) {
        max_sbb = max_sbb > sb_bytes(c.seg[i].type) ? max_sbb : sb_bytes(c.seg[i].type);
    }
    const size_t rows = c.TB == 2 ? 2 * kConsumerWarps : kConsumerWarps; // the two-token kernel takes two rows per warp
    const size_t min_tile = rows * (size_t)(((8 * max_sbb + 32 + 15) / 16) * 16);
    CostSplit cs; // ... and the byte-balanced row split works in 32-bit arithmetic
    return c.TB >= 2 && c.TB <= 4 && c.K <= 24576 && (size_t)tt * nb * kPackSB <= 56 * 1024 &&
           128 + (size_t)tt * nb * kPackSB + 2 * min_tile <= (size_t)kSmemBudget && cost_split(c, 2 * kSMs, cs);
}

cudaError_t launch_gemv_stream(cudaStream_t s, const CallDev & c, bool pdl_secondary) {
    StreamArgs a;
    a.c = c;
    if (c.TB == 2) {
        return launch_stream_tt<2, 2>(s, a, pdl_secondary);
    }
    if (c.TB == 3) {
        return launch_stream_tt<3, 1>(s, a, pdl_secondary);
    }
    return launch_stream_tt<4, 1>(s, a, pdl_secondary);
}

cudaError_t read_device_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_device_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    }
    return e;
}

// ---- parity instrument on the streaming kernel's decode path -------------------------------
// One CTA per weight row.  The row is copied into shared memory with the same misalignment
// it has in global memory, the activation pack of token t is built, and every (superblock,
// unit) is decoded and dotted by exactly the WUnit code the streaming kernel runs.
constexpr int kDotsChunk = 16; // superblocks staged at a time
template <int TYPE> __device__ constexpr int dots_per_sb() {
    return TYPE == kQ6_K ? 16 : 8;
}

template <int TYPE>
__device__ __forceinline__ void dots_chunk(uint32_t wbase, uint32_t pack, int sb0, int n, bool single, int32_t * wd) {
    PackA as{pack};
    if (single) { // the units a single-token call runs
        using U = Unit1<TYPE>;
        for (int i = threadIdx.x; i < U::H * n; i += blockDim.x) {
            const int b = i / U::H, u = i % U::H;
            typename U::Act act;
            U::load_act(as, b, u, act);
            // the unit writes at superblock index sb0 + b of the row's array
            U::exact(wbase + (uint32_t)(b * Fmt<TYPE>::SB), b, u, act, wd + dots_per_sb<TYPE>() * sb0);
        }
    } else { // the quarter units a 2..8 token call runs
        for (int i = threadIdx.x; i < 4 * n; i += blockDim.x) {
            const int b = i >> 2, u = i & 3;
            typename WUnit<TYPE>::Act act;
            load_act<TYPE>(as, b, u, 0, act);
            WUnit<TYPE> w;
            w.load(wbase + (uint32_t)(b * Fmt<TYPE>::SB), u);
            unit_exact<TYPE>(w, act, b, u, wd + dots_per_sb<TYPE>() * sb0);
        }
    }
}

__global__ void __launch_bounds__(128) unit_dots_kernel(const uint8_t * w, int type, int K, const int8_t * x8, int TB,
                                                        int t, int32_t * wd) {
    __shared__ __align__(16) uint8_t wbuf[kDotsChunk * 272 + 32];
    __shared__ __align__(16) uint8_t pbuf[kDotsChunk * kPackSB];
    const int nb = K >> 8, sbb = sb_bytes(type);
    const int D = type == kQ6_K ? K / 16 : K / 32;
    const uint8_t * row = w + (size_t)blockIdx.x * nb * sbb;
    int32_t * out = wd + (size_t)blockIdx.x * D;
    const uint32_t wb = smem_u32(wbuf), pk = smem_u32(pbuf);
    for (int sb0 = 0; sb0 < nb; sb0 += kDotsChunk) {
        const int n = min(kDotsChunk, nb - sb0);
        const uint8_t * src = row + (size_t)sb0 * sbb;
        const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15);
        __syncthreads();
        for (int i = threadIdx.x; i < n * sbb / 2; i += blockDim.x) { // blocks are 2-byte aligned
            reinterpret_cast<uint16_t *>(wbuf + mis)[i] = reinterpret_cast<const uint16_t *>(src)[i];
        }
        for (int i = threadIdx.x; i < 8 * n; i += blockDim.x) {
            const size_t gi = (size_t)(8 * sb0 + i) * TB + t;
            const uint4 * gx = reinterpret_cast<const uint4 *>(x8 + gi * 32);
            const uint4 x0 = __ldg(gx), x1 = __ldg(gx + 1);
            const uint32_t p = pack_addr(pk, i);
            sts128(p, x0.x, x0.y, x0.z, x0.w);
            sts128(p + 16, x1.x, x1.y, x1.z, x1.w);
            sts128(p + 32, 0, 0, 0, 0);
        }
        __syncthreads();
        switch (type) {
        case kQ4_K: dots_chunk<kQ4_K>(wb + mis, pk, sb0, n, TB == 1, out); break;
        case kQ5_K: dots_chunk<kQ5_K>(wb + mis, pk, sb0, n, TB == 1, out); break;
        case kQ6_K: dots_chunk<kQ6_K>(wb + mis, pk, sb0, n, TB == 1, out); break;
        case kIQ4_XS: dots_chunk<kIQ4_XS>(wb + mis, pk, sb0, n, TB == 1, out); break;
        default: dots_chunk<kQ8_0>(wb + mis, pk, sb0, n, TB == 1, out); break;
        }
    }
}

cudaError_t launch_unit_dots(cudaStream_t s, const uint8_t * w, int type, int K, int n_rows, const int8_t * x8, int TB,
                             int t, int32_t * wd) {
    unit_dots_kernel<<<(unsigned)n_rows, 128, 0, s>>>(w, type, K, x8, TB, t, wd);
    return cudaGetLastError();
}

} // namespace b200q
