// Grouped expert GEMV for routed MoE decode on the pinned-activation machinery of gemv_pinned.cu
// (this file is part of that translation unit).
//
// A routed pair p = (token t, its j-th expert e) is a small GEMV of its own: the rows of e's
// plane(s) against ONE activation vector (gate|up: token t's; down: pair p's intermediate).  That
// is the shape the single-token kernel is built for - every consumer thread keeps one 128-value
// unit of the activation in registers and meets one unit of one row per step - so the launch
// treats the call as n_pairs such GEMVs in CSR order (pairs of one expert next to each other: the
// second token of an expert finds the planes in L2) and cuts the flattened list (pair, row unit)
// into 148 equal, contiguous shares, one per CTA.  A CTA's share touches a few pairs; their
// activations are staged once, at the start, and a thread re-pins its registers when the share
// moves on to the next pair.
//
// gate|up: a step is H gate rows and the H up rows of the same indices (two bulk copies), the
// epilogue warp forms h = silu(gate) * up and stores it.  On request it also quantizes every
// finished 32-value group of h on the spot (shares are then made of whole 32-row units and H is a
// power of two); measured, that costs the launch more (3.9 us at 128 pairs) than the quantizer
// launch it replaces (1.8 us), so callers that can afford the launch do not ask for it.
// down: a step is R rows of the expert's down plane.
//
// Bulk copies are 1-D (cp.async.bulk, no multicast); all waits are bounded and report through
// the status word of this translation unit.
#pragma once

namespace b200q {

constexpr int kMoePinSegs = 8;    // (pair, row range) pieces a CTA's share may consist of
constexpr int kMoePinPairs = 2048; // CSR positions whose expert is tabulated in shared memory

struct MoePinArgs {
    PinArgs p; // thread and ring geometry (W, R, U, seg, P, Ppad, H, half_off, paired, stages, ...), p.c.K
    const uint8_t *bank_a, *bank_b; // gate and up planes, or the down plane in bank_a
    size_t plane_a, plane_b;
    const int32_t *off, *pair, *active, *n_active;
    const int8_t * x8; // activation views of TB vectors, group-major
    const float * xmeta;
    const int32_t * xsumq;
    float * out;
    NextAct hq; // gate|up: h quantized as b200q_xq(h, TB = n_pairs) would (x8 == nullptr: off)
    int32_t type, TB, top_k, n_rows, n_pairs, max_active, out_stride;
    int32_t row_bytes;
    int32_t unit_rows, upi; // rows (pairs of rows) per unit of the split, units per routed pair
    int32_t off_packs, pack_bytes, off_expert;
};

__device__ __forceinline__ float moe_pin_silu(float g) { // x / (1 + expf(-x)), as the streaming MoE kernel
    return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
}

// A CTA's share [u_lo, u_hi) of the units, walked as pieces (CSR position i, rows [lo, hi)).
struct MoeWalk {
    uint32_t u, u_hi;
    int i, lo, hi;
};
__device__ __forceinline__ MoeWalk moe_walk_begin(const MoePinArgs & a) {
    const unsigned long long T = (unsigned long long)a.n_pairs * (unsigned)a.upi;
    MoeWalk w;
    w.u = (uint32_t)(T * blockIdx.x / gridDim.x);
    w.u_hi = (uint32_t)(T * (blockIdx.x + 1) / gridDim.x);
    w.i = 0, w.lo = 0, w.hi = 0;
    return w;
}
__device__ __forceinline__ bool moe_walk_next(const MoePinArgs & a, MoeWalk & w) {
    if (w.u >= w.u_hi) {
        return false;
    }
    const uint32_t upi = (uint32_t)a.upi;
    const uint32_t i = w.u / upi, k0 = w.u - i * upi;
    const uint32_t k1 = min(upi, k0 + (w.u_hi - w.u));
    w.i = (int)i;
    w.lo = (int)k0 * a.unit_rows;
    w.hi = min(a.n_rows, (int)k1 * a.unit_rows);
    w.u += k1 - k0;
    return true;
}

// Pack (the pinned kernel's layout) of vector `vec` of the TB-vector activation views.
__device__ __forceinline__ void moe_pin_stage(uint32_t pack, const MoePinArgs & a, int vec, int tid, int nthr) {
    const int G = a.p.c.K >> 5;
    for (int g = tid; g < G; g += nthr) {
        const size_t gi = (size_t)g * a.TB + vec;
        const uint4 * gx = reinterpret_cast<const uint4 *>(a.x8 + gi * 32);
        const uint4 x0 = __ldcg(gx), x1 = __ldcg(gx + 1);
        const float sx = __ldcg(a.xmeta + 2 * gi);
        const int2 xs = __ldcg(reinterpret_cast<const int2 *>(a.xsumq) + gi);
        const uint32_t p = pin_pack_addr(pack, g);
        sts128(p, x0.x, x0.y, x0.z, x0.w);
        sts128(p + 16, x1.x, x1.y, x1.z, x1.w);
        sts128(p + 32, __float_as_uint(sx), (uint32_t)xs.x, (uint32_t)xs.y, __float_as_uint(sx * (float)(xs.x + xs.y)));
    }
}

template <int TYPE>
__device__ __forceinline__ bool moe_pin_piece(const MoePinArgs & a, const uint8_t * w0, const uint8_t * w1, int lo, int hi,
                                              uint32_t tiles, uint32_t red, const PinBars & bars, uint32_t pack, int slot,
                                              int unit, PinRing & pos) {
    ActPin pin;
    pin_from_pack<TYPE>(pack, unit, pin);
    return pin_consume_rows<TYPE>(a.p, a.p, w0, w1, lo, hi, tiles, red, bars, pin, slot, unit, pos);
}

__global__ void __launch_bounds__(kPinThreads, 1) moe_pinned_kernel(const __grid_constant__ MoePinArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const PinBars bars{base, base + 64, base + 128, base + 160};
    const uint32_t started = base + 192;
    const uint32_t red = base + kPinHdr, tiles = base + (uint32_t)a.p.off_tiles;
    const uint32_t packs = base + (uint32_t)a.off_packs;
    int32_t * expert_of = reinterpret_cast<int32_t *>(smem_raw + a.off_expert);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = a.p.W, S = a.p.stages, H = a.p.H, R = a.p.R;

    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        pin_init_barriers(bars, base, S, W);
    }
    // the expert lists come from the router, the activation from the quantizer or from gate|up
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        // expert of every CSR position; a position no active expert claims (a pair whose id was not
        // a valid expert: the CSR builder leaves it out) stays -1 and every role skips it
        for (int q = threadIdx.x; q < a.n_pairs; q += blockDim.x) {
            expert_of[q] = -1;
        }
        __syncthreads();
        const int n_act = min(*a.n_active, a.max_active);
        for (int s = threadIdx.x; s < n_act; s += blockDim.x) {
            const int e = a.active[s];
            const int q1 = min(a.off[e + 1], a.n_pairs);
            for (int q = max(a.off[e], 0); q < q1; q++) {
                expert_of[q] = e;
            }
        }
    }
    __syncthreads();

    if (warp == W) {
        // ---------------------------------------------------------------- producer (one thread)
        if (lane != 0) {
            return;
        }
        PinProd pr{0, 1, 0};
        const int step_rows = a.p.paired ? H : R;
        MoeWalk w = moe_walk_begin(a);
        while (moe_walk_next(a, w)) {
            const int e = expert_of[w.i];
            if (e < 0) {
                continue;
            }
            const uint8_t * wa = a.bank_a + (size_t)e * a.plane_a;
            const uint8_t * wb = a.p.paired ? a.bank_b + (size_t)e * a.plane_b : wa;
            for (int r0 = w.lo; r0 < w.hi; r0 += step_rows) {
                const int rows = min(step_rows, w.hi - r0);
                if (!mbar_wait_gated(bars.empty + 8 * pr.stage, pr.par, &g_pin_status, started)) {
                    pin_produce_drain(bars, S, pr);
                    return;
                }
                const uint32_t dst = tiles + (uint32_t)(pr.stage * a.p.stage_bytes);
                const uintptr_t A = reinterpret_cast<uintptr_t>(wa + (size_t)r0 * a.row_bytes);
                const uintptr_t A0 = A & ~uintptr_t(15);
                const uint32_t len = (uint32_t)(((A + (size_t)rows * a.row_bytes + 15) & ~uintptr_t(15)) - A0);
                if (a.p.paired) {
                    const uintptr_t B = reinterpret_cast<uintptr_t>(wb + (size_t)r0 * a.row_bytes);
                    const uintptr_t B0 = B & ~uintptr_t(15);
                    const uint32_t lenb = (uint32_t)(((B + (size_t)rows * a.row_bytes + 15) & ~uintptr_t(15)) - B0);
                    mbar_expect_tx(bars.full + 8 * pr.stage, len + lenb);
                    bulk_g2s(dst, reinterpret_cast<const void *>(A0), len, bars.full + 8 * pr.stage);
                    bulk_g2s(dst + (uint32_t)a.p.half_off, reinterpret_cast<const void *>(B0), lenb, bars.full + 8 * pr.stage);
                } else {
                    mbar_expect_tx(bars.full + 8 * pr.stage, len);
                    bulk_g2s(dst, reinterpret_cast<const void *>(A0), len, bars.full + 8 * pr.stage);
                }
                pr.issued++;
                if (++pr.stage == S) {
                    pr.stage = 0;
                    pr.par ^= 1;
                }
            }
        }
        return;
    }

    if (warp == W + 1) {
        // ---------------------------------------------------------------- epilogue warp
        int rb = 0;
        uint32_t rphase = 0;
        const int P = a.p.P, Ppad = a.p.Ppad;
        const uint32_t ring = red + (uint32_t)(kRedBufs * a.p.red_bytes); // 32 values of h behind the partials
        const int step_rows = a.p.paired ? H : R;
        MoeWalk w = moe_walk_begin(a);
        while (moe_walk_next(a, w)) {
            if (expert_of[w.i] < 0) {
                continue;
            }
            const int pr = a.pair[w.i];
            float * orow = a.out + (size_t)pr * a.out_stride;
            for (int r0 = w.lo; r0 < w.hi; r0 += step_rows) {
                const int rows = min(step_rows, w.hi - r0);
                if (!mbar_wait(bars.red_full + 8 * rb, rphase, &g_pin_status)) {
                    return;
                }
                const uint32_t rbuf = red + (uint32_t)(rb * a.p.red_bytes);
                if (a.p.paired) { // lane = pair of rows (H <= 32)
                    if (lane < rows) {
                        const uint32_t pg = rbuf + (uint32_t)(lane * Ppad) * 4u, pu = rbuf + (uint32_t)((H + lane) * Ppad) * 4u;
                        float g = 0.f, u = 0.f;
                        for (int j = 0; j < P; j++) {
                            g += __uint_as_float(lds32(pg + 4u * (uint32_t)j));
                            u += __uint_as_float(lds32(pu + 4u * (uint32_t)j));
                        }
                        const float hv = __fmul_rn(moe_pin_silu(g), u);
                        orow[r0 + lane] = hv;
                        sts32(ring + (uint32_t)((r0 + lane) & 31) * 4u, __float_as_uint(hv));
                    }
                } else {
                    for (int c0 = 0; c0 < rows; c0 += 32) { // lane = row slot; partials added in a fixed order
                        if (c0 + lane < rows) {
                            const uint32_t p = rbuf + (uint32_t)((c0 + lane) * Ppad) * 4u;
                            float sum = 0.f;
                            for (int j = 0; j < P; j++) {
                                sum += __uint_as_float(lds32(p + 4u * (uint32_t)j));
                            }
                            orow[r0 + c0 + lane] = sum;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bars.red_empty + 8 * rb);
                }
                if (++rb == kRedBufs) {
                    rb = 0;
                    rphase ^= 1;
                }
                if (a.hq.x8 && ((r0 + rows) & 31) == 0) { // a 32-value group of h is complete (H divides 32)
                    const int g = ((r0 + rows) >> 5) - 1;
                    const float v = __uint_as_float(lds32(ring + (uint32_t)lane * 4u));
                    float scale;
                    int s0, s1;
                    const int q = xq_group(v, lane, scale, s0, s1);
                    const size_t gi = (size_t)g * a.n_pairs + pr;
                    a.hq.x8[gi * 32 + lane] = (int8_t)q;
                    if (lane == 0) {
                        a.hq.xmeta[2 * gi] = scale;
                        a.hq.xmeta[2 * gi + 1] = 0.0f;
                        a.hq.xsumq[2 * gi] = s0;
                        a.hq.xsumq[2 * gi + 1] = s1;
                    }
                    __syncwarp();
                }
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    {
        // the activation of every pair this share touches, staged once
        MoeWalk w = moe_walk_begin(a);
        int s = 0, last = -1;
        while (moe_walk_next(a, w)) {
            if (expert_of[w.i] < 0) {
                continue;
            }
            if (w.i != last && s < kMoePinSegs) {
                const int pr = a.pair[w.i];
                moe_pin_stage(packs + (uint32_t)(s * a.pack_bytes), a, a.top_k > 0 ? pr / a.top_k : pr, (int)threadIdx.x, 32 * W);
                last = w.i;
                s++;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(32 * W) : "memory");
        if (threadIdx.x == 0) {
            asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(started), "r"(1u) : "memory");
        }
    }
    const int U = a.p.U;
    const int slot = (int)threadIdx.x / U, unit = (int)threadIdx.x - slot * U;
    PinRing pos{0, 0, 0, 0};
    MoeWalk w = moe_walk_begin(a);
    int s = -1, last = -1;
    while (moe_walk_next(a, w)) {
        if (expert_of[w.i] < 0) {
            continue;
        }
        if (w.i != last) {
            last = w.i;
            s++;
        }
        if (s >= kMoePinSegs) { // the host sizes shares so that this cannot happen
            atomicExch(&g_pin_status, B200Q_EINVAL);
            return;
        }
        const int e = expert_of[w.i];
        const uint8_t * wa = a.bank_a + (size_t)e * a.plane_a;
        const uint8_t * wb = a.p.paired ? a.bank_b + (size_t)e * a.plane_b : wa;
        const uint32_t pack = packs + (uint32_t)(s * a.pack_bytes);
        bool ok;
        switch (a.type) {
        case kQ4_K: ok = moe_pin_piece<kQ4_K>(a, wa, wb, w.lo, w.hi, tiles, red, bars, pack, slot, unit, pos); break;
        case kQ5_K: ok = moe_pin_piece<kQ5_K>(a, wa, wb, w.lo, w.hi, tiles, red, bars, pack, slot, unit, pos); break;
        case kQ6_K: ok = moe_pin_piece<kQ6_K>(a, wa, wb, w.lo, w.hi, tiles, red, bars, pack, slot, unit, pos); break;
        case kIQ4_XS: ok = moe_pin_piece<kIQ4_XS>(a, wa, wb, w.lo, w.hi, tiles, red, bars, pack, slot, unit, pos); break;
        default: ok = moe_pin_piece<kQ8_0>(a, wa, wb, w.lo, w.hi, tiles, red, bars, pack, slot, unit, pos); break;
        }
        if (!ok) {
            return;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------
static bool moe_pin_plan(int type_a, int type_b, int K, int n_rows, int fuse, long long n_pairs, bool want_hq,
                         MoePinArgs & a) {
    memset(&a, 0, sizeof(a));
    if ((K & 255) || n_rows < 1 || n_pairs < 1 || n_pairs > kMoePinPairs || (fuse && type_a != type_b)) {
        return false;
    }
    const int nb = K >> 8, U = K >> 7;
    const int row_bytes = nb * sb_bytes((uint32_t)type_a);
    if ((row_bytes & 15) || U > 32 * kPinMaxW) {
        return false;
    }
    int R, W;
    if (fuse && want_hq) {
        // H = R / 2 pairs per step, a power of two up to 32: a 32-row group of h is a whole number of steps
        if (n_rows & 31) {
            return false;
        }
        R = 64;
        while (R > 2 && R * U > 32 * kPinMaxW) {
            R >>= 1;
        }
        if (R * U > 32 * kPinMaxW) {
            return false;
        }
    } else {
        R = 32 * kPinMaxW / U;
        R = fuse ? (R > 64 ? 64 : R) & ~1 : (R > 256 ? 256 : R); // gate|up: at most 32 pairs per step (lane = pair)
        if (R < (fuse ? 2 : 1)) {
            return false;
        }
    }
    int seg = 1;
    while (seg < 32 && U % (2 * seg) == 0) {
        seg *= 2;
    }
    PinArgs & p = a.p;
    size_t off_tiles = 0;
    for (;; R = (fuse && want_hq) ? R / 2 : R - (fuse ? 2 : 1)) { // fewer row slots until three stages fit
        if (R < (fuse ? 2 : 1)) {
            return false;
        }
        W = (R * U + 31) / 32;
        p.W = W, p.R = R, p.U = U, p.seg = seg, p.P = U / seg, p.Ppad = p.P | 1;
        p.paired = fuse ? 1 : 0;
        p.H = fuse ? R / 2 : R;
        const size_t red = ((size_t)R * p.Ppad * 4 + 15) / 16 * 16;
        const size_t half = ((size_t)p.H * row_bytes + 32 + 15) / 16 * 16;
        const size_t stage = fuse ? (2 * half + 127) / 128 * 128 : ((size_t)R * row_bytes + 32 + 127) / 128 * 128;
        const size_t pack = ((size_t)U * kPinUnitBytes + 15) / 16 * 16;
        const size_t off_packs = kPinHdr + kRedBufs * red + 512;
        const size_t off_expert = off_packs + kMoePinSegs * pack;
        off_tiles = (off_expert + (size_t)n_pairs * 4 + 127) / 128 * 128;
        if (off_tiles + 3 * stage > (size_t)kPinSmem || stage >= (1u << 20)) {
            continue;
        }
        const int stages = (int)(((size_t)kPinSmem - off_tiles) / stage);
        p.half_off = fuse ? (int32_t)half : 0;
        p.stages = stages > 8 ? 8 : stages;
        p.stage_bytes = (int32_t)stage;
        p.red_bytes = (int32_t)red;
        p.off_tiles = (int32_t)off_tiles;
        a.off_packs = (int32_t)off_packs;
        a.pack_bytes = (int32_t)pack;
        a.off_expert = (int32_t)off_expert;
        break;
    }
    p.c.K = K;
    p.c.TB = 1;
    a.type = type_a;
    a.n_rows = n_rows;
    a.n_pairs = (int32_t)n_pairs;
    a.row_bytes = row_bytes;
    a.unit_rows = (fuse && want_hq) ? 32 : p.H; // a whole group of h, or one step
    a.upi = (n_rows + a.unit_rows - 1) / a.unit_rows;
    // pieces per share: a share of ceil(T / G) units spans at most that many pairs
    const long long T = n_pairs * a.upi, share = (T + kSMs - 1) / kSMs;
    if ((share + a.upi - 1) / a.upi + 1 > kMoePinSegs || T >= (1ll << 31)) {
        return false;
    }
    return true;
}

bool moe_pinned_supported(int type_a, int type_b, int K, int n_rows, int fuse_silu, long long n_pairs, bool want_hq) {
    MoePinArgs a;
    return moe_pin_plan(type_a, type_b, K, n_rows, fuse_silu, n_pairs, want_hq, a);
}

cudaError_t launch_moe_pinned(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                              size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                              const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                              const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                              float * out, int out_stride, int fuse_silu, const NextAct * hq) {
    const long long n_pairs = top_k > 0 ? (long long)TB * top_k : TB;
    MoePinArgs a;
    if (!moe_pin_plan(type_a, type_b, K, n_rows, fuse_silu, n_pairs, hq != nullptr, a)) {
        return cudaErrorInvalidConfiguration;
    }
    a.bank_a = static_cast<const uint8_t *>(bank_a);
    a.bank_b = static_cast<const uint8_t *>(bank_b);
    a.plane_a = plane_a;
    a.plane_b = plane_b;
    a.off = off;
    a.pair = pair;
    a.active = active;
    a.n_active = n_active;
    a.max_active = n_act_max;
    a.x8 = x8;
    a.xmeta = xmeta;
    a.xsumq = xsumq;
    a.TB = TB;
    a.top_k = top_k;
    a.out = out;
    a.out_stride = out_stride;
    a.hq = hq ? *hq : NextAct{nullptr, nullptr, nullptr};
    const size_t smem = (size_t)a.p.off_tiles + (size_t)a.p.stages * a.p.stage_bytes;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(moe_pinned_kernel), kPinSmem);
    if (e != cudaSuccess) {
        return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kSMs);
    cfg.blockDim = dim3((unsigned)(32 * (a.p.W + 2)));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, moe_pinned_kernel, a);
}

} // namespace b200q
