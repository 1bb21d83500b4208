// Single-token decode GEMV: the HBM-bound kernel of the library.
//
// Every consumer thread is pinned to ONE 128-value unit of the input vector (four activation
// groups) for the whole launch and keeps that unit's quantized activation - 128 int8 codes,
// four scales, the sums the min / offset terms need - in registers.  A step of the CTA is R
// whole weight rows; the 32*W consumer threads cover R row slots x U units (U = K / 128), so
// a thread's work per step is exactly one unit of one row: load 72..136 bytes of raw GGUF
// blocks from shared memory, unpack, dp4a against registers, apply the fp32 scales.  No
// activation is re-read from shared memory, lanes are fully used whatever K is (W is chosen
// per call so that R*U fills 32*W), and a call with few rows per SM loses nothing to ragged
// tiles.
//
// Data movement.  One CTA per SM.  A producer thread brings the R contiguous rows of a step
// into a ring of shared-memory stages with ONE bulk asynchronous copy (cp.async.bulk, the 1-D
// TMA path, no multicast) that completes on an mbarrier; the ring holds up to ~200 KB per SM.
// A copy starts on a 16-byte boundary: rows that start at address A are fetched from A & ~15
// and decoded from offset A & 15 (Q6_K / Q8_0 rows are only 2-byte aligned).
//
// Activation.  After the previous kernel has finished, ONE thread fetches the activation (the
// fp32 vector, or the already quantized views) into shared memory with bulk copies: 148 CTAs
// asking for the same 20 KB through per-thread loads serialise in the L2 slices that own those
// lines (measured 3.7 us), a copy engine's full-line requests do not.  The consumer warps then
// quantize it (8 threads per 32-value group) into a pack from which every thread takes its unit.
//
// Reduction.  Lanes are summed in aligned segments of `seg` lanes (the largest power of two
// that divides U, so a segment never straddles two rows) with butterfly shuffles; one lane per
// segment stores the partial into a small shared-memory array [slot][part]; a dedicated
// epilogue warp (lane = row slot) adds the U/seg partials of its row in a fixed order, applies
// alpha and the residual and stores the outputs (also into the peers' copies for row-sharded
// calls).  For a gate|up call it can also form silu(gate)*up and quantize
// it per 32 rows as soon as both halves of a group are complete, so the following down call
// needs no quantizer launch.
//
// Chaining.  The kernel is launched with programmatic stream serialization: its producer
// prefetches weights while the previous kernel of the stream is still draining; consumers and
// the epilogue execute griddepcontrol.wait before they touch the activation or any output.
// Early starts only happen behind kernels that trigger them (this library's own), and none of
// those writes weights.
//
// Every mbarrier wait is bounded by a clock budget; a wait that runs out records
// B200Q_ETIMEOUT in a status word the host reads (b200q_device_status) and the role returns.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "launch.h"
#include "stream_core.cuh"
#include "argmax.cuh"

namespace b200q {

constexpr int kPinMaxW = 18;                      // consumer warps
constexpr int kPinThreads = 32 * (kPinMaxW + 2);  // + producer warp + epilogue warp
constexpr int kPinSmem = 227 * 1024;
constexpr int kRedBufs = 4;   // partial-sum buffers in flight between consumers and the epilogue warp
constexpr int kPinHdr = 256;  // mbarriers and flags at the start of shared memory

__device__ int g_pin_status = 0;

struct PinArgs {
    CallDev c;
    CostSplit cost;
    const float * xq_x; // when set, every CTA quantizes this fp32 activation itself
    NormArgs norm;      // RMSNorm applied to xq_x before it is quantized (w == nullptr: off)
    int32_t * am_idx;   // argmax over the call's (single segment's) outputs, lowest index among equals (nullptr: off)
    float * am_val;
    NextAct next;       // the call's output, quantized, as the following call's activation (x8 == nullptr: off)
    PeerSync sync;      // row-sharded calls: wait for / signal the peers inside this launch
    int32_t W, R, U, seg, P, Ppad; // P = U / seg partials per row, rows Ppad words apart
    // paired mode (next.cnt != nullptr): a step is H gate rows and the H up rows of the same
    // indices; the up rows sit half_off bytes into the stage
    int32_t H, half_off, paired, next_mode;
    int32_t stages, stage_bytes, red_bytes;
    int32_t off_pack, off_tiles;
    int32_t off_xraw; // shared-memory landing zone of the raw activation (fp32 vector, or the three quantized views)
#ifdef B200Q_TUNING
    unsigned long long * trace; // [launch % 64][CTA][8] globaltimer stamps of the roles' milestones
    int32_t launch_idx;
#endif
};

#ifdef B200Q_TUNING
__device__ __forceinline__ void pin_stamp(const PinArgs & a, int ev) {
    if (a.trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.trace[((size_t)(a.launch_idx & 63) * 160 + blockIdx.x) * 8 + ev] = t;
    }
}
#define PIN_STAMP(ev) pin_stamp(a, ev)
static int g_trace_launches = 0; // every call, chained or not, gets its own slot of the trace
static void trace_slot(PinArgs & a, bool count) {
    const char * tp = getenv("B200Q_TRACE_PTR");
    a.trace = tp ? reinterpret_cast<unsigned long long *>(strtoull(tp, nullptr, 0)) : nullptr;
    a.launch_idx = g_trace_launches;
    g_trace_launches += count ? 1 : 0;
}
#else
#define PIN_STAMP(ev)
#endif

struct PinRing {
    int stage;
    uint32_t phase;
    int rb;
    uint32_t rphase;
    __device__ __forceinline__ void advance(int S) {
        if (++stage == S) {
            stage = 0;
            phase ^= 1;
        }
        if (++rb == kRedBufs) {
            rb = 0;
            rphase ^= 1;
        }
    }
};

// Calls that also emit the next call's activation split their rows (or gate|up pairs) in whole
// 32-row groups: the CTA that finishes a group holds all 32 values and quantizes it on the
// spot, with no exchange between CTAs.  Part p of G owns groups [n*p/G, n*(p+1)/G).
__device__ __forceinline__ RowRange group_rows(const CallDev & c, uint32_t p, uint32_t G) {
    const uint32_t n = (uint32_t)c.seg[0].n_rows >> 5;
    RowRange r;
    r.lo = (int)(32u * (n * p / G));
    r.hi = (int)(32u * (n * (p + 1) / G));
    return r;
}

// A wait whose clock budget only runs while `gate` (a shared-memory word) is non-zero: the
// producer must not time out while the consumers are still parked behind the previous kernel.
__device__ __forceinline__ bool mbar_wait_gated(uint32_t bar, uint32_t parity, int * status, uint32_t gate) {
    long long t0 = 0;
    for (uint32_t n = 0;; n++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) {
            return true;
        }
        if (n == 64) {
            t0 = clock64();
        } else if (n > 64 && clock64() - t0 > kSpinCycles) {
            uint32_t g;
            asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(g) : "r"(gate) : "memory");
            if (g) {
                break;
            }
            t0 = clock64();
        }
    }
    atomicExch(status, B200Q_ETIMEOUT);
    return false;
}

// ---- activation: quantize (8 threads per 32-value group) or fetch, then pin --------------------
// Pack layout of this kernel: 48 bytes per group (codes | sx | xs0 | xs1 | sx*(xs0+xs1)), the
// four groups of a unit back to back, units 208 bytes apart: an odd number of 16-byte chunks, so
// the eight lanes of a quarter-warp that fetch their units with 128-bit loads hit distinct banks
// (units 192 bytes apart would put them on two).
constexpr uint32_t kPinUnitBytes = 4 * kPackGroup + 16;
__device__ __forceinline__ uint32_t pin_pack_addr(uint32_t pack, int g) {
    return pack + (uint32_t)(g >> 2) * kPinUnitBytes + (uint32_t)(g & 3) * kPackGroup;
}

// The arithmetic is the standalone quantizer's (xq.cuh), bit for bit: max and integer sums are
// exact in any order, every fp32 operation is a single correctly rounded one.
// nw != nullptr: the value quantized is (x * nscale) * nw[i], the RMSNorm of the row (rmsnorm_row,
// src/backend/cpu/kernels/common.cpp:685-691 of the reference: two roundings, left to right).
template <bool NORM>
__device__ __forceinline__ void pin_quantize(uint32_t pack, const CallDev & c, uint32_t xraw, int G, int warp,
                                             int lane, int W, bool write_views, const float * nw, float nscale) {
    constexpr int kBatch = 4; // loads of several passes in flight before the first is used
    const int stride = 32 * W, n_tasks = 8 * G;
    for (int base0 = warp * 32; base0 < n_tasks; base0 += kBatch * stride) {
        float4 fb[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
            const int task = base0 + i * stride + lane;
            fb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (task < n_tasks) {
                const uint4 u = lds128(xraw + 16u * (uint32_t)task);
                fb[i] = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
                if (NORM && nw) {
                    const float4 wv = __ldg(reinterpret_cast<const float4 *>(nw) + task);
                    fb[i].x = __fmul_rn(__fmul_rn(fb[i].x, nscale), wv.x);
                    fb[i].y = __fmul_rn(__fmul_rn(fb[i].y, nscale), wv.y);
                    fb[i].z = __fmul_rn(__fmul_rn(fb[i].z, nscale), wv.z);
                    fb[i].w = __fmul_rn(__fmul_rn(fb[i].w, nscale), wv.w);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
            if (base0 + i * stride >= n_tasks) { // uniform per warp
                break;
            }
            const int task = base0 + i * stride + lane;
            const bool valid = task < n_tasks;
            const int g = task >> 3, j = task & 7;
            const float4 f = fb[i];
            float mx = fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w)));
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 4));
            const float inv = mx > 0.0f ? __fdiv_rn(127.0f, mx) : 0.0f;
            const float v[4] = {f.x, f.y, f.z, f.w};
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const float r = fminf(127.0f, fmaxf(-127.0f, roundf(__fmul_rn(v[b], inv))));
                word |= ((uint32_t)(int)r & 0xFFu) << (8 * b);
            }
            int s = __dp4a((int)word, 0x01010101, 0);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            const int other = __shfl_xor_sync(0xFFFFFFFFu, s, 4);
            const int s0 = (j & 4) ? other : s, s1 = (j & 4) ? s : other;
            const float sx = h2f(f2h_trunc(mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 0.0f));
            if (valid) {
                const uint32_t p = pin_pack_addr(pack, g);
                sts32(p + 4 * j, word);
                if (j == 0) {
                    sts128(p + 32, __float_as_uint(sx), (uint32_t)s0, (uint32_t)s1,
                           __float_as_uint(sx * (float)(s0 + s1)));
                }
                if (write_views) {
                    reinterpret_cast<uint32_t *>(const_cast<int8_t *>(c.x8))[task] = word;
                    if (j == 0) {
                        reinterpret_cast<float2 *>(const_cast<float *>(c.xmeta))[g] = make_float2(sx, 0.0f);
                        reinterpret_cast<int2 *>(const_cast<int32_t *>(c.xsumq))[g] = make_int2(s0, s1);
                    }
                }
            }
        }
    }
}

// Only what TYPE's decoder reads is loaded (Q4_K / Q5_K: scales and scale x sum; Q6_K: scales and
// the two 16-value sums; the others: scales), so the rest costs no registers in that type's loop.
template <int TYPE> __device__ __forceinline__ void pin_from_pack(uint32_t pack, int unit, ActPin & a) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t p = pin_pack_addr(pack, 4 * unit + i);
        const uint4 x0 = lds128(p), x1 = lds128(p + 16), m = lds128(p + 32);
        a.x[i][0] = x0.x, a.x[i][1] = x0.y, a.x[i][2] = x0.z, a.x[i][3] = x0.w;
        a.x[i][4] = x1.x, a.x[i][5] = x1.y, a.x[i][6] = x1.z, a.x[i][7] = x1.w;
        a.sx[i] = __uint_as_float(m.x);
        a.xs[i][0] = TYPE == kQ6_K ? (int)m.y : 0;
        a.xs[i][1] = TYPE == kQ6_K ? (int)m.z : 0;
        a.c[i] = (TYPE == kQ4_K || TYPE == kQ5_K) ? __uint_as_float(m.w) : 0.0f;
    }
}

// The pack from the caller's quantized views (one token), which lie in shared memory as
// [K codes][K/32 (scale, 0) pairs][K/32 sum pairs].
__device__ __forceinline__ void pin_stage_views(uint32_t pack, uint32_t xraw, int G, int tid, int nthr) {
    const uint32_t meta = xraw + 32u * (uint32_t)G, sums = meta + 8u * (uint32_t)G;
    for (int g = tid; g < G; g += nthr) { // one token: group index == array index
        const uint4 x0 = lds128(xraw + 32u * (uint32_t)g), x1 = lds128(xraw + 32u * (uint32_t)g + 16u);
        const float sx = __uint_as_float(lds32(meta + 8u * (uint32_t)g));
        const uint2 xs = lds64(sums + 8u * (uint32_t)g);
        const uint32_t p = pin_pack_addr(pack, g);
        sts128(p, x0.x, x0.y, x0.z, x0.w);
        sts128(p + 16, x1.x, x1.y, x1.z, x1.w);
        sts128(p + 32, __float_as_uint(sx), xs.x, xs.y, __float_as_uint(sx * (float)((int)xs.x + (int)xs.y)));
    }
}

// One thread, one unit (half h of the superblock at shared address sb) of one row.
template <int TYPE> __device__ __forceinline__ float pinned_term(uint32_t sb, int h, const ActPin & p) {
    if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        return HalfK45<TYPE>::term(sb, h, p);
    } else if constexpr (TYPE == kQ6_K) {
        return HalfQ6::term(sb, h, p);
    } else { // two quarter units of two groups each
        float r = 0.f;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            WUnit<TYPE> w;
            w.load(sb, 2 * h + e);
            ActG2 g;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                g.xa[k] = p.x[2 * e][k];
                g.xb[k] = p.x[2 * e + 1][k];
            }
            g.ma.sx = p.sx[2 * e];
            g.mb.sx = p.sx[2 * e + 1];
            r += w.term(g);
        }
        return r;
    }
}

struct PinBars {
    uint32_t full, empty, red_full, red_empty;
};

// The hot loop polls two mbarriers per step; nearly always the first try succeeds, and the
// bounded spin (clock reads, status word) is only entered when it does not.
__device__ __forceinline__ bool mbar_wait_fast(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok ? true : mbar_wait(bar, parity, &g_pin_status);
}

// Rows [lo, hi) of weight w0 - and, in paired mode, the same rows of w1 in the slots from H on.
template <int TYPE>
__device__ __forceinline__ bool pin_consume_rows(const PinArgs & a, const PinArgs & g, const uint8_t * w0,
                                                 const uint8_t * w1, int lo, int hi, uint32_t tiles, uint32_t red,
                                                 const PinBars & bars, const ActPin & pin, int slot, int unit,
                                                 PinRing & pos) {
    constexpr uint32_t SB = Fmt<TYPE>::SB;
    const int lane = threadIdx.x & 31;
    const int H = a.H, S = g.stages;
    const uint32_t row_bytes = (uint32_t)(a.c.K >> 8) * SB;
    const int part = slot >= H ? 1 : 0, sl = slot - part * H; // normal mode: H == R, part 0 only
    const bool mine = slot < a.R;
    const uint32_t wbase = (uint32_t)(reinterpret_cast<uintptr_t>(part ? w1 : w0) & 15);
    const uint32_t my_off = (uint32_t)(part * a.half_off) + (uint32_t)sl * row_bytes + (uint32_t)(unit >> 1) * SB;
    const int seg = a.seg;
    const bool writer = (lane & (seg - 1)) == 0 && mine;
    const int h = unit & 1;
    // everything that moves with the ring is kept as an address and stepped, not recomputed
    const uint32_t stage_bytes = (uint32_t)g.stage_bytes, red_bytes = (uint32_t)g.red_bytes;
    uint32_t st_addr = tiles + (uint32_t)pos.stage * stage_bytes + my_off;
    uint32_t rd_addr = red + (uint32_t)pos.rb * red_bytes + (uint32_t)(slot * a.Ppad + unit / seg) * 4u;
    // where a row's bytes start inside its 16-byte line: only the low four address bits matter
    uint32_t mis = (wbase + (uint32_t)lo * row_bytes) & 15u;
    const uint32_t mis_step = ((uint32_t)H * row_bytes) & 15u;
    for (int left = hi - lo; left > 0; left -= H) {
        if (!mbar_wait_fast(bars.full + 8 * pos.stage, pos.phase)) {
            return false;
        }
        const bool active = sl < left;
        float v = 0.f;
        if (mine && active) {
            v = pinned_term<TYPE>(st_addr + mis, h, pin);
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { // all lanes of a segment belong to the same row slot
            if (o < seg) {
                v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            }
        }
        if (!mbar_wait_fast(bars.red_empty + 8 * pos.rb, pos.rphase ^ 1)) {
            return false;
        }
        if (writer && active) {
            sts32(rd_addr, __float_as_uint(v));
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(bars.red_full + 8 * pos.rb);
            mbar_arrive(bars.empty + 8 * pos.stage);
        }
        mis = (mis + mis_step) & 15u;
        if (++pos.stage == S) {
            pos.stage = 0;
            pos.phase ^= 1;
            st_addr -= (uint32_t)(S - 1) * stage_bytes;
        } else {
            st_addr += stage_bytes;
        }
        if (++pos.rb == kRedBufs) {
            pos.rb = 0;
            pos.rphase ^= 1;
            rd_addr -= (kRedBufs - 1) * red_bytes;
        } else {
            rd_addr += red_bytes;
        }
    }
    return true;
}
template <int TYPE>
__device__ __forceinline__ bool pin_consume_call(const PinArgs & a, const PinArgs & g, int si, uint32_t cost_lo, uint32_t cost_hi,
                                                 uint32_t tiles, uint32_t red, const PinBars & bars, uint32_t pack,
                                                 int slot, int unit, PinRing & pos) {
    ActPin pin; // this thread's unit of the activation, for the whole segment
    pin_from_pack<TYPE>(pack, unit, pin);
    if (a.paired) { // gate rows and up rows together
        const RowRange pr = group_rows(a.c, blockIdx.x, gridDim.x);
        return pin_consume_rows<TYPE>(a, g, a.c.seg[0].w, a.c.seg[1].w, pr.lo, pr.hi, tiles, red, bars, pin, slot, unit, pos);
    }
    const RowRange rr = a.next.x8 ? group_rows(a.c, blockIdx.x, gridDim.x) : cta_rows(a.c, si, cost_lo, cost_hi);
    return pin_consume_rows<TYPE>(a, g, a.c.seg[si].w, a.c.seg[si].w, rr.lo, rr.hi, tiles, red, bars, pin, slot, unit, pos);
}

// Rows [32g, 32g+32) of the call's output as the next call's activation, quantized as b200q_xq
// would (one token): the output itself (one segment; lane i holds row 32g + i in gv), or
// silu(gate)*up (two segments; lane i holds gate and up of row 32g + i).
__device__ __forceinline__ void next_act_group(const PinArgs & a, int g, int lane, float gv, float uv) {
    const float v = a.paired ? __fmul_rn(silu_exact(gv), uv) : gv;
    float scale;
    int s0, s1;
    const int q = xq_group(v, lane, scale, s0, s1);
    a.next.x8[32 * g + lane] = (int8_t)q;
    if (lane == 0) {
        a.next.xmeta[2 * g] = scale;
        a.next.xmeta[2 * g + 1] = 0.0f;
        a.next.xsumq[2 * g] = s0;
        a.next.xsumq[2 * g + 1] = s1;
    }
}

// ---- the roles, one call each: both kernels below are built from these --------------------------
// a = the call; g = where the shared-memory geometry comes from (a itself, or the first call of a
// chain, whose geometry every call of the chain shares: a fixed place in the kernel parameters).
struct PinProd {
    int stage;
    uint32_t par; // parity of the empty barrier: a fresh slot is free
    int issued;
};

// Producer thread: one bulk copy (two in paired mode) per step of this CTA's rows of call a.
__device__ __forceinline__ bool pin_produce(const PinArgs & a, const PinArgs & g, uint32_t tiles, const PinBars & bars,
                                            uint32_t started, PinProd & pr) {
    const int S = g.stages, R = a.R, nb = a.c.K >> 8;
    bool alive = true;
    if (a.paired) { // H gate rows and the H up rows of the same indices per stage
        const RowRange rg = group_rows(a.c, blockIdx.x, gridDim.x);
        const size_t row_bytes = (size_t)nb * sb_bytes(a.c.seg[0].type);
        for (int p0 = rg.lo; p0 < rg.hi; p0 += a.H) {
            const int rows = min(a.H, rg.hi - p0);
            uintptr_t A0[2];
            uint32_t len[2];
            for (int e = 0; e < 2; e++) {
                const uintptr_t A = reinterpret_cast<uintptr_t>(a.c.seg[e].w + (size_t)p0 * row_bytes);
                A0[e] = A & ~uintptr_t(15);
                len[e] = (uint32_t)(((A + (size_t)rows * row_bytes + 15) & ~uintptr_t(15)) - A0[e]);
            }
            alive = mbar_wait_gated(bars.empty + 8 * pr.stage, pr.par, &g_pin_status, started);
            if (!alive) {
                return false;
            }
            mbar_expect_tx(bars.full + 8 * pr.stage, len[0] + len[1]);
            const uint32_t dst = tiles + (uint32_t)(pr.stage * g.stage_bytes);
            bulk_g2s(dst, reinterpret_cast<const void *>(A0[0]), len[0], bars.full + 8 * pr.stage);
            bulk_g2s(dst + (uint32_t)a.half_off, reinterpret_cast<const void *>(A0[1]), len[1], bars.full + 8 * pr.stage);
            pr.issued++;
            if (++pr.stage == S) {
                pr.stage = 0;
                pr.par ^= 1;
            }
        }
        return true;
    }
    const uint32_t cost_lo = cost_at(a.cost, blockIdx.x, gridDim.x), cost_hi = cost_at(a.cost, blockIdx.x + 1, gridDim.x);
    for (int si = 0; si < a.c.n_segs; si++) {
        const SegDev & sg = a.c.seg[si];
        const RowRange rr = a.next.x8 ? group_rows(a.c, blockIdx.x, gridDim.x) : cta_rows(a.c, si, cost_lo, cost_hi);
        const size_t row_bytes = (size_t)nb * sb_bytes(sg.type);
        for (int row0 = rr.lo; row0 < rr.hi; row0 += R) {
            const int rows = min(R, rr.hi - row0);
            const uintptr_t A = reinterpret_cast<uintptr_t>(sg.w + (size_t)row0 * row_bytes);
            const uintptr_t A0 = A & ~uintptr_t(15);
            const uint32_t len = (uint32_t)(((A + (size_t)rows * row_bytes + 15) & ~uintptr_t(15)) - A0);
            alive = mbar_wait_gated(bars.empty + 8 * pr.stage, pr.par, &g_pin_status, started);
            if (!alive) {
                return false;
            }
            mbar_expect_tx(bars.full + 8 * pr.stage, len);
            bulk_g2s(tiles + (uint32_t)(pr.stage * g.stage_bytes), reinterpret_cast<const void *>(A0), len,
                     bars.full + 8 * pr.stage);
            pr.issued++;
            if (++pr.stage == S) {
                pr.stage = 0;
                pr.par ^= 1;
            }
        }
    }
    return true;
}

// A producer that leaves early waits (bounded) until the copies still in flight have landed.
__device__ __forceinline__ void pin_produce_drain(const PinBars & bars, int S, const PinProd & pr) {
    for (int s = 0; s < S && s < pr.issued; s++) {
        const int last = ((pr.issued - 1 - s) / S) * S + s; // last step that filled stage s
        mbar_wait(bars.full + 8 * s, (uint32_t)(last / S) & 1u, &g_pin_status);
    }
}

// Epilogue warp: partial sums of each step -> alpha, residual, outputs (and the next call's
// activation).  rb / rphase walk the ring of partial-sum buffers and carry over between calls.
// AMAX: the argmax of the outputs is tracked and contributed (kernel images of their own).
template <bool AMAX>
__device__ __forceinline__ bool pin_epilogue(const PinArgs & a, const PinArgs & g, uint32_t red, const PinBars & bars,
                                             int & rb, uint32_t & rphase) {
    const int lane = threadIdx.x & 31;
    const int P = a.P, Ppad = a.Ppad, R = a.R;
    if (a.next.x8) {
        // The call's output doubles as the next call's activation.  One segment: lane = row
        // slot.  Two segments (gate|up, paired mode): lanes 0..15 take gate slots, lanes 16..31
        // the up slots of the same pairs, sixteen pairs at a time.  Every stored value is also
        // kept in a 64-row ring in shared memory; when a 32-row group completes, lane i takes
        // its row's value(s) from the ring and the warp quantizes the group (a CTA's range
        // is made of whole groups).
        const uint32_t ring = red + (uint32_t)(kRedBufs * g.red_bytes); // 2 x 64 floats behind the partials
        const RowRange pr = group_rows(a.c, blockIdx.x, gridDim.x);
        const int H = a.H, per = a.paired ? 16 : 32;
        const int e = a.paired ? lane >> 4 : 0, li = lane & (per - 1);
        const SegDev & sg = a.c.seg[e];
        for (int p0 = pr.lo; p0 < pr.hi; p0 += H) {
            const int rows = min(H, pr.hi - p0);
            if (!mbar_wait(bars.red_full + 8 * rb, rphase, &g_pin_status)) {
                return false;
            }
            const uint32_t rbuf = red + (uint32_t)(rb * g.red_bytes);
            for (int c0 = 0; c0 < rows; c0 += per) {
                if (c0 + li < rows) {
                    const uint32_t p = rbuf + (uint32_t)((e * H + c0 + li) * Ppad) * 4u;
                    float sum = 0.f;
                    for (int j = 0; j < P; j++) {
                        sum += __uint_as_float(lds32(p + 4u * (uint32_t)j));
                    }
                    const int row = p0 + c0 + li;
                    float v = sg.alpha * sum;
                    if (sg.residual) {
                        v += __ldcg(&sg.residual[row]);
                    }
                    sg.out[row] = v;
                    sts32(ring + (uint32_t)(e * 64 + (row & 63)) * 4u, __float_as_uint(v));
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
            // groups whose last row was stored in this step (H <= 32: at most two)
            for (int gi = p0 >> 5; 32 * gi + 32 <= p0 + rows; gi++) {
                const float gv = __uint_as_float(lds32(ring + (uint32_t)((32 * gi + lane) & 63) * 4u));
                const float uv = __uint_as_float(lds32(ring + (uint32_t)(64 + ((32 * gi + lane) & 63)) * 4u));
                next_act_group(a, gi, lane, gv, uv);
                __syncwarp();
            }
        }
        return true;
    }
    const uint32_t cost_lo = cost_at(a.cost, blockIdx.x, gridDim.x), cost_hi = cost_at(a.cost, blockIdx.x + 1, gridDim.x);
    float am_best = 0.0f; // this lane's best output so far (argmax option; rows come in increasing order)
    int am_i = -1;
    for (int si = 0; si < a.c.n_segs; si++) {
        const SegDev & sg = a.c.seg[si];
        const RowRange rr = cta_rows(a.c, si, cost_lo, cost_hi);
        for (int row0 = rr.lo; row0 < rr.hi; row0 += R) {
            const int rows = min(R, rr.hi - row0);
            if (!mbar_wait(bars.red_full + 8 * rb, rphase, &g_pin_status)) {
                return false;
            }
            const uint32_t rbuf = red + (uint32_t)(rb * g.red_bytes);
            for (int c0 = 0; c0 < rows; c0 += 32) { // lane = row slot; partials added in a fixed order
                if (c0 + lane < rows) {
                    const uint32_t p = rbuf + (uint32_t)((c0 + lane) * Ppad) * 4u;
                    float sum = 0.f;
                    for (int j = 0; j < P; j++) {
                        sum += __uint_as_float(lds32(p + 4u * (uint32_t)j));
                    }
                    const size_t o = (size_t)(row0 + c0 + lane); // one token
                    float v = sg.alpha * sum;
                    if (sg.residual) {
                        v += __ldcg(&sg.residual[o]);
                    }
                    store_out(a.c, &sg.out[o], v);
                    if (AMAX && (am_i < 0 || v > am_best)) {
                        am_best = v;
                        am_i = (int)o;
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
        }
    }
    if (AMAX) { // one segment (checked on the host): the CTA's best joins the grid's; the last CTA writes the result
        const unsigned long long k = argmax_warp(am_i >= 0 ? argmax_key(am_best, (uint32_t)am_i) : 0ull);
        if (lane == 0) {
            argmax_contribute(0, k, gridDim.x, a.c.seg[0].out, a.am_idx, a.am_val);
        }
    }
    return true;
}

// Consumer warps: fetch the call's activation with bulk copies (thread 0 issues them) and quantize
// or re-lay it into the pack, from which every thread then takes its unit into registers.
// NORM: the RMSNorm of the row is folded in (a kernel image of its own, so that the plain one carries none of it).
template <bool NORM>
__device__ __forceinline__ bool pin_activation(const PinArgs & a, const PinArgs & g, uint32_t base, uint32_t parity) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = a.W, nb = a.c.K >> 8;
    const uint32_t pack = base + (uint32_t)g.off_pack, xraw = base + (uint32_t)g.off_xraw, act_bar = base + 200;
    const uint32_t K = (uint32_t)a.c.K;
    if (threadIdx.x == 0) {
        if (a.xq_x) {
            mbar_expect_tx(act_bar, 4u * K);
            bulk_g2s(xraw, a.xq_x, 4u * K, act_bar);
        } else {
            mbar_expect_tx(act_bar, K + K / 2);
            bulk_g2s(xraw, a.c.x8, K, act_bar);
            bulk_g2s(xraw + K, a.c.xmeta, K / 4, act_bar);
            bulk_g2s(xraw + K + K / 4, a.c.xsumq, K / 4, act_bar);
        }
    }
    if (!mbar_wait(act_bar, parity, &g_pin_status)) {
        return false;
    }
    if (threadIdx.x == 0) {
        PIN_STAMP(7);
    }
    if (a.xq_x) {
        float nscale = 1.0f;
        if (NORM && a.norm.w) {
            // 1 / sqrt(sum(x^2) / K + eps), the sum in the order of the reference's widest host path
            // (sumsq_f32_avx512, common.cpp:278-290): sixteen accumulators acc[j] = fma(x, x, acc[j])
            // over i = 16k + j, halved 16 -> 8 -> 4, then (t0 + t2) + (t1 + t3)
            if (warp == 0) {
                float acc = 0.f;
                if (lane < 16) {
                    for (uint32_t i = (uint32_t)lane; i < K; i += 128) { // K is a multiple of 256
                        float v[8];
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            v[u] = __uint_as_float(lds32(xraw + 4u * (i + 16u * (uint32_t)u)));
                        }
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            acc = __fmaf_rn(v[u], v[u], acc);
                        }
                    }
                }
                acc = __fadd_rn(__shfl_down_sync(0xFFFFFFFFu, acc, 8), acc);
                acc = __fadd_rn(acc, __shfl_down_sync(0xFFFFFFFFu, acc, 4));
                acc = __fadd_rn(acc, __shfl_down_sync(0xFFFFFFFFu, acc, 2));
                acc = __fadd_rn(acc, __shfl_down_sync(0xFFFFFFFFu, acc, 1));
                if (lane == 0) {
                    const float sc = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(acc, (float)K), a.norm.eps)));
                    sts32(base + 208, __float_as_uint(sc));
                }
            }
            asm volatile("bar.sync 1, %0;" ::"r"(32 * W) : "memory");
            nscale = __uint_as_float(lds32(base + 208));
        }
        pin_quantize<NORM>(pack, a.c, xraw, 8 * nb, warp, lane, W, blockIdx.x == 0, a.norm.w, nscale);
    } else {
        pin_stage_views(pack, xraw, 8 * nb, (int)threadIdx.x, 32 * W);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(32 * W) : "memory");
    return true;
}

// Consumer warps: every step of this CTA's share of call a.
__device__ __forceinline__ bool pin_consume(const PinArgs & a, const PinArgs & g, uint32_t tiles, uint32_t red,
                                            const PinBars & bars, uint32_t pack, int slot, int unit, PinRing & pos) {
    const uint32_t cost_lo = cost_at(a.cost, blockIdx.x, gridDim.x), cost_hi = cost_at(a.cost, blockIdx.x + 1, gridDim.x);
    const int n_calls = a.paired ? 1 : a.c.n_segs; // paired mode walks both segments at once
    for (int si = 0; si < n_calls; si++) {
        bool ok;
        switch (a.c.seg[si].type) {
        case kQ4_K: ok = pin_consume_call<kQ4_K>(a, g, si, cost_lo, cost_hi, tiles, red, bars, pack, slot, unit, pos); break;
        case kQ5_K: ok = pin_consume_call<kQ5_K>(a, g, si, cost_lo, cost_hi, tiles, red, bars, pack, slot, unit, pos); break;
        case kQ6_K: ok = pin_consume_call<kQ6_K>(a, g, si, cost_lo, cost_hi, tiles, red, bars, pack, slot, unit, pos); break;
        case kIQ4_XS: ok = pin_consume_call<kIQ4_XS>(a, g, si, cost_lo, cost_hi, tiles, red, bars, pack, slot, unit, pos); break;
        default: ok = pin_consume_call<kQ8_0>(a, g, si, cost_lo, cost_hi, tiles, red, bars, pack, slot, unit, pos); break;
        }
        if (!ok) {
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void pin_init_barriers(const PinBars & bars, uint32_t base, int S, int W) {
    for (int s = 0; s < S; s++) {
        mbar_init(bars.full + 8 * s, 1);
        mbar_init(bars.empty + 8 * s, (uint32_t)W);
    }
    for (int b = 0; b < kRedBufs; b++) {
        mbar_init(bars.red_full + 8 * b, (uint32_t)W);
        mbar_init(bars.red_empty + 8 * b, 1);
    }
    mbar_init(base + 200, 1); // the activation's bulk copies
    sts32(base + 192, 0);     // "consumers have started": gates the producer's clock budget
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

template <bool NORM, bool AMAX>
__global__ void __launch_bounds__(kPinThreads, 1) gemv_pinned_kernel(const __grid_constant__ PinArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const PinBars bars{base, base + 64, base + 128, base + 160};
    const uint32_t started = base + 192;
    const uint32_t red = base + kPinHdr, tiles = base + (uint32_t)a.off_tiles;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = a.W;

    // let the next kernel of the stream be scheduled as soon as this grid is resident
    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        PIN_STAMP(0);
        pin_init_barriers(bars, base, a.stages, W);
    }
    __syncthreads();

    if (warp == W) {
        // ---------------------------------------------------------------- producer (one thread)
        if (lane != 0) {
            return;
        }
        PinProd pr{0, 1, 0};
        if (!pin_produce(a, a, tiles, bars, started, pr)) {
            pin_produce_drain(bars, a.stages, pr);
        }
        return;
    }

    // everything below reads the activation or writes outputs: wait for the previous kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        PIN_STAMP(1);
    }

    if (warp == W + 1) {
        // ---------------------------------------------------------------- epilogue warp
        int rb = 0;
        uint32_t rphase = 0;
        if (!pin_epilogue<AMAX>(a, a, red, bars, rb, rphase)) {
            return;
        }
        if (a.sync.signal) {
            // every CTA: publish its peer stores system-wide, then count itself; the last one
            // advances this rank's call count and writes it into every peer's flag array
            __threadfence_system();
            __syncwarp();
            if (lane == 0) {
                uint32_t * own = a.sync.flag[a.sync.rank];
                const uint32_t old = atomicAdd(own + 33, 1u);
                if (old == gridDim.x - 1) {
                    own[33] = 0;
                    uint32_t seq;
                    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(seq) : "l"(own + 32) : "memory");
                    seq += 1;
                    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(own + 32), "r"(seq) : "memory");
                    __threadfence_system();
                    for (int p = 0; p < a.sync.world; p++) {
                        if (p != a.sync.rank) {
                            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.sync.flag[p] + a.sync.rank), "r"(seq)
                                         : "memory");
                        }
                    }
                }
            }
        }
        if (lane == 0) {
            PIN_STAMP(5);
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    if (a.sync.wait) {
        // every peer must have finished storing the previous call's rows into this GPU's memory:
        // its signal count has to reach this rank's own (all ranks run the same call sequence)
        if (warp == 0 && lane < a.sync.world && lane != a.sync.rank) {
            const uint32_t * own = a.sync.flag[a.sync.rank];
            uint32_t expected;
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(expected) : "l"(own + 32) : "memory");
            const long long t0 = clock64();
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(own + lane) : "memory");
                if ((int32_t)(v - expected) >= 0) {
                    break;
                }
                if (clock64() - t0 > kSpinCycles) {
                    atomicExch(&g_pin_status, B200Q_ETIMEOUT);
                    break;
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(32 * W) : "memory");
    }
    const int U = a.U;
    const int slot = (int)threadIdx.x / U, unit = (int)threadIdx.x - slot * U;
    if (!pin_activation<NORM>(a, a, base, 0)) {
        return;
    }
    if (threadIdx.x == 0) {
        asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(started), "r"(1u) : "memory");
        PIN_STAMP(2);
    }
    PinRing pos{0, 0, 0, 0};
    if (!pin_consume(a, a, tiles, red, bars, base + (uint32_t)a.off_pack, slot, unit, pos)) {
        return;
    }
    if (threadIdx.x == 0) {
        PIN_STAMP(4);
    }
}

// ---- several dependent calls in one launch ------------------------------------------------------
// Calls whose activation is the previous call's output (o -> gate|up -> down) pay, as separate
// launches, a start-up and a drain each during which HBM does not stream for them.  Here the
// same roles walk the calls one after the other inside ONE launch: the producer keeps the ring
// full across the boundaries (weights depend on nothing), the epilogue warp counts its CTA in
// when its rows of a call are stored, and the consumers of every CTA wait for that count to reach
// (calls so far) x (CTAs) before they fetch the next activation.  All CTAs are resident (one per
// SM, at most one CTA per SM in the grid), so the wait cannot starve; it is bounded like every
// other wait.  All calls share one ring geometry and the same kChainW consumer warps.
constexpr int kChainMax = 4;
constexpr int kChainW = kPinMaxW; // consumer warps of every call of a chain
struct ChainArgs {
    PinArgs call[kChainMax];
    int32_t n;
};
// CTAs that have finished call 0, 1, ... of the running chain launch; the last arrival of the
// last call puts it back to zero.  One chain launch at a time per device.
__device__ uint32_t g_chain_count = 0;

__global__ void __launch_bounds__(32 * (kChainW + 2), 1) gemv_chain_kernel(const __grid_constant__ ChainArgs ch) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const PinBars bars{base, base + 64, base + 128, base + 160};
    const uint32_t started = base + 192;
    const uint32_t red = base + kPinHdr, tiles = base + (uint32_t)ch.call[0].off_tiles;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = ch.n, S = ch.call[0].stages;

    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x == 0) {
        {
            [[maybe_unused]] const PinArgs & a = ch.call[0];
            PIN_STAMP(0);
        }
        pin_init_barriers(bars, base, S, kChainW);
    }
    __syncthreads();

    if (warp == kChainW) {
        // ---------------------------------------------------------------- producer (one thread)
        if (lane != 0) {
            return;
        }
        PinProd pr{0, 1, 0};
        for (int ci = 0; ci < n; ci++) {
            if (!pin_produce(ch.call[ci], ch.call[0], tiles, bars, started, pr)) {
                pin_produce_drain(bars, S, pr);
                return;
            }
        }
        return;
    }

    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        [[maybe_unused]] const PinArgs & a = ch.call[0];
        PIN_STAMP(1);
    }

    if (warp == kChainW + 1) {
        // ---------------------------------------------------------------- epilogue warp
        int rb = 0;
        uint32_t rphase = 0;
        for (int ci = 0; ci < n; ci++) {
            const PinArgs & a = ch.call[ci];
            if (!pin_epilogue<false>(a, ch.call[0], red, bars, rb, rphase)) {
                return;
            }
            __threadfence(); // this CTA's outputs of the call, before it is counted in
            __syncwarp();
            if (lane == 0) {
                const uint32_t old = atomicAdd(&g_chain_count, 1u);
                if (old == (uint32_t)n * gridDim.x - 1u) {
                    atomicExch(&g_chain_count, 0u);
                }
                PIN_STAMP(5);
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    PinRing pos{0, 0, 0, 0};
    for (int ci = 0; ci < n; ci++) {
        const PinArgs & a = ch.call[ci];
        if (ci > 0) {
            if (threadIdx.x == 0) {
                PIN_STAMP(0);
            }
            // every consumer has taken its unit of the previous call out of the pack
            asm volatile("bar.sync 1, %0;" ::"r"(32 * kChainW) : "memory");
            if (threadIdx.x == 0) { // all CTAs have stored their rows of the previous call
                const uint32_t target = (uint32_t)ci * gridDim.x;
                const long long t0 = clock64();
                for (;;) {
                    uint32_t v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(&g_chain_count) : "memory");
                    if (v >= target) {
                        break;
                    }
                    if (clock64() - t0 > kSpinCycles) {
                        atomicExch(&g_pin_status, B200Q_ETIMEOUT);
                        break;
                    }
                }
                // the bulk copies below read, through the asynchronous proxy, what other CTAs stored
                asm volatile("fence.proxy.async;" ::: "memory");
                PIN_STAMP(1);
            }
        }
        const int U = a.U;
        const int slot = (int)threadIdx.x / U, unit = (int)threadIdx.x - slot * U;
        if (!pin_activation<false>(a, ch.call[0], base, (uint32_t)ci & 1u)) {
            return;
        }
        if (ci == 0 && threadIdx.x == 0) {
            asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(started), "r"(1u) : "memory");
        }
        if (threadIdx.x == 0) {
            PIN_STAMP(2);
        }
        if (!pin_consume(a, ch.call[0], tiles, red, bars, base + (uint32_t)ch.call[0].off_pack, slot, unit, pos)) {
            return;
        }
        if (threadIdx.x == 0) {
            PIN_STAMP(4);
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------
// Consumer warps W and row slots R for U units per row: the most warps whose lane use
// R*U / (32*W) is within 4 % of the best (more warps hide more latency).  w_fixed > 0: that W.
static void pick_shape(int U, bool even_rows, int w_fixed, int & W, int & R) {
    W = 0;
    R = 0;
    if (w_fixed > 0) {
        const int r = even_rows ? (32 * w_fixed / U) & ~1 : 32 * w_fixed / U;
        if (r >= 1) {
            W = w_fixed;
            R = r;
        }
        return;
    }
    double best = -1.0;
    for (int pass = 0; pass < 2; pass++) {
        for (int w = kPinMaxW; w >= 8; w--) {
            int r = 32 * w / U;
            r = even_rows ? r & ~1 : r;
            if (r < 1) {
                continue;
            }
            const double use = (double)r * U / (32.0 * w);
            if (pass == 0) {
                best = use > best ? use : best;
            } else if (use >= best - 0.04) {
                W = w;
                R = r;
                return;
            }
        }
    }
}

static uint32_t pin_grid(const CallDev & c, const PinArgs & a, int next_mode) {
    const int steps = next_mode ? c.seg[0].n_rows / 32 : (c.total_rows + a.R - 1) / a.R; // whole groups in next mode
    return (uint32_t)(steps < kSMs ? steps : kSMs);
}

// Thread geometry of a call.  next_mode: 0 = plain call, 1 = one segment whose output is quantized
// for the next call, 2 = gate|up pairs (silu(gate)*up quantized for the next call).
static bool pin_shape(const CallDev & c, int next_mode, int w_fixed, PinArgs & a) {
    const bool paired = next_mode == 2;
    if (c.TB != 1 || (c.K & 255)) {
        return false;
    }
    const int U = c.K >> 7;
    int W, R;
    pick_shape(U, paired, w_fixed, W, R);
    if (W == 0) {
        return false;
    }
    if (paired) { // at most 32 pairs per step (the epilogue's ring holds 64), same type and rows
        R = R > 64 ? 64 : R;
        if (c.n_segs != 2 || c.seg[0].type != c.seg[1].type || c.seg[0].n_rows != c.seg[1].n_rows) {
            return false;
        }
    }
    if (next_mode == 1) { // at most 32 rows per step
        R = R > 32 ? 32 : R;
        if (c.n_segs != 1) {
            return false;
        }
    }
    int seg = 1; // lanes summed by shuffles: the largest power of two dividing U, at most a warp
    while (seg < 32 && U % (2 * seg) == 0) {
        seg *= 2;
    }
    a.W = W, a.R = R, a.U = U, a.seg = seg, a.P = U / seg;
    a.Ppad = a.P | 1; // odd row pitch: the epilogue's lanes hit distinct banks
    a.paired = paired ? 1 : 0;
    a.next_mode = next_mode;
    return true;
}

// Shared memory a call needs with R row slots: partial sums per buffer, pack, landing zone of the
// raw activation (the fp32 vector, or the three quantized views: K + K/4 + K/4 bytes), one stage.
struct PinNeed {
    size_t red, pack, xraw, half, stage;
};
static PinNeed pin_need(const CallDev & c, const PinArgs & a, bool fp32_in, int R) {
    int max_sbb = 0;
    for (int i = 0; i < c.n_segs; i++) {
        max_sbb = max_sbb > sb_bytes(c.seg[i].type) ? max_sbb : sb_bytes(c.seg[i].type);
    }
    const size_t row_max = (size_t)(c.K >> 8) * max_sbb;
    PinNeed n;
    n.red = ((size_t)R * a.Ppad * 4 + 15) / 16 * 16;
    n.pack = (size_t)a.U * kPinUnitBytes;
    n.xraw = (fp32_in ? 4 : 1) * (size_t)c.K + (fp32_in ? 0 : c.K / 2);
    n.half = ((size_t)(R / 2) * row_max + 32 + 15) / 16 * 16;
    n.stage = a.paired ? (2 * n.half + 127) / 128 * 128 : ((size_t)R * row_max + 32 + 127) / 128 * 128;
    return n;
}
static void pin_set_layout(PinArgs & a, int R, const PinNeed & n, size_t red, size_t pack, size_t xraw, size_t stage) {
    const size_t off_pack = kPinHdr + kRedBufs * red + 512; // + the epilogue's value ring
    const size_t off_xraw = (off_pack + pack + 15) / 16 * 16;
    const size_t off_tiles = (off_xraw + xraw + 127) / 128 * 128;
    const int stages = off_tiles < (size_t)kPinSmem ? (int)(((size_t)kPinSmem - off_tiles) / stage) : 0;
    a.R = R;
    a.H = a.paired ? R / 2 : R;
    a.half_off = a.paired ? (int32_t)n.half : 0;
    a.stages = stages > 8 ? 8 : stages;
    a.stage_bytes = (int32_t)stage;
    a.red_bytes = (int32_t)red;
    a.off_pack = (int32_t)off_pack;
    a.off_xraw = (int32_t)off_xraw;
    a.off_tiles = (int32_t)off_tiles;
}

static bool pin_plan(const CallDev & c, int next_mode, bool fp32_in, PinArgs & a) {
    if (!pin_shape(c, next_mode, 0, a)) {
        return false;
    }
    for (int R = a.R;; R -= a.paired ? 2 : 1) { // fewer row slots when two stages of R rows do not fit
        if (R < 1) {
            return false;
        }
        const PinNeed n = pin_need(c, a, fp32_in, R);
        pin_set_layout(a, R, n, n.red, n.pack, n.xraw, n.stage);
        if (a.stages >= 2 && n.stage < (1u << 20)) {
            break;
        }
    }
    return cost_split(c, pin_grid(c, a, next_mode), a.cost);
}

// One geometry for all calls of a chain: every call on kChainW consumer warps, the largest
// need of any call for each region, at least three stages.
static bool chain_plan(const CallDev * calls, const float * const * xq_x, const NextAct * next, int n, ChainArgs & ch) {
    if (n < 1 || n > kChainMax) {
        return false;
    }
    PinNeed need[kChainMax];
    size_t red = 0, pack = 0, xraw = 0, stage = 0;
    for (int i = 0; i < n; i++) {
        PinArgs & a = ch.call[i];
        const CallDev & c = calls[i];
        const int next_mode = next[i].x8 ? (c.n_segs == 2 ? 2 : 1) : 0;
        if (c.n_peers > 0 || !pin_shape(c, next_mode, kChainW, a)) {
            return false;
        }
        need[i] = pin_need(c, a, xq_x[i] != nullptr, a.R);
        red = red > need[i].red ? red : need[i].red;
        pack = pack > need[i].pack ? pack : need[i].pack;
        xraw = xraw > need[i].xraw ? xraw : need[i].xraw;
        stage = stage > need[i].stage ? stage : need[i].stage;
    }
    for (int i = 0; i < n; i++) {
        PinArgs & a = ch.call[i];
        pin_set_layout(a, a.R, need[i], red, pack, xraw, stage);
        if (a.stages < 3 || stage >= (1u << 20) || !cost_split(calls[i], kSMs, a.cost)) {
            return false;
        }
    }
    ch.n = n;
    return true;
}

static bool views_aligned(const CallDev & c) { // bulk copies start on 16-byte boundaries
    return ((reinterpret_cast<uintptr_t>(c.x8) | reinterpret_cast<uintptr_t>(c.xmeta) | reinterpret_cast<uintptr_t>(c.xsumq)) & 15) == 0;
}

bool pinned_supported(const CallDev & c) {
    PinArgs a;
    return views_aligned(c) && pin_plan(c, 0, false, a);
}

bool pinned_next_supported(const CallDev & c) { // one segment, or gate|up pairs
    PinArgs a;
    return views_aligned(c) && pin_plan(c, c.n_segs == 2 ? 2 : 1, true, a);
}

bool pinned_quantizes(const CallDev & c, const float * x, const float * act_up) {
    // the fused silu(x)*up form evaluates a double-precision exp per value: every CTA repeating
    // that costs more than a launch; the vector loads of the in-kernel quantizer need 16-byte alignment
    PinArgs a;
    return c.TB == 1 && !act_up && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && views_aligned(c) &&
           pin_plan(c, 0, true, a);
}

cudaError_t launch_gemv_pinned(cudaStream_t s, const CallDev & c, const float * xq_x, const NextAct * next,
                               const PeerSync * sync, const NormArgs * norm, int32_t * am_idx, float * am_val) {
    PinArgs a;
    a.c = c;
    a.xq_x = xq_x;
    a.am_idx = am_idx;
    a.am_val = am_val;
    a.norm = (norm && xq_x) ? *norm : NormArgs{nullptr, 0.0f};
    a.next = next ? *next : NextAct{nullptr, nullptr, nullptr};
    memset(&a.sync, 0, sizeof(a.sync));
    if (sync) {
        a.sync = *sync;
    }
    if (!pin_plan(c, a.next.x8 ? (c.n_segs == 2 ? 2 : 1) : 0, xq_x != nullptr, a)) {
        return cudaErrorInvalidConfiguration;
    }
#ifdef B200Q_TUNING
    if (getenv("B200Q_CHAIN1")) { // A/B: the chain kernel for single calls too (one kernel image in the stream)
        const NextAct nx = a.next;
        if (!sync && !a.norm.w) {
            return launch_gemv_chain(s, &c, &xq_x, &nx, 1);
        }
    }
    trace_slot(a, true);
#endif
    const size_t smem = (size_t)a.off_tiles + (size_t)a.stages * a.stage_bytes;
    // The variants are kernel images of their own: the plain one carries neither option.  Two large
    // images taking turns in a stream run slower than either alone (a layer whose q|k|v and gate|up
    // launches carry a norm and whose o and down launches do not: 76 us against 60), so once a
    // call with a norm has been seen in this process every launch uses the image that can do it
    // (0.35 us per layer step dearer than the plain one when no norm is given).
    static std::atomic<bool> norm_image{false};
    if (a.norm.w) {
        norm_image.store(true, std::memory_order_relaxed);
    }
    const bool with_norm = norm_image.load(std::memory_order_relaxed);
    void (*kern)(PinArgs) = gemv_pinned_kernel<false, false>;
    if (with_norm && a.am_idx) {
        kern = gemv_pinned_kernel<true, true>;
    } else if (with_norm) {
        kern = gemv_pinned_kernel<true, false>;
    } else if (a.am_idx) {
        kern = gemv_pinned_kernel<false, true>;
    }
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(kern), kPinSmem);
    if (e != cudaSuccess) {
        return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pin_grid(c, a, a.next_mode));
    cfg.blockDim = dim3((unsigned)(32 * (a.W + 2)));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

static void chain_fill(ChainArgs & ch, const CallDev * calls, const float * const * xq_x, const NextAct * next, int n,
                       bool launching = false) {
    memset(&ch, 0, sizeof(ch));
    for (int i = 0; i < n; i++) {
        ch.call[i].c = calls[i];
        ch.call[i].xq_x = xq_x[i];
        ch.call[i].next = next[i];
#ifdef B200Q_TUNING
        trace_slot(ch.call[i], launching);
#endif
    }
}

bool chain_supported(const CallDev * calls, const float * const * xq_x, const NextAct * next, int n) {
    if (n < 2 || n > kChainMax) {
        return false;
    }
    // the waits between calls need every CTA of the grid resident: one per SM
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms < kSMs) {
        return false;
    }
    ChainArgs ch;
    chain_fill(ch, calls, xq_x, next, n);
    for (int i = 0; i < n; i++) {
        if (!views_aligned(calls[i]) || (reinterpret_cast<uintptr_t>(xq_x[i]) & 15)) {
            return false;
        }
    }
    return chain_plan(calls, xq_x, next, n, ch);
}

cudaError_t launch_gemv_chain(cudaStream_t s, const CallDev * calls, const float * const * xq_x, const NextAct * next,
                              int n) {
    ChainArgs ch;
    chain_fill(ch, calls, xq_x, next, n, true);
    if (!chain_plan(calls, xq_x, next, n, ch)) {
        return cudaErrorInvalidConfiguration;
    }
    const PinArgs & a = ch.call[0];
    const size_t smem = (size_t)a.off_tiles + (size_t)a.stages * a.stage_bytes;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(gemv_chain_kernel), kPinSmem);
    if (e != cudaSuccess) {
        return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kSMs); // one CTA per SM: all resident, which the waits between calls rely on
    cfg.blockDim = dim3(32 * (kChainW + 2));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_chain_kernel, ch);
}

cudaError_t read_pin_status(int * status, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(status, g_pin_status, sizeof(int));
    if (e == cudaSuccess && clear && *status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_pin_status, &zero, sizeof(int));
        if (e == cudaSuccess) { // a chain launch that gave up may have left its count behind
            const uint32_t none = 0;
            e = cudaMemcpyToSymbol(g_chain_count, &none, sizeof(none));
        }
        if (e == cudaSuccess) { // ... and an argmax tail its key and its count
            static const unsigned long long zk[kArgmaxRows] = {};
            static const unsigned int zd[kArgmaxRows] = {};
            e = cudaMemcpyToSymbol(g_argmax_key, zk, sizeof(zk));
            e = e == cudaSuccess ? cudaMemcpyToSymbol(g_argmax_done, zd, sizeof(zd)) : e;
        }
    }
    return e;
}

} // namespace b200q

namespace b200q {
cudaError_t launch_argmax(cudaStream_t s, const float * logits, int n, int32_t * out_idx, float * out_val, int M) {
    for (int r0 = 0; r0 < M; r0 += kArgmaxRows) { // a slot per row of a launch
        const int m = M - r0 < kArgmaxRows ? M - r0 : kArgmaxRows;
        int ctas = (n + 16383) / 16384; // at least 64 values per thread
        ctas = ctas < 1 ? 1 : (ctas > kSMs ? kSMs : ctas);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)ctas, (unsigned)m);
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_kernel, logits + (size_t)r0 * n, n, out_idx + r0,
                                           out_val ? out_val + r0 : static_cast<float *>(nullptr));
        if (e != cudaSuccess) {
            return e;
        }
    }
    return cudaSuccess;
}
} // namespace b200q

#include "moe_pinned.cuh"
