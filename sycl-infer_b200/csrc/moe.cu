// Routed mixture-of-experts on raw GGUF expert planes: router, token->expert CSR, grouped
// gate|up (silu(gate)*up fused), grouped down, weighted reduction.
//
// Arithmetic follows the reference's host twins (src/backend/cpu/kernels/moe.cpp of the
// reference): router = softmax over all experts with a sequential fp32 sum, top-k by rank
// counting with ties to the lower index, weights divided by max(sum, 6.103515625e-5)
// (:72-137); experts = int8 gate/up rows on the token's quantized activation, h = silu(g)*u,
// h re-quantized per 32 values, down rows on that (:476-559); reduce = out[t] += sum_j w*acc
// with a double accumulator (:562-574).  Expert e's plane starts at bank + e*plane_bytes.
//
// Expert kernels by regime (launch_moe_rows): up to four routed tokens per expert on average, every
// routed pair as a single-token GEMV (moe_pinned.cuh; moe_stream.cu for shapes it does not take);
// more, grouped tensor-core tiles over (expert, row tile) (gemm_mma.cu); the warp-per-row kernel
// below serves what neither takes (gate and up planes of different types with many tokens).
#include "decode.cuh"
#include "launch.h"

namespace b200q {

// ---- router --------------------------------------------------------------------------------
// Logits gate_inp . x with double accumulation: one CTA per kRouteExp experts, its warps splitting
// K, up to kRouteTok tokens per pass.  Every load of a sweep is independent of the others (the
// kernel is bound by memory latency, not by the fp64 pipe), a router row is read once for all
// tokens, and an activation row once per kRouteExp experts: with a CTA per expert the 256 CTAs of
// a 256-expert router re-read the same 128 KB of activations 256 times, and that L2 traffic
// (32 MB against 2 MB of router weights) was most of the kernel's time.
constexpr int kRouteTok = 16;
constexpr int kRouteExp = 2;
__global__ void __launch_bounds__(256) moe_logits_kernel(const float * __restrict__ gate_inp, const float * __restrict__ x,
                                                         int x_stride, int n_tok, int n_embd, int n_expert,
                                                         float * __restrict__ logits) {
    // chained launch: let the next kernel start its prologue, then wait for the producers of this one's inputs
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ double part[8][kRouteExp][kRouteTok];
    const int e0 = blockIdx.x * kRouteExp, ne = min(kRouteExp, n_expert - e0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float * w = gate_inp + (size_t)e0 * n_embd;
    const bool vec = (n_embd & 3) == 0 && (x_stride & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
    const int n_vec = vec ? n_embd : 0;
    for (int t0 = 0; t0 < n_tok; t0 += kRouteTok) {
        double a[kRouteExp][kRouteTok];
#pragma unroll
        for (int j = 0; j < kRouteExp; j++) {
#pragma unroll
            for (int i = 0; i < kRouteTok; i++) {
                a[j][i] = 0.0;
            }
        }
        for (int k = 4 * threadIdx.x; k < n_vec; k += 4 * 256) {
            float4 xv[kRouteTok], wk[kRouteExp];
#pragma unroll
            for (int j = 0; j < kRouteExp; j++) {
                wk[j] = j < ne ? __ldg(reinterpret_cast<const float4 *>(w + (size_t)j * n_embd + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < kRouteTok; i++) {
                xv[i] = t0 + i < n_tok ? __ldg(reinterpret_cast<const float4 *>(x + (size_t)(t0 + i) * x_stride + k))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < kRouteExp; j++) {
                if (j < ne) { // uniform
#pragma unroll
                    for (int i = 0; i < kRouteTok; i++) { // element order k, k+1, k+2, k+3 within a thread
                        a[j][i] += (double)wk[j].x * (double)xv[i].x;
                        a[j][i] += (double)wk[j].y * (double)xv[i].y;
                        a[j][i] += (double)wk[j].z * (double)xv[i].z;
                        a[j][i] += (double)wk[j].w * (double)xv[i].w;
                    }
                }
            }
        }
        for (int k = n_vec + threadIdx.x; k < n_embd; k += 256) {
#pragma unroll
            for (int j = 0; j < kRouteExp; j++) {
                if (j < ne) {
                    const double wkj = (double)__ldg(w + (size_t)j * n_embd + k);
#pragma unroll
                    for (int i = 0; i < kRouteTok; i++) {
                        if (t0 + i < n_tok) { // uniform
                            a[j][i] += wkj * (double)__ldg(x + (size_t)(t0 + i) * x_stride + k);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kRouteExp; j++) {
#pragma unroll
            for (int i = 0; i < kRouteTok; i++) {
                for (int o = 16; o > 0; o >>= 1) {
                    a[j][i] += __shfl_xor_sync(0xFFFFFFFFu, a[j][i], o);
                }
                if (lane == 0) {
                    part[warp][j][i] = a[j][i];
                }
            }
        }
        __syncthreads();
        if (threadIdx.x < kRouteExp * kRouteTok) {
            const int j = threadIdx.x / kRouteTok, i = threadIdx.x % kRouteTok;
            if (j < ne && t0 + i < n_tok) {
                double sum = 0.0;
                for (int q = 0; q < 8; q++) { // fixed order
                    sum += part[q][j][i];
                }
                logits[(size_t)(t0 + i) * n_expert + e0 + j] = (float)sum;
            }
        }
        __syncthreads();
    }
}

// The same logits for many tokens (prefill): a 32-token x 32-expert tile per CTA, K in chunks of 32
// through shared memory, so that an activation row is read once per 32 experts instead of once per
// CTA of two.  Every output is one thread's fp64 sum of the exact products (even and odd k apart).
// float -> double conversions run at a quarter of the fp64 FMA rate on this GPU: a value is converted
// once, by the thread that stages it, and the tiles lie in shared memory as doubles, k-major, so that a
// thread's two tokens (two experts) come with one 16-byte load.
constexpr int kLogitTiledFrom = 256; // tokens from which the tiled kernel is used
constexpr int kLogitTile = 32, kLogitPitch = kLogitTile + 2; // the pad spreads a warp's 32 stores of one column
// one chunk: 32 steps of k on the doubles in shared memory, every address a constant offset
__device__ __forceinline__ void logits_chunk(const double (*xs)[kLogitPitch], const double (*ws)[kLogitPitch], int ty, int tx,
                                             double (&a00)[2], double (&a01)[2], double (&a10)[2], double (&a11)[2]) {
#pragma unroll
    for (int k = 0; k < kLogitTile; k++) {
        const double2 xv = *reinterpret_cast<const double2 *>(&xs[k][2 * ty]);
        const double2 wv = *reinterpret_cast<const double2 *>(&ws[k][2 * tx]);
        a00[k & 1] += xv.x * wv.x;
        a01[k & 1] += xv.x * wv.y;
        a10[k & 1] += xv.y * wv.x;
        a11[k & 1] += xv.y * wv.y;
    }
}
__global__ void __launch_bounds__(256) moe_logits_tiled_kernel(const float * __restrict__ gate_inp, const float * __restrict__ x,
                                                               int x_stride, int n_tok, int n_embd, int n_expert,
                                                               float * __restrict__ logits) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // two chunks of [k][token] and [k][expert] doubles: one is summed while the next is stored
    __shared__ __align__(16) double xs[2][kLogitTile][kLogitPitch], ws[2][kLogitTile][kLogitPitch];
    const int e0 = blockIdx.x * kLogitTile, t0 = blockIdx.y * kLogitTile;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4; // experts 2tx, 2tx + 1; tokens 2ty, 2ty + 1
    // two sums per output (even and odd k), added at the end: twice as many independent fp64 chains
    double a00[2] = {0.0, 0.0}, a01[2] = {0.0, 0.0}, a10[2] = {0.0, 0.0}, a11[2] = {0.0, 0.0};
    float px[4], pw[4]; // a chunk's values of this thread, in flight while an earlier chunk is summed
    auto fetch = [&](int k0) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int idx = (int)threadIdx.x + 256 * j, r = idx >> 5, k = idx & 31;
            const bool kin = k0 + k < n_embd;
            px[j] = (kin && t0 + r < n_tok) ? __ldg(x + (size_t)(t0 + r) * x_stride + k0 + k) : 0.0f;
            pw[j] = (kin && e0 + r < n_expert) ? __ldg(gate_inp + (size_t)(e0 + r) * n_embd + k0 + k) : 0.0f;
        }
    };
    auto store = [&](int b) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int idx = (int)threadIdx.x + 256 * j, r = idx >> 5, k = idx & 31;
            xs[b][k][r] = (double)px[j];
            ws[b][k][r] = (double)pw[j];
        }
    };
    fetch(0);
    store(0);
    if (kLogitTile < n_embd) {
        fetch(kLogitTile);
    }
    for (int k0 = 0; k0 < n_embd; k0 += 2 * kLogitTile) { // two chunks per round: the buffer is a constant
        __syncthreads(); // chunk k0 is stored; buffer 1's readers are done
        if (k0 + kLogitTile < n_embd) {
            store(1);
            if (k0 + 2 * kLogitTile < n_embd) {
                fetch(k0 + 2 * kLogitTile);
            }
        }
        logits_chunk(xs[0], ws[0], ty, tx, a00, a01, a10, a11);
        if (k0 + kLogitTile >= n_embd) {
            break;
        }
        __syncthreads(); // chunk k0 + 32 is stored; buffer 0's readers are done
        if (k0 + 2 * kLogitTile < n_embd) {
            store(0);
            if (k0 + 3 * kLogitTile < n_embd) {
                fetch(k0 + 3 * kLogitTile);
            }
        }
        logits_chunk(xs[1], ws[1], ty, tx, a00, a01, a10, a11);
    }
    const int ta = t0 + 2 * ty, ea = e0 + 2 * tx;
    if (ta < n_tok && ea < n_expert) {
        logits[(size_t)ta * n_expert + ea] = (float)(a00[0] + a00[1]);
    }
    if (ta < n_tok && ea + 1 < n_expert) {
        logits[(size_t)ta * n_expert + ea + 1] = (float)(a01[0] + a01[1]);
    }
    if (ta + 1 < n_tok && ea < n_expert) {
        logits[(size_t)(ta + 1) * n_expert + ea] = (float)(a10[0] + a10[1]);
    }
    if (ta + 1 < n_tok && ea + 1 < n_expert) {
        logits[(size_t)(ta + 1) * n_expert + ea + 1] = (float)(a11[0] + a11[1]);
    }
}

// ---- token -> expert CSR (one CTA) -----------------------------------------------------------
// off[e]..off[e+1] index `pair`, which lists the (token, slot) pair ids routed to expert e in
// increasing pair order; active[0..n_active) lists the experts with at least one pair.
// cnt: shared memory, 2 * (n_expert + 1) words (+ n_pairs when ids_in_smem, + a cursor per warp and
// expert for lists of more than 1024 pairs): n_expert + 1 counts ->
// their prefix; then the active flags' prefix; then the ids.
__device__ __forceinline__ void csr_build(const int32_t * ids, int n_pairs, int n_expert, int32_t * off, int32_t * pair,
                                          int32_t * active, int32_t * n_active, int ids_in_smem, int32_t * cnt) {
    int32_t * act = cnt + n_expert + 1;
    int32_t * sid = act + n_expert + 1;
    for (int e = threadIdx.x; e <= n_expert; e += blockDim.x) {
        cnt[e] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = __ldcg(ids + i); // may have been written by other CTAs of this launch
        if (ids_in_smem) {
            sid[i] = e;
        }
        if (e >= 0 && e < n_expert) {
            atomicAdd(&cnt[e + 1], 1); // integer counts: order does not matter
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) { // warp 0: inclusive scans of the counts and of the "has pairs" flags, 32 at a time
        int carry = 0, acarry = 0;
        for (int e0 = 0; e0 < n_expert; e0 += 32) {
            const int e = e0 + threadIdx.x;
            const int c = e < n_expert ? cnt[e + 1] : 0;
            int v = c, f = c > 0 ? 1 : 0;
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xFFFFFFFFu, v, o), g = __shfl_up_sync(0xFFFFFFFFu, f, o);
                if ((int)threadIdx.x >= o) {
                    v += u;
                    f += g;
                }
            }
            if (e < n_expert) {
                cnt[e + 1] = carry + v;
                act[e + 1] = acarry + f; // experts with pairs among 0..e
            }
            carry += __shfl_sync(0xFFFFFFFFu, v, 31);
            acarry += __shfl_sync(0xFFFFFFFFu, f, 31);
        }
        if (threadIdx.x == 0) {
            act[0] = 0;
            *n_active = acarry;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= n_expert; e += blockDim.x) {
        off[e] = cnt[e];
    }
    const int32_t * idv = ids_in_smem ? sid : ids;
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
        if (act[e + 1] > act[e]) {
            active[act[e]] = e; // increasing expert order
        }
    }
    if (ids_in_smem && n_pairs <= 1024) {
        // a thread per pair: its place in its expert's list is the number of earlier pairs of the
        // same expert (a uniform scan of shared memory; the same lists as the loop below)
        for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
            const int e = idv[i];
            if (e < 0 || e >= n_expert) {
                continue;
            }
            int before = 0, j = 0;
            for (; j + 4 <= i; j += 4) {
                before += (idv[j] == e) + (idv[j + 1] == e) + (idv[j + 2] == e) + (idv[j + 3] == e);
            }
            for (; j < i; j++) {
                before += idv[j] == e;
            }
            pair[cnt[e] + before] = i;
        }
        return;
    }
    // long lists: every warp takes a contiguous range of the pairs.  Pass 1 counts the range's pairs
    // per expert, a prefix over the warps turns the counts into each warp's first free place in every
    // expert's list, pass 2 fills; lanes with the same expert in one step of 32 pairs are ranked by lane.
    // Lower ranges come first and a warp walks its range upwards: the lists stay in pair order.
    const int nw = (int)blockDim.x >> 5, warp = (int)threadIdx.x >> 5, lane = (int)threadIdx.x & 31;
    int32_t * wc = sid + (ids_in_smem ? n_pairs : 0); // [nw][n_expert]
    const int span = ((n_pairs + nw - 1) / nw + 31) & ~31;
    const int lo = min(warp * span, n_pairs), hi = min(lo + span, n_pairs);
    for (int e = threadIdx.x; e < nw * n_expert; e += blockDim.x) {
        wc[e] = 0;
    }
    __syncthreads();
    for (int pass = 0; pass < 2; pass++) {
        int32_t * mine = wc + warp * n_expert;
        for (int i0 = lo; i0 < hi; i0 += 32) {
            const int i = i0 + lane;
            int e = i < hi ? (ids_in_smem ? sid[i] : __ldcg(ids + i)) : -1; // other CTAs of this launch wrote the ids
            e = (e >= 0 && e < n_expert) ? e : -1;
            const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
            const int rank = __popc(same & ((1u << lane) - 1u));
            const int base = e >= 0 ? mine[e] : 0;
            __syncwarp();
            if (e >= 0 && rank == 0) {
                mine[e] = base + __popc(same);
            }
            __syncwarp();
            if (pass == 1 && e >= 0) {
                pair[base + rank] = i;
            }
        }
        __syncthreads();
        if (pass == 0) {
            for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
                int run = cnt[e];
                for (int w = 0; w < nw; w++) {
                    const int c = wc[w * n_expert + e];
                    wc[w * n_expert + e] = run;
                    run += c;
                }
            }
            __syncthreads();
        }
    }
}

__global__ void __launch_bounds__(256) moe_csr_kernel(const int32_t * __restrict__ ids, int n_pairs, int n_expert,
                                                      int32_t * off, int32_t * pair, int32_t * active,
                                                      int32_t * n_active, int ids_in_smem) {
    // chained launch: let the next kernel start its prologue, then wait for the producers of this one's inputs
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    extern __shared__ int32_t cnt[];
    csr_build(ids, n_pairs, n_expert, off, pair, active, n_active, ids_in_smem, cnt);
}

// Softmax and top-k of one token's logits (one CTA per token); the logits come from memory.
// With `off` set, the CTA that finishes last also builds the token -> expert CSR (one launch less).
__device__ unsigned int g_route_done = 0;
#ifdef B200Q_TUNING
__device__ unsigned long long * g_route_trace = nullptr; // [CTA][16] globaltimer stamps (set by the host, A/B only)
#define ROUTE_STAMP(k)                                                                                       \
    if (threadIdx.x == 0 && g_route_trace) {                                                                 \
        unsigned long long t_;                                                                               \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                              \
        g_route_trace[blockIdx.x * 16 + (k)] = t_;                                                           \
    }
#else
#define ROUTE_STAMP(k)
#endif
__global__ void __launch_bounds__(256) moe_route_kernel(const float * __restrict__ x, int x_stride, int n_embd,
                                                        int n_expert, int top_k, float * __restrict__ logits,
                                                        int32_t * ids, float * __restrict__ wts, int32_t * off,
                                                        int32_t * pair, int32_t * active, int32_t * n_active,
                                                        int ids_in_smem) {
    // chained launch: let the next kernel start its prologue, then wait for the producers of this one's inputs
    ROUTE_STAMP(0);
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    ROUTE_STAMP(1);
    extern __shared__ __align__(16) float p[]; // n_expert probabilities, then n_expert selection flags
    int * sel = reinterpret_cast<int *>(p + n_expert);
    __shared__ float s_max, s_inv, s_den;
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    float * lg = logits + (size_t)t * n_expert;
    (void)x, (void)x_stride, (void)n_embd;
    for (int e = tid; e < n_expert; e += blockDim.x) {
        p[e] = lg[e];
    }
    __syncthreads();
    if (tid < 32) { // the maximum is exact in any order
        float mx = -3.402823466e38f;
        for (int e = tid; e < n_expert; e += 32) {
            mx = fmaxf(mx, p[e]);
        }
        for (int o = 16; o > 0; o >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        }
        if (tid == 0) {
            s_max = mx;
        }
    }
    __syncthreads();
    ROUTE_STAMP(2);
    for (int e = tid; e < n_expert; e += blockDim.x) {
        p[e] = (float)exp((double)__fsub_rn(p[e], s_max)); // one rounding: a correctly rounded expf
    }
    __syncthreads();
    ROUTE_STAMP(3);
    if (tid == 0) {
        // expert order, like the reference's sum; sixteen loads in flight ahead of the chain of adds
        float sum = 0.f;
        for (int e0 = 0; e0 < n_expert; e0 += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; j++) {
                v[j] = p[min(e0 + j, n_expert - 1)];
            }
#pragma unroll
            for (int j = 0; j < 16; j++) {
                if (e0 + j < n_expert) {
                    sum = __fadd_rn(sum, v[j]);
                }
            }
        }
        s_inv = __fdiv_rn(1.f, sum);
    }
    __syncthreads();
    ROUTE_STAMP(4);
    for (int e = tid; e < n_expert; e += blockDim.x) {
        p[e] = __fmul_rn(p[e], s_inv);
        lg[e] = p[e]; // the reference leaves the probabilities in its logits scratch
    }
    __syncthreads();
    ROUTE_STAMP(5);
    for (int e = tid; e < n_expert; e += blockDim.x) {
        // rank = experts that beat this one: larger probability, or equal and a lower index
        const float pe = p[e];
        int rank = 0;
        for (int f = 0; f < n_expert; f++) {
            const float pf = p[f];
            rank += (pf > pe) || (pf == pe && f < e);
        }
        sel[e] = rank < top_k ? rank : -1;
    }
    __syncthreads();
    ROUTE_STAMP(6);
    {
        // the sum of the selected probabilities in expert order, like the reference's accumulation:
        // every warp marks its selected experts in a mask, one thread walks the marks
        __shared__ uint32_t s_mask[8];
        float wsum = 0.f;
        for (int e0 = 0; e0 < n_expert; e0 += blockDim.x) {
            const int e = e0 + tid;
            const uint32_t m = __ballot_sync(0xFFFFFFFFu, e < n_expert && sel[e] >= 0);
            if (lane == 0) {
                s_mask[warp] = m;
            }
            __syncthreads();
            if (tid == 0) {
                for (int w = 0; w < nw; w++) {
                    for (uint32_t mm = s_mask[w]; mm; mm &= mm - 1) {
                        wsum = __fadd_rn(wsum, p[e0 + 32 * w + __ffs((int)mm) - 1]);
                    }
                }
            }
            __syncthreads();
        }
        if (tid == 0) {
            s_den = fmaxf(wsum, 6.103515625e-5f);
        }
    }
    __syncthreads();
    for (int e = tid; e < n_expert; e += blockDim.x) {
        if (sel[e] >= 0) {
            ids[(size_t)t * top_k + sel[e]] = e;
            wts[(size_t)t * top_k + sel[e]] = __fdiv_rn(p[e], s_den);
        }
    }
    ROUTE_STAMP(7);
    if (off) {
        __shared__ int s_last;
        __syncthreads(); // this CTA's ids are written
        if (tid == 0) {
            __threadfence();
            s_last = atomicAdd(&g_route_done, 1u) == gridDim.x - 1;
            if (s_last) {
                g_route_done = 0; // ready for the next launch
                __threadfence();
            }
        }
        __syncthreads();
        ROUTE_STAMP(8);
        if (s_last) {
            csr_build(ids, (int)gridDim.x * top_k, n_expert, off, pair, active, n_active, ids_in_smem,
                      reinterpret_cast<int32_t *>(p));
            __syncthreads();
            ROUTE_STAMP(9);
        }
    }
}

// ---- grouped expert rows ---------------------------------------------------------------------
constexpr int kMoeTT = 4; // pairs of one expert handled per pass over a weight row

template <int TYPE, int TT>
__device__ __forceinline__ void expert_row(const uint8_t * wrow, int nb, const ActView & a, const int (&tok)[TT],
                                           float (&acc)[TT]) {
    const int lane = threadIdx.x & 31, j = lane & 7;
    for (int b = lane >> 3; b < nb; b += 4) {
        Part<TYPE, GmemW> p;
        p.load(wrow + (size_t)b * Fmt<TYPE>::SB, j);
#pragma unroll
        for (int i = 0; i < TT; i++) {
            acc[i] += p.term(a, 8 * b, tok[i]);
        }
    }
}

template <int TT>
__device__ __forceinline__ void expert_row_any(int type, const uint8_t * wrow, int nb, const ActView & a,
                                               const int (&tok)[TT], float (&acc)[TT]) {
    switch (type) {
    case kQ4_K: expert_row<kQ4_K, TT>(wrow, nb, a, tok, acc); break;
    case kQ5_K: expert_row<kQ5_K, TT>(wrow, nb, a, tok, acc); break;
    case kQ6_K: expert_row<kQ6_K, TT>(wrow, nb, a, tok, acc); break;
    case kIQ4_XS: expert_row<kIQ4_XS, TT>(wrow, nb, a, tok, acc); break;
    default: expert_row<kQ8_0, TT>(wrow, nb, a, tok, acc); break;
    }
}

struct MoeArgs {
    const uint8_t *bank_a, *bank_b; // gate and up planes (gate|up), or down plane in bank_a
    size_t plane_a, plane_b;
    int type_a, type_b;
    const int32_t *off, *pair, *active, *n_active;
    const int8_t * x8;
    const float * xmeta;
    const int32_t * xsumq;
    int TB;         // tokens (gate|up) or pairs (down) in the activation views
    int top_k;      // gate|up: token of pair p is p / top_k; down: 0 (activation row = pair)
    int K, n_rows;  // input length, rows per expert plane
    float * out;    // h[pair*out_stride + row] or acc[pair*out_stride + row]
    int out_stride;
    int fuse_silu;  // 1: out = silu(a) * b, 0: out = a
};

__device__ __forceinline__ float silu_host_like(float g) { // x / (1 + expf(-x)), expf rounded once
    const float e = (float)exp((double)(-g));
    return __fdiv_rn(g, __fadd_rn(1.0f, e));
}

// grid.x = row blocks (8 rows each), grid.y = expert slots; one warp per row of the expert
__global__ void __launch_bounds__(256) moe_rows_kernel(const __grid_constant__ MoeArgs m) {
    const int slot = blockIdx.y;
    if (slot >= *m.n_active) {
        return;
    }
    const int e = m.active[slot];
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= m.n_rows) {
        return;
    }
    const int nb = m.K >> 8;
    const int p0 = m.off[e], p1 = m.off[e + 1];
    const ActView a{m.x8, m.xmeta, m.xsumq, m.TB};
    const uint8_t * wa = m.bank_a + (size_t)e * m.plane_a + (size_t)row * nb * sb_bytes(m.type_a);
    const uint8_t * wb = m.fuse_silu ? m.bank_b + (size_t)e * m.plane_b + (size_t)row * nb * sb_bytes(m.type_b) : nullptr;
    for (int q = p0; q < p1; q += kMoeTT) {
        int pr[kMoeTT], tok[kMoeTT];
#pragma unroll
        for (int i = 0; i < kMoeTT; i++) {
            pr[i] = m.pair[min(q + i, p1 - 1)];
            tok[i] = m.top_k > 0 ? pr[i] / m.top_k : pr[i];
        }
        float ga[kMoeTT] = {0.f, 0.f, 0.f, 0.f}, ua[kMoeTT] = {0.f, 0.f, 0.f, 0.f};
        expert_row_any<kMoeTT>(m.type_a, wa, nb, a, tok, ga);
        if (m.fuse_silu) {
            expert_row_any<kMoeTT>(m.type_b, wb, nb, a, tok, ua);
        }
#pragma unroll
        for (int i = 0; i < kMoeTT; i++) {
            ga[i] = warp_sum(ga[i]);
            ua[i] = warp_sum(ua[i]);
        }
        if (lane < kMoeTT && q + lane < p1) {
            float g = 0.f, u = 0.f;
#pragma unroll
            for (int i = 0; i < kMoeTT; i++) {
                g = lane == i ? ga[i] : g;
                u = lane == i ? ua[i] : u;
            }
            int pi = pr[0];
#pragma unroll
            for (int i = 1; i < kMoeTT; i++) {
                pi = lane == i ? pr[i] : pi;
            }
            m.out[(size_t)pi * m.out_stride + row] = m.fuse_silu ? __fmul_rn(silu_host_like(g), u) : g;
        }
    }
}

// out[t*out_stride + c] += (float) sum_j (double)w[t,j] * acc[(t*top_k + j)*acc_stride + c]
__global__ void __launch_bounds__(256) moe_reduce_kernel(const float * __restrict__ acc, const float * __restrict__ wts,
                                                         int top_k, int n_tok, int n_embd, int acc_stride, float * out,
                                                         int out_stride) {
    // chained launch: let the next kernel start its prologue, then wait for the producers of this one's inputs
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tok * n_embd) {
        return;
    }
    const int t = (int)(i / n_embd), c = (int)(i - (long long)t * n_embd);
    double a = 0.0;
    for (int j = 0; j < top_k; j++) {
        const size_t pr = (size_t)t * top_k + j;
        a += (double)wts[pr] * (double)acc[pr * (size_t)acc_stride + c];
    }
    out[(size_t)t * out_stride + c] += (float)a;
}

// ---- launchers -----------------------------------------------------------------------------------
// every launch is programmatically chained to its predecessor in the stream (the kernels wait
// for it themselves before reading its results)
template <class... KArgs, class... Args>
static cudaError_t launch_chained(cudaStream_t s, void (*k)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k, static_cast<KArgs>(args)...);
}

// Shared memory of csr_build.  Lists of up to 1024 pairs are filled by a thread per pair, which needs the
// ids in shared memory; longer lists by the warp-parallel fill (a cursor per warp and expert), with the
// ids in shared memory while that stays within the 48 KB every launch may have (beyond that - many
// experts - the ids are read from global memory; the launchers raise the kernel's limit when even the
// cursors need more).
constexpr size_t kCsrPlainSmem = 48 * 1024;
static size_t csr_smem(int n_pairs, int n_expert, int & in_smem) {
    const size_t fixed = (size_t)2 * (n_expert + 1) + (n_pairs > 1024 ? (size_t)8 * n_expert : 0);
    in_smem = n_pairs <= 8192 ? 1 : 0;
    if (n_pairs > 1024 && (fixed + n_pairs) * sizeof(int32_t) > kCsrPlainSmem) {
        in_smem = 0;
    }
    return (fixed + (in_smem ? n_pairs : 0)) * sizeof(int32_t);
}

// off != nullptr: the CSR is built by the router's last CTA
cudaError_t launch_moe_route(cudaStream_t s, const float * gate_inp, const float * x, int x_stride, int n_tok,
                             int n_embd, int n_expert, int top_k, float * logits, int32_t * ids, float * wts,
                             int32_t * off, int32_t * pair, int32_t * active, int32_t * n_active) {
    if (gate_inp) {
        // the tiled kernel's grid is (experts / 32) x (tokens / 32) CTAs, each walking all of K: below 256
        // tokens that is too few CTAs (64 tokens: 16), and the kernel of two experts per CTA is faster
        cudaError_t e = n_tok >= kLogitTiledFrom
                            ? launch_chained(s, moe_logits_tiled_kernel,
                                             dim3((unsigned)((n_expert + kLogitTile - 1) / kLogitTile), (unsigned)((n_tok + kLogitTile - 1) / kLogitTile)),
                                             dim3(256), 0, gate_inp, x, x_stride, n_tok, n_embd, n_expert, logits)
                            : launch_chained(s, moe_logits_kernel, dim3((unsigned)((n_expert + kRouteExp - 1) / kRouteExp)),
                                             dim3(256), 0, gate_inp, x, x_stride, n_tok, n_embd, n_expert, logits);
        if (e != cudaSuccess) {
            return e;
        }
    }
#ifdef B200Q_TUNING
    {
        const char * tp = getenv("B200Q_ROUTE_TRACE_PTR");
        unsigned long long * ptr = tp ? reinterpret_cast<unsigned long long *>(strtoull(tp, nullptr, 0)) : nullptr;
        cudaMemcpyToSymbolAsync(g_route_trace, &ptr, sizeof(ptr), 0, cudaMemcpyHostToDevice, s);
    }
#endif
    int in_smem = 0;
    size_t smem = (size_t)n_expert * 8;
    if (off) {
        const size_t c = csr_smem(n_tok * top_k, n_expert, in_smem);
        smem = smem > c ? smem : c;
    }
    if (smem > kCsrPlainSmem) {
        const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(moe_route_kernel), (int)smem);
        if (e != cudaSuccess) {
            return e;
        }
    }
    return launch_chained(s, moe_route_kernel, dim3((unsigned)n_tok), dim3(256), smem, x, x_stride, n_embd, n_expert, top_k,
                          logits, ids, wts, off, pair, active, n_active, in_smem);
}

cudaError_t launch_moe_csr(cudaStream_t s, const int32_t * ids, int n_pairs, int n_expert, int32_t * off,
                           int32_t * pair, int32_t * active, int32_t * n_active) {
    int in_smem = 0;
    const size_t smem = csr_smem(n_pairs, n_expert, in_smem);
    if (smem > kCsrPlainSmem) {
        const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(moe_csr_kernel), (int)smem);
        if (e != cudaSuccess) {
            return e;
        }
    }
    return launch_chained(s, moe_csr_kernel, dim3(1), dim3(256), smem, ids, n_pairs, n_expert, off, pair, active, n_active,
                          in_smem);
}

static bool moe_force_rows() { // A/B builds only: B200Q_MOE_KERNEL=rows keeps the warp-per-row kernel
#ifdef B200Q_TUNING
    static const bool on = [] {
        const char * e = getenv("B200Q_MOE_KERNEL");
        return e && strcmp(e, "rows") == 0;
    }();
    return on;
#else
    return false;
#endif
}

bool moe_rows_takes_pinned(int type_a, int type_b, int K, int n_rows, int fuse_silu, int TB, int top_k, int n_act_max,
                           bool want_hq) {
#ifdef B200Q_TUNING
    static const bool off = [] {
        const char * e = getenv("B200Q_MOE_KERNEL");
        return e && (strcmp(e, "stream") == 0 || strcmp(e, "rows") == 0);
    }();
    if (off) {
        return false;
    }
#endif
    const long long n_pairs = top_k > 0 ? (long long)TB * top_k : TB;
    return n_pairs <= 4LL * n_act_max && moe_pinned_supported(type_a, type_b, K, n_rows, fuse_silu, n_pairs, want_hq);
}

cudaError_t launch_moe_rows(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                            size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                            const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                            const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                            float * out, int out_stride, int fuse_silu, const NextAct * hq) {
    // decode (at most a few routed tokens per expert on average): every pair as a GEMV of its own on
    // the pinned-activation kernel; shapes it does not take: the streaming kernel
    const long long n_pairs = top_k > 0 ? (long long)TB * top_k : TB;
    if (moe_rows_takes_pinned(type_a, type_b, K, n_rows, fuse_silu, TB, top_k, n_act_max, hq != nullptr)) {
        return launch_moe_pinned(s, bank_a, bank_b, type_a, type_b, plane_a, plane_b, off, pair, active, n_active, n_act_max,
                                 x8, xmeta, xsumq, TB, top_k, K, n_rows, out, out_stride, fuse_silu, hq);
    }
    if (hq) { // only the pinned kernel quantizes h itself; callers ask moe_rows_takes_pinned first
        return cudaErrorInvalidConfiguration;
    }
    // more than four routed tokens per expert on average (prefill): the expert GEMMs as tensor-core tiles
    if (n_pairs > 4LL * n_act_max && !moe_force_rows() && moe_mma_supported(type_a, type_b, K, n_rows, fuse_silu)) {
        return launch_moe_mma(s, bank_a, bank_b, type_a, type_b, plane_a, plane_b, off, pair, active, n_active, n_act_max, x8,
                              xmeta, xsumq, TB, top_k, K, n_rows, out, out_stride, fuse_silu);
    }
    if (n_pairs <= 4LL * n_act_max && n_act_max <= 1023 && moe_stream_supported(type_a, type_b, K, n_rows, fuse_silu)) {
        return launch_moe_stream(s, bank_a, bank_b, type_a, type_b, plane_a, plane_b, off, pair, active, n_active, n_act_max,
                                 x8, xmeta, xsumq, TB, top_k, K, n_rows, out, out_stride, fuse_silu);
    }
    MoeArgs m;
    m.bank_a = static_cast<const uint8_t *>(bank_a);
    m.bank_b = static_cast<const uint8_t *>(bank_b);
    m.plane_a = plane_a;
    m.plane_b = plane_b;
    m.type_a = type_a;
    m.type_b = type_b;
    m.off = off;
    m.pair = pair;
    m.active = active;
    m.n_active = n_active;
    m.x8 = x8;
    m.xmeta = xmeta;
    m.xsumq = xsumq;
    m.TB = TB;
    m.top_k = top_k;
    m.K = K;
    m.n_rows = n_rows;
    m.out = out;
    m.out_stride = out_stride;
    m.fuse_silu = fuse_silu;
    const dim3 grid((unsigned)((n_rows + 7) / 8), (unsigned)n_act_max);
    moe_rows_kernel<<<grid, 256, 0, s>>>(m);
    return cudaGetLastError();
}

cudaError_t launch_moe_reduce(cudaStream_t s, const float * acc, const float * wts, int top_k, int n_tok, int n_embd,
                              int acc_stride, float * out, int out_stride) {
    const long long n = (long long)n_tok * n_embd;
    return launch_chained(s, moe_reduce_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, acc, wts, top_k, n_tok, n_embd,
                          acc_stride, out, out_stride);
}

} // namespace b200q
