// The activation quantizer's arithmetic for one 32-value group, shared by the standalone
// quantizer kernel and the chained GEMV kernel.  Bit for bit the reference's cpu_xq
// (src/backend/cpu/kernels/xq.cpp:10-50 of the reference): every fp32 operation is a single
// correctly rounded IEEE operation in the same order.
#pragma once
#include "common.cuh"

namespace b200q {

// silu(x) = x / (1 + exp(-x)); exp in double, rounded once (equals a correctly rounded expf)
__device__ __forceinline__ float silu_exact(float a) {
    const float e = (float)exp((double)(-a));
    return __fdiv_rn(a, __fadd_rn(1.0f, e));
}

// One warp, lane i holds element i.  Returns the lane's int8 code; scale (f16-truncated
// max/127) and the two 16-value code sums come back in every lane.
__device__ __forceinline__ int xq_group(float a, int lane, float & scale, int & s0, int & s1) {
    const float mx = __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(fabsf(a))));
    const float inv = mx > 0.0f ? __fdiv_rn(127.0f, mx) : 0.0f;
    const float r = fminf(127.0f, fmaxf(-127.0f, roundf(__fmul_rn(a, inv))));
    const int q = (int)r;
    s0 = __reduce_add_sync(0xFFFFFFFFu, lane < 16 ? q : 0);
    s1 = __reduce_add_sync(0xFFFFFFFFu, lane < 16 ? 0 : q);
    scale = h2f(f2h_trunc(mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 0.0f));
    return q;
}

// The same arithmetic with one THREAD per group: v[0..31] in registers, no warp-wide
// reductions (max and integer sums are exact in any order).  Returns the 32 codes packed four
// per word (element i in byte i%4 of word i/4).
__device__ __forceinline__ void xq_group_thread(const float (&v)[32], uint32_t (&codes)[8], float & scale, int & s0,
                                                int & s1) {
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        mx = fmaxf(mx, fabsf(v[i]));
    }
    const float inv = mx > 0.0f ? __fdiv_rn(127.0f, mx) : 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const float r = fminf(127.0f, fmaxf(-127.0f, roundf(__fmul_rn(v[4 * w + b], inv))));
            word |= ((uint32_t)(int)r & 0xFFu) << (8 * b);
        }
        codes[w] = word;
    }
    int a = 0, b = 0;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        a = __dp4a((int)codes[w], 0x01010101, a);
        b = __dp4a((int)codes[4 + w], 0x01010101, b);
    }
    s0 = a;
    s1 = b;
    scale = h2f(f2h_trunc(mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 0.0f));
}

} // namespace b200q
