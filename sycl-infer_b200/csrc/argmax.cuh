// Row argmax on the device, standalone and as the tail of the single-token GEMV (the LM head of a
// greedy decode step): the index of the largest value, the LOWEST index among equals - what the
// reference's host scan `best = 0; if (row[i] > row[best]) best = i` yields
// (src/backend/cpu/cpu_backend.cpp:117-128; device twin src/backend/gpu/kernels/mtp_argmax.cpp).
// Part of the translation unit of gemv_pinned.cu (both kernels share the words below).
//
// A candidate is packed into one 64-bit key, (order-preserving image of the value) << 32 |
// (0xFFFFFFFF - index): the largest key is the largest value and, among equal values, the lowest
// index, so partial results combine with a plain maximum in any order.  -0 counts as +0 and a NaN
// never beats anything, as under the host's `>`.
#pragma once

namespace b200q {

constexpr int kArgmaxRows = 64; // rows (or chained launches) whose keys can be in flight at once

// per row: the running key and the number of CTAs that have contributed; the last contributor
// writes the result and puts both back to zero.  One argmax at a time per device and row slot.
__device__ unsigned long long g_argmax_key[kArgmaxRows];
__device__ unsigned int g_argmax_done[kArgmaxRows];

__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t idx) {
    uint32_t u = __float_as_uint(v == 0.0f ? 0.0f : v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    if (v != v) {
        u = 0;
    }
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}
__device__ __forceinline__ void argmax_unkey(unsigned long long k, int32_t & idx, uint32_t & ord) {
    idx = (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull));
    ord = (uint32_t)(k >> 32);
}
__device__ __forceinline__ unsigned long long argmax_warp(unsigned long long k) {
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, k, o);
        k = other > k ? other : k;
    }
    return k;
}
// One thread per contributing CTA, after its stores are done: merges the CTA's key; the last of
// `n_ctas` writes idx (and val = the row's value at idx, read back) and resets the slot.
__device__ __forceinline__ void argmax_contribute(int slot, unsigned long long key, unsigned int n_ctas, const float * row,
                                                  int32_t * out_idx, float * out_val) {
    atomicMax(&g_argmax_key[slot], key);
    __threadfence();
    if (atomicAdd(&g_argmax_done[slot], 1u) == n_ctas - 1) {
        __threadfence();
        const unsigned long long k = atomicExch(&g_argmax_key[slot], 0ull);
        g_argmax_done[slot] = 0;
        int32_t idx;
        uint32_t ord;
        argmax_unkey(k, idx, ord);
        *out_idx = idx;
        if (out_val) {
            *out_val = __ldcg(row + idx);
        }
    }
}

// grid (B, M): B CTAs share a row
__global__ void __launch_bounds__(256) argmax_kernel(const float * __restrict__ logits, int n, int32_t * out_idx,
                                                     float * out_val) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.y;
    const float * row = logits + (size_t)r * n;
    const int per = (n + gridDim.x - 1) / gridDim.x;
    const int lo = blockIdx.x * per, hi = min(n, lo + per);
    float best = 0.0f;
    int bi = -1;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) { // increasing i: `>` keeps the lowest index of equals
        const float v = __ldcg(row + i);
        if (bi < 0 || v > best) {
            best = v;
            bi = i;
        }
    }
    unsigned long long k = bi >= 0 ? argmax_key(best, (uint32_t)bi) : 0ull;
    k = argmax_warp(k);
    __shared__ unsigned long long part[8];
    if ((threadIdx.x & 31) == 0) {
        part[threadIdx.x >> 5] = k;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) {
            k = part[w] > k ? part[w] : k;
        }
        argmax_contribute(r % kArgmaxRows, k, gridDim.x, row, out_idx + r, out_val ? out_val + r : nullptr);
    }
}

} // namespace b200q
