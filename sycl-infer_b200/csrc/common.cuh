// Shared device/host helpers of the b200q kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

constexpr int kQ8_0 = B200Q_Q8_0, kQ4_K = B200Q_Q4_K, kQ5_K = B200Q_Q5_K, kQ6_K = B200Q_Q6_K,
              kIQ4_XS = B200Q_IQ4_XS;
constexpr int kWarp = 32;
constexpr int kSMs = 148; // B200: 2 dies x 74 SMs

// Bytes per 256-value superblock of each GGUF type (src/common/quant.h:12-41,292-298 of
// the reference; Q8_0 has no superblock: 8 blocks of 34 bytes) and the alignment every
// superblock has when the tensor base is 16-byte aligned.
template <int T> struct Fmt;
template <> struct Fmt<kQ4_K> { static constexpr int SB = 144, ALIGN = 16, NP = 2; };
template <> struct Fmt<kQ5_K> { static constexpr int SB = 176, ALIGN = 16, NP = 2; };
template <> struct Fmt<kQ6_K> { static constexpr int SB = 210, ALIGN = 2, NP = 4; };
template <> struct Fmt<kIQ4_XS> { static constexpr int SB = 136, ALIGN = 8, NP = 1; };
template <> struct Fmt<kQ8_0> { static constexpr int SB = 272, ALIGN = 2, NP = 1; };

__host__ __device__ inline int sb_bytes(uint32_t type) {
    switch (type) {
    case kQ4_K: return 144;
    case kQ5_K: return 176;
    case kQ6_K: return 210;
    case kIQ4_XS: return 136;
    case kQ8_0: return 272;
    default: return 0;
    }
}

// ---- f16 <-> f32 with the reference's semantics (src/common/quant.h:67-133): f32->f16
// truncates the mantissa, forms f16 subnormals by shifting, saturates to inf.
__host__ __device__ inline float h2f(uint16_t h) {
#ifdef __CUDA_ARCH__
    float f;
    asm("{.reg .b16 t; mov.b16 t, %1; cvt.f32.f16 %0, t;}" : "=f"(f) : "h"(h));
    return f; // exact for every f16 bit pattern, subnormals included
#else
    const uint32_t s = (uint32_t)(h >> 15) << 31;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, bits;
    if (e == 0) {
        if (m == 0) {
            bits = s;
        } else {
            int ex = 113;
            while (!(m & 0x400u)) {
                m <<= 1;
                ex--;
            }
            bits = s | ((uint32_t)ex << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) {
        bits = s | 0x7F800000u | (m << 13);
    } else {
        bits = s | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
#endif
}

__host__ __device__ inline uint16_t f2h_trunc(float f) {
#ifdef __CUDA_ARCH__
    const uint32_t bits = __float_as_uint(f);
#else
    uint32_t bits;
    memcpy(&bits, &f, 4);
#endif
    const uint32_t s = (bits >> 16) & 0x8000u;
    const int32_t e32 = (int32_t)((bits >> 23) & 0xFF);
    const int32_t e16 = e32 - 112;
    const uint32_t m = bits & 0x7FFFFFu;
    if (e16 >= 31) {
        return (uint16_t)(s | 0x7C00u);
    }
    if (e16 <= 0) {
        const int32_t sh = 126 - e32;
        return sh >= 32 ? (uint16_t)s : (uint16_t)(s | ((m | 0x800000u) >> sh));
    }
    return (uint16_t)(s | ((uint32_t)e16 << 10) | (m >> 13));
}

// ---- error plumbing shared by the C ABI translation units
void set_error(const char * fmt, ...);
int cuda_fail(cudaError_t e, const char * what);

#define B200Q_CUDA_OK(expr)                                                                                        \
    do {                                                                                                           \
        cudaError_t e__ = (expr);                                                                                  \
        if (e__ != cudaSuccess) {                                                                                  \
            return ::b200q::cuda_fail(e__, #expr);                                                                 \
        }                                                                                                          \
    } while (0)

// Segments of one call, passed to kernels by value (no device allocation, so launches
// stay legal inside CUDA-graph capture).
struct SegDev {
    const uint8_t * w;
    float * out;
    const float * residual;
    float alpha;
    int32_t type;
    int32_t n_rows;
    int32_t out_stride;
    int32_t row_end; // exclusive prefix sum of n_rows over the call
};

struct CallDev {
    SegDev seg[B200Q_MAX_SEGS];
    const int8_t * x8;
    const float * xmeta;
    const int32_t * xsumq;
    int32_t n_segs;
    int32_t K;
    int32_t TB;
    int32_t total_rows;
    // row-sharded calls: every output value is also stored into the same place of n_peers other
    // GPUs' mappings of the shared output arena (plain stores over NVLink, no multicast)
    int32_t n_peers;
    int64_t peer_delta[B200Q_MAX_PEERS];
};

// gate|up calls: where the quantized silu(gate)*up of the following call goes (b200q_next_act)
struct NextAct {
    int8_t * x8; // nullptr: feature off
    float * xmeta;
    int32_t * xsumq;
};

// RMSNorm folded into the in-kernel quantizer (b200q_norm); w == nullptr: off
struct NormArgs {
    const float * w;
    float eps;
};

// cross-GPU flag exchange folded into a GEMV launch (b200q_peer_sync)
struct PeerSync {
    uint32_t * flag[B200Q_MAX_PEERS + 1]; // rank p's flag array as mapped on this GPU
    int32_t world, rank;
    int32_t wait, signal;
};

#ifdef __CUDACC__
__device__ __forceinline__ void store_out(const CallDev & c, float * p, float v) {
    *p = v;
    for (int i = 0; i < c.n_peers; i++) {
        *reinterpret_cast<float *>(reinterpret_cast<char *>(p) + c.peer_delta[i]) = v;
    }
}
#endif

} // namespace b200q
