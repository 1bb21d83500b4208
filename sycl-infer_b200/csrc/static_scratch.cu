// b200q_quant_gemv_static: the fused quantize + GEMV call for hosts that must not allocate.
//
// Some embedders of this library run where device allocation is off the table: an engine
// that has already handed its whole memory budget to one weight blob and one arena, a
// plugin loaded into a process whose allocator it may not touch, or a call site inside a
// recorded launch sequence where cudaMalloc is illegal.  b200q_quant_gemv needs the caller
// to supply the int8 activation scratch; this variant keeps that scratch in a fixed array
// that is part of the library image instead.  The price is a size limit and shared state.
#include <mutex>

#include "launch.h"

namespace b200q {

// One token of at most B200Q_STATIC_MAX_K values: codes, (scale, 0) pairs, two sums per
// 32-value group.  48 KB of every GPU that loads the library, held until the process exits.
constexpr size_t kStaticX8 = B200Q_STATIC_MAX_K;
constexpr size_t kStaticMeta = (B200Q_STATIC_MAX_K / 32) * 2 * sizeof(float);
constexpr size_t kStaticSum = (B200Q_STATIC_MAX_K / 32) * 2 * sizeof(int32_t);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticX8 + kStaticMeta + kStaticSum];

// In host code the array's name is only a handle for the runtime, not an address a kernel
// can use.  The device address is looked up once per device, with that device current, and
// cached; kernels receive that address as an ordinary pointer argument.
constexpr int kMaxDevices = 64;
static void * g_scratch_addr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

static int scratch_for_current_device(unsigned char ** out) {
    int dev = -1;
    B200Q_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("b200q_quant_gemv_static: device ordinal %d is outside 0..%d", dev, kMaxDevices - 1);
        return B200Q_EUNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void * p = nullptr;
        B200Q_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
        g_scratch_addr[dev] = p;
    }
    *out = static_cast<unsigned char *>(g_scratch_addr[dev]);
    return B200Q_OK;
}

} // namespace b200q

using namespace b200q;

extern "C" int b200q_quant_gemv_static(void * stream, const b200q_seg * segs, int n_segs) {
    if (!segs || n_segs < 1) {
        set_error("b200q_quant_gemv_static: segs must be non-null and n_segs >= 1");
        return B200Q_EINVAL;
    }
    if (segs[0].K > B200Q_STATIC_MAX_K) {
        set_error("b200q_quant_gemv_static: K=%d exceeds the built-in scratch (at most %d values, one token); "
                  "use b200q_quant_gemv with caller-owned scratch",
                  segs[0].K, B200Q_STATIC_MAX_K);
        return B200Q_EUNSUPPORTED;
    }
    unsigned char * base = nullptr;
    int rc = scratch_for_current_device(&base);
    if (rc != B200Q_OK) {
        return rc;
    }
    int8_t * x8 = reinterpret_cast<int8_t *>(base);
    float * xmeta = reinterpret_cast<float *>(base + kStaticX8);
    int32_t * xsumq = reinterpret_cast<int32_t *>(base + kStaticX8 + kStaticMeta);
    // The quantizer (a kernel of its own, or the GEMV's prologue) rewrites every byte of the
    // scratch the GEMV reads (K codes, K/32 scale pairs and sum pairs), so nothing left over from
    // an earlier call is ever consumed and nothing needs clearing.
    return quant_gemv_call("b200q_quant_gemv_static", (cudaStream_t)stream, segs, n_segs, 1, x8, xmeta, xsumq, nullptr);
}
