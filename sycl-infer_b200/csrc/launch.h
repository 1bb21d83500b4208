// Host-side launcher declarations shared by the C-ABI translation unit.
#pragma once
#include "common.cuh"

namespace b200q {

cudaError_t launch_xq(cudaStream_t s, const float * x, const float * up, int x_stride, int up_stride, int8_t * x8,
                      float * xmeta, int32_t * xsumq, int TB, int K, bool pdl_primary);
cudaError_t launch_gemv_rows(cudaStream_t s, const CallDev & call, bool pdl_secondary);
bool stream_supported(const CallDev & call);
cudaError_t launch_gemv_stream(cudaStream_t s, const CallDev & call, bool pdl_secondary);
cudaError_t read_device_status(int * status, bool clear);
cudaError_t launch_unit_dots(cudaStream_t s, const uint8_t * w, int type, int K, int n_rows, const int8_t * x8, int TB,
                             int t, int32_t * wd);
cudaError_t launch_block_dots(cudaStream_t s, const uint8_t * w, int type, int K, int n_rows, const int8_t * x8,
                              int TB, int t, int32_t * wd);

// shared by the C-ABI translation units: validate + flatten a call, pick the GEMV kernel
int build_call(const b200q_seg * segs, int n_segs, int TB, const int8_t * x8, const float * xmeta,
               const int32_t * xsumq, CallDev & c);
cudaError_t launch_gemv(cudaStream_t s, const CallDev & c, bool pdl_secondary);

} // namespace b200q
