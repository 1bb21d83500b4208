// TEST INFRASTRUCTURE ONLY - never linked into or called from the product path.
//
// Thin extern "C" surface over the reference's own CPU implementation of the
// quantized GEMV/GEMM path.  It is compiled together with the reference's
// unmodified source files (see Makefile, target _ref/libsiref.so); nothing of
// the reference is copied here, the functions below only forward.
//
// Forwarded reference entry points (paths inside the reference project):
//   cpu_xq                 src/backend/cpu/kernels/xq.cpp:10-50
//   cpu_i8_gemv            src/backend/cpu/kernels/i8.cpp:498-516
//   cpu_i8_gemm            src/backend/cpu/kernels/i8.cpp:518-546
//   cpu_i8_gemv1_chunked   src/backend/cpu/kernels/i8.cpp:461-496
//   cpu_i8_expert_gemm     src/backend/cpu/kernels/i8.cpp:420-459
//   cpu_gemv_group         src/backend/cpu/kernels/gemv.cpp (fp32 fused path)
//   cpu_q8_0_down_grouped  src/backend/cpu/kernels/q4exp.cpp:472-484
//   cpu_moe_route          src/backend/cpu/kernels/moe.cpp:72-137
//   cpu_moe_experts_i8     src/backend/cpu/kernels/moe.cpp:476-559
//   cpu_moe_reduce         src/backend/cpu/kernels/moe.cpp:562-574
//   rmsnorm_row            src/backend/cpu/kernels/common.cpp:685-691 (sum of squares dispatched on the host ISA)
//   dequantize_row         src/common/quant.h
//   quant_row_bytes        src/common/quant.h:1177-1198
//   ggml_float_to_half / ggml_half_to_float   src/common/quant.h:67-133
#include <cstdint>
#include <cstring>

#include "cpu_types.h"
#include "kernels/common.h"
#include "common/cpu_isa.h"

using namespace si;

namespace {
cpu_gemv_seg make_seg(const void * w, uint32_t type, int K, int n_rows, const float * x, int x_stride,
                      const float * act_up, float * out, int out_stride, const float * residual, float alpha,
                      const int8_t * x8, const float * xmeta, const int32_t * xsumq) {
    cpu_gemv_seg s{};
    s.w = w;
    s.type = type;
    s.K = K;
    s.n_rows = n_rows;
    s.x = x;
    s.x_stride = x_stride;
    s.act_up = act_up;
    s.out = out;
    s.out_stride = out_stride;
    s.residual = residual;
    s.alpha = alpha;
    s.x8 = x8;
    s.xmeta = xmeta;
    s.xsumq = xsumq;
    s.i8 = true;
    return s;
}
} // namespace

extern "C" {

int siref_threads(void) {
    return cpu_thread_count();
}
void siref_set_threads(int n) {
    cpu_set_thread_count(n);
}
int siref_i8_supported_isa(void) {
    return isa().qgemv_sb != nullptr ? 1 : 0;
}

// 0 scalar, 1 AVX2, 2 AVX-512: which variant of the ISA-dispatched helpers (sum of squares) this host runs
int siref_isa(void) {
    return (int)cpu_best_isa();
}
void siref_rmsnorm_row(const float * x, const float * w, float * out, int n, float eps) {
    rmsnorm_row(x, w, out, n, eps);
}

uint16_t siref_f2h(float f) {
    return ggml_float_to_half(f);
}
float siref_h2f(uint16_t h) {
    return ggml_half_to_float(h);
}
uint64_t siref_row_bytes(uint32_t type, int64_t n) {
    return (uint64_t)quant_row_bytes(type, n);
}
void siref_dequantize_row(uint32_t type, const void * data, float * y, int64_t n) {
    dequantize_row(type, data, y, n);
}

void siref_xq(const float * x, const float * up, int x_stride, int up_stride, int8_t * x8, float * xmeta,
              int32_t * xsumq, int TB, int K) {
    cpu_xq(x, up, x_stride, up_stride, x8, xmeta, xsumq, nullptr, TB, K);
}

void siref_i8_gemv(const void * w, uint32_t type, int K, int n_rows, float * out, const float * residual, float alpha,
                   const int8_t * x8, const float * xmeta, const int32_t * xsumq) {
    cpu_gemv_seg s = make_seg(w, type, K, n_rows, nullptr, K, nullptr, out, n_rows, residual, alpha, x8, xmeta, xsumq);
    cpu_i8_gemv(s, 0);
}

void siref_i8_gemv1_chunked(const void * w, uint32_t type, int K, int n_rows, float * out, const float * residual,
                            float alpha, const int8_t * x8, const float * xmeta, const int32_t * xsumq, int n_chunks) {
    cpu_gemv_seg s = make_seg(w, type, K, n_rows, nullptr, K, nullptr, out, n_rows, residual, alpha, x8, xmeta, xsumq);
    cpu_i8_gemv1_chunked(s, n_chunks);
}

void siref_i8_gemm(const void * w, uint32_t type, int K, int n_rows, float * out, int out_stride,
                   const float * residual, float alpha, const int8_t * x8, const float * xmeta,
                   const int32_t * xsumq, int TB) {
    cpu_gemv_seg s =
        make_seg(w, type, K, n_rows, nullptr, K, nullptr, out, out_stride, residual, alpha, x8, xmeta, xsumq);
    cpu_i8_gemm(s, TB, 0);
}

void siref_i8_expert_gemm(uint32_t type, const void * w, const int8_t * x8, const float * xmeta,
                          const int32_t * xsumq, int K, int rows, int TB, float * out, int out_stride) {
    cpu_i8_expert_gemm(type, w, x8, xmeta, xsumq, K, rows, TB, out, out_stride);
}

// fp32 fused dequant GEMV of the reference (what it runs for Q8_0 / IQ4_XS on the host)
void siref_gemv_f32(const void * w, uint32_t type, int K, int n_rows, const float * x, int x_stride,
                    const float * act_up, float * out, int out_stride, const float * residual, float alpha, int TB) {
    cpu_gemv_seg s = make_seg(w, type, K, n_rows, x, x_stride, act_up, out, out_stride, residual, alpha, nullptr,
                              nullptr, nullptr);
    s.i8 = false;
    cpu_gemv_group(type, &s, 1, n_rows, TB, K / 256, 0, 0);
}

void siref_q8_0_down_grouped(const void * w, uint64_t row_bytes, const int8_t * x8, const float * xmeta,
                             const int32_t * xsumq, int xTB, int P, int N, int K, float * acc, int acc_stride) {
    cpu_q8_0_down_grouped(w, (size_t)row_bytes, x8, xmeta, xsumq, xTB, P, N, K, acc, acc_stride, nullptr);
}

void siref_moe_route(const float * x, int x_stride, const float * gate_inp, int n_tok, int n_embd, int n_expert,
                     int top_k, float * logits, int32_t * ids, float * wts) {
    cpu_moe_route(x, x_stride, gate_inp, GGML_TYPE_F32, n_tok, n_embd, n_expert, top_k, logits, ids, wts, false);
}

// gate/up of every pair of ONE token through the reference's int8 expert path.
// The reference's own down branch only knows Q5_1 / Q8_0 / its int8 store, so a
// Q8_0 down plane is what this forwards; K-quant down planes are composed by
// the caller from siref_i8_gemv1_chunked on the plane pointer.
void siref_moe_experts_i8_q8down(const void * gate, const void * up, const void * down, uint32_t gu_type,
                                 uint64_t gu_plane_bytes, uint64_t down_plane_bytes, uint64_t down_row_bytes,
                                 int n_expert, int n_embd, int n_ff, const float * x, int n_pairs,
                                 const int32_t * ids, float * acc, int acc_stride) {
    cpu_moe M{};
    M.gate_exps.data = (const char *)gate;
    M.gate_exps.type = gu_type;
    M.gate_exps.K = n_embd;
    M.gate_exps.N = n_ff;
    M.gate_exps.plane_bytes = (size_t)gu_plane_bytes;
    M.up_exps = M.gate_exps;
    M.up_exps.data = (const char *)up;
    M.down_exps.data = (const char *)down;
    M.down_exps.type = GGML_TYPE_Q8_0;
    M.down_exps.K = n_ff;
    M.down_exps.N = n_embd;
    M.down_exps.plane_bytes = (size_t)down_plane_bytes;
    M.down_raw = down;
    M.down_row_bytes = (size_t)down_row_bytes;
    M.down_type = GGML_TYPE_Q8_0;
    M.n_expert = n_expert;
    M.n_embd = n_embd;
    M.n_ff_exp = n_ff;
    cpu_moe_experts_i8(M, x, n_embd, n_pairs, ids, acc, acc_stride);
}

void siref_moe_reduce(const float * acc, const float * wts, int top_k, int n_tok, int n_embd, int acc_stride,
                      float * out, int out_stride) {
    cpu_moe_reduce(acc, wts, top_k, n_tok, n_embd, acc_stride, out, out_stride);
}

float siref_silu(float x) {
    return cpu_silu(x);
}

} // extern "C"
