/* TEST INFRASTRUCTURE ONLY - the product path never includes, links or calls this.
 *
 * Plain-C restatement of the reference's CPU arithmetic for the quantized
 * GEMV/GEMM hot path.  Every function cites the reference lines it follows
 * (paths inside the reference project).  Parity status: PINNED - the test
 * suite checks this file against the reference's own compiled CPU code
 * (_ref/libsiref*.so) and against committed vectors generated from it.
 *
 * fp32 contract: compiled with -ffp-contract=off, every expression below is
 * evaluated in the reference's association order with one rounding per
 * operation, so results are bit-equal to the reference built with
 * -ffp-contract=off and within a few ulp per term of its default build.
 */
#ifndef B200Q_ORACLE_H
#define B200Q_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q5_K = 13, ORC_Q6_K = 14, ORC_IQ4_XS = 23 };

typedef struct orc_seg {
    const void * w;
    uint32_t type;
    int32_t K;
    int32_t n_rows;
    float * out;
    int32_t out_stride;
    const float * residual;
    float alpha;
    const int8_t * x8;
    const float * xmeta;
    const int32_t * xsumq;
} orc_seg;

uint16_t orc_f2h(float f);
float orc_h2f(uint16_t h);
size_t orc_row_bytes(uint32_t type, int64_t n);
int orc_dots_per_row(uint32_t type, int K);
void orc_dequantize_row(uint32_t type, const void * data, float * y, int64_t n);

/* rmsnorm_row (src/backend/cpu/kernels/common.cpp:685-691).  `lanes` selects the order in which the
 * reference sums the squares on a host: 1 = the portable loop, 8 = its AVX2 helper (:259-276), 16 = its
 * AVX-512 helper (:278-290, sixteen fused-multiply-add accumulators combined by halving). */
void orc_rmsnorm(const float * x, const float * w, float * out, int n, float eps, int lanes);

void orc_xq(const float * x, const float * up, int x_stride, int up_stride, int8_t * x8, float * xmeta,
            int32_t * xsumq, int TB, int K);
void orc_block_dots(uint32_t type, const void * w, int K, int n_rows, const int8_t * x8, int TB, int t,
                    int32_t * wd);
float orc_row(uint32_t type, const void * wrow, const int8_t * x8, const float * xmeta, const int32_t * xsumq,
              int TB, int t, int K);
double orc_row_abs(uint32_t type, const void * wrow, const int8_t * x8, const float * xmeta, const int32_t * xsumq,
                   int TB, int t, int K);
void orc_i8_gemm(const orc_seg * seg, int TB);
void orc_i8_gemm_abs(const orc_seg * seg, int TB, double * abs_out);

void orc_moe_route(const float * x, int x_stride, const float * gate_inp, int n_tok, int n_embd, int n_expert,
                   int top_k, float * logits, int32_t * ids, float * wts);
void orc_moe_route_logits(int n_tok, int n_expert, int top_k, float * logits, int32_t * ids, float * wts);
void orc_moe_experts_i8(const void * gate, const void * up, const void * down, uint32_t gate_type, uint32_t up_type,
                        uint32_t down_type, size_t gate_plane, size_t up_plane, size_t down_plane, int n_embd,
                        int n_ff, const float * x, int x_stride, int n_tok, int top_k, const int32_t * ids,
                        float * h_out, float * acc, int acc_stride);
void orc_moe_reduce(const float * acc, const float * wts, int top_k, int n_tok, int n_embd, int acc_stride,
                    float * out, int out_stride);

#ifdef __cplusplus
}
#endif
#endif
