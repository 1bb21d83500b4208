// Host-side launcher declarations shared by the C-ABI translation unit.
#pragma once
#include "common.cuh"

namespace b200q {

// wait_for != nullptr: the quantizer first waits for the peers' signals (row-sharded calls)
cudaError_t launch_xq(cudaStream_t s, const float * x, const float * up, int x_stride, int up_stride, int8_t * x8,
                      float * xmeta, int32_t * xsumq, int TB, int K, bool pdl_primary,
                      const PeerSync * wait_for = nullptr);
cudaError_t read_xq_status(int * status, bool clear);
cudaError_t launch_gemv_rows(cudaStream_t s, const CallDev & call, bool pdl_secondary);
bool stream_supported(const CallDev & call);
cudaError_t launch_gemv_stream(cudaStream_t s, const CallDev & call, bool pdl_secondary);
cudaError_t read_device_status(int * status, bool clear);
// single-token kernel with the activation pinned in registers (gemv_pinned.cu)
bool pinned_supported(const CallDev & call);
bool pinned_next_supported(const CallDev & call); // a call that also emits the next call's activation
bool pinned_quantizes(const CallDev & call, const float * x, const float * act_up);
cudaError_t launch_gemv_pinned(cudaStream_t s, const CallDev & call, const float * xq_x, const NextAct * next,
                               const PeerSync * sync = nullptr, const NormArgs * norm = nullptr, int32_t * am_idx = nullptr,
                               float * am_val = nullptr);
// row argmax, lowest index among equals (argmax.cuh)
cudaError_t launch_argmax(cudaStream_t s, const float * logits, int n, int32_t * out_idx, float * out_val, int M);
// two to four dependent single-token calls in one launch (gemv_pinned.cu); xq_x[i] != nullptr: call i
// quantizes that fp32 vector itself; next[i].x8 != nullptr: call i emits the next call's activation
bool chain_supported(const CallDev * calls, const float * const * xq_x, const NextAct * next, int n);
cudaError_t launch_gemv_chain(cudaStream_t s, const CallDev * calls, const float * const * xq_x, const NextAct * next,
                              int n);
cudaError_t read_pin_status(int * status, bool clear);
// cudaFuncAttributeMaxDynamicSharedMemorySize is per device: set once per (kernel, device)
cudaError_t ensure_dynamic_smem(const void * func, int bytes);
// dump != nullptr: parity instrument, the raw int32 accumulators of token dump_t instead of outputs
cudaError_t launch_gemm_mma(cudaStream_t s, const CallDev & call, bool pdl_secondary, int32_t * dump = nullptr,
                            int dump_t = 0);
cudaError_t read_mma_status(int * status, bool clear);
// batched decode (2..32 tokens) on register-fragment int8 MMAs (gemm_frag.cu); dump as for launch_gemm_mma
bool frag_supported(const CallDev & call);
cudaError_t launch_gemm_frag(cudaStream_t s, const CallDev & call, int32_t * dump = nullptr, int dump_t = 0);
cudaError_t read_frag_status(int * status, bool clear);
cudaError_t launch_unit_dots(cudaStream_t s, const uint8_t * w, int type, int K, int n_rows, const int8_t * x8, int TB,
                             int t, int32_t * wd);
cudaError_t launch_block_dots(cudaStream_t s, const uint8_t * w, int type, int K, int n_rows, const int8_t * x8,
                              int TB, int t, int32_t * wd);

cudaError_t launch_moe_route(cudaStream_t s, const float * gate_inp, const float * x, int x_stride, int n_tok,
                             int n_embd, int n_expert, int top_k, float * logits, int32_t * ids, float * wts,
                             int32_t * off = nullptr, int32_t * pair = nullptr, int32_t * active = nullptr,
                             int32_t * n_active = nullptr);
cudaError_t launch_moe_csr(cudaStream_t s, const int32_t * ids, int n_pairs, int n_expert, int32_t * off,
                           int32_t * pair, int32_t * active, int32_t * n_active);
cudaError_t launch_moe_rows(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                            size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                            const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                            const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                            float * out, int out_stride, int fuse_silu, const NextAct * hq = nullptr);
// streaming form of the grouped expert rows (decode: a few routed tokens per expert)
bool moe_stream_supported(int type_a, int type_b, int K, int n_rows, int fuse_silu);
cudaError_t launch_moe_stream(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                              size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                              const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                              const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                              float * out, int out_stride, int fuse_silu);
// grouped expert rows on the pinned-activation kernel (moe_pinned.cuh): every routed pair as a GEMV of
// its own; hq != nullptr (gate|up only): also emits h quantized for the down launch
bool moe_pinned_supported(int type_a, int type_b, int K, int n_rows, int fuse_silu, long long n_pairs, bool want_hq);
cudaError_t launch_moe_pinned(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                              size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                              const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                              const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                              float * out, int out_stride, int fuse_silu, const NextAct * hq);
// grouped expert GEMMs on the tensor cores (gemm_mma.cu): more than a few routed tokens per expert
bool moe_mma_supported(int type_a, int type_b, int K, int n_rows, int fuse_silu);
cudaError_t launch_moe_mma(cudaStream_t s, const void * bank_a, const void * bank_b, int type_a, int type_b,
                           size_t plane_a, size_t plane_b, const int32_t * off, const int32_t * pair,
                           const int32_t * active, const int32_t * n_active, int n_act_max, const int8_t * x8,
                           const float * xmeta, const int32_t * xsumq, int TB, int top_k, int K, int n_rows,
                           float * out, int out_stride, int fuse_silu);
// which kernel launch_moe_rows picks for a shape: true = the pinned one (which can emit hq itself)
bool moe_rows_takes_pinned(int type_a, int type_b, int K, int n_rows, int fuse_silu, int TB, int top_k, int n_act_max,
                           bool want_hq = false);
cudaError_t read_moe_status(int * status, bool clear);
cudaError_t launch_moe_reduce(cudaStream_t s, const float * acc, const float * wts, int top_k, int n_tok, int n_embd,
                              int acc_stride, float * out, int out_stride);

// measurement instruments (probes.cu)
cudaError_t launch_probe_read(cudaStream_t s, const void * buf, size_t bytes, uint32_t * sink);
cudaError_t launch_probe_i8_mma(cudaStream_t s, int iters, uint32_t * sink);
cudaError_t read_probe_status(int * status, bool clear);

cudaError_t launch_peer_barrier(cudaStream_t s, uint32_t * const * flags, int world, int rank, uint32_t seq);
cudaError_t read_peer_status(int * status, bool clear);

// shared by the C-ABI translation units: validate + flatten a call, pick the GEMV kernel
int build_call(const b200q_seg * segs, int n_segs, int TB, const int8_t * x8, const float * xmeta,
               const int32_t * xsumq, CallDev & c);
cudaError_t launch_gemv(cudaStream_t s, const CallDev & c, bool pdl_secondary);
bool gemv_takes_stream(const CallDev & c);
bool gemv_takes_pinned(const CallDev & c);
int quant_gemv_call(const char * who, cudaStream_t stream, const b200q_seg * segs, int n_segs, int TB, int8_t * x8,
                    float * xmeta, int32_t * xsumq, const b200q_call_opts * opts);

} // namespace b200q
