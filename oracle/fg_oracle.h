/*
 * CPU oracle for the ferrograd B200 backend -- TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A plain C++ restatement of the arithmetic that the reference's generated GPU
 * kernels perform on the hot path.  Only tests, the smoke check and the benchmark's
 * CPU-baseline leg may load this library; nothing in the product path links or
 * calls it.
 *
 * Parity status.  The reference cannot be built or run here (Rust + HIP/wgpu), so
 * the oracle is pinned by the closed-form known answers of the reference's own
 * tests (crates/ferrograd/tests/std_wgsl.rs, tests/optim.rs): matmul forward/dA/dB,
 * softmax forward, elementwise mul/add forward+backward and the SGD update.
 * PARITY UNPINNED (no reference test or golden vector exists): AdamW (absent from
 * the reference), the CE and MSE loss kernels, tanh/relu/gelu forward and backward,
 * softmax backward with non-zero gradients, and bias broadcast.  For those the
 * oracle follows the cited source lines, or the standard definition where the
 * reference is absent or wrong (each such place has a REF_QUIRK_* switch that reproduces
 * the reference), and every function is compared with an independent float64 formula on
 * random inputs (tests/test_oracle_crosscheck.py).
 */
#ifndef FG_ORACLE_H
#define FG_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { REF_ACT_NONE = 0, REF_ACT_RELU = 1, REF_ACT_TANH = 2, REF_ACT_GELU = 3 };

/* Quirk switches: reproduce the reference's behaviour where it differs from the
 * standard definition.  0 everywhere = standard maths. */
enum {
    REF_QUIRK_RELU_MASK_GE0 = 1,  /* relu backward mask is saved_output >= 0 (op/unary.rs:453-472) */
    REF_QUIRK_GELU_BWD_T = 2,     /* gelu backward uses t = tanh(u) where x is meant (op/unary.rs:588-714) */
    REF_QUIRK_SOFTMAX_BWD_COL0 = 4,/* softmax backward updates only columns = 0 mod 256 (op/softmax.rs:601) */
    REF_QUIRK_CE_THROUGH_SOFTMAX = 8 /* the loss kernel's p - onehot is used as dL/dprobs and pushed through the
                                        softmax backward once more: the seed written by dispatch_loss
                                        (crates/fused_gpu/src/dispatch/mod.rs:713-718) is the upstream gradient of
                                        the graph's last node, the softmax (op/softmax.rs:448-688) */
};

int ref_num_threads(void);
void ref_set_num_threads(int n);

/* C = op(A)·op(B), f32, one fmaf per k in increasing k (op/matmul/generic.rs:98-319).
 * accumulate_f64 != 0 instead accumulates in double and rounds once. */
void ref_gemm_f32(int transA, int transB, uint32_t M, uint32_t N, uint32_t K,
                  const float* A, const float* B, float* C, int accumulate_f64);
void ref_bias_act_fwd(uint32_t rows, uint32_t cols, const float* z, const float* bias,
                      int act, float* y, float* preact_out);
void ref_act_bwd(uint64_t n, int act, const float* dy, const float* saved, float* dz, int quirks);
void ref_colsum(uint32_t rows, uint32_t cols, const float* x, float* out);

void ref_softmax_fwd(uint32_t rows, uint32_t cols, const float* x, float* y);
void ref_softmax_bwd(uint32_t rows, uint32_t cols, const float* y, const float* dy,
                     float* dx, int accumulate, int quirks);
void ref_ce_loss_grad(uint32_t rows, uint32_t cols, const float* probs, const uint32_t* labels,
                      float* loss, float* grad);
void ref_softmax_ce_fwd_bwd(uint32_t rows, uint32_t cols, const float* logits,
                            const uint32_t* labels, float grad_scale, float* loss_row,
                            float* loss_mean, float* dlogits, float* probs, uint32_t* argmax);
/* The same with quirk switches (REF_QUIRK_CE_THROUGH_SOFTMAX, REF_QUIRK_SOFTMAX_BWD_COL0). */
void ref_softmax_ce_fwd_bwd_q(uint32_t rows, uint32_t cols, const float* logits,
                              const uint32_t* labels, float grad_scale, float* loss_row,
                              float* loss_mean, float* dlogits, float* probs, uint32_t* argmax, int quirks);
void ref_mse_loss_grad(uint64_t n, const float* pred, const float* target, float grad_scale,
                       float* loss_elem, float* loss_sum, float* grad);
void ref_bce_loss_grad(uint64_t n, const float* pred, const float* target, float grad_scale,
                       int reference_formula, float* loss_elem, float* loss_sum, float* grad);

void ref_sgd_step(uint64_t n, float* w, float* g, float lr, float grad_scale, int zero_grad);
void ref_adamw_step(uint64_t n, float* w, float* g, float* m, float* v, float lr, float beta1,
                    float beta2, float eps, float weight_decay, uint32_t step, float grad_scale,
                    int zero_grad);

/* Elementwise chains: same program encoding as the product's fg_ew_instr. */
typedef struct ref_ew_instr { int32_t op, a, b; float imm; } ref_ew_instr;
void ref_eltwise_chain_fwd(uint64_t n, const ref_ew_instr* prog, int ninstr,
                           const float* const* inputs, int ninputs, float* out,
                           float* const* saved_out);
void ref_eltwise_chain_bwd(uint64_t n, const ref_ew_instr* prog, int ninstr,
                           const float* const* inputs, int ninputs, const float* seed,
                           float* const* grads, int accumulate, int quirks);
/* The same with 16-bit storage semantics: dt 0 = f32, 1 = f16, 2 = bf16.  Arrays stay float and hold
 * values of that type; every operation's result is rounded to it. */
void ref_eltwise_chain_fwd_dt(int dt, uint64_t n, const ref_ew_instr* prog, int ninstr,
                              const float* const* inputs, int ninputs, float* out,
                              float* const* saved_out);
void ref_eltwise_chain_bwd_dt(int dt, uint64_t n, const ref_ew_instr* prog, int ninstr,
                              const float* const* inputs, int ninputs, const float* seed,
                              float* const* grads, int accumulate, int quirks);
void ref_round_to(int dt, uint64_t n, const float* src, float* dst);

/* One training step of a dense MLP, composed in the reference's order
 * forward -> loss -> backward -> update (examples/save_load_model.rs:148-156).
 * dims[0..nlayers] are the layer widths, W[l] is [dims[l], dims[l+1]], b[l] is
 * [dims[l+1]].  loss_kind 0 = MSE (target f32 [batch, dims[nlayers]]), 1 = softmax-CE
 * (target = u32 labels).  opt_kind 0 = SGD, 1 = AdamW (m/v arrays per tensor).
 * grad_scale multiplies dL/dout (e.g. 1/batch).  Returns the summed loss. */
double ref_mlp_step(int nlayers, const uint32_t* dims, uint32_t batch, int hidden_act,
                    float** W, float** b, const float* x, const void* target, int loss_kind,
                    float grad_scale, int opt_kind, float lr, float beta1, float beta2,
                    float eps, float weight_decay, uint32_t step, float** mW, float** vW,
                    float** mb, float** vb, float** gW_out, float** gb_out, float* out_copy);

#ifdef __cplusplus
}
#endif
#endif
