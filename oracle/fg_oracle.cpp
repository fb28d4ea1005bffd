// CPU oracle -- TEST INFRASTRUCTURE, NOT PRODUCT (see fg_oracle.h for the parity status).
//
// Every function restates, in plain f32 C++, what the reference's generated kernels
// compute.  The generated HIP source is ordinary C++ apart from thread indices and
// shared memory (crates/fused_gpu/src/dispatch/backend/rocm/generate.rs:102-667), is
// compiled with fast-math off (rocm/mod.rs:148-156), and the IR optimiser contracts
// a*b+c to fma (kernel/optimize.rs:31-117); this file therefore uses fmaf where the
// reference's kernel body does and plain f32 operations elsewhere.
#include "fg_oracle.h"

#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr float kGeluA = 0.044715f;    // op/unary.rs:493
constexpr float kGeluB = 0.7978846f;   // op/unary.rs:494

inline float gelu_fwd(float x, float* t_out) {
    // op/unary.rs:501-587: 0.5*x * (1 + tanh(b*(x + a*x^3)))
    float xx = x * x;
    float xxx = xx * x;
    float u = kGeluB * (x + xxx * kGeluA);
    float t = std::tanh(u);
    if (t_out) *t_out = t;
    return (0.5f * x) * (1.0f + t);
}

inline float gelu_grad(float x, float t_for_x /*quirk: value used as x*/, float t) {
    // op/unary.rs:588-714: 0.5*((1+t) + (1-t^2) * x * b*(1 + 3a*x^2)); the reference feeds
    // the saved tanh where x is meant, reproduced when t_for_x != x.
    float xv = t_for_x;
    float c = kGeluA * 3.0f;
    float du = kGeluB * (1.0f + c * (xv * xv));
    float two = (1.0f + t) + (1.0f - t * t) * (xv * du);
    return 0.5f * two;
}

inline float act_fwd(int act, float z) {
    switch (act) {
        case REF_ACT_RELU: return z > 0.0f ? z : 0.0f;   // op/unary.rs:442-451 max(x, 0)
        case REF_ACT_TANH: return std::tanh(z);           // op/unary.rs:276
        case REF_ACT_GELU: return gelu_fwd(z, nullptr);
        default: return z;
    }
}

inline float act_grad(int act, float saved, int quirks) {
    switch (act) {
        case REF_ACT_RELU:
            if (quirks & REF_QUIRK_RELU_MASK_GE0) return saved >= 0.0f ? 1.0f : 0.0f;
            return saved > 0.0f ? 1.0f : 0.0f;
        case REF_ACT_TANH: return 1.0f - saved * saved;    // op/unary.rs:281-309, saved = y
        case REF_ACT_GELU: {
            float t;
            gelu_fwd(saved, &t);                            // saved = pre-activation
            if (quirks & REF_QUIRK_GELU_BWD_T) return gelu_grad(saved, t, t);
            return gelu_grad(saved, saved, t);
        }
        default: return 1.0f;
    }
}

// Register-blocked tiles, k strictly sequential, one fused multiply-add (single rounding,
// the same result as fmaf) per (i, j, k).  A tile is GEMM_MR rows by GEMM_NR columns.
constexpr uint32_t GEMM_MR = 6, GEMM_NR = 32;

// Generic / edge tile: scalar fmaf.
void gemm_tile_scalar(uint32_t ib, uint32_t jn, uint32_t K, const float* A, uint32_t lda,
                      const float* B, uint32_t ldb, float* C, uint32_t ldc) {
    float acc[GEMM_MR][GEMM_NR];
    for (uint32_t i = 0; i < ib; ++i)
        for (uint32_t j = 0; j < jn; ++j) acc[i][j] = 0.0f;
    for (uint32_t k = 0; k < K; ++k) {
        const float* b = B + (size_t)k * ldb;
        for (uint32_t i = 0; i < ib; ++i) {
            const float a = A[(size_t)i * lda + k];
            for (uint32_t j = 0; j < jn; ++j) acc[i][j] = __builtin_fmaf(a, b[j], acc[i][j]);
        }
    }
    for (uint32_t i = 0; i < ib; ++i)
        for (uint32_t j = 0; j < jn; ++j) C[(size_t)i * ldc + j] = acc[i][j];
}

// Full 6 x 32 tile with AVX-512: 2 vectors per row, 12 accumulators.
__attribute__((target("avx512f")))
void gemm_tile_avx512(uint32_t K, const float* A, uint32_t lda, const float* B, uint32_t ldb, float* C,
                      uint32_t ldc) {
    __m512 acc[GEMM_MR][2];
    for (uint32_t i = 0; i < GEMM_MR; ++i) acc[i][0] = acc[i][1] = _mm512_setzero_ps();
    for (uint32_t k = 0; k < K; ++k) {
        const float* b = B + (size_t)k * ldb;
        const __m512 b0 = _mm512_loadu_ps(b), b1 = _mm512_loadu_ps(b + 16);
        for (uint32_t i = 0; i < GEMM_MR; ++i) {
            const __m512 a = _mm512_set1_ps(A[(size_t)i * lda + k]);
            acc[i][0] = _mm512_fmadd_ps(a, b0, acc[i][0]);
            acc[i][1] = _mm512_fmadd_ps(a, b1, acc[i][1]);
        }
    }
    for (uint32_t i = 0; i < GEMM_MR; ++i) {
        _mm512_storeu_ps(C + (size_t)i * ldc, acc[i][0]);
        _mm512_storeu_ps(C + (size_t)i * ldc + 16, acc[i][1]);
    }
}

// Full 6 x 32 tile with AVX2 + FMA: two passes of 6 x 16 (2 vectors per row, 12 accumulators).
__attribute__((target("avx2,fma")))
void gemm_tile_avx2(uint32_t K, const float* A, uint32_t lda, const float* B, uint32_t ldb, float* C,
                    uint32_t ldc) {
    for (uint32_t jh = 0; jh < GEMM_NR; jh += 16) {
        __m256 acc[GEMM_MR][2];
        for (uint32_t i = 0; i < GEMM_MR; ++i) acc[i][0] = acc[i][1] = _mm256_setzero_ps();
        for (uint32_t k = 0; k < K; ++k) {
            const float* b = B + (size_t)k * ldb + jh;
            const __m256 b0 = _mm256_loadu_ps(b), b1 = _mm256_loadu_ps(b + 8);
            for (uint32_t i = 0; i < GEMM_MR; ++i) {
                const __m256 a = _mm256_broadcast_ss(A + (size_t)i * lda + k);
                acc[i][0] = _mm256_fmadd_ps(a, b0, acc[i][0]);
                acc[i][1] = _mm256_fmadd_ps(a, b1, acc[i][1]);
            }
        }
        for (uint32_t i = 0; i < GEMM_MR; ++i) {
            _mm256_storeu_ps(C + (size_t)i * ldc + jh, acc[i][0]);
            _mm256_storeu_ps(C + (size_t)i * ldc + jh + 8, acc[i][1]);
        }
    }
}

int gemm_isa() {   // 2 = AVX-512, 1 = AVX2+FMA, 0 = scalar
    static const int isa = __builtin_cpu_supports("avx512f") ? 2
                           : (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) ? 1 : 0;
    return isa;
}

void gemm_block_f32(uint32_t ib, uint32_t jn, uint32_t K, const float* A, uint32_t lda,
                    const float* B, uint32_t ldb, float* C, uint32_t ldc) {
    const int isa = gemm_isa();
    if (ib == GEMM_MR && jn == GEMM_NR && isa == 2) gemm_tile_avx512(K, A, lda, B, ldb, C, ldc);
    else if (ib == GEMM_MR && jn == GEMM_NR && isa == 1) gemm_tile_avx2(K, A, lda, B, ldb, C, ldc);
    else gemm_tile_scalar(ib, jn, K, A, lda, B, ldb, C, ldc);
}

void transpose(uint32_t R, uint32_t Cn, const float* x, float* y) {
    // y[Cn, R] = x[R, Cn]^T
#pragma omp parallel for schedule(static)
    for (int64_t rb = 0; rb < (int64_t)((R + 31) / 32); ++rb)
        for (uint32_t cb = 0; cb < Cn; cb += 32)
            for (uint32_t r = rb * 32; r < std::min<uint32_t>(R, rb * 32 + 32); ++r)
                for (uint32_t c = cb; c < std::min(Cn, cb + 32); ++c)
                    y[(size_t)c * R + r] = x[(size_t)r * Cn + c];
}

// The reference reduces a row with 256 threads: thread t folds columns t, t+256, ... and
// a shared-memory tree then halves the stride from 128 to 1 (op/softmax.rs:121-257 for max,
// :259-397 for the sum, :529-588 for the backward dot product).
template <typename F>
inline float tree256_sum(uint32_t cols, F term) {
    float part[256];
    for (uint32_t t = 0; t < 256; ++t) {
        float s = 0.0f;
        for (uint32_t c = t; c < cols; c += 256) s += term(c);
        part[t] = s;
    }
    for (uint32_t stride = 128; stride >= 1; stride >>= 1)
        for (uint32_t t = 0; t < stride; ++t) part[t] += part[t + stride];
    return part[0];
}

}  // namespace

extern "C" {

int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

void ref_gemm_f32(int transA, int transB, uint32_t M, uint32_t N, uint32_t K, const float* A,
                  const float* B, float* C, int accumulate_f64) {
    // op/matmul/mod.rs:75-101 selects the transposes for the backward edges
    // (dA = dC·B^T via transpose_b, dB = A^T·dC via transpose_a).
    std::vector<float> At, Bt;
    const float* a = A;
    const float* b = B;
    if (transA) { At.resize((size_t)M * K); transpose(K, M, A, At.data()); a = At.data(); }
    if (transB) { Bt.resize((size_t)K * N); transpose(N, K, B, Bt.data()); b = Bt.data(); }
    if (accumulate_f64) {
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < (int64_t)M; ++i) {
            std::vector<double> acc(N, 0.0);
            for (uint32_t k = 0; k < K; ++k) {
                double av = a[(size_t)i * K + k];
                const float* br = b + (size_t)k * N;
                for (uint32_t j = 0; j < N; ++j) acc[j] += av * (double)br[j];
            }
            for (uint32_t j = 0; j < N; ++j) C[(size_t)i * N + j] = (float)acc[j];
        }
        return;
    }
    const int64_t mb = (M + GEMM_MR - 1) / GEMM_MR, nb = (N + GEMM_NR - 1) / GEMM_NR;
    // Column panels outermost so that consecutive tiles reuse the same K x 32 panel of B from cache.
#pragma omp parallel for schedule(dynamic, 8) collapse(2)
    for (int64_t bj = 0; bj < nb; ++bj)
        for (int64_t bi = 0; bi < mb; ++bi) {
            uint32_t i0 = (uint32_t)bi * GEMM_MR, j0 = (uint32_t)bj * GEMM_NR;
            gemm_block_f32(std::min<uint32_t>(GEMM_MR, M - i0), std::min<uint32_t>(GEMM_NR, N - j0), K,
                           a + (size_t)i0 * K, K, b + j0, N, C + (size_t)i0 * N + j0, N);
        }
}

void ref_bias_act_fwd(uint32_t rows, uint32_t cols, const float* z, const float* bias, int act,
                      float* y, float* preact_out) {
    // add: op/binary.rs:74-234 (the build broadcasts bias[N] over rows); activations op/unary.rs.
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r)
        for (uint32_t c = 0; c < cols; ++c) {
            size_t i = (size_t)r * cols + c;
            float p = bias ? z[i] + bias[c] : z[i];
            if (preact_out) preact_out[i] = p;
            y[i] = act_fwd(act, p);
        }
}

void ref_act_bwd(uint64_t n, int act, const float* dy, const float* saved, float* dz, int quirks) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i)
        dz[i] = act == REF_ACT_NONE ? dy[i] : dy[i] * act_grad(act, saved[i], quirks);
}

void ref_colsum(uint32_t rows, uint32_t cols, const float* x, float* out) {
    // Bias gradient of a row-broadcast bias: sum over rows, accumulated in double.
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < (int64_t)cols; ++c) {
        double s = 0.0;
        for (uint32_t r = 0; r < rows; ++r) s += x[(size_t)r * cols + c];
        out[c] = (float)s;
    }
}

void ref_softmax_fwd(uint32_t rows, uint32_t cols, const float* x, float* y) {
    // op/softmax.rs:112-446.
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const float* xr = x + (size_t)r * cols;
        float* yr = y + (size_t)r * cols;
        float mx = -INFINITY;
        for (uint32_t c = 0; c < cols; ++c) mx = std::max(mx, xr[c]);   // max is order-independent
        for (uint32_t c = 0; c < cols; ++c) yr[c] = std::exp(xr[c] - mx);  // :318-347 stores e
        float sum = tree256_sum(cols, [&](uint32_t c) { return yr[c]; });
        float inv = 1.0f / sum;                                          // :408-416
        for (uint32_t c = 0; c < cols; ++c) yr[c] *= inv;                // :436 param_mul
    }
}

void ref_softmax_bwd(uint32_t rows, uint32_t cols, const float* y, const float* dy, float* dx,
                     int accumulate, int quirks) {
    // op/softmax.rs:448-688: dot = sum(dy*y); dx += y*(dy - dot).
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const float* yr = y + (size_t)r * cols;
        const float* dr = dy + (size_t)r * cols;
        float* xr = dx + (size_t)r * cols;
        float dot = tree256_sum(cols, [&](uint32_t c) { return dr[c] * yr[c]; });
        uint32_t step = (quirks & REF_QUIRK_SOFTMAX_BWD_COL0) ? 256 : 1;
        for (uint32_t c = 0; c < cols; c += step) {
            float g = yr[c] * (dr[c] - dot);
            xr[c] = accumulate ? xr[c] + g : g;
        }
    }
}

void ref_ce_loss_grad(uint32_t rows, uint32_t cols, const float* probs, const uint32_t* labels,
                      float* loss, float* grad) {
    // loss/basic_loss.rs:91-133; label read by row, compared with the column (kernel/loss.rs:92-162).
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r)
        for (uint32_t c = 0; c < cols; ++c) {
            size_t i = (size_t)r * cols + c;
            float p = probs[i];
            if (labels[r] == c) { loss[i] = -std::log(p); grad[i] = p - 1.0f; }
            else { loss[i] = 0.0f; grad[i] = p; }
        }
}

void ref_softmax_ce_fwd_bwd(uint32_t rows, uint32_t cols, const float* logits,
                            const uint32_t* labels, float grad_scale, float* loss_row,
                            float* loss_mean, float* dlogits, float* probs, uint32_t* argmax) {
    // softmax (op/softmax.rs:112-446) followed by CROSS_ENTROPY (loss/basic_loss.rs:91-133),
    // with p - onehot used directly as dlogits (the standard fused form).
    std::vector<float> lr(rows);
#pragma omp parallel
    {
        std::vector<float> p(cols);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)rows; ++r) {
            const float* xr = logits + (size_t)r * cols;
            ref_softmax_fwd(1, cols, xr, p.data());
            uint32_t am = 0;
            for (uint32_t c = 1; c < cols; ++c) if (xr[c] > xr[am]) am = c;
            if (argmax) argmax[r] = am;
            uint32_t lab = labels[r];
            lr[r] = lab < cols ? -std::log(p[lab]) : 0.0f;
            for (uint32_t c = 0; c < cols; ++c) {
                float g = (c == lab) ? p[c] - 1.0f : p[c];
                if (dlogits) dlogits[(size_t)r * cols + c] = g * grad_scale;
                if (probs) probs[(size_t)r * cols + c] = p[c];
            }
        }
    }
    double s = 0.0;
    for (uint32_t r = 0; r < rows; ++r) { s += lr[r]; if (loss_row) loss_row[r] = lr[r]; }
    if (loss_mean) *loss_mean = (float)(s / rows);
}

void ref_softmax_ce_fwd_bwd_q(uint32_t rows, uint32_t cols, const float* logits, const uint32_t* labels,
                              float grad_scale, float* loss_row, float* loss_mean, float* dlogits, float* probs,
                              uint32_t* argmax, int quirks) {
    if (!(quirks & REF_QUIRK_CE_THROUGH_SOFTMAX) || !dlogits) {
        ref_softmax_ce_fwd_bwd(rows, cols, logits, labels, grad_scale, loss_row, loss_mean, dlogits, probs, argmax);
        return;
    }
    // The reference's order: softmax forward, CROSS_ENTROPY on the probabilities (seed = p - onehot, unscaled:
    // loss/basic_loss.rs:91-133), then the softmax node's backward with that seed as dy (dispatch/mod.rs:713-718).
    std::vector<float> p((size_t)rows * cols), seed((size_t)rows * cols), unused((size_t)rows * cols);
    ref_softmax_ce_fwd_bwd(rows, cols, logits, labels, 1.0f, loss_row, loss_mean, nullptr, p.data(), argmax);
    ref_ce_loss_grad(rows, cols, p.data(), labels, unused.data(), seed.data());
    for (size_t i = 0; i < seed.size(); ++i) { seed[i] *= grad_scale; dlogits[i] = 0.0f; }
    ref_softmax_bwd(rows, cols, p.data(), seed.data(), dlogits, 0, quirks & REF_QUIRK_SOFTMAX_BWD_COL0);
    if (probs) std::memcpy(probs, p.data(), p.size() * sizeof(float));
}

void ref_mse_loss_grad(uint64_t n, const float* pred, const float* target, float grad_scale,
                       float* loss_elem, float* loss_sum, float* grad) {
    // loss/basic_loss.rs:3-27: diff = p - t; loss = diff*diff; grad = 2*diff (unreduced).
    double s = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : s)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        float d = pred[i] - target[i];
        float l = d * d;
        if (loss_elem) loss_elem[i] = l;
        if (grad) grad[i] = (2.0f * d) * grad_scale;
        s += l;
    }
    if (loss_sum) *loss_sum = (float)s;
}

void ref_bce_loss_grad(uint64_t n, const float* pred, const float* target, float grad_scale,
                       int reference_formula, float* loss_elem, float* loss_sum, float* grad) {
    // loss/basic_loss.rs:29-89.  grad = pred - target (:81-85).  The loss there is
    // (1-t)*log(1-t) - t*log(p): `one_minus_pred` is built from the target (:47-51) and the terms
    // are subtracted as term2 - term1 (:75-79).  reference_formula != 0 reproduces exactly that;
    // 0 gives the definition -(t*log(p) + (1-t)*log(1-p)).
    double s = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : s)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        const float p = pred[i], t = target[i];
        float l;
        if (reference_formula) {
            const float omt = 1.0f - t;
            l = omt * logf(omt) - t * logf(p);
        } else {
            l = -(t * logf(p) + (1.0f - t) * logf(1.0f - p));
        }
        if (loss_elem) loss_elem[i] = l;
        if (grad) grad[i] = (p - t) * grad_scale;
        s += l;
    }
    if (loss_sum) *loss_sum = (float)s;
}

void ref_sgd_step(uint64_t n, float* w, float* g, float lr, float grad_scale, int zero_grad) {
    // optim/basic_optim.rs:3-31: scaled = g*lr; w -= scaled; g = 0.
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        float gi = grad_scale == 1.0f ? g[i] : g[i] * grad_scale;
        float scaled = gi * lr;
        w[i] = w[i] - scaled;
        if (zero_grad) g[i] = 0.0f;
    }
}

void ref_adamw_step(uint64_t n, float* w, float* g, float* m, float* v, float lr, float beta1,
                    float beta2, float eps, float weight_decay, uint32_t step, float grad_scale,
                    int zero_grad) {
    // Not in the reference (optim/basic_optim.rs has SGD only): the standard decoupled form.
    const float bc1 = 1.0f - std::pow(beta1, (float)step);
    const float bc2 = 1.0f - std::pow(beta2, (float)step);
    const float inv_bc1 = 1.0f / bc1, inv_bc2 = 1.0f / bc2;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        float gi = g[i] * grad_scale;
        float mi = beta1 * m[i] + (1.0f - beta1) * gi;
        float vi = beta2 * v[i] + (1.0f - beta2) * (gi * gi);
        float mhat = mi * inv_bc1;
        float vhat = vi * inv_bc2;
        float upd = mhat / (std::sqrt(vhat) + eps) + weight_decay * w[i];
        w[i] = w[i] - lr * upd;
        m[i] = mi;
        v[i] = vi;
        if (zero_grad) g[i] = 0.0f;
    }
}

// ---- elementwise chains ------------------------------------------------------------
enum { EW_INPUT = 0, EW_CONST, EW_ADD, EW_SUB, EW_MUL, EW_DIV, EW_NEG, EW_ABS, EW_EXP, EW_LOG,
       EW_TANH, EW_RELU, EW_GELU, EW_ELU };

// Rounding to a 16-bit storage type (round to nearest even); dtype 0 = f32 = identity.
static inline float rnd(int dt, float x) {
    if (dt == 1) return (float)(_Float16)x;
    if (dt == 2) {
        uint32_t u;
        std::memcpy(&u, &x, 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) return x;            // NaN
        u += 0x7fffu + ((u >> 16) & 1u);
        u &= 0xffff0000u;
        std::memcpy(&x, &u, 4);
        return x;
    }
    return x;
}

static inline float ew_eval(int dt, const ref_ew_instr& in, const float* v, const float* const* inputs,
                            uint64_t i) {
    switch (in.op) {
        case EW_INPUT: return inputs[in.a][i];
        case EW_CONST: return rnd(dt, in.imm);
        case EW_ADD: return rnd(dt, v[in.a] + v[in.b]);                 // op/binary.rs:74
        case EW_SUB: return rnd(dt, v[in.a] - v[in.b]);                 // :449
        case EW_MUL: return rnd(dt, v[in.a] * v[in.b]);                 // :236
        case EW_DIV: return rnd(dt, v[in.a] / v[in.b]);                 // :644
        case EW_NEG: return -v[in.a];
        case EW_ABS: return std::fabs(v[in.a]);
        case EW_EXP: return rnd(dt, std::exp(v[in.a]));                 // op/unary.rs:741-756
        case EW_LOG: return rnd(dt, std::log(v[in.a]));
        case EW_TANH: return rnd(dt, std::tanh(v[in.a]));
        case EW_RELU: return v[in.a] > 0.0f ? v[in.a] : 0.0f;
        case EW_GELU: return rnd(dt, gelu_fwd(v[in.a], nullptr));
        case EW_ELU: return v[in.a] >= 0.0f ? v[in.a] : rnd(dt, std::exp(v[in.a]) - 1.0f);  // op/unary.rs:328-436
        default: return 0.0f;
    }
}

// The arrays are float; with dtype 1 (f16) or 2 (bf16) they hold values of that type and every operation's
// result is rounded to it, which is what arithmetic in the 16-bit type itself gives for + - * /
// (the reference computes f16 graphs in the storage type: crates/ferrograd/tests/nonf32.rs:10-99).
void ref_eltwise_chain_fwd_dt(int dt, uint64_t n, const ref_ew_instr* prog, int ninstr,
                              const float* const* inputs, int ninputs, float* out,
                              float* const* saved_out) {
    (void)ninputs;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        float v[64];
        for (int k = 0; k < ninstr; ++k) {
            v[k] = ew_eval(dt, prog[k], v, inputs, (uint64_t)i);
            if (saved_out && saved_out[k]) saved_out[k][i] = v[k];
        }
        out[i] = v[ninstr - 1];
    }
}

void ref_eltwise_chain_bwd_dt(int dt, uint64_t n, const ref_ew_instr* prog, int ninstr,
                              const float* const* inputs, int ninputs, const float* seed,
                              float* const* grads, int accumulate, int quirks) {
    // Reverse sweep; derivative forms from op/binary.rs (mul :344-418, sub :557-613,
    // div :752-851) and op/unary.rs.
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        float v[64], adj[64], gin[16];
        for (int k = 0; k < ninstr; ++k) { v[k] = ew_eval(dt, prog[k], v, inputs, (uint64_t)i); adj[k] = 0.0f; }
        for (int k = 0; k < ninputs; ++k) gin[k] = 0.0f;
        adj[ninstr - 1] = seed[i];
        auto R = [dt](float x) { return rnd(dt, x); };
        for (int k = ninstr - 1; k >= 0; --k) {
            const ref_ew_instr& in = prog[k];
            float g = adj[k];
            switch (in.op) {
                case EW_INPUT: gin[in.a] = R(gin[in.a] + g); break;
                case EW_ADD: adj[in.a] = R(adj[in.a] + g); adj[in.b] = R(adj[in.b] + g); break;
                case EW_SUB: adj[in.a] = R(adj[in.a] + g); adj[in.b] = R(adj[in.b] - g); break;
                case EW_MUL: { float va = v[in.a], vb = v[in.b];
                               adj[in.a] = R(adj[in.a] + R(g * vb)); adj[in.b] = R(adj[in.b] + R(g * va)); break; }
                case EW_DIV: { float va = v[in.a], vb = v[in.b];
                               adj[in.a] = R(adj[in.a] + R(g / vb));
                               adj[in.b] = R(adj[in.b] - R(R(g * va) / R(vb * vb))); break; }
                case EW_NEG: adj[in.a] = R(adj[in.a] - g); break;
                case EW_ABS: adj[in.a] = R(adj[in.a] + (v[in.a] >= 0.0f ? g : -g)); break;
                case EW_EXP: adj[in.a] = R(adj[in.a] + R(g * v[k])); break;
                case EW_LOG: adj[in.a] = R(adj[in.a] + R(g / v[in.a])); break;
                case EW_TANH: adj[in.a] = R(adj[in.a] + R(g * R(1.0f - R(v[k] * v[k])))); break;
                case EW_RELU: adj[in.a] = R(adj[in.a] + g * act_grad(REF_ACT_RELU, v[k], quirks)); break;
                case EW_GELU: adj[in.a] = R(adj[in.a] + R(g * R(act_grad(REF_ACT_GELU, v[in.a], quirks)))); break;
                case EW_ELU: adj[in.a] = R(adj[in.a] + (v[k] >= 0.0f ? g : R(g * R(v[k] + 1.0f)))); break;
                default: break;
            }
        }
        for (int k = 0; k < ninputs; ++k)
            if (grads[k]) grads[k][i] = accumulate ? R(grads[k][i] + gin[k]) : gin[k];
    }
}

void ref_eltwise_chain_fwd(uint64_t n, const ref_ew_instr* prog, int ninstr,
                           const float* const* inputs, int ninputs, float* out,
                           float* const* saved_out) {
    ref_eltwise_chain_fwd_dt(0, n, prog, ninstr, inputs, ninputs, out, saved_out);
}

void ref_eltwise_chain_bwd(uint64_t n, const ref_ew_instr* prog, int ninstr,
                           const float* const* inputs, int ninputs, const float* seed,
                           float* const* grads, int accumulate, int quirks) {
    ref_eltwise_chain_bwd_dt(0, n, prog, ninstr, inputs, ninputs, seed, grads, accumulate, quirks);
}

void ref_round_to(int dt, uint64_t n, const float* src, float* dst) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = rnd(dt, src[i]);
}

// ---- MLP training step --------------------------------------------------------------
double ref_mlp_step(int nlayers, const uint32_t* dims, uint32_t batch, int hidden_act, float** W,
                    float** b, const float* x, const void* target, int loss_kind,
                    float grad_scale, int opt_kind, float lr, float beta1, float beta2, float eps,
                    float weight_decay, uint32_t step, float** mW, float** vW, float** mb,
                    float** vb, float** gW_out, float** gb_out, float* out_copy) {
    std::vector<std::vector<float>> act(nlayers + 1), pre(nlayers);
    act[0].assign(x, x + (size_t)batch * dims[0]);
    for (int l = 0; l < nlayers; ++l) {
        size_t n = (size_t)batch * dims[l + 1];
        std::vector<float> z(n);
        act[l + 1].resize(n);
        pre[l].resize(n);
        ref_gemm_f32(0, 0, batch, dims[l + 1], dims[l], act[l].data(), W[l], z.data(), 0);
        int a = (l < nlayers - 1) ? hidden_act : REF_ACT_NONE;
        ref_bias_act_fwd(batch, dims[l + 1], z.data(), b ? b[l] : nullptr, a, act[l + 1].data(),
                         pre[l].data());
    }
    const uint32_t od = dims[nlayers];
    size_t on = (size_t)batch * od;
    if (out_copy) std::memcpy(out_copy, act[nlayers].data(), on * sizeof(float));
    std::vector<float> dz(on);
    double loss = 0.0;
    if (loss_kind == 0) {
        float s;
        ref_mse_loss_grad(on, act[nlayers].data(), (const float*)target, grad_scale, nullptr, &s,
                          dz.data());
        loss = s;
    } else {
        std::vector<float> lrow(batch);
        float mean;
        ref_softmax_ce_fwd_bwd(batch, od, act[nlayers].data(), (const uint32_t*)target, grad_scale,
                               lrow.data(), &mean, dz.data(), nullptr, nullptr);
        for (uint32_t r = 0; r < batch; ++r) loss += lrow[r];
    }
    for (int l = nlayers - 1; l >= 0; --l) {
        size_t wn = (size_t)dims[l] * dims[l + 1];
        std::vector<float> gW(wn), gb(dims[l + 1]), dprev;
        ref_gemm_f32(1, 0, dims[l], dims[l + 1], batch, act[l].data(), dz.data(), gW.data(), 0);
        ref_colsum(batch, dims[l + 1], dz.data(), gb.data());
        if (l > 0) {
            dprev.resize((size_t)batch * dims[l]);
            ref_gemm_f32(0, 1, batch, dims[l], dims[l + 1], dz.data(), W[l], dprev.data(), 0);
            const float* saved = hidden_act == REF_ACT_GELU ? pre[l - 1].data() : act[l].data();
            ref_act_bwd(dprev.size(), hidden_act, dprev.data(), saved, dprev.data(), 0);
        }
        if (gW_out && gW_out[l]) std::memcpy(gW_out[l], gW.data(), wn * sizeof(float));
        if (gb_out && gb_out[l]) std::memcpy(gb_out[l], gb.data(), dims[l + 1] * sizeof(float));
        if (opt_kind == 0) {
            ref_sgd_step(wn, W[l], gW.data(), lr, 1.0f, 1);
            if (b) ref_sgd_step(dims[l + 1], b[l], gb.data(), lr, 1.0f, 1);
        } else if (opt_kind == 1) {
            ref_adamw_step(wn, W[l], gW.data(), mW[l], vW[l], lr, beta1, beta2, eps, weight_decay,
                           step, 1.0f, 1);
            if (b) ref_adamw_step(dims[l + 1], b[l], gb.data(), mb[l], vb[l], lr, beta1, beta2, eps,
                                  weight_decay, step, 1.0f, 1);
        }
        if (l > 0) dz.swap(dprev);
    }
    return loss;
}

}  // extern "C"
