/*
 * CPU oracle for the ARCQ packed inference path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CPU
 * (PyTorch) implementation of the group-residual quantizer and of the packed
 * linear layer.  It is the checker for the CUDA kernels: tests, the smoke
 * check and the CPU-baseline leg of the benchmark may call it; the product
 * (the package and its shared library) never does.
 *
 * Parity status: PINNED against the reference run on CPU.  The reference has
 * no golden vectors of its own, so the pin is (1) a fixture generator that
 * imports the reference quantizer and packer and stores their outputs, and
 * (2) tests that compare this file against those stored outputs bit for bit.
 *
 * Reference citations use paths inside the reference project:
 *   FQ  = methods/fair_qat_framework
 *
 * Summation order.  Bit-exact codes need the same fp32 rounding as the
 * reference, whose reductions are torch CPU `sum(-1)` over `n` contiguous
 * floats.  That kernel (observed on torch 2.11, x86) works on 8-lane vectors
 * with 4 interleaved accumulators:
 *     chunk c (8 floats) of the row is added lane-wise to accumulator c % 4
 *     for the chunks of the full quads; left-over chunks go to accumulator 0;
 *     acc0 += acc1; acc0 += acc2; acc0 += acc3       (lane-wise)
 *     result = scalar tail (elements beyond the last full chunk, in order),
 *              then the 8 lanes of acc0 added one after the other.
 * `oracle_sum_f32` below is that order.  It is valid for n <= 512 (above that
 * the torch kernel adds a cascade level).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* All helper arithmetic must stay un-fused: compile with -ffp-contract=off. */

static float oracle_sum_f32(const float *x, int n) {
    float acc[4][8];
    memset(acc, 0, sizeof(acc));
    const int nvec = n / 8;
    const int quads = nvec / 4;
    for (int i = 0; i < quads; ++i)
        for (int k = 0; k < 4; ++k)
            for (int l = 0; l < 8; ++l)
                acc[k][l] = acc[k][l] + x[(i * 4 + k) * 8 + l];
    for (int c = quads * 4; c < nvec; ++c)
        for (int l = 0; l < 8; ++l)
            acc[0][l] = acc[0][l] + x[c * 8 + l];
    for (int k = 1; k < 4; ++k)
        for (int l = 0; l < 8; ++l)
            acc[0][l] = acc[0][l] + acc[k][l];
    float fin = 0.0f;
    for (int j = nvec * 8; j < n; ++j)
        fin = fin + x[j];
    for (int l = 0; l < 8; ++l)
        fin = fin + acc[0][l];
    return fin;
}

ORACLE_API int arcq_oracle_max_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API void arcq_oracle_set_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Exposed so tests can pin the summation order itself against torch. */
ORACLE_API void arcq_oracle_row_sums(const float *x, int64_t rows, int n, float *out) {
    for (int64_t r = 0; r < rows; ++r) out[r] = oracle_sum_f32(x + r * n, n);
}

/*
 * Group-residual quantizer, one shared codebook per tensor.
 * Follows FQ/quant/dcarcq.py:531-556 (ARCQPCQuantizer.forward) and
 * FQ/fair_qat/arcq_packed_linear.py:43-53 (_quantize_weight_reference):
 *   mu    = mean(x_g)
 *   r     = x_g - mu
 *   sigma = sqrt(mean(r*r) + eps)          eps inside the sqrt
 *   t     = r / sigma
 *   code  = #{ i : thresholds[i] < t }     torch.bucketize, right=False
 *   code_sum = sum(codebook[code])
 * x is [rows, cols] fp32 row-major, cols a multiple of gs, gs <= 512.
 * codes is one byte per element.  code_sum may be NULL.
 */
ORACLE_API int arcq_oracle_quantize(const float *x, int64_t rows, int64_t cols, int gs,
                                    const float *thresholds, const float *codebook, int levels,
                                    float eps, uint8_t *codes, float *mu, float *sigma,
                                    float *code_sum) {
    if (gs <= 0 || gs > 512 || cols % gs != 0 || levels < 2 || levels > 256) return -1;
    const int64_t groups = cols / gs;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        float r[512], sq[512], val[512];
        for (int64_t g = 0; g < groups; ++g) {
            const float *xg = x + row * cols + g * gs;
            uint8_t *cg = codes + row * cols + g * gs;
            const float m = oracle_sum_f32(xg, gs) / (float)gs;
            for (int j = 0; j < gs; ++j) {
                r[j] = xg[j] - m;
                sq[j] = r[j] * r[j];
            }
            const float var = oracle_sum_f32(sq, gs) / (float)gs;
            const float s = sqrtf(var + eps);
            for (int j = 0; j < gs; ++j) {
                const float t = r[j] / s;
                int c = 0;
                for (int i = 0; i < levels - 1; ++i) c += (thresholds[i] < t) ? 1 : 0;
                cg[j] = (uint8_t)c;
                val[j] = codebook[c];
            }
            mu[row * groups + g] = m;
            sigma[row * groups + g] = s;
            if (code_sum) code_sum[row * groups + g] = oracle_sum_f32(val, gs);
        }
    }
    return 0;
}

/*
 * Fake-quant reconstruction with the group mean of the code values removed
 * ("mean_preserve"), FQ/quant/dcarcq.py:556-563:
 *   x_hat = mu + sigma * (codebook[code] - mean_g(codebook[code]))
 */
ORACLE_API int arcq_oracle_dequant(const uint8_t *codes, int64_t rows, int64_t cols, int gs,
                                   const float *codebook, const float *mu, const float *sigma,
                                   float *x_hat) {
    if (gs <= 0 || gs > 512 || cols % gs != 0) return -1;
    const int64_t groups = cols / gs;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        float val[512];
        for (int64_t g = 0; g < groups; ++g) {
            const uint8_t *cg = codes + row * cols + g * gs;
            for (int j = 0; j < gs; ++j) val[j] = codebook[cg[j]];
            const float vm = oracle_sum_f32(val, gs) / (float)gs;
            const float m = mu[row * groups + g], s = sigma[row * groups + g];
            float *o = x_hat + row * cols + g * gs;
            for (int j = 0; j < gs; ++j) {
                const float th = val[j] - vm;
                const float p = s * th;
                o[j] = m + p;
            }
        }
    }
    return 0;
}

/*
 * Bit layout of packed codes, FQ/fair_qat/arcq_packed_py.py:8-78 (and
 * arcq_infer_cuda/arcq_pack_kernel.cu:8-36): code j of a row occupies bits
 * [j*bits, (j+1)*bits) of a little-endian bit stream, least significant bit
 * first inside each byte; every row starts on a byte and has
 * ceil(len*bits/8) bytes.
 */
ORACLE_API int64_t arcq_oracle_packed_cols(int64_t len, int bits) { return (len * bits + 7) / 8; }

ORACLE_API int arcq_oracle_pack(const uint8_t *codes, int64_t rows, int64_t len, int bits,
                                uint8_t *packed) {
    if (bits < 1 || bits > 8) return -1;
    const int64_t pc = arcq_oracle_packed_cols(len, bits);
    const unsigned mask = (1u << bits) - 1u;
    memset(packed, 0, (size_t)(rows * pc));
    for (int64_t r = 0; r < rows; ++r) {
        uint8_t *out = packed + r * pc;
        for (int64_t j = 0; j < len; ++j) {
            const int64_t bit = j * bits;
            const int64_t byte = bit >> 3;
            const int sh = (int)(bit & 7);
            const unsigned v = ((unsigned)codes[r * len + j] & mask) << sh;
            out[byte] |= (uint8_t)(v & 0xffu);
            if (sh + bits > 8) out[byte + 1] |= (uint8_t)((v >> 8) & 0xffu);
        }
    }
    return 0;
}

ORACLE_API int arcq_oracle_unpack(const uint8_t *packed, int64_t rows, int64_t len, int bits,
                                  uint8_t *codes) {
    if (bits < 1 || bits > 8) return -1;
    const int64_t pc = arcq_oracle_packed_cols(len, bits);
    const unsigned mask = (1u << bits) - 1u;
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t *in = packed + r * pc;
        for (int64_t j = 0; j < len; ++j) {
            const int64_t bit = j * bits;
            const int64_t byte = bit >> 3;
            const int sh = (int)(bit & 7);
            unsigned v = (unsigned)in[byte] >> sh;
            if (sh + bits > 8) v |= (unsigned)in[byte + 1] << (8 - sh);
            codes[r * len + j] = (uint8_t)(v & mask);
        }
    }
    return 0;
}

/*
 * Packed linear, code-sum decomposition, double accumulation.  Follows
 * FQ/fair_qat/arcq_infer_cuda/arcq_linear_kernel.cu:22-78:
 *   y[m,n] = bias[n] + sum_g [ gs*mu_a*mu_w
 *            + sigma_a*sigma_w*( sum_j cbA[ca_j]*cbW[cw_j] - Sa*Sw/gs ) ]
 * codes are one byte per element ([M,K] and [N,K]); stats are [M,G] / [N,G].
 */
ORACLE_API int arcq_oracle_linear_codesum(const uint8_t *ca, const float *mu_a, const float *sg_a,
                                          const float *cs_a, const uint8_t *cw, const float *mu_w,
                                          const float *sg_w, const float *cs_w, const float *cb_a,
                                          const float *cb_w, const float *bias, int64_t M, int64_t N,
                                          int64_t K, int gs, float *y) {
    if (gs <= 0 || K % gs != 0) return -1;
    const int64_t G = K / gs;
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            double acc = bias ? (double)bias[n] : 0.0;
            for (int64_t g = 0; g < G; ++g) {
                double cross = 0.0;
                const uint8_t *a = ca + m * K + g * gs, *w = cw + n * K + g * gs;
                for (int j = 0; j < gs; ++j) cross += (double)(cb_a[a[j]] * cb_w[w[j]]);
                const double mu_term = (double)gs * (double)mu_a[m * G + g] * (double)mu_w[n * G + g];
                const double res = (double)sg_a[m * G + g] * (double)sg_w[n * G + g] *
                                   (cross - (double)cs_a[m * G + g] * (double)cs_w[n * G + g] / (double)gs);
                acc += mu_term + res;
            }
            y[m * N + n] = (float)acc;
        }
    }
    return 0;
}

/*
 * Fake-quant linear, FQ/fair_qat/quant_backends.py:312-322:
 *   y = x_hat . w_hat^T + bias   on fp32 operands.
 * The reference contracts in fp32 with the BLAS library's own order; this
 * restatement accumulates in double and rounds once, which is the value the
 * reference approximates (difference ~1e-6 relative, far below the 2e-2
 * tolerance the linear output is judged with).
 */
ORACLE_API int arcq_oracle_linear_dense(const float *x_hat, const float *w_hat, const float *bias,
                                        int64_t M, int64_t N, int64_t K, float *y) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            double acc = bias ? (double)bias[n] : 0.0;
            const float *a = x_hat + m * K, *w = w_hat + n * K;
            for (int64_t k = 0; k < K; ++k) acc += (double)a[k] * (double)w[k];
            y[m * N + n] = (float)acc;
        }
    }
    return 0;
}
