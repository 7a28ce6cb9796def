/* TEST INFRASTRUCTURE ONLY — plain-C restatement of the reference's CPU kernels on the decoder path, with the
 * reference's own evaluation order (sequential sums in the storage type), so results can be compared with the
 * reference's unmodified kernels bit for bit where those exist.  Built by `make -C oracle port` into
 * oracle/librg_oracle.so.  Only tests, the smoke check and the benchmark's CPU-baseline leg load it.
 * File:line citations are relative to the reference repository root.
 *
 * Pinned against the reference's test vectors: rms_norm, softmax_asbuilt, mat_mul, gather.
 * PARITY UNPINNED (no reference implementation exists): softmax_intended on non-constant rows, attention,
 * rope, topk. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* RmsNormalizationCpu, src/04kernel/src/kernels/rms_normalization/cpu_kernel.cc:47-64 (T = float):
 * ss accumulated left to right in float; "1. / std::sqrt(ss)" is evaluated in double and stored to float. */
void oracle_rms_norm_f32(const float *x, const float *w, float *y, size_t rows, size_t dim, float eps) {
    for (size_t i = 0; i < rows; ++i) {
        const float *xr = x + i * dim;
        float *yr = y + i * dim;
        float ss = 0.f;
        for (size_t j = 0; j < dim; ++j) ss = ss + xr[j] * xr[j];
        ss /= (float) dim;
        ss += eps;
        ss = (float) (1. / sqrtf(ss));
        for (size_t j = 0; j < dim; ++j) yr[j] = xr[j] * ss * w[j];
    }
}

/* SoftmaxCpu as built, src/04kernel/src/kernels/softmax/cpu_kernel.cc:34-57 (T = float): the accumulator of
 * std::accumulate is an int (init literal 0), so every partial sum is truncated toward zero. */
void oracle_softmax_asbuilt_f32(const float *x, float *y, size_t pre, size_t mid, size_t post) {
    for (size_t i = 0; i < pre * post; ++i) {
        const size_t id = (i - i % post) * mid + i % post;
        size_t maxi = 0;
        for (size_t j = 1; j < mid; ++j)
            if (x[id + maxi * post] < x[id + j * post]) maxi = j;
        const float mx = x[id + maxi * post];
        int acc = 0;
        for (size_t j = 0; j < mid; ++j) {
            const size_t k = id + j * post;
            y[k] = expf(x[k] - mx);
            acc = (int) ((float) acc + y[k]);
        }
        for (size_t j = 0; j < mid; ++j) y[id + j * post] /= (float) acc;
    }
}

/* The same kernel with the accumulator seeded T(0): what the reference's CUDA kernels compute
 * (src/04kernel/src/kernels/softmax/cuda_kernel.cu:29-56). */
void oracle_softmax_intended_f32(const float *x, float *y, size_t pre, size_t mid, size_t post) {
    for (size_t i = 0; i < pre * post; ++i) {
        const size_t id = (i - i % post) * mid + i % post;
        float mx = x[id];
        for (size_t j = 1; j < mid; ++j)
            if (mx < x[id + j * post]) mx = x[id + j * post];
        float acc = 0.f;
        for (size_t j = 0; j < mid; ++j) {
            const size_t k = id + j * post;
            y[k] = expf(x[k] - mx);
            acc += y[k];
        }
        for (size_t j = 0; j < mid; ++j) y[id + j * post] /= acc;
    }
}

/* MatMulCPUMetaData::matrixMultiply, src/04kernel/src/kernels/mat_mul_common/cpu_template.hpp:18-30, one
 * [m,k]x[k,n] product with the strides of cpu_kernel.cc:41-44; y must already hold the broadcast bias when
 * beta != 0 (cpu_kernel.cc:36). */
void oracle_mat_mul_f32(const float *a, const float *b, float *y, size_t M, size_t K, size_t N, int trans_a,
                        int trans_b, float alpha, float beta) {
    const size_t sa0 = trans_a ? 1 : K, sa1 = trans_a ? M : 1;
    const size_t sb0 = trans_b ? 1 : N, sb1 = trans_b ? K : 1;
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; ++j) {
            float sum = 0;
            for (size_t k = 0; k < K; ++k) sum += a[i * sa0 + k * sa1] * b[k * sb0 + j * sb1];
            y[i * N + j] = beta * y[i * N + j] + alpha * sum;
        }
}

/* GatherCpu, src/04kernel/src/kernels/gather/cpu_kernel.cc:29-40. idx64 != 0: int64 indices, else int32. */
void oracle_gather(const uint8_t *data, const void *idx, int idx64, uint8_t *out, size_t prefix, size_t mid_in,
                   size_t mid_out, size_t postfix) {
    for (size_t i = 0; i < prefix * mid_out; ++i) {
        const size_t quot = i / mid_out, rem = i % mid_out;
        const int64_t k = idx64 ? ((const int64_t *) idx)[rem] : ((const int32_t *) idx)[rem];
        const int64_t q = k >= 0 ? (int64_t) quot : (int64_t) quot + 1;
        memcpy(out + postfix * i, data + postfix * (size_t) (q * (int64_t) mid_in + k), postfix);
    }
}

/* ---- definitions with no reference implementation (parity unpinned) ------------------------------------ */

/* x[tokens, heads, D]: rotate-half pairing (i, i + D/2), angle = pos * theta^(-2i/D). */
void oracle_rope_f32(const float *x, const int64_t *pos, float *y, size_t tokens, size_t heads, size_t D,
                     float theta) {
    const size_t half = D / 2;
    for (size_t t = 0; t < tokens; ++t)
        for (size_t h = 0; h < heads; ++h) {
            const float *xr = x + (t * heads + h) * D;
            float *yr = y + (t * heads + h) * D;
            for (size_t i = 0; i < half; ++i) {
                const double ang = (double) pos[t] * pow((double) theta, -2.0 * (double) i / (double) D);
                const double cs = cos(ang), sn = sin(ang);
                yr[i] = (float) (xr[i] * cs - xr[i + half] * sn);
                yr[i + half] = (float) (xr[i + half] * cs + xr[i] * sn);
            }
        }
}

/* Attention per the operator spec src/08-01llm/README.md:29-63: q[N,nH,S,D]; K,V[N,nKV,kv_tokens,D] already
 * holding the new keys at [past, past+S); row i sees j <= past+i. */
void oracle_attention_f32(const float *q, const float *K, const float *V, float *o, size_t N, size_t nH,
                          size_t nKV, size_t S, size_t D, size_t kv_tokens, size_t past) {
    const size_t rep = nH / nKV;
    const double scale = 1.0 / sqrt((double) D);
    double *p = (double *) malloc(sizeof(double) * (past + S));
    for (size_t n = 0; n < N; ++n)
        for (size_t h = 0; h < nH; ++h) {
            const float *Kb = K + (n * nKV + h / rep) * kv_tokens * D;
            const float *Vb = V + (n * nKV + h / rep) * kv_tokens * D;
            for (size_t i = 0; i < S; ++i) {
                const float *qr = q + ((n * nH + h) * S + i) * D;
                float *orow = o + ((n * nH + h) * S + i) * D;
                const size_t L = past + i + 1;
                double mx = -INFINITY;
                for (size_t j = 0; j < L; ++j) {
                    double d = 0;
                    for (size_t e = 0; e < D; ++e) d += (double) qr[e] * Kb[j * D + e];
                    p[j] = d * scale;
                    if (p[j] > mx) mx = p[j];
                }
                double sum = 0;
                for (size_t j = 0; j < L; ++j) {
                    p[j] = exp(p[j] - mx);
                    sum += p[j];
                }
                for (size_t e = 0; e < D; ++e) {
                    double acc = 0;
                    for (size_t j = 0; j < L; ++j) acc += p[j] * Vb[j * D + e];
                    orow[e] = (float) (acc / sum);
                }
            }
        }
    free(p);
}

/* TopK: value descending, ties by lower index, NaN lowest.  O(n*k) selection; indices int64. */
static uint32_t order_key(float f) {
    uint32_t b;
    if (f != f) return 0u;
    memcpy(&b, &f, 4);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
void oracle_topk_f32(const float *x, float *values, int64_t *indices, size_t rows, size_t n, size_t k) {
    uint8_t *used = (uint8_t *) malloc(n);
    for (size_t r = 0; r < rows; ++r) {
        const float *xr = x + r * n;
        memset(used, 0, n);
        for (size_t t = 0; t < k; ++t) {
            size_t best = n;
            uint32_t bk = 0;
            for (size_t j = 0; j < n; ++j) {
                if (used[j]) continue;
                const uint32_t key = order_key(xr[j]);
                if (best == n || key > bk) best = j, bk = key;
            }
            used[best] = 1;
            values[r * k + t] = xr[best];
            indices[r * k + t] = (int64_t) best;
        }
    }
    free(used);
}
