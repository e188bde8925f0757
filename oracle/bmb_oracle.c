/* bmb_oracle.c -- CPU restatement of the reference's GEMM / attention / nn /
 * train-step arithmetic.  TEST INFRASTRUCTURE ONLY: the tests, the smoke check
 * and the benchmark's cpu_baseline leg call it as the checker; nothing in the
 * shipped library links or loads it.
 *
 * The reference (OoEthanoO/bare-metal-bard) has no CPU code path at all: its
 * own tests compare one GPU implementation with another (cuBLAS in
 * src/bench.cu:259-273 and tools/test_gemm.cu:30-38; the unfused attention in
 * tools/test_flash.cu:1-6; finite differences in tools/test_grad.cu).  It also
 * stores no golden vectors.  Each function below therefore restates the body
 * of the reference kernel it cites, in plain C, and is pinned two ways:
 * (a) against the reference's own CUDA kernels compiled for sm_100a and run on
 * the same inputs (the GPU tests), and (b) against closed-form cases and
 * identities (the CPU tests).
 *
 * Build: gcc -O3 -march=native -ffp-contract=fast -fopenmp -shared -fPIC.
 * The GEMM inner products use fmaf() explicitly: one fused multiply-add per
 * term, the instruction nvcc emits for `acc += a*b` in the reference kernels,
 * so a sequential-k fp32 dot product agrees with the GPU's to the last bit.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ GEMM */
/* Element (m,k) of op(A) and (k,n) of op(B), src/gemm.h:6-11. */
static inline float a_at(const float *A, int ta, int M, int K, int m, int k) {
    return ta ? A[(size_t)k * M + m] : A[(size_t)m * K + k];
}
static inline float b_at(const float *B, int tb, int N, int K, int k, int n) {
    return tb ? B[(size_t)n * K + k] : B[(size_t)k * N + n];
}

/* One thread per output, k ascending, fp32 accumulator, then
 * C = alpha*acc + beta*C: the body of naive_kernel, src/kernels/k01_naive.cu:18-30,
 * with the transposes of gemm_generic, src/gemm.cu:169-197. */
void orc_gemm(int ta, int tb, int M, int N, int K, float alpha, const float *A, const float *B,
              float beta, float *C) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc = fmaf(a_at(A, ta, M, K, m, k), b_at(B, tb, N, K, k, n), acc);
            const size_t i = (size_t)m * N + n;
            C[i] = (beta == 0.0f) ? alpha * acc : alpha * acc + beta * C[i];
        }
}

/* Same sums in the same order (each output still accumulates k = 0..K-1 in
 * fp32), arranged i-k-j over packed copies so that the inner loop vectorises.
 * This is the form the CPU baseline is timed on. */
void orc_gemm_fast(int ta, int tb, int M, int N, int K, float alpha, const float *A, const float *B,
                   float beta, float *C) {
    float *Ap = NULL, *Bp = NULL;
    if (ta) {
        Ap = (float *)malloc((size_t)M * K * sizeof(float));
#pragma omp parallel for schedule(static)
        for (int m = 0; m < M; ++m)
            for (int k = 0; k < K; ++k) Ap[(size_t)m * K + k] = A[(size_t)k * M + m];
        A = Ap;
    }
    if (tb) {
        Bp = (float *)malloc((size_t)K * N * sizeof(float));
#pragma omp parallel for schedule(static)
        for (int k = 0; k < K; ++k)
            for (int n = 0; n < N; ++n) Bp[(size_t)k * N + n] = B[(size_t)n * K + k];
        B = Bp;
    }
#pragma omp parallel
    {
        float *acc = (float *)malloc((size_t)N * sizeof(float));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            for (int n = 0; n < N; ++n) acc[n] = 0.0f;
            for (int k = 0; k < K; ++k) {
                const float a = A[(size_t)m * K + k];
                const float *brow = B + (size_t)k * N;
                for (int n = 0; n < N; ++n) acc[n] = fmaf(a, brow[n], acc[n]);
            }
            float *crow = C + (size_t)m * N;
            if (beta == 0.0f) for (int n = 0; n < N; ++n) crow[n] = alpha * acc[n];
            else for (int n = 0; n < N; ++n) crow[n] = alpha * acc[n] + beta * crow[n];
        }
        free(acc);
    }
    free(Ap);
    free(Bp);
}

/* Double accumulator: separates "wrong" from "summed in another order". */
void orc_gemm_f64(int ta, int tb, int M, int N, int K, float alpha, const float *A, const float *B,
                  float beta, float *C) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int k = 0; k < K; ++k)
                acc += (double)a_at(A, ta, M, K, m, k) * (double)b_at(B, tb, N, K, k, n);
            const size_t i = (size_t)m * N + n;
            C[i] = (float)((double)alpha * acc + (beta == 0.0f ? 0.0 : (double)beta * (double)C[i]));
        }
}

void orc_batched_gemm(int ta, int tb, int batch, int M, int N, int K, float alpha, const float *A,
                      long long sA, const float *B, long long sB, float beta, float *C, long long sC) {
    for (int b = 0; b < batch; ++b)
        orc_gemm_fast(ta, tb, M, N, K, alpha, A + (size_t)b * sA, B + (size_t)b * sB, beta,
                      C + (size_t)b * sC);
}

/* cvt.rna.tf32.f32: nearest value with 10 mantissa bits, ties away from zero
 * (what wmma::__float_to_tf32 does at src/kernels/k09_tensorcore.cu:119-128). */
float orc_round_tf32(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) != 0x7f800000u) u += 0x1000u;
    u &= 0xffffe000u;
    memcpy(&x, &u, 4);
    return x;
}
void orc_round_tf32_n(float *dst, const float *src, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_round_tf32(src[i]);
}
/* fp32 -> bf16 -> fp32, round to nearest even. */
float orc_round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) != 0x7f800000u) u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}

/* Normwise error, max|got-ref| / max|ref|; NaN/Inf in got gives +inf
 * (src/bench.cu:133-147). */
double orc_normwise(const float *got, const float *ref, size_t n) {
    double max_abs = 0.0, ref_inf = 0.0;
    int bad = 0;
    for (size_t i = 0; i < n; ++i) {
        const double d = fabs((double)got[i] - (double)ref[i]);
        if (d > max_abs) max_abs = d;
        const double r = fabs((double)ref[i]);
        if (r > ref_inf) ref_inf = r;
        if (!isfinite((double)got[i])) bad = 1;
    }
    if (bad) return INFINITY;
    return max_abs / (ref_inf > 1e-30 ? ref_inf : 1e-30);
}

/* The reference harness's input generator: xorshift32 on a 0.001 grid in
 * [-1, 1) (src/bench.cu:59-66; tools/test_gemm.cu:40-45). */
void orc_fill_xorshift(float *v, size_t n, unsigned seed) {
    unsigned s = seed;
    for (size_t i = 0; i < n; ++i) {
        s ^= s << 13; s ^= s >> 17; s ^= s << 5;
        v[i] = (float)((int)(s % 2000) - 1000) / 1000.0f;
    }
}

/* ------------------------------------------------------------- attention */
/* Causal multi-head attention on the fused (B,T,3C) projection, the math of
 * attention_forward (src/attention.cu:132-163): S = q.k/sqrt(hs) on t2 <= t1,
 * row softmax with max shift, out = P v.  lse = max + log(sum) as the fused
 * kernel saves it (src/flash.cu:309).  att (B,NH,T,T) and lse may be NULL. */
void orc_attention_forward(float *out, float *lse, float *att, const float *qkv, int B, int T, int C,
                           int NH) {
    const int hs = C / NH;
    const float scale = 1.0f / sqrtf((float)hs);
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < NH; ++h) {
            float *p = (float *)malloc((size_t)T * sizeof(float));
            for (int t1 = 0; t1 < T; ++t1) {
                const float *q = qkv + ((size_t)b * T + t1) * 3 * C + (size_t)h * hs;
                float m = -INFINITY;
                for (int t2 = 0; t2 <= t1; ++t2) {
                    const float *k = qkv + ((size_t)b * T + t2) * 3 * C + C + (size_t)h * hs;
                    float s = 0.0f;
                    for (int i = 0; i < hs; ++i) s += q[i] * k[i];
                    s *= scale;
                    p[t2] = s;
                    if (s > m) m = s;
                }
                float sum = 0.0f;
                for (int t2 = 0; t2 <= t1; ++t2) { p[t2] = expf(p[t2] - m); sum += p[t2]; }
                const float inv = 1.0f / sum;
                float *o = out + ((size_t)b * T + t1) * C + (size_t)h * hs;
                for (int i = 0; i < hs; ++i) o[i] = 0.0f;
                for (int t2 = 0; t2 <= t1; ++t2) {
                    p[t2] *= inv;
                    const float *v = qkv + ((size_t)b * T + t2) * 3 * C + 2 * C + (size_t)h * hs;
                    for (int i = 0; i < hs; ++i) o[i] += p[t2] * v[i];
                }
                if (lse) lse[((size_t)b * NH + h) * T + t1] = m + logf(sum);
                if (att) {
                    float *arow = att + (((size_t)b * NH + h) * T + t1) * T;
                    for (int t2 = 0; t2 < T; ++t2) arow[t2] = (t2 <= t1) ? p[t2] : 0.0f;
                }
            }
            free(p);
        }
}

/* Backward of the above (src/attention.cu:165-200, identities at
 * src/flash.cu:447-453):  dV = P^T dO,  dP = dO V^T,
 * dS = P * (dP - rowsum(dP*P)),  dQ = scale dS K,  dK = scale dS^T Q.
 * dqkv is overwritten. */
void orc_attention_backward(float *dqkv, const float *dout, const float *qkv, int B, int T, int C,
                            int NH) {
    const int hs = C / NH;
    const float scale = 1.0f / sqrtf((float)hs);
    memset(dqkv, 0, (size_t)B * T * 3 * C * sizeof(float));
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < NH; ++h) {
            float *p = (float *)malloc((size_t)T * sizeof(float));
            float *dp = (float *)malloc((size_t)T * sizeof(float));
            for (int t1 = 0; t1 < T; ++t1) {
                const float *q = qkv + ((size_t)b * T + t1) * 3 * C + (size_t)h * hs;
                const float *go = dout + ((size_t)b * T + t1) * C + (size_t)h * hs;
                float m = -INFINITY;
                for (int t2 = 0; t2 <= t1; ++t2) {
                    const float *k = qkv + ((size_t)b * T + t2) * 3 * C + C + (size_t)h * hs;
                    float s = 0.0f;
                    for (int i = 0; i < hs; ++i) s += q[i] * k[i];
                    s *= scale;
                    p[t2] = s;
                    if (s > m) m = s;
                }
                float sum = 0.0f;
                for (int t2 = 0; t2 <= t1; ++t2) { p[t2] = expf(p[t2] - m); sum += p[t2]; }
                const float inv = 1.0f / sum;
                float dot = 0.0f;
                for (int t2 = 0; t2 <= t1; ++t2) {
                    p[t2] *= inv;
                    const float *v = qkv + ((size_t)b * T + t2) * 3 * C + 2 * C + (size_t)h * hs;
                    float d = 0.0f;
                    for (int i = 0; i < hs; ++i) d += go[i] * v[i];
                    dp[t2] = d;
                    dot += d * p[t2];
                }
                float *dq = dqkv + ((size_t)b * T + t1) * 3 * C + (size_t)h * hs;
                for (int t2 = 0; t2 <= t1; ++t2) {
                    const float ds = p[t2] * (dp[t2] - dot);
                    const float *k = qkv + ((size_t)b * T + t2) * 3 * C + C + (size_t)h * hs;
                    float *dk = dqkv + ((size_t)b * T + t2) * 3 * C + C + (size_t)h * hs;
                    float *dv = dqkv + ((size_t)b * T + t2) * 3 * C + 2 * C + (size_t)h * hs;
                    for (int i = 0; i < hs; ++i) {
                        dq[i] += scale * ds * k[i];
                        dk[i] += scale * ds * q[i];
                        dv[i] += p[t2] * go[i];
                    }
                }
            }
            free(p);
            free(dp);
        }
}

/* ------------------------------------------------------------- nn kernels */
/* src/nn.cu:23-36 */
void orc_encoder_forward(float *out, const int *tokens, const float *wte, const float *wpe, int B,
                         int T, int C) {
#pragma omp parallel for schedule(static)
    for (int bt = 0; bt < B * T; ++bt) {
        const int t = bt % T;
        const float *e = wte + (size_t)tokens[bt] * C, *p = wpe + (size_t)t * C;
        float *o = out + (size_t)bt * C;
        for (int c = 0; c < C; ++c) o[c] = e[c] + p[c];
    }
}
/* src/nn.cu:38-49 (accumulates) */
void orc_encoder_backward(float *dwte, float *dwpe, const float *dout, const int *tokens, int B, int T,
                          int C) {
    for (int bt = 0; bt < B * T; ++bt) {
        const int t = bt % T;
        const float *g = dout + (size_t)bt * C;
        float *a = dwte + (size_t)tokens[bt] * C, *b = dwpe + (size_t)t * C;
        for (int c = 0; c < C; ++c) { a[c] += g[c]; b[c] += g[c]; }
    }
}
/* src/nn.cu:54-78: mean, biased variance around it, rsqrt(var + 1e-5). */
void orc_layernorm_forward(float *out, float *mean, float *rstd, const float *inp, const float *w,
                           const float *b, int N, int C) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < N; ++r) {
        const float *x = inp + (size_t)r * C;
        float s = 0.0f;
        for (int i = 0; i < C; ++i) s += x[i];
        const float mu = s / C;
        float sq = 0.0f;
        for (int i = 0; i < C; ++i) { const float d = x[i] - mu; sq += d * d; }
        const float rs = 1.0f / sqrtf(sq / C + 1e-5f);
        mean[r] = mu; rstd[r] = rs;
        float *y = out + (size_t)r * C;
        for (int i = 0; i < C; ++i) y[i] = ((x[i] - mu) * rs) * w[i] + b[i];
    }
}
/* src/nn.cu:85-113: dinp, dweight, dbias are accumulated into. */
void orc_layernorm_backward(float *dinp, float *dweight, float *dbias, const float *dout,
                            const float *inp, const float *w, const float *mean, const float *rstd,
                            int N, int C) {
    for (int r = 0; r < N; ++r) {
        const float *x = inp + (size_t)r * C, *dy = dout + (size_t)r * C;
        float *dx = dinp + (size_t)r * C;
        const float mu = mean[r], rs = rstd[r];
        float s1 = 0.0f, s2 = 0.0f;
        for (int i = 0; i < C; ++i) {
            const float xh = (x[i] - mu) * rs, d = dy[i] * w[i];
            s1 += d; s2 += d * xh;
        }
        const float m1 = s1 / C, m2 = s2 / C;
        for (int i = 0; i < C; ++i) {
            const float xh = (x[i] - mu) * rs, d = dy[i] * w[i];
            dx[i] += rs * (d - m1 - xh * m2);
            dweight[i] += dy[i] * xh;
            dbias[i] += dy[i];
        }
    }
}
/* src/nn.cu:118-150 */
static inline float gelu1(float x) {
    const float s = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(s * (x + 0.044715f * x * x * x)));
}
void orc_gelu_forward(float *out, const float *inp, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) out[i] = gelu1(inp[i]);
}
void orc_gelu_backward(float *dinp, const float *inp, const float *dout, size_t n) {
    const float s = 0.7978845608028654f;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float x = inp[i];
        const float inner = s * (x + 0.044715f * x * x * x);
        const float t = tanhf(inner);
        const float sech2 = 1.0f - t * t;
        const float dinner = s * (1.0f + 3.0f * 0.044715f * x * x);
        dinp[i] = dout[i] * (0.5f * (1.0f + t) + 0.5f * x * sech2 * dinner);
    }
}
void orc_residual_forward(float *out, const float *a, const float *b, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}
/* src/nn.cu:171-191 */
void orc_bias_forward(float *out, const float *bias, int N, int C) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < N; ++r)
        for (int c = 0; c < C; ++c) out[(size_t)r * C + c] += bias[c];
}
void orc_bias_backward(float *dbias, const float *dout, int N, int C) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; ++c) {
        float acc = 0.0f;
        for (int r = 0; r < N; ++r) acc += dout[(size_t)r * C + c];
        dbias[c] += acc;
    }
}
/* src/nn.cu:197-221: max over real columns, p = exp(x-max)/sum, zero padding,
 * loss = -log(max(p[target], 1e-30)). */
void orc_softmax_crossentropy_forward(float *probs, float *losses, const float *logits,
                                      const int *targets, int N, int V, int Vp) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < N; ++r) {
        const float *x = logits + (size_t)r * Vp;
        float *p = probs + (size_t)r * Vp;
        float m = -3.402823466e38f;
        for (int i = 0; i < V; ++i) if (x[i] > m) m = x[i];
        float s = 0.0f;
        /* The reference sums with 128 threads striding the row and a shuffle tree
         * (src/nn.cu:207-214, src/reduce.cuh:46-60): 128 strided partial sums, then
         * pairwise folding.  A single running fp32 sum over 50k terms would itself be
         * off by ~5e-5, so the same order is kept here. */
        float part[128];
        for (int t = 0; t < 128; ++t) part[t] = 0.0f;
        for (int i = 0; i < V; ++i) { p[i] = expf(x[i] - m); part[i & 127] += p[i]; }
        for (int w = 0; w < 4; ++w)
            for (int off = 16; off > 0; off >>= 1)
                for (int t = 0; t < off; ++t) part[w * 32 + t] += part[w * 32 + t + off];
        s = (part[0] + part[64]) + (part[32] + part[96]);   /* xor-2 then xor-1 over the four warp sums */
        const float inv = 1.0f / s;
        for (int i = 0; i < V; ++i) p[i] *= inv;
        for (int i = V; i < Vp; ++i) p[i] = 0.0f;
        const float pt = p[targets[r]];
        losses[r] = -logf(pt > 1e-30f ? pt : 1e-30f);
    }
}
/* src/nn.cu:226-237 */
void orc_crossentropy_softmax_backward(float *dlogits, const float *probs, const int *targets, int N,
                                       int V, int Vp, float scale) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < N; ++r)
        for (int i = 0; i < Vp; ++i)
            dlogits[(size_t)r * Vp + i] =
                (i < V) ? (probs[(size_t)r * Vp + i] - (i == targets[r] ? 1.0f : 0.0f)) * scale : 0.0f;
}
/* src/nn.cu:240-254 with the bias corrections of src/nn.cu:339-340. */
void orc_adamw_update(float *params, const float *grads, float *m, float *v, size_t n, float lr,
                      float beta1, float beta2, float eps, float wd, int step, float gscale) {
    const float bc1 = 1.0f - powf(beta1, (float)step), bc2 = 1.0f - powf(beta2, (float)step);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        const float g = grads[i] * gscale;
        const float mi = beta1 * m[i] + (1.0f - beta1) * g;
        const float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
        m[i] = mi; v[i] = vi;
        const float mhat = mi / bc1, vhat = vi / bc2;
        params[i] -= lr * (mhat / (sqrtf(vhat) + eps) + wd * params[i]);
    }
}
/* src/nn.cu:336-355 (finished in double) */
float orc_grad_global_norm(const float *g, size_t n) {
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) s += (double)g[i] * (double)g[i];
    return (float)sqrt(s);
}
float orc_mean(const float *x, int n) {
    float acc = 0.0f;
    for (int i = 0; i < n; ++i) acc += x[i];
    return acc / n;
}

/* ------------------------------------------------------------ train step */
/* A GPT-2-shaped model on the host: tensor order and sizes of
 * src/gpt.cu:32-51, forward op list of src/gpt.cu:222-287, backward of
 * src/gpt.cu:290-385, optimiser step of src/train_gpt.cu:442-451. */
typedef struct orc_gpt {
    int maxT, V, Vp, L, NH, C, B, T;
    size_t psize[16], poff[16], num_params;
    float *params, *grads, *m, *v;
    /* activations */
    float *encoded, *ln1, *ln1_mean, *ln1_rstd, *qkv, *atty, *attproj, *res2, *ln2, *ln2_mean,
        *ln2_rstd, *fch, *fchg, *fcproj, *res3, *lnf, *lnf_mean, *lnf_rstd, *logits, *probs, *losses;
    float *dres, *dln1, *dln2, *datty, *dqkv, *dfch, *dfchg, *dlogits, *dlnf;
    int *tokens, *targets;
} orc_gpt;

static float *falloc(size_t n) { return (float *)calloc(n ? n : 1, sizeof(float)); }

orc_gpt *orc_gpt_create(int maxT, int V, int Vp, int L, int NH, int C, int B, int T) {
    orc_gpt *g = (orc_gpt *)calloc(1, sizeof(orc_gpt));
    g->maxT = maxT; g->V = V; g->Vp = Vp; g->L = L; g->NH = NH; g->C = C; g->B = B; g->T = T;
    const size_t l = L, c = C;
    const size_t sz[16] = {(size_t)Vp * c, (size_t)maxT * c, l * c, l * c, l * 3 * c * c, l * 3 * c,
                           l * c * c, l * c, l * c, l * c, l * 4 * c * c, l * 4 * c, l * c * 4 * c,
                           l * c, c, c};
    g->num_params = 0;
    for (int i = 0; i < 16; ++i) { g->psize[i] = sz[i]; g->poff[i] = g->num_params; g->num_params += sz[i]; }
    g->params = falloc(g->num_params); g->grads = falloc(g->num_params);
    g->m = falloc(g->num_params); g->v = falloc(g->num_params);
    const size_t BT = (size_t)B * T, BTC = BT * c;
    g->encoded = falloc(BTC);
    g->ln1 = falloc(BTC * l); g->ln1_mean = falloc(BT * l); g->ln1_rstd = falloc(BT * l);
    g->qkv = falloc(3 * BTC * l); g->atty = falloc(BTC * l); g->attproj = falloc(BTC * l);
    g->res2 = falloc(BTC * l); g->ln2 = falloc(BTC * l); g->ln2_mean = falloc(BT * l);
    g->ln2_rstd = falloc(BT * l); g->fch = falloc(4 * BTC * l); g->fchg = falloc(4 * BTC * l);
    g->fcproj = falloc(BTC * l); g->res3 = falloc(BTC * l);
    g->lnf = falloc(BTC); g->lnf_mean = falloc(BT); g->lnf_rstd = falloc(BT);
    g->logits = falloc(BT * Vp); g->probs = falloc(BT * Vp); g->losses = falloc(BT);
    g->dres = falloc(BTC); g->dln1 = falloc(BTC); g->dln2 = falloc(BTC); g->datty = falloc(BTC);
    g->dqkv = falloc(3 * BTC); g->dfch = falloc(4 * BTC); g->dfchg = falloc(4 * BTC);
    g->dlogits = falloc(BT * Vp); g->dlnf = falloc(BTC);
    g->tokens = (int *)calloc(BT, sizeof(int)); g->targets = (int *)calloc(BT, sizeof(int));
    return g;
}
void orc_gpt_destroy(orc_gpt *g) {
    if (!g) return;
    float **f[] = {&g->params, &g->grads, &g->m, &g->v, &g->encoded, &g->ln1, &g->ln1_mean, &g->ln1_rstd,
                   &g->qkv, &g->atty, &g->attproj, &g->res2, &g->ln2, &g->ln2_mean, &g->ln2_rstd, &g->fch,
                   &g->fchg, &g->fcproj, &g->res3, &g->lnf, &g->lnf_mean, &g->lnf_rstd, &g->logits,
                   &g->probs, &g->losses, &g->dres, &g->dln1, &g->dln2, &g->datty, &g->dqkv, &g->dfch,
                   &g->dfchg, &g->dlogits, &g->dlnf};
    for (size_t i = 0; i < sizeof(f) / sizeof(f[0]); ++i) free(*f[i]);
    free(g->tokens); free(g->targets); free(g);
}
size_t orc_gpt_num_params(const orc_gpt *g) { return g->num_params; }
float *orc_gpt_params(orc_gpt *g) { return g->params; }
float *orc_gpt_grads(orc_gpt *g) { return g->grads; }
void orc_gpt_set_batch(orc_gpt *g, const int *tokens, const int *targets) {
    memcpy(g->tokens, tokens, (size_t)g->B * g->T * sizeof(int));
    memcpy(g->targets, targets, (size_t)g->B * g->T * sizeof(int));
}

float orc_gpt_forward(orc_gpt *g) {
    const int B = g->B, T = g->T, C = g->C, L = g->L, NH = g->NH, Vp = g->Vp, V = g->V, N = B * T;
    const size_t BTC = (size_t)N * C, BT = N;
    const float *P = g->params;
    const size_t *o = g->poff;
    orc_encoder_forward(g->encoded, g->tokens, P + o[0], P + o[1], B, T, C);
    float *residual = g->encoded;
    for (int l = 0; l < L; ++l) {
        float *ln1 = g->ln1 + l * BTC, *qkv = g->qkv + l * 3 * BTC, *atty = g->atty + l * BTC;
        float *attproj = g->attproj + l * BTC, *res2 = g->res2 + l * BTC, *ln2 = g->ln2 + l * BTC;
        float *fch = g->fch + l * 4 * BTC, *fchg = g->fchg + l * 4 * BTC, *fcproj = g->fcproj + l * BTC;
        float *res3 = g->res3 + l * BTC;
        orc_layernorm_forward(ln1, g->ln1_mean + l * BT, g->ln1_rstd + l * BT, residual,
                              P + o[2] + (size_t)l * C, P + o[3] + (size_t)l * C, N, C);
        orc_gemm_fast(0, 1, N, 3 * C, C, 1.0f, ln1, P + o[4] + (size_t)l * 3 * C * C, 0.0f, qkv);
        orc_bias_forward(qkv, P + o[5] + (size_t)l * 3 * C, N, 3 * C);
        orc_attention_forward(atty, NULL, NULL, qkv, B, T, C, NH);
        orc_gemm_fast(0, 1, N, C, C, 1.0f, atty, P + o[6] + (size_t)l * C * C, 0.0f, attproj);
        orc_bias_forward(attproj, P + o[7] + (size_t)l * C, N, C);
        orc_residual_forward(res2, residual, attproj, BTC);
        orc_layernorm_forward(ln2, g->ln2_mean + l * BT, g->ln2_rstd + l * BT, res2,
                              P + o[8] + (size_t)l * C, P + o[9] + (size_t)l * C, N, C);
        orc_gemm_fast(0, 1, N, 4 * C, C, 1.0f, ln2, P + o[10] + (size_t)l * 4 * C * C, 0.0f, fch);
        orc_bias_forward(fch, P + o[11] + (size_t)l * 4 * C, N, 4 * C);
        orc_gelu_forward(fchg, fch, 4 * BTC);
        orc_gemm_fast(0, 1, N, C, 4 * C, 1.0f, fchg, P + o[12] + (size_t)l * C * 4 * C, 0.0f, fcproj);
        orc_bias_forward(fcproj, P + o[13] + (size_t)l * C, N, C);
        orc_residual_forward(res3, res2, fcproj, BTC);
        residual = res3;
    }
    orc_layernorm_forward(g->lnf, g->lnf_mean, g->lnf_rstd, residual, P + o[14], P + o[15], N, C);
    orc_gemm_fast(0, 1, N, Vp, C, 1.0f, g->lnf, P + o[0], 0.0f, g->logits);
    orc_softmax_crossentropy_forward(g->probs, g->losses, g->logits, g->targets, N, V, Vp);
    return orc_mean(g->losses, N);
}

void orc_gpt_backward(orc_gpt *g) {
    const int B = g->B, T = g->T, C = g->C, L = g->L, NH = g->NH, Vp = g->Vp, V = g->V, N = B * T;
    const size_t BTC = (size_t)N * C, BT = N;
    const float *P = g->params;
    float *G = g->grads;
    const size_t *o = g->poff;
    memset(G, 0, g->num_params * sizeof(float));
    orc_crossentropy_softmax_backward(g->dlogits, g->probs, g->targets, N, V, Vp, 1.0f / N);
    orc_gemm_fast(0, 0, N, C, Vp, 1.0f, g->dlogits, P + o[0], 0.0f, g->dlnf);
    orc_gemm_fast(1, 0, Vp, C, N, 1.0f, g->dlogits, g->lnf, 1.0f, G + o[0]);
    memset(g->dres, 0, BTC * sizeof(float));
    orc_layernorm_backward(g->dres, G + o[14], G + o[15], g->dlnf, g->res3 + (size_t)(L - 1) * BTC,
                           P + o[14], g->lnf_mean, g->lnf_rstd, N, C);
    for (int l = L - 1; l >= 0; --l) {
        float *residual = (l == 0) ? g->encoded : g->res3 + (size_t)(l - 1) * BTC;
        float *ln1 = g->ln1 + l * BTC, *qkv = g->qkv + l * 3 * BTC, *atty = g->atty + l * BTC;
        float *res2 = g->res2 + l * BTC, *ln2 = g->ln2 + l * BTC;
        float *fch = g->fch + l * 4 * BTC, *fchg = g->fchg + l * 4 * BTC;
        const size_t lC = (size_t)l * C;
        orc_gemm_fast(0, 0, N, 4 * C, C, 1.0f, g->dres, P + o[12] + (size_t)l * C * 4 * C, 0.0f, g->dfchg);
        orc_gemm_fast(1, 0, C, 4 * C, N, 1.0f, g->dres, fchg, 1.0f, G + o[12] + (size_t)l * C * 4 * C);
        orc_bias_backward(G + o[13] + lC, g->dres, N, C);
        orc_gelu_backward(g->dfch, fch, g->dfchg, 4 * BTC);
        orc_gemm_fast(0, 0, N, C, 4 * C, 1.0f, g->dfch, P + o[10] + (size_t)l * 4 * C * C, 0.0f, g->dln2);
        orc_gemm_fast(1, 0, 4 * C, C, N, 1.0f, g->dfch, ln2, 1.0f, G + o[10] + (size_t)l * 4 * C * C);
        orc_bias_backward(G + o[11] + 4 * lC, g->dfch, N, 4 * C);
        orc_layernorm_backward(g->dres, G + o[8] + lC, G + o[9] + lC, g->dln2, res2, P + o[8] + lC,
                               g->ln2_mean + l * BT, g->ln2_rstd + l * BT, N, C);
        orc_gemm_fast(0, 0, N, C, C, 1.0f, g->dres, P + o[6] + (size_t)l * C * C, 0.0f, g->datty);
        orc_gemm_fast(1, 0, C, C, N, 1.0f, g->dres, atty, 1.0f, G + o[6] + (size_t)l * C * C);
        orc_bias_backward(G + o[7] + lC, g->dres, N, C);
        orc_attention_backward(g->dqkv, g->datty, qkv, B, T, C, NH);
        orc_gemm_fast(0, 0, N, C, 3 * C, 1.0f, g->dqkv, P + o[4] + (size_t)l * 3 * C * C, 0.0f, g->dln1);
        orc_gemm_fast(1, 0, 3 * C, C, N, 1.0f, g->dqkv, ln1, 1.0f, G + o[4] + (size_t)l * 3 * C * C);
        orc_bias_backward(G + o[5] + 3 * lC, g->dqkv, N, 3 * C);
        orc_layernorm_backward(g->dres, G + o[2] + lC, G + o[3] + lC, g->dln1, residual, P + o[2] + lC,
                               g->ln1_mean + l * BT, g->ln1_rstd + l * BT, N, C);
    }
    orc_encoder_backward(G + o[0], G + o[1], g->dres, g->tokens, B, T, C);
}

/* One optimiser step, single rank: forward, backward, global-norm clip, AdamW
 * (src/train_gpt.cu:442-451 with nranks = 1).  Returns the loss. */
float orc_gpt_step(orc_gpt *g, float lr, float beta1, float beta2, float eps, float wd, float clip,
                   int step) {
    const float loss = orc_gpt_forward(g);
    orc_gpt_backward(g);
    const float gn = orc_grad_global_norm(g->grads, g->num_params);
    const float gs = (gn > clip) ? clip / gn : 1.0f;
    orc_adamw_update(g->params, g->grads, g->m, g->v, g->num_params, lr, beta1, beta2, eps, wd, step, gs);
    return loss;
}
