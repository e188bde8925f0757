// GEMM entry points: the transpose-aware gemm / batched_gemm of
// src/gemm.h:17-29 and the kernel registry of src/kernels.h:10-31, routed to
// the fp32 SIMT kernel or the tcgen05 tensor-core kernel.
#include "common.cuh"

namespace bmb {
int gemm_simt(int transA, int transB, int batch, int M, int N, int K, float alpha, const float *A,
              long long sA, const float *B, long long sB, float beta, float *C, long long sC,
              cudaStream_t st);
// Tensor-core path (gemm_tc.cu).  Returns BMB_E_UNSUPPORTED for shapes it does
// not take; the caller then falls back to the SIMT kernel (still on the GPU).
int gemm_tc(int math, int flags, int transA, int transB, int batch, int M, int N, int K,
            float alpha, const float *A, long long sA, const float *B, long long sB, float beta,
            float *C, long long sC, const float *bias, cudaStream_t st, float *aux_gelu = nullptr);
bool gemm_tc_accepts(int math, int transA, int transB, int batch, int M, int N, int K,
                     const float *A, long long sA, const float *B, long long sB, const float *C,
                     long long sC);

// C = alpha*op(A)op(B) + bias (broadcast over rows, may be null) + beta*C.
int gemm_any_bias(int math, int flags, int ta, int tb, int batch, int M, int N, int K, float alpha,
                  const float *A, long long sA, const float *B, long long sB, float beta, float *C,
                  long long sC, const float *bias, cudaStream_t st, float *aux_gelu) {
    int rc = BMB_OK;
    bool aux_done = false;
    if (math != BMB_MATH_FP32 && M > 0 && N > 0 && K > 0 && batch > 0 &&
        gemm_tc_accepts(math, ta, tb, batch, M, N, K, A, sA, B, sB, C, sC)) {
        rc = BMB_E_UNSUPPORTED;
        if (aux_gelu) {
            rc = gemm_tc(math, flags, ta, tb, batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, bias, st, aux_gelu);
            aux_done = (rc == BMB_OK);
        }
        if (rc == BMB_E_UNSUPPORTED) rc = gemm_tc(math, flags, ta, tb, batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, bias, st);
        if (rc != BMB_OK) return rc;
    } else {
        BMB_TRY(gemm_simt(ta, tb, batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, st));
        // SIMT route: the bias and the optional rounding are separate passes on the same stream.
        void *prev = bmb_get_stream();
        bmb_set_stream((void *)st);
        if (bias && batch == 1) rc = bmb_bias_forward(C, bias, M, N);
        if (rc == BMB_OK && (flags & BMB_GEMM_C_ROUNDED) && batch == 1)
            rc = bmb_round_tf32(C, C, (size_t)M * N, (void *)st);
        bmb_set_stream(prev);
        if (rc != BMB_OK) return rc;
    }
    if (aux_gelu && !aux_done) {
        if (batch != 1) return fail(BMB_E_ARG, "gemm: the activation output serves single products only");
        void *prev = bmb_get_stream();
        bmb_set_stream((void *)st);
        rc = bmb_gelu_forward(aux_gelu, C, M * N);
        bmb_set_stream(prev);
    }
    return rc;
}

int gemm_any(int math, int flags, int ta, int tb, int batch, int M, int N, int K, float alpha,
             const float *A, long long sA, const float *B, long long sB, float beta, float *C,
             long long sC, cudaStream_t st) {
    return gemm_any_bias(math, flags, ta, tb, batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, nullptr, st);
}
}  // namespace bmb

using namespace bmb;

extern "C" {

int bmb_gemm(int transA, int transB, int M, int N, int K, float alpha, const float *A,
             const float *B, float beta, float *C, void *stream) {
    return gemm_any(bmb_get_math_mode(), 0, transA, transB, 1, M, N, K, alpha, A, 0, B, 0, beta, C, 0,
                    (cudaStream_t)stream);
}

int bmb_gemm_ex(int math, int flags, int transA, int transB, int M, int N, int K, float alpha,
                const float *A, const float *B, float beta, float *C, void *stream) {
    if (math < BMB_MATH_FP32 || math > BMB_MATH_BF16) return fail(BMB_E_ARG, "gemm_ex: math %d", math);
    return gemm_any(math, flags, transA, transB, 1, M, N, K, alpha, A, 0, B, 0, beta, C, 0,
                    (cudaStream_t)stream);
}

int bmb_gemm_bias_gelu(int math, int flags, int M, int N, int K, const float *A, const float *W, const float *bias,
                       float *C, float *C_gelu, void *stream) {
    if (math < BMB_MATH_FP32 || math > BMB_MATH_BF16) return fail(BMB_E_ARG, "gemm_bias_gelu: math %d", math);
    if (!A || !W || !C || !C_gelu || M < 1 || N < 1 || K < 1) return fail(BMB_E_ARG, "gemm_bias_gelu: bad argument");
    const bool was = emit_rounded();
    set_emit_rounded((flags & BMB_GEMM_AUX_ROUNDED) != 0);
    const int rc = gemm_any_bias(math, flags & ~BMB_GEMM_AUX_ROUNDED, 0, 1, 1, M, N, K, 1.0f, A, 0, W, 0, 0.0f, C, 0, bias,
                                 (cudaStream_t)stream, C_gelu);
    set_emit_rounded(was);
    return rc;
}

int bmb_batched_gemm(int transA, int transB, int batch, int M, int N, int K, float alpha,
                     const float *A, long long strideA, const float *B, long long strideB,
                     float beta, float *C, long long strideC, void *stream) {
    return gemm_any(bmb_get_math_mode(), 0, transA, transB, batch, M, N, K, alpha, A, strideA, B,
                    strideB, beta, C, strideC, (cudaStream_t)stream);
}

int bmb_sgemm_simt(int M, int N, int K, float alpha, const float *A, const float *B, float beta,
                   float *C) {
    return gemm_simt(0, 0, 1, M, N, K, alpha, A, 0, B, 0, beta, C, 0, cur_stream());
}
int bmb_sgemm_tf32(int M, int N, int K, float alpha, const float *A, const float *B, float beta,
                   float *C) {
    return gemm_any(BMB_MATH_TF32, 0, 0, 0, 1, M, N, K, alpha, A, 0, B, 0, beta, C, 0, cur_stream());
}
int bmb_sgemm_bf16(int M, int N, int K, float alpha, const float *A, const float *B, float beta,
                   float *C) {
    return gemm_any(BMB_MATH_BF16, 0, 0, 0, 1, M, N, K, alpha, A, 0, B, 0, beta, C, 0, cur_stream());
}

// ---- registry -----------------------------------------------------------
// The reference's sgemm_fn returns void; errors surface through
// cudaGetLastError in its harness (src/bench.cu:96).  The table functions
// below keep that convention and drop the status.
static void reg_simt(int M, int N, int K, float a, const float *A, const float *B, float b, float *C) {
    (void)bmb_sgemm_simt(M, N, K, a, A, B, b, C);
}
static void reg_tf32(int M, int N, int K, float a, const float *A, const float *B, float b, float *C) {
    (void)bmb_sgemm_tf32(M, N, K, a, A, B, b, C);
}
static void reg_bf16(int M, int N, int K, float a, const float *A, const float *B, float b, float *C) {
    (void)bmb_sgemm_bf16(M, N, K, a, A, B, b, C);
}

static const bmb_kernel_entry g_table[] = {
    {1, "simt_fp32", reg_simt, "sm_100a FFMA, 128x128x16 tile, 8x8 per thread, register-prefetch double buffer", 1e-6},
    {2, "tcgen05_tf32", reg_tf32, "tcgen05.mma kind::tf32, TMA-fed 128B-swizzled ring, TMEM accumulators, rna-rounded operands", 5e-4},
    {3, "tcgen05_bf16", reg_bf16, "tcgen05.mma kind::f16 on bf16-rounded operands, fp32 accumulate in TMEM", 8e-3},
};

int bmb_num_kernels(void) { return (int)(sizeof(g_table) / sizeof(g_table[0])); }
const bmb_kernel_entry *bmb_kernel_table(void) { return g_table; }
const bmb_kernel_entry *bmb_find_kernel(int id) {
    for (int i = 0; i < bmb_num_kernels(); ++i)
        if (g_table[i].id == id) return &g_table[i];
    return nullptr;
}

}  // extern "C"
