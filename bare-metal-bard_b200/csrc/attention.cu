// Unfused causal attention (src/attention.h:18-24, src/attention.cu:132-200):
// head permute, batched Q@K^T, causal row softmax, batched P@V, head merge --
// and its seven-step backward.  It materialises the (B,NH,T,T) score matrix
// and is here as the reference point the fused kernels are compared with and
// for host code that asks for the unfused model; it is not tuned.
#include "common.cuh"
#include <cfloat>
#include <cmath>

namespace bmb {
namespace {

// which = 0: qkv (B,T,3C) -> q,k,v (B,NH,T,hs) back to back in qkvr
// which = 1: inverse scatter of dq,dk,dv into dqkv
__global__ void permute_qkv_k(float *__restrict__ dst, const float *__restrict__ src, int B, int T,
                              int NH, int hs, int which) {
    const long long total = (long long)B * NH * T * hs;
    const int C = NH * hs;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % hs);
        const int t = (int)((idx / hs) % T);
        const int h = (int)((idx / ((long long)hs * T)) % NH);
        const int b = (int)(idx / ((long long)hs * T * NH));
        const size_t flat = ((size_t)b * T + t) * 3 * C + (size_t)h * hs + i;
        if (which == 0) {
            dst[idx] = src[flat];
            dst[total + idx] = src[flat + C];
            dst[2 * total + idx] = src[flat + 2 * C];
        } else {
            dst[flat] = src[idx];
            dst[flat + C] = src[total + idx];
            dst[flat + 2 * C] = src[2 * total + idx];
        }
    }
}

// which = 0: (B,NH,T,hs) -> (B,T,C);  which = 1: (B,T,C) -> (B,NH,T,hs)
__global__ void permute_out_k(float *__restrict__ dst, const float *__restrict__ src, int B, int T,
                              int NH, int hs, int which) {
    const long long total = (long long)B * NH * T * hs;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % hs);
        const int t = (int)((idx / hs) % T);
        const int h = (int)((idx / ((long long)hs * T)) % NH);
        const int b = (int)(idx / ((long long)hs * T * NH));
        const size_t flat = ((size_t)b * T + t) * (NH * hs) + (size_t)h * hs + i;
        if (which == 0) dst[flat] = src[idx];
        else dst[idx] = src[flat];
    }
}

// Row t1 of every (b,h) attends to t2 <= t1; exact zeros beyond (src/attention.cu:86-111).
__global__ void softmax_causal_k(float *att, const float *preatt, int T) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const int len = (int)(row % T) + 1;
    const float *x = preatt + row * T;
    float *y = att + row * T;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < len; i += blockDim.x) m = fmaxf(m, x[i]);
    m = block_reduce<true>(m, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float e = __expf(x[i] - m);
        y[i] = e;
        s += e;
    }
    s = block_reduce<false>(s, red);
    const float inv = 1.0f / s;
    for (int i = threadIdx.x; i < len; i += blockDim.x) y[i] *= inv;
    for (int i = len + threadIdx.x; i < T; i += blockDim.x) y[i] = 0.0f;
}

// dx_i = y_i (dy_i - sum_j dy_j y_j) on the causal part, 0 beyond (src/attention.cu:113-129).
__global__ void softmax_causal_bwd_k(float *dpreatt, const float *datt, const float *att, int T) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const int len = (int)(row % T) + 1;
    const float *y = att + row * T, *dy = datt + row * T;
    float *dx = dpreatt + row * T;
    float dot = 0.0f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) dot += dy[i] * y[i];
    dot = block_reduce<false>(dot, red);
    for (int i = threadIdx.x; i < len; i += blockDim.x) dx[i] = y[i] * (dy[i] - dot);
    for (int i = len + threadIdx.x; i < T; i += blockDim.x) dx[i] = 0.0f;
}

inline int grid1d(long long n) {
    long long b = (n + 255) / 256, cap = (long long)sm_count() * 16;
    return (int)(b > cap ? cap : (b < 1 ? 1 : b));
}
}  // namespace
}  // namespace bmb

using namespace bmb;

extern "C" {

int bmb_attention_forward(float *out, float *qkvr, float *att, const float *qkv, int B, int T,
                          int C, int NH) {
    if (B <= 0 || T <= 0) return BMB_OK;
    if (NH <= 0 || C % NH) return fail(BMB_E_ARG, "attention: C=%d not divisible by NH=%d", C, NH);
    const int hs = C / NH;
    const long long total = (long long)B * NH * T * hs;
    const float scale = 1.0f / sqrtf((float)hs);
    const long long sHead = (long long)T * hs, sAtt = (long long)T * T;
    cudaStream_t st = cur_stream();
    const int math = bmb_get_math_mode();

    permute_qkv_k<<<grid1d(total), 256, 0, st>>>(qkvr, qkv, B, T, NH, hs, 0);
    count_launch();
    const float *q = qkvr, *k = qkvr + total, *v = qkvr + 2 * total;
    float *vaccum = qkvr + 3 * total;
    BMB_TRY(gemm_any(math, 0, 0, 1, B * NH, T, T, hs, scale, q, sHead, k, sHead, 0.0f, att, sAtt, st));
    softmax_causal_k<<<(unsigned)((long long)B * NH * T), 128, 0, st>>>(att, att, T);
    count_launch();
    BMB_TRY(gemm_any(math, 0, 0, 0, B * NH, T, hs, T, 1.0f, att, sAtt, v, sHead, 0.0f, vaccum, sHead, st));
    permute_out_k<<<grid1d(total), 256, 0, st>>>(out, vaccum, B, T, NH, hs, 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_attention_backward(float *dqkv, float *dqkvr, float *datt, float *dpreatt, const float *dout,
                           const float *qkvr, const float *att, int B, int T, int C, int NH) {
    if (B <= 0 || T <= 0) return BMB_OK;
    if (NH <= 0 || C % NH) return fail(BMB_E_ARG, "attention: C=%d not divisible by NH=%d", C, NH);
    const int hs = C / NH;
    const long long total = (long long)B * NH * T * hs;
    const float scale = 1.0f / sqrtf((float)hs);
    const long long sHead = (long long)T * hs, sAtt = (long long)T * T;
    cudaStream_t st = cur_stream();
    const int math = bmb_get_math_mode();

    const float *q = qkvr, *k = qkvr + total, *v = qkvr + 2 * total;
    float *dq = dqkvr, *dk = dqkvr + total, *dv = dqkvr + 2 * total;
    float *dvaccum = dqkvr + 3 * total;

    permute_out_k<<<grid1d(total), 256, 0, st>>>(dvaccum, dout, B, T, NH, hs, 1);
    count_launch();
    // datt = dvaccum @ v^T ;  dv = att^T @ dvaccum
    BMB_TRY(gemm_any(math, 0, 0, 1, B * NH, T, T, hs, 1.0f, dvaccum, sHead, v, sHead, 0.0f, datt, sAtt, st));
    BMB_TRY(gemm_any(math, 0, 1, 0, B * NH, T, hs, T, 1.0f, att, sAtt, dvaccum, sHead, 0.0f, dv, sHead, st));
    softmax_causal_bwd_k<<<(unsigned)((long long)B * NH * T), 128, 0, st>>>(dpreatt, datt, att, T);
    count_launch();
    // dq = scale * dpreatt @ k ;  dk = scale * dpreatt^T @ q
    BMB_TRY(gemm_any(math, 0, 0, 0, B * NH, T, hs, T, scale, dpreatt, sAtt, k, sHead, 0.0f, dq, sHead, st));
    BMB_TRY(gemm_any(math, 0, 1, 0, B * NH, T, hs, T, scale, dpreatt, sAtt, q, sHead, 0.0f, dk, sHead, st));
    permute_qkv_k<<<grid1d(total), 256, 0, st>>>(dqkv, dqkvr, B, T, NH, hs, 1);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // extern "C"
