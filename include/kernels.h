// Kernel registry with the reference's shape (src/kernels.h:10-31): a table of
// {id, name, launch function, note, normwise tolerance}.  libbmb.so defines
// these symbols with the reference's exact C++ signatures, so host code built
// against either header links against it.
//
// Every launch function computes, row-major,  C = alpha * A @ B + beta * C
// with A (M x K), B (K x N), C (M x N), on the calling thread's current
// stream (bmb_set_stream; the legacy default stream unless set).
#pragma once

typedef void (*sgemm_fn)(int M, int N, int K, float alpha, const float *A,
                         const float *B, float beta, float *C);

struct KernelEntry {
    int id;
    const char *name;
    sgemm_fn fn;
    const char *note;
    double tol;  // normwise bound against an fp32 product: max|got-ref| / max|ref|
};

extern const KernelEntry KERNELS[];
extern const int NUM_KERNELS;
const KernelEntry *find_kernel(int id);  // nullptr when the id is not registered

// The three sm_100a entries of the table.
void sgemm_simt_fp32(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_tcgen05_tf32(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_tcgen05_bf16(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);

// The reference's nine launch names (src/kernels.h:34-42) stay linkable: the
// eight fp32 stages all run the SIMT kernel, the tensor-core stage runs TF32.
void sgemm_naive(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_coalesced(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_smem(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_tile1d(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_tile2d(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_vectorized(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_warptile(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_doublebuffer(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
void sgemm_tensorcore(int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C);
