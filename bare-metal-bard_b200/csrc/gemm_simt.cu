// fp32 SIMT GEMM for sm_100a: C = alpha*op(A)@op(B) + beta*C, row-major,
// all four transpose cases, optional strided batch in gridDim.z.
//
// Shape of the kernel: a 128x128 output tile per 256-thread CTA, K walked in
// steps of 16; each thread owns an 8x8 accumulator split into four 4x4
// quadrants 64 apart so that every shared-memory fragment read is one
// 128-bit load.  Both operand tiles live in shared memory K-major
// ([k][128 m-or-n values]) whatever their layout in global memory, so the
// inner loop is the same for NN/NT/TN/TT; only the staging differs:
//   * source contiguous along m/n  -> straight 128-bit copies,
//   * source contiguous along k    -> 128-bit loads, transposing stores.
// The 128-wide rows are XOR-swizzled in units of 8 floats by (k/4)&3, which
// makes the transposing stores hit 32 distinct banks and leaves every
// fragment a contiguous, aligned float4.
// The next K-slice is fetched into registers while the current one is being
// multiplied and written to the other shared buffer afterwards: one barrier
// per K-slice.
//
// Replaces gemm_fast/gemm_generic (src/gemm.cu:35-197), bgemm_k
// (src/bgemm.cu:16-84) and the fp32 registry kernels (src/kernels/k01..k08).
#include "common.cuh"

namespace bmb {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, NTHREADS = 256;

__device__ __forceinline__ int swz(int k) { return ((k >> 2) & 3) << 3; }

// Stage one 16 x 128 operand slice into registers.
//   KCONTIG = true : source element (x, k) at src[x*ld + k]  (A when !TA, B when TB)
//   KCONTIG = false: source element (x, k) at src[k*ld + x]  (A when TA,  B when !TB)
// x0 / k0 are the tile origin; X / Kdim the matrix extents along x and k.
template <bool KCONTIG, bool GUARD>
__device__ __forceinline__ void fetch_slice(float4 (&r)[2], const float *__restrict__ src,
                                            long long ld, int x0, int k0, int X, int Kdim, int tid) {
    if (KCONTIG) {
        // 128 rows x 4 float4 along k.  thread -> (row = tid/4 + 64*i, kq = (tid%4)*4)
        const int kq = (tid & 3) * 4;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int x = x0 + (tid >> 2) + 64 * i;
            const float *p = src + (long long)x * ld + (k0 + kq);
            if (!GUARD) {
                r[i] = *reinterpret_cast<const float4 *>(p);
            } else {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = (x < X && k0 + kq + j < Kdim) ? p[j] : 0.0f;
                r[i] = make_float4(v[0], v[1], v[2], v[3]);
            }
        }
    } else {
        // 16 k-rows x 32 float4 along x.  thread -> (k = tid/32 + 8*i, xq = (tid%32)*4)
        const int xq = (tid & 31) * 4;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int k = k0 + (tid >> 5) + 8 * i;
            const float *p = src + (long long)k * ld + (x0 + xq);
            if (!GUARD) {
                r[i] = *reinterpret_cast<const float4 *>(p);
            } else {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = (k < Kdim && x0 + xq + j < X) ? p[j] : 0.0f;
                r[i] = make_float4(v[0], v[1], v[2], v[3]);
            }
        }
    }
}

template <bool KCONTIG>
__device__ __forceinline__ void store_slice(float *__restrict__ s, const float4 (&r)[2], int tid) {
    if (KCONTIG) {
        const int kq = (tid & 3) * 4;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int x = (tid >> 2) + 64 * i;
            const int xs = x ^ swz(kq);   // same swizzle for kq..kq+3
            s[(kq + 0) * 128 + xs] = r[i].x;
            s[(kq + 1) * 128 + xs] = r[i].y;
            s[(kq + 2) * 128 + xs] = r[i].z;
            s[(kq + 3) * 128 + xs] = r[i].w;
        }
    } else {
        const int xq = (tid & 31) * 4;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int k = (tid >> 5) + 8 * i;
            *reinterpret_cast<float4 *>(&s[k * 128 + (xq ^ swz(k))]) = r[i];
        }
    }
}

// Two fp32 fused multiply-adds in one instruction (sm_100): each half is an IEEE fma.rn, so results
// are bit-identical to fmaf; it halves the issue slots the inner product needs.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void ffma2(unsigned long long &d, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

template <bool TA, bool TB, bool GUARD>
__global__ void __launch_bounds__(NTHREADS, 2)
gemm_simt_k(int M, int N, int K, float alpha, const float *__restrict__ A, long long sA,
            const float *__restrict__ B, long long sB, float beta, float *__restrict__ C,
            long long sC) {
    __shared__ __align__(16) float As[2][BK * BM];
    __shared__ __align__(16) float Bs[2][BK * BN];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    A += (long long)blockIdx.z * sA;
    B += (long long)blockIdx.z * sB;
    C += (long long)blockIdx.z * sC;

    // A: x = m.  !TA: element (m,k) at A[m*K + k] (k contiguous).  TA: A[k*M + m].
    // B: x = n.  !TB: element (k,n) at B[k*N + n].                 TB: B[n*K + k] (k contiguous).
    constexpr bool A_KC = !TA, B_KC = TB;
    const long long lda = TA ? M : K, ldb = TB ? K : N;

    // acc2[i][jp] holds columns 2*jp and 2*jp+1 of row i of the 8 x 8 micro-tile
    unsigned long long acc2[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[i][j] = 0ull;

    float4 ra[2], rb[2];
    fetch_slice<A_KC, GUARD>(ra, A, lda, m0, 0, M, K, tid);
    fetch_slice<B_KC, GUARD>(rb, B, ldb, n0, 0, N, K, tid);
    store_slice<A_KC>(As[0], ra, tid);
    store_slice<B_KC>(Bs[0], rb, tid);
    __syncthreads();

    // Swizzled fragment offsets for the four (k/4)&3 classes.
    int am[4], bn[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) { am[c] = (ty * 4) ^ (c << 3); bn[c] = (tx * 4) ^ (c << 3); }

    const int nk = (K + BK - 1) / BK;
    for (int kt = 0; kt < nk; ++kt) {
        const int cur = kt & 1;
        const bool more = (kt + 1 < nk);
        if (more) {
            fetch_slice<A_KC, GUARD>(ra, A, lda, m0, (kt + 1) * BK, M, K, tid);
            fetch_slice<B_KC, GUARD>(rb, B, ldb, n0, (kt + 1) * BK, N, K, tid);
        }
        const float *as = As[cur], *bs = Bs[cur];
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const int c = (k >> 2) & 3;
            const float4 a0 = *reinterpret_cast<const float4 *>(&as[k * 128 + am[c]]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&as[k * 128 + 64 + am[c]]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&bs[k * 128 + bn[c]]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&bs[k * 128 + 64 + bn[c]]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const unsigned long long bp[4] = {pack2(b0.x, b0.y), pack2(b0.z, b0.w), pack2(b1.x, b1.y), pack2(b1.z, b1.w)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned long long aa = pack2(av[i], av[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) ffma2(acc2[i][j], aa, bp[j]);
            }
        }
        if (more) {
            store_slice<A_KC>(As[cur ^ 1], ra, tid);
            store_slice<B_KC>(Bs[cur ^ 1], rb, tid);
        }
        __syncthreads();
    }

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack2(acc2[i][j], acc[i][2 * j], acc[i][2 * j + 1]);
    // Epilogue.  Rows ty*4+{0..3} and 64+ty*4+{0..3}; columns likewise in tx.
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
        if (GUARD && m >= M) continue;
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const int n = n0 + tx * 4 + jh * 64;
            float *cp = C + (long long)m * N + n;
            if (!GUARD) {
                float4 o = make_float4(alpha * acc[i][jh * 4 + 0], alpha * acc[i][jh * 4 + 1],
                                       alpha * acc[i][jh * 4 + 2], alpha * acc[i][jh * 4 + 3]);
                if (beta != 0.0f) {
                    const float4 c = *reinterpret_cast<const float4 *>(cp);
                    o.x = fmaf(beta, c.x, o.x); o.y = fmaf(beta, c.y, o.y);
                    o.z = fmaf(beta, c.z, o.z); o.w = fmaf(beta, c.w, o.w);
                }
                *reinterpret_cast<float4 *>(cp) = o;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (n + j < N) {
                        float o = alpha * acc[i][jh * 4 + j];
                        if (beta != 0.0f) o = fmaf(beta, cp[j], o);
                        cp[j] = o;
                    }
                }
            }
        }
    }
}

template <bool TA, bool TB>
int launch_simt(int batch, int M, int N, int K, float alpha, const float *A, long long sA,
                const float *B, long long sB, float beta, float *C, long long sC,
                cudaStream_t st) {
    const bool aligned = (M % BM == 0) && (N % BN == 0) && (K % BK == 0) &&
                         (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) % 16 == 0) &&
                         (sA % 4 == 0) && (sB % 4 == 0) && (sC % 4 == 0);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    if (grid.y > 65535 || grid.z > 65535) return fail(BMB_E_ARG, "gemm: grid too large (M=%d batch=%d)", M, batch);
    if (aligned)
        gemm_simt_k<TA, TB, false><<<grid, NTHREADS, 0, st>>>(M, N, K, alpha, A, sA, B, sB, beta, C, sC);
    else
        gemm_simt_k<TA, TB, true><<<grid, NTHREADS, 0, st>>>(M, N, K, alpha, A, sA, B, sB, beta, C, sC);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

// K == 0 or alpha == 0: C = beta*C.
__global__ void scale_c_k(float *C, long long n, float beta) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        C[i] = (beta == 0.0f) ? 0.0f : beta * C[i];
}

}  // namespace

int gemm_simt_tma(int transA, int transB, int batch, int M, int N, int K, float alpha, const float *A, long long sA,
                  const float *B, long long sB, float beta, float *C, long long sC, cudaStream_t st);

int gemm_simt(int transA, int transB, int batch, int M, int N, int K, float alpha, const float *A,
              long long sA, const float *B, long long sB, float beta, float *C, long long sC,
              cudaStream_t st) {
    if (M < 0 || N < 0 || K < 0 || batch < 0) return fail(BMB_E_ARG, "gemm: negative dimension");
    if (M == 0 || N == 0 || batch == 0) return BMB_OK;
    if (!C || (K > 0 && (!A || !B))) return fail(BMB_E_ARG, "gemm: null operand");
    if (K == 0) {
        for (int b = 0; b < batch; ++b) {
            scale_c_k<<<ceil_div((long long)M * N, 256) > 1184 ? 1184 : ceil_div((long long)M * N, 256), 256, 0, st>>>(
                C + (long long)b * sC, (long long)M * N, beta);
            count_launch();
        }
        BMB_LAUNCH_CHECK();
        return BMB_OK;
    }
    // NN and TN on aligned shapes: the kernel fed by the copy engine (gemm_simt_tma.cu)
    {
        const int rc = gemm_simt_tma(transA, transB, batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, st);
        if (rc != BMB_E_UNSUPPORTED) return rc;
    }
    if (!transA && !transB) return launch_simt<false, false>(batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, st);
    if (!transA && transB)  return launch_simt<false, true >(batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, st);
    if (transA && !transB)  return launch_simt<true,  false>(batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, st);
    return launch_simt<true, true>(batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, st);
}

}  // namespace bmb
