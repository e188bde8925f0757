// fp32 SIMT GEMM fed by the copy engine: the NN and TN cases of C = alpha*op(A)@B + beta*C on
// aligned shapes (M, N multiples of 128, K a multiple of 32, 16-byte aligned dense operands).
//
// The register-staged kernel (gemm_simt.cu) brings every K slice through registers and a block-wide
// barrier: its FMA pipe idles while warps wait on global loads at the slice hand-over.  Here the
// operand slices arrive by TMA into a 3-deep shared-memory ring, each slot guarded by a pair of
// mbarriers, and the eight math warps issue nothing but shared-memory loads and fma.rn.f32x2:
//   * B (N contiguous) lands as [32 k][128 n], plain rows of 512 bytes: a thread's fragment is two
//     128-bit loads per k, and its values pair up along n for the packed multiply-add;
//   * A lands either as [32 k][128 m] (TN: M contiguous, read like B) or, when K is the contiguous
//     dimension (NN), as [128 m][32 k] in the 128-byte swizzle (16-byte units XOR row % 8): A is the
//     operand every packed multiply-add broadcasts, so reading it along k costs no repacking -- one
//     64-bit load per row per two k steps, conflict-free because rows four apart swizzle differently.
// No thread waits for a block-wide barrier in the main loop: a warp waits for a slot's "full"
// barrier, multiplies its 32 k steps and arrives on the slot's "empty" barrier; thread 0 re-arms and
// refills the slot that was emptied one iteration earlier, two slices (~8 us of arithmetic) ahead.
// The k order and the fused multiply-add are those of the register-staged kernel, so results are
// bit-identical to it and to the CPU oracle's sequential fmaf chain.
//
// Every mbarrier wait is bounded (tc_common.cuh); on expiry the CTA drains the copies it armed and
// raises the per-device status word.  No TMA load uses cluster multicast.
#include "tc_common.cuh"
#include <mutex>

namespace bmb {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3, NT = 256;
constexpr int TILE_BYTES = BM * BK * 4;                 // 16 KB per operand per slot
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 128 /*barriers*/;

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
__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds64(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

// A_KC: A is stored with K contiguous (the NN case); otherwise with M contiguous (TN).
template <bool A_KC>
__global__ void __launch_bounds__(NT, 2)
gemm_simt_tma_k(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                int M, int N, int K, float alpha, float beta, float *__restrict__ C, int *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + STAGES * STAGE_BYTES);       // [0..S) full, [S..2S) empty
    volatile int *giveup = reinterpret_cast<volatile int *>(bars + 2 * STAGES);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;

    const int tid = threadIdx.x, lane = tid & 31;
    const int tx = tid & 15, ty = tid >> 4;
    const int nk = K / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, NT / 32); }
        *giveup = 0;
        mbar_init_fence();
    }
    __syncthreads();

    // Thread 0 loads slice `kt` into slot kt % STAGES (armed on the slot's full barrier).
    auto load_slice = [&](int kt) {
        const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN, bi = blockIdx.z;
        // Row offsets of this problem inside the batch seen as one tall matrix.
        const int a_row0 = A_KC ? bi * M : bi * K, b_row0 = bi * K;
        const int s = kt % STAGES;
        const uint32_t fb = full0 + 8 * s, sa = base + s * STAGE_BYTES, sb = sa + TILE_BYTES;
        mbar_arrive_expect_tx(fb, STAGE_BYTES);
        if (A_KC) tma_load_2d(sa, &mapA, kt * BK, a_row0 + m0, fb);          // box 32 k x 128 m, swizzled rows of 128 B
        else tma_load_2d(sa, &mapA, m0, a_row0 + kt * BK, fb);               // box 128 m x 32 k, plain rows of 512 B
        tma_load_2d(sb, &mapB, n0, b_row0 + kt * BK, fb);                    // box 128 n x 32 k, plain rows of 512 B
    };
    int loaded = 0;
    if (tid == 0)
        for (; loaded < STAGES - 1 && loaded < nk; ++loaded) load_slice(loaded);

    unsigned long long acc2[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[i][j] = 0ull;

    // A fragment addressing (A_KC): rows ty*4+i and 64+ty*4+i; row % 8 = (ty & 1) * 4 + i for both halves.
    // The swizzle term of row ty*4+i is (k/4) ^ ((ty&1)*4 + i): its i part folds into compile-time offsets, its
    // ty part flips bit 6 of the byte offset, i.e. adds or subtracts 64 -- hence two base addresses per slot.
    const uint32_t a_row_off = (uint32_t)(ty * 4) * 128u, a_sw16 = (uint32_t)((ty & 1) * 64);
    const uint32_t frag_a = (uint32_t)(ty * 16), frag_b = (uint32_t)(tx * 16);   // byte offset of 4 floats in a [k][128] row
    bool ok = true;
    for (int kt = 0; kt < nk; ++kt) {
        const int s = kt % STAGES;
        const uint32_t par = (uint32_t)((kt / STAGES) & 1);
        if (tid == 0 && loaded < nk) {
            // the slot slice `loaded` goes into held slice loaded - STAGES = kt - 1: wait until all warps left it
            if (loaded >= STAGES && !mbar_wait(empty0 + 8 * (loaded % STAGES), (uint32_t)(((loaded / STAGES) - 1) & 1), giveup)) ok = false;
            if (ok) { load_slice(loaded); ++loaded; }
        }
        if (!mbar_wait(full0 + 8 * s, par, giveup)) { ok = false; }
        if (__any_sync(0xffffffffu, !ok) || *giveup) { ok = false; break; }
        const uint32_t sa = base + s * STAGE_BYTES, sb = sa + TILE_BYTES;
        if (A_KC) {
            const uint32_t pa = sa + a_row_off + a_sw16, qa = sa + a_row_off - a_sw16;
#pragma unroll 8                                    // (fully unrolled, the scheduler hoists loads until it spills)
            for (int kk = 0; kk < BK / 2; ++kk) {           // two k steps per round of A loads
                float2 a[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t cu = (uint32_t)(((kk >> 1) ^ (i & 3)) << 4);
                    const uint32_t off = (uint32_t)((i & 3) * 128 + (i >> 2) * 64 * 128 + (kk & 1) * 8) + cu;
                    a[i] = lds64(((cu & 64u) ? qa : pa) + off);
                }
#pragma unroll
                for (int dk = 0; dk < 2; ++dk) {
                    const uint32_t brow = sb + (uint32_t)((2 * kk + dk) * 512) + frag_b;
                    const float4 b0 = lds128(brow), b1 = lds128(brow + 256);
                    const unsigned long long bp[4] = {pack2(b0.x, b0.y), pack2(b0.z, b0.w), pack2(b1.x, b1.y), pack2(b1.z, b1.w)};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float av = dk ? a[i].y : a[i].x;
                        const unsigned long long aa = pack2(av, av);
#pragma unroll
                        for (int j = 0; j < 4; ++j) ffma2(acc2[i][j], aa, bp[j]);
                    }
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < BK; ++k) {
                const uint32_t arow = sa + (uint32_t)(k * 512) + frag_a, brow = sb + (uint32_t)(k * 512) + frag_b;
                const float4 a0 = lds128(arow), a1 = lds128(arow + 256);
                const float4 b0 = lds128(brow), b1 = lds128(brow + 256);
                const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const unsigned long long bp[4] = {pack2(b0.x, b0.y), pack2(b0.z, b0.w), pack2(b1.x, b1.y), pack2(b1.z, b1.w)};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const unsigned long long aa = pack2(av[i], av[i]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) ffma2(acc2[i][j], aa, bp[j]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);          // this warp has left the slot
    }
    // One vote for the whole CTA: a warp that got through its slices must not run ahead into the
    // epilogue while another gave up.
    if (!__syncthreads_and(ok && !*giveup)) {
        // Leave no copy in flight: every slice thread 0 armed must land before the CTA's memory goes away.
        if (tid == 0) {
            for (int kt = (loaded > STAGES ? loaded - STAGES : 0); kt < loaded; ++kt)
                mbar_drain(full0 + 8 * (kt % STAGES), (uint32_t)((kt / STAGES) & 1));
            *reinterpret_cast<volatile int *>(status) = 3;
            __threadfence_system();
        }
        return;
    }

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) unpack2(acc2[i][j], acc[i][2 * j], acc[i][2 * j + 1]);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    C += (size_t)blockIdx.z * M * N;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            float *cp = C + (size_t)m * N + (n0 + tx * 4 + jh * 64);
            float4 o = make_float4(alpha * acc[i][jh * 4 + 0], alpha * acc[i][jh * 4 + 1], alpha * acc[i][jh * 4 + 2], alpha * acc[i][jh * 4 + 3]);
            if (beta != 0.0f) {
                const float4 c = *reinterpret_cast<const float4 *>(cp);
                o.x = fmaf(beta, c.x, o.x); o.y = fmaf(beta, c.y, o.y); o.z = fmaf(beta, c.z, o.z); o.w = fmaf(beta, c.w, o.w);
            }
            *reinterpret_cast<float4 *>(cp) = o;
        }
    }
}

// Plain (unswizzled) 2-d map over a rows x cols fp32 matrix: box = box_cols x box_rows.
int make_map_plain(CUtensorMap *map, const void *ptr, long long rows, long long cols, int box_cols, int box_rows) {
    EncodeFn enc = encode_fn();
    if (!enc) return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled (plain) failed (%d) for %lld x %lld", (int)r, rows, cols);
    return BMB_OK;
}

bool g_attr[64][2];
std::mutex g_mu;

template <bool A_KC>
int launch(const CUtensorMap &mapA, const CUtensorMap &mapB, dim3 grid, int M, int N, int K, float alpha, float beta, float *C,
           int *status_dev, cudaStream_t st) {
    {
        std::lock_guard<std::mutex> lk(g_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !g_attr[d][A_KC ? 1 : 0]) {
            BMB_CUDA(cudaFuncSetAttribute(gemm_simt_tma_k<A_KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            g_attr[d][A_KC ? 1 : 0] = true;
        }
    }
    gemm_simt_tma_k<A_KC><<<grid, NT, SMEM_BYTES, st>>>(mapA, mapB, M, N, K, alpha, beta, C, status_dev);
    return BMB_OK;
}

}  // namespace

// The TMA-fed kernel for the shapes it takes; BMB_E_UNSUPPORTED (nothing launched, no error text)
// tells the caller to use the register-staged kernel.
int gemm_simt_tma(int transA, int transB, int batch, int M, int N, int K, float alpha, const float *A, long long sA,
                  const float *B, long long sB, float beta, float *C, long long sC, cudaStream_t st) {
    static const bool off = getenv("BMB_SIMT_NO_TMA") != nullptr;
    if (off || transB || M % BM || N % BN || K % BK || K < BK || batch < 1) return BMB_E_UNSUPPORTED;
    if ((((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) != 0) return BMB_E_UNSUPPORTED;
    if (batch > 1 && (sA != (long long)M * K || sB != (long long)K * N || sC != (long long)M * N)) return BMB_E_UNSUPPORTED;
    if (M / BM > 65535 || batch > 65535 || (long long)batch * (M > K ? M : K) >= (1LL << 31)) return BMB_E_UNSUPPORTED;
    if (!encode_fn()) return BMB_E_UNSUPPORTED;
    int *status_dev = nullptr;
    volatile int *status_host = nullptr;
    BMB_TRY(status_word(&status_dev, &status_host));
    if (*status_host != 0) return fail(BMB_E_TIMEOUT, "an earlier kernel on this device gave up waiting on a barrier");
    CUtensorMap mapA, mapB;
    if (!transA) BMB_TRY(make_map_2d(&mapA, A, 4, (long long)batch * M, K, (long long)K * 4, BM, false));   // [M][K]: 128-byte swizzled rows of 32 k
    else BMB_TRY(make_map_plain(&mapA, A, (long long)batch * K, M, BM, BK));                                // [K][M]
    BMB_TRY(make_map_plain(&mapB, B, (long long)batch * K, N, BN, BK));                                     // [K][N]
    dim3 grid(N / BN, M / BM, batch);
    if (!transA) BMB_TRY(launch<true>(mapA, mapB, grid, M, N, K, alpha, beta, C, status_dev, st));
    else BMB_TRY(launch<false>(mapA, mapB, grid, M, N, K, alpha, beta, C, status_dev, st));
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb
