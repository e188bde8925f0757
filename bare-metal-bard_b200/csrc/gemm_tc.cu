// Tensor-core GEMM for sm_100a: tcgen05.mma with the accumulator in tensor
// memory, operands brought into 128-byte-swizzled shared memory by TMA.
//
//   C[M,N] = alpha * op(A) @ op(B) + beta * C        (fp32 in global memory)
//
// kind::tf32 multiplies fp32 operands of which the tensor core reads only the
// upper 19 bits; feeding it raw fp32 therefore truncates, which biases every
// product low by about 2^-10.  The reference rounds to nearest instead
// (src/kernels/k09_tensorcore.cu:119-128), so operands are first rounded with
// cvt.rna.tf32.f32 -- by the prepass below into per-device scratch, or by the
// caller (BMB_GEMM_A_ROUNDED / BMB_GEMM_B_ROUNDED), in which case a K-contiguous
// operand is read in place.  kind::f16 takes the same route with a bf16 copy.
//
// Kernel shape.  One persistent CTA per SM, 192 threads in three roles:
//   warp 0      producer: one lane issues the TMA loads of a K-slice
//               (A 128 x 128 B, B 256 x 128 B) into a 4-deep ring, each slice
//               armed on an mbarrier with its byte count;
//   warp 1      issuer: one lane waits for a slice, issues 4 tcgen05.mma
//               (128 x 256 x 32 B of K each) and commits them to the slice's
//               "empty" barrier; after the last slice of a tile it commits to
//               the accumulator's "full" barrier.  This warp also owns the
//               TMEM allocation (512 columns: two 128 x 256 fp32 accumulators,
//               so the epilogue of tile i overlaps the main loop of tile i+1);
//   warps 2..5  epilogue: each warp reads its 32 TMEM lanes 32 columns at a
//               time (tcgen05.ld 32x32b.x32), applies alpha/beta and stores.
// Both operand tiles are K-major in shared memory (rows of 128 bytes of K,
// SWIZZLE_128B), so a K step of 32 bytes is a +2 on the descriptor's address
// field.  Tiles are visited in groups of 8 M-tiles so that concurrently
// resident CTAs share A and B slices in L2.
//
// Every wait on an mbarrier is bounded: when a wait runs out, the CTA raises a
// flag all roles poll, the producer waits (bounded again) for the copies it
// has in flight, the TMEM allocation is released, and the kernel writes a
// nonzero word into a host-visible status that the next call reports as
// BMB_E_TIMEOUT.  No TMA load uses cluster multicast.
#include "common.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <mutex>

namespace bmb {
namespace {

constexpr int BM = 128, BN = 256, STAGES = 4, KBYTES = 128;
constexpr int A_BYTES = BM * KBYTES, B_BYTES = BN * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NTHREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr long long WAIT_CYCLES = 4000000000LL;  // about two seconds at 2 GHz

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *giveup) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*giveup) return false;
        if (clock64() - t0 > WAIT_CYCLES) { *giveup = 1; return false; }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int KIND>  // 0 = tf32, 1 = f16 (bf16 inputs)
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if (KIND == 0)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// K-major, SWIZZLE_128B shared-memory matrix descriptor: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

struct TileSched {
    int tiles_m, tiles_n, num_tiles;
    __device__ __forceinline__ void coords(int tile, int &tm, int &tn) const {
        constexpr int GM = 8;
        const int per_group = GM * tiles_n;
        const int g = tile / per_group, first_m = g * GM;
        const int gsz = min(GM, tiles_m - first_m);
        const int r = tile - g * per_group;
        tm = first_m + r % gsz;
        tn = r / gsz;
    }
};

template <int KIND>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_k(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, int M, int N,
          int kblocks, int kelems_per_block, float alpha, float beta, float *__restrict__ C, int vec_ok,
          int *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + STAGES * STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *giveup = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *armed = reinterpret_cast<int *>(tmem_slot + 2);   // [STAGES] parity last armed per slice, -1 = never

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;

    TileSched sch;
    sch.tiles_m = (M + BM - 1) / BM;
    sch.tiles_n = (N + BN - 1) / BN;
    sch.num_tiles = sch.tiles_m * sch.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); armed[s] = -1; }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        *giveup = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < sch.num_tiles; tile += gridDim.x) {
                int tm, tn;
                sch.coords(tile, tm, tn);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, giveup)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * s;
                    mbar_arrive_expect_tx(fb, STAGE_BYTES);
                    armed[s] = (int)ph;
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
                    tma_load_2d(sa, &mapA, kb * kelems_per_block, tm * BM, fb);
                    tma_load_2d(sb, &mapB, kb * kelems_per_block, tn * BN, fb);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            if (!ok) {
                // Leave no copy in flight behind us: every armed slice must land.
                for (int i = 0; i < STAGES; ++i) {
                    if (armed[i] < 0) continue;
                    const long long t0 = clock64();
                    while (!mbar_try_wait(full0 + 8 * i, (uint32_t)armed[i]) && clock64() - t0 < WAIT_CYCLES) {}
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- issuer
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, A/B format, both K-major, N = 256, M = 128
            const uint32_t fmt = (KIND == 0) ? 2u : 1u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int s = 0, acc = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < sch.num_tiles; tile += gridDim.x) {
                if (!mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, giveup)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(full0 + 8 * s, ph, giveup)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
                    const uint64_t da = smem_desc_kmajor(sa), db = smem_desc_kmajor(sb);
#pragma unroll
                    for (int k = 0; k < KBYTES / 32; ++k)
                        tc_mma<KIND>(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);          // slice reusable once these MMAs retire
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                tc_commit(tfull0 + 8 * acc);            // accumulator complete
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                          // TMEM lane quadrant this warp may read
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < sch.num_tiles; tile += gridDim.x) {
            int tm, tn;
            sch.coords(tile, tm, tn);
            if (!mbar_wait(tfull0 + 8 * acc, acc_ph, giveup)) { ok = false; break; }
            tc_fence_after();
            const int m = tm * BM + q * 32 + lane;
            const uint32_t trow = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
            float *crow = C + (size_t)m * N;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                float v[32];
                tmem_ld32(trow + (uint32_t)(c * 32), v);
                const int n0 = tn * BN + c * 32;
                if (m < M && n0 < N) {
                    if (vec_ok && n0 + 32 <= N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(alpha * v[j], alpha * v[j + 1], alpha * v[j + 2], alpha * v[j + 3]);
                            if (beta != 0.0f) {
                                const float4 cc = *reinterpret_cast<const float4 *>(crow + n0 + j);
                                o.x = fmaf(beta, cc.x, o.x); o.y = fmaf(beta, cc.y, o.y);
                                o.z = fmaf(beta, cc.z, o.z); o.w = fmaf(beta, cc.w, o.w);
                            }
                            *reinterpret_cast<float4 *>(crow + n0 + j) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (n0 + j < N) {
                                float o = alpha * v[j];
                                if (beta != 0.0f) o = fmaf(beta, crow[n0 + j], o);
                                crow[n0 + j] = o;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *giveup) {
        *reinterpret_cast<volatile int *>(status) = 1;
        __threadfence_system();
    }
}

// ---- operand prepass --------------------------------------------------------
// dst[r][k] (row pitch Kp elements) = round(src(r, k)), zero for k in [K, Kp).
// KCONTIG: src(r,k) = src[r*K + k]; otherwise src(r,k) = src[k*R + r].
template <typename OUT>
__device__ __forceinline__ OUT cvt_out(float x);
template <> __device__ __forceinline__ float cvt_out<float>(float x) { return round_tf32(x); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename OUT>
__global__ void prep_rows_k(OUT *__restrict__ dst, const float *__restrict__ src, long long R, int K, int Kp) {
    const long long total = R * (long long)Kp;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / Kp;
        const int k = (int)(i - r * Kp);
        dst[i] = cvt_out<OUT>(k < K ? src[r * K + k] : 0.0f);
    }
}
__global__ void prep_rows_vec4_k(float *__restrict__ dst, const float *__restrict__ src, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(src)[i];
        reinterpret_cast<float4 *>(dst)[i] = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
    }
}
template <typename OUT>
__global__ void prep_transpose_k(OUT *__restrict__ dst, const float *__restrict__ src, int R, int K, int Kp) {
    __shared__ float t[32][33];
    const int r0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int k = k0 + j, r = r0 + threadIdx.x;
        t[j][threadIdx.x] = (k < K && r < R) ? src[(size_t)k * R + r] : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int r = r0 + j, k = k0 + threadIdx.x;
        if (r < R && k < Kp) dst[(size_t)r * Kp + k] = cvt_out<OUT>(t[threadIdx.x][j]);
    }
}

// ---- host side ----------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                             const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeFn encode_fn() {
    std::call_once(g_encode_once, [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = (EncodeFn)fn;
    });
    return g_encode;
}

// rows x Kelems matrix, K contiguous, row pitch `pitch_bytes`; box = 128 bytes of K x box_rows rows.
int make_map(CUtensorMap *map, const void *ptr, int esize, long long rows, long long kelems, long long pitch_bytes,
             int box_rows) {
    EncodeFn enc = encode_fn();
    if (!enc) return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)kelems, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(KBYTES / esize), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return BMB_OK;
}

struct DevState { int *status_dev = nullptr; int *status_host = nullptr; bool attr_set[2] = {false, false}; };
DevState g_dev[64];
std::mutex g_dev_mu;

int dev_state(DevState **out) {
    const int d = current_device();
    if (d < 0 || d >= 64) return fail(BMB_E_ARG, "device index %d out of range", d);
    std::lock_guard<std::mutex> lk(g_dev_mu);
    DevState &s = g_dev[d];
    if (!s.status_host) {
        BMB_CUDA(cudaHostAlloc((void **)&s.status_host, sizeof(int), cudaHostAllocMapped));
        *s.status_host = 0;
        BMB_CUDA(cudaHostGetDevicePointer((void **)&s.status_dev, s.status_host, 0));
    }
    *out = &s;
    return BMB_OK;
}

template <typename OUT>
int prepare_operand(OUT *dst, const float *src, bool kcontig, long long R, int K, int Kp, cudaStream_t st) {
    if (kcontig) {
        if (sizeof(OUT) == 4 && Kp == K && ((uintptr_t)src % 16 == 0) && ((R * (long long)K) % 4 == 0)) {
            const long long n4 = R * (long long)K / 4;
            long long blocks = (n4 + 255) / 256;
            if (blocks > 8LL * sm_count()) blocks = 8LL * sm_count();
            prep_rows_vec4_k<<<(int)blocks, 256, 0, st>>>(reinterpret_cast<float *>(dst), src, n4);
        } else {
            long long blocks = (R * (long long)Kp + 255) / 256;
            if (blocks > 8LL * sm_count()) blocks = 8LL * sm_count();
            prep_rows_k<OUT><<<(int)blocks, 256, 0, st>>>(dst, src, R, K, Kp);
        }
    } else {
        dim3 grid((unsigned)((R + 31) / 32), (unsigned)((Kp + 31) / 32));
        prep_transpose_k<OUT><<<grid, dim3(32, 8), 0, st>>>(dst, src, (int)R, K, Kp);
    }
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace

bool gemm_tc_accepts(int math, int, int, int batch, int M, int N, int K, const float *, long long, const float *,
                     long long, const float *C, long long) {
    if (math != BMB_MATH_TF32 && math != BMB_MATH_BF16) return false;
    if (batch != 1) return false;                // batched problems stay on the SIMT kernel for now
    // Smaller problems than one tile stay on the SIMT kernel (still fp32-exact).
    if (M < BM || N < BN || K < 32 || !C) return false;
    if ((long long)M * K >= (1LL << 40) || (long long)N * K >= (1LL << 40)) return false;
    return true;
}

int gemm_tc(int math, int flags, int transA, int transB, int batch, int M, int N, int K, float alpha,
            const float *A, long long, const float *B, long long, float beta, float *C, long long,
            cudaStream_t st) {
    (void)batch;
    DevState *ds = nullptr;
    BMB_TRY(dev_state(&ds));
    if (*ds->status_host != 0)
        return fail(BMB_E_TIMEOUT, "an earlier tensor-core GEMM on this device gave up waiting on a barrier");
    const bool bf16 = (math == BMB_MATH_BF16);
    const int esize = bf16 ? 2 : 4;
    const int kalign = 16 / esize;                       // elements per 16 bytes
    const bool a_kc = !transA, b_kc = transB != 0;
    // In-place use of a caller's operand: TF32 only, K-contiguous, already rounded, TMA-aligned.
    const bool a_direct = !bf16 && a_kc && (flags & BMB_GEMM_A_ROUNDED) && K % 4 == 0 && (uintptr_t)A % 16 == 0;
    const bool b_direct = !bf16 && b_kc && (flags & BMB_GEMM_B_ROUNDED) && K % 4 == 0 && (uintptr_t)B % 16 == 0;
    const int Kp = (K + kalign - 1) / kalign * kalign;
    const void *pa = A, *pb = B;
    long long pitch_a = (long long)K * 4, pitch_b = (long long)K * 4;
    long long kel_a = K, kel_b = K;
    if (!a_direct) {
        void *sa = device_scratch(SCR_GEMM_A, (size_t)M * Kp * esize);
        if (!sa) return BMB_E_CUDA;
        if (bf16) BMB_TRY(prepare_operand<__nv_bfloat16>((__nv_bfloat16 *)sa, A, a_kc, M, K, Kp, st));
        else BMB_TRY(prepare_operand<float>((float *)sa, A, a_kc, M, K, Kp, st));
        pa = sa; pitch_a = (long long)Kp * esize; kel_a = Kp;
    }
    if (!b_direct) {
        void *sb = device_scratch(SCR_GEMM_B, (size_t)N * Kp * esize);
        if (!sb) return BMB_E_CUDA;
        if (bf16) BMB_TRY(prepare_operand<__nv_bfloat16>((__nv_bfloat16 *)sb, B, b_kc, N, K, Kp, st));
        else BMB_TRY(prepare_operand<float>((float *)sb, B, b_kc, N, K, Kp, st));
        pb = sb; pitch_b = (long long)Kp * esize; kel_b = Kp;
    }
    CUtensorMap mapA, mapB;
    BMB_TRY(make_map(&mapA, pa, esize, M, kel_a, pitch_a, BM));
    BMB_TRY(make_map(&mapB, pb, esize, N, kel_b, pitch_b, BN));
    const int kper = KBYTES / esize;
    const int kblocks = (K + kper - 1) / kper;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    const int vec_ok = ((uintptr_t)C % 16 == 0) && (N % 4 == 0);
    const int kind = bf16 ? 1 : 0;
    if (!ds->attr_set[kind]) {
        if (bf16) BMB_CUDA(cudaFuncSetAttribute(gemm_tc_k<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        else BMB_CUDA(cudaFuncSetAttribute(gemm_tc_k<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        ds->attr_set[kind] = true;
    }
    if (bf16)
        gemm_tc_k<1><<<grid, NTHREADS, SMEM_BYTES, st>>>(mapA, mapB, M, N, kblocks, kper, alpha, beta, C, vec_ok, ds->status_dev);
    else
        gemm_tc_k<0><<<grid, NTHREADS, SMEM_BYTES, st>>>(mapA, mapB, M, N, kblocks, kper, alpha, beta, C, vec_ok, ds->status_dev);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb
