// Tensor-core GEMM for sm_100a: tcgen05.mma with the accumulator in tensor
// memory, operands brought into 128-byte-swizzled shared memory by TMA.
//
//   C[M,N] = alpha * op(A) @ op(B) + beta * C        (fp32 in global memory)
//
// kind::tf32 multiplies fp32 operands of which the tensor core reads only the
// upper 19 bits; feeding it raw fp32 therefore truncates, which biases every
// product low (measured on B200: normwise 6.4e-4 against 2.6e-4 with rounding).
// The reference rounds to nearest (src/kernels/k09_tensorcore.cu:119-128), so
// operands are first rounded with cvt.rna.tf32.f32 -- by the prepass below
// into per-device scratch, or by the caller (BMB_GEMM_A_ROUNDED /
// BMB_GEMM_B_ROUNDED), in which case the operand is read where it lies.
// kind::f16 takes the prepass route with a bf16 copy.
//
// All four transpose cases run without a transposed copy: an operand stored
// with K contiguous becomes a K-major tile (rows of 128 bytes of K), one
// stored with M (or N) contiguous becomes an MN-major tile (one 128-byte row
// of M/N per K index, 32-wide chunks side by side; for 32-bit elements the
// tensor core takes this only in the 128-byte swizzle with 32-byte atoms),
// and the instruction descriptor says which.
//
// Kernel shape.  One persistent CTA per SM, 192 threads in three roles:
//   warp 0      producer: one lane issues the TMA loads of a K-slice (32 fp32
//               or 64 bf16 of K: A 16 KB, B 32 KB) into a 4-deep ring, each
//               slice armed on an mbarrier with its byte count;
//   warp 1      issuer: one lane waits for a slice, issues 4 tcgen05.mma
//               (128 x 256 x 32 bytes of K each) and commits them to the
//               slice's "empty" barrier; after the last slice of a tile it
//               commits to the accumulator's "full" barrier.  This warp owns
//               the TMEM allocation (512 columns: two 128 x 256 fp32
//               accumulators, so the epilogue of tile i overlaps the main loop
//               of tile i+1);
//   warps 2..5  epilogue: each warp reads its 32 TMEM lanes 32 columns at a
//               time (tcgen05.ld 32x32b.x32), applies alpha/beta and stores.
// Tiles are visited in groups of 8 M-tiles so that concurrently resident CTAs
// share A and B slices in L2.
//
// Every wait on an mbarrier is bounded: when one runs out, the CTA raises a
// flag all roles poll, the producer waits (bounded again) for the copies it
// has in flight, the TMEM allocation is released, and the kernel stores a
// nonzero word into a host-visible status that the next call reports as
// BMB_E_TIMEOUT.  No TMA load uses cluster multicast.
#include "tc_common.cuh"
#include <cuda_bf16.h>
#include <mutex>

namespace bmb {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, STAGES = 4, KBYTES = 128;
constexpr int A_BYTES = BM * KBYTES, B_BYTES = BN * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NTHREADS = 192;
constexpr int EPI_PITCH = 36;                       // floats per parked row: 32 + 4 keeps 128-bit accesses conflict-free
constexpr int EPI_BYTES = 4 * 32 * EPI_PITCH * 4;   // one 32 x 32 staging block per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + EPI_BYTES;
constexpr int CHUNK_BYTES = 32 * KBYTES;   // one MN-major chunk: 32 K rows x 128 bytes of M/N

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

// KIND 0 = tf32 (fp32 operands), 1 = f16 (bf16 operands, always K-major).
// a_mn / b_mn: the operand's tile is MN-major (TF32 only).
template <int KIND>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_k(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, int M, int N,
          int kblocks, int kelems_per_block, int a_mn, int b_mn, float alpha, float beta, float *__restrict__ C,
          int vec_ok, int nsplit, const float *__restrict__ bias, int round_c, int *__restrict__ status) {
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
    // Split-K: a work unit is (tile, split); split s covers K slices [s*kbs, min(kblocks, (s+1)*kbs)).
    const int num_units = sch.num_tiles * nsplit;
    const int kbs = (kblocks + nsplit - 1) / nsplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); armed[s] = -1; }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        *giveup = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x) {
                int tm, tn;
                sch.coords(unit / nsplit, tm, tn);
                const int kb0 = (unit % nsplit) * kbs, kb1 = min(kblocks, kb0 + kbs);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, giveup)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * s;
                    mbar_arrive_expect_tx(fb, STAGE_BYTES);
                    armed[s] = (int)ph;
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
                    const int k0 = kb * kelems_per_block;
                    if (a_mn) {
#pragma unroll 1
                        for (int c = 0; c < BM / 32; ++c) tma_load_2d(sa + c * CHUNK_BYTES, &mapA, tm * BM + c * 32, k0, fb);
                    } else {
                        tma_load_2d(sa, &mapA, k0, tm * BM, fb);
                    }
                    if (b_mn) {
#pragma unroll 1
                        for (int c = 0; c < BN / 32; ++c) tma_load_2d(sb + c * CHUNK_BYTES, &mapB, tn * BN + c * 32, k0, fb);
                    } else {
                        tma_load_2d(sb, &mapB, k0, tn * BN, fb);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            if (!ok) {
                // Leave no copy in flight behind us: every armed slice must land.
                for (int i = 0; i < STAGES; ++i)
                    if (armed[i] >= 0) mbar_drain(full0 + 8 * i, (uint32_t)armed[i]);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc(KIND == 0 ? 2u : 1u, a_mn ? 1u : 0u, b_mn ? 1u : 0u, BN, BM);
            // per 32-byte K step: K-major tiles move 32 bytes along the row, MN-major tiles move 8 K rows
            const uint32_t a_step = a_mn ? 1024u : 32u, b_step = b_mn ? 1024u : 32u;
            int s = 0, acc = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x) {
                if (!mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, giveup)) { ok = false; break; }
                fence_after();
                const uint32_t d = tmem_base + (uint32_t)(acc * BN);
                const int kb0 = (unit % nsplit) * kbs, kb1 = min(kblocks, kb0 + kbs);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full0 + 8 * s, ph, giveup)) { ok = false; break; }
                    fence_after();
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
                    for (int k = 0; k < KBYTES / 32; ++k) {
                        const uint64_t da = a_mn ? smem_desc_mnmajor32(sa + k * a_step, CHUNK_BYTES) : smem_desc_kmajor(sa + k * a_step);
                        const uint64_t db = b_mn ? smem_desc_mnmajor32(sb + k * b_step, CHUNK_BYTES) : smem_desc_kmajor(sb + k * b_step);
                        if (KIND == 0) mma_tf32(d, da, db, idesc, ((kb - kb0) | k) ? 1u : 0u);
                        else mma_f16(d, da, db, idesc, ((kb - kb0) | k) ? 1u : 0u);
                    }
                    commit(empty0 + 8 * s);             // slice reusable once these MMAs retire
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                commit(tfull0 + 8 * acc);               // accumulator complete
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                          // TMEM lane quadrant this warp may read
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int unit = blockIdx.x; ok && unit < num_units; unit += gridDim.x) {
            int tm, tn;
            sch.coords(unit / nsplit, tm, tn);
            const bool first_split = (unit % nsplit) == 0;
            if (!mbar_wait(tfull0 + 8 * acc, acc_ph, giveup)) { ok = false; break; }
            fence_after();
            // The accumulator leaves TMEM one row per thread; the rows are parked in shared memory and
            // written out four rows per instruction, each row segment a contiguous 128 bytes, so that
            // the global stores (loads of C, atomics) are fully coalesced.
            const int row_base = tm * BM + q * 32;
            const uint32_t trow = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
            float *stg = reinterpret_cast<float *>(gen + STAGES * STAGE_BYTES + 256) + (warp - 2) * (32 * EPI_PITCH);
            const int sub_r = lane >> 3, sub_c = (lane & 7) * 4;
            const bool add_bias = bias && (nsplit == 1 || first_split);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int n0 = tn * BN + c * 32;
                if (n0 >= N) break;                      // warp-uniform
                float v[32];
                tmem_ld32(trow + (uint32_t)(c * 32), v);
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(stg + lane * EPI_PITCH + j) =
                        make_float4(alpha * v[j], alpha * v[j + 1], alpha * v[j + 2], alpha * v[j + 3]);
                __syncwarp();
                const int n = n0 + sub_c;
                const bool vec = vec_ok && (n + 4 <= N);
                float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
                if (add_bias && vec) bb = *reinterpret_cast<const float4 *>(bias + n);
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const int row = rr * 4 + sub_r, m = row_base + row;
                    float4 o = *reinterpret_cast<const float4 *>(stg + row * EPI_PITCH + sub_c);
                    if (m >= M) continue;
                    float *cp = C + (size_t)m * N + n;
                    if (vec) {
                        o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                        if (nsplit > 1) {
                            // split-K: partial products are added into C (the host has applied beta already)
                            atomicAdd(reinterpret_cast<float4 *>(cp), o);
                        } else {
                            if (beta != 0.0f) {
                                const float4 cc = *reinterpret_cast<const float4 *>(cp);
                                o.x = fmaf(beta, cc.x, o.x); o.y = fmaf(beta, cc.y, o.y);
                                o.z = fmaf(beta, cc.z, o.z); o.w = fmaf(beta, cc.w, o.w);
                            }
                            if (round_c) o = make_float4(round_tf32(o.x), round_tf32(o.y), round_tf32(o.z), round_tf32(o.w));
                            *reinterpret_cast<float4 *>(cp) = o;
                        }
                    } else {
                        const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (n + e >= N) continue;
                            float x = ov[e] + (add_bias ? bias[n + e] : 0.0f);
                            if (nsplit > 1) { atomicAdd(cp + e, x); continue; }
                            if (beta != 0.0f) x = fmaf(beta, cp[e], x);
                            cp[e] = round_c ? round_tf32(x) : x;
                        }
                    }
                }
                __syncwarp();
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
    }

    fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *giveup) {
        *reinterpret_cast<volatile int *>(status) = 1;
        __threadfence_system();
    }
}

// ---- operand prepass --------------------------------------------------------
template <typename OUT>
__device__ __forceinline__ OUT cvt_out(float x);
template <> __device__ __forceinline__ float cvt_out<float>(float x) { return round_tf32(x); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// dst[r][k] (row pitch Kp) = convert(src[r*K + k]), zero for k in [K, Kp).
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
// Same-layout rounding copy of n4 float4.
__global__ void prep_round_vec4_k(float *__restrict__ dst, const float *__restrict__ src, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(src)[i];
        reinterpret_cast<float4 *>(dst)[i] = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
    }
}
// dst[r][k] (row pitch Kp) = convert(src[k*R + r]): transposing copy through shared memory.
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

struct Operand {
    const void *ptr;      // what the tensor map points at
    bool mn_major;        // tile layout
    long long rows, cols, pitch_bytes;   // tensor-map geometry (cols contiguous)
    int box_rows;
};

inline int blocks_for(long long items) {
    long long b = (items + 255) / 256, cap = 8LL * sm_count();
    return (int)(b > cap ? cap : (b < 1 ? 1 : b));
}

// Decide how an operand reaches the tensor core.  X = its M or N extent, kcontig =
// element (x,k) at src[x*K + k], otherwise at src[k*X + x].
int stage_operand(Operand *op, const float *src, bool kcontig, long long X, int K, bool bf16, bool rounded,
                  ScratchSlot slot, int tile_rows, cudaStream_t st) {
    const bool aligned = ((uintptr_t)src % 16) == 0;
    if (!bf16) {
        const bool geom_ok = aligned && (kcontig ? (K % 4 == 0) : (X % 4 == 0));
        if (geom_ok) {
            const float *use = src;
            if (!rounded) {
                float *scr = (float *)device_scratch(slot, (size_t)X * K * sizeof(float));
                if (!scr) return BMB_E_CUDA;
                const long long n4 = X * (long long)K / 4;
                prep_round_vec4_k<<<blocks_for(n4), 256, 0, st>>>(scr, src, n4);
                count_launch();
                BMB_LAUNCH_CHECK();
                use = scr;
            }
            op->ptr = use;
            op->mn_major = !kcontig;
            if (kcontig) { op->rows = X; op->cols = K; op->pitch_bytes = (long long)K * 4; op->box_rows = tile_rows; }
            else { op->rows = K; op->cols = X; op->pitch_bytes = X * 4; op->box_rows = 32; }
            return BMB_OK;
        }
    }
    // General route: a K-major, padded, converted copy.
    const int esize = bf16 ? 2 : 4, kalign = 16 / esize;
    const int Kp = (K + kalign - 1) / kalign * kalign;
    void *scr = device_scratch(slot, (size_t)X * Kp * esize);
    if (!scr) return BMB_E_CUDA;
    if (kcontig) {
        if (bf16) prep_rows_k<__nv_bfloat16><<<blocks_for(X * (long long)Kp), 256, 0, st>>>((__nv_bfloat16 *)scr, src, X, K, Kp);
        else prep_rows_k<float><<<blocks_for(X * (long long)Kp), 256, 0, st>>>((float *)scr, src, X, K, Kp);
    } else {
        dim3 grid((unsigned)((X + 31) / 32), (unsigned)((Kp + 31) / 32));
        if (bf16) prep_transpose_k<__nv_bfloat16><<<grid, dim3(32, 8), 0, st>>>((__nv_bfloat16 *)scr, src, (int)X, K, Kp);
        else prep_transpose_k<float><<<grid, dim3(32, 8), 0, st>>>((float *)scr, src, (int)X, K, Kp);
    }
    count_launch();
    BMB_LAUNCH_CHECK();
    op->ptr = scr; op->mn_major = false;
    op->rows = X; op->cols = Kp; op->pitch_bytes = (long long)Kp * esize; op->box_rows = tile_rows;
    return BMB_OK;
}

bool g_attr_set[64][2];
std::mutex g_attr_mu;

}  // namespace

bool gemm_tc_accepts(int math, int, int, int batch, int M, int N, int K, const float *, long long, const float *,
                     long long, const float *C, long long) {
    if (math != BMB_MATH_TF32 && math != BMB_MATH_BF16) return false;
    if (batch != 1) return false;                // batched problems stay on the SIMT kernel
    // Problems smaller than one tile stay on the SIMT kernel (fp32-exact, so within any tensor-core tolerance).
    if (M < BM || N < BN || K < 32 || !C) return false;
    if ((long long)M * K >= (1LL << 40) || (long long)N * K >= (1LL << 40)) return false;
    return true;
}

namespace {
__global__ void scale_c_k(float *C, long long n, float beta) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        C[i] *= beta;
}

// Number of K splits for a problem with `tiles` output tiles and `kblocks` K slices on `sms` SMs: the
// split count that minimises (waves of work units) x (slices per unit + a fixed per-unit cost).
int choose_split(int tiles, int kblocks, int sms) {
    if (tiles * 4 >= sms * 3 || kblocks < 16) return 1;
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= 16 && s * 8 <= kblocks; ++s) {
        const int kbs = (kblocks + s - 1) / s;
        if ((s - 1) * kbs >= kblocks) continue;            // an empty split
        const long long waves = (tiles * s + sms - 1) / sms;
        const long long cost = waves * (kbs + 6);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

}  // namespace

int gemm_tc(int math, int flags, int transA, int transB, int batch, int M, int N, int K, float alpha,
            const float *A, long long, const float *B, long long, float beta, float *C, long long,
            const float *bias, cudaStream_t st) {
    (void)batch;
    int *status_dev = nullptr;
    volatile int *status_host = nullptr;
    BMB_TRY(tc::status_word(&status_dev, &status_host));
    if (*status_host != 0)
        return fail(BMB_E_TIMEOUT, "an earlier tensor-core kernel on this device gave up waiting on a barrier");
    const bool bf16 = (math == BMB_MATH_BF16);
    Operand a, b;
    BMB_TRY(stage_operand(&a, A, !transA, M, K, bf16, (flags & BMB_GEMM_A_ROUNDED) != 0, SCR_GEMM_A, BM, st));
    BMB_TRY(stage_operand(&b, B, transB != 0, N, K, bf16, (flags & BMB_GEMM_B_ROUNDED) != 0, SCR_GEMM_B, BN, st));
    const int esize = bf16 ? 2 : 4;
    CUtensorMap mapA, mapB;
    BMB_TRY(make_map_2d(&mapA, a.ptr, esize, a.rows, a.cols, a.pitch_bytes, a.box_rows, a.mn_major));
    BMB_TRY(make_map_2d(&mapB, b.ptr, esize, b.rows, b.cols, b.pitch_bytes, b.box_rows, b.mn_major));
    const int kper = KBYTES / esize;
    const int kblocks = (K + kper - 1) / kper;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int vec_ok = ((uintptr_t)C % 16 == 0) && (N % 4 == 0);
    // Split-K when the tiles cannot fill the GPU (the dW products of a training step: few tiles, long K).
    // The partial products are added atomically, so the summation order -- not the result beyond fp32
    // rounding -- varies from run to run; BMB_GEMM_NO_SPLIT keeps one CTA per tile.
    int nsplit = (flags & BMB_GEMM_NO_SPLIT) ? 1 : choose_split(tiles, kblocks, sm_count());
    if (nsplit > 1) {
        if (beta == 0.0f) BMB_CUDA(cudaMemsetAsync(C, 0, (size_t)M * N * sizeof(float), st));
        else if (beta != 1.0f) {
            scale_c_k<<<blocks_for((long long)M * N), 256, 0, st>>>(C, (long long)M * N, beta);
            count_launch();
        }
    }
    const int units = tiles * nsplit;
    const int grid = units < sm_count() ? units : sm_count();
    const int round_c = (flags & BMB_GEMM_C_ROUNDED) && nsplit == 1 ? 1 : 0;
    const int kind = bf16 ? 1 : 0;
    {
        std::lock_guard<std::mutex> lk(g_attr_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !g_attr_set[d][kind]) {
            if (bf16) BMB_CUDA(cudaFuncSetAttribute(gemm_tc_k<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            else BMB_CUDA(cudaFuncSetAttribute(gemm_tc_k<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            g_attr_set[d][kind] = true;
        }
    }
    if (bf16)
        gemm_tc_k<1><<<grid, NTHREADS, SMEM_BYTES, st>>>(mapA, mapB, M, N, kblocks, kper, 0, 0, alpha, beta, C, vec_ok, nsplit, bias,
                                                        round_c, status_dev);
    else
        gemm_tc_k<0><<<grid, NTHREADS, SMEM_BYTES, st>>>(mapA, mapB, M, N, kblocks, kper, a.mn_major ? 1 : 0,
                                                        b.mn_major ? 1 : 0, alpha, beta, C, vec_ok, nsplit, bias, round_c, status_dev);
    if (nsplit > 1 && (flags & BMB_GEMM_C_ROUNDED)) {
        count_launch();
        BMB_LAUNCH_CHECK();
        return bmb_round_tf32(C, C, (size_t)M * N, (void *)st);
    }
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb
