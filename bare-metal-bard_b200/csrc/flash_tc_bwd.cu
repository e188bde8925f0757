// Fused causal attention backward on the tensor cores (head size 64), two
// kernels as in the reference (src/flash.cu:434-470): dQ reduces over keys,
// dK and dV reduce over queries, so each keeps its accumulators on chip -- here
// in tensor memory -- and writes its part of dqkv with plain stores.
// P is rebuilt from the saved lse, P = exp(S - lse), and
// dS = P * (dP - D) with D = rowsum(dO * O)   (src/flash.cu:447-453).
//
// dQ kernel: a CTA owns 128 queries and walks key blocks of 64 up to the
//   diagonal.  Per block the issuer forms S = Q K^T and dP = dO V^T in TMEM
//   (double buffered, so block j+1 is being multiplied while block j is in the
//   registers); 256 threads -- a row of 128 per 32-column half -- turn them
//   into dS, rounded to TF32 and written back over dP in tensor memory, which
//   dQ += dS K (accumulated in TMEM over the whole walk) reads as its A operand.
// dK/dV kernel: a CTA owns 128 keys and walks query blocks of 64 from the
//   diagonal to the end, with everything transposed so that the owned keys are
//   again the rows: S^T = K Q^T, dP^T = V dO^T, P^T and dS^T written back in
//   place, then dV += P^T dO and dK += dS^T Q accumulate in TMEM.  lse and D
//   now vary along the columns; those of the whole walk sit in shared memory.
// K (dQ kernel) and Q, dO (dK/dV kernel) serve twice, once as a K-major operand
// and once with the head dimension as N, i.e. MN-major; the two uses need
// different swizzles (128-byte, and 128-byte with 32-byte atoms), so TMA brings
// each of those tiles in twice, into separate rings that are refilled as soon
// as their own consumer is done.
// Products are TF32 with fp32 accumulation; the exponentials, the subtraction
// of D and the scaling are fp32.  Waits are bounded as in the other kernels.
#include "tc_common.cuh"
#include <cmath>
#include <mutex>

namespace bmb {
int launch_flash_dsum(float *dsum, const float *dout, const float *out, int B, int T, int NH, int HS, cudaStream_t st);

namespace {

using namespace tc;

constexpr int HS = 64;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float4 out4(float a, float b, float c, float d, int rnd) {
    return rnd ? make_float4(round_tf32(a), round_tf32(b), round_tf32(c), round_tf32(d)) : make_float4(a, b, c, d);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

#ifdef BMB_FLASH_TRACE
__device__ long long g_trace_bwd[16];
#define TRB(i) do { if (tr) { const long long now_ = clock64(); g_trace_bwd[i] += now_ - tlast; tlast = now_; } } while (0)
#else
#define TRB(i)
#endif

// ============================================================== dQ kernel
namespace dq {
constexpr int QT = 128, KB = 64, STAGES = 3;
constexpr int OFF_Q = 0, OFF_DO = 32768;
constexpr int OFF_KK = 65536, KK_BYTES = 32768;         // per stage: K then V, K-major, 16 KB each
constexpr int OFF_KN = OFF_KK + STAGES * KK_BYTES;      // per stage: K, MN-major, 16 KB
constexpr int KN_BYTES = 16384;
constexpr int OFF_BAR = OFF_KN + STAGES * KN_BYTES;
constexpr int SMEM = OFF_BAR + 256 + 1024;
constexpr int THREADS = 320;
enum { Q_FULL = 0, KK_FULL = 1, KK_EMPTY = 4, KN_FULL = 7, KN_EMPTY = 10, SP_FULL = 13, DS_FULL = 15, DQ_DONE = 17, NBARS = 18 };
// TMEM columns: S [2] at 0 / 64, dP / dS [2] at 128 / 192, dQ at 256
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 256;
}  // namespace dq

// A CTA owns 128 queries and walks key blocks of 64 up to the diagonal.  S = Q K^T and dP = dO V^T
// land in tensor memory (double buffered); 256 threads (a query row each, 32 of the 64 key columns)
// turn them into dS, written back over dP, where the tensor core reads it as the A operand of
// dQ += dS K.  The K-major copies of a key block (K and V: operands of the first two products) and
// the MN-major copy of K (operand of the last) ride in separate 3-deep rings, each refilled as soon
// as its own consumer is done.
__global__ void __launch_bounds__(dq::THREADS, 1)
flash_bwd_dq_tc_k(const __grid_constant__ CUtensorMap mapQKV_k, const __grid_constant__ CUtensorMap mapQKV_n,
                  const __grid_constant__ CUtensorMap mapDO_k, float *__restrict__ dqkv,
                  const float *__restrict__ lse, const float *__restrict__ dsum, int T, int NH, float scale,
                  int round_out, int *__restrict__ status) {
    using namespace dq;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + OFF_BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    volatile int *giveup = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [bar0](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.x, b = bh / NH, h = bh % NH;
    const int C = NH * HS;
    const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * QT;   // CTAs are dispatched x first: every head's longest tile, then the next
    const int nb = min(T - 1, q0 + QT - 1) / KB + 1;       // key blocks up to the diagonal

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar(KK_FULL + s), 1); mbar_init(bar(KK_EMPTY + s), 1);
            mbar_init(bar(KN_FULL + s), 1); mbar_init(bar(KN_EMPTY + s), 1);
        }
        for (int s = 0; s < 2; ++s) { mbar_init(bar(SP_FULL + s), 1); mbar_init(bar(DS_FULL + s), 8); }
        mbar_init(bar(DQ_DONE), 1);
        *giveup = 0;
        mbar_init_fence();
    }
    if (warp == 9) tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            const int row0 = b * T;
            mbar_arrive_expect_tx(bar(Q_FULL), 65536);
            for (int half = 0; half < 2; ++half)
                for (int rr = 0; rr < 2; ++rr) {
                    tma_load_2d(base + OFF_Q + half * 16384 + rr * 8192, &mapQKV_k, h * HS + half * 32, row0 + q0 + rr * 64, bar(Q_FULL));
                    tma_load_2d(base + OFF_DO + half * 16384 + rr * 8192, &mapDO_k, h * HS + half * 32, row0 + q0 + rr * 64, bar(Q_FULL));
                }
            bool ok = true;
            int armed_k[STAGES], armed_n[STAGES];
            for (int s = 0; s < STAGES; ++s) { armed_k[s] = -1; armed_n[s] = -1; }
            for (int j = 0; j < nb; ++j) {
                const int st = j % STAGES;
                const uint32_t ph = (uint32_t)((j / STAGES) & 1);
                if (!mbar_wait(bar(KK_EMPTY + st), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(KK_FULL + st), KK_BYTES);
                armed_k[st] = (int)ph;
                const uint32_t sk = base + OFF_KK + st * KK_BYTES;
                for (int half = 0; half < 2; ++half) {
                    tma_load_2d(sk + half * 8192, &mapQKV_k, C + h * HS + half * 32, row0 + j * KB, bar(KK_FULL + st));
                    tma_load_2d(sk + 16384 + half * 8192, &mapQKV_k, 2 * C + h * HS + half * 32, row0 + j * KB, bar(KK_FULL + st));
                }
                if (!mbar_wait(bar(KN_EMPTY + st), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(KN_FULL + st), KN_BYTES);
                armed_n[st] = (int)ph;
                const uint32_t sn = base + OFF_KN + st * KN_BYTES;
                for (int half = 0; half < 2; ++half)
                    tma_load_2d(sn + half * 8192, &mapQKV_n, C + h * HS + half * 32, row0 + j * KB, bar(KN_FULL + st));
            }
            if (!ok) {
                mbar_drain(bar(Q_FULL), 0);
                for (int s = 0; s < STAGES; ++s) {
                    if (armed_k[s] >= 0) mbar_drain(bar(KK_FULL + s), (uint32_t)armed_k[s]);
                    if (armed_n[s] >= 0) mbar_drain(bar(KN_FULL + s), (uint32_t)armed_n[s]);
                }
            }
        }
    } else if (warp == 9) {
        // -------------------------------------------------------------- issuer
        if (lane == 0) {
            const uint32_t idesc_kk = make_idesc(2, 0, 0, KB, QT);     // [128 x 64] = A(K-major) x B(K-major)
            const uint32_t idesc_kn = make_idesc(2, 0, 1, HS, QT);     // dQ: dS (tensor memory) x K (MN-major)
            auto issue_sp = [&](int st, int buf) {
                const uint32_t sk = base + OFF_KK + st * KK_BYTES;
#pragma unroll
                for (int ks = 0; ks < HS / 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    mma_tf32(tmem_base + COL_S + (uint32_t)(buf * 64), smem_desc_kmajor(base + OFF_Q + half * 16384 + off),
                             smem_desc_kmajor(sk + half * 8192 + off), idesc_kk, ks ? 1u : 0u);
                }
#pragma unroll
                for (int ks = 0; ks < HS / 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    mma_tf32(tmem_base + COL_DP + (uint32_t)(buf * 64), smem_desc_kmajor(base + OFF_DO + half * 16384 + off),
                             smem_desc_kmajor(sk + 16384 + half * 8192 + off), idesc_kk, ks ? 1u : 0u);
                }
            };
            bool ok = mbar_wait(bar(Q_FULL), 0, giveup);
            if (ok) ok = mbar_wait(bar(KK_FULL + 0), 0, giveup);
            if (ok) { fence_after(); issue_sp(0, 0); commit(bar(SP_FULL + 0)); commit(bar(KK_EMPTY + 0)); }
            for (int j = 0; ok && j < nb; ++j) {
                const int st = j % STAGES, buf = j & 1;
                if (j + 1 < nb) {
                    // block j+1 goes into the other S / dP buffer; the product that read that buffer's dS
                    // (block j-1) was issued before this point, and the tensor core runs in order
                    const int s1 = (j + 1) % STAGES;
                    if (!mbar_wait(bar(KK_FULL + s1), (uint32_t)(((j + 1) / STAGES) & 1), giveup)) { ok = false; break; }
                    fence_after();
                    issue_sp(s1, (j + 1) & 1);
                    commit(bar(SP_FULL + ((j + 1) & 1)));
                    commit(bar(KK_EMPTY + s1));
                }
                if (!mbar_wait(bar(KN_FULL + st), (uint32_t)((j / STAGES) & 1), giveup)) { ok = false; break; }
                if (!mbar_wait(bar(DS_FULL + buf), (uint32_t)((j >> 1) & 1), giveup)) { ok = false; break; }
                fence_after();
                const uint32_t kn = base + OFF_KN + st * KN_BYTES;
#pragma unroll
                for (int ks = 0; ks < KB / 8; ++ks)
                    mma_tf32_ts(tmem_base + COL_DQ, tmem_base + COL_DP + (uint32_t)(buf * 64 + ks * 8),
                                smem_desc_mnmajor32(kn + ks * 1024, 8192), idesc_kn, (j | ks) ? 1u : 0u);
                commit(bar(KN_EMPTY + st));
            }
            if (ok) commit(bar(DQ_DONE));
        }
    } else {
        // ----------------------------------------------------------------- dS
        const int quad = warp & 3, colhalf = warp >> 2;
        const int r = quad * 32 + lane;
        const int qi = q0 + r;
        const float lse_r = (qi < T) ? lse[(size_t)bh * T + qi] * LOG2E : 0.0f;
        const float d_r = (qi < T) ? dsum[(size_t)bh * T + qi] : 0.0f;
        const float scale_log2e = scale * LOG2E;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        bool ok = true;
#ifdef BMB_FLASH_TRACE
        const bool tr = (blockIdx.x == 0 && blockIdx.y == 0 && warp == 0 && lane == 0);
        long long tlast = clock64();
#endif
        for (int j = 0; j < nb; ++j) {
            const int buf = j & 1;
            TRB(0);
            if (!mbar_wait(bar(SP_FULL + buf), (uint32_t)((j >> 1) & 1), giveup)) { ok = false; break; }
            fence_after();
            TRB(1);
            float s[32], dp[32];
            const uint32_t dp_addr = lane_addr + COL_DP + (uint32_t)(buf * 64 + colhalf * 32);
            tmem_ld32_nowait(lane_addr + COL_S + (uint32_t)(buf * 64 + colhalf * 32), s);
            tmem_ld32_nowait(dp_addr, dp);
            tmem_wait_ld();
            TRB(2);
            const int k0 = j * KB + colhalf * 32;
            const bool diag = (k0 + 31 > q0);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float p = fast_exp2(fmaf(s[i], scale_log2e, -lse_r));
                if (diag && (k0 + i > qi)) p = 0.0f;
                s[i] = round_tf32_alu(p * (dp[i] - d_r));
            }
            TRB(3);
            tmem_st32_nowait(dp_addr, s);                 // dS over dP: the A operand of dQ += dS K
            tmem_wait_st();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(DS_FULL + buf));
            TRB(4);
#ifdef BMB_FLASH_TRACE
            if (tr) g_trace_bwd[8] += 1;
#endif
        }
        if (ok && mbar_wait(bar(DQ_DONE), 0, giveup)) {
            fence_after();
            float v[32];
            tmem_ld32(lane_addr + COL_DQ + (uint32_t)(colhalf * 32), v);
            if (qi < T) {
                float *dst = dqkv + ((size_t)b * T + qi) * 3 * C + h * HS + colhalf * 32;
#pragma unroll
                for (int d = 0; d < 32; d += 4)
                    *reinterpret_cast<float4 *>(dst + d) = out4(v[d] * scale, v[d + 1] * scale, v[d + 2] * scale, v[d + 3] * scale, round_out);
            }
        }
    }

    fence_before();
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *giveup) {
        *reinterpret_cast<volatile int *>(status) = 3;
        __threadfence_system();
    }
}

// ============================================================ dK/dV kernel
namespace dkv {
constexpr int KT = 128, QB = 64, STAGES = 2;
constexpr int OFF_K = 0, OFF_V = 32768;
constexpr int OFF_STK = 65536, STK_BYTES = 32768;       // per stage: Q then dO, K-major, 16 KB each
constexpr int OFF_STN = OFF_STK + STAGES * STK_BYTES;   // per stage: Q then dO, MN-major, 16 KB each
constexpr int STN_BYTES = 32768;
constexpr int OFF_BAR = OFF_STN + STAGES * STN_BYTES;
constexpr int STAT_MAX = 4096;                          // queries whose lse and D fit in shared memory
constexpr int OFF_STAT = OFF_BAR + 256;                 // lse * log2(e), then D, STAT_MAX floats each
constexpr int SMEM = OFF_STAT + 2 * STAT_MAX * 4 + 1024;
constexpr int THREADS = 320;
enum { KV_FULL = 0, STK_FULL = 1, STK_EMPTY = 3, STN_FULL = 5, STN_EMPTY = 7, SP_FULL = 9, PD_FULL = 11, ACC_DONE = 13, NBARS = 14 };
// TMEM columns: S^T / P^T [2] at 0 / 64, dP^T / dS^T [2] at 128 / 192, dV at 256, dK at 320
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 320;
}  // namespace dkv

// A CTA owns 128 keys and walks query blocks of 64 from the diagonal to the end.  S^T = K Q^T and
// dP^T = V dO^T land in tensor memory; 256 threads (a key row each, 32 of the 64 query columns)
// turn them into P^T and dS^T and write those back over S^T and dP^T, where the tensor core reads
// them as the A operand of dV += P^T dO and dK += dS^T Q.  Nothing of the (T x T) matrices touches
// shared memory.  The K-major copies of a query block (operands of the first two products) and its
// MN-major copies (operands of the last two) ride in separate 2-deep rings, so each is refilled as
// soon as its own consumers are done.
__global__ void __launch_bounds__(dkv::THREADS, 1)
flash_bwd_dkv_tc_k(const __grid_constant__ CUtensorMap mapQKV_k64, const __grid_constant__ CUtensorMap mapQKV_n64,
                   const __grid_constant__ CUtensorMap mapDO_k64, const __grid_constant__ CUtensorMap mapDO_n64,
                   float *__restrict__ dqkv, const float *__restrict__ lse, const float *__restrict__ dsum,
                   int T, int NH, float scale, int round_out, int *__restrict__ status) {
    using namespace dkv;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + OFF_BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    volatile int *giveup = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [bar0](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.x, b = bh / NH, h = bh % NH;
    const int C = NH * HS;
    const int j0 = (int)blockIdx.y * KT;                   // first key of this CTA (earliest keys walk longest)
    const int ib0 = j0 / QB;                               // first query block that can see these keys
    const int nb = (T + QB - 1) / QB - ib0;                // query blocks to walk

    if (threadIdx.x == 0) {
        mbar_init(bar(KV_FULL), 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar(STK_FULL + s), 1); mbar_init(bar(STK_EMPTY + s), 1);
            mbar_init(bar(STN_FULL + s), 1); mbar_init(bar(STN_EMPTY + s), 1);
            mbar_init(bar(SP_FULL + s), 1); mbar_init(bar(PD_FULL + s), 8);
        }
        mbar_init(bar(ACC_DONE), 1);
        *giveup = 0;
        mbar_init_fence();
    }
    if (warp == 9) tmem_alloc(smem_u32(tmem_slot), 512);
    // Every thread needs the lse and D of every query the CTA walks: park them in shared memory once
    // (zero beyond the end of the sequence), lse already in log2 units.
    float *stat_l = reinterpret_cast<float *>(gen + OFF_STAT), *stat_d = stat_l + STAT_MAX;
    const int nstat = nb * QB;
    const bool stats_in_smem = nstat <= STAT_MAX;
    if (stats_in_smem) {
        for (int i = threadIdx.x; i < nstat; i += blockDim.x) {
            const int q = ib0 * QB + i;
            stat_l[i] = (q < T) ? __ldg(lse + (size_t)bh * T + q) * LOG2E : 0.0f;
            stat_d[i] = (q < T) ? __ldg(dsum + (size_t)bh * T + q) : 0.0f;
        }
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            const int row0 = b * T;
            mbar_arrive_expect_tx(bar(KV_FULL), 65536);
            for (int half = 0; half < 2; ++half)
                for (int rr = 0; rr < 2; ++rr) {
                    tma_load_2d(base + OFF_K + half * 16384 + rr * 8192, &mapQKV_k64, C + h * HS + half * 32, row0 + j0 + rr * 64, bar(KV_FULL));
                    tma_load_2d(base + OFF_V + half * 16384 + rr * 8192, &mapQKV_k64, 2 * C + h * HS + half * 32, row0 + j0 + rr * 64, bar(KV_FULL));
                }
            bool ok = true;
            int armed_k[STAGES] = {-1, -1}, armed_n[STAGES] = {-1, -1};
            for (int i = 0; i < nb; ++i) {
                const int st = i % STAGES;
                const uint32_t ph = (uint32_t)((i / STAGES) & 1);
                const int qrow = row0 + (ib0 + i) * QB;
                if (!mbar_wait(bar(STK_EMPTY + st), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(STK_FULL + st), STK_BYTES);
                armed_k[st] = (int)ph;
                const uint32_t sk = base + OFF_STK + st * STK_BYTES;
                for (int half = 0; half < 2; ++half) {
                    tma_load_2d(sk + half * 8192, &mapQKV_k64, h * HS + half * 32, qrow, bar(STK_FULL + st));
                    tma_load_2d(sk + 16384 + half * 8192, &mapDO_k64, h * HS + half * 32, qrow, bar(STK_FULL + st));
                }
                if (!mbar_wait(bar(STN_EMPTY + st), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(STN_FULL + st), STN_BYTES);
                armed_n[st] = (int)ph;
                const uint32_t sn = base + OFF_STN + st * STN_BYTES;
                for (int half = 0; half < 2; ++half) {
                    tma_load_2d(sn + half * 8192, &mapQKV_n64, h * HS + half * 32, qrow, bar(STN_FULL + st));
                    tma_load_2d(sn + 16384 + half * 8192, &mapDO_n64, h * HS + half * 32, qrow, bar(STN_FULL + st));
                }
            }
            if (!ok) {
                mbar_drain(bar(KV_FULL), 0);
                for (int s = 0; s < STAGES; ++s) {
                    if (armed_k[s] >= 0) mbar_drain(bar(STK_FULL + s), (uint32_t)armed_k[s]);
                    if (armed_n[s] >= 0) mbar_drain(bar(STN_FULL + s), (uint32_t)armed_n[s]);
                }
            }
        }
    } else if (warp == 9) {
        // -------------------------------------------------------------- issuer
        if (lane == 0) {
            const uint32_t idesc_st = make_idesc(2, 0, 0, QB, KT);     // [128 keys x 64 queries], both operands K-major
            const uint32_t idesc_acc = make_idesc(2, 0, 1, HS, KT);    // [128 keys x 64] = A (tensor memory) x B (MN-major)
            auto issue_sp = [&](int st) {
                const uint32_t sk = base + OFF_STK + st * STK_BYTES;
#pragma unroll
                for (int ks = 0; ks < HS / 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    mma_tf32(tmem_base + COL_S + (uint32_t)(st * 64), smem_desc_kmajor(base + OFF_K + half * 16384 + off),
                             smem_desc_kmajor(sk + half * 8192 + off), idesc_st, ks ? 1u : 0u);
                }
#pragma unroll
                for (int ks = 0; ks < HS / 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    mma_tf32(tmem_base + COL_DP + (uint32_t)(st * 64), smem_desc_kmajor(base + OFF_V + half * 16384 + off),
                             smem_desc_kmajor(sk + 16384 + half * 8192 + off), idesc_st, ks ? 1u : 0u);
                }
            };
            bool ok = mbar_wait(bar(KV_FULL), 0, giveup);
            if (ok && nb > 0) ok = mbar_wait(bar(STK_FULL + 0), 0, giveup);
            if (ok && nb > 0) {
                fence_after();
                issue_sp(0);
                commit(bar(SP_FULL + 0));
                commit(bar(STK_EMPTY + 0));
            }
            for (int i = 0; ok && i < nb; ++i) {
                const int st = i & 1;
                const uint32_t ph = (uint32_t)((i >> 1) & 1);
                if (i + 1 < nb) {
                    // block i+1 goes into the other S^T / dP^T buffer; the products that read that buffer's
                    // P^T / dS^T (block i-1) were issued before this point, and the tensor core runs in order
                    const int s1 = (i + 1) & 1;
                    if (!mbar_wait(bar(STK_FULL + s1), (uint32_t)(((i + 1) >> 1) & 1), giveup)) { ok = false; break; }
                    fence_after();
                    issue_sp(s1);
                    commit(bar(SP_FULL + s1));
                    commit(bar(STK_EMPTY + s1));
                }
                if (!mbar_wait(bar(STN_FULL + st), ph, giveup)) { ok = false; break; }
                if (!mbar_wait(bar(PD_FULL + st), ph, giveup)) { ok = false; break; }
                fence_after();
                const uint32_t sn = base + OFF_STN + st * STN_BYTES;
#pragma unroll
                for (int ks = 0; ks < QB / 8; ++ks)       // dV += P^T dO
                    mma_tf32_ts(tmem_base + COL_DV, tmem_base + COL_S + (uint32_t)(st * 64 + ks * 8),
                                smem_desc_mnmajor32(sn + 16384 + ks * 1024, 8192), idesc_acc, (i | ks) ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < QB / 8; ++ks)       // dK += dS^T Q
                    mma_tf32_ts(tmem_base + COL_DK, tmem_base + COL_DP + (uint32_t)(st * 64 + ks * 8),
                                smem_desc_mnmajor32(sn + ks * 1024, 8192), idesc_acc, (i | ks) ? 1u : 0u);
                commit(bar(STN_EMPTY + st));
            }
            if (ok) commit(bar(ACC_DONE));
        }
    } else {
        // ------------------------------------------------------- P^T and dS^T
        const int quad = warp & 3, colhalf = warp >> 2;
        const int r = quad * 32 + lane;
        const int kj = j0 + r;                             // this thread's key
        const float scale_log2e = scale * LOG2E;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        bool ok = true;
#ifdef BMB_FLASH_TRACE
        const bool tr = (blockIdx.x == 0 && blockIdx.y == 0 && warp == 0 && lane == 0);
        long long tlast = clock64();
#endif
        for (int i = 0; i < nb; ++i) {
            const int buf = i & 1;
            const int qc0 = (ib0 + i) * QB + colhalf * 32;     // first query column of this thread
            TRB(9);
            if (!mbar_wait(bar(SP_FULL + buf), (uint32_t)((i >> 1) & 1), giveup)) { ok = false; break; }
            fence_after();
            TRB(10);
            float s[32], dp[32];
            const uint32_t s_addr = lane_addr + COL_S + (uint32_t)(buf * 64 + colhalf * 32);
            const uint32_t dp_addr = lane_addr + COL_DP + (uint32_t)(buf * 64 + colhalf * 32);
            tmem_ld32_nowait(s_addr, s);
            tmem_ld32_nowait(dp_addr, dp);
            tmem_wait_ld();
            TRB(11);
            // per-column lse and D
            if (stats_in_smem) {
                const float4 *lp = reinterpret_cast<const float4 *>(stat_l + i * QB + colhalf * 32);
                const float4 *dp4 = reinterpret_cast<const float4 *>(stat_d + i * QB + colhalf * 32);
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 l4 = lp[c4], d4 = dp4[c4];          // the same address for the whole warp: broadcast
                    const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = c4 * 4 + e;
                        float p = fast_exp2(fmaf(s[c], scale_log2e, -lv[e]));
                        if (qc0 + c < kj || qc0 + c >= T) p = 0.0f;        // causal mask and the ragged end
                        s[c] = round_tf32_alu(p);
                        dp[c] = round_tf32_alu(p * (dp[c] - dv[e]));
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int q = qc0 + c;
                    const float lq = (q < T) ? __ldg(lse + (size_t)bh * T + q) * LOG2E : 0.0f;
                    const float dq_ = (q < T) ? __ldg(dsum + (size_t)bh * T + q) : 0.0f;
                    float p = fast_exp2(fmaf(s[c], scale_log2e, -lq));
                    if (q < kj || q >= T) p = 0.0f;        // causal mask and the ragged end
                    s[c] = round_tf32_alu(p);
                    dp[c] = round_tf32_alu(p * (dp[c] - dq_));
                }
            }
            TRB(12);
            tmem_st32_nowait(s_addr, s);
            tmem_st32_nowait(dp_addr, dp);
            tmem_wait_st();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(PD_FULL + buf));
            TRB(13);
#ifdef BMB_FLASH_TRACE
            if (tr) g_trace_bwd[14] += 1;
#endif
        }
        if (ok && nb > 0 && mbar_wait(bar(ACC_DONE), 0, giveup)) {
            fence_after();
            float v[32];
            tmem_ld32(lane_addr + COL_DV + (uint32_t)(colhalf * 32), v);
            if (kj < T) {
                float *dst = dqkv + ((size_t)b * T + kj) * 3 * C + 2 * C + h * HS + colhalf * 32;
#pragma unroll
                for (int d = 0; d < 32; d += 4)
                    *reinterpret_cast<float4 *>(dst + d) = out4(v[d], v[d + 1], v[d + 2], v[d + 3], round_out);
            }
            tmem_ld32(lane_addr + COL_DK + (uint32_t)(colhalf * 32), v);
            if (kj < T) {
                float *dst = dqkv + ((size_t)b * T + kj) * 3 * C + C + h * HS + colhalf * 32;
#pragma unroll
                for (int d = 0; d < 32; d += 4)
                    *reinterpret_cast<float4 *>(dst + d) = out4(v[d] * scale, v[d + 1] * scale, v[d + 2] * scale, v[d + 3] * scale, round_out);
            }
        }
    }

    fence_before();
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *giveup) {
        *reinterpret_cast<volatile int *>(status) = 4;
        __threadfence_system();
    }
}

__global__ void round_copy2_k(float *__restrict__ dst, const float *__restrict__ src, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(src)[i];
        reinterpret_cast<float4 *>(dst)[i] = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
    }
}

bool g_attr[64];
std::mutex g_mu;

}  // namespace

// dqkv is overwritten.  `rounded`: qkv and dout already hold TF32-representable
// values; otherwise rounded copies are made in per-device scratch first.
int flash_backward_tc(float *dqkv, float *dsum, const float *dout, const float *qkv, const float *out,
                      const float *lse, int B, int T, int C, int NH, bool rounded, cudaStream_t st) {
    int *status_dev = nullptr;
    volatile int *status_host = nullptr;
    BMB_TRY(tc::status_word(&status_dev, &status_host));
    if (*status_host != 0)
        return fail(BMB_E_TIMEOUT, "an earlier tensor-core kernel on this device gave up waiting on a barrier");
    BMB_TRY(launch_flash_dsum(dsum, dout, out, B, T, NH, HS, st));
    const float *q = qkv, *g = dout;
    if (!rounded) {
        const long long nq = (long long)B * T * 3 * C, ng = (long long)B * T * C;
        float *sq = (float *)device_scratch(SCR_GEMM_A, (size_t)nq * sizeof(float));
        float *sg = (float *)device_scratch(SCR_GEMM_B, (size_t)ng * sizeof(float));
        if (!sq || !sg) return BMB_E_CUDA;
        const long long cap = 8LL * sm_count();
        long long b1 = (nq / 4 + 255) / 256, b2 = (ng / 4 + 255) / 256;
        round_copy2_k<<<(int)(b1 > cap ? cap : b1), 256, 0, st>>>(sq, qkv, nq / 4);
        round_copy2_k<<<(int)(b2 > cap ? cap : b2), 256, 0, st>>>(sg, dout, ng / 4);
        count_launch(2);
        BMB_LAUNCH_CHECK();
        q = sq; g = sg;
    }
    const long long rows = (long long)B * T;
    CUtensorMap qk64, qn64, gk64, gn64;
    BMB_TRY(make_map_2d(&qk64, q, 4, rows, 3LL * C, 3LL * C * 4, 64, false));
    BMB_TRY(make_map_2d(&qn64, q, 4, rows, 3LL * C, 3LL * C * 4, 64, true));
    BMB_TRY(make_map_2d(&gk64, g, 4, rows, C, (long long)C * 4, 64, false));
    BMB_TRY(make_map_2d(&gn64, g, 4, rows, C, (long long)C * 4, 64, true));
    {
        std::lock_guard<std::mutex> lk(g_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !g_attr[d]) {
            BMB_CUDA(cudaFuncSetAttribute(flash_bwd_dq_tc_k, cudaFuncAttributeMaxDynamicSharedMemorySize, dq::SMEM));
            BMB_CUDA(cudaFuncSetAttribute(flash_bwd_dkv_tc_k, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::SMEM));
            g_attr[d] = true;
        }
    }
    const float scale = 1.0f / sqrtf((float)HS);
    // x = (batch, head), y = position: the dispatch order runs through all heads at the position with
    // the most work first, so the long CTAs start early and the short ones fill the tail.
    dim3 gkv(B * NH, (T + dkv::KT - 1) / dkv::KT), gq(B * NH, (T + dq::QT - 1) / dq::QT);
    flash_bwd_dkv_tc_k<<<gkv, dkv::THREADS, dkv::SMEM, st>>>(qk64, qn64, gk64, gn64, dqkv, lse, dsum, T, NH, scale, emit_rounded() ? 1 : 0, status_dev);
    flash_bwd_dq_tc_k<<<gq, dq::THREADS, dq::SMEM, st>>>(qk64, qn64, gk64, dqkv, lse, dsum, T, NH, scale, emit_rounded() ? 1 : 0, status_dev);
    count_launch(2);
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb

#ifdef BMB_FLASH_TRACE
extern "C" int bmb_dbg_flash_bwd_trace(long long *host16, int reset) {
    if (reset) { long long z[16] = {0}; return (int)cudaMemcpyToSymbol(bmb::g_trace_bwd, z, sizeof(z)); }
    return (int)cudaMemcpyFromSymbol(host16, bmb::g_trace_bwd, 16 * sizeof(long long));
}
#endif
