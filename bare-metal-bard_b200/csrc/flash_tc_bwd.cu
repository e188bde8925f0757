// Fused causal attention backward on the tensor cores (head size 64), split
// as in the reference (src/flash.cu:434-470): dQ reduces over keys, dK and dV
// reduce over queries, so each keeps its accumulators on chip -- here in tensor
// memory -- and writes its part of dqkv once, through shared memory and tile
// stores (no atomics).  The reference
// launches the two as separate kernels; here they are two kinds of CTA in one
// grid (flash_bwd_tc_k at the end of this file).
// P is rebuilt from the saved lse, P = exp(S - lse), and
// dS = P * (dP - D) with D = rowsum(dO * O)   (src/flash.cu:447-453).
//
// dQ CTAs: a CTA owns 128 queries and walks key blocks of 128 up to the
//   diagonal.  Per block S = Q K^T (double buffered) and dP = dO V^T land in
//   TMEM; 256 threads -- a row of 128 per 32-column half of each 64-key
//   granule -- turn them into dS, rounded to TF32 and written back over dP in
//   tensor memory, which dQ += dS K (accumulated in TMEM over the whole walk)
//   reads as its A operand.
// dK/dV CTAs: a CTA owns 128 keys and walks query blocks of 128 from the
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
float *column_partial_rows(size_t floats, bool *deferred);
int column_sum_finish(bool deferred, float *dst, const float *partial, int G, int ncols, cudaStream_t st);

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

// A warp's 32 rows x 32 columns leave through 4 KB of shared memory and one tile store: a thread writes its row's 128
// bytes with the 16-byte pieces permuted as the store's 128-byte swizzle expects (which also spreads the warp's rows
// over the banks).  Written straight to global memory, a row per thread costs a transaction per row and instruction.
// `stage` is 1024-byte aligned; rows at and beyond T are clipped by the tensor map.  The caller commits and waits.
__device__ __forceinline__ void stage_rows32(uint32_t stage, int lane, const float (&v)[32], float mul, int rnd) {
    const uint32_t row_addr = stage + (uint32_t)(lane * 128);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float4 w = out4(v[4 * c] * mul, v[4 * c + 1] * mul, v[4 * c + 2] * mul, v[4 * c + 3] * mul, rnd);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"r"(row_addr + (uint32_t)((c ^ (lane & 7)) << 4)), "f"(w.x), "f"(w.y), "f"(w.z), "f"(w.w) : "memory");
    }
}

#ifdef BMB_FLASH_TRACE
__device__ long long g_trace_bwd[32];
// phase times are summed in registers and written once, so a timer costs one clock read
#define TRB(i) do { const long long now_ = clock64(); tacc[(i) & 7] += now_ - tlast; tlast = now_; } while (0)
#define TRB_FLUSH(first, n) do { if (tr) for (int i_ = 0; i_ < (n); ++i_) g_trace_bwd[(first) + i_] += tacc[((first) + i_) & 7]; } while (0)
#else
#define TRB(i)
#define TRB_FLUSH(first, n)
#endif

// Column sums of the 32 x 32 block a warp has just staged (rows below `nvalid` only), one column per lane, written as
// one row of partial sums: the bias gradient of the projection that produced q, k, v is the column sum of dqkv, and
// the tile is at hand here.  The reads follow the staging layout's permutation, so a warp's 32 lanes hit 32 banks.
__device__ __forceinline__ void stage_colsum32(uint32_t stage, int lane, int nvalid, float *__restrict__ dst) {
    float s = 0.0f;
    const uint32_t piece = (uint32_t)(lane >> 2), within = (uint32_t)((lane & 3) * 4);
    for (int r = 0; r < nvalid; ++r) {
        float x;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x) : "r"(stage + (uint32_t)(r * 128) + ((piece ^ (uint32_t)(r & 7)) << 4) + within));
        s += x;
    }
    dst[lane] = s;
}

// ============================================================== dQ kernel
namespace dq {
constexpr int QT = 128, KB = 128, G = 64;               // keys per block (one S / dP product) and per granule (one dQ product)
constexpr int OFF_Q = 0, OFF_DO = 32768;
constexpr int OFF_KS = 65536, OFF_VK = OFF_KS + 2 * 32768;   // K and V blocks, K-major, two stages of 32 KB each
constexpr int OFF_KN = OFF_VK + 2 * 32768;              // K granules, MN-major, two slots of 16 KB
constexpr int OFF_BAR = OFF_KN + 2 * 16384;
constexpr int SMEM = OFF_BAR + 256 + 1024;
constexpr int THREADS = 384;
enum { Q_FULL = 0, KS_FULL = 1, KS_EMPTY = 3, VK_FULL = 5, VK_EMPTY = 7, KN_FULL = 9, KN_EMPTY = 11, S_FULL = 13, DP_FULL = 15,
       DS_FULL = 16, DQ_DONE = 18, S_EMPTY = 19, DO_FULL = 21, NBARS = 22 };
// TMEM columns: S [2] at 0 / 128, dP / dS at 256 (two granules of 64), dQ at 384
constexpr uint32_t COL_S = 0, COL_DP = 256, COL_DQ = 384;
}  // namespace dq

// A CTA owns 128 queries and walks key blocks of 128 up to the diagonal.  S = Q K^T (double
// buffered) and dP = dO V^T land in tensor memory as N = 128 products: an instruction of that width
// costs the tensor pipe its 64 cycles, whereas one thread cannot issue N = 64 instructions as fast as
// the pipe retires them.  256 threads (a query row each, 32 columns of each 64-key granule) rebuild P
// from S while dP is still being multiplied, then turn dP into dS granule by granule, written back
// over dP, where the tensor core reads it as the A operand of dQ += dS K; the second granule is
// computed while the first is multiplied.  The K-major copies of K and V (operands of S and dP) sit
// in 2-deep rings of whole blocks, the MN-major copy of K (operand of dQ) in two granule slots, each
// refilled as soon as its own consumer is done, by two loading threads so that neither ring waits
// for the other.
__device__ __forceinline__ void
flash_bwd_dq_body(const CUtensorMap &mapQKV_k, const CUtensorMap &mapQKV_n, const CUtensorMap &mapDO_k, const CUtensorMap &mapD,
                  const float *__restrict__ lse, const float *__restrict__ dsum, int T, int NH, float scale,
                  int round_out, int *__restrict__ status, int ypos, int ny, float *__restrict__ colpart) {
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
    const int q0 = (ny - 1 - ypos) * QT;                  // CTAs are dispatched x first: every head's longest tile, then the next
    const int nb = min(T - 1, q0 + QT - 1) / KB + 1;       // key blocks up to the diagonal
    const int row0 = b * T;

    // The loading thread sets up the barriers itself and goes straight on to its first copies; the other warps meet it
    // at a barrier it only arrives at, so the first operands are on their way while tensor memory is still being claimed.
    if (threadIdx.x == 256) {
        prefetch_tensormap(&mapQKV_k);
        prefetch_tensormap(&mapDO_k);
        mbar_init(bar(Q_FULL), 1);
        mbar_init(bar(DO_FULL), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(KS_FULL + s), 1); mbar_init(bar(KS_EMPTY + s), 1);
            mbar_init(bar(VK_FULL + s), 1); mbar_init(bar(VK_EMPTY + s), 1);
            mbar_init(bar(KN_FULL + s), 1); mbar_init(bar(KN_EMPTY + s), 1);
            mbar_init(bar(S_FULL + s), 1); mbar_init(bar(DS_FULL + s), 8); mbar_init(bar(S_EMPTY + s), 8);
        }
        mbar_init(bar(DP_FULL), 1);
        mbar_init(bar(DQ_DONE), 1);
        *giveup = 0;
        mbar_init_fence();
    }
    if (warp == 8) {
        __syncwarp();
        asm volatile("bar.arrive 2, 384;" ::: "memory");
    } else {
        if (warp == 9) tmem_alloc(smem_u32(tmem_slot), 512);
        fence_before();
        asm volatile("bar.sync 2, 384;" ::: "memory");
        fence_after();
    }
    const uint32_t tmem_base = (warp == 8) ? 0u : *tmem_slot;      // the loading warp has no use for it

    if (warp == 8) {
        // ------------------------------------- loads of Q, dO and the K-major K / V blocks
        if (lane == 0) {
            // in the order of first use: Q and the first K block (the scores), then dO and the first V block (dP)
            mbar_arrive_expect_tx(bar(Q_FULL), 32768);
            for (int half = 0; half < 2; ++half)
                for (int rr = 0; rr < 2; ++rr)
                    tma_load_2d(base + OFF_Q + half * 16384 + rr * 8192, &mapQKV_k, h * HS + half * 32, row0 + q0 + rr * 64, bar(Q_FULL));
            bool ok = true;
            int armed_k[2] = {-1, -1}, armed_v[2] = {-1, -1};
            for (int j = 0; j < nb; ++j) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (!mbar_wait(bar(KS_EMPTY + st), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(KS_FULL + st), 32768);
                armed_k[st] = (int)ph;
                for (int half = 0; half < 2; ++half)
                    for (int rr = 0; rr < 2; ++rr)
                        tma_load_2d(base + OFF_KS + st * 32768 + half * 16384 + rr * 8192, &mapQKV_k, C + h * HS + half * 32,
                                    row0 + j * KB + rr * 64, bar(KS_FULL + st));
                if (j == 0) {
                    mbar_arrive_expect_tx(bar(DO_FULL), 32768);
                    for (int half = 0; half < 2; ++half)
                        for (int rr = 0; rr < 2; ++rr)
                            tma_load_2d(base + OFF_DO + half * 16384 + rr * 8192, &mapDO_k, h * HS + half * 32, row0 + q0 + rr * 64, bar(DO_FULL));
                }
                if (!mbar_wait(bar(VK_EMPTY + st), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(VK_FULL + st), 32768);
                armed_v[st] = (int)ph;
                for (int half = 0; half < 2; ++half)
                    for (int rr = 0; rr < 2; ++rr)
                        tma_load_2d(base + OFF_VK + st * 32768 + half * 16384 + rr * 8192, &mapQKV_k, 2 * C + h * HS + half * 32,
                                    row0 + j * KB + rr * 64, bar(VK_FULL + st));
            }
            if (!ok) {
                mbar_drain(bar(Q_FULL), 0);
                if (armed_k[0] >= 0) mbar_drain(bar(DO_FULL), 0);    // armed right after the first K block
                for (int s = 0; s < 2; ++s) {
                    if (armed_k[s] >= 0) mbar_drain(bar(KS_FULL + s), (uint32_t)armed_k[s]);
                    if (armed_v[s] >= 0) mbar_drain(bar(VK_FULL + s), (uint32_t)armed_v[s]);
                }
            }
        }
    } else if (warp == 10) {
        // ------------------------------------------- loads of the MN-major K granules
        if (lane == 0) {
            bool ok = true;
            int armed_n[2] = {-1, -1};
            for (int j = 0; ok && j < nb; ++j)
                for (int g = 0; g < 2; ++g) {
                    const uint32_t ph = (uint32_t)(j & 1);
                    if (!mbar_wait(bar(KN_EMPTY + g), ph ^ 1, giveup)) { ok = false; break; }
                    mbar_arrive_expect_tx(bar(KN_FULL + g), 16384);
                    armed_n[g] = (int)ph;
                    for (int half = 0; half < 2; ++half)
                        tma_load_2d(base + OFF_KN + g * 16384 + half * 8192, &mapQKV_n, C + h * HS + half * 32,
                                    row0 + j * KB + g * G, bar(KN_FULL + g));
                }
            if (!ok)
                for (int g = 0; g < 2; ++g)
                    if (armed_n[g] >= 0) mbar_drain(bar(KN_FULL + g), (uint32_t)armed_n[g]);
        }
    } else if (warp == 9) {
        // ------------------------------------------------- issuer of S = Q K^T
        // Two threads feed the tensor core, because one cannot issue N = 64 instructions as fast as the
        // pipe retires them; this one runs ahead with the scores of the next block.
        if (lane == 0) {
            const uint32_t idesc_kk = make_idesc(2, 0, 0, KB, QT);     // [128 x 128] = A(K-major) x B(K-major)
            bool ok = mbar_wait(bar(Q_FULL), 0, giveup);
            for (int j = 0; ok && j < nb; ++j) {
                const int st = j & 1;
                if (!mbar_wait(bar(KS_FULL + st), (uint32_t)((j >> 1) & 1), giveup)) { ok = false; break; }
                // the threads have taken block j-2 out of this S buffer
                if (j >= 2 && !mbar_wait(bar(S_EMPTY + st), (uint32_t)(((j >> 1) & 1) ^ 1), giveup)) { ok = false; break; }
                fence_after();
                const uint32_t d = tmem_base + COL_S + (uint32_t)(st * 128), bsm = base + OFF_KS + st * 32768;
#pragma unroll
                for (int ks = 0; ks < HS / 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    mma_tf32(d, smem_desc_kmajor(base + OFF_Q + half * 16384 + off), smem_desc_kmajor(bsm + half * 16384 + off), idesc_kk, ks ? 1u : 0u);
                }
                commit(bar(S_FULL + st));
                commit(bar(KS_EMPTY + st));
            }
        }
    } else if (warp == 11) {
        // ----------------------------- issuer of dP = dO V^T and dQ += dS K
        if (lane == 0) {
            const uint32_t idesc_kk = make_idesc(2, 0, 0, KB, QT);     // [128 x 128] = A(K-major) x B(K-major)
            const uint32_t idesc_kn = make_idesc(2, 0, 1, HS, QT);     // dQ: dS (tensor memory) x K (MN-major)
            auto issue_dp = [&](uint32_t bsm) {
#pragma unroll
                for (int ks = 0; ks < HS / 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    mma_tf32(tmem_base + COL_DP, smem_desc_kmajor(base + OFF_DO + half * 16384 + off), smem_desc_kmajor(bsm + half * 16384 + off), idesc_kk, ks ? 1u : 0u);
                }
            };
#ifdef BMB_FLASH_TRACE
            // phases of this thread in CTA (0, 0): 16 prologue, 19 wait dS and K granule, 20 issue dQ, 21 wait V block, 22 issue dP
            const bool tr = (blockIdx.x == 0 && ypos == 0);
            long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long tlast = clock64();
#endif
            bool ok = mbar_wait(bar(DO_FULL), 0, giveup);
            if (ok) ok = mbar_wait(bar(VK_FULL + 0), 0, giveup);
            if (ok) {
                fence_after();
                issue_dp(base + OFF_VK);
                commit(bar(DP_FULL));
                commit(bar(VK_EMPTY + 0));
            }
            TRB(16);
            for (int j = 0; ok && j < nb; ++j) {
                const int s1 = (j + 1) & 1;
                for (int g = 0; g < 2; ++g) {
                    if (!mbar_wait(bar(KN_FULL + g), (uint32_t)(j & 1), giveup)) { ok = false; break; }
                    if (!mbar_wait(bar(DS_FULL + g), (uint32_t)(j & 1), giveup)) { ok = false; break; }
                    fence_after();
                    TRB(19);
                    const uint32_t kn = base + OFF_KN + g * 16384;
#pragma unroll
                    for (int ks = 0; ks < G / 8; ++ks)
                        mma_tf32_ts(tmem_base + COL_DQ, tmem_base + COL_DP + (uint32_t)(g * G + ks * 8),
                                    smem_desc_mnmajor32(kn + ks * 1024, 8192), idesc_kn, (j | g | ks) ? 1u : 0u);
                    commit(bar(KN_EMPTY + g));
                    TRB(20);
                }
                if (!ok) break;
                if (j + 1 < nb) {
                    // dP of block j+1 overwrites the dS just multiplied: the tensor core runs this thread's products in order
                    if (!mbar_wait(bar(VK_FULL + s1), (uint32_t)(((j + 1) >> 1) & 1), giveup)) { ok = false; break; }
                    fence_after();
                    TRB(21);
                    issue_dp(base + OFF_VK + s1 * 32768);
                    commit(bar(DP_FULL));
                    commit(bar(VK_EMPTY + s1));
                }
                TRB(22);
            }
            if (ok) commit(bar(DQ_DONE));
            TRB_FLUSH(16, 7);
        }
    } else if (warp < 8) {
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
        // phases of one thread of CTA (0, 0): 0 wait S, 1 load S + rebuild P, 2 wait dP, 3 dS of both granules
        const bool tr = (blockIdx.x == 0 && ypos == 0 && warp == 0 && lane == 0);
        long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tlast = clock64();
#endif
        for (int j = 0; j < nb; ++j) {
            const int buf = j & 1;
            if (!mbar_wait(bar(S_FULL + buf), (uint32_t)((j >> 1) & 1), giveup)) { ok = false; break; }
            fence_after();
            TRB(0);
            // P of this thread's 32 + 32 columns, kept in registers until dP arrives
            float p0[32], p1[32];
            const uint32_t s_addr = lane_addr + COL_S + (uint32_t)(buf * 128 + colhalf * 32);
            tmem_ld32_nowait(s_addr, p0);
            tmem_ld32_nowait(s_addr + G, p1);
            tmem_wait_ld();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(S_EMPTY + buf));       // the S buffer may take block j+2
            const int k0 = j * KB + colhalf * 32;
            const bool diag = (k0 + G + 31 > q0);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float a = fast_exp2(fmaf(p0[i], scale_log2e, -lse_r));
                float c = fast_exp2(fmaf(p1[i], scale_log2e, -lse_r));
                if (diag && (k0 + i > qi)) a = 0.0f;
                if (diag && (k0 + G + i > qi)) c = 0.0f;
                p0[i] = a;
                p1[i] = c;
            }
            TRB(1);
            if (!mbar_wait(bar(DP_FULL), (uint32_t)(j & 1), giveup)) { ok = false; break; }
            fence_after();
            TRB(2);
            const uint32_t dp_addr = lane_addr + COL_DP + (uint32_t)(colhalf * 32);
            {
                float dp[32];
                tmem_ld32(dp_addr, dp);
#pragma unroll
                for (int i = 0; i < 32; ++i) dp[i] = round_tf32_for_mma(p0[i] * (dp[i] - d_r));
                tmem_st32_nowait(dp_addr, dp);                 // dS over dP: the A operand of dQ += dS K
                tmem_wait_st();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(DS_FULL + 0));
            }
            {
                float dp[32];
                tmem_ld32(dp_addr + G, dp);
#pragma unroll
                for (int i = 0; i < 32; ++i) dp[i] = round_tf32_for_mma(p1[i] * (dp[i] - d_r));
                tmem_st32_nowait(dp_addr + G, dp);
                tmem_wait_st();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(DS_FULL + 1));
            }
            TRB(3);
        }
#ifdef BMB_FLASH_TRACE
        TRB_FLUSH(0, 4);
        if (tr) g_trace_bwd[8] += nb;
#endif
        if (ok && mbar_wait(bar(DQ_DONE), 0, giveup)) {
            fence_after();
            float v[32];
            tmem_ld32(lane_addr + COL_DQ + (uint32_t)(colhalf * 32), v);
            // Q and dO are no longer read (every product that does has retired): their space stages the output
            const uint32_t stage = base + OFF_Q + (uint32_t)(warp * 4096);
            stage_rows32(stage, lane, v, scale, round_out);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(&mapD, stage, h * HS + colhalf * 32, q0 + quad * 32, b);
                tma_store_commit();
            }
            if (colpart)       // partial row ((b, query block), quad): columns of q
                stage_colsum32(stage, lane, max(0, min(32, T - (q0 + quad * 32))),
                               colpart + ((size_t)(b * ny + q0 / QT) * 4 + quad) * (3 * C) + h * HS + colhalf * 32);
            if (lane == 0) tma_store_wait_read();        // shared memory has been read before the CTA may exit
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
constexpr int KT = 128, QB = 128, G = 64;               // queries per block (one S^T / dP^T product) and per granule
constexpr int OFF_K = 0, OFF_V = 32768;
constexpr int OFF_QK = 65536, OFF_DOK = OFF_QK + 32768; // Q and dO blocks, K-major, 32 KB each
constexpr int OFF_QN = OFF_DOK + 32768;                 // Q granules, MN-major, two slots of 16 KB
constexpr int OFF_DON = OFF_QN + 2 * 16384;             // dO granules, MN-major, two slots of 16 KB
constexpr int OFF_BAR = OFF_DON + 2 * 16384;
constexpr int STAT_MAX = 4096;                          // queries whose lse and D fit in shared memory
constexpr int OFF_STAT = OFF_BAR + 256;                 // lse * log2(e), then D, STAT_MAX floats each
constexpr int SMEM = OFF_STAT + 2 * STAT_MAX * 4 + 1024;
constexpr int THREADS = 384;
enum { KV_FULL = 0, QK_FULL = 1, QK_EMPTY = 2, DOK_FULL = 3, DOK_EMPTY = 4, N_FULL = 5, N_EMPTY = 7, S_FULL = 9, DP_FULL = 11,
       PD_FULL = 12, ACC_DONE = 14, V_FULL = 15, NBARS = 16 };
// TMEM columns: S^T / P^T [2] at 0 / 128, dP^T / dS^T at 256, dV at 384, dK at 448
constexpr uint32_t COL_S = 0, COL_DP = 256, COL_DV = 384, COL_DK = 448;
}  // namespace dkv

// A CTA owns 128 keys and walks query blocks of 128 from the diagonal to the end.  S^T = K Q^T
// (double buffered) and dP^T = V dO^T land in tensor memory as N = 128 products; 256 threads (a key
// row each, 32 columns of each 64-query granule) write P^T over S^T while dP^T is still being
// multiplied, then turn dP^T into dS^T granule by granule, in place, and the tensor core reads both
// as the A operands of dV += P^T dO and dK += dS^T Q; the second granule is computed while the first
// is multiplied.  Nothing of the (T x T) matrices touches shared memory.  The K-major copies of a
// query block (operands of the first two products) have one buffer each, refilled while the block
// is worked on; the MN-major copies (operands of the last two) sit in two granule slots, loaded by
// a thread of their own.
__device__ __forceinline__ void
flash_bwd_dkv_body(const CUtensorMap &mapQKV_k64, const CUtensorMap &mapQKV_n64, const CUtensorMap &mapDO_k64, const CUtensorMap &mapDO_n64,
                   const CUtensorMap &mapD, const float *__restrict__ lse, const float *__restrict__ dsum,
                   int T, int NH, float scale, int round_out, int *__restrict__ status, int ypos, int ny,
                   float *__restrict__ colpart) {
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
    const int j0 = ypos * KT;                              // first key of this CTA (earliest keys walk longest)
    const int ib0 = j0 / QB;                               // first query block that can see these keys
    const int nb = (T + QB - 1) / QB - ib0;                // query blocks to walk
    const int row0 = b * T;

    // As in the dQ body: the loading thread sets up the barriers and starts copying at once.
    if (threadIdx.x == 256) {
        prefetch_tensormap(&mapQKV_k64);
        prefetch_tensormap(&mapDO_k64);
        mbar_init(bar(KV_FULL), 1);
        mbar_init(bar(V_FULL), 1);
        mbar_init(bar(QK_FULL), 1); mbar_init(bar(QK_EMPTY), 1);
        mbar_init(bar(DOK_FULL), 1); mbar_init(bar(DOK_EMPTY), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(N_FULL + s), 1); mbar_init(bar(N_EMPTY + s), 2);     // both issuing threads release a granule slot
            mbar_init(bar(S_FULL + s), 1); mbar_init(bar(PD_FULL + s), 8);
        }
        mbar_init(bar(DP_FULL), 1);
        mbar_init(bar(ACC_DONE), 2);
        *giveup = 0;
        mbar_init_fence();
    }
    // Every thread needs the lse and D of every query the CTA walks: park them in shared memory once
    // (zero beyond the end of the sequence), lse already in log2 units.
    float *stat_l = reinterpret_cast<float *>(gen + OFF_STAT), *stat_d = stat_l + STAT_MAX;
    const int nstat = nb * QB;
    const bool stats_in_smem = nstat <= STAT_MAX;
    if (warp == 8) {
        __syncwarp();
        asm volatile("bar.arrive 2, 384;" ::: "memory");
    } else {
        if (warp == 9) tmem_alloc(smem_u32(tmem_slot), 512);
        fence_before();
        asm volatile("bar.sync 2, 384;" ::: "memory");
        fence_after();
    }
    const uint32_t tmem_base = (warp == 8) ? 0u : *tmem_slot;
    if (stats_in_smem && warp < 8) {
        // by the 256 arithmetic threads alone, after the block-wide barrier: the loading threads need not wait for it
        for (int i = threadIdx.x; i < nstat; i += 256) {
            const int q = ib0 * QB + i;
            stat_l[i] = (q < T) ? __ldg(lse + (size_t)bh * T + q) * LOG2E : 0.0f;
            stat_d[i] = (q < T) ? __ldg(dsum + (size_t)bh * T + q) : 0.0f;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
    }

    if (warp == 8) {
        // --------------------------- loads of K, V and the K-major Q / dO blocks
        if (lane == 0) {
            // in the order of first use: K and the first Q block (the scores), then V and the first dO block (dP)
            mbar_arrive_expect_tx(bar(KV_FULL), 32768);
            for (int half = 0; half < 2; ++half)
                for (int rr = 0; rr < 2; ++rr)
                    tma_load_2d(base + OFF_K + half * 16384 + rr * 8192, &mapQKV_k64, C + h * HS + half * 32, row0 + j0 + rr * 64, bar(KV_FULL));
            bool v_armed = false;
            bool ok = true;
            int armed_q = -1, armed_g = -1;
            for (int i = 0; i < nb; ++i) {
                const uint32_t ph = (uint32_t)(i & 1);
                const int qrow = row0 + (ib0 + i) * QB;
                if (!mbar_wait(bar(QK_EMPTY), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(QK_FULL), 32768);
                armed_q = (int)ph;
                for (int half = 0; half < 2; ++half)
                    for (int rr = 0; rr < 2; ++rr)
                        tma_load_2d(base + OFF_QK + half * 16384 + rr * 8192, &mapQKV_k64, h * HS + half * 32, qrow + rr * 64, bar(QK_FULL));
                if (i == 0) {
                    mbar_arrive_expect_tx(bar(V_FULL), 32768);
                    v_armed = true;
                    for (int half = 0; half < 2; ++half)
                        for (int rr = 0; rr < 2; ++rr)
                            tma_load_2d(base + OFF_V + half * 16384 + rr * 8192, &mapQKV_k64, 2 * C + h * HS + half * 32, row0 + j0 + rr * 64, bar(V_FULL));
                }
                if (!mbar_wait(bar(DOK_EMPTY), ph ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(DOK_FULL), 32768);
                armed_g = (int)ph;
                for (int half = 0; half < 2; ++half)
                    for (int rr = 0; rr < 2; ++rr)
                        tma_load_2d(base + OFF_DOK + half * 16384 + rr * 8192, &mapDO_k64, h * HS + half * 32, qrow + rr * 64, bar(DOK_FULL));
            }
            if (!ok) {
                mbar_drain(bar(KV_FULL), 0);
                if (v_armed) mbar_drain(bar(V_FULL), 0);
                if (armed_q >= 0) mbar_drain(bar(QK_FULL), (uint32_t)armed_q);
                if (armed_g >= 0) mbar_drain(bar(DOK_FULL), (uint32_t)armed_g);
            }
        }
    } else if (warp == 10) {
        // ------------------------------ loads of the MN-major Q and dO granules
        if (lane == 0) {
            bool ok = true;
            int armed_n[2] = {-1, -1};
            for (int i = 0; ok && i < nb; ++i)
                for (int g = 0; g < 2; ++g) {
                    const uint32_t ph = (uint32_t)(i & 1);
                    const int qrow = row0 + (ib0 + i) * QB + g * G;
                    if (!mbar_wait(bar(N_EMPTY + g), ph ^ 1, giveup)) { ok = false; break; }
                    mbar_arrive_expect_tx(bar(N_FULL + g), 32768);
                    armed_n[g] = (int)ph;
                    for (int half = 0; half < 2; ++half) {
                        tma_load_2d(base + OFF_QN + g * 16384 + half * 8192, &mapQKV_n64, h * HS + half * 32, qrow, bar(N_FULL + g));
                        tma_load_2d(base + OFF_DON + g * 16384 + half * 8192, &mapDO_n64, h * HS + half * 32, qrow, bar(N_FULL + g));
                    }
                }
            if (!ok)
                for (int g = 0; g < 2; ++g)
                    if (armed_n[g] >= 0) mbar_drain(bar(N_FULL + g), (uint32_t)armed_n[g]);
        }
    } else if (warp == 9 || warp == 11) {
        // ------------------------------------------------------------- issuers
        // Two threads feed the tensor core, because one cannot issue N = 64 instructions as fast as the
        // pipe retires them.  Warp 9 owns the S^T / P^T buffers: it issues S^T = K Q^T and dV += P^T dO.
        // Warp 11 owns the dP^T / dS^T buffer: dP^T = V dO^T and dK += dS^T Q.  Each buffer is written and
        // read by the products of one thread only, and the tensor core runs a thread's products in order.
        if (lane == 0) {
            const bool first = (warp == 9);
            const uint32_t idesc_st = make_idesc(2, 0, 0, QB, KT);     // [128 keys x 128 queries], both operands K-major
            const uint32_t idesc_acc = make_idesc(2, 0, 1, HS, KT);    // [128 keys x 64] = A (tensor memory) x B (MN-major)
            const int IN_FULL = first ? QK_FULL : DOK_FULL, IN_EMPTY = first ? QK_EMPTY : DOK_EMPTY;
            const uint32_t a_res = base + (first ? OFF_K : OFF_V), b_blk = base + (first ? OFF_QK : OFF_DOK);
            const uint32_t b_gran = base + (first ? OFF_DON : OFF_QN);
            const uint32_t acc = tmem_base + (first ? COL_DV : COL_DK);
            // D[128 x 128] = A (K or V, resident) x B^T (a K-major block of 128 queries)
            auto issue_st = [&](uint32_t d) {
#pragma unroll
                for (int ks = 0; ks < HS / 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    mma_tf32(d, smem_desc_kmajor(a_res + half * 16384 + off), smem_desc_kmajor(b_blk + half * 16384 + off), idesc_st, ks ? 1u : 0u);
                }
            };
#ifdef BMB_FLASH_TRACE
            // phases of warp 9 of CTA (0, 0): 24 prologue, 25 wait Q block, 26 issue S^T, 27 wait P^T / dS^T and granules, 28 issue dV
            const bool tr = (blockIdx.x == 0 && ypos == 0 && first);
            long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long tlast = clock64();
#endif
            bool ok = first ? mbar_wait(bar(KV_FULL), 0, giveup) : (nb <= 0 || mbar_wait(bar(V_FULL), 0, giveup));
            if (ok && nb > 0) ok = mbar_wait(bar(IN_FULL), 0, giveup);
            if (ok && nb > 0) {
                fence_after();
                issue_st(tmem_base + (first ? COL_S : COL_DP));
                commit(bar(first ? S_FULL + 0 : DP_FULL));
                commit(bar(IN_EMPTY));
            }
            TRB(24);
            for (int i = 0; ok && i < nb; ++i) {
                const int buf = i & 1, b1 = (i + 1) & 1;
                const uint32_t ph = (uint32_t)(i & 1), p1 = (uint32_t)((i + 1) & 1);
                if (first && i + 1 < nb) {
                    // S^T of block i+1 goes into the other buffer: the product that read its P^T (block i-1)
                    // was issued by this thread before this point
                    if (!mbar_wait(bar(QK_FULL), p1, giveup)) { ok = false; break; }
                    fence_after();
                    TRB(25);
                    issue_st(tmem_base + COL_S + (uint32_t)(b1 * 128));
                    commit(bar(S_FULL + b1));
                    commit(bar(QK_EMPTY));
                }
                TRB(26);
                for (int g = 0; g < 2; ++g) {
                    if (!mbar_wait(bar(N_FULL + g), ph, giveup)) { ok = false; break; }
                    if (!mbar_wait(bar(PD_FULL + g), ph, giveup)) { ok = false; break; }
                    fence_after();
                    TRB(27);
                    // dV += P^T dO   or   dK += dS^T Q
                    const uint32_t a_tm = tmem_base + (first ? COL_S + (uint32_t)(buf * 128) : COL_DP) + (uint32_t)(g * G);
                    const uint32_t bn = b_gran + g * 16384;
#pragma unroll
                    for (int ks = 0; ks < G / 8; ++ks)
                        mma_tf32_ts(acc, a_tm + (uint32_t)(ks * 8), smem_desc_mnmajor32(bn + ks * 1024, 8192), idesc_acc, (i | g | ks) ? 1u : 0u);
                    commit(bar(N_EMPTY + g));
                    TRB(28);
                }
                if (!ok) break;
                if (!first && i + 1 < nb) {
                    // dP^T of block i+1 overwrites the dS^T this thread has just had multiplied
                    if (!mbar_wait(bar(DOK_FULL), p1, giveup)) { ok = false; break; }
                    fence_after();
                    issue_st(tmem_base + COL_DP);
                    commit(bar(DP_FULL));
                    commit(bar(DOK_EMPTY));
                }
            }
            if (ok) commit(bar(ACC_DONE));
            TRB_FLUSH(24, 5);
        }
    } else if (warp < 8) {
        // ------------------------------------------------------- P^T and dS^T
        const int quad = warp & 3, colhalf = warp >> 2;
        const int r = quad * 32 + lane;
        const int kj = j0 + r;                             // this thread's key
        const float scale_log2e = scale * LOG2E;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        bool ok = true;
#ifdef BMB_FLASH_TRACE
        // phases of one thread of CTA (0, 0): 9 wait S^T, 10 P^T of both granules, 11 wait dP^T, 12 dS^T of both granules
        const bool tr = (blockIdx.x == 0 && ypos == 0 && warp == 0 && lane == 0);
        long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tlast = clock64();
#endif
        for (int i = 0; i < nb; ++i) {
            const int buf = i & 1;
            if (!mbar_wait(bar(S_FULL + buf), (uint32_t)((i >> 1) & 1), giveup)) { ok = false; break; }
            fence_after();
            TRB(9);
            // P^T of this thread's 32 + 32 query columns: unrounded in registers for dS^T, rounded into tensor memory
            float p[2][32];
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const int qc0 = (ib0 + i) * QB + g * G + colhalf * 32;       // first query column
                const uint32_t s_addr = lane_addr + COL_S + (uint32_t)(buf * 128 + g * G + colhalf * 32);
                float s[32];
                tmem_ld32(s_addr, s);
                // only the first block (the diagonal) and the last (the ragged end) have anything to mask
                const bool masked = (i == 0) || ((ib0 + i + 1) * QB > T);
                if (stats_in_smem) {
                    const float4 *lp = reinterpret_cast<const float4 *>(stat_l + i * QB + g * G + colhalf * 32);
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = lp[c4];                    // the same address for the whole warp: broadcast
                        const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = c4 * 4 + e;
                            p[g][c] = fast_exp2(fmaf(s[c], scale_log2e, -lv[e]));
                        }
                    }
                    if (masked) {
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (qc0 + c < kj || qc0 + c >= T) p[g][c] = 0.0f;  // causal mask and the ragged end
                    }
#pragma unroll
                    for (int c = 0; c < 32; ++c) s[c] = round_tf32_for_mma(p[g][c]);
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int q = qc0 + c;
                        const float lq = (q < T) ? __ldg(lse + (size_t)bh * T + q) * LOG2E : 0.0f;
                        float v = fast_exp2(fmaf(s[c], scale_log2e, -lq));
                        if (q < kj || q >= T) v = 0.0f;
                        p[g][c] = v;
                        s[c] = round_tf32_for_mma(v);
                    }
                }
                tmem_st32_nowait(s_addr, s);
            }
            TRB(10);
            if (!mbar_wait(bar(DP_FULL), (uint32_t)(i & 1), giveup)) { ok = false; break; }
            fence_after();
            TRB(11);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const int qc0 = (ib0 + i) * QB + g * G + colhalf * 32;
                const uint32_t dp_addr = lane_addr + COL_DP + (uint32_t)(g * G + colhalf * 32);
                float dp[32];
                tmem_ld32(dp_addr, dp);
                if (stats_in_smem) {
                    const float4 *dp4 = reinterpret_cast<const float4 *>(stat_d + i * QB + g * G + colhalf * 32);
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 d4 = dp4[c4];
                        const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = c4 * 4 + e;
                            dp[c] = round_tf32_for_mma(p[g][c] * (dp[c] - dv[e]));
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int q = qc0 + c;
                        const float dq_ = (q < T) ? __ldg(dsum + (size_t)bh * T + q) : 0.0f;
                        dp[c] = round_tf32_for_mma(p[g][c] * (dp[c] - dq_));
                    }
                }
                tmem_st32_nowait(dp_addr, dp);
                tmem_wait_st();                 // also covers this granule's P^T, stored above
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(PD_FULL + g));
            }
            TRB(12);
        }
#ifdef BMB_FLASH_TRACE
        TRB_FLUSH(9, 4);
        if (tr) g_trace_bwd[14] += nb;
#endif
        if (ok && nb > 0 && mbar_wait(bar(ACC_DONE), 0, giveup)) {
            fence_after();
            // K and V are no longer read (every product that does has retired): their space stages dV and dK
            const uint32_t stage_v = base + OFF_K + (uint32_t)(warp * 4096), stage_k = base + OFF_V + (uint32_t)(warp * 4096);
            float v[32];
            tmem_ld32(lane_addr + COL_DV + (uint32_t)(colhalf * 32), v);
            stage_rows32(stage_v, lane, v, 1.0f, round_out);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(&mapD, stage_v, 2 * C + h * HS + colhalf * 32, j0 + quad * 32, b);
                tma_store_commit();
            }
            // partial row ((b, key block), quad): columns of v, then of k
            const int nvalid = max(0, min(32, T - (j0 + quad * 32)));
            float *part = colpart ? colpart + ((size_t)(b * ny + ypos) * 4 + quad) * (3 * C) + h * HS + colhalf * 32 : nullptr;
            if (part) stage_colsum32(stage_v, lane, nvalid, part + 2 * C);
            tmem_ld32(lane_addr + COL_DK + (uint32_t)(colhalf * 32), v);
            stage_rows32(stage_k, lane, v, scale, round_out);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(&mapD, stage_k, C + h * HS + colhalf * 32, j0 + quad * 32, b);
                tma_store_commit();
            }
            if (part) stage_colsum32(stage_k, lane, nvalid, part + C);
            if (lane == 0) tma_store_wait_read();        // shared memory has been read before the CTA may exit
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

// Both backward kernels as one grid: CTAs with even blockIdx.y own 128 keys (dK/dV), those with odd
// blockIdx.y 128 queries (dQ), each family ordered from its longest walk to its shortest.  As two
// launches each would end in a partly filled wave of its own (768 CTAs on 148 SMs at B8 H12 T1024);
// together they end in one, and the short CTAs of either fill the gaps left by the long ones of both.
static_assert(dq::THREADS == dkv::THREADS && dq::SMEM == dkv::SMEM, "the two bodies share one launch configuration");
static_assert(dq::THREADS == 384, "the set-up barrier of both bodies counts 384 threads");
__global__ void __launch_bounds__(dkv::THREADS, 1)
flash_bwd_tc_k(const __grid_constant__ CUtensorMap mapQKV_k64, const __grid_constant__ CUtensorMap mapQKV_n64,
               const __grid_constant__ CUtensorMap mapDO_k64, const __grid_constant__ CUtensorMap mapDO_n64,
               const __grid_constant__ CUtensorMap mapD, const float *__restrict__ lse, const float *__restrict__ dsum,
               int T, int NH, float scale, int round_out, int *__restrict__ status, float *__restrict__ colpart) {
    const int ypos = (int)blockIdx.y >> 1, ny = (int)gridDim.y >> 1;
    if (blockIdx.y & 1) flash_bwd_dq_body(mapQKV_k64, mapQKV_n64, mapDO_k64, mapD, lse, dsum, T, NH, scale, round_out, status, ypos, ny, colpart);
    else flash_bwd_dkv_body(mapQKV_k64, mapQKV_n64, mapDO_k64, mapDO_n64, mapD, lse, dsum, T, NH, scale, round_out, status, ypos, ny, colpart);
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
// dbias_qkv (optional, 3C floats): += the column sums of dqkv (src/nn.cu bias_backward on dqkv: the bias gradient of
// the qkv projection), from partial sums the CTAs leave beside their tiles instead of another sweep over dqkv.
int flash_backward_tc(float *dqkv, float *dsum, const float *dout, const float *qkv, const float *out,
                      const float *lse, int B, int T, int C, int NH, bool rounded, cudaStream_t st, float *dbias_qkv) {
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
        BMB_TRY(scratch_acquire(SCR_GEMM_A, st));         // another stream's product may still read the staging slots
        BMB_TRY(scratch_acquire(SCR_GEMM_B, st));
        const long long cap = 8LL * sm_count();
        long long b1 = (nq / 4 + 255) / 256, b2 = (ng / 4 + 255) / 256;
        round_copy2_k<<<(int)(b1 > cap ? cap : b1), 256, 0, st>>>(sq, qkv, nq / 4);
        round_copy2_k<<<(int)(b2 > cap ? cap : b2), 256, 0, st>>>(sg, dout, ng / 4);
        count_launch(2);
        BMB_LAUNCH_CHECK();
        q = sq; g = sg;
    }
    const long long rows = (long long)B * T;
    CUtensorMap qk64, qn64, gk64, gn64, dmap;
    BMB_TRY(make_map_rows3d(&dmap, dqkv, 3LL * C, T, B, 32));
    BMB_TRY(make_map_2d(&qk64, q, 4, rows, 3LL * C, 3LL * C * 4, 64, false));
    BMB_TRY(make_map_2d(&qn64, q, 4, rows, 3LL * C, 3LL * C * 4, 64, true));
    BMB_TRY(make_map_2d(&gk64, g, 4, rows, C, (long long)C * 4, 64, false));
    BMB_TRY(make_map_2d(&gn64, g, 4, rows, C, (long long)C * 4, 64, true));
    {
        std::lock_guard<std::mutex> lk(g_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !g_attr[d]) {
            BMB_CUDA(cudaFuncSetAttribute(flash_bwd_tc_k, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::SMEM));
            g_attr[d] = true;
        }
    }
    const float scale = 1.0f / sqrtf((float)HS);
    // x = (batch, head), y = position: the dispatch order runs through all heads at the position with
    // the most work first, so the long CTAs start early and the short ones fill the tail.
    static_assert(dkv::KT == dq::QT, "one grid row pair per 128 positions");
    const int nblk = (T + dkv::KT - 1) / dkv::KT;
    dim3 grid(B * NH, 2 * nblk);
    // a row of partial column sums per (batch, block of 128 positions, quarter of the block): each (row, column) is
    // written by exactly one warp of one CTA
    const int part_rows = B * nblk * 4;
    bool deferred = false;
    float *colpart = nullptr;
    if (dbias_qkv) {
        colpart = column_partial_rows((size_t)part_rows * 3 * C, &deferred);
        if (!colpart) return BMB_E_CUDA;
    }
    flash_bwd_tc_k<<<grid, dkv::THREADS, dkv::SMEM, st>>>(qk64, qn64, gk64, gn64, dmap, lse, dsum, T, NH, scale, emit_rounded() ? 1 : 0, status_dev,
                                                           colpart);
    count_launch();
    BMB_LAUNCH_CHECK();
    if (dbias_qkv) BMB_TRY(column_sum_finish(deferred, dbias_qkv, colpart, part_rows, 3 * C, st));
    if (!rounded) {
        BMB_TRY(scratch_release(SCR_GEMM_A, st));
        BMB_TRY(scratch_release(SCR_GEMM_B, st));
    }
    return BMB_OK;
}

}  // namespace bmb

#ifdef BMB_FLASH_TRACE
extern "C" int bmb_dbg_flash_bwd_trace(long long *host16, int reset) {   // 32 counters
    if (reset) { long long z[32] = {0}; return (int)cudaMemcpyToSymbol(bmb::g_trace_bwd, z, sizeof(z)); }
    return (int)cudaMemcpyFromSymbol(host16, bmb::g_trace_bwd, 32 * sizeof(long long));
}
#endif
