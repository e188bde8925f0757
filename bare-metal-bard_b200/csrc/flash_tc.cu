// Fused causal attention forward on the tensor cores (head size 64):
// S = Q K^T and O += P V as tcgen05.mma kind::tf32 with S and P V in tensor
// memory, Q / K / V tiles brought in by TMA straight out of the fused
// (B,T,3C) projection, softmax in registers with one query row per thread.
// The (T x T) score matrix never leaves tensor memory and registers (src/flash.h:1-34).
//
// One CTA owns 256 consecutive queries of one (batch, head) as two tiles of
// 128 and walks the keys up to the diagonal: shared-memory stages cover 128
// keys, S products and softmax steps 64.  384 threads:
//   warps 0-3 / 4-7  softmax group of tile 0 / tile 1: a thread reads 64 scores
//                    of its row from TMEM (tcgen05.ld), masks the diagonal,
//                    updates the running max and sum (the scale rides in the
//                    exponent's multiply-add), writes P = exp2(.) rounded to
//                    TF32 back into tensor memory (tcgen05.st) and, after
//                    handing P to the tensor core, folds the previous step's
//                    P V into its output registers:
//                    o = o * exp2(m_old - m_new) + PV;
//   warp 8           producer: TMA loads of the two Q tiles, then K blocks into
//                    a 2-deep ring and V blocks into a 3-deep ring;
//   warp 9           issuer of S_t = Q_t K_j^T, 64 keys (one half of the tile's
//                    128-column S buffer) at a time, each half as soon as the
//                    group has taken that half of the previous block out of
//                    TMEM -- the next block's first scores are multiplied while
//                    the group still works on this block's second half;
//   warps 10, 11     issuers of PV_t = P_t V for tile 0 / tile 1 (A operand read from
//                    tensor memory, 64 keys per step) as soon as P_t is written.
// Three issuing threads keep the next block's scores from queueing behind a wait
// for the other tile's P and feed the N = 64 products to the pipe from two
// schedulers; the two tiles interleave, so one group's exponentials overlap the
// other's matrix products.
// V is the B operand of P V with the head dimension contiguous, i.e. MN-major:
// its TMA map uses the 128-byte swizzle with 32-byte atoms.  K and Q are
// K-major.  Keys beyond the end of a sequence are never seen unmasked: a key
// index >= T exceeds every valid query index, so the causal mask covers it.
// CTAs are dispatched longest first (grid x = (batch, head), y = query block
// counted from the end).
//
// All mbarrier waits are bounded (tc_common.cuh); on expiry the CTA drains its
// copies in flight, frees its TMEM columns and raises the device status word.
#include "tc_common.cuh"
#include <cmath>
#include <mutex>

namespace bmb {
namespace {

using namespace tc;

// KB keys per softmax step, KBLK = 2 KB keys per shared-memory stage and per S product
constexpr int HS = 64, QT = 128, NQ = 2, KB = 64, KBLK = 128, K_STAGES = 2, V_STAGES = 3;
constexpr int Q_TILE_BYTES = QT * HS * 4;          // 32 KB: two halves of 128 rows x 128 B
constexpr int KV_TILE_BYTES = KBLK * HS * 4;       // 32 KB: two halves / chunks of 128 rows x 128 B
constexpr int TILE_COLS = 256;                     // TMEM columns per query tile: S (128) | P (64) | P V (64)
constexpr int COL_P = 128, COL_PV = 192;
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + NQ * Q_TILE_BYTES;
constexpr int OFF_V = OFF_K + K_STAGES * KV_TILE_BYTES;
constexpr int OFF_BAR = OFF_V + V_STAGES * KV_TILE_BYTES;
constexpr int FWD_SMEM = OFF_BAR + 256 + 1024;
constexpr int FWD_THREADS = 384;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

#ifdef BMB_FLASH_TRACE
__device__ long long g_trace[16];
// phase times are summed in registers and written once, so a timer costs one clock read
#define TR(i) do { const long long now_ = clock64(); tacc[(i) & 7] += now_ - tlast; tlast = now_; } while (0)
#define TRI(i) TR(i)
#define TR_FLUSH(first, n) do { if (tr) for (int i_ = 0; i_ < (n); ++i_) g_trace[(first) + i_] += tacc[((first) + i_) & 7]; } while (0)
#else
#define TR(i)
#define TRI(i)
#define TR_FLUSH(first, n)
#endif

__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_tc_k(const __grid_constant__ CUtensorMap mapQK, const __grid_constant__ CUtensorMap mapV,
               float *__restrict__ out, float *__restrict__ lse, int T, int NH, float scale_log2e,
               int round_out, int *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + OFF_BAR);
    // barrier indices
    // S_FULL / S_EMPTY: one pair per query tile and per 64-key half of the S buffer (index 2 * tile + half)
    enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = K_FULL + K_STAGES, V_FULL = K_EMPTY + K_STAGES, V_EMPTY = V_FULL + V_STAGES,
           S_FULL = V_EMPTY + V_STAGES, S_EMPTY = S_FULL + 2 * NQ, P_FULL = S_EMPTY + 2 * NQ, PV_FULL = P_FULL + NQ, NBARS = PV_FULL + NQ };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    volatile int *giveup = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [bar0](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.x, b = bh / NH, h = bh % NH;
    const int C = NH * HS;
    // CTAs are dispatched x first: every head's last (longest) query block, then the next, so the
    // long CTAs start early and the short ones fill the tail.
    const int qblk = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int q0 = qblk * (NQ * QT);

    // per tile: softmax steps of KB keys up to the diagonal, and the blocks of KBLK keys that hold them
    int nstep[NQ], nblk[NQ];
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
        const int first = q0 + t * QT;
        nstep[t] = (first < T) ? (min(T - 1, first + QT - 1) / KB + 1) : 0;
        nblk[t] = (nstep[t] + 1) / 2;
    }
    const int maxblk = max(nblk[0], nblk[1]);

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < K_STAGES; ++s) { mbar_init(bar(K_FULL + s), 1); mbar_init(bar(K_EMPTY + s), 1); }
        for (int s = 0; s < V_STAGES; ++s) { mbar_init(bar(V_FULL + s), 1); mbar_init(bar(V_EMPTY + s), NQ); }   // one release per P V issuer
        for (int t = 0; t < NQ; ++t) {
            for (int hf = 0; hf < 2; ++hf) { mbar_init(bar(S_FULL + 2 * t + hf), 1); mbar_init(bar(S_EMPTY + 2 * t + hf), 4); }
            mbar_init(bar(P_FULL + t), 4); mbar_init(bar(PV_FULL + t), 1);
        }
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
            int ntiles = 0;
            for (int t = 0; t < NQ; ++t) ntiles += (nblk[t] > 0);
            mbar_arrive_expect_tx(bar(Q_FULL), (uint32_t)(ntiles * Q_TILE_BYTES));
            for (int t = 0; t < NQ; ++t) {
                if (nblk[t] == 0) continue;
                for (int half = 0; half < 2; ++half)
                    for (int rr = 0; rr < 2; ++rr)
                        tma_load_2d(base + OFF_Q + t * Q_TILE_BYTES + half * (QT * 128) + rr * (64 * 128), &mapQK,
                                    h * HS + half * 32, row0 + q0 + t * QT + rr * 64, bar(Q_FULL));
            }
            bool ok = true;
            int armed_k[K_STAGES], armed_v[V_STAGES];
            for (int s = 0; s < K_STAGES; ++s) armed_k[s] = -1;
            for (int s = 0; s < V_STAGES; ++s) armed_v[s] = -1;
            for (int j = 0; j < maxblk; ++j) {
                const int sk = j % K_STAGES, sv = j % V_STAGES;
                const uint32_t pk = (uint32_t)((j / K_STAGES) & 1), pv = (uint32_t)((j / V_STAGES) & 1);
                if (!mbar_wait(bar(K_EMPTY + sk), pk ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(K_FULL + sk), KV_TILE_BYTES);
                armed_k[sk] = (int)pk;
                for (int half = 0; half < 2; ++half)
                    for (int rr = 0; rr < 2; ++rr)
                        tma_load_2d(base + OFF_K + sk * KV_TILE_BYTES + half * (KBLK * 128) + rr * (64 * 128), &mapQK,
                                    C + h * HS + half * 32, row0 + j * KBLK + rr * 64, bar(K_FULL + sk));
                if (!mbar_wait(bar(V_EMPTY + sv), pv ^ 1, giveup)) { ok = false; break; }
                mbar_arrive_expect_tx(bar(V_FULL + sv), KV_TILE_BYTES);
                armed_v[sv] = (int)pv;
                for (int half = 0; half < 2; ++half)
                    for (int rr = 0; rr < 2; ++rr)
                        tma_load_2d(base + OFF_V + sv * KV_TILE_BYTES + half * (KBLK * 128) + rr * (64 * 128), &mapV,
                                    2 * C + h * HS + half * 32, row0 + j * KBLK + rr * 64, bar(V_FULL + sv));
            }
            if (!ok) {
                mbar_drain(bar(Q_FULL), 0);
                for (int s = 0; s < K_STAGES; ++s)
                    if (armed_k[s] >= 0) mbar_drain(bar(K_FULL + s), (uint32_t)armed_k[s]);
                for (int s = 0; s < V_STAGES; ++s)
                    if (armed_v[s] >= 0) mbar_drain(bar(V_FULL + s), (uint32_t)armed_v[s]);
            }
        }
    } else if (warp == 9) {
        // ----------------------------------------------------- issuer of S = Q K^T
        if (lane == 0) {
            // Q (K-major) x K (K-major), 64 keys at a time: each half of the 128-column S buffer is refilled as
            // soon as the softmax group has taken that half out of tensor memory, so the scores of the next
            // block's first 64 keys are being multiplied while the group still works on this block's last 64.
            // (An N = 64 instruction occupies the pipe longer than its 32 cycles of arithmetic; that is the
            // price of not leaving the pipe idle while a whole 128-key buffer drains.)
            const uint32_t idesc_s = make_idesc(2, 0, 0, KB, QT);
#ifdef BMB_FLASH_TRACE
            // issuer phases of CTA (0, 0): 9 wait K, 10 wait S_EMPTY, 11 issue S
            const bool tr = (blockIdx.x == 0 && blockIdx.y == 0);
            long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long tlast = clock64();
#endif
            bool ok = mbar_wait(bar(Q_FULL), 0, giveup);
            TRI(15);
            for (int j = 0; ok && j < maxblk; ++j) {
                const int st = j % K_STAGES;
                if (!mbar_wait(bar(K_FULL + st), (uint32_t)((j / K_STAGES) & 1), giveup)) { ok = false; break; }
                TRI(9);
                const uint32_t ka = base + OFF_K + st * KV_TILE_BYTES;
                for (int hf = 0; ok && hf < 2; ++hf) {
                    for (int t = 0; t < NQ; ++t) {
                        if (2 * j + hf >= nstep[t]) continue;
                        // the group has taken this half of block j-1's scores out of tensor memory
                        if (j > 0 && !mbar_wait(bar(S_EMPTY + 2 * t + hf), (uint32_t)((j - 1) & 1), giveup)) { ok = false; break; }
                        fence_after();
                        TRI(10);
                        const uint32_t qa = base + OFF_Q + t * Q_TILE_BYTES;
                        const uint32_t d = tmem_base + (uint32_t)(t * TILE_COLS + hf * KB);
                        const uint32_t kh = ka + (uint32_t)(hf * (KB * 128));          // key rows 64 hf .. 64 hf + 63 of the block
#pragma unroll
                        for (int ks = 0; ks < HS / 8; ++ks) {
                            const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                            mma_tf32(d, smem_desc_kmajor(qa + half * (QT * 128) + off),
                                     smem_desc_kmajor(kh + half * (KBLK * 128) + off), idesc_s, ks ? 1u : 0u);
                        }
                        commit(bar(S_FULL + 2 * t + hf));
                        TRI(11);
                    }
                }
                if (!ok) break;
                commit(bar(K_EMPTY + st));      // every product that reads this K block has been issued
            }
            TR_FLUSH(9, 3);
        }
    } else if (warp == 10 || warp == 11) {
        // ------------------------------------- issuers of O += P V, one per query tile
        if (lane == 0) {
            const int t = warp - 10;
            const uint32_t idesc_pv = make_idesc(2, 0, 1, HS, QT);   // P (tensor memory) x V (MN-major)
#ifdef BMB_FLASH_TRACE
            // tile 1's issuer: 12 wait V, 13 wait P_FULL, 14 issue PV
            const bool tr = (blockIdx.x == 0 && blockIdx.y == 0 && t == 1);
            long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long tlast = clock64();
#endif
            bool ok = true;
            const int maxstep = max(nstep[0], nstep[1]);
            const uint32_t pa = tmem_base + (uint32_t)(t * TILE_COLS + COL_P), d = tmem_base + (uint32_t)(t * TILE_COLS + COL_PV);
            for (int i = 0; ok && i < maxstep; ++i) {
                const int j = i >> 1, st = j % V_STAGES;
                if (!(i & 1) && !mbar_wait(bar(V_FULL + st), (uint32_t)((j / V_STAGES) & 1), giveup)) { ok = false; break; }
                TRI(12);
                if (i < nstep[t]) {
                    if (!mbar_wait(bar(P_FULL + t), (uint32_t)(i & 1), giveup)) { ok = false; break; }
                    fence_after();
                    TRI(13);
                    // P is read from tensor memory, where the softmax threads left it: 8 columns per K step
                    const uint32_t va = base + OFF_V + st * KV_TILE_BYTES + (uint32_t)((i & 1) * (KB * 128));
#pragma unroll
                    for (int ks = 0; ks < KB / 8; ++ks)
                        mma_tf32_ts(d, pa + (uint32_t)(ks * 8), smem_desc_mnmajor32(va + ks * 1024, KBLK * 128), idesc_pv, ks ? 1u : 0u);
                    commit(bar(PV_FULL + t));
                    TRI(14);
                }
                // this tile's products that read the V block have been issued (none, past the tile's diagonal)
                if ((i & 1) || i + 1 == maxstep) commit(bar(V_EMPTY + st));
            }
            TR_FLUSH(12, 3);
        }
    } else {
        // ------------------------------------------------------ softmax groups
        const int t = warp >> 2, quad = warp & 3;
        const int r = quad * 32 + lane;                 // row inside the tile = TMEM lane
        const int tile_q0 = q0 + t * QT;
        const int qi = tile_q0 + r;
        const int nb = nstep[t];
        if (nb > 0) {
            const uint32_t s_addr = tmem_base + (uint32_t)(t * TILE_COLS) + ((uint32_t)(quad * 32) << 16);
            const uint32_t p_addr = s_addr + COL_P, pv_addr = s_addr + COL_PV;
            float o[HS];
#pragma unroll
            for (int d = 0; d < HS; ++d) o[d] = 0.0f;
            float m = -INFINITY, l = 0.0f, alpha_prev = 1.0f;
            bool ok = true;
#ifdef BMB_FLASH_TRACE
            const bool tr = (blockIdx.x == 0 && blockIdx.y == 0 && warp == 4 && lane == 0);
            long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long tlast = clock64();
#endif
            for (int j = 0; j < nb; ++j) {
                TR(0);
                // every step has its own half of the S buffer: wait for its product, take it, hand the half back
                if (!mbar_wait(bar(S_FULL + 2 * t + (j & 1)), (uint32_t)((j >> 1) & 1), giveup)) { ok = false; break; }
                fence_after();
                TR(1);
                float s[KB];
                tmem_ld64(s_addr + (uint32_t)((j & 1) * KB), s);
                TR(2);
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(S_EMPTY + 2 * t + (j & 1)));       // this half may be overwritten

                // m is the running maximum of the raw scores (the scale is positive, so the order is
                // the same); the scale rides in the exponent's multiply-add.
                const int k0 = j * KB;
                if (k0 + KB - 1 > tile_q0) {                // the block touches the diagonal (warp-uniform)
#pragma unroll
                    for (int i = 0; i < KB; ++i)
                        if (k0 + i > qi) s[i] = -INFINITY;
                }
                float mx0 = fmax3(s[0], s[1], s[2]), mx1 = fmax3(s[3], s[4], s[5]);
#pragma unroll
                for (int i = 6; i + 3 < KB; i += 4) {
                    mx0 = fmax3(mx0, s[i], s[i + 1]);
                    mx1 = fmax3(mx1, s[i + 2], s[i + 3]);
                }
                const float m_new = fmax3(m, fmax3(mx0, mx1, s[KB - 2]), s[KB - 1]);   // finite: key 0 is visible to every row
                const float mb = m_new * scale_log2e;
                const float alpha = fast_exp2(fmaf(m, scale_log2e, -mb));
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int i = 0; i < KB; i += 2) {
                    const float p0 = fast_exp2(fmaf(s[i], scale_log2e, -mb));
                    const float p1 = fast_exp2(fmaf(s[i + 1], scale_log2e, -mb));
                    sum0 += p0;
                    sum1 += p1;
                    s[i] = round_tf32_for_mma(p0);
                    s[i + 1] = round_tf32_for_mma(p1);
                }
                l = l * alpha + (sum0 + sum1);
                m = m_new;
                TR(3);

                if (j > 0) {
                    // P V of the previous block is complete: the P buffer is free and PV readable.
                    if (!mbar_wait(bar(PV_FULL + t), (uint32_t)((j - 1) & 1), giveup)) { ok = false; break; }
                    fence_after();
                }
                TR(4);
                // P row -> this thread's lane of tensor memory, the A operand of P V
                tmem_st64(p_addr, s);
                TR(5);
                // The previous block's P V must be out of TMEM before the next product may overwrite it;
                // its fold into the output registers then runs while the tensor core works on this block.
                if (j > 0) {
                    float v0[32], v1[32];
                    tmem_ld32_nowait(pv_addr, v0);
                    tmem_ld32_nowait(pv_addr + 32, v1);
                    tmem_wait_ld();
                    TR(6);
                    fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(P_FULL + t));
#pragma unroll
                    for (int i = 0; i < 32; ++i) { o[i] = fmaf(o[i], alpha_prev, v0[i]); o[32 + i] = fmaf(o[32 + i], alpha_prev, v1[i]); }
                } else {
                    fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(P_FULL + t));
                }
                alpha_prev = alpha;
                TR(7);
            }
#ifdef BMB_FLASH_TRACE
            TR_FLUSH(0, 8);
            if (tr) g_trace[8] += nb;
#endif
            if (ok && mbar_wait(bar(PV_FULL + t), (uint32_t)((nb - 1) & 1), giveup)) {
                fence_after();
                float v[32];
                tmem_ld32(pv_addr, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = fmaf(o[i], alpha_prev, v[i]);
                tmem_ld32(pv_addr + 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[32 + i] = fmaf(o[32 + i], alpha_prev, v[i]);
                if (qi < T) {
                    const float inv = 1.0f / l;
                    float *dst = out + ((size_t)b * T + qi) * C + h * HS;
#pragma unroll
                    for (int d = 0; d < HS; d += 4)
                    {
                        float4 w = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
                        if (round_out) w = make_float4(round_tf32(w.x), round_tf32(w.y), round_tf32(w.z), round_tf32(w.w));
                        *reinterpret_cast<float4 *>(dst + d) = w;
                    }
                    lse[(size_t)bh * T + qi] = (m * scale_log2e + log2f(l)) * 0.6931471805599453f;
                }
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
        *reinterpret_cast<volatile int *>(status) = 2;
        __threadfence_system();
    }
}

__global__ void round_copy_k(float *__restrict__ dst, const float *__restrict__ src, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(src)[i];
        reinterpret_cast<float4 *>(dst)[i] = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
    }
}

bool g_fwd_attr[64];
std::mutex g_mu;

}  // namespace

bool flash_tc_supported(int T, int C, int NH, const float *qkv, const float *out) {
    if (NH <= 0 || C % NH || C / NH != HS) return false;
    if (T < 1 || (((uintptr_t)qkv | (uintptr_t)out) & 15)) return false;
    return true;
}

// qkv_rounded: the caller guarantees that qkv already holds TF32-representable
// values; otherwise a rounded copy is made in per-device scratch first.
int flash_forward_tc(float *out, float *lse, const float *qkv, int B, int T, int C, int NH, bool qkv_rounded,
                     cudaStream_t st) {
    int *status_dev = nullptr;
    volatile int *status_host = nullptr;
    BMB_TRY(tc::status_word(&status_dev, &status_host));
    if (*status_host != 0)
        return fail(BMB_E_TIMEOUT, "an earlier tensor-core kernel on this device gave up waiting on a barrier");
    const float *src = qkv;
    if (!qkv_rounded) {
        const long long n = (long long)B * T * 3 * C;
        float *scr = (float *)device_scratch(SCR_GEMM_A, (size_t)n * sizeof(float));
        if (!scr) return BMB_E_CUDA;
        long long blocks = (n / 4 + 255) / 256, cap = 8LL * sm_count();
        round_copy_k<<<(int)(blocks > cap ? cap : blocks), 256, 0, st>>>(scr, qkv, n / 4);
        count_launch();
        BMB_LAUNCH_CHECK();
        src = scr;
    }
    CUtensorMap mapQK, mapV;
    BMB_TRY(make_map_2d(&mapQK, src, 4, (long long)B * T, 3LL * C, 3LL * C * 4, 64, false));
    BMB_TRY(make_map_2d(&mapV, src, 4, (long long)B * T, 3LL * C, 3LL * C * 4, 64, true));
    {
        std::lock_guard<std::mutex> lk(g_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !g_fwd_attr[d]) {
            BMB_CUDA(cudaFuncSetAttribute(flash_fwd_tc_k, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
            g_fwd_attr[d] = true;
        }
    }
    const float scale_log2e = (1.0f / sqrtf((float)HS)) * 1.4426950408889634f;
    dim3 grid(B * NH, (T + NQ * QT - 1) / (NQ * QT));
    flash_fwd_tc_k<<<grid, FWD_THREADS, FWD_SMEM, st>>>(mapQK, mapV, out, lse, T, NH, scale_log2e,
                                                        emit_rounded() ? 1 : 0, status_dev);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb

#ifdef BMB_FLASH_TRACE
extern "C" int bmb_dbg_flash_trace(long long *host16, int reset) {
    if (reset) { long long z[16] = {0}; return (int)cudaMemcpyToSymbol(bmb::g_trace, z, sizeof(z)); }
    return (int)cudaMemcpyFromSymbol(host16, bmb::g_trace, 16 * sizeof(long long));
}
#endif
