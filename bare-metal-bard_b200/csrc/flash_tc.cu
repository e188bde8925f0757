// Fused causal attention forward on the tensor cores (head size 64):
// S = Q K^T and O += P V as tcgen05.mma kind::tf32 with S and P V in tensor
// memory, Q / K / V tiles brought in by TMA straight out of the fused
// (B,T,3C) projection, softmax in registers with one query row per thread.
// The (T x T) score matrix never leaves tensor memory and registers (src/flash.h:1-34).
//
// A work item is 256 consecutive queries of one (batch, head), handled as two tiles of 128 that walk the
// keys up to the diagonal: shared-memory stages cover 128 keys, S products and softmax steps 64.  The kernel is
// persistent: one CTA per SM takes its items in a fixed order (longest first) and every role carries its ring
// and barrier positions from one item to the next, so the next item's Q, K and V are in flight and its first
// scores multiplied while the softmax groups still normalise and store this item's output.  352 threads:
//   warps 0-3 / 4-7  softmax group of tile 0 / tile 1: a thread reads 64 scores
//                    of its row from TMEM (tcgen05.ld), masks the diagonal,
//                    updates the running max and sum (the scale rides in the
//                    exponent's multiply-add), writes P = exp2(.) rounded to
//                    TF32 back into tensor memory over the scores it took
//                    (tcgen05.st) and hands it to the tensor core, which
//                    accumulates O += P V in tensor memory.  The exponentials
//                    are taken against a maximum that follows the running one
//                    only in jumps of more than 2^8: O and the row sum are
//                    rescaled (a tensor-memory round trip) only then, so most
//                    steps never touch O;
//                    the finished tile goes to shared memory and from there to global memory by TMA store
//                    (a row per thread written straight to global memory costs one memory transaction per
//                    row and instruction: 3 us per item);
//   warp 8           producer: TMA loads of the two Q tiles, K blocks and V blocks into 2-deep rings;
//   warps 9, 10      issuer of tile 0 / tile 1: O_t += P_t V of step e - 2 (A operand read from tensor memory),
//                    then S_t = Q_t K^T of step e into the half of the tile's 128-column S buffer that P was
//                    just read from (products of one thread retire in order).  It waits for P only, so the two
//                    tiles never wait for one another (one issuer for both made them run in lockstep: each
//                    tile's next scores queued behind the other tile's release).
// V is the B operand of P V with the head dimension contiguous, i.e. MN-major:
// its TMA map uses the 128-byte swizzle with 32-byte atoms.  K and Q are
// K-major.  Keys beyond the end of a sequence are never seen unmasked: a key
// index >= T exceeds every valid query index, so the causal mask covers it.
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
constexpr int HS = 64, QT = 128, NQ = 2, KB = 64, KBLK = 128, K_STAGES = 2, V_STAGES = 2;
constexpr int Q_TILE_BYTES = QT * HS * 4;          // 32 KB: two halves of 128 rows x 128 B
constexpr int KV_TILE_BYTES = KBLK * HS * 4;       // 32 KB: two halves / chunks of 128 rows x 128 B
constexpr int TILE_COLS = 256;                     // TMEM columns per query tile: S / P halves (2 x 64) | O (64) | unused (64)
constexpr int COL_O = 128;
constexpr float RESCALE_LOG2 = 8.0f;               // O and the row sum are rescaled only when the running maximum has grown by more than 2^8
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + NQ * Q_TILE_BYTES;
constexpr int OFF_V = OFF_K + K_STAGES * KV_TILE_BYTES;
constexpr int O_STAGE_BYTES = QT * 128;             // 16 KB per tile: 4 KB per warp, its 32 rows x 32 columns of the output, swizzled for the tile store
constexpr int OFF_O = OFF_V + V_STAGES * KV_TILE_BYTES;
constexpr int OFF_BAR = OFF_O + NQ * O_STAGE_BYTES;
constexpr int FWD_SMEM = OFF_BAR + 256 + 1024;
constexpr int FWD_THREADS = 352;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


#ifdef BMB_FLASH_TRACE
// Developer timeline (compiled in only with -DBMB_FLASH_TRACE): per CTA, nanosecond stamps of kernel entry [0] and exit [1],
// and for the first softmax warp of query tile 0, per work item r < 5: first scores ready [2 + 4r], last block folded
// [3 + 4r], output stored [4 + 4r]; [22] / [23]: cycles that warp spent waiting for scores / for P V.
__device__ unsigned long long g_flash_trace[160][24];
__device__ __forceinline__ unsigned long long ftime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define FTR(i) do { g_flash_trace[blockIdx.x % 160][(i)] = ftime(); } while (0)
#define FTR_IF(c, i) do { if (c) FTR(i); } while (0)
#define FW_BEGIN() const long long fw_t0 = clock64()
#define FW_END(acc) acc += clock64() - fw_t0
// knock-out switches for timing experiments (results are then wrong): 1 no exponentials, 2 no P V load / fold,
// 4 no maximum, 8 no store of P, 16 no score products, 32 no P V products
__device__ int g_flash_ko;
#define KO_DECL() const int ko = g_flash_ko
#define KO(bit) (ko & (bit))
#else
#define KO_DECL() do { } while (0)
#define KO(bit) false
#define FTR(i) do { } while (0)
#define FTR_IF(c, i) do { } while (0)
#define FW_BEGIN() do { } while (0)
#define FW_END(acc) do { } while (0)
#endif

// A work item is (batch*head, block of 256 queries).  Items are numbered longest first (the last query
// block of every head, then the one before, ...) and dealt to the CTAs in rounds that alternate direction
// (CTA c takes items c, 2G-1-c, 2G+c, ...), which for four query blocks per head on 148 CTAs ends as evenly
// as a longest-first greedy assignment would.
struct FwdItem { int bh, q0, nstep[NQ], nblk[NQ], maxblk, maxstep; };
__device__ __forceinline__ bool fwd_item(int round, int T, int BH, int nqblk, FwdItem &it) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const long long w = (long long)round * G + ((round & 1) ? G - 1 - c : c);
    if (w >= (long long)BH * nqblk) return false;
    const int qblk = nqblk - 1 - (int)(w / BH);
    it.bh = (int)(w % BH);
    it.q0 = qblk * (NQ * QT);
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
        const int first = it.q0 + t * QT;
        it.nstep[t] = (first < T) ? (min(T - 1, first + QT - 1) / KB + 1) : 0;
        it.nblk[t] = (it.nstep[t] + 1) / 2;
    }
    it.maxblk = max(it.nblk[0], it.nblk[1]);
    it.maxstep = max(it.nstep[0], it.nstep[1]);
    return true;
}

// Named barriers of one softmax group (128 threads): plain, and one that also tells every thread whether all of
// them are still on course -- a thread whose bounded wait ran out must not leave the others at a barrier.
__device__ __forceinline__ bool group_all(int t, bool ok) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %2, 0;\n\tbar.red.and.pred p, %1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"(1 + t), "r"((uint32_t)ok) : "memory");
    return r != 0;
}

__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_tc_k(const __grid_constant__ CUtensorMap mapQK, const __grid_constant__ CUtensorMap mapV,
               const __grid_constant__ CUtensorMap mapO, float *__restrict__ lse, int T, int NH, int BH, int nqblk,
               float scale_log2e, int round_out, int *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + OFF_BAR);
    // One barrier per query tile and per 64-key half of the S buffer (index 2 * tile + half) for each of: S_FULL (the
    // scores are in the half), P_FULL (the group has written P over them), PV_DONE (the P V product that read the half
    // has retired).  Per half, because a parity wait tells the last phase from the one before only: the group may
    // be two steps ahead of the P V issue (both halves' scores are there before the first P V), and a thread that has
    // not waited for a while may be two products behind -- on one barrier for both halves either would alias.
    // O_FREE: the group has taken the finished item's O out of tensor memory
    enum { Q_FULL = 0, Q_EMPTY = 1, K_FULL = 2, K_EMPTY = K_FULL + K_STAGES, V_FULL = K_EMPTY + K_STAGES, V_EMPTY = V_FULL + V_STAGES,
           S_FULL = V_EMPTY + V_STAGES, P_FULL = S_FULL + 2 * NQ, PV_DONE = P_FULL + 2 * NQ, O_FREE = PV_DONE + 2 * NQ, NBARS = O_FREE + NQ };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NBARS);
    volatile int *giveup = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [bar0](int i) { return bar0 + 8u * (uint32_t)i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = NH * HS;

    if (threadIdx.x == 0) {
        // every ring slot and the Q tiles are released by both tiles' issuers
        mbar_init(bar(Q_FULL), 1);
        mbar_init(bar(Q_EMPTY), NQ);
        for (int s = 0; s < K_STAGES; ++s) { mbar_init(bar(K_FULL + s), 1); mbar_init(bar(K_EMPTY + s), NQ); }
        for (int s = 0; s < V_STAGES; ++s) { mbar_init(bar(V_FULL + s), 1); mbar_init(bar(V_EMPTY + s), NQ); }
        for (int t = 0; t < NQ; ++t) {
            for (int hf = 0; hf < 2; ++hf) mbar_init(bar(S_FULL + 2 * t + hf), 1);
            mbar_init(bar(O_FREE + t), 4);
            for (int hf = 0; hf < 2; ++hf) { mbar_init(bar(P_FULL + 2 * t + hf), 4); mbar_init(bar(PV_DONE + 2 * t + hf), 1); }
        }
        *giveup = 0;
        mbar_init_fence();
        FTR(0);
    }
    if (warp == 9) tmem_alloc(smem_u32(tmem_slot), 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    FwdItem it;

    if (warp == 8) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            bool ok = true;
            int kv = 0;                                   // key / value blocks loaded so far (all items)
            int armed_q = -1, armed_k[K_STAGES], armed_v[V_STAGES];
            for (int s = 0; s < K_STAGES; ++s) armed_k[s] = -1;
            for (int s = 0; s < V_STAGES; ++s) armed_v[s] = -1;
            for (int r = 0; ok && fwd_item(r, T, BH, nqblk, it); ++r) {
                const int b = it.bh / NH, h = it.bh % NH, row0 = b * T;
                for (int j = 0; j < it.maxblk; ++j, ++kv) {
                    const int sk = kv % K_STAGES, sv = kv % V_STAGES;
                    const uint32_t pk = (uint32_t)((kv / K_STAGES) & 1), pv = (uint32_t)((kv / V_STAGES) & 1);
                    if (!mbar_wait(bar(K_EMPTY + sk), pk ^ 1, giveup)) { ok = false; break; }
                    mbar_arrive_expect_tx(bar(K_FULL + sk), KV_TILE_BYTES);
                    armed_k[sk] = (int)pk;
                    for (int half = 0; half < 2; ++half)
                        for (int rr = 0; rr < 2; ++rr)
                            tma_load_2d(base + OFF_K + sk * KV_TILE_BYTES + half * (KBLK * 128) + rr * (64 * 128), &mapQK,
                                        C + h * HS + half * 32, row0 + j * KBLK + rr * 64, bar(K_FULL + sk));
                    if (j == 0) {
                        // the Q tiles may be replaced once the last score products of the previous item have retired
                        if (r > 0 && !mbar_wait(bar(Q_EMPTY), (uint32_t)((r - 1) & 1), giveup)) { ok = false; break; }
                        int ntiles = 0;
                        for (int t = 0; t < NQ; ++t) ntiles += (it.nblk[t] > 0);
                        mbar_arrive_expect_tx(bar(Q_FULL), (uint32_t)(ntiles * Q_TILE_BYTES));
                        armed_q = r & 1;
                        for (int t = 0; t < NQ; ++t) {
                            if (it.nblk[t] == 0) continue;
                            for (int half = 0; half < 2; ++half)
                                for (int rr = 0; rr < 2; ++rr)
                                    tma_load_2d(base + OFF_Q + t * Q_TILE_BYTES + half * (QT * 128) + rr * (64 * 128), &mapQK,
                                                h * HS + half * 32, row0 + it.q0 + t * QT + rr * 64, bar(Q_FULL));
                        }
                    }
                    if (!mbar_wait(bar(V_EMPTY + sv), pv ^ 1, giveup)) { ok = false; break; }
                    mbar_arrive_expect_tx(bar(V_FULL + sv), KV_TILE_BYTES);
                    armed_v[sv] = (int)pv;
                    for (int half = 0; half < 2; ++half)
                        for (int rr = 0; rr < 2; ++rr)
                            tma_load_2d(base + OFF_V + sv * KV_TILE_BYTES + half * (KBLK * 128) + rr * (64 * 128), &mapV,
                                        2 * C + h * HS + half * 32, row0 + j * KBLK + rr * 64, bar(V_FULL + sv));
                }
            }
            if (!ok) {
                if (armed_q >= 0) mbar_drain(bar(Q_FULL), (uint32_t)armed_q);
                for (int s = 0; s < K_STAGES; ++s)
                    if (armed_k[s] >= 0) mbar_drain(bar(K_FULL + s), (uint32_t)armed_k[s]);
                for (int s = 0; s < V_STAGES; ++s)
                    if (armed_v[s] >= 0) mbar_drain(bar(V_FULL + s), (uint32_t)armed_v[s]);
            }
        }
    } else if (warp == 9 || warp == 10) {
        // ------------------------------------- issuer of one query tile: S = Q K^T and O += P V
        if (lane == 0) {
            const int t = warp - 9;
            // Q (K-major) x K (K-major), 64 keys at a time; P (tensor memory) x V (MN-major), accumulated into O
            const uint32_t idesc_s = make_idesc(2, 0, 0, KB, QT), idesc_pv = make_idesc(2, 0, 1, HS, QT);
            const uint32_t qa = base + OFF_Q + t * Q_TILE_BYTES;
            const uint32_t s_tmem = tmem_base + (uint32_t)(t * TILE_COLS);
            const uint32_t od = s_tmem + COL_O;
            bool ok = true;
            KO_DECL();
            int kc = 0, vc = 0;                           // key blocks, value blocks consumed so far (all items)
            int pc[2] = {0, 0};                           // P tiles consumed so far from each half (all items)
            int items = 0;                                // items in which this tile had rows (all so far)
            for (int r = 0; ok && fwd_item(r, T, BH, nqblk, it); ++r) {
                const int mine = t ? it.nstep[1] : it.nstep[0];
                if (!mbar_wait(bar(Q_FULL), (uint32_t)(r & 1), giveup)) { ok = false; break; }
                // P V of step e - 2, then the scores of step e: the scores go to the half that P of step e - 2 was read
                // from, and products issued by one thread retire in order, so they land after that read.  Blocks past
                // this tile's diagonal (the other tile still needs them) are only waited for and released, which keeps
                // both issuers' releases of a ring slot in the same phase.
                for (int e = 0; ok && e < it.maxstep + 2; ++e) {
                    const int i = e - 2;
                    if (i >= 0) {
                        const int st = vc % V_STAGES;
                        if (!(i & 1) && !mbar_wait(bar(V_FULL + st), (uint32_t)((vc / V_STAGES) & 1), giveup)) { ok = false; break; }
                        if (i < mine) {
                            if (!mbar_wait(bar(P_FULL + 2 * t + (i & 1)), (uint32_t)(pc[i & 1] & 1), giveup)) { ok = false; break; }
                            // the first product of an item overwrites O: the group must have taken the last item's O
                            if (i == 0 && items > 0 && !mbar_wait(bar(O_FREE + t), (uint32_t)((items - 1) & 1), giveup)) { ok = false; break; }
                            fence_after();
                            // P is read from tensor memory, where the softmax threads left it: 8 columns per K step
                            const uint32_t va = base + OFF_V + st * KV_TILE_BYTES + (uint32_t)((i & 1) * (KB * 128));
                            const uint32_t pa = s_tmem + (uint32_t)((i & 1) * KB);
#pragma unroll
                            for (int ks = 0; ks < KB / 8; ++ks)
                                if (!KO(32)) mma_tf32_ts(od, pa + (uint32_t)(ks * 8), smem_desc_mnmajor32(va + ks * 1024, KBLK * 128), idesc_pv, (i > 0 || ks) ? 1u : 0u);
                            commit(bar(PV_DONE + 2 * t + (i & 1)));
                            ++pc[i & 1];
                        }
                        if ((i & 1) || i + 1 == it.maxstep) { commit(bar(V_EMPTY + st)); ++vc; }
                    }
                    if (e < it.maxstep) {
                        const int st = kc % K_STAGES, hf = e & 1;
                        if (!hf && !mbar_wait(bar(K_FULL + st), (uint32_t)((kc / K_STAGES) & 1), giveup)) { ok = false; break; }
                        if (e < mine) {
                            const uint32_t d = s_tmem + (uint32_t)(hf * KB);
                            const uint32_t kh = base + OFF_K + st * KV_TILE_BYTES + (uint32_t)(hf * (KB * 128));   // key rows 64 hf .. 64 hf + 63 of the block
#pragma unroll
                            for (int ks = 0; ks < HS / 8; ++ks) {
                                if (KO(16)) break;
                                const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                                mma_tf32(d, smem_desc_kmajor(qa + half * (QT * 128) + off),
                                         smem_desc_kmajor(kh + half * (KBLK * 128) + off), idesc_s, ks ? 1u : 0u);
                            }
                            commit(bar(S_FULL + 2 * t + hf));
                        }
                        if (hf || e + 1 == it.maxstep) { commit(bar(K_EMPTY + st)); ++kc; }   // this tile's products that read the K block have been issued
                        if (e + 1 == it.maxstep) commit(bar(Q_EMPTY));                       // ... and all that read this item's Q tile
                    }
                }
                if (mine > 0) ++items;
            }
        }
    } else {
        // ------------------------------------------------------ softmax groups
        const int t = warp >> 2, quad = warp & 3;
        const int rr = quad * 32 + lane;                // row inside the tile = TMEM lane
        KO_DECL();
        const uint32_t s_addr = tmem_base + (uint32_t)(t * TILE_COLS) + ((uint32_t)(quad * 32) << 16);
        const uint32_t o_addr = s_addr + COL_O;
        bool ok = true;
        int sc[2] = {0, 0};                             // score halves taken so far (all items)
        int pn[2] = {0, 0};                             // P tiles handed over so far from each half = P V products to expect (all items)
#ifdef BMB_FLASH_TRACE
        const bool tracer = (warp == 0 && lane == 0);
        long long fw_s = 0, fw_pv = 0;
#endif
        for (int r = 0; ok && fwd_item(r, T, BH, nqblk, it); ++r) {
            const int nb = t ? it.nstep[1] : it.nstep[0];
            if (nb == 0) continue;
            const int b = it.bh / NH, h = it.bh % NH;
            const int tile_q0 = it.q0 + t * QT;
            const int qi = tile_q0 + rr;
            // m is the maximum the exponentials are taken against; it follows the running maximum of the raw scores
            // (the scale is positive, so the order is the same) only in jumps of more than 2^8, and O and l are
            // rescaled only then: the output accumulates in tensor memory, and most steps never touch it.
            float m = -INFINITY, l = 0.0f;
            for (int j = 0; j < nb; ++j) {
                const int hf = j & 1;
                { FW_BEGIN(); if (!mbar_wait(bar(S_FULL + 2 * t + hf), (uint32_t)(sc[hf] & 1), giveup)) { ok = false; break; } FW_END(fw_s); }
                FTR_IF(tracer && j == 0 && r < 5, 2 + 4 * r);
                ++sc[hf];
                fence_after();
                float s[KB];
                tmem_ld64(s_addr + (uint32_t)(hf * KB), s);

                const int k0 = j * KB;
                if (k0 + KB - 1 > tile_q0) {                // the block touches the diagonal (warp-uniform)
#pragma unroll
                    for (int i = 0; i < KB; ++i)
                        if (k0 + i > qi) s[i] = -INFINITY;
                }
                float mx0 = fmax3(s[0], s[1], s[2]), mx1 = fmax3(s[3], s[4], s[5]);
                if (!KO(4)) {
#pragma unroll
                    for (int i = 6; i + 3 < KB; i += 4) {
                        mx0 = fmax3(mx0, s[i], s[i + 1]);
                        mx1 = fmax3(mx1, s[i + 2], s[i + 3]);
                    }
                }
                const float m_run = fmax3(m, fmax3(mx0, mx1, s[KB - 2]), s[KB - 1]);   // finite: key 0 is visible to every row
                if (j == 0) {
                    m = m_run;
                } else {
                    const bool grow = (m_run - m) * scale_log2e > RESCALE_LOG2;
                    if (__any_sync(0xffffffffu, grow)) {
                        // O must be whole (the previous block's product retired) while it is rescaled; the next
                        // product is not issued before this thread hands over P below.
                        // (the product before it on that half has retired: the scores this step waited for were issued after it)
                        { FW_BEGIN(); if (!mbar_wait(bar(PV_DONE + 2 * t + (hf ^ 1)), (uint32_t)((pn[hf ^ 1] - 1) & 1), giveup)) { ok = false; break; } FW_END(fw_pv); }
                        fence_after();
                        const float alpha = grow ? fast_exp2((m - m_run) * scale_log2e) : 1.0f;
                        float o[HS];
                        tmem_ld64(o_addr, o);
#pragma unroll
                        for (int d = 0; d < HS; ++d) o[d] *= alpha;
                        tmem_st64(o_addr, o);
                        l *= alpha;
                        if (grow) m = m_run;
                    }
                }
                const float mb = m * scale_log2e;
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int i = 0; i < KB; i += 2) {
                    const float e0 = fmaf(s[i], scale_log2e, -mb), e1 = fmaf(s[i + 1], scale_log2e, -mb);
                    const float p0 = KO(1) ? e0 : fast_exp2(e0);
                    const float p1 = KO(1) ? e1 : fast_exp2(e1);
                    sum0 += p0;
                    sum1 += p1;
                    s[i] = round_tf32_for_mma(p0);
                    s[i + 1] = round_tf32_for_mma(p1);
                }
                l += sum0 + sum1;
                // P row -> over the scores it came from, in this thread's lane of tensor memory: the A operand of P V
                if (!KO(8)) tmem_st64(s_addr + (uint32_t)(hf * KB), s);
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(P_FULL + 2 * t + hf));
                ++pn[hf];
            }
            FTR_IF(tracer && r < 5, 3 + 4 * r);
            // The last two products may both be in flight (the scores this thread waited for last were issued before
            // them); the ones before have retired.
            if (ok && nb > 1 && !mbar_wait(bar(PV_DONE + 2 * t + (nb & 1)), (uint32_t)((pn[nb & 1] - 1) & 1), giveup)) ok = false;
            if (ok && !mbar_wait(bar(PV_DONE + 2 * t + ((nb - 1) & 1)), (uint32_t)((pn[(nb - 1) & 1] - 1) & 1), giveup)) ok = false;
            if (!group_all(t, ok)) { ok = false; break; }
            fence_after();
            float o[HS];
            tmem_ld64(o_addr, o);
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(O_FREE + t));     // the next item's first product may overwrite O
            {
                // The tile leaves through shared memory, 32 columns at a time, each warp on its own with its 32 rows (4 KB of
                // the tile's staging buffer, one tile store): a thread writes its row's 128 bytes with the 16-byte pieces
                // permuted as the store's 128-byte swizzle expects (which also spreads the warp's rows over the banks);
                // rows at and beyond T are clipped by the tensor map.
                const float inv = 1.0f / l;
                const uint32_t stage = base + OFF_O + (uint32_t)(t * O_STAGE_BYTES) + (uint32_t)((rr >> 5) * 4096);
                const uint32_t row_addr = stage + (uint32_t)(lane * 128);
#pragma unroll
                for (int p = 0; p < 2; ++p) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int d = p * 32 + c * 4;
                        float4 w = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
                        if (round_out) w = make_float4(round_tf32(w.x), round_tf32(w.y), round_tf32(w.z), round_tf32(w.w));
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(row_addr + (uint32_t)(((c ^ (lane & 7)) << 4))), "f"(w.x), "f"(w.y), "f"(w.z), "f"(w.w) : "memory");
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&mapO, stage, h * HS + p * 32, tile_q0 + (rr >> 5) * 32, b);
                        tma_store_commit();
                        tma_store_wait_read();           // the staging buffer may be overwritten
                    }
                    __syncwarp();
                }
                if (qi < T) lse[(size_t)it.bh * T + qi] = (m * scale_log2e + log2f(l)) * 0.6931471805599453f;
            }
            FTR_IF(tracer && r < 5, 4 + 4 * r);
        }
#ifdef BMB_FLASH_TRACE
        if (tracer) { g_flash_trace[blockIdx.x % 160][22] = (unsigned long long)fw_s; g_flash_trace[blockIdx.x % 160][23] = (unsigned long long)fw_pv; }
#endif
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
    if (threadIdx.x == 0) FTR(1);
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
        BMB_TRY(scratch_acquire(SCR_GEMM_A, st));         // another stream's product may still read the staging slot
        long long blocks = (n / 4 + 255) / 256, cap = 8LL * sm_count();
        round_copy_k<<<(int)(blocks > cap ? cap : blocks), 256, 0, st>>>(scr, qkv, n / 4);
        count_launch();
        BMB_LAUNCH_CHECK();
        src = scr;
    }
    if (reinterpret_cast<uintptr_t>(out) % 16)
        return fail(BMB_E_ARG, "flash_attention_forward (tensor cores): the output must be 16-byte aligned");
    CUtensorMap mapQK, mapV, mapO;
    BMB_TRY(make_map_2d(&mapQK, src, 4, (long long)B * T, 3LL * C, 3LL * C * 4, 64, false));
    BMB_TRY(make_map_2d(&mapV, src, 4, (long long)B * T, 3LL * C, 3LL * C * 4, 64, true));
    BMB_TRY(make_map_rows3d(&mapO, out, C, T, B, 32));
    {
        std::lock_guard<std::mutex> lk(g_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !g_fwd_attr[d]) {
            BMB_CUDA(cudaFuncSetAttribute(flash_fwd_tc_k, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
            g_fwd_attr[d] = true;
        }
    }
    const float scale_log2e = (1.0f / sqrtf((float)HS)) * 1.4426950408889634f;
    const int nqblk = (T + NQ * QT - 1) / (NQ * QT);
    const long long items = (long long)B * NH * nqblk;
    int grid = (int)(items < sm_count() ? items : sm_count());             // persistent: one CTA per SM
    // BMB_FLASH_FWD_CTAS=n caps the grid, so that small problems also exercise CTAs that walk several work items (tests)
    if (const char *e = getenv("BMB_FLASH_FWD_CTAS")) { const int cap = atoi(e); if (cap >= 1 && cap < grid) grid = cap; }
    flash_fwd_tc_k<<<grid, FWD_THREADS, FWD_SMEM, st>>>(mapQK, mapV, mapO, lse, T, NH, B * NH, nqblk, scale_log2e,
                                                        emit_rounded() ? 1 : 0, status_dev);
    count_launch();
    BMB_LAUNCH_CHECK();
    if (!qkv_rounded) BMB_TRY(scratch_release(SCR_GEMM_A, st));
    return BMB_OK;
}

}  // namespace bmb

#ifdef BMB_FLASH_TRACE
extern "C" int bmb_dbg_flash_trace(unsigned long long *host_out /* 160 x 24 */) {
    cudaDeviceSynchronize();
    return cudaMemcpyFromSymbol(host_out, bmb::g_flash_trace, sizeof(unsigned long long) * 160 * 24) == cudaSuccess ? 0 : 1;
}
extern "C" int bmb_dbg_flash_ko(int ko) { return cudaMemcpyToSymbol(bmb::g_flash_ko, &ko, sizeof(int)) == cudaSuccess ? 0 : 1; }
extern "C" int bmb_dbg_flash_trace_clear() {
    static unsigned long long z[160 * 24];
    return cudaMemcpyToSymbol(bmb::g_flash_trace, z, sizeof(z)) == cudaSuccess ? 0 : 1;
}
#endif
