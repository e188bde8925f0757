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
// Kernel shape.  One persistent CTA per SM, 320 threads in three roles:
//   warp 0      producer: one lane issues the TMA loads of a K-slice (32 fp32
//               or 64 bf16 of K: A 16 KB, B 8..32 KB) into a 4-deep ring, each
//               slice armed on an mbarrier with its byte count.  A K-major
//               operand is one 2-d copy; an MN-major one is one 3-d copy that
//               lands all its 32-wide chunks (one copy per chunk starved the
//               tensor pipe);
//   warp 1      issuer: one lane waits for a slice, issues 4 tcgen05.mma
//               (128 x BN x 32 bytes of K each) and commits them to the
//               slice's "empty" barrier; after the last slice of a work item it
//               commits to the accumulator's "full" barrier.  This warp owns
//               the TMEM allocation (two fp32 accumulators, so the epilogue of
//               one item overlaps the main loop of the next);
//   warps 2..9  epilogue, two per TMEM lane quadrant taking alternate
//               32-column chunks.  Whole tiles with beta = 0 leave TMEM in the
//               16x256b shape and go straight from registers to global memory
//               in whole sectors; parts of tiles shared between CTAs, and
//               beta = 1, are parked in swizzled shared memory and added into C
//               by the copy engine (TMA reduce); any other case takes the
//               generic path (staging, then coalesced loads/stores/atomics).
// Tile width BN is 256, 192, 128 or 64 columns, chosen per problem; tiles are
// visited in groups of 8 M-tiles so that concurrently resident CTAs share A and
// B slices in L2; the tiles of a partly filled last wave are cut along K and
// shared between CTAs (WorkIter below).  A batch of dense problems is one long
// tile list.
//
// Every wait on an mbarrier is bounded: when one runs out, the CTA raises a
// flag all roles poll, the producer waits (bounded again) for the copies it
// has in flight, the TMEM allocation is released, and the kernel stores a
// nonzero word into a host-visible status that the next call reports as
// BMB_E_TIMEOUT.  No TMA load uses cluster multicast.
#include "tc_common.cuh"
#include <cuda_bf16.h>
#include <mutex>
#include <vector>

namespace bmb {
namespace {

using namespace tc;

// Output tile: 128 rows by 256, 192, 128 or 64 columns (chosen per problem to fill the last wave of CTAs;
// 64 serves outputs narrower than 128, e.g. the head-size-wide products of unfused attention).
constexpr int BM = 128, BN_WIDE = 256, BN_NARROW = 64, STAGES = 4, KBYTES = 128;
constexpr int A_BYTES = BM * KBYTES;
constexpr int EPI_WARPS = 8;                        // two per TMEM lane quadrant, taking alternate 32-column chunks
constexpr int NTHREADS = 64 + 32 * EPI_WARPS;
constexpr int EPI_BYTES = EPI_WARPS * 32 * 32 * 4;  // one 32 x 32 staging block per epilogue warp, 16-byte units XOR-swizzled by row
// A tile is MH (1 or 2) blocks of 128 rows tall.  Two blocks share every B slice: per K slice the SM then
// writes 64 KB and reads 96 KB of shared memory for 8 instructions, against 48 KB + 48 KB for 4 -- with
// fp32 operands it is shared-memory bandwidth, not the tensor pipe, that bounds the main loop.  The price:
// the two accumulators fill tensor memory, so the epilogue no longer overlaps the next tile, and the
// ring is 3 slices deep.
__host__ __device__ constexpr int stages_for(int mh) { return mh == 2 ? 3 : STAGES; }
constexpr int smem_bytes(int bn, int mh = 1) { return stages_for(mh) * (mh * A_BYTES + bn * KBYTES) + 1024 /*align*/ + 256 /*barriers*/ + EPI_BYTES; }
constexpr int CHUNK_BYTES = 32 * KBYTES;   // one MN-major chunk: 32 K rows x 128 bytes of M/N

#ifdef BMB_GEMM_TRACE
// Developer timeline (compiled in only with -DBMB_GEMM_TRACE): per CTA, nanosecond stamps of kernel entry,
// set-up done, first copy issued, first slice landed, last product issued, first accumulator ready,
// last tile stored, stores landed, exit.
__device__ unsigned long long g_gemm_trace[256][16];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define GTR(i) do { g_gemm_trace[blockIdx.x & 255][(i)] = gtime(); } while (0)
// cycles a role spent inside a wait: 10 issuer on full, 11 issuer on tmem-empty, 12 producer on empty, 13 epilogue warp 2 on tmem-full,
// 14 epilogue warp 2 working, 15 issuer total
// (summed in a register of the waiting thread, written once when its role ends)
#define GWAIT_DECL(v) long long v = 0
#define GWAIT_BEGIN() const long long gw0_ = clock64()
#define GWAIT_END(v) v += clock64() - gw0_
#define GWAIT_FLUSH(i, v) g_gemm_trace[blockIdx.x & 255][(i)] = (unsigned long long)(v)
#else
#define GTR(i)
#define GWAIT_DECL(v)
#define GWAIT_BEGIN()
#define GWAIT_END(v)
#define GWAIT_FLUSH(i, v)
#endif

struct TileSched {
    int tiles_m, tiles_n, num_tiles;
    __host__ __device__ __forceinline__ void coords(int tile, int &tm, int &tn) const {
        constexpr int GM = 8;
        const int per_group = GM * tiles_n;
        const int g = tile / per_group, first_m = g * GM;
        const int gsz = (tiles_m - first_m < GM) ? tiles_m - first_m : GM;
        const int r = tile - g * per_group;
        tm = first_m + r % gsz;
        tn = r / gsz;
    }
};

// The work of one CTA, as a list of items (tile, K slices [kb0, kb1)).  Tiles [0, dp_tiles) are
// handed out whole, round-robin.  The K slices of the remaining `sk_tiles` tiles -- the ones that
// would otherwise form a last, partly filled wave -- are laid end to end and cut into `g_sk` equal
// runs, one per CTA ("stream-K"), so a tile there is shared by the CTAs whose runs cross it.  Each
// CTA walks its run first, then its whole tiles.  Producer, issuer and epilogue warps each keep
// their own copy of this iterator and see the same sequence.
struct WorkIter {
    int dp_tiles, kblocks, g_sk, grid;
    long long R;            // K slices in the stream-K region
    long long it, hi;       // what is left of this CTA's run
    int dp_next;
    // Chunk-major form (g_sk < 0: -g_sk chunks; every tile is shared): the K range is cut into chunks and the items
    // (chunk, tile) are dealt round-robin in chunk-major order, so that at any time all CTAs work at about the same
    // depth of K -- CTAs that share an operand panel read the same slices at the same time, and panels too large for
    // L2 come from DRAM once instead of once per tile sharing them.
    int kchunks, ntiles;
    long long q;
    __host__ __device__ __forceinline__ long long run_start(int c) const { return ((long long)c * R) / g_sk; }
    __host__ __device__ __forceinline__ void init(int cta, int grid_, int dp_tiles_, int sk_tiles, int kblocks_, int g_sk_) {
        dp_tiles = dp_tiles_; kblocks = kblocks_; g_sk = g_sk_; grid = grid_;
        kchunks = 0; ntiles = sk_tiles; q = cta;
        if (g_sk_ < 0) { kchunks = -g_sk_; it = hi = 0; R = 0; dp_next = dp_tiles_; return; }
        R = (long long)sk_tiles * kblocks_;
        if (cta < g_sk_) { it = run_start(cta); hi = run_start(cta + 1); } else { it = hi = 0; }
        dp_next = cta;
    }
    __host__ __device__ __forceinline__ bool next(int &tile, int &kb0, int &kb1) {
        if (kchunks) {
            if (q >= (long long)ntiles * kchunks) return false;
            const int chunk = (int)(q / ntiles);
            tile = dp_tiles + (int)(q - (long long)chunk * ntiles);
            kb0 = (int)(((long long)chunk * kblocks) / kchunks);
            kb1 = (int)(((long long)(chunk + 1) * kblocks) / kchunks);
            q += grid;
            return true;
        }
        if (it < hi) {
            const long long t = it / kblocks;
            kb0 = (int)(it - t * kblocks);
            const long long n = ((long long)(kblocks - kb0) < hi - it) ? (long long)(kblocks - kb0) : hi - it;
            kb1 = kb0 + (int)n;
            tile = dp_tiles + (int)t;
            it += n;
            return true;
        }
        if (dp_next < dp_tiles) {
            tile = dp_next; kb0 = 0; kb1 = kblocks;
            dp_next += grid;
            return true;
        }
        return false;
    }
};

// One 128-bit group of the result: bias, beta * C, optional TF32 rounding, store (scalar at ragged edges).
__device__ __forceinline__ void store_result(float4 o, float *__restrict__ C, int M, int N, int m, int n, bool vec,
                                             float beta, const float *__restrict__ bias, int round_c) {
    if (m >= M) return;
    float *cp = C + (size_t)m * N + n;
    if (vec) {
        if (bias) {
            const float4 bb = *reinterpret_cast<const float4 *>(bias + n);
            o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
        }
        if (beta != 0.0f) {
            const float4 cc = *reinterpret_cast<const float4 *>(cp);
            o.x = fmaf(beta, cc.x, o.x); o.y = fmaf(beta, cc.y, o.y);
            o.z = fmaf(beta, cc.z, o.z); o.w = fmaf(beta, cc.w, o.w);
        }
        if (round_c) o = make_float4(round_tf32(o.x), round_tf32(o.y), round_tf32(o.z), round_tf32(o.w));
        *reinterpret_cast<float4 *>(cp) = o;
    } else {
        const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (n + e >= N) continue;
            float x = ov[e] + (bias ? bias[n + e] : 0.0f);
            if (beta != 0.0f) x = fmaf(beta, cp[e], x);
            cp[e] = round_c ? round_tf32(x) : x;
        }
    }
}

// One 128-bit group of a part of a stream-K tile: added into C, which the host has already
// multiplied by beta; the part that holds the first K slice brings the bias.
__device__ __forceinline__ void add_result(float4 o, float *__restrict__ C, int M, int N, int m, int n, bool vec,
                                           const float *__restrict__ bias) {
    if (m >= M) return;
    float *cp = C + (size_t)m * N + n;
    if (vec) {
        if (bias) {
            const float4 bb = *reinterpret_cast<const float4 *>(bias + n);
            o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
        }
        atomicAdd(reinterpret_cast<float4 *>(cp), o);
    } else {
        const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (n + e < N) atomicAdd(cp + e, ov[e] + (bias ? bias[n + e] : 0.0f));
    }
}

// KIND 0 = tf32 (fp32 operands), 1 = f16 (bf16 operands, always K-major).
// a_mn / b_mn: the operand's tile is MN-major (TF32 only); 2 = its tensor map is the 3-d one that
// brings all chunks of a slice in one copy.
template <int KIND, int BN, int MH, int AUX>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_k(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
          const __grid_constant__ CUtensorMap mapC, int c_mode, int batch, int M, int N,
          int kblocks, int kelems_per_block, int a_mn, int b_mn, float alpha, float beta, float *__restrict__ C,
          int vec_ok, int dp_tiles, int g_sk, const float *__restrict__ bias, int round_c, int *__restrict__ status,
          float *__restrict__ aux, int round_aux) {
    static_assert(MH == 1 || (MH == 2 && BN == 256), "two-block tiles are 256 columns wide");
    constexpr int STAGES = stages_for(MH), BMT = BM * MH;
    constexpr int B_BYTES = BN * KBYTES, STAGE_BYTES = MH * A_BYTES + B_BYTES;
    constexpr uint32_t ACC_COLS = BN > 128 ? 256 : 128; // TMEM columns set aside per 128-row accumulator
    constexpr int NACC = MH == 2 ? 1 : 2;               // accumulator sets: two blocks of rows fill tensor memory
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;        // allocations are powers of two
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    // operand ring | epilogue staging (1024-byte aligned: it is a TMA store source) | barriers
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + STAGES * STAGE_BYTES + EPI_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *giveup = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *armed = reinterpret_cast<int *>(tmem_slot + 2);   // [STAGES] parity last armed per slice, -1 = never

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;

    TileSched sch;
    sch.tiles_m = (M + BMT - 1) / BMT;
    sch.tiles_n = (N + BN - 1) / BN;
    // A batch of dense problems is one long list of tiles; its operands are seen as the 2-d matrices
    // [batch * rows][K] (K-major) or [batch * K][rows] (MN-major), so only a row offset tells batches apart.
    const int tiles_per_problem = sch.tiles_m * sch.tiles_n;
    sch.num_tiles = tiles_per_problem * batch;
    WorkIter wi;
    wi.init((int)blockIdx.x, (int)gridDim.x, dp_tiles, sch.num_tiles - dp_tiles, kblocks, g_sk);
    int tile, kb0, kb1;

    if (threadIdx.x == 0) {
        GTR(0);
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); armed[s] = -1; }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, EPI_WARPS); }
        *giveup = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) GTR(1);

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            GWAIT_DECL(gw_empty);
#ifdef BMB_GEMM_TRACE
            bool first_copy = true;
#endif
            while (ok && wi.next(tile, kb0, kb1)) {
                int tm, tn;
                const int bi = tile / tiles_per_problem;
                sch.coords(tile - bi * tiles_per_problem, tm, tn);
                const int a_row0 = bi * M, b_row0 = bi * N, k_row0 = bi * (kblocks * kelems_per_block);
                for (int kb = kb0; kb < kb1; ++kb) {
                    { GWAIT_BEGIN(); if (!mbar_wait(empty0 + 8 * s, ph ^ 1, giveup)) { ok = false; break; } GWAIT_END(gw_empty); }
                    const uint32_t fb = full0 + 8 * s;
                    mbar_arrive_expect_tx(fb, STAGE_BYTES);
                    armed[s] = (int)ph;
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + MH * A_BYTES;
                    const int k0 = kb * kelems_per_block;
                    if (a_mn == 2) {
                        tma_load_3d(sa, &mapA, 0, k_row0 + k0, tm * (BMT / 32), fb);       // all chunks in one copy
                    } else if (a_mn) {
#pragma unroll 1
                        for (int c = 0; c < BMT / 32; ++c) tma_load_2d(sa + c * CHUNK_BYTES, &mapA, tm * BMT + c * 32, k_row0 + k0, fb);
                    } else {
                        tma_load_2d(sa, &mapA, k0, a_row0 + tm * BMT, fb);
                    }
                    if (b_mn == 2) {
                        tma_load_3d(sb, &mapB, 0, k_row0 + k0, tn * (BN / 32), fb);
                    } else if (b_mn) {
#pragma unroll 1
                        for (int c = 0; c < BN / 32; ++c) tma_load_2d(sb + c * CHUNK_BYTES, &mapB, tn * BN + c * 32, k_row0 + k0, fb);
                    } else {
                        tma_load_2d(sb, &mapB, k0, b_row0 + tn * BN, fb);
                    }
#ifdef BMB_GEMM_TRACE
                    if (first_copy) { GTR(2); first_copy = false; }
#endif
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            GWAIT_FLUSH(12, gw_empty);
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
            GWAIT_DECL(gw_full);
            GWAIT_DECL(gw_tempty);
#ifdef BMB_GEMM_TRACE
            bool first_slice = true;
#endif
            while (ok && wi.next(tile, kb0, kb1)) {
                { GWAIT_BEGIN(); if (!mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, giveup)) { ok = false; break; } GWAIT_END(gw_tempty); }
                fence_after();
                const uint32_t d = tmem_base + (uint32_t)acc * ACC_COLS;
                for (int kb = kb0; kb < kb1; ++kb) {
                    { GWAIT_BEGIN(); if (!mbar_wait(full0 + 8 * s, ph, giveup)) { ok = false; break; } GWAIT_END(gw_full); }
                    fence_after();
#ifdef BMB_GEMM_TRACE
                    if (first_slice) { GTR(3); first_slice = false; }
#endif
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + MH * A_BYTES;
#pragma unroll
                    for (int k = 0; k < KBYTES / 32; ++k) {
                        const uint64_t db = b_mn ? smem_desc_mnmajor32(sb + k * b_step, CHUNK_BYTES) : smem_desc_kmajor(sb + k * b_step);
#pragma unroll
                        for (int hb = 0; hb < MH; ++hb) {       // the blocks of 128 rows, 16 KB apart in either layout
                            const uint32_t sah = sa + hb * A_BYTES + k * a_step;
                            const uint64_t da = a_mn ? smem_desc_mnmajor32(sah, CHUNK_BYTES) : smem_desc_kmajor(sah);
                            if (KIND == 0) mma_tf32(d + (uint32_t)hb * ACC_COLS, da, db, idesc, ((kb - kb0) | k) ? 1u : 0u);
                            else mma_f16(d + (uint32_t)hb * ACC_COLS, da, db, idesc, ((kb - kb0) | k) ? 1u : 0u);
                        }
                    }
                    commit(empty0 + 8 * s);             // slice reusable once these MMAs retire
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                commit(tfull0 + 8 * acc);               // accumulator complete
                GTR(4);
                if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
            }
            GWAIT_FLUSH(10, gw_full);
            GWAIT_FLUSH(11, gw_tempty);
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                          // TMEM lane quadrant this warp may read
        // the two warps of a quadrant take alternate 32-column chunks of one accumulator, or one block of rows each
        const int wgroup = (warp - 2) >> 2;
        const int chunk_first = MH == 2 ? 0 : wgroup, chunk_step = MH == 2 ? 1 : 2, hblock = MH == 2 ? wgroup : 0;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        GWAIT_DECL(gw_tfull);
        float *const C0 = C;
        while (ok && wi.next(tile, kb0, kb1)) {
            int tm, tn;
            const int bi = tile / tiles_per_problem;
            sch.coords(tile - bi * tiles_per_problem, tm, tn);
            float *C = C0 + (size_t)bi * M * N;          // this problem's result
            const bool whole = (kb0 == 0 && kb1 == kblocks);
            { GWAIT_BEGIN(); if (!mbar_wait(tfull0 + 8 * acc, acc_ph, giveup)) { ok = false; break; } GWAIT_END(gw_tfull); }
            fence_after();
#ifdef BMB_GEMM_TRACE
            if (warp == 2 && lane == 0 && g_gemm_trace[blockIdx.x & 255][9] == 0) { GTR(5); g_gemm_trace[blockIdx.x & 255][9] = 1; }
#endif
            // The accumulator leaves TMEM one row per thread; the rows are parked in shared memory and
            // written out four rows per instruction, each row segment a contiguous 128 bytes, so that
            // the global stores (loads of C, atomics) are fully coalesced.  A whole tile is stored; a
            // part of a stream-K tile is added into C.
            const int row_base = tm * BMT + hblock * BM + q * 32;
            const uint32_t trow = tmem_base + (uint32_t)(acc + hblock) * ACC_COLS + ((uint32_t)(q * 32) << 16);
            float *stg = reinterpret_cast<float *>(gen + STAGES * STAGE_BYTES) + (warp - 2) * (32 * 32);
            const int sub_r = lane >> 3, sub_u = lane & 7, sub_c = sub_u * 4;
            const float *part_bias = (kb0 == 0) ? bias : nullptr;
            if (whole && c_mode == 3) {
                // Direct path (beta 0, aligned C): the accumulator leaves TMEM in the 16x256b shape, where four
                // neighbouring lanes hold 32 contiguous bytes of a row, so the registers go straight to global
                // memory in whole sectors -- no trip through shared memory, whose bandwidth the main loop needs.
                // Two register sets: the tensor-memory load of the next 32-column chunk is in flight while this
                // chunk's stores are issued (the epilogue of a 256-row tile is not hidden behind a main loop).
                const int r0 = row_base + (lane >> 2), cq = 2 * (lane & 3);
                auto fetch = [&](int c, float (&lo)[16], float (&hi)[16]) {
                    tmem_ld_16x256b_x4_nowait(trow + (uint32_t)(c * 32), lo);                       // rows 0..15 of this quadrant
                    tmem_ld_16x256b_x4_nowait(trow + (uint32_t)(c * 32) + (16u << 16), hi);         // rows 16..31
                };
                auto put = [&](int c, const float (&lo)[16], const float (&hi)[16]) {
                    const int n0 = tn * BN + c * 32;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int n = n0 + 8 * j + cq;
                        if (n >= N) continue;
                        float2 bb = make_float2(0.f, 0.f);
                        if (bias) bb = *reinterpret_cast<const float2 *>(bias + n);
                        float2 o[4] = {make_float2(lo[4 * j], lo[4 * j + 1]), make_float2(lo[4 * j + 2], lo[4 * j + 3]),
                                       make_float2(hi[4 * j], hi[4 * j + 1]), make_float2(hi[4 * j + 2], hi[4 * j + 3])};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int m = r0 + 8 * k;
                            float2 x = make_float2(fmaf(alpha, o[k].x, bb.x), fmaf(alpha, o[k].y, bb.y));
                            if (round_c) x = make_float2(round_tf32(x.x), round_tf32(x.y));
                            if (m < M) *reinterpret_cast<float2 *>(C + (size_t)m * N + n) = x;
                            if (AUX && m < M) {                      // second output: GELU of the first
                                float2 g = (AUX == 2) ? make_float2(gelu_tanh_fast(x.x), gelu_tanh_fast(x.y))
                                                      : make_float2(gelu_tanh(x.x), gelu_tanh(x.y));
                                if (round_aux) g = make_float2(round_tf32(g.x), round_tf32(g.y));
                                *reinterpret_cast<float2 *>(aux + (size_t)m * N + n) = g;
                            }
                        }
                    }
                };
                auto live = [&](int c) { return c < BN / 32 && tn * BN + c * 32 < N; };     // warp-uniform
                float la[16], ha[16], lb[16], hb[16];
                int c = chunk_first;
                if (live(c)) fetch(c, la, ha);
#pragma unroll 1
                while (live(c)) {
                    tmem_wait_ld();
                    const int c2 = c + chunk_step;
                    if (live(c2)) fetch(c2, lb, hb);
                    put(c, la, ha);
                    if (!live(c2)) break;
                    tmem_wait_ld();
                    c = c2 + chunk_step;
                    if (live(c)) fetch(c, la, ha);
                    put(c2, lb, hb);
                }
            } else
#pragma unroll 1
            for (int c = chunk_first; c < BN / 32; c += chunk_step) {
                const int n0 = tn * BN + c * 32;
                if (n0 >= N) break;                      // warp-uniform
                float v[32];
                tmem_ld32(trow + (uint32_t)(c * 32), v);
                if (c_mode) {
                    // TMA path (C 16-byte aligned, N % 4 == 0, beta 0 or 1): finish the values in registers,
                    // park the 32 x 32 block in the swizzled layout the tensor map expects and let the
                    // copy engine store it (beta 0, whole tile) or add it into C (beta 1, stream-K parts).
                    if (row_base >= M) continue;         // warp-uniform; the box would lie outside C
                    const float *bsrc = whole ? bias : part_bias;
                    if (lane == 0) tma_store_wait_read();   // the previous block has left the staging buffer
                    __syncwarp();
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        float4 o = make_float4(alpha * v[4 * u], alpha * v[4 * u + 1], alpha * v[4 * u + 2], alpha * v[4 * u + 3]);
                        if (bsrc && n0 + 4 * u < N) {
                            const float4 bb = *reinterpret_cast<const float4 *>(bsrc + n0 + 4 * u);
                            o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                        }
                        if (round_c) o = make_float4(round_tf32(o.x), round_tf32(o.y), round_tf32(o.z), round_tf32(o.w));
                        *reinterpret_cast<float4 *>(stg + lane * 32 + ((u ^ (lane & 7)) << 2)) = o;
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (whole && c_mode == 1) tma_store_2d(&mapC, smem_u32(stg), n0, row_base);
                        else tma_reduce_add_2d(&mapC, smem_u32(stg), n0, row_base);
                        tma_store_commit();
                    }
                    continue;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    *reinterpret_cast<float4 *>(stg + lane * 32 + ((u ^ (lane & 7)) << 2)) =
                        make_float4(alpha * v[4 * u], alpha * v[4 * u + 1], alpha * v[4 * u + 2], alpha * v[4 * u + 3]);
                __syncwarp();
                const int n = n0 + sub_c;
                const bool vec = vec_ok && (n + 4 <= N);
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const int row = rr * 4 + sub_r;
                    const float4 o = *reinterpret_cast<const float4 *>(stg + row * 32 + ((sub_u ^ (row & 7)) << 2));
                    if (whole) store_result(o, C, M, N, row_base + row, n, vec, beta, bias, round_c);
                    else add_result(o, C, M, N, row_base + row, n, vec, part_bias);
                }
                __syncwarp();
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
            if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
#ifdef BMB_GEMM_TRACE
            if (warp == 2 && lane == 0) GTR(6);
#endif
        }
        if (warp == 2 && lane == 0) GWAIT_FLUSH(13, gw_tfull);
        if (c_mode && lane == 0) tma_store_wait_all();   // every block this warp handed to the copy engine has landed
#ifdef BMB_GEMM_TRACE
        if (warp == 2 && lane == 0) GTR(7);
#endif
    }

    fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *giveup) {
        *reinterpret_cast<volatile int *>(status) = 1;
        __threadfence_system();
    }
    if (threadIdx.x == 0) GTR(8);
}

// ---- the same GEMM on CTA pairs ----------------------------------------------------------------
// TF32 only.  Two CTAs (a cluster of 2, on neighbouring SMs) share one 256 x BN output tile: each loads
// its own 128 rows of A and HALF of the B slice, one thread of the leader CTA issues
// tcgen05.mma.cta_group::2 (M = 256) for both, and each CTA ends up with its 128 x BN block of the
// accumulator in its own tensor memory.  Against one CTA per 128 x 256 tile this halves the B bytes every
// SM has to land in and feed from shared memory (with fp32 operands it is shared-memory bandwidth that
// bounds a 128 x 256 tile at about two thirds of the tensor pipe's rate), and unlike the two-block tile
// of one CTA the accumulators stay double-buffered, so the epilogue of a tile still hides behind the
// next tile's products.
//   producer (warp 0, both CTAs)   waits for its own slot to be free, the leader arms its "full" barrier
//                                  with the bytes of BOTH CTAs, and each CTA's copies complete on the
//                                  leader's barrier (TMA without any multicast);
//   issuer (warp 1, leader only)   as in gemm_tc_k; when a slot's products retire it releases the slot in
//                                  both CTAs, and hands a finished accumulator to both CTAs' epilogues;
//   epilogue (warps 2..9, both)    as in gemm_tc_k, on the CTA's own 128 rows; the accumulator is handed
//                                  back by arriving on the leader's barrier.
// Work items are per pair.  Waits are bounded as everywhere; a pair leaves together (cluster barrier).
constexpr int PAIR_STAGES = 5;
constexpr int pair_smem_bytes(int bn) { return PAIR_STAGES * (A_BYTES + (bn / 2) * KBYTES) + 1024 + 256 + EPI_BYTES; }

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1)
gemm_tc_pair_k(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const __grid_constant__ CUtensorMap mapC, int c_mode, int M, int N, int kblocks, int kelems_per_block,
               int a_mn, int b_mn, float alpha, float beta, float *__restrict__ C, int vec_ok, int dp_tiles, int g_sk,
               const float *__restrict__ bias, int round_c, int *__restrict__ status) {
    constexpr int STAGES = PAIR_STAGES, BMT = 2 * BM, BH = BN / 2;
    constexpr int B_BYTES = BH * KBYTES, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t ACC_COLS = BN > 128 ? 256 : 128;
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + STAGES * STAGE_BYTES + EPI_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *giveup = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;

    TileSched sch;
    sch.tiles_m = (M + BMT - 1) / BMT;
    sch.tiles_n = (N + BN - 1) / BN;
    sch.num_tiles = sch.tiles_m * sch.tiles_n;
    WorkIter wi;
    wi.init((int)(blockIdx.x >> 1), (int)(gridDim.x >> 1), dp_tiles, sch.num_tiles - dp_tiles, kblocks, g_sk);
    int tile, kb0, kb1;

    if (threadIdx.x == 0) {
        GTR(0);
        // full: the leader's own arrival (with the byte count of both CTAs); empty, tmem_full: one arrival
        // from the leader's issuer per use; tmem_empty (used in the leader only): the epilogue warps of both CTAs
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 2 * EPI_WARPS); }
        *giveup = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    fence_before();
    __syncthreads();
    cluster_sync_all();                                // both CTAs' barriers exist before anyone signals across
    fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Each CTA asked its own SM for all the columns it will ever use, so both got the same address; the
    // pair instruction writes the same columns on both SMs and relies on that.
    if (threadIdx.x == 0 && rank == 0 && ld_shared_cluster_u32(map_to_cta(smem_u32(tmem_slot), 1)) != tmem_base) *giveup = 1;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (each CTA for its own tiles)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            GWAIT_DECL(gw_empty);
            int armed_par[STAGES];
            for (int i = 0; i < STAGES; ++i) armed_par[i] = -1;
            while (ok && wi.next(tile, kb0, kb1)) {
                int tm, tn;
                sch.coords(tile, tm, tn);
                const int a_x0 = tm * BMT + (int)rank * BM, b_x0 = tn * BN + (int)rank * BH;
                for (int kb = kb0; kb < kb1; ++kb) {
                    { GWAIT_BEGIN(); if (!mbar_wait(empty0 + 8 * s, ph ^ 1, giveup)) { ok = false; break; } GWAIT_END(gw_empty); }
                    const uint32_t fb_local = full0 + 8 * s;
                    if (rank == 0) { mbar_arrive_expect_tx(fb_local, 2 * STAGE_BYTES); armed_par[s] = (int)ph; }
                    const uint32_t fb = map_to_cta(fb_local, 0);
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
                    const int k0 = kb * kelems_per_block;
                    if (a_mn == 2) tma_load_3d_pair(sa, &mapA, 0, k0, a_x0 / 32, fb);
                    else tma_load_2d_pair(sa, &mapA, k0, a_x0, fb);
                    if (b_mn == 2) tma_load_3d_pair(sb, &mapB, 0, k0, b_x0 / 32, fb);
                    else tma_load_2d_pair(sb, &mapB, k0, b_x0, fb);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            GWAIT_FLUSH(12, gw_empty);
            // Do not leave while the issuer's releases of the last slots may still be on their way to this
            // CTA's barriers: wait until every slot has been handed back.
            for (int i = 0; ok && i < STAGES; ++i) {
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1, giveup)) ok = false;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (!ok && rank == 0) {
                // the leader's barriers count the bytes of both CTAs: once they have completed, no copy of
                // the pair is in flight any more (the peer stays until the cluster barrier at the end)
                for (int i = 0; i < STAGES; ++i)
                    if (armed_par[i] >= 0) mbar_drain(full0 + 8 * i, (uint32_t)armed_par[i]);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- issuer (leader only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc(2u, a_mn ? 1u : 0u, b_mn ? 1u : 0u, BN, BMT);
            const uint32_t a_step = a_mn ? 1024u : 32u, b_step = b_mn ? 1024u : 32u;
            const uint32_t peer_empty0 = map_to_cta(empty0, 1), peer_tfull0 = map_to_cta(tfull0, 1);
            int s = 0, acc = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            GWAIT_DECL(gw_full);
            GWAIT_DECL(gw_tempty);
            while (ok && wi.next(tile, kb0, kb1)) {
                { GWAIT_BEGIN(); if (!mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, giveup)) { ok = false; break; } GWAIT_END(gw_tempty); }
                fence_after();
                const uint32_t d = tmem_base + (uint32_t)acc * ACC_COLS;
                for (int kb = kb0; kb < kb1; ++kb) {
                    { GWAIT_BEGIN(); if (!mbar_wait(full0 + 8 * s, ph, giveup)) { ok = false; break; } GWAIT_END(gw_full); }
                    fence_after();
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
                    for (int k = 0; k < KBYTES / 32; ++k) {
                        const uint64_t db = b_mn ? smem_desc_mnmajor32(sb + k * b_step, CHUNK_BYTES) : smem_desc_kmajor(sb + k * b_step);
                        const uint64_t da = a_mn ? smem_desc_mnmajor32(sa + k * a_step, CHUNK_BYTES) : smem_desc_kmajor(sa + k * a_step);
                        mma_tf32_pair(d, da, db, idesc, ((kb - kb0) | k) ? 1u : 0u);
                    }
                    commit_pair(empty0 + 8 * s);                 // the slot is reusable, here ...
                    commit_pair(peer_empty0 + 8 * s);            // ... and in the peer CTA
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                commit_pair(tfull0 + 8 * acc);
                commit_pair(peer_tfull0 + 8 * acc);
                GTR(4);
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
            GWAIT_FLUSH(10, gw_full);
            GWAIT_FLUSH(11, gw_tempty);
        }
    } else {
        // ------------------------------------------------------------ epilogue (each CTA for its own 128 rows)
        const int q = warp & 3;
        const int wgroup = (warp - 2) >> 2;
        const uint32_t leader_tempty0 = map_to_cta(tempty0, 0);
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        GWAIT_DECL(gw_tfull);
        while (ok && wi.next(tile, kb0, kb1)) {
            int tm, tn;
            sch.coords(tile, tm, tn);
            const bool whole = (kb0 == 0 && kb1 == kblocks);
            { GWAIT_BEGIN(); if (!mbar_wait(tfull0 + 8 * acc, acc_ph, giveup)) { ok = false; break; } GWAIT_END(gw_tfull); }
            fence_after();
            const int row_base = tm * BMT + (int)rank * BM + q * 32;
            const uint32_t trow = tmem_base + (uint32_t)acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
            float *stg = reinterpret_cast<float *>(gen + STAGES * STAGE_BYTES) + (warp - 2) * (32 * 32);
            const int sub_r = lane >> 3, sub_u = lane & 7, sub_c = sub_u * 4;
            const float *part_bias = (kb0 == 0) ? bias : nullptr;
#pragma unroll 1
            for (int c = wgroup; c < BN / 32; c += 2) {
                const int n0 = tn * BN + c * 32;
                if (n0 >= N) break;
                if (whole && c_mode == 3) {
                    float lo[16], hi[16];
                    tmem_ld_16x256b_x4_nowait(trow + (uint32_t)(c * 32), lo);
                    tmem_ld_16x256b_x4_nowait(trow + (uint32_t)(c * 32) + (16u << 16), hi);
                    tmem_wait_ld();
                    const int r0 = row_base + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int n = n0 + 8 * j + cq;
                        if (n >= N) continue;
                        float2 bb = make_float2(0.f, 0.f);
                        if (bias) bb = *reinterpret_cast<const float2 *>(bias + n);
                        float2 o[4] = {make_float2(lo[4 * j], lo[4 * j + 1]), make_float2(lo[4 * j + 2], lo[4 * j + 3]),
                                       make_float2(hi[4 * j], hi[4 * j + 1]), make_float2(hi[4 * j + 2], hi[4 * j + 3])};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int m = r0 + 8 * k;
                            float2 x = make_float2(fmaf(alpha, o[k].x, bb.x), fmaf(alpha, o[k].y, bb.y));
                            if (round_c) x = make_float2(round_tf32(x.x), round_tf32(x.y));
                            if (m < M) *reinterpret_cast<float2 *>(C + (size_t)m * N + n) = x;
                        }
                    }
                    continue;
                }
                float v[32];
                tmem_ld32(trow + (uint32_t)(c * 32), v);
                if (c_mode) {
                    if (row_base >= M) continue;
                    const float *bsrc = whole ? bias : part_bias;
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        float4 o = make_float4(alpha * v[4 * u], alpha * v[4 * u + 1], alpha * v[4 * u + 2], alpha * v[4 * u + 3]);
                        if (bsrc && n0 + 4 * u < N) {
                            const float4 bb = *reinterpret_cast<const float4 *>(bsrc + n0 + 4 * u);
                            o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                        }
                        if (round_c) o = make_float4(round_tf32(o.x), round_tf32(o.y), round_tf32(o.z), round_tf32(o.w));
                        *reinterpret_cast<float4 *>(stg + lane * 32 + ((u ^ (lane & 7)) << 2)) = o;
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (whole && c_mode == 1) tma_store_2d(&mapC, smem_u32(stg), n0, row_base);
                        else tma_reduce_add_2d(&mapC, smem_u32(stg), n0, row_base);
                        tma_store_commit();
                    }
                    continue;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    *reinterpret_cast<float4 *>(stg + lane * 32 + ((u ^ (lane & 7)) << 2)) =
                        make_float4(alpha * v[4 * u], alpha * v[4 * u + 1], alpha * v[4 * u + 2], alpha * v[4 * u + 3]);
                __syncwarp();
                const int n = n0 + sub_c;
                const bool vec = vec_ok && (n + 4 <= N);
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const int row = rr * 4 + sub_r;
                    const float4 o = *reinterpret_cast<const float4 *>(stg + row * 32 + ((sub_u ^ (row & 7)) << 2));
                    if (whole) store_result(o, C, M, N, row_base + row, n, vec, beta, bias, round_c);
                    else add_result(o, C, M, N, row_base + row, n, vec, part_bias);
                }
                __syncwarp();
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tempty0 + 8 * acc);      // the issuer counts both CTAs' warps
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (warp == 2 && lane == 0) GWAIT_FLUSH(13, gw_tfull);
        if (c_mode && lane == 0) tma_store_wait_all();
    }

    fence_before();
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves (or frees tensor memory) while the other may still signal it
    if (warp == 1) {
        __syncwarp();
        fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *giveup) {
        *reinterpret_cast<volatile int *>(status) = 4;
        __threadfence_system();
    }
    if (threadIdx.x == 0) GTR(8);
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
    bool map3d;           // MN-major with the extent a multiple of 32: one 3-d copy per slice
    int tile_chunks;      // 32-wide chunks per tile (3-d map only)
    bool staged = false;  // ptr is a converted copy in the per-device staging scratch
};
// Marks the staging slots this call wrote as used by its stream when the call returns (its last launch reads
// them): the next caller on another stream of the device waits for that launch before overwriting them.
struct StagingRelease {
    const Operand &a, &b;
    cudaStream_t st;
    ~StagingRelease() {
        if (a.staged) scratch_release(SCR_GEMM_A, st);
        if (b.staged) scratch_release(SCR_GEMM_B, st);
    }
};

inline int blocks_for(long long items) {
    long long b = (items + 255) / 256, cap = 8LL * sm_count();
    return (int)(b > cap ? cap : (b < 1 ? 1 : b));
}

// Decide how an operand reaches the tensor core.  X = its M or N extent, kcontig =
// element (x,k) at src[x*K + k], otherwise at src[k*X + x].
// `batch` dense problems one after the other (batch > 1 only reaches here with geometry the direct route takes).
int stage_operand(Operand *op, const float *src, bool kcontig, long long X, int K, bool bf16, bool rounded,
                  ScratchSlot slot, int tile_rows, cudaStream_t st, int batch = 1) {
    const bool aligned = ((uintptr_t)src % 16) == 0;
    if (!bf16) {
        const bool geom_ok = aligned && (kcontig ? (K % 4 == 0) : (X % 4 == 0));
        if (geom_ok) {
            const float *use = src;
            if (!rounded) {
                float *scr = (float *)device_scratch(slot, (size_t)batch * X * K * sizeof(float));
                if (!scr) return BMB_E_CUDA;
                BMB_TRY(scratch_acquire(slot, st));
                op->staged = true;
                const long long n4 = (long long)batch * X * (long long)K / 4;
                prep_round_vec4_k<<<blocks_for(n4), 256, 0, st>>>(scr, src, n4);
                count_launch();
                BMB_LAUNCH_CHECK();
                use = scr;
            }
            op->ptr = use;
            op->mn_major = !kcontig;
            op->map3d = false;
            op->tile_chunks = 0;
            if (kcontig) { op->rows = X * batch; op->cols = K; op->pitch_bytes = (long long)K * 4; op->box_rows = tile_rows; }
            else { op->rows = (long long)K * batch; op->cols = X; op->pitch_bytes = X * 4; op->box_rows = 32; op->map3d = (X % 32 == 0); op->tile_chunks = tile_rows / 32; }
            return BMB_OK;
        }
    }
    // General route: a K-major, padded, converted copy.
    const int esize = bf16 ? 2 : 4, kalign = 16 / esize;
    const int Kp = (K + kalign - 1) / kalign * kalign;
    void *scr = device_scratch(slot, (size_t)X * Kp * esize);
    if (!scr) return BMB_E_CUDA;
    BMB_TRY(scratch_acquire(slot, st));
    op->staged = true;
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
    op->ptr = scr; op->mn_major = false; op->map3d = false; op->tile_chunks = 0;
    op->rows = X; op->cols = Kp; op->pitch_bytes = (long long)Kp * esize; op->box_rows = tile_rows;
    return BMB_OK;
}

std::mutex g_attr_mu;

}  // namespace

bool gemm_tc_accepts(int math, int transA, int transB, int batch, int M, int N, int K, const float *A, long long sA,
                     const float *B, long long sB, const float *C, long long sC) {
    if (math != BMB_MATH_TF32 && math != BMB_MATH_BF16) return false;
    // Problems smaller than one tile stay on the SIMT kernel (fp32-exact, so within any tensor-core tolerance).
    if (M < BM || N < BN_NARROW || K < 32 || !C) return false;
    if ((long long)M * K >= (1LL << 40) || (long long)N * K >= (1LL << 40)) return false;
    if (batch != 1) {
        // Batched: TF32, dense strides, operands the tensor maps can read where they lie; an MN-major
        // operand additionally needs K % 32 == 0 so that a K slice never runs into the next problem.
        if (math != BMB_MATH_TF32) return false;
        if (sA != (long long)M * K || sB != (long long)K * N || sC != (long long)M * N) return false;
        const bool a_kc = !transA, b_kc = transB != 0;
        if ((((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) != 0) return false;
        if ((a_kc ? K : M) % 4 != 0 || (b_kc ? K : N) % 4 != 0) return false;
        if ((!a_kc || !b_kc) && K % 32 != 0) return false;
        if ((long long)batch * M >= (1LL << 31) || (long long)batch * N >= (1LL << 31) || (long long)batch * K >= (1LL << 31)) return false;
    }
    return true;
}

namespace {

// C = beta * C over the tiles [dp_tiles, num_tiles) (the stream-K tiles), before their parts are added.
__global__ void __launch_bounds__(256) sk_prepare_k(float *__restrict__ C, int M, int N, int tiles_m, int tiles_n, int dp_tiles,
                                                    int bm, int bn, float beta, int vec_ok) {
    TileSched sch;
    sch.tiles_m = tiles_m; sch.tiles_n = tiles_n; sch.num_tiles = tiles_m * tiles_n;
    int tm, tn;
    sch.coords(dp_tiles + (int)blockIdx.x, tm, tn);
    const int m0 = tm * bm, n0 = tn * bn;
    const int rows = min(bm, M - m0), cols = min(bn, N - n0);
    if (vec_ok && cols % 4 == 0) {
        const int c4 = cols / 4;
        for (int i = threadIdx.x; i < rows * c4; i += blockDim.x) {
            float4 *p = reinterpret_cast<float4 *>(C + (size_t)(m0 + i / c4) * N + n0) + i % c4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (beta != 0.0f) { v = *p; v.x *= beta; v.y *= beta; v.z *= beta; v.w *= beta; }
            *p = v;
        }
    } else {
        for (int i = threadIdx.x; i < rows * cols; i += blockDim.x) {
            float *p = C + (size_t)(m0 + i / cols) * N + n0 + i % cols;
            *p = (beta != 0.0f) ? beta * *p : 0.0f;
        }
    }
}

// Relative cost of one K slice of a tile `bn` columns wide (the narrower tiles re-read A more often
// and amortise the epilogue less well).
double slice_cost(int bn) { return bn == 256 ? 256.0 : (bn == 192 ? 200.0 : (bn == 128 ? 150.0 : 110.0)); }

// Pick the tile width and how many tiles to hand out whole; the rest (a last, partly filled wave, or a
// problem smaller than one wave) is shared between CTAs along K.  Costs are in K-slice units of a
// 256-wide tile; a tile pays ~4 slices for its epilogue, sharing a tile ~6 more.
// A tile of two row blocks (256 x 256) costs `tall_slice` slices of a 128 x 256 tile per slice (fitted to
// measurements: 1.72 for twice the work) and, its epilogue no longer hidden, `tall_epi` slices more per
// tile; sharing such tiles between CTAs costs more than sharing the small ones.
void choose_schedule(int M, int N, int kblocks, int ctas, bool allow_split, int force_bn, int force_mh, bool tall_ok,
                     int *bn_out, int *mh_out, int *dp_tiles_out) {
    static const double tall_slice = [] { const char *e = getenv("BMB_GEMM_TALL_SLICE"); return e ? atof(e) : 1.72; }();
    static const double tall_epi = [] { const char *e = getenv("BMB_GEMM_TALL_EPI"); return e ? atof(e) : 8.0; }();
    const int widths[5] = {256, 256, 192, 128, 64};
    double best = -1.0;
    for (int cand = 0; cand < 5; ++cand) {
        const int w = widths[cand], mh = cand == 0 ? 2 : 1;
        const bool tall_possible = tall_ok && M >= 2 * BM && N >= 256;
        if (mh == 2 && (!tall_possible || force_mh == 1)) continue;
        if (mh == 1 && force_mh == 2 && tall_possible) continue;
        if (force_bn ? (w != force_bn) : ((w > 64 && N < w) || (w == 64 && N >= 128))) continue;
        const int tiles_m = (M + mh * BM - 1) / (mh * BM);
        const long long tiles = (long long)tiles_m * ((N + w - 1) / w);
        const long long full = tiles / ctas, rem = tiles % ctas;
        const double unit = mh == 2 ? tall_slice : slice_cost(w) / 256.0;
        const double epi = mh == 2 ? tall_epi : 4.0;
        const double whole = (double)(full + (rem ? 1 : 0)) * (kblocks + epi) * unit;
        double cost = whole;
        int dp = (int)tiles;
        if (allow_split && rem && kblocks >= 8) {
            const double run = (double)((rem * kblocks + ctas - 1) / ctas);          // K slices of a CTA's shared run
            const double shared = ((double)full * (kblocks + epi) + run + (mh == 2 ? 24.0 : 10.0)) * unit;
            // With a short K a shared run that is a sizeable part of a CTA's work costs more than the model says
            // (measured at 8192 x 768 x 768 on 74 CTAs: 45.3 us shared against 37.5 us with a third, partly filled
            // wave; the preparing launch and the parts' reductions do not shrink with K): keep such tiles whole.
            const bool short_k_big_run = kblocks <= 32 && run > 0.10 * ((double)full * (kblocks + epi) + run);
            if (shared < whole && !short_k_big_run) { cost = shared; dp = (int)(tiles - rem); }
        }
        if (best < 0.0 || cost < best) { best = cost; *bn_out = w; *mh_out = mh; *dp_tiles_out = dp; }
    }
}

// Everything the launch decides about how the tiles are handed out.
struct Plan { int bn, mh, kblocks, tiles_m, tiles_n, tiles, dp_tiles, sk_tiles, g_sk, grid; bool pair; };

// CTA pairs this device can keep resident at once for the pair kernel (one CTA per SM, clusters of 2).
int pair_clusters();

// Whether a problem goes to the pair kernel: TF32, one problem, at least one 256 x 256 tile, and operands
// the pair kernel's loads take (an M- or N-contiguous operand needs its extent to be a multiple of 32).
// BMB_GEMM_PAIR / BMB_GEMM_NO_PAIR in the flags decide for a call; the environment variable
// BMB_GEMM_PAIR=1 makes pairs the default where the shape allows.
bool wants_pair(bool bf16, int flags, int transA, int transB, int batch, int M, int N) {
    // Measured on the step's shapes the pair form runs within +-6 % of single CTAs (both sit at the same
    // shared-memory bandwidth bound: a CTA of a pair still feeds its half of B to both tensor cores), so it
    // is opt-in.
    static const bool env_on = [] { const char *e = getenv("BMB_GEMM_PAIR"); return e && atoi(e) != 0; }();
    if (bf16 || batch != 1 || M < 2 * BM || N < 256) return false;
    if ((transA && M % 32) || (!transB && N % 32)) return false;
    if (flags & BMB_GEMM_NO_PAIR) return false;
    if (flags & (BMB_GEMM_TILE_M128 | BMB_GEMM_TILE_M256)) return (flags & BMB_GEMM_PAIR) != 0;
    return (flags & BMB_GEMM_PAIR) ? true : env_on;
}

// The pair kernel's plan: 256 x 256 tiles handed to `clusters` CTA pairs; what does not fill a wave of
// pairs is shared along K like in the one-CTA kernel.
void plan_pair(Plan *p, int flags, int M, int N, int clusters) {
    p->pair = true;
    p->bn = 256;
    p->mh = 2;
    p->tiles_m = (M + 2 * BM - 1) / (2 * BM);
    p->tiles_n = (N + 255) / 256;
    p->tiles = p->tiles_m * p->tiles_n;
    const bool allow_split = !(flags & (BMB_GEMM_NO_SPLIT | BMB_GEMM_C_ROUNDED));
    const int full = p->tiles / clusters, rem = p->tiles % clusters;
    p->dp_tiles = p->tiles;
    if (allow_split && rem && p->kblocks >= 8) {
        const double whole = (double)(full + 1) * (p->kblocks + 4.0);
        const double shared = (double)full * (p->kblocks + 4.0) + (double)(((long long)rem * p->kblocks + clusters - 1) / clusters) + 10.0;
        if (shared < whole) p->dp_tiles = p->tiles - rem;
    }
    p->sk_tiles = p->tiles - p->dp_tiles;
    p->g_sk = 1;
    if (p->sk_tiles > 0) {
        const long long runs = (long long)p->sk_tiles * p->kblocks / 4;
        p->g_sk = (int)(runs < 1 ? 1 : (runs > clusters ? clusters : runs));
    }
    p->grid = p->sk_tiles > 0 ? (p->dp_tiles >= clusters ? clusters : (p->dp_tiles > p->g_sk ? p->dp_tiles : p->g_sk))
                              : (p->tiles < clusters ? p->tiles : clusters);          // in pairs
}

int plan_gemm(Plan *p, bool bf16, int flags, int batch, int M, int N, int K, int ctas) {
    const int kper = KBYTES / (bf16 ? 2 : 4);
    p->kblocks = (K + kper - 1) / kper;
    p->pair = false;
    // Sharing tiles between CTAs adds parts into C in whatever order they finish, so the last bits of
    // such a result vary from run to run, and a rounded result would need another pass: both
    // BMB_GEMM_NO_SPLIT and BMB_GEMM_C_ROUNDED keep every tile on one CTA; so do batched problems.
    const bool allow_split = !(flags & (BMB_GEMM_NO_SPLIT | BMB_GEMM_C_ROUNDED)) && batch == 1;
    static const int force_bn = [] { const char *e = getenv("BMB_GEMM_TILE_N"); const int v = e ? atoi(e) : 0; return (v == 256 || v == 192 || v == 128 || v == 64) ? v : 0; }();
    // BMB_GEMM_TILE_M = 128 or 256 forces the tile height where the shape allows it.  BF16 problems keep
    // the 128-row tile: measured at 8192^3, the tall tile ran at 889 TFLOP/s against 979.
    static const int force_mh = [] { const char *e = getenv("BMB_GEMM_TILE_M"); const int v = e ? atoi(e) : 0; return v == 256 ? 2 : (v == 128 ? 1 : 0); }();
    p->bn = BN_WIDE;
    p->mh = 1;
    p->dp_tiles = 0;
    // A call may force the height itself (BMB_GEMM_TILE_M128 / _M256), which wins over the environment.
    const int call_mh = (flags & BMB_GEMM_TILE_M256) ? 2 : ((flags & BMB_GEMM_TILE_M128) ? 1 : force_mh);
    choose_schedule(M, N, p->kblocks, ctas, allow_split, (force_bn && N >= force_bn) ? force_bn : 0, call_mh, batch == 1 && !bf16, &p->bn, &p->mh,
                    &p->dp_tiles);
    p->tiles_m = (M + p->mh * BM - 1) / (p->mh * BM);
    p->tiles_n = (N + p->bn - 1) / p->bn;
    const long long tiles_ll = (long long)p->tiles_m * p->tiles_n * batch;
    if (tiles_ll >= (1LL << 31)) return fail(BMB_E_LIMIT, "gemm_tc: %lld tiles", tiles_ll);
    p->tiles = (int)tiles_ll;
    if (batch > 1) p->dp_tiles = p->tiles;
    p->sk_tiles = p->tiles - p->dp_tiles;
    p->g_sk = 1;
    if (p->sk_tiles > 0) {
        const long long runs = (long long)p->sk_tiles * p->kblocks / 4;       // at least 4 K slices per run
        p->g_sk = (int)(runs < 1 ? 1 : (runs > ctas ? ctas : runs));
    }
    p->grid = p->sk_tiles > 0 ? (p->dp_tiles >= ctas ? ctas : (p->dp_tiles > p->g_sk ? p->dp_tiles : p->g_sk))
                              : (p->tiles < ctas ? p->tiles : ctas);
    // A problem shared as a whole (fewer tiles than would fill two waves, a long K) whose operands do not fit L2:
    // with end-to-end runs every CTA is at a different depth of K, and an operand panel shared by several tiles is
    // fetched from DRAM once per tile (measured at 8192 x 768 x 50304: 6.2 GB for 1.8 GB of operands, the launch
    // DRAM-bound).  The chunk-major order keeps all CTAs at about the same depth.  Chunks: the smallest count from 4
    // that fills the last round of items to 99 % (else the best up to 40), at least 16 K slices per item.
    static const bool no_chunks = getenv("BMB_GEMM_NO_KCHUNKS") != nullptr;
    const double operand_bytes = ((double)M + (double)N) * (double)K * (bf16 ? 2.0 : 4.0);
    // The bar is twice the 126 MB L2.  Weight-gradient products whose operands are about one L2 (2304 x 768 x 8192 on
    // half the SMs: 101 MB, 54 tiles) ran slower in this order (101 us against 79 us with end-to-end runs: three
    // partial-tile additions per CTA instead of one or two, for operands that mostly stay in L2 anyway).
    const double min_bytes = 252.0e6;
    if (!no_chunks && p->sk_tiles == p->tiles && p->dp_tiles == 0 && p->grid == ctas && p->g_sk == ctas && operand_bytes > min_bytes) {
        int best = 0;
        double best_eff = 0.0;
        for (int s = 4; s <= 40 && p->kblocks / s >= 16; ++s) {
            const long long items = (long long)p->tiles * s;
            const double eff = (double)items / (double)(((items + ctas - 1) / ctas) * ctas);
            if (eff > best_eff + 1e-9) { best_eff = eff; best = s; }
            if (eff >= 0.99) { best = s; best_eff = eff; break; }
        }
        if (best && best_eff >= 0.97) p->g_sk = -best;
    }
    return BMB_OK;
}

template <int KIND, int BN, int MH, int AUX = 0>
int launch_tc(int grid, cudaStream_t st, const CUtensorMap &mapA, const CUtensorMap &mapB, const CUtensorMap &mapC, int c_mode,
              int batch, int M, int N, int kblocks, int kper,
              int amn, int bmn, float alpha, float beta, float *C, int vec_ok, int dp_tiles, int g_sk, const float *bias,
              int round_c, int *status_dev, float *aux, int round_aux) {
    static bool attr_set[64];
    {
        std::lock_guard<std::mutex> lk(g_attr_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !attr_set[d]) {
            BMB_CUDA(cudaFuncSetAttribute(gemm_tc_k<KIND, BN, MH, AUX>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(BN, MH)));
            attr_set[d] = true;
        }
    }
    gemm_tc_k<KIND, BN, MH, AUX><<<grid, NTHREADS, smem_bytes(BN, MH), st>>>(mapA, mapB, mapC, c_mode, batch, M, N, kblocks, kper, amn, bmn, alpha, beta, C, vec_ok,
                                                                dp_tiles, g_sk, bias, round_c, status_dev, aux, round_aux);
    return BMB_OK;
}

template <int BN>
int launch_pair(int pairs, cudaStream_t st, const CUtensorMap &mapA, const CUtensorMap &mapB, const CUtensorMap &mapC, int c_mode,
                int M, int N, int kblocks, int kper, int amn, int bmn, float alpha, float beta, float *C, int vec_ok, int dp_tiles,
                int g_sk, const float *bias, int round_c, int *status_dev) {
    static bool attr_set[64];
    {
        std::lock_guard<std::mutex> lk(g_attr_mu);
        const int d = current_device();
        if (d >= 0 && d < 64 && !attr_set[d]) {
            BMB_CUDA(cudaFuncSetAttribute(gemm_tc_pair_k<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_bytes(BN)));
            attr_set[d] = true;
        }
    }
    gemm_tc_pair_k<BN><<<2 * pairs, NTHREADS, pair_smem_bytes(BN), st>>>(mapA, mapB, mapC, c_mode, M, N, kblocks, kper, amn, bmn, alpha, beta,
                                                                       C, vec_ok, dp_tiles, g_sk, bias, round_c, status_dev);
    return BMB_OK;
}

int pair_clusters() {
    static int cache[64];
    const int d = current_device();
    if (d < 0 || d >= 64) return 1;
    std::lock_guard<std::mutex> lk(g_attr_mu);
    if (cache[d] == 0) {
        int n = 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)(sm_count() / 2));
        cfg.blockDim = dim3(NTHREADS);
        cfg.dynamicSmemBytes = pair_smem_bytes(256);
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        cudaFuncSetAttribute(gemm_tc_pair_k<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_bytes(256));
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_k<256>, &cfg) != cudaSuccess || n < 1) { cudaGetLastError(); n = sm_count() / 2; }
        if (n > sm_count() / 2) n = sm_count() / 2;
        cache[d] = n;
    }
    return cache[d];
}

}  // namespace

// aux_gelu (optional): a second output, GELU (tanh form, src/nn.cu:118-127) of the result, rounded to TF32 when the
// library is emitting rounded operands -- the MLP's activation rides in the epilogue of the product before it.
// Served where every tile is stored by one CTA straight from registers (beta 0, aligned C, no tile shared
// along K, which costs a problem of many tiles about 1 %); otherwise the caller gets BMB_E_UNSUPPORTED with C
// untouched and applies the activation itself.
int gemm_tc(int math, int flags, int transA, int transB, int batch, int M, int N, int K, float alpha,
            const float *A, long long, const float *B, long long, float beta, float *C, long long,
            const float *bias, cudaStream_t st, float *aux_gelu) {
    if (aux_gelu) flags |= BMB_GEMM_NO_SPLIT | BMB_GEMM_NO_PAIR | BMB_GEMM_TILE_M128;
    int *status_dev = nullptr;
    volatile int *status_host = nullptr;
    BMB_TRY(tc::status_word(&status_dev, &status_host));
    if (*status_host != 0)
        return fail(BMB_E_TIMEOUT, "an earlier tensor-core kernel on this device gave up waiting on a barrier");
    const bool bf16 = (math == BMB_MATH_BF16);
    const int esize = bf16 ? 2 : 4;
    const int kper = KBYTES / esize;
    // BMB_GEMM_HALF_SMS: plan for half of the SMs, so that two such launches on two streams run side by side
    const int ctas = (flags & BMB_GEMM_HALF_SMS) ? (sm_count() + 1) / 2 : sm_count();
    Plan plan;
    BMB_TRY(plan_gemm(&plan, bf16, flags, batch, M, N, K, ctas));
    if (wants_pair(bf16, flags, transA, transB, batch, M, N))
        plan_pair(&plan, flags, M, N, (flags & BMB_GEMM_HALF_SMS) ? (pair_clusters() + 1) / 2 : pair_clusters());
    const int kblocks = plan.kblocks, bn = plan.bn, dp_tiles = plan.dp_tiles;
    Operand a, b;
    StagingRelease release_on_return{a, b, st};
    // per CTA: the pair kernel loads 128 rows of A and half of the B tile
    BMB_TRY(stage_operand(&a, A, !transA, M, K, bf16, (flags & BMB_GEMM_A_ROUNDED) != 0, SCR_GEMM_A, plan.pair ? BM : plan.mh * BM, st, batch));
    BMB_TRY(stage_operand(&b, B, transB != 0, N, K, bf16, (flags & BMB_GEMM_B_ROUNDED) != 0, SCR_GEMM_B, plan.pair ? bn / 2 : bn, st, batch));
    CUtensorMap mapA, mapB;
    if (a.map3d) BMB_TRY(make_map_mn3d(&mapA, a.ptr, a.rows, a.cols, a.pitch_bytes, a.tile_chunks));
    else BMB_TRY(make_map_2d(&mapA, a.ptr, esize, a.rows, a.cols, a.pitch_bytes, a.box_rows, a.mn_major));
    if (b.map3d) BMB_TRY(make_map_mn3d(&mapB, b.ptr, b.rows, b.cols, b.pitch_bytes, b.tile_chunks));
    else BMB_TRY(make_map_2d(&mapB, b.ptr, esize, b.rows, b.cols, b.pitch_bytes, b.box_rows, b.mn_major));
    const int tiles_m = plan.tiles_m, tiles_n = plan.tiles_n;
    const int vec_ok = ((uintptr_t)C % 16 == 0) && (N % 4 == 0);
    const int sk_tiles = plan.sk_tiles, g_sk = plan.g_sk, grid = plan.grid;
    if (sk_tiles > 0 && beta != 1.0f) {
        sk_prepare_k<<<sk_tiles, 256, 0, st>>>(C, M, N, tiles_m, tiles_n, dp_tiles, plan.mh * BM, bn, beta, vec_ok);
        count_launch();
    }
    const int round_c = (flags & BMB_GEMM_C_ROUNDED) ? 1 : 0;
    const int amn = bf16 ? 0 : (a.mn_major ? (a.map3d ? 2 : 1) : 0), bmn = bf16 ? 0 : (b.mn_major ? (b.map3d ? 2 : 1) : 0);
    // The epilogue hands finished 32 x 32 blocks to the copy engine when C allows a tensor map
    // (16-byte aligned rows) and beta is 0 (store) or 1 (add); otherwise the warps store themselves.
    CUtensorMap mapC;
    memset(&mapC, 0, sizeof(mapC));
    static const bool no_tma_store = getenv("BMB_GEMM_NO_TMA_STORE") != nullptr;
    static const bool no_direct = getenv("BMB_GEMM_NO_DIRECT") != nullptr;
    // 3 = whole tiles stored straight from registers (beta 0), parts of shared tiles added by the copy engine
    int c_mode = (!no_tma_store && vec_ok && (beta == 0.0f || beta == 1.0f)) ? (beta == 0.0f ? (no_direct ? 1 : 3) : 2) : 0;
    if (batch > 1 && c_mode != 3) c_mode = 0;        // the tensor map over C describes one problem only
    float *aux = aux_gelu;
    const int round_aux = emit_rounded() ? 1 : 0;
    if (aux && (c_mode != 3 || plan.pair || plan.sk_tiles > 0 || batch != 1 || ((uintptr_t)aux & 15) || bf16 || plan.mh != 1 || bn < 128))
        return fail(BMB_E_UNSUPPORTED, "gemm_tc: the fused activation needs beta 0, an aligned C and whole tiles");
    if (c_mode) BMB_TRY(make_map_2d(&mapC, C, 4, M, N, (long long)N * 4, 32, false));
    if (plan.pair) {
        // (a K-major operand may have gone the padded-copy route; an MN-major one is 3-d by wants_pair's rule)
        if ((a.mn_major && !a.map3d) || (b.mn_major && !b.map3d)) return fail(BMB_E_UNSUPPORTED, "gemm_tc: operand layout not served by the pair kernel");
        BMB_TRY((launch_pair<256>(grid, st, mapA, mapB, mapC, c_mode, M, N, kblocks, kper, amn, bmn, alpha, beta, C, vec_ok, dp_tiles, g_sk, bias,
                                  round_c, status_dev)));
        count_launch();
        BMB_LAUNCH_CHECK();
        return BMB_OK;
    }
#define BMB_TC_ARGS grid, st, mapA, mapB, mapC, c_mode, batch, M, N, kblocks, kper, amn, bmn, alpha, beta, C, vec_ok, dp_tiles, g_sk, bias, round_c, status_dev, aux, round_aux
    if (aux) {
        // the second output is compiled into instances of its own (the plain kernels stay as lean as they were:
        // the activation's code in every epilogue cost all products 13 %), three with the accurate tanh and three
        // with the approximate one (BMB_GEMM_AUX_FAST)
        if (flags & BMB_GEMM_AUX_FAST) {
            if (bn == 256) BMB_TRY((launch_tc<0, 256, 1, 2>(BMB_TC_ARGS)));
            else if (bn == 192) BMB_TRY((launch_tc<0, 192, 1, 2>(BMB_TC_ARGS)));
            else BMB_TRY((launch_tc<0, 128, 1, 2>(BMB_TC_ARGS)));
        } else if (bn == 256) BMB_TRY((launch_tc<0, 256, 1, 1>(BMB_TC_ARGS)));
        else if (bn == 192) BMB_TRY((launch_tc<0, 192, 1, 1>(BMB_TC_ARGS)));
        else BMB_TRY((launch_tc<0, 128, 1, 1>(BMB_TC_ARGS)));
    } else if (bf16) {
        if (plan.mh == 2) BMB_TRY((launch_tc<1, 256, 2>(BMB_TC_ARGS)));
        else if (bn == 256) BMB_TRY((launch_tc<1, 256, 1>(BMB_TC_ARGS)));
        else if (bn == 192) BMB_TRY((launch_tc<1, 192, 1>(BMB_TC_ARGS)));
        else if (bn == 128) BMB_TRY((launch_tc<1, 128, 1>(BMB_TC_ARGS)));
        else BMB_TRY((launch_tc<1, 64, 1>(BMB_TC_ARGS)));
    } else {
        if (plan.mh == 2) BMB_TRY((launch_tc<0, 256, 2>(BMB_TC_ARGS)));
        else if (bn == 256) BMB_TRY((launch_tc<0, 256, 1>(BMB_TC_ARGS)));
        else if (bn == 192) BMB_TRY((launch_tc<0, 192, 1>(BMB_TC_ARGS)));
        else if (bn == 128) BMB_TRY((launch_tc<0, 128, 1>(BMB_TC_ARGS)));
        else BMB_TRY((launch_tc<0, 64, 1>(BMB_TC_ARGS)));
    }
#undef BMB_TC_ARGS
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb

// Host-side replay of the tile schedule a tensor-core GEMM of this shape would use on `ctas` SMs:
// returns BMB_OK when the work items of all CTAs cover every (tile, K slice) exactly once, whole
// tiles only where no tile is shared.  Runs no kernel; the CPU tests sweep shapes through it.
extern "C" int bmb_gemm_schedule_check(int math, int flags, int batch, int M, int N, int K, int ctas, int *bm_out, int *bn_out,
                                       int *dp_tiles_out, int *grid_out) {
    using namespace bmb;
    if (M < 1 || N < 1 || K < 1 || batch < 1 || ctas < 1) return fail(BMB_E_ARG, "schedule_check: bad argument");
    Plan p;
    BMB_TRY(plan_gemm(&p, math == BMB_MATH_BF16, flags, batch, M, N, K, ctas));
    // the pair kernel's plan is replayed only when the call asks for it by flag (no device is consulted here):
    // `ctas` then counts CTA pairs
    if ((flags & BMB_GEMM_PAIR) && wants_pair(math == BMB_MATH_BF16, flags, 0, 1, batch, M, N)) plan_pair(&p, flags, M, N, ctas);
    if (bm_out) *bm_out = p.mh * BM;
    if (bn_out) *bn_out = p.bn;
    if (dp_tiles_out) *dp_tiles_out = p.dp_tiles;
    if (grid_out) *grid_out = p.grid;
    if (p.grid < 1 || p.grid > ctas) return fail(BMB_E_LIMIT, "schedule_check: grid %d", p.grid);
    if ((long long)p.tiles * p.kblocks > (1LL << 28)) return fail(BMB_E_LIMIT, "schedule_check: problem too large to replay");
    std::vector<unsigned char> seen((size_t)p.tiles * p.kblocks, 0);
    for (int c = 0; c < p.grid; ++c) {
        WorkIter wi;
        wi.init(c, p.grid, p.dp_tiles, p.sk_tiles, p.kblocks, p.g_sk);
        int tile, kb0, kb1;
        while (wi.next(tile, kb0, kb1)) {
            if (tile < 0 || tile >= p.tiles || kb0 < 0 || kb1 > p.kblocks || kb0 >= kb1)
                return fail(BMB_E_LIMIT, "schedule_check: CTA %d got item (%d, %d, %d)", c, tile, kb0, kb1);
            if (tile < p.dp_tiles && !(kb0 == 0 && kb1 == p.kblocks))
                return fail(BMB_E_LIMIT, "schedule_check: whole tile %d cut", tile);
            for (int k = kb0; k < kb1; ++k)
                if (seen[(size_t)tile * p.kblocks + k]++) return fail(BMB_E_LIMIT, "schedule_check: tile %d slice %d twice", tile, k);
        }
    }
    for (size_t i = 0; i < seen.size(); ++i)
        if (!seen[i]) return fail(BMB_E_LIMIT, "schedule_check: tile %zu slice %zu never computed", i / p.kblocks, i % p.kblocks);
    return BMB_OK;
}

#ifdef BMB_GEMM_TRACE
// Developer entry point: copy out (and clear) the per-CTA timeline of the last tensor-core GEMM launch.
extern "C" int bmb_dbg_gemm_trace(unsigned long long *host_256x16) {
    cudaError_t e = cudaMemcpyFromSymbol(host_256x16, bmb::g_gemm_trace, sizeof(unsigned long long) * 4096);
    if (e != cudaSuccess) return (int)e;
    static unsigned long long zeros[4096];
    return (int)cudaMemcpyToSymbol(bmb::g_gemm_trace, zeros, sizeof(zeros));
}
#endif
