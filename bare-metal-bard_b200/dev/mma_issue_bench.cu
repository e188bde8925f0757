// Developer micro-benchmark: how fast one thread can issue back-to-back tcgen05.mma kind::tf32
// (M = 128, K = 8 per instruction) for N = 64 / 128 / 256 and four operand sources:
//   0 both operands K-major in shared memory      1 A K-major, B MN-major
//   2 A in tensor memory, B MN-major              3 A in tensor memory, B K-major
// each written two ways: "plain" builds both descriptors from the shared-memory address inside the
// K loop and passes the accumulate flag as a value (a setp per instruction); "hoisted" builds the
// descriptors once per tile, adds a constant to the address field per K step and passes the flag as
// a literal.  One CTA on one SM, cycles per instruction from clock64.  Not part of libbmb.so.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Ibare-metal-bard_b200/csrc -Iinclude \
//        -o mma_issue_bench bare-metal-bard_b200/dev/mma_issue_bench.cu \
//        bare-metal-bard_b200/csrc/tc_common.cu bare-metal-bard_b200/csrc/runtime.cu && ./mma_issue_bench
#include "tc_common.cuh"
#include <cstdio>
using namespace bmb::tc;

// noise: what the other eight warps of the CTA do while warp 9 issues: 0 nothing, 1 a loop of fused
// multiply-adds and exp2, 2 loads and stores of tensor memory, 3 both (alternating).
template <int MODE, bool HOIST>
__global__ void __launch_bounds__(320, 1) k(int N, int reps, int noise, long long *out, float *sink) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    __shared__ uint64_t bar; __shared__ uint32_t slot;
    __shared__ volatile int stop;
    if (threadIdx.x == 0) { stop = 0; mbar_init(smem_u32(&bar), 1); mbar_init_fence(); }
    for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<float *>(smem_raw)[i] = 0.001f * (i & 1023);
    __syncthreads();
    fence_proxy_async();
    if (threadIdx.x < 32) tmem_alloc(smem_u32(&slot), 512);
    fence_before(); __syncthreads(); fence_after();
    const uint32_t tm = slot;
    if (threadIdx.x < 256 && noise) {
        // bounded: ends when the issuer raises `stop` or after a fixed number of rounds
        float v[32], acc = (float)threadIdx.x;
        const uint32_t ta = tm + 384 + ((uint32_t)((threadIdx.x >> 5) & 3) * 32u << 16) + (uint32_t)((threadIdx.x >> 7) * 32);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.001f * i;
        for (int round = 0; round < 200000 && !stop; ++round) {
            if (noise & 1) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = exp2f(fmaf(v[i], 0.5f, -acc)) + v[i];
            }
            if (noise & 2) {
                tmem_st32_nowait(ta, v);
                tmem_wait_st();
                tmem_ld32(ta, v);
            }
            acc += v[round & 31];
        }
        sink[threadIdx.x] = acc;
    }
    if (threadIdx.x == 288) {
        constexpr bool B_MN = (MODE == 1 || MODE == 2), A_TMEM = (MODE >= 2);
        const uint32_t idesc = make_idesc(2, 0, B_MN ? 1 : 0, N, 128);
        const uint32_t sa = base, sb = base + 65536;
        const long long t0 = clock64();
        if (HOIST) {
            const uint64_t da0 = smem_desc_kmajor(sa);
            const uint64_t db0 = B_MN ? smem_desc_mnmajor32(sb, 8192) : smem_desc_kmajor(sb);
            const uint64_t bhalf = (uint64_t)((N * 128) >> 4);
            for (int r = 0; r < reps; ++r) {
                const uint32_t d = tm + (r & 1) * 256;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint64_t da = da0 + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
                    const uint64_t db = B_MN ? db0 + (uint64_t)((ks * 1024) >> 4)
                                             : db0 + (uint64_t)(ks >> 2) * bhalf + (uint64_t)(((ks & 3) * 32) >> 4);
                    if (A_TMEM) {
                        if (ks == 0) mma_tf32_ts(d, tm + 128 + ks * 8, db, idesc, 0u);
                        else mma_tf32_ts(d, tm + 128 + ks * 8, db, idesc, 1u);
                    } else {
                        if (ks == 0) mma_tf32(d, da, db, idesc, 0u);
                        else mma_tf32(d, da, db, idesc, 1u);
                    }
                }
            }
        } else {
            for (int r = 0; r < reps; ++r) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                    const uint64_t da = smem_desc_kmajor(sa + half * 16384 + off);
                    const uint64_t db = B_MN ? smem_desc_mnmajor32(sb + ks * 1024, 8192) : smem_desc_kmajor(sb + half * (N * 128) + off);
                    if (A_TMEM) mma_tf32_ts(tm + (r & 1) * 256, tm + 128 + ks * 8, db, idesc, (r | ks) ? 1u : 0u);
                    else mma_tf32(tm + (r & 1) * 256, da, db, idesc, (r | ks) ? 1u : 0u);
                }
            }
        }
        const long long t1 = clock64();
        commit(smem_u32(&bar));
        volatile int gv = 0;
        mbar_wait(smem_u32(&bar), 0, &gv);
        const long long t2 = clock64();
        out[0] = t1 - t0; out[1] = t2 - t0;
        stop = 1;
    }
    fence_before(); __syncthreads();
    if (threadIdx.x < 32) { fence_after(); tmem_dealloc(tm, 512); }
}

template <int MODE, bool HOIST>
static void run(long long *d, float *sink, int noise) {
    static const char *what[4] = {"A K-major, B K-major", "A K-major, B MN-major", "A in TMEM, B MN-major", "A in TMEM, B K-major"};
    long long h[2];
    cudaFuncSetAttribute(k<MODE, HOIST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const int reps = 2000;
    for (int N : {64, 128, 256}) {
        for (int w = 0; w < 3; ++w) { k<MODE, HOIST><<<1, 320, 200 * 1024>>>(N, reps, noise, d, sink); cudaDeviceSynchronize(); }
        cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
        printf("%-22s %-7s noise %d N=%3d: issue %6.1f cyc/mma, complete %6.1f cyc/mma (tensor pipe at 2048 MAC/clk: %5.1f)  err=%s\n", what[MODE],
               HOIST ? "hoisted" : "plain", noise, N, (double)h[0] / (reps * 8), (double)h[1] / (reps * 8), 128.0 * N * 8 / 2048.0,
               cudaGetErrorString(cudaGetLastError()));
    }
}
int main() {
    long long *d; cudaMalloc(&d, 16);
    float *sink; cudaMalloc(&sink, 4096);
    for (int noise = 0; noise < 4; ++noise) {
        run<0, false>(d, sink, noise); run<0, true>(d, sink, noise);
        run<2, false>(d, sink, noise); run<2, true>(d, sink, noise);
    }
    run<1, false>(d, sink, 0); run<3, false>(d, sink, 0);
    return 0;
}
