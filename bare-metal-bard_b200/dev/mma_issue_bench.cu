// Developer micro-benchmark: how fast one thread can issue back-to-back tcgen05.mma kind::tf32
// (M = 128, K = 8 per instruction) for N = 64 / 128 / 256 and three operand sources: both operands
// K-major in shared memory; B MN-major; A in tensor memory with B MN-major.  One CTA on one SM,
// cycles per instruction from clock64.  Not part of libbmb.so.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Ibare-metal-bard_b200/csrc -Iinclude \
//        -o mma_issue_bench bare-metal-bard_b200/dev/mma_issue_bench.cu \
//        bare-metal-bard_b200/csrc/tc_common.cu bare-metal-bard_b200/csrc/runtime.cu && ./mma_issue_bench
#include "tc_common.cuh"
#include <cstdio>
using namespace bmb::tc;
__global__ void __launch_bounds__(128, 1) k(int N, int mode, int reps, long long *out) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    __shared__ uint64_t bar; __shared__ uint32_t slot;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); mbar_init_fence(); }
    for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<float *>(smem_raw)[i] = 0.001f * (i & 1023);
    __syncthreads();
    fence_proxy_async();
    if (threadIdx.x < 32) tmem_alloc(smem_u32(&slot), 512);
    fence_before(); __syncthreads(); fence_after();
    const uint32_t tm = slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = make_idesc(2, 0, mode == 1 ? 1 : 0, N, 128);
        const uint32_t sa = base, sb = base + 65536;
        long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t half = ks >> 2, off = (ks & 3) * 32;
                const uint64_t da = smem_desc_kmajor(sa + half * 16384 + off);
                if (mode == 0) mma_tf32(tm + (r & 1) * 256, da, smem_desc_kmajor(sb + half * (N * 128) + off), idesc, ks ? 1u : 0u);
                else if (mode == 1) mma_tf32(tm + (r & 1) * 256, da, smem_desc_mnmajor32(sb + ks * 1024, 8192), idesc, ks ? 1u : 0u);
                else mma_tf32_ts(tm + (r & 1) * 256, tm + 128 + ks * 8, smem_desc_mnmajor32(sb + ks * 1024, 8192), make_idesc(2, 0, 1, N, 128), ks ? 1u : 0u);
            }
        }
        long long t1 = clock64();
        commit(smem_u32(&bar));
        volatile int gv = 0;
        mbar_wait(smem_u32(&bar), 0, &gv);
        long long t2 = clock64();
        out[0] = t1 - t0; out[1] = t2 - t0;
    }
    fence_before(); __syncthreads();
    if (threadIdx.x < 32) { fence_after(); tmem_dealloc(tm, 512); }
}
int main() {
    long long *d; cudaMalloc(&d, 16); long long h[2];
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const int reps = 200;
    for (int mode = 0; mode < 3; ++mode)
        for (int N : {64, 128, 256}) {
            for (int w = 0; w < 2; ++w) { k<<<1, 128, 200 * 1024>>>(N, mode, reps, d); cudaDeviceSynchronize(); }
            cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
            printf("mode %d (0 B K-major, 1 B MN-major, 2 A from TMEM + B MN-major) N=%3d: issue %.1f cyc/mma, complete %.1f cyc/mma (at 2048 MAC/clk: %.1f)  err=%s\n",
                   mode, N, (double)h[0] / (reps * 8), (double)h[1] / (reps * 8), 128.0 * N * 8 / 2048.0, cudaGetErrorString(cudaGetLastError()));
        }
    return 0;
}
