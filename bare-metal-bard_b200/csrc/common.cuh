// Shared host/device helpers for libbmb: status plumbing, the per-thread
// stream, per-device scratch, and small device utilities.
#pragma once
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdarg>
#include <cstdint>
#include "../../include/bmb.h"

namespace bmb {

// ---- status -------------------------------------------------------------
int fail(int code, const char *fmt, ...);

#define BMB_CUDA(x)                                                           \
    do {                                                                      \
        cudaError_t e__ = (x);                                                \
        if (e__ != cudaSuccess)                                               \
            return ::bmb::fail(BMB_E_CUDA, "%s -> %s (%s:%d)", #x,            \
                               cudaGetErrorString(e__), __FILE__, __LINE__);  \
    } while (0)

// After a kernel launch: report a launch-configuration error, never sync.
#define BMB_LAUNCH_CHECK()                                                    \
    do {                                                                      \
        cudaError_t e__ = cudaGetLastError();                                 \
        if (e__ != cudaSuccess)                                               \
            return ::bmb::fail(BMB_E_CUDA, "launch -> %s (%s:%d)",            \
                               cudaGetErrorString(e__), __FILE__, __LINE__);  \
    } while (0)

#define BMB_TRY(x)                                                            \
    do {                                                                      \
        int s__ = (x);                                                        \
        if (s__ != BMB_OK) return s__;                                        \
    } while (0)

// ---- per-thread stream ----------------------------------------------------
cudaStream_t cur_stream();

// Per-thread switch read by the kernels that produce GEMM / attention operands
// (layernorm, GELU, bias add, cross-entropy backward, attention): when on, they
// store TF32-rounded values so that the tensor-core kernels can read them in
// place.  The training step turns it on in TF32 mode; the C ABI leaves it off.
bool emit_rounded();
void set_emit_rounded(bool on);

// ---- deferred column sums --------------------------------------------------
// The parameter-gradient sums of the backward kernels are two-stage: a kernel leaves G partial rows, a small
// launch adds them up in a fixed order.  While a collector is installed for the calling thread, those kernels take
// their partial rows from the collector's arena (instead of the shared per-device scratch, which the next call
// would overwrite) and only note the final sum as a job; one batched launch at the end of the backward pass then
// does all of them -- the same sums in the same order, a few dozen launches fewer.
struct ColumnAddJob {
    float *dst, *dst2, *dst3;     // as launch_column_add: columns [ncols_first, ..) go to dst2, from 2 * ncols_first on to dst3
    const float *partial;
    int ncols_first, G, ncols;
};
struct ColumnAddCollector {
    float *arena = nullptr;       // device memory for the partial rows of one backward pass
    size_t cap = 0, used = 0;     // floats
    ColumnAddJob *jobs = nullptr; // host array, filled while `record` is set (the job list is the same every pass)
    int max_jobs = 0, njobs = 0, max_cols = 0;
    bool record = false;
};
void set_column_add_collector(ColumnAddCollector *c);      // nullptr: sums are finished by their own launches again
int launch_column_add_jobs(const ColumnAddJob *jobs_dev, int njobs, int max_cols, cudaStream_t st);

// ---- data-parallel exchange: a list of ranges of a flat float buffer ------
// (offsets and lengths in floats, each a multiple of 4)
constexpr int DP_MAX_RANGES = 16;
struct DpRangeList {
    unsigned long long off[DP_MAX_RANGES], len[DP_MAX_RANGES];
    int n;
};

// ---- per-device scratch ---------------------------------------------------
// The reference keeps process-wide static device scratch (src/nn.cu:347, 362)
// that every rank thread shares regardless of device.  Here each device owns
// its own block, grown on demand and kept until process exit.
// Returns nullptr (and records an error) on failure.
enum ScratchSlot { SCR_REDUCE = 0, SCR_GEMM_A = 1, SCR_GEMM_B = 2, SCR_MISC = 3, SCR_SLOTS = 4 };
void *device_scratch(ScratchSlot slot, size_t bytes);
// Order the users of a scratch slot across streams of one device: acquire before the first launch that writes
// the slot, release after the last launch that reads it (both on the stream those launches go to).
int scratch_acquire(ScratchSlot slot, cudaStream_t st);
int scratch_release(ScratchSlot slot, cudaStream_t st);
// Counts the times any scratch block of the current device was (re)allocated.  A caller that keeps
// scratch addresses beyond one call (the trainer's captured graph) compares it before reusing them.
unsigned long long scratch_generation();
int current_device();
int sm_count();

// Launch counter (all kernels launched by this library in this process).
void count_launch(int n = 1);
long long launches_total();

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Internal GEMM dispatch shared by attention and the trainer: math is a
// BMB_MATH_* value, flags the BMB_GEMM_* bits, strides in elements.
int gemm_any(int math, int flags, int ta, int tb, int batch, int M, int N, int K, float alpha,
             const float *A, long long sA, const float *B, long long sB, float beta, float *C,
             long long sC, cudaStream_t st);
// Same with a bias row added to every output row (null = none).
int gemm_any_bias(int math, int flags, int ta, int tb, int batch, int M, int N, int K, float alpha,
                  const float *A, long long sA, const float *B, long long sB, float beta, float *C,
                  long long sC, const float *bias, cudaStream_t st, float *aux_gelu = nullptr);
// (aux_gelu: a second output of the same shape, GELU of the result -- in the product's epilogue where the
//  tensor-core kernel can, by a pass of its own otherwise)

}  // namespace bmb

// ---- device helpers ---------------------------------------------------------
#ifdef __CUDACC__
namespace bmb {
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Block-wide sum / max with the result in every thread.  `red` is a shared
// array of at least 32 floats; two barriers per call, safe to call repeatedly
// with the same array.
template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float *red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    v = (lane < nw) ? red[lane] : (IS_MAX ? -3.402823466e38f : 0.0f);
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    return v;
}
// tanh-approximation GELU with the accurate tanhf (src/nn.cu:118-127).
__device__ __forceinline__ float gelu_tanh(float x) {
    const float s = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(s * (x + 0.044715f * x * x * x)));
}
// The same form with the hardware's approximate tanh (one special-function instruction; absolute error of tanh about
// 2^-11, i.e. of the order of a TF32 rounding of the result): for an activation that is rounded to TF32 anyway.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    const float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    const float hx = 0.5f * x;
    return fmaf(hx, t, hx);
}
// Round to nearest TF32 (ties away), result as an fp32 bit pattern whose low
// 13 mantissa bits are zero.
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
// The same rounding with two integer instructions instead of a conversion (which shares the
// special-function unit with exp): add half a TF32 ulp to the magnitude, clear the low 13 bits.
// For finite values and infinities the result equals cvt.rna.tf32.f32.
__device__ __forceinline__ float round_tf32_alu(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}
// For a value that only the tensor core will read: kind::tf32 ignores the low 13 bits of an operand,
// so adding half a TF32 ulp is all it takes to turn that truncation into rounding to nearest.
__device__ __forceinline__ float round_tf32_for_mma(float x) { return __uint_as_float(__float_as_uint(x) + 0x1000u); }
}  // namespace bmb
#endif
