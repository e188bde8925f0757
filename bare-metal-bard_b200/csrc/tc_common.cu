// Host-side helpers of the tcgen05 kernels: the driver's tensor-map encoder
// (looked up at run time, so the library does not link against libcuda), and
// the per-device status word the kernels raise when a bounded wait runs out.
#include "tc_common.cuh"
#include <mutex>

namespace bmb {
namespace tc {

static EncodeFn g_encode = nullptr;
static std::once_flag g_encode_once;

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

int make_map_2d(CUtensorMap *map, const void *ptr, int esize, long long rows, long long cols, long long pitch_bytes,
                int box_rows, bool atom32) {
    EncodeFn enc = encode_fn();
    if (!enc) return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for %lld x %lld, pitch %lld", (int)r, rows, cols,
                    pitch_bytes);
    return BMB_OK;
}

// An MN-major fp32 operand (rows_k rows of K, cols_x contiguous M/N values, cols_x % 32 == 0) seen as
// [cols_x / 32 chunks][rows_k][32 floats]: one copy of a 32 x 32 x box_chunks box lands in shared memory
// as box_chunks consecutive chunks of 32 K rows x 128 bytes, the layout the MN-major descriptors read.
int make_map_mn3d(CUtensorMap *map, const void *ptr, long long rows_k, long long cols_x, long long pitch_bytes, int box_chunks) {
    EncodeFn enc = encode_fn();
    if (!enc) return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {32, (cuuint64_t)rows_k, (cuuint64_t)(cols_x / 32)};
    const cuuint64_t strides[2] = {(cuuint64_t)pitch_bytes, 128};
    const cuuint32_t box[3] = {32, 32, (cuuint32_t)box_chunks};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled (3-d) failed (%d) for %lld x %lld, pitch %lld", (int)r, rows_k, cols_x,
                    pitch_bytes);
    return BMB_OK;
}

// An fp32 array [batches][rows][cols] (cols % 32 == 0, contiguous) for tile stores of box_rows x 32 columns with the
// 128-byte swizzle: rows past the end of a batch are clipped instead of running into the next batch.
int make_map_rows3d(CUtensorMap *map, const void *ptr, long long cols, long long rows, long long batches, int box_rows) {
    EncodeFn enc = encode_fn();
    if (!enc) return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t strides[2] = {(cuuint64_t)(cols * 4), (cuuint64_t)(rows * cols * 4)};
    const cuuint32_t box[3] = {32, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(BMB_E_CUDA, "cuTensorMapEncodeTiled (3-d rows) failed (%d) for %lld x %lld x %lld", (int)r, batches, rows, cols);
    return BMB_OK;
}

struct Status { int *dev = nullptr; int *host = nullptr; };
static Status g_status[64];
static std::mutex g_status_mu;

int status_word(int **dev_ptr, volatile int **host_ptr) {
    const int d = current_device();
    if (d < 0 || d >= 64) return fail(BMB_E_ARG, "device index %d out of range", d);
    std::lock_guard<std::mutex> lk(g_status_mu);
    Status &s = g_status[d];
    if (!s.host) {
        BMB_CUDA(cudaHostAlloc((void **)&s.host, sizeof(int), cudaHostAllocMapped));
        *s.host = 0;
        BMB_CUDA(cudaHostGetDevicePointer((void **)&s.dev, s.host, 0));
    }
    *dev_ptr = s.dev;
    *host_ptr = s.host;
    return BMB_OK;
}

}  // namespace tc
}  // namespace bmb

// ---- the status word through the C ABI, and a self-test of the give-up path --------------------
namespace bmb {
namespace {
// One CTA waits, with the caller's cycle limit, on an mbarrier that nothing ever arrives on: the
// same bounded wait the GEMM and attention kernels use.  The wait runs out, the role raises the
// CTA's give-up flag and the kernel reports through the status word and returns by itself -- no
// trap, no fault, nothing left in flight (it issues no copy and holds no tensor memory).
__global__ void wait_expiry_selftest_k(long long limit_cycles, int *status, long long *waited_out) {
    __shared__ uint64_t bar;
    __shared__ int giveup;
    if (threadIdx.x == 0) {
        giveup = 0;
        tc::mbar_init(tc::smem_u32(&bar), 1);
        tc::mbar_init_fence();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        const bool ok = tc::mbar_wait_limit(tc::smem_u32(&bar), 0, &giveup, limit_cycles);
        if (waited_out) *waited_out = clock64() - t0;
        if (!ok) {
            *reinterpret_cast<volatile int *>(status) = 9;
            __threadfence_system();
        }
    }
}
}  // namespace
}  // namespace bmb

extern "C" {

int bmb_kernel_status(int *status_out) {
    int *dev = nullptr;
    volatile int *host = nullptr;
    BMB_TRY(bmb::tc::status_word(&dev, &host));
    if (status_out) *status_out = *host;
    return BMB_OK;
}

int bmb_kernel_status_clear(void) {
    int *dev = nullptr;
    volatile int *host = nullptr;
    BMB_TRY(bmb::tc::status_word(&dev, &host));
    BMB_CUDA(cudaDeviceSynchronize());        // no kernel that could still raise it is running
    *host = 0;
    return BMB_OK;
}

int bmb_selftest_wait_expiry(long long limit_cycles, long long *host_waited_cycles) {
    if (limit_cycles < 1 || limit_cycles > 100000000LL)
        return bmb::fail(BMB_E_ARG, "selftest_wait_expiry: limit must be 1..1e8 cycles");
    int *dev = nullptr;
    volatile int *host = nullptr;
    BMB_TRY(bmb::tc::status_word(&dev, &host));
    long long *d_waited = nullptr;
    BMB_CUDA(cudaMalloc(&d_waited, sizeof(long long)));
    bmb::wait_expiry_selftest_k<<<1, 32, 0, bmb::cur_stream()>>>(limit_cycles, dev, d_waited);
    bmb::count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(bmb::cur_stream());
    long long waited = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&waited, d_waited, sizeof(long long), cudaMemcpyDeviceToHost);
    cudaFree(d_waited);
    if (e != cudaSuccess) return bmb::fail(BMB_E_CUDA, "selftest_wait_expiry -> %s", cudaGetErrorString(e));
    if (host_waited_cycles) *host_waited_cycles = waited;
    return BMB_OK;
}

}  // extern "C"
