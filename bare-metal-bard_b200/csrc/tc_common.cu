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
