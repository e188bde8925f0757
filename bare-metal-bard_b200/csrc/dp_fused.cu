// Data-parallel gradient exchange fused with the optimiser, one process per GPU, over peer memory.
//
// The reference sums the whole gradient buffer on every rank (ddp_allreduce, src/ddp.cu:168-260) and
// then every rank runs the same AdamW step over all parameters (src/train_gpt.cu:438-451).  Here rank r
// owns slice r of the flat parameter space:
//   1. reduce: it sums slice r of every rank's gradient buffer by reading the peers' memory over
//      NVLink (fixed rank order, so every rank that ever sums a slice would get the same bits), keeps
//      the sum in its own buffer and leaves the slice's sum of squares on the device;
//   2. the ranks add their sums of squares (one 8-byte all-reduce, which is also the barrier between
//      the phases);
//   3. update + broadcast: it runs AdamW (with the clip factor of src/train_gpt.cu:442-448) on its
//      slice only and stores the new parameters straight into every rank's buffers (each rank rounds
//      its own TF32 shadow copy from them afterwards: a local pass is cheaper than a second trip
//      over NVLink).
// Per rank that is (n-1)/n of the buffer read and (n-1)/n written over NVLink, as in a ring
// all-reduce, but the optimiser touches 1/n of the parameters and no separate norm pass is needed.
// The peers' buffers are reached through CUDA IPC handles exchanged by the launcher.  The kernels only
// issue plain loads and stores to peer memory; ordering between ranks comes from collectives on the
// same stream (a rank's kernel cannot start before every rank has finished the phase before it), so
// no kernel spins on another GPU.
#include "common.cuh"
#include <cmath>

namespace bmb {
namespace {

constexpr int MAX_RANKS = 8;
struct PeerBufs {
    const float *grads[MAX_RANKS];
    float *params[MAX_RANKS];
};

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }

// out[off + i] = sum over ranks (in rank order) of grads_r[off + i], i < len (len % 4 == 0);
// partial[blockIdx.x] = this block's share of sum(out^2).
__global__ void __launch_bounds__(256)
dp_reduce_slice_k(PeerBufs pb, int nranks, float *__restrict__ out, size_t off, size_t len, float *__restrict__ partial) {
    __shared__ float red[32];
    float acc2 = 0.0f;
    const size_t n4 = len >> 2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const size_t e = off + i * 4;
        float4 v[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
            if (r < nranks) v[r] = ld4(pb.grads[r] + e);          // all loads in flight before the adds
        float4 s = v[0];
#pragma unroll
        for (int r = 1; r < MAX_RANKS; ++r)
            if (r < nranks) { s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w; }
        st4(out + e, s);
        acc2 += (s.x * s.x + s.y * s.y) + (s.z * s.z + s.w * s.w);
    }
    const float t = block_reduce<false>(acc2, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

__global__ void __launch_bounds__(256) dp_sumsq_finish_k(const float *__restrict__ partial, int nparts, double *__restrict__ out) {
    __shared__ double red[8];
    double s = 0.0;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += (double)partial[i];
    s = warp_sum_d(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < 8; ++i) t += red[i];
        *out = t;
    }
}

__device__ __forceinline__ float adamw_one(float p, float g, float &m, float &v, float lr, float b1, float b2, float eps,
                                           float wd, float bc1, float bc2) {
    const float mi = b1 * m + (1.0f - b1) * g;
    const float vi = b2 * v + (1.0f - b2) * g * g;
    m = mi; v = vi;
    const float mhat = mi / bc1, vhat = vi / bc2;
    return p - lr * (mhat / (sqrtf(vhat) + eps) + wd * p);
}

// AdamW (src/nn.cu:240-254) on [off, off + len) of this rank's buffers, gradient = the reduced slice
// scaled by the clip rule evaluated from the global squared norm *d_sumsq (sum over all ranks'
// slices); the new parameters go to every rank.
__global__ void __launch_bounds__(256)
dp_adamw_broadcast_k(PeerBufs pb, int nranks, int rank, const float *__restrict__ grads, float *__restrict__ m,
                     float *__restrict__ v, size_t off, size_t len, float lr, float b1, float b2, float eps, float wd,
                     float bc1, float bc2, const double *__restrict__ d_sumsq, float clip, float div) {
    const float gn = (float)sqrt(*d_sumsq) / div;
    const float gscale = ((gn > clip) ? clip / gn : 1.0f) / div;
    const float *params = pb.params[rank];
    const size_t n4 = len >> 2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const size_t e = off + i * 4;
        float4 p = ld4(params + e), mm = ld4(m + e), vv = ld4(v + e);
        const float4 g = ld4(grads + e);
        p.x = adamw_one(p.x, g.x * gscale, mm.x, vv.x, lr, b1, b2, eps, wd, bc1, bc2);
        p.y = adamw_one(p.y, g.y * gscale, mm.y, vv.y, lr, b1, b2, eps, wd, bc1, bc2);
        p.z = adamw_one(p.z, g.z * gscale, mm.z, vv.z, lr, b1, b2, eps, wd, bc1, bc2);
        p.w = adamw_one(p.w, g.w * gscale, mm.w, vv.w, lr, b1, b2, eps, wd, bc1, bc2);
        st4(m + e, mm);
        st4(v + e, vv);
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
            if (r < nranks) st4(pb.params[r] + e, p);
    }
}

}  // namespace

// State of the fused exchange for one trainer (rank).
struct DpFused {
    int rank = 0, nranks = 1;
    PeerBufs pb{};
    void *opened[3 * MAX_RANKS] = {nullptr};
    int nopened = 0;
    size_t slice = 0;       // floats per rank (multiple of 4; the last rank's slice ends at n)
};

int dp_fused_export(const float *grads, const float *params, const float *shadow, void *out192) {
    cudaIpcMemHandle_t h[3];
    memset(h, 0, sizeof(h));
    BMB_CUDA(cudaIpcGetMemHandle(&h[0], const_cast<float *>(grads)));
    BMB_CUDA(cudaIpcGetMemHandle(&h[1], const_cast<float *>(params)));
    (void)shadow;          // the third handle slot of the record stays empty: shadows are rounded locally
    memcpy(out192, h, sizeof(h));
    return BMB_OK;
}

int dp_fused_create(DpFused **out, int rank, int nranks, size_t n, float *grads, float *params, float * /*shadow*/,
                    const void *all_handles) {
    if (nranks < 2 || nranks > MAX_RANKS || rank < 0 || rank >= nranks)
        return fail(BMB_E_ARG, "fused data-parallel step: rank %d of %d (2..%d ranks)", rank, nranks, MAX_RANKS);
    if (n % 4) return fail(BMB_E_ARG, "fused data-parallel step: parameter count must be a multiple of 4");
    DpFused *d = new DpFused();
    d->rank = rank; d->nranks = nranks;
    d->slice = ((n / 4 + nranks - 1) / nranks) * 4;
    const cudaIpcMemHandle_t *h = static_cast<const cudaIpcMemHandle_t *>(all_handles);
    for (int r = 0; r < nranks; ++r) {
        if (r == rank) {
            d->pb.grads[r] = grads; d->pb.params[r] = params;
            continue;
        }
        void *pg = nullptr, *pp = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&pg, h[3 * r + 0], cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) { d->opened[d->nopened++] = pg; e = cudaIpcOpenMemHandle(&pp, h[3 * r + 1], cudaIpcMemLazyEnablePeerAccess); }
        if (e == cudaSuccess) d->opened[d->nopened++] = pp;
        if (e != cudaSuccess) {
            const int rc = fail(BMB_E_CUDA, "cudaIpcOpenMemHandle for rank %d -> %s", r, cudaGetErrorString(e));
            for (int i = 0; i < d->nopened; ++i) cudaIpcCloseMemHandle(d->opened[i]);
            delete d;
            cudaGetLastError();
            return rc;
        }
        d->pb.grads[r] = static_cast<const float *>(pg);
        d->pb.params[r] = static_cast<float *>(pp);
    }
    *out = d;
    return BMB_OK;
}

void dp_fused_destroy(DpFused *d) {
    if (!d) return;
    for (int i = 0; i < d->nopened; ++i) cudaIpcCloseMemHandle(d->opened[i]);
    delete d;
}

// Phase 1 on `st`: reduce this rank's slice and leave its sum of squares in *d_sumsq_slice.
int dp_fused_reduce(DpFused *d, size_t n, float *grads, double *d_sumsq_slice, cudaStream_t st) {
    const size_t off = d->slice * d->rank;
    const size_t len = off >= n ? 0 : (n - off < d->slice ? n - off : d->slice);
    float *partial = (float *)device_scratch(SCR_MISC, 4096 * sizeof(float));
    if (!partial) return BMB_E_CUDA;
    const int blocks = 4 * sm_count();
    dp_reduce_slice_k<<<blocks, 256, 0, st>>>(d->pb, d->nranks, grads, off, len, partial);
    dp_sumsq_finish_k<<<1, 256, 0, st>>>(partial, blocks, d_sumsq_slice);
    count_launch(2);
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

// Phase 3 on `st`: *d_sumsq_total holds the squared norm of the whole summed gradient.
int dp_fused_update(DpFused *d, size_t n, const float *grads, float *m, float *v, float lr, float beta1, float beta2,
                    float eps, float wd, int step, const double *d_sumsq_total, float clip, cudaStream_t st) {
    const size_t off = d->slice * d->rank;
    const size_t len = off >= n ? 0 : (n - off < d->slice ? n - off : d->slice);
    const float bc1 = 1.0f - powf(beta1, (float)step), bc2 = 1.0f - powf(beta2, (float)step);
    dp_adamw_broadcast_k<<<4 * sm_count(), 256, 0, st>>>(d->pb, d->nranks, d->rank, grads, m, v, off, len, lr, beta1, beta2, eps,
                                                        wd, bc1, bc2, d_sumsq_total, clip, (float)d->nranks);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb
