// Data-parallel gradient exchange fused with the optimiser, one process per GPU, over peer memory.
//
// The reference sums the whole gradient buffer on every rank (ddp_allreduce, src/ddp.cu:168-260) and
// then every rank runs the same AdamW step over all parameters (src/train_gpt.cu:438-451).  Here the flat
// parameter space is described by lists of ranges (a tensor, or the layers l0..l1 of a stacked tensor), and rank
// r owns the r-th of n equal pieces of every range -- so that any group of ranges (the tensors of some layers)
// can be exchanged as soon as its gradients are final, with the work spread over all ranks.  For a list:
//   1. reduce: rank r sums its pieces of every rank's gradient buffer by reading the peers' memory over
//      NVLink (fixed rank order, so every rank that ever sums a piece would get the same bits), keeps
//      the sum in its own buffer and leaves the pieces' sum of squares on the device;
//   2. the ranks add their sums of squares (one 8-byte all-reduce, which is also the barrier between
//      the phases);
//   3. update + broadcast: it runs AdamW (with the clip factor of src/train_gpt.cu:442-448) on its
//      pieces only and stores the new parameters straight into every rank's buffers (each rank rounds
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
#include <mutex>

namespace bmb {
namespace {

constexpr int MAX_RANKS = 8;
constexpr int DP_SLOTS = 4;
struct PeerBufs {
    const float *grads[MAX_RANKS];
    float *params[MAX_RANKS];
};

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }

// The piece of rank `rank` in a range of len4 float4s: [lo, hi).
__device__ __forceinline__ void my_piece(size_t len4, int rank, int nranks, size_t &lo, size_t &hi) {
    const size_t per = (len4 + nranks - 1) / nranks;
    lo = per * rank < len4 ? per * rank : len4;
    hi = lo + per < len4 ? lo + per : len4;
}

// For every range of the list, over this rank's piece of it: out[e] = sum over ranks (in rank order) of
// grads_r[e]; partial[blockIdx.x] = this block's share of sum(out^2).
// NR = 2, 4 or 8 bounds the rank count; a thread keeps NR * U = 8 sixteen-byte loads in flight, so that one block
// per SM (the grid used while the main stream's kernels own the SMs) still covers the NVLink round trip.
template <int NR, int U>
__global__ void __launch_bounds__(256)
dp_reduce_ranges_k(PeerBufs pb, int nranks, int rank, float *__restrict__ out, DpRangeList rl, float *__restrict__ partial) {
    __shared__ float red[32];
    float acc2 = 0.0f;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (int q = 0; q < rl.n; ++q) {
        size_t lo, hi;
        my_piece(rl.len[q] >> 2, rank, nranks, lo, hi);
        for (size_t i0 = lo + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i0 < hi; i0 += stride * U) {
            float4 v[U][NR];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t i = i0 + (size_t)u * stride;
#pragma unroll
                for (int r = 0; r < NR; ++r)
                    if (r < nranks && i < hi) v[u][r] = ld4(pb.grads[r] + rl.off[q] + i * 4);   // all loads in flight before the adds
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t i = i0 + (size_t)u * stride;
                if (i >= hi) continue;
                float4 s = v[u][0];
#pragma unroll
                for (int r = 1; r < NR; ++r)
                    if (r < nranks) { s.x += v[u][r].x; s.y += v[u][r].y; s.z += v[u][r].z; s.w += v[u][r].w; }
                st4(out + rl.off[q] + i * 4, s);
                acc2 += (s.x * s.x + s.y * s.y) + (s.z * s.z + s.w * s.w);
            }
        }
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

// AdamW (src/nn.cu:240-254) on this rank's pieces of the listed ranges, gradient = the reduced piece
// scaled by the clip rule evaluated from the global squared norm *d_sumsq (sum over all ranks'
// pieces of all ranges); the new parameters go to every rank.
__global__ void __launch_bounds__(256)
dp_adamw_broadcast_ranges_k(PeerBufs pb, int nranks, int rank, const float *__restrict__ grads, float *__restrict__ m,
                            float *__restrict__ v, DpRangeList rl, float lr, float b1, float b2, float eps, float wd,
                            float bc1, float bc2, const double *__restrict__ d_sumsq, float clip, float div) {
    const float gn = (float)sqrt(*d_sumsq) / div;
    const float gscale = ((gn > clip) ? clip / gn : 1.0f) / div;
    const float *params = pb.params[rank];
    for (int q = 0; q < rl.n; ++q) {
        size_t lo, hi;
        my_piece(rl.len[q] >> 2, rank, nranks, lo, hi);
        for (size_t i = lo + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
            const size_t e = rl.off[q] + i * 4;
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
}

// shadow[e] = params[e] rounded to TF32 over the whole of every listed range (local: each rank rounds what arrived).
__global__ void __launch_bounds__(256)
dp_round_ranges_k(DpRangeList rl, float *__restrict__ shadow, const float *__restrict__ params) {
    constexpr int U = 4;                                    // loads in flight per thread
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (int q = 0; q < rl.n; ++q) {
        const size_t n4 = rl.len[q] >> 2;
        for (size_t i0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i0 < n4; i0 += stride * U) {
            float4 p[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t i = i0 + (size_t)u * stride;
                if (i < n4) p[u] = ld4(params + rl.off[q] + i * 4);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t i = i0 + (size_t)u * stride;
                if (i < n4) st4(shadow + rl.off[q] + i * 4, make_float4(round_tf32(p[u].x), round_tf32(p[u].y), round_tf32(p[u].z), round_tf32(p[u].w)));
            }
        }
    }
}

}  // namespace

// State of the fused exchange for one trainer (rank).
struct DpFused {
    int rank = 0, nranks = 1;
    PeerBufs pb{};
    void *opened[3 * MAX_RANKS] = {nullptr};
    int nopened = 0;
    float *partial = nullptr;   // per-block sums of squares, DP_SLOTS reduce launches per step side by side
    int blocks = 0;             // largest grid of the exchange kernels (a slot of the partials holds this many)
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
    d->blocks = 4 * sm_count();
    if (cudaMalloc(&d->partial, (size_t)DP_SLOTS * d->blocks * sizeof(float)) != cudaSuccess) {
        delete d;
        cudaGetLastError();
        return fail(BMB_E_CUDA, "fused data-parallel step: no memory for the norm partials");
    }
    cudaMemset(d->partial, 0, (size_t)DP_SLOTS * d->blocks * sizeof(float));     // slots a trainer never uses stay zero
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
            cudaFree(d->partial);
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
    cudaFree(d->partial);
    delete d;
}

namespace {
int check_ranges(const DpRangeList &rl) {
    if (rl.n < 0 || rl.n > DP_MAX_RANGES) return fail(BMB_E_ARG, "fused data-parallel step: %d ranges (at most %d)", rl.n, DP_MAX_RANGES);
    for (int q = 0; q < rl.n; ++q)
        if ((rl.off[q] | rl.len[q]) & 3) return fail(BMB_E_ARG, "fused data-parallel step: range %d is not a multiple of 4 floats", q);
    return BMB_OK;
}
}  // namespace

// Phase 1 on `st`: reduce this rank's pieces of the listed ranges; their sum of squares goes to slot `slot`
// (0 .. DP_SLOTS-1) of the partials.  Slots not used in a step must be cleared with dp_fused_clear_slot.
// `alone`: nothing else is running on the GPU (the main stream is waiting for this), so the kernel may fill it; otherwise
// one block per SM, which leaves room for a GPU-filling kernel of the main stream beside it (four blocks per SM of
// these kernels take the whole register file, and the two streams then only take turns).
int dp_fused_reduce_ranges(DpFused *d, const DpRangeList &rl, float *grads, int slot, bool alone, cudaStream_t st) {
    BMB_TRY(check_ranges(rl));
    if (slot < 0 || slot >= DP_SLOTS) return fail(BMB_E_ARG, "fused data-parallel step: slot %d", slot);
    const int grid = alone ? d->blocks : sm_count();
    float *partial = d->partial + (size_t)slot * d->blocks;
    if (grid < d->blocks) BMB_CUDA(cudaMemsetAsync(partial + grid, 0, (size_t)(d->blocks - grid) * sizeof(float), st));
    if (d->nranks <= 2) dp_reduce_ranges_k<2, 4><<<grid, 256, 0, st>>>(d->pb, d->nranks, d->rank, grads, rl, partial);
    else if (d->nranks <= 4) dp_reduce_ranges_k<4, 2><<<grid, 256, 0, st>>>(d->pb, d->nranks, d->rank, grads, rl, partial);
    else dp_reduce_ranges_k<8, 1><<<grid, 256, 0, st>>>(d->pb, d->nranks, d->rank, grads, rl, partial);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
int dp_fused_clear_slot(DpFused *d, int slot, cudaStream_t st) {
    if (slot < 0 || slot >= DP_SLOTS) return fail(BMB_E_ARG, "fused data-parallel step: slot %d", slot);
    BMB_CUDA(cudaMemsetAsync(d->partial + (size_t)slot * d->blocks, 0, d->blocks * sizeof(float), st));
    return BMB_OK;
}
// *d_sumsq_pieces = the sum of all slots (a fixed order: the same bits every run).
int dp_fused_sumsq(DpFused *d, double *d_sumsq_pieces, cudaStream_t st) {
    dp_sumsq_finish_k<<<1, 256, 0, st>>>(d->partial, DP_SLOTS * d->blocks, d_sumsq_pieces);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

// Phase 3 on `st`: *d_sumsq_total holds the squared norm of the whole summed gradient.
int dp_fused_update_ranges(DpFused *d, const DpRangeList &rl, const float *grads, float *m, float *v, float lr, float beta1,
                           float beta2, float eps, float wd, int step, const double *d_sumsq_total, float clip, bool alone,
                           cudaStream_t st) {
    BMB_TRY(check_ranges(rl));
    const float bc1 = 1.0f - powf(beta1, (float)step), bc2 = 1.0f - powf(beta2, (float)step);
    dp_adamw_broadcast_ranges_k<<<alone ? d->blocks : sm_count(), 256, 0, st>>>(d->pb, d->nranks, d->rank, grads, m, v, rl, lr, beta1, beta2, eps,
                                                          wd, bc1, bc2, d_sumsq_total, clip, (float)d->nranks);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

// shadow = TF32-rounded params over the listed ranges, on `st`.
int dp_round_ranges(const DpRangeList &rl, float *shadow, const float *params, bool alone, cudaStream_t st) {
    BMB_TRY(check_ranges(rl));
    dp_round_ranges_k<<<(alone ? 4 : 1) * sm_count(), 256, 0, st>>>(rl, shadow, params);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace bmb
