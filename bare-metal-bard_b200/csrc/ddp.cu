// Gradient all-reduce for data-parallel training (src/ddp.h:32-69, src/ddp.cu).
//
// Two forms.
//
// (1) Single process, one rank per entry of `devices` -- the reference's own
//     calling convention.  The reference walks a ring of 2(n-1) host-stepped
//     peer copies with a host-wide sync after each (src/ddp.cu:216-251).  On
//     NVSwitch every GPU reaches every peer at full bandwidth, so the ring
//     order buys nothing; here the sum is a two-phase direct exchange:
//       reduce-scatter: rank r sums slice r of every rank's buffer, reading
//                       the peers' memory with 128-bit loads, in rank order
//                       0..n-1 (so the result is reproducible and identical
//                       on all ranks), and writes it into its own slice r;
//       all-gather:     rank r pulls every other reduced slice k from rank k.
//     The same bytes cross the links as in the ring, 2(n-1)/n * S per device,
//     in two launches per rank, ordered by events instead of host syncs.
//     Pairs without working peer access (or DDP_NO_P2P in the environment, as
//     src/ddp.cu:116-120) go through a pinned host bounce instead.
//     The same device may be named more than once (src/ddp.h:53-57): the
//     kernels then read ordinary local pointers and nothing waits on a flag.
//
// (2) One process per GPU: NCCL over NVLink/NVSwitch, opened with dlopen so
//     that the library loads (and everything else works) where NCCL is absent.
#include "common.cuh"
#include <dlfcn.h>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace bmb {
namespace {

constexpr int MAXR = 8;

struct SrcList { const float *p[MAXR]; };

// dst[i] = sum_k src.p[k][i] in rank order.  dst may alias one of the sources.
__global__ void reduce_slices_k(float *__restrict__ dst, SrcList src, int n, size_t len, int vec) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const size_t n4 = len >> 2;
        for (; i < n4; i += stride) {
            float4 a = reinterpret_cast<const float4 *>(src.p[0])[i];
            for (int k = 1; k < n; ++k) {
                const float4 b = reinterpret_cast<const float4 *>(src.p[k])[i];
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            }
            reinterpret_cast<float4 *>(dst)[i] = a;
        }
        i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        for (; i < len; i += stride) {
            float a = src.p[0][i];
            for (int k = 1; k < n; ++k) a += src.p[k][i];
            dst[i] = a;
        }
    } else {
        for (; i < len; i += stride) {
            float a = src.p[0][i];
            for (int k = 1; k < n; ++k) a += src.p[k][i];
            dst[i] = a;
        }
    }
}

__global__ void copy_slice_k(float *__restrict__ dst, const float *__restrict__ src, size_t len, int vec) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const size_t n4 = len >> 2;
        for (; i < n4; i += stride)
            reinterpret_cast<float4 *>(dst)[i] = reinterpret_cast<const float4 *>(src)[i];
        i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    }
    for (; i < len; i += stride) dst[i] = src[i];
}

struct Slice { size_t off, len; };
// Slice r of count elements split n ways; the last non-empty slice takes the
// remainder, later ones are empty (the convention of src/ddp.cu:34-40).
inline Slice slice_of(size_t count, int n, int r) {
    const size_t per = (count + (size_t)n - 1) / (size_t)n;
    const size_t off = per * (size_t)r;
    if (off >= count) return {count, 0};
    return {off, (off + per <= count) ? per : count - off};
}

}  // namespace
}  // namespace bmb

using namespace bmb;

struct bmb_ddp {
    int n = 0;
    int dev[MAXR];
    bool peer[MAXR][MAXR];
    bool any_peer = false, all_peer = false;
    cudaStream_t stream[MAXR] = {};
    cudaEvent_t ready[MAXR] = {}, reduced[MAXR] = {}, done[MAXR] = {};
    cudaEvent_t t0 = nullptr, t1 = nullptr, t2 = nullptr;
    float *recv[MAXR];
    size_t recv_cap = 0;
    float *host_stage = nullptr;
    size_t stage_cap = 0;
    bmb_ddp_timing last{0, 0, 0, 0};
};

static int ddp_probe_pair(bmb_ddp *d, int i, int j) {
    // Move four bytes i -> j and read them back: peer access being enabled is
    // not evidence that it works (src/ddp.cu:108-148).
    float *a = nullptr, *b = nullptr;
    const float probe = 1.0f + 100.0f * i + j;
    float back = -1.0f;
    BMB_CUDA(cudaSetDevice(d->dev[i]));
    BMB_CUDA(cudaMalloc(&a, sizeof(float)));
    BMB_CUDA(cudaMemcpy(a, &probe, sizeof(float), cudaMemcpyHostToDevice));
    BMB_CUDA(cudaSetDevice(d->dev[j]));
    BMB_CUDA(cudaMalloc(&b, sizeof(float)));
    BMB_CUDA(cudaMemset(b, 0, sizeof(float)));
    BMB_CUDA(cudaSetDevice(d->dev[i]));
    BMB_CUDA(cudaMemcpyPeer(b, d->dev[j], a, d->dev[i], sizeof(float)));
    BMB_CUDA(cudaSetDevice(d->dev[j]));
    BMB_CUDA(cudaMemcpy(&back, b, sizeof(float), cudaMemcpyDeviceToHost));
    if (back != probe) {
        printf("ddp       WARNING: peer %d->%d is enabled but moved the wrong bytes "
               "(sent %.1f, got %.1f); staging that pair through host memory.\n",
               d->dev[i], d->dev[j], probe, back);
        d->peer[i][j] = false;
    }
    BMB_CUDA(cudaSetDevice(d->dev[i]));
    BMB_CUDA(cudaFree(a));
    BMB_CUDA(cudaSetDevice(d->dev[j]));
    BMB_CUDA(cudaFree(b));
    return BMB_OK;
}

static int ddp_build(bmb_ddp *d);

extern "C" {

int bmb_ddp_create(bmb_ddp **out, int n, const int *devices) {
    if (!out || !devices || n < 1 || n > MAXR) return fail(BMB_E_ARG, "ddp: need 1 <= n <= %d ranks", MAXR);
    int ndev = 0;
    BMB_CUDA(cudaGetDeviceCount(&ndev));
    for (int r = 0; r < n; ++r)
        if (devices[r] < 0 || devices[r] >= ndev) return fail(BMB_E_ARG, "ddp: device %d not present", devices[r]);
    int prev = 0;
    BMB_CUDA(cudaGetDevice(&prev));
    bmb_ddp *d = new bmb_ddp();
    d->n = n;
    for (int r = 0; r < n; ++r) { d->dev[r] = devices[r]; d->recv[r] = nullptr; }
    const int rc = ddp_build(d);
    cudaSetDevice(prev);
    if (rc != BMB_OK) {
        bmb_ddp_destroy(d);               // streams and events made so far go with it
        return rc;
    }
    *out = d;
    return BMB_OK;
}

}  // extern "C"

static int ddp_build(bmb_ddp *d) {
    const int n = d->n;
    const bool no_p2p = getenv("DDP_NO_P2P") != nullptr;
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < n; ++j) {
            d->peer[i][j] = false;
            if (i == j) continue;
            // DDP_NO_P2P stages EVERY transfer through host memory, ranks sharing a device included
            // (src/ddp.cu:116-120 clears the whole matrix), so the staged route can be exercised anywhere.
            if (no_p2p) continue;
            if (d->dev[i] == d->dev[j]) { d->peer[i][j] = true; continue; }
            int can = 0;
            BMB_CUDA(cudaDeviceCanAccessPeer(&can, d->dev[i], d->dev[j]));
            if (can) {
                BMB_CUDA(cudaSetDevice(d->dev[i]));
                const cudaError_t e = cudaDeviceEnablePeerAccess(d->dev[j], 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) can = 0;
                cudaGetLastError();
            }
            d->peer[i][j] = can != 0;
        }
    if (no_p2p) printf("ddp       DDP_NO_P2P set: staging every transfer through host\n");
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < n; ++j)
            if (d->peer[i][j] && d->dev[i] != d->dev[j]) {
                const int s = ddp_probe_pair(d, i, j);
                if (s != BMB_OK) return s;
            }
    d->any_peer = false; d->all_peer = true;
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < n; ++j)
            if (i != j) { d->any_peer = d->any_peer || d->peer[i][j]; d->all_peer = d->all_peer && d->peer[i][j]; }
    for (int r = 0; r < n; ++r) {
        BMB_CUDA(cudaSetDevice(d->dev[r]));
        BMB_CUDA(cudaStreamCreate(&d->stream[r]));
        BMB_CUDA(cudaEventCreateWithFlags(&d->ready[r], cudaEventDisableTiming));
        BMB_CUDA(cudaEventCreateWithFlags(&d->reduced[r], cudaEventDisableTiming));
        BMB_CUDA(cudaEventCreateWithFlags(&d->done[r], cudaEventDisableTiming));
    }
    BMB_CUDA(cudaSetDevice(d->dev[0]));
    BMB_CUDA(cudaEventCreate(&d->t0));
    BMB_CUDA(cudaEventCreate(&d->t1));
    BMB_CUDA(cudaEventCreate(&d->t2));
    return BMB_OK;
}

extern "C" {

int bmb_ddp_destroy(bmb_ddp *d) {
    if (!d) return BMB_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    for (int r = 0; r < d->n; ++r) {
        cudaSetDevice(d->dev[r]);
        if (d->recv[r]) cudaFree(d->recv[r]);
        if (d->stream[r]) cudaStreamDestroy(d->stream[r]);
        if (d->ready[r]) cudaEventDestroy(d->ready[r]);
        if (d->reduced[r]) cudaEventDestroy(d->reduced[r]);
        if (d->done[r]) cudaEventDestroy(d->done[r]);
    }
    cudaSetDevice(d->dev[0]);
    if (d->t0) cudaEventDestroy(d->t0);
    if (d->t1) cudaEventDestroy(d->t1);
    if (d->t2) cudaEventDestroy(d->t2);
    if (d->host_stage) cudaFreeHost(d->host_stage);
    cudaSetDevice(prev);
    delete d;
    return BMB_OK;
}

// Host-bounced copy for a pair without peer access.  Blocking.
static int staged_copy(bmb_ddp *d, int src_rank, const float *src, int dst_rank, float *dst, size_t len) {
    if (len == 0) return BMB_OK;
    BMB_CUDA(cudaSetDevice(d->dev[src_rank]));
    BMB_CUDA(cudaMemcpyAsync(d->host_stage, src, len * sizeof(float), cudaMemcpyDeviceToHost, d->stream[src_rank]));
    BMB_CUDA(cudaStreamSynchronize(d->stream[src_rank]));
    BMB_CUDA(cudaSetDevice(d->dev[dst_rank]));
    BMB_CUDA(cudaMemcpyAsync(dst, d->host_stage, len * sizeof(float), cudaMemcpyHostToDevice, d->stream[dst_rank]));
    BMB_CUDA(cudaStreamSynchronize(d->stream[dst_rank]));
    return BMB_OK;
}

static int sync_all(bmb_ddp *d) {
    for (int r = 0; r < d->n; ++r) {
        BMB_CUDA(cudaSetDevice(d->dev[r]));
        BMB_CUDA(cudaStreamSynchronize(d->stream[r]));
    }
    return BMB_OK;
}

int bmb_ddp_allreduce(bmb_ddp *d, float **bufs, size_t count) {
    if (!d || !bufs) return fail(BMB_E_ARG, "ddp_allreduce: null argument");
    const int n = d->n;
    if (n == 1 || count == 0) { d->last = {0.0, 0.0, 0.0, 0}; return BMB_OK; }
    int prev = 0;
    BMB_CUDA(cudaGetDevice(&prev));
    const size_t per = (count + (size_t)n - 1) / (size_t)n;
    const int nsm = sm_count();

    if (!d->all_peer) {
        if (d->recv_cap < per) {
            for (int r = 0; r < n; ++r) {
                BMB_CUDA(cudaSetDevice(d->dev[r]));
                if (d->recv[r]) BMB_CUDA(cudaFree(d->recv[r]));
                BMB_CUDA(cudaMalloc(&d->recv[r], per * sizeof(float)));
            }
            d->recv_cap = per;
        }
        if (d->stage_cap < per) {
            if (d->host_stage) BMB_CUDA(cudaFreeHost(d->host_stage));
            BMB_CUDA(cudaMallocHost(&d->host_stage, per * sizeof(float)));
            d->stage_cap = per;
        }
    }

    // Every rank's buffer must be complete before any rank reads it.
    for (int r = 0; r < n; ++r) {
        BMB_CUDA(cudaSetDevice(d->dev[r]));
        BMB_CUDA(cudaEventRecord(d->ready[r], d->stream[r]));
    }
    for (int r = 0; r < n; ++r) {
        BMB_CUDA(cudaSetDevice(d->dev[r]));
        for (int k = 0; k < n; ++k)
            if (k != r) BMB_CUDA(cudaStreamWaitEvent(d->stream[r], d->ready[k], 0));
    }
    BMB_CUDA(cudaSetDevice(d->dev[0]));
    BMB_CUDA(cudaEventRecord(d->t0, d->stream[0]));

    // ---- reduce-scatter: rank r produces the sum of slice r ----
    if (d->all_peer) {
        for (int r = 0; r < n; ++r) {
            const Slice s = slice_of(count, n, r);
            if (s.len == 0) continue;
            SrcList src;
            bool vec = true;
            for (int k = 0; k < n; ++k) {
                src.p[k] = bufs[k] + s.off;
                vec = vec && (((uintptr_t)src.p[k]) % 16 == 0);
            }
            BMB_CUDA(cudaSetDevice(d->dev[r]));
            long long blocks = (long long)((s.len / 4 + 255) / 256);
            if (blocks > 4LL * nsm) blocks = 4LL * nsm;
            if (blocks < 1) blocks = 1;
            reduce_slices_k<<<(int)blocks, 256, 0, d->stream[r]>>>(bufs[r] + s.off, src, n, s.len, vec ? 1 : 0);
            count_launch();
            BMB_LAUNCH_CHECK();
        }
    } else {
        // Slice r of every other rank is brought to rank r and added in rank
        // order; pairs with peer access copy directly, the others bounce.
        BMB_TRY(sync_all(d));
        for (int r = 0; r < n; ++r) {
            const Slice s = slice_of(count, n, r);
            if (s.len == 0) continue;
            for (int k = 0; k < n; ++k) {
                if (k == r) continue;
                if (d->peer[k][r]) {
                    BMB_CUDA(cudaSetDevice(d->dev[r]));
                    BMB_CUDA(cudaMemcpyPeerAsync(d->recv[r], d->dev[r], bufs[k] + s.off, d->dev[k],
                                                 s.len * sizeof(float), d->stream[r]));
                } else {
                    BMB_TRY(staged_copy(d, k, bufs[k] + s.off, r, d->recv[r], s.len));
                }
                BMB_CUDA(cudaSetDevice(d->dev[r]));
                SrcList src;
                src.p[0] = bufs[r] + s.off;
                src.p[1] = d->recv[r];
                const bool vec = ((uintptr_t)src.p[0] % 16 == 0) && ((uintptr_t)src.p[1] % 16 == 0);
                long long blocks = (long long)((s.len / 4 + 255) / 256);
                if (blocks > 4LL * nsm) blocks = 4LL * nsm;
                if (blocks < 1) blocks = 1;
                reduce_slices_k<<<(int)blocks, 256, 0, d->stream[r]>>>(bufs[r] + s.off, src, 2, s.len, vec ? 1 : 0);
                count_launch();
                BMB_LAUNCH_CHECK();
                BMB_CUDA(cudaStreamSynchronize(d->stream[r]));
            }
        }
    }
    for (int r = 0; r < n; ++r) {
        BMB_CUDA(cudaSetDevice(d->dev[r]));
        BMB_CUDA(cudaEventRecord(d->reduced[r], d->stream[r]));
    }
    for (int r = 0; r < n; ++r) {
        BMB_CUDA(cudaSetDevice(d->dev[r]));
        for (int k = 0; k < n; ++k)
            if (k != r) BMB_CUDA(cudaStreamWaitEvent(d->stream[r], d->reduced[k], 0));
    }
    BMB_CUDA(cudaSetDevice(d->dev[0]));
    BMB_CUDA(cudaEventRecord(d->t1, d->stream[0]));

    // ---- all-gather: rank r pulls reduced slice k from rank k ----
    for (int r = 0; r < n; ++r) {
        for (int k = 0; k < n; ++k) {
            if (k == r) continue;
            const Slice s = slice_of(count, n, k);
            if (s.len == 0) continue;
            if (d->peer[r][k]) {
                BMB_CUDA(cudaSetDevice(d->dev[r]));
                const float *src = bufs[k] + s.off;
                float *dst = bufs[r] + s.off;
                const bool vec = ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0);
                long long blocks = (long long)((s.len / 4 + 255) / 256);
                if (blocks > 2LL * nsm) blocks = 2LL * nsm;
                if (blocks < 1) blocks = 1;
                copy_slice_k<<<(int)blocks, 256, 0, d->stream[r]>>>(dst, src, s.len, vec ? 1 : 0);
                count_launch();
                BMB_LAUNCH_CHECK();
            } else {
                BMB_TRY(staged_copy(d, k, bufs[k] + s.off, r, bufs[r] + s.off, s.len));
            }
        }
    }
    // Stream 0's second mark must follow every rank's gather.
    for (int r = 0; r < n; ++r) {
        BMB_CUDA(cudaSetDevice(d->dev[r]));
        BMB_CUDA(cudaEventRecord(d->done[r], d->stream[r]));
    }
    BMB_CUDA(cudaSetDevice(d->dev[0]));
    for (int r = 1; r < n; ++r) BMB_CUDA(cudaStreamWaitEvent(d->stream[0], d->done[r], 0));
    BMB_CUDA(cudaEventRecord(d->t2, d->stream[0]));
    BMB_TRY(sync_all(d));

    float ms1 = 0.f, ms2 = 0.f;
    BMB_CUDA(cudaSetDevice(d->dev[0]));
    BMB_CUDA(cudaEventElapsedTime(&ms1, d->t0, d->t1));
    BMB_CUDA(cudaEventElapsedTime(&ms2, d->t1, d->t2));
    d->last.reduce_scatter_ms = ms1;
    d->last.all_gather_ms = ms2;
    d->last.total_ms = ms1 + ms2;
    d->last.bytes_per_device = (size_t)(2 * (n - 1)) * per * sizeof(float);
    BMB_CUDA(cudaSetDevice(prev));
    return BMB_OK;
}

int bmb_ddp_slice(size_t count, int n, int r, size_t *off_out, size_t *len_out) {
    if (n < 1 || r < 0 || r >= n || !off_out || !len_out) return fail(BMB_E_ARG, "ddp_slice: bad argument");
    const Slice s = slice_of(count, n, r);
    *off_out = s.off;
    *len_out = s.len;
    return BMB_OK;
}

int bmb_ddp_timing_get(const bmb_ddp *d, bmb_ddp_timing *out) {
    if (!d || !out) return fail(BMB_E_ARG, "ddp_timing: null argument");
    *out = d->last;
    return BMB_OK;
}

int bmb_ddp_peer_matrix(const bmb_ddp *d, int *n_out, int *dev_out, unsigned char *peer_out) {
    if (!d) return fail(BMB_E_ARG, "ddp_peer_matrix: null handle");
    if (n_out) *n_out = d->n;
    for (int i = 0; i < d->n; ++i) {
        if (dev_out) dev_out[i] = d->dev[i];
        if (peer_out)
            for (int j = 0; j < d->n; ++j) peer_out[i * d->n + j] = d->peer[i][j] ? 1 : 0;
    }
    return BMB_OK;
}

int bmb_ddp_report_topology(const bmb_ddp *d) {
    if (!d) return fail(BMB_E_ARG, "ddp_report_topology: null handle");
    printf("ddp       %d rank(s) on device(s)", d->n);
    for (int r = 0; r < d->n; ++r) printf(" %d", d->dev[r]);
    bool same = true;
    for (int r = 1; r < d->n; ++r) same = same && (d->dev[r] == d->dev[0]);
    if (same && d->n > 1) printf("  [SIMULATED: one physical GPU]");
    printf("\n");
    if (d->n > 1) {
        printf("links     ");
        if (d->all_peer) printf("peer-to-peer enabled on every pair\n");
        else if (d->any_peer) printf("peer-to-peer on some pairs; others staged through host\n");
        else printf("NO peer access -- every transfer staged through host memory\n");
    }
    return BMB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------- NCCL form
namespace {
typedef struct { char internal[128]; } nccl_uid;
typedef void *nccl_comm_t;
struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(nccl_uid *) = nullptr;
    int (*CommInitRank)(nccl_comm_t *, int, nccl_uid, int) = nullptr;
    int (*CommDestroy)(nccl_comm_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool tried = false;
};
NcclApi g_nccl;

int nccl_load() {
    if (g_nccl.lib) return BMB_OK;
    if (g_nccl.tried) return fail(BMB_E_NCCL, "libnccl.so.2 could not be opened");
    g_nccl.tried = true;
    const char *names[] = {getenv("BMB_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *nm : names) {
        if (!nm) continue;
        lib = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
    }
    if (!lib) return fail(BMB_E_NCCL, "libnccl.so.2 could not be opened: %s", dlerror());
    g_nccl.GetUniqueId = (int (*)(nccl_uid *))dlsym(lib, "ncclGetUniqueId");
    g_nccl.CommInitRank = (int (*)(nccl_comm_t *, int, nccl_uid, int))dlsym(lib, "ncclCommInitRank");
    g_nccl.CommDestroy = (int (*)(nccl_comm_t))dlsym(lib, "ncclCommDestroy");
    g_nccl.AllReduce = (int (*)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t))dlsym(lib, "ncclAllReduce");
    g_nccl.GetErrorString = (const char *(*)(int))dlsym(lib, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllReduce)
        return fail(BMB_E_NCCL, "libnccl.so.2 lacks an expected symbol");
    g_nccl.lib = lib;
    return BMB_OK;
}
int nccl_fail(const char *what, int code) {
    return fail(BMB_E_NCCL, "%s -> %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(code) : "error");
}
}  // namespace

struct bmb_comm {
    nccl_comm_t comm = nullptr;
    int nranks = 1, rank = 0;
};

extern "C" {

int bmb_comm_unique_id(unsigned char id_out[128]) {
    BMB_TRY(nccl_load());
    nccl_uid id;
    const int rc = g_nccl.GetUniqueId(&id);
    if (rc) return nccl_fail("ncclGetUniqueId", rc);
    memcpy(id_out, id.internal, 128);
    return BMB_OK;
}

int bmb_comm_create(bmb_comm **out, const unsigned char id[128], int nranks, int rank) {
    if (!out || !id || nranks < 1 || rank < 0 || rank >= nranks) return fail(BMB_E_ARG, "comm_create: bad argument");
    BMB_TRY(nccl_load());
    nccl_uid uid;
    memcpy(uid.internal, id, 128);
    bmb_comm *c = new bmb_comm();
    c->nranks = nranks; c->rank = rank;
    const int rc = g_nccl.CommInitRank(&c->comm, nranks, uid, rank);
    if (rc) { delete c; return nccl_fail("ncclCommInitRank", rc); }
    *out = c;
    return BMB_OK;
}

int bmb_comm_destroy(bmb_comm *c) {
    if (!c) return BMB_OK;
    if (c->comm) g_nccl.CommDestroy(c->comm);
    delete c;
    return BMB_OK;
}

int bmb_comm_allreduce(bmb_comm *c, float *buf, size_t count, void *stream) {
    if (!c || !c->comm) return fail(BMB_E_ARG, "comm_allreduce: null communicator");
    if (count == 0 || c->nranks == 1) return BMB_OK;
    const int rc = g_nccl.AllReduce(buf, buf, count, /*ncclFloat32*/ 7, /*ncclSum*/ 0, c->comm, (cudaStream_t)stream);
    if (rc) return nccl_fail("ncclAllReduce", rc);
    return BMB_OK;
}

// Sum of `count` doubles across the ranks (the squared-norm exchange of the fused data-parallel step).
int bmb_comm_allreduce_f64(bmb_comm *c, double *buf, size_t count, void *stream) {
    if (!c || !c->comm) return fail(BMB_E_ARG, "comm_allreduce_f64: null communicator");
    if (count == 0 || c->nranks == 1) return BMB_OK;
    const int rc = g_nccl.AllReduce(buf, buf, count, /*ncclFloat64*/ 8, /*ncclSum*/ 0, c->comm, (cudaStream_t)stream);
    if (rc) return nccl_fail("ncclAllReduce", rc);
    return BMB_OK;
}

}  // extern "C"
