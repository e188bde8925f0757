// In-place sum all-reduce across the GPUs of one process, with the
// reference's types and signatures (src/ddp.h:32-69).  The struct keeps the
// reference's fields and layout so that callers which place a DDP on their
// stack link against libbmb.so unchanged; this implementation keeps its own
// state behind `host_stage`, which it owns (treat every field as read-only).
// `n`, `dev`, `peer`, `any_peer` and `last` are filled in for the caller.
#pragma once
#include <cstddef>
#include <cuda_runtime.h>

struct DDPTiming {
    double reduce_scatter_ms;
    double all_gather_ms;
    double total_ms;
    size_t bytes_per_device;  // moved by one device over both phases
};

struct DDP {
    int n;
    int dev[8];
    bool peer[8][8];     // peer[i][j]: rank i reaches rank j's memory directly
    bool any_peer;
    float *recv[8];      // unused here
    size_t recv_cap;     // unused here
    float *host_stage;   // opaque handle of this implementation
    size_t stage_cap;    // unused here
    cudaStream_t stream[8];             // unused here
    cudaEvent_t start[8], stop[8];      // unused here
    DDPTiming last;
};

// `devices` may name one physical device several times: the whole exchange
// then runs on one GPU, which is how it is rehearsed without a second one.
void ddp_init(DDP &d, int n, const int *devices);
void ddp_free(DDP &d);
// bufs[r] lives on dev[r]; afterwards every buffer holds the sum.  Returns
// when the exchange is complete on every rank.
void ddp_allreduce(DDP &d, float **bufs, size_t count);
const DDPTiming &ddp_timing(const DDP &d);
void ddp_report_topology(const DDP &d);
