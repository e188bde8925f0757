// GPT training step on one GPU, the caller of every kernel in this library:
// the host-side loop of src/gpt.cu:222-385 (forward, backward) and
// src/train_gpt.cu:397-464 (all-reduce, global-norm clip, AdamW), restated
// so that one optimiser step issues no blocking call: tokens arrive by async
// copy, the loss mean and the gradient norm stay on the device, and the
// all-reduce is enqueued on the same stream as the backward pass.
//
// Parameter and gradient storage is one flat buffer in the reference's tensor
// order (src/gpt.cu:32-51), so raw parameter dumps are interchangeable.
#include "common.cuh"
#include <cmath>
#include <cstring>
#include <random>
#include <string>
#include <vector>

namespace bmb {
int layernorm_bwd_blocks(int N);
bool flash_tc_supported(int T, int C, int NH, const float *qkv, const float *out);
int flash_forward_tc(float *out, float *lse, const float *qkv, int B, int T, int C, int NH, bool qkv_rounded,
                     cudaStream_t st);
int flash_backward_tc(float *dqkv, float *dsum, const float *dout, const float *qkv, const float *out,
                      const float *lse, int B, int T, int C, int NH, bool rounded, cudaStream_t st, float *dbias_qkv = nullptr);
namespace tc {
int status_word(int **dev_ptr, volatile int **host_ptr);
}
struct DpFused;
int dp_fused_export(const float *grads, const float *params, const float *shadow, void *out192);
int dp_fused_create(DpFused **out, int rank, int nranks, size_t n, float *grads, float *params, float *shadow,
                    const void *all_handles);
void dp_fused_destroy(DpFused *d);
int dp_fused_reduce_ranges(DpFused *d, const DpRangeList &rl, float *grads, int slot, bool alone, cudaStream_t st);
int dp_fused_sumsq(DpFused *d, double *d_sumsq_pieces, cudaStream_t st);
int dp_fused_update_ranges(DpFused *d, const DpRangeList &rl, const float *grads, float *m, float *v, float lr, float beta1,
                           float beta2, float eps, float wd, int step, const double *d_sumsq_total, float clip, bool alone,
                           cudaStream_t st);
int dp_round_ranges(const DpRangeList &rl, float *shadow, const float *params, bool alone, cudaStream_t st);
}
using namespace bmb;

namespace {
constexpr int NPT = 16;  // parameter tensors
}

struct bmb_trainer {
    bmb_train_config c;
    int dev = 0;
    cudaStream_t st = nullptr;
    size_t psize[NPT], poff[NPT], num_params = 0;
    float *params = nullptr, *grads = nullptr, *m = nullptr, *v = nullptr;
    float *shadow = nullptr;  // TF32-rounded parameters (tensor-core modes only)
    float *acts = nullptr, *bacts = nullptr;
    size_t num_acts = 0, num_bacts = 0;
    int *d_tokens = nullptr, *d_targets = nullptr;
    float *d_loss = nullptr;
    double *d_sumsq = nullptr;
    bmb_comm *comm = nullptr;
    int nranks = 1;
    DpFused *dp = nullptr;        // fused gradient exchange + optimiser over peer memory, when attached
    float *d_token = nullptr;     // one float the ranks all-reduce where the step only needs a barrier
    // activation pointers
    float *encoded, *ln1, *ln1_mean, *ln1_rstd, *qkv, *qkvr, *att, *lse, *atty, *attproj, *residual2,
        *ln2, *ln2_mean, *ln2_rstd, *fch, *fch_gelu, *fcproj, *residual3, *lnf, *lnf_mean, *lnf_rstd,
        *logits, *probs, *losses;
    float *dres, *dln1, *dln2, *datty, *dqkv, *dqkvr, *datt, *dsum, *dfch, *dfch_gelu, *dlogits, *dlnf;
    // The forward and backward pass of a step, captured once into a CUDA graph and replayed: the
    // ~370 launches of a step then follow one another without a host round trip each.
    // The step is a list of pieces (runs of units: embedding, layers, head, and their backward counterparts), one
    // graph each: a single piece without the fused exchange, five with it (see plan_pieces).
    bool use_graph = true, graph_failed = false;
    int eager_passes = 0;                 // the first pass runs eagerly (it sizes the library's scratch)
    struct Piece {
        int u0 = 0, u1 = 0;               // units [u0, u1)
        int needs = -1;                   // chunk whose new parameters must have arrived before the piece starts
        int reduces = -1;                 // chunk whose gradients are final when the piece ends
        cudaGraphExec_t exec = nullptr;
        long long launches = 0;
    };
    std::vector<Piece> pieces;
    unsigned long long graph_scratch_gen = 0;   // the device's scratch generation the graphs were captured under
    // Fused exchange, overlapped forms: the parameter space is cut into three chunks -- A: embeddings + layer 0,
    // B: layers 1 .. c2-1, C: layers c2 .. L-1 + final layernorm.  Backward finishes C, then B, then A, and each
    // chunk's reduce runs on the exchange stream while backward goes on; the next forward needs A, then B, then
    // C, and each chunk's update + broadcast is awaited only by the first piece that reads it.
    static constexpr int NCHUNK = 3;
    DpRangeList chunk[NCHUNK];
    int chunk_split = 0;                  // c2
    // BMB_TRAINER_OVERLAP: 0 (default) one chunk, exchanged after backward; 1 three chunks, each reduced while backward
    // goes on, all updated after the last reduce; 2 also the updates overlapped, with the next step's forward.
    // Measured at 2 and 4 GPUs (per-step timelines, BMB_TRAINER_TIMELINE): what the overlapped forms hide they give
    // back -- the kernels of the main stream run slower beside the exchange's memory traffic by about the time the
    // exchange takes -- so 0 is never worse there: 17.52 / 17.73 / 17.85 ms per step at 2 GPUs for 0 / 1 / 2.
    int overlap = 0;
    cudaStream_t st_x = nullptr;          // exchange stream
    cudaEvent_t ev_seg[NCHUNK] = {nullptr, nullptr, nullptr};   // main stream: the chunk's gradients are final
    cudaEvent_t ev_upd[NCHUNK] = {nullptr, nullptr, nullptr};   // exchange stream: the chunk's new parameters are in place
    bool upd_pending[NCHUNK] = {false, false, false};
    // Developer timeline (BMB_TRAINER_TIMELINE=<step>): timed events at the ends of the pieces and of the exchange's
    // phases in that step and the next, printed to stderr once both have drained.
    int tl_step = 0;
    std::vector<std::pair<std::string, cudaEvent_t>> tl;
    float *gen_probs = nullptr;   // one row of next-token probabilities, allocated by the first sampling call
    // The two products of a linear layer's backward (dX = dY W and dW = dY^T X: the same FLOP count, both waiting only
    // for dY) run side by side, each on half of the SMs: dX on the main stream, dW on this one, forked and joined
    // by events -- one launch gap, one ramp and one tail per pair instead of two.
    cudaStream_t st_dw = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    bool side_by_side = true;
    // BMB_TRAINER_FUSE_GELU=1 (fused TF32 mode): the MLP's activation in the epilogue of the product before it.  Off by
    // default: measured at the 124M shapes the product gets 37 us slower (its epilogue is no longer hidden behind
    // the next tile's main loop) for the 35 us pass it saves.
    bool qkv_bias_in_attention = true;   // BMB_TRAINER_QKV_BIAS_IN_ATTENTION=0: a sweep over dqkv of its own again
    int fuse_gelu = 0;           // 0: GELU is a kernel of its own; 1: it rides in the fc product's epilogue; 2: with the approximate tanh
    // Deferred column sums (single-piece steps): the backward kernels' partial rows go to this arena and one batched
    // launch at the end of backward finishes all the parameter-gradient sums (BMB_TRAINER_DEFER_COLSUMS=0: each
    // sum by a launch of its own, right after its kernel).
    bool defer_colsums = true;
    ColumnAddCollector col;
    std::vector<ColumnAddJob> col_jobs_host;
    ColumnAddJob *col_jobs_dev = nullptr;
    bool col_jobs_uploaded = false, col_active = false;
    int col_njobs = 0, col_max_cols = 0;
    bool unit_span_whole = false;         // the units being run cover the whole backward pass (set by run_units)
    // profiling
    bool prof = false;
    std::vector<cudaEvent_t> ev;
    size_t ev_used = 0;
    double prof_flop = 0.0, prof_ms = 0.0;
    long long prof_calls = 0, launches0 = 0;
};

namespace {

void param_sizes(size_t *s, const bmb_train_config &c) {
    const size_t L = c.n_layer, C = c.n_embd, Vp = c.padded_vocab, maxT = c.max_seq_len;
    const size_t sz[NPT] = {Vp * C, maxT * C, L * C, L * C, L * 3 * C * C, L * 3 * C, L * C * C, L * C,
                            L * C,  L * C,    L * 4 * C * C, L * 4 * C, L * C * 4 * C, L * C, C, C};
    for (int i = 0; i < NPT; ++i) s[i] = sz[i];
}
enum { P_WTE, P_WPE, P_LN1W, P_LN1B, P_QKVW, P_QKVB, P_APW, P_APB, P_LN2W, P_LN2B, P_FCW, P_FCB, P_FPW, P_FPB, P_LNFW, P_LNFB };

// Entry points run on the trainer's device and stream.  Unless told otherwise they first make the main stream
// wait for what the last step left running on the exchange stream (parameter chunks still being updated).
struct Scope {
    int prev_dev = 0;
    void *prev_stream;
    explicit Scope(bmb_trainer *t, bool join = true) {
        cudaGetDevice(&prev_dev);
        cudaSetDevice(t->dev);
        prev_stream = bmb_get_stream();
        bmb_set_stream(t->st);
        if (join)
            for (int c = 0; c < bmb_trainer::NCHUNK; ++c)
                if (t->upd_pending[c]) { cudaStreamWaitEvent(t->st, t->ev_upd[c], 0); t->upd_pending[c] = false; }
    }
    ~Scope() { set_emit_rounded(false); bmb_set_stream(prev_stream); cudaSetDevice(prev_dev); }
};

// "Fused" TF32 mode: every kernel that produces a GEMM or attention operand
// stores it already rounded to TF32 (so the tensor-core kernels read activations
// and gradients where they lie), and the bias add rides in the GEMM epilogue.
bool fused_tf32(const bmb_train_config &c) { return c.fused && c.math == BMB_MATH_TF32; }

// Attention kernel configuration for this trainer's arithmetic: the SIMT fp32
// kernels, or the tensor-core pair (config 2 of both tables) when the GEMMs
// run on tensor cores and the head size is the one those kernels serve.
int attn_cfg(const bmb_train_config &c) {
    return (c.math != BMB_MATH_FP32 && c.n_embd / c.n_head == 64) ? 2 : 0;
}

int collect_profile(bmb_trainer *t) {
    for (size_t i = 0; i + 1 < t->ev_used; i += 2) {
        float ms = 0.f;
        BMB_CUDA(cudaEventElapsedTime(&ms, t->ev[i], t->ev[i + 1]));
        t->prof_ms += ms;
    }
    t->ev_used = 0;
    return BMB_OK;
}

// One matmul of the model, optionally bracketed by events.
int mm(bmb_trainer *t, int flags, int ta, int tb, int M, int N, int K, const float *A, const float *B,
       float beta, float *C, const float *bias = nullptr, cudaStream_t on = nullptr, float *aux_gelu = nullptr) {
    if (on) return gemm_any_bias(t->c.math, flags, ta, tb, 1, M, N, K, 1.0f, A, 0, B, 0, beta, C, 0, bias, on, aux_gelu);
    if (t->prof) {
        if (t->ev_used + 2 > t->ev.size()) {
            for (int i = 0; i < 64; ++i) {
                cudaEvent_t e;
                BMB_CUDA(cudaEventCreate(&e));
                t->ev.push_back(e);
            }
        }
        BMB_CUDA(cudaEventRecord(t->ev[t->ev_used], t->st));
    }
    BMB_TRY(gemm_any_bias(t->c.math, flags, ta, tb, 1, M, N, K, 1.0f, A, 0, B, 0, beta, C, 0, bias, t->st, aux_gelu));
    if (t->prof) {
        BMB_CUDA(cudaEventRecord(t->ev[t->ev_used + 1], t->st));
        t->ev_used += 2;
        t->prof_flop += 2.0 * M * N * K;
        t->prof_calls += 1;
    }
    return BMB_OK;
}

// Shapes and operand conventions shared by the units of a pass.
struct Dims {
    int B, T, C, L, NH, Vp, V, N;
    size_t BTC, BT, BT3C, BT4C, qkvr_sz, att_sz, lse_sz;
    const float *W, *P;      // weights as the GEMMs read them (the pre-rounded shadow copy in the tensor-core modes), and as stored
    float *G;
    bool fz;
    int wflag;               // products with a weight: A = an activation or gradient (rounded by its producer when fused), B = the weight
    int gflag;               // weight-gradient products: both operands are activations / gradients
};
Dims dims_of(bmb_trainer *t) {
    const bmb_train_config &c = t->c;
    Dims d;
    d.B = c.B; d.T = c.T; d.C = c.n_embd; d.L = c.n_layer; d.NH = c.n_head; d.Vp = c.padded_vocab; d.V = c.vocab_size;
    d.N = d.B * d.T;
    d.BTC = (size_t)d.N * d.C; d.BT = d.N; d.BT3C = 3 * d.BTC; d.BT4C = 4 * d.BTC;
    d.qkvr_sz = 4 * d.BTC; d.att_sz = (size_t)d.B * d.NH * d.T * d.T; d.lse_sz = (size_t)d.B * d.NH * d.T;
    d.W = (c.math == BMB_MATH_FP32 || !t->shadow) ? t->params : t->shadow;
    d.P = t->params;
    d.G = t->grads;
    d.fz = fused_tf32(c);
    d.wflag = ((d.W == t->shadow) ? BMB_GEMM_B_ROUNDED : 0) | (d.fz ? BMB_GEMM_A_ROUNDED : 0);
    d.gflag = d.fz ? (BMB_GEMM_A_ROUNDED | BMB_GEMM_B_ROUNDED) : 0;
    return d;
}

int fwd_embed(bmb_trainer *t, const Dims &d) {
    BMB_TRY(bmb_encoder_forward(t->encoded, t->d_tokens, d.P + t->poff[P_WTE], d.P + t->poff[P_WPE], d.B, d.T, d.C));
    // The first layernorm stands alone; every later one (and the final one) rides with the
    // residual add that produces its input.
    return bmb_layernorm_forward(t->ln1, t->ln1_mean, t->ln1_rstd, t->encoded, d.P + t->poff[P_LN1W], d.P + t->poff[P_LN1B], d.N, d.C);
}

int fwd_layer(bmb_trainer *t, const Dims &d, int l) {
    const bmb_train_config &c = t->c;
    const int N = d.N, C = d.C, L = d.L, NH = d.NH, B = d.B, T = d.T;
    const size_t BTC = d.BTC, BT = d.BT;
    const float *W = d.W, *P = d.P;
    const int wflag = d.wflag;
    const bool fz = d.fz;
    float *residual = (l == 0) ? t->encoded : t->residual3 + (size_t)(l - 1) * BTC;
    float *ln1 = t->ln1 + l * BTC, *qkv = t->qkv + l * d.BT3C, *atty = t->atty + l * BTC;
    float *attproj = t->attproj + l * BTC, *res2 = t->residual2 + l * BTC, *ln2 = t->ln2 + l * BTC;
    float *fch = t->fch + l * d.BT4C, *fchg = t->fch_gelu + l * d.BT4C, *fcproj = t->fcproj + l * BTC;
    float *res3 = t->residual3 + l * BTC;
    if (fz) {
        BMB_TRY(mm(t, wflag | BMB_GEMM_C_ROUNDED, 0, 1, N, 3 * C, C, ln1, W + t->poff[P_QKVW] + (size_t)l * 3 * C * C, 0.0f, qkv,
                   P + t->poff[P_QKVB] + (size_t)l * 3 * C));
    } else {
        BMB_TRY(mm(t, wflag, 0, 1, N, 3 * C, C, ln1, W + t->poff[P_QKVW] + (size_t)l * 3 * C * C, 0.0f, qkv));
        BMB_TRY(bmb_bias_forward(qkv, P + t->poff[P_QKVB] + (size_t)l * 3 * C, N, 3 * C));
    }
    if (c.use_flash && fz && attn_cfg(c) == 2)
        BMB_TRY(flash_forward_tc(atty, t->lse + l * d.lse_sz, qkv, B, T, C, NH, true, t->st));
    else if (c.use_flash)
        BMB_TRY(bmb_flash_attention_forward_cfg(attn_cfg(c), atty, t->lse + l * d.lse_sz, qkv, B, T, C, NH));
    else
        BMB_TRY(bmb_attention_forward(atty, t->qkvr + l * d.qkvr_sz, t->att + l * d.att_sz, qkv, B, T, C, NH));
    if (fz) {
        BMB_TRY(mm(t, wflag, 0, 1, N, C, C, atty, W + t->poff[P_APW] + (size_t)l * C * C, 0.0f, attproj,
                   P + t->poff[P_APB] + (size_t)l * C));
    } else {
        BMB_TRY(mm(t, wflag, 0, 1, N, C, C, atty, W + t->poff[P_APW] + (size_t)l * C * C, 0.0f, attproj));
        BMB_TRY(bmb_bias_forward(attproj, P + t->poff[P_APB] + (size_t)l * C, N, C));
    }
    BMB_TRY(bmb_residual_layernorm_forward(res2, ln2, t->ln2_mean + l * BT, t->ln2_rstd + l * BT, residual, attproj,
                                           P + t->poff[P_LN2W] + (size_t)l * C, P + t->poff[P_LN2B] + (size_t)l * C, N, C));
    if (fz) {
        // bias and GELU ride in the product's epilogue: fch and fch_gelu leave the accumulator together
        BMB_TRY(mm(t, wflag | (t->fuse_gelu == 2 ? BMB_GEMM_AUX_FAST : 0), 0, 1, N, 4 * C, C, ln2, W + t->poff[P_FCW] + (size_t)l * 4 * C * C, 0.0f, fch,
                   P + t->poff[P_FCB] + (size_t)l * 4 * C, nullptr, t->fuse_gelu ? fchg : nullptr));
        if (!t->fuse_gelu) BMB_TRY(bmb_gelu_forward(fchg, fch, (int)d.BT4C));
    } else {
        BMB_TRY(mm(t, wflag, 0, 1, N, 4 * C, C, ln2, W + t->poff[P_FCW] + (size_t)l * 4 * C * C, 0.0f, fch));
        BMB_TRY(bmb_bias_forward(fch, P + t->poff[P_FCB] + (size_t)l * 4 * C, N, 4 * C));
        BMB_TRY(bmb_gelu_forward(fchg, fch, (int)d.BT4C));
    }
    if (fz) {
        BMB_TRY(mm(t, wflag, 0, 1, N, C, 4 * C, fchg, W + t->poff[P_FPW] + (size_t)l * C * 4 * C, 0.0f, fcproj,
                   P + t->poff[P_FPB] + (size_t)l * C));
    } else {
        BMB_TRY(mm(t, wflag, 0, 1, N, C, 4 * C, fchg, W + t->poff[P_FPW] + (size_t)l * C * 4 * C, 0.0f, fcproj));
        BMB_TRY(bmb_bias_forward(fcproj, P + t->poff[P_FPB] + (size_t)l * C, N, C));
    }
    if (l + 1 < L)
        return bmb_residual_layernorm_forward(res3, t->ln1 + (l + 1) * BTC, t->ln1_mean + (l + 1) * BT, t->ln1_rstd + (l + 1) * BT,
                                              res2, fcproj, P + t->poff[P_LN1W] + (size_t)(l + 1) * C,
                                              P + t->poff[P_LN1B] + (size_t)(l + 1) * C, N, C);
    return bmb_residual_layernorm_forward(res3, t->lnf, t->lnf_mean, t->lnf_rstd, res2, fcproj, P + t->poff[P_LNFW],
                                          P + t->poff[P_LNFB], N, C);
}

int fwd_head(bmb_trainer *t, const Dims &d, bool with_loss) {
    BMB_TRY(mm(t, d.wflag, 0, 1, d.N, d.Vp, d.C, t->lnf, d.W + t->poff[P_WTE], 0.0f, t->logits));
    if (!with_loss) return BMB_OK;        // sampling reads the logits only
    // Loss and its gradient with respect to the logits in one sweep (mean loss: dloss = 1/N).
    BMB_TRY(bmb_softmax_crossentropy_fused(t->dlogits, t->losses, t->logits, t->d_targets, d.N, d.V, d.Vp, 1.0f / d.N));
    return bmb_reduce_mean_device(t->losses, d.N, t->d_loss);
}

// dX = dY * W with W stored [out, in]: W is the MN-major operand of this product.
int dx(bmb_trainer *t, const Dims &d, int flags, int M_, int N_, int K_, const float *dY, int id, size_t woff, float *dX) {
    return mm(t, flags, 0, 0, M_, N_, K_, dY, d.W + t->poff[id] + woff, 0.0f, dX);
}

// dX and dW of one linear layer.  Side by side (fused TF32 mode, not while GEMMs are being timed one by one):
// the weight gradient goes to the second stream, both planned for half of the SMs.
// (only where both read their operands in place: a product that first rounds an operand into the per-device
// staging scratch must not share it with another in flight)
int dx_dw(bmb_trainer *t, const Dims &d, int xflags, int Mx, int Nx, int Kx, const float *dY, int id, size_t woff, float *dX,
          int Mw, int Nw, const float *act, float *dW) {
    const bool sbs = t->side_by_side && d.fz && !t->prof && t->st_dw;
    if (!sbs) {
        BMB_TRY(dx(t, d, xflags, Mx, Nx, Kx, dY, id, woff, dX));
        return mm(t, d.gflag, 1, 0, Mw, Nw, Mx, dY, act, 1.0f, dW);
    }
    BMB_CUDA(cudaEventRecord(t->ev_fork, t->st));
    BMB_CUDA(cudaStreamWaitEvent(t->st_dw, t->ev_fork, 0));
    BMB_TRY(mm(t, d.gflag | BMB_GEMM_HALF_SMS, 1, 0, Mw, Nw, Mx, dY, act, 1.0f, dW, nullptr, t->st_dw));
    BMB_TRY(dx(t, d, xflags | BMB_GEMM_HALF_SMS, Mx, Nx, Kx, dY, id, woff, dX));
    BMB_CUDA(cudaEventRecord(t->ev_join, t->st_dw));
    BMB_CUDA(cudaStreamWaitEvent(t->st, t->ev_join, 0));
    return BMB_OK;
}

// Whether `st` is being captured into a graph.
bool stream_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) { cudaGetLastError(); return false; }
    return cs != cudaStreamCaptureStatusNone;
}

int bwd_head(bmb_trainer *t, const Dims &d) {
    const int N = d.N, C = d.C, L = d.L, Vp = d.Vp;
    float *G = d.G;
    // Column sums are deferred to one launch at the end of backward when the whole step is one piece (nothing
    // reads a gradient before the embedding's backward is done).  The job list is recorded during the first such
    // pass, which is never a captured one, and uploaded then.
    t->col_active = t->defer_colsums && t->col.arena && t->pieces.size() <= 1 && t->unit_span_whole &&
                    (t->col_jobs_uploaded || !stream_capturing(t->st));
    if (t->col_active) {
        t->col.used = 0; t->col.njobs = 0; t->col.max_cols = 0;
        t->col.record = !t->col_jobs_uploaded;
        set_column_add_collector(&t->col);
    }
    BMB_CUDA(cudaMemsetAsync(G, 0, t->num_params * sizeof(float), t->st));
    BMB_TRY(dx(t, d, d.wflag, N, C, Vp, t->dlogits, P_WTE, 0, t->dlnf));
    BMB_TRY(mm(t, d.gflag, 1, 0, Vp, C, N, t->dlogits, t->lnf, 1.0f, G + t->poff[P_WTE]));
    float *last_res = t->residual3 + (size_t)(L - 1) * d.BTC;
    BMB_CUDA(cudaMemsetAsync(t->dres, 0, d.BTC * sizeof(float), t->st));
    // Each layernorm backward also sums the columns of the residual-stream gradient it leaves behind:
    // that is the bias gradient of the projection feeding that point of the stream.
    return bmb_layernorm_backward_colsum(t->dres, G + t->poff[P_LNFW], G + t->poff[P_LNFB],
                                         G + t->poff[P_FPB] + (size_t)(L - 1) * C, t->dlnf, last_res,
                                         d.P + t->poff[P_LNFW], t->lnf_mean, t->lnf_rstd, N, C);
}

int bwd_layer(bmb_trainer *t, const Dims &d, int l) {
    const bmb_train_config &c = t->c;
    const int N = d.N, C = d.C, NH = d.NH, B = d.B, T = d.T;
    const size_t BTC = d.BTC, BT = d.BT;
    const float *P = d.P;
    float *G = d.G;
    const int wflag = d.wflag;
    const bool fz = d.fz;
    float *residual = (l == 0) ? t->encoded : t->residual3 + (size_t)(l - 1) * BTC;
    float *ln1 = t->ln1 + l * BTC, *qkv = t->qkv + l * d.BT3C, *atty = t->atty + l * BTC;
    float *res2 = t->residual2 + l * BTC, *ln2 = t->ln2 + l * BTC;
    float *fch = t->fch + l * d.BT4C, *fchg = t->fch_gelu + l * d.BT4C;
    const size_t lC = (size_t)l * C;

    BMB_TRY(dx_dw(t, d, wflag, N, 4 * C, C, t->dres, P_FPW, (size_t)l * C * 4 * C, t->dfch_gelu,
                  C, 4 * C, fchg, G + t->poff[P_FPW] + (size_t)l * C * 4 * C));
    BMB_TRY(bmb_gelu_backward_colsum(t->dfch, G + t->poff[P_FCB] + 4 * lC, fch, t->dfch_gelu, N, 4 * C));
    BMB_TRY(dx_dw(t, d, wflag, N, C, 4 * C, t->dfch, P_FCW, (size_t)l * 4 * C * C, t->dln2,
                  4 * C, C, ln2, G + t->poff[P_FCW] + (size_t)l * 4 * C * C));
    BMB_TRY(bmb_layernorm_backward_colsum(t->dres, G + t->poff[P_LN2W] + lC, G + t->poff[P_LN2B] + lC,
                                          G + t->poff[P_APB] + lC, t->dln2, res2,
                                          P + t->poff[P_LN2W] + lC, t->ln2_mean + l * BT, t->ln2_rstd + l * BT, N, C));
    BMB_TRY(dx_dw(t, d, wflag | (fz ? BMB_GEMM_C_ROUNDED : 0), N, C, C, t->dres, P_APW, (size_t)l * C * C, t->datty,
                  C, C, atty, G + t->poff[P_APW] + (size_t)l * C * C));
    // the tensor-core attention backward leaves the qkv bias gradient (column sums of dqkv) from its own epilogue
    const bool bias_in_attention = c.use_flash && fz && attn_cfg(c) == 2 && t->qkv_bias_in_attention;
    if (c.use_flash && fz && attn_cfg(c) == 2)
        BMB_TRY(flash_backward_tc(t->dqkv, t->dsum, t->datty, qkv, atty, t->lse + l * d.lse_sz, B, T, C, NH, true, t->st,
                                  bias_in_attention ? G + t->poff[P_QKVB] + 3 * lC : nullptr));
    else if (c.use_flash)
        BMB_TRY(bmb_flash_attention_backward_cfg(attn_cfg(c), t->dqkv, t->dsum, t->datty, qkv, atty, t->lse + l * d.lse_sz, B, T, C, NH));
    else
        BMB_TRY(bmb_attention_backward(t->dqkv, t->dqkvr, t->datt, t->datt, t->datty, t->qkvr + l * d.qkvr_sz,
                                       t->att + l * d.att_sz, B, T, C, NH));
    BMB_TRY(dx_dw(t, d, wflag, N, C, 3 * C, t->dqkv, P_QKVW, (size_t)l * 3 * C * C, t->dln1,
                  3 * C, C, ln1, G + t->poff[P_QKVW] + (size_t)l * 3 * C * C));
    if (!bias_in_attention) BMB_TRY(bmb_bias_backward(G + t->poff[P_QKVB] + 3 * lC, t->dqkv, N, 3 * C));
    return bmb_layernorm_backward_colsum(t->dres, G + t->poff[P_LN1W] + lC, G + t->poff[P_LN1B] + lC,
                                         l > 0 ? G + t->poff[P_FPB] + lC - C : nullptr, t->dln1, residual,
                                         P + t->poff[P_LN1W] + lC, t->ln1_mean + l * BT, t->ln1_rstd + l * BT, N, C);
}

int bwd_embed(bmb_trainer *t, const Dims &d) {
    BMB_TRY(bmb_encoder_backward(d.G + t->poff[P_WTE], d.G + t->poff[P_WPE], t->dres, t->d_tokens, d.B, d.T, d.C));
    if (!t->col_active) return BMB_OK;
    set_column_add_collector(nullptr);
    t->col_active = false;
    if (!t->col_jobs_uploaded) {
        BMB_CUDA(cudaMemcpyAsync(t->col_jobs_dev, t->col_jobs_host.data(), (size_t)t->col.njobs * sizeof(ColumnAddJob),
                                 cudaMemcpyHostToDevice, t->st));
        BMB_CUDA(cudaStreamSynchronize(t->st));          // (once per trainer: the host list may not change under the copy)
        t->col_jobs_uploaded = true;
        t->col_njobs = t->col.njobs;
        t->col_max_cols = t->col.max_cols;
    }
    return launch_column_add_jobs(t->col_jobs_dev, t->col_njobs, t->col_max_cols, t->st);
}

// The units of a pass, in execution order: 0 embedding; 1 .. L the layers; L+1 the head with the loss;
// L+2 the head's backward; L+3 .. 2L+2 the layers' backward (last layer first); 2L+3 the embedding's backward.
int num_units(const bmb_trainer *t) { return 2 * t->c.n_layer + 4; }
int run_units(bmb_trainer *t, int u0, int u1, bool with_loss = true) {
    const Dims d = dims_of(t);
    const int L = d.L;
    set_emit_rounded(d.fz);
    t->unit_span_whole = (u0 <= L + 2 && u1 == num_units(t));      // head backward .. embedding backward in this call
    int rc = BMB_OK;
    for (int u = u0; u < u1 && rc == BMB_OK; ++u) {
        if (u == 0) rc = fwd_embed(t, d);
        else if (u <= L) rc = fwd_layer(t, d, u - 1);
        else if (u == L + 1) rc = fwd_head(t, d, with_loss);
        else if (u == L + 2) rc = bwd_head(t, d);
        else if (u <= 2 * L + 2) rc = bwd_layer(t, d, 2 * L + 2 - u);
        else rc = bwd_embed(t, d);
    }
    if (t->col_active) { set_column_add_collector(nullptr); t->col_active = false; }    // (only after a failure part-way)
    return rc;
}
int forward(bmb_trainer *t, bool with_loss = true) { return run_units(t, 0, t->c.n_layer + 2, with_loss); }
int backward(bmb_trainer *t) { return run_units(t, t->c.n_layer + 2, num_units(t)); }

void drop_graphs(bmb_trainer *t) {
    for (auto &pc : t->pieces) {
        if (pc.exec) cudaGraphExecDestroy(pc.exec);
        pc.exec = nullptr;
        pc.launches = 0;
    }
}

// The chunks of the parameter space (see bmb_trainer) as range lists, and the pieces of a step.
// Without the fused exchange the step is one piece.  With it (overlap 2):
//   [embedding, layer 0] needs A | [layers 1 .. c2-1] needs B | [layers c2 .. L-1, head, head backward,
//   backward of layers L-1 .. c2] needs C, finishes C | [backward of layers c2-1 .. 1] finishes B |
//   [backward of layer 0, embedding backward] finishes A;
// with overlap 1 the first three are one piece that needs all chunks.
// Every gradient of a layer is written during that layer's backward or the unit before it (the bias of its
// second MLP projection comes out of the following layernorm's backward), so a chunk is final when the last of
// its layers is done.
struct StepPlan {
    DpRangeList chunk[bmb_trainer::NCHUNK];
    int split = 0;
    int npieces = 0;
    struct { int u0, u1, needs, reduces; } piece[5];
};
void make_plan(const bmb_train_config &c, int overlap, StepPlan &pl) {
    const bool chunks = overlap > 0;
    size_t psize[NPT], poff[NPT], total = 0;
    param_sizes(psize, c);
    for (int i = 0; i < NPT; ++i) { poff[i] = total; total += psize[i]; }
    const int L = c.n_layer, U = 2 * L + 4;
    for (int k = 0; k < bmb_trainer::NCHUNK; ++k) pl.chunk[k].n = 0;
    pl.npieces = 0;
    auto add = [&](int k, size_t off, size_t len) {
        if (!len) return;
        DpRangeList &rl = pl.chunk[k];
        rl.off[rl.n] = off; rl.len[rl.n] = len; ++rl.n;
    };
    auto piece = [&](int u0, int u1, int needs, int reduces) {
        if (u0 >= u1) return;
        pl.piece[pl.npieces].u0 = u0; pl.piece[pl.npieces].u1 = u1;
        pl.piece[pl.npieces].needs = needs; pl.piece[pl.npieces].reduces = reduces;
        ++pl.npieces;
    };
    if (!chunks || L < 2) {               // (a single layer also applies the final layernorm: nothing to split)
        add(0, 0, total);
        piece(0, U, 0, 0);                 // (needs / reduces are read by the fused exchange only)
        pl.split = L;
        return;
    }
    const int c2 = 1 + (L - 1) / 2;
    pl.split = c2;
    add(0, poff[P_WTE], psize[P_WTE]);
    add(0, poff[P_WPE], psize[P_WPE]);
    for (int id = P_LN1W; id <= P_FPB; ++id) {                 // the twelve tensors stacked over the layers
        const size_t per = psize[id] / L;
        add(0, poff[id], per);
        add(1, poff[id] + per, per * (size_t)(c2 - 1));
        add(2, poff[id] + per * (size_t)c2, per * (size_t)(L - c2));
    }
    add(2, poff[P_LNFW], psize[P_LNFW]);
    add(2, poff[P_LNFB], psize[P_LNFB]);
    // forward units: 0 embedding, 1 + l layer l, L + 1 head; backward: L + 2 head, 2L + 2 - l layer l, 2L + 3 embedding
    if (overlap >= 2) {
        piece(0, 2, 0, -1);
        piece(2, 1 + c2, 1, -1);
        piece(1 + c2, 2 * L + 3 - c2, 2, 2);
    } else {
        piece(0, 2 * L + 3 - c2, 2, 2);    // waits for the last chunk's update, i.e. for all of them (one stream)
    }
    piece(2 * L + 3 - c2, 2 * L + 2, -1, 1);
    piece(2 * L + 2, U, -1, 0);
}

void plan_pieces(bmb_trainer *t) {
    drop_graphs(t);
    t->pieces.clear();
    StepPlan pl;
    make_plan(t->c, t->dp ? t->overlap : 0, pl);
    for (int k = 0; k < bmb_trainer::NCHUNK; ++k) t->chunk[k] = pl.chunk[k];
    t->chunk_split = pl.split;
    for (int i = 0; i < pl.npieces; ++i) {
        bmb_trainer::Piece pc;
        pc.u0 = pl.piece[i].u0; pc.u1 = pl.piece[i].u1; pc.needs = pl.piece[i].needs; pc.reduces = pl.piece[i].reduces;
        t->pieces.push_back(pc);
    }
}

// One piece on t->st: replay of its captured graph, or eager launches (`eager`: first pass, GEMM event
// profiling on, graphs switched off, or a capture failed).
int run_piece(bmb_trainer *t, bmb_trainer::Piece &pc, bool eager) {
    if (eager || t->graph_failed) return run_units(t, pc.u0, pc.u1);
    if (!pc.exec) {
        const long long before = launches_total();
        const unsigned long long gen_before = scratch_generation();
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(t->st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();
            t->graph_failed = true;
            return run_units(t, pc.u0, pc.u1);
        }
        const int rc = run_units(t, pc.u0, pc.u1);
        const cudaError_t e = cudaStreamEndCapture(t->st, &graph);
        if (rc != BMB_OK || e != cudaSuccess || !graph || gen_before != scratch_generation() ||
            cudaGraphInstantiate(&pc.exec, graph, 0) != cudaSuccess) {
            // nothing ran during the capture: fall back to eager launches for good and run this piece now
            cudaGetLastError();
            if (graph) cudaGraphDestroy(graph);
            pc.exec = nullptr;
            t->graph_failed = true;
            return run_units(t, pc.u0, pc.u1);
        }
        cudaGraphDestroy(graph);
        t->graph_scratch_gen = gen_before;
        pc.launches = launches_total() - before;
        count_launch((int)-pc.launches);        // counted again at every replay, this first one included
    }
    BMB_CUDA(cudaGraphLaunch(pc.exec, t->st));
    count_launch((int)pc.launches);
    return BMB_OK;
}

// Whether this step's pieces run eagerly.  The captured launches carry the addresses of the library's
// per-device scratch: if another caller on this device has made that scratch grow since (the old block was
// freed), the graphs are dropped and built again -- one eager pass to size the scratch, then new captures.
bool step_is_eager(bmb_trainer *t) {
    if (!t->use_graph || t->graph_failed || t->prof) return true;
    bool any = false;
    for (auto &pc : t->pieces) any = any || pc.exec;
    if (any && t->graph_scratch_gen != scratch_generation()) {
        drop_graphs(t);
        t->eager_passes = 0;
        any = false;
    }
    if (!any && t->eager_passes < 1) {
        t->eager_passes++;
        return true;
    }
    return false;
}

// The tensor-core kernels report a bounded wait that ran out through a host-mapped word; the eager
// entry points look at it before every launch, a replayed graph does not, so the trainer looks after
// it has synchronised.
int check_kernel_status() {
    int *dev = nullptr;
    volatile int *host = nullptr;
    BMB_TRY(tc::status_word(&dev, &host));
    if (*host != 0) return fail(BMB_E_TIMEOUT, "a tensor-core kernel gave up waiting on a barrier (status %d)", *host);
    return BMB_OK;
}

int refresh_shadow(bmb_trainer *t) {
    if (!t->shadow) return BMB_OK;
    return bmb_round_tf32(t->shadow, t->params, t->num_params, t->st);
}

int trainer_build(bmb_trainer *t, const bmb_train_config &c, unsigned seed);

}  // namespace

extern "C" {

int bmb_trainer_create(bmb_trainer **out, const bmb_train_config *cfg, unsigned seed) {
    if (!out || !cfg) return fail(BMB_E_ARG, "trainer_create: null argument");
    const bmb_train_config &c = *cfg;
    if (c.n_layer < 1 || c.n_head < 1 || c.n_embd < 4 || c.n_embd % c.n_head || c.n_embd % 4 ||
        c.B < 1 || c.T < 1 || c.T > c.max_seq_len || c.vocab_size < 1 || c.padded_vocab < c.vocab_size ||
        c.padded_vocab % 4)
        return fail(BMB_E_ARG, "trainer_create: inconsistent configuration");
    if (c.math < BMB_MATH_FP32 || c.math > BMB_MATH_BF16) return fail(BMB_E_ARG, "trainer_create: math %d", c.math);
    const int hs = c.n_embd / c.n_head;
    if (c.use_flash && hs != 32 && hs != 64 && hs != 128)
        return fail(BMB_E_UNSUPPORTED, "trainer_create: fused attention needs head size 32, 64 or 128 (got %d)", hs);

    bmb_trainer *t = new bmb_trainer();
    const int rc = trainer_build(t, c, seed);
    if (rc != BMB_OK) {
        // a failed allocation part-way (a busy device) must not strand the gigabytes already taken
        bmb_trainer_destroy(t);
        return rc;
    }
    *out = t;
    return BMB_OK;
}

}  // extern "C"

namespace {
int trainer_build(bmb_trainer *t, const bmb_train_config &c, unsigned seed) {
    t->c = c;
    if (const char *g = getenv("BMB_TRAINER_GRAPH")) t->use_graph = atoi(g) != 0;
    BMB_CUDA(cudaGetDevice(&t->dev));
    BMB_CUDA(cudaStreamCreateWithFlags(&t->st, cudaStreamNonBlocking));
    BMB_CUDA(cudaStreamCreateWithFlags(&t->st_dw, cudaStreamNonBlocking));
    BMB_CUDA(cudaEventCreateWithFlags(&t->ev_fork, cudaEventDisableTiming));
    BMB_CUDA(cudaEventCreateWithFlags(&t->ev_join, cudaEventDisableTiming));
    if (const char *e = getenv("BMB_TRAINER_SIDE_BY_SIDE")) t->side_by_side = atoi(e) != 0;
    if (const char *e = getenv("BMB_TRAINER_OVERLAP")) { const int v = atoi(e); t->overlap = v < 0 ? 0 : (v > 2 ? 2 : v); }
    if (const char *e = getenv("BMB_TRAINER_FUSE_GELU")) t->fuse_gelu = atoi(e);
    if (const char *e = getenv("BMB_TRAINER_QKV_BIAS_IN_ATTENTION")) t->qkv_bias_in_attention = atoi(e) != 0;
    if (const char *e = getenv("BMB_TRAINER_TIMELINE")) t->tl_step = atoi(e);
    if (const char *e = getenv("BMB_TRAINER_DEFER_COLSUMS")) t->defer_colsums = atoi(e) != 0;
    {
        // The exchange stream outranks the main stream: its small kernels (barrier collectives, piece-wise reduce
        // and update) must get the SMs that free up between two of the main stream's GPU-filling kernels, or they
        // queue behind a whole piece of the step and nothing overlaps.
        int lo = 0, hi = 0;
        BMB_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        BMB_CUDA(cudaStreamCreateWithPriority(&t->st_x, cudaStreamNonBlocking, hi));
    }
    for (int c = 0; c < bmb_trainer::NCHUNK; ++c) {
        BMB_CUDA(cudaEventCreateWithFlags(&t->ev_seg[c], cudaEventDisableTiming));
        BMB_CUDA(cudaEventCreateWithFlags(&t->ev_upd[c], cudaEventDisableTiming));
    }
    param_sizes(t->psize, c);
    t->num_params = 0;
    for (int i = 0; i < NPT; ++i) { t->poff[i] = t->num_params; t->num_params += t->psize[i]; }
    const size_t pb = t->num_params * sizeof(float);
    BMB_CUDA(cudaMalloc(&t->params, pb));
    BMB_CUDA(cudaMalloc(&t->grads, pb));
    BMB_CUDA(cudaMalloc(&t->m, pb));
    BMB_CUDA(cudaMalloc(&t->v, pb));
    BMB_CUDA(cudaMemset(t->m, 0, pb));
    BMB_CUDA(cudaMemset(t->v, 0, pb));
    BMB_CUDA(cudaMemset(t->grads, 0, pb));
    if (c.math != BMB_MATH_FP32) BMB_CUDA(cudaMalloc(&t->shadow, pb));

    const size_t B = c.B, T = c.T, C = c.n_embd, L = c.n_layer, NH = c.n_head, Vp = c.padded_vocab;
    const size_t BT = B * T, BTC = BT * C, BT3C = 3 * BTC, BT4C = 4 * BTC;
    const size_t qkvr = 4 * BTC, att = B * NH * T * T, lse = B * NH * T;
    // Every tensor starts on a 256-byte boundary: the first call sizes the
    // arena (base = nullptr), the second hands out the pointers.
    auto layout_fwd = [&](float *base) -> size_t {
        size_t off = 0;
        auto take = [&](size_t n) { float *r = base + off; off += (n + 63) & ~(size_t)63; return r; };
        t->encoded = take(BTC);
        t->ln1 = take(BTC * L); t->ln1_mean = take(BT * L); t->ln1_rstd = take(BT * L);
        t->qkv = take(BT3C * L);
        t->qkvr = c.use_flash ? nullptr : take(qkvr * L);
        t->att = c.use_flash ? nullptr : take(att * L);
        t->lse = c.use_flash ? take(lse * L) : nullptr;
        t->atty = take(BTC * L); t->attproj = take(BTC * L); t->residual2 = take(BTC * L);
        t->ln2 = take(BTC * L); t->ln2_mean = take(BT * L); t->ln2_rstd = take(BT * L);
        t->fch = take(BT4C * L); t->fch_gelu = take(BT4C * L); t->fcproj = take(BTC * L);
        t->residual3 = take(BTC * L);
        t->lnf = take(BTC); t->lnf_mean = take(BT); t->lnf_rstd = take(BT);
        t->logits = take(BT * Vp); t->probs = nullptr; t->losses = take(BT);
        return off;
    };
    auto layout_bwd = [&](float *base) -> size_t {
        size_t off = 0;
        auto take = [&](size_t n) { float *r = base + off; off += (n + 63) & ~(size_t)63; return r; };
        t->dres = take(BTC); t->dln1 = take(BTC); t->dln2 = take(BTC); t->datty = take(BTC);
        t->dqkv = take(BT3C);
        t->dqkvr = c.use_flash ? nullptr : take(qkvr);
        t->datt = c.use_flash ? nullptr : take(att);
        t->dsum = c.use_flash ? take(lse) : nullptr;
        t->dfch = take(BT4C); t->dfch_gelu = take(BT4C);
        t->dlogits = take(BT * Vp); t->dlnf = take(BTC);
        return off;
    };
    t->num_acts = layout_fwd(nullptr);
    BMB_CUDA(cudaMalloc(&t->acts, t->num_acts * sizeof(float)));
    layout_fwd(t->acts);
    t->num_bacts = layout_bwd(nullptr);
    BMB_CUDA(cudaMalloc(&t->bacts, t->num_bacts * sizeof(float)));
    layout_bwd(t->bacts);

    if (t->defer_colsums) {
        // partial rows of one backward pass: per layer two layernorm backwards (3C columns), the GELU backward (4C) and
        // the qkv bias (3C), each at most 4 rows per SM; the final layernorm; a job each (+ a few spare)
        const size_t rows = 4 * (size_t)sm_count();
        t->col.cap = ((size_t)L * (2 * 3 * C + 4 * C + 3 * C) + 3 * C) * rows + 64 * (4 * L + 8);
        t->col.max_jobs = 4 * (int)L + 8;
        BMB_CUDA(cudaMalloc(&t->col.arena, t->col.cap * sizeof(float)));
        BMB_CUDA(cudaMalloc(&t->col_jobs_dev, t->col.max_jobs * sizeof(ColumnAddJob)));
        t->col_jobs_host.resize(t->col.max_jobs);
        t->col.jobs = t->col_jobs_host.data();
    }
    BMB_CUDA(cudaMalloc(&t->d_tokens, BT * sizeof(int)));
    BMB_CUDA(cudaMalloc(&t->d_targets, BT * sizeof(int)));
    BMB_CUDA(cudaMemset(t->d_tokens, 0, BT * sizeof(int)));
    BMB_CUDA(cudaMemset(t->d_targets, 0, BT * sizeof(int)));
    BMB_CUDA(cudaMalloc(&t->d_loss, sizeof(float)));
    BMB_CUDA(cudaMalloc(&t->d_sumsq, sizeof(double)));
    BMB_CUDA(cudaMemset(t->d_loss, 0, sizeof(float)));
    BMB_CUDA(cudaMalloc(&t->d_token, sizeof(float)));
    BMB_CUDA(cudaMemset(t->d_token, 0, sizeof(float)));

    // GPT-2 initialisation with the reference's draw order (src/gpt.cu:189-218):
    // one mt19937 stream; a fresh normal_distribution per tensor; N(0, 0.02)
    // except the two residual projections at 0.02/sqrt(2L); gains 1, biases 0.
    {
        std::vector<float> h(t->num_params, 0.0f);
        std::mt19937 rng(seed);
        const float resid = 0.02f / sqrtf(2.0f * c.n_layer);
        auto fill = [&](int i, float sd) {
            std::normal_distribution<float> d(0.0f, sd);
            float *dst = h.data() + t->poff[i];
            for (size_t k = 0; k < t->psize[i]; ++k) dst[k] = d(rng);
        };
        auto ones = [&](int i) {
            float *dst = h.data() + t->poff[i];
            for (size_t k = 0; k < t->psize[i]; ++k) dst[k] = 1.0f;
        };
        fill(P_WTE, 0.02f); fill(P_WPE, 0.02f); ones(P_LN1W);
        fill(P_QKVW, 0.02f); fill(P_APW, resid); ones(P_LN2W);
        fill(P_FCW, 0.02f); fill(P_FPW, resid); ones(P_LNFW);
        BMB_CUDA(cudaMemcpy(t->params, h.data(), pb, cudaMemcpyHostToDevice));
    }
    {
        Scope sc(t);
        BMB_TRY(refresh_shadow(t));
        BMB_CUDA(cudaStreamSynchronize(t->st));
    }
    return BMB_OK;
}
}  // namespace

extern "C" {

int bmb_trainer_destroy(bmb_trainer *t) {
    if (!t) return BMB_OK;
    cudaSetDevice(t->dev);
    if (t->st) cudaStreamSynchronize(t->st);
    if (t->st_x) cudaStreamSynchronize(t->st_x);
    for (cudaEvent_t e : t->ev) cudaEventDestroy(e);
    drop_graphs(t);
    for (int c = 0; c < bmb_trainer::NCHUNK; ++c) {
        if (t->ev_seg[c]) cudaEventDestroy(t->ev_seg[c]);
        if (t->ev_upd[c]) cudaEventDestroy(t->ev_upd[c]);
    }
    if (t->st_x) cudaStreamDestroy(t->st_x);
    cudaFree(t->params); cudaFree(t->grads); cudaFree(t->m); cudaFree(t->v);
    if (t->shadow) cudaFree(t->shadow);
    cudaFree(t->acts); cudaFree(t->bacts); cudaFree(t->d_tokens); cudaFree(t->d_targets);
    cudaFree(t->d_loss); cudaFree(t->d_sumsq); cudaFree(t->d_token);
    if (t->gen_probs) cudaFree(t->gen_probs);
    if (t->col.arena) cudaFree(t->col.arena);
    if (t->col_jobs_dev) cudaFree(t->col_jobs_dev);
    dp_fused_destroy(t->dp);
    if (t->ev_fork) cudaEventDestroy(t->ev_fork);
    if (t->ev_join) cudaEventDestroy(t->ev_join);
    if (t->st_dw) cudaStreamDestroy(t->st_dw);
    if (t->st) cudaStreamDestroy(t->st);
    delete t;
    return BMB_OK;
}

int bmb_trainer_attach_comm(bmb_trainer *t, bmb_comm *c, int nranks) {
    if (!t || nranks < 1) return fail(BMB_E_ARG, "trainer_attach_comm: bad argument");
    t->comm = c;
    t->nranks = nranks;
    return BMB_OK;
}

int bmb_trainer_ipc_export(bmb_trainer *t, void *record192) {
    if (!t || !record192) return fail(BMB_E_ARG, "trainer_ipc_export: null argument");
    Scope sc(t);
    return dp_fused_export(t->grads, t->params, t->shadow, record192);
}

int bmb_trainer_attach_peers(bmb_trainer *t, int rank, int nranks, const void *records) {
    if (!t) return fail(BMB_E_ARG, "trainer_attach_peers: null handle");
    if (records && (!t->comm || t->nranks != nranks))
        return fail(BMB_E_ARG, "trainer_attach_peers: attach the communicator of %d ranks first", nranks);
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    BMB_CUDA(cudaStreamSynchronize(t->st_x));
    dp_fused_destroy(t->dp);
    t->dp = nullptr;
    int rc = BMB_OK;
    if (records)                          // (null: detach, back to the communicator's all-reduce)
        rc = dp_fused_create(&t->dp, rank, nranks, t->num_params, t->grads, t->params, t->shadow, records);
    plan_pieces(t);                       // the step's pieces follow the exchange
    return rc;
}

int bmb_trainer_step_plan(const bmb_train_config *cfg, int overlapped, unsigned long long *ranges, int *nranges, int *pieces,
                          int *npieces) {
    if (!cfg || !ranges || !nranges || !pieces || !npieces || cfg->n_layer < 1) return fail(BMB_E_ARG, "trainer_step_plan: bad argument");
    StepPlan pl;
    make_plan(*cfg, overlapped < 0 ? 0 : (overlapped > 2 ? 2 : overlapped), pl);
    for (int k = 0; k < bmb_trainer::NCHUNK; ++k) {
        nranges[k] = pl.chunk[k].n;
        for (int q = 0; q < DP_MAX_RANGES; ++q) {
            ranges[(k * DP_MAX_RANGES + q) * 2 + 0] = q < pl.chunk[k].n ? pl.chunk[k].off[q] : 0;
            ranges[(k * DP_MAX_RANGES + q) * 2 + 1] = q < pl.chunk[k].n ? pl.chunk[k].len[q] : 0;
        }
    }
    *npieces = pl.npieces;
    for (int i = 0; i < pl.npieces; ++i) {
        pieces[4 * i + 0] = pl.piece[i].u0; pieces[4 * i + 1] = pl.piece[i].u1;
        pieces[4 * i + 2] = pl.piece[i].needs; pieces[4 * i + 3] = pl.piece[i].reduces;
    }
    return BMB_OK;
}

size_t bmb_trainer_num_params(const bmb_trainer *t) { return t ? t->num_params : 0; }

int bmb_trainer_get_params(bmb_trainer *t, float *host_out) {
    if (!t || !host_out) return fail(BMB_E_ARG, "trainer_get_params: null argument");
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    BMB_CUDA(cudaMemcpy(host_out, t->params, t->num_params * sizeof(float), cudaMemcpyDeviceToHost));
    return BMB_OK;
}
int bmb_trainer_set_params(bmb_trainer *t, const float *host_in) {
    if (!t || !host_in) return fail(BMB_E_ARG, "trainer_set_params: null argument");
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    BMB_CUDA(cudaMemcpy(t->params, host_in, t->num_params * sizeof(float), cudaMemcpyHostToDevice));
    BMB_TRY(refresh_shadow(t));
    BMB_CUDA(cudaStreamSynchronize(t->st));
    return BMB_OK;
}
int bmb_trainer_get_grads(bmb_trainer *t, float *host_out) {
    if (!t || !host_out) return fail(BMB_E_ARG, "trainer_get_grads: null argument");
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    BMB_CUDA(cudaMemcpy(host_out, t->grads, t->num_params * sizeof(float), cudaMemcpyDeviceToHost));
    return BMB_OK;
}

int bmb_trainer_upload(bmb_trainer *t, const int *host_tokens, const int *host_targets) {
    if (!t || !host_tokens || !host_targets) return fail(BMB_E_ARG, "trainer_upload: null argument");
    Scope sc(t, /*join=*/false);          // token buffers only: nothing the exchange stream touches
    const size_t n = (size_t)t->c.B * t->c.T * sizeof(int);
    // cudaMemcpyDefault: the source may also be a batch already staged in device memory
    BMB_CUDA(cudaMemcpyAsync(t->d_tokens, host_tokens, n, cudaMemcpyDefault, t->st));
    BMB_CUDA(cudaMemcpyAsync(t->d_targets, host_targets, n, cudaMemcpyDefault, t->st));
    return BMB_OK;
}

int bmb_trainer_forward_backward(bmb_trainer *t) {
    if (!t) return fail(BMB_E_ARG, "trainer: null handle");
    Scope sc(t);
    return run_units(t, 0, num_units(t));
}

namespace {
void tl_mark(bmb_trainer *t, int step, cudaStream_t st, const char *what, int idx = -1) {
    if (!t->tl_step || (step != t->tl_step && step != t->tl_step + 1)) return;
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    cudaEventRecord(e, st);
    char name[64];
    if (idx >= 0) snprintf(name, sizeof name, "step %d %s %d", step, what, idx);
    else snprintf(name, sizeof name, "step %d %s", step, what);
    t->tl.emplace_back(name, e);
}
void tl_flush(bmb_trainer *t, int step) {
    if (!t->tl_step || step != t->tl_step + 2 || t->tl.empty()) return;
    cudaDeviceSynchronize();
    for (auto &m : t->tl) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, t->tl.front().second, m.second);
        fprintf(stderr, "[timeline dev %d] %8.3f ms  %s\n", t->dev, ms, m.first.c_str());
    }
    for (auto &m : t->tl) cudaEventDestroy(m.second);
    t->tl.clear();
}
}  // namespace

int bmb_trainer_step(bmb_trainer *t, float lr, int step) {
    if (!t || step < 1) return fail(BMB_E_ARG, "trainer_step: bad argument");
    Scope sc(t, /*join=*/false);
    if (t->pieces.empty()) plan_pieces(t);
    tl_flush(t, step);
    const bool eager = step_is_eager(t);
    tl_mark(t, step, t->st, "start (main)");
    if (!t->dp) {
        for (auto &pc : t->pieces) BMB_TRY(run_piece(t, pc, eager));
        if (t->comm && t->nranks > 1) BMB_TRY(bmb_comm_allreduce(t->comm, t->grads, t->num_params, t->st));
        BMB_TRY(bmb_grad_sumsq_device(t->grads, t->num_params, t->d_sumsq));
        BMB_TRY(bmb_adamw_update_clipped(t->params, t->grads, t->m, t->v, t->num_params, lr, t->c.beta1, t->c.beta2,
                                         t->c.eps, t->c.weight_decay, step, t->d_sumsq, t->c.grad_clip,
                                         (float)t->nranks, t->shadow));
        return BMB_OK;
    }
    // Fused exchange.  Everything that crosses GPUs runs on the exchange stream, ordered across ranks by small
    // collectives on that stream: no rank reads a chunk's gradients before every rank has finished them, none
    // updates before every piece of the gradient is summed (the norm), and none reads a chunk's new parameters
    // before every rank has stored its pieces of them.  The main stream only waits where it needs a result.
    for (auto &pc : t->pieces) {
        if (pc.needs >= 0 && t->upd_pending[pc.needs]) {
            BMB_CUDA(cudaStreamWaitEvent(t->st, t->ev_upd[pc.needs], 0));
            t->upd_pending[pc.needs] = false;
        }
        tl_mark(t, step, t->st, "piece waits done, starts (main), first unit", pc.u0);
        BMB_TRY(run_piece(t, pc, eager));
        tl_mark(t, step, t->st, "piece ends (main), end unit", pc.u1);
        const int c = pc.reduces;
        if (c < 0 || t->chunk[c].n == 0) continue;
        BMB_CUDA(cudaEventRecord(t->ev_seg[c], t->st));
        BMB_CUDA(cudaStreamWaitEvent(t->st_x, t->ev_seg[c], 0));
        BMB_TRY(bmb_comm_allreduce(t->comm, t->d_token, 1, t->st_x));
        tl_mark(t, step, t->st_x, "barrier before reduce done (exchange), chunk", c);
        // the last piece's chunk is reduced with the main stream waiting; the others while backward goes on
        BMB_TRY(dp_fused_reduce_ranges(t->dp, t->chunk[c], t->grads, c, /*alone=*/&pc == &t->pieces.back(), t->st_x));
        tl_mark(t, step, t->st_x, "reduce done (exchange), chunk", c);
    }
    BMB_TRY(dp_fused_sumsq(t->dp, t->d_sumsq, t->st_x));
    BMB_TRY(bmb_comm_allreduce_f64(t->comm, t->d_sumsq, 1, t->st_x));
    tl_mark(t, step, t->st_x, "norm done (exchange)");
    if (t->overlap < 2) {
        // All chunks updated with the main stream waiting: every update may fill the GPU, one barrier for all, then
        // the rounded copies; the next step's first piece waits for the last event.
        for (int c = 0; c < bmb_trainer::NCHUNK; ++c) {
            if (t->chunk[c].n == 0) continue;
            BMB_TRY(dp_fused_update_ranges(t->dp, t->chunk[c], t->grads, t->m, t->v, lr, t->c.beta1, t->c.beta2, t->c.eps,
                                           t->c.weight_decay, step, t->d_sumsq, t->c.grad_clip, /*alone=*/true, t->st_x));
        }
        tl_mark(t, step, t->st_x, "updates + broadcasts done (exchange)");
        BMB_TRY(bmb_comm_allreduce(t->comm, t->d_token, 1, t->st_x));
        for (int c = 0; c < bmb_trainer::NCHUNK; ++c) {
            if (t->chunk[c].n == 0) continue;
            if (t->shadow) BMB_TRY(dp_round_ranges(t->chunk[c], t->shadow, t->params, /*alone=*/true, t->st_x));
            BMB_CUDA(cudaEventRecord(t->ev_upd[c], t->st_x));
            t->upd_pending[c] = true;
        }
        tl_mark(t, step, t->st_x, "rounded copies done (exchange)");
        return BMB_OK;
    }
    for (int c = 0; c < bmb_trainer::NCHUNK; ++c) {           // in the order the next forward needs them
        if (t->chunk[c].n == 0) continue;
        // the first chunk is updated with the main stream waiting for it; the others while the next forward has begun
        const bool alone = (c == 0);
        BMB_TRY(dp_fused_update_ranges(t->dp, t->chunk[c], t->grads, t->m, t->v, lr, t->c.beta1, t->c.beta2, t->c.eps,
                                       t->c.weight_decay, step, t->d_sumsq, t->c.grad_clip, alone, t->st_x));
        tl_mark(t, step, t->st_x, "update + broadcast done (exchange), chunk", c);
        BMB_TRY(bmb_comm_allreduce(t->comm, t->d_token, 1, t->st_x));
        tl_mark(t, step, t->st_x, "barrier after update done (exchange), chunk", c);
        // The rounded copy of the token embedding is read by the head's product only, at the end of the forward
        // pass (the embedding look-up reads the fp32 rows): it is rounded after chunk A's event,
        // still ahead of chunk C's, which the piece holding the head waits for.
        const bool wte_later = t->shadow && c == 0 && t->chunk[0].n > 1 && t->chunk[0].off[0] == t->poff[P_WTE];
        if (t->shadow) {
            DpRangeList first = t->chunk[c];
            if (wte_later) {
                for (int q = 1; q < first.n; ++q) { first.off[q - 1] = first.off[q]; first.len[q - 1] = first.len[q]; }
                --first.n;
            }
            BMB_TRY(dp_round_ranges(first, t->shadow, t->params, alone, t->st_x));
        }
        BMB_CUDA(cudaEventRecord(t->ev_upd[c], t->st_x));
        t->upd_pending[c] = true;
        tl_mark(t, step, t->st_x, "rounded copy done (exchange), chunk", c);
        if (wte_later) {
            DpRangeList wte;
            wte.n = 1; wte.off[0] = t->chunk[0].off[0]; wte.len[0] = t->chunk[0].len[0];
            BMB_TRY(dp_round_ranges(wte, t->shadow, t->params, /*alone=*/false, t->st_x));
        }
    }
    return BMB_OK;
}

int bmb_trainer_loss_async(bmb_trainer *t, float *pinned_host_loss) {
    if (!t || !pinned_host_loss) return fail(BMB_E_ARG, "trainer_loss_async: null argument");
    Scope sc(t, /*join=*/false);
    BMB_CUDA(cudaMemcpyAsync(pinned_host_loss, t->d_loss, sizeof(float), cudaMemcpyDeviceToHost, t->st));
    return BMB_OK;
}

int bmb_trainer_loss(bmb_trainer *t, float *host_loss) {
    if (!t || !host_loss) return fail(BMB_E_ARG, "trainer_loss: null argument");
    Scope sc(t, /*join=*/false);
    BMB_CUDA(cudaMemcpyAsync(host_loss, t->d_loss, sizeof(float), cudaMemcpyDeviceToHost, t->st));
    BMB_CUDA(cudaStreamSynchronize(t->st));
    return check_kernel_status();
}

void *bmb_trainer_stream(bmb_trainer *t) { return t ? (void *)t->st : nullptr; }

int bmb_trainer_sync(bmb_trainer *t) {
    if (!t) return fail(BMB_E_ARG, "trainer: null handle");
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    return BMB_OK;
}

int bmb_trainer_profile(bmb_trainer *t, int on) {
    if (!t) return fail(BMB_E_ARG, "trainer: null handle");
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    BMB_TRY(collect_profile(t));
    t->prof = on != 0;
    t->prof_flop = 0.0; t->prof_ms = 0.0; t->prof_calls = 0;
    t->launches0 = launches_total();
    return BMB_OK;
}

int bmb_trainer_profile_read(bmb_trainer *t, double *gemm_flop, double *gemm_ms, long long *gemm_calls,
                             long long *kernel_launches) {
    if (!t) return fail(BMB_E_ARG, "trainer: null handle");
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    BMB_TRY(collect_profile(t));
    if (gemm_flop) *gemm_flop = t->prof_flop;
    if (gemm_ms) *gemm_ms = t->prof_ms;
    if (gemm_calls) *gemm_calls = t->prof_calls;
    if (kernel_launches) *kernel_launches = launches_total() - t->launches0;
    return BMB_OK;
}


// ---- memory report, gradient norm, forward-only loss -------------------------------------------
int bmb_trainer_memory(const bmb_trainer *t, size_t *param_floats, size_t *activation_floats, size_t *scratch_floats) {
    if (!t) return fail(BMB_E_ARG, "trainer_memory: null handle");
    if (param_floats) *param_floats = t->num_params;
    if (activation_floats) *activation_floats = t->num_acts;
    if (scratch_floats) *scratch_floats = t->num_bacts;
    return BMB_OK;
}

int bmb_trainer_grad_norm(bmb_trainer *t, float *host_norm) {
    if (!t || !host_norm) return fail(BMB_E_ARG, "trainer_grad_norm: null argument");
    Scope sc(t);
    double ss = 0.0;
    BMB_CUDA(cudaMemcpyAsync(&ss, t->d_sumsq, sizeof(double), cudaMemcpyDeviceToHost, t->st));
    BMB_CUDA(cudaStreamSynchronize(t->st));
    *host_norm = (float)(sqrt(ss) / (double)t->nranks);
    return BMB_OK;
}

int bmb_trainer_forward_loss(bmb_trainer *t, float *host_loss) {
    if (!t || !host_loss) return fail(BMB_E_ARG, "trainer_forward_loss: null argument");
    Scope sc(t);
    BMB_TRY(forward(t));
    BMB_CUDA(cudaMemcpyAsync(host_loss, t->d_loss, sizeof(float), cudaMemcpyDeviceToHost, t->st));
    BMB_CUDA(cudaStreamSynchronize(t->st));
    return check_kernel_status();
}

// ---- GPT1 checkpoints (src/train_gpt.cu:175-227) -------------------------------------------------
// Layout, all little-endian as the reference writes it with fwrite:
//   int32 magic 0x47505431 ("GPT1") | GPTConfig as six int32 (max_seq_len, vocab_size, padded_vocab,
//   n_layer, n_head, n_embd; src/gpt.h:10-17) | int32 nvocab | nvocab bytes (token id -> character) |
//   num_params fp32 in the tensor order of src/gpt.cu:32-51.
// The reference's reader stops there.  Optionally this library appends the optimiser state, which
// the reference does not keep:  int32 magic 0x4F424D42 ("BMBO") | int32 step | m | v (fp32 each).
namespace {
constexpr int GPT1_MAGIC = 0x47505431, OPT_MAGIC = 0x4F424D42;
struct Gpt1Header { int cfg[6]; int nvocab; std::string itos; long params_at; };

int read_gpt1_header(FILE *f, const char *path, Gpt1Header *h) {
    int magic = 0;
    if (fread(&magic, sizeof(int), 1, f) != 1 || magic != GPT1_MAGIC) return fail(BMB_E_ARG, "%s is not a GPT1 checkpoint", path);
    if (fread(h->cfg, sizeof(int), 6, f) != 6 || fread(&h->nvocab, sizeof(int), 1, f) != 1 || h->nvocab < 0 || h->nvocab > (1 << 24))
        return fail(BMB_E_ARG, "%s: truncated or corrupt header", path);
    h->itos.resize((size_t)h->nvocab);
    if (h->nvocab && fread(&h->itos[0], 1, (size_t)h->nvocab, f) != (size_t)h->nvocab) return fail(BMB_E_ARG, "%s: truncated vocabulary", path);
    h->params_at = ftell(f);
    return BMB_OK;
}
}  // namespace

int bmb_trainer_save(bmb_trainer *t, const char *path, const char *itos, int nvocab, int with_optimizer_state, int step) {
    if (!t || !path || nvocab < 0 || (nvocab && !itos)) return fail(BMB_E_ARG, "trainer_save: bad argument");
    Scope sc(t);
    BMB_CUDA(cudaStreamSynchronize(t->st));
    std::vector<float> h(t->num_params);
    FILE *f = fopen(path, "wb");
    if (!f) return fail(BMB_E_ARG, "trainer_save: cannot write %s", path);
    const int cfg[6] = {t->c.max_seq_len, t->c.vocab_size, t->c.padded_vocab, t->c.n_layer, t->c.n_head, t->c.n_embd};
    bool ok = fwrite(&GPT1_MAGIC, sizeof(int), 1, f) == 1 && fwrite(cfg, sizeof(int), 6, f) == 6 &&
              fwrite(&nvocab, sizeof(int), 1, f) == 1 && (nvocab == 0 || fwrite(itos, 1, (size_t)nvocab, f) == (size_t)nvocab);
    auto dump = [&](const float *dev) {
        if (!ok) return;
        ok = cudaMemcpy(h.data(), dev, t->num_params * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess &&
             fwrite(h.data(), sizeof(float), t->num_params, f) == t->num_params;
    };
    dump(t->params);
    if (with_optimizer_state) {
        ok = ok && fwrite(&OPT_MAGIC, sizeof(int), 1, f) == 1 && fwrite(&step, sizeof(int), 1, f) == 1;
        dump(t->m);
        dump(t->v);
    }
    ok = (fclose(f) == 0) && ok;
    return ok ? BMB_OK : fail(BMB_E_CUDA, "trainer_save: writing %s failed", path);
}

int bmb_checkpoint_header(const char *path, bmb_train_config *cfg_out, int *nvocab_out, char *itos_out, int itos_cap,
                          int *has_optimizer_state, int *step_out) {
    if (!path) return fail(BMB_E_ARG, "checkpoint_header: null path");
    FILE *f = fopen(path, "rb");
    if (!f) return fail(BMB_E_ARG, "cannot open %s", path);
    Gpt1Header h;
    int rc = read_gpt1_header(f, path, &h);
    if (rc == BMB_OK) {
        if (cfg_out) {
            cfg_out->max_seq_len = h.cfg[0]; cfg_out->vocab_size = h.cfg[1]; cfg_out->padded_vocab = h.cfg[2];
            cfg_out->n_layer = h.cfg[3]; cfg_out->n_head = h.cfg[4]; cfg_out->n_embd = h.cfg[5];
        }
        if (nvocab_out) *nvocab_out = h.nvocab;
        if (itos_out) memcpy(itos_out, h.itos.data(), (size_t)(h.nvocab < itos_cap ? h.nvocab : (itos_cap > 0 ? itos_cap : 0)));
        bmb_train_config c{};
        c.max_seq_len = h.cfg[0]; c.vocab_size = h.cfg[1]; c.padded_vocab = h.cfg[2]; c.n_layer = h.cfg[3]; c.n_head = h.cfg[4]; c.n_embd = h.cfg[5];
        int opt = 0, step = 0;
        if (c.n_layer > 0 && c.n_embd > 0 && c.padded_vocab > 0 && c.max_seq_len > 0) {
            size_t ps[NPT], n = 0;
            param_sizes(ps, c);
            for (int i = 0; i < NPT; ++i) n += ps[i];
            int magic = 0;
            if (fseek(f, h.params_at + (long)(n * sizeof(float)), SEEK_SET) == 0 && fread(&magic, sizeof(int), 1, f) == 1 &&
                magic == OPT_MAGIC && fread(&step, sizeof(int), 1, f) == 1)
                opt = 1;
        }
        if (has_optimizer_state) *has_optimizer_state = opt;
        if (step_out) *step_out = opt ? step : 0;
    }
    fclose(f);
    return rc;
}

int bmb_trainer_load(bmb_trainer *t, const char *path, int load_optimizer_state, int *step_out) {
    if (!t || !path) return fail(BMB_E_ARG, "trainer_load: null argument");
    FILE *f = fopen(path, "rb");
    if (!f) return fail(BMB_E_ARG, "cannot open %s", path);
    Gpt1Header h;
    int rc = read_gpt1_header(f, path, &h);
    const int mine[6] = {t->c.max_seq_len, t->c.vocab_size, t->c.padded_vocab, t->c.n_layer, t->c.n_head, t->c.n_embd};
    // the context length only sizes the position table: a trainer may run shorter sequences than the file's
    if (rc == BMB_OK && memcmp(h.cfg, mine, sizeof(mine)) != 0)
        rc = fail(BMB_E_ARG, "%s holds a %d-layer %d-head %d-wide model (ctx %d, vocab %d/%d); this trainer is %d/%d/%d (ctx %d, vocab %d/%d)",
                  path, h.cfg[3], h.cfg[4], h.cfg[5], h.cfg[0], h.cfg[1], h.cfg[2], mine[3], mine[4], mine[5], mine[0], mine[1], mine[2]);
    std::vector<float> buf(rc == BMB_OK ? t->num_params : 0);
    Scope sc(t);
    auto slurp = [&](float *dev, const char *what) {
        if (rc != BMB_OK) return;
        if (fread(buf.data(), sizeof(float), t->num_params, f) != t->num_params) { rc = fail(BMB_E_ARG, "%s: %s truncated", path, what); return; }
        if (cudaMemcpy(dev, buf.data(), t->num_params * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
            rc = fail(BMB_E_CUDA, "trainer_load: copy of %s failed", what);
    };
    if (rc == BMB_OK) cudaStreamSynchronize(t->st);
    slurp(t->params, "parameters");
    int step = 0;
    if (rc == BMB_OK && load_optimizer_state) {
        int magic = 0;
        if (fread(&magic, sizeof(int), 1, f) != 1 || magic != OPT_MAGIC || fread(&step, sizeof(int), 1, f) != 1)
            rc = fail(BMB_E_ARG, "%s carries no optimiser state", path);
        slurp(t->m, "first moments");
        slurp(t->v, "second moments");
    }
    fclose(f);
    if (rc != BMB_OK) return rc;
    if (step_out) *step_out = step;
    BMB_TRY(refresh_shadow(t));
    BMB_CUDA(cudaStreamSynchronize(t->st));
    return BMB_OK;
}

// ---- sampling (src/train_gpt.cu:46-102) ------------------------------------------------------------
int bmb_trainer_next_token_probs(bmb_trainer *t, const int *host_tokens, int pos, float *host_probs) {
    if (!t || !host_tokens || !host_probs || pos < 0 || pos >= t->c.B * t->c.T) return fail(BMB_E_ARG, "next_token_probs: bad argument");
    Scope sc(t);
    const int Vp = t->c.padded_vocab, V = t->c.vocab_size;
    if (!t->gen_probs) BMB_CUDA(cudaMalloc(&t->gen_probs, ((size_t)Vp + 1) * sizeof(float)));
    BMB_CUDA(cudaMemcpyAsync(t->d_tokens, host_tokens, (size_t)t->c.B * t->c.T * sizeof(int), cudaMemcpyDefault, t->st));
    BMB_TRY(forward(t, false));
    set_emit_rounded(false);
    // the softmax of the reference's loss kernel over that one row (src/nn.cu:197-237); its target only picks which
    // loss is written, so row `pos` of the resident targets serves
    BMB_TRY(bmb_softmax_crossentropy_forward(t->gen_probs, t->gen_probs + Vp, t->logits + (size_t)pos * Vp, t->d_targets + pos, 1, V, Vp));
    BMB_CUDA(cudaMemcpyAsync(host_probs, t->gen_probs, (size_t)Vp * sizeof(float), cudaMemcpyDeviceToHost, t->st));
    BMB_CUDA(cudaStreamSynchronize(t->st));
    return check_kernel_status();
}

int bmb_trainer_generate(bmb_trainer *t, int start_token, int steps, unsigned seed, float temperature, int *host_tokens_out) {
    if (!t || steps < 0 || (steps && !host_tokens_out) || start_token < 0 || start_token >= t->c.vocab_size || !(temperature > 0.0f))
        return fail(BMB_E_ARG, "trainer_generate: bad argument");
    const int T = t->c.T, Vp = t->c.padded_vocab, V = t->c.vocab_size;
    std::vector<int> ctx((size_t)t->c.B * T, 0);
    std::vector<float> row((size_t)Vp);
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> uni(0.0f, 1.0f);
    int cur_len = 1;
    ctx[0] = start_token;
    for (int s = 0; s < steps; ++s) {
        BMB_TRY(bmb_trainer_next_token_probs(t, ctx.data(), cur_len - 1, row.data()));
        if (temperature != 1.0f) {
            float sum = 0.0f;
            for (int i = 0; i < V; ++i) { row[i] = powf(row[i], 1.0f / temperature); sum += row[i]; }
            for (int i = 0; i < V; ++i) row[i] /= sum;
        }
        const float coin = uni(rng);
        float cdf = 0.0f;
        int tok = V - 1;
        for (int i = 0; i < V; ++i) { cdf += row[i]; if (coin < cdf) { tok = i; break; } }
        host_tokens_out[s] = tok;
        if (cur_len < T) ctx[cur_len++] = tok;
        else {                               // context full: slide the window left by one
            for (int i = 0; i < T - 1; ++i) ctx[i] = ctx[i + 1];
            ctx[T - 1] = tok;
        }
    }
    return BMB_OK;
}

}  // extern "C"
