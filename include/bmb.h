/* bmb.h -- the C ABI of libbmb.so: a B200 (sm_100a) implementation of the
 * GEMM / attention / nn / data-parallel hot path of bare-metal-bard.
 *
 * Every entry point takes plain pointers and sizes, returns an int status
 * (0 = ok, otherwise one of BMB_E_*; bmb_last_error() gives the text for the
 * calling thread) and never takes ownership of a caller's buffer.  Pointers
 * are device pointers on the current CUDA device unless a parameter is named
 * host_*.  Calls are asynchronous on the calling thread's "current stream"
 * (bmb_set_stream; the legacy default stream unless set) except where a
 * parameter named `stream` is given or the comment says the call blocks.
 *
 * The C++ headers beside this file (kernels.h, gemm.h, flash.h, attention.h,
 * nn.h, ddp.h, gpt.h) are inline shims with the reference's own names and
 * signatures over these functions, so gpt.cu / train_gpt.cu-shaped host code
 * compiles against them unchanged.  Each declaration cites the reference
 * interface it replaces as path:line inside the reference project.
 */
#ifndef BMB_H
#define BMB_H
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BMB_OK 0
#define BMB_E_ARG 1      /* bad argument (shape, alignment, null pointer)     */
#define BMB_E_CUDA 2     /* a CUDA runtime / driver call failed               */
#define BMB_E_UNSUPPORTED 3 /* valid request this build cannot serve          */
#define BMB_E_TIMEOUT 4  /* a bounded device-side wait expired                */
#define BMB_E_NCCL 5     /* NCCL missing or an NCCL call failed               */
#define BMB_E_LIMIT 6    /* size beyond a stated maximum                      */

const char *bmb_last_error(void);
const char *bmb_version(void);
/* No counterpart in the reference.  Replays on the host the tile schedule a tensor-core GEMM of
 * this shape would use on `ctas` SMs (tile height and width, whole tiles, tiles shared along K) and returns 0
 * when every (tile, K slice) is computed exactly once.  Launches nothing; usable without a GPU. */
int bmb_gemm_schedule_check(int math, int flags, int batch, int M, int N, int K, int ctas,
                            int *tile_m_out, int *tile_n_out, int *whole_tiles_out, int *grid_out);
/* Kernels this library has launched in this process so far (launches replayed from a CUDA
 * graph included).  No counterpart in the reference; bench.py reports it. */
long long bmb_launch_count(void);

/* ---- device-side waits that ran out ------------------------------------ */
/* No counterparts in the reference.  Every wait inside the tensor-core kernels (on a copy, on the
 * tensor core, on another role of the CTA) is bounded; when one runs out the kernel drains what it
 * has in flight, returns, and leaves a nonzero word per device that makes every later tensor-core
 * call on that device return BMB_E_TIMEOUT.  bmb_kernel_status reads the word of the current device
 * (0 = nothing happened).  bmb_kernel_status_clear waits for the device to go idle and resets it,
 * so that a process can carry on after it has dealt with the failed step.
 * bmb_selftest_wait_expiry exercises that path without any fault: one CTA waits at most
 * limit_cycles (1..1e8 SM clocks) on a barrier that nothing arrives on, gives up, raises the word
 * and returns; the call blocks until then and reports the cycles the wait took.  Afterwards the
 * status is set, exactly as after a real expiry, until bmb_kernel_status_clear. */
int bmb_kernel_status(int *status_out);
int bmb_kernel_status_clear(void);
int bmb_selftest_wait_expiry(long long limit_cycles, long long *host_waited_cycles);

/* ---- per-thread launch context ---------------------------------------- */
/* Stream used by every entry point without a `stream` parameter.  Thread
 * local: rank threads of one process do not disturb one another. */
int bmb_set_stream(void *cuda_stream);
void *bmb_get_stream(void);

/* Arithmetic used by bmb_gemm / bmb_batched_gemm / flash attention when the
 * caller does not say.  fp32 = SIMT FFMA, bit-comparable with the reference's
 * fp32 kernels up to summation order; tf32 = tcgen05 kind::tf32 with operands
 * rounded to nearest TF32 first and fp32 accumulation in tensor memory;
 * bf16 = tcgen05 kind::f16 on bf16-rounded operands. */
#define BMB_MATH_FP32 0
#define BMB_MATH_TF32 1
#define BMB_MATH_BF16 2
int bmb_set_math_mode(int mode);   /* process wide */
int bmb_get_math_mode(void);

/* ---- registry (src/kernels.h:10-31, src/registry.cu:4-23) -------------- */
typedef void (*bmb_sgemm_fn)(int M, int N, int K, float alpha, const float *A,
                             const float *B, float beta, float *C);
typedef struct bmb_kernel_entry {
    int id;
    const char *name;
    bmb_sgemm_fn fn;
    const char *note;
    double tol; /* normwise tolerance against an fp32 reference product */
} bmb_kernel_entry;
int bmb_num_kernels(void);
const bmb_kernel_entry *bmb_kernel_table(void);
const bmb_kernel_entry *bmb_find_kernel(int id);
/* Row-major C = alpha*A@B + beta*C, the three registry kernels
 * (replaces sgemm_naive..sgemm_tensorcore, src/kernels.h:34-42). */
int bmb_sgemm_simt(int M, int N, int K, float alpha, const float *A,
                   const float *B, float beta, float *C);
int bmb_sgemm_tf32(int M, int N, int K, float alpha, const float *A,
                   const float *B, float beta, float *C);
int bmb_sgemm_bf16(int M, int N, int K, float alpha, const float *A,
                   const float *B, float beta, float *C);

/* ---- GEMM (src/gemm.h:17-19, 26-29) ----------------------------------- */
/* C[M,N] = alpha*op(A)@op(B) + beta*C, row-major, dense leading dimensions
 * exactly as src/gemm.h:6-11 defines them. */
int bmb_gemm(int transA, int transB, int M, int N, int K, float alpha,
             const float *A, const float *B, float beta, float *C,
             void *stream);
/* Same, with the arithmetic stated per call (BMB_MATH_*) and flags. */
#define BMB_GEMM_A_ROUNDED 1 /* A already holds TF32-representable values */
#define BMB_GEMM_B_ROUNDED 2 /* B already holds TF32-representable values */
#define BMB_GEMM_C_ROUNDED 4 /* store C rounded to TF32 (it feeds another tensor-core kernel) */
#define BMB_GEMM_NO_SPLIT 8  /* never split K across CTAs (keeps the summation order fixed) */
#define BMB_GEMM_TILE_M128 16 /* TF32 tensor-core path: 128-row tiles whatever the cost model says */
#define BMB_GEMM_TILE_M256 32 /* TF32 tensor-core path: 256-row tiles where the shape allows (M >= 256, N >= 256) */
#define BMB_GEMM_PAIR 64      /* TF32: run on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles) where the shape allows
                                 (M >= 256, N >= 256, an M- or N-contiguous operand a multiple of 32 wide); opt-in */
#define BMB_GEMM_NO_PAIR 128  /* TF32: never use CTA pairs for this call */
#define BMB_GEMM_HALF_SMS 256 /* tensor-core path: occupy only half of the SMs (one CTA each), so that two products
                                 launched on two streams share the GPU side by side instead of one after the other */
int bmb_gemm_ex(int math, int flags, int transA, int transB, int M, int N,
                int K, float alpha, const float *A, const float *B, float beta,
                float *C, void *stream);
/* The MLP's first half in one call (no counterpart in the reference; equals gemm + bias_forward + gelu_forward of
 * src/gpt.cu:268-272): C = A W^T + bias (A [M,K], W [N,K], bias [N] or NULL, all row-major) and
 * C_gelu = GELU(C), bit-identical to bmb_gelu_forward on C.  On the tensor-core paths both leave the
 * accumulator in the product's epilogue when C and C_gelu are 16-byte aligned and N % 4 == 0 (no tile is then
 * split along K); otherwise, and for BMB_MATH_FP32, the activation is a pass of its own.
 * BMB_GEMM_AUX_ROUNDED: C_gelu is stored rounded to TF32 (it feeds another tensor-core product).
 * BMB_GEMM_AUX_FAST: where the activation rides in the epilogue, its tanh is the hardware's approximate one (absolute
 * error about 2^-11, of the order of the TF32 rounding of C_gelu; no longer bit-identical to bmb_gelu_forward). */
#define BMB_GEMM_AUX_ROUNDED 512
#define BMB_GEMM_AUX_FAST 1024
int bmb_gemm_bias_gelu(int math, int flags, int M, int N, int K, const float *A, const float *W, const float *bias,
                       float *C, float *C_gelu, void *stream);
int bmb_batched_gemm(int transA, int transB, int batch, int M, int N, int K,
                     float alpha, const float *A, long long strideA,
                     const float *B, long long strideB, float beta, float *C,
                     long long strideC, void *stream);
/* Round n floats to the nearest TF32 value (ties away from zero, the
 * cvt.rna.tf32.f32 rule the reference applies at k09_tensorcore.cu:119-128). */
int bmb_round_tf32(float *dst, const float *src, size_t n, void *stream);

/* ---- fused causal attention (src/flash.h:36-62) ------------------------ */
int bmb_flash_attention_forward(float *out, float *lse, const float *qkv,
                                int B, int T, int C, int NH);
int bmb_flash_attention_backward(float *dqkv, float *dsum, const float *dout,
                                 const float *qkv, const float *out,
                                 const float *lse, int B, int T, int C, int NH);
int bmb_flash_num_configs(void);
const char *bmb_flash_config_name(int cfg);
int bmb_flash_default_config(void);
/* status BMB_E_UNSUPPORTED <=> the reference's `false` (config cannot run for
 * this head size). */
int bmb_flash_attention_forward_cfg(int cfg, float *out, float *lse,
                                    const float *qkv, int B, int T, int C,
                                    int NH);
int bmb_flash_num_bwd_configs(void);
const char *bmb_flash_bwd_config_name(int cfg);
int bmb_flash_default_bwd_config(void);
int bmb_flash_attention_backward_cfg(int cfg, float *dqkv, float *dsum,
                                     const float *dout, const float *qkv,
                                     const float *out, const float *lse, int B,
                                     int T, int C, int NH);
/* No counterpart in the reference: the _cfg calls with a flag word.  BMB_FLASH_OPERANDS_ROUNDED
 * tells the TF32 tensor-core configuration that qkv (and dout) already hold TF32-representable
 * values, as the training step's producers leave them: the kernels then read them where they
 * lie instead of rounding copies first.  Ignored by the fp32 configurations. */
#define BMB_FLASH_OPERANDS_ROUNDED 1
int bmb_flash_attention_forward_ex(int cfg, int flags, float *out, float *lse,
                                   const float *qkv, int B, int T, int C, int NH);
int bmb_flash_attention_backward_ex(int cfg, int flags, float *dqkv, float *dsum,
                                    const float *dout, const float *qkv, const float *out,
                                    const float *lse, int B, int T, int C, int NH);

/* ---- unfused attention (src/attention.h:18-24) ------------------------- */
int bmb_attention_forward(float *out, float *qkvr, float *att,
                          const float *qkv, int B, int T, int C, int NH);
int bmb_attention_backward(float *dqkv, float *dqkvr, float *datt,
                           float *dpreatt, const float *dout,
                           const float *qkvr, const float *att, int B, int T,
                           int C, int NH);

/* ---- nn kernels (src/nn.h:10-60) -------------------------------------- */
int bmb_encoder_forward(float *out, const int *tokens, const float *wte,
                        const float *wpe, int B, int T, int C);
int bmb_encoder_backward(float *dwte, float *dwpe, const float *dout,
                         const int *tokens, int B, int T, int C);
int bmb_layernorm_forward(float *out, float *mean, float *rstd,
                          const float *inp, const float *weight,
                          const float *bias, int N, int C);
/* dinp, dweight and dbias are accumulated into (+=), as src/nn.cu:108-111. */
int bmb_layernorm_backward(float *dinp, float *dweight, float *dbias,
                           const float *dout, const float *inp,
                           const float *weight, const float *mean,
                           const float *rstd, int N, int C);
/* Same result as bmb_layernorm_backward, for callers that must not allocate.  No
 * counterpart in the reference.  A training loop that has handed all of its device memory
 * out at start-up (as gpt_alloc does) cannot afford the library's lazy cudaMalloc in the
 * middle of a step: it may fail on a full device, and it synchronises the whole device.
 * This entry point calls no cudaMalloc / cudaFree or any allocating routine: its partial
 * sums live in a fixed 4 MiB array inside the library image, present on every GPU that
 * loads libbmb.so.  Limits: C <= 1024, C % 4 == 0, 16-byte aligned buffers; a wider row
 * returns BMB_E_LIMIT.  The first call on each device looks up the array's device address
 * (once, with that device current), so make that first call before any stream capture.
 * All calls on a device share the one array: calls that overlap on the GPU (two streams,
 * two threads) race on it and must be serialised by the caller.  Nothing in the array needs
 * clearing between calls. */
int bmb_layernorm_backward_noalloc(float *dinp, float *dweight, float *dbias,
                                   const float *dout, const float *inp,
                                   const float *weight, const float *mean,
                                   const float *rstd, int N, int C);
/* No counterparts in the reference (fusions the training step uses):
 * residual_layernorm_forward: sum_out = a + b, then layernorm_forward(out, mean, rstd, sum_out, ...)
 *   (residual_forward + layernorm_forward, src/nn.cu:54-81, 152-159) in one pass over the rows.
 * layernorm_backward_colsum: layernorm_backward, and dcolsum += column sums of the updated dinp --
 *   the bias gradient (bias_backward, src/nn.cu:184-191) of the projection whose output gradient
 *   dinp is.  dcolsum may be NULL. */
/* gelu_backward over an (N x C) matrix, and dcolsum += column sums of dinp (the bias gradient
 * of the projection that produced the GELU input).  No counterpart in the reference. */
int bmb_gelu_backward_colsum(float *dinp, float *dcolsum, const float *inp,
                             const float *dout, int N, int C);
int bmb_residual_layernorm_forward(float *sum_out, float *out, float *mean, float *rstd,
                                   const float *a, const float *b, const float *weight,
                                   const float *bias, int N, int C);
int bmb_layernorm_backward_colsum(float *dinp, float *dweight, float *dbias, float *dcolsum,
                                  const float *dout, const float *inp, const float *weight,
                                  const float *mean, const float *rstd, int N, int C);
int bmb_gelu_forward(float *out, const float *inp, int n);
int bmb_gelu_backward(float *dinp, const float *inp, const float *dout, int n);
int bmb_residual_forward(float *out, const float *a, const float *b, int n);
int bmb_add_inplace(float *dst, const float *src, int n);
int bmb_bias_forward(float *out, const float *bias, int N, int C);
/* dbias += column sums of dout (src/nn.cu:184-191). */
int bmb_bias_backward(float *dbias, const float *dout, int N, int C);
int bmb_softmax_crossentropy_forward(float *probs, float *losses,
                                     const float *logits, const int *targets,
                                     int N, int V, int Vp);
int bmb_crossentropy_softmax_backward(float *dlogits, const float *probs,
                                      const int *targets, int N, int V, int Vp,
                                      float dloss_scale);
/* No counterpart in the reference: softmax_crossentropy_forward and
 * crossentropy_softmax_backward (src/nn.cu:197-237) in one sweep.  losses as
 * the forward writes them; dlogits = (softmax(logits) - onehot) * dloss_scale
 * on the V real columns, 0 on the padding.  The probabilities are not kept. */
int bmb_softmax_crossentropy_fused(float *dlogits, float *losses,
                                   const float *logits, const int *targets,
                                   int N, int V, int Vp, float dloss_scale);
int bmb_adamw_update(float *params, float *grads, float *m, float *v, int n,
                     float lr, float beta1, float beta2, float eps,
                     float weight_decay, int step, float grad_scale);
/* Blocks; *host_norm = sqrt(sum g^2) (src/nn.cu:336-355). */
int bmb_grad_global_norm(const float *grads, int n, float *host_norm);
int bmb_zero_buffer(float *p, size_t n);
/* Blocks; *host_mean = mean of n device values (src/nn.cu:359-368). */
int bmb_reduce_mean(const float *d_values, int n, float *host_mean);

/* Device-resident variants used by the training step so that a step has no
 * host round trip: the squared norm and the loss stay on the device, and the
 * optimiser derives its clip factor from the device value.
 * sumsq_out[0] = sum g^2 (double).  */
int bmb_grad_sumsq_device(const float *grads, size_t n, double *sumsq_out);
int bmb_reduce_mean_device(const float *d_values, int n, float *d_mean);
/* grad_scale = (norm/div > clip ? clip/(norm/div) : 1)/div with
 * norm = sqrt(*d_sumsq), the rule of src/train_gpt.cu:442-448 (div = ranks).
 * shadow (may be null) receives the TF32-rounded copy of the new params. */
int bmb_adamw_update_clipped(float *params, const float *grads, float *m,
                             float *v, size_t n, float lr, float beta1,
                             float beta2, float eps, float weight_decay,
                             int step, const double *d_sumsq, float clip,
                             float div, float *shadow);

/* ---- data-parallel all-reduce (src/ddp.h:32-69) ------------------------ */
typedef struct bmb_ddp_timing {
    double reduce_scatter_ms;
    double all_gather_ms;
    double total_ms;
    size_t bytes_per_device;
} bmb_ddp_timing;

/* Single-process form, one rank per entry of `devices` (a device may repeat,
 * src/ddp.h:53-57).  The handle is opaque; the C++ shim keeps it inside the
 * reference-shaped DDP struct. */
typedef struct bmb_ddp bmb_ddp;
int bmb_ddp_create(bmb_ddp **out, int n, const int *devices);
int bmb_ddp_destroy(bmb_ddp *d);
/* In-place sum over ranks of bufs[r][0..count); blocks until complete. */
int bmb_ddp_allreduce(bmb_ddp *d, float **bufs, size_t count);
int bmb_ddp_timing_get(const bmb_ddp *d, bmb_ddp_timing *out);
/* The part of a count-element buffer that rank r reduces and then serves to
 * the others: ceil(count/n) elements from r*ceil(count/n), clipped to the end
 * (the chunking of src/ddp.cu:34-40).  Host-only arithmetic. */
int bmb_ddp_slice(size_t count, int n, int r, size_t *off_out, size_t *len_out);
/* peer[i*n+j] = 1 when rank i reaches rank j's memory directly. */
int bmb_ddp_peer_matrix(const bmb_ddp *d, int *n_out, int *dev_out,
                        unsigned char *peer_out);
int bmb_ddp_report_topology(const bmb_ddp *d);

/* One-process-per-GPU form (NCCL over NVLink/NVSwitch; libnccl.so.2 is
 * opened on first use).  id is the 128-byte NCCL unique id made by rank 0 and
 * handed to every rank by the launcher. */
typedef struct bmb_comm bmb_comm;
int bmb_comm_unique_id(unsigned char id_out[128]);
int bmb_comm_create(bmb_comm **out, const unsigned char id[128], int nranks,
                    int rank);
int bmb_comm_destroy(bmb_comm *c);
/* In-place sum of count floats over all ranks, asynchronous on `stream`. */
int bmb_comm_allreduce(bmb_comm *c, float *buf, size_t count, void *stream);
int bmb_comm_allreduce_f64(bmb_comm *c, double *buf, size_t count, void *stream);

/* ---- GPT training step (caller of all of the above; src/gpt.h:10-79,
 *      src/train_gpt.cu:397-464) ---------------------------------------- */
typedef struct bmb_trainer bmb_trainer;
typedef struct bmb_train_config {
    int max_seq_len, vocab_size, padded_vocab, n_layer, n_head, n_embd;
    int B, T;          /* per-rank batch and sequence length               */
    int use_flash;     /* 1 fused attention, 0 the unfused path             */
    int math;          /* BMB_MATH_* for the GEMMs and attention            */
    int fused;         /* 1 = fused epilogues, 0 = the reference's op list  */
    float beta1, beta2, eps, weight_decay, grad_clip;
} bmb_train_config;
int bmb_trainer_create(bmb_trainer **out, const bmb_train_config *cfg,
                       unsigned seed);
int bmb_trainer_destroy(bmb_trainer *t);
int bmb_trainer_attach_comm(bmb_trainer *t, bmb_comm *c, int nranks);
/* Fused gradient exchange + optimiser over peer memory (one process per GPU, 2..8 ranks; replaces
 * ddp_allreduce + grad norm + adamw_update of src/train_gpt.cu:431-451 inside bmb_trainer_step):
 * rank r owns the r-th of n equal pieces of every tensor (of every layer group of a stacked tensor); it
 * sums its pieces of all ranks' gradients by reading the peers' buffers, the ranks add their squared
 * norms, every rank updates its pieces and stores the new parameters into all ranks' buffers.  All of it
 * runs on a second (exchange) stream, so bmb_trainer_step returns with the exchange still in flight; the
 * next step and every other entry point wait for it first.  BMB_TRAINER_OVERLAP=1 exchanges the parameter
 * space in three chunks (embeddings + layer 0 | the first half of the other layers | the second half + final
 * layernorm) and sums a chunk's gradients as soon as backward has finished them; =2 also lets the next step's
 * forward begin on the chunks that have arrived.  Both measured no faster than the default at 2 and 4 GPUs.
 * bmb_trainer_ipc_export writes this rank's 192-byte handle record; the launcher
 * gathers the records of all ranks in rank order and hands them to bmb_trainer_attach_peers
 * (after bmb_trainer_attach_comm, whose communicator carries the small collectives that order
 * the phases).  records = NULL detaches (back to the communicator's all-reduce); all ranks must
 * attach or none.  After a fused step bmb_trainer_get_grads returns summed values only inside
 * this rank's pieces. */
int bmb_trainer_ipc_export(bmb_trainer *t, void *record192);
int bmb_trainer_attach_peers(bmb_trainer *t, int rank, int nranks, const void *records);
/* The step's plan for a configuration (host only, no GPU needed; no counterpart in the reference): the chunks
 * as ranges of the flat parameter space -- ranges[(chunk * 16 + i) * 2 + {0, 1}] = offset, length in floats,
 * nranges[chunk] of them, 3 chunks -- and the pieces the step is captured in: pieces[4 * i + {0..3}] = first
 * unit, end unit, chunk whose update the piece waits for (-1: none), chunk whose gradients are final when it ends
 * (-1: none); units are 0 embedding, 1 + l layer l, L + 1 head and loss, L + 2 head backward, 2L + 2 - l layer
 * l backward, 2L + 3 embedding backward.  overlapped = 0 gives the single-chunk, single-piece plan. */
int bmb_trainer_step_plan(const bmb_train_config *cfg, int overlapped, unsigned long long *ranges /* [3][16][2] */,
                          int *nranges /* [3] */, int *pieces /* [5][4] */, int *npieces);
size_t bmb_trainer_num_params(const bmb_trainer *t);
int bmb_trainer_get_params(bmb_trainer *t, float *host_out);
int bmb_trainer_set_params(bmb_trainer *t, const float *host_in);
int bmb_trainer_get_grads(bmb_trainer *t, float *host_out);
/* Make tokens/targets (B*T ints each) the resident batch: an asynchronous copy on the trainer's
 * stream from host memory (pinned or pageable) or from device memory where a batch was staged. */
int bmb_trainer_upload(bmb_trainer *t, const int *host_tokens,
                       const int *host_targets);
/* One optimiser step on the resident batch: forward, backward, gradient
 * all-reduce (if a comm is attached), global-norm clip, AdamW.  Asynchronous;
 * the mean loss of the step lands in a device scalar. `step` counts from 1. */
int bmb_trainer_step(bmb_trainer *t, float lr, int step);
/* Forward+backward only (gradients left in place), for gradient parity. */
int bmb_trainer_forward_backward(bmb_trainer *t);
/* Blocks: waits for the stream and returns the last step's mean loss. */
int bmb_trainer_loss(bmb_trainer *t, float *host_loss);
/* The same read without the wait: enqueues the 4-byte device-to-host copy of the last step's mean
 * loss on the trainer's stream and returns; `pinned_host_loss` must be page-locked and is valid once
 * the stream has passed this point (an event recorded after the call, or bmb_trainer_sync).  Lets a
 * training loop read every step's loss one step late instead of draining the GPU every step. */
int bmb_trainer_loss_async(bmb_trainer *t, float *pinned_host_loss);
int bmb_trainer_sync(bmb_trainer *t);
/* Floats held by one replica: parameters (x4 with gradients and the two AdamW moments), forward
 * activations, backward scratch -- the figures the reference prints before training and under
 * --alloc-only (src/train_gpt.cu:339-355). */
int bmb_trainer_memory(const bmb_trainer *t, size_t *param_floats, size_t *activation_floats,
                       size_t *scratch_floats);
/* Blocks: the gradient norm the last bmb_trainer_step clipped against, ||sum over ranks of g|| / ranks
 * (src/train_gpt.cu:442-446). */
int bmb_trainer_grad_norm(bmb_trainer *t, float *host_norm);
/* Blocks: forward pass only on the resident batch, mean loss returned (the evaluate() of
 * src/train_gpt.cu:163-173 calls gpt_forward this way).  Parameters and gradients are untouched. */
int bmb_trainer_forward_loss(bmb_trainer *t, float *host_loss);

/* ---- GPT1 checkpoints and sampling (src/train_gpt.cu:175-227, 46-102) ---- */
/* Write the parameters in the reference's GPT1 layout: int32 magic 0x47505431, the six int32 of GPTConfig,
 * int32 nvocab, nvocab bytes mapping token id -> character, then num_params fp32 in the reference's tensor
 * order.  A file written here loads in the reference's `train_gpt --load` and the other way round.
 * with_optimizer_state != 0 appends what the reference does not keep -- int32 magic 0x4F424D42, int32 step,
 * the AdamW first and second moments -- after the point where the reference's reader stops. */
int bmb_trainer_save(bmb_trainer *t, const char *path, const char *itos, int nvocab,
                     int with_optimizer_state, int step);
/* Read a GPT1 file's header: fills the six model fields of *cfg_out (the others are left alone), the
 * vocabulary (at most itos_cap bytes of it), whether the optimiser-state section is present and its step. */
int bmb_checkpoint_header(const char *path, bmb_train_config *cfg_out, int *nvocab_out, char *itos_out,
                          int itos_cap, int *has_optimizer_state, int *step_out);
/* Load parameters (and, if asked, the optimiser state and *step_out) into a trainer whose six model fields
 * equal the file's; BMB_E_ARG otherwise, or when the state is asked for and absent. */
int bmb_trainer_load(bmb_trainer *t, const char *path, int load_optimizer_state, int *step_out);
/* Forward pass on host_tokens (B*T ints) and the softmax of row `pos` (0 <= pos < B*T) of the logits:
 * host_probs receives padded_vocab floats, zeros on the padding (what src/train_gpt.cu:73-78 reads). Blocks. */
int bmb_trainer_next_token_probs(bmb_trainer *t, const int *host_tokens, int pos, float *host_probs);
/* The reference's generate(): starts from start_token, draws `steps` tokens with mt19937(seed) and a
 * uniform float per token, probabilities raised to 1/temperature and renormalised when temperature != 1,
 * the window sliding once the context is full.  host_tokens_out receives the drawn token ids. Blocks. */
int bmb_trainer_generate(bmb_trainer *t, int start_token, int steps, unsigned seed, float temperature,
                         int *host_tokens_out);
/* The CUDA stream every step of this trainer is enqueued on (for events). */
void *bmb_trainer_stream(bmb_trainer *t);
/* Per-call event timing of the GEMMs inside steps (on = 1 / off = 0); the
 * totals since the last reset: flop count, device milliseconds, launches. */
int bmb_trainer_profile(bmb_trainer *t, int on);
int bmb_trainer_profile_read(bmb_trainer *t, double *gemm_flop,
                             double *gemm_ms, long long *gemm_calls,
                             long long *kernel_launches);

#ifdef __cplusplus
}
#endif
#endif /* BMB_H */
