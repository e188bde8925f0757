// extern "C" doors onto the UNMODIFIED reference kernels, for the tests and
// the benchmark's reference arm.  TEST INFRASTRUCTURE ONLY.
//
// This file is compiled together with the reference's own sources, taken
// where they lie in the reference checkout (see the Makefile beside it), into
// oracle/_ref/libbmbref.so.  Nothing of the reference is copied here: every
// function below only forwards to the reference's public API (src/kernels.h,
// src/gemm.h, src/flash.h, src/attention.h, src/nn.h, src/ddp.h, src/gpt.h).
// The train-step driver repeats the call sequence of src/train_gpt.cu:397-464
// because the reference's CLI cannot express a configuration with a chosen
// head count, width or vocabulary (src/train_gpt.cu:256-277).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#include <cuda_runtime.h>
#include "kernels.h"
#include "gemm.h"
#include "flash.h"
#include "attention.h"
#include "nn.h"
#include "ddp.h"
#include "gpt.h"

extern "C" {

int ref_num_kernels() { return NUM_KERNELS; }
const char *ref_kernel_name(int id) { const KernelEntry *k = find_kernel(id); return k ? k->name : nullptr; }
double ref_kernel_tol(int id) { const KernelEntry *k = find_kernel(id); return k ? k->tol : -1.0; }
int ref_sgemm(int id, int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C) {
    const KernelEntry *k = find_kernel(id);
    if (!k) return 1;
    k->fn(M, N, K, alpha, A, B, beta, C);
    return 0;
}
void ref_gemm(int ta, int tb, int M, int N, int K, float alpha, const float *A, const float *B, float beta, float *C) {
    gemm(ta != 0, tb != 0, M, N, K, alpha, A, B, beta, C, 0);
}
void ref_batched_gemm(int ta, int tb, int batch, int M, int N, int K, float alpha, const float *A, long long sA,
                      const float *B, long long sB, float beta, float *C, long long sC) {
    batched_gemm(ta != 0, tb != 0, batch, M, N, K, alpha, A, sA, B, sB, beta, C, sC, 0);
}
void ref_flash_attention_forward(float *out, float *lse, const float *qkv, int B, int T, int C, int NH) {
    flash_attention_forward(out, lse, qkv, B, T, C, NH);
}
void ref_flash_attention_backward(float *dqkv, float *dsum, const float *dout, const float *qkv, const float *out,
                                  const float *lse, int B, int T, int C, int NH) {
    flash_attention_backward(dqkv, dsum, dout, qkv, out, lse, B, T, C, NH);
}
int ref_flash_num_configs() { return flash_num_configs(); }
int ref_flash_num_bwd_configs() { return flash_num_bwd_configs(); }
void ref_attention_forward(float *out, float *qkvr, float *att, const float *qkv, int B, int T, int C, int NH) {
    attention_forward(out, qkvr, att, qkv, B, T, C, NH);
}
void ref_attention_backward(float *dqkv, float *dqkvr, float *datt, float *dpreatt, const float *dout,
                            const float *qkvr, const float *att, int B, int T, int C, int NH) {
    attention_backward(dqkv, dqkvr, datt, dpreatt, dout, qkvr, att, B, T, C, NH);
}
void ref_encoder_forward(float *out, const int *tokens, const float *wte, const float *wpe, int B, int T, int C) {
    encoder_forward(out, tokens, wte, wpe, B, T, C);
}
void ref_encoder_backward(float *dwte, float *dwpe, const float *dout, const int *tokens, int B, int T, int C) {
    encoder_backward(dwte, dwpe, dout, tokens, B, T, C);
}
void ref_layernorm_forward(float *out, float *mean, float *rstd, const float *inp, const float *w, const float *b, int N, int C) {
    layernorm_forward(out, mean, rstd, inp, w, b, N, C);
}
void ref_layernorm_backward(float *dinp, float *dw, float *db, const float *dout, const float *inp, const float *w,
                            const float *mean, const float *rstd, int N, int C) {
    layernorm_backward(dinp, dw, db, dout, inp, w, mean, rstd, N, C);
}
void ref_gelu_forward(float *out, const float *inp, int n) { gelu_forward(out, inp, n); }
void ref_gelu_backward(float *dinp, const float *inp, const float *dout, int n) { gelu_backward(dinp, inp, dout, n); }
void ref_residual_forward(float *out, const float *a, const float *b, int n) { residual_forward(out, a, b, n); }
void ref_bias_forward(float *out, const float *bias, int N, int C) { bias_forward(out, bias, N, C); }
void ref_bias_backward(float *dbias, const float *dout, int N, int C) { bias_backward(dbias, dout, N, C); }
void ref_softmax_crossentropy_forward(float *probs, float *losses, const float *logits, const int *targets, int N, int V, int Vp) {
    softmax_crossentropy_forward(probs, losses, logits, targets, N, V, Vp);
}
void ref_crossentropy_softmax_backward(float *dlogits, const float *probs, const int *targets, int N, int V, int Vp, float s) {
    crossentropy_softmax_backward(dlogits, probs, targets, N, V, Vp, s);
}
void ref_adamw_update(float *p, float *g, float *m, float *v, int n, float lr, float b1, float b2, float eps, float wd,
                      int step, float gs) {
    adamw_update(p, g, m, v, n, lr, b1, b2, eps, wd, step, gs);
}
float ref_grad_global_norm(const float *g, int n) { return grad_global_norm(g, n); }
float ref_reduce_mean(const float *v, int n) { return reduce_mean(v, n); }

// ---- ring all-reduce ------------------------------------------------------
void *ref_ddp_create(int n, const int *devices) {
    DDP *d = new DDP();
    ddp_init(*d, n, devices);
    return d;
}
void ref_ddp_allreduce(void *h, float **bufs, size_t count) { ddp_allreduce(*(DDP *)h, bufs, count); }
double ref_ddp_total_ms(void *h) { return ddp_timing(*(DDP *)h).total_ms; }
void ref_ddp_destroy(void *h) { ddp_free(*(DDP *)h); delete (DDP *)h; }

// ---- training step, n ranks in one process as src/train_gpt.cu does --------
struct RefTrainer {
    int n;
    std::vector<int> devs;
    std::vector<GPT> reps;
    DDP ddp;
    float b1, b2, eps, wd, clip;
};

void *ref_trainer_create(int max_seq_len, int vocab, int padded_vocab, int n_layer, int n_head, int n_embd, int B,
                         int T, int use_flash, unsigned seed, int nranks, float b1, float b2, float eps, float wd,
                         float clip) {
    RefTrainer *t = new RefTrainer();
    t->n = nranks;
    t->b1 = b1; t->b2 = b2; t->eps = eps; t->wd = wd; t->clip = clip;
    int ndev = 1;
    cudaGetDeviceCount(&ndev);
    t->devs.resize(nranks);
    t->reps.resize(nranks);
    for (int r = 0; r < nranks; ++r) t->devs[r] = r % ndev;
    for (int r = 0; r < nranks; ++r) {
        cudaSetDevice(t->devs[r]);
        GPT &g = t->reps[r];
        g.use_flash = use_flash != 0;
        g.config = {max_seq_len, vocab, padded_vocab, n_layer, n_head, n_embd};
        g.B = B; g.T = T;   // per-rank batch
        gpt_alloc(g);
        gpt_init(g, seed);  // same seed: identical replicas (src/train_gpt.cu:326-328)
    }
    ddp_init(t->ddp, nranks, t->devs.data());
    cudaSetDevice(t->devs[0]);
    return t;
}
size_t ref_trainer_num_params(void *h) { return ((RefTrainer *)h)->reps[0].num_params; }
void ref_trainer_get_params(void *h, float *out) {
    RefTrainer *t = (RefTrainer *)h;
    cudaSetDevice(t->devs[0]);
    cudaMemcpy(out, t->reps[0].params_mem, t->reps[0].num_params * sizeof(float), cudaMemcpyDeviceToHost);
}
void ref_trainer_set_params(void *h, const float *in) {
    RefTrainer *t = (RefTrainer *)h;
    for (int r = 0; r < t->n; ++r) {
        cudaSetDevice(t->devs[r]);
        cudaMemcpy(t->reps[r].params_mem, in, t->reps[r].num_params * sizeof(float), cudaMemcpyHostToDevice);
    }
    cudaSetDevice(t->devs[0]);
}
void ref_trainer_get_grads(void *h, float *out) {
    RefTrainer *t = (RefTrainer *)h;
    cudaSetDevice(t->devs[0]);
    cudaMemcpy(out, t->reps[0].grads_mem, t->reps[0].num_params * sizeof(float), cudaMemcpyDeviceToHost);
}
// Forward + backward on rank 0 only (gradient parity).
float ref_trainer_forward_backward(void *h, const int *tokens, const int *targets) {
    RefTrainer *t = (RefTrainer *)h;
    cudaSetDevice(t->devs[0]);
    const float loss = gpt_forward(t->reps[0], tokens, targets);
    gpt_backward(t->reps[0]);
    cudaDeviceSynchronize();
    return loss;
}
// One optimiser step over all ranks; tokens/targets hold nranks*B*T ints, rank
// r taking rows [r*B, (r+1)*B).  Returns the mean loss over ranks.
float ref_trainer_step(void *h, const int *tokens, const int *targets, float lr, int step) {
    RefTrainer *t = (RefTrainer *)h;
    const int n = t->n;
    std::vector<float> rank_loss(n, 0.0f);
    const size_t shard = (size_t)t->reps[0].B * t->reps[0].T;
    if (n == 1) {
        cudaSetDevice(t->devs[0]);
        rank_loss[0] = gpt_forward(t->reps[0], tokens, targets);
        gpt_backward(t->reps[0]);
    } else {
        std::vector<std::thread> workers;
        for (int r = 0; r < n; ++r)
            workers.emplace_back([&, r] {
                cudaSetDevice(t->devs[r]);
                rank_loss[r] = gpt_forward(t->reps[r], tokens + r * shard, targets + r * shard);
                gpt_backward(t->reps[r]);
                cudaDeviceSynchronize();
            });
        for (auto &w : workers) w.join();
    }
    double loss_sum = 0.0;
    for (int r = 0; r < n; ++r) loss_sum += rank_loss[r];
    for (int r = 0; r < n; ++r) { cudaSetDevice(t->devs[r]); cudaDeviceSynchronize(); }
    std::vector<float *> gbufs(n);
    for (int r = 0; r < n; ++r) gbufs[r] = t->reps[r].grads_mem;
    ddp_allreduce(t->ddp, gbufs.data(), t->reps[0].num_params);
    auto opt_step = [&](int r) {
        cudaSetDevice(t->devs[r]);
        const float gn = grad_global_norm(t->reps[r].grads_mem, (int)t->reps[r].num_params) / n;
        const float gs = ((gn > t->clip) ? t->clip / gn : 1.0f) / n;
        adamw_update(t->reps[r].params_mem, t->reps[r].grads_mem, t->reps[r].m_mem, t->reps[r].v_mem,
                     (int)t->reps[r].num_params, lr, t->b1, t->b2, t->eps, t->wd, step, gs);
        cudaDeviceSynchronize();
    };
    if (n == 1) opt_step(0);
    else {
        std::vector<std::thread> workers;
        for (int r = 0; r < n; ++r) workers.emplace_back(opt_step, r);
        for (auto &w : workers) w.join();
    }
    for (int r = 0; r < n; ++r) { cudaSetDevice(t->devs[r]); cudaDeviceSynchronize(); }
    cudaSetDevice(t->devs[0]);
    return (float)(loss_sum / n);
}
// The loss of the last forward pass recomputed from the probability matrix the reference's own
// softmax_crossentropy_forward left behind: mean over rows (and ranks) of -log(max(p[target], 1e-30)).
// Why it exists: in the reference's kernel thread 0 reads p[target] for the loss right after the loop
// that normalises p, with no barrier in between (src/nn.cu:216-220), so at a large vocabulary it can
// read a value another thread has not normalised yet; the loss gpt_forward returns is then too low for
// that row.  The probabilities themselves (and with them the gradients) are unaffected, and after the
// kernel has finished they give the loss the formula defines.
__global__ void shim_target_prob_k(const float *__restrict__ probs, const int *__restrict__ targets,
                                   float *__restrict__ out, int N, int Vp) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < N) out[r] = probs[(size_t)r * Vp + targets[r]];
}
float ref_trainer_loss_from_probs(void *h) {
    RefTrainer *t = (RefTrainer *)h;
    double total = 0.0;
    for (int r = 0; r < t->n; ++r) {
        cudaSetDevice(t->devs[r]);
        GPT &g = t->reps[r];
        const int N = g.B * g.T, Vp = g.config.padded_vocab;
        float *d = nullptr;
        cudaMalloc(&d, N * sizeof(float));
        shim_target_prob_k<<<(N + 255) / 256, 256>>>(g.acts.probs, g.d_targets, d, N, Vp);
        std::vector<float> hp(N);
        cudaMemcpy(hp.data(), d, N * sizeof(float), cudaMemcpyDeviceToHost);
        cudaFree(d);
        double s = 0.0;
        for (int i = 0; i < N; ++i) s += -log((double)fmaxf(hp[i], 1e-30f));
        total += s / N;
    }
    cudaSetDevice(t->devs[0]);
    return (float)(total / t->n);
}

void ref_trainer_destroy(void *h) {
    RefTrainer *t = (RefTrainer *)h;
    for (int r = 0; r < t->n; ++r) {
        cudaSetDevice(t->devs[r]);
        GPT &g = t->reps[r];
        cudaFree(g.params_mem); cudaFree(g.grads_mem); cudaFree(g.m_mem); cudaFree(g.v_mem);
        cudaFree(g.acts_mem); cudaFree(g.grads_act_mem); cudaFree(g.d_tokens); cudaFree(g.d_targets);
    }
    ddp_free(t->ddp);
    delete t;
}

}  // extern "C"
