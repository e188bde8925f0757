// Bandwidth-bound transformer kernels with the reference's signatures
// (src/nn.h:10-60).  Activations are row-major (B, T, C) seen as N = B*T rows;
// weights are (out_features, in_features).  All calls are asynchronous on the
// calling thread's current stream except grad_global_norm and reduce_mean,
// which return a host value and therefore wait.
#pragma once
#include <cstddef>
#include <cuda_runtime.h>

void encoder_forward(float *out, const int *tokens, const float *wte,
                     const float *wpe, int B, int T, int C);
void encoder_backward(float *dwte, float *dwpe, const float *dout,
                      const int *tokens, int B, int T, int C);

void layernorm_forward(float *out, float *mean, float *rstd, const float *inp,
                       const float *weight, const float *bias, int N, int C);
// Accumulates (+=) into dinp, dweight and dbias.
void layernorm_backward(float *dinp, float *dweight, float *dbias,
                        const float *dout, const float *inp,
                        const float *weight, const float *mean,
                        const float *rstd, int N, int C);

void gelu_forward(float *out, const float *inp, int n);
void gelu_backward(float *dinp, const float *inp, const float *dout, int n);
void residual_forward(float *out, const float *a, const float *b, int n);
void add_inplace(float *dst, const float *src, int n);

void bias_forward(float *out, const float *bias, int N, int C);
void bias_backward(float *dbias, const float *dout, int N, int C);  // dbias += column sums

// V real columns out of Vp stored; columns [V, Vp) get probability 0.
void softmax_crossentropy_forward(float *probs, float *losses,
                                  const float *logits, const int *targets,
                                  int N, int V, int Vp);
void crossentropy_softmax_backward(float *dlogits, const float *probs,
                                   const int *targets, int N, int V, int Vp,
                                   float dloss_scale);

// grad_scale multiplies every gradient on the way in (clipping, 1/ranks).
void adamw_update(float *params, float *grads, float *m, float *v, int n,
                  float lr, float beta1, float beta2, float eps,
                  float weight_decay, int step, float grad_scale);
float grad_global_norm(const float *grads, int n);

void zero_buffer(float *p, size_t n);
float reduce_mean(const float *d_values, int n);
