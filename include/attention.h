// Unfused causal attention with the reference's signatures
// (src/attention.h:18-24): permute, batched Q@K^T, causal softmax, batched
// P@V, head merge.  hs = C / NH.
//   qkv   (B, T, 3C)
//   qkvr  (4, B, NH, T, hs)  q, k, v head-major, plus one scratch slot
//   att   (B, NH, T, T)      post-softmax weights, kept for backward
//   out   (B, T, C)
#pragma once

void attention_forward(float *out, float *qkvr, float *att, const float *qkv,
                       int B, int T, int C, int NH);
// dpreatt may be the same buffer as datt.
void attention_backward(float *dqkv, float *dqkvr, float *datt, float *dpreatt,
                        const float *dout, const float *qkvr, const float *att,
                        int B, int T, int C, int NH);
