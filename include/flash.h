// Fused causal multi-head attention with the reference's signatures
// (src/flash.h:36-62).  The (B,NH,T,T) score matrix is never written.
//   qkv  (B, T, 3C)  fused projection, [q|k|v] along the last axis
//   out  (B, T, C)
//   lse  (B, NH, T)  row log-sum-exp, all the backward pass needs to rebuild P
//   dqkv (B, T, 3C)  overwritten, not accumulated
//   dsum (B, NH, T)  backward scratch, rowsum(dout * out)
// Head sizes 32, 64 and 128; any other is fatal (message, exit(1)) as in the
// reference (src/flash.cu:426-431).
#pragma once
#include <cuda_runtime.h>

void flash_attention_forward(float *out, float *lse, const float *qkv, int B,
                             int T, int C, int NH);
void flash_attention_backward(float *dqkv, float *dsum, const float *dout,
                              const float *qkv, const float *out,
                              const float *lse, int B, int T, int C, int NH);

// Tuning harness: enumerate and run each kernel configuration.  The _cfg calls
// return false when a configuration cannot serve this head size.
int flash_num_configs();
const char *flash_config_name(int cfg);
int flash_default_config();
bool flash_attention_forward_cfg(int cfg, float *out, float *lse,
                                 const float *qkv, int B, int T, int C, int NH);
int flash_num_bwd_configs();
const char *flash_bwd_config_name(int cfg);
int flash_default_bwd_config();
bool flash_attention_backward_cfg(int cfg, float *dqkv, float *dsum,
                                  const float *dout, const float *qkv,
                                  const float *out, const float *lse, int B,
                                  int T, int C, int NH);
