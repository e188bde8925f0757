// Bandwidth-bound kernels of the transformer (src/nn.h:10-60, src/nn.cu):
// embeddings, layernorm, GELU, residual, bias, softmax-cross-entropy, AdamW,
// gradient norm.  Every kernel moves each byte once with 128-bit accesses
// where the shape allows, and every reduction that the reference does with
// atomics on parameter gradients (src/nn.cu:110-111) is done here in two
// deterministic stages through per-device scratch.
#include "common.cuh"
#include <cfloat>
#include <cmath>
#include <mutex>

namespace bmb {
namespace {

#define LD4(p) (*reinterpret_cast<const float4 *>(p))
#define ST4(p) (*reinterpret_cast<float4 *>(p))

// Values headed for a tensor-core GEMM or attention kernel are stored already
// rounded to TF32 when the caller (the training step in TF32 mode) asks for it.
__device__ __forceinline__ float rnd1(float v, int rnd) { return rnd ? round_tf32(v) : v; }
__device__ __forceinline__ float4 rnd4(float4 v, int rnd) {
    return rnd ? make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w)) : v;
}

inline int grid_for(long long work_items, int threads, int per_sm) {
    long long b = (work_items + threads - 1) / threads;
    long long cap = (long long)sm_count() * per_sm;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

// ------------------------------------------------------------------ encoder
// out[b,t,:] = wte[tokens[b,t],:] + wpe[t,:]        (src/nn.cu:23-36)
__global__ void encoder_fwd_k(float *__restrict__ out, const int *__restrict__ tokens,
                              const float *__restrict__ wte, const float *__restrict__ wpe, int T,
                              int C, long long n4) {
    const int C4 = C >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const long long bt = i / C4;
        const int c = (int)(i - bt * C4) * 4;
        const int t = (int)(bt % T);
        const int tok = tokens[bt];
        float4 e = LD4(wte + (size_t)tok * C + c);
        const float4 p = LD4(wpe + (size_t)t * C + c);
        e.x += p.x; e.y += p.y; e.z += p.z; e.w += p.w;
        ST4(out + i * 4) = e;
    }
}

// dwpe[t,:] += sum_b dout[b,t,:]   -- no conflicts, so no atomics.
__global__ void encoder_bwd_wpe_k(float *__restrict__ dwpe, const float *__restrict__ dout, int B,
                                  int T, int C) {
    const long long n4 = (long long)T * C / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        float4 s = LD4(dwpe + i * 4);
        for (int b = 0; b < B; ++b) {
            const float4 g = LD4(dout + ((size_t)b * T * C) + i * 4);
            s.x += g.x; s.y += g.y; s.z += g.z; s.w += g.w;
        }
        ST4(dwpe + i * 4) = s;
    }
}

// dwte[tokens[b,t],:] += dout[b,t,:].  Positions that share a token id are
// genuine conflicts (src/nn.cu:44-48); one 128-bit atomic per four floats.
__global__ void encoder_bwd_wte_k(float *__restrict__ dwte, const float *__restrict__ dout,
                                  const int *__restrict__ tokens, int C, long long n4) {
    const int C4 = C >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const long long bt = i / C4;
        const int c = (int)(i - bt * C4) * 4;
        const float4 g = LD4(dout + i * 4);
        atomicAdd(reinterpret_cast<float4 *>(dwte + (size_t)tokens[bt] * C + c), g);
    }
}

// ---------------------------------------------------------------- layernorm
// One warp per row, the row held in registers between the mean pass, the
// variance pass and the write (src/nn.cu:54-78: two-pass biased variance,
// rsqrtf(var + 1e-5)).  C % 4 == 0 and C <= 32*4*V4 floats.
// With `addend`: the row normalised is inp + addend, and that sum is also stored to `sum_out`
// (the residual add of a transformer block riding in the layernorm that follows it).
template <int V4>
__global__ void __launch_bounds__(256)
layernorm_fwd_warp_k(float *__restrict__ out, float *__restrict__ mean, float *__restrict__ rstd,
                     const float *__restrict__ inp, const float *__restrict__ weight,
                     const float *__restrict__ bias, int N, int C, int rnd,
                     const float *__restrict__ addend = nullptr, float *__restrict__ sum_out = nullptr) {
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int C4 = C >> 2;
    for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < N;
         row += gridDim.x * warps_per_block) {
        const float *x = inp + (size_t)row * C;
        float4 v[V4];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            const int c4 = lane + 32 * i;
            v[i] = (c4 < C4) ? LD4(x + c4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (addend && c4 < C4) {
                const float4 a = LD4(addend + (size_t)row * C + c4 * 4);
                v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
                ST4(sum_out + (size_t)row * C + c4 * 4) = v[i];
            }
            sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        const float mu = warp_sum(sum) / C;
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            if (lane + 32 * i < C4) {
                const float a = v[i].x - mu, b = v[i].y - mu, c = v[i].z - mu, d = v[i].w - mu;
                sq += (a * a + b * b) + (c * c + d * d);
            }
        }
        const float var = warp_sum(sq) / C;
        const float rs = rsqrtf(var + 1e-5f);
        if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
        float *y = out + (size_t)row * C;
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            const int c4 = lane + 32 * i;
            if (c4 < C4) {
                const float4 w = LD4(weight + c4 * 4), b = LD4(bias + c4 * 4);
                float4 o;
                o.x = ((v[i].x - mu) * rs) * w.x + b.x;
                o.y = ((v[i].y - mu) * rs) * w.y + b.y;
                o.z = ((v[i].z - mu) * rs) * w.z + b.z;
                o.w = ((v[i].w - mu) * rs) * w.w + b.w;
                ST4(y + c4 * 4) = rnd4(o, rnd);
            }
        }
    }
}

// Any C: one block per row, three passes over the row (second and third hit L1/L2).
__global__ void layernorm_fwd_block_k(float *__restrict__ out, float *__restrict__ mean,
                                      float *__restrict__ rstd, const float *__restrict__ inp,
                                      const float *__restrict__ weight,
                                      const float *__restrict__ bias, int C, int rnd) {
    __shared__ float red[32];
    const int row = blockIdx.x;
    const float *x = inp + (size_t)row * C;
    float s = 0.0f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) s += x[i];
    const float mu = block_reduce<false>(s, red) / C;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) { const float d = x[i] - mu; sq += d * d; }
    const float var = block_reduce<false>(sq, red) / C;
    const float rs = rsqrtf(var + 1e-5f);
    if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
    float *y = out + (size_t)row * C;
    for (int i = threadIdx.x; i < C; i += blockDim.x) y[i] = rnd1(((x[i] - mu) * rs) * weight[i] + bias[i], rnd);
}

// Backward (src/nn.cu:85-113):
//   dx += rstd * (dxhat - mean(dxhat) - xhat * mean(dxhat * xhat)),  dxhat = dy*w
//   dw += sum_rows dy*xhat,   db += sum_rows dy
// A warp walks rows; each lane keeps the dw/db partial sums of its own columns
// in registers for all the rows the warp visits.  The warps of a block then
// fold their partials through shared memory, and the block writes one row of
// `partial` ([gridDim.x][2*C]: dw then db).  column_add_k finishes the sum in a
// fixed order, so the parameter gradients are reproducible run to run.
// COLSUM: `partial` rows are 3*C wide and the third part holds the column sums of the updated dinp
// (as stored), which is the bias gradient of the projection that produced this layer's input.
template <int V4, bool COLSUM>
__global__ void __launch_bounds__(128)
layernorm_bwd_warp_k(float *__restrict__ dinp, float *__restrict__ partial,
                     const float *__restrict__ dout, const float *__restrict__ inp,
                     const float *__restrict__ weight, const float *__restrict__ mean,
                     const float *__restrict__ rstd, int N, int C, int rnd) {
    extern __shared__ float fold[];  // 2*C floats (3*C with COLSUM)
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    const int C4 = C >> 2;
    float4 dw[V4], db[V4], dc[COLSUM ? V4 : 1];
#pragma unroll
    for (int i = 0; i < V4; ++i) {
        dw[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        db[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (COLSUM) dc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int row = blockIdx.x * warps_per_block + wid; row < N; row += gridDim.x * warps_per_block) {
        const float *x = inp + (size_t)row * C;
        const float *dy = dout + (size_t)row * C;
        float *dx = dinp + (size_t)row * C;
        const float mu = mean[row], rs = rstd[row];
        float4 xh[V4], g[V4], acc[V4];
        float s1 = 0.0f, s2 = 0.0f;
        // all three rows are requested before anything is consumed: one memory round trip per row
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            const int c4 = lane + 32 * i;
            if (c4 < C4) { xh[i] = LD4(x + c4 * 4); g[i] = LD4(dy + c4 * 4); acc[i] = LD4(dx + c4 * 4); }
        }
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            const int c4 = lane + 32 * i;
            if (c4 < C4) {
                const float4 xv = xh[i], wv = LD4(weight + c4 * 4);   // weight row stays in L1
                xh[i].x = (xv.x - mu) * rs; xh[i].y = (xv.y - mu) * rs;
                xh[i].z = (xv.z - mu) * rs; xh[i].w = (xv.w - mu) * rs;
                dw[i].x += g[i].x * xh[i].x; dw[i].y += g[i].y * xh[i].y;
                dw[i].z += g[i].z * xh[i].z; dw[i].w += g[i].w * xh[i].w;
                db[i].x += g[i].x; db[i].y += g[i].y; db[i].z += g[i].z; db[i].w += g[i].w;
                const float a = g[i].x * wv.x, b = g[i].y * wv.y, c = g[i].z * wv.z, d = g[i].w * wv.w;
                g[i] = make_float4(a, b, c, d);                       // from here on g holds dxhat = dy * w
                s1 += (a + b) + (c + d);
                s2 += (a * xh[i].x + b * xh[i].y) + (c * xh[i].z + d * xh[i].w);

            }
        }
        const float m1 = warp_sum(s1) / C, m2 = warp_sum(s2) / C;
#pragma unroll
        for (int i = 0; i < V4; ++i) {
            const int c4 = lane + 32 * i;
            if (c4 < C4) {
                float4 d = acc[i];
                d.x += rs * (g[i].x - m1 - xh[i].x * m2);
                d.y += rs * (g[i].y - m1 - xh[i].y * m2);
                d.z += rs * (g[i].z - m1 - xh[i].z * m2);
                d.w += rs * (g[i].w - m1 - xh[i].w * m2);
                d = rnd4(d, rnd);
                ST4(dx + c4 * 4) = d;
                if (COLSUM) { dc[i].x += d.x; dc[i].y += d.y; dc[i].z += d.z; dc[i].w += d.w; }
            }
        }
    }
    // Fold the warps of this block, one warp at a time (fixed order).
    for (int turn = 0; turn < warps_per_block; ++turn) {
        if (wid == turn) {
#pragma unroll
            for (int i = 0; i < V4; ++i) {
                const int c4 = lane + 32 * i;
                if (c4 < C4) {
                    float4 a = dw[i], b = db[i];
                    if (turn > 0) {
                        const float4 pa = LD4(fold + c4 * 4), pb = LD4(fold + C + c4 * 4);
                        a.x += pa.x; a.y += pa.y; a.z += pa.z; a.w += pa.w;
                        b.x += pb.x; b.y += pb.y; b.z += pb.z; b.w += pb.w;
                    }
                    ST4(fold + c4 * 4) = a;
                    ST4(fold + C + c4 * 4) = b;
                    if (COLSUM) {
                        float4 c = dc[i];
                        if (turn > 0) {
                            const float4 pc = LD4(fold + 2 * C + c4 * 4);
                            c.x += pc.x; c.y += pc.y; c.z += pc.z; c.w += pc.w;
                        }
                        ST4(fold + 2 * C + c4 * 4) = c;
                    }
                }
            }
        }
        __syncthreads();
    }
    constexpr int PARTS = COLSUM ? 3 : 2;
    float *dst = partial + (size_t)blockIdx.x * PARTS * C;
    for (int i = threadIdx.x; i < PARTS * C; i += blockDim.x) dst[i] = fold[i];
}

// Any C: block per row, parameter-gradient partials through atomics on a
// [PARTS][2C] scratch (rows hashed to parts) -- only ragged test shapes get here.
__global__ void layernorm_bwd_block_k(float *__restrict__ dinp, float *__restrict__ partial, int parts,
                                      const float *__restrict__ dout, const float *__restrict__ inp,
                                      const float *__restrict__ weight, const float *__restrict__ mean,
                                      const float *__restrict__ rstd, int C, int rnd) {
    __shared__ float red[32];
    const int row = blockIdx.x;
    const float *x = inp + (size_t)row * C, *dy = dout + (size_t)row * C;
    float *dx = dinp + (size_t)row * C;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
        const float xh = (x[i] - mu) * rs, d = dy[i] * weight[i];
        s1 += d; s2 += d * xh;
    }
    const float m1 = block_reduce<false>(s1, red) / C;
    const float m2 = block_reduce<false>(s2, red) / C;
    float *p = partial + (size_t)(row % parts) * 2 * C;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
        const float xh = (x[i] - mu) * rs, d = dy[i] * weight[i];
        dx[i] = rnd1(dx[i] + rs * (d - m1 - xh * m2), rnd);
        atomicAdd(&p[i], dy[i] * xh);
        atomicAdd(&p[C + i], dy[i]);
    }
}

// dst[c] += sum_{g < G} partial[g][c]   for c < ncols, in a fixed order: a block
// covers 32 columns, its 32 warps each sum every 32nd row of `partial`, and the 32
// sub-sums are added in warp order.  If dst2 != nullptr the columns
// [ncols_first, ncols) go to dst2; if dst3 != nullptr those from 2 * ncols_first on go to dst3.
__device__ __forceinline__ void column_add_body(float *__restrict__ dst, float *__restrict__ dst2, int ncols_first,
                                                const float *__restrict__ partial, int G, int ncols, float *__restrict__ dst3,
                                                int block_x, float (*red)[33]) {
    const int cx = threadIdx.x & 31, gy = threadIdx.x >> 5;
    const int c = block_x * 32 + cx;
    // 32 warps share the G rows; four loads are in flight per thread before the first add
    float s = 0.0f;
    if (c < ncols) {
        int g = gy;
        for (; g + 96 < G; g += 128) {
            const float a0 = partial[(size_t)g * ncols + c], a1 = partial[(size_t)(g + 32) * ncols + c];
            const float a2 = partial[(size_t)(g + 64) * ncols + c], a3 = partial[(size_t)(g + 96) * ncols + c];
            s += a0; s += a1; s += a2; s += a3;
        }
        for (; g < G; g += 32) s += partial[(size_t)g * ncols + c];
    }
    red[gy][cx] = s;
    __syncthreads();
    if (gy == 0 && c < ncols) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) t += red[i][cx];
        if (dst3 && c >= 2 * ncols_first) dst3[c - 2 * ncols_first] += t;
        else if (dst2 && c >= ncols_first) dst2[c - ncols_first] += t;
        else dst[c] += t;
    }
}
__global__ void __launch_bounds__(1024)
column_add_k(float *__restrict__ dst, float *__restrict__ dst2, int ncols_first,
             const float *__restrict__ partial, int G, int ncols, float *__restrict__ dst3 = nullptr) {
    __shared__ float red[32][33];
    column_add_body(dst, dst2, ncols_first, partial, G, ncols, dst3, (int)blockIdx.x, red);
}
// The same sum for a list of jobs (blockIdx.y), each over its own partial rows.
__global__ void __launch_bounds__(1024) column_add_jobs_k(const ColumnAddJob *__restrict__ jobs) {
    __shared__ float red[32][33];
    const ColumnAddJob j = jobs[blockIdx.y];
    if ((int)blockIdx.x * 32 >= j.ncols) return;          // (uniform per block)
    column_add_body(j.dst, j.dst2, j.ncols_first, j.partial, j.G, j.ncols, j.dst3, (int)blockIdx.x, red);
}

// --------------------------------------------------------------------- gelu
// tanh-approximation GELU with the accurate tanhf (src/nn.cu:118-150).
__device__ __forceinline__ float gelu1(float x) { return gelu_tanh(x); }
__device__ __forceinline__ float dgelu1(float x, float g) {
    const float s = 0.7978845608028654f;
    const float inner = s * (x + 0.044715f * x * x * x);
    const float t = tanhf(inner);
    const float sech2 = 1.0f - t * t;
    const float dinner = s * (1.0f + 3.0f * 0.044715f * x * x);
    return g * (0.5f * (1.0f + t) + 0.5f * x * sech2 * dinner);
}

__global__ void gelu_fwd_k(float *__restrict__ out, const float *__restrict__ inp, long long n4, int rnd) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        float4 v = LD4(inp + i * 4);
        v.x = gelu1(v.x); v.y = gelu1(v.y); v.z = gelu1(v.z); v.w = gelu1(v.w);
        ST4(out + i * 4) = rnd4(v, rnd);
    }
}
__global__ void gelu_bwd_k(float *__restrict__ dinp, const float *__restrict__ inp,
                           const float *__restrict__ dout, long long n4, int rnd) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 x = LD4(inp + i * 4), g = LD4(dout + i * 4);
        float4 d;
        d.x = dgelu1(x.x, g.x); d.y = dgelu1(x.y, g.y); d.z = dgelu1(x.z, g.z); d.w = dgelu1(x.w, g.w);
        ST4(dinp + i * 4) = rnd4(d, rnd);
    }
}

// element-wise forms for operands that are not 16-byte aligned or whose count is not a multiple of 4
__global__ void gelu_fwd_scalar_k(float *__restrict__ out, const float *__restrict__ inp, long long n, int rnd) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float g = gelu1(inp[i]);
        out[i] = rnd ? round_tf32(g) : g;
    }
}
__global__ void gelu_bwd_scalar_k(float *__restrict__ dinp, const float *__restrict__ inp, const float *__restrict__ dout,
                                  long long n, int rnd) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float d = dgelu1(inp[i], dout[i]);
        dinp[i] = rnd ? round_tf32(d) : d;
    }
}

// ------------------------------------------------------- residual and bias
__global__ void add3_k(float *__restrict__ out, const float *__restrict__ a,
                       const float *__restrict__ b, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 x = LD4(a + i * 4), y = LD4(b + i * 4);
        ST4(out + i * 4) = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
}
__global__ void add3_scalar_k(float *__restrict__ out, const float *__restrict__ a, const float *__restrict__ b, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = a[i] + b[i];
}
__global__ void bias_fwd_k(float *__restrict__ out, const float *__restrict__ bias, int C,
                           long long n4, int rnd) {
    const int C4 = C >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % C4) * 4;
        float4 v = LD4(out + i * 4);
        const float4 b = LD4(bias + c);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        ST4(out + i * 4) = rnd4(v, rnd);
    }
}
// Column sums of dout (N x C): blockIdx.x picks a strip of 256 float4 columns,
// blockIdx.y a residue class of rows; partial[blockIdx.y][C].
__global__ void __launch_bounds__(256)
bias_bwd_partial_k(float *__restrict__ partial, const float *__restrict__ dout, int N, int C) {
    const int c4 = blockIdx.x * 256 + threadIdx.x;
    if (c4 * 4 >= C) return;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    // rows n = blockIdx.y + k*gridDim.y, four loads in flight at a time, summed in row order
    const int step = gridDim.y;
    int n = blockIdx.y;
    for (; n + 3 * step < N; n += 4 * step) {
        const float4 g0 = LD4(dout + (size_t)n * C + c4 * 4);
        const float4 g1 = LD4(dout + (size_t)(n + step) * C + c4 * 4);
        const float4 g2 = LD4(dout + (size_t)(n + 2 * step) * C + c4 * 4);
        const float4 g3 = LD4(dout + (size_t)(n + 3 * step) * C + c4 * 4);
        s.x += g0.x; s.y += g0.y; s.z += g0.z; s.w += g0.w;
        s.x += g1.x; s.y += g1.y; s.z += g1.z; s.w += g1.w;
        s.x += g2.x; s.y += g2.y; s.z += g2.z; s.w += g2.w;
        s.x += g3.x; s.y += g3.y; s.z += g3.z; s.w += g3.w;
    }
    for (; n < N; n += step) {
        const float4 g = LD4(dout + (size_t)n * C + c4 * 4);
        s.x += g.x; s.y += g.y; s.z += g.z; s.w += g.w;
    }
    ST4(partial + (size_t)blockIdx.y * C + c4 * 4) = s;
}
// GELU backward over an (N x C) matrix that also leaves the column sums of its result (the bias
// gradient of the projection that produced the GELU input) in partial[blockIdx.y][C]: the grid is
// that of bias_bwd_partial_k, each thread walks its float4 column down a residue class of rows.
__global__ void __launch_bounds__(256)
gelu_bwd_colsum_k(float *__restrict__ partial, float *__restrict__ dinp, const float *__restrict__ inp,
                  const float *__restrict__ dout, int N, int C, int rnd) {
    const int c4 = blockIdx.x * 256 + threadIdx.x;
    if (c4 * 4 >= C) return;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    const int step = gridDim.y;
    int n = blockIdx.y;
    for (; n + step < N; n += 2 * step) {          // two rows in flight
        const size_t o0 = (size_t)n * C + c4 * 4, o1 = (size_t)(n + step) * C + c4 * 4;
        const float4 x0 = LD4(inp + o0), g0 = LD4(dout + o0), x1 = LD4(inp + o1), g1 = LD4(dout + o1);
        float4 d0, d1;
        d0.x = dgelu1(x0.x, g0.x); d0.y = dgelu1(x0.y, g0.y); d0.z = dgelu1(x0.z, g0.z); d0.w = dgelu1(x0.w, g0.w);
        d1.x = dgelu1(x1.x, g1.x); d1.y = dgelu1(x1.y, g1.y); d1.z = dgelu1(x1.z, g1.z); d1.w = dgelu1(x1.w, g1.w);
        d0 = rnd4(d0, rnd); d1 = rnd4(d1, rnd);
        ST4(dinp + o0) = d0; ST4(dinp + o1) = d1;
        s.x += d0.x; s.y += d0.y; s.z += d0.z; s.w += d0.w;
        s.x += d1.x; s.y += d1.y; s.z += d1.z; s.w += d1.w;
    }
    for (; n < N; n += step) {
        const size_t o0 = (size_t)n * C + c4 * 4;
        const float4 x0 = LD4(inp + o0), g0 = LD4(dout + o0);
        float4 d0;
        d0.x = dgelu1(x0.x, g0.x); d0.y = dgelu1(x0.y, g0.y); d0.z = dgelu1(x0.z, g0.z); d0.w = dgelu1(x0.w, g0.w);
        d0 = rnd4(d0, rnd);
        ST4(dinp + o0) = d0;
        s.x += d0.x; s.y += d0.y; s.z += d0.z; s.w += d0.w;
    }
    ST4(partial + (size_t)blockIdx.y * C + c4 * 4) = s;
}
__global__ void bias_bwd_scalar_k(float *__restrict__ dbias, const float *__restrict__ dout, int N,
                                  int C) {
    __shared__ float red[32];
    const int c = blockIdx.x;
    float acc = 0.0f;
    for (int n = threadIdx.x; n < N; n += blockDim.x) acc += dout[(size_t)n * C + c];
    acc = block_reduce<false>(acc, red);
    if (threadIdx.x == 0) dbias[c] += acc;
}

// ------------------------------------------------------- softmax + xent
// One block per row (src/nn.cu:197-221): max over the V real columns, then
// p = __expf(x - max) / sum, zeros in [V, Vp), loss = -logf(max(p[target], 1e-30)).
// The row is read from DRAM once; the second and third sweeps are served by
// L2, which holds every row in flight (2 blocks x 1024 threads per SM).
// GRAD = true writes the gradient of the mean loss with respect to the logits,
// (p - onehot) * grad_scale (optionally TF32-rounded), where GRAD = false writes p: the training
// step then needs no separate backward sweep over the (N, Vp) matrix.
template <bool GRAD>
__global__ void __launch_bounds__(1024)
softmax_xent_fwd_k(float *__restrict__ probs, float *__restrict__ losses,
                   const float *__restrict__ logits, const int *__restrict__ targets, int V,
                   int Vp, float grad_scale, int rnd) {
    __shared__ float red[32];
    const int row = blockIdx.x;
    const int tgt = targets[row];
    const float *x = logits + (size_t)row * Vp;
    float *p = probs + (size_t)row * Vp;
    const bool vec = (Vp & 3) == 0;
    const int Vp4 = Vp >> 2;

    float m = -FLT_MAX;
    if (vec) {
        for (int i = threadIdx.x; i < Vp4; i += blockDim.x) {
            const float4 v = LD4(x + i * 4);
            const int c = i * 4;
            if (c + 0 < V) m = fmaxf(m, v.x);
            if (c + 1 < V) m = fmaxf(m, v.y);
            if (c + 2 < V) m = fmaxf(m, v.z);
            if (c + 3 < V) m = fmaxf(m, v.w);
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, x[i]);
    }
    m = block_reduce<true>(m, red);

    float s = 0.0f;
    if (vec) {
        for (int i = threadIdx.x; i < Vp4; i += blockDim.x) {
            const float4 v = LD4(x + i * 4);
            const int c = i * 4;
            if (c + 0 < V) s += __expf(v.x - m);
            if (c + 1 < V) s += __expf(v.y - m);
            if (c + 2 < V) s += __expf(v.z - m);
            if (c + 3 < V) s += __expf(v.w - m);
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(x[i] - m);
    }
    s = block_reduce<false>(s, red);
    const float inv = 1.0f / s;

    if (vec) {
        for (int i = threadIdx.x; i < Vp4; i += blockDim.x) {
            const float4 v = LD4(x + i * 4);
            const int c = i * 4;
            float4 o;
            o.x = (c + 0 < V) ? __expf(v.x - m) * inv : 0.0f;
            o.y = (c + 1 < V) ? __expf(v.y - m) * inv : 0.0f;
            o.z = (c + 2 < V) ? __expf(v.z - m) * inv : 0.0f;
            o.w = (c + 3 < V) ? __expf(v.w - m) * inv : 0.0f;
            if (GRAD) {
                o.x = (c + 0 < V) ? (o.x - (c + 0 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
                o.y = (c + 1 < V) ? (o.y - (c + 1 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
                o.z = (c + 2 < V) ? (o.z - (c + 2 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
                o.w = (c + 3 < V) ? (o.w - (c + 3 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
                o = rnd4(o, rnd);
            }
            ST4(p + i * 4) = o;
        }
    } else {
        for (int i = threadIdx.x; i < Vp; i += blockDim.x) {
            float o = (i < V) ? __expf(x[i] - m) * inv : 0.0f;
            if (GRAD) o = rnd1((i < V) ? (o - (i == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f, rnd);
            p[i] = o;
        }
    }
    if (threadIdx.x == 0) {
        const int t = tgt;
        const float pt = __expf(x[t] - m) * inv;
        losses[row] = -logf(fmaxf(pt, 1e-30f));
    }
}

// The training step's classifier: loss and dlogits = (softmax(x) - onehot) * grad_scale, one block per row,
// Vp % 4 == 0.  Two sweeps instead of three: the first (the one that comes from DRAM) keeps a running
// maximum and a running sum of exponentials per thread (the sum is rescaled whenever the maximum moves),
// the second re-reads the row from L2 and writes the gradient with streaming stores, so that the 1.65 GB
// of output does not push the rows still waiting for their second sweep out of L2.
__global__ void __launch_bounds__(1024)
softmax_xent_grad_k(float *__restrict__ dlogits, float *__restrict__ losses, const float *__restrict__ logits,
                    const int *__restrict__ targets, int V, int Vp, float grad_scale, int rnd) {
    __shared__ float red[32];
    const int row = blockIdx.x;
    const int tgt = targets[row];
    const float *x = logits + (size_t)row * Vp;
    float *p = dlogits + (size_t)row * Vp;
    const int Vp4 = Vp >> 2;
    float m = -FLT_MAX, s = 0.0f;
    for (int i = threadIdx.x; i < Vp4; i += blockDim.x) {
        float4 v = LD4(x + i * 4);
        const int c = i * 4;
        if (c + 3 >= V) {                      // the row's last real columns (and the padding after them)
            if (c + 0 >= V) v.x = -FLT_MAX;
            if (c + 1 >= V) v.y = -FLT_MAX;
            if (c + 2 >= V) v.z = -FLT_MAX;
            if (c + 3 >= V) v.w = -FLT_MAX;
        }
        const float mn = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
        s = s * __expf(m - mn) + ((__expf(v.x - mn) + __expf(v.y - mn)) + (__expf(v.z - mn) + __expf(v.w - mn)));
        m = mn;
    }
    const float M = block_reduce<true>(m, red);
    s = block_reduce<false>(s * __expf(m - M), red);
    const float inv = 1.0f / s;
    for (int i = threadIdx.x; i < Vp4; i += blockDim.x) {
        const float4 v = LD4(x + i * 4);
        const int c = i * 4;
        float4 o;
        o.x = (c + 0 < V) ? (__expf(v.x - M) * inv - (c + 0 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
        o.y = (c + 1 < V) ? (__expf(v.y - M) * inv - (c + 1 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
        o.z = (c + 2 < V) ? (__expf(v.z - M) * inv - (c + 2 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
        o.w = (c + 3 < V) ? (__expf(v.w - M) * inv - (c + 3 == tgt ? 1.0f : 0.0f)) * grad_scale : 0.0f;
        __stcs(reinterpret_cast<float4 *>(p + i * 4), rnd4(o, rnd));
    }
    if (threadIdx.x == 0) {
        const float pt = __expf(x[tgt] - M) * inv;
        losses[row] = -logf(fmaxf(pt, 1e-30f));
    }
}

// dlogits = (p - onehot) * scale on real columns, 0 on padding (src/nn.cu:226-237).
__global__ void xent_bwd_k(float *__restrict__ dlogits, const float *__restrict__ probs,
                           const int *__restrict__ targets, int V, int Vp, float scale,
                           long long n4, int rnd) {
    const int Vp4 = Vp >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / Vp4;
        const int c = (int)(i - row * Vp4) * 4;
        const int t = targets[row];
        const float4 p = LD4(probs + i * 4);
        float4 d;
        d.x = (c + 0 < V) ? (p.x - (c + 0 == t ? 1.0f : 0.0f)) * scale : 0.0f;
        d.y = (c + 1 < V) ? (p.y - (c + 1 == t ? 1.0f : 0.0f)) * scale : 0.0f;
        d.z = (c + 2 < V) ? (p.z - (c + 2 == t ? 1.0f : 0.0f)) * scale : 0.0f;
        d.w = (c + 3 < V) ? (p.w - (c + 3 == t ? 1.0f : 0.0f)) * scale : 0.0f;
        ST4(dlogits + i * 4) = rnd4(d, rnd);
    }
}
__global__ void xent_bwd_scalar_k(float *__restrict__ dlogits, const float *__restrict__ probs,
                                  const int *__restrict__ targets, int V, int Vp, float scale, int rnd) {
    const int row = blockIdx.x;
    const float *p = probs + (size_t)row * Vp;
    float *d = dlogits + (size_t)row * Vp;
    const int t = targets[row];
    for (int i = threadIdx.x; i < Vp; i += blockDim.x)
        d[i] = rnd1((i < V) ? (p[i] - (i == t ? 1.0f : 0.0f)) * scale : 0.0f, rnd);
}

// ---------------------------------------------------------------- optimizer
// AdamW exactly as src/nn.cu:240-254: decay on every parameter, bias
// corrections passed in, gradient pre-multiplied by gscale.
__device__ __forceinline__ float adamw1(float p, float g, float &m, float &v, float lr, float b1,
                                        float b2, float eps, float wd, float bc1, float bc2) {
    const float mi = b1 * m + (1.0f - b1) * g;
    const float vi = b2 * v + (1.0f - b2) * g * g;
    m = mi; v = vi;
    const float mhat = mi / bc1, vhat = vi / bc2;
    return p - lr * (mhat / (sqrtf(vhat) + eps) + wd * p);
}

// d_sumsq == nullptr: gscale is used as given.  Otherwise the clip rule of
// src/train_gpt.cu:442-448 is evaluated from the device-resident squared norm.
__global__ void adamw_k(float *__restrict__ params, const float *__restrict__ grads,
                        float *__restrict__ m, float *__restrict__ v, size_t n, float lr, float b1,
                        float b2, float eps, float wd, float bc1, float bc2, float gscale,
                        const double *__restrict__ d_sumsq, float clip, float div,
                        float *__restrict__ shadow) {
    if (d_sumsq) {
        const float gn = (float)sqrt(*d_sumsq) / div;
        gscale = ((gn > clip) ? clip / gn : 1.0f) / div;
    }
    const size_t n4 = n >> 2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4;
         i += (size_t)gridDim.x * blockDim.x) {
        float4 p = LD4(params + i * 4), mm = LD4(m + i * 4), vv = LD4(v + i * 4);
        const float4 g = LD4(grads + i * 4);
        p.x = adamw1(p.x, g.x * gscale, mm.x, vv.x, lr, b1, b2, eps, wd, bc1, bc2);
        p.y = adamw1(p.y, g.y * gscale, mm.y, vv.y, lr, b1, b2, eps, wd, bc1, bc2);
        p.z = adamw1(p.z, g.z * gscale, mm.z, vv.z, lr, b1, b2, eps, wd, bc1, bc2);
        p.w = adamw1(p.w, g.w * gscale, mm.w, vv.w, lr, b1, b2, eps, wd, bc1, bc2);
        ST4(params + i * 4) = p; ST4(m + i * 4) = mm; ST4(v + i * 4) = vv;
        if (shadow)
            ST4(shadow + i * 4) = make_float4(round_tf32(p.x), round_tf32(p.y), round_tf32(p.z), round_tf32(p.w));
    }
    // tail (n % 4 elements)
    const size_t t = n4 * 4 + blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (t < n) {
        float mm = m[t], vv = v[t];
        const float p = adamw1(params[t], grads[t] * gscale, mm, vv, lr, b1, b2, eps, wd, bc1, bc2);
        params[t] = p; m[t] = mm; v[t] = vv;
        if (shadow) shadow[t] = round_tf32(p);
    }
}

// Sum of squares: per-block float partials (src/nn.cu:258-267), finished in
// double by one block so that the value never leaves the device.
__global__ void __launch_bounds__(256)
sumsq_partial_k(const float *__restrict__ g, float *__restrict__ partial, size_t n) {
    __shared__ float red[32];
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    const size_t n4 = ((uintptr_t)g % 16 == 0) ? (n >> 2) : 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4;
         i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = LD4(g + i * 4);
        a0 += v.x * v.x; a1 += v.y * v.y; a2 += v.z * v.z; a3 += v.w * v.w;
    }
    for (size_t i = n4 * 4 + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        a0 += g[i] * g[i];
    const float s = block_reduce<false>((a0 + a1) + (a2 + a3), red);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256)
sumsq_finish_k(const float *__restrict__ partial, int nparts, double *__restrict__ out) {
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

__global__ void __launch_bounds__(1024) reduce_mean_k(const float *__restrict__ in, float *__restrict__ out, int n) {
    __shared__ float red[32];
    float acc = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += in[i];
    acc = block_reduce<false>(acc, red);
    if (threadIdx.x == 0) *out = acc / n;
}

__global__ void round_tf32_k(float *__restrict__ dst, const float *__restrict__ src, size_t n) {
    const bool vec = (((uintptr_t)dst | (uintptr_t)src) % 16) == 0;
    const size_t n4 = vec ? (n >> 2) : 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4;
         i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = LD4(src + i * 4);
        ST4(dst + i * 4) = make_float4(round_tf32(v.x), round_tf32(v.y), round_tf32(v.z), round_tf32(v.w));
    }
    for (size_t i = n4 * 4 + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = round_tf32(src[i]);
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

static thread_local ColumnAddCollector *g_collector = nullptr;
void set_column_add_collector(ColumnAddCollector *c) { g_collector = c; }
int launch_column_add_jobs(const ColumnAddJob *jobs_dev, int njobs, int max_cols, cudaStream_t st) {
    if (njobs <= 0) return BMB_OK;
    column_add_jobs_k<<<dim3(ceil_div(max_cols, 32), njobs), 1024, 0, st>>>(jobs_dev);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
namespace {
// Partial rows for a two-stage sum: from the installed collector's arena, else from the per-device scratch.
// *deferred says which; a full arena or job list falls back to the scratch (and an immediate sum) for that call.
float *partial_rows(size_t floats, bool *deferred) {
    ColumnAddCollector *cc = g_collector;
    *deferred = false;
    if (cc && cc->njobs < cc->max_jobs) {
        const size_t need = (floats + 3) & ~(size_t)3;
        if (cc->used + need <= cc->cap) {
            float *p = cc->arena + cc->used;
            cc->used += need;
            *deferred = true;
            return p;
        }
    }
    return (float *)device_scratch(SCR_REDUCE, floats * sizeof(float));
}
// Finish a two-stage sum now, or note it for the batched launch.
int finish_column_sum(bool deferred, float *dst, float *dst2, int ncols_first, const float *partial, int G, int ncols,
                      cudaStream_t st, float *dst3 = nullptr);
}  // namespace

// Shared with other translation units of the library.
int launch_column_add(float *dst, float *dst2, int ncols_first, const float *partial, int G,
                      int ncols, cudaStream_t st, float *dst3 = nullptr) {
    column_add_k<<<ceil_div(ncols, 32), 1024, 0, st>>>(dst, dst2, ncols_first, partial, G, ncols, dst3);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

namespace {
int finish_column_sum(bool deferred, float *dst, float *dst2, int ncols_first, const float *partial, int G, int ncols,
                      cudaStream_t st, float *dst3) {
    if (!deferred) return launch_column_add(dst, dst2, ncols_first, partial, G, ncols, st, dst3);
    ColumnAddCollector *cc = g_collector;
    if (cc->record) cc->jobs[cc->njobs] = ColumnAddJob{dst, dst2, dst3, partial, ncols_first, G, ncols};
    cc->njobs++;
    if (ncols > cc->max_cols) cc->max_cols = ncols;
    return BMB_OK;
}
}  // namespace

// Column sums whose partial rows another kernel's epilogue leaves (the attention backward, for the qkv bias): where
// those rows go (the deferred-sum arena while a collector is installed, else per-device scratch) and how the sum into
// dst (+=) is finished (noted for the batched launch, or launched now).
float *column_partial_rows(size_t floats, bool *deferred) { return partial_rows(floats, deferred); }
int column_sum_finish(bool deferred, float *dst, const float *partial, int G, int ncols, cudaStream_t st) {
    return finish_column_sum(deferred, dst, nullptr, ncols, partial, G, ncols, st);
}

// Layernorm backward with the scratch supplied by the caller: `partial` holds
// at least layernorm_bwd_blocks(N) * 2 * C floats.
int layernorm_bwd_blocks(int N) {
    int g = ceil_div(N, 4);
    const int cap = 3 * sm_count();     // 128-thread blocks, three resident per SM
    return g > cap ? cap : (g < 1 ? 1 : g);
}
// dcolsum != nullptr: also dcolsum += column sums of the updated dinp; `partial` then holds
// G * 3 * C floats.
int layernorm_backward_with_scratch(float *dinp, float *dweight, float *dbias, const float *dout,
                                    const float *inp, const float *weight, const float *mean,
                                    const float *rstd, int N, int C, float *partial, int G,
                                    cudaStream_t st, float *dcolsum = nullptr, bool deferred = false) {
    const int rnd = emit_rounded() ? 1 : 0;
    // registers follow the row length: V4 float4 per lane cover C <= 128 * V4
#define BMB_LN_BWD(V4_)                                                                                                   \
    do {                                                                                                                  \
        if (dcolsum) layernorm_bwd_warp_k<V4_, true><<<G, 128, 3 * C * sizeof(float), st>>>(dinp, partial, dout, inp, weight, mean, rstd, N, C, rnd); \
        else layernorm_bwd_warp_k<V4_, false><<<G, 128, 2 * C * sizeof(float), st>>>(dinp, partial, dout, inp, weight, mean, rstd, N, C, rnd);        \
    } while (0)
    if (C <= 256) BMB_LN_BWD(2);
    else if (C <= 512) BMB_LN_BWD(4);
    else if (C <= 768) BMB_LN_BWD(6);
    else BMB_LN_BWD(8);
#undef BMB_LN_BWD
    count_launch();
    BMB_LAUNCH_CHECK();
    return finish_column_sum(deferred, dweight, dbias, C, partial, G, (dcolsum ? 3 : 2) * C, st, dcolsum);
}

}  // namespace bmb

using namespace bmb;

extern "C" {

int bmb_encoder_forward(float *out, const int *tokens, const float *wte, const float *wpe, int B,
                        int T, int C) {
    if (C % 4) return fail(BMB_E_ARG, "encoder_forward: C=%d must be a multiple of 4", C);
    if (!aligned16(out) || !aligned16(wte) || !aligned16(wpe)) return fail(BMB_E_ARG, "encoder_forward: out, wte and wpe must be 16-byte aligned");
    const long long n4 = (long long)B * T * C / 4;
    if (n4 == 0) return BMB_OK;
    encoder_fwd_k<<<grid_for(n4, 256, 8), 256, 0, cur_stream()>>>(out, tokens, wte, wpe, T, C, n4);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_encoder_backward(float *dwte, float *dwpe, const float *dout, const int *tokens, int B,
                         int T, int C) {
    if (C % 4) return fail(BMB_E_ARG, "encoder_backward: C=%d must be a multiple of 4", C);
    if (!aligned16(dwte) || !aligned16(dwpe) || !aligned16(dout)) return fail(BMB_E_ARG, "encoder_backward: dwte, dwpe and dout must be 16-byte aligned");
    const long long n4 = (long long)B * T * C / 4;
    if (n4 == 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    encoder_bwd_wpe_k<<<grid_for((long long)T * C / 4, 256, 8), 256, 0, st>>>(dwpe, dout, B, T, C);
    encoder_bwd_wte_k<<<grid_for(n4, 256, 8), 256, 0, st>>>(dwte, dout, tokens, C, n4);
    count_launch(2);
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_layernorm_forward(float *out, float *mean, float *rstd, const float *inp,
                          const float *weight, const float *bias, int N, int C) {
    if (N <= 0 || C <= 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    const bool fast = (C % 4 == 0) && C <= 1024 && aligned16(out) && aligned16(inp) &&
                      aligned16(weight) && aligned16(bias);
    if (fast) {
        int g = ceil_div(N, 8);
        const int cap = sm_count() * 8;
        if (g > cap) g = cap;
        const int rnd = emit_rounded() ? 1 : 0;
        if (C <= 256) layernorm_fwd_warp_k<2><<<g, 256, 0, st>>>(out, mean, rstd, inp, weight, bias, N, C, rnd);
        else if (C <= 512) layernorm_fwd_warp_k<4><<<g, 256, 0, st>>>(out, mean, rstd, inp, weight, bias, N, C, rnd);
        else if (C <= 768) layernorm_fwd_warp_k<6><<<g, 256, 0, st>>>(out, mean, rstd, inp, weight, bias, N, C, rnd);
        else layernorm_fwd_warp_k<8><<<g, 256, 0, st>>>(out, mean, rstd, inp, weight, bias, N, C, rnd);
    } else {
        layernorm_fwd_block_k<<<N, 128, 0, st>>>(out, mean, rstd, inp, weight, bias, C, emit_rounded() ? 1 : 0);
    }
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_residual_layernorm_forward(float *sum_out, float *out, float *mean, float *rstd, const float *a,
                                   const float *b, const float *weight, const float *bias, int N, int C) {
    if (N <= 0 || C <= 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    const bool fast = (C % 4 == 0) && C <= 1024 && aligned16(out) && aligned16(a) && aligned16(b) &&
                      aligned16(sum_out) && aligned16(weight) && aligned16(bias);
    if (!fast) {
        const long long n = (long long)N * C;
        add3_scalar_k<<<grid_for(n, 256, 8), 256, 0, st>>>(sum_out, a, b, n);
        count_launch();
        BMB_LAUNCH_CHECK();
        return bmb_layernorm_forward(out, mean, rstd, sum_out, weight, bias, N, C);
    }
    int g = ceil_div(N, 8);
    const int cap = sm_count() * 8;
    if (g > cap) g = cap;
    const int rnd = emit_rounded() ? 1 : 0;
    if (C <= 256) layernorm_fwd_warp_k<2><<<g, 256, 0, st>>>(out, mean, rstd, a, weight, bias, N, C, rnd, b, sum_out);
    else if (C <= 512) layernorm_fwd_warp_k<4><<<g, 256, 0, st>>>(out, mean, rstd, a, weight, bias, N, C, rnd, b, sum_out);
    else if (C <= 768) layernorm_fwd_warp_k<6><<<g, 256, 0, st>>>(out, mean, rstd, a, weight, bias, N, C, rnd, b, sum_out);
    else layernorm_fwd_warp_k<8><<<g, 256, 0, st>>>(out, mean, rstd, a, weight, bias, N, C, rnd, b, sum_out);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_layernorm_backward_colsum(float *dinp, float *dweight, float *dbias, float *dcolsum, const float *dout,
                                  const float *inp, const float *weight, const float *mean,
                                  const float *rstd, int N, int C) {
    if (N <= 0 || C <= 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    const bool fast = (C % 4 == 0) && C <= 1024 && aligned16(dinp) && aligned16(inp) &&
                      aligned16(dout) && aligned16(weight);
    if (!fast || !dcolsum) {
        BMB_TRY(bmb_layernorm_backward(dinp, dweight, dbias, dout, inp, weight, mean, rstd, N, C));
        return dcolsum ? bmb_bias_backward(dcolsum, dinp, N, C) : BMB_OK;
    }
    const int G = layernorm_bwd_blocks(N);
    bool deferred = false;
    float *partial = partial_rows((size_t)G * 3 * C, &deferred);
    if (!partial) return BMB_E_CUDA;
    return layernorm_backward_with_scratch(dinp, dweight, dbias, dout, inp, weight, mean, rstd, N, C, partial, G, st, dcolsum, deferred);
}

int bmb_layernorm_backward(float *dinp, float *dweight, float *dbias, const float *dout,
                           const float *inp, const float *weight, const float *mean,
                           const float *rstd, int N, int C) {
    if (N <= 0 || C <= 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    const bool fast = (C % 4 == 0) && C <= 1024 && aligned16(dinp) && aligned16(inp) &&
                      aligned16(dout) && aligned16(weight);
    if (fast) {
        const int G = layernorm_bwd_blocks(N);
        bool deferred = false;
        float *partial = partial_rows((size_t)G * 2 * C, &deferred);
        if (!partial) return BMB_E_CUDA;
        return layernorm_backward_with_scratch(dinp, dweight, dbias, dout, inp, weight, mean, rstd, N,
                                               C, partial, G, st, nullptr, deferred);
    }
    const int parts = 32;
    float *partial = (float *)device_scratch(SCR_REDUCE, (size_t)parts * 2 * C * sizeof(float));
    if (!partial) return BMB_E_CUDA;
    BMB_CUDA(cudaMemsetAsync(partial, 0, (size_t)parts * 2 * C * sizeof(float), st));
    layernorm_bwd_block_k<<<N, 128, 0, st>>>(dinp, partial, parts, dout, inp, weight, mean, rstd, C, emit_rounded() ? 1 : 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return launch_column_add(dweight, dbias, C, partial, parts, 2 * C, st);
}

}  // extern "C"

// ---- layernorm backward without any allocation ---------------------------------
// The two-stage parameter-gradient sum needs a block of per-CTA partial rows.
// bmb_layernorm_backward takes it from per-device scratch that is cudaMalloc'ed on
// first use; this variant keeps it in the library image instead: a fixed 4 MiB
// array in device memory (every GPU that loads libbmb.so holds it until exit).
namespace {
constexpr int NOALLOC_MAX_C = 1024;       // widest row served
constexpr int NOALLOC_MAX_BLOCKS = 512;   // most partial rows ever written
static __device__ __align__(256) float g_ln_noalloc_scratch[(size_t)NOALLOC_MAX_BLOCKS * 2 * NOALLOC_MAX_C];
float *g_ln_noalloc_ptr[64];              // device address of the array, per device, 0 = not looked up yet
std::mutex g_ln_noalloc_mu;
}  // namespace

extern "C" {

int bmb_layernorm_backward_noalloc(float *dinp, float *dweight, float *dbias, const float *dout,
                                   const float *inp, const float *weight, const float *mean,
                                   const float *rstd, int N, int C) {
    if (N <= 0 || C <= 0) return BMB_OK;
    if (C > NOALLOC_MAX_C)
        return fail(BMB_E_LIMIT, "layernorm_backward_noalloc: C=%d exceeds the built-in scratch (C <= %d)", C, NOALLOC_MAX_C);
    if (C % 4 != 0 || !aligned16(dinp) || !aligned16(inp) || !aligned16(dout) || !aligned16(weight))
        return fail(BMB_E_ARG, "layernorm_backward_noalloc: needs C %% 4 == 0 and 16-byte aligned buffers");
    const int dev = current_device();
    if (dev < 0 || dev >= 64) return fail(BMB_E_ARG, "device index %d out of range", dev);
    float *partial = nullptr;
    {
        // Set-up, once per device, with that device current: in host code the array's name is only a
        // stand-in, the kernel needs the address the runtime reports for this device.
        std::lock_guard<std::mutex> lk(g_ln_noalloc_mu);
        if (!g_ln_noalloc_ptr[dev]) {
            void *p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_ln_noalloc_scratch);
            if (e != cudaSuccess || !p)
                return fail(BMB_E_CUDA, "cudaGetSymbolAddress(layernorm scratch) -> %s", cudaGetErrorString(e));
            g_ln_noalloc_ptr[dev] = static_cast<float *>(p);
        }
        partial = g_ln_noalloc_ptr[dev];
    }
    int G = layernorm_bwd_blocks(N);
    if (G > NOALLOC_MAX_BLOCKS) G = NOALLOC_MAX_BLOCKS;   // the kernel strides rows over any grid
    // Every partial row that is read was written by this launch first, so nothing needs clearing.
    return layernorm_backward_with_scratch(dinp, dweight, dbias, dout, inp, weight, mean, rstd, N, C, partial, G,
                                           cur_stream());
}

int bmb_gelu_forward(float *out, const float *inp, int n) {
    if (n <= 0) return BMB_OK;
    if (n % 4 || !aligned16(out) || !aligned16(inp))
        gelu_fwd_scalar_k<<<grid_for(n, 256, 8), 256, 0, cur_stream()>>>(out, inp, n, emit_rounded() ? 1 : 0);
    else
        gelu_fwd_k<<<grid_for(n / 4, 256, 8), 256, 0, cur_stream()>>>(out, inp, n / 4, emit_rounded() ? 1 : 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
int bmb_gelu_backward(float *dinp, const float *inp, const float *dout, int n) {
    if (n <= 0) return BMB_OK;
    if (n % 4 || !aligned16(dinp) || !aligned16(inp) || !aligned16(dout))
        gelu_bwd_scalar_k<<<grid_for(n, 256, 8), 256, 0, cur_stream()>>>(dinp, inp, dout, n, emit_rounded() ? 1 : 0);
    else
        gelu_bwd_k<<<grid_for(n / 4, 256, 8), 256, 0, cur_stream()>>>(dinp, inp, dout, n / 4, emit_rounded() ? 1 : 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
int bmb_gelu_backward_colsum(float *dinp, float *dcolsum, const float *inp, const float *dout, int N, int C) {
    if (N <= 0 || C <= 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    if (C % 4 != 0 || !aligned16(dinp) || !aligned16(inp) || !aligned16(dout) || !dcolsum) {
        BMB_TRY(bmb_gelu_backward(dinp, inp, dout, N * C));
        return dcolsum ? bmb_bias_backward(dcolsum, dinp, N, C) : BMB_OK;
    }
    const int strips = ceil_div(C / 4, 256);
    int gy = (4 * sm_count()) / strips;
    if (gy < 1) gy = 1;
    if (gy > N) gy = N;
    bool deferred = false;
    float *partial = partial_rows((size_t)gy * C, &deferred);
    if (!partial) return BMB_E_CUDA;
    gelu_bwd_colsum_k<<<dim3(strips, gy), 256, 0, st>>>(partial, dinp, inp, dout, N, C, emit_rounded() ? 1 : 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return finish_column_sum(deferred, dcolsum, nullptr, C, partial, gy, C, st);
}
int bmb_residual_forward(float *out, const float *a, const float *b, int n) {
    if (n % 4) return fail(BMB_E_ARG, "residual_forward: n=%d must be a multiple of 4", n);
    if (!aligned16(out) || !aligned16(a) || !aligned16(b)) return fail(BMB_E_ARG, "residual_forward: the operands must be 16-byte aligned");
    if (n == 0) return BMB_OK;
    add3_k<<<grid_for(n / 4, 256, 8), 256, 0, cur_stream()>>>(out, a, b, n / 4);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
int bmb_add_inplace(float *dst, const float *src, int n) {
    return bmb_residual_forward(dst, dst, src, n);
}
int bmb_bias_forward(float *out, const float *bias, int N, int C) {
    if (C % 4) return fail(BMB_E_ARG, "bias_forward: C=%d must be a multiple of 4", C);
    if (!aligned16(out) || !aligned16(bias)) return fail(BMB_E_ARG, "bias_forward: out and bias must be 16-byte aligned");
    const long long n4 = (long long)N * C / 4;
    if (n4 == 0) return BMB_OK;
    bias_fwd_k<<<grid_for(n4, 256, 8), 256, 0, cur_stream()>>>(out, bias, C, n4, emit_rounded() ? 1 : 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
int bmb_bias_backward(float *dbias, const float *dout, int N, int C) {
    if (N <= 0 || C <= 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    if (C % 4 == 0 && aligned16(dout)) {
        const int strips = ceil_div(C / 4, 256);
        int gy = (2 * sm_count()) / strips;
        if (gy < 1) gy = 1;
        if (gy > N) gy = N;
        bool deferred = false;
        float *partial = partial_rows((size_t)gy * C, &deferred);
        if (!partial) return BMB_E_CUDA;
        bias_bwd_partial_k<<<dim3(strips, gy), 256, 0, st>>>(partial, dout, N, C);
        count_launch();
        BMB_LAUNCH_CHECK();
        return finish_column_sum(deferred, dbias, nullptr, C, partial, gy, C, st);
    }
    bias_bwd_scalar_k<<<C, 256, 0, st>>>(dbias, dout, N, C);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_softmax_crossentropy_forward(float *probs, float *losses, const float *logits,
                                     const int *targets, int N, int V, int Vp) {
    if (N <= 0) return BMB_OK;
    if (V <= 0 || V > Vp) return fail(BMB_E_ARG, "softmax_xent: need 0 < V <= Vp (V=%d Vp=%d)", V, Vp);
    softmax_xent_fwd_k<false><<<N, Vp >= 4096 ? 1024 : 128, 0, cur_stream()>>>(probs, losses, logits, targets, V, Vp, 0.0f, 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
int bmb_softmax_crossentropy_fused(float *dlogits, float *losses, const float *logits,
                                   const int *targets, int N, int V, int Vp, float dloss_scale) {
    if (N <= 0) return BMB_OK;
    if (V <= 0 || V > Vp) return fail(BMB_E_ARG, "softmax_xent: need 0 < V <= Vp (V=%d Vp=%d)", V, Vp);
    if (Vp % 4 == 0 && aligned16(dlogits) && aligned16(logits))
        softmax_xent_grad_k<<<N, Vp >= 4096 ? 1024 : 128, 0, cur_stream()>>>(dlogits, losses, logits, targets, V, Vp, dloss_scale,
                                                                              emit_rounded() ? 1 : 0);
    else
        softmax_xent_fwd_k<true><<<N, Vp >= 4096 ? 1024 : 128, 0, cur_stream()>>>(dlogits, losses, logits, targets, V, Vp, dloss_scale,
                                                                                   emit_rounded() ? 1 : 0);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
int bmb_crossentropy_softmax_backward(float *dlogits, const float *probs, const int *targets, int N,
                                      int V, int Vp, float dloss_scale) {
    if (N <= 0) return BMB_OK;
    cudaStream_t st = cur_stream();
    if (Vp % 4 == 0 && aligned16(dlogits) && aligned16(probs)) {
        const long long n4 = (long long)N * Vp / 4;
        xent_bwd_k<<<grid_for(n4, 256, 8), 256, 0, st>>>(dlogits, probs, targets, V, Vp, dloss_scale, n4, emit_rounded() ? 1 : 0);
    } else {
        xent_bwd_scalar_k<<<N, 128, 0, st>>>(dlogits, probs, targets, V, Vp, dloss_scale, emit_rounded() ? 1 : 0);
    }
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

static int adamw_launch(float *params, const float *grads, float *m, float *v, size_t n, float lr,
                        float beta1, float beta2, float eps, float wd, int step, float gscale,
                        const double *d_sumsq, float clip, float div, float *shadow) {
    if (n == 0) return BMB_OK;
    if (!aligned16(params) || !aligned16(grads) || !aligned16(m) || !aligned16(v) ||
        (shadow && !aligned16(shadow)))
        return fail(BMB_E_ARG, "adamw: buffers must be 16-byte aligned");
    const float bc1 = 1.0f - powf(beta1, (float)step);
    const float bc2 = 1.0f - powf(beta2, (float)step);
    const int grid = grid_for((long long)(n / 4 + 4), 256, 8);
    adamw_k<<<grid, 256, 0, cur_stream()>>>(params, grads, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2,
                                           gscale, d_sumsq, clip, div, shadow);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_adamw_update(float *params, float *grads, float *m, float *v, int n, float lr, float beta1,
                     float beta2, float eps, float weight_decay, int step, float grad_scale) {
    if (n < 0) return fail(BMB_E_ARG, "adamw: n < 0");
    return adamw_launch(params, grads, m, v, (size_t)n, lr, beta1, beta2, eps, weight_decay, step,
                        grad_scale, nullptr, 0.f, 1.f, nullptr);
}

int bmb_adamw_update_clipped(float *params, const float *grads, float *m, float *v, size_t n,
                             float lr, float beta1, float beta2, float eps, float weight_decay,
                             int step, const double *d_sumsq, float clip, float div, float *shadow) {
    if (!d_sumsq) return fail(BMB_E_ARG, "adamw_update_clipped: d_sumsq is null");
    return adamw_launch(params, grads, m, v, n, lr, beta1, beta2, eps, weight_decay, step, 1.0f,
                        d_sumsq, clip, div, shadow);
}

int bmb_grad_sumsq_device(const float *grads, size_t n, double *sumsq_out) {
    cudaStream_t st = cur_stream();
    const int nparts = 2 * sm_count();
    float *partial = (float *)device_scratch(SCR_MISC, 4096 * sizeof(float));
    if (!partial) return BMB_E_CUDA;
    sumsq_partial_k<<<nparts, 256, 0, st>>>(grads, partial, n);
    sumsq_finish_k<<<1, 256, 0, st>>>(partial, nparts, sumsq_out);
    count_launch(2);
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_grad_global_norm(const float *grads, int n, float *host_norm) {
    if (n < 0 || !host_norm) return fail(BMB_E_ARG, "grad_global_norm: bad argument");
    float *scr = (float *)device_scratch(SCR_MISC, 4096 * sizeof(float));
    if (!scr) return BMB_E_CUDA;
    double *d_out = reinterpret_cast<double *>(scr + 2048);
    BMB_TRY(bmb_grad_sumsq_device(grads, (size_t)n, d_out));
    double h = 0.0;
    BMB_CUDA(cudaMemcpyAsync(&h, d_out, sizeof(double), cudaMemcpyDeviceToHost, cur_stream()));
    BMB_CUDA(cudaStreamSynchronize(cur_stream()));
    *host_norm = (float)sqrt(h);
    return BMB_OK;
}

int bmb_zero_buffer(float *p, size_t n) {
    if (n == 0) return BMB_OK;
    BMB_CUDA(cudaMemsetAsync(p, 0, n * sizeof(float), cur_stream()));
    return BMB_OK;
}

int bmb_reduce_mean_device(const float *d_values, int n, float *d_mean) {
    if (n <= 0) return fail(BMB_E_ARG, "reduce_mean: n=%d", n);
    reduce_mean_k<<<1, 1024, 0, cur_stream()>>>(d_values, d_mean, n);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

int bmb_reduce_mean(const float *d_values, int n, float *host_mean) {
    if (!host_mean) return fail(BMB_E_ARG, "reduce_mean: null result pointer");
    float *scr = (float *)device_scratch(SCR_MISC, 4096 * sizeof(float));
    if (!scr) return BMB_E_CUDA;
    float *d_out = scr + 3072;
    BMB_TRY(bmb_reduce_mean_device(d_values, n, d_out));
    BMB_CUDA(cudaMemcpyAsync(host_mean, d_out, sizeof(float), cudaMemcpyDeviceToHost, cur_stream()));
    BMB_CUDA(cudaStreamSynchronize(cur_stream()));
    return BMB_OK;
}

int bmb_round_tf32(float *dst, const float *src, size_t n, void *stream) {
    if (n == 0) return BMB_OK;
    round_tf32_k<<<grid_for((long long)(n / 4 + 1), 256, 8), 256, 0, (cudaStream_t)stream>>>(dst, src, n);
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // extern "C"
