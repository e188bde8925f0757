// Fused causal attention, fp32 SIMT path (src/flash.h:36-62, src/flash.cu).
//
// The score matrix never reaches global memory: the forward walks key tiles
// with a running row max / row sum and writes out (B,T,C) plus
// lse = max + log(sum) (src/flash.cu:292-310); the backward rebuilds
// P = exp(S - lse) and uses  dS = P * (dP - D),  D = rowsum(dO * O)
// (src/flash.cu:447-453), in two kernels so that dQ (reduced over keys) and
// dK/dV (reduced over queries) each stay in registers and are written with
// plain stores -- dqkv is overwritten, not accumulated.
//
// Thread mapping ("row group"): a query row (or, in the dK/dV kernel, a key
// row) belongs to G = HS/32 adjacent lanes, each holding a 32-float slice of
// the head dimension in registers.  Key/value (or query/dO) rows are staged
// in shared memory and read as warp-wide broadcasts; dot products finish with
// log2(G) shuffles.  Scores are processed KC keys at a time so that the
// running max is rescaled once per chunk, not once per key.
// q, k and v are read straight out of the fused (B,T,3C) projection.
#include "common.cuh"
#include <cfloat>
#include <cmath>

namespace bmb {
bool flash_tc_supported(int T, int C, int NH, const float *qkv, const float *out);
int flash_forward_tc(float *out, float *lse, const float *qkv, int B, int T, int C, int NH, bool qkv_rounded,
                     cudaStream_t st);
int flash_backward_tc(float *dqkv, float *dsum, const float *dout, const float *qkv, const float *out,
                      const float *lse, int B, int T, int C, int NH, bool rounded, cudaStream_t st, float *dbias_qkv = nullptr);
namespace {

#define LD4(p) (*reinterpret_cast<const float4 *>(p))
#define ST4(p) (*reinterpret_cast<float4 *>(p))

constexpr int FT = 128;    // threads per block
// Rows staged per tile: 64, or 32 at head size 128 (static shared memory stays under 48 KB).
template <int HS> struct tile_rows { static constexpr int value = (HS >= 128) ? 32 : 64; };

template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = 1; o < G; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Copy TILE rows of HS floats (row r at src + r*ld) into dense smem [TILE][HS];
// rows at or beyond `valid` are zero filled.
template <int HS, int TILE>
__device__ __forceinline__ void stage_rows(float *__restrict__ dst, const float *__restrict__ src,
                                           long long ld, int valid, int tid) {
    constexpr int V4 = HS / 4;
    for (int lin = tid; lin < TILE * V4; lin += FT) {
        const int r = lin / V4, c = (lin % V4) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < valid) v = LD4(src + (long long)r * ld + c);
        ST4(dst + r * HS + c) = v;
    }
}

// ------------------------------------------------------------------ forward
template <int HS, int KC>
__global__ void __launch_bounds__(FT)
flash_fwd_simt_k(float *__restrict__ out, float *__restrict__ lse, const float *__restrict__ qkv,
                 int T, int NH, float scale) {
    constexpr int G = HS / 32, R = FT / G, TILE = tile_rows<HS>::value;
    __shared__ __align__(16) float Ks[TILE * HS];
    __shared__ __align__(16) float Vs[TILE * HS];

    const int tid = threadIdx.x, sub = tid % G;
    const int bh = blockIdx.y, b = bh / NH, h = bh % NH;
    const int C = NH * HS;
    const int i0 = blockIdx.x * R;
    const int row = i0 + tid / G;                 // this thread's query
    const long long ld = 3LL * C;
    const float *base = qkv + (long long)b * T * ld + h * HS;

    float q[32], o[32];
    if (row < T) {
#pragma unroll
        for (int d = 0; d < 32; d += 4) {
            const float4 v = LD4(base + (long long)row * ld + sub * 32 + d);
            q[d] = v.x * scale; q[d + 1] = v.y * scale; q[d + 2] = v.z * scale; q[d + 3] = v.w * scale;
        }
    } else {
#pragma unroll
        for (int d = 0; d < 32; ++d) q[d] = 0.0f;
    }
#pragma unroll
    for (int d = 0; d < 32; ++d) o[d] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    // Last query row any lane of this warp owns: chunks past it are skipped.
    const int warp_last = min(T - 1, i0 + ((tid | 31) / G));
    const int jmax = min(T, i0 + R);

    for (int j0 = 0; j0 < jmax; j0 += TILE) {
        __syncthreads();
        stage_rows<HS, TILE>(Ks, base + (long long)j0 * ld + C, ld, T - j0, tid);
        stage_rows<HS, TILE>(Vs, base + (long long)j0 * ld + 2 * C, ld, T - j0, tid);
        __syncthreads();

        for (int c0 = 0; c0 < TILE; c0 += KC) {
            if (j0 + c0 > warp_last) break;       // warp-uniform
            float s[KC];
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const float *kr = Ks + (c0 + c) * HS + sub * 32;
                float a = 0.0f;
#pragma unroll
                for (int d = 0; d < 32; d += 4) {
                    const float4 kv = LD4(kr + d);
                    a = fmaf(q[d], kv.x, a); a = fmaf(q[d + 1], kv.y, a);
                    a = fmaf(q[d + 2], kv.z, a); a = fmaf(q[d + 3], kv.w, a);
                }
                a = group_sum<G>(a);
                const int kg = j0 + c0 + c;
                s[c] = (kg > row || kg >= T) ? -INFINITY : a;
            }
            float cmax = s[0];
#pragma unroll
            for (int c = 1; c < KC; ++c) cmax = fmaxf(cmax, s[c]);
            const float mnew = fmaxf(m, cmax);
            const bool live = mnew > -INFINITY;
            const float resc = live ? __expf(m - mnew) : 1.0f;
            float csum = 0.0f;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                s[c] = live ? __expf(s[c] - mnew) : 0.0f;
                csum += s[c];
            }
            m = mnew;
            l = l * resc + csum;
#pragma unroll
            for (int d = 0; d < 32; ++d) o[d] *= resc;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const float *vr = Vs + (c0 + c) * HS + sub * 32;
#pragma unroll
                for (int d = 0; d < 32; d += 4) {
                    const float4 vv = LD4(vr + d);
                    o[d] = fmaf(s[c], vv.x, o[d]); o[d + 1] = fmaf(s[c], vv.y, o[d + 1]);
                    o[d + 2] = fmaf(s[c], vv.z, o[d + 2]); o[d + 3] = fmaf(s[c], vv.w, o[d + 3]);
                }
            }
        }
    }

    if (row < T) {
        const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
        float *dst = out + ((long long)b * T + row) * C + h * HS + sub * 32;
#pragma unroll
        for (int d = 0; d < 32; d += 4)
            ST4(dst + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
        if (sub == 0) lse[(long long)bh * T + row] = m + __logf(l);
    }
}

// Forward, register-tiled ("rows4"): a thread owns RQ = 4 consecutive query rows x 16 of the head's columns, a row
// group is HS/16 adjacent lanes.  Every 16-float slice of a K or V row read from shared memory now feeds 4 rows'
// products (64 multiply-adds per 4 128-bit loads instead of 16), and the products are issued as two-wide
// fma.rn.f32x2 (each half an IEEE fma); scores finish with log2(HS/16) shuffles.  Measured at B8 H12 T1024 hs64:
// 0.90 ms against 0.94 ms for the kernel above -- both sit at a fifth of the multiply-add peak, held there by
// dependent-issue and shared-memory-load latency at 8 warps per SM (213 registers per thread), not by any pipe.
// The same tiling of the two backward kernels (2 rows x 16 columns) measured 4 % slower than theirs and was dropped.
__device__ __forceinline__ unsigned long long f2pack(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2unpack(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void f2fma(unsigned long long &d, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

template <int HS, int KC>
__global__ void __launch_bounds__(FT)
flash_fwd_rows4_k(float *__restrict__ out, float *__restrict__ lse, const float *__restrict__ qkv,
                  int T, int NH, float scale) {
    constexpr int GL = HS / 16, RQ = 4, ROWS = FT / GL * RQ, TILE = tile_rows<HS>::value;
    __shared__ __align__(16) float Ks[TILE * HS];
    __shared__ __align__(16) float Vs[TILE * HS];

    const int tid = threadIdx.x, sub = tid % GL;
    const int bh = blockIdx.y, b = bh / NH, h = bh % NH;
    const int C = NH * HS;
    const int i0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * ROWS;      // longest blocks first
    const int row0 = i0 + (tid / GL) * RQ;        // this thread's first query
    const long long ld = 3LL * C;
    const float *base = qkv + (long long)b * T * ld + h * HS;

    // q and o as pairs of neighbouring columns: q2[r][i] = columns 2i, 2i+1 of this thread's slice
    unsigned long long q2[RQ][8], o2[RQ][8];
#pragma unroll
    for (int r = 0; r < RQ; ++r) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row0 + r < T) v = LD4(base + (long long)(row0 + r) * ld + sub * 16 + 2 * i);
            q2[r][i] = f2pack(v.x * scale, v.y * scale);
            q2[r][i + 1] = f2pack(v.z * scale, v.w * scale);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) o2[r][i] = 0ull;
    }
    float m[RQ], l[RQ];
#pragma unroll
    for (int r = 0; r < RQ; ++r) { m[r] = -INFINITY; l[r] = 0.0f; }

    // Last query row any lane of this warp owns: chunks past it are skipped.
    const int warp_last = min(T - 1, i0 + ((tid | 31) / GL) * RQ + RQ - 1);
    const int jmax = min(T, i0 + ROWS);

    for (int j0 = 0; j0 < jmax; j0 += TILE) {
        __syncthreads();
        stage_rows<HS, TILE>(Ks, base + (long long)j0 * ld + C, ld, T - j0, tid);
        stage_rows<HS, TILE>(Vs, base + (long long)j0 * ld + 2 * C, ld, T - j0, tid);
        __syncthreads();

        for (int c0 = 0; c0 < TILE; c0 += KC) {
            if (j0 + c0 > warp_last) break;       // warp-uniform
            float s[RQ][KC];
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const float *kr = Ks + (c0 + c) * HS + sub * 16;
                unsigned long long k2[8];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const float4 kv = LD4(kr + 2 * i);
                    k2[i] = f2pack(kv.x, kv.y);
                    k2[i + 1] = f2pack(kv.z, kv.w);
                }
#pragma unroll
                for (int r = 0; r < RQ; ++r) {
                    unsigned long long acc = 0ull;
#pragma unroll
                    for (int i = 0; i < 8; ++i) f2fma(acc, q2[r][i], k2[i]);
                    float lo, hi;
                    f2unpack(acc, lo, hi);
                    s[r][c] = lo + hi;
                }
            }
#pragma unroll
            for (int r = 0; r < RQ; ++r) {
                const int row = row0 + r;
                float cmax = -INFINITY;
#pragma unroll
                for (int c = 0; c < KC; ++c) {
                    const float a = group_sum<GL>(s[r][c]);
                    const int kg = j0 + c0 + c;
                    s[r][c] = (kg > row || kg >= T) ? -INFINITY : a;
                    cmax = fmaxf(cmax, s[r][c]);
                }
                const float mnew = fmaxf(m[r], cmax);
                const bool live = mnew > -INFINITY;
                const float resc = live ? __expf(m[r] - mnew) : 1.0f;
                float csum = 0.0f;
#pragma unroll
                for (int c = 0; c < KC; ++c) {
                    s[r][c] = live ? __expf(s[r][c] - mnew) : 0.0f;
                    csum += s[r][c];
                }
                m[r] = mnew;
                l[r] = l[r] * resc + csum;
                const unsigned long long resc2 = f2pack(resc, resc);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    unsigned long long z = 0ull;
                    f2fma(z, o2[r][i], resc2);                  // o * resc + 0
                    o2[r][i] = z;
                }
            }
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const float *vr = Vs + (c0 + c) * HS + sub * 16;
                unsigned long long v2[8];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const float4 vv = LD4(vr + 2 * i);
                    v2[i] = f2pack(vv.x, vv.y);
                    v2[i + 1] = f2pack(vv.z, vv.w);
                }
#pragma unroll
                for (int r = 0; r < RQ; ++r) {
                    const unsigned long long p2 = f2pack(s[r][c], s[r][c]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) f2fma(o2[r][i], p2, v2[i]);
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < RQ; ++r) {
        const int row = row0 + r;
        if (row >= T) continue;
        const float inv = (l[r] > 0.0f) ? 1.0f / l[r] : 0.0f;
        float *dst = out + ((long long)b * T + row) * C + h * HS + sub * 16;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float a0, a1, a2, a3;
            f2unpack(o2[r][i], a0, a1);
            f2unpack(o2[r][i + 1], a2, a3);
            ST4(dst + 2 * i) = make_float4(a0 * inv, a1 * inv, a2 * inv, a3 * inv);
        }
        if (sub == 0) lse[(long long)bh * T + row] = m[r] + __logf(l[r]);
    }
}

// ----------------------------------------------------------------- backward
// D[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per row (src/flash.cu:471-489).
__global__ void flash_dsum_k(float *__restrict__ dsum, const float *__restrict__ dout,
                             const float *__restrict__ out, int T, int NH, int HS, long long rows) {
    const int lane = threadIdx.x & 31;
    const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    if (w >= rows) return;
    const int t = (int)(w % T);
    const int h = (int)((w / T) % NH);
    const long long b = w / ((long long)T * NH);
    const long long off = (b * T + t) * (long long)(NH * HS) + (long long)h * HS;
    float a = 0.0f;
    for (int d = lane; d < HS; d += 32) a += dout[off + d] * out[off + d];
    a = warp_sum(a);
    if (lane == 0) dsum[w] = a;
}

// The same sums with 128-bit loads over the (B*T, C) arrays in storage order: GL = HS/4 consecutive
// lanes hold one head of one token and add up with shuffles.  Needs 16-byte aligned rows.
template <int GL>
__global__ void __launch_bounds__(256) flash_dsum_vec_k(float *__restrict__ dsum, const float *__restrict__ dout,
                                                        const float *__restrict__ out, int T, int NH, long long n4) {
    const int c4 = NH * GL;                                // 128-bit words per token
    const long long stride = (long long)gridDim.x * blockDim.x;
    // whole warps stay in the loop for the shuffles
    const long long n4_up = (n4 + 31) & ~31LL;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n4_up; e += stride) {
        float a = 0.0f;
        if (e < n4) {
            const float4 x = __ldg(reinterpret_cast<const float4 *>(dout) + e);
            const float4 y = __ldg(reinterpret_cast<const float4 *>(out) + e);
            a = x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
        }
#pragma unroll
        for (int o = GL / 2; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (e < n4 && (threadIdx.x & (GL - 1)) == 0) {
            const long long bt = e / c4;
            const int h = (int)(e - bt * c4) / GL;
            const long long b = bt / T;
            const int t = (int)(bt - b * T);
            dsum[(b * NH + h) * T + t] = a;
        }
    }
}

// dQ: a row group owns a query row; keys stream through shared memory.
template <int HS, int KC>
__global__ void __launch_bounds__(FT)
flash_bwd_q_simt_k(float *__restrict__ dqkv, const float *__restrict__ qkv,
                   const float *__restrict__ dout, const float *__restrict__ lse,
                   const float *__restrict__ dsum, int T, int NH, float scale) {
    constexpr int G = HS / 32, R = FT / G, TILE = tile_rows<HS>::value;
    __shared__ __align__(16) float Ks[TILE * HS];
    __shared__ __align__(16) float Vs[TILE * HS];

    const int tid = threadIdx.x, sub = tid % G;
    const int bh = blockIdx.y, b = bh / NH, h = bh % NH;
    const int C = NH * HS;
    const int i0 = blockIdx.x * R;
    const int row = i0 + tid / G;
    const long long ld = 3LL * C;
    const float *base = qkv + (long long)b * T * ld + h * HS;

    float q[32], go[32], dq[32];
    float lrow = 0.0f, drow = 0.0f;
    if (row < T) {
        const float *dor = dout + ((long long)b * T + row) * C + h * HS + sub * 32;
#pragma unroll
        for (int d = 0; d < 32; d += 4) {
            const float4 v = LD4(base + (long long)row * ld + sub * 32 + d);
            q[d] = v.x * scale; q[d + 1] = v.y * scale; q[d + 2] = v.z * scale; q[d + 3] = v.w * scale;
            const float4 g = LD4(dor + d);
            go[d] = g.x; go[d + 1] = g.y; go[d + 2] = g.z; go[d + 3] = g.w;
        }
        lrow = lse[(long long)bh * T + row];
        drow = dsum[(long long)bh * T + row];
    } else {
#pragma unroll
        for (int d = 0; d < 32; ++d) { q[d] = 0.0f; go[d] = 0.0f; }
    }
#pragma unroll
    for (int d = 0; d < 32; ++d) dq[d] = 0.0f;

    const int warp_last = min(T - 1, i0 + ((tid | 31) / G));
    const int jmax = min(T, i0 + R);
    for (int j0 = 0; j0 < jmax; j0 += TILE) {
        __syncthreads();
        stage_rows<HS, TILE>(Ks, base + (long long)j0 * ld + C, ld, T - j0, tid);
        stage_rows<HS, TILE>(Vs, base + (long long)j0 * ld + 2 * C, ld, T - j0, tid);
        __syncthreads();
        for (int c0 = 0; c0 < TILE; c0 += KC) {
            if (j0 + c0 > warp_last) break;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const float *kr = Ks + (c0 + c) * HS + sub * 32;
                const float *vr = Vs + (c0 + c) * HS + sub * 32;
                float s = 0.0f, dp = 0.0f;
                float kreg[32];
#pragma unroll
                for (int d = 0; d < 32; d += 4) {
                    const float4 kv = LD4(kr + d), vv = LD4(vr + d);
                    kreg[d] = kv.x; kreg[d + 1] = kv.y; kreg[d + 2] = kv.z; kreg[d + 3] = kv.w;
                    s = fmaf(q[d], kv.x, s); s = fmaf(q[d + 1], kv.y, s);
                    s = fmaf(q[d + 2], kv.z, s); s = fmaf(q[d + 3], kv.w, s);
                    dp = fmaf(go[d], vv.x, dp); dp = fmaf(go[d + 1], vv.y, dp);
                    dp = fmaf(go[d + 2], vv.z, dp); dp = fmaf(go[d + 3], vv.w, dp);
                }
                s = group_sum<G>(s);
                dp = group_sum<G>(dp);
                const int kg = j0 + c0 + c;
                const bool on = (kg <= row) && (kg < T) && (row < T);
                const float p = on ? __expf(s - lrow) : 0.0f;
                const float ds = p * (dp - drow);
#pragma unroll
                for (int d = 0; d < 32; ++d) dq[d] = fmaf(ds, kreg[d], dq[d]);
            }
        }
    }
    if (row < T) {
        float *dst = dqkv + ((long long)b * T + row) * ld + h * HS + sub * 32;
#pragma unroll
        for (int d = 0; d < 32; d += 4)
            ST4(dst + d) = make_float4(dq[d] * scale, dq[d + 1] * scale, dq[d + 2] * scale, dq[d + 3] * scale);
    }
}

// dK, dV: a row group owns a key row; queries at or after it stream through
// shared memory together with dO, lse and D.
template <int HS, int KC>
__global__ void __launch_bounds__(FT)
flash_bwd_kv_simt_k(float *__restrict__ dqkv, const float *__restrict__ qkv,
                    const float *__restrict__ dout, const float *__restrict__ lse,
                    const float *__restrict__ dsum, int T, int NH, float scale) {
    constexpr int G = HS / 32, R = FT / G;
    constexpr int QT = 32;   // queries staged per tile
    __shared__ __align__(16) float Qs[QT * HS];
    __shared__ __align__(16) float Os[QT * HS];
    __shared__ float Ls[QT], Ds[QT];

    const int tid = threadIdx.x, sub = tid % G;
    const int bh = blockIdx.y, b = bh / NH, h = bh % NH;
    const int C = NH * HS;
    const int j0 = blockIdx.x * R;
    const int key = j0 + tid / G;
    const long long ld = 3LL * C;
    const float *base = qkv + (long long)b * T * ld + h * HS;

    float k[32], v[32], dk[32], dv[32];
    if (key < T) {
#pragma unroll
        for (int d = 0; d < 32; d += 4) {
            const float4 a = LD4(base + (long long)key * ld + C + sub * 32 + d);
            const float4 c = LD4(base + (long long)key * ld + 2 * C + sub * 32 + d);
            k[d] = a.x; k[d + 1] = a.y; k[d + 2] = a.z; k[d + 3] = a.w;
            v[d] = c.x; v[d + 1] = c.y; v[d + 2] = c.z; v[d + 3] = c.w;
        }
    } else {
#pragma unroll
        for (int d = 0; d < 32; ++d) { k[d] = 0.0f; v[d] = 0.0f; }
    }
#pragma unroll
    for (int d = 0; d < 32; ++d) { dk[d] = 0.0f; dv[d] = 0.0f; }

    // First key row of this warp: queries before it contribute nothing.
    const int warp_first = j0 + ((tid & ~31) / G);
    constexpr int V4 = HS / 4;
    for (int i0 = (j0 / QT) * QT; i0 < T; i0 += QT) {
        __syncthreads();
        for (int lin = tid; lin < QT * V4; lin += FT) {
            const int r = lin / V4, c = (lin % V4) * 4;
            float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), gv = qv;
            if (i0 + r < T) {
                qv = LD4(base + (long long)(i0 + r) * ld + c);
                gv = LD4(dout + ((long long)b * T + i0 + r) * C + h * HS + c);
            }
            ST4(Qs + r * HS + c) = qv;
            ST4(Os + r * HS + c) = gv;
        }
        if (tid < QT) {
            const bool ok = i0 + tid < T;
            Ls[tid] = ok ? lse[(long long)bh * T + i0 + tid] : 0.0f;
            Ds[tid] = ok ? dsum[(long long)bh * T + i0 + tid] : 0.0f;
        }
        __syncthreads();
        if (i0 + QT - 1 < warp_first) continue;   // warp-uniform; barriers are outside
#pragma unroll 2
        for (int r = 0; r < QT; ++r) {
            const int qg = i0 + r;
            const float *qr = Qs + r * HS + sub * 32;
            const float *gr = Os + r * HS + sub * 32;
            float s = 0.0f, dp = 0.0f;
            float qreg[32], greg[32];
#pragma unroll
            for (int d = 0; d < 32; d += 4) {
                const float4 qv = LD4(qr + d), gv = LD4(gr + d);
                qreg[d] = qv.x; qreg[d + 1] = qv.y; qreg[d + 2] = qv.z; qreg[d + 3] = qv.w;
                greg[d] = gv.x; greg[d + 1] = gv.y; greg[d + 2] = gv.z; greg[d + 3] = gv.w;
                s = fmaf(qv.x, k[d], s); s = fmaf(qv.y, k[d + 1], s);
                s = fmaf(qv.z, k[d + 2], s); s = fmaf(qv.w, k[d + 3], s);
                dp = fmaf(gv.x, v[d], dp); dp = fmaf(gv.y, v[d + 1], dp);
                dp = fmaf(gv.z, v[d + 2], dp); dp = fmaf(gv.w, v[d + 3], dp);
            }
            s = group_sum<G>(s) * scale;
            dp = group_sum<G>(dp);
            const bool on = (qg >= key) && (qg < T) && (key < T);
            const float p = on ? __expf(s - Ls[r]) : 0.0f;
            const float ds = p * (dp - Ds[r]);
#pragma unroll
            for (int d = 0; d < 32; ++d) {
                dv[d] = fmaf(p, greg[d], dv[d]);
                dk[d] = fmaf(ds, qreg[d], dk[d]);
            }
        }
    }
    if (key < T) {
        float *dkp = dqkv + ((long long)b * T + key) * ld + C + h * HS + sub * 32;
        float *dvp = dkp + C;
#pragma unroll
        for (int d = 0; d < 32; d += 4) {
            ST4(dkp + d) = make_float4(dk[d] * scale, dk[d + 1] * scale, dk[d + 2] * scale, dk[d + 3] * scale);
            ST4(dvp + d) = make_float4(dv[d], dv[d + 1], dv[d + 2], dv[d + 3]);
        }
    }
}

struct FwdCfg { int kc; const char *name; };
struct BwdCfg { int kc; const char *name; };
// Forward config 2 is the tensor-core kernel (flash_tc.cu), head size 64 only.
// Forward config 0 is the register-tiled kernel (4 rows x 16 columns per thread), 1 the row-per-lane-group one.
const FwdCfg FWD[] = {{8, "simt-fp32 rows4 keys8"}, {16, "simt-fp32 rowgroup keys16"},
                      {0, "tcgen05-tf32 q2x128 k64 (head size 64 only)"}};
// Backward config 2 is the tensor-core kernel pair (flash_tc_bwd.cu), head size 64 only.
const BwdCfg BWD[] = {{4, "simt-fp32 rowgroup keys4"}, {8, "simt-fp32 rowgroup keys8"},
                      {0, "tcgen05-tf32 dq128x128 dkv128x128 (head size 64 only)"}};
constexpr int NFWD = 3, NBWD = 3, FWD_TC = 2, BWD_TC = 2;

bool shape_ok(const float *a, const float *b, int C, int NH) {
    return NH > 0 && C % NH == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0;
}

template <int HS>
int run_fwd(int cfg, float *out, float *lse, const float *qkv, int B, int T, int NH, float scale,
            cudaStream_t st) {
    if (cfg == 0) {
        constexpr int ROWS = FT / (HS / 16) * 4;
        dim3 grid(ceil_div(T, ROWS), B * NH);
        flash_fwd_rows4_k<HS, 8><<<grid, FT, 0, st>>>(out, lse, qkv, T, NH, scale);
    } else {
        constexpr int R = FT / (HS / 32);
        dim3 grid(ceil_div(T, R), B * NH);
        flash_fwd_simt_k<HS, 16><<<grid, FT, 0, st>>>(out, lse, qkv, T, NH, scale);
    }
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

template <int HS>
int run_bwd(int cfg, float *dqkv, float *dsum, const float *dout, const float *qkv, const float *out,
            const float *lse, int B, int T, int NH, float scale, cudaStream_t st) {
    constexpr int R = FT / (HS / 32);
    const long long rows = (long long)B * NH * T;
    flash_dsum_k<<<ceil_div(rows * 32, 256), 256, 0, st>>>(dsum, dout, out, T, NH, HS, rows);
    dim3 grid(ceil_div(T, R), B * NH);
    if (BWD[cfg].kc == 4) {
        flash_bwd_kv_simt_k<HS, 4><<<grid, FT, 0, st>>>(dqkv, qkv, dout, lse, dsum, T, NH, scale);
        flash_bwd_q_simt_k<HS, 4><<<grid, FT, 0, st>>>(dqkv, qkv, dout, lse, dsum, T, NH, scale);
    } else {
        flash_bwd_kv_simt_k<HS, 8><<<grid, FT, 0, st>>>(dqkv, qkv, dout, lse, dsum, T, NH, scale);
        flash_bwd_q_simt_k<HS, 8><<<grid, FT, 0, st>>>(dqkv, qkv, dout, lse, dsum, T, NH, scale);
    }
    count_launch(3);
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}

}  // namespace

int launch_flash_dsum(float *dsum, const float *dout, const float *out, int B, int T, int NH, int HS, cudaStream_t st) {
    const long long rows = (long long)B * NH * T;
    const bool vec = (HS == 32 || HS == 64 || HS == 128) && (((uintptr_t)dout | (uintptr_t)out) & 15) == 0;
    if (vec) {
        const long long n4 = rows * (HS / 4);
        long long blocks = (n4 + 255) / 256;
        const long long cap = 16LL * sm_count();
        if (blocks > cap) blocks = cap;
        if (HS == 32) flash_dsum_vec_k<8><<<(int)blocks, 256, 0, st>>>(dsum, dout, out, T, NH, n4);
        else if (HS == 64) flash_dsum_vec_k<16><<<(int)blocks, 256, 0, st>>>(dsum, dout, out, T, NH, n4);
        else flash_dsum_vec_k<32><<<(int)blocks, 256, 0, st>>>(dsum, dout, out, T, NH, n4);
    } else {
        flash_dsum_k<<<ceil_div(rows * 32, 256), 256, 0, st>>>(dsum, dout, out, T, NH, HS, rows);
    }
    count_launch();
    BMB_LAUNCH_CHECK();
    return BMB_OK;
}
}  // namespace bmb

using namespace bmb;

extern "C" {

int bmb_flash_num_configs(void) { return NFWD; }
const char *bmb_flash_config_name(int cfg) { return (cfg >= 0 && cfg < NFWD) ? FWD[cfg].name : "?"; }
// fp32 arithmetic: the SIMT kernel; TF32/BF16 math modes: the tensor-core kernel.
int bmb_flash_default_config(void) { return bmb_get_math_mode() == BMB_MATH_FP32 ? 0 : FWD_TC; }

int bmb_flash_attention_forward_cfg(int cfg, float *out, float *lse, const float *qkv, int B, int T,
                                    int C, int NH) {
    return bmb_flash_attention_forward_ex(cfg, 0, out, lse, qkv, B, T, C, NH);
}

int bmb_flash_attention_forward_ex(int cfg, int flags, float *out, float *lse, const float *qkv, int B, int T,
                                   int C, int NH) {
    if (cfg < 0 || cfg >= NFWD) return fail(BMB_E_UNSUPPORTED, "flash: no forward config %d", cfg);
    if (B <= 0 || T <= 0) return BMB_OK;
    if (!shape_ok(out, qkv, C, NH)) return fail(BMB_E_ARG, "flash: bad shape or alignment (C=%d NH=%d)", C, NH);
    const int hs = C / NH;
    const float scale = 1.0f / sqrtf((float)hs);
    cudaStream_t st = cur_stream();
    if (cfg == FWD_TC) {
        if (!flash_tc_supported(T, C, NH, qkv, out))
            return fail(BMB_E_UNSUPPORTED, "flash: the tensor-core config needs head size 64 (got %d)", hs);
        return flash_forward_tc(out, lse, qkv, B, T, C, NH, (flags & BMB_FLASH_OPERANDS_ROUNDED) != 0, st);
    }
    switch (hs) {
    case 32:  return run_fwd<32>(cfg, out, lse, qkv, B, T, NH, scale, st);
    case 64:  return run_fwd<64>(cfg, out, lse, qkv, B, T, NH, scale, st);
    case 128: return run_fwd<128>(cfg, out, lse, qkv, B, T, NH, scale, st);
    default:  return fail(BMB_E_UNSUPPORTED, "flash: no tile config for head size %d", hs);
    }
}

int bmb_flash_attention_forward(float *out, float *lse, const float *qkv, int B, int T, int C,
                                int NH) {
    int cfg = bmb_flash_default_config();
    // The preferred config may not serve this head size: fall back through the table (src/flash.cu:419-432).
    if (cfg == FWD_TC && !(NH > 0 && C % NH == 0 && flash_tc_supported(T, C, NH, qkv, out))) cfg = 0;
    return bmb_flash_attention_forward_cfg(cfg, out, lse, qkv, B, T, C, NH);
}

int bmb_flash_num_bwd_configs(void) { return NBWD; }
const char *bmb_flash_bwd_config_name(int cfg) { return (cfg >= 0 && cfg < NBWD) ? BWD[cfg].name : "?"; }
int bmb_flash_default_bwd_config(void) { return bmb_get_math_mode() == BMB_MATH_FP32 ? 0 : BWD_TC; }

int bmb_flash_attention_backward_cfg(int cfg, float *dqkv, float *dsum, const float *dout,
                                     const float *qkv, const float *out, const float *lse, int B,
                                     int T, int C, int NH) {
    return bmb_flash_attention_backward_ex(cfg, 0, dqkv, dsum, dout, qkv, out, lse, B, T, C, NH);
}

int bmb_flash_attention_backward_ex(int cfg, int flags, float *dqkv, float *dsum, const float *dout,
                                    const float *qkv, const float *out, const float *lse, int B,
                                    int T, int C, int NH) {
    if (cfg < 0 || cfg >= NBWD) return fail(BMB_E_UNSUPPORTED, "flash: no backward config %d", cfg);
    if (B <= 0 || T <= 0) return BMB_OK;
    if (!shape_ok(dqkv, qkv, C, NH) || !shape_ok(dout, out, C, NH))
        return fail(BMB_E_ARG, "flash: bad shape or alignment (C=%d NH=%d)", C, NH);
    const int hs = C / NH;
    const float scale = 1.0f / sqrtf((float)hs);
    cudaStream_t st = cur_stream();
    if (cfg == BWD_TC) {
        if (!flash_tc_supported(T, C, NH, qkv, dqkv))
            return fail(BMB_E_UNSUPPORTED, "flash: the tensor-core config needs head size 64 (got %d)", hs);
        return flash_backward_tc(dqkv, dsum, dout, qkv, out, lse, B, T, C, NH, (flags & BMB_FLASH_OPERANDS_ROUNDED) != 0, st);
    }
    switch (hs) {
    case 32:  return run_bwd<32>(cfg, dqkv, dsum, dout, qkv, out, lse, B, T, NH, scale, st);
    case 64:  return run_bwd<64>(cfg, dqkv, dsum, dout, qkv, out, lse, B, T, NH, scale, st);
    case 128: return run_bwd<128>(cfg, dqkv, dsum, dout, qkv, out, lse, B, T, NH, scale, st);
    default:  return fail(BMB_E_UNSUPPORTED, "flash: no backward tile config for head size %d", hs);
    }
}

int bmb_flash_attention_backward(float *dqkv, float *dsum, const float *dout, const float *qkv,
                                 const float *out, const float *lse, int B, int T, int C, int NH) {
    int cfg = bmb_flash_default_bwd_config();
    if (cfg == BWD_TC && !(NH > 0 && C % NH == 0 && flash_tc_supported(T, C, NH, qkv, dqkv))) cfg = 0;
    return bmb_flash_attention_backward_cfg(cfg, dqkv, dsum, dout, qkv, out, lse, B, T, C, NH);
}

}  // extern "C"
