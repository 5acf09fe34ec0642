// stack_kernels.cuh — CUDA kernels (sm_100a) of the layer-stack models: a residual stream that passes a configurable
// list of layers, each one mixer (minGRU recurrence | latent attention with a sliding window and a soft-max sink |
// gated delta rule | generalized delta rule | differential sliding-window attention) and an optional feed-forward
// (clamped gated unit | polynomial activation with norms), either one sub-layer after the other with grouped RMS norms
// before and after each, or both reading the same residual behind causal convolutions of their normed inputs.
// Every size and constant is a kernel argument; nothing is specialised for one model. stack_kernels_mix.cuh holds the kernels of
// further mechanisms (element-wise norm, depth average, retention, sigmoid attention, routed mixture) on top of these.
//
// Precision: the residual stream, norms, positions and angles, attention scores and weights, recurrent states and
// everything that enters a recurrence are float32. Matrix products take float32 activations and weights in the
// model's storage type WT (bfloat16 or float32) and accumulate in float32; the tensor-core product (k_gemm_bf16_mma)
// rounds its activation operand to bfloat16.
#pragma once
#include <cuda_bf16.h>
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {
namespace stk {


__device__ __forceinline__ float wf(const float * p, size_t i) { return p[i]; }
__device__ __forceinline__ float wf(const __nv_bfloat16 * p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// what a step works on: written by the host (or by a memcpy node of the replayed decode graph) before the launches
struct StepState {
    int32_t pos0;       // position of the step's first token within its sequence
    int32_t n_tokens;
};

// ---- RMS norm of one group by one warp: y = x / sqrt(mean(x^2) + eps) * w ------------------------------------------------
__device__ __forceinline__ void warp_group_norm(const float * __restrict__ x, const float * __restrict__ w, int gs, float eps, float * __restrict__ y, int lane) {
    float ss = 0.f;
    for (int i = lane; i < gs; i += 32) { const float v = x[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float) gs + eps);
    for (int i = lane; i < gs; i += 32) y[i] = x[i] * r * w[i];
}

// ---- embedding fused with the first layer's input norm: X[t] = embed[token[t]], Hn[t] = norm(X[t]) * w ---------------------
template <typename WT>
__global__ void k_embed_rows(const WT * __restrict__ embed, const int32_t * __restrict__ tokens, int E, int n_vocab, float * __restrict__ X,
                             const float * __restrict__ w, int groups, float eps, float * __restrict__ Hn) {
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : tok >= n_vocab ? n_vocab - 1 : tok;      // ids are validated on the host; never read outside the table
    for (int i = threadIdx.x; i < E; i += blockDim.x) X[(size_t) t * E + i] = wf(embed, (size_t) tok * E + i);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, gs = E / groups;
    for (int g = warp; g < groups; g += nw) warp_group_norm(X + (size_t) t * E + g * gs, w + g * gs, gs, eps, Hn + (size_t) t * E + g * gs, lane);
}

// ---- end of a sub-layer, fused: X[t] += norm(Y[t]) * w_post, then (w_next != nullptr) Hn[t] = norm(X[t]) * w_next, the input
// norm of the sub-layer that follows. Same groups for both; one block per row, one warp per group.
constexpr int POST_NPL = 16;       // elements per lane k_post_norm_add keeps in registers (groups of up to 512)
__global__ void k_post_norm_add(const float * __restrict__ Y, const float * __restrict__ w_post, float * __restrict__ X,
                                const float * __restrict__ w_next, float * __restrict__ Hn, int n, int groups, float eps) {
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, gs = n / groups;
    for (int g = warp; g < groups; g += nw) {
        const size_t b = (size_t) row * n + (size_t) g * gs;
        const float * y = Y + b;
        float * x = X + b;
        if (gs <= 32 * POST_NPL) {
            // the group lives in registers: one round trip to memory instead of three dependent passes (a decode step is latency-bound)
            float yv[POST_NPL], xv[POST_NPL];
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < POST_NPL; k++) {
                const int i = lane + 32 * k;
                yv[k] = i < gs ? y[i] : 0.f; xv[k] = i < gs ? x[i] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < POST_NPL; k++) ss = fmaf(yv[k], yv[k], ss);
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float) gs + eps);
            float s2 = 0.f;
#pragma unroll
            for (int k = 0; k < POST_NPL; k++) {
                const int i = lane + 32 * k;
                if (i < gs) { xv[k] = xv[k] + yv[k] * r * w_post[g * gs + i]; x[i] = xv[k]; s2 = fmaf(xv[k], xv[k], s2); }
            }
            if (w_next) {
                s2 = warp_sum(s2);
                const float r2 = 1.0f / sqrtf(s2 / (float) gs + eps);
#pragma unroll
                for (int k = 0; k < POST_NPL; k++) { const int i = lane + 32 * k; if (i < gs) Hn[b + i] = xv[k] * r2 * w_next[g * gs + i]; }
            }
            continue;
        }
        float ss = 0.f;
        for (int i = lane; i < gs; i += 32) ss = fmaf(y[i], y[i], ss);
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float) gs + eps);
        float s2 = 0.f;
        for (int i = lane; i < gs; i += 32) { const float v = x[i] + y[i] * r * w_post[g * gs + i]; x[i] = v; s2 = fmaf(v, v, s2); }
        if (w_next) {
            s2 = warp_sum(s2);
            const float r2 = 1.0f / sqrtf(s2 / (float) gs + eps);
            for (int i = lane; i < gs; i += 32) Hn[b + i] = x[i] * r2 * w_next[g * gs + i];     // each lane re-reads what it wrote
        }
    }
}

// ---- RMS norm in `groups` equal consecutive parts; eps inside the root ----------------------------------------------
// one block per row, one warp per group (round robin). rows != nullptr gathers input rows (the head's wanted rows).
// accumulate == 0: Y[row] = norm(X[row]) * w;  accumulate == 1: Y[row] += norm(X[row]) * w  (the residual sum)
__global__ void k_group_norm(const float * __restrict__ X, int ldx, const int32_t * __restrict__ rows, const float * __restrict__ w,
                             int n, int groups, float eps, float * __restrict__ Y, int ldy, int accumulate) {
    const int row = blockIdx.x, src = rows ? rows[row] : row;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int gs = n / groups;
    const float * x = X + (size_t) src * ldx;
    float * y = Y + (size_t) row * ldy;
    for (int g = warp; g < groups; g += nw) {
        const int b = g * gs;
        float ss = 0.f;
        for (int i = lane; i < gs; i += 32) { const float v = x[b + i]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float) gs + eps);
        for (int i = lane; i < gs; i += 32) {
            const float v = x[b + i] * r * w[b + i];
            y[b + i] = accumulate ? y[b + i] + v : v;
        }
    }
}

// ---- matrix products: Y[t][n] = sum_k X[t][k] * W[n][k] (+ bias[n]); W row-major [N][K] -------------------------------
// blockIdx.z runs over a batch of independent products (per-head matrices) with element strides sX / sW / sY.
struct LinArgs {
    const float * X; const void * W; const float * bias; float * Y;
    int T, N, K, ldx, ldy;
    long long sX, sW, sY;
    int vec;            // 1: K, ldx and all bases allow 16-byte loads
    int glu;            // 1: rows of W are interleaved (2i: gate_i, 2i + 1: up_i); the epilogue writes the clamped gated unit
    float limit, alpha; //    y_i = g sigmoid(alpha g) (u + 1), g = min(gate_i, limit), u = clamp(up_i, -limit, limit), to Y[t][i] (N / 2 wide)
    int w_kn, ldw;      // k_gemm_simt only. w_kn = 1: W is given [K][N] with row stride ldw (the attention's weights x cached rows);
                        // w_kn = 0 and ldw > 0: W is [N][K] with row stride ldw (keys inside wider cached rows)
    int nz2 = 1;        // k_gemm_simt only: blockIdx.z = z1 * nz2 + z2, a second batch level with the strides below
    long long sX2 = 0, sW2 = 0, sY2 = 0;
    float up_shift = 1.0f;                  // the gated unit's (u + up_shift)
    // tile kernels: batch entry z works on rows seg[z] .. seg[z + 1] - 1 of X and Y (rows sorted by the matrix they meet: a routed
    // mixture's experts); T is then only the most rows an entry can have
    const int32_t * seg = nullptr;
    // k_gemv: entry z meets matrix w_index[z] of the batch and reads the rows of entry z / x_share
    const int32_t * w_index = nullptr;
    int x_share = 1;
    // k_gemv: entry z's input row is x_scale[z] times the row it reads (a routed expert that runs on a weighted input); no bias then
    const float * x_scale = nullptr;
    int accum = 0;      // k_gemm_simt only: Y += the product (a second set of keys joining a weighted sum)
};
__device__ __forceinline__ float clamped_glu(float gate, float up, float limit, float alpha, float shift) {
    const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);      // limit = +inf: no clamp
    return g * sigmoidf_(alpha * g) * (u + shift);
}

constexpr int GEMV_MAX_T = 4;
// decode and very short portions: one warp per output row, the row of W streamed once with 16-byte loads
template <typename WT, int RPW>
__global__ void __launch_bounds__(256) k_gemv(const LinArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = (blockIdx.x * (blockDim.x >> 5) + warp) * RPW;      // RPW = 2: a (gate, up) pair per warp
    if (n >= a.N) return;
    const WT * w = reinterpret_cast<const WT *>(a.W) + (size_t) (a.w_index ? a.w_index[blockIdx.z] : blockIdx.z) * a.sW + (size_t) n * a.K;
    const float * x = a.X + (size_t) (blockIdx.z / a.x_share) * a.sX;
    float acc[RPW][GEMV_MAX_T];
#pragma unroll
    for (int r = 0; r < RPW; r++)
#pragma unroll
        for (int t = 0; t < GEMV_MAX_T; t++) acc[r][t] = 0.f;
    constexpr int VEC = 16 / (int) sizeof(WT);
    if (a.vec) {
        // U chunks of 16 bytes per row and lane are requested before any is used: a mat-vec is bound by the bytes in flight
        constexpr int U = RPW == 2 ? 2 : 4;
        for (int kb = lane * VEC; kb < a.K; kb += 32 * VEC * U) {
            uint4 raw[RPW][U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int k = kb + u * 32 * VEC;
#pragma unroll
                for (int r = 0; r < RPW; r++) raw[r][u] = k < a.K ? *reinterpret_cast<const uint4 *>(w + (size_t) r * a.K + k) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int k = kb + u * 32 * VEC;
                if (k >= a.K) break;
                float wv[RPW][VEC];
#pragma unroll
                for (int r = 0; r < RPW; r++) {
                    const uint32_t uu[4] = { raw[r][u].x, raw[r][u].y, raw[r][u].z, raw[r][u].w };
                    if constexpr (sizeof(WT) == 2) {
#pragma unroll
                        for (int i = 0; i < 4; i++) { wv[r][2 * i] = __uint_as_float(uu[i] << 16); wv[r][2 * i + 1] = __uint_as_float(uu[i] & 0xffff0000u); }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++) wv[r][i] = __uint_as_float(uu[i]);
                    }
                }
#pragma unroll
                for (int t = 0; t < GEMV_MAX_T; t++) {
                    if (t < a.T) {
                        const float * xt = x + (size_t) t * a.ldx + k;
#pragma unroll
                        for (int i = 0; i < VEC; i += 4) {
                            const float4 xv = *reinterpret_cast<const float4 *>(xt + i);
#pragma unroll
                            for (int r = 0; r < RPW; r++) {
                                acc[r][t] = fmaf(wv[r][i], xv.x, acc[r][t]); acc[r][t] = fmaf(wv[r][i + 1], xv.y, acc[r][t]);
                                acc[r][t] = fmaf(wv[r][i + 2], xv.z, acc[r][t]); acc[r][t] = fmaf(wv[r][i + 3], xv.w, acc[r][t]);
                            }
                        }
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < a.K; k += 32) {
#pragma unroll
            for (int r = 0; r < RPW; r++) {
                const float wv = wf(w, (size_t) r * a.K + k);
#pragma unroll
                for (int t = 0; t < GEMV_MAX_T; t++) if (t < a.T) acc[r][t] = fmaf(wv, x[(size_t) t * a.ldx + k], acc[r][t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < GEMV_MAX_T; t++) {
        if (t < a.T) {
            float s[RPW];
#pragma unroll
            for (int r = 0; r < RPW; r++) s[r] = warp_sum(acc[r][t]) * (a.x_scale ? a.x_scale[blockIdx.z] : 1.0f) + (a.bias ? a.bias[n + r] : 0.f);
            if (lane == 0) {
                float * y = a.Y + (size_t) blockIdx.z * a.sY + (size_t) t * a.ldy;
                if constexpr (RPW == 2) y[n >> 1] = clamped_glu(s[0], s[1], a.limit, a.alpha, a.up_shift);
                else y[n] = s[0];
            }
        }
    }
}

// prompt portions in true float32 (and every shape the tensor-core kernel does not take): 64 x 64 x 16 tiles on the CUDA
// cores, 256 threads with 4 x 4 outputs each
template <typename WT>
__global__ void __launch_bounds__(256) k_gemm_simt(const LinArgs a) {
    __shared__ __align__(16) float Xs[16][64 + 4];
    __shared__ __align__(16) float Ws[16][64 + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int z1 = blockIdx.z / a.nz2, z2 = blockIdx.z - z1 * a.nz2;
    const int r0 = a.seg ? a.seg[blockIdx.z] : 0, T = a.seg ? a.seg[blockIdx.z + 1] - r0 : a.T;
    if (m0 >= T) return;
    const float * X = a.seg ? a.X + (size_t) r0 * a.ldx : a.X + (size_t) z1 * a.sX + (size_t) z2 * a.sX2;
    const WT * W = reinterpret_cast<const WT *>(a.W) + (size_t) z1 * a.sW + (size_t) z2 * a.sW2;
    const int lr = tid >> 2, lk = (tid & 3) * 4;          // this thread stages 4 consecutive k of row lr
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += 16) {
        {
            const int m = m0 + lr;
            float v[4] = { 0.f, 0.f, 0.f, 0.f };
            if (m < T) {
                const float * p = X + (size_t) m * a.ldx + k0 + lk;
                if (a.vec && k0 + lk + 3 < a.K) { const float4 f = *reinterpret_cast<const float4 *>(p); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
                else for (int i = 0; i < 4; i++) if (k0 + lk + i < a.K) v[i] = p[i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++) Xs[lk + i][lr] = v[i];
        }
        if (a.w_kn && sizeof(WT) == 4 && a.vec) {
            // [K][N] operand with 16-byte aligned rows: a thread takes 4 consecutive n of one k, the block one 16 x 64 tile
            const int kk = tid >> 4, n4 = (tid & 15) * 4, k = k0 + kk, n = n0 + n4;
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < a.K && n < a.N) {
                const float * p = reinterpret_cast<const float *>(W) + (size_t) k * a.ldw + n;
                if (n + 3 < a.N) f = *reinterpret_cast<const float4 *>(p);
                else { f.x = p[0]; if (n + 1 < a.N) f.y = p[1]; if (n + 2 < a.N) f.z = p[2]; }
            }
            *reinterpret_cast<float4 *>(&Ws[kk][n4]) = f;
        } else {
            const int n = n0 + lr;
            float v[4] = { 0.f, 0.f, 0.f, 0.f };
            if (n < a.N) {
                if (a.w_kn) {
                    for (int i = 0; i < 4; i++) if (k0 + lk + i < a.K) v[i] = wf(W, (size_t) (k0 + lk + i) * a.ldw + n);
                } else {
                    const size_t o = (size_t) n * (a.ldw > 0 ? a.ldw : a.K) + k0 + lk;
                    if (sizeof(WT) == 4 && a.vec && k0 + lk + 3 < a.K) {
                        const float4 f = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(W) + o);
                        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                    } else for (int i = 0; i < 4; i++) if (k0 + lk + i < a.K) v[i] = wf(W, o + i);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) Ws[lk + i][lr] = v[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; k++) {
            const float4 xv = *reinterpret_cast<const float4 *>(&Xs[k][ty * 4]);
            const float4 wv = *reinterpret_cast<const float4 *>(&Ws[k][tx * 4]);
            const float xa[4] = { xv.x, xv.y, xv.z, xv.w }, wa[4] = { wv.x, wv.y, wv.z, wv.w };
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xa[i], wa[j], acc[i][j]);
        }
        __syncthreads();
    }
    float * Y = a.seg ? a.Y + (size_t) r0 * a.ldy : a.Y + (size_t) z1 * a.sY + (size_t) z2 * a.sY2;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= T) continue;
        if (a.glu) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < a.N) Y[(size_t) m * a.ldy + (n >> 1)] = clamped_glu(acc[i][j] + (a.bias ? a.bias[n] : 0.f), acc[i][j + 1] + (a.bias ? a.bias[n + 1] : 0.f), a.limit, a.alpha, a.up_shift);
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < a.N) Y[(size_t) m * a.ldy + n] = acc[i][j] + (a.bias ? a.bias[n] : 0.f) + (a.accum ? Y[(size_t) m * a.ldy + n] : 0.f);
        }
    }
}

// the same float32 product for operands large enough to fill 128 x 128 tiles (the attention's products over a tile of tokens x all
// heads): 256 threads with 8 x 8 outputs each (two 4 x 4 quarters 64 apart, so that the 16-byte shared-memory reads of a
// half-warp stay free of bank conflicts), twice the FMAs per shared-memory read of the 64 x 64 kernel, the next K slice
// of both operands in registers while the current one is multiplied. float32 operands with 16-byte aligned rows only (a.vec);
// plain or accumulating stores; no bias, no gated unit, no segments.
constexpr int SG_BM = 128, SG_BN = 128, SG_BK = 16;
__global__ void __launch_bounds__(256, 2) k_gemm_simt_big(const LinArgs a) {
    __shared__ __align__(16) float Xs[SG_BK][SG_BM + 4];
    __shared__ __align__(16) float Ws[SG_BK][SG_BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    const int z1 = blockIdx.z / a.nz2, z2 = blockIdx.z - z1 * a.nz2;
    const float * X = a.X + (size_t) z1 * a.sX + (size_t) z2 * a.sX2;
    const float * W = reinterpret_cast<const float *>(a.W) + (size_t) z1 * a.sW + (size_t) z2 * a.sW2;
    const int ldw = a.ldw > 0 ? a.ldw : a.K;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
    float4 xr[2], wr[2];
    // a K slice of both operands from global memory into registers: rows lr and lr + 64, 4 consecutive k each ([N][K] operands);
    // a [K][N] operand: k rows kk and kk + 8, 4 consecutive n each
    const int lr = tid >> 2, lk = (tid & 3) * 4, kk = tid >> 5, n4 = (tid & 31) * 4;
    const auto fetch = [&](int k0) {
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = m0 + lr + 64 * h;
            xr[h] = zero;
            if (m < a.T && k0 + lk < a.K) xr[h] = *reinterpret_cast<const float4 *>(X + (size_t) m * a.ldx + k0 + lk);      // K is a multiple of 4
            wr[h] = zero;
            if (a.w_kn) {
                const int k = k0 + kk + 8 * h, n = n0 + n4;
                if (k < a.K && n < a.N) {
                    const float * p = W + (size_t) k * ldw + n;
                    if (n + 3 < a.N) wr[h] = *reinterpret_cast<const float4 *>(p);
                    else { wr[h].x = p[0]; if (n + 1 < a.N) wr[h].y = p[1]; if (n + 2 < a.N) wr[h].z = p[2]; }
                }
            } else {
                const int n = n0 + lr + 64 * h;
                if (n < a.N && k0 + lk < a.K) wr[h] = *reinterpret_cast<const float4 *>(W + (size_t) n * ldw + k0 + lk);
            }
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < a.K; k0 += SG_BK) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const float xv[4] = { xr[h].x, xr[h].y, xr[h].z, xr[h].w };
#pragma unroll
            for (int i = 0; i < 4; i++) Xs[lk + i][lr + 64 * h] = xv[i];
            if (a.w_kn) *reinterpret_cast<float4 *>(&Ws[kk + 8 * h][n4]) = wr[h];
            else {
                const float wv[4] = { wr[h].x, wr[h].y, wr[h].z, wr[h].w };
#pragma unroll
                for (int i = 0; i < 4; i++) Ws[lk + i][lr + 64 * h] = wv[i];
            }
        }
        __syncthreads();
        if (k0 + SG_BK < a.K) fetch(k0 + SG_BK);
#pragma unroll
        for (int k = 0; k < SG_BK; k++) {
            const float4 x0 = *reinterpret_cast<const float4 *>(&Xs[k][ty * 4]), x1 = *reinterpret_cast<const float4 *>(&Xs[k][64 + ty * 4]);
            const float4 w0 = *reinterpret_cast<const float4 *>(&Ws[k][tx * 4]), w1 = *reinterpret_cast<const float4 *>(&Ws[k][64 + tx * 4]);
            const float xa[8] = { x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w }, wa[8] = { w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w };
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(xa[i], wa[j], acc[i][j]);
        }
        __syncthreads();
    }
    float * Y = a.Y + (size_t) z1 * a.sY + (size_t) z2 * a.sY2;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (m >= a.T) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
            if (n < a.N) Y[(size_t) m * a.ldy + n] = acc[i][j] + (a.accum ? Y[(size_t) m * a.ldy + n] : 0.f);
        }
    }
}

// prompt portions with bfloat16 weights on the tensor cores: mma.sync m16n8k16 (bf16 x bf16 -> f32), CTA tile 128 (tokens)
// x 128 (rows of W) x 32, 8 warps of 64 x 32, operands staged through registers into padded shared memory (the float32
// activations are rounded to bfloat16 on the way), double-buffered. Needs K % 8 == 0 and 16-byte aligned rows (a.vec).
constexpr int MM_BM = 128, MM_BN = 128, MM_BK = 32, MM_LD = MM_BK + 8;     // row stride 80 B: conflict-free ldmatrix
__device__ __forceinline__ uint32_t smem_addr(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
__global__ void __launch_bounds__(256) k_gemm_bf16_mma(const LinArgs a) {
    __shared__ __align__(16) __nv_bfloat16 As[2][MM_BM][MM_LD];
    __shared__ __align__(16) __nv_bfloat16 Bs[2][MM_BN][MM_LD];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
    const int m0 = blockIdx.y * MM_BM, n0 = blockIdx.x * MM_BN;
    const int r0 = a.seg ? a.seg[blockIdx.z] : 0, T = a.seg ? a.seg[blockIdx.z + 1] - r0 : a.T;
    if (m0 >= T) return;
    const float * X = a.seg ? a.X + (size_t) r0 * a.ldx : a.X + (size_t) blockIdx.z * a.sX;
    const __nv_bfloat16 * W = reinterpret_cast<const __nv_bfloat16 *>(a.W) + (size_t) blockIdx.z * a.sW;
    // staging: 128 rows x 32 k per operand; thread -> (row = tid / 2 [+ 0], 16 consecutive k starting at (tid & 1) * 16)
    const int sr = tid >> 1, sk = (tid & 1) * 16;
    float4 xa[4]; uint4 wb[2];
    const auto fetch = [&](int k0) {
        const int m = m0 + sr, n = n0 + sr;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int k = k0 + sk + 4 * i;
            xa[i] = (m < T && k < a.K) ? *reinterpret_cast<const float4 *>(X + (size_t) m * a.ldx + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int k = k0 + sk + 8 * i;
            wb[i] = (n < a.N && k < a.K) ? *reinterpret_cast<const uint4 *>(W + (size_t) n * a.K + k) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    const auto stash = [&](int buf) {
        uint4 p0, p1;
        p0.x = pack_bf16(xa[0].x, xa[0].y); p0.y = pack_bf16(xa[0].z, xa[0].w); p0.z = pack_bf16(xa[1].x, xa[1].y); p0.w = pack_bf16(xa[1].z, xa[1].w);
        p1.x = pack_bf16(xa[2].x, xa[2].y); p1.y = pack_bf16(xa[2].z, xa[2].w); p1.z = pack_bf16(xa[3].x, xa[3].y); p1.w = pack_bf16(xa[3].z, xa[3].w);
        *reinterpret_cast<uint4 *>(&As[buf][sr][sk]) = p0;
        *reinterpret_cast<uint4 *>(&As[buf][sr][sk + 8]) = p1;
        *reinterpret_cast<uint4 *>(&Bs[buf][sr][sk]) = wb[0];
        *reinterpret_cast<uint4 *>(&Bs[buf][sr][sk + 8]) = wb[1];
    };
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f;
    const int nk = (a.K + MM_BK - 1) / MM_BK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kt = 0; kt < nk; kt++) {
        const int buf = kt & 1;
        if (kt + 1 < nk) fetch((kt + 1) * MM_BK);
#pragma unroll
        for (int ks = 0; ks < MM_BK; ks += 16) {
            uint32_t af[4][4], bf[2][4];
#pragma unroll
            for (int i = 0; i < 4; i++)      // A fragment of rows wm + 16 i ..: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
                ldsm_x4(af[i], smem_addr(&As[buf][wm + 16 * i + (lane & 15)][ks + (lane >> 4) * 8]));
#pragma unroll
            for (int j = 0; j < 2; j++)      // B: two n-tiles of 8 per ldmatrix.x4: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                ldsm_x4(bf[j], smem_addr(&Bs[buf][wn + 16 * j + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]));
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) mma_bf16(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
        }
        if (kt + 1 < nk) stash(buf ^ 1);
        __syncthreads();
    }
    float * Y = a.seg ? a.Y + (size_t) r0 * a.ldy : a.Y + (size_t) blockIdx.z * a.sY;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int m = m0 + wm + 16 * i + (lane >> 2) + (e >> 1) * 8;
                const int n = n0 + wn + 8 * j + (lane & 3) * 2 + (e & 1);
                if (a.glu) {            // this thread holds the (gate, up) pair of unit n / 2 in elements e, e + 1
                    if (!(e & 1) && m < T && n + 1 < a.N)
                        Y[(size_t) m * a.ldy + (n >> 1)] = clamped_glu(acc[i][j][e] + (a.bias ? a.bias[n] : 0.f), acc[i][j][e + 1] + (a.bias ? a.bias[n + 1] : 0.f), a.limit, a.alpha, a.up_shift);
                } else if (m < T && n < a.N) Y[(size_t) m * a.ldy + n] = acc[i][j][e] + (a.bias ? a.bias[n] : 0.f);
            }
}

// ---- prompt portions with bfloat16 weights on the 5th-generation tensor cores -------------------------------------------------
// tcgen05.mma (kind::f16, bf16 x bf16 -> f32) with the accumulator in tensor memory: D[128 tokens][256 rows of W] per CTA.
//   operands   both K-major in the canonical no-swizzle core-matrix order [8-row group][k-chunk][8 rows][16 B]: a 16-byte
//              cp.async per (row, k-chunk) drops global rows straight into that order (zero-fill past T, N or K), four stages of
//              K = 64 deep; the activations were rounded to bfloat16 by k_to_bf16 beforehand
//   issue      one thread: four K = 16 MMAs per stage, tcgen05.commit -> the stage's mbarrier (frees the stage for the refill)
//   epilogue   warp w owns TMEM lanes 32 (w & 3) .. + 31 (= tokens) and column half w >> 2: tcgen05.ld, bias / gated unit, stores
// Every wait on an mbarrier is bounded: on a timeout the CTA raises *err, skips what is left and still frees its tensor memory.
__global__ void k_to_bf16(const float * __restrict__ X, int ldx, int T, int K, long long sX, __nv_bfloat16 * __restrict__ Xb, long long sXb) {
    const float * x = X + (size_t) blockIdx.z * sX + (size_t) blockIdx.y * ldx;
    __nv_bfloat16 * o = Xb + (size_t) blockIdx.z * sXb + (size_t) blockIdx.y * K;
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < K; k += gridDim.x * blockDim.x) o[k] = __float2bfloat16_rn(x[k]);
}
constexpr int UM_BM = 128, UM_BN = 256, UM_BK = 64, UM_STAGES = 4;
constexpr int UM_A_BYTES = UM_BM * UM_BK * 2, UM_B_BYTES = UM_BN * UM_BK * 2, UM_STAGE_BYTES = UM_A_BYTES + UM_B_BYTES;
constexpr int UM_SMEM = UM_STAGES * UM_STAGE_BYTES + 1024;                 // + alignment slack
__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, volatile int * failed, int * err) {
    if (*failed) return false;
    for (uint32_t spins = 0; spins < (1u << 22); spins++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    *failed = 1;
    atomicExch(err, 1);
    return false;
}
__global__ void __launch_bounds__(256, 1) k_gemm_bf16_umma(const LinArgs a, const __nv_bfloat16 * __restrict__ Xb, long long sXb, int * err) {
    extern __shared__ uint8_t um_raw[];
    __shared__ __align__(8) uint64_t done[UM_STAGES];
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t smem0 = (smem_addr(um_raw) + 1023u) & ~1023u;
    const int m0 = blockIdx.y * UM_BM, n0 = blockIdx.x * UM_BN;
    const int r0 = a.seg ? a.seg[blockIdx.z] : 0, T = a.seg ? a.seg[blockIdx.z + 1] - r0 : a.T;
    if (m0 >= T) return;                      // the whole block, before anything is allocated
    const __nv_bfloat16 * X = a.seg ? Xb + (size_t) r0 * a.K : Xb + (size_t) blockIdx.z * sXb;
    const __nv_bfloat16 * W = reinterpret_cast<const __nv_bfloat16 *>(a.W) + (size_t) blockIdx.z * a.sW;
    volatile int * failed = &failed_s;
    if (tid == 0) {
        failed_s = 0;
        for (int s = 0; s < UM_STAGES; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_addr(&done[s])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_addr(&tmem_base_s)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    const int nk = (a.K + UM_BK - 1) / UM_BK;
    // one stage: 128 x 8 chunks of A (4 per thread) and 256 x 8 chunks of B (8 per thread); a warp's 32 chunks are 512 contiguous bytes
    const auto issue_copies = [&](int kt, int slot) {
        const uint32_t sa = smem0 + (uint32_t) slot * UM_STAGE_BYTES, sb = sa + UM_A_BYTES;
        const int k0 = kt * UM_BK;
#pragma unroll
        for (int i = 0; i < 12; i++) {
            const int idx = tid + 256 * (i < 4 ? i : i - 4);
            const int r_in = idx & 7, kc = (idx >> 3) & 7, rg = idx >> 6;
            const int k = k0 + kc * 8;
            const uint32_t off = (uint32_t) rg * 1024u + (uint32_t) kc * 128u + (uint32_t) r_in * 16u;
            if (i < 4) {
                const int m = m0 + rg * 8 + r_in;
                const bool ok = m < T && k < a.K;
                cp_async16(sa + off, ok ? (const void *) (X + (size_t) m * a.K + k) : (const void *) X, ok ? 16u : 0u);
            } else {
                const int n = n0 + rg * 8 + r_in;
                const bool ok = n < a.N && k < a.K;
                cp_async16(sb + off, ok ? (const void *) (W + (size_t) n * a.K + k) : (const void *) W, ok ? 16u : 0u);
            }
        }
    };
    for (int s = 0; s < UM_STAGES - 1; s++) {
        if (s < nk) issue_copies(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // instruction descriptor: D f32, A and B bf16, both K-major, N = 256, M = 128
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (UM_BN >> 3) << 17) | ((uint32_t) (UM_BM >> 4) << 24);
    for (int kt = 0; kt < nk; kt++) {
        const int slot = kt % UM_STAGES;
        asm volatile("cp.async.wait_group %0;" :: "n"(UM_STAGES - 2) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // the copies' writes -> visible to the tensor core's reads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && !*failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = smem0 + (uint32_t) slot * UM_STAGE_BYTES, sb = sa + UM_A_BYTES;
#pragma unroll
            for (int ks = 0; ks < UM_BK / 16; ks++) {
                // K-major, no swizzle: start >> 4 | (k-chunk stride 128 B) >> 4 << 16 | (8-row group stride 1024 B) >> 4 << 32 | version 1
                const uint64_t da = (uint64_t) (((sa + ks * 256u) >> 4) & 0x3fffu) | ((uint64_t) (128u >> 4) << 16) | ((uint64_t) (1024u >> 4) << 32) | (1ull << 46);
                const uint64_t db = (uint64_t) (((sb + ks * 256u) >> 4) & 0x3fffu) | ((uint64_t) (128u >> 4) << 16) | ((uint64_t) (1024u >> 4) << 32) | (1ull << 46);
                const uint32_t accumulate = (kt | ks) ? 1u : 0u;
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                             :: "r"(tmem), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_addr(&done[slot])) : "memory");
        }
        // refill the slot of stage kt - 1 with stage kt + STAGES - 1 once its MMAs have read it
        const int nxt = kt + UM_STAGES - 1;
        if (nxt < nk) {
            if (kt >= 1) mbar_wait_limited(smem_addr(&done[(kt - 1) % UM_STAGES]), (uint32_t) (((kt - 1) / UM_STAGES) & 1), failed, err);
            if (!*failed) issue_copies(nxt, nxt % UM_STAGES);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const bool ok = mbar_wait_limited(smem_addr(&done[(nk - 1) % UM_STAGES]), (uint32_t) (((nk - 1) / UM_STAGES) & 1), failed, err);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        const int m = m0 + 32 * (warp & 3) + lane, cbase = (warp >> 2) * (UM_BN / 2);
        const uint32_t taddr = tmem + ((uint32_t) (32 * (warp & 3)) << 16) + (uint32_t) cbase;
        float * Y = (a.seg ? a.Y + (size_t) r0 * a.ldy : a.Y + (size_t) blockIdx.z * a.sY) + (size_t) m * a.ldy;
#pragma unroll 1
        for (int c = 0; c < UM_BN / 2; c += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t r0, r1, r2, r3;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(taddr + (uint32_t) (c + 4 * j)) : "memory");
                v[4 * j] = __uint_as_float(r0); v[4 * j + 1] = __uint_as_float(r1); v[4 * j + 2] = __uint_as_float(r2); v[4 * j + 3] = __uint_as_float(r3);
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (m < T) {
                const int nb = n0 + cbase + c;
                if (!a.glu && nb + 15 < a.N && (a.ldy & 3) == 0 && ((uintptr_t) (Y + nb) & 15) == 0) {       // whole 16-byte stores
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        if (a.bias) { o.x += a.bias[nb + j]; o.y += a.bias[nb + j + 1]; o.z += a.bias[nb + j + 2]; o.w += a.bias[nb + j + 3]; }
                        *reinterpret_cast<float4 *>(Y + nb + j) = o;
                    }
                    continue;
                }
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const int n = n0 + cbase + c + j;
                    if (a.glu) {
                        if (n + 1 < a.N) Y[n >> 1] = clamped_glu(v[j] + (a.bias ? a.bias[n] : 0.f), v[j + 1] + (a.bias ? a.bias[n + 1] : 0.f), a.limit, a.alpha, a.up_shift);
                    } else {
                        if (n < a.N) Y[n] = v[j] + (a.bias ? a.bias[n] : 0.f);
                        if (n + 1 < a.N) Y[n + 1] = v[j + 1] + (a.bias ? a.bias[n + 1] : 0.f);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(256u) : "memory");
    }
}

// ---- minGRU: S_t = (1 - z) S_(t-1) + z * cand, gates from the current token only ----------------------------------------
// P[t] = [ z pre-activation | candidate pre-activation u | output-gate pre-activation ] (3 * width, biases included);
// cand = u + 1/2 for u >= 0, sigmoid(u) below. A[t] = S_t * silu(gate). One thread per channel walks the portion in order.
__global__ void k_mingru_scan(const float * __restrict__ P, int T, int width, float * __restrict__ state, float * __restrict__ A) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    float s = state[c];
    const int ld = 3 * width;
    constexpr int TB = 8;                 // tokens whose inputs are fetched together: the walk itself is serial, its loads are not
    for (int t0 = 0; t0 < T; t0 += TB) {
        float zp[TB], up[TB], gp[TB];
#pragma unroll
        for (int i = 0; i < TB; i++) {
            const float * p = P + (size_t) min(t0 + i, T - 1) * ld;
            zp[i] = p[c]; up[i] = p[width + c]; gp[i] = p[2 * width + c];
        }
#pragma unroll
        for (int i = 0; i < TB; i++) {
            if (t0 + i < T) {
                const float z = sigmoidf_(zp[i]), u = up[i];
                const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
                s = (1.0f - z) * s + z * cand;
                A[(size_t) (t0 + i) * width + c] = s * siluf_(gp[i]);
            }
        }
    }
    state[c] = s;
}

// ---- rotary positions on the first `dims` entries of a vector: pair i is (i, i + dims/2) ('rotate half') or, with
// adjacent = 1, the neighbours (2i, 2i + 1) -------------------------------------------------------------------------------
struct RopeArgs {
    const float * freq;   // [dims / 2] frequencies after any YaRN blend (host-built)
    int dims;
    float mag;            // factor on cos and sin (YaRN: 0.1 ln(factor) + 1; else 1)
    int adjacent;         // 0: pair i = entries (i, i + dims/2); 1: entries (2i, 2i + 1)
};
__device__ __forceinline__ int rope_lo(const RopeArgs & r, int i) { return r.adjacent ? 2 * i : i; }
__device__ __forceinline__ int rope_hi(const RopeArgs & r, int i) { return r.adjacent ? 2 * i + 1 : i + r.dims / 2; }
__device__ __forceinline__ void rope_pair(const RopeArgs & r, int pos, int i, float u, float v, float & ou, float & ov) {
    const float ang = (float) pos * r.freq[i];
    const float c = cosf(ang) * r.mag, s = sinf(ang) * r.mag;
    ou = u * c - v * s;
    ov = v * c + u * s;
}

// ---- latent attention, step 1: cache row + rotated query parts -------------------------------------------------------------
// P[t] = [ q: H x (D + R) | down-projection: rank + R ]. Per token: latent c = RMS norm of the first `rank` entries of the
// down-projection (plain weight), the last R entries are the rotated key part all heads share. The cache row of position p is
// [ c | rotated key part ] (rank + R floats): nothing else of a key or value is kept. The query row of head h is
// QK[t][h] = [ absorbed query (written by the per-head product q_unrotated . W_uk) | rotated query part ].
// dkv_off: where the down-projection starts in a row of P (H (D + R) in the layout above; a design whose queries pass a
// latent of their own keeps [ query latent | down-projection | ... ] there and has no rotated parts: R = 0).
// qnorm != nullptr: the first q_rank entries of the row (the query latent) are RMS-normed in place with that weight by a warp of their own.
__global__ void k_latent_prep(float * __restrict__ P, int ldp, int H, int D, int R, int rank, const float * __restrict__ cnorm, float eps,
                              RopeArgs rope, const StepState * __restrict__ st, float * __restrict__ cache, float * __restrict__ QK, int dkv_off,
                              const float * __restrict__ qnorm, int q_rank) {
    const int t = blockIdx.x, pos = st->pos0 + t, bk = blockIdx.y, nblk = gridDim.y;      // grid (T, blocks): the rotated vectors are dealt over the blocks of a token
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float * p = P + (size_t) t * ldp;
    const float * dkv = p + dkv_off;
    if (qnorm && bk == 0 && warp == (nw > 1 ? 1 : 0)) warp_group_norm(p, qnorm, q_rank, eps, p, lane);
    float * row = cache + (size_t) pos * (rank + R);
    const int half = rope.dims / 2;
    if (warp == 0 && bk == nblk - 1) {
        float ss = 0.f;
        for (int i = lane; i < rank; i += 32) ss = fmaf(dkv[i], dkv[i], ss);
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float) rank + eps);
        for (int i = lane; i < rank; i += 32) row[i] = dkv[i] * r * cnorm[i];
    }
    // rotated vectors: index H is the shared key part, 0..H-1 the heads' query parts
    for (int v = bk * nw + warp; v <= H; v += nw * nblk) {
        const float * src = v == H ? dkv + rank : p + (size_t) v * (D + R) + D;
        float * dst = v == H ? row + rank : QK + ((size_t) t * H + v) * (rank + R) + rank;
        for (int i = lane; i < R; i += 32) {
            if (i < half) { const int lo = rope_lo(rope, i), hi = rope_hi(rope, i); float a, b; rope_pair(rope, pos, i, src[lo], src[hi], a, b); dst[lo] = a; dst[hi] = b; }
            if (i >= rope.dims) dst[i] = src[i];
        }
    }
}

// ---- latent attention, step 2: scores over the window, soft-max with a sink, weighted sum of the cached latents -------------------
// Keys j with 0 <= p - j < window (window <= 0: every earlier position). The score of key j is (QK[t][h] . cache[j]) * scale
// over all rank + R entries: the absorbed query against the latent plus the rotated parts. The denominator also holds
// exp(sink[h]), which has no key and no value. OL[t][h] = sum_j w_j c_j (rank entries); the per-head value matrix is applied
// afterwards (W_uv (sum_j w_j c_j) = sum_j w_j v_j).
// All heads share one cached row per key, and neighbouring tokens share almost all their keys: a block takes TQ consecutive
// tokens x HQ heads (NQ = TQ HQ <= 16 queries) and one of `nsplit` slices of the tile's key range, so every cached row it
// loads serves NQ queries. nsplit == 1: the block finishes its queries. nsplit > 1 (decode: few queries, many SMs): it
// leaves the un-normalised sum and (max, sum of exponentials) of its slice; k_latent_combine merges the slices.
struct LatAttnArgs {
    const float * QK; const float * cache; const float * sink; const StepState * st;
    float * OL;            // [T][H][rank]
    float * part;          // [T][H][nsplit][rank]
    float * ml;            // [T][H][nsplit][2]
    int T, H, rank, R, window;
    float scale;
    int TQ, HQ, nsplit, smax;      // smax: score-row stride = the most keys one block can get
};
constexpr int LAT_NQ_MAX = 16, LAT_RPT = 2;
__global__ void __launch_bounds__(256) k_latent_attn(const LatAttnArgs a) {
    extern __shared__ float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int W = a.rank + a.R, NQ = a.TQ * a.HQ;
    const int t0 = blockIdx.x * a.TQ, h0 = blockIdx.y * a.HQ, z = blockIdx.z;
    const int nt = min(a.TQ, a.T - t0);
    const int p_first = a.st->pos0 + t0, p_last = p_first + nt - 1;
    const int jlo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int nkeys = p_last - jlo + 1;
    const int chunk = (nkeys + a.nsplit - 1) / a.nsplit;
    const int jb = jlo + z * chunk, je = min(jb + chunk, p_last + 1), nk = max(je - jb, 0);      // this block's keys [jb, je)
    float * q = sm;                       // [NQ][W]
    float * s = q + (size_t) NQ * W;      // [NQ][smax]
    float * inv = s + (size_t) NQ * a.smax;   // [NQ] factor on the weighted sum
    for (int i = tid; i < NQ * W; i += 256) {
        const int qi = i / W, e = i % W, tq = qi / a.HQ, h = h0 + qi % a.HQ;
        q[i] = (tq < nt && h < a.H) ? a.QK[((size_t) (t0 + tq) * a.H + h) * W + e] : 0.f;
    }
    __syncthreads();
    // scores: one warp per key, four queries at a time against the key row
    for (int j = warp; j < nk; j += 8) {
        const float * c = a.cache + (size_t) (jb + j) * W;
        for (int qb = 0; qb < NQ; qb += 4) {
            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
            for (int e = lane; e < W; e += 32) {
                const float kv = c[e];
#pragma unroll
                for (int k = 0; k < 4; k++) if (qb + k < NQ) acc[k] = fmaf(q[(size_t) (qb + k) * W + e], kv, acc[k]);
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                if (qb + k >= NQ) continue;
                const float v = warp_sum(acc[k]) * a.scale;
                const int qi = qb + k, tq = qi / a.HQ, p = p_first + tq, key = jb + j;
                const bool ok = tq < nt && h0 + qi % a.HQ < a.H && key <= p && (a.window <= 0 || p - key < a.window);
                if (lane == 0) s[(size_t) qi * a.smax + j] = ok ? v : -INFINITY;
            }
        }
    }
    __syncthreads();
    // soft-max per query: one warp per query
    for (int qi = warp; qi < NQ; qi += 8) {
        float * row = s + (size_t) qi * a.smax;
        const int tq = qi / a.HQ, h = h0 + qi % a.HQ;
        const bool live = tq < nt && h < a.H;
        float mx = -INFINITY;
        for (int j = lane; j < nk; j += 32) mx = fmaxf(mx, row[j]);
        mx = warp_max(mx);
        const float snk = (a.sink && live) ? a.sink[h] : -INFINITY;
        const float m = a.nsplit == 1 ? fmaxf(mx, snk) : mx;
        float sum = 0.f;
        for (int j = lane; j < nk; j += 32) { const float e = m == -INFINITY ? 0.f : expf(row[j] - m); row[j] = e; sum += e; }
        sum = warp_sum(sum);
        if (lane == 0) {
            if (a.nsplit == 1) {
                const float den = sum + (snk == -INFINITY ? 0.f : expf(snk - m));
                inv[qi] = den > 0.f ? 1.0f / den : 0.f;
            } else {
                inv[qi] = 1.0f;
                if (live) {
                    float * o = a.ml + (((size_t) (t0 + tq) * a.H + h) * a.nsplit + z) * 2;
                    o[0] = m; o[1] = sum;
                }
            }
        }
    }
    __syncthreads();
    // weighted sum of the latents: a thread owns LAT_RPT entries of the latent for all NQ queries
    for (int rb = 0; rb < a.rank; rb += 256 * LAT_RPT) {
        float acc[LAT_NQ_MAX][LAT_RPT];
#pragma unroll
        for (int qi = 0; qi < LAT_NQ_MAX; qi++)
#pragma unroll
            for (int k = 0; k < LAT_RPT; k++) acc[qi][k] = 0.f;
        for (int j = 0; j < nk; j++) {
            const float * c = a.cache + (size_t) (jb + j) * W + rb + tid;
            float cv[LAT_RPT];
#pragma unroll
            for (int k = 0; k < LAT_RPT; k++) cv[k] = rb + tid + 256 * k < a.rank ? c[256 * k] : 0.f;
#pragma unroll
            for (int qi = 0; qi < LAT_NQ_MAX; qi++) {
                if (qi < NQ) {
                    const float w = s[(size_t) qi * a.smax + j];
#pragma unroll
                    for (int k = 0; k < LAT_RPT; k++) acc[qi][k] = fmaf(w, cv[k], acc[qi][k]);
                }
            }
        }
#pragma unroll
        for (int qi = 0; qi < LAT_NQ_MAX; qi++) {
            if (qi >= NQ) continue;
            const int tq = qi / a.HQ, h = h0 + qi % a.HQ;
            if (tq >= nt || h >= a.H) continue;
            const size_t th = (size_t) (t0 + tq) * a.H + h;
            float * o = a.nsplit == 1 ? a.OL + th * a.rank : a.part + (th * a.nsplit + z) * a.rank;
#pragma unroll
            for (int k = 0; k < LAT_RPT; k++) {
                const int r = rb + tid + 256 * k;
                if (r < a.rank) o[r] = acc[qi][k] * inv[qi];
            }
        }
    }
}
// The same step for decode when a block's key slice fits shared memory: asynchronous copies bring the slice's cached rows in
// all at once (no chain of dependent loads), and scores and weighted sum read them from there. One to eight lanes own a
// (query, key) score; the weighted sum keeps k_latent_attn's ownership (LAT_RPT latent entries, all queries). VEC: rows are
// whole 16-byte chunks (rank + R a multiple of 4); otherwise 4-byte copies. Rows are padded so that the keys of a warp fall
// into different banks. Same results layout (OL, or part / ml for k_latent_combine) as k_latent_attn.
template <bool VEC>
__global__ void __launch_bounds__(256) k_latent_attn_staged(const LatAttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int W = a.rank + a.R, WP = VEC ? W + 4 : (W | 1), NQ = a.TQ * a.HQ;
    const int t0 = blockIdx.x * a.TQ, h0 = blockIdx.y * a.HQ, z = blockIdx.z;
    const int nt = min(a.TQ, a.T - t0);
    const int p_first = a.st->pos0 + t0, p_last = p_first + nt - 1;
    const int jlo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int nkeys = p_last - jlo + 1;
    const int chunk = (nkeys + a.nsplit - 1) / a.nsplit;
    const int jb = jlo + z * chunk, je = min(jb + chunk, p_last + 1), nk = max(je - jb, 0);      // this block's keys [jb, je)
    float * q = sm;                                   // [NQ][W]
    float * keys = q + (size_t) NQ * W;               // [smax][WP]
    float * s = keys + (size_t) a.smax * WP;          // [NQ][smax]
    float * inv = s + (size_t) NQ * a.smax;           // [NQ]
    {   // the slice's cached rows and the block's queries: every copy is issued before any is waited for
        const float * src = a.cache + (size_t) jb * W;
        const uint32_t dst = (uint32_t) __cvta_generic_to_shared(keys), qdst = (uint32_t) __cvta_generic_to_shared(q);
        if (VEC) {
            const int w4 = W >> 2;
            for (int i = tid; i < nk * w4; i += 256) {
                const int j = i / w4, e = (i - j * w4) << 2;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst + (uint32_t) (j * WP + e) * 4u), "l"(src + (size_t) j * W + e) : "memory");
            }
            for (int i = tid; i < NQ * w4; i += 256) {
                const int qi = i / w4, e = (i - qi * w4) << 2, tq = qi / a.HQ, h = h0 + qi % a.HQ;
                if (tq < nt && h < a.H)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(qdst + (uint32_t) (qi * W + e) * 4u), "l"(a.QK + ((size_t) (t0 + tq) * a.H + h) * W + e) : "memory");
                else *reinterpret_cast<float4 *>(q + (size_t) qi * W + e) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        } else {
            for (int i = tid; i < nk * W; i += 256) {
                const int j = i / W, e = i - j * W;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(dst + (uint32_t) (j * WP + e) * 4u), "l"(src + (size_t) j * W + e) : "memory");
            }
            for (int i = tid; i < NQ * W; i += 256) {
                const int qi = i / W, e = i - qi * W, tq = qi / a.HQ, h = h0 + qi % a.HQ;
                if (tq < nt && h < a.H)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(qdst + (uint32_t) (qi * W + e) * 4u), "l"(a.QK + ((size_t) (t0 + tq) * a.H + h) * W + e) : "memory");
                else q[(size_t) qi * W + e] = 0.f;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    // scores: `spl` neighbouring lanes share one (query, key) dot product when there are fewer scores than threads
    const int npairs = NQ * nk;
    int spl = 1;
    while (spl < 8 && npairs * spl * 2 <= 256) spl *= 2;
    for (int base = 0; base < npairs; base += 256 / spl) {
        const int pr = base + tid / spl, part = tid & (spl - 1);
        const bool live = pr < npairs;
        const int qi = live ? pr / nk : 0, j = live ? pr - qi * nk : 0;
        const float * qv = q + (size_t) qi * W, * kv = keys + (size_t) j * WP;
        const int lim = live ? W : 0;
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
        if (VEC) {
            for (int e = part * 4; e < lim; e += 4 * spl) {
                const float4 x = *reinterpret_cast<const float4 *>(qv + e), y = *reinterpret_cast<const float4 *>(kv + e);
                acc0 = fmaf(x.x, y.x, acc0); acc1 = fmaf(x.y, y.y, acc1); acc2 = fmaf(x.z, y.z, acc2); acc3 = fmaf(x.w, y.w, acc3);
            }
        } else {
            for (int e = part; e < lim; e += spl) acc0 = fmaf(qv[e], kv[e], acc0);
        }
        float v = (acc0 + acc1) + (acc2 + acc3);
        for (int o = 1; o < spl; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        v *= a.scale;
        const int tq = qi / a.HQ, p = p_first + tq, key = jb + j;
        const bool ok = tq < nt && h0 + qi % a.HQ < a.H && key <= p && (a.window <= 0 || p - key < a.window);
        if (live && part == 0) s[(size_t) qi * a.smax + j] = ok ? v : -INFINITY;
    }
    __syncthreads();
    // soft-max per query: one warp per query
    for (int qi = warp; qi < NQ; qi += 8) {
        float * row = s + (size_t) qi * a.smax;
        const int tq = qi / a.HQ, h = h0 + qi % a.HQ;
        const bool live = tq < nt && h < a.H;
        float mx = -INFINITY;
        for (int j = lane; j < nk; j += 32) mx = fmaxf(mx, row[j]);
        mx = warp_max(mx);
        const float snk = (a.sink && live) ? a.sink[h] : -INFINITY;
        const float m = a.nsplit == 1 ? fmaxf(mx, snk) : mx;
        float sum = 0.f;
        for (int j = lane; j < nk; j += 32) { const float e = m == -INFINITY ? 0.f : expf(row[j] - m); row[j] = e; sum += e; }
        sum = warp_sum(sum);
        if (lane == 0) {
            if (a.nsplit == 1) {
                const float den = sum + (snk == -INFINITY ? 0.f : expf(snk - m));
                inv[qi] = den > 0.f ? 1.0f / den : 0.f;
            } else {
                inv[qi] = 1.0f;
                if (live) {
                    float * o = a.ml + (((size_t) (t0 + tq) * a.H + h) * a.nsplit + z) * 2;
                    o[0] = m; o[1] = sum;
                }
            }
        }
    }
    __syncthreads();
    // weighted sum of the latents: a thread owns LAT_RPT entries of the latent for all NQ queries
    for (int rb = 0; rb < a.rank; rb += 256 * LAT_RPT) {
        float acc[LAT_NQ_MAX][LAT_RPT];
#pragma unroll
        for (int qi = 0; qi < LAT_NQ_MAX; qi++)
#pragma unroll
            for (int k = 0; k < LAT_RPT; k++) acc[qi][k] = 0.f;
        for (int j = 0; j < nk; j++) {
            const float * c = keys + (size_t) j * WP + rb + tid;
            float cv[LAT_RPT];
#pragma unroll
            for (int k = 0; k < LAT_RPT; k++) cv[k] = rb + tid + 256 * k < a.rank ? c[256 * k] : 0.f;
#pragma unroll
            for (int qi = 0; qi < LAT_NQ_MAX; qi++) {
                if (qi < NQ) {
                    const float w = s[(size_t) qi * a.smax + j];
#pragma unroll
                    for (int k = 0; k < LAT_RPT; k++) acc[qi][k] = fmaf(w, cv[k], acc[qi][k]);
                }
            }
        }
#pragma unroll
        for (int qi = 0; qi < LAT_NQ_MAX; qi++) {
            if (qi >= NQ) continue;
            const int tq = qi / a.HQ, h = h0 + qi % a.HQ;
            if (tq >= nt || h >= a.H) continue;
            const size_t th = (size_t) (t0 + tq) * a.H + h;
            float * o = a.nsplit == 1 ? a.OL + th * a.rank : a.part + (th * a.nsplit + z) * a.rank;
#pragma unroll
            for (int k = 0; k < LAT_RPT; k++) {
                const int r = rb + tid + 256 * k;
                if (r < a.rank) o[r] = acc[qi][k] * inv[qi];
            }
        }
    }
}

// merge of the key slices of one (token, head): weights exp(m_z - M) with M the largest maximum (the sink included)
__global__ void __launch_bounds__(256) k_latent_combine(const LatAttnArgs a) {       // grid (T, H, ceil(rank / 64)): 64 latent entries x 4 groups of slices
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t th = (size_t) t * a.H + h;
    const float * ml = a.ml + th * a.nsplit * 2;
    const float snk = a.sink ? a.sink[h] : -INFINITY;
    float M = snk;
    for (int z = 0; z < a.nsplit; z++) M = fmaxf(M, ml[2 * z]);
    float den = snk == -INFINITY ? 0.f : expf(snk - M);
    for (int z = 0; z < a.nsplit; z++) if (ml[2 * z] != -INFINITY) den += ml[2 * z + 1] * expf(ml[2 * z] - M);
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    __shared__ float wz[64];            // nsplit <= 64
    __shared__ float red[4][64];
    if (threadIdx.x < a.nsplit) wz[threadIdx.x] = ml[2 * threadIdx.x] != -INFINITY ? expf(ml[2 * threadIdx.x] - M) * inv : 0.f;
    __syncthreads();
    const int r = blockIdx.z * 64 + (threadIdx.x & 63), g = threadIdx.x >> 6;
    float acc = 0.f;
    if (r < a.rank) {
#pragma unroll 8
        for (int z = g; z < a.nsplit; z += 4) acc = fmaf(a.part[(th * a.nsplit + z) * a.rank + r], wz[z], acc);     // empty slices wrote zeros
    }
    red[g][threadIdx.x & 63] = acc;
    __syncthreads();
    if (g == 0 && r < a.rank) a.OL[th * a.rank + r] = (red[0][threadIdx.x] + red[1][threadIdx.x]) + (red[2][threadIdx.x] + red[3][threadIdx.x]);
}

// Prompt portions compute the same attention as two float32 products around a row soft-max (all on the CUDA cores: scores and
// weights stay 32-bit): per tile of TQ tokens, S = QK_tile (TQ H rows) x cached rows [jlo, jlo + nk)^T, then this kernel, then
// OL_tile = S x cached latents. Row (t, h) of tile i = t / TQ sees key jlo_i + n, jlo_i = pos0 + i TQ - span + 1 (window > 0)
// or 0; keys outside 0 <= p - j < window (or j < 0) get weight 0. One warp per row; the sink joins maximum and denominator.
__global__ void k_latent_softmax_rows(float * __restrict__ S, int n_rows, int H, int TQ, int nk, int window, int span, const float * __restrict__ sink,
                                      const StepState * __restrict__ st, float scale, int tile0) {
    const int lane = threadIdx.x & 31, row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);      // row = (t - tile0 TQ) H + h
    if (row >= n_rows) return;
    const int tl = row / H, h = row % H, t = tile0 * TQ + tl, p = st->pos0 + t;
    const int jlo = window > 0 ? st->pos0 + (t / TQ) * TQ - span + 1 : 0;      // span = min(window, positions so far): the range the product covered
    float * s = S + (size_t) row * nk;
    // valid n: j = jlo + n in [max(0, p - window + 1), p]
    const int n_lo = max(window > 0 ? p - window + 1 : 0, 0) - jlo, n_hi = p - jlo;         // inclusive
    float mx = -INFINITY;
    for (int n = n_lo + lane; n <= n_hi; n += 32) mx = fmaxf(mx, s[n] * scale);
    mx = warp_max(mx);
    const float snk = sink ? sink[h] : -INFINITY;
    const float m = fmaxf(mx, snk);
    float sum = 0.f;
    for (int n = n_lo + lane; n <= n_hi; n += 32) sum += expf(s[n] * scale - m);
    sum = warp_sum(sum);
    const float inv = 1.0f / (sum + (sink ? expf(snk - m) : 0.f));
    for (int n = lane; n < nk; n += 32) s[n] = (n >= n_lo && n <= n_hi) ? expf(s[n] * scale - m) * inv : 0.f;
}

// ---- gated delta rule --------------------------------------------------------------------------------------------------
// P[t] = [ q: KH x D | k: KH x D | v: H x V | beta logit: H | decay input: H | output-gate pre-activation: H x V ].
// Step 1: short causal convolution over time per channel of q | k | v (k_causal_conv with silu), then the steps below.

// ---- causal convolution over time on each channel ----------------------------------------------------------------------------
// y_t = sum_k w[c][k] x_(t - taps + 1 + k): the last weight is the current token's, inputs before the sequence's start are zero,
// no bias. hist holds the taps - 1 inputs before the portion ([taps - 1][C]); it is part of the sequence's state and is moved
// on by k_causal_conv_hist after the portion. act: 0 none, 1 silu. add_input: Y = X + conv(X) (a convolution around a
// residual path). blockIdx.z runs over a batch of independent convolutions (element strides sX / sW / sH / sY). Channels from
// `split` on can be written to the row of the token's position in a per-position cache instead of Y (an attention's keys and
// values after their convolution).
struct ConvArgs {
    const float * X; int ldx; long long sX;
    const float * w; long long sW;
    float * hist; long long sH;
    float * Y; int ldy; long long sY;
    int T, C, taps, act, add_input;
    const StepState * st; float * cache; int ldc, split;      // cache == nullptr: everything goes to Y
    int fuse_hist;                                            // T == 1: the thread also moves its channel's history on (no second launch)
};
__global__ void k_causal_conv(const ConvArgs a) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y, z = blockIdx.z;
    if (c >= a.C) return;
    const float * X = a.X + (size_t) z * a.sX;
    const float * w = a.w + (size_t) z * a.sW + (size_t) c * a.taps;
    const float * hist = a.hist + (size_t) z * a.sH;
    float y = 0.f;
    for (int k = 0; k < a.taps; k++) {
        const int tau = t - (a.taps - 1) + k;
        const float in = tau >= 0 ? X[(size_t) tau * a.ldx + c] : hist[(size_t) (a.taps - 1 + tau) * a.C + c];
        y = fmaf(w[k], in, y);
    }
    if (a.add_input) y += X[(size_t) t * a.ldx + c];
    if (a.act == 1) y = siluf_(y);
    if (a.cache && c >= a.split) a.cache[(size_t) (a.st->pos0 + t) * a.ldc + (c - a.split)] = y;
    else a.Y[(size_t) z * a.sY + (size_t) t * a.ldy + c] = y;
    if (a.fuse_hist && a.taps > 1) {                          // one token: drop the oldest input of this channel, append the new one
        float * h = a.hist + (size_t) z * a.sH;
        for (int i = 0; i + 2 < a.taps; i++) h[(size_t) i * a.C + c] = h[(size_t) (i + 1) * a.C + c];
        h[(size_t) (a.taps - 2) * a.C + c] = X[c];
    }
}
// afterwards: the history becomes the last taps - 1 inputs of (history ++ portion)
__global__ void k_causal_conv_hist(const ConvArgs a) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, z = blockIdx.z;
    if (c >= a.C) return;
    const float * X = a.X + (size_t) z * a.sX;
    float * hist = a.hist + (size_t) z * a.sH;
    for (int i = 0; i < a.taps - 1; i++) {          // ascending: entry i reads old entries at T + i > i only
        const int f = a.T + i;                       // index into (history ++ portion)
        hist[(size_t) i * a.C + c] = f < a.taps - 1 ? hist[(size_t) f * a.C + c] : X[(size_t) (f - (a.taps - 1)) * a.ldx + c];
    }
}
// Step 2, per token: q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q is also scaled by D^(-1/2);
// beta = sigmoid(beta logit); decay g = exp(-exp(A_log) * softplus(decay input + dt_bias)). BG[t] = [ beta: H | g: H ].
__global__ void k_delta_gates(float * __restrict__ CV, int C, const float * __restrict__ P, int ldp, int H, int KH, int D, int V,
                              const float * __restrict__ A_log, const float * __restrict__ dt_bias, float * __restrict__ BG) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float * cv = CV + (size_t) t * C;
    for (int v = warp; v < 2 * KH; v += nw) {     // q heads, then k heads
        float * x = cv + (size_t) v * D;
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        float r = 1.0f / sqrtf(ss + 1e-6f);
        if (v < KH) r *= 1.0f / sqrtf((float) D);
        for (int i = lane; i < D; i += 32) x[i] *= r;
    }
    const float * p = P + (size_t) t * ldp + 2 * KH * D + H * V;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        BG[(size_t) t * 2 * H + h] = sigmoidf_(p[h]);
        BG[(size_t) t * 2 * H + H + h] = expf(-expf(A_log[h]) * softplusf_(p[H + h] + dt_bias[h]));
    }
}
// Step 3, the recurrence per head, in this order: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q — the read-out
// sees the current token's write. S is [D][V] per head in float32; one thread owns one column of S (D registers) and walks
// the portion token by token; head h reads q / k head h / (H / KH). DMAX >= D is the register tile (rows beyond D stay zero).
template <int DMAX>
__global__ void __launch_bounds__(128) k_delta_scan(const float * __restrict__ CV, int C, const float * __restrict__ BG, int T, int H, int KH, int D, int V,
                                                    float * __restrict__ S, float * __restrict__ O) {
    constexpr int TT = 8;
    __shared__ float ks[TT][DMAX], qs[TT][DMAX], bg[TT][2], vs[TT][128];
    const int h = blockIdx.x, col = blockIdx.y * blockDim.x + threadIdx.x, kh = h / (H / KH);
    const bool live = col < V;
    float s[DMAX];
    float * Sh = S + (size_t) h * D * V;
#pragma unroll
    for (int d = 0; d < DMAX; d++) s[d] = (live && d < D) ? Sh[(size_t) d * V + col] : 0.f;
    for (int t0 = 0; t0 < T; t0 += TT) {
        const int nt = min(TT, T - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * DMAX; i += blockDim.x) {
            const int tt = i / DMAX, d = i % DMAX;
            const float * cv = CV + (size_t) (t0 + tt) * C;
            qs[tt][d] = d < D ? cv[(size_t) kh * D + d] : 0.f;
            ks[tt][d] = d < D ? cv[(size_t) (KH + kh) * D + d] : 0.f;
        }
        if (threadIdx.x < 2 * nt) bg[threadIdx.x >> 1][threadIdx.x & 1] = BG[(size_t) (t0 + (threadIdx.x >> 1)) * 2 * H + (threadIdx.x & 1) * H + h];
        // this column's values of the tile, fetched together (the walk below is serial, its loads are not)
#pragma unroll
        for (int tt = 0; tt < TT; tt++) vs[tt][threadIdx.x] = (live && tt < nt) ? CV[(size_t) (t0 + tt) * C + (size_t) 2 * KH * D + (size_t) h * V + col] : 0.f;
        __syncthreads();
        if (!live) continue;
        for (int tt = 0; tt < nt; tt++) {
            const int t = t0 + tt;
            const float beta = bg[tt][0], g = bg[tt][1];
            const float v = vs[tt][threadIdx.x];
            float dot = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; d++) { s[d] *= g; dot = fmaf(s[d], ks[tt][d], dot); }
            const float u = beta * (v - dot);
            float o = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; d++) { s[d] = fmaf(ks[tt][d], u, s[d]); o = fmaf(s[d], qs[tt][d], o); }
            O[(size_t) t * H * V + (size_t) h * V + col] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; d++) if (d < D) Sh[(size_t) d * V + col] = s[d];
    }
}
// Step 4: each head's read-out over its root mean square (eps inside the root), times a weight (w_stride 0: one [V] shared by
// the heads; V: [H][V]), times the activated output gate (silu, or sigmoid when gate_sigmoid). One warp per (token, head).
__global__ void k_delta_out(const float * __restrict__ O, const float * __restrict__ P, int ldp, int gate_off, int H, int V,
                            const float * __restrict__ normw, int w_stride, int gate_sigmoid, float eps, float * __restrict__ A) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = blockIdx.y * nw + warp; h < H; h += gridDim.y * nw) {
        const float * o = O + (size_t) t * H * V + (size_t) h * V;
        const float * gp = P + (size_t) t * ldp + gate_off + (size_t) h * V;
        float ss = 0.f;
        for (int i = lane; i < V; i += 32) ss = fmaf(o[i], o[i], ss);
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float) V + eps);
        const float * nw = normw ? normw + (size_t) h * w_stride : nullptr;      // nullptr: no weight
        for (int i = lane; i < V; i += 32) A[(size_t) t * H * V + (size_t) h * V + i] = o[i] * r * (nw ? nw[i] : 1.0f) * (gate_sigmoid ? sigmoidf_(gp[i]) : siluf_(gp[i]));
    }
}

// ---- generalized delta rule: per-channel decay and per-channel removal along the unit key ------------------------------------
// P[t] = [ r: H x D | k: H x D | v: H x V | output-gate pre-activation: H x V | removal logit: H x D (bias included) | decay latent ].
// Per token and head, all in float32:
//   w = exp(-e^(-1/2) sigmoid(decay logit))      decay of each key channel, in (e^(-e^(-1/2)), 1)
//   u = k / sqrt(sum k^2 + 1e-6)                 unit key
//   b = sigmoid(removal logit) * u
// G[t][h] = [ w | u | b ] (3 D floats). One block per (token, head).
constexpr float GDELTA_DECAY_RATE = 0.60653065971263342f;      // e^(-1/2)
// The decay logits are a low-rank product computed here: logit = w0 + W2 tanh(latent), latent = the last `lora` entries of the
// row (lat_off), W2 [H D][lora] in the model's storage type; the block keeps tanh(latent) in shared memory.
template <typename WT>
__global__ void k_gdelta_prep(const float * __restrict__ P, int ldp, int k_off, int a_off, int lat_off, int lora, const WT * __restrict__ W2, const float * __restrict__ w0,
                              int H, int D, float * __restrict__ G) {
    extern __shared__ float sm_prep[];
    float * lat = sm_prep, * wl = sm_prep + lora;            // tanh(latent) [lora], decay logits of this head [D]
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int i = threadIdx.x; i < lora; i += blockDim.x) lat[i] = tanhf(P[(size_t) t * ldp + lat_off + i]);
    __syncthreads();
    // a warp per row of W2, lanes striding the latent (the row is read in whole lines), PREP_RB rows at a time so that their
    // loads are in flight together
    constexpr int PREP_RB = 8;
    for (int i0 = warp * PREP_RB; i0 < D; i0 += nw * PREP_RB) {
        float acc[PREP_RB];
#pragma unroll
        for (int q = 0; q < PREP_RB; q++) acc[q] = 0.f;
        for (int j = lane; j < lora; j += 32) {
            const float x = lat[j];
#pragma unroll
            for (int q = 0; q < PREP_RB; q++) if (i0 + q < D) acc[q] = fmaf(wf(W2, ((size_t) h * D + i0 + q) * lora + j), x, acc[q]);
        }
#pragma unroll
        for (int q = 0; q < PREP_RB; q++) {
            const float v = warp_sum(acc[q]);
            if (lane == 0 && i0 + q < D) wl[i0 + q] = v + w0[(size_t) h * D + i0 + q];
        }
    }
    const float * k = P + (size_t) t * ldp + k_off + (size_t) h * D;
    const float * al = P + (size_t) t * ldp + a_off + (size_t) h * D;
    float * g = G + ((size_t) t * H + h) * 3 * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) ss = fmaf(k[i], k[i], ss);      // every warp for itself: no second barrier round
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss + 1e-6f);
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float u = k[i] * r;
        g[i] = expf(-GDELTA_DECAY_RATE * sigmoidf_(wl[i]));
        g[D + i] = u;
        g[2 * D + i] = sigmoidf_(al[i]) * u;
    }
}
// The recurrence per head; both corrections read the old state:
//   S_t = diag(w) S_(t-1) - b (u^T S_(t-1)) + k v^T,   o_t = S_t^T r
// S is [D][V] per head in float32 and stays in registers for the whole portion. Four neighbouring lanes share one column of S,
// each holding a quarter of its rows (DMAX / 4 registers): dot = sum_m u_m s_m and o = sum_i s_i r_i are partial sums closed
// by two shuffles, s_i <- w_i s_i - b_i dot + k_i v in between. A block of up to 512 threads (128 columns) walks the portion
// token by token; r, k, w, u, b of a few tokens arrive in shared memory by asynchronous copies while the tokens before
// them are walked (two buffers), each quarter of the rows padded apart so that the four lanes' 16-byte reads fall into
// different banks.
constexpr int GD_RG = 4, GD_PAD = 4;
__device__ __forceinline__ void cp_async4(float * dst, const float * src, bool real) {      // real == false: the destination gets a zero
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" :: "r"((uint32_t) __cvta_generic_to_shared(dst)), "l"(src), "r"(real ? 4u : 0u) : "memory");
}
template <int DMAX>
__global__ void __launch_bounds__(512) k_gdelta_scan(const float * __restrict__ P, int ldp, int r_off, int k_off, int v_off, const float * __restrict__ G,
                                                     int T, int H, int D, int V, float * __restrict__ S, float * __restrict__ O) {
    // two buffers of GD_TT tokens: asynchronous copies fill one while the other is walked
    constexpr int TT = DMAX > 128 ? 2 : 4, DR = DMAX / GD_RG, ROW = GD_RG * (DR + GD_PAD);
    __shared__ __align__(16) float rs[2][TT][ROW], ks[2][TT][ROW], ws[2][TT][ROW], us[2][TT][ROW], bs[2][TT][ROW], vs[2][TT][128];
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, rg = lane & 3, ncols = blockDim.x / GD_RG;
    const int cl = (tid >> 5) * 8 + (lane >> 2), col = blockIdx.y * ncols + cl;     // a warp covers 8 columns x 4 quarters
    const bool live = col < V;
    const auto stage = [&](int t0, int buf) {
        const int nt = min(TT, T - t0);
        for (int i = tid; i < nt * DMAX; i += blockDim.x) {
            const int tt = i / DMAX, d = i % DMAX, at = (d / DR) * (DR + GD_PAD) + d % DR;
            const bool in = d < D;
            const float * p = P + (size_t) (t0 + tt) * ldp + (size_t) h * D + (in ? d : 0);
            const float * g = G + ((size_t) (t0 + tt) * H + h) * 3 * D + (in ? d : 0);
            cp_async4(&rs[buf][tt][at], p + r_off, in);
            cp_async4(&ks[buf][tt][at], p + k_off, in);
            cp_async4(&ws[buf][tt][at], g, in);
            cp_async4(&us[buf][tt][at], g + D, in);
            cp_async4(&bs[buf][tt][at], g + 2 * D, in);
        }
        for (int i = tid; i < nt * ncols; i += blockDim.x) {
            const int tt = i / ncols, c = i % ncols;
            const bool in = blockIdx.y * ncols + c < V;
            cp_async4(&vs[buf][tt][c], P + (size_t) (t0 + tt) * ldp + v_off + (size_t) h * V + (in ? blockIdx.y * ncols + c : 0), in);
        }
    };
    stage(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    float s[DR];
    float * Sh = S + (size_t) h * D * V;
#pragma unroll
    for (int i = 0; i < DR; i++) { const int d = rg * DR + i; s[i] = (live && d < D) ? Sh[(size_t) d * V + col] : 0.f; }
    const int base = rg * (DR + GD_PAD);
    for (int t0 = 0, buf = 0; t0 < T; t0 += TT, buf ^= 1) {
        const int nt = min(TT, T - t0);
        if (t0 + TT < T) stage(t0 + TT, buf ^ 1);            // its last readers passed the barrier that closed the previous walk
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this tile's copies (the group before the one just committed) have landed
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {                    // every lane walks (the shuffles need the whole warp); dead columns hold zeros
            const float v = vs[buf][tt][cl];
            float dp[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
            for (int i = 0; i < DR; i++) dp[i & 3] = fmaf(us[buf][tt][base + i], s[i], dp[i & 3]);
            float dot = (dp[0] + dp[1]) + (dp[2] + dp[3]);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            float op[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
            for (int i = 0; i < DR; i++) {
                s[i] = fmaf(ws[buf][tt][base + i], s[i], fmaf(ks[buf][tt][base + i], v, -bs[buf][tt][base + i] * dot));
                op[i & 3] = fmaf(s[i], rs[buf][tt][base + i], op[i & 3]);
            }
            float o = (op[0] + op[1]) + (op[2] + op[3]);
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (rg == 0 && live) O[(size_t) (t0 + tt) * H * V + (size_t) h * V + col] = o;
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DR; i++) { const int d = rg * DR + i; if (d < D) Sh[(size_t) d * V + col] = s[i]; }
    }
}

// ---- differential soft-max attention over a sliding window, grouped key/value heads -------------------------------------------
// Every query head carries two score maps over the same values: Q[t] = [ head h: map 1 (D) | map 2 (D) ], the cached row of
// position j is [ key head g: map 1 | map 2 (G x 2 x D) | value head g (G x V) ], query head h reads key/value head
// h / (H / G). Position p sees j with 0 <= p - j < window (window <= 0: every j <= p). With a1, a2 the two maps' soft-max
// averages of the values: o = a1 - lambda a2, divided by its root mean square over the V values (eps inside the root, no
// weight), times out_scale. No positions enter the scores. Everything in float32.
// A block takes TQ consecutive tokens of one head; the 8 / TQ warps of a query walk its keys in alternating chunks of 32 (one
// lane per key for the scores, one lane per 32nd value channel for the weighted sum, running maximum and denominator per
// map) and are merged through shared memory; decode (TQ = 1) so spreads one query's window over the whole block.
struct DiffAttnArgs {
    const float * Q; int ldq;
    const float * cache; int ldc;
    const StepState * st;
    float * A;                  // [T][H x V]
    int T, H, G, D, V, window;
    float scale, lambda, out_scale, eps;
    int TQ, vec;                // vec: D and ldc are multiples of 4 and the cache is 16-byte aligned
    int nsplit;                 // > 1: blockIdx.z takes every nsplit-th group of chunks; the block that finishes last merges
    float * part;               // [T][H][nsplit][4 + 64 VPL] partial (maxima, denominators, sums)
    int * counter;              // [T][H] blocks done; the merging block puts it back to 0
};
template <int VPL>
__global__ void __launch_bounds__(256) k_diff_attn(const DiffAttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int WPQ = 8 / a.TQ, qi = warp / WPQ, wq = warp % WPQ;
    const int h = blockIdx.y, g = h / (a.H / a.G), t0 = blockIdx.x * a.TQ, t = t0 + qi;
    const int D2 = 2 * a.D;
    float * qs = sm;                                        // [TQ][2 D]
    float * mg = sm + (size_t) a.TQ * D2;                   // [8 warps][4 + 2 x 32 VPL]
    constexpr int MGW = 4 + 64 * VPL;
    for (int i = tid; i < a.TQ * D2; i += 256) {
        const int q = i / D2, e = i - q * D2;
        qs[i] = t0 + q < a.T ? a.Q[(size_t) (t0 + q) * a.ldq + (size_t) h * D2 + e] : 0.f;
    }
    __syncthreads();
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f;
    float acc1[VPL], acc2[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++) { acc1[i] = 0.f; acc2[i] = 0.f; }
    if (t < a.T) {
        const int p = a.st->pos0 + t;
        const int jlo = a.window > 0 ? max(0, p - a.window + 1) : 0;
        const int nchunk = (p - jlo + 1 + 31) / 32;
        const float * q1 = qs + (size_t) qi * D2, * q2 = q1 + a.D;
        const size_t koff = (size_t) g * D2, voff = (size_t) a.G * D2 + (size_t) g * a.V;
        for (int c = blockIdx.z * WPQ + wq; c < nchunk; c += WPQ * a.nsplit) {
            const int jb = jlo + c * 32, j = jb + lane, cnt = min(32, p - jb + 1);
            float s1 = -INFINITY, s2 = -INFINITY;
            if (lane < cnt) {
                const float * k1 = a.cache + (size_t) j * a.ldc + koff, * k2 = k1 + a.D;
                float x0 = 0.f, x1 = 0.f, y0 = 0.f, y1 = 0.f;
                if (a.vec) {
#pragma unroll 8
                    for (int e = 0; e < a.D; e += 4) {                // unrolled: the loads of several steps are in flight together
                        const float4 ka = __ldg(reinterpret_cast<const float4 *>(k1 + e)), kb = __ldg(reinterpret_cast<const float4 *>(k2 + e));
                        const float4 qa = *reinterpret_cast<const float4 *>(q1 + e), qb = *reinterpret_cast<const float4 *>(q2 + e);
                        x0 = fmaf(qa.x, ka.x, x0); x1 = fmaf(qa.y, ka.y, x1); x0 = fmaf(qa.z, ka.z, x0); x1 = fmaf(qa.w, ka.w, x1);
                        y0 = fmaf(qb.x, kb.x, y0); y1 = fmaf(qb.y, kb.y, y1); y0 = fmaf(qb.z, kb.z, y0); y1 = fmaf(qb.w, kb.w, y1);
                    }
                } else {
                    for (int e = 0; e < a.D; e++) { x0 = fmaf(q1[e], k1[e], x0); y0 = fmaf(q2[e], k2[e], y0); }
                }
                s1 = (x0 + x1) * a.scale; s2 = (y0 + y1) * a.scale;
            }
            const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));      // finite: the chunk holds at least one key
            const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
            const float e1 = lane < cnt ? expf(s1 - n1) : 0.f, e2 = lane < cnt ? expf(s2 - n2) : 0.f;
            l1 = l1 * c1 + warp_sum(e1); l2 = l2 * c2 + warp_sum(e2);
            m1 = n1; m2 = n2;
#pragma unroll
            for (int i = 0; i < VPL; i++) { acc1[i] *= c1; acc2[i] *= c2; }
            const float * vrow = a.cache + (size_t) jb * a.ldc + voff;
#pragma unroll 4
            for (int kk = 0; kk < cnt; kk++) {
                const float w1 = __shfl_sync(0xffffffffu, e1, kk), w2 = __shfl_sync(0xffffffffu, e2, kk);
#pragma unroll
                for (int i = 0; i < VPL; i++) {
                    const int vi = lane + 32 * i;
                    const float v = vi < a.V ? __ldg(vrow + (size_t) kk * a.ldc + vi) : 0.f;
                    acc1[i] = fmaf(w1, v, acc1[i]); acc2[i] = fmaf(w2, v, acc2[i]);
                }
            }
        }
    }
    {
        float * o = mg + (size_t) warp * MGW;
        if (lane == 0) { o[0] = m1; o[1] = l1; o[2] = m2; o[3] = l2; }
#pragma unroll
        for (int i = 0; i < VPL; i++) { o[4 + lane + 32 * i] = acc1[i]; o[4 + 32 * VPL + lane + 32 * i] = acc2[i]; }
    }
    __syncthreads();
    if (wq != 0 || t >= a.T) return;
    // merge of the query's warps (a warp that had no chunk left m = -inf, l = 0), then the difference and its norm
    float M1 = -INFINITY, M2 = -INFINITY;
    for (int w = 0; w < WPQ; w++) { const float * o = mg + (size_t) (warp + w) * MGW; M1 = fmaxf(M1, o[0]); M2 = fmaxf(M2, o[2]); }
    float L1 = 0.f, L2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i++) { acc1[i] = 0.f; acc2[i] = 0.f; }
    for (int w = 0; w < WPQ; w++) {
        const float * o = mg + (size_t) (warp + w) * MGW;
        const float f1 = o[0] == -INFINITY ? 0.f : expf(o[0] - M1), f2 = o[2] == -INFINITY ? 0.f : expf(o[2] - M2);
        L1 = fmaf(o[1], f1, L1); L2 = fmaf(o[3], f2, L2);
#pragma unroll
        for (int i = 0; i < VPL; i++) { acc1[i] = fmaf(o[4 + lane + 32 * i], f1, acc1[i]); acc2[i] = fmaf(o[4 + 32 * VPL + lane + 32 * i], f2, acc2[i]); }
    }
    if (a.nsplit > 1) {
        // leave this block's share; the block that arrives last (per token and head) merges all shares the same way
        const size_t th = (size_t) t * a.H + h;
        float * o = a.part + (th * a.nsplit + blockIdx.z) * MGW;
        if (lane == 0) { o[0] = M1; o[1] = L1; o[2] = M2; o[3] = L2; }
#pragma unroll
        for (int i = 0; i < VPL; i++) { o[4 + lane + 32 * i] = acc1[i]; o[4 + 32 * VPL + lane + 32 * i] = acc2[i]; }
        __threadfence();
        int done = 0;
        if (lane == 0) done = atomicAdd(a.counter + th, 1);
        done = __shfl_sync(0xffffffffu, done, 0);
        if (done != a.nsplit - 1) return;
        __threadfence();
        if (lane == 0) a.counter[th] = 0;
        const float * ps = a.part + th * a.nsplit * MGW;
        M1 = -INFINITY; M2 = -INFINITY;
        for (int z = 0; z < a.nsplit; z++) { M1 = fmaxf(M1, __ldcg(ps + (size_t) z * MGW)); M2 = fmaxf(M2, __ldcg(ps + (size_t) z * MGW + 2)); }
        L1 = 0.f; L2 = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; i++) { acc1[i] = 0.f; acc2[i] = 0.f; }
        for (int z = 0; z < a.nsplit; z++) {
            const float * q = ps + (size_t) z * MGW;
            const float z1 = __ldcg(q), z2 = __ldcg(q + 2);
            const float f1 = z1 == -INFINITY ? 0.f : expf(z1 - M1), f2 = z2 == -INFINITY ? 0.f : expf(z2 - M2);
            L1 = fmaf(__ldcg(q + 1), f1, L1); L2 = fmaf(__ldcg(q + 3), f2, L2);
#pragma unroll
            for (int i = 0; i < VPL; i++) { acc1[i] = fmaf(__ldcg(q + 4 + lane + 32 * i), f1, acc1[i]); acc2[i] = fmaf(__ldcg(q + 4 + 32 * VPL + lane + 32 * i), f2, acc2[i]); }
        }
    }
    const float i1 = 1.0f / L1, i2 = a.lambda / L2;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        const float d = lane + 32 * i < a.V ? acc1[i] * i1 - acc2[i] * i2 : 0.f;
        acc1[i] = d; ss = fmaf(d, d, ss);
    }
    ss = warp_sum(ss);
    const float r = a.out_scale / sqrtf(ss / (float) a.V + a.eps);
#pragma unroll
    for (int i = 0; i < VPL; i++) if (lane + 32 * i < a.V) a.A[(size_t) t * a.H * a.V + (size_t) h * a.V + lane + 32 * i] = acc1[i] * r;
}

// Prompt portions compute the same attention as float32 products, like the latent attention: per tile of TQ tokens and per
// key/value head g, S_m = Q_(g,m) K_(g,m)^T for both maps (rows: the tile's tokens x the R = H / G query heads of the group), then
// k_diff_softmax_rows turns the pair of score rows into ONE row of weights P = softmax(S_1) - lambda softmax(S_2) (both maps
// weigh the same values, so the difference can be taken on the weights), then O = P V_g, then k_diff_norm_out.
// k_diff_q_layout: queries [T][H][2][D] -> Qr[g][m][Tpad][R][D] (rows of one group and map contiguous; rows past T zero)
__global__ void k_diff_q_layout(const float * __restrict__ Q, int ldq, int T, int Tpad, int H, int G, int D, float * __restrict__ Qr) {
    const int t = blockIdx.x, R = H / G, nq = H * 2 * D;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        const int h = i / (2 * D), m = (i / D) & 1, d = i % D, g = h / R, hq = h - g * R;
        Qr[((((size_t) g * 2 + m) * Tpad + t) * R + hq) * D + d] = t < T ? Q[(size_t) t * ldq + i] : 0.f;
    }
}
// S holds, for a group of ng tiles starting at tile0, [g][m][ng TQ R rows][nk]; row (tile, token, head) sees key jlo + n with
// jlo = pos0 + tile TQ - span + 1 (window > 0) or 0, as in k_latent_softmax_rows. The weights replace map 1's row.
__global__ void k_diff_softmax_rows(float * __restrict__ S, int n_rows, int G, int R, int TQ, int nk, int window, int span,
                                    const StepState * __restrict__ st, float scale, float lambda, int tile0, int T) {
    const int lane = threadIdx.x & 31, id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (id >= n_rows * G) return;
    const int g = id / n_rows, r = id - g * n_rows;
    const int tile = tile0 + r / (TQ * R), t = tile * TQ + (r % (TQ * R)) / R, p = st->pos0 + t;
    float * s1 = S + ((size_t) (2 * g) * n_rows + r) * nk;
    const float * s2 = s1 + (size_t) n_rows * nk;
    if (t >= T) { for (int n = lane; n < nk; n += 32) s1[n] = 0.f; return; }
    const int jlo = window > 0 ? st->pos0 + tile * TQ - span + 1 : 0;
    const int n_lo = max(window > 0 ? p - window + 1 : 0, 0) - jlo, n_hi = p - jlo;         // inclusive
    float m1 = -INFINITY, m2 = -INFINITY;
    for (int n = n_lo + lane; n <= n_hi; n += 32) { m1 = fmaxf(m1, s1[n] * scale); m2 = fmaxf(m2, s2[n] * scale); }
    m1 = warp_max(m1); m2 = warp_max(m2);
    float l1 = 0.f, l2 = 0.f;
    for (int n = n_lo + lane; n <= n_hi; n += 32) { l1 += expf(s1[n] * scale - m1); l2 += expf(s2[n] * scale - m2); }
    l1 = warp_sum(l1); l2 = warp_sum(l2);
    const float i1 = 1.0f / l1, i2 = lambda / l2;
    for (int n = lane; n < nk; n += 32) s1[n] = (n >= n_lo && n <= n_hi) ? expf(s1[n] * scale - m1) * i1 - expf(s2[n] * scale - m2) * i2 : 0.f;
}
// Or[g][Tpad][R][V] -> A[t][h][V]: each head's vector over its root mean square (eps inside the root), times out_scale
__global__ void k_diff_norm_out(const float * __restrict__ Or, int Tpad, int H, int G, int V, float eps, float out_scale, float * __restrict__ A) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, R = H / G;
    for (int h = blockIdx.y * nw + warp; h < H; h += gridDim.y * nw) {
        const int g = h / R, hq = h - g * R;
        const float * o = Or + (((size_t) g * Tpad + t) * R + hq) * V;
        float ss = 0.f;
        for (int i = lane; i < V; i += 32) ss = fmaf(o[i], o[i], ss);
        ss = warp_sum(ss);
        const float r = out_scale / sqrtf(ss / (float) V + eps);
        for (int i = lane; i < V; i += 32) A[(size_t) t * H * V + (size_t) h * V + i] = o[i] * r;
    }
}

// ---- blocks whose two sub-layers read the same residual: x <- x + mixer(n1(x)) + ff(n2(x)) -----------------------------------
// End of one layer and start of the next in one pass over a row: X[t] += Ya[t] + Yb[t] (either may be absent), the new row also
// goes to Xc (row stride ldc; the input of a product that follows) when given, then H1[t] = X^ w1 and H2[t] = X^ w2 with
// X^ = X / sqrt(mean(X^2) + eps): both norms share the root mean square, the weights arrive as 1 + w. One block per row.
__global__ void __launch_bounds__(256) k_add_norm2(float * __restrict__ X, const float * __restrict__ Ya, const float * __restrict__ Yb, float * __restrict__ Xc, int ldc,
                                                   const float * __restrict__ w1, const float * __restrict__ w2, float * __restrict__ H1, float * __restrict__ H2, int n, float eps) {
    __shared__ float red[8];
    const int row = blockIdx.x, tid = threadIdx.x;
    float * x = X + (size_t) row * n;
    float ss = 0.f;
    for (int i = tid; i < n; i += 256) {
        float v = x[i];
        if (Ya) v += Ya[(size_t) row * n + i];
        if (Yb) v += Yb[(size_t) row * n + i];
        if (Ya || Yb) x[i] = v;
        if (Xc) Xc[(size_t) row * ldc + i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!w1) return;
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot += red[w];
    const float r = 1.0f / sqrtf(tot / (float) n + eps);
    for (int i = tid; i < n; i += 256) {
        const float v = x[i] * r;                 // each thread re-reads what it wrote
        H1[(size_t) row * n + i] = v * w1[i];
        if (w2) H2[(size_t) row * n + i] = v * w2[i];
    }
}

// The same for a one-token step, with the causal convolutions of both normed inputs (weights cw [2][n][taps], history
// hist [2][taps - 1][n]) in the same launch: U_i = h_i + conv_i(h_i) to U (planes of `plane` floats), the history moves on.
// One thread-block cluster of CANON1_CTAS blocks: each block owns a slice of the row, the sum of squares is reduced across the
// cluster through distributed shared memory, so that no block reads an entry of X another block rewrites.
constexpr int CANON1_CTAS = 8;
__global__ void __cluster_dims__(CANON1_CTAS, 1, 1) __launch_bounds__(256)
k_add_norm2_canon1(float * __restrict__ X, const float * __restrict__ Ya, const float * __restrict__ Yb, const float * __restrict__ w1, const float * __restrict__ w2,
                   const float * __restrict__ cw, float * __restrict__ hist, float * __restrict__ U, long long plane, int n, int taps, float eps) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float red[8];
    __shared__ float part;
    const int tid = threadIdx.x, first = (int) cluster.block_rank() * 256 + tid, step = 256 * CANON1_CTAS;
    float ss = 0.f;
    for (int i = first; i < n; i += step) {
        float v = X[i];
        if (Ya) v += Ya[i];
        if (Yb) v += Yb[i];
        if (Ya || Yb) X[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) { float p = 0.f; for (int w = 0; w < 8; w++) p += red[w]; part = p; }
    cluster.sync();
    float tot = 0.f;
    for (int r = 0; r < CANON1_CTAS; r++) tot += *cluster.map_shared_rank(&part, r);      // the same order in every block
    cluster.sync();                                    // no block leaves while its share may still be read
    const float r = 1.0f / sqrtf(tot / (float) n + eps);
    for (int i = first; i < n; i += step) {
        const float v = X[i] * r;                      // each thread re-reads what it wrote
        for (int z = 0; z < (w2 ? 2 : 1); z++) {
            const float h = v * (z ? w2[i] : w1[i]);
            const float * c = cw + ((size_t) z * n + i) * taps;
            float * hs = hist + (size_t) z * (taps - 1) * n;
            float y = fmaf(c[taps - 1], h, h);
            for (int k = 0; k + 1 < taps; k++) y = fmaf(c[k], hs[(size_t) k * n + i], y);
            U[(size_t) z * plane + i] = y;
            for (int k = 0; k + 2 < taps; k++) hs[(size_t) k * n + i] = hs[(size_t) (k + 1) * n + i];
            if (taps > 1) hs[(size_t) (taps - 2) * n + i] = h;
        }
    }
}

// embedding without a norm: X[t] = embed[token[t]]; X0 (row stride ld0), when given, keeps the same row for later layers
template <typename WT>
__global__ void k_embed_plain(const WT * __restrict__ embed, const int32_t * __restrict__ tokens, int E, int n_vocab, float * __restrict__ X, float * __restrict__ X0, int ld0) {
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : tok >= n_vocab ? n_vocab - 1 : tok;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float v = wf(embed, (size_t) tok * E + i);
        X[(size_t) t * E + i] = v;
        if (X0) X0[(size_t) t * ld0 + i] = v;
    }
}

// ---- polynomial activation with norms: y = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N divides a row by its
// root mean square (eps inside the root); coef = [a, b, c, e]. One block per row, in place, float32.
__global__ void __launch_bounds__(256) k_polynorm(float * __restrict__ Z, int n, const float * __restrict__ coef, float eps) {
    __shared__ float red[3][8];
    float * z = Z + (size_t) blockIdx.x * n;
    const int tid = threadIdx.x;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = tid; i < n; i += 256) { const float v = z[i], v2 = v * v, v3 = v2 * v; s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6); }
    s2 = warp_sum(s2); s4 = warp_sum(s4); s6 = warp_sum(s6);
    if ((tid & 31) == 0) { red[0][tid >> 5] = s2; red[1][tid >> 5] = s4; red[2][tid >> 5] = s6; }
    __syncthreads();
    float t2 = 0.f, t4 = 0.f, t6 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) { t2 += red[0][w]; t4 += red[1][w]; t6 += red[2][w]; }
    const float r1 = coef[0] / sqrtf(t2 / (float) n + eps), r2 = coef[1] / sqrtf(t4 / (float) n + eps), r3 = coef[2] / sqrtf(t6 / (float) n + eps), e = coef[3];
    for (int i = tid; i < n; i += 256) { const float v = z[i], v2 = v * v; z[i] = fmaf(v, r1, fmaf(v2, r2, fmaf(v2 * v, r3, e))); }
}

// ---- small element-wise steps ---------------------------------------------------------------------------------------------------
// output gate: A[t][h][0..V) *= sigmoid(gate[t][h]) (one number per head), or with per_entry = 1 A[t][i] *= sigmoid(gate[t][i])
// (one number per entry); gate rows of stride ldg. grid (T, slices of a row)
__global__ void k_head_gate(float * __restrict__ A, const float * __restrict__ gate, int ldg, int H, int V, int per_entry) {
    const int t = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H * V; i += blockDim.x * gridDim.y) A[(size_t) t * H * V + i] *= sigmoidf_(gate[(size_t) t * ldg + (per_entry ? i : i / V)]);
}
// soft cap on the logits: x <- cap tanh(x / cap)
__global__ void k_softcap(float * __restrict__ x, size_t n, float cap) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// ---- arg-max of one row of logits (lowest index wins ties) -----------------------------------------------------------------
__global__ void __launch_bounds__(1024) k_argmax_row(const float * __restrict__ x, int n, int32_t * __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    float best = -INFINITY; int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = x[i]; if (v > best || (v == best && i < idx)) { best = v; idx = i; } }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int) (blockDim.x >> 5); w++) if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        *out = idx == 0x7fffffff ? 0 : idx;
    }
}

// the device-resident greedy loop's last kernel: arg-max of the token's logits becomes the next step's token at the next
// position (header in device memory), and is appended to the list the host reads after the burst
__global__ void __launch_bounds__(1024) k_argmax_advance(const float * __restrict__ x, int n, StepState * st, int32_t * token_slot,
                                                         int32_t * __restrict__ out, int32_t * counter) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    float best = -INFINITY; int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = x[i]; if (v > best || (v == best && i < idx)) { best = v; idx = i; } }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int) (blockDim.x >> 5); w++) if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        if (idx == 0x7fffffff) idx = 0;
        out[*counter] = idx;
        *counter += 1;
        *token_slot = idx;
        st->pos0 += 1;
    }
}

}  // namespace stk
}  // namespace b200
