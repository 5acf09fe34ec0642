// stack_kernels_hyper.cuh — CUDA kernels (sm_100a) of further mechanisms of the layer-stack models, on top of stack_kernels.cuh:
// a residual kept as several streams that every sub-layer reads through a weighted sum and writes through a small mixing
// matrix (hyper-connections), RMS norms whose weight is one number, and a soft-max attention over grouped key/value heads
// whose options are all arguments: per-head RMS norm of queries and keys, rotation of neighbouring or half-split pairs on part
// of a head, a cap on the scores, a logarithmic distance penalty, a sink in the denominator, values mixed with an earlier
// layer's, a per-head output gate, and three masks (causal | chunks counted from position 0 | a sliding window with the means
// of whole blocks of cached keys and values standing in for what lies before the window).
// Everything here is float32: streams, norms, positions and angles, scores and weights.
#pragma once
#include "stack_kernels.cuh"

namespace b200 {
namespace stk {

constexpr int HC_MAX = 8;              // most residual streams
struct HcW {                           // one sub-layer's connection weights
    float in[HC_MAX];                  // u = sum_s in[s] x_s
    float mix[HC_MAX * HC_MAX];        // x_t <- sum_s mix[s * S + t] x_s + out[t] y
    float out[HC_MAX];
};

// sum over a block of up to 1024 threads (a multiple of 32); every thread gets the total. red: 32 floats of shared memory
__device__ __forceinline__ float block_sum(float v, float * red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    const int nw = blockDim.x >> 5;
    for (int w = 0; w < nw; w++) t += red[w];
    __syncthreads();
    return t;
}
// threads per row of the stream kernels: steps of few tokens spread a row over a whole block (`per_thread` entries per thread), so
// that the loads of a row are in flight together; prompt portions have rows enough to fill the SMs with smaller blocks
inline int hc_threads(int T, int E, int per_thread = 2, int most = 1024) {
    const int n = (E / per_thread + 31) / 32 * 32;
    return T > 16 ? 256 : n < 128 ? 128 : n > most ? most : n;
}

// embedding into all S streams, fused with the first sub-layer's read-in and norm:
// XS[s][t] = embed[token[t]]; Hn[t] = u / sqrt(mean(u^2) + eps) * g with u = sum_s in[s] XS[s][t]
template <typename WT>
__global__ void __launch_bounds__(1024) k_hc_embed(const WT * __restrict__ embed, const int32_t * __restrict__ tokens, int E, int n_vocab, int S,
                                                  float * __restrict__ XS, long long plane, HcW w, float g, float eps, float * __restrict__ Hn) {
    __shared__ float red[32];
    const int t = blockIdx.x, nt = blockDim.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : tok >= n_vocab ? n_vocab - 1 : tok;      // ids are validated on the host; never read outside the table
    const size_t row = (size_t) t * E;
    float a = 0.f;
    for (int s = 0; s < S; s++) a += w.in[s];
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += nt) {
        const float x = wf(embed, (size_t) tok * E + i);
        for (int s = 0; s < S; s++) XS[(size_t) s * plane + row + i] = x;
        const float u = a * x;
        Hn[row + i] = u;
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, red);
    const float r = g / sqrtf(ss / (float) E + eps);
    for (int i = threadIdx.x; i < E; i += nt) Hn[row + i] *= r;
}

// end of a sub-layer: all streams at once from the old ones, x_t <- sum_s mix[s][t] x_s + out[t] y, where y is the sub-layer's
// output: Ya[t] (may be nullptr) plus, for a routed mixture, the chosen experts' outputs Yk[slot(t, k)], k < top, as they are
// (slot_of == nullptr: slot t top + k). Then, for the sub-layer that follows, u = sum_t nin[t] x_t and Hn[t] = u / rms(u) * g
// (Hn == nullptr: nothing follows), and Xsum[t] = sum_t x_t when the residual itself is wanted. One block per token
// (hc_threads threads).
struct HcJoinArgs {
    float * XS; long long plane; int S, E;
    const float * Ya;
    const float * Yk; const int32_t * slot_of; int top;
    HcW w;
    float nin[HC_MAX]; float g; float eps; float * Hn;
    float * Xsum;
};
// VEC = 4: rows are walked in 16-byte chunks (E a multiple of 4, 16-byte aligned rows); VEC = 1: any E.
template <int VEC> __device__ __forceinline__ void ld_chunk(const float * p, float (&v)[VEC]) {
    if constexpr (VEC == 4) { const float4 f = *reinterpret_cast<const float4 *>(p); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
    else v[0] = p[0];
}
template <int VEC> __device__ __forceinline__ void st_chunk(float * p, const float (&v)[VEC]) {
    if constexpr (VEC == 4) *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else p[0] = v[0];
}
constexpr int HC_OWN = 2;              // read-in chunks a thread keeps in registers until the row's sum of squares is known
template <int VEC>
__global__ void __launch_bounds__(VEC == 4 ? 512 : 1024) k_hc_join(const HcJoinArgs a) {
    __shared__ float red[32];
    const int t = blockIdx.x, S = a.S, nt = blockDim.x, nchunk = a.E / VEC;
    const size_t row = (size_t) t * a.E;
    const bool own = nchunk <= HC_OWN * nt;
    float ss = 0.f, keep[HC_OWN][VEC];
    int n_own = 0;
    for (int c = threadIdx.x; c < nchunk; c += nt) {
        const int i = c * VEC;
        float y[VEC], old[HC_MAX][VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) y[e] = 0.f;
        if (a.Ya) ld_chunk<VEC>(a.Ya + row + i, y);
#pragma unroll
        for (int s = 0; s < HC_MAX; s++) if (s < S) ld_chunk<VEC>(a.XS + (size_t) s * a.plane + row + i, old[s]);
        if (a.Yk) for (int k = 0; k < a.top; k++) {
            const int sl = t * a.top + k;
            float v[VEC];
            ld_chunk<VEC>(a.Yk + (size_t) (a.slot_of ? a.slot_of[sl] : sl) * a.E + i, v);
#pragma unroll
            for (int e = 0; e < VEC; e++) y[e] += v[e];
        }
        float u[VEC], sum[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) u[e] = sum[e] = 0.f;
#pragma unroll
        for (int q = 0; q < HC_MAX; q++) {
            if (q < S) {
                float v[VEC];
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    v[e] = a.w.out[q] * y[e];
#pragma unroll
                    for (int s = 0; s < HC_MAX; s++) if (s < S) v[e] = fmaf(a.w.mix[s * S + q], old[s][e], v[e]);
                    u[e] = fmaf(a.nin[q], v[e], u[e]);
                    sum[e] += v[e];
                }
                st_chunk<VEC>(a.XS + (size_t) q * a.plane + row + i, v);
            }
        }
        if (a.Xsum) st_chunk<VEC>(a.Xsum + row + i, sum);
        if (a.Hn) {
#pragma unroll
            for (int e = 0; e < VEC; e++) ss = fmaf(u[e], u[e], ss);
            if (own) {
#pragma unroll
                for (int k = 0; k < HC_OWN; k++) if (k == n_own) {
#pragma unroll
                    for (int e = 0; e < VEC; e++) keep[k][e] = u[e];
                }
                n_own++;
            } else st_chunk<VEC>(a.Hn + row + i, u);
        }
    }
    if (!a.Hn) return;
    ss = block_sum(ss, red);
    const float r = a.g / sqrtf(ss / (float) a.E + a.eps);
    if (own) {
#pragma unroll
        for (int k = 0; k < HC_OWN; k++) if (k < n_own) {
            float v[VEC];
#pragma unroll
            for (int e = 0; e < VEC; e++) v[e] = keep[k][e] * r;
            st_chunk<VEC>(a.Hn + row + ((size_t) threadIdx.x + (size_t) k * nt) * VEC, v);
        }
    } else for (int i = threadIdx.x; i < a.E; i += nt) a.Hn[row + i] *= r;
}

// ---- soft-max attention over grouped key/value heads ------------------------------------------------------------------------------
// P[t] = [ q: H x D | k: G x D | v: G x V | ... ]. Query head h reads key/value head h / (H / G).
// Step 1, per token: every q and k head over its own root mean square (eps inside the root) times a weight [D] shared by the heads
// (qw / kw; nullptr: no norm), then the rotation of the first rope.dims entries by the token's position. Queries go to Q[t]
// (H x D), keys and values to the cache row of the position: [ k: G x D | v: G x V ]. Values: vmode 1 also leaves them in
// vfirst[t] (the first mixing layer of the model); vmode 2 stores (1 - lambda) v + lambda vfirst[t] (a later mixing layer; the
// mixed values are what the cache keeps). grid (T, blocks): a warp per head, the heads and the value entries dealt over the blocks of a token.
enum { GQA_V_PLAIN = 0, GQA_V_FIRST = 1, GQA_V_MIX = 2 };
struct GqaPrepArgs {
    const float * P; int ldp;
    int H, G, D, V;
    const float * qw; const float * kw; float eps;
    RopeArgs rope;
    const StepState * st;
    float * Q; float * cache; int ldc;
    float * vfirst; int vmode; float lambda;
};
__global__ void __launch_bounds__(256) k_gqa_prep(const GqaPrepArgs a) {
    const int t = blockIdx.x, pos = a.st->pos0 + t, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nq = a.H * a.D, nk = a.G * a.D, nv = a.G * a.V;
    const float * q = a.P + (size_t) t * a.ldp, * k = q + nq, * v = k + nk;
    float * row = a.cache + (size_t) pos * a.ldc;
    const int half = a.rope.dims / 2;
    const int nblk = gridDim.y, bk = blockIdx.y;
    for (int vec = bk * 8 + warp; vec < a.H + a.G; vec += 8 * nblk) {
        const bool is_q = vec < a.H;
        const float * src = is_q ? q + (size_t) vec * a.D : k + (size_t) (vec - a.H) * a.D;
        const float * w = is_q ? a.qw : a.kw;
        float * dst = is_q ? a.Q + (size_t) t * nq + (size_t) vec * a.D : row + (size_t) (vec - a.H) * a.D;
        float r = 1.0f;
        if (w) {
            float ss = 0.f;
            for (int i = lane; i < a.D; i += 32) ss = fmaf(src[i], src[i], ss);
            ss = warp_sum(ss);
            r = 1.0f / sqrtf(ss / (float) a.D + a.eps);
        }
        for (int i = lane; i < half; i += 32) {
            const int lo = rope_lo(a.rope, i), hi = rope_hi(a.rope, i);
            const float x = w ? src[lo] * r * w[lo] : src[lo], y = w ? src[hi] * r * w[hi] : src[hi];
            float ox, oy;
            rope_pair(a.rope, pos, i, x, y, ox, oy);
            dst[lo] = ox; dst[hi] = oy;
        }
        for (int i = a.rope.dims + lane; i < a.D; i += 32) dst[i] = w ? src[i] * r * w[i] : src[i];
    }
    for (int i = bk * 256 + tid; i < nv; i += 256 * nblk) {
        float x = v[i];
        if (a.vmode == GQA_V_MIX) x = fmaf(a.lambda, a.vfirst[(size_t) t * nv + i], (1.0f - a.lambda) * x);
        else if (a.vmode == GQA_V_FIRST) a.vfirst[(size_t) t * nv + i] = x;
        row[nk + i] = x;
    }
}

// means of whole blocks of P cached rows: pool[b] = (1 / P) sum_(j < P) cache[b P + j], for every block whose last position
// b P + P - 1 lies in this step (its rows are all in the cache then). grid (n_tokens / P + 1, slices of the row).
__global__ void k_pool_rows(const float * __restrict__ cache, int ldc, float * __restrict__ pool, int P, const StepState * __restrict__ st) {
    const int b = st->pos0 / P + blockIdx.x;
    if ((long long) (b + 1) * P > (long long) st->pos0 + st->n_tokens) return;
    const float * src = cache + (size_t) b * P * ldc;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < ldc; i += blockDim.x * gridDim.y) {
        float s = 0.f;
        for (int j = 0; j < P; j++) s += src[(size_t) j * ldc + i];
        pool[(size_t) b * ldc + i] = s / (float) P;
    }
}

// what position p sees: `nb` leading block means (rows 0 .. nb - 1 of the pool) and the tokens jlo .. p
enum { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_CHUNK = 2 };
struct GqaMask { int kind, size, P; };
__host__ __device__ __forceinline__ int gqa_first_token(const GqaMask & m, int p) {
    return m.kind == MASK_WINDOW ? (p - m.size + 1 > 0 ? p - m.size + 1 : 0) : m.kind == MASK_CHUNK ? (p / m.size) * m.size : 0;
}
__host__ __device__ __forceinline__ int gqa_blocks_seen(const GqaMask & m, int p) {      // blocks b with b P + P - 1 <= p - size
    return m.kind == MASK_WINDOW && m.P > 0 && p - m.size >= 0 ? (p - m.size + 1) / m.P : 0;
}
// score of one key from the dot product: scale, cap, distance penalty (tokens only)
struct GqaScore { float scale, cap; };
__device__ __forceinline__ float gqa_score(const GqaScore & sc, float dot, float r1, float r2, int dist) {
    float s = dot * sc.scale;
    if (sc.cap > 0.f) s = sc.cap * tanhf(s / sc.cap);
    if (dist > 0) s -= r1 * log1pf(r2 * (float) dist);      // ln(1 + 0) = 0: the token itself and block means carry no penalty
    return s;
}

// Step 2 for steps of few tokens: a block takes TQ consecutive tokens of one head; the 8 / TQ warps of a query and the nsplit
// blocks of blockIdx.z walk its keys (block means first, then tokens) in alternating chunks of 32: a lane per key for the score,
// a lane per 32nd value channel for the weighted sum, a running maximum and denominator per warp. The query's warps merge in
// shared memory, the blocks through `part`, merged by the block that finishes last (an atomic counter, no waiting). The sink
// joins the denominator once at the very end; the output is multiplied by sigmoid(gate[t][h]) when a gate is given.
struct GqaAttnArgs {
    const float * Q; int ldq;
    const float * cache; const float * pool; int ldc;
    const StepState * st;
    float * A;                                  // [T][H x V]
    const float * r1; const float * r2; const float * sink;      // [H] each; r1 == nullptr: no penalty; sink == nullptr: none
    const float * gate; int ldg;                // gate pre-activations, one per head, rows of stride ldg (nullptr: none)
    int T, H, G, D, V;
    GqaScore sc;
    GqaMask mask;
    int TQ, vec, nsplit;
    float * part;                               // [T][H][nsplit][2 + 32 VPL]
    int * counter;                              // [T][H]
};
template <int VPL>
__global__ void __launch_bounds__(256) k_gqa_attn(const GqaAttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int WPQ = 8 / a.TQ, qi = warp / WPQ, wq = warp % WPQ;
    const int h = blockIdx.y, g = h / (a.H / a.G), t0 = blockIdx.x * a.TQ, t = t0 + qi;
    constexpr int MGW = 2 + 32 * VPL;
    float * qs = sm;                                        // [TQ][D]
    float * mg = sm + (size_t) a.TQ * a.D;                  // [8 warps][MGW]
    // asked for together with the queries (one round trip to memory, not one each): the step's position and the head's constants
    const int pos0 = a.st->pos0;
    const float r1 = a.r1 ? a.r1[h] : 0.f, r2 = a.r1 ? a.r2[h] : 0.f, snk = a.sink ? a.sink[h] : 0.f;
    const float gate_in = a.gate && t < a.T ? a.gate[(size_t) t * a.ldg + h] : 0.f;
    for (int i = tid; i < a.TQ * a.D; i += 256) {
        const int q = i / a.D, e = i - q * a.D;
        qs[i] = t0 + q < a.T ? a.Q[(size_t) (t0 + q) * a.ldq + (size_t) h * a.D + e] : 0.f;
    }
    __syncthreads();
    float acc[VPL], m = -INFINITY, l = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i++) acc[i] = 0.f;
    if (t < a.T) {
        const int p = pos0 + t;
        const int jlo = gqa_first_token(a.mask, p), nb = gqa_blocks_seen(a.mask, p), ntot = nb + p - jlo + 1;
        const float * q1 = qs + (size_t) qi * a.D;
        const size_t koff = (size_t) g * a.D, voff = (size_t) a.G * a.D + (size_t) g * a.V;
        const float * tokens = a.cache + ((long long) jlo - nb) * a.ldc;      // entry n >= nb is token jlo + n - nb
        for (int c = blockIdx.z * WPQ + wq; c * 32 < ntot; c += WPQ * a.nsplit) {
            const int nbase = c * 32, n = nbase + lane, cnt = min(32, ntot - nbase);
            float s = -INFINITY;
            if (lane < cnt) {
                const float * k1 = (n < nb ? a.pool + (size_t) n * a.ldc : tokens + (long long) n * a.ldc) + koff;
                // the lane's key row and value row are asked for now, whole: the dot product and the weighted sum then find them in L2
                const char * kp = reinterpret_cast<const char *>(k1), * vp = reinterpret_cast<const char *>(k1 - koff + voff);
                for (int b = 128; b < a.D * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" :: "l"(kp + b));
                for (int b = 0; b < a.V * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" :: "l"(vp + b));
                float x0 = 0.f, x1 = 0.f;
                if (a.vec) {
#pragma unroll 8
                    for (int e = 0; e < a.D; e += 4) {
                        const float4 ka = __ldg(reinterpret_cast<const float4 *>(k1 + e));
                        const float4 qa = *reinterpret_cast<const float4 *>(q1 + e);
                        x0 = fmaf(qa.x, ka.x, x0); x1 = fmaf(qa.y, ka.y, x1); x0 = fmaf(qa.z, ka.z, x0); x1 = fmaf(qa.w, ka.w, x1);
                    }
                } else {
                    for (int e = 0; e < a.D; e++) x0 = fmaf(q1[e], k1[e], x0);
                }
                s = gqa_score(a.sc, x0 + x1, r1, r2, n < nb ? 0 : p - (jlo + n - nb));
            }
            const float mn = fmaxf(m, warp_max(s));
            const float corr = m == -INFINITY ? 0.f : expf(m - mn);
            const float w = lane < cnt ? expf(s - mn) : 0.f;
            l = fmaf(l, corr, warp_sum(w));
#pragma unroll
            for (int i = 0; i < VPL; i++) acc[i] *= corr;
            m = mn;
#pragma unroll 8
            for (int kk = 0; kk < cnt; kk++) {
                const float wk = __shfl_sync(0xffffffffu, w, kk);
                const int nn = nbase + kk;
                const float * vrow = (nn < nb ? a.pool + (size_t) nn * a.ldc : tokens + (long long) nn * a.ldc) + voff;
#pragma unroll
                for (int i = 0; i < VPL; i++) {
                    const int vi = lane + 32 * i;
                    const float v = vi < a.V ? __ldg(vrow + vi) : 0.f;
                    acc[i] = fmaf(wk, v, acc[i]);
                }
            }
        }
    }
    if (lane == 0) { mg[(size_t) warp * MGW] = m; mg[(size_t) warp * MGW + 1] = l; }
#pragma unroll
    for (int i = 0; i < VPL; i++) mg[(size_t) warp * MGW + 2 + lane + 32 * i] = acc[i];
    __syncthreads();
    if (wq != 0 || t >= a.T) return;
    // the query's warps: one maximum, rescaled sums
    m = -INFINITY;
    for (int w = 0; w < WPQ; w++) m = fmaxf(m, mg[(size_t) (warp + w) * MGW]);
    l = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; i++) acc[i] = 0.f;
    for (int w = 0; w < WPQ; w++) {
        const float * o = mg + (size_t) (warp + w) * MGW;
        const float f = o[0] == -INFINITY ? 0.f : expf(o[0] - m);
        l = fmaf(o[1], f, l);
#pragma unroll
        for (int i = 0; i < VPL; i++) acc[i] = fmaf(o[2 + lane + 32 * i], f, acc[i]);
    }
    if (a.nsplit > 1) {
        const size_t th = (size_t) t * a.H + h;
        float * o = a.part + (th * a.nsplit + blockIdx.z) * MGW;
        if (lane == 0) { o[0] = m; o[1] = l; }
#pragma unroll
        for (int i = 0; i < VPL; i++) o[2 + lane + 32 * i] = acc[i];
        __threadfence();
        int done = 0;
        if (lane == 0) done = atomicAdd(a.counter + th, 1);
        done = __shfl_sync(0xffffffffu, done, 0);
        if (done != a.nsplit - 1) return;
        __threadfence();
        if (lane == 0) a.counter[th] = 0;
        const float * ps = a.part + th * a.nsplit * MGW;
        m = -INFINITY;
        for (int z = 0; z < a.nsplit; z++) m = fmaxf(m, __ldcg(ps + (size_t) z * MGW));
        l = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; i++) acc[i] = 0.f;
        for (int z = 0; z < a.nsplit; z++) {
            const float mz = __ldcg(ps + (size_t) z * MGW);
            const float f = mz == -INFINITY ? 0.f : expf(mz - m);
            l = fmaf(__ldcg(ps + (size_t) z * MGW + 1), f, l);
#pragma unroll
            for (int i = 0; i < VPL; i++) acc[i] = fmaf(__ldcg(ps + (size_t) z * MGW + 2 + lane + 32 * i), f, acc[i]);
        }
    }
    float f = 1.0f;
    if (a.sink) {                                           // exp(sink) joins the denominator: no key, no value
        const float mm = fmaxf(m, snk);
        f = expf(m - mm);
        l = fmaf(l, f, expf(snk - mm));
    }
    f /= l;
    if (a.gate) f *= sigmoidf_(gate_in);
#pragma unroll
    for (int i = 0; i < VPL; i++) if (lane + 32 * i < a.V) a.A[(size_t) t * a.H * a.V + (size_t) h * a.V + lane + 32 * i] = acc[i] * f;
}

// Prompt portions run the same attention as float32 products around a row soft-max, like the other attentions of the family:
// per tile of TQ tokens and key/value head g, S = Q_g K_g^T (rows: the tile's tokens x the R = H / G query heads of the group),
// this kernel turns scores into weights, then O = W V_g. A row of S holds [ npc columns of block means | nk columns of tokens ]:
// token column n is position jlo + n with jlo = pos0 + tile TQ - span + 1 (span: the most tokens any row looks back, no more
// than the sequence so far; the cache has a zero margin in front) or 0 when the products start at position 0 (span == 0).
// S holds [g][n_rows = ng TQ R][npc + nk] for a group of ng tiles starting at tile0. One warp per row.
__global__ void k_gqa_softmax_rows(float * __restrict__ S, int n_rows, int G, int R, int TQ, int npc, int nk, int span, GqaMask mask, GqaScore sc,
                                   const float * __restrict__ r1v, const float * __restrict__ r2v, const float * __restrict__ sink,
                                   const StepState * __restrict__ st, int tile0, int T) {
    const int lane = threadIdx.x & 31, id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (id >= n_rows * G) return;
    const int g = id / n_rows, r = id - g * n_rows, h = g * R + r % R;
    const int t = tile0 * TQ + r / R, p = st->pos0 + t;
    float * s = S + (size_t) id * (npc + nk);
    if (t >= T) { for (int n = lane; n < npc + nk; n += 32) s[n] = 0.f; return; }
    const int jlo = span > 0 ? st->pos0 + (t / TQ) * TQ - span + 1 : 0;
    const int n_lo = npc + gqa_first_token(mask, p) - jlo, n_hi = npc + p - jlo, nb = gqa_blocks_seen(mask, p);     // token columns n_lo .. n_hi, block columns 0 .. nb - 1
    const float r1 = r1v ? r1v[h] : 0.f, r2 = r1v ? r2v[h] : 0.f;
    float mx = -INFINITY;
    for (int n = lane; n < nb; n += 32) { const float v = gqa_score(sc, s[n], 0.f, 0.f, 0); s[n] = v; mx = fmaxf(mx, v); }
    for (int n = n_lo + lane; n <= n_hi; n += 32) { const float v = gqa_score(sc, s[n], r1, r2, n_hi - n); s[n] = v; mx = fmaxf(mx, v); }
    mx = warp_max(mx);
    const float snk = sink ? sink[h] : -INFINITY;
    const float m = fmaxf(mx, snk);
    float sum = 0.f;
    for (int n = lane; n < nb; n += 32) sum += expf(s[n] - m);
    for (int n = n_lo + lane; n <= n_hi; n += 32) sum += expf(s[n] - m);
    sum = warp_sum(sum);
    const float inv = 1.0f / (sum + (sink ? expf(snk - m) : 0.f));
    __syncwarp();                                           // the last pass walks the row from column 0: other lanes' columns
    for (int n = lane; n < npc + nk; n += 32) s[n] = (n < nb || (n >= n_lo && n <= n_hi)) ? expf(s[n] - m) * inv : 0.f;
}

}  // namespace stk
}  // namespace b200
