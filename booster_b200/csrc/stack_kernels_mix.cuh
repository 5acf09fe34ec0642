// stack_kernels_mix.cuh — more CUDA kernels (sm_100a) of the layer-stack models, beside stack_kernels.cuh: an element-wise
// norm without statistics (dynamic tanh), the sub-layer join with a depth-weighted average over the outputs of all earlier
// layers, retention (matrix state with a constant decay per head), sigmoid attention with a linear distance penalty over
// grouped key/value heads, and the routed mixture of gated units (router with group-limited choice, expert-sorted rows for
// the segmented products of prompt portions, indexed mat-vecs for single tokens).
// Every size and constant is a kernel argument. Everything here is float32: norms, positions and angles, scores and
// weights, the recurrent state, the router.
#pragma once
#include "stack_kernels.cuh"

namespace b200 {
namespace stk {

// ---- dynamic tanh: y = tanh(alpha x) w + b, element by element: no statistic of the row enters -----------------------------------------
struct DytW { const float * w; const float * b; float alpha; };
__device__ __forceinline__ float dytf_(float x, const DytW & n, int i) { return fmaf(tanhf(n.alpha * x), n.w[i], n.b[i]); }

// embedding under that norm: X[t] = dyt_e(embed[token[t]]) (also kept as plane 0 of the depth history when given),
// Hn[t] = dyt_1(X[t]) for the first layer
template <typename WT>
__global__ void k_embed_dyt(const WT * __restrict__ embed, const int32_t * __restrict__ tokens, int E, int n_vocab, DytW ne, DytW n1,
                            float * __restrict__ X, float * __restrict__ keep0, float * __restrict__ Hn) {
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : tok >= n_vocab ? n_vocab - 1 : tok;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float v = dytf_(wf(embed, (size_t) tok * E + i), ne, i);
        X[(size_t) t * E + i] = v;
        if (keep0) keep0[(size_t) t * E + i] = v;
        Hn[(size_t) t * E + i] = dytf_(v, n1, i);
    }
}
// the head's input: Y[r] = dyt(X[rows[r]]) on the wanted rows
__global__ void k_dyt_rows(const float * __restrict__ X, int ldx, const int32_t * __restrict__ rows, DytW n, int E, float * __restrict__ Y, int ldy) {
    const int r = blockIdx.x, src = rows ? rows[r] : r;
    for (int i = threadIdx.x; i < E; i += blockDim.x) Y[(size_t) r * ldy + i] = dytf_(X[(size_t) src * ldx + i], n, i);
}

// ---- end of a sub-layer ---------------------------------------------------------------------------------------------------------
// v = X[t] + y[t], where y is one of
//   plain     Ya[t]
//   pair      (rms(Ya[t]) wa + rms(Yb[t]) wb) / 2: two branches that read the same input, each over its root mean square across
//             the row (eps inside the root) times a plain weight
//   mixture   sum_k wt[t][k] Yk[slot(t, k)] (+ sg[t] Ysh[t]): the chosen experts' outputs, found through slot_of when the rows were
//             sorted by expert (nullptr: slot t top + k), plus the gated shared unit
// then, when the layer ends here and the design averages over depth: keep[n_keep - 1][t] = v and
// v <- sum_(j < n_keep) coef[j] keep[j][t] (planes of `plane` floats; plane 0 is the embedding output); X[t] = v; and
// Hn[t] = dyt(v) for the sub-layer that follows. grid (T, slices of JOIN_SLICE entries); a pair's two sums of squares are taken
// by every slice's block over the whole row.
constexpr int JOIN_SLICE = 256;        // one entry per thread: a one-token step still spreads over several SMs
struct JoinArgs {
    float * X; int E;
    const float * Ya; const float * Yb; const float * wa; const float * wb; float eps;      // Yb != nullptr: pair
    const float * Yk; const float * wt; const int32_t * slot_of; int top; const float * Ysh; const float * sg;   // Yk != nullptr: mixture
    float * keep; long long plane; const float * coef; int n_keep;                          // keep != nullptr: depth average
    const float * nw; const float * nb; float alpha; float * Hn;                            // nw != nullptr: the next norm
};
__global__ void __launch_bounds__(256) k_join(const JoinArgs a) {
    __shared__ float red[2][8];
    const int t = blockIdx.x, tid = threadIdx.x;
    const size_t row = (size_t) t * a.E;
    float ra = 1.f, rb = 1.f;
    if (a.Yb) {
        float sa = 0.f, sb = 0.f;
        for (int i = tid; i < a.E; i += 256) { const float u = a.Ya[row + i], v = a.Yb[row + i]; sa = fmaf(u, u, sa); sb = fmaf(v, v, sb); }
        sa = warp_sum(sa); sb = warp_sum(sb);
        if ((tid & 31) == 0) { red[0][tid >> 5] = sa; red[1][tid >> 5] = sb; }
        __syncthreads();
        float ta = 0.f, tb = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) { ta += red[0][w]; tb += red[1][w]; }
        ra = 1.0f / sqrtf(ta / (float) a.E + a.eps); rb = 1.0f / sqrtf(tb / (float) a.E + a.eps);
    }
    const int i1 = min(a.E, (int) (blockIdx.y + 1) * JOIN_SLICE);
    for (int i = blockIdx.y * JOIN_SLICE + tid; i < i1; i += 256) {
        float y;
        if (a.Yb) y = 0.5f * fmaf(a.Ya[row + i] * ra, a.wa[i], a.Yb[row + i] * rb * a.wb[i]);
        else if (a.Yk) {
            y = 0.f;
            for (int k = 0; k < a.top; k++) {
                const int s = t * a.top + k;
                y = fmaf(a.wt[s], a.Yk[(size_t) (a.slot_of ? a.slot_of[s] : s) * a.E + i], y);
            }
            if (a.Ysh) y = fmaf(a.sg[t], a.Ysh[row + i], y);
        } else y = a.Ya[row + i];
        float v = a.X[row + i] + y;
        if (a.keep) {
            a.keep[(size_t) (a.n_keep - 1) * a.plane + row + i] = v;
            float z = a.coef[a.n_keep - 1] * v;
            for (int j = a.n_keep - 2; j >= 0; j--) z = fmaf(a.coef[j], a.keep[(size_t) j * a.plane + row + i], z);
            v = z;
        }
        a.X[row + i] = v;
        if (a.nw) a.Hn[row + i] = fmaf(tanhf(a.alpha * v), a.nw[i], a.nb[i]);
    }
}

// ---- retention: S <- decay_h S + k v^T, o = S^T q per head: a plain decayed sum, nothing divides the read-out --------------------------------------
// P[t] = [ q: H x D | k: H x D | v: H x V | output-gate pre-activation: H x V ].
// Step 1, per token, in place: the first rope.dims entries of every q and k head are rotated by the token's position
// ('rotate half' pairs), then k is scaled by k_scale (D^(-1/2)). grid (T, ceil(2 H / warps per block)): a warp per head.
__global__ void k_retention_prep(float * __restrict__ P, int ldp, int q_off, int k_off, int H, int D, RopeArgs rope, float k_scale, const StepState * __restrict__ st) {
    const int t = blockIdx.x, pos = st->pos0 + t;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, half = rope.dims / 2;
    for (int v = blockIdx.y * nw + warp; v < 2 * H; v += gridDim.y * nw) {
        const bool is_k = v >= H;
        float * x = P + (size_t) t * ldp + (is_k ? k_off + (size_t) (v - H) * D : q_off + (size_t) v * D);
        const float f = is_k ? k_scale : 1.0f;
        for (int i = lane; i < D; i += 32) {
            if (i < half) { float a, b; rope_pair(rope, pos, i, x[i], x[i + half], a, b); x[i] = a * f; x[i + half] = b * f; }
            else if (i >= rope.dims && is_k) x[i] *= f;
        }
    }
}
// Step 2, the recurrence. S is [D][V] per head in float32 and stays in registers for the whole portion; four neighbouring lanes
// share one column of S, each holding a quarter of its rows, and close the read-out with two shuffles. q and k of a few tokens
// arrive in shared memory by asynchronous copies while the tokens before them are walked (two buffers); each quarter of the rows
// is padded apart so that the four lanes' reads fall into different banks. A head's columns are spread over gridDim.y blocks.
template <int DMAX>
__global__ void __launch_bounds__(512) k_retention_scan(const float * __restrict__ P, int ldp, int q_off, int k_off, int v_off, const float * __restrict__ decay,
                                                        int T, int H, int D, int V, float * __restrict__ S, float * __restrict__ O) {
    constexpr int TT = DMAX > 128 ? 4 : 8, DR = DMAX / GD_RG, ROW = GD_RG * (DR + GD_PAD);
    __shared__ __align__(16) float qs[2][TT][ROW], ks[2][TT][ROW], vs[2][TT][128];
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, rg = lane & 3, ncols = blockDim.x / GD_RG;
    const int cl = (tid >> 5) * 8 + (lane >> 2), col = blockIdx.y * ncols + cl;
    const bool live = col < V;
    const float g = decay[h];
    const auto stage = [&](int t0, int buf) {
        const int nt = min(TT, T - t0);
        for (int i = tid; i < nt * DMAX; i += blockDim.x) {
            const int tt = i / DMAX, d = i % DMAX, at = (d / DR) * (DR + GD_PAD) + d % DR;
            const bool in = d < D;
            const float * p = P + (size_t) (t0 + tt) * ldp + (size_t) h * D + (in ? d : 0);
            cp_async4(&qs[buf][tt][at], p + q_off, in);
            cp_async4(&ks[buf][tt][at], p + k_off, in);
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
        if (t0 + TT < T) stage(t0 + TT, buf ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float v = vs[buf][tt][cl];
            float op[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
            for (int i = 0; i < DR; i++) {
                s[i] = fmaf(g, s[i], ks[buf][tt][base + i] * v);
                op[i & 3] = fmaf(s[i], qs[buf][tt][base + i], op[i & 3]);
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

// Long prompt portions run the same recurrence chunk by chunk (RC tokens), so that only the short walk over chunks is serial.
// With t, j local to chunk c of n_c tokens, S_c the state before it and g the head's decay:
//   U_c = sum_j g^(n_c - 1 - j) k_j v_j^T                               k_retention_chunk_kv     (all chunks at once)
//   S_(c+1) = g^(n_c) S_c + U_c                                         k_retention_chunk_state  (in place: U_c's slot then holds S_c)
//   o_t = g^(t + 1) S_c^T q_t + sum_(j <= t) g^(t - j) (q_t . k_j) v_j  k_retention_chunk_out    (all chunks at once)
// Same float32 arithmetic as the walk, sums in another order. SB [H][chunks][D][V] is a working buffer of the pass.
constexpr int RC = 32;
// rows [0, n_rows) x columns [0, n_cols) of a row-major source into a shared tile of `rows` x `cols` (row stride dst_ld), zeros
// elsewhere, by asynchronous copies that are all issued before any is awaited (16 bytes each when `vec`: every address a multiple of 16)
__device__ __forceinline__ void stage_tile_async(float * dst, int dst_ld, const float * src, size_t src_ld, int rows, int cols, int n_rows, int n_cols, bool vec, int tid, int nthreads) {
    if (vec) {
        const int c4 = cols >> 2;
        for (int i = tid; i < rows * c4; i += nthreads) {
            const int j = i / c4, x = (i - j * c4) << 2;
            const bool in = j < n_rows && x < n_cols;
            cp_async16((uint32_t) __cvta_generic_to_shared(dst + j * dst_ld + x), in ? (const void *) (src + (size_t) j * src_ld + x) : (const void *) src, in ? 16u : 0u);
        }
    } else {
        for (int i = tid; i < rows * cols; i += nthreads) {
            const int j = i / cols, x = i - j * cols;
            const bool in = j < n_rows && x < n_cols;
            cp_async4(dst + j * dst_ld + x, in ? src + (size_t) j * src_ld + x : src, in);
        }
    }
}
__device__ __forceinline__ void async_copies_done() {
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}
// grid (H, chunks, ceil(V / 128)), 256 threads: thread (ty, tx) owns 8 x 8 of a 128 x 128 tile of U_c; keys and decay-scaled values
// of the chunk are staged in shared memory
__global__ void __launch_bounds__(256) k_retention_chunk_kv(const float * __restrict__ P, int ldp, int k_off, int v_off, const float * __restrict__ decay,
                                                            int T, int H, int D, int V, float * __restrict__ SB) {
    __shared__ __align__(16) float Ks[RC][128], Vs[RC][128];
    const int h = blockIdx.x, c = blockIdx.y, v0 = blockIdx.z * 128, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int t0 = c * RC, nt = min(RC, T - t0), nch = gridDim.y;
    __shared__ float pw[RC];
    const float g = decay[h];
    const bool vec = ((ldp | k_off | v_off | D | V) & 3) == 0;
    if (tid < RC) pw[tid] = tid < nt ? powf(g, (float) (nt - 1 - tid)) : 0.f;
    stage_tile_async(&Vs[0][0], 128, P + (size_t) t0 * ldp + v_off + (size_t) h * V + v0, (size_t) ldp, RC, 128, nt, V - v0, vec, tid, 256);
    float * U = SB + ((size_t) h * nch + c) * D * V;
    for (int d0 = 0; d0 < D; d0 += 128) {
        __syncthreads();
        stage_tile_async(&Ks[0][0], 128, P + (size_t) t0 * ldp + k_off + (size_t) h * D + d0, (size_t) ldp, RC, 128, nt, D - d0, vec, tid, 256);
        async_copies_done();
        __syncthreads();
        float acc[8][8];
#pragma unroll
        for (int a = 0; a < 8; a++)
#pragma unroll
            for (int b = 0; b < 8; b++) acc[a][b] = 0.f;
#pragma unroll 4
        for (int j = 0; j < RC; j++) {
            const float4 ka = *reinterpret_cast<const float4 *>(&Ks[j][ty * 8]), kb = *reinterpret_cast<const float4 *>(&Ks[j][ty * 8 + 4]);
            const float4 va = *reinterpret_cast<const float4 *>(&Vs[j][tx * 8]), vb = *reinterpret_cast<const float4 *>(&Vs[j][tx * 8 + 4]);
            const float f = pw[j];                      // the key's decay until the chunk's end
            const float kk[8] = { ka.x * f, ka.y * f, ka.z * f, ka.w * f, kb.x * f, kb.y * f, kb.z * f, kb.w * f }, vv[8] = { va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w };
#pragma unroll
            for (int a = 0; a < 8; a++)
#pragma unroll
                for (int b = 0; b < 8; b++) acc[a][b] = fmaf(kk[a], vv[b], acc[a][b]);
        }
#pragma unroll
        for (int a = 0; a < 8; a++) {
            const int d = d0 + ty * 8 + a;
            if (d >= D) continue;
#pragma unroll
            for (int b = 0; b < 8; b++) { const int v = v0 + tx * 8 + b; if (v < V) U[(size_t) d * V + v] = acc[a][b]; }
        }
    }
}
// grid (H, ceil(D V / 256)): a thread owns one entry of the state and walks the chunks
__global__ void k_retention_chunk_state(const float * __restrict__ decay, int T, int D, int V, int nch, float * __restrict__ S, float * __restrict__ SB) {
    const int h = blockIdx.x, e = blockIdx.y * blockDim.x + threadIdx.x, n = D * V;
    if (e >= n) return;
    const float g = decay[h], gfull = powf(g, (float) RC), glast = powf(g, (float) (T - (nch - 1) * RC));
    float s = S[(size_t) h * n + e];
    float * sb = SB + (size_t) h * nch * n + e;
    for (int c0 = 0; c0 < nch; c0 += 8) {
        float u[8];
#pragma unroll
        for (int i = 0; i < 8; i++) u[i] = c0 + i < nch ? sb[(size_t) (c0 + i) * n] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (c0 + i < nch) {
                sb[(size_t) (c0 + i) * n] = s;
                s = fmaf(c0 + i == nch - 1 ? glast : gfull, s, u[i]);
            }
        }
    }
    S[(size_t) h * n + e] = s;
}
// grid (H, chunks, ceil(V / 128)), 128 threads: warp w owns tokens 8 w .. 8 w + 7 of the chunk, a lane four value channels.
// Dynamic shared memory: q and k of the chunk [RC][D + 4] each, the masked scores [RC][RC + 4], the values [RC][128], the powers of g.
__global__ void __launch_bounds__(128) k_retention_chunk_out(const float * __restrict__ P, int ldp, int q_off, int k_off, int v_off, const float * __restrict__ decay,
                                                             int T, int H, int D, int V, const float * __restrict__ SB, float * __restrict__ O) {
    extern __shared__ __align__(16) float csm[];
    const int Dp = D + 4;
    constexpr int AP = RC + 4;                         // score rows padded to whole 16-byte chunks
    float * Qs = csm, * Ks = Qs + RC * Dp, * As = Ks + RC * Dp, * Vs = As + RC * AP, * pw = Vs + RC * 128;
    const int h = blockIdx.x, c = blockIdx.y, v0 = blockIdx.z * 128, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = c * RC, nt = min(RC, T - t0), nch = gridDim.y;
    const float g = decay[h];
    {
        const bool al = ((ldp | q_off | k_off | v_off | D | V) & 3) == 0;
        const float * row0 = P + (size_t) t0 * ldp + (size_t) h * D;
        stage_tile_async(Qs, Dp, row0 + q_off, (size_t) ldp, RC, D, nt, D, al, tid, 128);
        stage_tile_async(Ks, Dp, row0 + k_off, (size_t) ldp, RC, D, nt, D, al, tid, 128);
        stage_tile_async(Vs, 128, P + (size_t) t0 * ldp + v_off + (size_t) h * V + v0, (size_t) ldp, RC, 128, nt, V - v0, al, tid, 128);
        if (tid <= RC) pw[tid] = powf(g, (float) tid);
        async_copies_done();
    }
    __syncthreads();
    const int D4 = (D & 3) ? 0 : D;                    // 16-byte reads along d need whole chunks per row (D + 4 is then a multiple of 4 too)
    {   // scores of the chunk against itself: lane = key j, the warp's 8 tokens; 16-byte reads along d (a lane's own key row, the
        // tokens' query rows as broadcasts) when D is a multiple of 4, else entry by entry
        float sc[8] = { 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f };
        const float * kr = Ks + lane * Dp;
        for (int d = 0; d < D4; d += 4) {
            const float4 k4 = *reinterpret_cast<const float4 *>(kr + d);
#pragma unroll
            for (int a = 0; a < 8; a++) {
                const float4 q4 = *reinterpret_cast<const float4 *>(Qs + (warp * 8 + a) * Dp + d);
                sc[a] = fmaf(q4.x, k4.x, fmaf(q4.y, k4.y, fmaf(q4.z, k4.z, fmaf(q4.w, k4.w, sc[a]))));
            }
        }
        for (int d = D4; d < D; d++)
#pragma unroll
            for (int a = 0; a < 8; a++) sc[a] = fmaf(Qs[(warp * 8 + a) * Dp + d], kr[d], sc[a]);
#pragma unroll
        for (int a = 0; a < 8; a++) { const int t = warp * 8 + a; As[t * AP + lane] = lane <= t ? sc[a] * pw[t - lane] : 0.f; }
    }
    __syncthreads();
    float acc[8][4];
#pragma unroll
    for (int a = 0; a < 8; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.f;
    const float * Sc = SB + ((size_t) h * nch + c) * D * V;
    const int v = v0 + lane * 4;
    const bool vec = (V & 3) == 0 && v + 3 < V;
    const auto srow = [&](int d, float (&sv)[4]) {
        if (vec) { const float4 f = __ldg(reinterpret_cast<const float4 *>(Sc + (size_t) d * V + v)); sv[0] = f.x; sv[1] = f.y; sv[2] = f.z; sv[3] = f.w; }
        else {
#pragma unroll
            for (int b = 0; b < 4; b++) sv[b] = v + b < V ? __ldg(Sc + (size_t) d * V + v + b) : 0.f;
        }
    };
#pragma unroll 2
    for (int d = 0; d < D4; d += 4) {                   // four rows of the chunk's entry state per step, the queries as 16-byte broadcasts
        float sv[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++) srow(d + r, sv[r]);
#pragma unroll
        for (int a = 0; a < 8; a++) {
            const float4 q4 = *reinterpret_cast<const float4 *>(Qs + (warp * 8 + a) * Dp + d);
#pragma unroll
            for (int b = 0; b < 4; b++) acc[a][b] = fmaf(q4.x, sv[0][b], fmaf(q4.y, sv[1][b], fmaf(q4.z, sv[2][b], fmaf(q4.w, sv[3][b], acc[a][b]))));
        }
    }
    for (int d = D4; d < D; d++) {
        float sv[4];
        srow(d, sv);
#pragma unroll
        for (int a = 0; a < 8; a++) {
            const float qv = Qs[(warp * 8 + a) * Dp + d];
#pragma unroll
            for (int b = 0; b < 4; b++) acc[a][b] = fmaf(qv, sv[b], acc[a][b]);
        }
    }
#pragma unroll
    for (int a = 0; a < 8; a++) {
        const float f = pw[warp * 8 + a + 1];
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] *= f;
    }
    for (int j = 0; j < RC; j += 4) {
        float4 f[4];
#pragma unroll
        for (int r = 0; r < 4; r++) f[r] = *reinterpret_cast<const float4 *>(Vs + (j + r) * 128 + lane * 4);
#pragma unroll
        for (int a = 0; a < 8; a++) {
            const float4 w = *reinterpret_cast<const float4 *>(As + (warp * 8 + a) * AP + j);
            acc[a][0] = fmaf(w.x, f[0].x, fmaf(w.y, f[1].x, fmaf(w.z, f[2].x, fmaf(w.w, f[3].x, acc[a][0]))));
            acc[a][1] = fmaf(w.x, f[0].y, fmaf(w.y, f[1].y, fmaf(w.z, f[2].y, fmaf(w.w, f[3].y, acc[a][1]))));
            acc[a][2] = fmaf(w.x, f[0].z, fmaf(w.y, f[1].z, fmaf(w.z, f[2].z, fmaf(w.w, f[3].z, acc[a][2]))));
            acc[a][3] = fmaf(w.x, f[0].w, fmaf(w.y, f[1].w, fmaf(w.z, f[2].w, fmaf(w.w, f[3].w, acc[a][3]))));
        }
    }
#pragma unroll
    for (int a = 0; a < 8; a++) {
        const int tl = warp * 8 + a;
        if (tl >= nt) continue;
#pragma unroll
        for (int b = 0; b < 4; b++) if (v + b < V) O[(size_t) (t0 + tl) * H * V + (size_t) h * V + v + b] = acc[a][b];
    }
}

// The whole mixer core for a one-token step in one launch (steps 1 and 2 and the read-out's norm and gate): one block per head.
// Rotation and key scale happen on the way into shared memory, the state is updated tile by tile of up to 128 columns (the same
// four-lanes-per-column layout), the head's read-out is kept in shared memory, then A[h] = o / rms(o) * silu(gate) (eps inside the
// root, no weight). Dynamic shared memory: V floats.
template <int DMAX>
__global__ void __launch_bounds__(512) k_retention_token(const float * __restrict__ P, int q_off, int k_off, int v_off, int g_off, const float * __restrict__ decay,
                                                         RopeArgs rope, float k_scale, const StepState * __restrict__ st, int H, int D, int V, float eps,
                                                         float * __restrict__ S, float * __restrict__ A) {
    constexpr int DR = DMAX / GD_RG, ROW = GD_RG * (DR + GD_PAD);
    extern __shared__ float o_s[];                      // [V]
    __shared__ __align__(16) float qs[ROW], ks[ROW];
    __shared__ float red[16];
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, rg = lane & 3, ncols = blockDim.x / GD_RG;
    const int pos = st->pos0, half = rope.dims / 2;
    const float * q = P + q_off + (size_t) h * D, * k = P + k_off + (size_t) h * D;
    for (int i = tid; i < 2 * DMAX; i += blockDim.x) {
        const bool is_k = i >= DMAX;
        const int d = is_k ? i - DMAX : i, at = (d / DR) * (DR + GD_PAD) + d % DR;
        float v = 0.f;
        if (d < D) {
            const float * x = is_k ? k : q;
            if (d < half) { float a, b; rope_pair(rope, pos, d, x[d], x[d + half], a, b); v = a; }
            else if (d < rope.dims) { float a, b; rope_pair(rope, pos, d - half, x[d - half], x[d], a, b); v = b; }
            else v = x[d];
            if (is_k) v *= k_scale;
        }
        (is_k ? ks : qs)[at] = v;
    }
    __syncthreads();
    const float g = decay[h];
    float * Sh = S + (size_t) h * D * V;
    const int base = rg * (DR + GD_PAD), cl = warp * 8 + (lane >> 2);
    float ss = 0.f;
    for (int c0 = 0; c0 < V; c0 += ncols) {
        const int col = c0 + cl;
        const bool live = col < V;
        const float v = live ? P[v_off + (size_t) h * V + col] : 0.f;
        float op[4] = { 0.f, 0.f, 0.f, 0.f };
        constexpr int CH = DR < 16 ? DR : 16;           // rows whose loads are in flight together (the stores would order them otherwise)
#pragma unroll 1
        for (int i0 = 0; i0 < DR; i0 += CH) {
            float sv[CH];
#pragma unroll
            for (int i = 0; i < CH; i++) { const int d = rg * DR + i0 + i; sv[i] = (live && d < D) ? Sh[(size_t) d * V + col] : 0.f; }
#pragma unroll
            for (int i = 0; i < CH; i++) {
                const int d = rg * DR + i0 + i;
                sv[i] = fmaf(g, sv[i], ks[base + i0 + i] * v);
                if (live && d < D) Sh[(size_t) d * V + col] = sv[i];
                op[i & 3] = fmaf(sv[i], qs[base + i0 + i], op[i & 3]);
            }
        }
        float o = (op[0] + op[1]) + (op[2] + op[3]);
        o += __shfl_xor_sync(0xffffffffu, o, 1);
        o += __shfl_xor_sync(0xffffffffu, o, 2);
        if (rg == 0 && live) { o_s[col] = o; ss = fmaf(o, o, ss); }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (int) (blockDim.x >> 5); w++) tot += red[w];
    const float r = 1.0f / sqrtf(tot / (float) V + eps);
    for (int i = tid; i < V; i += blockDim.x) A[(size_t) h * V + i] = o_s[i] * r * siluf_(P[g_off + (size_t) h * V + i]);
}

// ---- sigmoid attention over grouped key/value heads -------------------------------------------------------------------------------
// P[t] = [ q: H x D | k: G x D | v: G x V ]. Query head h reads key/value head h / (H / G); position p sees every j <= p.
// The weight of key j for head h is sigmoid((q . k_j) scale - slope[h] (p - j) + pb[h]); a row's weights are used as they are (they need not sum to one).
// Step 1, per token: q and k are each divided by the root mean square of their WHOLE projection (all heads at once, eps inside
// the root) and multiplied by plain weights; q is also multiplied by the position's temperature
// 1 + coef ln(floor((p + 1) / every) + 1); every value head is divided by its own root mean square (no weight). Queries go to
// Q[t] (H x D), keys and values to the cache row of the position: [ k: G x D | v: G x V ]. One block per token.
__global__ void __launch_bounds__(256) k_sigattn_prep(const float * __restrict__ P, int ldp, int H, int G, int D, int V, const float * __restrict__ qw, const float * __restrict__ kw,
                                                      float eps, float t_coef, int t_every, const StepState * __restrict__ st, float * __restrict__ Q, float * __restrict__ cache) {
    __shared__ float red[2][8];
    const int t = blockIdx.x, pos = st->pos0 + t, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nq = H * D, nk = G * D;
    const float * q = P + (size_t) t * ldp, * k = q + nq, * v = k + nk;
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < nq; i += 256) sq = fmaf(q[i], q[i], sq);
    for (int i = tid; i < nk; i += 256) sk = fmaf(k[i], k[i], sk);
    sq = warp_sum(sq); sk = warp_sum(sk);
    if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) { tq += red[0][w]; tk += red[1][w]; }
    const float temp = t_every > 0 ? 1.0f + t_coef * logf((float) ((pos + 1) / t_every) + 1.0f) : 1.0f;
    const float rq = temp / sqrtf(tq / (float) nq + eps), rk = 1.0f / sqrtf(tk / (float) nk + eps);
    float * row = cache + (size_t) pos * (nk + G * V);
    for (int i = tid; i < nq; i += 256) Q[(size_t) t * nq + i] = q[i] * rq * qw[i];
    for (int i = tid; i < nk; i += 256) row[i] = k[i] * rk * kw[i];
    for (int g = warp; g < G; g += 8) {
        const float * x = v + (size_t) g * V;
        float ss = 0.f;
        for (int i = lane; i < V; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float) V + eps);
        for (int i = lane; i < V; i += 32) row[nk + (size_t) g * V + i] = x[i] * r;
    }
}
// Step 2 for steps of few tokens: a block takes TQ consecutive tokens of one head; the 8 / TQ warps of a query and the nsplit blocks
// of blockIdx.z walk its keys in alternating chunks of 32 (a lane per key for the score, a lane per 32nd value channel for the
// weighted sum). Without a soft-max the partial sums simply add: the query's warps through shared memory, the blocks through
// `part`, summed in a fixed order by the block that finishes last (an atomic counter, no waiting).
struct SigAttnArgs {
    const float * Q; int ldq;
    const float * cache; int ldc;
    const StepState * st;
    float * A;                  // [T][H x V]
    const float * slope; const float * pb;      // [H] each
    int T, H, G, D, V;
    float scale;
    int TQ, vec, nsplit;
    float * part;               // [T][H][nsplit][32 VPL]
    int * counter;              // [T][H]
};
template <int VPL>
__global__ void __launch_bounds__(256) k_sig_attn(const SigAttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int WPQ = 8 / a.TQ, qi = warp / WPQ, wq = warp % WPQ;
    const int h = blockIdx.y, g = h / (a.H / a.G), t0 = blockIdx.x * a.TQ, t = t0 + qi;
    float * qs = sm;                                        // [TQ][D]
    float * mg = sm + (size_t) a.TQ * a.D;                  // [8 warps][32 VPL]
    constexpr int MGW = 32 * VPL;
    for (int i = tid; i < a.TQ * a.D; i += 256) {
        const int q = i / a.D, e = i - q * a.D;
        qs[i] = t0 + q < a.T ? a.Q[(size_t) (t0 + q) * a.ldq + (size_t) h * a.D + e] : 0.f;
    }
    __syncthreads();
    float acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++) acc[i] = 0.f;
    if (t < a.T) {
        const int p = a.st->pos0 + t;
        const int nchunk = (p + 1 + 31) / 32;
        const float * q1 = qs + (size_t) qi * a.D;
        const float slope = a.slope[h], pb = a.pb[h];
        const size_t koff = (size_t) g * a.D, voff = (size_t) a.G * a.D + (size_t) g * a.V;
        for (int c = blockIdx.z * WPQ + wq; c < nchunk; c += WPQ * a.nsplit) {
            const int jb = c * 32, j = jb + lane, cnt = min(32, p - jb + 1);
            float w = 0.f;
            if (lane < cnt) {
                // the lane's key row and value row are asked for now, whole: the dot product and the weighted sum then find them in L2
                // instead of paying one memory round trip per batch of loads
                const char * kp = reinterpret_cast<const char *>(a.cache + (size_t) j * a.ldc + koff);
                const char * vp = reinterpret_cast<const char *>(a.cache + (size_t) j * a.ldc + voff);
                for (int b = 128; b < a.D * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" :: "l"(kp + b));
                for (int b = 0; b < a.V * 4; b += 128) asm volatile("prefetch.global.L2 [%0];" :: "l"(vp + b));
                const float * k1 = a.cache + (size_t) j * a.ldc + koff;
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
                w = sigmoidf_(fmaf(x0 + x1, a.scale, pb - slope * (float) (p - j)));
            }
            const float * vrow = a.cache + (size_t) jb * a.ldc + voff;
#pragma unroll 8
            for (int kk = 0; kk < cnt; kk++) {
                const float wk = __shfl_sync(0xffffffffu, w, kk);
#pragma unroll
                for (int i = 0; i < VPL; i++) {
                    const int vi = lane + 32 * i;
                    const float v = vi < a.V ? __ldg(vrow + (size_t) kk * a.ldc + vi) : 0.f;
                    acc[i] = fmaf(wk, v, acc[i]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < VPL; i++) mg[(size_t) warp * MGW + lane + 32 * i] = acc[i];
    __syncthreads();
    if (wq != 0 || t >= a.T) return;
#pragma unroll
    for (int i = 0; i < VPL; i++) acc[i] = 0.f;
    for (int w = 0; w < WPQ; w++)
#pragma unroll
        for (int i = 0; i < VPL; i++) acc[i] += mg[(size_t) (warp + w) * MGW + lane + 32 * i];
    if (a.nsplit > 1) {
        const size_t th = (size_t) t * a.H + h;
        float * o = a.part + (th * a.nsplit + blockIdx.z) * MGW;
#pragma unroll
        for (int i = 0; i < VPL; i++) o[lane + 32 * i] = acc[i];
        __threadfence();
        int done = 0;
        if (lane == 0) done = atomicAdd(a.counter + th, 1);
        done = __shfl_sync(0xffffffffu, done, 0);
        if (done != a.nsplit - 1) return;
        __threadfence();
        if (lane == 0) a.counter[th] = 0;
        const float * ps = a.part + th * a.nsplit * MGW;
#pragma unroll
        for (int i = 0; i < VPL; i++) acc[i] = 0.f;
        for (int z = 0; z < a.nsplit; z++)
#pragma unroll
            for (int i = 0; i < VPL; i++) acc[i] += __ldcg(ps + (size_t) z * MGW + lane + 32 * i);
    }
#pragma unroll
    for (int i = 0; i < VPL; i++) if (lane + 32 * i < a.V) a.A[(size_t) t * a.H * a.V + (size_t) h * a.V + lane + 32 * i] = acc[i];
}
// Prompt portions run the same attention as two float32 products around an element-wise pass, like the other attentions of the
// family: per tile of TQ tokens and key/value head g, S = Q_g K_g^T (rows: the tile's tokens x the R = H / G query heads of the
// group), k_sig_weight_rows turns scores into weights, then O = W V_g.
// queries [T][H][D] -> Qr[g][Tpad][R][D] (rows past T are zero)
__global__ void k_group_q_layout(const float * __restrict__ Q, int ldq, int T, int Tpad, int H, int G, int D, float * __restrict__ Qr) {
    const int t = blockIdx.x, R = H / G, nq = H * D;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        const int h = i / D, d = i - h * D, g = h / R, hq = h - g * R;
        Qr[(((size_t) g * Tpad + t) * R + hq) * D + d] = t < T ? Q[(size_t) t * ldq + i] : 0.f;
    }
}
// S holds [g][n_rows = ng TQ R][nk] for a group of ng tiles starting at tile0; column n is key n (no window: the products
// start at position 0). One warp per row.
__global__ void k_sig_weight_rows(float * __restrict__ S, int n_rows, int G, int R, int TQ, int nk, const StepState * __restrict__ st, float scale,
                                  const float * __restrict__ slope, const float * __restrict__ pb, int tile0, int T) {
    const int lane = threadIdx.x & 31, id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (id >= n_rows * G) return;
    const int g = id / n_rows, r = id - g * n_rows, h = g * R + r % R;
    const int t = tile0 * TQ + r / R, p = st->pos0 + t;
    float * s = S + (size_t) id * nk;
    const float sl = slope[h], b = pb[h];
    for (int n = lane; n < nk; n += 32) s[n] = (t < T && n <= p) ? sigmoidf_(fmaf(s[n], scale, b - sl * (float) (p - n))) : 0.f;
}
// Or[g][Tpad][R][V] -> A[t][h][V], times sigmoid(gate[t][h]) when a gate is given (one number per head, rows of stride ldg)
__global__ void k_group_o_layout(const float * __restrict__ Or, int Tpad, int H, int G, int V, float * __restrict__ A, const float * __restrict__ gate = nullptr, int ldg = 0) {
    const int t = blockIdx.x, R = H / G;
    for (int i = threadIdx.x; i < H * V; i += blockDim.x) {
        const int h = i / V, d = i - h * V, g = h / R, hq = h - g * R;
        const float o = Or[(((size_t) g * Tpad + t) * R + hq) * V + d];
        A[(size_t) t * H * V + i] = gate ? o * sigmoidf_(gate[(size_t) t * ldg + h]) : o;
    }
}

// ---- routed mixture of gated units --------------------------------------------------------------------------------------------------
// Router, per token, in float32: z = W_r h, s = softmax(z) over all n experts (score_fn 0) or s_i = sigmoid(z_i), each expert by
// itself (score_fn 1). The expert list is cut into n_groups consecutive blocks
// of equal size; a block ranks by the best s inside it and the choice is confined to the `keep` best-ranked blocks: of their experts
// the `top` with the largest s are taken (lowest index first among equals), each weighing in with s * scale as it is.
// sel[t][top], wt[t][top]; sg[t] = sigmoid(w_sg . h) is the shared unit's gate (w_sg == nullptr: no shared unit).
// grid (T, ceil(rows / (8 / wpr))) with rows = n (+ 1 for the shared gate): wpr warps per row of the router (1, or 8 for steps of few
// tokens, whose rows would otherwise be walked by one warp each), several 16-byte loads in flight;
// the logits go to z[t][n + 1], and the block of a token that finishes last (an atomic counter, no waiting) makes the choice with
// one warp. Dynamic shared memory: 2 n + n_groups floats.
struct RouteArgs {
    const float * Hn; int ld, E;
    const float * Wr; const float * w_sg;
    int n, top, n_groups, keep;
    float scale;
    int32_t * sel; float * wt; float * sg;
    float * z; int * counter;
    int score_fn;       // 0: soft-max over the experts; 1: sigmoid of each logit
    int wpr;            // warps per router row: 1 (a block takes 8 rows) or 8 (a block takes one row, each warp an eighth of it: steps of few tokens)
};
__global__ void __launch_bounds__(256) k_moe_route(const RouteArgs a) {
    extern __shared__ float rsm[];
    __shared__ int last_s;
    float * s = rsm, * elig = rsm + a.n, * gbest = rsm + 2 * a.n;
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float * h = a.Hn + (size_t) t * a.ld;
    __shared__ float psum[8];
    const int wpr = a.wpr, kw = warp % wpr;
    const int rows = a.n + (a.w_sg ? 1 : 0), e = blockIdx.y * (8 / wpr) + warp / wpr;
    float * z = a.z + (size_t) t * (a.n + 1);
    if (e < rows) {
        const float * w = e < a.n ? a.Wr + (size_t) e * a.E : a.w_sg;
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
        if ((a.E & 3) == 0 && (a.ld & 3) == 0 && (((uintptr_t) w | (uintptr_t) h) & 15) == 0) {
#pragma unroll 4
            for (int i = (kw * 32 + lane) * 4; i < a.E; i += 128 * wpr) {
                const float4 x = *reinterpret_cast<const float4 *>(h + i), y = __ldg(reinterpret_cast<const float4 *>(w + i));
                acc0 = fmaf(x.x, y.x, acc0); acc1 = fmaf(x.y, y.y, acc1); acc2 = fmaf(x.z, y.z, acc2); acc3 = fmaf(x.w, y.w, acc3);
            }
        } else {
            for (int i = kw * 32 + lane; i < a.E; i += 32 * wpr) acc0 = fmaf(w[i], h[i], acc0);
        }
        float acc = warp_sum((acc0 + acc1) + (acc2 + acc3));
        if (wpr > 1) {                                      // the row's warps: partial sums through shared memory, in a fixed order
            if (lane == 0) psum[warp] = acc;
            __syncthreads();
            acc = 0.f;
            for (int k = 0; k < wpr; k++) acc += psum[k];
        }
        if (lane == 0 && kw == 0) { if (e < a.n) z[e] = acc; else a.sg[t] = sigmoidf_(acc); }
    }
    if (gridDim.y > 1) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) last_s = atomicAdd(a.counter + t, 1) == (int) gridDim.y - 1;
        __syncthreads();
        if (!last_s) return;
        __threadfence();
        if (threadIdx.x == 0) a.counter[t] = 0;
    } else __syncthreads();
    if (warp != 0) return;
    const int per = a.n / a.n_groups;
    if (a.score_fn == 1) {
        for (int i = lane; i < a.n; i += 32) { s[i] = sigmoidf_(__ldcg(z + i)); elig[i] = -1.f; }
    } else {
        float mx = -INFINITY;
        for (int i = lane; i < a.n; i += 32) { const float v = __ldcg(z + i); s[i] = v; mx = fmaxf(mx, v); }
        mx = warp_max(mx);
        float sum = 0.f;
        for (int i = lane; i < a.n; i += 32) { const float v = expf(s[i] - mx); s[i] = v; sum += v; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int i = lane; i < a.n; i += 32) { s[i] *= inv; elig[i] = -1.f; }
    }
    __syncwarp();
    for (int g = lane; g < a.n_groups; g += 32) {
        float b = -1.f;
        for (int i = 0; i < per; i++) b = fmaxf(b, s[g * per + i]);
        gbest[g] = b;
    }
    __syncwarp();
    // the best groups, one at a time; then the best eligible experts, one at a time (value, then lowest index)
    for (int r = 0; r < a.keep; r++) {
        float bv = -2.f; int bi = 0x7fffffff;
        for (int g = lane; g < a.n_groups; g += 32) if (gbest[g] > bv) { bv = gbest[g]; bi = g; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi != 0x7fffffff) {
            for (int i = lane; i < per; i += 32) elig[bi * per + i] = s[bi * per + i];
            if (lane == 0) gbest[bi] = -3.f;
        }
        __syncwarp();
    }
    for (int r = 0; r < a.top; r++) {
        float bv = -0.5f; int bi = 0x7fffffff;
        for (int i = lane; i < a.n; i += 32) if (elig[i] > bv) { bv = elig[i]; bi = i; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) { bi = 0; bv = 0.f; }        // fewer eligible experts than `top` (refused at load): a slot of weight 0
        if (lane == 0) { a.sel[t * a.top + r] = bi; a.wt[t * a.top + r] = bv * a.scale; elig[bi] = -1.f; }
        __syncwarp();
    }
}
// Prompt portions: the n_slots = T top (token, choice) slots sorted by expert, stably, so that every expert's rows are contiguous:
// seg[e] .. seg[e + 1] - 1 are expert e's rows, slot_of[slot] the row a slot got, src_row[row] the token it reads. One block of
// 1024 threads: `tpe` threads per expert (a power of two) each count one contiguous part of the slots, a block-wide prefix sum
// over (expert, part) gives every thread its first row, a second walk places the slots. Dynamic shared memory: the slots'
// experts when they fit (in_smem), then n tpe counters.
__global__ void __launch_bounds__(1024) k_moe_sort(const int32_t * __restrict__ sel, int n_slots, int top, int n, int tpe, int in_smem,
                                                   int32_t * __restrict__ seg, int32_t * __restrict__ slot_of, int32_t * __restrict__ src_row) {
    extern __shared__ int ssm[];
    __shared__ int wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int * cnt = ssm + (in_smem ? n_slots : 0);
    const int32_t * es = sel;
    if (in_smem) {
        for (int i = tid; i < n_slots; i += 1024) ssm[i] = sel[i];
        es = ssm;
    }
    __syncthreads();
    const int chunk = (n_slots + tpe - 1) / tpe, part = tid & (tpe - 1), epb = 1024 / tpe;
    const int s0 = min(part * chunk, n_slots), s1 = min(s0 + chunk, n_slots);
    for (int e = tid / tpe; e < n; e += epb) {
        int c = 0;
        for (int i = s0; i < s1; i++) c += es[i] == e;
        cnt[e * tpe + part] = c;
    }
    __syncthreads();
    // exclusive prefix sum over the M = n tpe counters, in place: a thread owns `own` consecutive entries
    const int M = n * tpe, own = (M + 1023) / 1024, b0 = min(tid * own, M), b1 = min(b0 + own, M);
    int mine = 0;
    for (int i = b0; i < b1; i++) mine += cnt[i];
    int inc = mine;
    for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += v; }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int v = wsum[lane];
        for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
        wsum[lane] = v;
    }
    __syncthreads();
    int at = inc - mine + (warp ? wsum[warp - 1] : 0);
    for (int i = b0; i < b1; i++) { const int c = cnt[i]; cnt[i] = at; at += c; }
    __syncthreads();
    for (int e = tid; e < n; e += 1024) seg[e] = cnt[e * tpe];
    if (tid == 0) seg[n] = n_slots;
    for (int e = tid / tpe; e < n; e += epb) {
        int r = cnt[e * tpe + part];
        for (int i = s0; i < s1; i++) if (es[i] == e) { slot_of[i] = r; src_row[r] = i / top; r++; }
    }
}
// Y[r] = X[src_row[r]]
__global__ void k_gather_rows(const float * __restrict__ X, int ldx, const int32_t * __restrict__ src_row, int E, float * __restrict__ Y) {
    const int r = blockIdx.x;
    const float * x = X + (size_t) src_row[r] * ldx;
    if ((E & 3) == 0 && (ldx & 3) == 0) {
        for (int i = threadIdx.x * 4; i < E; i += blockDim.x * 4) *reinterpret_cast<float4 *>(Y + (size_t) r * E + i) = *reinterpret_cast<const float4 *>(x + i);
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) Y[(size_t) r * E + i] = x[i];
    }
}

// Y[slot_of[s]] = wt[s] X[s / top]: every (token, choice) slot's input row, weighted by the choice's score, at the row the sort
// gave the slot (an expert that runs on the weighted input)
__global__ void k_spread_rows(const float * __restrict__ X, int ldx, const int32_t * __restrict__ slot_of, const float * __restrict__ wt, int top, int E, float * __restrict__ Y) {
    const int s = blockIdx.x;
    const float * x = X + (size_t) (s / top) * ldx;
    float * y = Y + (size_t) slot_of[s] * E;
    const float w = wt[s];
    for (int i = threadIdx.x; i < E; i += blockDim.x) y[i] = w * x[i];
}

}  // namespace stk
}  // namespace b200
