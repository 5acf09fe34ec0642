// stack.cu — the layer-stack model family on the B200 engine: configuration (config.json), weights (model.safetensors),
// per-sequence state (attention cache + recurrent state), the step function for prompt portions and single tokens, and
// the registry of designs and mixers. Kernels: stack_kernels.cuh, stack_kernels_mix.cuh, stack_kernels_hyper.cuh. C-ABI dispatch: engine.cu.
//
// A design is a name in config.json ("architecture") mapped to a builder that turns the configuration into a list of
// LayerSpec; a mixer is a name ("type") mapped to a loader of its tensors and a forward routine. Four designs are registered:
//   Matulorn   sequential sub-layers with grouped norms before and after each; mixers minGRU | latent attention (rotated
//              part, window, sink) | gated delta rule; clamped gated feed-forward
//   Dopilorn   both sub-layers read the same residual (x += mixer(n1 x) + ff(n2 x)) behind a causal convolution of their
//              inputs; mixers latent attention (query latent, head gates) | generalized delta rule | differential
//              sliding-window attention; polynomial feed-forward; a span of layers run several times with the same weights
//              (each pass with a state of its own); soft-capped logits
//   Tosevik    pre-norm sub-layers with element-wise norms (dynamic tanh); after every layer the stream becomes a weighted sum of
//              the embedding output and all layers' results so far; mixers retention | parallel (sigmoid attention with a distance
//              penalty beside a retention, each normed, averaged); routed mixture of gated units with group-limited choice and a
//              gated shared unit
//   Rumurax    the residual is several streams; every sub-layer reads their weighted sum through an RMS norm whose weight is one
//              number and writes all streams at once through a mixing matrix (hyper-connections). Mixers: soft-max attention
//              over grouped heads with normed queries and keys, under a chunk mask (score cap, logarithmic distance penalty,
//              sink, per-head gate) or under a sliding window that also sees means of whole blocks of older cached keys and
//              values (rotation of neighbouring pairs); both may mix their values with the first such layer's | latent
//              attention (causal, gated entry by entry). Routed mixture: sigmoid scores, experts run on the weighted input,
//              an ungated shared unit
// A model is executed as a list of layer RUNS: (layer, state slot), one per layer unless the design repeats some.
#include "stack.hpp"
#include "safetensors.hpp"
#include "stack_kernels.cuh"
#include "stack_kernels_mix.cuh"
#include "stack_kernels_hyper.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <vector>

namespace b200 {
using namespace stk;

#define SCU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) \
    throw std::runtime_error(std::string(#call) + ": " + cudaGetErrorString(e_)); } while (0)

namespace {

enum MixerKind { MIX_MINGRU = 0, MIX_LATENT, MIX_DELTA, MIX_GDELTA, MIX_DIFFATTN, MIX_RETENTION, MIX_SIGATTN, MIX_PAIR, MIX_GQATTN };
enum BlockKind { BLOCK_SEQUENTIAL = 0, BLOCK_PARALLEL, BLOCK_PRENORM, BLOCK_HYPER };
enum FfKind { FF_GLU = 0, FF_POLY, FF_MOE };
constexpr int CHUNK_MAX = 512;          // tokens per pass of a prompt portion (longer steps run as several passes)
constexpr float GLU_ALPHA = 1.702f;     // the feed-forward's sigmoid slope: fixed by the design

struct DMat {                            // a weight matrix [N][K] (or a batch of them) in the model's storage type
    void * w = nullptr;
    float * bias = nullptr;
    int N = 0, K = 0;
    int64_t bytes = 0;
};

struct LayerSpec {
    int kind = 0;
    bool has_mlp = false;
    float * norm1 = nullptr, * norm1b = nullptr, * norm2 = nullptr, * norm2b = nullptr;
    // minGRU
    int width = 0;
    DMat zxg, o;                         // z | candidate | gate stacked row-wise; o shared by all mixers
    // latent attention
    int H = 0, D = 0, R = 0, V = 0, rank = 0, window = 0;
    float scale = 1.f;
    float * cnorm = nullptr, * sink = nullptr, * rope_freq = nullptr;
    int rope_dims = 0;
    float rope_mag = 1.f;
    DMat qdkv, ukT, uv;                  // q | down-projection stacked; per head: W_uk transposed [rank][D], W_uv [V][rank]
    int q_rank = 0;                      // > 0: queries pass a latent of their own; qdkv is then [ query latent | down-projection | head gates ]
    DMat uq;                             // query latent -> H x D
    float * qnorm = nullptr;
    bool head_gate = false;
    int gate_rows = 0;                   // rows of the gate projection: H (one number per head) or H x V (one per entry)
    bool rope_adjacent = false;          // rotation pairs are neighbours (2i, 2i + 1) instead of (i, i + dims / 2)
    // gated delta rule
    int KH = 0, taps = 0;
    DMat proj;                           // q | k | v | beta | decay | gate stacked
    float * wconv = nullptr, * A_log = nullptr, * dt_bias = nullptr, * dnorm = nullptr;
    // generalized delta rule: proj = r | k | v | gate | removal | decay latent; w2 maps the decay latent to H x D (bias: w0)
    int lora = 0;
    DMat w2;
    // differential attention: proj = q | k | v with biases; G = KH; lambda is one number per layer
    float lambda = 0.f, diff = 0.f;
    // feed-forward
    int ff = 0, ff_kind = FF_GLU;
    float limit = 0.f;
    DMat gateup, down;                   // FF_POLY: gateup is the plain up-projection; FF_MOE: the shared unit (ff = 0: none)
    float * act = nullptr;               // FF_POLY: the four coefficients
    // FF_MOE: routed mixture of gated units. e_gateup [n_exp][2 e_ff][E] (gate / up interleaved), e_down [n_exp][E][e_ff]
    int n_exp = 0, top = 0, n_groups = 1, keep_groups = 1, e_ff = 0;
    float r_scale = 1.f;
    int route_fn = 0;                    // 0: soft-max over the experts; 1: sigmoid of each logit
    bool scale_input = false;            // the choice's weight multiplies the expert's input instead of its output
    float * router = nullptr, * w_sg = nullptr;      // float32: the router is computed in 32-bit
    DMat e_gateup, e_down;
    // element-wise norms (dynamic tanh): weight in norm1 / norm2, bias and slope here
    float * n1_b = nullptr, * n2_b = nullptr;
    float n1_alpha = 1.f, n2_alpha = 1.f;
    // depth average after the layer: coefficients over the embedding output and every layer's result so far
    float * dwa = nullptr;
    int n_dwa = 0;
    // retention: constant decay per head; rotation of q and k (rope_freq / rope_dims above)
    float * decay = nullptr;
    float k_scale = 1.f;
    // sigmoid attention: weights of the whole-projection norms, per-head score offset and distance slope, query temperature
    float * qw = nullptr, * kw = nullptr, * pb = nullptr, * slope = nullptr;
    float t_coef = 0.f;
    int t_every = 0;
    // soft-max attention over grouped heads (MIX_GQATTN): proj = q | k | v | head gates; window = the mask's size; qw / kw are the
    // per-head norm weights [D]
    int mask_kind = 0, pool = 0;         // MASK_*; pool > 0: means of whole blocks of `pool` cached rows stand in for what lies before the window
    float cap = 0.f;                     // > 0: score <- cap tanh(score / cap)
    float * r1 = nullptr, * r2 = nullptr;
    int vmode = 0;                       // GQA_V_*: values left for later layers / mixed with the first mixing layer's
    float vlambda = 0.f;
    // hyper-connections (BLOCK_HYPER): the weights of both sub-layers, and norm weights that are one number
    HcW hc[2];
    float g1 = 1.f, g2 = 1.f;
    // a pair of mixers side by side (MIX_PAIR): each over its root mean square times a weight, then their mean
    std::vector<LayerSpec> parts;
    float * pair_w[2] = { nullptr, nullptr };
    // parallel blocks: weights of the causal convolution in front of each sub-layer, [2][E][taps]
    float * canon = nullptr;
    // state a sequence keeps for one run of this layer
    size_t n_rec = 0;                    // recurrent slab (floats): minGRU state | delta S + conv history | ... ; then the input convolutions' history
    size_t cache_row = 0;                // attention: floats per cached position (0: no cache)
    int64_t bytes = 0;                   // weights one token reads in this layer
};

struct RunSpec {                         // one execution of a layer within a step
    int layer = 0;
    int pass = -1;                       // >= 0: this run opens pass `pass` of the repeated span (x <- W_in [x; x0] + step[pass] first)
    size_t off_rec = 0;
    int cache_index = -1;
};

}  // namespace

struct StackModel {
    int device = 0, dtype = STACK_BF16;
    std::string design;
    int vocab = 0, E = 0, groups = 1;
    float eps = 1e-6f;
    int block = BLOCK_SEQUENTIAL;
    int canon_taps = 0;                   // parallel blocks: taps of the input convolutions (0: none)
    float softcap = 0.f;                  // > 0: logits <- cap tanh(logits / cap)
    bool dyt = false;                     // the model's norm is the element-wise dynamic tanh (weight, bias, slope)
    float * embed_w = nullptr, * embed_b = nullptr, * final_b = nullptr;
    float embed_alpha = 1.f, final_alpha = 1.f;
    bool depth_avg = false;               // every layer hands on a weighted sum of all results so far
    bool has_pair = false;
    int streams = 1;                      // BLOCK_HYPER: copies of the residual
    float final_g = 1.f;                  // BLOCK_HYPER: the model's norm weight (one number)
    bool rope_adjacent = false;           // the design rotates neighbouring pairs
    int vfirst_width = 0, vfirst_heads = 0;   // key/value heads x vdim, and key/value heads, of the first value-mixing layer (0: none so far)
    int max_slots = 0, max_eff = 0, max_exp = 0;      // routed mixtures: choices per token, expert width, experts
    size_t max_ret_state = 0;             // retention: the largest heads x dim x vdim
    int max_ret_dim = 0;
    DMat loop_in;                         // repeated span: [E][2 E]
    float * loop_step = nullptr;          // [times][E]
    std::vector<LayerSpec> layers;
    std::vector<RunSpec> runs;
    void * embed = nullptr;
    float * final_norm = nullptr;
    DMat head;
    int64_t weight_bytes = 0;
    std::vector<void *> allocs;
    // buffer widths
    int maxP = 0, maxA = 0, maxQK = 0, maxOL = 0, maxCV = 0, maxBG = 0;
    size_t rec_floats = 0;
    int n_caches = 0;
};

struct StepDev {                          // device image of a step's header
    StepState st;
    int32_t tokens[CHUNK_MAX];
    int32_t rows[CHUNK_MAX];
};

struct StackCtx {
    StackModel * m = nullptr;
    int n_ctx = 0, n_past = 0, cap = 0;
    cudaStream_t st = nullptr;
    float * XS = nullptr, * VF = nullptr; // hyper-connections: the streams [S][cap][E]; value mixing: the first mixing layer's values of this pass [cap][G V]
    std::vector<float *> pools;           // per attention cache: means of whole blocks of cached rows (nullptr: the layer keeps none)
    float * Y2 = nullptr, * U = nullptr, * XC = nullptr;     // parallel blocks: the feed-forward's output, the convolved inputs [2][cap][E], [x; x0] rows
    const float * in = nullptr;           // what the mixer being enqueued reads ([T][E]) ...
    float * out = nullptr;                // ... and writes
    float * X = nullptr, * Hn = nullptr, * Y = nullptr, * P = nullptr, * A = nullptr, * QK = nullptr, * OL = nullptr, * CV = nullptr, * BG = nullptr, * O = nullptr;
    float * rec = nullptr;                // recurrent slab
    std::vector<float *> caches;          // per run of an attention layer: [n_ctx][cache_row]
    StepDev * d_step = nullptr, * h_step = nullptr;
    float * d_logits = nullptr, * h_logits = nullptr;
    int64_t logit_rows_cap = 0;
    float * h_last = nullptr;             // last computed row (inside h_logits)
    int64_t d_last_row = -1;              // its row in d_logits
    int32_t * d_arg = nullptr, * h_arg = nullptr;
    cudaGraphExec_t g_token = nullptr;    // one token: header in -> layers -> head -> logits out
    cudaGraphExec_t g_greedy = nullptr;   // one token of the device-resident greedy loop: layers -> head -> arg-max -> next header
    int64_t n_greedy_launches = 0;
    int32_t * d_out_tokens = nullptr, * d_counter = nullptr;
    bool graph_failed = false;
    int64_t n_token_launches = 0;         // kernels per replay of g_token
    size_t attn_smem = 0;                 // the most dynamic shared memory any attention launch of this context asks for
    float * att_scores = nullptr;         // prompt attention: scores / weights of a group of tiles
    size_t att_scores_floats = 0;
    std::vector<float *> cache_allocs;    // the caches with their zero margins (caches[] point behind the front margin)
    float * att_part = nullptr, * att_ml = nullptr;   // key-slice partials of the latent attention (decode)
    float * ret_sb = nullptr;             // retention, long portions: per-chunk states [heads][chunks][dim][vdim]
    float * keep = nullptr;               // depth average: [layers + 1][cap][E] results of this pass's tokens
    float * Xp = nullptr, * Ap = nullptr, * Yk = nullptr, * r_wt = nullptr, * r_sg = nullptr;      // routed mixture: rows by slot, weights, shared gate
    int32_t * r_sel = nullptr, * r_slot = nullptr, * r_src = nullptr, * r_seg = nullptr;
    float * r_z = nullptr;                // router logits [cap][experts + 1]
    int * r_counter = nullptr;            // per token: router blocks done
    float * da_part = nullptr;            // key-slice partials of the differential / sigmoid attention (few-token steps)
    int * da_counter = nullptr;           // per (token, head): slices done
    int sm_count = 148;
    __nv_bfloat16 * xb = nullptr;         // activations of a prompt pass rounded to bfloat16 (operand of the tcgen05 product)
    size_t xb_elems = 0;
    int * d_err = nullptr, * h_err = nullptr;   // raised by a kernel whose bounded wait ran out
    bool taps = false;
    std::vector<float> tap_data;
    int tap_T = 0;
    int64_t launches = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f;
};

namespace {

// ---- uploads --------------------------------------------------------------------------------------------------
void * dev_alloc(StackModel & m, size_t bytes) {
    void * p = nullptr;
    SCU(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
    m.allocs.push_back(p);
    return p;
}
float * up_f32(StackModel & m, const std::vector<float> & v) {
    float * d = (float *) dev_alloc(m, v.size() * 4);
    SCU(cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
    return d;
}
uint16_t bf16_bits(float f) {             // round to nearest even (weights stored as bfloat16 convert exactly)
    uint32_t u; std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t) ((u >> 16) | 0x40);
    return (uint16_t) ((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
DMat up_mat(StackModel & m, const std::vector<float> & w, int N, int K, const std::vector<float> * bias, int batch = 1) {
    DMat d;
    d.N = N; d.K = K;
    const size_t n = (size_t) batch * N * K;
    if (w.size() != n) throw std::runtime_error("internal: matrix size mismatch");
    if (m.dtype == STACK_F32) {
        d.w = dev_alloc(m, n * 4);
        SCU(cudaMemcpy(d.w, w.data(), n * 4, cudaMemcpyHostToDevice));
        d.bytes = (int64_t) n * 4;
    } else {
        std::vector<uint16_t> h(n);
        for (size_t i = 0; i < n; i++) h[i] = bf16_bits(w[i]);
        d.w = dev_alloc(m, n * 2);
        SCU(cudaMemcpy(d.w, h.data(), n * 2, cudaMemcpyHostToDevice));
        d.bytes = (int64_t) n * 2;
    }
    if (bias) { d.bias = up_f32(m, *bias); d.bytes += (int64_t) bias->size() * 4; }
    m.weight_bytes += d.bytes;
    return d;
}
void append(std::vector<float> & a, const std::vector<float> & b) { a.insert(a.end(), b.begin(), b.end()); }

int need_int(const Json & j, const char * k, int lo = 1) {
    const int64_t v = j.integer(k);
    if (v < lo || v > (1 << 30)) throw std::runtime_error(std::string("config: '") + k + "' is out of range");
    return (int) v;
}

// ---- mixers: tensors '<layer>.mix.*' ----------------------------------------------------------------------------------------
void load_mingru(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const int E = m.E, w = L.width = need_int(mx, "width");
    std::vector<float> W = sf.read_f32(p + "z", {w, E}), b = sf.read_f32(p + "z.b", {w});
    append(W, sf.read_f32(p + "x", {w, E})); append(b, sf.read_f32(p + "x.b", {w}));
    append(W, sf.read_f32(p + "g", {w, E})); b.resize((size_t) 3 * w, 0.f);
    L.zxg = up_mat(m, W, 3 * w, E, &b);
    L.o = up_mat(m, sf.read_f32(p + "o", {E, w}), E, w, nullptr);
    L.n_rec = (size_t) w;
    m.maxP = std::max(m.maxP, 3 * w); m.maxA = std::max(m.maxA, w);
}

void load_latent(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const int E = m.E;
    const int H = L.H = need_int(mx, "heads"), D = L.D = need_int(mx, "dim"), R = L.R = (int) mx.integer("rot_dim", 0);
    const int V = L.V = need_int(mx, "vdim"), rank = L.rank = need_int(mx, "kv_rank");
    if (R < 0) throw std::runtime_error("config: rot_dim must not be negative");
    L.scale = (float) mx.number("scale");
    L.window = mx.has("mask") ? (int) mx.at("mask").integer("size", 0) : 0;       // 0: every earlier position
    if (L.window < 0) throw std::runtime_error("config: mask.size must not be negative");
    const int qr = L.q_rank = (int) mx.integer("q_rank", 0);
    if (qr < 0) throw std::runtime_error("config: q_rank must not be negative");
    if (const st_tensor * gt = sf.find(p + "g")) {
        // one gate per head ([H][E]) or one per entry of the concatenated heads ([H V][E])
        if (gt->shape.size() != 2 || (gt->shape[0] != H && gt->shape[0] != (int64_t) H * V)) throw std::runtime_error("tensor '" + p + "g' must have heads or heads x vdim rows");
        L.head_gate = true;
        L.gate_rows = (int) gt->shape[0];
    }
    L.rope_adjacent = m.rope_adjacent;
    if (qr > 0) {
        // queries through a latent: [ W_dq | W_dkv | W_g ] in one product, then norm and W_uq
        if (R) throw std::runtime_error("latent attention: a query latent with a rotated part is not implemented");
        std::vector<float> W = sf.read_f32(p + "dq", {qr, E});
        append(W, sf.read_f32(p + "dkv", {rank, E}));
        if (L.head_gate) append(W, sf.read_f32(p + "g", {L.gate_rows, E}));
        L.qdkv = up_mat(m, W, qr + rank + L.gate_rows, E, nullptr);
        L.qnorm = up_f32(m, sf.read_f32(p + "dq.norm", {qr}));
        L.uq = up_mat(m, sf.read_f32(p + "uq", {H * D, qr}), H * D, qr, nullptr);
    } else {
        std::vector<float> W = sf.read_f32(p + "q", {H * (D + R), E});
        append(W, sf.read_f32(p + "dkv", {rank + R, E}));
        if (L.head_gate) append(W, sf.read_f32(p + "g", {L.gate_rows, E}));
        L.qdkv = up_mat(m, W, H * (D + R) + rank + R + L.gate_rows, E, nullptr);
    }
    L.cnorm = up_f32(m, sf.read_f32(p + "dkv.norm", {rank}));
    // W_uk [H*D][rank] -> per head transposed [rank][D]: the unrotated score q_h . (W_uk,h c) = (W_uk,h^T q_h) . c
    const std::vector<float> uk = sf.read_f32(p + "uk", {H * D, rank});
    std::vector<float> ukT((size_t) H * rank * D);
    for (int h = 0; h < H; h++) for (int d = 0; d < D; d++) for (int r = 0; r < rank; r++)
        ukT[((size_t) h * rank + r) * D + d] = uk[((size_t) h * D + d) * rank + r];
    L.ukT = up_mat(m, ukT, rank, D, nullptr, H);
    L.uv = up_mat(m, sf.read_f32(p + "uv", {H * V, rank}), V, rank, nullptr, H);
    L.sink = sf.find(p + "sink") ? up_f32(m, sf.read_f32(p + "sink", {H})) : nullptr;
    L.o = up_mat(m, sf.read_f32(p + "o", {E, H * V}), E, H * V, nullptr);
    // rotary frequencies: f_i = base^(-2i/dims), blended by YaRN when rot.scaling is given
    L.rope_dims = 0; L.rope_mag = 1.f;
    std::vector<float> freq(1, 0.f);
    if (R > 0 && mx.has("rot")) {
        const Json & rot = mx.at("rot");
        const int dims = L.rope_dims = (int) rot.integer("dims", R);
        if (dims < 0 || dims > R || dims % 2) throw std::runtime_error("config: rot.dims must be even and at most rot_dim");
        const double base = rot.number("base");
        freq.assign((size_t) std::max(dims / 2, 1), 0.f);
        double factor = 1.0, lo = 0, hi = 0;
        const bool yarn = rot.has("scaling");
        if (yarn) {
            const Json & sc = rot.at("scaling");
            factor = sc.number("factor");
            const double orig = sc.number("original"), fast = sc.number("fast"), slow = sc.number("slow");
            const auto dim_of = [&](double t) { return dims * std::log(orig / (2 * M_PI * t)) / (2 * std::log(base)); };
            lo = std::max(std::floor(dim_of(fast)), 0.0);
            hi = std::min(std::ceil(dim_of(slow)), (double) dims - 1);
            L.rope_mag = (float) (0.1 * std::log(factor) + 1.0);
        }
        for (int i = 0; i < dims / 2; i++) {
            double f = std::pow(base, -2.0 * i / dims);
            if (yarn) {
                const double ramp = std::min(std::max((i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
                f = f / factor * ramp + f * (1.0 - ramp);
            }
            freq[(size_t) i] = (float) f;
        }
    }
    L.rope_freq = up_f32(m, freq);
    L.cache_row = (size_t) rank + R;
    m.maxP = std::max(m.maxP, L.qdkv.N); m.maxA = std::max({ m.maxA, H * V, qr > 0 ? H * D : 0 });
    m.maxQK = std::max(m.maxQK, H * (rank + R)); m.maxOL = std::max(m.maxOL, H * rank);
}

void load_delta(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const int E = m.E;
    const int H = L.H = need_int(mx, "heads"), KH = L.KH = (int) mx.integer("kv_heads", H), D = L.D = need_int(mx, "dim"), V = L.V = need_int(mx, "vdim");
    const int taps = L.taps = (int) mx.integer("conv", 1);
    if (KH < 1 || H % KH) throw std::runtime_error("config: delta heads must be a multiple of kv_heads");
    if (taps < 1 || taps > 64) throw std::runtime_error("config: delta conv taps out of range");
    if (D > 256) throw std::runtime_error("delta rule: dim above 256 is not supported by the recurrence kernel");
    std::vector<float> W = sf.read_f32(p + "q", {KH * D, E}), wc = sf.read_f32(p + "q.conv", {KH * D, taps});
    append(W, sf.read_f32(p + "k", {KH * D, E})); append(wc, sf.read_f32(p + "k.conv", {KH * D, taps}));
    append(W, sf.read_f32(p + "v", {H * V, E}));  append(wc, sf.read_f32(p + "v.conv", {H * V, taps}));
    append(W, sf.read_f32(p + "b", {H, E}));
    append(W, sf.read_f32(p + "a", {H, E}));
    append(W, sf.read_f32(p + "g", {H * V, E}));
    const int C = 2 * KH * D + H * V, NP = C + 2 * H + H * V;
    L.proj = up_mat(m, W, NP, E, nullptr);
    L.wconv = up_f32(m, wc);
    L.A_log = up_f32(m, sf.read_f32(p + "A_log", {H}));
    L.dt_bias = up_f32(m, sf.read_f32(p + "dt_bias", {H}));
    L.dnorm = up_f32(m, sf.read_f32(p + "norm", {V}));
    L.o = up_mat(m, sf.read_f32(p + "o", {E, H * V}), E, H * V, nullptr);
    L.n_rec = (size_t) H * D * V + (size_t) (taps - 1) * C;
    m.maxP = std::max(m.maxP, NP); m.maxA = std::max(m.maxA, H * V);
    m.maxCV = std::max(m.maxCV, C); m.maxBG = std::max(m.maxBG, 2 * H);
}

// generalized delta rule: '<layer>.mix.{r,k,v,g,a,a.b,w1,w2,w0,norm,o}'
void load_gdelta(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const int E = m.E;
    const int H = L.H = need_int(mx, "heads"), D = L.D = need_int(mx, "dim"), V = L.V = (int) mx.integer("vdim", D);
    if (V < 1) throw std::runtime_error("config: vdim out of range");
    if (D > 256) throw std::runtime_error("generalized delta rule: dim above 256 is not supported by the recurrence kernel");
    const st_tensor * w1 = sf.find(p + "w1");
    if (!w1 || w1->shape.size() != 2) throw std::runtime_error("tensor '" + p + "w1' is missing or not a matrix");
    const int lr = L.lora = (int) w1->shape[0];
    std::vector<float> W = sf.read_f32(p + "r", {H * D, E}), b((size_t) 2 * H * D + 2 * H * V, 0.f);
    append(W, sf.read_f32(p + "k", {H * D, E}));
    append(W, sf.read_f32(p + "v", {H * V, E}));
    append(W, sf.read_f32(p + "g", {H * V, E}));
    append(W, sf.read_f32(p + "a", {H * D, E})); append(b, sf.read_f32(p + "a.b", {H * D}));
    append(W, sf.read_f32(p + "w1", {lr, E}));   b.resize(b.size() + (size_t) lr, 0.f);
    const int NP = 3 * H * D + 2 * H * V + lr;
    L.proj = up_mat(m, W, NP, E, &b);
    const std::vector<float> w0 = sf.read_f32(p + "w0", {H * D});
    L.w2 = up_mat(m, sf.read_f32(p + "w2", {H * D, lr}), H * D, lr, &w0);
    L.dnorm = up_f32(m, sf.read_f32(p + "norm", {H * V}));
    L.o = up_mat(m, sf.read_f32(p + "o", {E, H * V}), E, H * V, nullptr);
    L.n_rec = (size_t) H * D * V;
    m.maxP = std::max(m.maxP, NP); m.maxA = std::max(m.maxA, H * V);
    if (lr > 8192) throw std::runtime_error("generalized delta rule: a decay latent above 8192 is not supported");
    m.maxCV = std::max(m.maxCV, 3 * H * D);
}

// differential sliding-window attention: '<layer>.mix.{q,k,v}' with '.b' and '.conv', 'lq1','lk1','lq2','lk2', 'o'
void load_diffattn(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const int E = m.E;
    const int H = L.H = need_int(mx, "heads"), G = L.KH = (int) mx.integer("kv_heads", H), D = L.D = need_int(mx, "dim"), V = L.V = need_int(mx, "vdim");
    if (G < 1 || H % G) throw std::runtime_error("config: attention heads must be a multiple of kv_heads");
    if (V > 256) throw std::runtime_error("differential attention: vdim above 256 is not supported by the attention kernel");
    if (D > 256) throw std::runtime_error("differential attention: dim above 256 is not supported by the attention kernel");
    const int taps = L.taps = (int) mx.integer("conv", 0);              // 0: no convolution after the projections
    if (taps < 0 || taps > 64) throw std::runtime_error("config: attention conv taps out of range");
    L.scale = (float) mx.number("scale");
    L.diff = (float) mx.number("diff");
    L.window = mx.has("mask") ? (int) mx.at("mask").integer("size", 0) : 0;
    if (L.window < 0) throw std::runtime_error("config: mask.size must not be negative");
    const int nq = H * 2 * D, nk = G * 2 * D, nv = G * V, C = nq + nk + nv;
    std::vector<float> W = sf.read_f32(p + "q", {nq, E}), b = sf.read_f32(p + "q.b", {nq}), wc;
    append(W, sf.read_f32(p + "k", {nk, E})); append(b, sf.read_f32(p + "k.b", {nk}));
    append(W, sf.read_f32(p + "v", {nv, E})); append(b, sf.read_f32(p + "v.b", {nv}));
    L.proj = up_mat(m, W, C, E, &b);
    if (taps > 0) {
        wc = sf.read_f32(p + "q.conv", {nq, taps});
        append(wc, sf.read_f32(p + "k.conv", {nk, taps}));
        append(wc, sf.read_f32(p + "v.conv", {nv, taps}));
    } else {
        wc.assign((size_t) C, 1.f);                                       // no convolution: one unit tap (the pass that moves keys and values into the cache)
        L.taps = 1;
    }
    L.wconv = up_f32(m, wc);
    const std::vector<float> lq1 = sf.read_f32(p + "lq1", {D}), lk1 = sf.read_f32(p + "lk1", {D}), lq2 = sf.read_f32(p + "lq2", {D}), lk2 = sf.read_f32(p + "lk2", {D});
    float d1 = 0.f, d2 = 0.f;                                             // one number per layer, float32 like everything around the scores
    for (int i = 0; i < D; i++) { d1 = std::fmaf(lq1[(size_t) i], lk1[(size_t) i], d1); d2 = std::fmaf(lq2[(size_t) i], lk2[(size_t) i], d2); }
    L.lambda = std::exp(d1) - std::exp(d2) + L.diff;
    L.o = up_mat(m, sf.read_f32(p + "o", {E, H * V}), E, H * V, nullptr);
    L.n_rec = (size_t) (L.taps - 1) * C;
    L.cache_row = (size_t) nk + nv;
    m.maxP = std::max(m.maxP, C); m.maxA = std::max(m.maxA, H * V);
    m.maxCV = std::max(m.maxCV, nq);
    m.maxQK = std::max(m.maxQK, nq); m.maxOL = std::max(m.maxOL, H * V);      // prompt portions: regrouped queries, per-group outputs
}

// plain rotary frequencies f_i = base^(-2i/dims) of a mixer's "rot" object (absent: no rotation)
void load_rot(StackModel & m, LayerSpec & L, const Json & mx, int D) {
    L.rope_dims = 0; L.rope_mag = 1.f;
    std::vector<float> freq(1, 0.f);
    if (mx.has("rot")) {
        const Json & rot = mx.at("rot");
        const int dims = L.rope_dims = (int) rot.integer("dims", D);
        if (dims < 0 || dims > D || dims % 2) throw std::runtime_error("config: rot.dims must be even and at most dim");
        const double base = rot.number("base");
        freq.assign((size_t) std::max(dims / 2, 1), 0.f);
        for (int i = 0; i < dims / 2; i++) freq[(size_t) i] = (float) std::pow(base, -2.0 * i / dims);
    }
    L.rope_freq = up_f32(m, freq);
}

// retention: '<prefix>{q,k,v,g,o}'; decay per head from the configuration
void load_retention(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const int E = m.E;
    const int H = L.H = need_int(mx, "heads"), D = L.D = need_int(mx, "dim"), V = L.V = need_int(mx, "vdim");
    if (D > 256) throw std::runtime_error("retention: dim above 256 is not supported by the recurrence kernel");
    const Json & dj = mx.at("decay");
    if (dj.kind != Json::Arr || (int) dj.arr.size() != H) throw std::runtime_error("config: 'decay' must list one number per head");
    std::vector<float> dec((size_t) H);
    for (int h = 0; h < H; h++) { if (dj.arr[(size_t) h].kind != Json::Num) throw std::runtime_error("config: 'decay' must hold numbers"); dec[(size_t) h] = (float) dj.arr[(size_t) h].num; }
    L.decay = up_f32(m, dec);
    load_rot(m, L, mx, D);
    L.k_scale = (float) (1.0 / std::sqrt((double) D));
    std::vector<float> W = sf.read_f32(p + "q", {H * D, E});
    append(W, sf.read_f32(p + "k", {H * D, E}));
    append(W, sf.read_f32(p + "v", {H * V, E}));
    append(W, sf.read_f32(p + "g", {H * V, E}));
    L.proj = up_mat(m, W, 2 * H * D + 2 * H * V, E, nullptr);
    L.o = up_mat(m, sf.read_f32(p + "o", {E, H * V}), E, H * V, nullptr);
    L.n_rec = (size_t) H * D * V;
    m.maxP = std::max(m.maxP, L.proj.N); m.maxA = std::max(m.maxA, H * V);
    m.max_ret_state = std::max(m.max_ret_state, L.n_rec); m.max_ret_dim = std::max(m.max_ret_dim, D);
}

// sigmoid attention: '<prefix>{q,k,v,q.norm,k.norm,pb,o}'; slopes 2^(-8 (h + 1) / H) are fixed by the mechanism
void load_sigattn(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const int E = m.E;
    const int H = L.H = need_int(mx, "heads"), G = L.KH = (int) mx.integer("kv_heads", H), D = L.D = need_int(mx, "dim"), V = L.V = need_int(mx, "vdim");
    if (G < 1 || H % G) throw std::runtime_error("config: attention heads must be a multiple of kv_heads");
    if (V > 256 || D > 256) throw std::runtime_error("sigmoid attention: dim and vdim above 256 are not supported by the attention kernel");
    L.scale = (float) mx.number("scale");
    if (mx.has("q_temp")) {
        L.t_coef = (float) mx.at("q_temp").number("coef");
        L.t_every = need_int(mx.at("q_temp"), "every");
    }
    std::vector<float> W = sf.read_f32(p + "q", {H * D, E});
    append(W, sf.read_f32(p + "k", {G * D, E}));
    append(W, sf.read_f32(p + "v", {G * V, E}));
    L.proj = up_mat(m, W, H * D + G * D + G * V, E, nullptr);
    L.qw = up_f32(m, sf.read_f32(p + "q.norm", {H * D}));
    L.kw = up_f32(m, sf.read_f32(p + "k.norm", {G * D}));
    L.pb = up_f32(m, sf.read_f32(p + "pb", {H}));
    std::vector<float> sl((size_t) H);
    for (int h = 0; h < H; h++) sl[(size_t) h] = (float) std::exp2(-8.0 * (h + 1) / H);
    L.slope = up_f32(m, sl);
    L.o = up_mat(m, sf.read_f32(p + "o", {E, H * V}), E, H * V, nullptr);
    L.cache_row = (size_t) G * D + (size_t) G * V;
    m.maxP = std::max(m.maxP, L.proj.N); m.maxA = std::max(m.maxA, H * V);
    m.maxCV = std::max(m.maxCV, H * D);
    m.maxQK = std::max(m.maxQK, H * D); m.maxOL = std::max(m.maxOL, H * V);
}

float read_scalar(const safetensors_file & sf, const std::string & name);
// soft-max attention over grouped heads: '<prefix>{q,k,v,o}', optional 'q.norm' / 'k.norm' [dim], 'r1' / 'r2' [heads] (distance
// penalty), 'sink' [heads], 'g' [heads][E] (output gate), 'vmix' (one number). Configuration: heads, kv_heads, dim, vdim, scale,
// softcap, rot.{base,dims}, mask.{size,pool}, v_mix. The mask's kind belongs to the mixer's name (chunks | window).
void load_gqattn(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p, int mask_kind) {
    const int E = m.E;
    const int H = L.H = need_int(mx, "heads"), G = L.KH = (int) mx.integer("kv_heads", H), D = L.D = need_int(mx, "dim"), V = L.V = need_int(mx, "vdim");
    if (G < 1 || H % G) throw std::runtime_error("config: attention heads must be a multiple of kv_heads");
    if (V > 256) throw std::runtime_error("attention: vdim above 256 is not supported by the attention kernel");
    L.scale = (float) mx.number("scale");
    L.cap = (float) mx.number("softcap", 0.0);
    if (L.cap < 0.f) throw std::runtime_error("config: softcap must not be negative");
    L.mask_kind = MASK_CAUSAL; L.window = 0; L.pool = 0;
    if (mx.has("mask")) {
        L.mask_kind = mask_kind;
        L.window = need_int(mx.at("mask"), "size");
        if (mask_kind == MASK_WINDOW) L.pool = (int) mx.at("mask").integer("pool", 0);
        if (L.pool < 0) throw std::runtime_error("config: mask.pool must not be negative");
    }
    load_rot(m, L, mx, D);
    L.rope_adjacent = m.rope_adjacent;
    std::vector<float> W = sf.read_f32(p + "q", {H * D, E});
    append(W, sf.read_f32(p + "k", {G * D, E}));
    append(W, sf.read_f32(p + "v", {G * V, E}));
    if (sf.find(p + "g")) { append(W, sf.read_f32(p + "g", {H, E})); L.head_gate = true; L.gate_rows = H; }
    L.proj = up_mat(m, W, H * D + G * D + G * V + L.gate_rows, E, nullptr);
    if (sf.find(p + "q.norm")) L.qw = up_f32(m, sf.read_f32(p + "q.norm", {D}));
    if (sf.find(p + "k.norm")) L.kw = up_f32(m, sf.read_f32(p + "k.norm", {D}));
    if (sf.find(p + "r1")) { L.r1 = up_f32(m, sf.read_f32(p + "r1", {H})); L.r2 = up_f32(m, sf.read_f32(p + "r2", {H})); }
    if (sf.find(p + "sink")) L.sink = up_f32(m, sf.read_f32(p + "sink", {H}));
    L.vmode = GQA_V_PLAIN;
    if (mx.has("v_mix") && mx.at("v_mix").kind == Json::Bool && mx.at("v_mix").b) {
        if (m.vfirst_width == 0) { L.vmode = GQA_V_FIRST; m.vfirst_width = G * V; m.vfirst_heads = G; }      // the first mixing layer's own weight is unused
        else {
            if (m.vfirst_width != G * V || m.vfirst_heads != G) throw std::runtime_error("config: value-mixing layers must agree in kv_heads and vdim");
            L.vmode = GQA_V_MIX;
            L.vlambda = read_scalar(sf, p + "vmix");
        }
    }
    L.o = up_mat(m, sf.read_f32(p + "o", {E, H * V}), E, H * V, nullptr);
    L.cache_row = (size_t) G * D + (size_t) G * V;
    m.maxP = std::max(m.maxP, L.proj.N); m.maxA = std::max(m.maxA, H * V);
    m.maxCV = std::max(m.maxCV, H * D);
    m.maxQK = std::max(m.maxQK, H * D); m.maxOL = std::max(m.maxOL, H * V);
}
void load_gqattn_chunks(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) { load_gqattn(m, L, mx, sf, p, MASK_CHUNK); }
void load_gqattn_window(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) { load_gqattn(m, L, mx, sf, p, MASK_WINDOW); }

struct MixerEntry;
const MixerEntry & find_mixer(const std::string & type, size_t layer);
void load_pair(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p);

struct MixerEntry { const char * name; int kind; void (*load)(StackModel &, LayerSpec &, const Json &, const safetensors_file &, const std::string &); };
const MixerEntry MIXERS[] = {
    { "mingru", MIX_MINGRU, load_mingru },
    { "latent_attention", MIX_LATENT, load_latent },
    { "delta", MIX_DELTA, load_delta },
    { "general_delta", MIX_GDELTA, load_gdelta },
    { "attention", MIX_DIFFATTN, load_diffattn },
    { "retention", MIX_RETENTION, load_retention },
    { "sigmoid_attention", MIX_SIGATTN, load_sigattn },
    { "parallel", MIX_PAIR, load_pair },
    { "chunk_attention", MIX_GQATTN, load_gqattn_chunks },
    { "window_attention", MIX_GQATTN, load_gqattn_window },
};

const MixerEntry & find_mixer(const std::string & type, size_t layer) {
    for (const MixerEntry & e : MIXERS) if (type == e.name) return e;
    throw std::runtime_error("config: layer " + std::to_string(layer) + " has unknown mixer type '" + type + "'");
}

// two mixers side by side on the same input: '<prefix>left.*' and '<prefix>right.*', each branch's output over its root mean
// square times '<prefix>left.out' / '<prefix>right.out', then their mean. A branch names its mixer by "type" (absent: a sigmoid
// attention on the left, a retention on the right).
void load_pair(StackModel & m, LayerSpec & L, const Json & mx, const safetensors_file & sf, const std::string & p) {
    const char * side[2] = { "left", "right" }, * dflt[2] = { "sigmoid_attention", "retention" };
    L.parts.resize(2);
    L.n_rec = 0; L.cache_row = 0;
    for (int i = 0; i < 2; i++) {
        const Json & bj = mx.at(side[i]);
        const MixerEntry & me = find_mixer(bj.string("type", dflt[i]), 0);
        if (me.kind == MIX_PAIR) throw std::runtime_error("config: a branch of a parallel mixer cannot be a parallel mixer");
        LayerSpec & B = L.parts[(size_t) i];
        B.kind = me.kind;
        me.load(m, B, bj, sf, p + side[i] + ".");
        L.pair_w[i] = up_f32(m, sf.read_f32(p + side[i] + ".out", {m.E}));
        L.n_rec += (B.n_rec + 3) / 4 * 4;
    }
    m.has_pair = true;
}

// the attention caches one run of a layer needs (a pair: its branches')
int n_layer_caches(const LayerSpec & L) {
    if (L.kind != MIX_PAIR) return L.cache_row ? 1 : 0;
    int n = 0;
    for (const LayerSpec & B : L.parts) n += B.cache_row ? 1 : 0;
    return n;
}

// one run of `layer`: its slice of the recurrent slab and, for attention, a cache of its own
void add_run(StackModel & m, int layer, int pass) {
    const LayerSpec & L = m.layers[(size_t) layer];
    RunSpec r;
    r.layer = layer; r.pass = pass;
    r.off_rec = m.rec_floats;
    m.rec_floats += (L.n_rec + 3) / 4 * 4;
    if (const int nc = n_layer_caches(L)) { r.cache_index = m.n_caches; m.n_caches += nc; }
    m.weight_bytes += L.bytes;
    m.runs.push_back(r);
}

// ---- designs ----------------------------------------------------------------------------------------------------------
// Matulorn: embed -> layers (x += norm1b(mixer(norm1 x)); x += norm2b(ff(norm2 x)) when the layer has one) -> final norm -> head
void build_matulorn(StackModel & m, const Json & cfg, const safetensors_file & sf) {
    m.vocab = need_int(cfg, "vocab"); m.E = need_int(cfg, "width");
    const Json & nj = cfg.at("norm");
    m.eps = (float) nj.number("eps");
    m.groups = (int) nj.integer("groups", 1);
    if (m.groups < 1 || m.E % m.groups) throw std::runtime_error("config: width must be a multiple of norm.groups");
    const int E = m.E;
    {
        const std::vector<float> e = sf.read_f32("embed", {m.vocab, E});
        DMat d = up_mat(m, e, m.vocab, E, nullptr);
        m.embed = d.w;
        m.weight_bytes -= d.bytes;                 // one row per token is read, not the table
    }
    const Json & layers = cfg.at("layers");
    if (layers.kind != Json::Arr || layers.arr.empty()) throw std::runtime_error("config: 'layers' must be a non-empty list");
    for (size_t i = 0; i < layers.arr.size(); i++) {
        const Json & lj = layers.arr[i];
        const std::string type = lj.string("type", ""), p = "l" + std::to_string(i) + ".";
        const MixerEntry * me = &find_mixer(type, i);
        if (me->kind != MIX_MINGRU && me->kind != MIX_LATENT && me->kind != MIX_DELTA) throw std::runtime_error("config: mixer '" + type + "' is not part of the Matulorn design");
        const int64_t bytes0 = m.weight_bytes;
        m.layers.emplace_back();
        LayerSpec & L = m.layers.back();
        L.kind = me->kind;
        L.norm1 = up_f32(m, sf.read_f32(p + "norm1", {E}));
        L.norm1b = up_f32(m, sf.read_f32(p + "norm1b", {E}));
        me->load(m, L, lj.at("mixer"), sf, p + "mix.");
        if (lj.has("mlp")) {
            const Json & mj = lj.at("mlp");
            const std::string kind = mj.string("kind", "dense");
            if (kind != "dense") throw std::runtime_error("config: feed-forward kind '" + kind + "' is not implemented (dense)");
            L.has_mlp = true;
            const int ff = L.ff = need_int(mj, "ff");
            L.limit = (float) mj.number("limit");
            L.norm2 = up_f32(m, sf.read_f32(p + "norm2", {E}));
            L.norm2b = up_f32(m, sf.read_f32(p + "norm2b", {E}));
            // gate and up interleaved row by row (2i: gate_i, 2i + 1: up_i): the product's epilogue holds both halves of a unit
            const std::vector<float> Wg = sf.read_f32(p + "mlp.gate", {ff, E}), bg = sf.read_f32(p + "mlp.gate.b", {ff});
            const std::vector<float> Wu = sf.read_f32(p + "mlp.up", {ff, E}), bu = sf.read_f32(p + "mlp.up.b", {ff});
            std::vector<float> W((size_t) 2 * ff * E), b((size_t) 2 * ff);
            for (int i = 0; i < ff; i++) {
                std::memcpy(&W[(size_t) (2 * i) * E], &Wg[(size_t) i * E], (size_t) E * 4);
                std::memcpy(&W[(size_t) (2 * i + 1) * E], &Wu[(size_t) i * E], (size_t) E * 4);
                b[(size_t) 2 * i] = bg[(size_t) i]; b[(size_t) 2 * i + 1] = bu[(size_t) i];
            }
            L.gateup = up_mat(m, W, 2 * ff, E, &b);
            const std::vector<float> db = sf.read_f32(p + "mlp.down.b", {E});
            L.down = up_mat(m, sf.read_f32(p + "mlp.down", {E, ff}), E, ff, &db);
            m.maxA = std::max(m.maxA, ff);
        }
        m.weight_bytes += (int64_t) E * 4 * (L.has_mlp ? 4 : 2);
        L.bytes = m.weight_bytes - bytes0;
        m.weight_bytes = bytes0;                       // counted per run
        add_run(m, (int) i, -1);
    }
    m.final_norm = up_f32(m, sf.read_f32("final.norm", {E}));
    m.head = up_mat(m, sf.read_f32("head", {m.vocab, E}), m.vocab, E, nullptr);
}

// Dopilorn: embed -> runs of layers (x += mixer(n1 x + conv) + ff(n2 x + conv), norms with zero-centred weights) with a
// span of layers repeated `loop.times` times (x <- W_in [x; x0] + step[t] in front of every pass) -> final norm -> head -> soft cap
void build_dopilorn(StackModel & m, const Json & cfg, const safetensors_file & sf) {
    m.block = BLOCK_PARALLEL;
    m.vocab = need_int(cfg, "vocab"); m.E = need_int(cfg, "width");
    m.eps = (float) cfg.at("norm").number("eps");
    m.groups = 1;
    m.canon_taps = cfg.has("canon") ? need_int(cfg.at("canon"), "taps") : 0;
    if (m.canon_taps > 64) throw std::runtime_error("config: canon.taps out of range");
    m.softcap = (float) cfg.number("logit_softcap", 0.0);
    const int E = m.E, ct = m.canon_taps;
    const auto one_plus = [](std::vector<float> w) { for (float & v : w) v = 1.0f + v; return w; };      // zero-centred norm weights: the file holds w, the norm multiplies by 1 + w
    {
        DMat d = up_mat(m, sf.read_f32("embed", {m.vocab, E}), m.vocab, E, nullptr);
        m.embed = d.w;
        m.weight_bytes -= d.bytes;
    }
    const Json & layers = cfg.at("layers");
    if (layers.kind != Json::Arr || layers.arr.empty()) throw std::runtime_error("config: 'layers' must be a non-empty list");
    const int n = (int) layers.arr.size();
    for (int i = 0; i < n; i++) {
        const Json & lj = layers.arr[(size_t) i];
        const std::string type = lj.string("type", ""), p = "l" + std::to_string(i) + ".";
        const MixerEntry * me = &find_mixer(type, (size_t) i);
        if (me->kind != MIX_LATENT && me->kind != MIX_GDELTA && me->kind != MIX_DIFFATTN) throw std::runtime_error("config: mixer '" + type + "' is not part of the Dopilorn design");
        const int64_t bytes0 = m.weight_bytes;
        m.layers.emplace_back();
        LayerSpec & L = m.layers.back();
        L.kind = me->kind;
        L.has_mlp = lj.has("mlp");
        L.norm1 = up_f32(m, one_plus(sf.read_f32(p + "norm1", {E})));
        if (L.has_mlp) L.norm2 = up_f32(m, one_plus(sf.read_f32(p + "norm2", {E})));
        me->load(m, L, lj.at("mixer"), sf, p + "mix.");
        if (L.kind == MIX_LATENT && (L.R || L.sink || L.window)) throw std::runtime_error("config: the Dopilorn latent attention has no rotated part, sink or window");
        if (ct > 0) {
            std::vector<float> wc = sf.read_f32(p + "canon1", {E, ct});
            if (L.has_mlp) append(wc, sf.read_f32(p + "canon2", {E, ct}));
            L.canon = up_f32(m, wc);
            if (ct > 1) L.n_rec += (size_t) (L.has_mlp ? 2 : 1) * (ct - 1) * E;       // behind the mixer's own state
        }
        if (L.has_mlp) {
            const Json & mj = lj.at("mlp");
            const std::string kind = mj.string("kind", "dense");
            if (kind != "dense") throw std::runtime_error("config: feed-forward kind '" + kind + "' is not implemented (dense)");
            const int ff = L.ff = need_int(mj, "ff");
            L.ff_kind = FF_POLY;
            L.gateup = up_mat(m, sf.read_f32(p + "mlp.up", {ff, E}), ff, E, nullptr);
            L.down = up_mat(m, sf.read_f32(p + "mlp.down", {E, ff}), E, ff, nullptr);
            L.act = up_f32(m, sf.read_f32(p + "mlp.act", {4}));
            m.maxA = std::max(m.maxA, ff);
        }
        m.weight_bytes += (int64_t) E * 4 * (L.has_mlp ? 2 : 1) * (1 + ct);
        L.bytes = m.weight_bytes - bytes0;
        m.weight_bytes = bytes0;
    }
    int start = 0, stop = 0, times = 0;
    if (cfg.has("loop")) {
        const Json & lp = cfg.at("loop");
        start = need_int(lp, "start", 0); stop = need_int(lp, "stop", 0); times = need_int(lp, "times", 0);
        if (start > stop || stop > n) throw std::runtime_error("config: loop.start .. loop.stop must lie within the layers");
        if (stop > start && times > 0) {
            m.loop_in = up_mat(m, sf.read_f32("loop.in", {E, 2 * E}), E, 2 * E, nullptr);
            m.weight_bytes += m.loop_in.bytes * (times - 1);
            m.loop_step = up_f32(m, sf.read_f32("loop.step", {times, E}));
        } else { start = stop = times = 0; }
    }
    for (int i = 0; i < start; i++) add_run(m, i, -1);
    for (int t = 0; t < times; t++) for (int i = start; i < stop; i++) add_run(m, i, i == start ? t : -1);
    for (int i = stop; i < n; i++) add_run(m, i, -1);
    m.final_norm = up_f32(m, one_plus(sf.read_f32("final.norm", {E})));
    m.head = up_mat(m, sf.read_f32("head", {m.vocab, E}), m.vocab, E, nullptr);
}

// Tosevik: x0 = dyt(embed) -> layers (y = z + mixer(dyt1 z); y += mixture(dyt2 y) when the layer has a feed-forward; the next layer
// reads z = sum_j dwa[j] x_j over the embedding output and all results so far) -> dyt -> head. Norms are element-wise (dynamic
// tanh: weight, bias '.b', slope '.alpha'). Mixers: retention | parallel (sigmoid attention beside retention).
float read_scalar(const safetensors_file & sf, const std::string & name) {
    const st_tensor * t = sf.find(name);
    if (!t || t->numel() != 1) throw std::runtime_error("tensor " + name + " is missing or not a single number");
    return sf.read_f32(name, t->shape)[0];
}
DMat load_glu_pair(StackModel & m, const safetensors_file & sf, const std::string & p, int ff, int E, std::vector<float> * into) {
    // gate and up interleaved row by row (2i: gate_i, 2i + 1: up_i): the product's epilogue holds both halves of a unit
    const std::vector<float> Wg = sf.read_f32(p + "gate", {ff, E}), Wu = sf.read_f32(p + "up", {ff, E});
    std::vector<float> W((size_t) 2 * ff * E);
    for (int i = 0; i < ff; i++) {
        std::memcpy(&W[(size_t) (2 * i) * E], &Wg[(size_t) i * E], (size_t) E * 4);
        std::memcpy(&W[(size_t) (2 * i + 1) * E], &Wu[(size_t) i * E], (size_t) E * 4);
    }
    if (into) { append(*into, W); return DMat(); }
    return up_mat(m, W, 2 * ff, E, nullptr);
}
// what a design fixes about its routed mixture: the score function, where a choice's weight is applied, a gate on the shared unit
struct MixtureKind { int route_fn; bool scale_input; bool shared_gate; };
void load_mixture(StackModel & m, LayerSpec & L, const Json & mj, const safetensors_file & sf, const std::string & p, const MixtureKind & mk) {
    const int E = m.E;
    L.route_fn = mk.route_fn; L.scale_input = mk.scale_input;
    const Json & rj = mj.at("router");
    const int n = L.n_exp = need_int(rj, "experts"), top = L.top = need_int(rj, "top");
    L.r_scale = (float) rj.number("scale", 1.0);
    L.n_groups = rj.has("groups") ? need_int(rj.at("groups"), "count") : 1;
    L.keep_groups = rj.has("groups") ? need_int(rj.at("groups"), "keep") : 1;
    if (n % L.n_groups) throw std::runtime_error("config: experts must be a multiple of groups.count");
    if (L.keep_groups > L.n_groups) throw std::runtime_error("config: groups.keep exceeds groups.count");
    if (top > L.keep_groups * (n / L.n_groups)) throw std::runtime_error("config: router.top exceeds the experts of the kept groups");
    if (n > 4096 || top > 64) throw std::runtime_error("config: more than 4096 experts or 64 choices per token are not supported");
    const int ff = L.e_ff = need_int(mj.at("expert"), "ff");
    L.ff_kind = FF_MOE;
    L.router = up_f32(m, sf.read_f32(p + "router", {n, E}));
    std::vector<float> GU, DN;
    for (int e = 0; e < n; e++) {
        const std::string ep = p + "e" + std::to_string(e) + ".";
        load_glu_pair(m, sf, ep, ff, E, &GU);
        append(DN, sf.read_f32(ep + "down", {E, ff}));
    }
    const int64_t before = m.weight_bytes;
    L.e_gateup = up_mat(m, GU, 2 * ff, E, nullptr, n);
    L.e_down = up_mat(m, DN, E, ff, nullptr, n);
    m.weight_bytes = before + (m.weight_bytes - before) / n * top + (int64_t) n * E * 4;      // a token reads its chosen experts and the router
    L.ff = 0;
    if (mj.has("shared")) {
        const int sff = L.ff = need_int(mj.at("shared"), "ff");
        L.gateup = load_glu_pair(m, sf, p + "shared.", sff, E, nullptr);
        L.down = up_mat(m, sf.read_f32(p + "shared.down", {E, sff}), E, sff, nullptr);
        if (mk.shared_gate) L.w_sg = up_f32(m, sf.read_f32(p + "shared.sg", {1, E}));
        m.maxA = std::max(m.maxA, sff);
    }
    m.max_slots = std::max(m.max_slots, top); m.max_eff = std::max(m.max_eff, ff); m.max_exp = std::max(m.max_exp, n);
}
void build_tosevik(StackModel & m, const Json & cfg, const safetensors_file & sf) {
    m.block = BLOCK_PRENORM;
    m.dyt = true; m.depth_avg = true;
    m.vocab = need_int(cfg, "vocab"); m.E = need_int(cfg, "width");
    m.eps = (float) cfg.at("norm").number("eps");
    m.groups = 1;
    const int E = m.E;
    {
        DMat d = up_mat(m, sf.read_f32("embed", {m.vocab, E}), m.vocab, E, nullptr);
        m.embed = d.w;
        m.weight_bytes -= d.bytes;
    }
    m.embed_w = up_f32(m, sf.read_f32("embed.norm", {E})); m.embed_b = up_f32(m, sf.read_f32("embed.norm.b", {E})); m.embed_alpha = read_scalar(sf, "embed.norm.alpha");
    const Json & layers = cfg.at("layers");
    if (layers.kind != Json::Arr || layers.arr.empty()) throw std::runtime_error("config: 'layers' must be a non-empty list");
    const int n = (int) layers.arr.size();
    for (int i = 0; i < n; i++) {
        const Json & lj = layers.arr[(size_t) i];
        const std::string type = lj.string("type", ""), p = "l" + std::to_string(i) + ".";
        const MixerEntry * me = &find_mixer(type, (size_t) i);
        if (me->kind != MIX_RETENTION && me->kind != MIX_PAIR) throw std::runtime_error("config: mixer '" + type + "' is not part of the Tosevik design");
        const int64_t bytes0 = m.weight_bytes;
        m.layers.emplace_back();
        LayerSpec & L = m.layers.back();
        L.kind = me->kind;
        L.has_mlp = lj.has("mlp");
        L.norm1 = up_f32(m, sf.read_f32(p + "norm1", {E})); L.n1_b = up_f32(m, sf.read_f32(p + "norm1.b", {E})); L.n1_alpha = read_scalar(sf, p + "norm1.alpha");
        me->load(m, L, lj.at("mixer"), sf, p + "mix.");
        if (L.has_mlp) {
            const Json & mj = lj.at("mlp");
            const std::string kind = mj.string("kind", "moe");
            if (kind != "moe") throw std::runtime_error("config: feed-forward kind '" + kind + "' is not part of the Tosevik design (moe)");
            L.norm2 = up_f32(m, sf.read_f32(p + "norm2", {E})); L.n2_b = up_f32(m, sf.read_f32(p + "norm2.b", {E})); L.n2_alpha = read_scalar(sf, p + "norm2.alpha");
            load_mixture(m, L, mj, sf, p + "mlp.", MixtureKind{0, false, true});
        }
        L.n_dwa = i + 2;
        L.dwa = up_f32(m, sf.read_f32(p + "dwa", {i + 2}));
        m.weight_bytes += (int64_t) E * 4 * (L.has_mlp ? 4 : 2);
        L.bytes = m.weight_bytes - bytes0;
        m.weight_bytes = bytes0;
        add_run(m, i, -1);
    }
    m.final_norm = up_f32(m, sf.read_f32("final.norm", {E})); m.final_b = up_f32(m, sf.read_f32("final.norm.b", {E})); m.final_alpha = read_scalar(sf, "final.norm.alpha");
    m.head = up_mat(m, sf.read_f32("head", {m.vocab, E}), m.vocab, E, nullptr);
}

// Rumurax: embed -> S equal streams -> layers (per sub-layer: u = sum_s in[s] x_s; y = f(norm(u) g); x_t <- sum_s mix[s][t] x_s +
// out[t] y, tensors '<layer>.hc1.*' for the mixer and '<layer>.hc2.*' for the mixture) -> sum of the streams -> norm -> head.
// Norm weights are one number each. The design's mixer names map to registry entries; rotations pair neighbours.
HcW load_hc(const safetensors_file & sf, const std::string & p, int S) {
    HcW w{};
    if (!sf.find(p + "in")) {
        if (S != 1) throw std::runtime_error("tensor '" + p + "in' is missing");
        w.in[0] = w.mix[0] = w.out[0] = 1.f;                 // one stream and no weights: the plain residual sum
        return w;
    }
    const std::vector<float> a = sf.read_f32(p + "in", {S}), b = sf.read_f32(p + "out", {S}), M = sf.read_f32(p + "mix", {S, S});
    for (int i = 0; i < S; i++) { w.in[i] = a[(size_t) i]; w.out[i] = b[(size_t) i]; }
    for (int i = 0; i < S * S; i++) w.mix[i] = M[(size_t) i];      // [from][to]
    return w;
}
void build_rumurax(StackModel & m, const Json & cfg, const safetensors_file & sf) {
    static const char * const alias[][2] = { { "attention", "chunk_attention" }, { "attention_2", "window_attention" }, { "latent_attention", "latent_attention" } };
    m.block = BLOCK_HYPER;
    m.rope_adjacent = true;
    m.vocab = need_int(cfg, "vocab"); m.E = need_int(cfg, "width");
    m.eps = (float) cfg.at("norm").number("eps");
    m.groups = 1;
    const int S = m.streams = (int) cfg.integer("streams", 1);
    if (S < 1 || S > HC_MAX) throw std::runtime_error("config: 'streams' must lie between 1 and " + std::to_string(HC_MAX));
    const int E = m.E;
    {
        DMat d = up_mat(m, sf.read_f32("embed", {m.vocab, E}), m.vocab, E, nullptr);
        m.embed = d.w;
        m.weight_bytes -= d.bytes;
    }
    const Json & layers = cfg.at("layers");
    if (layers.kind != Json::Arr || layers.arr.empty()) throw std::runtime_error("config: 'layers' must be a non-empty list");
    const int n = (int) layers.arr.size();
    for (int i = 0; i < n; i++) {
        const Json & lj = layers.arr[(size_t) i];
        const std::string type = lj.string("type", ""), p = "l" + std::to_string(i) + ".";
        const char * entry = nullptr;
        for (const auto & a : alias) if (type == a[0]) entry = a[1];
        if (!entry) throw std::runtime_error("config: layer " + std::to_string(i) + ": mixer '" + type + "' is not part of the Rumurax design");
        const MixerEntry * me = &find_mixer(entry, (size_t) i);
        const int64_t bytes0 = m.weight_bytes;
        m.layers.emplace_back();
        LayerSpec & L = m.layers.back();
        L.kind = me->kind;
        L.has_mlp = lj.has("mlp");
        L.g1 = read_scalar(sf, p + "norm1");
        L.hc[0] = load_hc(sf, p + "hc1.", S);
        me->load(m, L, lj.at("mixer"), sf, p + "mix.");
        if (L.kind == MIX_LATENT && (L.q_rank || L.sink || L.window)) throw std::runtime_error("config: the Rumurax latent attention has no query latent, sink or window");
        if (L.has_mlp) {
            const Json & mj = lj.at("mlp");
            const std::string kind = mj.string("kind", "moe");
            if (kind != "moe") throw std::runtime_error("config: feed-forward kind '" + kind + "' is not part of the Rumurax design (moe)");
            L.g2 = read_scalar(sf, p + "norm2");
            L.hc[1] = load_hc(sf, p + "hc2.", S);
            load_mixture(m, L, mj, sf, p + "mlp.", MixtureKind{1, true, false});
        }
        L.bytes = m.weight_bytes - bytes0;
        m.weight_bytes = bytes0;
        add_run(m, i, -1);
    }
    m.final_g = read_scalar(sf, "final.norm");
    m.head = up_mat(m, sf.read_f32("head", {m.vocab, E}), m.vocab, E, nullptr);
}

struct DesignEntry { const char * name; void (*build)(StackModel &, const Json &, const safetensors_file &); };
const DesignEntry DESIGNS[] = {
    { "Matulorn", build_matulorn },
    { "Dopilorn", build_dopilorn },
    { "Tosevik", build_tosevik },
    { "Rumurax", build_rumurax },
};

// ---- launches ---------------------------------------------------------------------------------------------------------
bool mma_enabled() {
    static const bool on = [] { const char * e = std::getenv("BOOSTER_B200_STACK_MMA"); return !(e && e[0] == '0'); }();
    return on;
}

bool umma_enabled() {
    static const bool on = [] { const char * e = std::getenv("BOOSTER_B200_STACK_UMMA"); return !(e && e[0] == '0'); }();
    return on;
}
// what the tcgen05 product needs beside its operands: room for the activations rounded to bfloat16 and the error flag its
// bounded waits raise
struct UmmaScratch { __nv_bfloat16 * xb = nullptr; size_t elems = 0; int * err = nullptr; };

// what a product may ask for beyond its operands: the gated unit's constants (y = g sigmoid(alpha g) (u + shift), g and u clamped
// at +-limit), rows sorted into segments per batch entry (tile kernels), an indexed batch (mat-vec)
struct LinOpt {
    float alpha = GLU_ALPHA, shift = 1.f;
    const int32_t * seg = nullptr;
    const int32_t * w_index = nullptr;
    int x_share = 1;
    const float * x_scale = nullptr;        // mat-vec: entry z runs on x_scale[z] times its input row
};
void linear_on(cudaStream_t st, int dtype, int64_t * launches, const float * X, int ldx, const void * W, const float * bias, float * Y, int ldy,
               int T, int N, int K, int batch = 1, long long sX = 0, long long sW = 0, long long sY = 0, bool glu = false, float glu_limit = 0.f,
               const UmmaScratch * us = nullptr, const LinOpt * opt = nullptr) {
    if (T <= 0 || N <= 0) return;
    LinArgs a{X, W, bias, Y, T, N, K, ldx, ldy, sX, sW, sY, 0, glu ? 1 : 0, glu_limit, GLU_ALPHA, 0, 0};
    if (opt) { a.alpha = opt->alpha; a.up_shift = opt->shift; a.seg = opt->seg; a.w_index = opt->w_index; a.x_share = opt->x_share; a.x_scale = opt->x_scale; }
    const int xbatch = a.seg ? 1 : batch;      // segments: X is one matrix of T rows
    const int vecw = dtype == STACK_F32 ? 4 : 8;
    const auto al16 = [](const void * p) { return ((uintptr_t) p & 15) == 0; };
    a.vec = K % vecw == 0 && ldx % 4 == 0 && sX % 4 == 0 && sW % vecw == 0 && al16(X) && al16(W);
    if (launches) (*launches)++;
    if (T <= GEMV_MAX_T) {
        if (a.glu) {
            const dim3 grid((unsigned) ((N / 2 + 7) / 8), 1, (unsigned) batch);
            if (dtype == STACK_F32) k_gemv<float, 2><<<grid, 256, 0, st>>>(a); else k_gemv<__nv_bfloat16, 2><<<grid, 256, 0, st>>>(a);
        } else {
            const dim3 grid((unsigned) ((N + 7) / 8), 1, (unsigned) batch);
            if (dtype == STACK_F32) k_gemv<float, 1><<<grid, 256, 0, st>>>(a); else k_gemv<__nv_bfloat16, 1><<<grid, 256, 0, st>>>(a);
        }
    } else if (dtype == STACK_BF16 && a.vec && us && us->xb && umma_enabled() && T >= 64 && N >= 128 && K >= 64 && (size_t) xbatch * T * K <= us->elems) {
        // tensor memory path: activations to bfloat16 once, then tcgen05.mma over cp.async-fed stages
        static const bool attr = [] { return cudaFuncSetAttribute(k_gemm_bf16_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_SMEM) == cudaSuccess; }();
        if (!attr) throw std::runtime_error("cannot reserve shared memory for k_gemm_bf16_umma");
        k_to_bf16<<<dim3((unsigned) std::min((K + 255) / 256, 64), (unsigned) T, (unsigned) xbatch), 256, 0, st>>>(X, ldx, T, K, sX, us->xb, (long long) T * K);
        const dim3 grid((unsigned) ((N + UM_BN - 1) / UM_BN), (unsigned) ((T + UM_BM - 1) / UM_BM), (unsigned) batch);
        k_gemm_bf16_umma<<<grid, 256, UM_SMEM, st>>>(a, us->xb, (long long) T * K, us->err);
        if (launches) (*launches)++;
    } else if (dtype == STACK_BF16 && a.vec && mma_enabled()) {
        const dim3 grid((unsigned) ((N + MM_BN - 1) / MM_BN), (unsigned) ((T + MM_BM - 1) / MM_BM), (unsigned) batch);
        k_gemm_bf16_mma<<<grid, 256, 0, st>>>(a);
    } else {
        const dim3 grid((unsigned) ((N + 63) / 64), (unsigned) ((T + 63) / 64), (unsigned) batch);
        if (dtype == STACK_F32) k_gemm_simt<float><<<grid, 256, 0, st>>>(a); else k_gemm_simt<__nv_bfloat16><<<grid, 256, 0, st>>>(a);
    }
    SCU(cudaGetLastError());
}

void linear(StackCtx * c, const float * X, int ldx, const DMat & W, float * Y, int ldy, int T, int batch = 1, long long sX = 0, long long sY = 0, bool glu = false, float glu_limit = 0.f,
            const LinOpt * opt = nullptr) {
    const UmmaScratch us{c->xb, c->xb_elems, c->d_err};
    linear_on(c->st, c->m->dtype, &c->launches, X, ldx, W.w, W.bias, Y, ldy, T, W.N, W.K, batch, sX, (long long) W.N * W.K, sY, glu, glu_limit, &us, opt);
}

// end of a sub-layer: X += norm(Y) * w_post; Hn = norm(X) * w_next when another sub-layer follows
void post_norm_add(StackCtx * c, const float * w_post, const float * w_next, int T) {
    const StackModel & m = *c->m;
    k_post_norm_add<<<T, std::min(256, 32 * m.groups), 0, c->st>>>(c->Y, w_post, c->X, w_next, c->Hn, m.E, m.groups, m.eps);
    c->launches++;
}

void norm(StackCtx * c, const float * X, int ldx, const int32_t * rows, const float * w, int n, int groups, float * Y, int ldy, int T, bool accumulate) {
    const int threads = std::min(256, 32 * groups);
    k_group_norm<<<T, threads, 0, c->st>>>(X, ldx, rows, w, n, groups, c->m->eps, Y, ldy, accumulate ? 1 : 0);
    c->launches++;
    SCU(cudaGetLastError());
}

template <int DMAX>
void launch_delta_scan(StackCtx * c, const LayerSpec & L, int T, int C, float * S) {
    const int threads = std::min(128, (L.V + 31) / 32 * 32);
    const dim3 grid((unsigned) L.H, (unsigned) ((L.V + threads - 1) / threads));
    k_delta_scan<DMAX><<<grid, threads, 0, c->st>>>(c->CV, C, c->BG, T, L.H, L.KH, L.D, L.V, S, c->O);
}

// mixers: c->in [T][E] -> c->out [T][E]; R names the run's state
void mixer_mingru(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    linear(c, c->in, c->m->E, L.zxg, c->P, 3 * L.width, T);
    k_mingru_scan<<<(L.width + 127) / 128, 128, 0, c->st>>>(c->P, T, L.width, c->rec + R.off_rec, c->A);
    c->launches++;
    linear(c, c->A, L.width, L.o, c->out, c->m->E, T);
}

// launch shape of the latent attention for a pass of T tokens: queries per block, key slices, shared memory
struct AttnPlan { int TQ, HQ, nsplit, smax; size_t smem; bool staged; };
AttnPlan plan_attention(const LayerSpec & L, int n_ctx, int T, int sm_count) {
    AttnPlan p;
    p.TQ = std::min(T, 4);
    const int W = L.rank + L.R;
    const int keys = L.window > 0 ? std::min(L.window + p.TQ - 1, n_ctx) : n_ctx;     // the most keys a tile can see
    {   // staged: a block takes as many heads as it may (every cached row is fetched once per token tile) and a slice of >= 8 keys that fits shared memory
        p.staged = true;
        p.HQ = std::min(L.H, std::max(1, LAT_NQ_MAX / p.TQ));
        int blocks = ((T + p.TQ - 1) / p.TQ) * ((L.H + p.HQ - 1) / p.HQ);
        const int WP = W % 4 == 0 ? W + 4 : (W | 1);
        p.nsplit = std::max(1, std::min({ 2 * sm_count / blocks, (keys + 7) / 8, 64 }));
        while (blocks * p.nsplit < sm_count && p.HQ > 4) {      // SMs left idle: fewer heads per block (the rows come from L2 again)
            p.HQ = (p.HQ + 1) / 2;
            blocks = ((T + p.TQ - 1) / p.TQ) * ((L.H + p.HQ - 1) / p.HQ);
        }
        for (;;) {
            p.smax = (keys + p.nsplit - 1) / p.nsplit;
            p.smem = ((size_t) p.TQ * p.HQ * (W + p.smax + 1) + (size_t) p.smax * WP + 8) * 4;
            if (p.smem <= 160 * 1024 || p.nsplit >= 64) break;
            p.nsplit = std::min(64, p.nsplit * 2);
        }
        if (p.smem <= 160 * 1024) return p;
    }
    p.staged = false;                     // long unmasked contexts: the slices stay in global memory
    p.HQ = std::min(L.H, std::max(1, LAT_NQ_MAX / p.TQ));
    if (T < 8) p.HQ = std::min(p.HQ, 4);
    const int blocks = ((T + p.TQ - 1) / p.TQ) * ((L.H + p.HQ - 1) / p.HQ);
    p.nsplit = 1;
    if (blocks < sm_count) p.nsplit = std::max(1, std::min({ 2 * sm_count / blocks, (keys + 31) / 32, 64 }));
    for (;;) {
        p.smax = (keys + p.nsplit - 1) / p.nsplit;
        p.smem = ((size_t) p.TQ * p.HQ * (W + p.smax + 1) + 8) * 4;
        if (p.smem <= 200 * 1024 || p.nsplit >= 64) break;
        p.nsplit *= 2;                    // slice the keys until the scores of a block fit
    }
    while (p.smem > 200 * 1024 && p.HQ > 1) { p.HQ = (p.HQ + 1) / 2; p.smem = ((size_t) p.TQ * p.HQ * (W + p.smax + 1) + 8) * 4; }
    return p;
}

bool simt_big_enabled() {
    static const bool on = [] { const char * e = std::getenv("BOOSTER_B200_STACK_SIMT_BIG"); return !(e && e[0] == '0'); }();
    return on;
}
// float32 product on the CUDA cores with explicit operand layout (the attention's two products over cached rows)
// A second batch level (nz2 products per first-level index, strides sX2 / sW2 / sY2) serves operands that are cut twice: tiles x heads.
void gemm_f32(StackCtx * c, const float * X, int ldx, long long sX, const float * W, int w_kn, int ldw, long long sW, float * Y, int ldy, long long sY,
              int M, int N, int K, int batch, int nz2 = 1, long long sX2 = 0, long long sW2 = 0, long long sY2 = 0, int accum = 0) {
    const auto al16 = [](const void * p) { return ((uintptr_t) p & 15) == 0; };
    LinArgs a{X, W, nullptr, Y, M, N, K, ldx, ldy, sX, sW, sY, 0, 0, 0.f, 0.f, w_kn, ldw, nz2, sX2, sW2, sY2};
    a.vec = K % 4 == 0 && ldx % 4 == 0 && sX % 4 == 0 && sW % 4 == 0 && sX2 % 4 == 0 && sW2 % 4 == 0 && ldw % 4 == 0 && al16(X) && al16(W);
    a.accum = accum;
    if (a.vec && M >= SG_BM && N >= SG_BN && simt_big_enabled())       // operands that fill 128 x 128 tiles
        k_gemm_simt_big<<<dim3((unsigned) ((N + SG_BN - 1) / SG_BN), (unsigned) ((M + SG_BM - 1) / SG_BM), (unsigned) (batch * nz2)), 256, 0, c->st>>>(a);
    else k_gemm_simt<float><<<dim3((unsigned) ((N + 63) / 64), (unsigned) ((M + 63) / 64), (unsigned) (batch * nz2)), 256, 0, c->st>>>(a);
    c->launches++;
}
constexpr int ATT_TQ = 16;                 // tokens per tile of the prompt attention
constexpr size_t ATT_SCORE_BYTES = (size_t) 256 << 20;

// the latent attention's last steps: per-head values A[t][h] = W_uv,h (sum_j w_j c_j), head gates, output product
void latent_values_out(StackCtx * c, const LayerSpec & L, int T, int ldp, int gate_off) {
    const int H = L.H, V = L.V, rank = L.rank;
    linear(c, c->OL, H * rank, L.uv, c->A, H * V, T, H, rank, V);
    if (L.head_gate) { k_head_gate<<<dim3((unsigned) T, T <= 16 ? (unsigned) ((H * V + 255) / 256) : 1u), 256, 0, c->st>>>(c->A, c->P + gate_off, ldp, H, V, L.gate_rows == H ? 0 : 1); c->launches++; }
    linear(c, c->A, H * V, L.o, c->out, c->m->E, T);
}

void mixer_latent(StackCtx * c, const LayerSpec & L, const RunSpec & Rn, int T) {
    const int E = c->m->E, H = L.H, D = L.D, R = L.R, rank = L.rank, W = rank + R;
    const int ldp = L.qdkv.N;
    float * cache = c->caches[(size_t) Rn.cache_index];
    linear(c, c->in, E, L.qdkv, c->P, ldp, T);
    const RopeArgs rope{L.rope_freq, L.rope_dims, L.rope_mag, L.rope_adjacent ? 1 : 0};
    int gate_off;
    if (L.q_rank > 0) {
        // P[t] = [ query latent | down-projection | head gates ]: norm of the query latent in place, q = W_uq c_q into A, cache row, absorbed queries from A
        gate_off = L.q_rank + rank;
        k_latent_prep<<<dim3((unsigned) T, T <= 16 ? (unsigned) ((H + 4) / 4) : 1u), 128, 0, c->st>>>(c->P, ldp, H, D, 0, rank, L.cnorm, c->m->eps, rope, &c->d_step->st, cache, c->QK, L.q_rank, L.qnorm, L.q_rank);
        linear(c, c->P, ldp, L.uq, c->A, H * D, T);
        linear(c, c->A, H * D, L.ukT, c->QK, H * W, T, H, D, W);
    } else {
        gate_off = H * (D + R) + W;
        k_latent_prep<<<dim3((unsigned) T, T <= 16 ? (unsigned) ((H + 4) / 4) : 1u), 128, 0, c->st>>>(c->P, ldp, H, D, R, rank, L.cnorm, c->m->eps, rope, &c->d_step->st, cache, c->QK, H * (D + R), nullptr, 0);
        // absorbed queries, one product per head: QK[t][h][0..rank) = W_uk,h^T q[t][h][0..D)
        linear(c, c->P, ldp, L.ukT, c->QK, H * W, T, H, D + R, W);
    }
    if (T >= 8) {
        // prompt portion: scores, row soft-max and weighted sum as float32 products over tiles of ATT_TQ tokens x all heads
        const int TQ = ATT_TQ, M = TQ * H, ntile = (T + TQ - 1) / TQ;
        const int pos0 = c->h_step->st.pos0;                                       // of this pass (set by the step function before the launches)
        // keys a tile's rows can see: the window (no wider than the sequence so far) plus the tile; unmasked: all so far. Padded for 16-byte rows
        const int span = L.window > 0 ? std::min(L.window, pos0 + ntile * TQ) : 0;
        const int nk = ((L.window > 0 ? span + TQ - 1 : pos0 + ntile * TQ) + 3) / 4 * 4;
        const int per_group = (int) std::max<size_t>(1, c->att_scores_floats / ((size_t) M * nk));
        for (int g0 = 0; g0 < ntile; g0 += per_group) {
            const int ng = std::min(per_group, ntile - g0);
            const long long jlo = L.window > 0 ? (long long) pos0 + (long long) g0 * TQ - span + 1 : 0;     // may be negative: the cache has a zero margin in front
            const float * keys = cache + jlo * W;
            const long long sK = L.window > 0 ? (long long) TQ * W : 0;
            gemm_f32(c, c->QK + (size_t) g0 * M * W, W, (long long) M * W, keys, 0, 0, sK, c->att_scores, nk, (long long) M * nk, M, nk, W, ng);
            const int rows = (std::min(T, (g0 + ng) * TQ) - g0 * TQ) * H;
            k_latent_softmax_rows<<<(rows + 7) / 8, 256, 0, c->st>>>(c->att_scores, rows, H, TQ, nk, L.window, span, L.sink, &c->d_step->st, L.scale, g0);
            gemm_f32(c, c->att_scores, nk, (long long) M * nk, keys, 1, W, sK, c->OL + (size_t) g0 * M * rank, rank, (long long) M * rank, M, rank, nk, ng);
            c->launches++;
        }
        c->launches++;
        latent_values_out(c, L, T, ldp, gate_off);
        return;
    }
    const AttnPlan ap = plan_attention(L, c->n_ctx, T, c->sm_count);
    const LatAttnArgs aa{c->QK, cache, L.sink, &c->d_step->st, c->OL, c->att_part, c->att_ml, T, H, rank, R, L.window, L.scale, ap.TQ, ap.HQ, ap.nsplit, ap.smax};
    const dim3 grid((unsigned) ((T + ap.TQ - 1) / ap.TQ), (unsigned) ((H + ap.HQ - 1) / ap.HQ), (unsigned) ap.nsplit);
    if (!ap.staged) k_latent_attn<<<grid, 256, ap.smem, c->st>>>(aa);
    else if (W % 4 == 0) k_latent_attn_staged<true><<<grid, 256, ap.smem, c->st>>>(aa);
    else k_latent_attn_staged<false><<<grid, 256, ap.smem, c->st>>>(aa);
    if (ap.nsplit > 1) { k_latent_combine<<<dim3((unsigned) T, (unsigned) H, (unsigned) ((rank + 63) / 64)), 256, 0, c->st>>>(aa); c->launches++; }
    c->launches += 2;
    latent_values_out(c, L, T, ldp, gate_off);
}

// causal convolution of a portion's rows with the history a sequence keeps (k_causal_conv), then the history moves on
void causal_conv(StackCtx * c, ConvArgs a, int batch = 1) {
    a.fuse_hist = a.T == 1 ? 1 : 0;
    k_causal_conv<<<dim3((unsigned) ((a.C + 127) / 128), (unsigned) a.T, (unsigned) batch), 128, 0, c->st>>>(a);
    c->launches++;
    if (a.taps > 1 && !a.fuse_hist) { k_causal_conv_hist<<<dim3((unsigned) ((a.C + 127) / 128), 1, (unsigned) batch), 128, 0, c->st>>>(a); c->launches++; }
}

void mixer_delta(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    const int E = c->m->E, H = L.H, KH = L.KH, D = L.D, V = L.V, C = 2 * KH * D + H * V, ldp = C + 2 * H + H * V;
    float * S = c->rec + R.off_rec, * hist = S + (size_t) H * D * V;
    linear(c, c->in, E, L.proj, c->P, ldp, T);
    causal_conv(c, ConvArgs{c->P, ldp, 0, L.wconv, 0, hist, 0, c->CV, C, 0, T, C, L.taps, 1, 0, nullptr, nullptr, 0, 0, 0});
    k_delta_gates<<<T, 128, 0, c->st>>>(c->CV, C, c->P, ldp, H, KH, D, V, L.A_log, L.dt_bias, c->BG);
    if (D <= 32) launch_delta_scan<32>(c, L, T, C, S);
    else if (D <= 64) launch_delta_scan<64>(c, L, T, C, S);
    else if (D <= 128) launch_delta_scan<128>(c, L, T, C, S);
    else launch_delta_scan<256>(c, L, T, C, S);
    k_delta_out<<<dim3((unsigned) T, (unsigned) ((H + 3) / 4)), 128, 0, c->st>>>(c->O, c->P, ldp, C + 2 * H, H, V, L.dnorm, 0, 0, c->m->eps, c->A);
    c->launches += 3;
    linear(c, c->A, H * V, L.o, c->out, E, T);
}

template <int DMAX>
void launch_gdelta_scan(StackCtx * c, const LayerSpec & L, int T, int ldp, float * S) {
    // four lanes per column of the state; a head's columns are spread over blocks of >= 16 until the grid fills the SMs (every
    // block stages the same r, k, w, u, b of a token tile, which is little beside its share of the walk)
    int ncols = std::min(128, (L.V + 7) / 8 * 8);
    while (ncols > 16 && L.H * ((L.V + ncols - 1) / ncols) < c->sm_count) ncols = (ncols / 2 + 7) / 8 * 8;
    const int threads = GD_RG * ncols, HD = L.H * L.D;
    const dim3 grid((unsigned) L.H, (unsigned) ((L.V + ncols - 1) / ncols));
    k_gdelta_scan<DMAX><<<grid, threads, 0, c->st>>>(c->P, ldp, 0, HD, 2 * HD, c->CV, T, L.H, L.D, L.V, S, c->O);
}

// generalized delta rule: P[t] = [ r | k | v | gate | removal logit | decay latent ]
void mixer_gdelta(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    const int E = c->m->E, H = L.H, D = L.D, V = L.V, HD = H * D, HV = H * V, ldp = L.proj.N, lat_off = 3 * HD + 2 * HV;
    float * S = c->rec + R.off_rec;
    linear(c, c->in, E, L.proj, c->P, ldp, T);
    const dim3 pgrid((unsigned) T, (unsigned) H);
    if (c->m->dtype == STACK_F32) k_gdelta_prep<float><<<pgrid, 128, (size_t) (L.lora + D) * 4, c->st>>>(c->P, ldp, HD, 2 * HD + 2 * HV, lat_off, L.lora, (const float *) L.w2.w, L.w2.bias, H, D, c->CV);
    else k_gdelta_prep<__nv_bfloat16><<<pgrid, 128, (size_t) (L.lora + D) * 4, c->st>>>(c->P, ldp, HD, 2 * HD + 2 * HV, lat_off, L.lora, (const __nv_bfloat16 *) L.w2.w, L.w2.bias, H, D, c->CV);
    if (D <= 32) launch_gdelta_scan<32>(c, L, T, ldp, S);
    else if (D <= 64) launch_gdelta_scan<64>(c, L, T, ldp, S);
    else if (D <= 128) launch_gdelta_scan<128>(c, L, T, ldp, S);
    else launch_gdelta_scan<256>(c, L, T, ldp, S);
    k_delta_out<<<dim3((unsigned) T, (unsigned) ((H + 3) / 4)), 128, 0, c->st>>>(c->O, c->P, ldp, 2 * HD + HV, H, V, L.dnorm, V, 1, c->m->eps, c->A);
    c->launches += 3;
    linear(c, c->A, HV, L.o, c->out, E, T);
}

constexpr int DIFF_MAX_SPLIT = 16;
size_t diffattn_smem(const LayerSpec & L, int TQ) {
    const int VPL = L.V <= 32 ? 1 : L.V <= 64 ? 2 : L.V <= 128 ? 4 : 8;
    return ((size_t) TQ * 2 * L.D + (size_t) 8 * (4 + 64 * VPL)) * 4;
}

// differential sliding-window attention: P[t] = [ q | k | v ] (biases included) -> convolution over time -> queries to CV, keys
// and values to the cache row of the token's position -> attention with the difference and its norm -> output product
void mixer_diffattn(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    const int E = c->m->E, H = L.H, G = L.KH, D = L.D, V = L.V, nq = H * 2 * D, row = (int) L.cache_row, C = nq + row;
    float * cache = c->caches[(size_t) R.cache_index];
    linear(c, c->in, E, L.proj, c->P, C, T);
    causal_conv(c, ConvArgs{c->P, C, 0, L.wconv, 0, c->rec + R.off_rec, 0, c->CV, nq, 0, T, C, L.taps, 0, 0, &c->d_step->st, cache, row, nq, 0});
    const float * Q = c->CV;
    const int ldq = nq;
    if (T >= 8) {
        // prompt portion: float32 products over tiles of ATT_TQ tokens, one batch entry per (tile, key/value head, map)
        const int TQ = ATT_TQ, Rh = H / G, M = TQ * Rh, ntile = (T + TQ - 1) / TQ, Tpad = ntile * TQ;
        const int pos0 = c->h_step->st.pos0;
        k_diff_q_layout<<<Tpad, 256, 0, c->st>>>(Q, ldq, T, Tpad, H, G, D, c->QK);
        const int span = L.window > 0 ? std::min(L.window, pos0 + Tpad) : 0;
        const int nk = ((L.window > 0 ? span + TQ - 1 : pos0 + Tpad) + 3) / 4 * 4;
        const int per_group = (int) std::max<size_t>(1, c->att_scores_floats / ((size_t) 2 * G * M * nk));
        for (int g0 = 0; g0 < ntile; g0 += per_group) {
            const int ng = std::min(per_group, ntile - g0);
            const long long jlo = L.window > 0 ? (long long) pos0 + (long long) g0 * TQ - span + 1 : 0;     // may be negative: zero margin in front of the cache
            const float * keys = cache + jlo * row;
            const long long sK = L.window > 0 ? (long long) TQ * row : 0;
            const long long grp = (long long) ng * M * nk;                                               // one (head group, map) of this group of tiles
            gemm_f32(c, c->QK + (size_t) g0 * M * D, D, (long long) M * D, keys, 0, row, sK, c->att_scores, nk, (long long) M * nk, M, nk, D, ng,
                     2 * G, (long long) Tpad * Rh * D, D, grp);
            const int rows = ng * M * G;
            k_diff_softmax_rows<<<(rows + 7) / 8, 256, 0, c->st>>>(c->att_scores, ng * M, G, Rh, TQ, nk, L.window, span, &c->d_step->st, L.scale, L.lambda, g0, T);
            gemm_f32(c, c->att_scores, nk, (long long) M * nk, keys + (size_t) G * 2 * D, 1, row, sK, c->OL + (size_t) g0 * M * V, V, (long long) M * V, M, V, nk, ng,
                     G, 2 * grp, V, (long long) Tpad * Rh * V);
            c->launches++;
        }
        k_diff_norm_out<<<dim3((unsigned) T, (unsigned) ((H + 3) / 4)), 128, 0, c->st>>>(c->OL, Tpad, H, G, V, c->m->eps, 1.0f - L.diff, c->A);
        c->launches += 2;
        linear(c, c->A, H * V, L.o, c->out, E, T);
        return;
    }
    const int TQ = T >= 4 ? 4 : T >= 2 ? 2 : 1, WPQ = 8 / TQ;
    // few queries: the keys of one query are spread over 8 / TQ warps and nsplit blocks until the grid fills the SMs
    const int blocks = ((T + TQ - 1) / TQ) * H, max_keys = L.window > 0 ? std::min(L.window, c->n_ctx) : c->n_ctx;
    const int nsplit = std::max(1, std::min({ 2 * c->sm_count / blocks, ((max_keys + 31) / 32 + WPQ - 1) / WPQ, DIFF_MAX_SPLIT }));
    DiffAttnArgs a{Q, ldq, cache, row, &c->d_step->st, c->A, T, H, G, D, V, L.window, L.scale, L.lambda, 1.0f - L.diff, c->m->eps, TQ,
                   (D % 4 == 0 && row % 4 == 0 && ((uintptr_t) cache & 15) == 0) ? 1 : 0, nsplit, c->da_part, c->da_counter};
    const dim3 grid((unsigned) ((T + TQ - 1) / TQ), (unsigned) H, (unsigned) nsplit);
    const size_t smem = diffattn_smem(L, TQ);
    if (V <= 32) k_diff_attn<1><<<grid, 256, smem, c->st>>>(a);
    else if (V <= 64) k_diff_attn<2><<<grid, 256, smem, c->st>>>(a);
    else if (V <= 128) k_diff_attn<4><<<grid, 256, smem, c->st>>>(a);
    else k_diff_attn<8><<<grid, 256, smem, c->st>>>(a);
    c->launches++;
    linear(c, c->A, H * V, L.o, c->out, E, T);
}

constexpr int RET_CHUNK_MIN_T = 128;      // shorter portions walk token by token
size_t retention_chunk_smem(int D) { return ((size_t) 2 * RC * (D + 4) + (size_t) RC * (RC + 4) + (size_t) RC * 128 + RC + 1) * 4; }
bool retention_chunks_enabled() {
    static const bool on = [] { const char * e = std::getenv("BOOSTER_B200_STACK_RET_CHUNKS"); return !(e && e[0] == '0'); }();
    return on;
}

template <int DMAX>
void launch_retention_scan(StackCtx * c, const LayerSpec & L, int T, int ldp, float * S) {
    // four lanes per column of the state; a head's columns are spread over blocks of >= 16 until the grid fills the SMs
    int ncols = std::min(128, (L.V + 7) / 8 * 8);
    while (ncols > 16 && L.H * ((L.V + ncols - 1) / ncols) < c->sm_count) ncols = (ncols / 2 + 7) / 8 * 8;
    const int HD = L.H * L.D;
    const dim3 grid((unsigned) L.H, (unsigned) ((L.V + ncols - 1) / ncols));
    k_retention_scan<DMAX><<<grid, GD_RG * ncols, 0, c->st>>>(c->P, ldp, 0, HD, 2 * HD, L.decay, T, L.H, L.D, L.V, S, c->O);
}

// retention: P[t] = [ q | k | v | gate ] -> rotation, key scale -> recurrence -> per-head unit norm, silu gate -> output product
void mixer_retention(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    const int E = c->m->E, H = L.H, D = L.D, V = L.V, HD = H * D, HV = H * V, ldp = L.proj.N;
    float * S = c->rec + R.off_rec;
    linear(c, c->in, E, L.proj, c->P, ldp, T);
    if (T == 1) {
        // one token: rotation, state update, read-out norm and gate in one launch, a block per head
        const RopeArgs rope{L.rope_freq, L.rope_dims, 1.0f};
        const int threads = GD_RG * std::min(128, (V + 7) / 8 * 8);
        const size_t sm = (size_t) V * 4;
        const StepState * st = &c->d_step->st;
        if (D <= 32) k_retention_token<32><<<H, threads, sm, c->st>>>(c->P, 0, HD, 2 * HD, 2 * HD + HV, L.decay, rope, L.k_scale, st, H, D, V, c->m->eps, S, c->A);
        else if (D <= 64) k_retention_token<64><<<H, threads, sm, c->st>>>(c->P, 0, HD, 2 * HD, 2 * HD + HV, L.decay, rope, L.k_scale, st, H, D, V, c->m->eps, S, c->A);
        else if (D <= 128) k_retention_token<128><<<H, threads, sm, c->st>>>(c->P, 0, HD, 2 * HD, 2 * HD + HV, L.decay, rope, L.k_scale, st, H, D, V, c->m->eps, S, c->A);
        else k_retention_token<256><<<H, threads, sm, c->st>>>(c->P, 0, HD, 2 * HD, 2 * HD + HV, L.decay, rope, L.k_scale, st, H, D, V, c->m->eps, S, c->A);
        c->launches++;
        linear(c, c->A, HV, L.o, c->out, E, T);
        return;
    }
    k_retention_prep<<<dim3((unsigned) T, (unsigned) ((2 * H + 3) / 4)), 128, 0, c->st>>>(c->P, ldp, 0, HD, H, D, RopeArgs{L.rope_freq, L.rope_dims, 1.0f}, L.k_scale, &c->d_step->st);
    if (T >= RET_CHUNK_MIN_T && c->ret_sb && retention_chunks_enabled()) {
        // long portions: per-chunk products in parallel, a short walk over the chunks in between
        const int nch = (T + RC - 1) / RC, vt = (V + 127) / 128;
        const dim3 grid((unsigned) H, (unsigned) nch, (unsigned) vt);
        const size_t sm = retention_chunk_smem(D);
        k_retention_chunk_kv<<<grid, 256, 0, c->st>>>(c->P, ldp, HD, 2 * HD, L.decay, T, H, D, V, c->ret_sb);
        k_retention_chunk_state<<<dim3((unsigned) H, (unsigned) ((D * V + 255) / 256)), 256, 0, c->st>>>(L.decay, T, D, V, nch, S, c->ret_sb);
        k_retention_chunk_out<<<grid, 128, sm, c->st>>>(c->P, ldp, 0, HD, 2 * HD, L.decay, T, H, D, V, c->ret_sb, c->O);
        c->launches += 2;
    }
    else if (D <= 32) launch_retention_scan<32>(c, L, T, ldp, S);
    else if (D <= 64) launch_retention_scan<64>(c, L, T, ldp, S);
    else if (D <= 128) launch_retention_scan<128>(c, L, T, ldp, S);
    else launch_retention_scan<256>(c, L, T, ldp, S);
    k_delta_out<<<dim3((unsigned) T, (unsigned) ((H + 3) / 4)), 128, 0, c->st>>>(c->O, c->P, ldp, 2 * HD + HV, H, V, nullptr, 0, 0, c->m->eps, c->A);
    c->launches += 3;
    linear(c, c->A, HV, L.o, c->out, E, T);
}

constexpr int SIG_MAX_SPLIT = 16;
int sig_vpl(const LayerSpec & L) { return L.V <= 32 ? 1 : L.V <= 64 ? 2 : L.V <= 128 ? 4 : 8; }

// sigmoid attention: P[t] = [ q | k | v ] -> norms, temperature; keys and values to the cache row of the token's position ->
// weights sigmoid(score - slope distance + offset) over all earlier positions -> output product
void mixer_sigattn(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    const int E = c->m->E, H = L.H, G = L.KH, D = L.D, V = L.V, nq = H * D, row = (int) L.cache_row;
    float * cache = c->caches[(size_t) R.cache_index];
    linear(c, c->in, E, L.proj, c->P, L.proj.N, T);
    k_sigattn_prep<<<T, 256, 0, c->st>>>(c->P, L.proj.N, H, G, D, V, L.qw, L.kw, c->m->eps, L.t_coef, L.t_every, &c->d_step->st, c->CV, cache);
    c->launches++;
    if (T >= 8) {
        // prompt portion: float32 products over tiles of ATT_TQ tokens, one batch entry per (tile, key/value head)
        const int TQ = ATT_TQ, Rh = H / G, M = TQ * Rh, ntile = (T + TQ - 1) / TQ, Tpad = ntile * TQ;
        const int pos0 = c->h_step->st.pos0;
        k_group_q_layout<<<Tpad, 256, 0, c->st>>>(c->CV, nq, T, Tpad, H, G, D, c->QK);
        const size_t nk_max = (size_t) (pos0 + Tpad + 3) / 4 * 4;
        const int per_group = (int) std::max<size_t>(1, c->att_scores_floats / ((size_t) G * M * nk_max));
        for (int g0 = 0; g0 < ntile; g0 += per_group) {
            const int ng = std::min(per_group, ntile - g0);
            const int nk = (pos0 + (g0 + ng) * TQ + 3) / 4 * 4;                                           // no key beyond this group's last token is seen
            const long long grp = (long long) ng * M * nk;
            gemm_f32(c, c->QK + (size_t) g0 * M * D, D, (long long) M * D, cache, 0, row, 0, c->att_scores, nk, (long long) M * nk, M, nk, D, ng,
                     G, (long long) Tpad * Rh * D, D, grp);
            const int rows = ng * M * G;
            k_sig_weight_rows<<<(rows + 7) / 8, 256, 0, c->st>>>(c->att_scores, ng * M, G, Rh, TQ, nk, &c->d_step->st, L.scale, L.slope, L.pb, g0, T);
            gemm_f32(c, c->att_scores, nk, (long long) M * nk, cache + (size_t) G * D, 1, row, 0, c->OL + (size_t) g0 * M * V, V, (long long) M * V, M, V, nk, ng,
                     G, grp, V, (long long) Tpad * Rh * V);
            c->launches++;
        }
        k_group_o_layout<<<T, 256, 0, c->st>>>(c->OL, Tpad, H, G, V, c->A);
        c->launches += 2;
        linear(c, c->A, H * V, L.o, c->out, E, T);
        return;
    }
    const int TQ = T >= 4 ? 4 : T >= 2 ? 2 : 1, WPQ = 8 / TQ;
    const int blocks = ((T + TQ - 1) / TQ) * H;
    const int nsplit = std::max(1, std::min({ 2 * c->sm_count / blocks, ((c->n_ctx + 31) / 32 + WPQ - 1) / WPQ, SIG_MAX_SPLIT }));
    SigAttnArgs a{c->CV, nq, cache, row, &c->d_step->st, c->A, L.slope, L.pb, T, H, G, D, V, L.scale, TQ,
                  (D % 4 == 0 && row % 4 == 0 && ((uintptr_t) cache & 15) == 0) ? 1 : 0, nsplit, c->da_part, c->da_counter};
    const dim3 grid((unsigned) ((T + TQ - 1) / TQ), (unsigned) H, (unsigned) nsplit);
    const int VPL = sig_vpl(L);
    const size_t smem = ((size_t) TQ * D + (size_t) 8 * 32 * VPL) * 4;
    if (VPL == 1) k_sig_attn<1><<<grid, 256, smem, c->st>>>(a);
    else if (VPL == 2) k_sig_attn<2><<<grid, 256, smem, c->st>>>(a);
    else if (VPL == 4) k_sig_attn<4><<<grid, 256, smem, c->st>>>(a);
    else k_sig_attn<8><<<grid, 256, smem, c->st>>>(a);
    c->launches++;
    linear(c, c->A, H * V, L.o, c->out, E, T);
}

constexpr int GQA_MAX_SPLIT = 16;
int gqa_vpl(const LayerSpec & L) { return L.V <= 32 ? 1 : L.V <= 64 ? 2 : L.V <= 128 ? 4 : 8; }
bool gqa_tiles_enabled() {
    static const bool on = [] { const char * e = std::getenv("BOOSTER_B200_STACK_GQA_TILES"); return !(e && e[0] == '0'); }();
    return on;
}

// soft-max attention over grouped heads: P[t] = [ q | k | v | head gates ] -> per-head norms, rotation, value mixing; keys and
// values to the cache row of the token's position (and the means of the blocks this step completes to the pool) -> attention
// under the layer's mask -> gate -> output product
void mixer_gqattn(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    const int E = c->m->E, H = L.H, G = L.KH, D = L.D, V = L.V, nq = H * D, row = (int) L.cache_row, ldp = L.proj.N;
    float * cache = c->caches[(size_t) R.cache_index], * pool = c->pools[(size_t) R.cache_index];
    const StepState * st = &c->d_step->st;
    linear(c, c->in, E, L.proj, c->P, ldp, T);
    const GqaPrepArgs pa{c->P, ldp, H, G, D, V, L.qw, L.kw, c->m->eps, RopeArgs{L.rope_freq, L.rope_dims, 1.0f, L.rope_adjacent ? 1 : 0}, st, c->CV, cache, row,
                         c->VF, L.vmode, L.vlambda};
    k_gqa_prep<<<dim3((unsigned) T, T <= 16 ? (unsigned) ((H + G + 7) / 8) : 1u), 256, 0, c->st>>>(pa);      // few tokens: a token's heads over several blocks
    c->launches++;
    if (L.pool > 0) { k_pool_rows<<<dim3((unsigned) (T / L.pool + 1), (unsigned) ((row + 127) / 128)), 128, 0, c->st>>>(cache, row, pool, L.pool, st); c->launches++; }
    const float * gate = L.head_gate ? c->P + nq + row : nullptr;
    const GqaMask mask{L.mask_kind, L.window, L.pool};
    const GqaScore sc{L.scale, L.cap};
    if (T >= 8 && gqa_tiles_enabled()) {
        // prompt portion: float32 products over tiles of ATT_TQ tokens, one batch entry per (tile, key/value head). A row's columns
        // are [ block means | tokens ]; the token columns of a masked layer start `span` - 1 positions before the tile
        const int TQ = ATT_TQ, Rh = H / G, M = TQ * Rh, ntile = (T + TQ - 1) / TQ, Tpad = ntile * TQ;
        const int pos0 = c->h_step->st.pos0;
        k_group_q_layout<<<Tpad, 256, 0, c->st>>>(c->CV, nq, T, Tpad, H, G, D, c->QK);
        const bool masked = L.mask_kind != MASK_CAUSAL;
        const int span = masked ? std::min(L.window, pos0 + Tpad) : 0;
        const size_t nk_max = (size_t) ((masked ? span + TQ - 1 : pos0 + Tpad) + 3) / 4 * 4;
        const int npc_max = (gqa_blocks_seen(mask, pos0 + T - 1) + 3) / 4 * 4;
        const int per_group = (int) std::max<size_t>(1, c->att_scores_floats / ((size_t) G * M * (nk_max + npc_max)));
        for (int g0 = 0; g0 < ntile; g0 += per_group) {
            const int ng = std::min(per_group, ntile - g0);
            const int nk = masked ? (int) nk_max : (pos0 + (g0 + ng) * TQ + 3) / 4 * 4;           // unmasked: no key beyond this group's last token is seen
            const int npc = (gqa_blocks_seen(mask, pos0 + std::min(T, (g0 + ng) * TQ) - 1) + 3) / 4 * 4, ld = npc + nk;
            const long long jlo = masked ? (long long) pos0 + (long long) g0 * TQ - span + 1 : 0; // may be negative: zero margin in front of the cache
            const float * keys = cache + jlo * row;
            const long long sK = masked ? (long long) TQ * row : 0;
            const long long grp = (long long) ng * M * ld;
            gemm_f32(c, c->QK + (size_t) g0 * M * D, D, (long long) M * D, keys, 0, row, sK, c->att_scores + npc, ld, (long long) M * ld, M, nk, D, ng,
                     G, (long long) Tpad * Rh * D, D, grp);
            if (npc) gemm_f32(c, c->QK + (size_t) g0 * M * D, D, (long long) M * D, pool, 0, row, 0, c->att_scores, ld, (long long) M * ld, M, npc, D, ng,
                              G, (long long) Tpad * Rh * D, D, grp);
            const int rows = ng * M * G;
            k_gqa_softmax_rows<<<(rows + 7) / 8, 256, 0, c->st>>>(c->att_scores, ng * M, G, Rh, TQ, npc, nk, span, mask, sc, L.r1, L.r2, L.sink, st, g0, T);
            gemm_f32(c, c->att_scores + npc, ld, (long long) M * ld, keys + (size_t) G * D, 1, row, sK, c->OL + (size_t) g0 * M * V, V, (long long) M * V, M, V, nk, ng,
                     G, grp, V, (long long) Tpad * Rh * V);
            if (npc) gemm_f32(c, c->att_scores, ld, (long long) M * ld, pool + (size_t) G * D, 1, row, 0, c->OL + (size_t) g0 * M * V, V, (long long) M * V, M, V, npc, ng,
                              G, grp, V, (long long) Tpad * Rh * V, 1);
            c->launches++;
        }
        k_group_o_layout<<<T, 256, 0, c->st>>>(c->OL, Tpad, H, G, V, c->A, gate, ldp);      // the head gates ride on the regrouping
        c->launches += 2;
        linear(c, c->A, H * V, L.o, c->out, E, T);
        return;
    }
    const int TQ = T >= 4 ? 4 : T >= 2 ? 2 : 1, WPQ = 8 / TQ;
    const int blocks = ((T + TQ - 1) / TQ) * H;
    const int max_keys = L.mask_kind == MASK_CAUSAL ? c->n_ctx : std::min(c->n_ctx, L.window + (L.pool > 0 ? c->n_ctx / L.pool : 0));
    const int nsplit = std::max(1, std::min({ 2 * c->sm_count / blocks, ((max_keys + 31) / 32 + WPQ - 1) / WPQ, GQA_MAX_SPLIT }));
    const GqaAttnArgs a{c->CV, nq, cache, pool, row, st, c->A, L.r1, L.r2, L.sink, gate, ldp, T, H, G, D, V, sc, mask, TQ,
                        (D % 4 == 0 && row % 4 == 0 && ((uintptr_t) cache & 15) == 0 && ((uintptr_t) pool & 15) == 0) ? 1 : 0, nsplit, c->da_part, c->da_counter};
    const dim3 grid((unsigned) ((T + TQ - 1) / TQ), (unsigned) H, (unsigned) nsplit);
    const int VPL = gqa_vpl(L);
    const size_t smem = ((size_t) TQ * D + (size_t) 8 * (2 + 32 * VPL)) * 4;
    if (VPL == 1) k_gqa_attn<1><<<grid, 256, smem, c->st>>>(a);
    else if (VPL == 2) k_gqa_attn<2><<<grid, 256, smem, c->st>>>(a);
    else if (VPL == 4) k_gqa_attn<4><<<grid, 256, smem, c->st>>>(a);
    else k_gqa_attn<8><<<grid, 256, smem, c->st>>>(a);
    c->launches++;
    linear(c, c->A, H * V, L.o, c->out, E, T);
}

void tap_layer(StackCtx * c, size_t ri, int T) {
    const size_t E = (size_t) c->m->E, n = (size_t) T * E;
    SCU(cudaMemcpyAsync(c->tap_data.data() + ri * n, c->X, n * 4, cudaMemcpyDeviceToHost, c->st));
}

void run_mixer(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T);
// two mixers on the same input: the first leaves its output in c->out, the second in c->Y2 (the layer's join norms and averages them)
void mixer_pair(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    float * out = c->out;
    RunSpec B = R;
    for (size_t i = 0; i < L.parts.size(); i++) {
        const LayerSpec & P = L.parts[i];
        c->out = i == 0 ? out : c->Y2;
        run_mixer(c, P, B, T);
        B.off_rec += (P.n_rec + 3) / 4 * 4;
        if (P.cache_row) B.cache_index++;
    }
    c->out = out;
}

void run_mixer(StackCtx * c, const LayerSpec & L, const RunSpec & R, int T) {
    switch (L.kind) {
        case MIX_RETENTION: mixer_retention(c, L, R, T); break;
        case MIX_SIGATTN:   mixer_sigattn(c, L, R, T); break;
        case MIX_PAIR:      mixer_pair(c, L, R, T); break;
        case MIX_GQATTN:    mixer_gqattn(c, L, R, T); break;
        case MIX_MINGRU:   mixer_mingru(c, L, R, T); break;
        case MIX_LATENT:   mixer_latent(c, L, R, T); break;
        case MIX_DELTA:    mixer_delta(c, L, R, T); break;
        case MIX_GDELTA:   mixer_gdelta(c, L, R, T); break;
        default:           mixer_diffattn(c, L, R, T); break;
    }
}

// sequential blocks: x += n1b(mixer(n1 x)); x += n2b(ff(n2 x))
void enqueue_layers_sequential(StackCtx * c, int T) {
    StackModel & m = *c->m;
    const int E = m.E;
    const int nthreads = std::min(256, std::max(128, 32 * m.groups));
    const float * w0 = m.layers[(size_t) m.runs[0].layer].norm1;
    if (m.dtype == STACK_F32) k_embed_rows<float><<<T, nthreads, 0, c->st>>>((const float *) m.embed, c->d_step->tokens, E, m.vocab, c->X, w0, m.groups, m.eps, c->Hn);
    else k_embed_rows<__nv_bfloat16><<<T, nthreads, 0, c->st>>>((const __nv_bfloat16 *) m.embed, c->d_step->tokens, E, m.vocab, c->X, w0, m.groups, m.eps, c->Hn);
    c->launches++;
    c->in = c->Hn; c->out = c->Y;
    for (size_t ri = 0; ri < m.runs.size(); ri++) {
        const RunSpec & R = m.runs[ri];
        const LayerSpec & L = m.layers[(size_t) R.layer];
        const float * next_in = ri + 1 < m.runs.size() ? m.layers[(size_t) m.runs[ri + 1].layer].norm1 : nullptr;     // the final norm runs on the wanted rows only
        run_mixer(c, L, R, T);                         // Hn holds norm1(x)
        post_norm_add(c, L.norm1b, L.has_mlp ? L.norm2 : next_in, T);
        if (L.has_mlp) {
            linear(c, c->Hn, E, L.gateup, c->A, L.ff, T, 1, 0, 0, true, L.limit);      // clamped gated unit in the epilogue
            linear(c, c->A, L.ff, L.down, c->Y, E, T);
            post_norm_add(c, L.norm2b, next_in, T);
        }
        if (c->taps) tap_layer(c, ri, T);
    }
    SCU(cudaGetLastError());
}

// parallel blocks: x += mixer(u1) + ff(u2), u_i = h_i + conv_i(h_i), h_i = n_i(x). The sum of a layer's two outputs is folded
// into the kernel that norms the next layer's inputs (k_add_norm2) unless a pass of the repeated span begins in between.
void enqueue_layers_parallel(StackCtx * c, int T) {
    StackModel & m = *c->m;
    const int E = m.E, ct = m.canon_taps;
    const size_t plane = (size_t) c->cap * E;
    const bool looped = m.loop_step != nullptr;
    if (m.dtype == STACK_F32) k_embed_plain<float><<<T, 128, 0, c->st>>>((const float *) m.embed, c->d_step->tokens, E, m.vocab, c->X, looped ? c->XC + E : nullptr, 2 * E);
    else k_embed_plain<__nv_bfloat16><<<T, 128, 0, c->st>>>((const __nv_bfloat16 *) m.embed, c->d_step->tokens, E, m.vocab, c->X, looped ? c->XC + E : nullptr, 2 * E);
    c->launches++;
    const float * ya = nullptr, * yb = nullptr;        // outputs of the layer before, not yet added to X
    for (size_t ri = 0; ri < m.runs.size(); ri++) {
        const RunSpec & R = m.runs[ri];
        const LayerSpec & L = m.layers[(size_t) R.layer];
        float * H1 = c->Hn, * H2 = c->Hn + plane;
        if (R.pass >= 0) {
            // x <- W_in [x; x0] + step[pass]: the finished x goes to the left half of XC (x0 is in the right half since the embedding)
            k_add_norm2<<<T, 256, 0, c->st>>>(c->X, ya, yb, c->XC, 2 * E, nullptr, nullptr, nullptr, nullptr, E, m.eps);
            c->launches++;
            ya = yb = nullptr;
            DMat w = m.loop_in;
            w.bias = m.loop_step + (size_t) R.pass * E;
            linear(c, c->XC, 2 * E, w, c->X, E, T);
        }
        const int nsub = L.has_mlp ? 2 : 1;
        const float * u1 = H1, * u2 = H2;
        float * hist = c->rec + R.off_rec + (L.n_rec - (size_t) nsub * std::max(ct - 1, 0) * E);
        if (T == 1 && ct > 0) {                        // one token: sum, both norms, both input convolutions and their history in one launch
            k_add_norm2_canon1<<<CANON1_CTAS, 256, 0, c->st>>>(c->X, ya, yb, L.norm1, L.has_mlp ? L.norm2 : nullptr, L.canon, hist, c->U, (long long) plane, E, ct, m.eps);
            c->launches++;
            u1 = c->U; u2 = c->U + plane;
        } else {
            k_add_norm2<<<T, 256, 0, c->st>>>(c->X, ya, yb, nullptr, 0, L.norm1, L.has_mlp ? L.norm2 : nullptr, H1, H2, E, m.eps);
            c->launches++;
        }
        if (ct > 0 && T > 1) {
            causal_conv(c, ConvArgs{c->Hn, E, (long long) plane, L.canon, (long long) E * ct, hist, (long long) (ct - 1) * E, c->U, E, (long long) plane,
                                    T, E, ct, 0, 1, nullptr, nullptr, 0, 0, 0}, nsub);
            u1 = c->U; u2 = c->U + plane;
        }
        c->in = u1; c->out = c->Y;
        run_mixer(c, L, R, T);
        ya = c->Y; yb = nullptr;
        if (L.has_mlp) {
            linear(c, u2, E, L.gateup, c->A, L.ff, T);
            k_polynorm<<<T, 256, 0, c->st>>>(c->A, L.ff, L.act, m.eps);
            c->launches++;
            linear(c, c->A, L.ff, L.down, c->Y2, E, T);
            yb = c->Y2;
        }
        if (c->taps || ri + 1 == m.runs.size()) {      // the residual stream itself is wanted now
            k_add_norm2<<<T, 256, 0, c->st>>>(c->X, ya, yb, nullptr, 0, nullptr, nullptr, nullptr, nullptr, E, m.eps);
            c->launches++;
            ya = yb = nullptr;
            if (c->taps) tap_layer(c, ri, T);
        }
    }
    SCU(cudaGetLastError());
}

// routed mixture on c->Hn (a design whose experts run on the weighted input gets outputs that are added as they are): the chosen experts' outputs by slot in c->Yk (slot order in *slot_of: nullptr = t top + k), the
// shared unit's in c->Y; the layer's join weighs and adds them
void mixture_ff(StackCtx * c, const LayerSpec & L, int T, const int32_t ** slot_of) {
    const int E = c->m->E, top = L.top, ff = L.e_ff, slots = T * top;
    const RouteArgs ra{c->Hn, E, E, L.router, L.w_sg, L.n_exp, top, L.n_groups, L.keep_groups, L.r_scale, c->r_sel, c->r_wt, c->r_sg, c->r_z, c->r_counter, L.route_fn, T <= 16 ? 8 : 1};
    k_moe_route<<<dim3((unsigned) T, (unsigned) ((L.n_exp + (L.w_sg ? 1 : 0) + 8 / ra.wpr - 1) / (8 / ra.wpr))), 256, (size_t) (2 * L.n_exp + L.n_groups) * 4, c->st>>>(ra);
    c->launches++;
    LinOpt o;
    o.alpha = 1.f; o.shift = 0.f;               // silu(gate) * up, no clamp
    if (T <= GEMV_MAX_T) {
        // few tokens: one mat-vec per (token, choice) against the chosen expert's matrices
        o.w_index = c->r_sel; o.x_share = top;
        if (L.scale_input) o.x_scale = c->r_wt;     // W (w h) = w (W h): the weight meets the products before the gated unit
        linear(c, c->Hn, E, L.e_gateup, c->Ap, ff, 1, slots, E, ff, true, INFINITY, &o);
        o.x_share = 1; o.x_scale = nullptr;
        linear(c, c->Ap, ff, L.e_down, c->Yk, E, 1, slots, ff, E, false, 0.f, &o);
        *slot_of = nullptr;
    } else {
        // prompt portion: rows sorted by expert, one segmented product per projection
        int tpe = 1;
        while (tpe * 2 * L.n_exp <= 1024 && tpe * 2 <= slots) tpe *= 2;
        const size_t cnt_bytes = (size_t) L.n_exp * tpe * 4;
        const int in_smem = (size_t) slots * 4 + cnt_bytes <= 40 * 1024 ? 1 : 0;
        k_moe_sort<<<1, 1024, cnt_bytes + (in_smem ? (size_t) slots * 4 : 0), c->st>>>(c->r_sel, slots, top, L.n_exp, tpe, in_smem, c->r_seg, c->r_slot, c->r_src);
        if (L.scale_input) k_spread_rows<<<slots, 128, 0, c->st>>>(c->Hn, E, c->r_slot, c->r_wt, top, E, c->Xp);
        else k_gather_rows<<<slots, 128, 0, c->st>>>(c->Hn, E, c->r_src, E, c->Xp);
        c->launches += 2;
        o.seg = c->r_seg;
        linear(c, c->Xp, E, L.e_gateup, c->Ap, ff, slots, L.n_exp, 0, 0, true, INFINITY, &o);
        linear(c, c->Ap, ff, L.e_down, c->Yk, E, slots, L.n_exp, 0, 0, false, 0.f, &o);
        *slot_of = c->r_slot;
    }
    if (L.ff > 0) {
        LinOpt s;
        s.alpha = 1.f; s.shift = 0.f;
        linear(c, c->Hn, E, L.gateup, c->A, L.ff, T, 1, 0, 0, true, INFINITY, &s);
        linear(c, c->A, L.ff, L.down, c->Y, E, T);
    }
}

// pre-norm blocks with element-wise norms: y = z + mixer(dyt1 z); y += ff(dyt2 y); the next layer reads the depth average of
// the embedding output and all layers' y so far. Every sub-layer ends in one k_join launch that also norms the next one's input.
void enqueue_layers_prenorm(StackCtx * c, int T) {
    StackModel & m = *c->m;
    const int E = m.E;
    const long long plane = (long long) c->cap * E;
    const dim3 jgrid((unsigned) T, (unsigned) ((E + JOIN_SLICE - 1) / JOIN_SLICE));
    {
        const LayerSpec & L0 = m.layers[(size_t) m.runs[0].layer];
        const DytW ne{m.embed_w, m.embed_b, m.embed_alpha}, n1{L0.norm1, L0.n1_b, L0.n1_alpha};
        if (m.dtype == STACK_F32) k_embed_dyt<float><<<T, 256, 0, c->st>>>((const float *) m.embed, c->d_step->tokens, E, m.vocab, ne, n1, c->X, m.depth_avg ? c->keep : nullptr, c->Hn);
        else k_embed_dyt<__nv_bfloat16><<<T, 256, 0, c->st>>>((const __nv_bfloat16 *) m.embed, c->d_step->tokens, E, m.vocab, ne, n1, c->X, m.depth_avg ? c->keep : nullptr, c->Hn);
        c->launches++;
    }
    for (size_t ri = 0; ri < m.runs.size(); ri++) {
        const RunSpec & R = m.runs[ri];
        const LayerSpec & L = m.layers[(size_t) R.layer];
        const LayerSpec * N = ri + 1 < m.runs.size() ? &m.layers[(size_t) m.runs[ri + 1].layer] : nullptr;      // the final norm runs on the wanted rows only
        c->in = c->Hn; c->out = c->Y;
        run_mixer(c, L, R, T);
        JoinArgs j{};
        j.X = c->X; j.E = E; j.eps = m.eps; j.Ya = c->Y;
        if (L.kind == MIX_PAIR) { j.Yb = c->Y2; j.wa = L.pair_w[0]; j.wb = L.pair_w[1]; }
        const auto layer_end = [&](JoinArgs & a) {
            if (m.depth_avg) { a.keep = c->keep; a.plane = plane; a.coef = L.dwa; a.n_keep = L.n_dwa; }
            if (N) { a.nw = N->norm1; a.nb = N->n1_b; a.alpha = N->n1_alpha; a.Hn = c->Hn; }
        };
        if (L.has_mlp) { j.nw = L.norm2; j.nb = L.n2_b; j.alpha = L.n2_alpha; j.Hn = c->Hn; } else layer_end(j);
        k_join<<<jgrid, 256, 0, c->st>>>(j);
        c->launches++;
        if (L.has_mlp) {
            JoinArgs f{};
            f.X = c->X; f.E = E; f.eps = m.eps;
            mixture_ff(c, L, T, &f.slot_of);
            f.Yk = c->Yk; f.wt = c->r_wt; f.top = L.top;
            if (L.ff > 0) { f.Ysh = c->Y; f.sg = c->r_sg; }
            layer_end(f);
            k_join<<<jgrid, 256, 0, c->st>>>(f);
            c->launches++;
        }
        if (c->taps) tap_layer(c, ri, T);
    }
    SCU(cudaGetLastError());
}

// hyper-connected blocks: the residual is m.streams rows per token; every sub-layer ends in one k_hc_join launch that writes all
// streams and norms the read-in of the sub-layer that follows; the last one leaves the model's norm of the sum of the streams in
// c->Hn for the head. c->X gets the sum of the streams when the residual after a layer is tapped.
void enqueue_layers_hyper(StackCtx * c, int T) {
    StackModel & m = *c->m;
    const int E = m.E, S = m.streams;
    const long long plane = (long long) c->cap * E;
    {
        const LayerSpec & L0 = m.layers[(size_t) m.runs[0].layer];
        if (m.dtype == STACK_F32) k_hc_embed<float><<<T, hc_threads(T, E), 0, c->st>>>((const float *) m.embed, c->d_step->tokens, E, m.vocab, S, c->XS, plane, L0.hc[0], L0.g1, m.eps, c->Hn);
        else k_hc_embed<__nv_bfloat16><<<T, hc_threads(T, E), 0, c->st>>>((const __nv_bfloat16 *) m.embed, c->d_step->tokens, E, m.vocab, S, c->XS, plane, L0.hc[0], L0.g1, m.eps, c->Hn);
        c->launches++;
    }
    for (size_t ri = 0; ri < m.runs.size(); ri++) {
        const RunSpec & R = m.runs[ri];
        const LayerSpec & L = m.layers[(size_t) R.layer];
        const LayerSpec * N = ri + 1 < m.runs.size() ? &m.layers[(size_t) m.runs[ri + 1].layer] : nullptr;      // the final norm runs on the wanted rows only
        const auto join = [&](int q, HcJoinArgs & j) {
            j.XS = c->XS; j.plane = plane; j.S = S; j.E = E; j.eps = m.eps;
            j.w = L.hc[q];
            const bool last_sub = q == 1 || !L.has_mlp;
            const HcW * nw = !last_sub ? &L.hc[1] : N ? &N->hc[0] : nullptr;
            if (nw) { for (int s = 0; s < HC_MAX; s++) j.nin[s] = nw->in[s]; j.g = !last_sub ? L.g2 : N->g1; j.Hn = c->Hn; }
            else { for (int s = 0; s < S; s++) j.nin[s] = 1.f; j.g = m.final_g; j.Hn = c->Hn; }      // after the last layer: the model's norm of the sum of the streams
            if (last_sub && c->taps) j.Xsum = c->X;
            if (E % 4 == 0) k_hc_join<4><<<T, hc_threads(T, E, 4, 512), 0, c->st>>>(j);      // every buffer of a context is 16-byte aligned and its rows are E floats apart
            else k_hc_join<1><<<T, hc_threads(T, E), 0, c->st>>>(j);
            c->launches++;
        };
        c->in = c->Hn; c->out = c->Y;
        run_mixer(c, L, R, T);
        HcJoinArgs j{};
        j.Ya = c->Y;
        join(0, j);
        if (L.has_mlp) {
            HcJoinArgs f{};
            mixture_ff(c, L, T, &f.slot_of);
            f.Yk = c->Yk; f.top = L.top;
            if (L.ff > 0) f.Ya = c->Y;
            join(1, f);
        }
        if (c->taps) tap_layer(c, ri, T);
    }
    SCU(cudaGetLastError());
}

// the layers over the T tokens whose header (positions, ids) is already on the device
void enqueue_layers(StackCtx * c, int T) {
    if (c->m->block == BLOCK_PARALLEL) enqueue_layers_parallel(c, T);
    else if (c->m->block == BLOCK_PRENORM) enqueue_layers_prenorm(c, T);
    else if (c->m->block == BLOCK_HYPER) enqueue_layers_hyper(c, T);
    else enqueue_layers_sequential(c, T);
}

// final norm + head on n_rows rows of the pass (row indices in d_step->rows) -> d_logits[row_off ..]
void enqueue_head(StackCtx * c, int n_rows, int64_t row_off, bool one_token = false) {
    StackModel & m = *c->m;
    if (m.block == BLOCK_HYPER) {
        // the last join left the normed sum of the streams in Hn for every row of the pass: the wanted rows are gathered for the head
        const float * hn = c->Hn;
        if (!one_token) { k_gather_rows<<<n_rows, 128, 0, c->st>>>(c->Hn, m.E, c->d_step->rows, m.E, c->Y); c->launches++; hn = c->Y; }
        linear(c, hn, m.E, m.head, c->d_logits + row_off * m.vocab, m.vocab, n_rows);
        return;
    }
    if (m.dyt) { k_dyt_rows<<<n_rows, 256, 0, c->st>>>(c->X, m.E, c->d_step->rows, DytW{m.final_norm, m.final_b, m.final_alpha}, m.E, c->Hn, m.E); c->launches++; }
    else norm(c, c->X, m.E, c->d_step->rows, m.final_norm, m.E, m.groups, c->Hn, m.E, n_rows, false);
    linear(c, c->Hn, m.E, m.head, c->d_logits + row_off * m.vocab, m.vocab, n_rows);
    if (m.softcap > 0.f) {
        const size_t n = (size_t) n_rows * m.vocab;
        k_softcap<<<(unsigned) ((n + 255) / 256), 256, 0, c->st>>>(c->d_logits + row_off * m.vocab, n, m.softcap);
        c->launches++;
    }
}

void ensure_logit_rows(StackCtx * c, int64_t rows) {
    if (rows <= c->logit_rows_cap) return;
    SCU(cudaStreamSynchronize(c->st));
    const int64_t cap = std::max<int64_t>(rows, 16);
    float * d = nullptr, * h = nullptr;
    SCU(cudaMalloc(&d, (size_t) cap * c->m->vocab * 4));
    if (cudaMallocHost(&h, (size_t) cap * c->m->vocab * 4) != cudaSuccess) { cudaFree(d); throw std::runtime_error("out of pinned host memory for the logits"); }
    cudaFree(c->d_logits);
    cudaFreeHost(c->h_logits);
    c->d_logits = d; c->h_logits = h; c->logit_rows_cap = cap;
    c->h_last = nullptr; c->d_last_row = -1;
    if (c->g_token) { cudaGraphExecDestroy(c->g_token); c->g_token = nullptr; }      // they hold the old addresses
    if (c->g_greedy) { cudaGraphExecDestroy(c->g_greedy); c->g_greedy = nullptr; }
}

bool graph_enabled() {
    static const bool on = [] { const char * e = std::getenv("BOOSTER_B200_STACK_GRAPH"); return !(e && e[0] == '0'); }();
    return on;
}

// one token: header in, layers, head, logits out — the body of the replayed graph and of its un-captured twin
void enqueue_token_step(StackCtx * c) {
    SCU(cudaMemcpyAsync(c->d_step, c->h_step, sizeof(StepState) + sizeof(int32_t), cudaMemcpyHostToDevice, c->st));
    SCU(cudaMemsetAsync(c->d_step->rows, 0, sizeof(int32_t), c->st));      // the wanted row is the token itself (a prompt pass leaves its own rows here)
    enqueue_layers(c, 1);
    enqueue_head(c, 1, 0, true);
    SCU(cudaMemcpyAsync(c->h_logits, c->d_logits, (size_t) c->m->vocab * 4, cudaMemcpyDeviceToHost, c->st));
}

}  // namespace

// ---- public ------------------------------------------------------------------------------------------------------------
bool stack_knows(const std::string & architecture) {
    for (const DesignEntry & d : DESIGNS) if (architecture == d.name) return true;
    return false;
}

void stack_model_free(StackModel * m) {
    if (!m) return;
    cudaSetDevice(m->device);
    for (void * p : m->allocs) cudaFree(p);
    delete m;
}

StackModel * stack_model_load(const std::string & dir, int device, int dtype) {
    const Json cfg = json_parse_file(dir + "/config.json");
    const std::string arch = cfg.string("architecture", "");
    const DesignEntry * de = nullptr;
    for (const DesignEntry & d : DESIGNS) if (arch == d.name) de = &d;
    if (!de) throw std::runtime_error("unsupported architecture '" + arch + "' in " + dir + "/config.json");
    safetensors_file sf;
    sf.open(dir + "/model.safetensors");
    std::unique_ptr<StackModel> m(new StackModel());
    m->device = device; m->dtype = dtype; m->design = arch;
    SCU(cudaSetDevice(device));
    try {
        de->build(*m, cfg, sf);
    } catch (...) {
        stack_model_free(m.release());
        cudaGetLastError();
        throw;
    }
    return m.release();
}

void stack_model_info(const StackModel * m, int32_t info[16]) {
    std::memset(info, 0, sizeof(int32_t) * 16);
    info[0] = m->vocab; info[1] = m->E; info[2] = (int32_t) m->layers.size();
    for (const LayerSpec & L : m->layers) {
        if (L.H && !info[3]) { info[3] = L.H; info[4] = L.KH ? L.KH : 1; info[6] = L.D + L.R; }
        if (L.has_mlp && !info[5]) info[5] = L.ff;
    }
    info[8] = 0; info[9] = (int32_t) m->layers.size(); info[10] = m->dtype == STACK_F32 ? 0 : 32;   // ggml file types: 0 all F32, 32 BF16
}
int64_t stack_model_weight_bytes(const StackModel * m) { return m->weight_bytes; }
int stack_model_device(const StackModel * m) { return m->device; }
int stack_model_n_vocab(const StackModel * m) { return m->vocab; }

void stack_ctx_free(StackCtx * c) {
    if (!c) return;
    cudaSetDevice(c->m->device);
    if (c->st) cudaStreamSynchronize(c->st);
    if (c->g_token) cudaGraphExecDestroy(c->g_token);
    if (c->g_greedy) cudaGraphExecDestroy(c->g_greedy);
    cudaFree(c->d_out_tokens); cudaFree(c->d_counter);
    for (float * p : c->pools) cudaFree(p);
    for (float * p : { c->XS, c->VF }) cudaFree(p);
    for (float * p : { c->Y2, c->U, c->XC, c->keep, c->ret_sb, c->Xp, c->Ap, c->Yk, c->r_wt, c->r_sg, c->r_z }) cudaFree(p);
    cudaFree(c->r_counter);
    for (int32_t * p : { c->r_sel, c->r_slot, c->r_src, c->r_seg }) cudaFree(p);
    for (float * p : { c->X, c->Hn, c->Y, c->P, c->A, c->QK, c->OL, c->CV, c->BG, c->O, c->rec, c->d_logits }) cudaFree(p);
    for (float * p : c->cache_allocs) cudaFree(p);
    cudaFree(c->att_scores); cudaFree(c->da_part); cudaFree(c->da_counter);
    cudaFree(c->xb); cudaFree(c->d_err); cudaFreeHost(c->h_err);
    cudaFree(c->d_step); cudaFree(c->d_arg); cudaFree(c->att_part); cudaFree(c->att_ml);
    cudaFreeHost(c->h_step); cudaFreeHost(c->h_logits); cudaFreeHost(c->h_arg);
    if (c->ev0) { cudaEventDestroy(c->ev0); cudaEventDestroy(c->ev1); }
    if (c->st) cudaStreamDestroy(c->st);
    delete c;
}

StackCtx * stack_ctx_new(StackModel * m, int n_ctx) {
    if (n_ctx <= 0) throw std::runtime_error("n_ctx must be positive (this model names no trained context length)");
    std::unique_ptr<StackCtx> c(new StackCtx());
    c->m = m; c->n_ctx = n_ctx; c->cap = std::min(n_ctx, CHUNK_MAX);
    SCU(cudaSetDevice(m->device));
    try {
        SCU(cudaStreamCreateWithFlags(&c->st, cudaStreamNonBlocking));
        const size_t cap = (size_t) c->cap;
        // zero-filled: rows that a tile computes beyond the portion, and cached rows no token has written, must hold finite numbers
        const auto fl = [&](float ** p, size_t n) { SCU(cudaMalloc(p, std::max<size_t>(n, 4) * 4)); SCU(cudaMemsetAsync(*p, 0, std::max<size_t>(n, 4) * 4, c->st)); };
        const size_t cap_t = (cap + ATT_TQ - 1) / ATT_TQ * ATT_TQ;
        const bool par = m->block == BLOCK_PARALLEL;
        fl(&c->X, cap * m->E); fl(&c->Hn, cap * m->E * (par ? 2 : 1)); fl(&c->Y, cap * m->E);
        if (par) { fl(&c->Y2, cap * m->E); fl(&c->U, cap * m->E * 2); fl(&c->XC, cap * m->E * 2); }
        else if (m->has_pair) fl(&c->Y2, cap * m->E);
        if (m->depth_avg) fl(&c->keep, (m->layers.size() + 1) * cap * m->E);
        if (m->block == BLOCK_HYPER) fl(&c->XS, (size_t) m->streams * cap * m->E);
        if (m->vfirst_width > 0) fl(&c->VF, cap * (size_t) m->vfirst_width);
        if (m->max_ret_state > 0 && c->cap >= RET_CHUNK_MIN_T) {
            fl(&c->ret_sb, (size_t) ((c->cap + RC - 1) / RC) * m->max_ret_state);
            static size_t attr = 48 * 1024;
            const size_t need = retention_chunk_smem(m->max_ret_dim);
            if (need > attr) { SCU(cudaFuncSetAttribute(k_retention_chunk_out, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) need)); attr = need; }
        }
        size_t moe_rows = 0;
        if (m->max_slots > 0) {
            moe_rows = cap * (size_t) m->max_slots;
            fl(&c->Xp, moe_rows * m->E); fl(&c->Ap, moe_rows * m->max_eff); fl(&c->Yk, moe_rows * m->E);
            fl(&c->r_wt, moe_rows); fl(&c->r_sg, cap); fl(&c->r_z, cap * ((size_t) m->max_exp + 1)); fl((float **) &c->r_counter, cap);
            fl((float **) &c->r_sel, moe_rows); fl((float **) &c->r_slot, moe_rows); fl((float **) &c->r_src, moe_rows); fl((float **) &c->r_seg, (size_t) m->max_exp + 1);
        }
        fl(&c->P, cap * m->maxP); fl(&c->A, cap * m->maxA); fl(&c->QK, cap_t * m->maxQK); fl(&c->OL, cap_t * m->maxOL);
        fl(&c->CV, cap * m->maxCV); fl(&c->BG, cap * m->maxBG); fl(&c->O, cap * m->maxA);
        fl(&c->rec, m->rec_floats);
        if (m->dtype == STACK_BF16) {
            c->xb_elems = std::max(cap * (size_t) std::max({ 2 * m->E, m->maxA, m->maxOL, m->maxP }), moe_rows * (size_t) std::max(m->E, m->max_eff));
            SCU(cudaMalloc(&c->xb, c->xb_elems * 2));
        }
        SCU(cudaMalloc(&c->d_err, 4)); SCU(cudaMemsetAsync(c->d_err, 0, 4, c->st));
        SCU(cudaMallocHost(&c->h_err, 4)); *c->h_err = 0;
        c->caches.assign((size_t) m->n_caches, nullptr);
        c->pools.assign((size_t) m->n_caches, nullptr);
        cudaDeviceProp prop;
        SCU(cudaGetDeviceProperties(&prop, m->device));
        c->sm_count = prop.multiProcessorCount;
        size_t smem = 0, part = 0, ml = 0, da_part = 0, da_cnt = 0;
        struct Cached { const LayerSpec * L; int index; };
        std::vector<Cached> cached;           // every attention cache of every run (a pair's branches each have their own)
        for (const RunSpec & R : m->runs) {
            const LayerSpec & L = m->layers[(size_t) R.layer];
            if (R.cache_index < 0) continue;
            if (L.kind != MIX_PAIR) { cached.push_back({ &L, R.cache_index }); continue; }
            int at = R.cache_index;
            for (const LayerSpec & B : L.parts) if (B.cache_row) cached.push_back({ &B, at++ });
        }
        for (const Cached & cd : cached) {
            const LayerSpec & L = *cd.L;
            {   // [ window - 1 zero rows | n_ctx positions | one tile of slack ]: a tile's key range may start before position 0 and end past the portion
                const size_t front = (size_t) std::max(L.window, 1), rows = front + (size_t) n_ctx + 2 * ATT_TQ;
                float * base = nullptr;
                fl(&base, rows * L.cache_row);
                c->cache_allocs.push_back(base);
                c->caches[(size_t) cd.index] = base + front * L.cache_row;
                size_t nk = (L.window > 0 ? (size_t) L.window + ATT_TQ - 1 : (size_t) n_ctx + ATT_TQ) + 3;
                if (L.pool > 0) {             // means of whole blocks: [ n_ctx / pool rows | a tile of slack for padded products ]
                    const size_t prow = (size_t) n_ctx / (size_t) L.pool + ATT_TQ;
                    fl(&c->pools[(size_t) cd.index], prow * L.cache_row);
                    nk += prow;
                }
                const size_t one = (size_t) ATT_TQ * L.H * nk * (L.kind == MIX_DIFFATTN ? 2 : 1);     // one tile's scores (two maps per head)
                const size_t all = (cap_t / ATT_TQ) * one;
                c->att_scores_floats = std::max(c->att_scores_floats, std::min(all, std::max(one, ATT_SCORE_BYTES / 4)));
            }
            if (L.kind == MIX_DIFFATTN) {
                const size_t mgw = 4 + 64 * (size_t) (L.V <= 32 ? 1 : L.V <= 64 ? 2 : L.V <= 128 ? 4 : 8);
                da_part = std::max(da_part, (size_t) 8 * L.H * DIFF_MAX_SPLIT * mgw);
                da_cnt = std::max(da_cnt, (size_t) 8 * L.H);
                continue;
            }
            if (L.kind == MIX_SIGATTN) {
                da_part = std::max(da_part, (size_t) 8 * L.H * SIG_MAX_SPLIT * 32 * (size_t) sig_vpl(L));
                da_cnt = std::max(da_cnt, (size_t) 8 * L.H);
                continue;
            }
            if (L.kind == MIX_GQATTN) {       // key slices only while (tokens x heads x slices) stays under 8 per SM; one counter per (token, head) of a pass
                da_part = std::max(da_part, (size_t) (8 * c->sm_count + 64) * (2 + 32 * (size_t) gqa_vpl(L)));
                da_cnt = std::max(da_cnt, cap * (size_t) L.H);
                continue;
            }
            for (int T = 1; T <= std::min(c->cap, 7); T++) {      // the pass sizes that take the decode kernels: the buffers cover the largest plan
                const AttnPlan ap = plan_attention(L, n_ctx, T, c->sm_count);
                smem = std::max(smem, ap.smem);
                if (ap.nsplit > 1) { part = std::max(part, (size_t) T * L.H * ap.nsplit * L.rank); ml = std::max(ml, (size_t) T * L.H * ap.nsplit * 2); }
            }
        }
        if (smem > 227 * 1024) throw std::runtime_error("latent attention: a context of " + std::to_string(n_ctx) + " positions without a window does not fit one block's shared memory; use a smaller n_ctx");
        c->attn_smem = smem;
        fl(&c->att_part, part); fl(&c->att_ml, ml);
        if (da_part) { fl(&c->da_part, da_part); fl((float **) &c->da_counter, da_cnt); }
        if (c->att_scores_floats) fl(&c->att_scores, c->att_scores_floats);
        {   // the opt-in limit is a property of the kernel, not of a context: it only ever grows
            static size_t attr = 48 * 1024;
            if (smem > attr) {
                SCU(cudaFuncSetAttribute(k_latent_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
                SCU(cudaFuncSetAttribute(k_latent_attn_staged<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
                SCU(cudaFuncSetAttribute(k_latent_attn_staged<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
                attr = smem;
            }
        }
        SCU(cudaMalloc(&c->d_step, sizeof(StepDev)));
        SCU(cudaMemsetAsync(c->d_step, 0, sizeof(StepDev), c->st));
        SCU(cudaMallocHost(&c->h_step, sizeof(StepDev)));
        std::memset(c->h_step, 0, sizeof(StepDev));
        SCU(cudaMalloc(&c->d_out_tokens, (size_t) (n_ctx + 1) * 4)); SCU(cudaMalloc(&c->d_counter, 4));
        SCU(cudaMalloc(&c->d_arg, 4));
        SCU(cudaMallocHost(&c->h_arg, 4));
        SCU(cudaEventCreate(&c->ev0)); SCU(cudaEventCreate(&c->ev1));
        ensure_logit_rows(c.get(), 16);
        SCU(cudaMemsetAsync(c->rec, 0, std::max<size_t>(m->rec_floats, 4) * 4, c->st));
        SCU(cudaStreamSynchronize(c->st));
    } catch (...) {
        stack_ctx_free(c.release());
        cudaGetLastError();
        throw;
    }
    return c.release();
}

int stack_ctx_n_ctx(const StackCtx * c) { return c->n_ctx; }
int stack_ctx_n_past(const StackCtx * c) { return c->n_past; }
int64_t stack_ctx_launches(const StackCtx * c) { return c->launches; }
float stack_last_device_ms(const StackCtx * c) { return c->last_ms; }

void stack_ctx_clear(StackCtx * c) {
    SCU(cudaSetDevice(c->m->device));
    // recurrent state back to zero; cached positions need no clearing: a sequence only reads positions it wrote
    SCU(cudaMemsetAsync(c->rec, 0, std::max<size_t>(c->m->rec_floats, 4) * 4, c->st));
    SCU(cudaStreamSynchronize(c->st));
    c->n_past = 0;
    c->h_last = nullptr; c->d_last_row = -1;
}

void stack_set_taps(StackCtx * c, bool on) { c->taps = on; c->tap_data.clear(); c->tap_T = 0; }
int64_t stack_get_taps(StackCtx * c, float * out, int64_t cap) {
    const int64_t n = (int64_t) c->tap_data.size();
    if (out) std::memcpy(out, c->tap_data.data(), (size_t) std::min(n, cap) * 4);
    return n;
}

void stack_decode(StackCtx * c, const int32_t * tokens, int n, int pos0, const int32_t * rows, int n_rows, float * logits_out) {
    StackModel & m = *c->m;
    if (!tokens || n <= 0) throw std::runtime_error("empty step");
    if (pos0 != c->n_past) throw std::runtime_error("this model carries recurrent state: a step must continue the sequence at position " +
                                                    std::to_string(c->n_past) + " (got " + std::to_string(pos0) + "); clear the context to start a new one");
    if ((int64_t) pos0 + n > c->n_ctx) throw std::runtime_error("the step exceeds the context of " + std::to_string(c->n_ctx) + " positions");
    for (int i = 0; i < n; i++) if (tokens[i] < 0 || tokens[i] >= m.vocab) throw std::runtime_error("token id " + std::to_string(tokens[i]) + " is outside the vocabulary");
    const int32_t last_row = n - 1;
    if (!rows) { rows = &last_row; n_rows = 1; }
    for (int i = 0; i < n_rows; i++) if (rows[i] < 0 || rows[i] >= n || (i && rows[i] <= rows[i - 1])) throw std::runtime_error("wanted rows must be ascending indices into the step");
    SCU(cudaSetDevice(m.device));
    ensure_logit_rows(c, std::max(n_rows, 1));
    SCU(cudaEventRecord(c->ev0, c->st));
    if (n == 1 && n_rows == 1 && !c->taps && graph_enabled() && !c->graph_failed) {
        c->h_step->st.pos0 = pos0; c->h_step->st.n_tokens = 1; c->h_step->tokens[0] = tokens[0];
        if (!c->g_token) {
            SCU(cudaStreamSynchronize(c->st));
            const int64_t before = c->launches;
            cudaGraph_t g = nullptr;
            bool ok = cudaStreamBeginCapture(c->st, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
            if (ok) {
                try { enqueue_token_step(c); } catch (...) { ok = false; }
                if (cudaStreamEndCapture(c->st, &g) != cudaSuccess) ok = false;
            }
            if (ok && cudaGraphInstantiate(&c->g_token, g, 0) != cudaSuccess) { ok = false; c->g_token = nullptr; }
            if (g) cudaGraphDestroy(g);
            c->n_token_launches = c->launches - before;
            c->launches = before;
            if (!ok) { cudaGetLastError(); c->graph_failed = true; }
        }
        if (c->g_token) {
            SCU(cudaGraphLaunch(c->g_token, c->st));
            c->launches += c->n_token_launches;
        } else {
            enqueue_token_step(c);
        }
        SCU(cudaEventRecord(c->ev1, c->st));
        SCU(cudaStreamSynchronize(c->st));
        c->d_last_row = 0; c->h_last = c->h_logits;
    } else {
        if (c->taps) { c->tap_data.assign(m.runs.size() * (size_t) n * m.E, 0.f); c->tap_T = n; if (n > c->cap) throw std::runtime_error("taps need a step of at most one pass"); }
        int64_t row_off = 0;
        int ri = 0;
        for (int i0 = 0; i0 < n; i0 += c->cap) {
            const int T = std::min(c->cap, n - i0);
            SCU(cudaStreamSynchronize(c->st));              // the pinned header is free again
            c->h_step->st.pos0 = pos0 + i0; c->h_step->st.n_tokens = T;
            std::memcpy(c->h_step->tokens, tokens + i0, (size_t) T * 4);
            int nr = 0;
            while (ri < n_rows && rows[ri] < i0 + T) c->h_step->rows[nr++] = rows[ri++] - i0;
            SCU(cudaMemcpyAsync(c->d_step, c->h_step, sizeof(StepState) + (size_t) T * 4, cudaMemcpyHostToDevice, c->st));
            if (nr) SCU(cudaMemcpyAsync(c->d_step->rows, c->h_step->rows, (size_t) nr * 4, cudaMemcpyHostToDevice, c->st));
            enqueue_layers(c, T);
            if (nr) { enqueue_head(c, nr, row_off); row_off += nr; }
        }
        if (row_off) SCU(cudaMemcpyAsync(c->h_logits, c->d_logits, (size_t) row_off * m.vocab * 4, cudaMemcpyDeviceToHost, c->st));
        SCU(cudaMemcpyAsync(c->h_err, c->d_err, 4, cudaMemcpyDeviceToHost, c->st));
        SCU(cudaEventRecord(c->ev1, c->st));
        SCU(cudaStreamSynchronize(c->st));
        if (*c->h_err) throw std::runtime_error("a tensor-core product gave up waiting for its pipeline (k_gemm_bf16_umma); the step's results are invalid");
        if (row_off) { c->d_last_row = row_off - 1; c->h_last = c->h_logits + (size_t) (row_off - 1) * m.vocab; }
    }
    cudaEventElapsedTime(&c->last_ms, c->ev0, c->ev1);
    c->n_past = pos0 + n;
    if (logits_out && n_rows > 0) std::memcpy(logits_out, c->h_logits, (size_t) n_rows * m.vocab * 4);
}

// Device-resident greedy loop: token -> layers -> head -> arg-max -> next token, n_steps times, one graph replay per token and
// no host round trip in between; out_tokens[n_steps] receives the ids.
void stack_generate_greedy(StackCtx * c, int32_t first_token, int pos0, int n_steps, int32_t * out_tokens) {
    StackModel & m = *c->m;
    if (n_steps <= 0 || !out_tokens) throw std::runtime_error("bad arguments");
    if (pos0 != c->n_past) throw std::runtime_error("the burst must continue the sequence at position " + std::to_string(c->n_past));
    if ((int64_t) pos0 + n_steps > c->n_ctx) throw std::runtime_error("the burst exceeds the context of " + std::to_string(c->n_ctx) + " positions");
    if (first_token < 0 || first_token >= m.vocab) throw std::runtime_error("token id outside the vocabulary");
    if (c->taps || !graph_enabled() || c->graph_failed) {
        int32_t tok = first_token;
        float ms = 0.f;
        for (int i = 0; i < n_steps; i++) { stack_decode(c, &tok, 1, pos0 + i, nullptr, 1, nullptr); ms += c->last_ms; out_tokens[i] = tok = stack_argmax(c); }
        c->last_ms = ms;
        return;
    }
    SCU(cudaSetDevice(m.device));
    ensure_logit_rows(c, 1);
    SCU(cudaStreamSynchronize(c->st));
    c->h_step->st.pos0 = pos0; c->h_step->st.n_tokens = 1; c->h_step->tokens[0] = first_token;
    const auto body = [&]() {
        enqueue_layers(c, 1);
        enqueue_head(c, 1, 0, true);
        k_argmax_advance<<<1, 1024, 0, c->st>>>(c->d_logits, m.vocab, &c->d_step->st, c->d_step->tokens, c->d_out_tokens, c->d_counter);
        c->launches++;
    };
    if (!c->g_greedy) {
        const int64_t before = c->launches;
        cudaGraph_t g = nullptr;
        bool ok = cudaStreamBeginCapture(c->st, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if (ok) {
            try { body(); } catch (...) { ok = false; }
            if (cudaStreamEndCapture(c->st, &g) != cudaSuccess) ok = false;
        }
        if (ok && cudaGraphInstantiate(&c->g_greedy, g, 0) != cudaSuccess) { ok = false; c->g_greedy = nullptr; }
        if (g) cudaGraphDestroy(g);
        c->n_greedy_launches = c->launches - before;
        c->launches = before;
        if (!ok) { cudaGetLastError(); c->graph_failed = true; stack_generate_greedy(c, first_token, pos0, n_steps, out_tokens); return; }
    }
    SCU(cudaMemcpyAsync(c->d_step, c->h_step, sizeof(StepState) + sizeof(int32_t), cudaMemcpyHostToDevice, c->st));
    SCU(cudaMemsetAsync(c->d_step->rows, 0, sizeof(int32_t), c->st));
    SCU(cudaMemsetAsync(c->d_counter, 0, 4, c->st));
    SCU(cudaEventRecord(c->ev0, c->st));
    for (int i = 0; i < n_steps; i++) SCU(cudaGraphLaunch(c->g_greedy, c->st));
    SCU(cudaEventRecord(c->ev1, c->st));
    SCU(cudaMemcpyAsync(out_tokens, c->d_out_tokens, (size_t) n_steps * 4, cudaMemcpyDeviceToHost, c->st));
    SCU(cudaStreamSynchronize(c->st));
    cudaEventElapsedTime(&c->last_ms, c->ev0, c->ev1);
    c->launches += c->n_greedy_launches * n_steps;
    c->n_past = pos0 + n_steps;
    c->d_last_row = 0; c->h_last = nullptr;       // the last token's logits are on the device only
}

void stack_sync(StackCtx * c) {
    SCU(cudaSetDevice(c->m->device));
    SCU(cudaStreamSynchronize(c->st));
}

float * stack_logits_view(StackCtx * c) {
    if (!c->h_last && c->d_last_row >= 0) {         // after a device-resident burst: fetch the row now
        SCU(cudaSetDevice(c->m->device));
        SCU(cudaMemcpyAsync(c->h_logits, c->d_logits + (size_t) c->d_last_row * c->m->vocab, (size_t) c->m->vocab * 4, cudaMemcpyDeviceToHost, c->st));
        SCU(cudaStreamSynchronize(c->st));
        c->h_last = c->h_logits;
    }
    if (!c->h_last) throw std::runtime_error("no logits yet: the last step asked for none");
    return c->h_last;
}

int32_t stack_argmax(StackCtx * c) {
    if (c->d_last_row < 0) throw std::runtime_error("no logits yet: the last step asked for none");
    SCU(cudaSetDevice(c->m->device));
    k_argmax_row<<<1, 1024, 0, c->st>>>(c->d_logits + (size_t) c->d_last_row * c->m->vocab, c->m->vocab, c->d_arg);
    c->launches++;
    SCU(cudaMemcpyAsync(c->h_arg, c->d_arg, 4, cudaMemcpyDeviceToHost, c->st));
    SCU(cudaStreamSynchronize(c->st));
    return *c->h_arg;
}

float stack_time_linear(int device, int dtype, int T, int N, int K, int reps) {
    SCU(cudaSetDevice(device));
    float * X = nullptr, * Y = nullptr; void * W = nullptr;
    UmmaScratch us;
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    float ms = 0.f;
    // several distinct weight matrices so that a repetition does not find its operand in L2
    const size_t wbytes = (size_t) N * K * (dtype == STACK_F32 ? 4 : 2);
    const int copies = (int) std::min<size_t>(8, std::max<size_t>(1, ((size_t) 256 << 20) / std::max<size_t>(wbytes, 1) + 1));
    try {
        SCU(cudaMalloc(&X, (size_t) T * K * 4)); SCU(cudaMalloc(&Y, (size_t) T * N * 4)); SCU(cudaMalloc(&W, wbytes * copies));
        SCU(cudaMemset(X, 0, (size_t) T * K * 4)); SCU(cudaMemset(W, 0, wbytes * copies));
        us.elems = (size_t) T * K;
        SCU(cudaMalloc(&us.xb, us.elems * 2)); SCU(cudaMalloc(&us.err, 4)); SCU(cudaMemset(us.err, 0, 4));
        SCU(cudaStreamCreate(&st)); SCU(cudaEventCreate(&e0)); SCU(cudaEventCreate(&e1));
        for (int i = 0; i < 3; i++) linear_on(st, dtype, nullptr, X, K, (char *) W + wbytes * (size_t) (i % copies), nullptr, Y, N, T, N, K, 1, 0, 0, 0, false, 0.f, &us);
        SCU(cudaStreamSynchronize(st));
        SCU(cudaEventRecord(e0, st));
        for (int i = 0; i < reps; i++) linear_on(st, dtype, nullptr, X, K, (char *) W + wbytes * (size_t) (i % copies), nullptr, Y, N, T, N, K, 1, 0, 0, 0, false, 0.f, &us);
        SCU(cudaEventRecord(e1, st));
        SCU(cudaStreamSynchronize(st));
        cudaEventElapsedTime(&ms, e0, e1);
    } catch (...) {
        cudaFree(X); cudaFree(Y); cudaFree(W); cudaFree(us.xb); cudaFree(us.err);
        if (st) cudaStreamDestroy(st);
        throw;
    }
    cudaFree(X); cudaFree(Y); cudaFree(W); cudaFree(us.xb); cudaFree(us.err);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaStreamDestroy(st);
    return ms / (float) std::max(reps, 1);
}

void stack_linear(int device, int dtype, int T, int N, int K, const float * x, const float * w, const float * bias, int glu, float limit, float * y) {
    SCU(cudaSetDevice(device));
    StackModel tmp;                      // owns the device copies
    tmp.device = device; tmp.dtype = dtype;
    float * X = nullptr, * Y = nullptr;
    UmmaScratch us;
    int herr = 0;
    const int ny = glu ? N / 2 : N;
    try {
        const std::vector<float> wv(w, w + (size_t) N * K);
        std::vector<float> bv;
        if (bias) bv.assign(bias, bias + N);
        const DMat d = up_mat(tmp, wv, N, K, bias ? &bv : nullptr);
        SCU(cudaMalloc(&X, (size_t) T * K * 4)); SCU(cudaMalloc(&Y, (size_t) T * ny * 4));
        SCU(cudaMemcpy(X, x, (size_t) T * K * 4, cudaMemcpyHostToDevice));
        us.elems = (size_t) T * K;
        SCU(cudaMalloc(&us.xb, us.elems * 2)); SCU(cudaMalloc(&us.err, 4)); SCU(cudaMemset(us.err, 0, 4));
        linear_on(nullptr, dtype, nullptr, X, K, d.w, d.bias, Y, ny, T, N, K, 1, 0, 0, 0, glu != 0, limit, &us);
        SCU(cudaDeviceSynchronize());
        SCU(cudaMemcpy(y, Y, (size_t) T * ny * 4, cudaMemcpyDeviceToHost));
        SCU(cudaMemcpy(&herr, us.err, 4, cudaMemcpyDeviceToHost));
    } catch (...) {
        cudaFree(X); cudaFree(Y); cudaFree(us.xb); cudaFree(us.err);
        for (void * p : tmp.allocs) cudaFree(p);
        throw;
    }
    cudaFree(X); cudaFree(Y); cudaFree(us.xb); cudaFree(us.err);
    for (void * p : tmp.allocs) cudaFree(p);
    if (herr) throw std::runtime_error("k_gemm_bf16_umma gave up waiting for its pipeline");
}

}  // namespace b200
