// stack.hpp — host interface of the layer-stack model family (stack.cu): models described by a config.json whose
// "layers" list names, per layer, a mixer (minGRU | latent attention | gated delta rule | generalized delta rule |
// differential sliding-window attention | retention | a sigmoid attention beside a retention | soft-max attention over grouped
// heads under a chunk mask or a window with block means) and an optional feed-forward (gated unit | polynomial | routed mixture
// of gated units); four designs (Matulorn, Dopilorn, Tosevik, Rumurax) arrange them.
// engine.cu dispatches the C-ABI (b200_model_load, b200_ctx_new, b200_decode, ...) here when the model path is a folder
// with config.json + model.safetensors; the GGUF LLaMA path stays where it was. Functions throw std::runtime_error.
#pragma once
#include <cstdint>
#include <string>

namespace b200 {

struct StackModel;
struct StackCtx;

enum { STACK_BF16 = 0, STACK_F32 = 1 };

// designs the registry knows (config.json "architecture")
bool stack_knows(const std::string & architecture);

StackModel * stack_model_load(const std::string & dir, int device, int dtype);
void         stack_model_free(StackModel * m);
// B200_INFO_* slots the family can fill (vocab, width, layers, ...)
void         stack_model_info(const StackModel * m, int32_t info[16]);
int64_t      stack_model_weight_bytes(const StackModel * m);
int          stack_model_device(const StackModel * m);
int          stack_model_n_vocab(const StackModel * m);

// One sequence per context, like the LLaMA contexts: a cache of n_ctx positions for the attention layers and the
// recurrent state (minGRU state, delta-rule matrices, convolution history) of the other mixers, all in float32. A layer
// that a design runs several times per token keeps one cache / state per run.
StackCtx * stack_ctx_new(StackModel * m, int n_ctx);
void       stack_ctx_free(StackCtx * c);
int        stack_ctx_n_ctx(const StackCtx * c);
int        stack_ctx_n_past(const StackCtx * c);
void       stack_ctx_clear(StackCtx * c);            // the sequence ends: state zeroed, positions start at 0 again
int64_t    stack_ctx_launches(const StackCtx * c);

// The step function: the next n tokens of the sequence (pos0 must equal the number of tokens the context holds).
// rows[n_rows] (ascending indices into the step's tokens; nullptr: the last token only) are the places whose logits
// are computed; logits_out (host, [n_rows][n_vocab]) may be nullptr — the last row then stays available through
// stack_logits_view / stack_argmax. One token steps replay a captured CUDA graph.
void    stack_decode(StackCtx * c, const int32_t * tokens, int n, int pos0, const int32_t * rows, int n_rows, float * logits_out);
void    stack_generate_greedy(StackCtx * c, int32_t first_token, int pos0, int n_steps, int32_t * out_tokens);
void    stack_sync(StackCtx * c);
float * stack_logits_view(StackCtx * c);             // pinned host copy of the last computed row of logits
int32_t stack_argmax(StackCtx * c);                  // arg-max of that row, computed on the device
// residual stream after every layer run of the LAST step, host [n_runs][n][width] (parity tests); enable before the step
void    stack_set_taps(StackCtx * c, bool on);
int64_t stack_get_taps(StackCtx * c, float * out, int64_t cap);
float   stack_last_device_ms(const StackCtx * c);

// micro-benchmark of one product shape through the family's own kernels (bench.py): ms per call, CUDA events
float   stack_time_linear(int device, int dtype, int T, int N, int K, int reps);
// one product y[T][N] = x[T][K] w[N][K]^T (+ bias; glu: rows of w interleaved gate/up, y[T][N/2] = the clamped gated unit)
// through the kernel the family would pick for that shape (parity tests)
void    stack_linear(int device, int dtype, int T, int N, int K, const float * x, const float * w, const float * bias, int glu, float limit, float * y);

}  // namespace b200
