// Engine-facing op set: the attention entry points of the reference's gpu.h with the same names,
// argument order and meaning, implemented over the C ABI of include/kiln_b200.h.
//
//   attention()    engine/src/gpu.h:152-153, engine/src/kernels.cu:828-866
//   attention16()  engine/src/gpu.h:155-156, engine/src/kernels.cu:868-873
//   rmsnorm()      engine/src/gpu.h:133,     engine/src/kernels.cu:668-673   (rows of 128: the per-head Q/K norm)
//   rope_half()    engine/src/gpu.h:145,     engine/src/kernels.cu:773-777
//   linear16()     engine/src/gpu.h (Epi16, linear16), engine/src/kernels.cu:559-609   (LoRAs unmerged, as a second product)
//   nag_combine is the k_nag launch of engine/src/dit.cu:486 (fp16 rows) / :524 (fp32 rows)
//
// Like the reference ops they run on one stream, take device pointers the caller owns, and throw
// std::runtime_error on failure (the reference's CK/CB macros, engine/src/gpu.h:15-16); the engine's job
// wrapper turns that into an {"ev":"error"} event (engine/src/engine.h:785-791).
// The reference keeps stream and scratch arena in a global `Gpu G` (engine/src/gpu.h:63-90); the
// equivalent here is OpContext, set once by the engine with G.stream and a slice of G.arena.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace kiln_b200 {

struct OpContext {
    cudaStream_t stream = nullptr;
    void* workspace = nullptr;       // fp16 staging of Q/K/V: kb_attn_workspace_bytes(...) for the largest call
    size_t workspace_bytes = 0;
};
void set_context(const OpContext& ctx);
const OpContext& context();

// q [Tq, ldq], k/v [Tk, ld*], out [Tq, ldo] fp32; head h at column h*Dh; npad zero keys join the softmax.
// The fused kernels take what the reference's own fast path takes (engine/src/kernels.cu:830: not causal, Dh == 128, row strides
// that are multiples of 4). The reference's dispatcher sends everything else - the causal text encoder (engine/src/te.cu:90),
// the Dh = 64 adapter (engine/src/dit.cu:106-169) - to its exact fp32 path (engine/src/kernels.cu:842-865), which is not
// part of this library: the engine registers that path here once and attention() falls through to it exactly as the
// reference's dispatcher does; without a registered path such a call throws.
using ExactAttentionFn = void (*)(float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                                  int Tq, int Tk, int H, int Dh, bool causal, int npad);
void set_exact_attention(ExactAttentionFn fn);
bool attention_eligible(int Dh, bool causal, int ldq, int ldk, int ldv, int ldo);
void attention(float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
               int Tq, int Tk, int H, int Dh, bool causal, int npad = 0);
void attention16(__half* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                 int Tq, int Tk, int H, int Dh, int npad = 0);

// In-place fp32 RMSNorm over rows of 128 with a bf16 weight (the reference passes a Weight*; its ->p is this pointer).
// A null weight normalises with weight 1, as the reference does (engine/src/kernels.cu:650-673).
void rmsnorm(float* y, const float* x, const uint16_t* w_bf16, int rows, int dim, float eps);
void rope_half(float* x, int T, int H, int Dh, const float* cos_t, const float* sin_t);

// Fused forms the DiT block driver can call instead of the unfused sequences:
// rmsnorm(Q) + rmsnorm(K) + rope_half(Q) + rope_half(K) + attention16 per batch element -> one call for the whole batch
void self_attention16(__half* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                      int B, int T, int H, const uint16_t* qn_w, const uint16_t* kn_w, const float* rope_cos,
                      const float* rope_sin, float eps);
// rmsnorm(Q) + attention16(pos) + attention16(neg) + k_nag -> one call
void nag_attention16(__half* out, int ldo, const float* q, int ldq, const uint16_t* qn_w, const float* k_pos, const float* v_pos,
                     int Tk_pos, int npad_pos, const float* k_neg, const float* v_neg, int Tk_neg, int npad_neg, int ld_kv,
                     float scale, float tau, float alpha, int Tq, int H, float eps);

// The fp16-activation linear layer y = epi(x16 [T, in] . W^T), W an fp16 [out, in] weight (the reference's Weight with
// f16 set; a bf16 weight is converted by the caller once, as the reference does into G.wbuf). Epilogues as the reference's
// Epi16 (engine/src/kernels.cu:597-603); y is fp32 for F32 / Resid and fp16 for F16 / Gelu16.
enum class Epi16 { F32 = 0, F16 = 1, Gelu16 = 2, Resid = 3 };
// The LoRAs of one weight, stacked and converted ONCE (pack_lora below). The reference's linear16 rebuilds these two
// matrices from the bf16 LoRA tensors on every call (engine/src/kernels.cu:578-590); they depend only on the weights.
struct Lora16 {
    const __half* a_cat = nullptr;   // [rank, in]  the down-projections, one under the other
    const __half* b_cat = nullptr;   // [out, rank] the up-projections side by side, each times its LoRA's scale
    int rank = 0;                    // stacked rank padded to a multiple of 8 with zero rows / columns
};
struct LoraAdd16 {                   // one LoRA as the reference holds it (LoraAdd, engine/src/gpu.h:37), bf16 on the device
    const uint16_t* A; int r;        // [r, in]
    const uint16_t* B;               // [out, r]
    float scale;
};
inline int lora_rank_padded(const LoraAdd16* adds, int n) { int r = 0; for (int i = 0; i < n; i++) r += adds[i].r; return (r + 7) / 8 * 8; }
// Fills a_cat [rank, in] and b_cat [out, rank] (device buffers of the caller, rank = lora_rank_padded) on the context's stream.
void pack_lora(__half* a_cat, __half* b_cat, int out, int in, const LoraAdd16* adds, int n);
struct Weight16 {
    const __half* p = nullptr;
    int rows = 0, cols = 0;          // out, in
    const Lora16* lora = nullptr;    // null: none. With LoRAs a call first forms t = x16 . a_cat^T ([T, rank] fp16, at the start
                                     // of the context's workspace) and the GEMM adds t . b_cat^T before its epilogue
};
void linear16(void* y, int ldy, const __half* x16, int T, const Weight16& W, Epi16 epi, const float* gate = nullptr);
// linear16 + rmsnorm + rope_half of engine/src/dit.cu:461-468 in one launch, fp16 out: what attention consumes directly
void linear16_heads(__half* y, int ldy, const __half* x16, int T, const Weight16& W, const uint16_t* norm_w_bf16,
                    const float* rope_cos, const float* rope_sin, int rope_T, float eps);

// the three linear16_heads / linear16 calls of a block's q, k, v projections in one launch (outputs fp16 [T, ldy]; q and k
// normalised with their own weights and rotated, v plain)
void linear16_qkv(__half* q, __half* k, __half* v, int ldy, const __half* x16, int T, const Weight16& Wq, const Weight16& Wk,
                  const Weight16& Wv, const uint16_t* qn_w_bf16, const uint16_t* kn_w_bf16, const float* rope_cos, const float* rope_sin,
                  int rope_T, float eps);

// Cross-attention K and V of one context for one block (the body of Dit::cache_context's loop, engine/src/dit.cu:228-230:
// linear + rmsnorm + linear), emitted fp16 and already normalised: attention16 / nag_attention16 then read them without the
// per-call conversion, and the cache is half the size. ctx fp32 [L, Wk.cols]; k16, v16 [L, ldy]; kn_w bf16[128].
void cross_kv16(__half* k16, __half* v16, int ldy, const float* ctx, int L, const Weight16& Wk, const Weight16& Wv, const uint16_t* kn_w_bf16,
                float eps);

// The trainer's exact attention backward (attention_bwd, engine/src/train.cu:216-242; an anonymous-namespace function there, with
// D = 2048 fixed): q, dout [Tq, H*128], k, v [Tk, H*128] fp32 rows -> dq, dk, dv (written). npad zero keys of score 0 join the
// softmax. Nothing of size Tq x Tk is materialised; scratch comes from the context's workspace (kb_attn_bwd_workspace_bytes).
void attention_bwd(float* dq, float* dk, float* dv, const float* q, const float* k, const float* v, const float* dout, int Tq, int Tk, int npad,
                   int H = 16);

}  // namespace kiln_b200
