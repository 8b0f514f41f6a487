// The binding of the reference's five attention-path ops to the library (TEST INFRASTRUCTURE, shared by the two builds of
// the reference's driver over this repository's kernels: oracle/ref_wrap.cu and oracle/ref_engine_bind.cu).
//
// Read with the reference's gpu.h already included under the renames attention -> ref_own_attention (and likewise
// attention16, rmsnorm, rope_half, linear16), so that Weight, Epi16, G and the ref_own_* declarations are visible and the
// plain names are free. It defines the plain names with the reference's signatures (engine/src/gpu.h:133,145,152-156 and
// linear16 there): each call goes to the library and falls back to the reference's own op for what the library does not
// cover (head sizes other than 128, causal attention, weights that are not fp16 in VRAM), which is how an engine
// maintainer would bind the library.
#pragma once
#include "gpu_ops.h"
#include "kiln_b200.h"

// ---- the binding: the reference's signatures (engine/src/gpu.h:133,145,152-156 and linear16 there), the library underneath ----
// The library's staging area (fp16 copies of fp32 operands, LoRA down-projections, the backward's scratch): one block outside
// the engine's arena, sized for the largest call the engine makes (8192 image tokens). Taken at the first bound call, or
// earlier by whoever sizes the engine's scratch (oracle/ref_engine_bind.cu does, so that the arena leaves room for it).
static void* g_bind_ws = nullptr;
static size_t g_bind_ws_bytes = 0;
static size_t bind_workspace_bytes() {
    const size_t fwd = kb_attn_workspace_bytes(8192, 8192, 2, 16, KB_F32, 1, 1), bwd = kb_attn_bwd_workspace_bytes(1, 8192, 8192, 16, KB_F32);
    return (fwd > bwd ? fwd : bwd) + ((size_t)64 << 20);   // + room for LoRA down-projections
}
static void bind_workspace_reserve() {
    if (g_bind_ws) return;
    g_bind_ws_bytes = bind_workspace_bytes();
    if (cudaMalloc(&g_bind_ws, g_bind_ws_bytes) != cudaSuccess) { g_bind_ws = nullptr; throw std::runtime_error("workspace allocation failed"); }
    kiln_b200::set_exact_attention([](float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                                      int Tq, int Tk, int H, int Dh, bool causal, int npad) {
        ref_own_attention(out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, Dh, causal, npad);
    });
}
static void bind_context() {
    bind_workspace_reserve();
    kiln_b200::OpContext c;
    c.stream = G.stream; c.workspace = g_bind_ws; c.workspace_bytes = g_bind_ws_bytes;
    kiln_b200::set_context(c);
}
void attention(float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
               int Tq, int Tk, int H, int Dh, bool causal, int npad = 0) {
    // a job that asks for exact arithmetic (G.fp16 off: engine/src/kernels.cu:830 keeps it off the fast kernels) stays on the reference's fp32 path
    if (!G.fp16) { ref_own_attention(out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, Dh, causal, npad); return; }
    bind_context();
    kiln_b200::attention(out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, Dh, causal, npad);   // falls through to ref_own_attention when not eligible
}
void attention16(__half* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                 int Tq, int Tk, int H, int Dh, int npad = 0) {
    bind_context();
    kiln_b200::attention16(out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, Dh, npad);
}
void rmsnorm(float* y, const float* x, const Weight* w, int rows, int dim, float eps) {
    if (dim != 128) { ref_own_rmsnorm(y, x, w, rows, dim, eps); return; }                   // the 2048- and 1024-wide norms are not on the path
    bind_context();
    kiln_b200::rmsnorm(y, x, w ? w->p : nullptr, rows, dim, eps);
}
void rope_half(float* x, int T, int H, int Dh, const float* cos_t, const float* sin_t) {
    if (Dh != 128) { ref_own_rope_half(x, T, H, Dh, cos_t, sin_t); return; }
    bind_context();
    kiln_b200::rope_half(x, T, H, Dh, cos_t, sin_t);
}
void linear16(void* y, int ldy, const __half* x16, int T, const Weight& Win, Epi16 epi, const float* gate = nullptr) {
    if (!Win.f16 || Win.on_host || Win.cols % 64) { ref_own_linear16(y, ldy, x16, T, Win, epi, gate); return; }
    bind_context();
    kiln_b200::Weight16 W;
    W.p = (const __half*)Win.p; W.rows = (int)Win.rows; W.cols = (int)Win.cols;
    kiln_b200::Lora16 L;
    const size_t m = G.arena.mark();
    if (Win.lora && !Win.lora->empty()) {                          // stacked per call into the arena, as engine/src/kernels.cu:578-590 does
        std::vector<kiln_b200::LoraAdd16> adds;
        for (auto& l : *Win.lora) adds.push_back({l.A.p, (int)l.A.rows, l.B.p, l.scale});
        const int rank = kiln_b200::lora_rank_padded(adds.data(), (int)adds.size());
        __half* ac = (__half*)G.arena.f(((size_t)rank * W.cols + 1) / 2);
        __half* bc = (__half*)G.arena.f(((size_t)W.rows * rank + 1) / 2);
        kiln_b200::pack_lora(ac, bc, W.rows, W.cols, adds.data(), (int)adds.size());
        L.a_cat = ac; L.b_cat = bc; L.rank = rank;
        W.lora = &L;
    }
    kiln_b200::linear16(y, ldy, x16, T, W, (kiln_b200::Epi16)(int)epi, gate);
    G.arena.release(m);
}
