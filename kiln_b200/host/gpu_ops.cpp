// Implementation of the engine-facing op set over the C ABI (see gpu_ops.h for the reference citations).
#include "gpu_ops.h"

#include <chrono>
#include <stdexcept>
#include <string>

#include "kiln_b200.h"

namespace kiln_b200 {

namespace {
OpContext g_ctx;

void check(int rc, const char* what) {
    if (rc != KB_OK) throw std::runtime_error(std::string(what) + ": " + kb_error_string(rc));
}
void need_d128(int Dh, const char* what) {
    // same wording as the reference's attention16 (engine/src/kernels.cu:870)
    if (Dh != 128) throw std::runtime_error(std::string(what) + ": unsupported head size or row stride");
}
}  // namespace

void set_context(const OpContext& ctx) { g_ctx = ctx; }
const OpContext& context() { return g_ctx; }

void attention(float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, int Tq, int Tk,
               int H, int Dh, bool causal, int npad) {
    need_d128(Dh, "attention");
    if (causal) throw std::runtime_error("attention: causal attention is not on the fused path");
    check(kb_attn_cross(out, q, nullptr, k, v, Tq, Tk, npad, H, ldq, ldk, ldv, ldo, KB_F32, KB_F32, 1e-6f, g_ctx.workspace,
                        g_ctx.workspace_bytes, g_ctx.stream),
          "attention");
}

void attention16(__half* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, int Tq, int Tk,
                 int H, int Dh, int npad) {
    need_d128(Dh, "attention16");
    check(kb_attn_cross(out, q, nullptr, k, v, Tq, Tk, npad, H, ldq, ldk, ldv, ldo, KB_F32, KB_F16, 1e-6f, g_ctx.workspace,
                        g_ctx.workspace_bytes, g_ctx.stream),
          "attention16");
}

void rmsnorm(float* y, const float* x, const uint16_t* w_bf16, int rows, int dim, float eps) {
    if (dim != 128) throw std::runtime_error("rmsnorm: only the per-head rows of 128 are on this path");
    // rows of 128 are (token, head) pairs: one "head" per row
    check(kb_qk_prep(y, 128, KB_F32, x, 128, KB_F32, rows, 1, 1, w_bf16, eps, nullptr, nullptr, g_ctx.stream), "rmsnorm");
}

void rope_half(float* x, int T, int H, int Dh, const float* cos_t, const float* sin_t) {
    need_d128(Dh, "rope_half");
    check(kb_qk_prep(x, H * 128, KB_F32, x, H * 128, KB_F32, T, H, T, nullptr, 0.f, cos_t, sin_t, g_ctx.stream), "rope_half");
}

void self_attention16(__half* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, int B, int T,
                      int H, const uint16_t* qn_w, const uint16_t* kn_w, const float* rope_cos, const float* rope_sin, float eps) {
    check(kb_attn_self(out, q, k, v, qn_w, kn_w, rope_cos, rope_sin, B, T, H, ldq, ldk, ldv, ldo, KB_F32, KB_F16, eps,
                       g_ctx.workspace, g_ctx.workspace_bytes, g_ctx.stream),
          "self_attention16");
}

void nag_attention16(__half* out, int ldo, const float* q, int ldq, const uint16_t* qn_w, const float* k_pos, const float* v_pos,
                     int Tk_pos, int npad_pos, const float* k_neg, const float* v_neg, int Tk_neg, int npad_neg, int ld_kv,
                     float scale, float tau, float alpha, int Tq, int H, float eps) {
    check(kb_attn_nag(out, q, qn_w, k_pos, v_pos, Tk_pos, npad_pos, k_neg, v_neg, Tk_neg, npad_neg, scale, tau, alpha, Tq, H, ldq,
                      ld_kv, ldo, KB_F32, KB_F16, eps, g_ctx.workspace, g_ctx.workspace_bytes, g_ctx.stream),
          "nag_attention16");
}

void linear16(void* y, int ldy, const __half* x16, int T, const Weight16& W, Epi16 epi, const float* gate) {
    if (W.rows % 128 || W.cols % 64) throw std::runtime_error("linear16: the weight is not tensor-core eligible");   // engine/src/kernels.cu:560
    check(kb_linear16(y, ldy, x16, W.cols, W.p, W.cols, T, W.rows, W.cols, (int)epi, gate, nullptr, nullptr, nullptr, 0, 0.f, g_ctx.stream),
          "linear16");
}

void linear16_heads(__half* y, int ldy, const __half* x16, int T, const Weight16& W, const uint16_t* norm_w_bf16, const float* rope_cos,
                    const float* rope_sin, int rope_T, float eps) {
    if (W.rows % 128 || W.cols % 64) throw std::runtime_error("linear16: the weight is not tensor-core eligible");
    check(kb_linear16(y, ldy, x16, W.cols, W.p, W.cols, T, W.rows, W.cols, KB_EPI_HEADS16, nullptr, norm_w_bf16, rope_cos, rope_sin, rope_T,
                      eps, g_ctx.stream),
          "linear16_heads");
}

void linear16_qkv(__half* q, __half* k, __half* v, int ldy, const __half* x16, int T, const Weight16& Wq, const Weight16& Wk,
                  const Weight16& Wv, const uint16_t* qn_w_bf16, const uint16_t* kn_w_bf16, const float* rope_cos, const float* rope_sin,
                  int rope_T, float eps) {
    if (Wq.rows % 128 || Wq.cols % 64 || Wk.rows != Wq.rows || Wv.rows != Wq.rows || Wk.cols != Wq.cols || Wv.cols != Wq.cols)
        throw std::runtime_error("linear16_qkv: the three weights must share one tensor-core eligible shape");
    void* const C3[3] = {q, k, v};
    const void* const W3[3] = {Wq.p, Wk.p, Wv.p};
    const void* const hw3[3] = {qn_w_bf16, kn_w_bf16, nullptr};
    const int rope3[3] = {rope_cos != nullptr, rope_cos != nullptr, 0};
    check(kb_linear16_qkv(C3, ldy, x16, Wq.cols, W3, Wq.cols, T, Wq.rows, Wq.cols, hw3, rope3, rope_cos, rope_sin, rope_T, eps, g_ctx.stream),
          "linear16_qkv");
}

}  // namespace kiln_b200

// C trampolines so the shim can be exercised from the test-suite without a C++ test runner:
// each returns 0, or -1 after copying the exception text into `err`.
extern "C" {
static int guard(char* err, int n, void (*fn)(void*), void* arg) {
    try { fn(arg); return 0; }
    catch (const std::exception& e) { if (err && n > 0) { snprintf(err, n, "%s", e.what()); } return -1; }
}
void kbh_set_context(void* stream, void* workspace, size_t bytes) {
    kiln_b200::OpContext c; c.stream = (cudaStream_t)stream; c.workspace = workspace; c.workspace_bytes = bytes;
    kiln_b200::set_context(c);
}
struct A16 { void* out; int ldo; const float *q; int ldq; const float* k; int ldk; const float* v; int ldv; int Tq, Tk, H, Dh, npad; int causal; int f32out; };
int kbh_attention(void* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, int Tq, int Tk, int H,
                  int Dh, int causal, int npad, int f32out, char* err, int n) {
    A16 a{out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, Dh, npad, causal, f32out};
    return guard(err, n, [](void* p) {
        A16& a = *(A16*)p;
        if (a.f32out) kiln_b200::attention((float*)a.out, a.ldo, a.q, a.ldq, a.k, a.ldk, a.v, a.ldv, a.Tq, a.Tk, a.H, a.Dh, a.causal != 0, a.npad);
        else kiln_b200::attention16((__half*)a.out, a.ldo, a.q, a.ldq, a.k, a.ldk, a.v, a.ldv, a.Tq, a.Tk, a.H, a.Dh, a.npad);
    }, &a);
}
struct NR { float* x; const uint16_t* w; int rows, T, H; float eps; const float *c, *s; };
int kbh_rmsnorm_rope(float* x, const uint16_t* w, int T, int H, float eps, const float* c, const float* s, char* err, int n) {
    NR a{x, w, T * H, T, H, eps, c, s};
    return guard(err, n, [](void* p) {
        NR& a = *(NR*)p;
        kiln_b200::rmsnorm(a.x, a.x, a.w, a.rows, 128, a.eps);
        kiln_b200::rope_half(a.x, a.T, a.H, 128, a.c, a.s);
    }, &a);
}
struct L16 { void* y; int ldy; const void* x; int T; const void* w; int rows, cols, epi; const float* gate; const uint16_t* nw; const float *c, *s; int rope_T; float eps; };
int kbh_linear16(void* y, int ldy, const void* x16, int T, const void* w16, int rows, int cols, int epi, const float* gate,
                 const uint16_t* norm_w, const float* c, const float* s, int rope_T, float eps, char* err, int n) {
    L16 a{y, ldy, x16, T, w16, rows, cols, epi, gate, norm_w, c, s, rope_T, eps};
    return guard(err, n, [](void* p) {
        L16& a = *(L16*)p;
        kiln_b200::Weight16 W; W.p = (const __half*)a.w; W.rows = a.rows; W.cols = a.cols;
        if (a.epi == 4) kiln_b200::linear16_heads((__half*)a.y, a.ldy, (const __half*)a.x, a.T, W, a.nw, a.c, a.s, a.rope_T, a.eps);
        else kiln_b200::linear16(a.y, a.ldy, (const __half*)a.x, a.T, W, (kiln_b200::Epi16)a.epi, a.gate);
    }, &a);
}
// Host cost of enqueueing one fp16 cross-attention call through the C ABI (argument checks, four tensor-map encodes, one
// launch), in microseconds: wall clock around n back-to-back calls that are not waited for, then one synchronise.
double kbh_enqueue_cost_us(void* out, const void* q, const void* k, const void* v, int Tq, int Tk, int npad, int H, int n) {
    const int ld = H * 128;
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < n; i++)
        if (kb_attn_cross(out, q, nullptr, k, v, Tq, Tk, npad, H, ld, ld, ld, ld, KB_F16, KB_F16, 1e-6f, nullptr, 0, nullptr) != KB_OK) return -1.0;
    const auto t1 = std::chrono::steady_clock::now();
    cudaStreamSynchronize(nullptr);
    return std::chrono::duration<double, std::micro>(t1 - t0).count() / n;
}
}
