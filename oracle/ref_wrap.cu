// GPU-side oracle: the reference's OWN kernels, compiled for sm_100a from the reference tree.
//
// TEST INFRASTRUCTURE ONLY. This translation unit contains no reference code; it #includes the
// reference's source files by path (given with -I at build time, see oracle/build.py) and exports
// thin extern "C" launchers so tests and the benchmark can run, on the same device buffers:
//   * ref_attn        bench/tfa_test.cu:11-33        fp32 two-pass attention (the harness's own reference)
//   * tfa::launch     engine/src/tcflash.cuh:161-167 the mma.sync FlashAttention-2 kernel (the kernel to beat)
//   * k_rmsnorm_warp  engine/src/kernels.cu:656-666
//   * k_rope_half     engine/src/kernels.cu:759-772
//   * k_nag<T>        engine/src/dit.cu:295-324
//   * cosmos_rope     engine/src/dit.cu:196-215      (host table builder)
// All launches go to the legacy default stream, as the reference's harness does (bench/tfa_test.cu:49-56).
// Every function returns cudaGetLastError() as an int (0 = ok).
//   * Dit::forward_batch  engine/src/dit.cu:356-545  the reference's own DiT driver (kref_dit_* below): blocks of
//                         layernorm_mod16 -> linear16 q/k/v -> rmsnorm -> rope_half -> attention16 -> linear16(Resid), cross
//                         attention against cache_context's K/V (dit.cu:217-234), NAG, MLP.
//
// Built twice. As it is: the reference's driver over the reference's ops (oracle/_ref/libkiln_ref.so). With
// -DKILN_OPS_FROM_SHIM: the SAME driver source, with the five ops of the attention path - attention, attention16,
// rmsnorm, rope_half, linear16 - taken from kiln_b200/host/gpu_ops.h instead (oracle/_ref/libkiln_ref_shim.so). The
// reference's definitions are renamed while kernels.cu is read and stay reachable as ref_own_*: the bound ops fall back
// to them for what the library does not cover (head sizes other than 128, causal attention, bf16 weights still to convert),
// which is how an engine maintainer would bind the library.
#ifdef KILN_OPS_FROM_SHIM
#define attention ref_own_attention
#define attention16 ref_own_attention16
#define rmsnorm ref_own_rmsnorm
#define rope_half ref_own_rope_half
#define linear16 ref_own_linear16
#endif
#include <functional>
#define main kiln_ref_unused_main
#include "tfa_test.cu"   // ref_attn + flash.cuh + tcflash.cuh (its main() is renamed and never called)
#undef main
#include "kernels.cu"    // k_rmsnorm_warp, k_rope_half (and the op set they belong to)
#ifdef KILN_OPS_FROM_SHIM
#undef attention
#undef attention16
#undef rmsnorm
#undef rope_half
#undef linear16
#include "ref_ops_binding.h"
#endif
#include "dit.cu"        // k_nag<T>, cosmos_rope, Dit::forward_batch
// The LoRA trainer's file defines the same model constants as dit.cu (each is its own translation unit in the engine): rename them
// while it is read. Wanted from it: attention_bwd (engine/src/train.cu:216-242), the exact attention backward.
#define D kref_train_D
#define NH kref_train_NH
#define DH kref_train_DH
#define FF kref_train_FF
#define EPS kref_train_EPS
#include "train.cu"
#undef D
#undef NH
#undef DH
#undef FF
#undef EPS

// The symbols the included files need from the reference's Win32-only loader; never reached here.
float st_elem_f32(const StTensor&, int64_t) { return 0.f; }
SafeTensors::SafeTensors(const std::string& path) : path_(path) {}
SafeTensors::~SafeTensors() {}
const StTensor& SafeTensors::get(const std::string&) const { static StTensor none; return none; }
void rope_table(std::vector<float>&, std::vector<float>&, int, int, float) {}  // text-encoder table (engine/src/te.cu), unused here

extern "C" {

int kref_ref_attn(float* out, const float* q, const float* k, const float* v, int T, int Tk, int H, int ld, int npad) {
    ref_attn<<<(T * H + 127) / 128, 128>>>(out, q, k, v, T, Tk, H, ld, npad);
    return (int)cudaGetLastError();
}

int kref_tfa_f32(float* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                 int Tq, int Tk, int H, int npad) {
    if (!tfa::eligible(128, ldq, ldk, ldv, ldo)) return -1;
    tfa::launch<float>(out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, npad, 0);
    return (int)cudaGetLastError();
}

int kref_tfa_f16(void* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                 int Tq, int Tk, int H, int npad) {
    if (!tfa::eligible(128, ldq, ldk, ldv, ldo)) return -1;
    tfa::launch<__half>((__half*)out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, npad, 0);
    return (int)cudaGetLastError();
}

// average milliseconds of `reps` back-to-back tfa launches (fp16 output) after `warm` warm-ups
float kref_time_tfa_f16(void* out, int ldo, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                        int Tq, int Tk, int H, int npad, int warm, int reps) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < warm; i++) tfa::launch<__half>((__half*)out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, npad, 0);
    cudaEventRecord(e0);
    for (int i = 0; i < reps; i++) tfa::launch<__half>((__half*)out, ldo, q, ldq, k, ldk, v, ldv, Tq, Tk, H, npad, 0);
    cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms = 0.f; cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return cudaGetLastError() == cudaSuccess ? ms / reps : -1.f;
}

// the reference's fp16-activation GEMM (tc16::launch, engine/src/tcgemm16.cuh:198-201); A2 / W2 / K2 are the LoRA
// second product as linear16 hands it over (engine/src/kernels.cu:596), null / 0 for none;
// epi: 0 fp32 store, 1 fp16 store, 2 fp16 GELU, 3 gated add into fp32 C
static void ref_gemm16(void* C, int ldc, const void* A16, const void* W16, int M, int N, int K, int epi, const float* gate,
                       const void* A2 = nullptr, const void* W2 = nullptr, int K2 = 0) {
    tc16::Args a;
    a.A = (const __half*)A16; a.W = (const __half*)W16; a.K = K;
    a.A2 = (const __half*)A2; a.W2 = (const __half*)W2; a.K2 = K2;
    a.C = C; a.ldc = ldc; a.gate = gate; a.M = M; a.N = N;
    switch (epi) {
        case 0: tc16::launch<tc16::EPI_F32>(a, 0, 100); break;
        case 1: tc16::launch<tc16::EPI_F16>(a, 0, 100); break;
        case 2: tc16::launch<tc16::EPI_GELU16>(a, 0, 100); break;
        default: tc16::launch<tc16::EPI_RESID>(a, 0, 100); break;
    }
}

int kref_linear16(void* C, int ldc, const void* A16, const void* W16, int M, int N, int K, int epi, const float* gate) {
    if (!tc16::eligible(M, N, K) || epi < 0 || epi > 3) return -1;
    ref_gemm16(C, ldc, A16, W16, M, N, K, epi, gate);
    return (int)cudaGetLastError();
}

// the same kernel with the second product: A2 fp16 [M, K2], W2 fp16 [N, K2], K2 a multiple of the reference's k tile
int kref_linear16_lora(void* C, int ldc, const void* A16, const void* W16, const void* A2, const void* W2, int K2, int M, int N, int K,
                       int epi, const float* gate) {
    if (!tc16::eligible(M, N, K) || epi < 0 || epi > 3 || K2 <= 0 || K2 % tc16::BK) return -1;
    ref_gemm16(C, ldc, A16, W16, M, N, K, epi, gate, A2, W2, K2);
    return (int)cudaGetLastError();
}

// k_lora_pack (engine/src/kernels.cu:548-554): dst[r * ld + col0 + c] = fp16(scale * src[r, c]), src bf16 [rows, cols]
int kref_lora_pack(void* dst16, int ld, int col0, const uint16_t* src_bf16, int rows, int cols, float scale) {
    k_lora_pack<<<nblk((size_t)rows * cols), 256>>>((__half*)dst16, ld, col0, src_bf16, rows, cols, scale);
    return (int)cudaGetLastError();
}

// average milliseconds of `reps` back-to-back launches after `warm` warm-ups
float kref_time_linear16(void* C, int ldc, const void* A16, const void* W16, int M, int N, int K, int epi, const float* gate,
                         int warm, int reps) {
    if (!tc16::eligible(M, N, K) || epi < 0 || epi > 3) return -1.f;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < warm; i++) ref_gemm16(C, ldc, A16, W16, M, N, K, epi, gate);
    cudaEventRecord(e0);
    for (int i = 0; i < reps; i++) ref_gemm16(C, ldc, A16, W16, M, N, K, epi, gate);
    cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms = 0.f; cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return cudaGetLastError() == cudaSuccess ? ms / reps : -1.f;
}

int kref_rmsnorm(float* y, const float* x, const uint16_t* w_bf16, int rows, int dim, float eps) {
    if (dim > 256) return -1;
    k_rmsnorm_warp<<<nblk(rows, 8), 256>>>(y, x, w_bf16, rows, dim, eps);
    return (int)cudaGetLastError();
}

int kref_rope_half(float* x, int T, int H, int Dh, const float* cos_t, const float* sin_t) {
    size_t n = (size_t)T * H * (Dh / 2);
    k_rope_half<<<nblk(n), 256>>>(x, T, H, Dh, cos_t, sin_t);
    return (int)cudaGetLastError();
}

int kref_nag_f32(float* a, const float* an, int T, int dim, float s, float tau, float alpha) {
    k_nag<float><<<(unsigned)T, 256>>>(a, an, dim, s, tau, alpha);
    return (int)cudaGetLastError();
}

int kref_nag_f16(void* a, const void* an, int T, int dim, float s, float tau, float alpha) {
    k_nag<__half><<<(unsigned)T, 256>>>((__half*)a, (const __half*)an, dim, s, tau, alpha);
    return (int)cudaGetLastError();
}

// host tables [Hp*Wp, 64] each
int kref_cosmos_rope(float* c, float* s, int Hp, int Wp) {
    std::vector<float> cv, sv;
    cosmos_rope(cv, sv, Hp, Wp);
    memcpy(c, cv.data(), cv.size() * 4);
    memcpy(s, sv.data(), sv.size() * 4);
    return 0;
}

int kref_sync() { return (int)cudaDeviceSynchronize(); }

// attention_bwd (engine/src/train.cu:216-242): q [Tq, 2048], k, v [Tk, 2048], dout [Tq, 2048] fp32 -> dq, dk, dv (16 heads of 128;
// five cuBLAS SGEMMs per head group + k_softmax_pad / k_dsoftmax). Needs kref_engine_init (the arena holds P and dP).
int kref_attention_bwd(float* dq, float* dk, float* dv, const float* q, const float* k, const float* v, const float* dout, int Tq, int Tk,
                       int npad, char* err, int n) {
    try { attention_bwd(dq, dk, dv, q, k, v, dout, Tq, Tk, npad); gpu_sync(); return 0; }
    catch (const std::exception& e) { if (err && n > 0) snprintf(err, n, "%s", e.what()); return -1; }
}

// ------------------------------------------------------------------ the reference's DiT driver on seeded random weights
// p[i] = bf16(bias + amp * u), u uniform in (-1, 1) from a hash of (seed, i): the same weights in every build of this file
__global__ void k_fill_bf16(uint16_t* p, size_t n, uint32_t seed, float amp, float bias) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t h = (uint32_t)i * 2654435761u ^ (uint32_t)(i >> 32) ^ (seed * 0x9E3779B9u);
    h ^= h >> 16; h *= 0x7feb352du; h ^= h >> 15; h *= 0x846ca68bu; h ^= h >> 16;
    const float u = ((float)(h >> 8) + 0.5f) * (2.f / 16777216.f) - 1.f;
    p[i] = __bfloat16_as_ushort(__float2bfloat16_rn(bias + amp * u));
}

static Weight make_weight(int rows, int cols, uint32_t seed, float amp, float bias = 0.f) {
    Weight w;
    const size_t n = (size_t)rows * cols;
    CK(cudaMalloc(&w.p, n * 2));
    w.rows = rows; w.cols = cols;
    k_fill_bf16<<<nblk(n), 256, 0, G.stream>>>(w.p, n, seed, amp, bias);
    return w;
}

static int guarded(char* err, int n, const std::function<void()>& fn) {
    try { fn(); return 0; }
    catch (const std::exception& e) { if (err && n > 0) snprintf(err, n, "%s", e.what()); return -1; }
}

// the engine's start-up (gpu_init, engine/src/kernels.cu:206-221) with the fp16-activation path switched on instead of raced
int kref_engine_init(size_t arena_bytes, char* err, int n) {
    return guarded(err, n, [&] {
        if (G.stream) return;
        setenv("KILN_TC16", "1", 1);
        gpu_init(0);
        gpu_alloc_scratch((size_t)8192 * 2048, arena_bytes);
    });
}

// exact != 0: the engine's exact mode (G.fp16 = false: fp32 cuBLAS GEMMs and the exact attention path, engine/src/gpu.h:76) -
// the yardstick both fp16-activation builds are measured against
void kref_set_exact(int exact) { G.fp16 = !exact; }

// A Dit of `nblocks` blocks with uniform random weights of variance 1/in (norm weights 1 +- 0.1), GEMM weights converted
// to fp16 as Dit::load does (half_weights, engine/src/dit.cu:99-104). with_lora: unmerged LoRAs on block 0's self-attention
// q projection (ranks 8 + 16) and cross-attention output projection (rank 16), as lora.cu would attach them.
void* kref_dit_create(int nblocks, unsigned seed, int with_lora, char* err, int n) {
    Dit* d = nullptr;
    const int rc = guarded(err, n, [&] {
        d = new Dit();
        uint32_t s = seed * 1000u;
        auto W = [&](int rows, int cols, float gain = 1.f) { return make_weight(rows, cols, ++s, gain * sqrtf(3.f / (float)cols)); };
        auto Nw = [&](int dim) { return make_weight(1, dim, ++s, 0.1f, 1.f); };
        d->blocks.resize(nblocks);
        for (auto& b : d->blocks) {
            b.sa_q = W(D, D); b.sa_k = W(D, D); b.sa_v = W(D, D); b.sa_o = W(D, D); b.sa_qn = Nw(DH); b.sa_kn = Nw(DH);
            b.ca_q = W(D, D); b.ca_k = W(D, AD); b.ca_v = W(D, AD); b.ca_o = W(D, D); b.ca_qn = Nw(DH); b.ca_kn = Nw(DH);
            b.mlp1 = W(4 * D, D); b.mlp2 = W(D, 4 * D);
            b.mod_sa1 = W(256, D); b.mod_sa2 = W(3 * D, 256); b.mod_ca1 = W(256, D); b.mod_ca2 = W(3 * D, 256);
            b.mod_mlp1 = W(256, D); b.mod_mlp2 = W(3 * D, 256);
        }
        d->x_embed = W(D, 68); d->t_lin1 = W(D, D); d->t_lin2 = W(3 * D, D, 0.3f); d->t_norm = Nw(D);
        d->final_mod1 = W(256, D); d->final_mod2 = W(2 * D, 256); d->final_lin = W(64, D);
        if (with_lora) {
            auto& b = d->blocks[0];
            b.sa_q.lora = new std::vector<LoraAdd>{{W(8, D), W(D, 8), 1.5f}, {W(16, D), W(D, 16), -0.75f}};
            b.ca_o.lora = new std::vector<LoraAdd>{{W(16, D), W(D, 16), 2.0f}};
        }
        d->half_weights();
        gpu_sync();
    });
    return rc == 0 ? d : nullptr;
}

// forward_batch (engine/src/dit.cu:356) of one latent [16, Hl, Wl] under B contexts [len_b, 1024] of which real_b rows are
// text; cache_mask bit b: context b goes through cache_context (dit.cu:217) first, else its K/V are made per block
// (dit.cu:407-413). nag_ctx != null: NAG on batch item 0 with that negative context (bit 2 of cache_mask caches it).
// outs[b] [16, Hl, Wl]. Everything device memory of the caller.
int kref_dit_forward(void* dit, float* const* outs, const float* latent, int Hl, int Wl, float t, const float* const* ctx, const int* len,
                     const int* real, int B, const float* nag_ctx, int nag_len, int nag_real, float nag_scale, float nag_tau,
                     float nag_alpha, int cache_mask, char* err, int n) {
    return guarded(err, n, [&] {
        Dit& d = *(Dit*)dit;
        const size_t m = G.arena.mark();
        std::vector<Context> cs(B);
        std::vector<const Context*> cp(B);
        for (int b = 0; b < B; b++) { cs[b].p = const_cast<float*>(ctx[b]); cs[b].len = len[b]; cs[b].real = real[b]; cp[b] = &cs[b]; }
        Context neg;
        d.drop_context_cache();
        for (int b = 0; b < B; b++) if (cache_mask >> b & 1) d.cache_context(cs[b]);
        d.nag = Dit::Nag();
        if (nag_ctx) {
            neg.p = const_cast<float*>(nag_ctx); neg.len = nag_len; neg.real = nag_real;
            if (cache_mask >> 2 & 1) d.cache_context(neg);
            d.nag.neg = &neg; d.nag.scale = nag_scale; d.nag.tau = nag_tau; d.nag.alpha = nag_alpha;
        }
        d.forward_batch(outs, latent, Hl, Wl, t, cp.data(), B);
        gpu_sync();
        d.nag = Dit::Nag();
        d.drop_context_cache();
        G.arena.release(m);
    });
}

}  // extern "C"
