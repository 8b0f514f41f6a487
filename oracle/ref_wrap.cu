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
#define main kiln_ref_unused_main
#include "tfa_test.cu"   // ref_attn + flash.cuh + tcflash.cuh (its main() is renamed and never called)
#undef main
#include "kernels.cu"    // k_rmsnorm_warp, k_rope_half (and the op set they belong to)
#include "dit.cu"        // k_nag<T>, cosmos_rope

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

// the reference's fp16-activation GEMM (tc16::launch, engine/src/tcgemm16.cuh:198-201) without the LoRA product;
// epi: 0 fp32 store, 1 fp16 store, 2 fp16 GELU, 3 gated add into fp32 C
static void ref_gemm16(void* C, int ldc, const void* A16, const void* W16, int M, int N, int K, int epi, const float* gate) {
    tc16::Args a;
    a.A = (const __half*)A16; a.W = (const __half*)W16; a.K = K;
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

}  // extern "C"
