// Start-up known-answer test: each kernel family on a small seeded problem against a plain
// one-thread-per-(row, head) fp32 kernel. It follows the idea of the reference's start-up cross-check of
// its tensor-core GEMM against its plain GEMM (engine/src/kernels.cu:106-151, 192-202): a fast path is
// only trusted on a GPU where it reproduces the simple one. The plain kernels here restate the
// arithmetic of bench/tfa_test.cu:11-33 (attention with npad) and engine/src/dit.cu:295-324 (NAG).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace kb {

__device__ __forceinline__ float hash_unit(uint32_t x) {  // (-1, 1), deterministic
    x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
    return (float)(x & 0xffffff) * (2.0f / 16777216.0f) - 1.0f;
}

template <typename T>
__global__ void sc_fill_kernel(T* x, size_t n, uint32_t seed, float amp) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = amp * (hash_unit((uint32_t)i * 2654435761u + seed) + hash_unit((uint32_t)i * 40503u + seed * 31u + 7u));
    if constexpr (sizeof(T) == 4) x[i] = v;
    else if constexpr (std::is_same<T, __half>::value) x[i] = __float2half_rn(v);
    else x[i] = __float2bfloat16_rn(v);
}

template <typename T> __device__ __forceinline__ float sc_ld(const T* p) {
    if constexpr (std::is_same<T, __half>::value) return __half2float(*p);
    else return __bfloat162float(*p);
}

template <typename T>
__global__ void sc_naive_attn_kernel(float* out, const T* q, const T* k, const T* v, int Tq, int Tk, int H, int ld, int npad) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Tq * H) return;
    int t = i / H, h = i % H;
    const T* qr = q + (size_t)t * ld + h * 128;
    const float scale = 0.08838834764831845f;
    float m = npad ? 0.f : -INFINITY;
    for (int j = 0; j < Tk; j++) {
        const T* kr = k + (size_t)j * ld + h * 128;
        float s = 0.f;
        for (int d = 0; d < 128; d++) s += sc_ld(qr + d) * sc_ld(kr + d);
        m = fmaxf(m, s * scale);
    }
    float l = npad * expf(-m);
    float* o = out + (size_t)t * ld + h * 128;
    for (int d = 0; d < 128; d++) o[d] = 0.f;
    for (int j = 0; j < Tk; j++) {
        const T* kr = k + (size_t)j * ld + h * 128;
        const T* vr = v + (size_t)j * ld + h * 128;
        float s = 0.f;
        for (int d = 0; d < 128; d++) s += sc_ld(qr + d) * sc_ld(kr + d);
        float p = expf(s * scale - m);
        l += p;
        for (int d = 0; d < 128; d++) o[d] += p * sc_ld(vr + d);
    }
    for (int d = 0; d < 128; d++) o[d] /= l;
}

// one thread per token row (tiny problem sizes only)
__global__ void sc_naive_nag_kernel(float* a, const float* an, int T, int dim, float s, float tau, float alpha) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    float* p = a + (size_t)t * dim;
    const float* n = an + (size_t)t * dim;
    float lp = 0.f, lg = 0.f;
    for (int i = 0; i < dim; i++) { lp += fabsf(p[i]); lg += fabsf(p[i] * s - n[i] * (s - 1.f)); }
    float ratio = lg / fmaxf(lp, 1e-12f);
    float kc = ratio > tau ? tau / ratio : 1.f;
    for (int i = 0; i < dim; i++) p[i] = alpha * (p[i] * s - n[i] * (s - 1.f)) * kc + (1.f - alpha) * p[i];
}

// max |a-b| into *out (non-negative floats order like their bit patterns); NaN counts as a huge error
__global__ void sc_maxdiff_kernel(const float* a, const float* b, size_t n, unsigned int* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float d = fabsf(a[i] - b[i]);
    if (!(d == d)) d = 1e30f;
    atomicMax(out, __float_as_uint(d));
}

}  // namespace kb
