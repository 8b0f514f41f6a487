// Row pre-pass for Q and K: per (token, head) RMSNorm with a bf16 weight[128] and rotate-half RoPE,
// written once as 16-bit operands for the attention kernel. It restates, fused into one pass,
//   k_rmsnorm_warp  engine/src/kernels.cu:656-666   y = x * rsqrt(mean(x^2) + eps) * w
//   k_rope_half     engine/src/kernels.cu:759-772   pairs (i, i+64): a*c - b*s, b*c + a*s, tables [T, 64]
// in the reference's order (norm, then RoPE; engine/src/dit.cu:464-468). With neither norm nor RoPE
// it is the fp32 -> 16-bit staging conversion the reference does inside its kernel
// (engine/src/tcflash.cuh:56-64).
// The attention kernel's tensor-core operands are always fp16 (as in the reference, which converts to
// fp16 while staging): bf16 and fp32 inputs are converted here, fp16 inputs that need neither norm nor
// RoPE skip this pass entirely.
// HBM-bound: one warp per (row, head), 4 elements per lane, fully coalesced 128-byte segments.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace kb {

template <typename T> struct Io;
template <> struct Io<float> {
    static __device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void st2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Io<__half> {
    static __device__ __forceinline__ float2 ld2(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
    static __device__ __forceinline__ void st2(__half* p, float a, float b) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b); }
};
template <> struct Io<__nv_bfloat16> {
    static __device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
    static __device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
};

// One launch stages up to five tensors (Q, K, V, or Q and the four context tensors of NAG).
struct PrepSeg {
    const void* in;              // [rows, ld_in], head h at columns h*128
    void* out;                   // [rows, ld_out]
    const __nv_bfloat16* w;      // RMSNorm weight[128] or null
    const float* cos_t;          // RoPE tables [T, 64] or null; row r uses table row r % T
    const float* sin_t;
    int rows, ld_in, ld_out, T;
    long long item0;             // first (row, head) item of this segment in the launch
};
struct PrepParams {
    PrepSeg seg[5];
    int nseg, H;
    float eps;
    long long items;             // total (row, head) items
};

template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
qk_prep_kernel(const PrepParams pp) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= pp.items) return;
    int si = 0;
#pragma unroll
    for (int i = 1; i < 5; i++)
        if (i < pp.nseg && item >= pp.seg[i].item0) si = i;
    const PrepSeg& sg = pp.seg[si];
    const long long local = item - sg.item0;
    const int r = (int)(local / pp.H), h = (int)(local % pp.H);
    const InT* src = static_cast<const InT*>(sg.in) + (size_t)r * sg.ld_in + h * 128;
    float2 a = Io<InT>::ld2(src + 2 * lane);            // elements 2l, 2l+1
    float2 b = Io<InT>::ld2(src + 64 + 2 * lane);       // elements 64+2l, 65+2l: the RoPE partners
    if (sg.w) {
        float ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rs = rsqrtf(ss * (1.f / 128.f) + pp.eps);
        const float2 wa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sg.w + 2 * lane));
        const float2 wb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sg.w + 64 + 2 * lane));
        a.x = a.x * rs * wa.x; a.y = a.y * rs * wa.y;
        b.x = b.x * rs * wb.x; b.y = b.y * rs * wb.y;
    }
    if (sg.cos_t) {
        const size_t tr = (size_t)(r % sg.T) * 64 + 2 * lane;
        const float2 c = *reinterpret_cast<const float2*>(sg.cos_t + tr);
        const float2 s = *reinterpret_cast<const float2*>(sg.sin_t + tr);
        const float ax = a.x * c.x - b.x * s.x, bx = b.x * c.x + a.x * s.x;
        const float ay = a.y * c.y - b.y * s.y, by = b.y * c.y + a.y * s.y;
        a.x = ax; a.y = ay; b.x = bx; b.y = by;
    }
    OutT* dst = static_cast<OutT*>(sg.out) + (size_t)r * sg.ld_out + h * 128;
    Io<OutT>::st2(dst + 2 * lane, a.x, a.y);
    Io<OutT>::st2(dst + 64 + 2 * lane, b.x, b.y);
}

}  // namespace kb
