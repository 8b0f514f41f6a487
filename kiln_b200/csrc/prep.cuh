// Row pre-pass for Q and K: per (token, head) RMSNorm with a bf16 weight[128] and rotate-half RoPE,
// written once as 16-bit operands for the attention kernel. It restates, fused into one pass,
//   k_rmsnorm_warp  engine/src/kernels.cu:656-666   y = x * rsqrt(mean(x^2) + eps) * w
//   k_rope_half     engine/src/kernels.cu:759-772   pairs (i, i+64): a*c - b*s, b*c + a*s, tables [T, 64]
// in the reference's order (norm, then RoPE; engine/src/dit.cu:464-468). With neither norm nor RoPE
// it is the fp32 -> 16-bit staging conversion the reference does inside its kernel
// (engine/src/tcflash.cuh:56-64).
// HBM-bound: one warp per (row, head), 4 elements per lane, fully coalesced 128-byte segments.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace kb {

template <typename T> struct Io;
template <> struct Io<float> {
    static __device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Io<__half> {
    static __device__ __forceinline__ float2 ld2(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
    static __device__ __forceinline__ void st2(__half* p, float a, float b) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b); }
};
template <> struct Io<__nv_bfloat16> {
    static __device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
    static __device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
};

// in [R, ld_in] (head h at columns h*128), out [R, ld_out]; w = bf16 weight[128] or null;
// cos_t/sin_t = fp32 [T, 64] or null, row r uses table row r % T.
template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
qk_prep_kernel(OutT* __restrict__ out, int ld_out, const InT* __restrict__ in, int ld_in, int R, int H, int T,
               const __nv_bfloat16* __restrict__ w, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (long long)R * H) return;
    const int r = (int)(item / H), h = (int)(item % H);
    const InT* src = in + (size_t)r * ld_in + h * 128;
    float2 a = Io<InT>::ld2(src + 2 * lane);            // elements 2l, 2l+1
    float2 b = Io<InT>::ld2(src + 64 + 2 * lane);       // elements 64+2l, 65+2l: the RoPE partners
    if (w) {
        float ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rs = rsqrtf(ss * (1.f / 128.f) + eps);
        const float2 wa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + 2 * lane));
        const float2 wb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + 64 + 2 * lane));
        a.x = a.x * rs * wa.x; a.y = a.y * rs * wa.y;
        b.x = b.x * rs * wb.x; b.y = b.y * rs * wb.y;
    }
    if (cos_t) {
        const size_t tr = (size_t)(r % T) * 64 + 2 * lane;
        const float2 c = *reinterpret_cast<const float2*>(cos_t + tr);
        const float2 s = *reinterpret_cast<const float2*>(sin_t + tr);
        const float ax = a.x * c.x - b.x * s.x, bx = b.x * c.x + a.x * s.x;
        const float ay = a.y * c.y - b.y * s.y, by = b.y * c.y + a.y * s.y;
        a.x = ax; a.y = ay; b.x = bx; b.y = by;
    }
    OutT* dst = out + (size_t)r * ld_out + h * 128;
    Io<OutT>::st2(dst + 2 * lane, a.x, a.y);
    Io<OutT>::st2(dst + 64 + 2 * lane, b.x, b.y);
}

}  // namespace kb
