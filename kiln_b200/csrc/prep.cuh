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
// HBM-bound: half a warp per (row, head), 8 elements (16 bytes) per lane, one pass at full occupancy.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace kb {

// eight consecutive elements as fp32
struct F8 { float v[8]; };
struct F4 { float v[4]; };
template <typename T> struct Io;
template <> struct Io<float> {
    static __device__ __forceinline__ F4 ld4(const float* p) { const float4 a = *reinterpret_cast<const float4*>(p); return F4{{a.x, a.y, a.z, a.w}}; }
    static __device__ __forceinline__ void st4(float* p, const F4& r) { *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]); }
    static __device__ __forceinline__ F8 ld8(const float* p) {
        F8 r;
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w; r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
        return r;
    }
    static __device__ __forceinline__ void st8(float* p, const F8& r) {
        reinterpret_cast<float4*>(p)[0] = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(r.v[4], r.v[5], r.v[6], r.v[7]);
    }
};
template <> struct Io<__half> {
    static __device__ __forceinline__ F4 ld4(const __half* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        return F4{{a.x, a.y, b.x, b.y}};
    }
    static __device__ __forceinline__ void st4(__half* p, const F4& r) {
        const __half2 a = __floats2half2_rn(r.v[0], r.v[1]), b = __floats2half2_rn(r.v[2], r.v[3]);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
    }
    static __device__ __forceinline__ F8 ld8(const __half* p) {
        F8 r;
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            r.v[2 * i] = f.x; r.v[2 * i + 1] = f.y;
        }
        return r;
    }
    static __device__ __forceinline__ void st8(__half* p, const F8& r) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 h = __floats2half2_rn(r.v[2 * i], r.v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Io<__nv_bfloat16> {
    static __device__ __forceinline__ F4 ld4(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        return F4{{__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u)}};
    }
    static __device__ __forceinline__ void st4(__nv_bfloat16* p, const F4& r) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(r.v[0], r.v[1]), b = __floats2bfloat162_rn(r.v[2], r.v[3]);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
    }
    static __device__ __forceinline__ F8 ld8(const __nv_bfloat16* p) {
        F8 r;
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {   // a bf16 is the top half of an fp32
            r.v[2 * i] = __uint_as_float(w[i] << 16); r.v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
        return r;
    }
    static __device__ __forceinline__ void st8(__nv_bfloat16* p, const F8& r) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(r.v[2 * i], r.v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// One launch stages up to five tensors (Q, K, V, or Q and the four context tensors of NAG).
struct PrepSeg {
    const void* in;              // [rows, ld_in], head h at columns h*128
    void* out;                   // [rows, ld_out]
    const __nv_bfloat16* w;      // RMSNorm weight[128] or null
    const float* cos_t;          // RoPE tables [T, 64] or null; row r uses table row r % T
    const float* sin_t;
    int rows, ld_in, ld_out, T;
    unsigned block0;             // first thread block of this segment in the launch
};
struct PrepParams {
    PrepSeg seg[5];
    int nseg, H;
    float eps;
    unsigned blocks;             // total thread blocks
    unsigned int* zero_ptr;      // optional: zero_n words the first thread block clears (counters and flags that the
    int zero_n;                  // attention kernel launched next on the stream expects at zero)
};

// Measured on B200: a plain one-16-byte-load-per-thread conversion runs at the speed of a device copy
// (101 MB in 18.6 us), and unrolling for more loads in flight buys nothing; what costs bandwidth is
// occupancy and narrow accesses. So: no loop, one pass, 16-byte accesses for 16-bit data everywhere, and a thread
// block belongs to exactly one tensor so the tensor lookup is block-uniform.
//   without RoPE: one (row, head) per half-warp, lane `sub` holds elements [8 sub, 8 sub + 8);
//   with RoPE   : one (row, head) per quarter-warp, lane `sub` holds elements [8 sub, 8 sub + 8) AND their rotation
//                 partners [64 + 8 sub, ...), so the rotation needs no shuffle and each table entry is loaded once.
constexpr int PREP_ITEMS_PER_BLOCK = 16;        // 256 threads / 16 lanes
constexpr int PREP_ITEMS_PER_BLOCK_ROPE = 32;   // 256 threads / 8 lanes

template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
qk_prep_kernel(const __grid_constant__ PrepParams pp) {
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < pp.zero_n; i += 256) pp.zero_ptr[i] = 0u;
    int si = 0;
#pragma unroll
    for (int i = 1; i < 5; i++)
        if (i < pp.nseg && blockIdx.x >= pp.seg[i].block0) si = i;
    const PrepSeg& sg = pp.seg[si];
    if (sg.cos_t) {
        const int sub = threadIdx.x & 7;
        const long long item = (long long)(blockIdx.x - sg.block0) * PREP_ITEMS_PER_BLOCK_ROPE + (threadIdx.x >> 3);
        const bool live = item < (long long)sg.rows * pp.H;  // uniform across a quarter-warp
        const int r = live ? (int)(item / pp.H) : 0, h = live ? (int)(item % pp.H) : 0;
        F8 a, b;
#pragma unroll
        for (int e = 0; e < 8; e++) a.v[e] = b.v[e] = 0.f;
        const InT* src = static_cast<const InT*>(sg.in) + (size_t)r * sg.ld_in + h * 128 + 8 * sub;
        if (live) { a = Io<InT>::ld8(src); b = Io<InT>::ld8(src + 64); }
        if (sg.w) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) ss += a.v[e] * a.v[e] + b.v[e] * b.v[e];
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rs = rsqrtf(ss * (1.f / 128.f) + pp.eps);
            const F8 wa = Io<__nv_bfloat16>::ld8(sg.w + 8 * sub), wb = Io<__nv_bfloat16>::ld8(sg.w + 64 + 8 * sub);
#pragma unroll
            for (int e = 0; e < 8; e++) { a.v[e] = a.v[e] * rs * wa.v[e]; b.v[e] = b.v[e] * rs * wb.v[e]; }
        }
        const size_t tr = (size_t)(r % sg.T) * 64 + 8 * sub;
        const F8 c = Io<float>::ld8(sg.cos_t + tr), s = Io<float>::ld8(sg.sin_t + tr);
        F8 x, y;
#pragma unroll
        for (int e = 0; e < 8; e++) {                         // engine/src/kernels.cu:769-771
            x.v[e] = a.v[e] * c.v[e] - b.v[e] * s.v[e];
            y.v[e] = b.v[e] * c.v[e] + a.v[e] * s.v[e];
        }
        if (live) {
            OutT* dst = static_cast<OutT*>(sg.out) + (size_t)r * sg.ld_out + h * 128 + 8 * sub;
            Io<OutT>::st8(dst, x);
            Io<OutT>::st8(dst + 64, y);
        }
        return;
    }
    const int sub = threadIdx.x & 15;
    const long long item = (long long)(blockIdx.x - sg.block0) * PREP_ITEMS_PER_BLOCK + (threadIdx.x >> 4);
    const bool live = item < (long long)sg.rows * pp.H;      // uniform across a half-warp
    const int r = live ? (int)(item / pp.H) : 0, h = live ? (int)(item % pp.H) : 0;
    // no RoPE: lane `sub` holds elements [8 sub, 8 sub + 8) (16-byte accesses for 16-bit data)
    F8 x;
    if (live) x = Io<InT>::ld8(static_cast<const InT*>(sg.in) + (size_t)r * sg.ld_in + h * 128 + 8 * sub);
    else {
#pragma unroll
        for (int e = 0; e < 8; e++) x.v[e] = 0.f;
    }
    if (sg.w) {                                               // block-uniform
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) ss += x.v[e] * x.v[e];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rs = rsqrtf(ss * (1.f / 128.f) + pp.eps);
        const F8 w = Io<__nv_bfloat16>::ld8(sg.w + 8 * sub);
#pragma unroll
        for (int e = 0; e < 8; e++) x.v[e] = x.v[e] * rs * w.v[e];
    }
    if (live) Io<OutT>::st8(static_cast<OutT*>(sg.out) + (size_t)r * sg.ld_out + h * 128 + 8 * sub, x);
}

}  // namespace kb
