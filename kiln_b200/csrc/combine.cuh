// Stand-alone NAG combine and the arrival wait used by head-split runs.
//
// nag_combine_kernel restates k_nag (engine/src/dit.cu:295-324) as a single pass: a block per token row
// keeps the row of Z+ and Z- in registers, reduces |Z+|_1 and |g|_1 over ALL channels of the row, then
// writes a <- alpha * g * min(1, tau / ratio) + (1 - alpha) * Z+. Three HBM passes (read a, read an, write a)
// instead of the reference's five. It is the drop-in for the engine's k_nag launch and the blend step of
// head-split NAG, where Z+ and Z- are gathered from all GPUs first.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "prep.cuh"
#include "ptx.cuh"

namespace kb {

constexpr int NAG_MAX_CHUNKS = 4;   // 256 threads x 8 elements x 4 = rows of up to 8192 channels

template <typename T>
__global__ void __launch_bounds__(256)
nag_combine_kernel(T* __restrict__ a, const T* __restrict__ an, int dim, int lda, int ldn, float s, float tau, float alpha) {
    T* p = a + (size_t)blockIdx.x * lda;
    const T* n = an + (size_t)blockIdx.x * ldn;
    __shared__ float red[2][8];
    F8 pv[NAG_MAX_CHUNKS], gv[NAG_MAX_CHUNKS];
    float lp = 0.f, lg = 0.f;
    const float sm1 = s - 1.f;
#pragma unroll
    for (int c = 0; c < NAG_MAX_CHUNKS; c++) {
        const int i = (c * 256 + threadIdx.x) * 8;
        if (i < dim) {
            pv[c] = Io<T>::ld8(p + i);
            const F8 nv = Io<T>::ld8(n + i);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                gv[c].v[e] = pv[c].v[e] * s - nv.v[e] * sm1;
                lp += fabsf(pv[c].v[e]);
                lg += fabsf(gv[c].v[e]);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { lp += __shfl_xor_sync(0xffffffffu, lp, o); lg += __shfl_xor_sync(0xffffffffu, lg, o); }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = lp; red[1][threadIdx.x >> 5] = lg; }
    __syncthreads();
    float tp = 0.f, tg = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) { tp += red[0][w]; tg += red[1][w]; }   // same order in every thread
    const float ratio = tg / fmaxf(tp, 1e-12f);
    const float k = ratio > tau ? tau / ratio : 1.f;
    const float ag = alpha * k, ap = 1.f - alpha;
#pragma unroll
    for (int c = 0; c < NAG_MAX_CHUNKS; c++) {
        const int i = (c * 256 + threadIdx.x) * 8;
        if (i < dim) {
            F8 o;
#pragma unroll
            for (int e = 0; e < 8; e++) o.v[e] = ag * gv[c].v[e] + ap * pv[c].v[e];
            Io<T>::st8(p + i, o);
        }
    }
}

// One thread waits (bounded) until *ctr >= target: every tile of every GPU has landed in this GPU's buffer.
// Peers bump the counter with system-scope atomics after a system-scope fence; kernels launched after this
// one on the same stream may read the gathered rows.
__global__ void wait_arrivals_kernel(const unsigned long long* ctr, unsigned long long target, unsigned int* status, unsigned int err_bit) {
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
        if (v >= target) return;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { atomicOr(status, err_bit); return; }
        __nanosleep(200);
    }
}

// One thread per listed counter adds 1 with system scope after a system-scope fence: "this GPU has finished what came
// before this kernel on its stream" - the release side of the buffer-reuse protocol of head-split runs.
struct BumpList {
    unsigned long long* ctr[8];
    int n;
};
__global__ void bump_counters_kernel(const BumpList bl) {
    if ((int)threadIdx.x < bl.n) {
        __threadfence_system();
        atomicAdd_system(bl.ctr[threadIdx.x], 1ull);
    }
}

}  // namespace kb
