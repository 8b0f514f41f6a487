// fp16 GEMM for the projections around attention on sm_100a: C = epilogue(A[M,K] * W[N,K]^T), fp32 accumulation
// in TMEM, TMA-fed tcgen05 MMAs, persistent CTAs with two accumulator buffers so that the epilogue of one tile runs
// under the main loop of the next.
//
// Two shapes of the same kernel. PAIR: two CTAs of a cluster share one 256x256 tile through cta_group::2 MMAs; each
// loads its own 128 rows of A and 128 of the 256 W rows per 64-wide k step (32 KiB) and keeps its 128x256 half of the
// accumulator, so a CTA moves half the shared-memory bytes per flop of the single-CTA shape. That matters because
// measured on B200 a 128x128 single-CTA tile is bound by shared-memory bandwidth (TMA writes plus operand reads,
// about 100 B/clk/SM), not by the tensor pipe. Single: one CTA per 128x128 tile, for N not a multiple of 256 or M <= 128.
//
// It takes the place of the reference's fp16-activation GEMM tc16::k_gemm16 (engine/src/tcgemm16.cuh:57-175,
// host wrapper linear16 at engine/src/kernels.cu:559-609) with its four epilogues — fp32 store, fp16 store,
// fp16 GELU, gated add into the fp32 residual stream (engine/src/tcgemm16.cuh:145-174) — and adds a fifth that the
// attention path wants: EPI_HEADS16 treats every 128 output columns as one attention head and applies the
// per-head RMSNorm (engine/src/kernels.cu:656-666) and rotate-half RoPE (engine/src/kernels.cu:759-772) to the
// accumulator row before storing fp16. A thread of the epilogue owns one token row of one head (tcgen05.ld
// 32x32b), so both are thread-local. With it the Q and K projections emit exactly what the attention kernel
// consumes, and the separate rmsnorm / rope_half launches and the staging pre-pass disappear.
// (The reference accumulates each 32-wide k tile in fp16 before flushing to fp32; here every product is
// accumulated in fp32.)
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "attn_sm100.cuh"   // pack16, store32, ST_TIMEOUT
#include "ptx.cuh"

namespace kb {

constexpr int EPI_F32 = 0, EPI_F16 = 1, EPI_GELU16 = 2, EPI_RESID = 3, EPI_HEADS16 = 4;

constexpr int GB_M = 128;                                  // accumulator rows per CTA (TMEM lanes)
constexpr int GB_K = 64;                                   // k step: one 128-byte swizzle atom of fp16
constexpr int G_STAGE_BYTES = (GB_M + 128) * GB_K * 2;     // 32 KiB: this CTA's A rows then its W rows, each [128][64] fp16
constexpr int G_STAGES = 5;
constexpr int G_EPI_WARPS = 8;                             // two per TMEM lane quarter, each taking every other column chunk
constexpr int G_THREADS = 32 * (G_EPI_WARPS + 4);          // warps 0-7 epilogue; third warpgroup: warp 8 MMA issue, warp 9 TMA loads, two idle
constexpr int G_GROUP_M = 8;                               // row tiles per raster group (engine/src/tcgemm16.cuh:18)
constexpr int G_STAGING = G_EPI_WARPS * 32 * 256;          // per epilogue warp 32 rows x 256 bytes of output being re-ordered
constexpr int G_SMEM = G_STAGES * G_STAGE_BYTES + G_STAGING + 2048 + 1024;   // = 227 KiB with the alignment slack

struct GemmParams {
    void* C;
    int ldc;
    int M, N, K;
    int tiles_m, tiles_n;          // in tiles of the launched shape (256x256 for PAIR, 128x128 otherwise)
    const float* gate;             // EPI_RESID: C[r, c] += gate[c] * acc (null = 1)
    const __nv_bfloat16* head_w;   // EPI_HEADS16: RMSNorm weight[128] or null
    const float* rope_cos;         // EPI_HEADS16: tables [rope_T, 64] or null; row r uses table row r % rope_T
    const float* rope_sin;
    int rope_T;
    float eps;
    uint32_t* status;
};

enum { GBAR_FULL = 0, GBAR_EMPTY = G_STAGES, GBAR_ACC_FULL = 2 * G_STAGES, GBAR_ACC_EMPTY = 2 * G_STAGES + 2, GBAR_COUNT = 2 * G_STAGES + 4 };

__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }   // engine/src/tcgemm16.cuh:55

// tile w -> (row tile, column tile): groups of G_GROUP_M row tiles x every column tile, column-major inside a group, so
// the CTAs running at the same time share weight tiles in L2 (engine/src/tcgemm16.cuh:66-69)
__device__ __forceinline__ void gemm_tile(int w, const GemmParams& p, int& tm, int& tn) {
    const int per_group = G_GROUP_M * p.tiles_n;
    const int first = (w / per_group) * G_GROUP_M, gsz = min(p.tiles_m - first, G_GROUP_M), in_g = w % per_group;
    tm = first + in_g % gsz;
    tn = in_g / gsz;
}

// per-head RMSNorm and rotate-half RoPE on one accumulator row of one head (engine/src/kernels.cu:656-666, 759-772)
__device__ __forceinline__ void head_norm_rope(float (&v)[128], const GemmParams& p, int row) {
    if (p.head_w) {
        uint4 wv[16];
#pragma unroll
        for (int q = 0; q < 16; q++) wv[q] = __ldg(reinterpret_cast<const uint4*>(p.head_w) + q);
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < 128; c++) ss = fmaf(v[c], v[c], ss);
        const float rs = rsqrtf(ss * (1.f / 128.f) + p.eps);
#pragma unroll
        for (int q = 0; q < 16; q++) {
            const uint32_t wd[4] = {wv[q].x, wv[q].y, wv[q].z, wv[q].w};
#pragma unroll
            for (int m = 0; m < 4; m++) {   // a bf16 is the top half of an fp32
                v[8 * q + 2 * m] = v[8 * q + 2 * m] * rs * __uint_as_float(wd[m] << 16);
                v[8 * q + 2 * m + 1] = v[8 * q + 2 * m + 1] * rs * __uint_as_float(wd[m] & 0xffff0000u);
            }
        }
    }
    if (p.rope_cos) {
        const int tr = min(row, p.M - 1) % p.rope_T;
        const float4* cr = reinterpret_cast<const float4*>(p.rope_cos + (size_t)tr * 64);
        const float4* sr = reinterpret_cast<const float4*>(p.rope_sin + (size_t)tr * 64);
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            float4 cv[8], sv[8];
#pragma unroll
            for (int q = 0; q < 8; q++) { cv[q] = __ldg(cr + hf * 8 + q); sv[q] = __ldg(sr + hf * 8 + q); }
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float cc[4] = {cv[q].x, cv[q].y, cv[q].z, cv[q].w}, sn[4] = {sv[q].x, sv[q].y, sv[q].z, sv[q].w};
#pragma unroll
                for (int m = 0; m < 4; m++) {
                    const int e = hf * 32 + q * 4 + m;
                    const float x0 = v[e], x1 = v[e + 64];
                    v[e] = x0 * cc[m] - x1 * sn[m];
                    v[e + 64] = x1 * cc[m] + x0 * sn[m];
                }
            }
        }
    }
}

template <int EPI, bool PAIR>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const GemmParams p) {
    constexpr int BN = PAIR ? 256 : 128;                                  // accumulator columns per tile
    constexpr int TILE_M = PAIR ? 256 : 128;                              // tile rows over the CTA group
    constexpr bool OUT32 = (EPI == EPI_F32 || EPI == EPI_RESID);
    constexpr int CW = OUT32 ? 64 : 128;                                  // columns per 256-byte output row chunk
    constexpr int NCH = BN / CW;
    constexpr uint32_t TMEM_COLS = 2 * BN;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* const smem = smem_raw + (base - raw);
    const uint32_t sRing = base;
    uint8_t* const stage_out = smem + G_STAGES * G_STAGE_BYTES;
    uint8_t* const ctrl = stage_out + G_STAGING;
    const uint32_t bars = sRing + G_STAGES * G_STAGE_BYTES + G_STAGING;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 512);
    volatile uint32_t* const abort_flag = reinterpret_cast<volatile uint32_t*>(ctrl + 516);
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;                  // 0 issues the MMAs
    const int group = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_groups = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int n_tiles = p.tiles_m * p.tiles_n, ksteps = p.K / GB_K;

    if (tid == 0) {
        for (int i = 0; i < GBAR_COUNT; i++) mbar_init(bar(i), (i >= GBAR_ACC_EMPTY) ? (PAIR ? 2u : 1u) * G_EPI_WARPS : 1u);   // acc_empty: one arrival per epilogue warp of the group
        *abort_flag = 0u;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == G_EPI_WARPS + 1 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmW); }
    if (warp == G_EPI_WARPS) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);                       // two accumulator buffers
        tmem_relinquish();
    }
    tc_fence_before();
    if (PAIR) { cluster_arrive(); cluster_wait(); } else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < G_EPI_WARPS) {
        setmaxnreg_inc<224>();                                            // the row buffers of the epilogue live in registers
        // ------------------------------------------------------------------ epilogue: one output row per thread
        const int quarter = warp & 3, chunk0 = warp >> 2;                // TMEM lanes [32 quarter, +32); chunks chunk0, chunk0 + 2, ...
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        uint8_t* const my_stage = stage_out + warp * 32 * 256;           // this warp's 32 rows, re-read by this warp only
        uint32_t use[2] = {0, 0};
        int k = 0;
        for (int w = group; w < n_tiles; w += n_groups, ++k) {
            const int buf = k & 1;
            int tm, tn;
            gemm_tile(w, p, tm, tn);
            const int m0 = tm * TILE_M + (int)rank * GB_M, n0 = tn * BN;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(GBAR_ACC_FULL + buf), use[buf] & 1u, abort_flag));
            ++use[buf];
            if (!ok) break;                                               // warps are independent from here on
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const int nrow = p.M - (m0 + quarter * 32);                      // rows of this warp inside the matrix
#pragma unroll 1
            for (int ch = chunk0; ch < NCH; ch += 2) {
                float v[CW];
                {
                    uint32_t a[CW / 32][32];
#pragma unroll
                    for (int q = 0; q < CW / 32; q++) tmem_ld32(tmem_base + lane_base + (uint32_t)(buf * BN + ch * CW + 32 * q), a[q]);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < CW / 32; q++) {
                        reg_fence32(a[q]);
#pragma unroll
                        for (int e = 0; e < 32; e++) v[32 * q + e] = __uint_as_float(a[q][e]);
                    }
                }
                if (ch + 2 >= NCH) {                                      // this warp's last chunk is in registers: the MMA warp may reuse it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR && rank != 0) mbar_arrive_cluster(mapa_u32(bar(GBAR_ACC_EMPTY + buf), 0));
                        else mbar_arrive(bar(GBAR_ACC_EMPTY + buf));
                    }
                }
                if constexpr (EPI == EPI_GELU16) {
#pragma unroll
                    for (int c = 0; c < CW; c++) v[c] = gelu_erf(v[c]);
                }
                if constexpr (EPI == EPI_HEADS16) head_norm_rope(v, p, row);
                // re-order through shared memory (16-byte pieces XOR-swizzled by row) so that whole 256-byte row chunks go out
                __syncwarp();
                uint8_t* const my_row = my_stage + lane * 256;
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    uint4 pk;
                    if constexpr (OUT32) {
                        pk = make_uint4(__float_as_uint(v[4 * c]), __float_as_uint(v[4 * c + 1]), __float_as_uint(v[4 * c + 2]), __float_as_uint(v[4 * c + 3]));
                    } else {
                        pk.x = pack16<DT_F16>(v[8 * c + 0], v[8 * c + 1]); pk.y = pack16<DT_F16>(v[8 * c + 2], v[8 * c + 3]);
                        pk.z = pack16<DT_F16>(v[8 * c + 4], v[8 * c + 5]); pk.w = pack16<DT_F16>(v[8 * c + 6], v[8 * c + 7]);
                    }
                    *reinterpret_cast<uint4*>(my_row + ((c ^ (lane & 15)) << 4)) = pk;
                }
                __syncwarp();
                uint2 vals[32];
#pragma unroll
                for (int rr = 0; rr < 32; rr++)
                    vals[rr] = *reinterpret_cast<const uint2*>(my_stage + rr * 256 + (((lane >> 1) ^ (rr & 15)) << 4) + (lane & 1) * 8);
                if constexpr (OUT32) {
                    float* g = static_cast<float*>(p.C) + (size_t)(m0 + quarter * 32) * p.ldc + n0 + ch * CW + lane * 2;
                    if (EPI == EPI_RESID) {
                        const float2 gt = p.gate ? __ldg(reinterpret_cast<const float2*>(p.gate + n0 + ch * CW + lane * 2)) : make_float2(1.f, 1.f);
                        float2 old[32];
#pragma unroll
                        for (int rr = 0; rr < 32; rr++)
                            if (rr < nrow) old[rr] = *reinterpret_cast<const float2*>(g + (size_t)rr * p.ldc);
#pragma unroll
                        for (int rr = 0; rr < 32; rr++)
                            if (rr < nrow)
                                *reinterpret_cast<float2*>(g + (size_t)rr * p.ldc) =
                                    make_float2(fmaf(gt.x, __uint_as_float(vals[rr].x), old[rr].x), fmaf(gt.y, __uint_as_float(vals[rr].y), old[rr].y));
                    } else {
#pragma unroll
                        for (int rr = 0; rr < 32; rr++)
                            if (rr < nrow) *reinterpret_cast<uint2*>(g + (size_t)rr * p.ldc) = vals[rr];
                    }
                } else {
                    __half* g = static_cast<__half*>(p.C) + (size_t)(m0 + quarter * 32) * p.ldc + n0 + ch * CW + lane * 4;
#pragma unroll
                    for (int rr = 0; rr < 32; rr++)
                        if (rr < nrow) *reinterpret_cast<uint2*>(g + (size_t)rr * p.ldc) = vals[rr];
                }
            }
        }
    } else if (warp == G_EPI_WARPS) {
        setmaxnreg_dec<56>();
        // ------------------------------------------------------------------ MMA issue (one lane of the group's first CTA)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t IDESC = idesc_f16(0, 0, 0, 0, TILE_M, BN);
            uint32_t ring = 0, use[2] = {0, 0};
            bool good = true;
            int k = 0;
            for (int w = group; w < n_tiles && good; w += n_groups, ++k) {
                const int buf = k & 1;
                // the epilogues have drained this accumulator (passes at once for the first two tiles)
                good = mbar_wait(bar(GBAR_ACC_EMPTY + buf), (use[buf] & 1u) ^ 1u, abort_flag);
                ++use[buf];
                if (!good) break;
                tc_fence_after();
                for (int ks = 0; ks < ksteps && good; ++ks, ++ring) {
                    const uint32_t st = ring % G_STAGES;
                    good = mbar_wait(bar(GBAR_FULL + st), (ring / G_STAGES) & 1u, abort_flag);
                    if (!good) break;
                    tc_fence_after();
                    const uint32_t a_s = sRing + st * G_STAGE_BYTES;
                    const uint64_t adesc = smem_desc_sw128(a_s, 16, 1024), wdesc = smem_desc_sw128(a_s + GB_M * GB_K * 2, 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
                        if (PAIR) mma_ss_pair(tmem_base + (uint32_t)(buf * BN), adesc + (uint64_t)(kk * 2), wdesc + (uint64_t)(kk * 2), IDESC, acc);
                        else mma_ss(tmem_base + (uint32_t)(buf * BN), adesc + (uint64_t)(kk * 2), wdesc + (uint64_t)(kk * 2), IDESC, acc);
                    }
                    if (PAIR) tc_commit_pair(bar(GBAR_EMPTY + st), 3); else tc_commit(bar(GBAR_EMPTY + st));
                }
                if (good) {
                    if (PAIR) tc_commit_pair(bar(GBAR_ACC_FULL + buf), 3); else tc_commit(bar(GBAR_ACC_FULL + buf));
                }
            }
        }
        __syncwarp();
    } else {
        setmaxnreg_dec<56>();
        // ------------------------------------------------------------------ TMA loads (one lane of every CTA)
        if (warp == G_EPI_WARPS + 1 && lane == 0) {
            uint32_t ring = 0;
            bool good = true;
            for (int w = group; w < n_tiles && good; w += n_groups) {
                int tm, tn;
                gemm_tile(w, p, tm, tn);
                const int m0 = tm * TILE_M + (int)rank * GB_M, wrow0 = tn * BN + (int)rank * 128;
                for (int ks = 0; ks < ksteps && good; ++ks, ++ring) {
                    const uint32_t st = ring % G_STAGES;
                    good = mbar_wait(bar(GBAR_EMPTY + st), ((ring / G_STAGES) & 1u) ^ 1u, abort_flag);
                    if (!good) break;
                    const uint32_t a_s = sRing + st * G_STAGE_BYTES;
                    if (PAIR) {
                        // both CTAs' bytes complete on the issuing CTA's barrier
                        if (rank == 0) mbar_expect_tx(bar(GBAR_FULL + st), 2 * G_STAGE_BYTES);
                        const uint32_t fb = mapa_u32(bar(GBAR_FULL + st), 0);
                        tma_load_3d_pair(a_s, &tmA, fb, ks * GB_K, m0, 0);
                        tma_load_3d_pair(a_s + GB_M * GB_K * 2, &tmW, fb, ks * GB_K, wrow0, 0);
                    } else {
                        mbar_expect_tx(bar(GBAR_FULL + st), G_STAGE_BYTES);
                        tma_load_3d(a_s, &tmA, bar(GBAR_FULL + st), ks * GB_K, m0, 0);
                        tma_load_3d(a_s + GB_M * GB_K * 2, &tmW, bar(GBAR_FULL + st), ks * GB_K, wrow0, 0);
                    }
                }
            }
            if (!good || *abort_flag) {                                   // let copies in flight land before the memory goes away
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 20000ull) {}
            }
        }
        __syncwarp();
    }
    tc_fence_before();
    if (PAIR) { cluster_arrive(); cluster_wait(); } else __syncthreads();
    if (warp == G_EPI_WARPS) {
        if (lane == 0 && *abort_flag) atomicOr(p.status, ST_TIMEOUT);
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace kb
