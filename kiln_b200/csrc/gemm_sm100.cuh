// fp16 GEMM for the projections around attention on sm_100a: C = epilogue(A[M,K] * W[N,K]^T), fp32 accumulation
// in TMEM, TMA-fed tcgen05 MMAs, persistent CTAs with two accumulator buffers so that the epilogue of one tile runs
// under the main loop of the next.
//
// Two shapes of the same kernel. PAIR: two CTAs of a cluster share one 256x256 tile through cta_group::2 MMAs; each
// loads its own 128 rows of A and 128 of the 256 W rows per 64-wide k step (32 KiB) and keeps its 128x256 half of the
// accumulator, so a CTA moves half the shared-memory bytes per flop of the single-CTA shape. That matters because
// measured on B200 a 128x128 single-CTA tile is bound by shared-memory bandwidth (TMA writes plus operand reads,
// about 100 B/clk/SM), not by the tensor pipe. Single: one CTA per 128x128 tile, for N not a multiple of 256, M <= 128,
// or when the pair shape would fill the device worse (the host decides).
//
// It takes the place of the reference's fp16-activation GEMM tc16::k_gemm16 (engine/src/tcgemm16.cuh:57-175,
// host wrapper linear16 at engine/src/kernels.cu:559-609) with its four epilogues — fp32 store, fp16 store,
// fp16 GELU, gated add into the fp32 residual stream (engine/src/tcgemm16.cuh:145-174) — and adds a fifth that the
// attention path wants: EPI_HEADS16 treats every 128 output columns as one attention head and applies the
// per-head RMSNorm (engine/src/kernels.cu:656-666) and rotate-half RoPE (engine/src/kernels.cu:759-772) to the
// accumulator row before storing fp16 (how the epilogue warps share that work is described at the code). With it the
// Q and K projections emit exactly what the attention kernel consumes, and the separate rmsnorm / rope_half launches
// and the staging pre-pass disappear. Up to three weight matrices can share one launch (q, k, v of one activation).
// Outputs leave through TMA stores, the residual epilogue through a TMA reduce-add.
// (The reference accumulates each 32-wide k tile in fp16 before flushing to fp32; here every product is
// accumulated in fp32.)
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "attn_sm100.cuh"   // pack16, ST_TIMEOUT
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
    // Second product (LoRA side path, engine/src/tcgemm16.cuh:26-28): the accumulator of segment s also takes
    // A2_s[M, K2_s] * W2_s[N, K2_s]^T, as further k steps after the first product's, so every epilogue sees the sum.
    // K2 = 0: none. A last partial k step reads zeros past column K2 (the tensor maps fill out-of-range elements).
    int K2[3];
    int tiles_m, tiles_n;          // in tiles of the launched shape (256x256 for PAIR, 128x128 otherwise)
    // Up to three weight matrices [N, K] share one launch (the q, k, v projections of one activation): column tile tn
    // belongs to segment tn / tiles_n_seg, which has its own W and C tensor maps and its own head epilogue settings.
    int tiles_n_seg;               // column tiles per segment (= tiles_n for a single matrix)
    const float* gate;             // EPI_RESID: C[r, c] += gate[c] * acc (null = 1)
    const __nv_bfloat16* head_w[3];   // EPI_HEADS16: RMSNorm weight[128] of the segment, or null
    int rope_on[3];                // EPI_HEADS16: the segment's heads are rotated (tables below)
    const float* rope_cos;         // EPI_HEADS16: tables [rope_T, 64] or null; row r uses table row r % rope_T
    const float* rope_sin;
    int rope_T;
    float eps;
    uint32_t* status;
};

struct alignas(64) GemmMaps {
    CUtensorMap w[3];              // per segment: the weight matrix, box 64 columns x 128 rows
    CUtensorMap c[3];              // per segment: the output, box as the epilogue stores it
    CUtensorMap a2[3];             // per segment: left operand [M, K2] of the second product (unused when K2 = 0)
    CUtensorMap w2[3];             // per segment: right operand [N, K2] of the second product
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

// dst[r * ld + col0 + c] = fp16(scale * src[r, c]) for a bf16 LoRA matrix [rows, cols]: how the stacked operands of the
// second product are laid out, with the LoRA's scale folded into its up-projection (engine/src/kernels.cu:548-554)
__global__ void lora_pack_kernel(__half* dst, int ld, int col0, const __nv_bfloat16* src, int rows, int cols, float scale) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    const int r = (int)(i / cols), c = (int)(i % cols);
    dst[(size_t)r * ld + col0 + c] = __float2half_rn(scale * __bfloat162float(src[i]));
}

template <int EPI, bool PAIR>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ GemmMaps maps, const GemmParams p) {
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
    const int n_tiles = p.tiles_m * p.tiles_n, ksteps1 = p.K / GB_K;

    if (tid == 0) {
        for (int i = 0; i < GBAR_COUNT; i++) mbar_init(bar(i), (i >= GBAR_ACC_EMPTY) ? (PAIR ? 2u : 1u) * G_EPI_WARPS : 1u);   // acc_empty: one arrival per epilogue warp of the group
        *abort_flag = 0u;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == G_EPI_WARPS + 1 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&maps.w[0]); tma_prefetch_desc(&maps.c[0]); }
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
        if constexpr (EPI == EPI_HEADS16) {
            // The two warps of a TMEM lane quarter split every head by RoPE half: warp half hs owns columns [32 hs, +32) and
            // their rotation partners [64 + 32 hs, +32). A thread normalises its row of the accumulator, the warp turns its
            // 32 rows x 64 values through shared memory, and the rotation runs after the turn, one (i, i + 64) pair per
            // lane per row: there a table row is one coalesced 128-byte read (measured: reading the tables in the
            // thread-per-row layout, 32 different lines per instruction, cost 4 us per tile). The 32 + 32 table values of
            // a lane are loaded once per tile, before the accumulator is waited for, and serve both heads of the tile.
            constexpr int NH = BN / 128;
            const int quarter = warp & 3, hs = warp >> 2;
            const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
            uint8_t* const my_stage = stage_out + warp * 32 * 256;        // 32 rows x 64 fp32, written and re-read by this warp only
            float* const ss_buf = reinterpret_cast<float*>(ctrl + 1024) + quarter * 64;
            volatile uint32_t* const ok_buf = reinterpret_cast<volatile uint32_t*>(ctrl + 640) + quarter * 2;
            const int pair_bar = 1 + quarter;
            uint4 w0[4], w1[4];                                           // RMSNorm weights of this warp's 32 + 32 columns (bf16)
            int w_seg = -1;                                               // segment they belong to
            uint32_t use[2] = {0, 0};
            int k = 0;
            for (int w = group; w < n_tiles; w += n_groups, ++k) {
                const int buf = k & 1;
                int tm, tn;
                gemm_tile(w, p, tm, tn);
                const int seg = tn / p.tiles_n_seg;
                const int m0 = tm * TILE_M + (int)rank * GB_M, n0 = (tn - seg * p.tiles_n_seg) * BN;
                const int row0 = m0 + quarter * 32;
                const int nrow = p.M - row0;
                const __nv_bfloat16* const head_w = seg == 0 ? p.head_w[0] : seg == 1 ? p.head_w[1] : p.head_w[2];
                const bool rope = (seg == 0 ? p.rope_on[0] : seg == 1 ? p.rope_on[1] : p.rope_on[2]) != 0;
                if (head_w && seg != w_seg) {                             // L1 hits after the first tile of a segment
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        w0[q] = __ldg(reinterpret_cast<const uint4*>(head_w + hs * 32) + q);
                        w1[q] = __ldg(reinterpret_cast<const uint4*>(head_w + 64 + hs * 32) + q);
                    }
                    w_seg = seg;
                }
                float cr[32], sr[32];
                if (rope) {
                    int tr = min(row0, p.M - 1) % p.rope_T;
#pragma unroll
                    for (int rr = 0; rr < 32; rr++) {
                        cr[rr] = __ldg(p.rope_cos + (size_t)tr * 64 + hs * 32 + lane);
                        sr[rr] = __ldg(p.rope_sin + (size_t)tr * 64 + hs * 32 + lane);
                        if (row0 + rr + 1 < p.M) tr = (tr + 1 == p.rope_T) ? 0 : tr + 1;
                    }
                }
                bool ok = __all_sync(0xffffffffu, mbar_wait(bar(GBAR_ACC_FULL + buf), use[buf] & 1u, abort_flag));
                ++use[buf];
                if (lane == 0) ok_buf[hs] = ok ? 1u : 0u;                 // leave only together: the pair meets at named barriers below
                named_bar_sync(pair_bar, 64);
                ok = ok_buf[0] != 0u && ok_buf[1] != 0u;
                named_bar_sync(pair_bar, 64);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int h = 0; h < NH; h++) {
                    float x0[32], x1[32];
                    {
                        uint32_t a0[32], a1[32];
                        tmem_ld32(tmem_base + lane_base + (uint32_t)(buf * BN + h * 128 + hs * 32), a0);
                        tmem_ld32(tmem_base + lane_base + (uint32_t)(buf * BN + h * 128 + 64 + hs * 32), a1);
                        tmem_wait_ld();
                        reg_fence32(a0);
                        reg_fence32(a1);
#pragma unroll
                        for (int e = 0; e < 32; e++) { x0[e] = __uint_as_float(a0[e]); x1[e] = __uint_as_float(a1[e]); }
                    }
                    if (h == NH - 1) {                                    // this warp's share of the accumulator is in registers
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (PAIR && rank != 0) mbar_arrive_cluster(mapa_u32(bar(GBAR_ACC_EMPTY + buf), 0));
                            else mbar_arrive(bar(GBAR_ACC_EMPTY + buf));
                        }
                    }
                    if (head_w) {                                         // engine/src/kernels.cu:656-666
                        float ss = 0.f;
#pragma unroll
                        for (int e = 0; e < 32; e++) ss = fmaf(x0[e], x0[e], fmaf(x1[e], x1[e], ss));
                        ss_buf[hs * 32 + lane] = ss;
                        named_bar_sync(pair_bar, 64);
                        const float rs = rsqrtf((ss + ss_buf[(hs ^ 1) * 32 + lane]) * (1.f / 128.f) + p.eps);
                        named_bar_sync(pair_bar, 64);                     // both sums are read before the next head overwrites them
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const uint32_t d0[4] = {w0[q].x, w0[q].y, w0[q].z, w0[q].w}, d1[4] = {w1[q].x, w1[q].y, w1[q].z, w1[q].w};
#pragma unroll
                            for (int m = 0; m < 4; m++) {                 // a bf16 is the top half of an fp32
                                x0[8 * q + 2 * m] = x0[8 * q + 2 * m] * rs * __uint_as_float(d0[m] << 16);
                                x0[8 * q + 2 * m + 1] = x0[8 * q + 2 * m + 1] * rs * __uint_as_float(d0[m] & 0xffff0000u);
                                x1[8 * q + 2 * m] = x1[8 * q + 2 * m] * rs * __uint_as_float(d1[m] << 16);
                                x1[8 * q + 2 * m + 1] = x1[8 * q + 2 * m + 1] * rs * __uint_as_float(d1[m] & 0xffff0000u);
                            }
                        }
                    }
                    if (lane == 0) tma_store_wait_read();                 // the boxes of the last head have left shared memory
                    __syncwarp();
                    uint8_t* const my_row = my_stage + lane * 256;
#pragma unroll
                    for (int j = 0; j < 8; j++) {                         // 16-byte pieces j (first half) and 8 + j (partners), XOR-swizzled by row
                        *reinterpret_cast<float4*>(my_row + ((j ^ (lane & 15)) << 4)) = make_float4(x0[4 * j], x0[4 * j + 1], x0[4 * j + 2], x0[4 * j + 3]);
                        *reinterpret_cast<float4*>(my_row + (((8 + j) ^ (lane & 15)) << 4)) = make_float4(x1[4 * j], x1[4 * j + 1], x1[4 * j + 2], x1[4 * j + 3]);
                    }
                    __syncwarp();
                    uint32_t pk[32];
#pragma unroll
                    for (int rr = 0; rr < 32; rr++) {
                        const uint8_t* src = my_stage + rr * 256 + (lane & 3) * 4;
                        float a = *reinterpret_cast<const float*>(src + (((lane >> 2) ^ (rr & 15)) << 4));
                        float b = *reinterpret_cast<const float*>(src + (((8 + (lane >> 2)) ^ (rr & 15)) << 4));
                        if (rope) {                                       // engine/src/kernels.cu:769-771
                            const float ra = a * cr[rr] - b * sr[rr];
                            b = b * cr[rr] + a * sr[rr];
                            a = ra;
                        }
                        const float other = __shfl_xor_sync(0xffffffffu, (lane & 1) ? a : b, 1);
                        pk[rr] = (lane & 1) ? pack16<DT_F16>(other, b) : pack16<DT_F16>(a, other);
                    }
                    // back into shared memory as two 32-row x 64-byte boxes (first half, partners), which leave by TMA
                    __syncwarp();
                    uint8_t* const my_out = my_stage + (lane & 1) * 2048 + (lane >> 1) * 4;
#pragma unroll
                    for (int rr = 0; rr < 32; rr++) *reinterpret_cast<uint32_t*>(my_out + rr * 64) = pk[rr];
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && nrow > 0) {
                        const int x = n0 + h * 128 + hs * 32;
                        tma_store_3d(&maps.c[seg], smem_u32(my_stage), x, row0, 0);
                        tma_store_3d(&maps.c[seg], smem_u32(my_stage) + 2048, x + 64, row0, 0);
                        tma_store_commit();
                    }
                }
            }
            if (lane == 0) tma_store_wait_all();
        } else {
            const int quarter = warp & 3, chunk0 = warp >> 2;                // TMEM lanes [32 quarter, +32); chunks chunk0, chunk0 + 2, ...
            const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
            uint8_t* const my_stage = stage_out + warp * 32 * 256;           // this warp's 32 rows x 256 bytes on their way out
            uint32_t use[2] = {0, 0};
            int k = 0;
            for (int w = group; w < n_tiles; w += n_groups, ++k) {
                const int buf = k & 1;
                int tm, tn;
                gemm_tile(w, p, tm, tn);
                const int seg = tn / p.tiles_n_seg;
                const int m0 = tm * TILE_M + (int)rank * GB_M, n0 = (tn - seg * p.tiles_n_seg) * BN;
                const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(GBAR_ACC_FULL + buf), use[buf] & 1u, abort_flag));
                ++use[buf];
                if (!ok) break;                                               // warps are independent from here on
                tc_fence_after();
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
                    if constexpr (EPI == EPI_RESID) {
                        if (p.gate) {
#pragma unroll
                            for (int c = 0; c < CW; c += 4) {
                                const float4 gt = __ldg(reinterpret_cast<const float4*>(p.gate + n0 + ch * CW + c));
                                v[c] *= gt.x; v[c + 1] *= gt.y; v[c + 2] *= gt.z; v[c + 3] *= gt.w;
                            }
                        }
                    }
                    // the 32 x 256-byte piece of the output goes through shared memory as two 128-byte-swizzled boxes and
                    // leaves by TMA (measured: 32 row stores per warp took 3 us, the issue rate of plain global stores from
                    // eight warps; the bulk copy takes them off the warp)
                    if (lane == 0) tma_store_wait_read();                     // the boxes of the last chunk have been read
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < 16; c++) {
                        uint4 pk;
                        if constexpr (OUT32) {
                            pk = make_uint4(__float_as_uint(v[4 * c]), __float_as_uint(v[4 * c + 1]), __float_as_uint(v[4 * c + 2]), __float_as_uint(v[4 * c + 3]));
                        } else {
                            pk.x = pack16<DT_F16>(v[8 * c + 0], v[8 * c + 1]); pk.y = pack16<DT_F16>(v[8 * c + 2], v[8 * c + 3]);
                            pk.z = pack16<DT_F16>(v[8 * c + 4], v[8 * c + 5]); pk.w = pack16<DT_F16>(v[8 * c + 6], v[8 * c + 7]);
                        }
                        *reinterpret_cast<uint4*>(my_stage + (c >> 3) * 4096 + lane * 128 + (((c & 7) ^ (lane & 7)) << 4)) = pk;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    const int x = n0 + ch * CW, y = m0 + quarter * 32;
                    if (lane == 0 && nrow > 0 && x < p.N) {                   // a narrow last column tile stores only the boxes that begin inside it
                        if constexpr (EPI == EPI_RESID) {
                            tma_reduce_add_3d(&maps.c[seg], smem_u32(my_stage), x, y, 0);
                            tma_reduce_add_3d(&maps.c[seg], smem_u32(my_stage) + 4096, x + CW / 2, y, 0);
                        } else {
                            tma_store_3d(&maps.c[seg], smem_u32(my_stage), x, y, 0);
                            if (x + CW / 2 < p.N) tma_store_3d(&maps.c[seg], smem_u32(my_stage) + 4096, x + CW / 2, y, 0);
                        }
                        tma_store_commit();
                    }
                }
            }
            if (lane == 0) tma_store_wait_all();
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
                int tm, tn;
                gemm_tile(w, p, tm, tn);
                const int ksteps = ksteps1 + (p.K2[tn / p.tiles_n_seg] + GB_K - 1) / GB_K;
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
                const int seg = tn / p.tiles_n_seg;
                const int m0 = tm * TILE_M + (int)rank * GB_M, wrow0 = (tn - seg * p.tiles_n_seg) * BN + (int)rank * 128;
                const int ksteps = ksteps1 + (p.K2[seg] + GB_K - 1) / GB_K;
                for (int ks = 0; ks < ksteps && good; ++ks, ++ring) {
                    const bool second = ks >= ksteps1;                    // the k steps of the second product follow the first's
                    const CUtensorMap* const tmL = second ? &maps.a2[seg] : &tmA;
                    const CUtensorMap* const tmW = second ? &maps.w2[seg] : &maps.w[seg];
                    const int k0 = (second ? ks - ksteps1 : ks) * GB_K;
                    const uint32_t st = ring % G_STAGES;
                    good = mbar_wait(bar(GBAR_EMPTY + st), ((ring / G_STAGES) & 1u) ^ 1u, abort_flag);
                    if (!good) break;
                    const uint32_t a_s = sRing + st * G_STAGE_BYTES;
                    if (PAIR) {
                        // both CTAs' bytes complete on the issuing CTA's barrier
                        if (rank == 0) mbar_expect_tx(bar(GBAR_FULL + st), 2 * G_STAGE_BYTES);
                        const uint32_t fb = mapa_u32(bar(GBAR_FULL + st), 0);
                        tma_load_3d_pair(a_s, tmL, fb, k0, m0, 0);
                        tma_load_3d_pair(a_s + GB_M * GB_K * 2, tmW, fb, k0, wrow0, 0);
                    } else {
                        mbar_expect_tx(bar(GBAR_FULL + st), G_STAGE_BYTES);
                        tma_load_3d(a_s, tmL, bar(GBAR_FULL + st), k0, m0, 0);
                        tma_load_3d(a_s + GB_M * GB_K * 2, tmW, bar(GBAR_FULL + st), k0, wrow0, 0);
                    }
                }
            }
            if (!good || *abort_flag) {
                // let the copies already requested land before the memory goes away: a bounded wait on the FULL barrier of every
                // stage with a request outstanding. In a pair those barriers live in the first CTA; the second one cannot poll
                // them and waits a fixed 20 us instead (both then meet at the cluster barrier below).
                if (!PAIR || rank == 0) {
                    for (uint32_t k = ring > (uint32_t)G_STAGES ? ring - G_STAGES : 0u; k < ring; ++k) drain_wait(bar(GBAR_FULL + k % G_STAGES), (k / G_STAGES) & 1u);
                } else {
                    const uint64_t t0 = globaltimer_ns();
                    while (globaltimer_ns() - t0 < 20000ull) {}
                }
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
