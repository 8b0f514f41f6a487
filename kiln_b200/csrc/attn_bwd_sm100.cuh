// Attention backward on sm_100a: dQ, dK, dV of softmax(Q K^T / sqrt(128)) V per head, from Q, K, V and dO.
//
// It takes the place of the reference's exact backward attention_bwd (engine/src/train.cu:216-242: five batched cuBLAS SGEMMs
// per head group around k_softmax_pad, train.cu:103-121, and k_dsoftmax, train.cu:124-131, with the [heads, Tq, Tk]
// probabilities P and their gradient dP materialised in the arena) for the LoRA trainer's two call sites (train.cu:334, 344).
// Here nothing of size Tq x Tk exists in memory: like the forward kernel the products are formed tile by tile on the tensor
// cores (fp16 operands, fp32 accumulation in TMEM) and P is recomputed from a per-row statistic.
//
// Four launches (kb_attn_bwd): the staging pre-pass (Q, K, V, dO -> fp16), the forward kernel, which also leaves
// L_i = log2 of the softmax denominator of row i (npad zero keys included) in the "stats" array, a small kernel for
// D_i = sum_d dO[i, d] O[i, d] (= sum_j P_ij dP_ij, what k_dsoftmax sums), and this file's kernel, whose thread blocks
// play one of two roles:
//
//   BWD_DKV  one thread block per (key block j, head, image), query blocks i streamed through a two-stage ring:
//              S^T  = K_j Q_i^T            dP^T = V_j dO_i^T                      (two SS products into TMEM)
//              P^T  = 2^(c S^T - L_i)      dS^T = P^T (dP^T - D_i)                (softmax warps; fp16, written over S^T / dP^T)
//              dV_j += P^T dO_i            dK_j += dS^T Q_i                       (A operand from TMEM, B the same shared-memory
//                                                                                  tiles read MN-major)
//   BWD_DQ   one thread block per (query block i, head, image), key blocks j streamed:
//              S = Q_i K_j^T,  dP = dO_i V_j^T,  dS = 2^(c S - L_i) (dP - D_i),  dQ_i += dS K_j
//
// Two roles instead of one with atomics: every output element is written once by one thread block, in a fixed order, so
// results are bit-identical from run to run (the reference's are too). The price is that S and dP are formed twice.
// The npad zero keys only enter through L_i: their dP is 0 and their K is 0, so they add nothing to any gradient
// (train.cu:124 says the same of the reference). Rows past Tq or Tk are zero-filled by TMA; a zero Q/dO row has dS = 0 and
// adds nothing to dK / dV, a zero K row adds nothing to dQ, so ragged sizes need no masking - only finite statistics, which
// the stats array (padded to whole query blocks) always holds.
//
// TMEM (512 columns): T0 [0,128) S or S^T, T1 [128,256) dP or dP^T, acc0 [256,384), acc1 [384,512). Measured on B200 (clock
// stamps in a private build): the kernel is bound by the thread that issues the products - an SS product costs ~650 cycles
// per 128x128x128 however its N is cut (the A operand is re-read from shared memory for every instruction), the softmax
// warps need ~1100 per step. So the products keep N = 128 and the step is software-pipelined across the two products instead:
//   softmax phase 1: S^T ready -> P^T = 2^(c S^T - L) (kept in registers), fp16 P^T stored, "P0" signalled;
//   softmax phase 2: dP^T ready -> dS^T = P^T (dP^T - D) stored, "P1" signalled;
//   issue order:     [P0] dV += P^T dO | S^T of the next step | [P1] dK += dS^T Q | dP^T of the next step
// so that phase 1 of the next step runs under the dK and dP^T products and phase 2 under the dV and S^T products of the step
// after (in-order execution of one thread's tcgen05.mma keeps a product from overwriting what the one before still reads).
// BWD_DQ has one accumulating product: S of the next step is issued as soon as the softmax warps have read S (phase 1
// signals that), under phase 2. Each of the eight softmax warps (lane quarter x column half) owns 64 columns of T0 / T1 and
// writes its fp16 results over the first 32 of those same columns, so no warp overwrites what another still has to read.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "attn_sm100.cuh"
#include "ptx.cuh"

namespace kb {

constexpr int BWD_DKV = 0, BWD_DQ = 1;
constexpr int BWD_THREADS = 384;                              // warps 0-7 softmax / epilogue, 8 MMA issue, 9 TMA loads, 10-11 idle
constexpr int BWD_SOFTMAX_REGS = 224, BWD_OTHER_REGS = 56;    // 384 x 168 = 256 x 224 + 128 x 56
constexpr int BWD_STAGE_BYTES = 2 * TILE_BYTES + 1024;        // two streamed tiles + the statistics of a query block
constexpr int BWD_SMEM = 2 * TILE_BYTES + 2 * BWD_STAGE_BYTES + 1024;   // resident pair, two stages, control block

struct BwdParams {
    int B, H, Tq, Tk;
    // BWD_DKV with few key blocks (cross-attention to a short context): the query blocks of a (key block, head, image) are cut
    // into qsplit ranges of q_per blocks, one thread block each, whose partial dK / dV go to scratch (image index s * B + b of
    // the output tensor maps) and are summed in a fixed order by bwd_reduce_kernel. qsplit = 1: no cut, outputs written directly.
    int qsplit, q_per;
    const float* stats;     // [B][H][ceil(Tq/128)][2][128]: L (log2 of the softmax denominator, in units of c * score), then D
    float scale_log2;       // c = log2(e) / sqrt(128)
    float scale;            // 1 / sqrt(128)
    uint32_t* status;
};

enum { BB_RES = 0, BB_XFULL = 1, BB_XEMPTY = 3, BB_TFULL = 5, BB_PFULL = 7, BB_ACC = 9, BB_COUNT = 10 };   // TFULL/PFULL: [0] first product / phase 1, [1] second

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// D_i = sum_d dO[i, d] * O[i, d] per (row, head) into the stats array; one warp per (row, head), rows of whole query blocks
// (rows past Tq get 0). dO fp16 as staged for the tensor cores, O fp16 from the forward pass (its 16-bit output path: bulk
// tensor stores instead of per-thread fp32 row stores; the rounding moves D by ~1e-4 of the dP it is subtracted from).
__global__ void bwd_delta_kernel(float* stats, const __half* dout, int ld_do, const __half* o, int ld_o, int B, int Tq, int H) {
    const int nqb = (Tq + BM - 1) / BM;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const long long total = (long long)B * H * nqb * BM;
    if (w >= total) return;
    const int r = (int)(w % (nqb * BM)), h = (int)((w / (nqb * BM)) % H), b = (int)(w / ((long long)nqb * BM * H));
    float s = 0.f;
    if (r < Tq) {
        const uint2 gv = *reinterpret_cast<const uint2*>(dout + ((size_t)b * Tq + r) * (size_t)ld_do + (size_t)h * HD + lane * 4);
        const uint2 ow = *reinterpret_cast<const uint2*>(o + ((size_t)b * Tq + r) * (size_t)ld_o + (size_t)h * HD + lane * 4);
        const float2 ga = __half22float2(*reinterpret_cast<const __half2*>(&gv.x)), gb = __half22float2(*reinterpret_cast<const __half2*>(&gv.y));
        const float2 oa = __half22float2(*reinterpret_cast<const __half2*>(&ow.x)), ob = __half22float2(*reinterpret_cast<const __half2*>(&ow.y));
        s = ga.x * oa.x + ga.y * oa.y + gb.x * ob.x + gb.y * ob.y;
    }
    for (int o2 = 16; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
    if (lane == 0) stats[(((size_t)b * H + h) * nqb + r / BM) * 256 + 128 + (r % BM)] = s;
}

// One thread block's work in either role: (blk, h, b) = (key block, head, image) for BWD_DKV, (query block, head, image) for BWD_DQ.
template <int MODE>
__device__ __forceinline__ void attn_bwd_body(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmdO,
                                              const CUtensorMap& tmOut0, const CUtensorMap& tmOut1, const BwdParams& p, const int blk, const int h,
                                              const int b, const int part) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {                                           // never seen; without it every tile would be garbage
        if (threadIdx.x == 0) atomicOr(p.status, ST_TIMEOUT);
        return;
    }
    const uint32_t sR0 = base, sR1 = base + TILE_BYTES;            // resident: K_j, V_j (BWD_DKV) or Q_i, dO_i (BWD_DQ)
    const uint32_t sX = base + 2 * TILE_BYTES;                     // stages: X0 (Q_i or K_j), X1 (dO_i or V_j), statistics
    uint8_t* const ctrl = smem_raw + 2 * TILE_BYTES + 2 * BWD_STAGE_BYTES;
    const uint32_t bars = sX + 2 * BWD_STAGE_BYTES;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 128);
    volatile uint32_t* const abort_flag = reinterpret_cast<volatile uint32_t*>(ctrl + 132);
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nqb = (p.Tq + BM - 1) / BM;
    const int i0 = MODE == BWD_DKV ? part * p.q_per : 0;           // first streamed block of this thread block
    const int n_it = MODE == BWD_DKV ? min(nqb - i0, p.q_per) : (p.Tk + BN - 1) / BN;

    if (tid == 0) {
        for (int i = 0; i < BB_COUNT; i++) mbar_init(bar(i), (i == BB_PFULL || i == BB_PFULL + 1) ? 8u : 1u);   // P: one arrival per softmax warp
        *abort_flag = 0u;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 9 && lane == 0) { tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO); }
    if (warp == 8) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        setmaxnreg_inc<BWD_SOFTMAX_REGS>();
        // ------------------------------------------------------------------ softmax warps: TMEM lane quarter x column half
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;                          // row of the resident block (= TMEM lane)
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t tT0 = tmem_base + lane_base, tT1 = tmem_base + lane_base + 128u;
        const float c = p.scale_log2;
        float Lr = 0.f, Dr = 0.f;                                   // BWD_DQ: this row's statistics
        if (MODE == BWD_DQ) {
            const float* st = p.stats + (((size_t)b * p.H + h) * nqb + blk) * 256;
            Lr = __ldg(st + r);
            Dr = __ldg(st + 128 + r);
        }
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int st = it & 1;
            // ---- phase 1: P = 2^(c S - L) for this warp's 64 columns
            ok = __all_sync(0xffffffffu, mbar_wait(bar(BB_TFULL + 0), (uint32_t)it & 1u, abort_flag));
            if (!ok) break;
            tc_fence_after();
            const float* sStats = reinterpret_cast<const float*>(smem_raw + 2 * TILE_BYTES + st * BWD_STAGE_BYTES + 2 * TILE_BYTES);
            if (MODE == BWD_DKV) {                                  // the statistics came with the stage's tiles (already complete: the
                ok = __all_sync(0xffffffffu, mbar_wait(bar(BB_XFULL + st), ((uint32_t)it >> 1) & 1u, abort_flag));   // products read them)
                if (!ok) break;
            }
            float pv[64];
            {
                uint32_t s0[32], s1[32];
                tmem_ld32(tT0 + (uint32_t)(half * 64), s0);
                tmem_ld32(tT0 + (uint32_t)(half * 64 + 32), s1);
                tmem_wait_ld();
                reg_fence32(s0); reg_fence32(s1);
                if (MODE == BWD_DQ) {                               // S has been read: the next step's S may be formed
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(BB_PFULL + 0));
                }
#pragma unroll
                for (int e = 0; e < 64; e += 2) {
                    float L0 = Lr, L1 = Lr;
                    if (MODE == BWD_DKV) {                          // per column: the query row's statistic (a broadcast read)
                        const float2 l2 = *reinterpret_cast<const float2*>(sStats + half * 64 + e);
                        L0 = l2.x; L1 = l2.y;
                    }
                    const uint32_t a = e < 32 ? s0[e & 31] : s1[e & 31], bq = e < 32 ? s0[(e & 31) + 1] : s1[(e & 31) + 1];
                    pv[e] = ex2(fmaf(__uint_as_float(a), c, -L0));
                    pv[e + 1] = ex2(fmaf(__uint_as_float(bq), c, -L1));
                }
            }
            if (MODE == BWD_DKV) {
                uint32_t pk[32];
#pragma unroll
                for (int e = 0; e < 32; e++) pk[e] = pack16<DT_F16>(pv[2 * e], pv[2 * e + 1]);
                // element pair (2c, 2c+1) of this warp's contraction range in column c of its OWN columns: only what this
                // thread has just read is overwritten
                tmem_st32(tT0 + (uint32_t)(half * 64), pk);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BB_PFULL + 0));
            }
            // ---- phase 2: dS = P (dP - D)
            ok = __all_sync(0xffffffffu, mbar_wait(bar(BB_TFULL + 1), (uint32_t)it & 1u, abort_flag));
            if (!ok) break;
            tc_fence_after();
            {
                uint32_t d0[32], d1[32], dk[32];
                tmem_ld32(tT1 + (uint32_t)(half * 64), d0);
                tmem_ld32(tT1 + (uint32_t)(half * 64 + 32), d1);
                tmem_wait_ld();
                reg_fence32(d0); reg_fence32(d1);
#pragma unroll
                for (int e = 0; e < 64; e += 2) {
                    float D0 = Dr, D1 = Dr;
                    if (MODE == BWD_DKV) {
                        const float2 dd = *reinterpret_cast<const float2*>(sStats + 128 + half * 64 + e);
                        D0 = dd.x; D1 = dd.y;
                    }
                    const uint32_t a = e < 32 ? d0[e & 31] : d1[e & 31], bq = e < 32 ? d0[(e & 31) + 1] : d1[(e & 31) + 1];
                    dk[e >> 1] = pack16<DT_F16>(pv[e] * (__uint_as_float(a) - D0), pv[e + 1] * (__uint_as_float(bq) - D1));
                }
                tmem_st32(tT1 + (uint32_t)(half * 64), dk);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(BB_PFULL + 1));
        }
        // ------------------------------------------------------------------ epilogue: accumulators -> global
        // Each warp turns its 32 rows x 64 columns of an accumulator into two 32 x 32 fp32 boxes (128-byte rows, 128-byte
        // swizzle) in the stage area, which is free now, and one lane hands them to bulk tensor stores: rows past the end are
        // clipped by the tensor map. (Per-thread row stores, 32 scattered 16-byte pieces per instruction, took ~4 us per
        // thread block here, as they did in the projection GEMM.)
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(BB_ACC), 0u, abort_flag));
        if (ok) {
            tc_fence_after();
            uint8_t* const my_stage = smem_raw + 2 * TILE_BYTES + warp * 16384;          // four 4 KiB boxes per warp
#pragma unroll
            for (int a = 0; a < (MODE == BWD_DKV ? 2 : 1); a++) {
                const float k = (MODE == BWD_DKV && a == 0) ? 1.f : p.scale;   // dV unscaled; dK and dQ carry 1/sqrt(128)
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    uint32_t o[32];
                    tmem_ld32(tmem_base + lane_base + 256u + (uint32_t)(a * 128 + half * 64 + 32 * q), o);
                    tmem_wait_ld();
                    reg_fence32(o);
                    uint8_t* const box = my_stage + (a * 2 + q) * 4096 + lane * 128;
#pragma unroll
                    for (int cc = 0; cc < 8; cc++)
                        *reinterpret_cast<float4*>(box + ((cc ^ (lane & 7)) << 4)) =
                            make_float4(__uint_as_float(o[4 * cc]) * k, __uint_as_float(o[4 * cc + 1]) * k, __uint_as_float(o[4 * cc + 2]) * k,
                                        __uint_as_float(o[4 * cc + 3]) * k);
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                const int row0 = blk * BM + quarter * 32;
                if (row0 < (MODE == BWD_DKV ? p.Tk : p.Tq)) {
#pragma unroll
                    for (int a = 0; a < (MODE == BWD_DKV ? 2 : 1); a++)
#pragma unroll
                        for (int q = 0; q < 2; q++)
                            tma_store_3d(a ? &tmOut1 : &tmOut0, smem_u32(my_stage + (a * 2 + q) * 4096), h * HD + half * 64 + 32 * q, row0,
                                         MODE == BWD_DKV ? part * p.B + b : b);
                    tma_store_commit();
                }
                tma_store_wait_all();                                       // the stage area goes away with the thread block
            }
        }
    } else {
        setmaxnreg_dec<BWD_OTHER_REGS>();
        if (warp == 8 && lane == 0) {
            // ------------------------------------------------------------------ MMA issue
            constexpr uint32_t IDESC_T = idesc_f16(0, 0, 0, 0, BM, BN);   // T = R X^T, both operands K-major (rows of 128 head channels)
            constexpr uint32_t IDESC_A = idesc_f16(0, 0, 0, 1, BM, HD);   // acc += (fp16 in TMEM) X, X MN-major (rows = contraction index)
            constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
            auto issue_T = [&](uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr) {
                const uint32_t alo = smem_desc_lo(a_saddr, 16), blo = smem_desc_lo(b_saddr, 16);
                mma_ss_w<0>(d_tmem, alo, blo, DESC_HI, IDESC_T);
#pragma unroll
                for (int kk = 1; kk < 8; kk++) {
                    const uint32_t off = ((uint32_t)(kk >> 2) * HALF_BYTES + (uint32_t)(kk & 3) * 32u) >> 4;
                    mma_ss_w<1>(d_tmem, alo + off, blo + off, DESC_HI, IDESC_T);
                }
            };
            // the fp16 A operand sits in two pieces: contraction elements [64 hh, 64 hh + 64) at columns [64 hh, 64 hh + 32)
            auto issue_A = [&](uint32_t d_tmem, uint32_t a_region, uint32_t b_saddr, bool first) {
                const uint32_t blo = smem_desc_lo(b_saddr, HALF_BYTES);
#pragma unroll
                for (int kk = 0; kk < 8; kk++) {
                    const uint32_t a_t = a_region + (uint32_t)(64 * (kk >> 2) + 8 * (kk & 3));
                    if (kk == 0 && first) mma_ts_w<0>(d_tmem, a_t, blo, DESC_HI, IDESC_A);
                    else mma_ts_w<1>(d_tmem, a_t, blo + (uint32_t)(kk * 128), DESC_HI, IDESC_A);
                }
            };
            auto xaddr = [&](int st) { return sX + (uint32_t)st * BWD_STAGE_BYTES; };
            bool good = mbar_wait(bar(BB_RES), 0u, abort_flag);
            if (good) {
                good = mbar_wait(bar(BB_XFULL + 0), 0u, abort_flag);
                if (good) {
                    tc_fence_after();
                    issue_T(tmem_base, sR0, xaddr(0));
                    tc_commit(bar(BB_TFULL + 0));
                    issue_T(tmem_base + 128u, sR1, xaddr(0) + TILE_BYTES);
                    tc_commit(bar(BB_TFULL + 1));
                }
            }
            for (int it = 0; it < n_it && good; ++it) {
                const int st = it & 1;
                const uint32_t x0 = xaddr(st), x1 = x0 + TILE_BYTES;
                const bool more = it + 1 < n_it;
                // phase 1 of this step is over: P^T is stored (BWD_DKV) / S has been read (BWD_DQ)
                good = mbar_wait(bar(BB_PFULL + 0), (uint32_t)it & 1u, abort_flag);
                if (!good) break;
                tc_fence_after();
                if (MODE == BWD_DKV) issue_A(tmem_base + 256u, tmem_base, x1, it == 0);               // dV += P^T dO_i
                if (more) {
                    good = mbar_wait(bar(BB_XFULL + (st ^ 1)), ((uint32_t)(it + 1) >> 1) & 1u, abort_flag);
                    if (!good) break;
                    tc_fence_after();
                    issue_T(tmem_base, sR0, xaddr(st ^ 1));                                           // the next step's S / S^T
                    tc_commit(bar(BB_TFULL + 0));
                }
                good = mbar_wait(bar(BB_PFULL + 1), (uint32_t)it & 1u, abort_flag);
                if (!good) break;
                tc_fence_after();
                if (MODE == BWD_DKV) issue_A(tmem_base + 384u, tmem_base + 128u, x0, it == 0);        // dK += dS^T Q_i
                else issue_A(tmem_base + 256u, tmem_base + 128u, x0, it == 0);                        // dQ += dS K_j
                tc_commit(bar(BB_XEMPTY + st));                                    // every product on this stage has been issued
                if (more) {
                    issue_T(tmem_base + 128u, sR1, xaddr(st ^ 1) + TILE_BYTES);                       // the next step's dP / dP^T
                    tc_commit(bar(BB_TFULL + 1));
                }
            }
            if (good) tc_commit(bar(BB_ACC));
        } else if (warp == 9 && lane == 0) {
            // ------------------------------------------------------------------ TMA loads
            auto load_tile = [&](uint32_t dst, const CUtensorMap* tm, uint32_t mbar, int row0) {
                tma_load_3d(dst, tm, mbar, h * HD, row0, b);
                tma_load_3d(dst + HALF_BYTES, tm, mbar, h * HD + 64, row0, b);
            };
            mbar_expect_tx(bar(BB_RES), 2 * TILE_BYTES);
            load_tile(sR0, MODE == BWD_DKV ? &tmK : &tmQ, bar(BB_RES), blk * BM);
            load_tile(sR1, MODE == BWD_DKV ? &tmV : &tmdO, bar(BB_RES), blk * BM);
            bool good = true;
            int issued = 0;
            for (int it = 0; it < n_it && good; ++it) {
                const int st = it & 1;
                good = mbar_wait(bar(BB_XEMPTY + st), (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag);
                if (!good) break;
                issued = it + 1;
                const uint32_t x0 = sX + st * BWD_STAGE_BYTES, x1 = x0 + TILE_BYTES;
                mbar_expect_tx(bar(BB_XFULL + st), 2 * TILE_BYTES + (MODE == BWD_DKV ? 1024 : 0));
                load_tile(x0, MODE == BWD_DKV ? &tmQ : &tmK, bar(BB_XFULL + st), (i0 + it) * BM);
                load_tile(x1, MODE == BWD_DKV ? &tmdO : &tmV, bar(BB_XFULL + st), (i0 + it) * BM);
                if (MODE == BWD_DKV) bulk_load_1d(x1 + TILE_BYTES, p.stats + (((size_t)b * p.H + h) * nqb + (i0 + it)) * 256, 1024, bar(BB_XFULL + st));
            }
            if (!good || *abort_flag) {                               // let the copies already requested land before the memory goes away
                drain_wait(bar(BB_RES), 0u);
                for (int k = issued > 2 ? issued - 2 : 0; k < issued; ++k) drain_wait(bar(BB_XFULL + (k & 1)), ((uint32_t)k >> 1) & 1u);
            }
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        if (lane == 0 && *abort_flag) atomicOr(p.status, ST_TIMEOUT);
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// dk / dv [B*Tk, ld] = sum over the qsplit partial results [qsplit][B*Tk][cols] in scratch, in the order of the parts
// (bit-identical from run to run); one thread per four columns of a row, both tensors in one launch (blockIdx.y).
__global__ void bwd_reduce_kernel(float* dk, int ld_dk, float* dv, int ld_dv, const float* part_dk, const float* part_dv, int rows, int cols, int qsplit) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t per_row = (size_t)cols / 4;
    if (i >= (size_t)rows * per_row) return;
    const size_t r = i / per_row, c4 = i % per_row;
    const float* src = blockIdx.y ? part_dv : part_dk;
    float* dst = blockIdx.y ? dv + r * (size_t)ld_dv + c4 * 4 : dk + r * (size_t)ld_dk + c4 * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < qsplit; s++) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + ((size_t)s * rows + r) * (size_t)cols) + c4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(dst) = acc;
}

// Both roles in ONE launch: thread blocks [0, n_dkv) are the dK/dV blocks, the rest the dQ blocks. The two halves are independent
// (disjoint outputs, common read-only inputs); launched together, the dQ blocks start on the SMs that the last, partial round of
// dK/dV blocks leaves idle: 2 x 512 blocks at the DiT size are 6.9 rounds on 148 SMs instead of 3.46 rounds twice, each rounded up.
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const __grid_constant__ CUtensorMap tmdO, const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                const __grid_constant__ CUtensorMap tmDV, const __grid_constant__ BwdParams p, const int n_dkv) {
    const int nkb = (p.Tk + BN - 1) / BN, nqb = (p.Tq + BM - 1) / BM;
    int idx = (int)blockIdx.x;
    if (idx < n_dkv) {
        const int part = idx % p.qsplit;
        idx /= p.qsplit;
        attn_bwd_body<BWD_DKV>(tmQ, tmK, tmV, tmdO, tmDV, tmDK, p, idx % nkb, (idx / nkb) % p.H, idx / (nkb * p.H), part);
    } else {
        idx -= n_dkv;
        attn_bwd_body<BWD_DQ>(tmQ, tmK, tmV, tmdO, tmDQ, tmDQ, p, idx % nqb, (idx / nqb) % p.H, idx / (nqb * p.H), 0);
    }
}

}  // namespace kb
