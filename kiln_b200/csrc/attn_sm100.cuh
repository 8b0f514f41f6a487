// Fused multi-head attention forward for head size 128 on sm_100a (B200):
// TMA-staged fp16 Q/K/V tiles (128-byte swizzle), tcgen05 MMAs with the S and O accumulators in TMEM,
// online softmax with one thread per query row, P handed to the second MMA through TMEM.
//
// It replaces the reference's mma.sync FlashAttention-2 kernel tfa::k_flash
// (engine/src/tcflash.cuh:20-157) and keeps its contract: non-causal, keys >= Tk ignored, `npad`
// all-zero keys joining the softmax analytically (engine/src/tcflash.cuh:136-147), fp32 statistics,
// base-2 exponent with the scale log2(e)/sqrt(128) (engine/src/tcflash.cuh:164).
//
// The kernel is PERSISTENT: one CTA per SM walks a list of work segments, so TMEM allocation, barrier
// set-up and the TMA/MMA pipeline fill are paid once, and the loads of the next segment run under the
// epilogue of the current one. A segment runs TWO softmax streams that share the tensor core:
//   MODE_PAIR : two 128-row query tiles of one (batch, head) against a range of 128-key blocks of one
//               K/V sequence (self-attention and plain cross-attention);
//   MODE_NAG  : one 128-row query tile of one head against TWO K/V sequences (positive and negative
//               context), followed by the NAG combine of engine/src/dit.cu:295-324 in the epilogue.
//               The combine needs per-token L1 norms over ALL heads: the CTAs that hold the heads of
//               one query tile (adjacent items, so they run at the same time) publish their partial
//               norms in a small global scratch, bump a per-tile counter and wait, bounded, for the
//               other heads. Nothing but the blended result is written as output.
//
// Warp roles (384 threads): warps 0-3 / 4-7: softmax of stream 0 / 1 (warp w owns TMEM lanes 32*(w%4)..+31,
// one query row per thread), warps 8 / 10 issue the MMAs of stream 0 / 1 (one lane each), warp 9 issues TMA loads
// (one lane), warp 11 idle.
//
// TMEM (512 columns): R [0,128) P0 [128,192) P1 [192,256) O0 [256,384) O1 [384,512).
// R is ONE score staging area shared by both streams: an S = Q K^T lands there, the stream's softmax threads
// read it into registers at once and hand R back. P (fp16 pairs, 64 columns) has its own place per stream.
// With P written over S (the usual layout) a stream's next S cannot be issued before its own P*V has
// consumed P, so its cycle is  softmax + P*V + S + two hand-offs  and two streams keep the tensor core ~58 % busy.
// Here the next S of a stream does not depend on its P: the softmax threads ask for it while they are still
// in their exponentials (`s_req`), it runs on the tensor core under the rest of that softmax, and the
// threads go from one block straight into the next; P*V follows whenever P is complete.
//
// Balanced schedule (MODE_PAIR, `split`). Items x key blocks rarely divide by the SM count (4096 tokens:
// 256 items on 148 SMs = 1.73 rounds). With `split` every CTA takes an equal, contiguous range of
// (item, key block) steps. An item cut by a range boundary is finished by the CTA that holds its FIRST blocks
// (always the last thing that CTA does); the CTAs holding its later blocks (always the first thing they do)
// write their unnormalised (m, l, O) to a global scratch and raise a flag; the finisher waits (bounded) and
// merges. All CTAs are resident (cooperative launch), so nothing the finisher waits for can be queued behind it.
//
// (Tried and dropped: 64-key half blocks with two S buffers per stream: an S MMA with N = 64 reads as many
// shared-memory bytes per FLOP for its A operand as it saves on B and runs at half rate, 1.5x slower. Both
// warpgroups on one stream's block with half of the keys per thread: the exponentials are bound by the
// 16-per-clock MUFU unit whatever the thread count, and the two softmaxes can then no longer overlap, 12 % slower.
// 2^x by polynomial on the FMA pipe for part of the scores: packed f32x2 instructions issue at half rate on B200
// (measured: 2 cycles per warp instruction), so the polynomial costs more pipe time than the MUFU it saves.
// Exponentials against the stale maximum with the block maximum tracked on the side and a redo on overflow: the extra
// instructions in the exponential loop cost more than the ~400-cycle maximum phase they remove, 12 % slower.
// Strict turns of the two streams at their exponential phase, so that one stream's MUFU work runs under the other's
// MUFU-free work: a warpgroup alone runs its exponentials at ~24 cycles per score pair, not the 16 MUFU allows, so two
// overlapping exponential phases use MUFU better than two exclusive ones, 15 % slower.)
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <type_traits>

#include "ptx.cuh"

namespace kb {

constexpr int MODE_PAIR = 0, MODE_NAG = 1;
constexpr int DT_F16 = 0, DT_BF16 = 1;

constexpr int HD = 128;                 // head size
constexpr int BM = 128;                 // query rows per stream tile
constexpr int BN = 128;                 // keys per block
constexpr int TILE_BYTES = BM * HD * 2; // 32 KiB: one Q, K or V tile (two 64-column swizzled halves)
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int NSTAGE = 4;               // K/V ring depth
#ifndef KB_POLY_PAIRS
#define KB_POLY_PAIRS 0
#endif
constexpr int POLY_PAIRS = KB_POLY_PAIRS; // of every 8 score pairs, this many take 2^x on the FMA pipe instead of MUFU
constexpr int ATTN_THREADS = 384;
// Registers per thread after the warpgroups re-divide the 384 x 168 the block starts with: 256 softmax threads x 224 + 128
// threads of the MMA / TMA / helper warps x 56 = 64512 exactly (a larger second number would leave the softmax warps'
// increase waiting forever). At 224 the softmax code compiles without a spill, which matters more than usual here: with
// 227 KB of the SM's 256 KB configured as shared memory there is almost no L1 left, so every spill access is an L2 round trip.
#ifndef KB_SOFTMAX_REGS
#define KB_SOFTMAX_REGS 224
#endif
constexpr int SOFTMAX_REGS = KB_SOFTMAX_REGS, OTHER_REGS = (ATTN_THREADS * 168 - 256 * SOFTMAX_REGS) / 128;
static_assert(256 * SOFTMAX_REGS + 128 * OTHER_REGS == ATTN_THREADS * 168 && OTHER_REGS % 8 == 0 && OTHER_REGS >= 24, "register split");
// Shared memory (dynamic, 1024-byte aligned): MODE_PAIR: Q0, Q1, K/V ring, one tile of output staging (a 64-column half per
// stream, so that a Q tile is free for the next segment's Q as soon as the segment's last S product is done - head-split
// runs still stage in the Q tile), 1 KB of barriers and shared words. MODE_NAG: Q, two tiles holding the previous item's unblended g and Z+ as fp16 (see the
// NAG epilogue), K/V ring, 3 KB control block (barriers, words, 2.5 KB of epilogue scratch): exactly the 227 KB a thread
// block may have.
constexpr int CTRL_BYTES_PAIR = 1024, CTRL_BYTES_NAG = 3072;
constexpr int ATTN_TILES_PAIR = 3 + NSTAGE, ATTN_TILES_NAG = 3 + NSTAGE;
constexpr int ATTN_SMEM_PAIR = ATTN_TILES_PAIR * TILE_BYTES + CTRL_BYTES_PAIR;
constexpr int ATTN_SMEM_NAG = ATTN_TILES_NAG * TILE_BYTES + CTRL_BYTES_NAG;
static_assert(ATTN_SMEM_NAG <= 232448, "shared memory per thread block on sm_100");

// error bits written to the status word
constexpr uint32_t ST_TIMEOUT = 1u;

constexpr int MAX_PEERS = 8;

// Scratch one CTA needs for the partial result of a cut item: per stream O[128 columns][128 rows], m[128], l[128] (fp32)
constexpr int PART_STREAM_FLOATS = HD * BM + 2 * BM;
constexpr size_t PART_CTA_BYTES = 2 * (size_t)PART_STREAM_FLOATS * sizeof(float);

struct AttnParams {
    void* out;          // [B*Tq, ldo]
    int ldo;
    // Head-split runs (MODE_PAIR, 16-bit output): the output tile is stored into the [B*Tq, ldo] buffer of every
    // GPU in `out_peers` (this GPU's own buffer included) at column offset col0, and each finished 128-row tile
    // bumps the arrival counter of every peer. n_peers = 0 on the ordinary single-buffer path.
    void* out_peers[MAX_PEERS];
    unsigned long long* ctr_peers[MAX_PEERS];
    int n_peers, col0;
    int Tq, H, B;
    int n_items;        // MODE_PAIR: ceil(Tq/256) * H * B; MODE_NAG: ceil(Tq/128) * H
    int Tk[2];          // MODE_PAIR uses [0]; MODE_NAG: positive, negative context
    int npad[2];
    float scale_log2;   // log2(e) / sqrt(128)
    float nag_s, nag_tau, nag_alpha;
    float* nag_part;    // MODE_NAG scratch [ceil(Tq/128)][nag_heads][2 column halves][2][128]: per head and half of its columns |Z+|_1 and |g|_1 of each row
    unsigned int* nag_flag;  // MODE_NAG [ceil(Tq/128)] arrival counters: a tile is complete at nag_epoch * nag_heads
    // The per-token norms span ALL heads of the model. Single GPU: nag_heads = H, nag_h0 = 0, nag_epoch = 1 and the counters
    // are zeroed before the launch. Head split: this GPU holds heads [nag_h0, nag_h0 + H) of nag_heads; every CTA stores its
    // head's two norms per row into the scratch of EVERY GPU (nag_part_peers) and bumps every GPU's counter
    // (nag_flag_peers), so each GPU blends with the norms over all heads; the counters only grow (nag_epoch-th call).
    int nag_heads, nag_h0;
    unsigned int nag_epoch;
    // MODE_PAIR, optional (the backward pass): [B][H][ceil(Tq/128)][2][128] floats; the first 128 of a query block receive
    // L = log2 of each row's softmax denominator in units of scale_log2 * score (so that P = 2^(scale_log2 * s - L))
    float* stats;
    float* nag_part_peers[MAX_PEERS];
    unsigned int* nag_flag_peers[MAX_PEERS];
    int split;          // MODE_PAIR: balanced (item, key block) ranges per CTA with partial results merged
    float* part;        // split: [gridDim.x] slots of PART_CTA_BYTES
    unsigned int* part_flag;  // split: [gridDim.x][2 streams], zero before the launch; 1 = slot written
    uint32_t* status;   // device word, OR-ed with ST_* on failure
};

// barrier slots inside the control block
enum { BAR_QFULL = 0, BAR_QEMPTY = 2, BAR_SFULL = 4, BAR_SREQ = 6, BAR_PFULL = 8, BAR_PEMPTY = 10, BAR_ODONE = 12, BAR_OFREE = 14,
       BAR_SFREE = 16, BAR_PARKED = 17, BAR_NORMS = 18, BAR_KVFULL = 20, BAR_KVEMPTY = 20 + NSTAGE, BAR_COUNT = 20 + 2 * NSTAGE };
// when a stream asks for its next S: 0 = before its exponentials, 1 = after the first half of them, 2 = with P (no overlap)
#ifndef KB_SREQ_AT
#define KB_SREQ_AT 1
#endif

// full-CTA barrier usable from divergent role branches (same id and count everywhere)
__device__ __forceinline__ void cta_sync() { named_bar_sync(2, ATTN_THREADS); }

template <int DT>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
    if constexpr (DT == DT_BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}

// store 32 consecutive output columns of one row
template <typename OutT>
__device__ __forceinline__ void store32(OutT* dst, const float (&v)[32]) {
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
        for (int i = 0; i < 8; i++) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
        constexpr int DT = std::is_same<OutT, __nv_bfloat16>::value ? DT_BF16 : DT_F16;
#pragma unroll
        for (int i = 0; i < 4; i++)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(pack16<DT>(v[8 * i], v[8 * i + 1]), pack16<DT>(v[8 * i + 2], v[8 * i + 3]),
                                                          pack16<DT>(v[8 * i + 4], v[8 * i + 5]), pack16<DT>(v[8 * i + 6], v[8 * i + 7]));
    }
}

// One work segment: which rows, head and batch element, and which 128-key blocks [jb, je[i]) each stream runs
// (je[i] <= jb: the stream does not exist in this segment). nb = blocks of the whole item (MODE_PAIR).
struct Seg {
    int q0, h, b, qt;
    int jb, je[2], nb;
};

// Every role of a CTA walks the same segment list.
template <int MODE>
struct SegIter {
    long long s, s_end;     // split: steps (item * nb + block) of this CTA
    int w, nb;
    const AttnParams& p;
    __device__ __forceinline__ SegIter(const AttnParams& p_) : p(p_) {
        nb = (p.Tk[0] + BN - 1) / BN;
        w = blockIdx.x;
        s = s_end = 0;
        if (MODE == MODE_PAIR && p.split) {
            const long long n = (long long)p.n_items * nb;
            s = n * blockIdx.x / gridDim.x;
            s_end = n * (blockIdx.x + 1) / gridDim.x;
        }
    }
    __device__ __forceinline__ bool next(Seg& o) {
        int item, jb, je;
        if (MODE == MODE_PAIR && p.split) {
            if (s >= s_end) return false;
            item = (int)(s / nb);
            jb = (int)(s % nb);
            const long long rem = s_end - s;
            je = (rem < (long long)(nb - jb)) ? jb + (int)rem : nb;
            s += je - jb;
        } else {
            if (w >= p.n_items) return false;
            item = w;
            jb = 0;
            je = nb;
            w += gridDim.x;
        }
        o.jb = jb;
        o.nb = nb;
        if (MODE == MODE_PAIR) {
            const int nqp = (p.Tq + 2 * BM - 1) / (2 * BM);       // query-tile pairs per (batch, head), fastest: K/V reuse in L2
            const int qp = item % nqp, hb = item / nqp;
            o.h = hb % p.H;
            o.b = hb / p.H;
            o.q0 = qp * 2 * BM;
            o.qt = qp;
            o.je[0] = je;
            o.je[1] = (o.q0 + BM < p.Tq) ? je : jb;
        } else {
            o.h = item % p.H;                                     // heads fastest: the heads of a query tile run side by side
            o.qt = item / p.H;
            o.b = 0;
            o.q0 = o.qt * BM;
            o.je[0] = (p.Tk[0] + BN - 1) / BN;
            o.je[1] = (p.Tk[1] + BN - 1) / BN;
        }
        return true;
    }
};

// K/V ring bookkeeping. The loader fills ring entries in a fixed order and every consumer counts the same way:
//   MODE_PAIR segment: K(jb), then per key block V(j), K(j+1): K(j) is entry 2(j-jb), V(j) entry 2(j-jb)+1 of the segment;
//   MODE_NAG item: K0(0), K1(0), then per block j and stream i (0 first): V_i(j), K_i(j+1).
// nag_entry returns the entry of V_i(j) within the item (K_i(j+1), when it exists, is the next one).
__device__ __forceinline__ int nag_entry(int i, int j, int L0, int L1) {
    int e = (L0 > 0) + (L1 > 0);
    const int L[2] = {L0, L1};
#pragma unroll
    for (int ii = 0; ii < 2; ii++) {
        if (L[ii] <= 0) continue;
        const int full = j < L[ii] ? j : L[ii];                  // blocks of stream ii before block j
        e += 2 * full - (j >= L[ii] ? 1 : 0);                     // two entries per block, the last block only its V
        if (ii < i && j < L[ii]) e += 1 + (j + 1 < L[ii] ? 1 : 0);   // stream 0's entries of block j come first
    }
    return e;
}
__device__ __forceinline__ int seg_entries(int mode, int jb, const int (&je)[2]) {
    if (mode == MODE_PAIR) return 2 * (je[0] - jb);
    return (je[0] > 0 ? 2 * je[0] : 0) + (je[1] > 0 ? 2 * je[1] : 0);
}

template <int MODE, typename OutT>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK0,
                const __grid_constant__ CUtensorMap tmV0, const __grid_constant__ CUtensorMap tmK1,
                const __grid_constant__ CUtensorMap tmV1, const __grid_constant__ CUtensorMap tmO, const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];         // 128-byte swizzle wants 1024-byte aligned tiles
    const uint32_t base = smem_u32(smem_raw);
    uint8_t* const smem = smem_raw;
    if (base & 1023u) {                                           // never seen; without it every tile would be garbage
        if (threadIdx.x == 0) atomicOr(p.status, ST_TIMEOUT);
        return;
    }
    constexpr int N_FRONT = MODE == MODE_NAG ? 3 : 2;             // tiles in front of the K/V ring
    const uint32_t sQ = base;
    const uint32_t sKV = base + N_FRONT * TILE_BYTES;             // NSTAGE tiles
    constexpr int N_BACK = MODE == MODE_PAIR ? 1 : 0;             // MODE_PAIR: the output staging tile behind the ring
    uint8_t* const ctrl = smem + (N_FRONT + NSTAGE + N_BACK) * TILE_BYTES;
    const uint32_t bars = sKV + (NSTAGE + N_BACK) * TILE_BYTES;   // BAR_COUNT x 8 bytes
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 256);
    volatile uint32_t* const abort_flag = reinterpret_cast<volatile uint32_t*>(ctrl + 260);
    volatile uint32_t* const warp_ok = reinterpret_cast<volatile uint32_t*>(ctrl + 264);   // [8] per softmax warp
    volatile uint32_t* const wg_stop = reinterpret_cast<volatile uint32_t*>(ctrl + 296);   // [2] per softmax warpgroup
    volatile uint32_t* const wg_here = reinterpret_cast<volatile uint32_t*>(ctrl + 304);   // [2] per softmax warpgroup; NAG: [1] = warp 11's norm totals are good
    volatile uint32_t* const sm_item = reinterpret_cast<volatile uint32_t*>(ctrl + 312);   // [1] NAG: query tile of the item just parked
    volatile uint32_t* const sm_store = reinterpret_cast<volatile uint32_t*>(ctrl + 316);  // [3] NAG: {a blended tile waits in the Q tile, its head, its first row}
    float* const fbuf = reinterpret_cast<float*>(ctrl + 512);     // MODE_NAG epilogue scratch: 1/l of both streams [2][128], norm totals [2][128]
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int i = 0; i < BAR_COUNT; i++) {
            uint32_t count = 1;
            if (i >= BAR_SREQ && i < BAR_SREQ + 2) count = 4;               // one arrival per softmax warp of the stream
            if (i >= BAR_PFULL && i < BAR_PFULL + 2) count = 4;
            if (i == BAR_SFREE) count = 4;
            if (i >= BAR_KVEMPTY && i < BAR_KVEMPTY + NSTAGE) count = MODE == MODE_PAIR ? 2 : 1;   // PAIR: both streams use every K/V tile
            if (i >= BAR_OFREE && i < BAR_OFREE + 2) count = MODE == MODE_NAG ? 8 : 4;   // NAG: both warpgroups read both O
            mbar_init(bar(i), count);
        }
        *abort_flag = 0u;
        sm_store[0] = 0u;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK0); tma_prefetch_desc(&tmV0);
        if (MODE == MODE_NAG) { tma_prefetch_desc(&tmK1); tma_prefetch_desc(&tmV1); }
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // 384 threads start with 168 registers each; the MMA/TMA warpgroup gives most of its share to the
    // softmax ones. Everything a softmax thread runs from here on sits inside this branch so that the
    // register budget of the branch is known at compile time; the final full-CTA barrier is therefore
    // written as the same bar.sync id from both branches.
    if (warp < 8) {
        setmaxnreg_inc<SOFTMAX_REGS>();
        // ------------------------------------------------------------------ softmax, one row per thread
        const int i = warp >> 2;                                   // stream = warpgroup
        const int t = tid & 127;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tR = tmem_base + lane_base;                                  // score staging, shared by both streams
        const uint32_t tP = tmem_base + lane_base + 128u + (uint32_t)(i * 64);
        const uint32_t tO = tmem_base + lane_base + 256u + (uint32_t)(i * 128);
        const float c = p.scale_log2;
        uint32_t sf_cnt = 0, od_cnt = 0, pe_cnt = 0;               // uses of s_full[i] / o_done[i] / p_empty[i] so far (phase parity)
        uint32_t ring0 = 0;                                        // K/V ring entries of all earlier segments

        // MODE_NAG, 16-bit output: the item parked in shared memory, waiting for its blend
        bool pend_valid = false, pend_go = false;
        int pend_h = 0, pend_q0 = 0;
        float pend_tp = 0.f, pend_tg = 0.f;                        // its |Z+|_1 and |g|_1 over all heads, this thread's row
        uint32_t norms_cnt = 0;                                    // parked items whose norms have been taken over so far
        float* const f_tot = fbuf + 256;                           // [2][128] norm totals of the parked item, written by warp 11
        constexpr int NORM_STRIDE = 512;                           // floats per (query tile, head) in the norm scratch
        // one thread waits (bounded) until all heads of query tile qt have published their norms; result in wg_here[0]
        auto nag_wait_norms = [&](int qt) {
            if (tid == 0) {
                const uint32_t target = p.nag_epoch * (uint32_t)p.nag_heads;
                const uint64_t t0 = globaltimer_ns();
                uint32_t seen = 0;
                for (;;) {
                    if (p.n_peers == 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.nag_flag + qt) : "memory");
                    else asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.nag_flag + qt) : "memory");
                    if (seen >= target || *abort_flag) break;
                    if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { *abort_flag = 1u; break; }
                    __nanosleep(32);
                }
                wg_here[0] = (seen >= target) ? 1u : 0u;
            }
            named_bar_sync(1, 256);
        };
        // The parked item, in two steps. Step one (blend = false): take over the norms of all heads that warp 11 has summed
        // into shared memory during the main loop. Step two (blend = true): blend the parked tiles in place and start the
        // store. Every barrier inside depends only on pend_valid and n_peers, which all 256 threads agree on.
        auto nag_finish = [&](bool blend) {
            if (MODE != MODE_NAG || sizeof(OutT) != 2 || !pend_valid) return;
            if (!blend) {
                const bool got = __all_sync(0xffffffffu, mbar_wait(bar(BAR_NORMS), norms_cnt & 1u, abort_flag));
                ++norms_cnt;
                pend_go = got && wg_here[1] != 0u;
                pend_tp = f_tot[t];
                pend_tg = f_tot[128 + t];
                return;
            }
            constexpr int ODT = std::is_same<OutT, __nv_bfloat16>::value ? DT_BF16 : DT_F16;
            const int wg = warp >> 2;
            // The blend below writes into the Q tile: both streams' MMAs of the current item must be complete first (each
            // warpgroup has waited for its own stream's last P*V only, and the streams may differ in length).
            named_bar_sync(1, 256);
            const float ratio = pend_tg / fmaxf(pend_tp, 1e-12f);
            const float kclamp = ratio > p.nag_tau ? p.nag_tau / ratio : 1.f;
            const float ag = p.nag_alpha * kclamp, ap = 1.f - p.nag_alpha;
            // The blended tile goes into the Q tile, which is dead here (every S MMA of the current item has completed and the
            // loader is only told so once the store below has read it): the parking tiles are free for the current item at once.
            uint8_t* const stage = smem;
            if (pend_go) {
                uint8_t* const to = stage + wg * HALF_BYTES + t * 128;
                const uint8_t* const tg = smem + TILE_BYTES + wg * HALF_BYTES + t * 128;
                const uint8_t* const tz = smem + 2 * TILE_BYTES + wg * HALF_BYTES + t * 128;
#pragma unroll
                for (int cc = 0; cc < 8; cc++) {
                    const uint4 g4 = *reinterpret_cast<const uint4*>(tg + ((cc ^ (t & 7)) << 4));
                    const uint4 z4 = *reinterpret_cast<const uint4*>(tz + ((cc ^ (t & 7)) << 4));
                    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, zw[4] = {z4.x, z4.y, z4.z, z4.w};
                    uint32_t ow[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&gw[e]));
                        const float2 zf = __half22float2(*reinterpret_cast<const __half2*>(&zw[e]));
                        ow[e] = pack16<ODT>(ag * gf.x + ap * zf.x, ag * gf.y + ap * zf.y);
                    }
                    *reinterpret_cast<uint4*>(to + ((cc ^ (t & 7)) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                }
                if (p.n_peers == 0) fence_proxy_async_smem();
            }
            named_bar_sync(1, 256);                                           // the blended tile is complete, the parking tiles are read out
            if (p.n_peers == 0) {
                // the loader warp stores the tile (bulk tensor store, rows past Tq clipped by the tensor map) before it loads the
                // next Q into the same space: nobody here waits for the store to read the tile
                if (tid == 0) { sm_store[1] = (uint32_t)pend_h; sm_store[2] = (uint32_t)pend_q0; sm_store[0] = pend_go ? 1u : 0u; }
            } else {
                // head split: each of the eight warps copies 16 rows out as whole 256-byte rows to every GPU's buffer
                if (pend_go) {
                    const int lr0 = 16 * warp;
                    const int row0 = pend_q0 + lr0;
                    const int nrow = p.Tq - row0;                             // rows of this warp that exist (warp-uniform)
                    uint2 vals[16];
#pragma unroll
                    for (int rr = 0; rr < 16; rr++)
                        vals[rr] = *reinterpret_cast<const uint2*>(stage + (lane >> 4) * HALF_BYTES + (lr0 + rr) * 128 +
                                                                   ((((lane >> 1) & 7) ^ ((lr0 + rr) & 7)) << 4) + (lane & 1) * 8);
                    const size_t off = (size_t)row0 * (size_t)p.ldo + (size_t)(p.col0 + pend_h * HD) + (size_t)lane * 4;
                    for (int pe = 0; pe < p.n_peers; pe++) {
                        OutT* g = reinterpret_cast<OutT*>(p.out_peers[pe]) + off;
#pragma unroll
                        for (int rr = 0; rr < 16; rr++)
                            if (rr < nrow) *reinterpret_cast<uint2*>(g + (size_t)rr * (size_t)p.ldo) = vals[rr];
                    }
                    __threadfence_system();                                   // the tile is visible to every GPU before the arrival
                }
                named_bar_sync(1, 256);                                       // every warp is done with the parked tile
                if (pend_go && tid < p.n_peers) atomicAdd_system(p.ctr_peers[tid], 1ull);
                if (tid == 0) sm_store[0] = 0u;
            }
            pend_valid = false;
        };

        SegIter<MODE> iter(p);
        Seg it;
        while (iter.next(it)) {
            const int jb = it.jb, je = it.je[i];
            const int Tk = p.Tk[MODE == MODE_NAG ? i : 0];
            const int j_last = (Tk + BN - 1) / BN - 1;             // the block that may be ragged
            float row_m = -INFINITY, row_l = 0.f;
            bool ok = true;
            // this stream's K/V ring entries: a slot goes back to the loader when the MMAs that read it are done, which the
            // softmax threads see anyway (S done: s_full; P*V done: p_empty / o_done) - a plain arrive by one thread instead
            // of a tcgen05.commit by the MMA warp, each of which costs the tensor pipe ~100 cycles (measured)
            const bool two = MODE == MODE_PAIR && it.je[1] > jb;
            auto release = [&](uint32_t entry) {
                if (t == 0) {
                    mbar_arrive(bar(BAR_KVEMPTY + (ring0 + entry) % NSTAGE));
                    if (MODE == MODE_PAIR && !two) mbar_arrive(bar(BAR_KVEMPTY + (ring0 + entry) % NSTAGE));   // stream 1 is absent: its share too
                }
            };
            auto k_entry = [&](int j) { return (uint32_t)(MODE == MODE_PAIR ? 2 * (j - jb) : (j == 0 ? (i == 1 && it.je[0] > 0 ? 1 : 0) : nag_entry(i, j - 1, it.je[0], it.je[1]) + 1)); };
            auto v_entry = [&](int j) { return (uint32_t)(MODE == MODE_PAIR ? 2 * (j - jb) + 1 : nag_entry(i, j, it.je[0], it.je[1])); };
            for (int j = jb; j < je; ++j) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_SFULL + i), sf_cnt & 1u, abort_flag));
                ++sf_cnt;
                if (!ok) break;
                tc_fence_after();
                // the segment's last S product is done: nothing reads this stream's Q tile any more, the next segment's Q may
                // load under the rest of this one (head-split runs stage their output in the Q tile and release it later)
                if (MODE == MODE_PAIR && j == je - 1 && t == 0 && (sizeof(OutT) == 4 || p.n_peers == 0)) mbar_arrive(bar(BAR_QEMPTY + i));
                uint32_t s[4][32];
#pragma unroll
                for (int q = 0; q < 4; q++) tmem_ld32(tR + 32u * q, s[q]);
                tmem_wait_ld();
#pragma unroll
                for (int q = 0; q < 4; q++) reg_fence32(s[q]);
                // the scores are in registers: the staging area may take the next S (of the other stream, normally)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_SFREE));
                release(k_entry(j));                               // S_i(j) is complete: this stream is done with K(j)
                if (j == j_last && (Tk & (BN - 1))) {              // ragged last block: keys >= Tk score -inf
                    const int valid = Tk - j * BN;
#pragma unroll
                    for (int q = 0; q < 4; q++)
#pragma unroll
                        for (int e = 0; e < 32; e++)
                            if (q * 32 + e >= valid) s[q][e] = 0xff800000u;
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {                  // 3-input max: two scores per instruction
                    mx0 = max3(mx0, __uint_as_float(s[0][e]), __uint_as_float(s[0][e + 1]));
                    mx1 = max3(mx1, __uint_as_float(s[1][e]), __uint_as_float(s[1][e + 1]));
                    mx2 = max3(mx2, __uint_as_float(s[2][e]), __uint_as_float(s[2][e + 1]));
                    mx3 = max3(mx3, __uint_as_float(s[3][e]), __uint_as_float(s[3][e + 1]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
                if (KB_SREQ_AT == 0 && j + 1 < je) { __syncwarp(); if (lane == 0) mbar_arrive(bar(BAR_SREQ + i)); }
                // The previous P*V of this stream reads P_i and writes O_i: it must be complete before either is touched.
                // That wait sits as late as possible: before the first store of P, or before a rescale of O.
                bool pv_done = false;
                auto wait_pv = [&]() {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_PEMPTY + i), (pe_cnt & 1u) ^ 1u, abort_flag));
                    ++pe_cnt;
                    tc_fence_after();
                    pv_done = true;
                    if (ok && j > jb) release(v_entry(j - 1));     // P_i(j-1) V(j-1) is complete: this stream is done with V(j-1)
                };
                if (j == jb) {
                    row_m = mx;
                } else {
                    // Keep a stale maximum while the new one is less than 2^8 above it: P stays <= 256, which
                    // fp16 and the fp32 sums hold exactly as well, and O needs no rescale.
                    const bool need = (mx - row_m) * c > 8.f;
                    if (__any_sync(0xffffffffu, need)) {
                        wait_pv();
                        if (!ok) break;
                        const float mn = fmaxf(row_m, mx);
                        const float a = ex2((row_m - mn) * c);
                        row_l *= a;
                        row_m = mn;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint32_t o[32];
                            tmem_ld32(tO + 32u * q, o);
                            tmem_wait_ld();
                            reg_fence32(o);
#pragma unroll
                            for (int e = 0; e < 32; e++) o[e] = __float_as_uint(__uint_as_float(o[e]) * a);
                            tmem_st32(tO + 32u * q, o);
                        }
                    }
                }
                // p = 2^(s*c - m*c) on packed pairs: one FFMA2 per two scores, then MUFU ex2 (and the FMA-pipe
                // polynomial for POLY_PAIRS of every 8 pairs, when enabled).
                const uint64_t c2 = pack2(c, c), nmc2 = pack2(-row_m * c, -row_m * c);
                uint64_t sum2a = pack2(0.f, 0.f), sum2b = sum2a;
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    uint32_t pk[32];
#pragma unroll
                    for (int e = 0; e < 32; e++) {                 // pair e of this half: scores 2e, 2e+1 of chunk 2q + e/16
                        const int ch = 2 * q + (e >> 4), ee = (e & 15) * 2;
                        const uint64_t x2 = fma2(pack2u(s[ch][ee], s[ch][ee + 1]), c2, nmc2);
                        uint64_t p2;
                        if ((e & 7) >= 8 - POLY_PAIRS) {
                            p2 = ex2_poly2(x2);
                        } else {
                            float x0, x1;
                            unpack2(x2, x0, x1);
                            p2 = pack2(ex2(x0), ex2(x1));
                        }
                        if (e & 1) sum2b = add2(sum2b, p2); else sum2a = add2(sum2a, p2);
                        float p0, p1;
                        unpack2(p2, p0, p1);
                        pk[e] = pack16<DT_F16>(p0, p1);
                    }
                    if (q == 0) {
                        reg_fence32(pk);                           // the first half is computed before the wait below, not after it
                        if (!pv_done) wait_pv();
                        if (!ok) break;
                    }
                    tmem_st32(tP + 32u * q, pk);                   // P: key pair (2c, 2c+1) in column c
                    if (q == 0) {
                        // Ask for the next S of this stream now: it runs on the tensor core under the second half of the
                        // exponentials. The register fences keep that second half from being scheduled ahead of the request.
                        if (KB_SREQ_AT == 1 && j + 1 < je) { __syncwarp(); if (lane == 0) mbar_arrive(bar(BAR_SREQ + i)); }
                        reg_fence32(s[2]);
                        reg_fence32(s[3]);
                    }
                }
                if (!ok) break;
                float sum0, sum1, sum2, sum3;
                unpack2(sum2a, sum0, sum1);
                unpack2(sum2b, sum2, sum3);
                row_l += (sum0 + sum2) + (sum1 + sum3);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (KB_SREQ_AT == 2 && j + 1 < je) mbar_arrive(bar(BAR_SREQ + i));
                    mbar_arrive(bar(BAR_PFULL + i));
                }
            }
            const bool mine = je > jb;                                         // this stream exists in the segment
            nag_finish(false);                                                 // the parked item's norms, fetched under the wait below
            if (ok && mine) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_ODONE + i), od_cnt & 1u, abort_flag));
                tc_fence_after();
                if (ok) release(v_entry(je - 1));                              // the last P*V is complete: done with its V
            }
            if (mine) ++od_cnt;
            ring0 += (uint32_t)seg_entries(MODE, jb, it.je);

            // ---------------------------------------------------------------- epilogue of the segment
            if (MODE == MODE_PAIR) {
                if (mine) {
                    // Make `ok` uniform over the stream's four warps before barriers only they take part in; this
                    // barrier is reached unconditionally, so a warp that gave up cannot leave the others waiting.
                    if (lane == 0) warp_ok[warp] = ok ? 1u : 0u;
                    named_bar_sync(3 + i, 128);
                    const int w0 = warp & 4;
                    ok = (warp_ok[w0] & warp_ok[w0 + 1] & warp_ok[w0 + 2] & warp_ok[w0 + 3]) != 0u;
                    const float M = row_m * c;                                 // running maximum in log2 units
                    if (jb > 0) {
                        // later blocks of a cut item: the unnormalised result goes to this CTA's scratch slot, four columns of a
                        // row together and rows adjacent (16-byte stores, coalesced over rows), and the stream's flag is raised
                        float* const slot = p.part + (size_t)blockIdx.x * (2 * PART_STREAM_FLOATS) + (size_t)i * PART_STREAM_FLOATS;
                        if (ok) {
                            slot[HD * BM + t] = M;
                            slot[HD * BM + BM + t] = row_l;
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                uint32_t o[32];
                                tmem_ld32(tO + 32u * q, o);
                                tmem_wait_ld();
                                reg_fence32(o);
#pragma unroll
                                for (int e4 = 0; e4 < 8; e4++)                 // [column / 4][row][4]: a warp writes 512 contiguous bytes
                                    reinterpret_cast<float4*>(slot)[(size_t)(q * 8 + e4) * BM + t] =
                                        make_float4(__uint_as_float(o[4 * e4]), __uint_as_float(o[4 * e4 + 1]), __uint_as_float(o[4 * e4 + 2]),
                                                    __uint_as_float(o[4 * e4 + 3]));
                            }
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar(BAR_OFREE + i));
                            if (t == 0 && sizeof(OutT) == 2 && p.n_peers != 0) mbar_arrive(bar(BAR_QEMPTY + i));
                        }
                        __threadfence();
                        named_bar_sync(3 + i, 128);                            // every thread's stores are ordered before the flag
                        if (ok && t == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.part_flag + 2 * blockIdx.x + i), "r"(1u) : "memory");
                    } else {
                        // CTAs after this one whose range starts inside this item hold the rest of it
                        int n_rest = 0;
                        if (p.split && je < it.nb) {
                            const long long n = (long long)p.n_items * it.nb, item_end = iter.s - je + it.nb;   // iter.s: this segment's end
                            for (int cc = blockIdx.x + 1; cc < (int)gridDim.x && n * cc / gridDim.x < item_end; cc++) n_rest++;
                        }
                        if (n_rest > 0) {
                            if (t == 0) {
                                bool here = true;
                                const uint64_t t0 = globaltimer_ns();
                                for (int r = 1; r <= n_rest && here; r++) {
                                    for (;;) {
                                        uint32_t seen;
                                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.part_flag + 2 * (blockIdx.x + r) + i) : "memory");
                                        if (seen) break;
                                        if (*abort_flag) { here = false; break; }
                                        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { *abort_flag = 1u; here = false; break; }
                                        __nanosleep(64);
                                    }
                                }
                                wg_here[i] = here ? 1u : 0u;
                            }
                            named_bar_sync(3 + i, 128);
                            ok = ok && wg_here[i] != 0u;
                        }
                        if (ok) {
                            // statistics of all parts first, then one pass over the columns
                            float Mf = M;
                            for (int r = 1; r <= n_rest; r++)
                                Mf = fmaxf(Mf, __ldcg(p.part + (size_t)(blockIdx.x + r) * (2 * PART_STREAM_FLOATS) + (size_t)i * PART_STREAM_FLOATS + HD * BM + t));
                            const float a_mine = ex2(M - Mf);
                            float l = row_l * a_mine;
                            for (int r = 1; r <= n_rest; r++) {
                                const float* slot = p.part + (size_t)(blockIdx.x + r) * (2 * PART_STREAM_FLOATS) + (size_t)i * PART_STREAM_FLOATS;
                                l += __ldcg(slot + HD * BM + BM + t) * ex2(__ldcg(slot + HD * BM + t) - Mf);
                            }
                            float scale = 1.f;
                            if (p.npad[0]) {                                   // engine/src/tcflash.cuh:140-144
                                const float mn = fmaxf(Mf, 0.f);
                                scale = exp2f(Mf - mn);
                                l = l * scale + (float)p.npad[0] * exp2f(-mn);
                            }
                            const float inv = scale / l;
                            const float k_mine = a_mine * inv;
                            if (p.stats)
                                p.stats[(((size_t)it.b * p.H + it.h) * ((p.Tq + BM - 1) / BM) + (size_t)(it.q0 / BM + i)) * 256 + t] =
                                    (p.npad[0] ? fmaxf(Mf, 0.f) : Mf) + log2f(l);
                            // one 32-column chunk of the merged, normalised row
                            auto chunk = [&](int q, float (&v)[32]) {
                                uint32_t o[32];
                                tmem_ld32(tO + 32u * q, o);
                                tmem_wait_ld();
                                reg_fence32(o);
#pragma unroll
                                for (int e = 0; e < 32; e++) v[e] = __uint_as_float(o[e]) * k_mine;
                                for (int r = 1; r <= n_rest; r++) {
                                    const float* slot = p.part + (size_t)(blockIdx.x + r) * (2 * PART_STREAM_FLOATS) + (size_t)i * PART_STREAM_FLOATS;
                                    const float k_r = ex2(__ldcg(slot + HD * BM + t) - Mf) * inv;
#pragma unroll
                                    for (int e4 = 0; e4 < 8; e4++) {
                                        const float4 pv = __ldcg(reinterpret_cast<const float4*>(slot) + (size_t)(q * 8 + e4) * BM + t);
                                        v[4 * e4] += pv.x * k_r; v[4 * e4 + 1] += pv.y * k_r; v[4 * e4 + 2] += pv.z * k_r; v[4 * e4 + 3] += pv.w * k_r;
                                    }
                                }
                            };
                            if constexpr (sizeof(OutT) == 2) {
                                constexpr int ODT = std::is_same<OutT, __nv_bfloat16>::value ? DT_BF16 : DT_F16;
                                if (p.n_peers == 0) {
                                    // 16-bit output: the tile leaves in two rounds of 64 columns through this stream's own
                                    // [128][64] staging half (128-byte rows, 128-byte swizzle: what a bulk tensor store reads);
                                    // rows past Tq are clipped by the tensor map
                                    uint8_t* const half_stage = smem + (2 + NSTAGE) * TILE_BYTES + i * HALF_BYTES;
#pragma unroll
                                    for (int hh = 0; hh < 2; hh++) {
#pragma unroll
                                        for (int q2 = 0; q2 < 2; q2++) {
                                            float v[32];
                                            chunk(2 * hh + q2, v);
#pragma unroll
                                            for (int cc = 0; cc < 4; cc++) {
                                                uint4 pk;
                                                pk.x = pack16<ODT>(v[8 * cc + 0], v[8 * cc + 1]);
                                                pk.y = pack16<ODT>(v[8 * cc + 2], v[8 * cc + 3]);
                                                pk.z = pack16<ODT>(v[8 * cc + 4], v[8 * cc + 5]);
                                                pk.w = pack16<ODT>(v[8 * cc + 6], v[8 * cc + 7]);
                                                *reinterpret_cast<uint4*>(half_stage + t * 128 + (((4 * q2 + cc) ^ (t & 7)) << 4)) = pk;
                                            }
                                        }
                                        if (hh == 1) {
                                            tc_fence_before();
                                            __syncwarp();
                                            if (lane == 0) mbar_arrive(bar(BAR_OFREE + i));   // O_i is read out: the next segment's P*V may start
                                        }
                                        fence_proxy_async_smem();
                                        named_bar_sync(3 + i, 128);              // the staged half is complete
                                        if (t == 0) {
                                            tma_store_3d(&tmO, smem_u32(half_stage), it.h * HD + 64 * hh, it.q0 + i * BM, it.b);
                                            tma_store_commit();
                                            tma_store_wait_read();               // the half may be overwritten
                                        }
                                        if (hh == 0) named_bar_sync(3 + i, 128);
                                    }
                                } else {
                                    // head-split runs: the tile is staged in this stream's Q tile (dead: every S product of the
                                    // stream has completed), then written as whole 256-byte rows to every peer buffer
                                    uint8_t* const stage = smem + i * TILE_BYTES;
#pragma unroll
                                    for (int q = 0; q < 4; q++) {
                                        float v[32];
                                        chunk(q, v);
#pragma unroll
                                        for (int cc = 0; cc < 4; cc++) {
                                            uint4 pk;
                                            pk.x = pack16<ODT>(v[8 * cc + 0], v[8 * cc + 1]);
                                            pk.y = pack16<ODT>(v[8 * cc + 2], v[8 * cc + 3]);
                                            pk.z = pack16<ODT>(v[8 * cc + 4], v[8 * cc + 5]);
                                            pk.w = pack16<ODT>(v[8 * cc + 6], v[8 * cc + 7]);
                                            *reinterpret_cast<uint4*>(stage + (q >> 1) * HALF_BYTES + t * 128 + ((((4 * q + cc) & 7) ^ (t & 7)) << 4)) = pk;
                                        }
                                    }
                                    tc_fence_before();
                                    __syncwarp();
                                    if (lane == 0) mbar_arrive(bar(BAR_OFREE + i));
                                    named_bar_sync(3 + i, 128);                  // the staged tile is complete
                                    // each warp copies 32 rows out as whole 256-byte rows to every peer buffer
                                    // (all shared-memory reads first, then the stores)
                                    const int lr0 = 32 * (warp & 3);
                                    const int row0 = it.q0 + i * BM + lr0;
                                    const int nrow = p.Tq - row0;                // rows of this warp that exist (warp-uniform)
                                    uint2 vals[32];
#pragma unroll
                                    for (int rr = 0; rr < 32; rr++)
                                        vals[rr] = *reinterpret_cast<const uint2*>(stage + (lane >> 4) * HALF_BYTES + (lr0 + rr) * 128 +
                                                                                   ((((lane >> 1) & 7) ^ ((lr0 + rr) & 7)) << 4) + (lane & 1) * 8);
                                    const size_t off = ((size_t)it.b * p.Tq + (size_t)row0) * (size_t)p.ldo + (size_t)(p.col0 + it.h * HD) + (size_t)lane * 4;
                                    for (int pe = 0; pe < p.n_peers; pe++) {
                                        OutT* g = reinterpret_cast<OutT*>(p.out_peers[pe]) + off;
#pragma unroll
                                        for (int rr = 0; rr < 32; rr++)
                                            if (rr < nrow) *reinterpret_cast<uint2*>(g + (size_t)rr * (size_t)p.ldo) = vals[rr];
                                    }
                                    __threadfence_system();                      // the tile is visible to every GPU before the arrival
                                    named_bar_sync(3 + i, 128);                  // every warp is done with the staging tile
                                    if (t < p.n_peers) atomicAdd_system(p.ctr_peers[t], 1ull);
                                }
                            } else {
                                const int row = it.q0 + i * BM + t;
                                OutT* dst = reinterpret_cast<OutT*>(p.out) + ((size_t)it.b * p.Tq + (size_t)row) * (size_t)p.ldo + (size_t)it.h * HD;
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    float v[32];
                                    chunk(q, v);
                                    if (row < p.Tq) store32<OutT>(dst + 32 * q, v);
                                }
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(bar(BAR_OFREE + i));
                            }
                            // head-split runs: the Q tile (the staging space in it) may now be overwritten by the next segment's Q
                            if (t == 0 && sizeof(OutT) == 2 && p.n_peers != 0) mbar_arrive(bar(BAR_QEMPTY + i));
                        }
                    }
                }
            } else {
                // NAG combine (engine/src/dit.cu:295-324) on Z+ = O0/l0 and Z- = O1/l1 straight from TMEM.
                // The clamp factor of a token needs |Z+|_1 and |g|_1 over ALL heads, i.e. from up to nag_heads other thread
                // blocks: publish this head's norms, get the others'. 16-bit outputs do not wait for that exchange: the item's
                // unblended g and Z+ are parked as fp16 tiles in shared memory, TMEM is handed back, the next item runs, and
                // the parked item is blended and stored one item later, when the other heads' norms have long arrived.
                float* const f_inv = fbuf;             // [2][128]  1/l per stream
                const int wg = i;                      // warpgroup wg takes head columns [64 wg, 64 wg + 64) of both outputs
                const uint32_t tOp = tmem_base + lane_base + 256u + (uint32_t)(wg * 64);
                const uint32_t tOn = tmem_base + lane_base + 384u + (uint32_t)(wg * 64);
                const float s = p.nag_s, sm1 = p.nag_s - 1.f;
                constexpr bool DEFER = sizeof(OutT) == 2;
                if constexpr (DEFER) {
                    if (tid == 0 && !pend_valid) sm_store[0] = 0u;        // nothing parked (first item): the Q tile is simply free
                    nag_finish(true);                                     // the parked item: blend into the Q tile
                    // every S MMA of the current item has completed and the blended tile (if any) is staged: the loader may
                    // store it and load the next Q
                    if (tid == 0 && ok) mbar_arrive(bar(BAR_QEMPTY + 0));
                }
                {
                    const float mc = row_m * p.scale_log2;
                    float scale = 1.f, l = row_l;
                    if (p.npad[wg]) {
                        const float mn = fmaxf(mc, 0.f);
                        scale = exp2f(mc - mn);
                        l = l * scale + (float)p.npad[wg] * exp2f(-mn);
                    }
                    f_inv[wg * 128 + t] = scale / l;
                }
                if (lane == 0) warp_ok[warp] = ok ? 1u : 0u;
                tc_fence_before();
                named_bar_sync(1, 256);                                   // both streams' O and 1/l are final
                ok = (warp_ok[0] & warp_ok[1] & warp_ok[2] & warp_ok[3] & warp_ok[4] & warp_ok[5] & warp_ok[6] & warp_ok[7]) != 0u;
                if (!DEFER && tid == 0 && ok) mbar_arrive(bar(BAR_QEMPTY + 0));   // every S MMA of the item has completed: the next Q may load
                const float ip = f_inv[t], in = f_inv[128 + t];
                float lp = 0.f, lg = 0.f;
                if (ok) {
                    tc_fence_after();
                    // DEFER: g and Z+ of this item are parked as two [128][128] fp16 tiles in the layout TMA stores (two
                    // 128-byte-swizzled halves), straight from the registers of this pass
                    uint8_t* const tg = smem + TILE_BYTES + wg * HALF_BYTES + t * 128;
                    uint8_t* const tz = smem + 2 * TILE_BYTES + wg * HALF_BYTES + t * 128;
#pragma unroll
                    for (int q = 0; q < 2; q++) {
                        uint32_t a[32], n[32];
                        tmem_ld32(tOp + 32u * q, a);
                        tmem_ld32(tOn + 32u * q, n);
                        tmem_wait_ld();
                        reg_fence32(a);
                        reg_fence32(n);
#pragma unroll
                        for (int cc = 0; cc < 4; cc++) {                      // 16-byte chunk 4q + cc of this thread's 128-byte half row
                            uint32_t gw[4], zw[4];
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const int k = 8 * cc + 2 * e;
                                const float pv0 = __uint_as_float(a[k]) * ip, pv1 = __uint_as_float(a[k + 1]) * ip;
                                const float g0 = pv0 * s - __uint_as_float(n[k]) * in * sm1, g1 = pv1 * s - __uint_as_float(n[k + 1]) * in * sm1;
                                lp += fabsf(pv0) + fabsf(pv1);
                                lg += fabsf(g0) + fabsf(g1);
                                gw[e] = pack16<DT_F16>(g0, g1);
                                zw[e] = pack16<DT_F16>(pv0, pv1);
                            }
                            if constexpr (DEFER) {
                                *reinterpret_cast<uint4*>(tg + (((4 * q + cc) ^ (t & 7)) << 4)) = make_uint4(gw[0], gw[1], gw[2], gw[3]);
                                *reinterpret_cast<uint4*>(tz + (((4 * q + cc) ^ (t & 7)) << 4)) = make_uint4(zw[0], zw[1], zw[2], zw[3]);
                            }
                        }
                    }
                    if constexpr (DEFER) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) { mbar_arrive(bar(BAR_OFREE + 0)); mbar_arrive(bar(BAR_OFREE + 1)); }   // both O read out
                    }
                }
                // publish this head's norms, per half of its columns: plain stores now, one fence and the arrival by one thread
                // after the barrier below (the barrier orders every thread's stores before that thread's release)
                const size_t tile_off = ((size_t)it.qt * p.nag_heads) * NORM_STRIDE;   // [nag_heads][2 halves][2 norms][128] of this query tile
                const size_t mine_off = tile_off + (size_t)(p.nag_h0 + it.h) * NORM_STRIDE + wg * 256 + t;
                if (p.n_peers == 0) {
                    p.nag_part[mine_off] = lp;
                    p.nag_part[mine_off + 128] = lg;
                } else {
                    for (int pe = 0; pe < p.n_peers; pe++) { p.nag_part_peers[pe][mine_off] = lp; p.nag_part_peers[pe][mine_off + 128] = lg; }   // plain stores over NVLink
                }
                named_bar_sync(1, 256);                                   // norms stored by everyone
                // The arrival on the tile's counter needs a fence that waits for those stores (a few thousand cycles): in the
                // deferred form warp 11 does both, so that nobody here waits for it. (The barrier above orders every thread's
                // stores before thread 0's mbarrier arrive, which warp 11 acquires before its own fence and release.)
                auto publish = [&](int qt) {
                    if (p.n_peers == 0) {
                        asm volatile("fence.acq_rel.gpu;" ::: "memory");
                        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.nag_flag + qt), "r"(1u) : "memory");
                    } else {
                        asm volatile("fence.acq_rel.sys;" ::: "memory");
                        for (int pe = 0; pe < p.n_peers; pe++)
                            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.nag_flag_peers[pe] + qt), "r"(1u) : "memory");
                    }
                };
                if constexpr (DEFER) {
                    // warp 11 publishes, then fetches this item's norms over all heads (it waits for the other heads itself); the
                    // totals of the item before were taken over by every thread before the barrier above
                    if (tid == 0) { sm_item[0] = (uint32_t)it.qt; mbar_arrive(bar(BAR_PARKED)); }
                    pend_valid = ok;
                    pend_h = it.h; pend_q0 = it.q0;
                } else {
                    // fp32 output: wait here for the other heads, blend from TMEM, store rows
                    if (tid == 0) publish(it.qt);
                    nag_wait_norms(it.qt);
                    const bool all_here = wg_here[0] != 0u;
                    float tp = 0.f, tg = 0.f;
                    if (all_here)
                        for (int hh = 0; hh < 2 * p.nag_heads; hh++) {        // head and half order: same sum everywhere
                            tp += __ldcg(p.nag_part + tile_off + (size_t)hh * 256 + t);
                            tg += __ldcg(p.nag_part + tile_off + (size_t)hh * 256 + 128 + t);
                        }
                    const float ratio = tg / fmaxf(tp, 1e-12f);
                    const float kclamp = ratio > p.nag_tau ? p.nag_tau / ratio : 1.f;
                    const float ag = p.nag_alpha * kclamp, ap = 1.f - p.nag_alpha;
                    const int row = it.q0 + t;
                    OutT* dst = reinterpret_cast<OutT*>(p.out) + (size_t)row * (size_t)p.ldo + (size_t)it.h * HD + wg * 64;
                    if (ok && all_here) {
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            uint32_t a[32], n[32];
                            float v[32];
                            tmem_ld32(tOp + 32u * q, a);
                            tmem_ld32(tOn + 32u * q, n);
                            tmem_wait_ld();
                            reg_fence32(a);
                            reg_fence32(n);
#pragma unroll
                            for (int e = 0; e < 32; e++) {
                                const float pv = __uint_as_float(a[e]) * ip;
                                const float nv = __uint_as_float(n[e]) * in;
                                v[e] = ag * (pv * s - nv * sm1) + ap * pv;
                            }
                            if (row < p.Tq) store32<OutT>(dst + 32 * q, v);
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) { mbar_arrive(bar(BAR_OFREE + 0)); mbar_arrive(bar(BAR_OFREE + 1)); }   // both O read out
                    }
                }
            }
            // leave the segment loop together once any role has given up (uniform per warpgroup; in NAG mode per CTA)
            if (MODE == MODE_PAIR) {
                if (t == 0) wg_stop[i] = *abort_flag;
                named_bar_sync(3 + i, 128);
                const bool stop = wg_stop[i] != 0u;
                named_bar_sync(3 + i, 128);
                if (stop) break;
            } else {
                named_bar_sync(1, 256);
                if (tid == 0) wg_stop[1] = *abort_flag;
                named_bar_sync(1, 256);
                if (wg_stop[1] != 0u) break;
            }
        }
        if (MODE == MODE_NAG && sizeof(OutT) == 2) {                      // the last parked item; the loader stores it
            const bool last = pend_valid;
            nag_finish(false);
            nag_finish(true);
            if (tid == 0 && last) mbar_arrive(bar(BAR_QEMPTY + 0));
        }
        if (lane == 0) tma_store_wait_all();                              // bulk stores issued by this thread have landed
        tc_fence_before();
        cta_sync();
    } else {
        setmaxnreg_dec<OTHER_REGS>();
        if (warp == 8 || warp == 10) {
            // ------------------------------------------------------------------ MMA issue: one warp (one lane) per stream
            // Two issuing threads, because one thread's waits, fences and commits between two batches of eight MMAs take
            // longer than the tensor core's instruction queue lasts: with a single issuer the pipe drained between batches
            // and paid its start-up latency every time (measured: ~850 cycles per batch against 520 back to back).
            // Now one thread's bookkeeping runs under the other's MMAs.
            const int i = (warp - 8) >> 1;
            if (lane == 0) {
                // Operands are fp16 throughout (bf16/fp32 inputs are staged as fp16 by the pre-pass): with bf16
                // P the 2^-9 rounding of each weight alone costs ~1e-3 relative error on outputs that are sums
                // of random-sign terms, and tcgen05 does not take an fp16 A with a bf16 B.
                constexpr uint32_t IDESC_S = idesc_f16(0, 0, 0, 0, BM, BN);   // S = Q K^T, both K-major
                constexpr uint32_t IDESC_PV = idesc_f16(0, 0, 0, 1, BM, HD);  // O += P V, V is MN-major (rows = keys)
                // descriptor words: the high word is common to every tile here (stride between 8-row groups 1024 bytes, 128-byte
                // swizzle), the low word is the tile's base plus a constant per k step
                constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
                const uint32_t q_lo = smem_desc_lo(sQ + (MODE == MODE_NAG ? 0 : i) * TILE_BYTES, 16);
                const uint32_t tO = tmem_base + 256u + (uint32_t)(i * 128), tP = tmem_base + 128u + (uint32_t)(i * 64);
                uint32_t ring = 0;                                            // ring slot index, counted exactly as the loader counts
                uint32_t n_s = 0;                                             // S products issued so far by BOTH warps (they share the staging area in turn)
                uint32_t qf_cnt = 0, pf_cnt = 0, of_cnt = 0, sr_cnt = 0;
                bool good = true;
                auto kv_wait = [&](uint32_t idx) { return mbar_wait(bar(BAR_KVFULL + idx % NSTAGE), (idx / NSTAGE) & 1u, abort_flag); };
                auto kv_addr = [&](uint32_t idx) { return sKV + (idx % NSTAGE) * TILE_BYTES; };
                auto q_wait = [&]() { const bool r = mbar_wait(bar(BAR_QFULL + (MODE == MODE_NAG ? 0 : i)), qf_cnt & 1u, abort_flag); ++qf_cnt; return r; };
                auto p_wait = [&]() { const bool r = mbar_wait(bar(BAR_PFULL + i), pf_cnt & 1u, abort_flag); ++pf_cnt; tc_fence_after(); return r; };
                auto sreq_wait = [&]() { const bool r = mbar_wait(bar(BAR_SREQ + i), sr_cnt & 1u, abort_flag); ++sr_cnt; return r; };
                // O_i (in NAG mode both O) of the previous segment has been read out; passes at once for the first one
                auto o_free_wait = [&]() { const bool r = mbar_wait(bar(BAR_OFREE + i), (of_cnt & 1u) ^ 1u, abort_flag); ++of_cnt; tc_fence_after(); return r; };
                // S = Q_i K^T into the shared staging area as its g-th user, once user g-1 has read its scores out (at once for g = 0)
                auto issue_S = [&](uint32_t g, uint32_t k_saddr) {
                    if (!mbar_wait(bar(BAR_SFREE), (g & 1u) ^ 1u, abort_flag)) return false;
                    tc_fence_after();
                    const uint32_t blo = smem_desc_lo(k_saddr, 16);
                    mma_ss_w<0>(tmem_base, q_lo, blo, DESC_HI, IDESC_S);
#pragma unroll
                    for (int kk = 1; kk < 8; kk++) {
                        const uint32_t off = ((uint32_t)(kk >> 2) * HALF_BYTES + (uint32_t)(kk & 3) * 32u) >> 4;
                        mma_ss_w<1>(tmem_base, q_lo + off, blo + off, DESC_HI, IDESC_S);
                    }
                    tc_commit(bar(BAR_SFULL + i));
                    return true;
                };
                // O_i (+)= P_i V; P_i may be overwritten and O_i rescaled once these MMAs are done
                auto issue_PV = [&](uint32_t v_saddr, int j, int Tk, bool first) {
                    const int valid = min(BN, Tk - j * BN);
                    const int nkk = (valid + 15) >> 4;                        // 16 keys per MMA; P is 0 past `valid`
                    const uint32_t blo = smem_desc_lo(v_saddr, HALF_BYTES);
                    if (first) mma_ts_w<0>(tO, tP, blo, DESC_HI, IDESC_PV);
                    else mma_ts_w<1>(tO, tP, blo, DESC_HI, IDESC_PV);
#pragma unroll
                    for (int kk = 1; kk < 8; kk++)
                        if (kk < nkk) mma_ts_w<1>(tO, tP + (uint32_t)(kk * 8), blo + (uint32_t)(kk * 128), DESC_HI, IDESC_PV);
                    tc_commit(bar(BAR_PEMPTY + i));
                };
                SegIter<MODE> iter(p);
                Seg it;
                while (good && iter.next(it)) {
                    if (MODE == MODE_PAIR) {
                        // ring order (loader): K(jb), then per block V(j), K(j+1). A K/V tile serves both streams; its slot is handed
                        // back by the softmax threads once they have seen the MMAs on it complete.
                        const int jb = it.jb, je = it.je[0];
                        const bool two = it.je[1] > jb;
                        const bool mine = i == 0 || two;
                        const uint32_t per_blk = two ? 2u : 1u;               // S products per key block, in the order stream 0, stream 1
                        if (mine) {
                            good = q_wait() && kv_wait(ring) && issue_S(n_s + (uint32_t)i, kv_addr(ring));
                            if (!good) break;
                        }
                        ++ring;
                        for (int j = jb; j < je && good; ++j) {
                            const uint32_t nv = ring, nk = ring + 1;          // V(j), K(j+1)
                            const bool more = j + 1 < je;
                            if (mine) {
                                if (more) {
                                    good = sreq_wait() && kv_wait(nk) && issue_S(n_s + per_blk * (uint32_t)(j + 1 - jb) + (uint32_t)i, kv_addr(nk));
                                    if (!good) break;
                                }
                                good = kv_wait(nv) && (j > jb || o_free_wait()) && p_wait();
                                if (!good) break;
                                issue_PV(kv_addr(nv), j, p.Tk[0], j == jb);
                                if (!more) tc_commit(bar(BAR_ODONE + i));
                            }
                            ring += more ? 2u : 1u;
                        }
                        n_s += per_blk * (uint32_t)(je - jb);
                    } else {
                        // ring order (loader): K0(0), K1(0), then per block j and stream: V_i(j), K_i(j+1). Every tile belongs to
                        // one stream. Staging-area order: S0(0), S1(0), then S_i(j+1) in the same (j, i) order.
                        good = q_wait();
                        uint32_t g = n_s;
                        for (int ii = 0; ii < 2 && good; ii++) {
                            if (it.je[ii] <= 0) continue;
                            if (ii == i) {
                                good = kv_wait(ring) && issue_S(g, kv_addr(ring));
                            }
                            ++ring;
                            ++g;
                        }
                        const int nmax = max(it.je[0], it.je[1]);
                        for (int j = 0; j < nmax && good; ++j) {
                            for (int ii = 0; ii < 2 && good; ii++) {
                                if (j >= it.je[ii]) continue;
                                const bool more = j + 1 < it.je[ii];
                                if (ii == i) {
                                    if (more) {                               // ring: V_i(j), then K_i(j+1)
                                        good = sreq_wait() && kv_wait(ring + 1) && issue_S(g, kv_addr(ring + 1));
                                        if (!good) break;
                                    }
                                    good = kv_wait(ring) && (j > 0 || o_free_wait()) && p_wait();
                                    if (!good) break;
                                    issue_PV(kv_addr(ring), j, p.Tk[i], j == 0);
                                    if (!more) tc_commit(bar(BAR_ODONE + i));
                                }
                                ring += more ? 2u : 1u;
                                if (more) ++g;
                            }
                        }
                        n_s = g;
                    }
                }
            }
            __syncwarp();
        } else if (warp == 9) {
            // ------------------------------------------------------------------ TMA loads (one lane)
            if (lane == 0) {
                uint32_t n = 0;
                uint32_t qe_cnt[2] = {0, 0};
                uint32_t q_loads[2] = {0, 0};                             // Q tiles requested so far, per stream
                bool good = true;
                Seg it = {};
                // one 128x128 tile = two 64-column boxes, each landing as a 128-byte-swizzled [128][64] half
                auto load_tile = [&](uint32_t dst, const CUtensorMap* tm, uint32_t mbar, int row0, int bb) {
                    tma_load_3d(dst, tm, mbar, it.h * HD, row0, bb);
                    tma_load_3d(dst + HALF_BYTES, tm, mbar, it.h * HD + 64, row0, bb);
                };
                // MODE_NAG, 16-bit output: the softmax threads leave the blended tile of the item before in the Q tile; store it
                auto store_staged = [&]() {
                    if (MODE == MODE_NAG && sizeof(OutT) == 2 && sm_store[0]) {
                        tma_store_3d(&tmO, sQ, (int)sm_store[1] * HD, (int)sm_store[2], 0);
                        tma_store_3d(&tmO, sQ + HALF_BYTES, (int)sm_store[1] * HD + 64, (int)sm_store[2], 0);
                        tma_store_commit();
                        tma_store_wait_read();                                // the tile has been read: Q may land on it
                    }
                };
                auto load_q = [&](int i) {
                    // the previous segment's S MMAs (and its output staging in the same space) are done with this tile
                    good = mbar_wait(bar(BAR_QEMPTY + i), (qe_cnt[i] & 1u) ^ 1u, abort_flag);
                    ++qe_cnt[i];
                    if (!good) return;
                    store_staged();
                    mbar_expect_tx(bar(BAR_QFULL + i), TILE_BYTES);
                    load_tile(sQ + i * TILE_BYTES, &tmQ, bar(BAR_QFULL + i), it.q0 + i * BM, it.b);
                    ++q_loads[i];
                };
                auto load_kv = [&](const CUtensorMap* tm, int row0) {
                    const uint32_t st = n % NSTAGE;
                    good = mbar_wait(bar(BAR_KVEMPTY + st), ((n / NSTAGE) & 1u) ^ 1u, abort_flag);
                    if (!good) return;
                    mbar_expect_tx(bar(BAR_KVFULL + st), TILE_BYTES);
                    load_tile(sKV + st * TILE_BYTES, tm, bar(BAR_KVFULL + st), row0, MODE == MODE_NAG ? 0 : it.b);
                    ++n;
                };
                SegIter<MODE> iter(p);
                bool any = false;
                while (good && iter.next(it)) {
                    any = true;
                    if (MODE == MODE_NAG) {
                        // the first K tiles do not depend on the Q tile, which the previous item's output may still occupy
                        if (it.je[0] > 0) load_kv(&tmK0, 0);
                        if (good && it.je[1] > 0) load_kv(&tmK1, 0);
                        if (!good) break;
                    }
                    load_q(0);
                    if (!good) break;
                    if (MODE == MODE_PAIR) {
                        const int jb = it.jb, je = it.je[0];
                        load_kv(&tmK0, jb * BN);
                        if (good && it.je[1] > jb) load_q(1);
                        for (int j = jb; j < je && good; ++j) {
                            load_kv(&tmV0, j * BN);
                            if (good && j + 1 < je) load_kv(&tmK0, (j + 1) * BN);
                        }
                    } else {
                        const int nmax = max(it.je[0], it.je[1]);
                        for (int j = 0; j < nmax && good; ++j) {
                            for (int i = 0; i < 2 && good; i++) {
                                if (j >= it.je[i]) continue;
                                load_kv(i ? &tmV1 : &tmV0, j * BN);
                                if (good && j + 1 < it.je[i]) load_kv(i ? &tmK1 : &tmK0, (j + 1) * BN);
                            }
                        }
                    }
                }
                if (MODE == MODE_NAG && sizeof(OutT) == 2 && good && any) {
                    // two hand-overs are still to come: the last epilogue's (it staged the item before the last) and the final
                    // one after the loop (the last item)
                    for (int k = 0; k < 2 && good; k++) {
                        good = mbar_wait(bar(BAR_QEMPTY + 0), (qe_cnt[0] & 1u) ^ 1u, abort_flag);
                        ++qe_cnt[0];
                        if (good) store_staged();
                    }
                    tma_store_wait_all();
                }
                // on failure, let the copies already requested land before the CTA's shared memory goes away: a bounded wait on
                // the FULL barrier of every ring slot and Q tile that still has a request outstanding
                if (!good || *abort_flag) {
                    for (uint32_t k = n > (uint32_t)NSTAGE ? n - NSTAGE : 0u; k < n; ++k) drain_wait(bar(BAR_KVFULL + k % NSTAGE), (k / NSTAGE) & 1u);
                    for (int i = 0; i < 2; i++)
                        if (q_loads[i]) drain_wait(bar(BAR_QFULL + i), (q_loads[i] - 1u) & 1u);
                }
            }
            __syncwarp();
        }
        if (warp == 11 && MODE == MODE_NAG && sizeof(OutT) == 2) {
            // ------------------------------------------------------------------ norm fetcher (MODE_NAG, 16-bit output)
            // For every item the softmax threads park: wait (bounded) until all heads of its query tile have published their
            // norms, sum them per row in a fixed order (same bits in every thread block) and leave the totals in shared memory,
            // all under the main loop of the next item.
            float* const f_tot = fbuf + 256;
            SegIter<MODE> iter(p);
            Seg it;
            uint32_t n = 0;
            bool good = true;
            while (good && iter.next(it)) {
                good = __all_sync(0xffffffffu, mbar_wait(bar(BAR_PARKED), n & 1u, abort_flag));
                ++n;
                if (!good) break;
                const int qt = (int)sm_item[0];
                uint32_t here = 0;
                if (lane == 0) {
                    // this thread block's norms of the item are stored (ordered before the arrival just acquired): make them
                    // visible and count this head in, then wait for the other heads
                    if (p.n_peers == 0) {
                        asm volatile("fence.acq_rel.gpu;" ::: "memory");
                        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.nag_flag + qt), "r"(1u) : "memory");
                    } else {
                        asm volatile("fence.acq_rel.sys;" ::: "memory");
                        for (int pe = 0; pe < p.n_peers; pe++)
                            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.nag_flag_peers[pe] + qt), "r"(1u) : "memory");
                    }
                    const uint32_t target = p.nag_epoch * (uint32_t)p.nag_heads;
                    const uint64_t t0 = globaltimer_ns();
                    uint32_t seen = 0;
                    for (;;) {
                        if (p.n_peers == 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.nag_flag + qt) : "memory");
                        else asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.nag_flag + qt) : "memory");
                        if (seen >= target || *abort_flag) break;
                        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { *abort_flag = 1u; break; }
                        __nanosleep(64);
                    }
                    here = seen >= target ? 1u : 0u;
                }
                here = __shfl_sync(0xffffffffu, here, 0);
                // rows 4 lane .. 4 lane + 3: 16-byte loads, four (head, half) entries in flight at a time
                const float4* src = reinterpret_cast<const float4*>(p.nag_part + ((size_t)qt * p.nag_heads) * 512) + lane;
                float4 tp = make_float4(0.f, 0.f, 0.f, 0.f), tg = tp;
                if (here) {
                    const int n_e = 2 * p.nag_heads;                          // head and half order: same sum everywhere
                    for (int h0 = 0; h0 < n_e; h0 += 4) {
                        float4 a[4], b[4];
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            if (h0 + u < n_e) { a[u] = __ldcg(src + (size_t)(h0 + u) * 64); b[u] = __ldcg(src + (size_t)(h0 + u) * 64 + 32); }
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            if (h0 + u < n_e) {
                                tp.x += a[u].x; tp.y += a[u].y; tp.z += a[u].z; tp.w += a[u].w;
                                tg.x += b[u].x; tg.y += b[u].y; tg.z += b[u].z; tg.w += b[u].w;
                            }
                    }
                }
                reinterpret_cast<float4*>(f_tot)[lane] = tp;
                reinterpret_cast<float4*>(f_tot + 128)[lane] = tg;
                if (lane == 0) wg_here[1] = here;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_NORMS));
            }
        }
        cta_sync();
        if (warp == 8) {
            if (lane == 0 && *abort_flag) atomicOr(p.status, ST_TIMEOUT);
            tc_fence_after();
            tmem_dealloc(tmem_base, 512);
        }
    }
}

}  // namespace kb
