// C ABI of the sm_100a attention path (declarations and contracts: include/kiln_b200.h).
// Host side only: argument validation, TMA tensor-map construction, kernel selection by dtype, launches.
// There is no CPU fallback and no second backend: on anything but an sm_100 device the entry points fail.
#include <cuda.h>
#include <cuda_runtime.h>

#include <string.h>

#include <mutex>

#include "../../include/kiln_b200.h"
#include "attn_sm100.cuh"
#include "prep.cuh"
#include "combine.cuh"
#include "selfcheck.cuh"
#include "gemm_sm100.cuh"
#include "attn_bwd_sm100.cuh"

namespace {

using namespace kb;

// One word per device that kernels OR error bits into (ST_*). File-scope device memory: no allocation.
__device__ unsigned int g_status_word;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Optional per-category kernel timing, the counterpart of the reference's ProfScope / prof_report
// (engine/src/kernels.cu:18-58): an event pair around every launch while enabled, summed on read.
constexpr int PROF_POOL = 8192;
struct Prof {
    bool on = false;
    int used = 0;
    cudaEvent_t* ev = nullptr;      // 2 * PROF_POOL events, created when profiling is first enabled
    unsigned char* cat = nullptr;   // category of each pair
};

struct DeviceState {
    bool ready = false;
    int err = KB_OK;
    unsigned int* status = nullptr;
    int sm_count = 148;
    Prof prof;
};

struct ProfScope {
    Prof* p = nullptr;
    int slot = -1;
    cudaStream_t stream;
    ProfScope(DeviceState* st, int category, cudaStream_t s) : stream(s) {
        if (st && st->prof.on && st->prof.used < PROF_POOL) {
            p = &st->prof;
            slot = p->used++;
            p->cat[slot] = (unsigned char)category;
            cudaEventRecord(p->ev[2 * slot], stream);
        }
    }
    ~ProfScope() { if (p) cudaEventRecord(p->ev[2 * slot + 1], stream); }
};

constexpr int MAX_DEVICES = 64;
DeviceState g_dev[MAX_DEVICES];
EncodeTiledFn g_encode = nullptr;
std::mutex g_mu;

template <typename K>
int set_smem(K kernel, int bytes) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return KB_ERR_CUDA;
    return KB_OK;
}

template <int EPI>
int set_gemm_smem() {
    if (cudaFuncSetAttribute(gemm16_kernel<EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm16_kernel<EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM) != cudaSuccess)
        return KB_ERR_CUDA;
    return KB_OK;
}

int init_device(DeviceState& st, int dev) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return KB_ERR_DEVICE;
    if (prop.major != 10) return KB_ERR_DEVICE;  // tcgen05 / TMEM exist on sm_100 only
    st.sm_count = prop.multiProcessorCount;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || !fn)
            return KB_ERR_CUDA;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    int rc;
    if ((rc = set_smem(attn_bwd_kernel, BWD_SMEM))) return rc;
    if ((rc = set_smem(attn_fwd_kernel<MODE_PAIR, __half>, ATTN_SMEM_PAIR))) return rc;
    if ((rc = set_smem(attn_fwd_kernel<MODE_PAIR, __nv_bfloat16>, ATTN_SMEM_PAIR))) return rc;
    if ((rc = set_smem(attn_fwd_kernel<MODE_PAIR, float>, ATTN_SMEM_PAIR))) return rc;
    if ((rc = set_smem(attn_fwd_kernel<MODE_NAG, __half>, ATTN_SMEM_NAG))) return rc;
    if ((rc = set_smem(attn_fwd_kernel<MODE_NAG, __nv_bfloat16>, ATTN_SMEM_NAG))) return rc;
    if ((rc = set_smem(attn_fwd_kernel<MODE_NAG, float>, ATTN_SMEM_NAG))) return rc;
    if ((rc = set_gemm_smem<EPI_F32>()) || (rc = set_gemm_smem<EPI_F16>()) || (rc = set_gemm_smem<EPI_GELU16>()) ||
        (rc = set_gemm_smem<EPI_RESID>()) || (rc = set_gemm_smem<EPI_HEADS16>()))
        return rc;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return KB_ERR_CUDA;
    st.status = static_cast<unsigned int*>(p);
    if (cudaMemset(st.status, 0, sizeof(unsigned int)) != cudaSuccess) return KB_ERR_CUDA;
    return KB_OK;
}

// state of the current device, initialised on first use
int get_state(DeviceState** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return KB_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        st.err = init_device(st, dev);
        st.ready = true;
        if (st.err != KB_OK) cudaGetLastError();
    }
    *out = &st;
    return st.err;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

// [batches][rows][H*128] view of a row-major fp16 matrix with row stride ld; box = 64 columns x 128 rows
int make_tmap(CUtensorMap* tm, const void* ptr, int rows, int H, int batches, int ld) {
    const cuuint64_t dims[3] = {(cuuint64_t)H * 128, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)rows * (cuuint64_t)ld * 2};
    const cuuint32_t box[3] = {64, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                          const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KB_OK : KB_ERR_CUDA;
}

int check_mat(const void* p, int ld, int H, int dtype) {
    if (!p) return KB_ERR_ARG;
    if (!aligned16(p) || (ld & (dtype == KB_F32 ? 3 : 7))) return KB_ERR_ALIGN;
    if (ld < H * 128) return KB_ERR_SHAPE;
    return KB_OK;
}

int check_out(const void* p, int ld, int H, int out_dtype) {
    if (!p) return KB_ERR_ARG;
    if (out_dtype != KB_F16 && out_dtype != KB_BF16 && out_dtype != KB_F32) return KB_ERR_ARG;
    if (!aligned16(p) || (ld & (out_dtype == KB_F32 ? 3 : 7))) return KB_ERR_ALIGN;
    if (ld < H * 128) return KB_ERR_SHAPE;
    return KB_OK;
}

// Collects the tensors one launch of the pre-pass stages.
struct PrepBatch {
    PrepParams pp = {};
    // words the pre-pass clears on the way (arrival counters / flags the attention kernel expects at zero)
    void zero(unsigned int* ptr, int n) { pp.zero_ptr = ptr; pp.zero_n = n; }
    void add(void* out, int ld_out, const void* in, int ld_in, int rows, int T, const void* w, const float* c, const float* s) {
        PrepSeg& sg = pp.seg[pp.nseg++];
        sg.in = in; sg.out = out; sg.w = static_cast<const __nv_bfloat16*>(w); sg.cos_t = c; sg.sin_t = s;
        sg.rows = rows; sg.ld_in = ld_in; sg.ld_out = ld_out; sg.T = T > 0 ? T : 1;
        sg.block0 = pp.blocks;
        const int per_block = c ? PREP_ITEMS_PER_BLOCK_ROPE : PREP_ITEMS_PER_BLOCK;
        pp.blocks += (unsigned)(((long long)rows * pp.H + per_block - 1) / per_block);
    }
};

int launch_prep(DeviceState* st, const PrepBatch& pb, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (pb.pp.blocks == 0) {
        // nothing to stage: the words still have to be cleared before the attention kernel starts
        if (pb.pp.zero_n > 0 && cudaMemsetAsync(pb.pp.zero_ptr, 0, (size_t)pb.pp.zero_n * sizeof(unsigned int), stream) != cudaSuccess) return KB_ERR_CUDA;
        return KB_OK;
    }
    ProfScope ps(st, KB_PROF_NORM_ROPE, stream);
    const unsigned grid = pb.pp.blocks;
#define KB_PREP(IN, OUT) qk_prep_kernel<IN, OUT><<<grid, 256, 0, stream>>>(pb.pp)
    if (out_dtype == KB_F32) {
        KB_PREP(float, float);        // in-place fp32 norm / RoPE as the engine's own ops do (validated by the caller)
    } else if (out_dtype == KB_F16) {
        if (in_dtype == KB_F16) KB_PREP(__half, __half);
        else if (in_dtype == KB_BF16) KB_PREP(__nv_bfloat16, __half);
        else KB_PREP(float, __half);
    } else {
        if (in_dtype == KB_F16) KB_PREP(__half, __nv_bfloat16);
        else if (in_dtype == KB_BF16) KB_PREP(__nv_bfloat16, __nv_bfloat16);
        else KB_PREP(float, __nv_bfloat16);
    }
#undef KB_PREP
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

template <int MODE, typename OutT>
int launch_attn_t(const CUtensorMap& tq, const CUtensorMap& tk0, const CUtensorMap& tv0, const CUtensorMap& tk1,
                  const CUtensorMap& tv1, const CUtensorMap& to, const AttnParams& p, int sm_count, cudaStream_t stream) {
    // persistent kernel: one CTA per SM (its shared memory and TMEM fill an SM) walks the work items
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(ATTN_THREADS, 1, 1);
    cfg.gridDim = dim3((unsigned)((p.split || p.n_items >= sm_count) ? sm_count : p.n_items), 1, 1);
    cfg.dynamicSmemBytes = MODE == MODE_NAG ? ATTN_SMEM_NAG : ATTN_SMEM_PAIR;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = 0;
    if (MODE == MODE_NAG || p.split) {
        // the CTAs holding the heads of one query tile (NAG) or the parts of a cut item (split) wait for each other:
        // all CTAs must be resident at once
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, attn_fwd_kernel<MODE, OutT>, tq, tk0, tv0, tk1, tv1, to, p);
    return e == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

template <int MODE>
int launch_attn(int out_dtype, const CUtensorMap& tq, const CUtensorMap& tk0, const CUtensorMap& tv0, const CUtensorMap& tk1,
                const CUtensorMap& tv1, const AttnParams& p, int sm_count, cudaStream_t stream) {
    // 16-bit outputs of single-GPU calls leave through TMA stores: [B][Tq][H*128] view of `out`, box = 64 columns x 128 rows
    CUtensorMap to;
    memset(&to, 0, sizeof(to));
    if (out_dtype != KB_F32 && p.n_peers == 0) {
        const cuuint64_t dims[3] = {(cuuint64_t)p.H * 128, (cuuint64_t)p.Tq, (cuuint64_t)p.B};
        const cuuint64_t strides[2] = {(cuuint64_t)p.ldo * 2, (cuuint64_t)p.Tq * (cuuint64_t)p.ldo * 2};
        const cuuint32_t box[3] = {64, 128, 1};
        const cuuint32_t estr[3] = {1, 1, 1};
        if (g_encode(&to, out_dtype == KB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, p.out, dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return KB_ERR_CUDA;
    }
    if (out_dtype == KB_F32) return launch_attn_t<MODE, float>(tq, tk0, tv0, tk1, tv1, to, p, sm_count, stream);
    if (out_dtype == KB_BF16) return launch_attn_t<MODE, __nv_bfloat16>(tq, tk0, tv0, tk1, tv1, to, p, sm_count, stream);
    return launch_attn_t<MODE, __half>(tq, tk0, tv0, tk1, tv1, to, p, sm_count, stream);
}

constexpr float SCALE_LOG2 = 1.4426950408889634f * 0.08838834764831845f;  // log2(e) / sqrt(128)

inline bool valid_in_dtype(int d) { return d == KB_F16 || d == KB_BF16 || d == KB_F32; }

// A tensor is staged (copied as fp16 into the workspace) when it is not fp16 already or needs norm/RoPE.
struct Stage {
    char* ws;
    size_t left;
    bool overflow = false;
    void* take(size_t rows, int H) { return take_bytes(rows * (size_t)H * 128 * 2); }
    void* take_bytes(size_t bytes) {
        const size_t n = align256(bytes);
        if (!ws || n > left) { overflow = true; return nullptr; }
        void* p = ws;
        ws += n; left -= n;
        return p;
    }
};

// where a head-split run stores its output: every GPU's [B*Tq, ld_o] buffer (own included) and arrival counter
struct PeerSpec {
    void* const* out_peers;
    unsigned long long* const* ctr_peers;
    int n_peers, col0;
};

#ifndef KB_SPLIT_MARGIN
#define KB_SPLIT_MARGIN 7
#endif
constexpr int MAX_HEADS = 4096;   // keeps every byte count below in range
constexpr size_t NAG_NORM_FLOATS = 512;   // per (query tile, head): [2 column halves][|Z+|_1, |g|_1][128 rows]

// fp16 staging bytes of one attention call (the part of the workspace the pre-pass writes)
size_t staging_bytes(size_t rows_q, size_t rows_k, int n_ctx, int H, int dtype, bool norm_q, bool norm_k) {
    const bool conv = dtype != KB_F16;
    size_t n = 0;
    if (conv || norm_q) n += align256(rows_q * H * 128 * 2);
    if (conv || norm_k) n += (size_t)n_ctx * align256(rows_k * H * 128 * 2);   // K of every context
    if (conv) n += (size_t)n_ctx * align256(rows_k * H * 128 * 2);             // V of every context
    return n;
}

// Balanced (item, key block) ranges per SM against whole items per SM, in key-block steps on the slowest SM. Measured on B200
// (4096 / 3456 / 2560 / 2048 / 1536 / 1024 tokens x 16 heads, device time inside a CUDA graph): a key-block step costs ~1.86 us
// and the balanced schedule a fixed ~15 us on top (one more segment to fill and drain per SM, the partial results written and
// merged; the cooperative launch itself measured free): it wins at 2560 and 3456 tokens (63.8 vs 83.5 us, 97.6 vs 111.7 us), ties
// or wins at 4096 (128.2 vs 127.4 us on one GPU, 126.9 vs 140.0 us on another), ties at 2048 and loses at 1536 and 1024 (36.8 vs
// 29.3 us, 28.7 vs 21.3 us). So it is taken when it saves at least eight steps.
bool split_pays(int n_items, int nb, int sm_count) {
    const long long steps = (long long)n_items * nb;
    if (nb < 2 || steps < 2LL * sm_count) return false;
    const long long whole = (long long)((n_items + sm_count - 1) / sm_count) * nb;
    const long long balanced = (steps + sm_count - 1) / sm_count + KB_SPLIT_MARGIN;
    return balanced < whole;
}

// shared body of self- and cross-attention: q [B*Tq], k/v [B*Tk]
int attn_pair(void* out, const void* q, const void* k, const void* v, const void* qn_w, const void* kn_w,
              const float* rope_cos, const float* rope_sin, int B, int Tq, int Tk, int npad, int H, int ld_q, int ld_k,
              int ld_v, int ld_o, int dtype, int out_dtype, float eps, void* workspace, size_t workspace_bytes,
              cudaStream_t stream, const PeerSpec* peers = nullptr, float* stats = nullptr) {
    if (!valid_in_dtype(dtype)) return KB_ERR_ARG;
    if (B <= 0 || Tq <= 0 || Tk <= 0 || H <= 0 || npad < 0) return KB_ERR_ARG;
    if (peers) {
        if (peers->n_peers < 1 || peers->n_peers > MAX_PEERS || peers->col0 < 0 || (peers->col0 & 7) || out_dtype == KB_F32) return KB_ERR_ARG;
        if (ld_o < peers->col0 + H * 128) return KB_ERR_SHAPE;
        for (int i = 0; i < peers->n_peers; i++) {
            if (!peers->out_peers[i] || !peers->ctr_peers[i]) return KB_ERR_ARG;
            if (!aligned16(peers->out_peers[i])) return KB_ERR_ALIGN;
        }
        out = peers->out_peers[0];
    }
    if ((rope_cos == nullptr) != (rope_sin == nullptr)) return KB_ERR_ARG;
    if (H > MAX_HEADS) return KB_ERR_SHAPE;
    // the pre-pass reads norm weights and RoPE tables with 16-byte vector loads
    if (!aligned16(qn_w) || !aligned16(kn_w) || !aligned16(rope_cos) || !aligned16(rope_sin)) return KB_ERR_ALIGN;
    int rc;
    if ((rc = check_mat(q, ld_q, H, dtype)) || (rc = check_mat(k, ld_k, H, dtype)) || (rc = check_mat(v, ld_v, H, dtype)) ||
        (rc = check_out(out, ld_o, H, out_dtype)))
        return rc;
    DeviceState* st;
    if ((rc = get_state(&st))) return rc;

    const bool conv = dtype != KB_F16;
    const bool stage_q = conv || qn_w || rope_cos, stage_k = conv || kn_w || rope_cos, stage_v = conv;
    if ((stage_q || stage_k || stage_v) && (!workspace || !aligned16(workspace))) return KB_ERR_WORKSPACE;
    Stage sg{static_cast<char*>(workspace), workspace_bytes};
    PrepBatch pb;
    pb.pp.H = H; pb.pp.eps = eps;
    const void *qq = q, *kk = k, *vv = v;
    int ldq = ld_q, ldk = ld_k, ldv = ld_v;
    if (stage_q) { void* d = sg.take((size_t)B * Tq, H); if (d) pb.add(d, H * 128, q, ld_q, B * Tq, Tq, qn_w, rope_cos, rope_sin); qq = d; ldq = H * 128; }
    if (stage_k) { void* d = sg.take((size_t)B * Tk, H); if (d) pb.add(d, H * 128, k, ld_k, B * Tk, Tk, kn_w, rope_cos, rope_sin); kk = d; ldk = H * 128; }
    if (stage_v) { void* d = sg.take((size_t)B * Tk, H); if (d) pb.add(d, H * 128, v, ld_v, B * Tk, Tk, nullptr, nullptr, nullptr); vv = d; ldv = H * 128; }
    if (sg.overflow) return KB_ERR_WORKSPACE;
    AttnParams p = {};
    p.out = out; p.ldo = ld_o; p.Tq = Tq; p.H = H; p.B = B;
    p.Tk[0] = Tk; p.Tk[1] = 0; p.npad[0] = npad; p.npad[1] = 0;
    p.n_items = ((Tq + 2 * BM - 1) / (2 * BM)) * H * B;
    p.scale_log2 = SCALE_LOG2;
    p.status = st->status;
    p.stats = stats;
    // Balanced schedule: worth it when equal (item, key block) ranges per SM beat whole items per SM by more than the
    // cost of writing and merging the cut items' partial results (about two key blocks), and the workspace has room for
    // those partial results; otherwise every CTA takes whole items.
    if (split_pays(p.n_items, (Tk + BN - 1) / BN, st->sm_count) && workspace && aligned16(workspace)) {
        Stage trial = sg;
        float* part = static_cast<float*>(trial.take_bytes((size_t)st->sm_count * PART_CTA_BYTES));
        unsigned int* flags = static_cast<unsigned int*>(trial.take_bytes((size_t)st->sm_count * 2 * sizeof(unsigned int)));   // one per SM and stream
        if (!trial.overflow) {
            sg = trial;
            p.split = 1; p.part = part; p.part_flag = flags;
            pb.zero(flags, st->sm_count * 2);
        }
    }
    if ((rc = launch_prep(st, pb, dtype, KB_F16, stream))) return rc;
    CUtensorMap tq, tk, tv;
    if ((rc = make_tmap(&tq, qq, Tq, H, B, ldq)) || (rc = make_tmap(&tk, kk, Tk, H, B, ldk)) || (rc = make_tmap(&tv, vv, Tk, H, B, ldv)))
        return rc;
    if (peers) {
        p.n_peers = peers->n_peers;
        p.col0 = peers->col0;
        for (int i = 0; i < peers->n_peers; i++) { p.out_peers[i] = peers->out_peers[i]; p.ctr_peers[i] = peers->ctr_peers[i]; }
    }
    ProfScope ps(st, KB_PROF_ATTENTION, stream);
    return launch_attn<MODE_PAIR>(out_dtype, tq, tk, tv, tk, tv, p, st->sm_count, stream);
}

}  // namespace

extern "C" {

const char* kb_error_string(int code) {
    switch (code) {
        case KB_OK: return "ok";
        case KB_ERR_ARG: return "bad argument (null pointer, non-positive size or unknown dtype)";
        case KB_ERR_ALIGN: return "pointer not 16-byte aligned or row stride not a multiple of 8 elements";
        case KB_ERR_SHAPE: return "unsupported shape";
        case KB_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case KB_ERR_CUDA: return "CUDA call failed";
        case KB_ERR_DEVICE: return "no sm_100 device is current";
        case KB_ERR_TIMEOUT: return "a kernel gave up on a bounded wait";
        case KB_ERR_SELFCHECK: return "start-up self-check exceeded its tolerance";
        case KB_ERR_STATIC_SCRATCH: return "problem needs more staging scratch than the library's built-in buffer (KB_STATIC_SCRATCH_BYTES); use kb_attn_self with a workspace";
        default: return "unknown error";
    }
}

int kb_version(void) { return 110; }



int kb_init(void) {
    DeviceState* st;
    return get_state(&st);
}

size_t kb_attn_workspace_bytes(int rows_q, int rows_k, int n_ctx, int H, int dtype, int norm_q, int norm_k) {
    if (rows_q < 0 || rows_k < 0 || H <= 0 || H > MAX_HEADS || n_ctx < 1) return 0;
    size_t n = staging_bytes((size_t)rows_q, (size_t)rows_k, n_ctx, H, dtype, norm_q != 0, norm_k != 0);
    if (n_ctx == 2) {                                                                  // NAG: per-head norm partials and arrival counters
        const size_t n_qt = ((size_t)rows_q + 127) / 128;
        n += align256(n_qt * H * NAG_NORM_FLOATS * sizeof(float)) + align256(n_qt * sizeof(unsigned int));
    } else {
        // room for the balanced schedule's partial results (one slot and one flag per SM); a smaller workspace still works,
        // the call then runs whole items per SM
        int sms = 148;
        DeviceState* st;
        if (get_state(&st) == KB_OK) sms = st->sm_count;
        n += align256((size_t)sms * PART_CTA_BYTES) + align256((size_t)sms * 2 * sizeof(unsigned int));
    }
    return n;
}

int kb_attn_self(void* out, const void* q, const void* k, const void* v, const void* qn_w, const void* kn_w,
                 const float* rope_cos, const float* rope_sin, int B, int T, int H, int ld_q, int ld_k, int ld_v, int ld_o,
                 int dtype, int out_dtype, float eps, void* workspace, size_t workspace_bytes, void* stream) {
    return attn_pair(out, q, k, v, qn_w, kn_w, rope_cos, rope_sin, B, T, T, 0, H, ld_q, ld_k, ld_v, ld_o, dtype, out_dtype, eps,
                     workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int kb_attn_cross(void* out, const void* q, const void* qn_w, const void* k, const void* v, int Tq, int Tk, int npad, int H,
                  int ld_q, int ld_k, int ld_v, int ld_o, int dtype, int out_dtype, float eps, void* workspace,
                  size_t workspace_bytes, void* stream) {
    return attn_pair(out, q, k, v, qn_w, nullptr, nullptr, nullptr, 1, Tq, Tk, npad, H, ld_q, ld_k, ld_v, ld_o, dtype, out_dtype,
                     eps, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

// Head split of the NAG kernel: where the norms of all heads and the output tiles go on every GPU
struct NagPeerSpec {
    void* const* out_peers;
    unsigned long long* const* ctr_peers;
    float* const* part_peers;
    unsigned int* const* flag_peers;
    int n_peers, self, col0, h0, heads_total;
    unsigned int epoch;
};

static int nag_impl(void* out, const void* q, const void* qn_w, const void* k_pos, const void* v_pos, int Tk_pos, int npad_pos,
                    const void* k_neg, const void* v_neg, int Tk_neg, int npad_neg, float scale, float tau, float alpha, int Tq,
                    int H, int ld_q, int ld_kv, int ld_o, int dtype, int out_dtype, float eps, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream, const NagPeerSpec* peers) {
    if (!valid_in_dtype(dtype)) return KB_ERR_ARG;
    if (Tq <= 0 || Tk_pos <= 0 || Tk_neg <= 0 || H <= 0 || npad_pos < 0 || npad_neg < 0) return KB_ERR_ARG;
    if (H > 64) return KB_ERR_SHAPE;                   // the heads of a query tile run on H different SMs at once
    if (!aligned16(qn_w)) return KB_ERR_ALIGN;         // read with 16-byte vector loads by the pre-pass
    if (peers) {
        if (peers->n_peers < 1 || peers->n_peers > MAX_PEERS || peers->self < 0 || peers->self >= peers->n_peers || peers->col0 < 0 ||
            (peers->col0 & 7) || peers->h0 < 0 || peers->heads_total < peers->h0 + H || peers->epoch == 0 || out_dtype == KB_F32)
            return KB_ERR_ARG;
        if (ld_o < peers->col0 + H * 128) return KB_ERR_SHAPE;
        for (int i = 0; i < peers->n_peers; i++) {
            if (!peers->out_peers[i] || !peers->ctr_peers[i] || !peers->part_peers[i] || !peers->flag_peers[i]) return KB_ERR_ARG;
            if (!aligned16(peers->out_peers[i])) return KB_ERR_ALIGN;
        }
        out = peers->out_peers[peers->self];
    }
    int rc;
    if ((rc = check_mat(q, ld_q, H, dtype)) || (rc = check_mat(k_pos, ld_kv, H, dtype)) || (rc = check_mat(v_pos, ld_kv, H, dtype)) ||
        (rc = check_mat(k_neg, ld_kv, H, dtype)) || (rc = check_mat(v_neg, ld_kv, H, dtype)) || (rc = check_out(out, ld_o, peers ? 0 : H, out_dtype)))
        return rc;
    DeviceState* st;
    if ((rc = get_state(&st))) return rc;
    const bool conv = dtype != KB_F16;
    const int n_qt = (Tq + BM - 1) / BM;
    Stage sg{static_cast<char*>(workspace), workspace_bytes};
    PrepBatch pb;
    pb.pp.H = H; pb.pp.eps = eps;
    float* nag_part = nullptr;
    unsigned int* nag_flag = nullptr;
    if (!peers) {
        if (!workspace || !aligned16(workspace)) return KB_ERR_WORKSPACE;   // always: the cross-head norm exchange lives there
        nag_part = static_cast<float*>(sg.take_bytes((size_t)n_qt * H * NAG_NORM_FLOATS * sizeof(float)));
        nag_flag = static_cast<unsigned int*>(sg.take_bytes((size_t)n_qt * sizeof(unsigned int)));
        if (sg.overflow) return KB_ERR_WORKSPACE;
        pb.zero(nag_flag, n_qt);                       // cleared by the pre-pass, or by a memset when nothing is staged
    } else {
        if ((conv || qn_w) && (!workspace || !aligned16(workspace))) return KB_ERR_WORKSPACE;
        nag_part = peers->part_peers[peers->self];     // the exchange lives in the peer-visible buffers; their counters only grow
        nag_flag = peers->flag_peers[peers->self];
    }
    const void* qq = q;
    const void* kv[4] = {k_pos, v_pos, k_neg, v_neg};
    const int kv_rows[4] = {Tk_pos, Tk_pos, Tk_neg, Tk_neg};
    int ldq = ld_q, ldkv = ld_kv;
    if (conv || qn_w) { void* d = sg.take((size_t)Tq, H); if (d) pb.add(d, H * 128, q, ld_q, Tq, Tq, qn_w, nullptr, nullptr); qq = d; ldq = H * 128; }
    if (conv) {
        for (int i = 0; i < 4; i++) {
            void* d = sg.take((size_t)kv_rows[i], H);
            if (d) pb.add(d, H * 128, kv[i], ld_kv, kv_rows[i], kv_rows[i], nullptr, nullptr, nullptr);
            kv[i] = d;
        }
        ldkv = H * 128;
    }
    if (sg.overflow) return KB_ERR_WORKSPACE;
    if ((rc = launch_prep(st, pb, dtype, KB_F16, stream))) return rc;
    CUtensorMap tq, tk0, tv0, tk1, tv1;
    if ((rc = make_tmap(&tq, qq, Tq, H, 1, ldq)) || (rc = make_tmap(&tk0, kv[0], Tk_pos, H, 1, ldkv)) ||
        (rc = make_tmap(&tv0, kv[1], Tk_pos, H, 1, ldkv)) || (rc = make_tmap(&tk1, kv[2], Tk_neg, H, 1, ldkv)) ||
        (rc = make_tmap(&tv1, kv[3], Tk_neg, H, 1, ldkv)))
        return rc;
    AttnParams p = {};
    p.out = out; p.ldo = ld_o; p.Tq = Tq; p.H = H; p.B = 1;
    p.Tk[0] = Tk_pos; p.Tk[1] = Tk_neg; p.npad[0] = npad_pos; p.npad[1] = npad_neg;
    p.n_items = n_qt * H;
    p.nag_part = nag_part; p.nag_flag = nag_flag;
    p.nag_heads = H; p.nag_h0 = 0; p.nag_epoch = 1;
    if (peers) {
        p.n_peers = peers->n_peers; p.col0 = peers->col0;
        p.nag_heads = peers->heads_total; p.nag_h0 = peers->h0; p.nag_epoch = peers->epoch;
        for (int i = 0; i < peers->n_peers; i++) {
            p.out_peers[i] = peers->out_peers[i]; p.ctr_peers[i] = peers->ctr_peers[i];
            p.nag_part_peers[i] = peers->part_peers[i]; p.nag_flag_peers[i] = peers->flag_peers[i];
        }
    }
    p.scale_log2 = SCALE_LOG2;
    p.nag_s = scale; p.nag_tau = tau; p.nag_alpha = alpha;
    p.status = st->status;
    ProfScope ps(st, KB_PROF_NAG, stream);
    return launch_attn<MODE_NAG>(out_dtype, tq, tk0, tv0, tk1, tv1, p, st->sm_count, stream);
}

int kb_attn_nag(void* out, const void* q, const void* qn_w, const void* k_pos, const void* v_pos, int Tk_pos, int npad_pos,
                const void* k_neg, const void* v_neg, int Tk_neg, int npad_neg, float scale, float tau, float alpha, int Tq,
                int H, int ld_q, int ld_kv, int ld_o, int dtype, int out_dtype, float eps, void* workspace,
                size_t workspace_bytes, void* stream_) {
    return nag_impl(out, q, qn_w, k_pos, v_pos, Tk_pos, npad_pos, k_neg, v_neg, Tk_neg, npad_neg, scale, tau, alpha, Tq, H, ld_q, ld_kv,
                    ld_o, dtype, out_dtype, eps, workspace, workspace_bytes, static_cast<cudaStream_t>(stream_), nullptr);
}

int kb_qk_prep(void* out, int ld_out, int out_dtype, const void* in, int ld_in, int in_dtype, int rows, int H, int T,
               const void* w_bf16, float eps, const float* rope_cos, const float* rope_sin, void* stream) {
    if (!out || !in || rows < 0 || H <= 0 || T <= 0) return KB_ERR_ARG;
    if (out_dtype != KB_F16 && out_dtype != KB_BF16 && out_dtype != KB_F32) return KB_ERR_ARG;
    if (in_dtype != KB_F16 && in_dtype != KB_BF16 && in_dtype != KB_F32) return KB_ERR_ARG;
    if (out_dtype == KB_F32 && in_dtype != KB_F32) return KB_ERR_ARG;
    if ((rope_cos == nullptr) != (rope_sin == nullptr)) return KB_ERR_ARG;
    if (!aligned16(out) || !aligned16(in) || (ld_out & (out_dtype == KB_F32 ? 3 : 7)) || (ld_in & (in_dtype == KB_F32 ? 3 : 7))) return KB_ERR_ALIGN;
    if (!aligned16(w_bf16) || !aligned16(rope_cos) || !aligned16(rope_sin)) return KB_ERR_ALIGN;   // 16-byte vector loads
    if (ld_out < H * 128 || ld_in < H * 128) return KB_ERR_SHAPE;
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    PrepBatch pb;
    pb.pp.H = H; pb.pp.eps = eps;
    pb.add(out, ld_out, in, ld_in, rows, T, w_bf16, rope_cos, rope_sin);
    return launch_prep(st, pb, in_dtype, out_dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

namespace {

// [rows][cols] view of the output with row stride ld; box = 128 bytes of columns x 32 rows with 128-byte swizzle, or
// (half_heads: the fused head epilogue stores 32-column half-heads) 64 bytes x 32 rows unswizzled
int make_tmap_out(CUtensorMap* tm, void* ptr, int rows, int cols, int ld, bool f32, bool half_heads) {
    const cuuint64_t esz = f32 ? 4 : 2;
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
    const cuuint64_t strides[2] = {(cuuint64_t)ld * esz, (cuuint64_t)rows * (cuuint64_t)ld * esz};
    const cuuint32_t box[3] = {half_heads ? 32u : (cuuint32_t)(128 / esz), 32, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, ptr, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, half_heads ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KB_OK : KB_ERR_CUDA;
}

// [rows][cols] view of a row-major fp16 matrix with row stride ld; box = 64 columns x 128 rows, 128-byte swizzle
int make_tmap_mat(CUtensorMap* tm, const void* ptr, int rows, int cols, int ld) {
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
    const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)rows * (cuuint64_t)ld * 2};
    const cuuint32_t box[3] = {64, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KB_OK : KB_ERR_CUDA;
}

// p.N is the width of ONE segment; the launch covers n_seg of them side by side
template <int EPI, bool PAIR>
int launch_gemm_shape(DeviceState* st, const CUtensorMap& ta, const GemmMaps& maps, GemmParams p, int n_seg, cudaStream_t stream) {
    const int tile = PAIR ? 256 : 128, per_group = PAIR ? 2 : 1;
    p.tiles_m = (p.M + tile - 1) / tile;
    p.tiles_n_seg = (p.N + tile - 1) / tile;
    p.tiles_n = p.tiles_n_seg * n_seg;
    const int n_tiles = p.tiles_m * p.tiles_n, max_groups = st->sm_count / per_group;
    const int groups = n_tiles < max_groups ? n_tiles : max_groups;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(groups * per_group));
    cfg.blockDim = dim3(G_THREADS);
    cfg.dynamicSmemBytes = G_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = per_group; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ProfScope ps(st, KB_PROF_LINEAR, stream);
    return cudaLaunchKernelEx(&cfg, gemm16_kernel<EPI, PAIR>, ta, maps, p) == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

// CTA pairs on 256x256 tiles when that fills the device better. Measured on B200 a CTA of a pair spends about 11/8 of the
// time a single CTA spends per 64-wide k step while doing twice the work, so compare waves x time per step.
template <int EPI>
int launch_gemm(DeviceState* st, const CUtensorMap& ta, const GemmMaps& maps, const GemmParams& p, int n_seg, cudaStream_t stream) {
    if (p.N % 256 == 0 && p.M > 128) {
        const long long tp = (long long)((p.M + 255) / 256) * (p.N / 256) * n_seg, ts = (long long)((p.M + 127) / 128) * (p.N / 128) * n_seg;
        const long long gp = st->sm_count / 2, gs = st->sm_count;
        const long long pair_cost = ((tp + gp - 1) / gp) * 11, single_cost = ((ts + gs - 1) / gs) * 8;
        if (pair_cost <= single_cost) return launch_gemm_shape<EPI, true>(st, ta, maps, p, n_seg, stream);
    }
    return launch_gemm_shape<EPI, false>(st, ta, maps, p, n_seg, stream);
}

// The second product of a segment (null = none): A2 [M, K2] with row stride lda2, W2 [N, K2] with row stride ldw2.
struct SecondProduct {
    const void* const* A2 = nullptr;
    const void* const* W2 = nullptr;
    const int* K2 = nullptr;
    const int* lda2 = nullptr;
    const int* ldw2 = nullptr;
};

// shared body of kb_linear16 (one weight matrix) and kb_linear16_qkv (three, one launch)
int linear16_segments(void* const* C, int ldc, const void* A, int lda, const void* const* W, int ldw, int n_seg, int M, int N, int K, int epi,
                      const float* gate, const void* const* head_w, const int* rope_on, const float* rope_cos, const float* rope_sin,
                      int rope_T, float eps, cudaStream_t stream, const SecondProduct& sp = SecondProduct()) {
    if (!A || M < 0 || N <= 0 || K <= 0 || n_seg < 1 || n_seg > 3) return KB_ERR_ARG;
    if (epi < KB_EPI_F32 || epi > KB_EPI_HEADS16) return KB_ERR_ARG;
    if ((rope_cos == nullptr) != (rope_sin == nullptr)) return KB_ERR_ARG;
    if (rope_cos && rope_T <= 0) return KB_ERR_ARG;
    if (epi != KB_EPI_RESID && gate) return KB_ERR_ARG;
    const bool c32 = epi == KB_EPI_F32 || epi == KB_EPI_RESID;
    if (!aligned16(A) || (lda & 7) || (ldw & 7) || (ldc & (c32 ? 3 : 7))) return KB_ERR_ALIGN;
    if (gate && !aligned16(gate)) return KB_ERR_ALIGN;
    if (rope_cos && (!aligned16(rope_cos) || !aligned16(rope_sin))) return KB_ERR_ALIGN;
    bool any_rope = false;
    for (int i = 0; i < n_seg; i++) {
        if (!C[i] || !W[i]) return KB_ERR_ARG;
        if (!aligned16(C[i]) || !aligned16(W[i]) || (head_w[i] && !aligned16(head_w[i]))) return KB_ERR_ALIGN;
        if (epi != KB_EPI_HEADS16 && (head_w[i] || rope_on[i])) return KB_ERR_ARG;
        any_rope = any_rope || rope_on[i];
    }
    if (any_rope && !rope_cos) return KB_ERR_ARG;
    // A plain store epilogue of one matrix also takes a width that is no multiple of the 128-column tile (the rank of a
    // LoRA down-projection): the weight rows past N read as zeros and the stores past N are left out.
    const bool narrow_ok = n_seg == 1 && (epi == KB_EPI_F32 || epi == KB_EPI_F16 || epi == KB_EPI_GELU16);
    if ((narrow_ok ? (N % 8) : (N % 128)) || (K % GB_K) || lda < K || ldw < K || ldc < N) return KB_ERR_SHAPE;
    for (int i = 0; i < n_seg && sp.K2; i++) {
        if (sp.K2[i] < 0) return KB_ERR_ARG;
        if (sp.K2[i] == 0) continue;
        if (!sp.A2 || !sp.W2 || !sp.lda2 || !sp.ldw2 || !sp.A2[i] || !sp.W2[i]) return KB_ERR_ARG;
        if (!aligned16(sp.A2[i]) || !aligned16(sp.W2[i]) || (sp.lda2[i] & 7) || (sp.ldw2[i] & 7)) return KB_ERR_ALIGN;
        if ((sp.K2[i] % 8) || sp.lda2[i] < sp.K2[i] || sp.ldw2[i] < sp.K2[i]) return KB_ERR_SHAPE;
    }
    if (M == 0) return KB_OK;
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    CUtensorMap ta;
    GemmMaps maps;
    memset(&maps, 0, sizeof(maps));
    if ((rc = make_tmap_mat(&ta, A, M, K, lda))) return rc;
    GemmParams p = {};
    for (int i = 0; i < n_seg; i++) {
        if ((rc = make_tmap_mat(&maps.w[i], W[i], N, K, ldw)) || (rc = make_tmap_out(&maps.c[i], C[i], M, N, ldc, c32, epi == KB_EPI_HEADS16))) return rc;
        p.head_w[i] = static_cast<const __nv_bfloat16*>(head_w[i]);
        p.rope_on[i] = rope_on[i] ? 1 : 0;
        if (sp.K2 && sp.K2[i] > 0) {
            p.K2[i] = sp.K2[i];
            if ((rc = make_tmap_mat(&maps.a2[i], sp.A2[i], M, sp.K2[i], sp.lda2[i])) || (rc = make_tmap_mat(&maps.w2[i], sp.W2[i], N, sp.K2[i], sp.ldw2[i]))) return rc;
        }
    }
    p.C = C[0]; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
    p.gate = gate;
    p.rope_cos = rope_cos; p.rope_sin = rope_sin; p.rope_T = rope_T > 0 ? rope_T : 1; p.eps = eps;
    p.status = st->status;
    switch (epi) {
        case KB_EPI_F32: return launch_gemm<EPI_F32>(st, ta, maps, p, n_seg, stream);
        case KB_EPI_F16: return launch_gemm<EPI_F16>(st, ta, maps, p, n_seg, stream);
        case KB_EPI_GELU16: return launch_gemm<EPI_GELU16>(st, ta, maps, p, n_seg, stream);
        case KB_EPI_RESID: return launch_gemm<EPI_RESID>(st, ta, maps, p, n_seg, stream);
        default: return launch_gemm<EPI_HEADS16>(st, ta, maps, p, n_seg, stream);
    }
}

}  // namespace

extern "C" {

int kb_linear16(void* C, int ldc, const void* A, int lda, const void* W, int ldw, int M, int N, int K, int epi,
                const float* gate, const void* head_w_bf16, const float* rope_cos, const float* rope_sin, int rope_T,
                float eps, void* stream) {
    if (epi != KB_EPI_HEADS16 && (head_w_bf16 || rope_cos)) return KB_ERR_ARG;
    void* const cs[1] = {C};
    const void* const ws[1] = {W};
    const void* const hw[1] = {head_w_bf16};
    const int rope_on[1] = {rope_cos != nullptr};
    return linear16_segments(cs, ldc, A, lda, ws, ldw, 1, M, N, K, epi, gate, hw, rope_on, rope_cos, rope_sin, rope_T, eps,
                             static_cast<cudaStream_t>(stream));
}

int kb_linear16_qkv(void* const* C3, int ldc, const void* A, int lda, const void* const* W3, int ldw, int M, int N, int K,
                    const void* const* head_w3, const int* rope_on3, const float* rope_cos, const float* rope_sin, int rope_T,
                    float eps, void* stream) {
    if (!C3 || !W3 || !head_w3 || !rope_on3) return KB_ERR_ARG;
    return linear16_segments(C3, ldc, A, lda, W3, ldw, 3, M, N, K, KB_EPI_HEADS16, nullptr, head_w3, rope_on3, rope_cos, rope_sin, rope_T, eps,
                             static_cast<cudaStream_t>(stream));
}

int kb_linear16_lora(void* C, int ldc, const void* A, int lda, const void* W, int ldw, const void* A2, int lda2, const void* W2,
                     int ldw2, int K2, int M, int N, int K, int epi, const float* gate, const void* head_w_bf16,
                     const float* rope_cos, const float* rope_sin, int rope_T, float eps, void* stream) {
    if (epi != KB_EPI_HEADS16 && (head_w_bf16 || rope_cos)) return KB_ERR_ARG;
    void* const cs[1] = {C};
    const void* const ws[1] = {W};
    const void* const hw[1] = {head_w_bf16};
    const int rope_on[1] = {rope_cos != nullptr};
    const void* const a2[1] = {A2};
    const void* const w2[1] = {W2};
    SecondProduct sp;
    sp.A2 = a2; sp.W2 = w2; sp.K2 = &K2; sp.lda2 = &lda2; sp.ldw2 = &ldw2;
    return linear16_segments(cs, ldc, A, lda, ws, ldw, 1, M, N, K, epi, gate, hw, rope_on, rope_cos, rope_sin, rope_T, eps,
                             static_cast<cudaStream_t>(stream), sp);
}

int kb_linear16_qkv_lora(void* const* C3, int ldc, const void* A, int lda, const void* const* W3, int ldw, const void* const* A2_3,
                         const int* lda2_3, const void* const* W2_3, const int* ldw2_3, const int* K2_3, int M, int N, int K,
                         const void* const* head_w3, const int* rope_on3, const float* rope_cos, const float* rope_sin, int rope_T,
                         float eps, void* stream) {
    if (!C3 || !W3 || !head_w3 || !rope_on3 || !K2_3) return KB_ERR_ARG;
    SecondProduct sp;
    sp.A2 = A2_3; sp.W2 = W2_3; sp.K2 = K2_3; sp.lda2 = lda2_3; sp.ldw2 = ldw2_3;
    return linear16_segments(C3, ldc, A, lda, W3, ldw, 3, M, N, K, KB_EPI_HEADS16, nullptr, head_w3, rope_on3, rope_cos, rope_sin, rope_T, eps,
                             static_cast<cudaStream_t>(stream), sp);
}

// ------------------------------------------------------------------------------------------- attention backward
namespace {
size_t bwd_stats_bytes(int B, int Tq, int H) { return align256((size_t)B * H * ((Tq + 127) / 128) * 256 * sizeof(float)); }
// How the dK/dV role cuts its query blocks when there are too few (key block, head, image) triples to fill the GPU
// (cross-attention to a short context): parts of q_per query blocks each; 1 part = no cut.
void bwd_qsplit(int B, int Tq, int Tk, int H, int sm_count, int* qsplit, int* q_per) {
    const long long triples = (long long)B * H * ((Tk + 127) / 128);
    const int nqb = (Tq + 127) / 128;
    int want = (int)(sm_count / (triples > 0 ? triples : 1));
    if (want > nqb) want = nqb;
    if (want < 2) { *qsplit = 1; *q_per = nqb; return; }
    *q_per = (nqb + want - 1) / want;
    *qsplit = (nqb + *q_per - 1) / *q_per;
}
size_t bwd_partial_bytes(int B, int Tk, int H, int qsplit) { return qsplit > 1 ? 2 * align256((size_t)qsplit * B * Tk * H * 128 * sizeof(float)) : 0; }
size_t bwd_fixed_bytes(int B, int Tq, int Tk, int H, int dtype) {
    size_t n = bwd_stats_bytes(B, Tq, H) + align256((size_t)B * Tq * H * 128 * 2);                         // statistics, O (fp16)
    if (dtype != KB_F16) n += 2 * align256((size_t)B * Tq * H * 128 * 2) + 2 * align256((size_t)B * Tk * H * 128 * 2);   // fp16 Q, dO, K, V
    return n;
}
}  // namespace

size_t kb_attn_bwd_workspace_bytes(int B, int Tq, int Tk, int H, int dtype) {
    if (B <= 0 || Tq <= 0 || Tk <= 0 || H <= 0 || H > MAX_HEADS || !valid_in_dtype(dtype)) return 0;
    // + the partial dK / dV of a cut query range, + what the forward pass inside wants for its balanced schedule (it runs on
    // fp16 operands: no staging of its own)
    int sms = 148, qsplit, q_per;
    DeviceState* st;
    if (get_state(&st) == KB_OK) sms = st->sm_count;
    bwd_qsplit(B, Tq, Tk, H, sms, &qsplit, &q_per);
    return bwd_fixed_bytes(B, Tq, Tk, H, dtype) + bwd_partial_bytes(B, Tk, H, qsplit) + kb_attn_workspace_bytes(B * Tq, B * Tk, 1, H, KB_F16, 0, 0);
}

int kb_attn_bwd(void* dq, void* dk, void* dv, const void* q, const void* k, const void* v, const void* dout, int B, int Tq, int Tk,
                int npad, int H, int ld_q, int ld_k, int ld_v, int ld_do, int ld_dq, int ld_dk, int ld_dv, int dtype, void* workspace,
                size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!dq || !dk || !dv || !q || !k || !v || !dout || !valid_in_dtype(dtype)) return KB_ERR_ARG;
    if (B <= 0 || Tq <= 0 || Tk <= 0 || H <= 0 || npad < 0) return KB_ERR_ARG;
    if (H > MAX_HEADS) return KB_ERR_SHAPE;
    int rc;
    if ((rc = check_mat(q, ld_q, H, dtype)) || (rc = check_mat(k, ld_k, H, dtype)) || (rc = check_mat(v, ld_v, H, dtype)) ||
        (rc = check_mat(dout, ld_do, H, dtype)) || (rc = check_out(dq, ld_dq, H, KB_F32)) || (rc = check_out(dk, ld_dk, H, KB_F32)) ||
        (rc = check_out(dv, ld_dv, H, KB_F32)))
        return rc;
    if (!workspace || !aligned16(workspace)) return KB_ERR_WORKSPACE;
    DeviceState* st;
    if ((rc = get_state(&st))) return rc;
    Stage sg{static_cast<char*>(workspace), workspace_bytes};
    float* stats = static_cast<float*>(sg.take_bytes(bwd_stats_bytes(B, Tq, H)));
    __half* o16 = static_cast<__half*>(sg.take_bytes((size_t)B * Tq * H * 128 * 2));
    int qsplit, q_per;
    bwd_qsplit(B, Tq, Tk, H, st->sm_count, &qsplit, &q_per);
    float* part_dk = nullptr;
    float* part_dv = nullptr;
    if (qsplit > 1) {
        part_dk = static_cast<float*>(sg.take_bytes((size_t)qsplit * B * Tk * H * 128 * sizeof(float)));
        part_dv = static_cast<float*>(sg.take_bytes((size_t)qsplit * B * Tk * H * 128 * sizeof(float)));
    }
    const void *qq = q, *kk = k, *vv = v, *gg = dout;
    int ldq = ld_q, ldk = ld_k, ldv = ld_v, ldg = ld_do;
    PrepBatch pb;
    pb.pp.H = H; pb.pp.eps = 0.f;
    if (dtype != KB_F16) {
        void* d;
        d = sg.take((size_t)B * Tq, H); if (d) pb.add(d, H * 128, q, ld_q, B * Tq, Tq, nullptr, nullptr, nullptr); qq = d; ldq = H * 128;
        d = sg.take((size_t)B * Tq, H); if (d) pb.add(d, H * 128, dout, ld_do, B * Tq, Tq, nullptr, nullptr, nullptr); gg = d; ldg = H * 128;
        d = sg.take((size_t)B * Tk, H); if (d) pb.add(d, H * 128, k, ld_k, B * Tk, Tk, nullptr, nullptr, nullptr); kk = d; ldk = H * 128;
        d = sg.take((size_t)B * Tk, H); if (d) pb.add(d, H * 128, v, ld_v, B * Tk, Tk, nullptr, nullptr, nullptr); vv = d; ldv = H * 128;
    }
    if (sg.overflow) return KB_ERR_WORKSPACE;
    if ((rc = launch_prep(st, pb, dtype, KB_F16, stream))) return rc;
    // forward on the fp16 operands: O for D, and L into the statistics
    if ((rc = attn_pair(o16, qq, kk, vv, nullptr, nullptr, nullptr, nullptr, B, Tq, Tk, npad, H, ldq, ldk, ldv, H * 128, KB_F16, KB_F16, 0.f,
                        sg.ws, sg.left, stream, nullptr, stats)))
        return rc;
    {
        const long long warps = (long long)B * H * ((Tq + 127) / 128) * 128;
        const unsigned grid = (unsigned)((warps + 7) / 8);
        // dO as the tensor cores see it (fp16), so that the rows of dS sum to zero as exactly as the products allow
        bwd_delta_kernel<<<grid, 256, 0, stream>>>(stats, static_cast<const __half*>(gg), ldg, o16, H * 128, B, Tq, H);
        if (cudaGetLastError() != cudaSuccess) return KB_ERR_CUDA;
    }
    CUtensorMap tq, tk, tv, tg;
    if ((rc = make_tmap(&tq, qq, Tq, H, B, ldq)) || (rc = make_tmap(&tk, kk, Tk, H, B, ldk)) || (rc = make_tmap(&tv, vv, Tk, H, B, ldv)) ||
        (rc = make_tmap(&tg, gg, Tq, H, B, ldg)))
        return rc;
    BwdParams p = {};
    p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk;
    p.qsplit = qsplit; p.q_per = q_per;
    p.stats = stats; p.scale_log2 = SCALE_LOG2; p.scale = 0.08838834764831845f;
    p.status = st->status;
    ProfScope ps(st, KB_PROF_ATTENTION, stream);
    // fp32 [B][T][H*128] views of the three outputs, 32 columns x 32 rows per box (128-byte rows, 128-byte swizzle)
    CUtensorMap tdq, tdk, tdv;
    {
        // a cut query range writes its dK / dV parts to scratch: dense [qsplit * B][Tk][H*128]
        struct { CUtensorMap* tm; void* ptr; int T, ld, nb; } outs[3] = {{&tdq, dq, Tq, ld_dq, B},
                                                                         {&tdk, qsplit > 1 ? (void*)part_dk : dk, Tk, qsplit > 1 ? H * 128 : ld_dk, qsplit * B},
                                                                         {&tdv, qsplit > 1 ? (void*)part_dv : dv, Tk, qsplit > 1 ? H * 128 : ld_dv, qsplit * B}};
        for (auto& o : outs) {
            const cuuint64_t dims[3] = {(cuuint64_t)H * 128, (cuuint64_t)o.T, (cuuint64_t)o.nb};
            const cuuint64_t strides[2] = {(cuuint64_t)o.ld * 4, (cuuint64_t)o.T * (cuuint64_t)o.ld * 4};
            const cuuint32_t box[3] = {32, 32, 1};
            const cuuint32_t estr[3] = {1, 1, 1};
            if (g_encode(o.tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, o.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return KB_ERR_CUDA;
        }
    }
    const long long n_dkv = (long long)B * H * ((Tk + 127) / 128) * qsplit, n_dq = (long long)B * H * ((Tq + 127) / 128);
    if (n_dkv + n_dq > 0x7fffffffLL) return KB_ERR_SHAPE;
    attn_bwd_kernel<<<(unsigned)(n_dkv + n_dq), BWD_THREADS, BWD_SMEM, stream>>>(tq, tk, tv, tg, tdq, tdk, tdv, p, (int)n_dkv);
    if (cudaGetLastError() != cudaSuccess) return KB_ERR_CUDA;
    if (qsplit > 1) {
        const size_t n = (size_t)B * Tk * H * 32;                 // one thread per four columns
        bwd_reduce_kernel<<<dim3((unsigned)((n + 255) / 256), 2), 256, 0, stream>>>(static_cast<float*>(dk), ld_dk, static_cast<float*>(dv), ld_dv, part_dk,
                                                                                   part_dv, B * Tk, H * 128, qsplit);
    }
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

int kb_cross_kv(void* k16, void* v16, int ld_out, const void* ctx, int ld_ctx, int ctx_dtype, int L, int N, int K, const void* Wk,
                const void* Wv, int ldw, const void* kn_w_bf16, float eps, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!k16 || !v16 || !ctx || !Wk || !Wv || L < 0 || N <= 0 || K <= 0 || !valid_in_dtype(ctx_dtype)) return KB_ERR_ARG;
    if ((N % 128) || (K % 128) || ld_ctx < K) return KB_ERR_SHAPE;
    if (!aligned16(ctx) || (ld_ctx & (ctx_dtype == KB_F32 ? 3 : 7))) return KB_ERR_ALIGN;
    if (L == 0) return KB_OK;
    const void* x16 = ctx;
    int ldx = ld_ctx;
    if (ctx_dtype != KB_F16) {                                   // the context as fp16 rows in the workspace, as the GEMM reads it
        const size_t need = (size_t)L * K * 2;
        if (!workspace || workspace_bytes < need) return KB_ERR_WORKSPACE;
        if (!aligned16(workspace)) return KB_ERR_ALIGN;
        DeviceState* st;
        int rc;
        if ((rc = get_state(&st))) return rc;
        PrepBatch pb;
        pb.pp.H = K / 128; pb.pp.eps = eps;
        pb.add(workspace, K, ctx, ld_ctx, L, L, nullptr, nullptr, nullptr);
        if ((rc = launch_prep(st, pb, ctx_dtype, KB_F16, stream))) return rc;
        x16 = workspace;
        ldx = K;
    }
    void* const cs[2] = {k16, v16};
    const void* const ws[2] = {Wk, Wv};
    const void* const hw[2] = {kn_w_bf16, nullptr};
    const int rope_on[2] = {0, 0};
    return linear16_segments(cs, ld_out, x16, ldx, ws, ldw, 2, L, N, K, KB_EPI_HEADS16, nullptr, hw, rope_on, nullptr, nullptr, 0, eps, stream);
}

int kb_lora_pack(void* dst_f16, int ld, int col0, const void* src_bf16, int rows, int cols, float scale, void* stream) {
    if (!dst_f16 || !src_bf16 || rows < 0 || cols < 0 || col0 < 0 || ld < col0 + cols) return KB_ERR_ARG;
    const size_t n = (size_t)rows * cols;
    if (!n) return KB_OK;
    lora_pack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half*>(dst_f16), ld, col0, static_cast<const __nv_bfloat16*>(src_bf16), rows, cols, scale);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

int kb_status(unsigned* status_bits) {
    if (!status_bits) return KB_ERR_ARG;
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    unsigned v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return KB_ERR_CUDA;
    if (cudaMemcpy(&v, st->status, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return KB_ERR_CUDA;
    if (v && cudaMemset(st->status, 0, sizeof(v)) != cudaSuccess) return KB_ERR_CUDA;
    *status_bits = v;
    return (v & ST_TIMEOUT) ? KB_ERR_TIMEOUT : KB_OK;
}

int kb_prof_enable(int on) {
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    Prof& pf = st->prof;
    if (on && !pf.ev) {
        pf.ev = new cudaEvent_t[2 * PROF_POOL];
        pf.cat = new unsigned char[PROF_POOL];
        for (int i = 0; i < 2 * PROF_POOL; i++)
            if (cudaEventCreate(&pf.ev[i]) != cudaSuccess) return KB_ERR_CUDA;
    }
    pf.on = on != 0;
    pf.used = 0;
    return KB_OK;
}

int kb_prof_read(int category, double* total_ms, int* launches) {
    if (!total_ms || !launches || category < 0 || category >= KB_PROF_CATEGORIES) return KB_ERR_ARG;
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    Prof& pf = st->prof;
    if (cudaDeviceSynchronize() != cudaSuccess) return KB_ERR_CUDA;
    double sum = 0;
    int n = 0;
    for (int i = 0; i < pf.used; i++) {
        if (pf.cat[i] != category) continue;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, pf.ev[2 * i], pf.ev[2 * i + 1]) != cudaSuccess) return KB_ERR_CUDA;
        sum += ms;
        n++;
    }
    *total_ms = sum;
    *launches = n;
    return KB_OK;
}

int kb_nag_combine(void* a, const void* an, int T, int dim, int lda, int ldn, float scale, float tau, float alpha, int dtype, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a || !an || T < 0 || dim <= 0 || !valid_in_dtype(dtype)) return KB_ERR_ARG;
    if ((dim & 7) || dim > 256 * 8 * NAG_MAX_CHUNKS || lda < dim || ldn < dim) return KB_ERR_SHAPE;
    const int m = dtype == KB_F32 ? 3 : 7;
    if (!aligned16(a) || !aligned16(an) || (lda & m) || (ldn & m)) return KB_ERR_ALIGN;
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    if (T == 0) return KB_OK;
    ProfScope ps(st, KB_PROF_NAG, stream);
    if (dtype == KB_F16) nag_combine_kernel<__half><<<T, 256, 0, stream>>>((__half*)a, (const __half*)an, dim, lda, ldn, scale, tau, alpha);
    else if (dtype == KB_BF16) nag_combine_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)an, dim, lda, ldn, scale, tau, alpha);
    else nag_combine_kernel<float><<<T, 256, 0, stream>>>((float*)a, (const float*)an, dim, lda, ldn, scale, tau, alpha);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------- head split
int kb_peer_alloc(size_t bytes, void** ptr) {
    if (!ptr || !bytes) return KB_ERR_ARG;
    if (cudaMalloc(ptr, bytes) != cudaSuccess) { cudaGetLastError(); return KB_ERR_CUDA; }
    if (cudaMemset(*ptr, 0, bytes) != cudaSuccess) return KB_ERR_CUDA;
    return KB_OK;
}
int kb_peer_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? KB_OK : KB_ERR_CUDA; }
int kb_ipc_export(void* ptr, unsigned char* handle64) {
    if (!ptr || !handle64) return KB_ERR_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) { cudaGetLastError(); return KB_ERR_CUDA; }
    memcpy(handle64, &h, 64);
    return KB_OK;
}
int kb_ipc_import(const unsigned char* handle64, void** ptr) {
    if (!ptr || !handle64) return KB_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return KB_ERR_CUDA; }
    return KB_OK;
}
int kb_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? KB_OK : KB_ERR_CUDA; }

int kb_attn_push(void* const* out_peers, unsigned long long* const* ctr_peers, int n_peers, int col0, const void* q, const void* k,
                 const void* v, const void* qn_w, const void* kn_w, const float* rope_cos, const float* rope_sin, int B, int Tq, int Tk,
                 int npad, int H_local, int ld_q, int ld_k, int ld_v, int ld_o, int dtype, int out_dtype, float eps, void* workspace,
                 size_t workspace_bytes, void* stream) {
    if (!out_peers || !ctr_peers) return KB_ERR_ARG;
    PeerSpec ps{out_peers, ctr_peers, n_peers, col0};
    return attn_pair(nullptr, q, k, v, qn_w, kn_w, rope_cos, rope_sin, B, Tq, Tk, npad, H_local, ld_q, ld_k, ld_v, ld_o, dtype, out_dtype, eps,
                     workspace, workspace_bytes, static_cast<cudaStream_t>(stream), &ps);
}

int kb_attn_nag_push(void* const* out_peers, unsigned long long* const* ctr_peers, float* const* part_peers, unsigned int* const* flag_peers,
                     int n_peers, int self, int col0, int h0, int heads_total, unsigned epoch, const void* q, const void* qn_w,
                     const void* k_pos, const void* v_pos, int Tk_pos, int npad_pos, const void* k_neg, const void* v_neg, int Tk_neg,
                     int npad_neg, float scale, float tau, float alpha, int Tq, int H_local, int ld_q, int ld_kv, int ld_o, int dtype,
                     int out_dtype, float eps, void* workspace, size_t workspace_bytes, void* stream) {
    if (!out_peers || !ctr_peers || !part_peers || !flag_peers) return KB_ERR_ARG;
    NagPeerSpec ps{out_peers, ctr_peers, part_peers, flag_peers, n_peers, self, col0, h0, heads_total, epoch};
    return nag_impl(nullptr, q, qn_w, k_pos, v_pos, Tk_pos, npad_pos, k_neg, v_neg, Tk_neg, npad_neg, scale, tau, alpha, Tq, H_local, ld_q,
                    ld_kv, ld_o, dtype, out_dtype, eps, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), &ps);
}

size_t kb_nag_exchange_bytes(int Tq, int heads_total) {
    if (Tq <= 0 || heads_total <= 0) return 0;
    const size_t n_qt = ((size_t)Tq + 127) / 128;
    return align256(n_qt * heads_total * NAG_NORM_FLOATS * sizeof(float)) + align256(n_qt * sizeof(unsigned int));
}

size_t kb_nag_exchange_counter_offset(int Tq, int heads_total) {
    if (Tq <= 0 || heads_total <= 0) return 0;
    return align256((((size_t)Tq + 127) / 128) * heads_total * NAG_NORM_FLOATS * sizeof(float));
}

int kb_bump_counters(unsigned long long* const* ctr_peers, int n_peers, void* stream) {
    if (!ctr_peers || n_peers < 1 || n_peers > MAX_PEERS) return KB_ERR_ARG;
    BumpList bl = {};
    for (int i = 0; i < n_peers; i++) { if (!ctr_peers[i]) return KB_ERR_ARG; bl.ctr[i] = ctr_peers[i]; }
    bl.n = n_peers;
    bump_counters_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(bl);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

unsigned long long kb_push_arrivals_per_call(int B, int Tq, int H_local, int n_peers) {
    return (unsigned long long)n_peers * (unsigned long long)B * (unsigned long long)H_local * (unsigned long long)((Tq + 127) / 128);
}

int kb_wait_arrivals(const unsigned long long* ctr, unsigned long long target, void* stream) {
    if (!ctr) return KB_ERR_ARG;
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    wait_arrivals_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(ctr, target, st->status, ST_TIMEOUT);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_CUDA;
}

// ---------------------------------------------------------------------------------------------
// Self-attention for callers that cannot hand over scratch memory and must not allocate any.
// The fp16 staging copies of Q, K and V go to a fixed array that is part of the library's device
// image, so the call makes no cudaMalloc / cudaFree and needs no caller workspace. The price: every
// GPU that loads the library carries the array until the process exits, problems whose staging
// does not fit are refused, and the array is shared by all calls on that GPU.
static __device__ __align__(256) unsigned char g_static_scratch[KB_STATIC_SCRATCH_BYTES];

namespace {
void* g_static_scratch_addr[MAX_DEVICES] = {};   // device address of the array, per device
std::mutex g_static_mu;

// The array's name is only a host-side handle here; kernels need its device address, looked up once
// per device while that device is current.
int static_scratch_addr(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return KB_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_scratch_addr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return KB_ERR_CUDA;
        }
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return KB_OK;
}
}  // namespace

int kb_attn_self_static(void* out, const void* q, const void* k, const void* v, const void* qn_w, const void* kn_w,
                        const float* rope_cos, const float* rope_sin, int B, int T, int H, int ld_q, int ld_k, int ld_v, int ld_o,
                        int dtype, int out_dtype, float eps, void* stream) {
    if (!valid_in_dtype(dtype) || B <= 0 || T <= 0 || H <= 0) return KB_ERR_ARG;
    if (H > MAX_HEADS) return KB_ERR_SHAPE;
    if ((long long)B * T > (long long)KB_STATIC_SCRATCH_BYTES) return KB_ERR_STATIC_SCRATCH;   // keeps the size arithmetic in range
    // only the staging copies must fit; what is left of the array serves the balanced schedule when it is enough for it
    const size_t need = staging_bytes((size_t)B * T, (size_t)B * T, 1, H, dtype, qn_w || rope_cos, kn_w || rope_cos);
    if (need > (size_t)KB_STATIC_SCRATCH_BYTES) return KB_ERR_STATIC_SCRATCH;
    void* scratch = nullptr;
    int rc;
    if ((rc = static_scratch_addr(&scratch))) return rc;
    // Nothing in the array has to start at zero: the pre-pass overwrites every staged row before the
    // attention kernel's TMA loads read it, and rows past the end are never read (the tensor maps bound them).
    return attn_pair(out, q, k, v, qn_w, kn_w, rope_cos, rope_sin, B, T, T, 0, H, ld_q, ld_k, ld_v, ld_o, dtype, out_dtype, eps, scratch,
                     (size_t)KB_STATIC_SCRATCH_BYTES, static_cast<cudaStream_t>(stream));
}

// 128 bf16 ones in the library's device image: the weight of an RMSNorm "without weight" (the engine's rmsnorm takes a null
// weight and still normalises: w ? bf(w[i]) : 1, engine/src/kernels.cu:650-673)
#define KB_R8(x) x, x, x, x, x, x, x, x
static __device__ __align__(16) unsigned short g_unit_weight[128] = {KB_R8(KB_R8(0x3f80)), KB_R8(KB_R8(0x3f80))};
#undef KB_R8

const void* kb_unit_norm_weight(void) {
    DeviceState* st;
    if (get_state(&st) != KB_OK) return nullptr;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_unit_weight) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}

size_t kb_selfcheck_workspace_bytes(void) { return (size_t)4 << 20; }

int kb_attn_selfcheck(void* workspace, size_t workspace_bytes, float* max_abs_err_out, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!workspace || workspace_bytes < kb_selfcheck_workspace_bytes() || !aligned16(workspace)) return KB_ERR_WORKSPACE;
    DeviceState* st;
    int rc;
    if ((rc = get_state(&st))) return rc;
    // small ragged shapes: neither Tq nor Tk a multiple of the tile sizes
    const int H = 2, ld = H * 128, Tq = 300, Tk = 200, Tc = 77, Tn = 26;
    char* ws = static_cast<char*>(workspace);
    auto take = [&](size_t bytes) { char* p = ws; ws += align256(bytes); return p; };
    void* q = take((size_t)Tq * ld * 2); void* k = take((size_t)Tq * ld * 2); void* v = take((size_t)Tq * ld * 2);
    void* k2 = take((size_t)Tq * ld * 2); void* v2 = take((size_t)Tq * ld * 2);
    float* out = (float*)take((size_t)Tq * ld * 4); float* ref = (float*)take((size_t)Tq * ld * 4);
    float* ref2 = (float*)take((size_t)Tq * ld * 4);
    unsigned int* err = (unsigned int*)take(256);
    const size_t stage_bytes = kb_attn_workspace_bytes(Tq, Tq, 2, H, KB_BF16, 1, 1);   // fp16 staging of bf16 inputs + NAG scratch
    void* stage = take(stage_bytes);
    const size_t n = (size_t)Tq * ld;
    const unsigned fb = (unsigned)((n + 255) / 256), ab = (unsigned)((Tq * H + 127) / 128);
    if (cudaMemsetAsync(err, 0, 4, stream) != cudaSuccess) return KB_ERR_CUDA;
    for (int dtype = 0; dtype < 2; dtype++) {
        if (dtype == KB_F16) {
            sc_fill_kernel<__half><<<fb, 256, 0, stream>>>((__half*)q, n, 11u, 1.2f);
            sc_fill_kernel<__half><<<fb, 256, 0, stream>>>((__half*)k, n, 12u, 1.2f);
            sc_fill_kernel<__half><<<fb, 256, 0, stream>>>((__half*)v, n, 13u, 0.8f);
            sc_fill_kernel<__half><<<fb, 256, 0, stream>>>((__half*)k2, n, 14u, 1.2f);
            sc_fill_kernel<__half><<<fb, 256, 0, stream>>>((__half*)v2, n, 15u, 0.8f);
        } else {
            sc_fill_kernel<__nv_bfloat16><<<fb, 256, 0, stream>>>((__nv_bfloat16*)q, n, 21u, 1.2f);
            sc_fill_kernel<__nv_bfloat16><<<fb, 256, 0, stream>>>((__nv_bfloat16*)k, n, 22u, 1.2f);
            sc_fill_kernel<__nv_bfloat16><<<fb, 256, 0, stream>>>((__nv_bfloat16*)v, n, 23u, 0.8f);
            sc_fill_kernel<__nv_bfloat16><<<fb, 256, 0, stream>>>((__nv_bfloat16*)k2, n, 24u, 1.2f);
            sc_fill_kernel<__nv_bfloat16><<<fb, 256, 0, stream>>>((__nv_bfloat16*)v2, n, 25u, 0.8f);
        }
        auto naive = [&](float* o, const void* kk, const void* vv, int tk, int npad) {
            if (dtype == KB_F16) sc_naive_attn_kernel<__half><<<ab, 128, 0, stream>>>(o, (const __half*)q, (const __half*)kk, (const __half*)vv, Tq, tk, H, ld, npad);
            else sc_naive_attn_kernel<__nv_bfloat16><<<ab, 128, 0, stream>>>(o, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kk, (const __nv_bfloat16*)vv, Tq, tk, H, ld, npad);
        };
        // self-shaped (Tq x Tk keys, no padding)
        if ((rc = kb_attn_cross(out, q, nullptr, k, v, Tq, Tk, 0, H, ld, ld, ld, ld, dtype, KB_F32, 1e-6f, stage, stage_bytes, stream))) return rc;
        naive(ref, k, v, Tk, 0);
        sc_maxdiff_kernel<<<fb, 256, 0, stream>>>(out, ref, n, err);
        // cross with analytic padding
        if ((rc = kb_attn_cross(out, q, nullptr, k, v, Tq, Tc, 512 - Tc, H, ld, ld, ld, ld, dtype, KB_F32, 1e-6f, stage, stage_bytes, stream))) return rc;
        naive(ref, k, v, Tc, 512 - Tc);
        sc_maxdiff_kernel<<<fb, 256, 0, stream>>>(out, ref, n, err);
        // NAG: two contexts, reference defaults s=5 tau=2.5 alpha=0.25 (engine/src/models.h:80)
        if ((rc = kb_attn_nag(out, q, nullptr, k, v, Tc, 512 - Tc, k2, v2, Tn, 512 - Tn, 5.f, 2.5f, 0.25f, Tq, H, ld, ld, ld, dtype, KB_F32,
                              1e-6f, stage, stage_bytes, stream)))
            return rc;
        naive(ref2, k2, v2, Tn, 512 - Tn);
        sc_naive_nag_kernel<<<(Tq + 127) / 128, 128, 0, stream>>>(ref, ref2, Tq, ld, 5.f, 2.5f, 0.25f);
        sc_maxdiff_kernel<<<fb, 256, 0, stream>>>(out, ref, n, err);
    }
    unsigned int bits = 0;
    if (cudaMemcpyAsync(&bits, err, 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return KB_ERR_CUDA;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return KB_ERR_CUDA;
    float e;
    memcpy(&e, &bits, 4);
    if (max_abs_err_out) *max_abs_err_out = e;
    unsigned sb = 0;
    if ((rc = kb_status(&sb))) return rc;
    return e <= 2e-3f ? KB_OK : KB_ERR_SELFCHECK;
}

}  // extern "C"
