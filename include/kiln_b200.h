/*
 * kiln_b200 — C ABI of the B200 (sm_100a) attention path for the kiln engine's Anima DiT.
 *
 * Conventions (all entry points):
 *   - plain C, no exceptions; every function returns an int status (KB_OK = 0, negative = error,
 *     kb_error_string() names it) unless stated otherwise;
 *   - every buffer is owned by the caller and lives on the current CUDA device; nothing is
 *     allocated per call, optional scratch is passed in as `workspace`;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*) and the call returns without
 *     synchronising; no hidden streams, no device-wide syncs;
 *   - activations are row-major [rows, ld] with head h at columns [h*128, (h+1)*128), the layout of
 *     the engine's op set (reference: engine/src/gpu.h:149-156); `ld_*` are in ELEMENTS;
 *   - head size is 128 (the only size the reference's fused kernels take: engine/src/tcflash.cuh:170-172);
 *   - row pointers must be 16-byte aligned and ld a multiple of 8 elements, 4 for fp32 (reference:
 *     engine/src/tcflash.cuh:169); the workspace must be 16-byte aligned.
 *
 * `npad` has the reference's meaning (engine/src/gpu.h:149-151): npad extra keys that are exactly
 * zero (K = 0, V = 0) join the softmax analytically. Reference semantics for a padded text context
 * are (Tk = real, npad = len - real); masking the padding out instead is (Tk = real, npad = 0).
 */
#ifndef KILN_B200_H
#define KILN_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of Q/K/V (`dtype`) and of the output (`out_dtype`), chosen independently.
 * The tensor-core operands are always fp16 with fp32 accumulation, as in the reference kernel, which
 * converts its fp32 inputs to fp16 while staging (engine/src/tcflash.cuh:56-64): KB_F16 inputs that need
 * neither norm nor RoPE are read in place; KB_BF16 / KB_F32 inputs, and any tensor that gets RMSNorm or
 * RoPE, are staged once as fp16 in the caller's workspace by a fused pre-pass. KB_F32 inputs are what the
 * engine holds today (engine/src/dit.cu:429-430). */
enum { KB_F16 = 0, KB_BF16 = 1, KB_F32 = 2 };

enum {
    KB_OK = 0,
    KB_ERR_ARG = -1,        /* null pointer, non-positive size, unknown dtype */
    KB_ERR_ALIGN = -2,      /* pointer not 16-byte aligned or ld not a multiple of 8 */
    KB_ERR_SHAPE = -3,      /* unsupported shape (ld < H*128, H not a cluster size for NAG, ...) */
    KB_ERR_WORKSPACE = -4,  /* workspace missing or too small */
    KB_ERR_CUDA = -5,       /* a CUDA runtime/driver call failed; cudaGetLastError has the detail */
    KB_ERR_DEVICE = -6,     /* not an sm_100 device, or no device */
    KB_ERR_TIMEOUT = -7,    /* a kernel gave up on a bounded wait (reported by kb_status) */
    KB_ERR_SELFCHECK = -8,  /* kb_attn_selfcheck: error above tolerance */
    KB_ERR_STATIC_SCRATCH = -9  /* kb_attn_self_static: the problem does not fit the built-in scratch */
};

const char* kb_error_string(int code);
int kb_version(void);

/* Prepare the current device (kernel attributes, status word). Idempotent and implied by every
 * launch entry point; call it once up front to keep the first launch cheap. */
int kb_init(void);

/* Bytes of scratch an attention call needs: room for the fp16 staging copies of Q (when dtype is not
 * KB_F16 or norm_q != 0), of K per context (dtype not KB_F16 or norm_k != 0) and of V per context
 * (dtype not KB_F16). rows_q = B*Tq, rows_k = B*Tk (the largest context for NAG), n_ctx = 1, or 2 for
 * kb_attn_nag. norm_q / norm_k: that tensor gets RMSNorm and/or RoPE. */
size_t kb_attn_workspace_bytes(int rows_q, int rows_k, int n_ctx, int H, int dtype, int norm_q, int norm_k);

/* Self-attention of B images, T tokens each (Tq = Tk = T), no padding.
 * Replaces, per DiT block, the reference sequence rmsnorm(Q), rmsnorm(K), rope_half(Q), rope_half(K),
 * attention16() (engine/src/dit.cu:464-470; ops at engine/src/kernels.cu:668-673, 773-777, 868-873).
 *   qn_w / kn_w : bf16 RMSNorm weight[128] for Q / K, or NULL for "already normalised"
 *   rope_cos / rope_sin : fp32 tables [T, 64] (engine/src/dit.cu:196-215), or NULL for no RoPE
 * q, k, v: [B*T, ld_*]; out: [B*T, ld_o]. */
int kb_attn_self(void* out, const void* q, const void* k, const void* v,
                 const void* qn_w, const void* kn_w, const float* rope_cos, const float* rope_sin,
                 int B, int T, int H, int ld_q, int ld_k, int ld_v, int ld_o,
                 int dtype, int out_dtype, float eps,
                 void* workspace, size_t workspace_bytes, void* stream);

/* kb_attn_self for callers that can neither pass a workspace nor allocate one. (No counterpart in the
 * reference: its ops bump-allocate scratch from the engine's arena.)
 *
 * Who needs it: code that runs with the GPU memory already carved up and no allocator to ask — an engine
 * whose arena was sized to the user's VRAM budget at start-up and is full, a plugin or callback that is
 * only given input and output buffers, a latency-sensitive loop where cudaMalloc (which synchronises the
 * device and can fail once another application has taken the remaining memory) is not acceptable.
 *
 * Same arguments and results as kb_attn_self, minus the workspace: the fp16 staging copies of Q, K and V
 * live in a fixed KB_STATIC_SCRATCH_BYTES array inside the library's device image. Consequences:
 *   - every GPU on which the library is loaded holds those 32 MiB until the process exits;
 *   - a problem whose staging (kb_attn_workspace_bytes(B*T, B*T, 1, H, dtype, norm_q, norm_k)) exceeds
 *     KB_STATIC_SCRATCH_BYTES is refused with KB_ERR_STATIC_SCRATCH and nothing is launched
 *     (e.g. bf16 or fp32 inputs: B*T*H <= 43690 rows-times-heads; 1536 tokens x 16 heads fit, 4096 x 16 do not);
 *   - the array is shared by every call on that GPU and keeps the previous call's contents (nothing in it
 *     needs clearing: each call overwrites what it later reads); two calls whose kernels overlap on the GPU
 *     (different streams, or different host threads) race on it — keep such calls on one stream;
 *   - the first call on each device looks up the array's device address (and, like every entry point,
 *     prepares the device); make that first call before any stream capture begins.
 * It calls no cudaMalloc / cudaFree and no allocating library routine. */
#define KB_STATIC_SCRATCH_BYTES (32u << 20)
int kb_attn_self_static(void* out, const void* q, const void* k, const void* v,
                        const void* qn_w, const void* kn_w, const float* rope_cos, const float* rope_sin,
                        int B, int T, int H, int ld_q, int ld_k, int ld_v, int ld_o,
                        int dtype, int out_dtype, float eps, void* stream);

/* Cross-attention of Tq latent tokens to one text context of Tk real rows + npad zero rows.
 * Replaces rmsnorm(Q) + attention16(..., Tk = real, npad) (engine/src/dit.cu:476-481). K is taken as
 * already normalised, as the reference's per-image K/V cache holds it (engine/src/dit.cu:217-234). */
int kb_attn_cross(void* out, const void* q, const void* qn_w, const void* k, const void* v,
                  int Tq, int Tk, int npad, int H, int ld_q, int ld_k, int ld_v, int ld_o,
                  int dtype, int out_dtype, float eps,
                  void* workspace, size_t workspace_bytes, void* stream);

/* NAG cross-attention: attention to the positive and the negative context from one Q, then
 *   g = s*Z+ - (s-1)*Z-;  ratio = |g|_1 / max(|Z+|_1, 1e-12) per token over all H*128 channels;
 *   out = alpha * g * (ratio > tau ? tau/ratio : 1) + (1 - alpha) * Z+
 * in one kernel. Replaces attention16 x2 + k_nag (engine/src/dit.cu:482-487, 295-324).
 * The per-token norms span all heads: the thread blocks holding the heads of one query tile exchange
 * their partial norms through a few KB of the workspace, so a workspace is ALWAYS required here
 * (kb_attn_workspace_bytes(Tq, max(Tk_pos, Tk_neg), 2, H, dtype, norm_q, 0)), H <= 64, and the launch is
 * cooperative (all its thread blocks are resident at once). */
int kb_attn_nag(void* out, const void* q, const void* qn_w,
                const void* k_pos, const void* v_pos, int Tk_pos, int npad_pos,
                const void* k_neg, const void* v_neg, int Tk_neg, int npad_neg,
                float scale, float tau, float alpha,
                int Tq, int H, int ld_q, int ld_kv, int ld_o,
                int dtype, int out_dtype, float eps,
                void* workspace, size_t workspace_bytes, void* stream);

/* The NAG combine on its own, in place on `a` (Z+) with `an` (Z-): the engine's k_nag launch
 * (engine/src/dit.cu:486, 524; kernel :295-324). Rows of `dim` channels (all heads together, dim % 8 == 0,
 * dim <= 8192), row strides lda / ldn in elements, dtype KB_F16 / KB_BF16 / KB_F32 for both. One pass:
 * the row stays in registers between the norm and the blend. kb_attn_nag fuses this into the attention
 * kernel; this entry point serves callers that already hold Z+ and Z- (head-split runs, the unfused engine path). */
int kb_nag_combine(void* a, const void* an, int T, int dim, int lda, int ldn,
                   float scale, float tau, float alpha, int dtype, void* stream);

/* ---- Head split at batch 1 (no counterpart in the reference, which is single-GPU: one cudaSetDevice at
 * engine/src/kernels.cu:207, no peer access, no collective). Each of G GPUs owns H/G heads: its Q/K/V are
 * [rows, (H/G)*128] slices, and every GPU needs the full [Tq, H*128] output for the following projection.
 * kb_attn_push is kb_attn_self / kb_attn_cross over the local heads whose epilogue writes each finished
 * 128-row tile into the output buffer of EVERY GPU (peer-mapped pointers, plain stores over NVLink) at
 * column col0 = rank*(H/G)*128, then bumps every GPU's arrival counter (system-scope fence + atomic).
 * kb_wait_arrivals enqueues a one-thread kernel that waits, bounded, until this GPU's counter reaches
 * `target`; work enqueued after it on the stream may read the gathered rows. Counters only grow: after
 * the n-th call target = n * kb_push_arrivals_per_call(...). Buffers for peers come from kb_peer_alloc
 * (cudaMalloc + zero fill, at set-up time) and travel between processes as 64-byte IPC handles. */
int kb_peer_alloc(size_t bytes, void** ptr);
int kb_peer_free(void* ptr);
int kb_ipc_export(void* ptr, unsigned char* handle64);
int kb_ipc_import(const unsigned char* handle64, void** ptr);
int kb_ipc_close(void* ptr);
int kb_attn_push(void* const* out_peers, unsigned long long* const* ctr_peers, int n_peers, int col0,
                 const void* q, const void* k, const void* v, const void* qn_w, const void* kn_w,
                 const float* rope_cos, const float* rope_sin,
                 int B, int Tq, int Tk, int npad, int H_local, int ld_q, int ld_k, int ld_v, int ld_o,
                 int dtype, int out_dtype, float eps, void* workspace, size_t workspace_bytes, void* stream);
/* Head-split NAG: kb_attn_nag over the local heads of one GPU. The per-token norms of the combine span all heads of the
 * model, so every thread block stores its head's two norms per row (2 floats per token and head, engine/src/dit.cu:295-324
 * computes them over the full row; here per half of the head's columns) into the exchange area of EVERY GPU (part_peers, plain peer stores) and bumps every
 * GPU's per-query-tile counter (flag_peers); it then waits, bounded, until its own GPU's counter shows all heads_total
 * heads of the tile, blends in fp32 exactly as the single-GPU kernel does, and stores the finished tile into every GPU's
 * output buffer at column col0 (then bumps ctr_peers as kb_attn_push does). Only final tiles and 16 bytes per token and
 * head cross NVLink. All GPUs must make the matching call (it is a collective). `self` = this GPU's index in the peer
 * arrays, h0 = its first head, epoch = 1, 2, 3 ... = how many times this exchange area has been used including this call
 * (its counters only grow and are never cleared, so a fast GPU's arrivals for the next call cannot be lost); an exchange
 * area is kb_nag_exchange_bytes(Tq, heads_total) bytes of zero-initialised peer-visible memory: the norms first, the
 * counters after them. A call may follow the previous one only when every GPU has finished that previous kernel
 * (kb_bump_counters / kb_wait_arrivals carry that hand-shake between streams of different GPUs). */
int kb_attn_nag_push(void* const* out_peers, unsigned long long* const* ctr_peers, float* const* part_peers, unsigned int* const* flag_peers,
                     int n_peers, int self, int col0, int h0, int heads_total, unsigned epoch,
                     const void* q, const void* qn_w, const void* k_pos, const void* v_pos, int Tk_pos, int npad_pos,
                     const void* k_neg, const void* v_neg, int Tk_neg, int npad_neg, float scale, float tau, float alpha,
                     int Tq, int H_local, int ld_q, int ld_kv, int ld_o, int dtype, int out_dtype, float eps,
                     void* workspace, size_t workspace_bytes, void* stream);
size_t kb_nag_exchange_bytes(int Tq, int heads_total);
size_t kb_nag_exchange_counter_offset(int Tq, int heads_total);   /* where the counters start inside an exchange area */
/* Buffer reuse across GPUs. Nothing above stops a fast GPU from pushing call n+1 into a buffer that a slow GPU is still
 * reading for call n. The hand-shake: when a GPU is done with a buffer it enqueues kb_bump_counters on the "released"
 * counters of that buffer on every GPU (one system-scope add each, ordered after everything enqueued before it on the
 * stream); before a GPU pushes use n+1 it enqueues kb_wait_arrivals on its OWN released counter with target n * n_gpus.
 * Counters only grow. */
int kb_bump_counters(unsigned long long* const* ctr_peers, int n_peers, void* stream);
unsigned long long kb_push_arrivals_per_call(int B, int Tq, int H_local, int n_peers);
int kb_wait_arrivals(const unsigned long long* ctr, unsigned long long target, void* stream);

/* Row pre-pass on its own: out[r, h*128..] = rope(rmsnorm(in[r, h*128..])) as 16-bit, or a plain
 * conversion when w, cos and sin are NULL. in_dtype may be KB_F32 (the engine keeps Q/K/V in fp32:
 * engine/src/dit.cu:429-430); with in_dtype = out_dtype = KB_F32 it is the engine's in-place fp32
 * rmsnorm / rope_half (out may equal in: every element is read before it is written by the same lane). Replaces rmsnorm + rope_half (engine/src/kernels.cu:668-673, 773-777)
 * and the fp32 -> fp16 staging inside the reference kernel (engine/src/tcflash.cuh:56-64). */
int kb_qk_prep(void* out, int ld_out, int out_dtype, const void* in, int ld_in, int in_dtype,
               int rows, int H, int T, const void* w_bf16, float eps,
               const float* rope_cos, const float* rope_sin, void* stream);

/* Device address (on the current device) of 128 bf16 ones: the `w_bf16` of a norm without weight. The engine's rmsnorm
 * normalises with weight 1 when it is given no weight (engine/src/kernels.cu:650-673); here a null weight means "no norm",
 * so a caller that wants the engine's behaviour passes this. NULL on failure. */
const void* kb_unit_norm_weight(void);

/* The projections either side of attention: C = epilogue(A[M,K] * W[N,K]^T), A and W fp16 row-major
 * (row strides lda, ldw in elements), fp32 accumulation. Replaces the engine's fp16-activation GEMM
 * linear16 -> tc16::launch (engine/src/kernels.cu:559-609, engine/src/tcgemm16.cuh:57-190; call sites
 * engine/src/dit.cu:461-463 (q/k/v), 471 (o-proj into the residual), 475, 488); its LoRA second product is
 * kb_linear16_lora below. Epilogues as there (engine/src/tcgemm16.cuh:145-174):
 *   KB_EPI_F32     C fp32 = acc
 *   KB_EPI_F16     C fp16 = acc
 *   KB_EPI_GELU16  C fp16 = gelu_erf(acc)
 *   KB_EPI_RESID   C fp32 += gate[c] * acc   (gate NULL = 1)
 * and one the engine does not have:
 *   KB_EPI_HEADS16 C fp16 = rope(rmsnorm(acc)) per 128-column head: head_w bf16[128] or NULL, rope tables
 *                  fp32 [rope_T, 64] or NULL (row r uses table row r % rope_T). It fuses the engine's
 *                  rmsnorm + rope_half launches (engine/src/dit.cu:464-468) and this library's staging
 *                  pre-pass into the q / k projection, so the attention entry points get fp16 operands
 *                  that need no further pass.
 * N must be a multiple of 128 and K of 64 (the engine asks N % 128 == 0, K % 32 == 0; every DiT weight
 * has K = 2048 or 8192); M is free. The three plain store epilogues (F32, F16, GELU16) also take any N that is a
 * multiple of 8: a LoRA down-projection t = x . A_cat^T has the stacked rank for its width. Pointers 16-byte aligned, strides multiples of 8 (fp16) / 4 (fp32). */
enum { KB_EPI_F32 = 0, KB_EPI_F16 = 1, KB_EPI_GELU16 = 2, KB_EPI_RESID = 3, KB_EPI_HEADS16 = 4 };
int kb_linear16(void* C, int ldc, const void* A, int lda, const void* W, int ldw, int M, int N, int K, int epi,
                const float* gate, const void* head_w_bf16, const float* rope_cos, const float* rope_sin, int rope_T,
                float eps, void* stream);

/* The q, k and v projections of one activation in ONE launch: C3[i] = heads16(A . W3[i]^T) for i = 0..2, every output
 * fp16 [M, ldc] with N = 128 * heads columns, every weight fp16 [N, ldw]; head_w3[i] (bf16[128] or NULL) and
 * rope_on3[i] choose the per-head RMSNorm and the RoPE of each projection (the engine: q and k normalised and
 * rotated, v neither: engine/src/dit.cu:461-468). Same arithmetic as three kb_linear16(KB_EPI_HEADS16) calls — the
 * results are bit-identical — with one pass over the tile schedule: 3x the tiles per launch fill the last wave
 * better and two launches, two pipeline fills and two drains go away. The engine has no counterpart (it issues three
 * linear16 calls, engine/src/dit.cu:461-463). */
int kb_linear16_qkv(void* const* C3, int ldc, const void* A, int lda, const void* const* W3, int ldw, int M, int N, int K,
                    const void* const* head_w3, const int* rope_on3, const float* rope_cos, const float* rope_sin, int rope_T,
                    float eps, void* stream);

/* kb_linear16 with a second product, the engine's unmerged LoRA side path (Args::A2, W2, K2 of
 * engine/src/tcgemm16.cuh:26-28, consumed at tcgemm16.cuh:70-76; composed by linear16, engine/src/kernels.cu:578-596):
 *   C = epilogue(A . W^T + A2 . W2^T),   A2 fp16 [M, K2] (row stride lda2), W2 fp16 [N, K2] (row stride ldw2).
 * In the engine A2 is t = x . A_cat^T (the stacked down-projections) and W2 is B_cat = [s1 B1 | s2 B2 | ...] with the
 * LoRA scales folded in, so every epilogue sees the LoRA-adjusted value. K2 is a multiple of 8 (the engine pads the
 * stacked rank to 32; here a last partial 64-wide k step reads zeros), K2 = 0 is kb_linear16. The second product's k
 * steps follow the first's in the same accumulator: no extra launch, no extra pass over C. Same argument rules as
 * kb_linear16 otherwise. */
int kb_linear16_lora(void* C, int ldc, const void* A, int lda, const void* W, int ldw, const void* A2, int lda2, const void* W2,
                     int ldw2, int K2, int M, int N, int K, int epi, const float* gate, const void* head_w_bf16,
                     const float* rope_cos, const float* rope_sin, int rope_T, float eps, void* stream);

/* kb_linear16_qkv with a second product per projection: A2_3[i] fp16 [M, K2_3[i]] with row stride lda2_3[i],
 * W2_3[i] fp16 [N, K2_3[i]] with row stride ldw2_3[i] (K2_3[i] = 0: projection i has no LoRA and its pointers may be NULL). Bit-identical to three kb_linear16_lora calls. */
int kb_linear16_qkv_lora(void* const* C3, int ldc, const void* A, int lda, const void* const* W3, int ldw, const void* const* A2_3,
                         const int* lda2_3, const void* const* W2_3, const int* ldw2_3, const int* K2_3, int M, int N, int K,
                         const void* const* head_w3, const int* rope_on3, const float* rope_cos, const float* rope_sin, int rope_T,
                         float eps, void* stream);

/* Attention backward: dq [B*Tq, ld_dq], dk, dv [B*Tk, ld_*] (fp32, written) of out = softmax(q k^T / sqrt(128)) v per head,
 * from q, k, v and dout (the gradient of out), all in `dtype`; npad zero keys of score 0 join the softmax as in the forward
 * calls. Replaces the engine's exact backward attention_bwd (engine/src/train.cu:216-242 with k_softmax_pad, train.cu:103-121,
 * and k_dsoftmax, train.cu:124-131; call sites train.cu:334 (cross-attention, npad) and train.cu:344 (self-attention)), which
 * materialises the [heads, Tq, Tk] probabilities and their gradients in the arena: here they are recomputed tile by tile on
 * the tensor cores (fp16 operands, fp32 accumulation; the engine's is fp32 throughout), nothing of size Tq x Tk is stored,
 * and every output element is written once in a fixed order (bit-identical from run to run). Launches: staging pre-pass
 * (unless dtype is KB_F16), the forward kernel (for the per-row softmax statistics and O), a reduction for
 * sum_d dout * O, and one launch whose thread blocks form dK/dV (one per key block) or dQ (one per query block). The workspace (kb_attn_bwd_workspace_bytes) is always required. */
size_t kb_attn_bwd_workspace_bytes(int B, int Tq, int Tk, int H, int dtype);
int kb_attn_bwd(void* dq, void* dk, void* dv, const void* q, const void* k, const void* v, const void* dout, int B, int Tq, int Tk,
                int npad, int H, int ld_q, int ld_k, int ld_v, int ld_do, int ld_dq, int ld_dk, int ld_dv, int dtype, void* workspace,
                size_t workspace_bytes, void* stream);

/* The cross-attention K/V of one context for one block, as the engine's per-generation cache makes them
 * (Dit::cache_context, engine/src/dit.cu:217-234, and per block at dit.cu:407-413):
 *   K = rmsnorm_per_head(ctx . Wk^T, kn_w),  V = ctx . Wv^T
 * but emitted as fp16 [L, ld_out] and already normalised: what kb_attn_cross / kb_attn_nag read with dtype KB_F16
 * and no staging pass, in half the engine's cache (which holds fp32 K and V and converts them in every attention call).
 * ctx [L, K] (K = 1024 in the engine) fp32, fp16 or bf16 with row stride ld_ctx; Wk, Wv fp16 [N, ldw]; kn_w bf16[128]
 * or NULL. One conversion launch when ctx is not fp16 (L * K * 2 bytes of workspace) and ONE GEMM launch for both
 * projections. N and K multiples of 128. */
int kb_cross_kv(void* k16, void* v16, int ld_out, const void* ctx, int ld_ctx, int ctx_dtype, int L, int N, int K, const void* Wk,
                const void* Wv, int ldw, const void* kn_w_bf16, float eps, void* workspace, size_t workspace_bytes, void* stream);

/* dst[r * ld + col0 + c] = fp16(scale * src[r, c]) for a bf16 matrix [rows, cols]: builds the stacked operands A_cat
 * (scale 1) and B_cat (the LoRA's scale) of the second product (k_lora_pack, engine/src/kernels.cu:548-554). */
int kb_lora_pack(void* dst_f16, int ld, int col0, const void* src_bf16, int rows, int cols, float scale, void* stream);

/* Read and clear the device status word of the current device (synchronises the device).
 * *status_bits = 0 when every kernel since the last call finished normally; returns KB_ERR_TIMEOUT
 * when a kernel gave up on a bounded wait. */
int kb_status(unsigned* status_bits);

/* Per-category kernel timing, the counterpart of the engine's ProfScope / prof_report
 * (engine/src/kernels.cu:18-58; categories "norm"+"rope" and "attention" there). kb_prof_enable(1)
 * (re)starts recording one CUDA event pair per kernel launch on the launch's stream, up to 8192 launches;
 * the event pool is created on the first enable, never per call. kb_prof_read synchronises the device
 * and returns the summed kernel time and launch count of one category since the last enable. */
enum { KB_PROF_NORM_ROPE = 0, KB_PROF_ATTENTION = 1, KB_PROF_NAG = 2, KB_PROF_LINEAR = 3, KB_PROF_CATEGORIES = 4 };
int kb_prof_enable(int on);
int kb_prof_read(int category, double* total_ms, int* launches);

/* Start-up known-answer test on the current device, in the spirit of the reference's start-up GEMM
 * cross-check (engine/src/kernels.cu:106-151): runs each kernel family on a small seeded problem and
 * compares with a one-thread-per-row fp32 kernel. workspace >= kb_selfcheck_workspace_bytes(). */
size_t kb_selfcheck_workspace_bytes(void);
int kb_attn_selfcheck(void* workspace, size_t workspace_bytes, float* max_abs_err_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KILN_B200_H */
