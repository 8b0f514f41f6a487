// The reference's whole engine over this repository's library (TEST INFRASTRUCTURE; see oracle/build.py build_ref_engine).
//
// The engine is built from its own translation units where they lie, unchanged. For the build over the library, its
// kernels.cu is compiled with the five attention-path ops renamed (-Dattention=ref_own_attention and so on), every other
// unit keeps calling the plain names, and this unit supplies them: the binding of oracle/ref_ops_binding.h.
// gpu_alloc_scratch (engine/src/kernels.cu:239-247) is bound the same way: the engine sizes its arena to all the memory
// that is free (engine/src/engine.h:257-265), so the library's workspace is taken first and the arena made that much smaller.
#define attention ref_own_attention
#define attention16 ref_own_attention16
#define rmsnorm ref_own_rmsnorm
#define rope_half ref_own_rope_half
#define linear16 ref_own_linear16
#define gpu_alloc_scratch ref_own_gpu_alloc_scratch
#include "gpu.h"   // the reference's op declarations, as kernels.cu sees them under the same renames
#undef attention
#undef attention16
#undef rmsnorm
#undef rope_half
#undef linear16
#undef gpu_alloc_scratch
#include <functional>
#include <vector>

#include "ref_ops_binding.h"

void gpu_alloc_scratch(size_t wbuf_elems, size_t arena_bytes) {
    bind_workspace_reserve();
    // the engine sized the arena from the memory that was free before the workspace was taken: keep its own margin
    // (engine.h:259: the weight staging buffer + 160 MB) free now; an arena it already capped (--vram-budget) is left alone
    size_t free_now = 0, total = 0;
    CK(cudaMemGetInfo(&free_now, &total));
    const size_t keep = wbuf_elems * 4 + ((size_t)160 << 20);
    if (arena_bytes + keep > free_now && free_now > keep) arena_bytes = free_now - keep;
    ref_own_gpu_alloc_scratch(wbuf_elems, arena_bytes);
}

// for oracle/ref_engine_train_bind.cu: the trainer's backward bound in its own translation unit
void kiln_bound_attention_bwd(float* dq, float* dk, float* dv, const float* q, const float* k, const float* v, const float* dout,
                              int Tq, int Tk, int npad) {
    bind_context();
    kiln_b200::attention_bwd(dq, dk, dv, q, k, v, dout, Tq, Tk, npad, 16);
}
