// The reference's LoRA trainer (engine/src/train.cu) with its attention backward bound to the library (TEST
// INFRASTRUCTURE; part of oracle/_ref/kiln-engine-shim, see oracle/build.py build_ref_engine).
//
// attention_bwd (engine/src/train.cu:216-242) lives in that file's anonymous namespace, so it cannot be replaced at link
// time like the five forward ops. The file is read unchanged under one macro that appends an argument to every mention of
// the name: the reference's definition becomes attention_bwd(..., int npad, int()) - an unnamed parameter of
// function-pointer type - and its two call sites (train.cu:334, 344) become attention_bwd(..., npad, int()), a call with a
// value-initialised int, which can only select the overload declared here first. That overload sends the call to the
// library (fp16 operands, fp32 accumulation, nothing of size Tq x Tk in memory) while the engine is in its fp16 mode and
// to the reference's own exact backward otherwise (G.fp16 off: a job that asked for exact arithmetic).
#include "gpu.h"

void kiln_bound_attention_bwd(float* dq, float* dk, float* dv, const float* q, const float* k, const float* v, const float* dout,
                              int Tq, int Tk, int npad);

namespace {
void attention_bwd(float* dq, float* dk, float* dv, const float* q, const float* k, const float* v, const float* dout, int Tq, int Tk,
                   int npad, int bound);
}

#define attention_bwd(...) attention_bwd(__VA_ARGS__, int())
#include "train.cu"
#undef attention_bwd

namespace {
void attention_bwd(float* dq, float* dk, float* dv, const float* q, const float* k, const float* v, const float* dout, int Tq, int Tk,
                   int npad, int) {
    if (!G.fp16) {
        attention_bwd(dq, dk, dv, q, k, v, dout, Tq, Tk, npad, (int (*)()) nullptr);   // the reference's own (exact) backward
        return;
    }
    ProfScope ps("bwd_attention");
    kiln_bound_attention_bwd(dq, dk, dv, q, k, v, dout, Tq, Tk, npad);
}
}  // namespace
