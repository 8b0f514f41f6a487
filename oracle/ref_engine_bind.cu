// The reference's whole engine over this repository's library (TEST INFRASTRUCTURE; see oracle/build.py build_ref_engine).
//
// The engine is built from its own translation units where they lie, unchanged. For the build over the library, its
// kernels.cu is compiled with the five attention-path ops renamed (-Dattention=ref_own_attention and so on), every other
// unit keeps calling the plain names, and this unit supplies them: the binding of oracle/ref_ops_binding.h.
#define attention ref_own_attention
#define attention16 ref_own_attention16
#define rmsnorm ref_own_rmsnorm
#define rope_half ref_own_rope_half
#define linear16 ref_own_linear16
#include "gpu.h"   // the reference's op declarations, as kernels.cu sees them under the same renames
#undef attention
#undef attention16
#undef rmsnorm
#undef rope_half
#undef linear16
#include <functional>
#include <vector>

#include "ref_ops_binding.h"
