// Test infrastructure only: compiles the reference's OWN rounding / requantisation functions for the oracle to be
// checked against.  The function bodies are not in this repository: the build recipe cuts the line ranges
//   include/tpu_mlir/Support/MathUtils.h   (the RoundingMode enum)
//   lib/Support/MathUtils.cpp              (to_int, RightShiftRound, MultiplyByQuantizedMultiplier,
//                                           applyMultiplierAndRShift)
// out of the reference checkout into generated include files beside the built library (a git-ignored folder) and
// this file supplies the few names those bodies expect from the rest of the reference (the RequantMode enum of
// TpuOps.td:160-172, module::isCV18xx(), llvm_unreachable).
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <string>

#include "_ref/mathutils_enum.inc"

namespace tpu {
enum class RequantMode { TFLite_LShift = 0, TFLite = 1, MultiplierShift = 2, OnlyShift = 3, QDM = 4, OnlyScale = 5 };
}
namespace module {
static bool g_cv18xx = false;
static bool isCV18xx() { return g_cv18xx; }
}  // namespace module
#define llvm_unreachable(msg) abort()

#include "_ref/mathutils_body.inc"

extern "C" {
long long ref_to_int_f32(float v, int rmode) { return to_int<float>(v, (RoundingMode)rmode); }
long long ref_rshift_round(long long v, int shift, int rmode) { return RightShiftRound<long long>(v, shift, (RoundingMode)rmode); }
int ref_mbqm(int x, int m, int shift, int rmode) { return MultiplyByQuantizedMultiplier(x, m, shift, (RoundingMode)rmode); }
long long ref_apply_multiplier_rshift(long long v, long long m, long long rshift, int qmode, int rmode, int cv18xx) {
  module::g_cv18xx = cv18xx != 0;
  return applyMultiplierAndRShift(v, m, rshift, (tpu::RequantMode)qmode, (RoundingMode)rmode);
}
}
