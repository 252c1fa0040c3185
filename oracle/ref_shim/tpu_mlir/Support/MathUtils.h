// Test infrastructure only.  Stands in for the reference's include/tpu_mlir/Support/MathUtils.h (which pulls in MLIR)
// while the reference's lib/Support/Float16.cpp is compiled, where it lies, into the checker library: it supplies the
// RoundingMode enum and RightShiftRound (both cut out of the reference checkout by the build recipe into generated
// include files), and stand-ins for the two other names that file uses.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <math.h>
namespace tpu_mlir {
#include "../../../_ref/mathutils_enum.inc"
#include "../../../_ref/mathutils_rsr.inc"
namespace module {
inline bool isCV18xx() { return false; }  // the BM168x conversion (bm_f32_to_bf16) is the one pinned
}  // namespace module
inline int omp_schedule(int count) { return count > 64 ? count / 64 : 1; }  // only a loop chunk size
}  // namespace tpu_mlir
