// Test infrastructure only: C entry points to the reference's own float conversions (lib/Support/Float16.cpp,
// compiled from the reference checkout together with this file).
#include <cstdint>
namespace tpu_mlir {
uint16_t f32_to_bf16(float src, bool is_tpu);
float bf16_to_f32(uint16_t src);
uint16_t f32_to_f16(float src);
float f16_to_f32(uint16_t src);
}  // namespace tpu_mlir
extern "C" {
unsigned ref_f32_to_bf16(float v) { return tpu_mlir::f32_to_bf16(v, true); }
float ref_bf16_to_f32(unsigned b) { return tpu_mlir::bf16_to_f32((uint16_t)b); }
unsigned ref_f32_to_f16(float v) { return tpu_mlir::f32_to_f16(v); }
float ref_f16_to_f32(unsigned b) { return tpu_mlir::f16_to_f32((uint16_t)b); }
}
