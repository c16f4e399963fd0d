// Evaluator<float>: every kernel instantiation of the float path is compiled in this translation unit.
#include "evaluator.cuh"

namespace smx {

std::unique_ptr<EvaluatorBase> make_evaluator_f32(HostModel&& m, int device) {
    return std::make_unique<Evaluator<float>>(std::move(m), device);
}
double measure_fma_peak_f32(int device) { return measure_fma_peak<float>(device); }

}  // namespace smx
