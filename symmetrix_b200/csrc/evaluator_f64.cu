// Evaluator<double>: every kernel instantiation of the double path is compiled in this translation unit.
#include "evaluator.cuh"

namespace smx {

std::unique_ptr<EvaluatorBase> make_evaluator_f64(HostModel&& m, int device) {
    return std::make_unique<Evaluator<double>>(std::move(m), device);
}
double measure_fma_peak_f64(int device) { return measure_fma_peak<double>(device); }

}  // namespace smx
