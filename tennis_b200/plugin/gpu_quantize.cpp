// Operator "quantize" on TenniS's "gpu" device, over libtennis_b200.so.
//
// Same shell as the CPU operator: attribute parsing, infer() and run() come from ts::base::Quantize
// (src/backend/base/base_quantize.cpp:12-49); only the compute hook differs from
// ts::cpu::Quantize (src/kernels/cpu/quantize.cpp:127-147).
#include <backend/base/base_quantize.h>
#include <backend/name.h>
#include <global/operator_factory.h>
#include <kernels/gpu/operator_on_gpu.h>

#include "b200_common.h"

namespace ts {
    namespace b200 {
        class Quantize : public gpu::OperatorOnGPU<base::Quantize> {
        public:
            using self = Quantize;
            using supper = gpu::OperatorOnGPU<base::Quantize>;

            void quantize(const Tensor &x, std::vector<float> quantize_scales, Tensor &out) override {
                // all tensors live on the GPU, as given by running_memory_device(); the same two input types as the CPU
                // operator's dispatch (src/kernels/cpu/quantize.cpp:130-141) and its error text for the rest
                if (x.dtype() == FLOAT32) {
                    check(tsb_quantize_f32_i8(x.data<float>(), out.data<int8_t>(), int64_t(out.count()),
                                              quantize_scales.data(), int(quantize_scales.size()), stream_on_context()),
                          this->op());
                } else if (x.dtype() == FLOAT64) {
                    check(tsb_quantize_f64_i8(x.data<double>(), out.data<int8_t>(), int64_t(out.count()),
                                              quantize_scales.data(), int(quantize_scales.size()), stream_on_context()),
                          this->op());
                } else {
                    TS_LOG_ERROR << this->op() << " not support this data type: " << x.dtype() << eject;
                }
            }
        };
    }
}

using namespace ts;
using namespace b200;
TS_REGISTER_OPERATOR(Quantize, ts::GPU, name::layer::quantize())
