// Operator "conv2d_quantized" on TenniS's "gpu" device, over libtennis_b200.so.
//
// The shell (fields, init, infer, run, scratch frame) is ts::base::Conv2DQuantized
// (src/backend/base/base_conv2d_quantized.cpp:13-219); the compute core below takes the place of
// ts::cpu::Conv2DQuantizedCore (src/kernels/cpu/quantized/conv2d_quantized_core.cpp:128-147), composed the way
// the reference composes its GPU convolution (include/kernels/gpu/conv2d.h:11).
#include <backend/base/base_conv2d_quantized.h>
#include <backend/base/base_conv2d_quantized_core.h>
#include <backend/name.h>
#include <core/tensor_builder.h>
#include <global/operator_factory.h>
#include <kernels/gpu/operator_on_gpu.h>

#include <cstring>

#include "b200_common.h"

namespace ts {
    namespace b200 {
        class Conv2DQuantizedCore : public base::Conv2DQuantizedCore {
        public:
            ~Conv2DQuantizedCore() override {
                if (m_plan) tsb_conv2d_i8_plan_destroy(m_plan);
            }

            void conv2d(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                        const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                        std::vector<float> dequantize_scales, Tensor &out, Stack &stack) override {
                (void) stack;
                if (format != FORMAT_NCHW) {
                    TS_LOG_ERROR << "Conv2D_quantized only support NCHW" << eject;
                }
                if (x.dtype() != INT8) {
                    TS_LOG_ERROR << "Conv2D_quantized not support this data type: " << type_str(x.dtype()) << eject;
                }
                const std::string op = "conv2d_quantized";
                auto stream = stream_on_context();
                auto device = out.device();

                tsb_conv_desc desc;
                std::memset(&desc, 0, sizeof(desc));
                desc.n = x.size(0); desc.c = x.size(1); desc.h = x.size(2); desc.w = x.size(3);
                desc.o = w.size(0); desc.kh = w.size(2); desc.kw = w.size(3);
                desc.pad_top = padding.top; desc.pad_bottom = padding.bottom;
                desc.pad_left = padding.left; desc.pad_right = padding.right;
                desc.stride_h = stride.height; desc.stride_w = stride.width;
                desc.dilation_h = dilation.height; desc.dilation_w = dilation.width;
                desc.padding_value = padding_value;
                desc.kernel = TSB_KERNEL_AUTO;

                // Weights are a stack input, constant across runs (src/runtime/program.cpp:91-107): the plan, the
                // packed weights and the device copy of the scales are built on the first run and kept while the
                // geometry and the weight pointer stay the same.
                const void *w_ptr = w.data();
                if (m_plan == nullptr || std::memcmp(&desc, &m_desc, sizeof(desc)) != 0 || w_ptr != m_weights) {
                    if (m_plan) tsb_conv2d_i8_plan_destroy(m_plan);
                    m_plan = nullptr;
                    check(tsb_conv2d_i8_plan_create(&desc, &m_plan), op);
                    m_desc = desc;
                    m_weights = w_ptr;
                    m_workspace_bytes = tsb_conv2d_i8_workspace_bytes(m_plan);
                    m_workspace = Tensor(device, INT8, Shape({int(m_workspace_bytes)}));
                    m_scales = tensor::build(FLOAT32, dequantize_scales).view(device);
                    check(tsb_conv2d_i8_set_weights(m_plan, w.data<int8_t>(), m_workspace.data(), m_workspace_bytes, stream), op);
                }

                tsb_conv_epilogue epilogue;
                std::memset(&epilogue, 0, sizeof(epilogue));
                epilogue.dequantize_scales = m_scales.data<float>();
                epilogue.activation = TSB_ACT_NONE;
                epilogue.out_f32 = out.data<float>();
                epilogue.out_f32_layout = TSB_LAYOUT_NCHW;
                check(tsb_conv2d_i8_run(m_plan, x.data<int8_t>(), TSB_LAYOUT_NCHW, &epilogue, m_workspace.data(),
                                        m_workspace_bytes, stream), op);
            }

        private:
            tsb_conv_plan *m_plan = nullptr;
            tsb_conv_desc m_desc;
            const void *m_weights = nullptr;
            size_t m_workspace_bytes = 0;
            Tensor m_workspace;
            Tensor m_scales;
        };

        using Conv2DQuantized = base::Conv2DWithCore<gpu::OperatorOnGPU<base::Conv2DQuantized>, Conv2DQuantizedCore>;
    }
}

using namespace ts;
using namespace b200;
TS_REGISTER_OPERATOR(Conv2DQuantized, ts::GPU, name::layer::conv2d_quantized())
