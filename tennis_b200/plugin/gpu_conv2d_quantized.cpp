// Operator "conv2d_quantized" on TenniS's "gpu" device, over libtennis_b200.so, and the compile-time rewrite that
// folds the add_bias and activation after it into the same launch.
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
#include <backend/common_function.h>
#include <compiler/option/zipper_option.h>
#include <module/menu.h>

#include <atomic>

#include <cstring>

#include "b200_common.h"

namespace ts {
    namespace b200 {
        class Conv2DQuantizedCore : public base::Conv2DQuantizedCore {
        public:
            ~Conv2DQuantizedCore() override {
                // the last run's status word has not been looked at yet: wait for it and at least say so (a destructor
                // cannot eject)
                if (m_status_pending && m_status_event && cudaEventSynchronize(m_status_event) == cudaSuccess &&
                    m_status_host && *m_status_host != 0 && tsb_conv2d_i8_status_decode(*m_status_host) != TSB_OK) {
                    TS_LOG_ERROR << "conv2d_quantized: " << tsb_last_error();
                }
                if (m_status_event) cudaEventDestroy(m_status_event);
                if (m_status_host) cudaFreeHost(m_status_host);
                if (m_plan) tsb_conv2d_i8_plan_destroy(m_plan);
            }

            // Failure detection without a synchronisation on the workbench's stream: every run enqueues a 4-byte copy
            // of the kernel's status word into pinned memory and records an event; the NEXT run (or the destructor)
            // looks at the word once the event has passed.  A kernel that gave up on one of its bounded waits
            // therefore ejects, with the name of the wait, instead of handing on invalid output silently.
            void check_previous_run(cudaStream_t stream, const std::string &op) {
                if (!m_status_pending || cudaEventQuery(m_status_event) != cudaSuccess) return;
                m_status_pending = false;
                if (*m_status_host == 0) return;
                const int word = *m_status_host;
                *m_status_host = 0;
                if (m_plan) cudaMemsetAsync(m_workspace.data(), 0, sizeof(int), stream);   // reported once, then cleared
                check(tsb_conv2d_i8_status_decode(word), op);
            }

            void note_run(cudaStream_t stream, const std::string &op) {
                if (tsb_conv2d_i8_kernel(m_plan) != TSB_KERNEL_TCGEN05) return;
                if (!m_status_host) {
                    if (cudaMallocHost(reinterpret_cast<void **>(&m_status_host), sizeof(int)) != cudaSuccess) { m_status_host = nullptr; return; }
                    *m_status_host = 0;
                    if (cudaEventCreateWithFlags(&m_status_event, cudaEventDisableTiming) != cudaSuccess) { m_status_event = nullptr; return; }
                }
                if (!m_status_event) return;
                check(tsb_conv2d_i8_status_async(m_plan, m_workspace.data(), m_status_host, stream), op);
                if (cudaEventRecord(m_status_event, stream) == cudaSuccess) m_status_pending = true;
            }

            void conv2d(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                        const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                        std::vector<float> dequantize_scales, Tensor &out, Stack &stack) override {
                conv2d_fused(x, padding, padding_value, w, stride, dilation, format, dequantize_scales, out, stack, nullptr,
                             TSB_ACT_NONE, 0.0f);
            }

            // conv2d_quantized -> add_bias -> relu | leaky_relu in one launch (bias: device pointer or null)
            void conv2d_fused(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                              const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                              std::vector<float> dequantize_scales, Tensor &out, Stack &stack, const float *bias,
                              int activation, float leaky, const std::vector<float> *quantize_scales = nullptr) {
                (void) stack;
                if (format != FORMAT_NCHW) {
                    TS_LOG_ERROR << "Conv2D_quantized only support NCHW" << eject;
                }
                // quantize_scales given: x is the fp32 tensor the folded quantize operator would have read
                if (quantize_scales == nullptr && x.dtype() != INT8) {
                    TS_LOG_ERROR << "Conv2D_quantized not support this data type: " << type_str(x.dtype()) << eject;
                }
                if (quantize_scales != nullptr && x.dtype() != FLOAT32) {
                    TS_LOG_ERROR << "quantize not support data type(" << x.dtype() << "): " << type_str(x.dtype()) << eject;
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
                check_previous_run(stream, op);
                if (m_plan == nullptr || std::memcmp(&desc, &m_desc, sizeof(desc)) != 0 || w_ptr != m_weights) {
                    if (m_plan) tsb_conv2d_i8_plan_destroy(m_plan);
                    m_plan = nullptr;
                    m_status_pending = false;
                    check(tsb_conv2d_i8_plan_create(&desc, &m_plan), op);
                    if (tsb_conv2d_i8_kernel(m_plan) != TSB_KERNEL_TCGEN05) {
                        // the CUDA-core kernel is a correctness path (non-zero padding_value, filters beyond the
                        // tensor-map limits) and many times slower: say so once per plan
                        char text[256];
                        if (tsb_conv2d_i8_plan_describe(m_plan, text, sizeof(text)) > 0) {
                            TS_LOG_INFO << op << ": this layer runs on the CUDA-core kernel, not on the tensor cores: " << text;
                        }
                    }
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
                epilogue.bias = bias;
                epilogue.activation = activation;
                epilogue.leaky_scale = leaky;
                epilogue.out_f32 = out.data<float>();
                epilogue.out_f32_layout = TSB_LAYOUT_NCHW;
                if (quantize_scales != nullptr) {
                    // fp32 NCHW -> the plan's own staged int8 layout, then the convolution reads it in place
                    check(tsb_conv2d_i8_quantize_input(m_plan, x.data<float>(), quantize_scales->data(), int(quantize_scales->size()),
                                                       m_workspace.data(), m_workspace_bytes, stream), op);
                    check(tsb_conv2d_i8_run(m_plan, nullptr, TSB_LAYOUT_STAGED, &epilogue, m_workspace.data(), m_workspace_bytes,
                                            stream), op);
                    note_run(stream, op);
                    return;
                }
                check(tsb_conv2d_i8_run(m_plan, x.data<int8_t>(), TSB_LAYOUT_NCHW, &epilogue, m_workspace.data(),
                                        m_workspace_bytes, stream), op);
                note_run(stream, op);
            }

        private:
            tsb_conv_plan *m_plan = nullptr;
            tsb_conv_desc m_desc;
            const void *m_weights = nullptr;
            size_t m_workspace_bytes = 0;
            Tensor m_workspace;
            Tensor m_scales;
            int *m_status_host = nullptr;          // pinned: the status word of the last run lands here
            cudaEvent_t m_status_event = nullptr;
            bool m_status_pending = false;
        };

        using Conv2DQuantized = base::Conv2DWithCore<gpu::OperatorOnGPU<base::Conv2DQuantized>, Conv2DQuantizedCore>;

        // "b200_conv2d_quantized_fused": conv2d_quantized with the add_bias and relu / leaky_relu that follow it folded
        // into the convolution's epilogue.  Same inputs (x int8, w int8), attributes and fp32 NCHW output as
        // conv2d_quantized, plus the bias (a constant of the graph) and the activation as attributes.  Never written by
        // hand: the zipper option below puts it into the graph when a module is compiled for the gpu device.
        class Conv2DQuantizedFused : public gpu::OperatorOnGPU<base::Conv2DQuantized> {
        public:
            using self = Conv2DQuantizedFused;
            using supper = gpu::OperatorOnGPU<base::Conv2DQuantized>;

            Conv2DQuantizedFused() {
                field(fused_bias(), OPTIONAL);
                field(fused_activation(), OPTIONAL, tensor::from<int32_t>(TSB_ACT_NONE));
                field(fused_leaky(), OPTIONAL, tensor::from<float>(0.0f));
                field(fused_quantize_scale(), OPTIONAL);
            }

            static const std::string &op_name() { static const std::string n = "b200_conv2d_quantized_fused"; return n; }
            static const std::string &fused_bias() { static const std::string n = "b200_bias"; return n; }
            static const std::string &fused_activation() { static const std::string n = "b200_activation"; return n; }
            static const std::string &fused_leaky() { static const std::string n = "b200_leaky_scale"; return n; }
            // present when the quantize operator in front of the convolution was folded in: the operator's first input
            // is then the fp32 tensor, and this is that operator's quantize_scale attribute (one scale per sample)
            static const std::string &fused_quantize_scale() { static const std::string n = "b200_quantize_scale"; return n; }

            void init() override {
                supper::init();
                m_activation = tensor::to_int(get(fused_activation()));
                m_leaky = tensor::to_float(get(fused_leaky()));
                m_has_bias = has(fused_bias());
                if (m_has_bias) m_bias_host = tensor::cast(FLOAT32, get(fused_bias()));
                m_folded_quantize = has(fused_quantize_scale());
                if (m_folded_quantize) {
                    m_quantize_scales = tensor::array::to_float(get(fused_quantize_scale()));
                    // the shell keeps its parsed attributes private; the folded path needs them again (the shell's init()
                    // above has already validated them: src/backend/base/base_conv2d_quantized.cpp:36-117)
                    if (tensor::to_string(get(name::format)) != name::NCHW) {
                        TS_LOG_ERROR << op_name() << " folds quantize only for format NCHW" << eject;
                    }
                    auto padding = tensor::cast(INT32, get(name::padding));
                    auto stride = tensor::cast(INT32, get(name::stride));
                    auto dilation = tensor::cast(INT32, has(name::dilation) ? get(name::dilation) : get(name::typo::dialations));
                    m_padding = Padding2D(padding.data<int32_t>(4), padding.data<int32_t>(5), padding.data<int32_t>(6), padding.data<int32_t>(7));
                    m_stride = Stride2D(stride.data<int32_t>(2), stride.data<int32_t>(3));
                    m_dilation = Dilation2D(dilation.data<int32_t>(2), dilation.data<int32_t>(3));
                    m_padding_value = tensor::to_float(get(name::padding_value));
                    m_dequantize_scales = tensor::array::to_float(get(name::dequantize_scales));
                }
            }

            // With the quantize folded in, the first input is fp32: the shell's infer/run (which insist on int8) are
            // replaced by the same steps on the fp32 tensor.
            int infer(Stack &stack, std::vector<Tensor::Prototype> &output) override {
                if (!m_folded_quantize) return supper::infer(stack, output);
                TS_AUTO_CHECK(stack.size() == 2);
                auto x = stack[0];
                auto w = stack[1];
                TS_AUTO_CHECK(x.dims() == 4);
                TS_AUTO_CHECK(w.dims() == 4);
                TS_AUTO_CHECK(x.dtype() == FLOAT32);
                TS_AUTO_CHECK(w.dtype() == INT8);
                TS_AUTO_CHECK(w.size(1) == x.size(1));
                TS_AUTO_CHECK(int(m_quantize_scales.size()) == x.size(0));      // base_quantize.cpp:26
                TS_AUTO_CHECK(int(m_dequantize_scales.size()) == w.size(0));
                Size2D y = conv2d_forward(Size2D(x.size(2), x.size(3)), m_padding, Size2D(w.size(2), w.size(3)), m_stride, m_dilation);
                output.resize(1);
                output[0] = Tensor::Prototype(FLOAT32, {x.size(0), w.size(0), y.height, y.width});
                return 1;
            }

            int run(Stack &stack) override {
                if (!m_folded_quantize) return supper::run(stack);
                std::vector<Tensor::Prototype> protos;
                infer(stack, protos);
                auto memory_device = running_memory_device();
                Tensor x = stack[0].view(memory_device);
                Tensor w = stack[1].view(memory_device);
                Tensor out = *stack.push(protos[0], memory_device);
                run_core(x, m_padding, m_padding_value, w, m_stride, m_dilation, FORMAT_NCHW, m_dequantize_scales, out, stack,
                         &m_quantize_scales);
                return 1;
            }

            void conv2d(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                        const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                        std::vector<float> dequantize_scales, Tensor &out, Stack &stack) override {
                run_core(x, padding, padding_value, w, stride, dilation, format, dequantize_scales, out, stack, nullptr);
            }

            void run_core(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                          const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                          const std::vector<float> &dequantize_scales, Tensor &out, Stack &stack,
                          const std::vector<float> *quantize_scales) {
                const float *bias = nullptr;
                if (m_has_bias) {
                    if (m_bias_host.count() != w.size(0)) {
                        TS_LOG_ERROR << op_name() << ": bias has " << m_bias_host.count() << " entries for " << w.size(0)
                                     << " output channels" << eject;
                    }
                    if (m_bias_device.count() != m_bias_host.count()) m_bias_device = m_bias_host.view(out.device()).clone();
                    bias = m_bias_device.data<float>();
                }
                m_core.conv2d_fused(x, padding, padding_value, w, stride, dilation, format, dequantize_scales, out, stack, bias,
                                    m_activation, m_leaky, quantize_scales);
                fused_runs().fetch_add(1);
                if (quantize_scales) folded_quantize_runs().fetch_add(1);
            }

            static std::atomic<long> &fused_runs() { static std::atomic<long> n(0); return n; }
            static std::atomic<long> &folded_quantize_runs() { static std::atomic<long> n(0); return n; }

        private:
            b200::Conv2DQuantizedCore m_core;   // the class above, not the base interface of the same name
            int m_activation = TSB_ACT_NONE;
            float m_leaky = 0.0f;
            bool m_has_bias = false;
            Tensor m_bias_host, m_bias_device;
            bool m_folded_quantize = false;
            std::vector<float> m_quantize_scales, m_dequantize_scales;
            Padding2D m_padding;
            Stride2D m_stride;
            Dilation2D m_dilation;
            float m_padding_value = 0.0f;
        };

        // Graph rewrite at compile time (src/compiler/zipper.cpp:20-62 visits every node of the module once):
        //   relu | leaky_relu ( add_bias ( conv2d_quantized(x, w), <const bias> ) )  ->  b200_conv2d_quantized_fused(x, w)
        //   ... and with x = quantize(x32) read by nothing else                       ->  b200_conv2d_quantized_fused(x32, w)
        // on the gpu device, when the bias is a constant over the channel dimension of an NCHW tensor and neither
        // intermediate result has another consumer.  The fused node keeps the name of the activation node, so the
        // module's outputs are found as before.
        class ConvBiasActivationZipper : public ZipperOption {
        public:
            bool zip(const ComputingDevice &device, Node node, Node &zipped_node) const override {
                if (device.type() != GPU) return false;
                const Bubble &act = node.bubble();
                int activation;
                float leaky = 0.0f;
                if (act.op() == name::layer::relu()) activation = TSB_ACT_RELU;
                else if (act.op() == "leaky_relu") {   // src/backend/base/base_leaky_relu.cpp registers it under this name
                    activation = TSB_ACT_LEAKY_RELU;
                    if (!act.has(name::scale)) return false;
                    leaky = tensor::to_float(act.get(name::scale));
                } else return false;
                auto act_inputs = node.inputs();
                if (act_inputs.size() != 1) return false;
                Node biased = act_inputs[0];
                if (biased.bubble().op() != name::layer::add_bias() || biased.outputs().size() != 1) return false;
                if (biased.bubble().has(name::format)) {
                    if (tensor::to_string(biased.bubble().get(name::format)) != name::NCHW) return false;
                } else if (biased.bubble().has(name::dim)) {
                    if (tensor::to_int(biased.bubble().get(name::dim)) != 1) return false;
                } else return false;
                auto biased_inputs = biased.inputs();
                if (biased_inputs.size() != 2) return false;
                Node conv = biased_inputs[0], bias = biased_inputs[1];
                if (conv.bubble().op() != name::layer::conv2d_quantized() || conv.outputs().size() != 1) return false;
                if (bias.bubble().op() != Bubble::Const || !bias.bubble().has(name::value)) return false;
                if (conv.bubble().has(name::format) && tensor::to_string(conv.bubble().get(name::format)) != name::NCHW) return false;

                // quantize(x) in front of the convolution, read by nothing else: the fused operator takes x itself and
                // quantizes it straight into the layout its kernel reads
                std::vector<Node> fused_inputs = conv.inputs();
                if (fused_inputs.size() != 2) return false;
                Tensor folded_scales;
                {
                    Node q = fused_inputs[0];
                    if (q.bubble().op() == name::layer::quantize() && q.outputs().size() == 1 && q.inputs().size() == 1 &&
                        q.bubble().has(name::quantize_scale)) {
                        folded_scales = tensor::cast(FLOAT32, q.bubble().get(name::quantize_scale));
                        fused_inputs[0] = q.input(0);
                    }
                }
                Node fused = bubble::op(act.name(), Conv2DQuantizedFused::op_name(), fused_inputs);
                for (auto &param : conv.bubble().params()) {
                    if (!param.first.empty() && param.first[0] == Bubble::retention_param_sign) continue;   // #name, #op, ...
                    fused.bubble().set(param.first, param.second);
                }
                fused.bubble().set(Conv2DQuantizedFused::fused_bias(), tensor::cast(FLOAT32, bias.bubble().get(name::value)));
                fused.bubble().set(Conv2DQuantizedFused::fused_activation(), tensor::from<int32_t>(activation));
                fused.bubble().set(Conv2DQuantizedFused::fused_leaky(), tensor::from<float>(leaky));
                if (!folded_scales.empty()) fused.bubble().set(Conv2DQuantizedFused::fused_quantize_scale(), folded_scales);
                zipped_node = fused;
                return true;
            }
        };
    }
}

// how many times the fused operator has run in this process (drop-in tests read it)
extern "C" __attribute__((visibility("default"))) long tsb_plugin_fused_runs() {
    return ts::b200::Conv2DQuantizedFused::fused_runs().load();
}
// ... and how many of those runs had the quantize operator folded in
extern "C" __attribute__((visibility("default"))) long tsb_plugin_folded_quantize_runs() {
    return ts::b200::Conv2DQuantizedFused::folded_quantize_runs().load();
}

using namespace ts;
using namespace b200;
TS_REGISTER_OPERATOR(Conv2DQuantized, ts::GPU, name::layer::conv2d_quantized())
TS_REGISTER_OPERATOR(Conv2DQuantizedFused, ts::GPU, Conv2DQuantizedFused::op_name())
TS_REGISTER_ZIPPER_OPTION(ConvBiasActivationZipper)
