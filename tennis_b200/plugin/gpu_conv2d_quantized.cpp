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
#include <runtime/inferer.h>

#include <atomic>
#include <chrono>
#include <memory>

#include <cstring>

#include "b200_common.h"

namespace ts {
    namespace b200 {
        class Conv2DQuantizedCore : public base::Conv2DQuantizedCore {
        public:
            ~Conv2DQuantizedCore() override {
                // a time-out of the last runs that nobody has looked at yet: let the device finish and at least say so (a
                // destructor cannot eject)
                if (m_status_host && m_ran) {
                    cudaDeviceSynchronize();
                    const int word = *static_cast<volatile int *>(m_status_host);
                    if (word != 0 && tsb_conv2d_i8_status_decode(word) != TSB_OK) TS_LOG_ERROR << "conv2d_quantized: " << tsb_last_error();
                }
                if (m_plan) tsb_conv2d_i8_plan_destroy(m_plan);
                if (m_status_host) cudaFreeHost(m_status_host);
            }

            // Failure detection without a synchronisation, a copy or an event on the workbench's stream: the plan's kernels
            // report a bounded wait that gave up into a word of MAPPED pinned host memory (nothing is written there
            // otherwise), and every run looks at that word as plain memory before it launches.  A kernel that gave up
            // therefore makes the next run (or the destructor) eject with the name of the wait, instead of handing on
            // invalid output silently.
            void check_previous_run(const std::string &op) {
                if (!m_status_host) return;
                const int word = *static_cast<volatile int *>(m_status_host);
                if (word == 0) return;
                *static_cast<volatile int *>(m_status_host) = 0;                                  // reported once, then cleared
                check(tsb_conv2d_i8_status_decode(word), op);
            }

            void bind_status_word(const std::string &op) {
                if (tsb_conv2d_i8_kernel(m_plan) != TSB_KERNEL_TCGEN05) return;
                if (!m_status_host) {
                    void *host = nullptr;
                    if (cudaHostAlloc(&host, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return;   // (the workspace word stays in use)
                    m_status_host = static_cast<int *>(host);
                    *m_status_host = 0;
                }
                void *dev = nullptr;
                if (cudaHostGetDevicePointer(&dev, m_status_host, 0) != cudaSuccess) return;
                check(tsb_conv2d_i8_set_status_word(m_plan, static_cast<int *>(dev)), op);
            }

            void conv2d(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                        const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                        std::vector<float> dequantize_scales, Tensor &out, Stack &stack) override {
                conv2d_fused(x, padding, padding_value, w, stride, dilation, format, dequantize_scales, out, stack, nullptr,
                             TSB_ACT_NONE, 0.0f);
            }

            // What the compile-time rewrite can ask of one launch beyond bias and activation.
            struct Extras {
                const std::vector<float> *quantize_scales = nullptr;   // x is fp32 NCHW: quantize it into the staged layout first
                bool x_nhwc = false;                                   // x is int8 NHWC_PAD [N,H,W,Cp], written by another fused node
                const std::vector<float> *out_scales = nullptr;        // out is int8 NHWC_PAD [N,OH,OW,Cp]: the consumer's quantize
                const float *residual = nullptr;                       // fp32 NCHW shortcut (operator "add"), device pointer
                bool residual_after = false;                           // added after the activation instead of before it
            };

            // conv2d_quantized -> add_bias -> relu | leaky_relu in one launch (bias: device pointer or null)
            void conv2d_fused(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                              const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                              std::vector<float> dequantize_scales, Tensor &out, Stack &stack, const float *bias,
                              int activation, float leaky, const std::vector<float> *quantize_scales = nullptr,
                              const Extras *extras = nullptr) {
                (void) stack;
                Extras ex;
                if (extras) ex = *extras;
                if (quantize_scales) ex.quantize_scales = quantize_scales;
                quantize_scales = ex.quantize_scales;
                if (format != FORMAT_NCHW) {
                    TS_LOG_ERROR << "Conv2D_quantized only support NCHW" << eject;
                }
                // quantize_scales given: x is the fp32 tensor the folded quantize operator would have read
                if (ex.x_nhwc && (x.dtype() != INT8 || x.size(3) != tsb_padded_channels(w.size(1)))) {
                    TS_LOG_ERROR << "b200_conv2d_quantized_fused: the int8 NHWC_PAD input does not match the weights" << eject;
                }
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
                if (ex.x_nhwc) { desc.n = x.size(0); desc.c = w.size(1); desc.h = x.size(1); desc.w = x.size(2); }
                else { desc.n = x.size(0); desc.c = x.size(1); desc.h = x.size(2); desc.w = x.size(3); }
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
                check_previous_run(op);
                if (m_plan == nullptr || std::memcmp(&desc, &m_desc, sizeof(desc)) != 0 || w_ptr != m_weights) {
                    if (m_plan) tsb_conv2d_i8_plan_destroy(m_plan);
                    m_plan = nullptr;
                    check(tsb_conv2d_i8_plan_create(&desc, &m_plan), op);
                    bind_status_word(op);
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
                if (ex.out_scales != nullptr) {
                    // int8 NHWC_PAD for the next fused convolution: the requantize of the epilogue with that layer's scales
                    epilogue.out_i8 = out.data<int8_t>();
                    epilogue.out_i8_layout = TSB_LAYOUT_NHWC_PAD;
                    epilogue.requant_scales_host = ex.out_scales->data();
                    epilogue.n_requant_scales = int(ex.out_scales->size());
                } else {
                    epilogue.out_f32 = out.data<float>();
                    epilogue.out_f32_layout = TSB_LAYOUT_NCHW;
                }
                epilogue.residual = ex.residual;
                epilogue.residual_after_activation = ex.residual_after ? 1 : 0;
                if (ex.x_nhwc) {
                    check(tsb_conv2d_i8_run(m_plan, x.data<int8_t>(), TSB_LAYOUT_NHWC_PAD, &epilogue, m_workspace.data(),
                                            m_workspace_bytes, stream), op);
                    m_ran = true;
                    return;
                }
                if (quantize_scales != nullptr) {
                    // fp32 NCHW -> the plan's own staged int8 layout, then the convolution reads it in place
                    check(tsb_conv2d_i8_quantize_input(m_plan, x.data<float>(), quantize_scales->data(), int(quantize_scales->size()),
                                                       m_workspace.data(), m_workspace_bytes, stream), op);
                    check(tsb_conv2d_i8_run(m_plan, nullptr, TSB_LAYOUT_STAGED, &epilogue, m_workspace.data(), m_workspace_bytes,
                                            stream), op);
                    m_ran = true;
                    return;
                }
                check(tsb_conv2d_i8_run(m_plan, x.data<int8_t>(), TSB_LAYOUT_NCHW, &epilogue, m_workspace.data(),
                                        m_workspace_bytes, stream), op);
                m_ran = true;
            }

        private:
            tsb_conv_plan *m_plan = nullptr;
            tsb_conv_desc m_desc;
            const void *m_weights = nullptr;
            size_t m_workspace_bytes = 0;
            Tensor m_workspace;
            Tensor m_scales;
            int *m_status_host = nullptr;          // mapped pinned memory: the plan's kernels report a wait that gave up here
            bool m_ran = false;
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
                field(fused_in_nhwc(), OPTIONAL, tensor::from<int32_t>(0));
                field(fused_out_scale(), OPTIONAL);
                field(fused_residual(), OPTIONAL, tensor::from<int32_t>(0));
            }

            static const std::string &op_name() { static const std::string n = "b200_conv2d_quantized_fused"; return n; }
            static const std::string &fused_bias() { static const std::string n = "b200_bias"; return n; }
            static const std::string &fused_activation() { static const std::string n = "b200_activation"; return n; }
            static const std::string &fused_leaky() { static const std::string n = "b200_leaky_scale"; return n; }
            // present when the quantize operator in front of the convolution was folded in: the operator's first input
            // is then the fp32 tensor, and this is that operator's quantize_scale attribute (one scale per sample)
            static const std::string &fused_quantize_scale() { static const std::string n = "b200_quantize_scale"; return n; }
            // 1: the first input is the int8 NHWC_PAD tensor [N,H,W,Cp] another fused node wrote (the quantize between the
            // two layers was folded into that node's epilogue)
            static const std::string &fused_in_nhwc() { static const std::string n = "b200_input_nhwc"; return n; }
            // present: the output is int8 NHWC_PAD [N,OH,OW,Cp], requantized with these scales (the quantize_scale attribute of
            // the quantize operator that followed this layer and fed the next convolution alone)
            static const std::string &fused_out_scale() { static const std::string n = "b200_output_quantize_scale"; return n; }
            // 1: a third input, fp32 NCHW of the output's shape, is added between add_bias and the activation (a ResNet
            // shortcut); 2: it is added after the activation (a Darknet shortcut)
            static const std::string &fused_residual() { static const std::string n = "b200_residual"; return n; }

            void init() override {
                supper::init();
                m_activation = tensor::to_int(get(fused_activation()));
                m_leaky = tensor::to_float(get(fused_leaky()));
                m_has_bias = has(fused_bias());
                if (m_has_bias) m_bias_host = tensor::cast(FLOAT32, get(fused_bias()));
                m_folded_quantize = has(fused_quantize_scale());
                m_in_nhwc = tensor::to_int(get(fused_in_nhwc())) != 0;
                m_residual = tensor::to_int(get(fused_residual()));
                m_has_out_scale = has(fused_out_scale());
                if (m_has_out_scale) m_out_scales = tensor::array::to_float(get(fused_out_scale()));
                m_extended = m_folded_quantize || m_in_nhwc || m_residual != 0 || m_has_out_scale;
                if (m_extended) {
                    if (m_folded_quantize) m_quantize_scales = tensor::array::to_float(get(fused_quantize_scale()));
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
                if (!m_extended) return supper::infer(stack, output);
                TS_AUTO_CHECK(stack.size() == (m_residual ? 3 : 2));
                auto x = stack[0];
                auto w = stack[1];
                TS_AUTO_CHECK(x.dims() == 4);
                TS_AUTO_CHECK(w.dims() == 4);
                TS_AUTO_CHECK(w.dtype() == INT8);
                int height, width;
                if (m_in_nhwc) {
                    TS_AUTO_CHECK(x.dtype() == INT8);
                    TS_AUTO_CHECK(x.size(3) == tsb_padded_channels(w.size(1)));
                    height = x.size(1); width = x.size(2);
                } else {
                    TS_AUTO_CHECK(x.dtype() == (m_folded_quantize ? FLOAT32 : INT8));
                    TS_AUTO_CHECK(w.size(1) == x.size(1));
                    height = x.size(2); width = x.size(3);
                }
                if (m_folded_quantize) TS_AUTO_CHECK(int(m_quantize_scales.size()) == x.size(0));      // base_quantize.cpp:26
                if (m_has_out_scale) TS_AUTO_CHECK(int(m_out_scales.size()) == x.size(0));
                TS_AUTO_CHECK(int(m_dequantize_scales.size()) == w.size(0));
                Size2D y = conv2d_forward(Size2D(height, width), m_padding, Size2D(w.size(2), w.size(3)), m_stride, m_dilation);
                Shape y_shape = {x.size(0), w.size(0), y.height, y.width};
                DTYPE y_dtype = FLOAT32;
                if (m_residual && !shortcut_fits(stack[2], y_shape)) {
                    // operator "add" broadcasts and up-casts (src/backend/base/element_wise_reduce.cpp:21-138): such a
                    // shortcut goes through the device's own add operator after the convolution, see run()
                    std::vector<Tensor::Prototype> sum;
                    stack.push(Tensor::Prototype(FLOAT32, y_shape), MemoryDevice(CPU));
                    stack.push(stack[2]);
                    InferOperator(reference_add(), stack, 2, sum);      // takes its two arguments off the stack
                    TS_AUTO_CHECK(sum.size() == 1);
                    y_shape = sum[0].sizes();
                    y_dtype = sum[0].dtype();
                }
                output.resize(1);
                if (m_has_out_scale) {
                    TS_AUTO_CHECK(y_shape.size() == 4 && y_dtype == FLOAT32);
                    output[0] = Tensor::Prototype(INT8, {y_shape[0], y_shape[2], y_shape[3], tsb_padded_channels(y_shape[1])});
                } else {
                    output[0] = Tensor::Prototype(y_dtype, y_shape);
                }
                return 1;
            }

            // the shortcut can go into the convolution's epilogue: fp32 and of the convolution's own output shape
            static bool shortcut_fits(const Tensor &r, const Shape &y_shape) {
                return r.dtype() == FLOAT32 && r.has_shape(y_shape);
            }

            // host time spent inside run() of this operator, summed over the process (what the runtime around it adds is the
            // rest of a pass: the drop-in tests and the benchmark read both)
            struct HostClock {
                std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
                ~HostClock() {
                    host_ns().fetch_add(std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count());
                }
            };
            static std::atomic<long long> &host_ns() { static std::atomic<long long> n(0); return n; }

            int run(Stack &stack) override {
                HostClock clock;
                if (!m_extended) return supper::run(stack);
                std::vector<Tensor::Prototype> protos;
                infer(stack, protos);
                auto memory_device = running_memory_device();
                Tensor x = stack[0].view(memory_device);
                Tensor w = stack[1].view(memory_device);
                b200::Conv2DQuantizedCore::Extras extras;
                extras.quantize_scales = m_folded_quantize ? &m_quantize_scales : nullptr;
                extras.x_nhwc = m_in_nhwc;
                const int height = m_in_nhwc ? x.size(1) : x.size(2), width = m_in_nhwc ? x.size(2) : x.size(3);
                Size2D y = conv2d_forward(Size2D(height, width), m_padding, Size2D(w.size(2), w.size(3)), m_stride, m_dilation);
                const Shape y_shape = {x.size(0), w.size(0), y.height, y.width};
                if (m_residual && !shortcut_fits(stack[2], y_shape)) return run_with_reference_add(stack, x, w, y_shape, protos[0], extras);
                Tensor shortcut;
                if (m_residual) shortcut = stack[2].view(memory_device);
                Tensor out = *stack.push(protos[0], memory_device);
                extras.out_scales = m_has_out_scale ? &m_out_scales : nullptr;
                extras.residual = m_residual ? shortcut.data<float>() : nullptr;
                extras.residual_after = m_residual == 2;
                run_core(x, m_padding, m_padding_value, w, m_stride, m_dilation, FORMAT_NCHW, m_dequantize_scales, out, stack,
                         &extras, m_activation);
                return 1;
            }

            // A shortcut the epilogue cannot take (another shape: "add" broadcasts; another type: it up-casts).  The graph
            // was rewritten before any shape was known (the compiler strips "#shape" from the module's inputs), so the
            // decision falls here, per run: the convolution with its bias (and the activation, where the shortcut comes
            // after it) runs fused, then the gpu device's own add -- and activation -- operators finish the layer.
            int run_with_reference_add(Stack &stack, const Tensor &x, const Tensor &w, const Shape &y_shape,
                                       const Tensor::Prototype &result, b200::Conv2DQuantizedCore::Extras extras) {
                auto memory_device = running_memory_device();
                Tensor conv_out = *stack.push(Tensor::Prototype(FLOAT32, y_shape), memory_device);
                run_core(x, m_padding, m_padding_value, w, m_stride, m_dilation, FORMAT_NCHW, m_dequantize_scales, conv_out, stack,
                         &extras, m_residual == 2 ? m_activation : TSB_ACT_NONE);
                stack.push(stack[2]);
                RunOperator(reference_add(), stack, 2);
                if (m_residual == 1 && m_activation != TSB_ACT_NONE) RunOperator(reference_activation(), stack, 1);
                reference_add_runs().fetch_add(1);
                if (!m_has_out_scale) return 1;
                Tensor sum = stack[-1].view(memory_device);
                Tensor out = *stack.push(result, memory_device);
                check(tsb_quantize_f32_nchw_to_nhwc(sum.data<float>(), out.data<int8_t>(), sum.size(0), sum.size(1), sum.size(2),
                                                    sum.size(3), m_out_scales.data(), int(m_out_scales.size()), stream_on_context()),
                      op_name());
                return 1;
            }

            Operator::shared reference_add() {
                if (!m_add) {
                    m_add = OperatorCreator::Create(GPU, name::layer::add(), false);
                    m_add->set(Bubble::RetentionParam::op, tensor::from(name::layer::add()));
                    m_add->set(Bubble::RetentionParam::name, tensor::from(name() + ".add"));
                    m_add->init();
                }
                return m_add;
            }

            Operator::shared reference_activation() {
                if (!m_act) {
                    const std::string act = m_activation == TSB_ACT_RELU ? name::layer::relu() : std::string("leaky_relu");
                    m_act = OperatorCreator::Create(GPU, act, false);
                    m_act->set(Bubble::RetentionParam::op, tensor::from(act));
                    m_act->set(Bubble::RetentionParam::name, tensor::from(name() + ".activation"));
                    if (m_activation == TSB_ACT_LEAKY_RELU) m_act->set(name::scale, tensor::from<float>(m_leaky));
                    m_act->init();
                }
                return m_act;
            }

            void conv2d(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                        const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                        std::vector<float> dequantize_scales, Tensor &out, Stack &stack) override {
                run_core(x, padding, padding_value, w, stride, dilation, format, dequantize_scales, out, stack, nullptr, m_activation);
            }

            void run_core(const Tensor &x, const Padding2D &padding, float padding_value, const Tensor &w,
                          const Stride2D &stride, const Dilation2D &dilation, Conv2DFormat format,
                          const std::vector<float> &dequantize_scales, Tensor &out, Stack &stack,
                          const b200::Conv2DQuantizedCore::Extras *extras, int activation) {
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
                                    activation, m_leaky, nullptr, extras);
                fused_runs().fetch_add(1);
                if (extras && extras->quantize_scales) folded_quantize_runs().fetch_add(1);
                if (extras && extras->x_nhwc) int8_handover_runs().fetch_add(1);
                if (extras && extras->residual) residual_runs().fetch_add(1);
            }

            static std::atomic<long> &fused_runs() { static std::atomic<long> n(0); return n; }
            static std::atomic<long> &folded_quantize_runs() { static std::atomic<long> n(0); return n; }
            static std::atomic<long> &int8_handover_runs() { static std::atomic<long> n(0); return n; }
            static std::atomic<long> &residual_runs() { static std::atomic<long> n(0); return n; }
            static std::atomic<long> &reference_add_runs() { static std::atomic<long> n(0); return n; }

        private:
            b200::Conv2DQuantizedCore m_core;   // the class above, not the base interface of the same name
            int m_activation = TSB_ACT_NONE;
            float m_leaky = 0.0f;
            bool m_has_bias = false;
            Tensor m_bias_host, m_bias_device;
            Operator::shared m_add, m_act;      // the device's own operators, for a shortcut the epilogue cannot take
            bool m_folded_quantize = false, m_in_nhwc = false, m_has_out_scale = false, m_extended = false;
            int m_residual = 0;
            std::vector<float> m_quantize_scales, m_dequantize_scales, m_out_scales;
            Padding2D m_padding;
            Stride2D m_stride;
            Dilation2D m_dilation;
            float m_padding_value = 0.0f;
        };

        // Graph rewrite at compile time.  src/compiler/zipper.cpp:20-62 walks the module from its outputs towards its
        // inputs, offers every node to the registered options once, and goes on with the inputs of what an option returned.
        // On the gpu device this option turns a quantized layer -- as a TenniS graph spells it -- into ONE node:
        //
        //   relu | leaky_relu ( add_bias ( conv2d_quantized(x, w), <const bias> ) )                      plain layer
        //   add_bias ( conv2d_quantized(x, w), <const bias> )       with no activation behind it: projection shortcut
        //   relu | leaky_relu ( add ( add_bias(conv2d_quantized(x, w), <const bias>), shortcut ) )       ResNet block tail
        //   add ( relu | leaky_relu ( add_bias(conv2d_quantized(x, w), <const bias>) ), shortcut )       Darknet shortcut
        //                                                            ->  b200_conv2d_quantized_fused(x, w [, shortcut])
        //
        // with NCHW tensors, a constant per-channel bias, and no other reader of the intermediate results.  No shape is
        // known here (the compiler strips "#shape" from the module's inputs before this pass), so whether a shortcut has
        // the layer's own output shape -- "add" broadcasts -- is settled by the fused operator at run time: it folds the
        // shortcut into its epilogue when the shapes agree and finishes the layer with the device's add operator when not.
        // Around the fused node the quantize operators go as well:
        //   * x = quantize(x32), read by this convolution alone: the node takes x32 and quantizes it straight into the layout
        //     its kernel reads;
        //   * x = quantize(y) where y is the top of another such layer that nothing else reads: that layer's node writes int8
        //     in the convolution path's own layout, requantized in its epilogue with this quantize's scales, and this node
        //     reads it as it is -- int8 travels between the layers and no fp32 tensor is written or read in between.
        // Both ends of a hand-over are decided by the same test on the unchanged graph, whichever node is visited first.
        // The fused node keeps the name of the node it replaces, so the module's outputs are found as before.
        class ConvBiasActivationZipper : public ZipperOption {
        public:
            struct Chain {           // (ts::Node has no empty state: the nodes are held by pointer until they are known)
                std::shared_ptr<Node> conv, bias;         // the conv2d_quantized node and the constant of its add_bias
                int activation = TSB_ACT_NONE;
                float leaky = 0.0f;
                int residual = 0;        // 0 none, 1 added before the activation, 2 after it
                std::shared_ptr<Node> shortcut;
            };

            // The readers of a node in the graph as the module gave it: fused nodes this option has already created (the
            // walk goes from the outputs inwards, so a consumer is rewritten before its producer) read the same tensor in
            // place of the quantize -> convolution pair they replace, and are not counted a second time.
            static std::vector<Node> users(const Node &n) {
                std::vector<Node> out;
                for (auto &u : n.outputs())
                    if (u.bubble().op() != Conv2DQuantizedFused::op_name()) out.push_back(u);
                return out;
            }

            static bool is_activation(const Node &n, int &activation, float &leaky) {
                const Bubble &b = n.bubble();
                leaky = 0.0f;
                if (b.op() == name::layer::relu()) { activation = TSB_ACT_RELU; return n.inputs().size() == 1; }
                if (b.op() == "leaky_relu") {     // src/backend/base/base_leaky_relu.cpp registers it under this name
                    if (!b.has(name::scale) || n.inputs().size() != 1) return false;
                    activation = TSB_ACT_LEAKY_RELU;
                    leaky = tensor::to_float(b.get(name::scale));
                    return true;
                }
                return false;
            }

            static bool is_add(const Node &n) {
                return n.bubble().op() == name::layer::add() && n.inputs().size() == 2 && n.input(0) != n.input(1);
            }

            // add_bias(conv2d_quantized(x, w), const) over the channel dimension of NCHW tensors; the convolution's result
            // is read by the add_bias alone
            static bool is_biased_conv(const Node &biased) {
                if (biased.bubble().op() != name::layer::add_bias()) return false;
                if (biased.bubble().has(name::format)) {
                    if (tensor::to_string(biased.bubble().get(name::format)) != name::NCHW) return false;
                } else if (biased.bubble().has(name::dim)) {
                    if (tensor::to_int(biased.bubble().get(name::dim)) != 1) return false;
                } else return false;
                auto in = biased.inputs();
                if (in.size() != 2) return false;
                Node conv = in[0], bias = in[1];
                if (conv.bubble().op() != name::layer::conv2d_quantized() || users(conv).size() != 1) return false;
                if (conv.inputs().size() != 2) return false;
                if (bias.bubble().op() != Bubble::Const || !bias.bubble().has(name::value)) return false;
                if (conv.bubble().has(name::format) && tensor::to_string(conv.bubble().get(name::format)) != name::NCHW) return false;
                return true;
            }

            // ... read by one node only / an activation on such a node, itself read by one node only
            static bool is_biased_chain(const Node &n) { return is_biased_conv(n) && users(n).size() == 1; }
            static bool is_activated_chain(const Node &n) {
                int activation; float leaky;
                return is_activation(n, activation, leaky) && users(n).size() == 1 && is_biased_chain(n.input(0));
            }

            // An "add" goes into ONE layer: style 1, act(add(add_bias(conv), other)), for its first operand that is a biased
            // convolution when an activation alone reads the sum; else style 2, add(act(add_bias(conv)), other), for its
            // first operand that is an activated layer.
            static bool add_owner(const Node &sum, int &operand, int &style) {
                if (!is_add(sum)) return false;
                auto readers = users(sum);
                int activation; float leaky;
                if (readers.size() == 1 && is_activation(readers[0], activation, leaky)) {
                    for (int i = 0; i < 2; ++i) if (is_biased_chain(sum.input(i))) { operand = i; style = 1; return true; }
                }
                for (int i = 0; i < 2; ++i) if (is_activated_chain(sum.input(i))) { operand = i; style = 2; return true; }
                return false;
            }

            // The layer around one conv2d_quantized node, read off the graph as the module gave it: what follows the
            // convolution up to the layer's last node `top` (the add_bias itself where no activation follows: a projection
            // shortcut).  Every question about a layer -- is this node a top, will that convolution be replaced -- goes
            // through here, so all nodes of the walk agree.
            static bool layer_of(const Node &conv, Chain &m, std::shared_ptr<Node> &top) {
                if (conv.bubble().op() != name::layer::conv2d_quantized()) return false;
                auto readers = users(conv);
                if (readers.size() != 1 || !is_biased_conv(readers[0]) || readers[0].input(0) != conv) return false;
                Node biased = readers[0];
                m = Chain();
                m.conv = std::make_shared<Node>(conv);
                m.bias = std::make_shared<Node>(biased.input(1));
                top = std::make_shared<Node>(biased);
                readers = users(biased);
                if (readers.size() != 1) return true;
                Node next = readers[0];
                int operand, style;
                if (is_activation(next, m.activation, m.leaky)) {
                    top = std::make_shared<Node>(next);
                    readers = users(next);
                    if (readers.size() == 1 && add_owner(readers[0], operand, style) && style == 2 && readers[0].input(operand) == next) {
                        m.residual = 2;
                        m.shortcut = std::make_shared<Node>(readers[0].input(1 - operand));
                        top = std::make_shared<Node>(readers[0]);
                    }
                    return true;
                }
                m.activation = TSB_ACT_NONE;
                m.leaky = 0.0f;
                if (add_owner(next, operand, style) && style == 1 && next.input(operand) == biased) {
                    Node act = users(next)[0];
                    is_activation(act, m.activation, m.leaky);
                    m.residual = 1;
                    m.shortcut = std::make_shared<Node>(next.input(1 - operand));
                    top = std::make_shared<Node>(act);
                }
                return true;
            }

            // `node` is the last node of a quantized layer this option replaces
            static bool match(const Node &node, Chain &m) {
                std::vector<Node> convs;        // the convolutions whose layer could end in this node
                auto below_bias = [&](const Node &n) { if (n.bubble().op() == name::layer::add_bias() && n.inputs().size() == 2) convs.push_back(n.input(0)); };
                int activation; float leaky;
                if (node.bubble().op() == name::layer::add_bias()) {
                    below_bias(node);
                } else if (is_activation(node, activation, leaky)) {
                    Node in = node.input(0);
                    below_bias(in);
                    if (is_add(in)) for (int i = 0; i < 2; ++i) below_bias(in.input(i));
                } else if (is_add(node)) {
                    for (int i = 0; i < 2; ++i)
                        if (is_activation(node.input(i), activation, leaky)) below_bias(node.input(i).input(0));
                }
                for (auto &conv : convs) {
                    Chain t;
                    std::shared_ptr<Node> top;
                    if (layer_of(conv, t, top) && *top == node) { m = t; return true; }
                }
                return false;
            }

            // the convolution `conv` belongs to a layer this option replaces
            static bool layer_top(const Node &conv) {
                Chain m;
                std::shared_ptr<Node> top;
                return layer_of(conv, m, top);
            }

            // y -> quantize q -> convolution `consumer`, nothing else reading y or q, both layers replaced by fused nodes:
            // int8 can travel from the first node to the second
            static bool handover(const Node &producer_top, const Node &q, const Node &consumer) {
                if (q.bubble().op() != name::layer::quantize() || !q.bubble().has(name::quantize_scale)) return false;
                if (q.inputs().size() != 1 || q.outputs().size() != 1 || users(producer_top).size() != 1) return false;
                if (q.input(0) != producer_top || q.outputs()[0] != consumer) return false;
                if (consumer.bubble().op() != name::layer::conv2d_quantized() || consumer.input(0) != q) return false;
                Chain pm;
                return match(producer_top, pm) && layer_top(consumer);
            }

            bool zip(const ComputingDevice &device, Node node, Node &zipped_node) const override {
                if (device.type() != GPU) return false;
                Chain m;
                if (!match(node, m)) return false;
                std::vector<Node> fused_inputs = m.conv->inputs();       // x (int8), w
                Tensor folded_scales;
                bool in_nhwc = false;
                {
                    Node q = fused_inputs[0];
                    if (q.bubble().op() == name::layer::quantize() && q.outputs().size() == 1 && q.inputs().size() == 1 &&
                        q.bubble().has(name::quantize_scale)) {
                        if (handover(q.input(0), q, *m.conv)) in_nhwc = true;    // the producer writes what this kernel reads
                        else folded_scales = tensor::cast(FLOAT32, q.bubble().get(name::quantize_scale));
                        fused_inputs[0] = q.input(0);
                    }
                }
                Tensor out_scales;
                if (users(node).size() == 1) {
                    Node q = users(node)[0];
                    if (q.outputs().size() == 1 && handover(node, q, q.outputs()[0]))
                        out_scales = tensor::cast(FLOAT32, q.bubble().get(name::quantize_scale));
                }
                if (m.residual) fused_inputs.push_back(*m.shortcut);
                Node fused = bubble::op(node.bubble().name(), Conv2DQuantizedFused::op_name(), fused_inputs);
                for (auto &param : m.conv->bubble().params()) {
                    if (!param.first.empty() && param.first[0] == Bubble::retention_param_sign) continue;   // #name, #op, ...
                    fused.bubble().set(param.first, param.second);
                }
                fused.bubble().set(Conv2DQuantizedFused::fused_bias(), tensor::cast(FLOAT32, m.bias->bubble().get(name::value)));
                fused.bubble().set(Conv2DQuantizedFused::fused_activation(), tensor::from<int32_t>(m.activation));
                fused.bubble().set(Conv2DQuantizedFused::fused_leaky(), tensor::from<float>(m.leaky));
                if (!folded_scales.empty()) fused.bubble().set(Conv2DQuantizedFused::fused_quantize_scale(), folded_scales);
                if (in_nhwc) fused.bubble().set(Conv2DQuantizedFused::fused_in_nhwc(), tensor::from<int32_t>(1));
                if (!out_scales.empty()) fused.bubble().set(Conv2DQuantizedFused::fused_out_scale(), out_scales);
                if (m.residual) fused.bubble().set(Conv2DQuantizedFused::fused_residual(), tensor::from<int32_t>(m.residual));
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
// ... how many took their input as int8 from another fused node, and how many had a shortcut folded in
extern "C" __attribute__((visibility("default"))) long tsb_plugin_int8_handover_runs() {
    return ts::b200::Conv2DQuantizedFused::int8_handover_runs().load();
}
extern "C" __attribute__((visibility("default"))) long tsb_plugin_residual_runs() {
    return ts::b200::Conv2DQuantizedFused::residual_runs().load();
}
// host nanoseconds spent inside the fused operator's run() so far
extern "C" __attribute__((visibility("default"))) long long tsb_plugin_host_ns() {
    return ts::b200::Conv2DQuantizedFused::host_ns().load();
}
// ... and how many finished a shortcut of another shape or type with the device's own add operator
extern "C" __attribute__((visibility("default"))) long tsb_plugin_reference_add_runs() {
    return ts::b200::Conv2DQuantizedFused::reference_add_runs().load();
}

using namespace ts;
using namespace b200;
TS_REGISTER_OPERATOR(Conv2DQuantized, ts::GPU, name::layer::conv2d_quantized())
TS_REGISTER_OPERATOR(Conv2DQuantizedFused, ts::GPU, Conv2DQuantizedFused::op_name())
TS_REGISTER_ZIPPER_OPTION(ConvBiasActivationZipper)
