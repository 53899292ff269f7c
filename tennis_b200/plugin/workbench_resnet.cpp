// A ResNet-50-shaped quantized network written with the reference's own graph API, loaded with Workbench::Load and run
// with Workbench::run on TenniS's "gpu" device, where libtennis_b200_ops.so has registered its operators and its graph
// rewrite.  A host program in miniature: bench.py times it beside the same network driven through the C ABI, and
// tests/test_gpu_plugin.py compares it with the cpu device.  Everything that is not a quantized convolution layer
// (max pool, average pool, flatten, inner product) runs on the reference's own gpu operators.
#include <runtime/workbench.h>
#include <module/graph.h>
#include <module/menu.h>
#include <module/module.h>
#include <core/tensor_builder.h>
#include <backend/name.h>
#include <utils/ctxmgr_lite.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "tennis_b200.h"

extern "C" long tsb_plugin_fused_runs();             // gpu_conv2d_quantized.cpp
extern "C" long tsb_plugin_int8_handover_runs();
extern "C" long tsb_plugin_residual_runs();
extern "C" long long tsb_plugin_host_ns();

using namespace ts;

namespace {

Tensor int_tensor(const std::vector<int32_t> &v, const Shape &shape) {
    Tensor t(INT32, shape);
    std::memcpy(t.data(), v.data(), v.size() * sizeof(int32_t));
    return t;
}

Tensor float_vector(const std::vector<float> &v) {
    Tensor t(FLOAT32, Shape({int(v.size())}));
    std::memcpy(t.data(), v.data(), v.size() * sizeof(float));
    return t;
}

long mismatches_f32(const Tensor &a, const Tensor &b) {
    if (!a.has_shape(b.sizes())) return -1;
    long bad = 0;
    const float *pa = a.data<float>(), *pb = b.data<float>();
    for (int i = 0; i < a.count(); ++i) {
        uint32_t ua, ub;
        std::memcpy(&ua, pa + i, 4);
        std::memcpy(&ub, pb + i, 4);
        if (ua != ub && !(pa[i] == 0.0f && pb[i] == 0.0f)) ++bad;
    }
    return bad;
}

// ---- a ResNet-50-shaped network as ONE TenniS graph ----------------------------------------------------------------
// Seeded synthetic int8 weights; dequantize scales sized so that activations stay within a few units; every
// convolution has its own quantize operator in front, as a model converter writes it.
struct LayerData {
    Tensor w, bias;
    std::vector<float> dq;
};

LayerData make_layer(int c, int o, int k, float in_scale, std::mt19937 &rng) {
    LayerData d;
    d.w = Tensor(INT8, Shape({o, c, k, k}));
    for (int i = 0; i < d.w.count(); ++i) d.w.data<int8_t>()[i] = int8_t(int(rng() % 255) - 127);
    d.dq.resize(o);
    std::vector<float> bias(o);
    // int8 weights ~ U(-127,127) (sigma 73), int8 activations of sigma about 30: the accumulator's sigma is 73*30*sqrt(K)
    const float unit = 1.0f / (73.0f * 30.0f * std::sqrt(float(c * k * k)));
    for (int i = 0; i < o; ++i) {
        d.dq[i] = unit * (0.5f + float(rng() >> 8) / float(1 << 24)) * (127.0f / 4.0f) / in_scale;
        bias[i] = (float(rng() >> 8) / float(1 << 24) - 0.5f) * 0.2f;
    }
    d.bias = float_vector(bias);
    return d;
}

// quantize -> conv2d_quantized -> add_bias, the part every layer has
Node biased_conv(const std::string &name, Node in, int n, const LayerData &d, int k, int stride, int pad, float in_scale) {
    auto q = bubble::op(name + ".q", name::layer::quantize(), {in});
    q.bubble().set(name::quantize_scale, float_vector(std::vector<float>(n, in_scale)));
    auto conv = bubble::op(name + ".conv", name::layer::conv2d_quantized(), {q, bubble::data(name + ".w", d.w)});
    Bubble &b = conv.bubble();
    b.set(name::format, tensor::from("NCHW"));
    b.set(name::padding, int_tensor({0, 0, 0, 0, pad, pad, pad, pad}, Shape({4, 2})));
    b.set(name::stride, int_tensor({1, 1, stride, stride}, Shape({4})));
    b.set(name::dilation, int_tensor({1, 1, 1, 1}, Shape({4})));
    b.set(name::dequantize_scales, float_vector(d.dq));
    auto biased = bubble::op(name + ".biased", name::layer::add_bias(), {conv, bubble::data(name + ".b", d.bias)});
    biased.bubble().set(name::format, tensor::from("NCHW"));
    return biased;
}

struct ResNetGraph {
    Graph graph;
    std::shared_ptr<Module> module;
    int convolutions = 0;
};

// stem 7x7/2 -> max pool 3x3/2 -> [3, 4, 6, 3] bottlenecks (projection shortcut on the first block of a stage, stride
// on the 3x3) -> global average pool -> inner product: 53 convolutions.
void build_resnet50(ResNetGraph &net, int n, int image, unsigned seed, bool head, int max_blocks = 16) {
    std::mt19937 rng(seed);
    ctx::bind<Graph> _graph(net.graph);
    const float act_scale = 127.0f / 4.0f;
    auto x = bubble::param("x", FLOAT32, Shape({n, 3, image, image}));
    int count = 0;
    auto layer = [&](const std::string &name, Node in, int c, int o, int k, int stride, int pad, float in_scale) {
        ++count;
        return biased_conv(name, in, n, make_layer(c, o, k, in_scale, rng), k, stride, pad, in_scale);
    };
    Node y = bubble::op("stem.act", name::layer::relu(), {layer("stem", x, 3, 64, 7, 2, 3, 127.0f / 2.5f)});
    y = bubble::op("pool", name::layer::pooling2d(), {y});
    y.bubble().set(name::format, tensor::from("NCHW"));
    y.bubble().set(name::type, tensor::from<int32_t>(0));
    y.bubble().set(name::padding, int_tensor({0, 0, 0, 0, 1, 0, 1, 0}, Shape({4, 2})));
    y.bubble().set(name::ksize, int_tensor({1, 1, 3, 3}, Shape({4})));
    y.bubble().set(name::stride, int_tensor({1, 1, 2, 2}, Shape({4})));
    const int widths[4] = {64, 128, 256, 512}, blocks[4] = {3, 4, 6, 3};
    int cin = 64, built = 0;
    for (int s = 0; s < 4; ++s) {
        for (int bi = 0; bi < blocks[s] && built < max_blocks; ++bi, ++built) {
            const std::string name = "s" + std::to_string(s + 1) + "b" + std::to_string(bi + 1);
            const int width = widths[s], cout = 4 * width, stride = (bi == 0 && s > 0) ? 2 : 1;
            Node a = bubble::op(name + ".conv1.act", name::layer::relu(), {layer(name + ".conv1", y, cin, width, 1, 1, 0, act_scale)});
            Node b = bubble::op(name + ".conv2.act", name::layer::relu(), {layer(name + ".conv2", a, width, width, 3, stride, 1, act_scale)});
            Node c = layer(name + ".conv3", b, width, cout, 1, 1, 0, act_scale);
            Node shortcut = bi == 0 ? layer(name + ".proj", y, cin, cout, 1, stride, 0, act_scale) : y;
            Node sum = bubble::op(name + ".sum", name::layer::add(), {c, shortcut});
            y = bubble::op(name + ".out", name::layer::relu(), {sum});
            cin = cout;
        }
    }
    net.convolutions = count;
    if (!head) {         // the trunk alone: everything up to here is exact on both devices
        net.module = std::make_shared<Module>();
        net.module->load(net.graph, {y.bubble().name()});
        return;
    }
    y = bubble::op("gap", name::layer::global_pooling2d(), {y});
    y.bubble().set(name::format, tensor::from("NCHW"));
    y.bubble().set(name::type, tensor::from<int32_t>(1));
    y = bubble::op("flat", name::layer::flatten(), {y});
    Tensor fc_w(FLOAT32, Shape({cin, 1000}));
    for (int i = 0; i < fc_w.count(); ++i) fc_w.data<float>()[i] = (float(rng() >> 8) / float(1 << 24) - 0.5f) * 0.02f;
    y = bubble::op("fc", name::layer::inner_prod(), {y, bubble::data("fc.w", fc_w)});
    net.module = std::make_shared<Module>();
    net.module->load(net.graph, {"fc"});
}

}  // namespace

// A ResNet-50-shaped TenniS graph (53 convolutions) through Workbench::Load / Workbench::run on the gpu device.
// check > 0: the trunk alone, its first check - 1 blocks (17: all of them) (the last block's output is the module's output: the average pool and inner product
// behind it are floating-point reductions of the two devices' own operators), also run on the cpu device and compared
// bit for bit.  reps timed passes after two warm-up passes, each with the host input bound again (Workbench::input +
// run: the upload from pageable host memory is part of the pass) and the logits read back; check == -1: the input is
// bound once as a tensor in device memory instead, so a pass is what the device and the runtime's run loop take.
// out[0] = milliseconds per pass (wall clock, device idle at both ends), out[1] = kernel launches of this library per
// pass, out[2] = fused nodes run per pass, out[3] = int8 hand-overs per pass, out[4] = shortcuts folded per pass,
// out[5] = mismatching elements (-1 when not checked), out[6] = host milliseconds per pass spent inside the fused operator.
extern "C" __attribute__((visibility("default")))
int tsb_workbench_resnet50(int batch, int image, int reps, int check, unsigned seed, double *out, char *msg, int msglen) {
    const char *phase = "build";
    try {
        ResNetGraph net;
        build_resnet50(net, batch, image, seed, check <= 0, check <= 0 ? 16 : check - 1);
        Tensor input(FLOAT32, Shape({batch, 3, image, image}));
        {
            std::mt19937 rng(seed + 99);
            for (int i = 0; i < input.count(); ++i) {
                float v = 0;
                for (int r = 0; r < 4; ++r) v += float(rng() >> 8) / float(1 << 24) - 0.5f;
                input.data<float>()[i] = v * 1.7f;
            }
        }
        phase = "gpu device";
        ComputingDevice gpu(GPU, 0);
        Workbench::shared bench = Workbench::Load(net.module, gpu);
        Tensor logits;
        const bool resident = check == -1;
        if (resident) bench->input("x", input.view(MemoryDevice(GPU, 0)));
        auto pass = [&]() {
            if (!resident) bench->input("x", input);
            bench->run();
            logits = bench->output(0).view(MemoryDevice(CPU));      // waits for the device and copies the result back
        };
        pass();
        pass();
        const long fused0 = tsb_plugin_fused_runs(), hand0 = tsb_plugin_int8_handover_runs(), res0 = tsb_plugin_residual_runs();
        const int64_t launches0 = tsb_kernel_launch_count();
        const long long host0 = tsb_plugin_host_ns();
        const auto t0 = std::chrono::steady_clock::now();
        for (int r = 0; r < reps; ++r) pass();
        const auto t1 = std::chrono::steady_clock::now();
        out[0] = std::chrono::duration<double, std::milli>(t1 - t0).count() / reps;
        out[1] = double(tsb_kernel_launch_count() - launches0) / reps;
        out[2] = double(tsb_plugin_fused_runs() - fused0) / reps;
        out[3] = double(tsb_plugin_int8_handover_runs() - hand0) / reps;
        out[4] = double(tsb_plugin_residual_runs() - res0) / reps;
        out[5] = -1;
        out[6] = double(tsb_plugin_host_ns() - host0) / 1e6 / reps;      // ms per pass inside the fused operator's run()
        Tensor y_gpu = logits.clone();
        if (check > 0) {
            phase = "cpu device";
            ComputingDevice cpu(CPU, 0);
            Workbench::shared ref = Workbench::Load(net.module, cpu);
            ref->runtime().set_computing_thread_number(1);   // as everywhere in this file: the reference's multi-scale quantize is only deterministic on one thread
            ref->input("x", input);
            ref->run();
            Tensor y_cpu = ref->output(0).view(MemoryDevice(CPU)).clone();
            const long bad = mismatches_f32(y_cpu, y_gpu);
            out[5] = double(bad);
            std::snprintf(msg, msglen, "resnet50 graph: %d convolutions, trunk mismatches=%ld of %d; per pass: fused nodes=%g int8 hand-overs=%g shortcuts folded=%g kernel launches=%g",
                          net.convolutions, bad, y_cpu.count(), out[2], out[3], out[4], out[1]);
            return bad == 0 ? 0 : 1;
        }
        std::snprintf(msg, msglen, "resnet50 graph: %d convolutions, %.3f ms per pass", net.convolutions, out[0]);
        return 0;
    } catch (const std::exception &e) {
        std::snprintf(msg, msglen, "exception (%s): %s", phase, e.what());
        return -1;
    }
}

// A module file (.tsm, Module::Load: src/module/module.cpp:295-333) compiled by Workbench::Load for `device` ("cpu" or
// "gpu") and run on one fp32 input; the fp32 output is copied to `out` (null: only its shape is wanted).  out_shape
// receives the number of dimensions, then the shape.  counters (may be null) receives what the pass ran of this library:
// {fused nodes, int8 hand-overs, shortcuts folded, kernel launches}.
extern "C" __attribute__((visibility("default")))
int tsb_workbench_run_tsm(const char *path, const char *device, const float *x, const int *shape, int ndims, float *out,
                          long out_capacity, int *out_shape, double *counters, char *msg, int msglen) {
    try {
        Module::shared module = Module::Load(path);
        ComputingDevice where(device, 0);
        Workbench::shared bench = Workbench::Load(module, where);
        if (where.type() == CPU) bench->runtime().set_computing_thread_number(1);
        Tensor input(FLOAT32, Shape(shape, shape + ndims));
        std::memcpy(input.data(), x, size_t(input.count()) * sizeof(float));
        bench->input(0, input);
        bench->run();       // first run: plans, packed weights
        const long fused0 = tsb_plugin_fused_runs(), hand0 = tsb_plugin_int8_handover_runs(), res0 = tsb_plugin_residual_runs();
        const int64_t launches0 = tsb_kernel_launch_count();
        bench->run();
        Tensor y = bench->output(0).view(MemoryDevice(CPU));
        if (counters) {
            counters[0] = double(tsb_plugin_fused_runs() - fused0);
            counters[1] = double(tsb_plugin_int8_handover_runs() - hand0);
            counters[2] = double(tsb_plugin_residual_runs() - res0);
            counters[3] = double(tsb_kernel_launch_count() - launches0);
        }
        if (y.dtype() != FLOAT32) throw Exception("the module's output is not fp32");
        out_shape[0] = y.dims();
        for (int i = 0; i < y.dims() && i < 8; ++i) out_shape[1 + i] = y.size(i);
        if (out) {
            if (long(y.count()) > out_capacity) throw Exception("output buffer too small");
            std::memcpy(out, y.data(), size_t(y.count()) * sizeof(float));
        }
        std::snprintf(msg, msglen, "ok");
        return 0;
    } catch (const std::exception &e) {
        std::snprintf(msg, msglen, "exception: %s", e.what());
        return -1;
    }
}
