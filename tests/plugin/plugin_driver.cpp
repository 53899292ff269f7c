// Drop-in test driver (test infrastructure): runs the SAME TenniS graph -- quantize -> conv2d_quantized ->
// add_bias -> relu, built with the reference's own graph API and loaded with Workbench::Load -- once on the
// reference's CPU device and once on its "gpu" device, where tennis_b200/plugin has registered the B200
// operators and the compile-time rewrite that folds add_bias and relu into the convolution, and compares the outputs.  Also runs the two operators alone through offline_create/offline_run.
//
// Built against the reference headers and linked to the CUDA host build of the reference
// (oracle/_ref/libtennis_cuda.so) and to libtennis_b200_ops.so, whose static initialisers do the registration.
#include <runtime/workbench.h>
#include <module/graph.h>
#include <module/menu.h>
#include <module/module.h>
#include <core/tensor_builder.h>
#include <backend/name.h>
#include <utils/ctxmgr_lite.h>
#include <global/operator_factory.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "tennis_b200.h"

extern "C" long tsb_plugin_fused_runs();             // tennis_b200/plugin/gpu_conv2d_quantized.cpp
extern "C" long tsb_plugin_folded_quantize_runs();

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

struct Case {
    int n, c, h, w, o, k, stride, pad;
};

struct Data {
    Tensor x, w, bias;
    std::vector<float> qscales, dq;
};

Data make_data(const Case &cs, unsigned seed) {
    std::mt19937 rng(seed);
    Data d;
    d.x = Tensor(FLOAT32, Shape({cs.n, cs.c, cs.h, cs.w}));
    float amax = 0;
    for (int i = 0; i < d.x.count(); ++i) {
        // sum of uniforms: bell-shaped, portable across standard libraries
        float v = 0;
        for (int r = 0; r < 4; ++r) v += float(rng() >> 8) / float(1 << 24) - 0.5f;
        d.x.data<float>()[i] = v * 1.7f;
        amax = std::max(amax, std::fabs(v * 1.7f));
    }
    d.qscales.assign(cs.n, 127.0f / amax);
    d.w = Tensor(INT8, Shape({cs.o, cs.c, cs.k, cs.k}));
    for (int i = 0; i < d.w.count(); ++i) d.w.data<int8_t>()[i] = int8_t(int(rng() % 255) - 127);
    d.dq.resize(cs.o);
    std::vector<float> bias(cs.o);
    for (int i = 0; i < cs.o; ++i) {
        d.dq[i] = (0.001f + 0.009f * float(rng() >> 8) / float(1 << 24)) / d.qscales[0];
        bias[i] = (float(rng() >> 8) / float(1 << 24) - 0.5f) * 0.2f;
    }
    d.bias = float_vector(bias);
    return d;
}

void set_conv_params(Bubble &b, const Case &cs, const Data &d) {
    b.set(name::format, tensor::from("NCHW"));
    b.set(name::padding, int_tensor({0, 0, 0, 0, cs.pad, cs.pad, cs.pad, cs.pad}, Shape({4, 2})));
    b.set(name::stride, int_tensor({1, 1, cs.stride, cs.stride}, Shape({4})));
    b.set(name::dilation, int_tensor({1, 1, 1, 1}, Shape({4})));
    b.set(name::dequantize_scales, float_vector(d.dq));
}

// the quantized layer as a TenniS graph, compiled and run on `device`
// keep_q: the quantized tensor is a second output of the module, so the quantize operator has to stay in the program
// leaky > 0: the activation is leaky_relu with that scale instead of relu
Tensor run_graph(const std::string &device, const Case &cs, const Data &d, bool keep_q = false, float leaky = 0.0f) {
    Graph g;
    ctx::bind<Graph> _graph(g);
    auto x = bubble::param("x");
    auto w = bubble::data("w", d.w);
    auto b = bubble::data("b", d.bias);
    auto q = bubble::op("q", name::layer::quantize(), {x});
    q.bubble().set(name::quantize_scale, float_vector(d.qscales));
    auto conv = bubble::op("conv", name::layer::conv2d_quantized(), {q, w});
    set_conv_params(conv.bubble(), cs, d);
    auto biased = bubble::op("biased", name::layer::add_bias(), {conv, b});
    biased.bubble().set(name::format, tensor::from("NCHW"));
    auto y = bubble::op("y", leaky > 0.0f ? std::string("leaky_relu") : name::layer::relu(), {biased});
    if (leaky > 0.0f) y.bubble().set(name::scale, tensor::from<float>(leaky));
    std::shared_ptr<Module> m = std::make_shared<Module>();
    if (keep_q) m->load(g, std::vector<std::string>{"y", "q"});
    else m->load(g, {"y"});
    ComputingDevice cd(device, 0);
    Workbench::shared bench = Workbench::Load(m, cd);
    if (device == CPU) bench->runtime().set_computing_thread_number(1);
    bench->input("x", d.x);
    bench->run();
    bench->run();  // the second run reuses the operator's plan and packed weights
    return bench->output("y").view(MemoryDevice(CPU)).clone();
}

// the two operators alone
void run_ops(const std::string &device, const Case &cs, const Data &d, Tensor &xq, Tensor &y) {
    ComputingDevice cd(device, 0);
    Workbench bench(cd, 1);
    Bubble qb(name::layer::quantize(), "q", 1);
    qb.set(name::quantize_scale, float_vector(d.qscales));
    auto q_op = bench.offline_create(qb, true);
    Bubble cb(name::layer::conv2d_quantized(), "conv", 1);
    set_conv_params(cb, cs, d);
    auto c_op = bench.offline_create(cb, true);
    if (!q_op || !c_op) throw Exception("operator missing on " + device);
    std::vector<Tensor> o1, o2;
    bench.offline_run(q_op, {d.x}, o1);
    bench.offline_run(c_op, {o1[0], d.w}, o2);
    xq = o1[0].view(MemoryDevice(CPU)).clone();
    y = o2[0].view(MemoryDevice(CPU)).clone();
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

}  // namespace

extern "C" __attribute__((visibility("default")))
int tsplug_selftest(int n, int c, int h, int w, int o, int k, int stride, int pad, unsigned seed, char *msg, int msglen) {
    try {
        Case cs{n, c, h, w, o, k, stride, pad};
        Data d = make_data(cs, seed);
        const int64_t launches0 = tsb_kernel_launch_count();
        Tensor xq_cpu, y_cpu, xq_gpu, y_gpu;
        run_ops(CPU, cs, d, xq_cpu, y_cpu);
        run_ops(GPU, cs, d, xq_gpu, y_gpu);
        long bad_q = std::memcmp(xq_cpu.data(), xq_gpu.data(), size_t(xq_cpu.count())) != 0;
        long bad_y = mismatches_f32(y_cpu, y_gpu);
        const int64_t launches_ops = tsb_kernel_launch_count() - launches0;
        Tensor g_cpu = run_graph(CPU, cs, d);
        const long fused0 = tsb_plugin_fused_runs();
        const long folded_start = tsb_plugin_folded_quantize_runs();
        Tensor g_gpu = run_graph(GPU, cs, d);
        // compiling for the gpu device folds add_bias and relu into the convolution (two runs of the graph)
        const long fused = tsb_plugin_fused_runs() - fused0;
        const long folded0 = tsb_plugin_folded_quantize_runs();
        // ... and, the quantize being read by the convolution alone, folds it in as well.  A module that also outputs
        // the quantized tensor keeps its quantize operator for that output and must still give the same y.
        Tensor g_gpu_q = run_graph(GPU, cs, d, true);
        const long folded = folded0 - folded_start;   // the two runs of the first gpu graph
        // the same layer with leaky_relu(0.1): the other activation the rewrite folds
        Tensor l_cpu = run_graph(CPU, cs, d, false, 0.1f);
        const long fused_l0 = tsb_plugin_fused_runs();
        Tensor l_gpu = run_graph(GPU, cs, d, false, 0.1f);
        const long fused_leaky = tsb_plugin_fused_runs() - fused_l0;
        const long bad_l = mismatches_f32(l_cpu, l_gpu);
        long bad_g = mismatches_f32(g_cpu, g_gpu) + mismatches_f32(g_cpu, g_gpu_q) + bad_l;
        const int64_t launches_all = tsb_kernel_launch_count() - launches0;
        std::snprintf(msg, msglen, "quantize mismatch=%ld conv mismatches=%ld graph mismatches=%ld of %d; b200 kernel launches: ops=%lld total=%lld; fused operator runs=%ld; quantize folded=%d",
                      bad_q, bad_y, bad_g, g_cpu.count(), (long long) launches_ops, (long long) launches_all, fused,
                      int(folded >= 2));
        if (launches_ops < 2) return 2;  // the gpu workbench did not reach the B200 operators (CPU fallback)
        if (fused != 2) return 3;        // the graph rewrite did not happen
        if (folded < 2 || fused_leaky != 2) return 4;
        return (bad_q == 0 && bad_y == 0 && bad_g == 0) ? 0 : 1;
    } catch (const std::exception &e) {
        std::snprintf(msg, msglen, "exception: %s", e.what());
        return -1;
    }
}
