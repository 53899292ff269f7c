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
extern "C" long tsb_plugin_int8_handover_runs();
extern "C" long tsb_plugin_residual_runs();
extern "C" long tsb_plugin_reference_add_runs();

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

// One quantized layer of a larger graph: quantize -> conv2d_quantized -> add_bias [-> add shortcut] -> relu | leaky_relu
// [-> add shortcut], as a model converter writes it.  shortcut_mode: 0 none, 1 before the activation, 2 after it.
Node quantized_layer(const std::string &name, Node in, const Case &cs, const Data &d, float in_scale, float leaky, int shortcut_mode,
                     const Node *shortcut) {
    auto q = bubble::op(name + ".q", name::layer::quantize(), {in});
    q.bubble().set(name::quantize_scale, float_vector(std::vector<float>(cs.n, in_scale)));
    auto conv = bubble::op(name + ".conv", name::layer::conv2d_quantized(), {q, bubble::data(name + ".w", d.w)});
    set_conv_params(conv.bubble(), cs, d);
    auto biased = bubble::op(name + ".biased", name::layer::add_bias(), {conv, bubble::data(name + ".b", d.bias)});
    biased.bubble().set(name::format, tensor::from("NCHW"));
    Node pre = biased;
    if (shortcut_mode == 1) pre = bubble::op(name + ".sum", name::layer::add(), {biased, *shortcut});
    auto act = bubble::op(name + ".act", leaky > 0.0f ? std::string("leaky_relu") : name::layer::relu(), {pre});
    if (leaky > 0.0f) act.bubble().set(name::scale, tensor::from<float>(leaky));
    if (shortcut_mode == 2) return bubble::op(name + ".sum", name::layer::add(), {act, *shortcut});
    return act;
}

// A bottleneck block with a shortcut -- 1x1 c->m, 3x3 m->m, 1x1 m->c, the sum with the block's input before the last
// relu (darknet: after a leaky_relu) -- as ONE TenniS graph, loaded with Workbench::Load.
// broadcast: the shortcut is a second input of shape [1, c, 1, 1] instead, which operator "add" broadcasts;
// tail: a fourth layer (1x1 c->m) reads the block's result, so the block's last node hands int8 on as well.
Tensor run_block(const std::string &device, int n, int c, int m, int h, int w, const Data d[4], const float scales[4], bool darknet,
                 bool broadcast, bool tail, const Tensor &side) {
    Graph g;
    ctx::bind<Graph> _graph(g);
    auto x = bubble::param("x", FLOAT32, Shape({n, c, h, w}));
    auto s = broadcast ? bubble::param("s", FLOAT32, Shape({1, c, 1, 1})) : x;
    const float leaky = darknet ? 0.1f : 0.0f;
    Case c1{n, c, h, w, m, 1, 1, 0}, c2{n, m, h, w, m, 3, 1, 1}, c3{n, m, h, w, c, 1, 1, 0};
    Node y1 = quantized_layer("l1", x, c1, d[0], scales[0], leaky, 0, nullptr);
    Node y2 = quantized_layer("l2", y1, c2, d[1], scales[1], leaky, 0, nullptr);
    Node y3 = quantized_layer("l3", y2, c3, d[2], scales[2], leaky, darknet ? 2 : 1, &s);
    Node top = tail ? quantized_layer("l4", y3, c1, d[3], scales[3], leaky, 0, nullptr) : y3;
    std::shared_ptr<Module> mod = std::make_shared<Module>();
    mod->load(g, {top.bubble().name()});
    ComputingDevice cd(device, 0);
    Workbench::shared bench = Workbench::Load(mod, cd);
    if (device == CPU) bench->runtime().set_computing_thread_number(1);
    Tensor input(FLOAT32, Shape({n, c, h, w}));
    std::memcpy(input.data(), d[0].x.data(), size_t(input.count()) * sizeof(float));
    bench->input("x", input);
    if (broadcast) bench->input("s", side);
    bench->run();
    bench->run();
    return bench->output(0).view(MemoryDevice(CPU)).clone();
}

}  // namespace

// The bottleneck block on the cpu and on the gpu device.  On the gpu device the layers must become fused nodes that pass
// int8 between them: per run one staging quantize of the block's input and one convolution launch per layer, nothing
// else from this library.  variant: bit 0 Darknet-style shortcut, bit 1 broadcast shortcut (the fused node then finishes
// the layer with the device's own add), bit 2 a fourth layer behind the block.
extern "C" __attribute__((visibility("default")))
int tsplug_block(int n, int c, int m, int h, int w, int variant, unsigned seed, char *msg, int msglen) {
    const char *phase = "setup";
    try {
        const bool darknet = variant & 1, broadcast = variant & 2, tail = variant & 4;
        const int layers = tail ? 4 : 3;
        Data d[4] = {make_data(Case{n, c, h, w, m, 1, 1, 0}, seed), make_data(Case{n, m, h, w, m, 3, 1, 1}, seed + 1),
                     make_data(Case{n, m, h, w, c, 1, 1, 0}, seed + 2), make_data(Case{n, c, h, w, m, 1, 1, 0}, seed + 3)};
        // activation scales between the layers: 127 / (a plausible maximum of the previous layer's output)
        const float scales[4] = {d[0].qscales[0], 127.0f / 3.0f, 127.0f / 2.5f, 127.0f / 4.0f};
        for (int l = 1; l < 4; ++l)
            for (auto &v : d[l].dq) v = v * d[l].qscales[0] / scales[l];      // weight scale / this layer's input scale
        Tensor side(FLOAT32, Shape({1, c, 1, 1}));
        for (int i = 0; i < c; ++i) side.data<float>()[i] = 0.25f * float((i * 7) % 11) - 1.0f;
        phase = "cpu device";
        Tensor y_cpu = run_block(CPU, n, c, m, h, w, d, scales, darknet, broadcast, tail, side);
        const long fused0 = tsb_plugin_fused_runs(), hand0 = tsb_plugin_int8_handover_runs(), res0 = tsb_plugin_residual_runs();
        const long folded0 = tsb_plugin_folded_quantize_runs(), ref0 = tsb_plugin_reference_add_runs();
        const int64_t launches0 = tsb_kernel_launch_count();
        phase = "gpu device";
        Tensor y_gpu = run_block(GPU, n, c, m, h, w, d, scales, darknet, broadcast, tail, side);
        const long fused = tsb_plugin_fused_runs() - fused0, hand = tsb_plugin_int8_handover_runs() - hand0;
        const long res = tsb_plugin_residual_runs() - res0, folded = tsb_plugin_folded_quantize_runs() - folded0;
        const long ref_add = tsb_plugin_reference_add_runs() - ref0;
        const int64_t launches = tsb_kernel_launch_count() - launches0;
        const long bad = mismatches_f32(y_cpu, y_gpu);
        std::snprintf(msg, msglen, "block mismatches=%ld of %d; per 2 runs: fused nodes=%ld int8 hand-overs=%ld shortcuts folded=%ld shortcuts by the add operator=%ld input quantizes folded=%ld kernel launches=%lld",
                      bad, y_cpu.count(), fused, hand, res, ref_add, folded, (long long) launches);
        // the rewrite must have produced the chain of fused nodes
        if (fused != 2 * layers || hand != 2 * (layers - 1) || folded != 2) return 3;
        if (res != (broadcast ? 0 : 2) || ref_add != (broadcast ? 2 : 0)) return 3;
        // two runs x (1 staging quantize + the convolutions [+ the quantize behind a shortcut the add operator took]),
        // plus the weight repacks of the first run
        if (launches != 2 * (1 + layers + (broadcast && tail ? 1 : 0)) + layers) return 4;
        return bad == 0 ? 0 : 1;
    } catch (const std::exception &e) {
        std::snprintf(msg, msglen, "exception (%s): %s", phase, e.what());
        return -1;
    }
}

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

// The compile-time use of quantize (src/compiler/compiler.cpp:386-461: a node whose inputs are all constants is run once,
// on the compiling workbench's device, and replaced by its result): a module that carries its convolution weights in fp32
// with a quantize node behind them, one scale per output channel.  Compiled for the gpu device, that node runs through
// this repo's quantize operator while the module is loaded; the graph's result must equal the cpu device's.
extern "C" __attribute__((visibility("default")))
int tsplug_const_weights(int n, int c, int h, int w, int o, int k, int stride, int pad, unsigned seed, char *msg, int msglen) {
    try {
        Case cs{n, c, h, w, o, k, stride, pad};
        Data d = make_data(cs, seed);
        std::mt19937 rng(seed + 7);
        Tensor wf(FLOAT32, Shape({o, c, k, k}));
        std::vector<float> wscales(o);
        const int per_channel = c * k * k;
        for (int oc = 0; oc < o; ++oc) {
            float amax = 0;
            for (int i = 0; i < per_channel; ++i) {
                const float v = (float(rng() >> 8) / float(1 << 24) - 0.5f) * (0.2f + 0.01f * float(oc % 7));
                wf.data<float>()[oc * per_channel + i] = v;
                amax = std::max(amax, std::fabs(v));
            }
            wscales[oc] = 127.0f / amax;
            d.dq[oc] = 1.0f / (wscales[oc] * d.qscales[0]);
        }
        auto run = [&](const std::string &device, int64_t *launches_at_load) {
            Graph g;
            ctx::bind<Graph> _graph(g);
            auto x = bubble::param("x");
            auto q = bubble::op("q", name::layer::quantize(), {x});
            q.bubble().set(name::quantize_scale, float_vector(d.qscales));
            auto wq = bubble::op("wq", name::layer::quantize(), {bubble::data("w32", wf)});
            wq.bubble().set(name::quantize_scale, float_vector(wscales));
            auto conv = bubble::op("conv", name::layer::conv2d_quantized(), {q, wq});
            set_conv_params(conv.bubble(), cs, d);
            auto biased = bubble::op("biased", name::layer::add_bias(), {conv, bubble::data("b", d.bias)});
            biased.bubble().set(name::format, tensor::from("NCHW"));
            auto y = bubble::op("y", name::layer::relu(), {biased});
            std::shared_ptr<Module> m = std::make_shared<Module>();
            m->load(g, {"y"});
            ComputingDevice cd(device, 0);
            const int64_t before = tsb_kernel_launch_count();
            Workbench::shared bench = Workbench::Load(m, cd);
            if (launches_at_load) *launches_at_load = tsb_kernel_launch_count() - before;
            if (device == CPU) bench->runtime().set_computing_thread_number(1);
            bench->input("x", d.x);
            bench->run();
            return bench->output("y").view(MemoryDevice(CPU)).clone();
        };
        Tensor y_cpu = run(CPU, nullptr);
        int64_t at_load = 0;
        const long fused0 = tsb_plugin_fused_runs();
        Tensor y_gpu = run(GPU, &at_load);
        const long fused = tsb_plugin_fused_runs() - fused0;
        const long bad = mismatches_f32(y_cpu, y_gpu);
        std::snprintf(msg, msglen, "constant weights: mismatches=%ld of %d; kernel launches while loading=%lld; fused operator runs=%ld",
                      bad, y_cpu.count(), (long long) at_load, fused);
        if (at_load < 1) return 2;       // the weights were not quantized by this library's operator at compile time
        if (fused != 1) return 3;
        return bad == 0 ? 0 : 1;
    } catch (const std::exception &e) {
        std::snprintf(msg, msglen, "exception: %s", e.what());
        return -1;
    }
}
