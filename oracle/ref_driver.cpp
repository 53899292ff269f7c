// Test infrastructure, not product code.
//
// Plain-C entry points over the reference's own CPU operators, so that Python tests and the
// benchmark's CPU arm can run the unmodified reference arithmetic.  Every call builds a
// ts::Workbench on the CPU device with ONE computing thread (the reference's dequantize loop
// advances a shared pointer inside an OpenMP loop, src/kernels/cpu/quantized/conv2d_quantized_core.cpp:86-106,
// so its output is only defined at one thread), creates the operator with offline_create
// (src/runtime/workbench.cpp:274-288), sets the same attributes a compiled module would carry and runs it
// with offline_run (:290-312).
//
// Compiled against the reference headers where they lie; linked to _ref/libtennis_ref.so.
#include <runtime/workbench.h>
#include <module/bubble.h>
#include <module/module.h>
#include <core/tensor_builder.h>
#include <backend/name.h>
#include <utils/except.h>

#include <chrono>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

using namespace ts;

static thread_local std::string g_error;

#define TSREF_GUARD_BEGIN try {
#define TSREF_GUARD_END                                                   \
    } catch (const std::exception &e) { g_error = e.what(); return -1; }  \
      catch (...) { g_error = "unknown exception"; return -1; }

static Tensor make_tensor(DTYPE dtype, const int *shape, int ndims, const void *data) {
    Shape s(shape, shape + ndims);
    Tensor t(dtype, s);
    if (data) std::memcpy(t.data(), data, size_t(t.count()) * type_bytes(dtype));
    return t;
}

static Tensor int_tensor(const std::vector<int32_t> &v, const Shape &shape) {
    Tensor t(INT32, shape);
    std::memcpy(t.data(), v.data(), v.size() * sizeof(int32_t));
    return t;
}

static Tensor float_vector(const float *v, int n) {
    Tensor t(FLOAT32, Shape({n}));
    std::memcpy(t.data(), v, size_t(n) * sizeof(float));
    return t;
}

static Tensor run1(Workbench &bench, const Bubble &bubble, const std::vector<Tensor> &inputs) {
    auto op = bench.offline_create(bubble, true);
    if (!op) throw Exception("operator not found on cpu: " + bubble.op());
    std::vector<Tensor> outputs;
    bench.offline_run(op, inputs, outputs);
    if (outputs.size() != 1) throw Exception("operator returned != 1 outputs");
    return outputs[0].view(MemoryDevice(CPU));
}

static Bubble quantize_bubble(const float *scales, int nscales) {
    Bubble b(name::layer::quantize(), "q", 1);
    b.set(name::quantize_scale, float_vector(scales, nscales));
    return b;
}

static Bubble conv_bubble(const int *pad_tblr, float padding_value, int sh, int sw, int dh, int dw,
                          const float *dq, int O, int have_padding_value) {
    Bubble b(name::layer::conv2d_quantized(), "conv", 1);
    b.set(name::format, tensor::from("NCHW"));
    b.set(name::padding, int_tensor({0, 0, 0, 0, pad_tblr[0], pad_tblr[1], pad_tblr[2], pad_tblr[3]}, Shape({4, 2})));
    b.set(name::stride, int_tensor({1, 1, sh, sw}, Shape({4})));
    b.set(name::dilation, int_tensor({1, 1, dh, dw}, Shape({4})));
    b.set(name::dequantize_scales, float_vector(dq, O));
    if (have_padding_value) b.set(name::padding_value, tensor::from(padding_value));
    return b;
}

extern "C" {

__attribute__((visibility("default"))) const char *tsref_last_error() { return g_error.c_str(); }

// "quantize": src/backend/base/base_quantize.cpp:12-49, src/kernels/cpu/quantize.cpp:69-147.
__attribute__((visibility("default")))
int tsref_quantize(const float *x, const int *shape, int ndims, const float *scales, int nscales,
                   int8_t *y, int threads) {
    TSREF_GUARD_BEGIN
    Workbench bench(ComputingDevice(CPU, 0), threads);
    Tensor out = run1(bench, quantize_bubble(scales, nscales), {make_tensor(FLOAT32, shape, ndims, x)});
    std::memcpy(y, out.data(), size_t(out.count()));
    return 0;
    TSREF_GUARD_END
}

// the same operator on a FLOAT64 tensor: the generic branch, src/kernels/cpu/quantize.cpp:38-67 and :134.
__attribute__((visibility("default")))
int tsref_quantize_f64(const double *x, const int *shape, int ndims, const float *scales, int nscales,
                       int8_t *y, int threads) {
    TSREF_GUARD_BEGIN
    Workbench bench(ComputingDevice(CPU, 0), threads);
    Tensor out = run1(bench, quantize_bubble(scales, nscales), {make_tensor(FLOAT64, shape, ndims, x)});
    std::memcpy(y, out.data(), size_t(out.count()));
    return 0;
    TSREF_GUARD_END
}

// "pooling2d", type max, format NCHW, padding_type black (the default): src/backend/base/base_pooling2d.cpp:14-118,
// src/kernels/cpu/pooling2d_core.cpp.  out_shape receives {N,C,OH,OW}; y may be null to ask for the shape only.
__attribute__((visibility("default")))
int tsref_max_pooling2d(const float *x, const int *shape, int k, int stride, const int *pad_tblr, float *y,
                        int *out_shape, int threads) {
    TSREF_GUARD_BEGIN
    Workbench bench(ComputingDevice(CPU, 0), threads);
    Bubble b(name::layer::pooling2d(), "pool", 1);
    b.set(name::format, tensor::from("NCHW"));
    b.set(name::type, tensor::from<int32_t>(0));
    b.set(name::padding, int_tensor({0, 0, 0, 0, pad_tblr[0], pad_tblr[1], pad_tblr[2], pad_tblr[3]}, Shape({4, 2})));
    b.set(name::ksize, int_tensor({1, 1, k, k}, Shape({4})));
    b.set(name::stride, int_tensor({1, 1, stride, stride}, Shape({4})));
    Tensor out = run1(bench, b, {make_tensor(FLOAT32, shape, 4, x)});
    for (int i = 0; i < 4; ++i) out_shape[i] = out.size(i);
    if (y) std::memcpy(y, out.data(), size_t(out.count()) * sizeof(float));
    return 0;
    TSREF_GUARD_END
}

// "conv2d_quantized": src/backend/base/base_conv2d_quantized.cpp:13-219,
// src/kernels/cpu/quantized/conv2d_quantized_core.cpp:18-147.  out_shape receives {N,O,OH,OW}.
__attribute__((visibility("default")))
int tsref_conv2d_quantized(const int8_t *x, const int *xshape, const int8_t *w, const int *wshape,
                           const int *pad_tblr, float padding_value, int have_padding_value,
                           int sh, int sw, int dh, int dw, const float *dq, int ndq,
                           float *out, int *out_shape, int threads) {
    TSREF_GUARD_BEGIN
    Workbench bench(ComputingDevice(CPU, 0), threads);
    Bubble b = conv_bubble(pad_tblr, padding_value, sh, sw, dh, dw, dq, ndq, have_padding_value);
    Tensor y = run1(bench, b, {make_tensor(INT8, xshape, 4, x), make_tensor(INT8, wshape, 4, w)});
    for (int i = 0; i < 4; ++i) out_shape[i] = y.size(i);
    if (out) std::memcpy(out, y.data(), size_t(y.count()) * sizeof(float));
    return 0;
    TSREF_GUARD_END
}

// "add_bias" with format NCHW: src/backend/base/base_add_bias.cpp:17-87, src/kernels/cpu/add_bias.cpp:47-85.
__attribute__((visibility("default")))
int tsref_add_bias(const float *x, const int *shape, int ndims, const float *bias, int nbias, float *y, int threads) {
    TSREF_GUARD_BEGIN
    Workbench bench(ComputingDevice(CPU, 0), threads);
    Bubble b(name::layer::add_bias(), "bias", 1);
    b.set(name::format, tensor::from("NCHW"));
    Tensor out = run1(bench, b, {make_tensor(FLOAT32, shape, ndims, x), float_vector(bias, nbias)});
    std::memcpy(y, out.data(), size_t(out.count()) * sizeof(float));
    return 0;
    TSREF_GUARD_END
}

// "relu": src/kernels/cpu/relu.cpp:30-52.
__attribute__((visibility("default")))
int tsref_relu(const float *x, const int *shape, int ndims, float *y, int threads) {
    TSREF_GUARD_BEGIN
    Workbench bench(ComputingDevice(CPU, 0), threads);
    Bubble b(name::layer::relu(), "relu", 1);
    Tensor out = run1(bench, b, {make_tensor(FLOAT32, shape, ndims, x)});
    std::memcpy(y, out.data(), size_t(out.count()) * sizeof(float));
    return 0;
    TSREF_GUARD_END
}

// "leaky_relu": src/backend/base/base_leaky_relu.cpp:13-24, src/kernels/cpu/leaky_relu.cpp:39-67.
__attribute__((visibility("default")))
int tsref_leaky_relu(const float *x, const int *shape, int ndims, float scale, float *y, int threads) {
    TSREF_GUARD_BEGIN
    Workbench bench(ComputingDevice(CPU, 0), threads);
    Bubble b("leaky_relu", "leaky", 1);
    b.set(name::scale, tensor::from(scale));
    Tensor out = run1(bench, b, {make_tensor(FLOAT32, shape, ndims, x)});
    std::memcpy(y, out.data(), size_t(out.count()) * sizeof(float));
    return 0;
    TSREF_GUARD_END
}

// Timing of the reference hot path on host cores: quantize -> conv2d_quantized -> add_bias -> relu|leaky_relu
// on one layer, `workers` independent Workbenches in as many host threads (one Workbench per thread is how the
// reference is used from several threads; each keeps ONE computing thread so its output stays valid), each
// running `images` samples `repeats` times.  seconds_out = wall time of the slowest worker for ONE repeat
// (minimum over repeats).  act: 0 none, 1 relu, 2 leaky_relu(leaky).
__attribute__((visibility("default")))
int tsref_time_layer(const float *x, int images, int C, int H, int W,
                     const int8_t *w, int O, int KH, int KW, const int *pad_tblr, int sh, int sw, int dh, int dw,
                     float qscale, const float *dq, const float *bias, int act, float leaky,
                     int workers, int repeats, double *seconds_out, double *quantize_seconds_out) {
    TSREF_GUARD_BEGIN
    std::vector<double> best(workers, 1e30), best_q(workers, 1e30);
    std::vector<std::string> errors(workers);
    auto body = [&](int wid) {
        try {
            Workbench bench(ComputingDevice(CPU, 0), 1);
            int xs[4] = {images, C, H, W};
            int ws[4] = {O, C, KH, KW};
            Tensor tx = make_tensor(FLOAT32, xs, 4, x);
            Tensor tw = make_tensor(INT8, ws, 4, w);
            std::vector<float> qs(images, qscale);
            auto q_op = bench.offline_create(quantize_bubble(qs.data(), images), true);
            auto c_op = bench.offline_create(conv_bubble(pad_tblr, 0.f, sh, sw, dh, dw, dq, O, 0), true);
            Bubble bb(name::layer::add_bias(), "bias", 1);
            bb.set(name::format, tensor::from("NCHW"));
            auto b_op = bench.offline_create(bb, true);
            Operator::shared a_op;
            if (act == 1) a_op = bench.offline_create(Bubble(name::layer::relu(), "relu", 1), true);
            if (act == 2) {
                Bubble lb("leaky_relu", "leaky", 1);
                lb.set(name::scale, tensor::from(leaky));
                a_op = bench.offline_create(lb, true);
            }
            Tensor tb = float_vector(bias, O);
            for (int r = 0; r < repeats; ++r) {
                std::vector<Tensor> o1, o2, o3, o4;
                auto t0 = std::chrono::steady_clock::now();
                bench.offline_run(q_op, {tx}, o1);
                auto t1 = std::chrono::steady_clock::now();
                bench.offline_run(c_op, {o1[0], tw}, o2);
                bench.offline_run(b_op, {o2[0], tb}, o3);
                if (a_op) bench.offline_run(a_op, {o3[0]}, o4);
                auto t2 = std::chrono::steady_clock::now();
                best[wid] = std::min(best[wid], std::chrono::duration<double>(t2 - t0).count());
                best_q[wid] = std::min(best_q[wid], std::chrono::duration<double>(t1 - t0).count());
            }
        } catch (const std::exception &e) { errors[wid] = e.what(); }
    };
    std::vector<std::thread> pool;
    for (int i = 1; i < workers; ++i) pool.emplace_back(body, i);
    body(0);
    for (auto &t : pool) t.join();
    double worst = 0, worst_q = 0;
    for (int i = 0; i < workers; ++i) {
        if (!errors[i].empty()) throw Exception(errors[i]);
        worst = std::max(worst, best[i]);
        worst_q = std::max(worst_q, best_q[i]);
    }
    *seconds_out = worst;
    if (quantize_seconds_out) *quantize_seconds_out = worst_q;
    return 0;
    TSREF_GUARD_END
}

// tensor::load + tensor::save (include/core/tensor_builder.h:153-159): reads a .t file with the reference and writes it
// back with the reference, so a file written elsewhere can be compared byte for byte with the reference's own.
// info receives {fields, dtype of field 0, dims of field 0, shape...} (up to 3 + 8 ints).
__attribute__((visibility("default")))
int tsref_tensor_roundtrip(const char *path_in, const char *path_out, int *info) {
    TSREF_GUARD_BEGIN
    Tensor t = tensor::load(path_in);
    info[0] = int(t.fields_count());
    info[1] = int(t.dtype());
    info[2] = int(t.dims());
    for (int i = 0; i < t.dims() && i < 8; ++i) info[3 + i] = t.size(i);
    if (path_out) tensor::save(path_out, t);
    return 0;
    TSREF_GUARD_END
}

// Module::Load of a .tsm file (src/module/module.cpp:295-333), compiled for the cpu device with Workbench::Load and run
// on one fp32 input.  out may be null to ask for the output's shape only (out_shape: dims, then the shape).
__attribute__((visibility("default")))
int tsref_run_module(const char *path, const float *x, const int *shape, int ndims, float *out, long out_capacity,
                     int *out_shape, int *node_count, int threads) {
    TSREF_GUARD_BEGIN
    Module::shared module = Module::Load(path);
    if (node_count) *node_count = 0;
    ComputingDevice device(CPU, 0);
    Workbench::shared bench = Workbench::Load(module, device);
    bench->runtime().set_computing_thread_number(threads);
    bench->input(0, make_tensor(FLOAT32, shape, ndims, x));
    bench->run();
    Tensor y = bench->output(0).view(MemoryDevice(CPU));
    if (y.dtype() != FLOAT32) throw Exception("module output is not fp32");
    out_shape[0] = y.dims();
    for (int i = 0; i < y.dims() && i < 8; ++i) out_shape[1 + i] = y.size(i);
    if (out) {
        if (long(y.count()) > out_capacity) throw Exception("output buffer too small");
        std::memcpy(out, y.data(), size_t(y.count()) * sizeof(float));
    }
    return 0;
    TSREF_GUARD_END
}

}  // extern "C"
