"""Writes BASELINE configurations 0 and 1 as case folders for the reference's tools/run_test (one folder per operator
call: 0.<operator>.txt, 1.<attribute>.t, 2.input_<i>.t, 3.output_<i>.t).  The wanted outputs come from the reference's own
compiled CPU operators (oracle/_ref/libtsref.so), so `run_test <folder> gpu` compares this repo's operators on the gpu
device with the reference's CPU results, within run_test's own tolerances (tools/run_test/test_case.hpp:491-492).

    python tests/run_test_cases.py <output folder> [--batch N]

Test infrastructure: imports the oracle package."""
import argparse
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import oracle as orc          # noqa: E402
from tennis_b200 import tsfile             # noqa: E402

# (name, batch, C, H/W, O, kernel, stride, pad): configuration 0, then the five shapes of configuration 1
CONFIG0 = ("config0_3x3_64_64_56", 1, 64, 56, 64, 3, 1, 1)
CONFIG1 = [("config1a_1x1_256_1024_14", 32, 256, 14, 1024, 1, 1, 0),
           ("config1b_3x3_128_128_28", 32, 128, 28, 128, 3, 1, 1),
           ("config1c_3x3s2_256_512_28", 32, 256, 28, 512, 3, 2, 1),
           ("config1d_1x1_2048_512_7", 32, 2048, 7, 512, 1, 1, 0),
           ("config1e_7x7s2_3_64_224", 32, 3, 224, 64, 7, 2, 3)]


def layer_tensors(n, c, hw, o, k, seed=0):
    """The value distributions BASELINE.json states: x ~ N(0,1), per-tensor scale 127 / max|x|, int8 weights uniform in
    [-127, 127], per-channel weight scales ~ U(0.001, 0.01), bias ~ N(0, 0.1)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, c, hw, hw), dtype=np.float32)
    scale = np.float32(127.0) / np.float32(np.abs(x).max())
    w = rng.integers(-127, 128, size=(o, c, k, k), dtype=np.int8)
    sw = rng.uniform(0.001, 0.01, size=o).astype(np.float32)
    bias = (rng.standard_normal(o) * 0.1).astype(np.float32)
    dq = (sw / scale).astype(np.float32)
    return x, scale, w, dq, bias


def write_layer_cases(folder, spec, ref, batch=None, seed=0):
    """quantize, conv2d_quantized, add_bias and relu of one layer, each as a case of its own; returns the folder names."""
    name, n, c, hw, o, k, stride, pad = spec
    n = batch or n
    x, scale, w, dq, bias = layer_tensors(n, c, hw, o, k, seed)
    scales = np.full(n, scale, dtype=np.float32)
    xq = ref.quantize(x, scales)
    y = ref.conv2d_quantized(xq, w, (pad,) * 4, (stride,) * 2, (1, 1), dq)
    yb = ref.add_bias(y, bias)
    yr = np.maximum(yb, np.float32(0))
    out = []
    tsfile.write_case(os.path.join(folder, name + ".quantize"), "quantize", {"quantize_scale": scales}, [x], [xq])
    out.append(name + ".quantize")
    tsfile.write_case(os.path.join(folder, name + ".conv2d_quantized"), "conv2d_quantized", tsfile.conv_attributes(pad, stride, dq),
                      [xq, w], [y])
    out.append(name + ".conv2d_quantized")
    tsfile.write_case(os.path.join(folder, name + ".add_bias"), "add_bias", {"format": "NCHW"}, [y, bias], [yb])
    out.append(name + ".add_bias")
    tsfile.write_case(os.path.join(folder, name + ".relu"), "relu", {}, [yb], [yr])
    out.append(name + ".relu")
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("folder")
    ap.add_argument("--batch", type=int, default=None, help="override the batch of every case (default: 1 and 32 as configured)")
    args = ap.parse_args()
    ref = orc.Reference(threads=1)
    names = []
    for spec in [CONFIG0] + CONFIG1:
        names += write_layer_cases(args.folder, spec, ref, args.batch)
    print("\n".join(names))


if __name__ == "__main__":
    main()
