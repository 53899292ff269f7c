"""Compile libtennis_b200.so for sm_100a with nvcc (cross-compiles without a GPU)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))


def build(verbose=False):
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), "-j4"]
    out = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or out.returncode != 0:
        print(out.stdout)
    if out.returncode != 0:
        raise RuntimeError("building libtennis_b200.so failed")
    return os.path.join(_HERE, "libtennis_b200.so")


if __name__ == "__main__":
    print(build(verbose=True))
