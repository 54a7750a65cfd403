"""Makes tests/golden/primitives.json: outputs of the reference's own C primitives on fixed inputs.

computerex/dlgo's model code is Go (no toolchain here), but the C kernels its forward pass calls on
amd64 (quant/simd_dot.c: vec_softmax :940, vec_swiglu :911, vec_dot_f32 :991, vec_scale_add :1033)
compile with gcc.  This script compiles that file into a shared library in a temporary folder, runs
the four primitives on seeded inputs and stores inputs and outputs.  They use a 5-digit polynomial
exp (quant/simd_dot.c:874-905), so tests compare at 1e-4 relative, not bit for bit.

    python tests/golden/make_primitives.py /path/to/dlgo
"""
import ctypes
import json
import os
import random
import subprocess
import sys
import tempfile


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref = sys.argv[1]
    src = os.path.join(ref, "quant", "simd_dot.c")
    with tempfile.TemporaryDirectory() as tmp:
        so = os.path.join(tmp, "simd_dot.so")
        subprocess.check_call(["gcc", "-O2", "-mavx2", "-mfma", "-mf16c", "-shared", "-fPIC", "-o", so, src, "-lm"])
        lib = ctypes.CDLL(so)
        lib.vec_dot_f32.restype = ctypes.c_float
        rnd = random.Random(20240501)
        f32 = lambda v: ctypes.c_float(v).value

        def arr(vals):
            return (ctypes.c_float * len(vals))(*vals)

        out = {"source": "computerex/dlgo quant/simd_dot.c compiled with gcc -O2 -mavx2 -mfma", "cases": []}
        for n in (1, 7, 8, 33, 64, 200):
            x = [f32(rnd.uniform(-6, 6)) for _ in range(n)]
            g = [f32(rnd.uniform(-8, 8)) for _ in range(n)]
            u = [f32(rnd.uniform(-3, 3)) for _ in range(n)]
            sm = arr(x)
            lib.vec_softmax(sm, ctypes.c_int(n))
            sw = arr([0.0] * n)
            lib.vec_swiglu(sw, arr(g), arr(u), ctypes.c_int(n))
            dot = lib.vec_dot_f32(arr(g), arr(u), ctypes.c_int(n))
            acc = arr(x)
            lib.vec_scale_add(acc, ctypes.c_float(0.375), arr(u), ctypes.c_int(n))
            out["cases"].append({"n": n, "x": x, "gate": g, "up": u, "softmax": list(sm), "swiglu": list(sw),
                                 "dot": dot, "scale_add_0.375": list(acc)})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "primitives.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
