"""Makes tests/golden/linear_golden.json from the reference's own C operator.

The reference's model code is Rust and cannot be built without a Rust toolchain,
so the plain implementation rests on the formulas.  The one piece of reference
code that does build with a C compiler is its CPU ``linear`` plugin
(native/cpu/safetyraise_cpu.c), the operator every projection of the model goes
through.  This script compiles that file unchanged into a temporary folder,
runs it on a small seeded case (float32 and float16 weights) and on the
reference's own round-trip case (src/backend/mod.rs:705-726), and stores inputs
and outputs.  tests/test_plain.py checks the plain ``linear`` against them.

    python tests/golden/make_linear_golden.py /path/to/reference
"""
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile

import numpy as np


class Options(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("struct_size", C.c_uint32), ("flags", C.c_uint64)]


def main(ref):
    tmp = tempfile.mkdtemp()
    so = os.path.join(tmp, "libsafetyraise_cpu.so")
    subprocess.check_call(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-I", os.path.join(ref, "native/include"),
                           os.path.join(ref, "native/cpu/safetyraise_cpu.c"), "-o", so, "-lm"])
    lib = C.CDLL(so)
    lib.safetyraise_kernel_abi_version.restype = C.c_uint32
    ctx = C.c_void_p()
    opts = Options(lib.safetyraise_kernel_abi_version(), C.sizeof(Options), 0)
    assert lib.safetyraise_kernel_create_context(C.byref(opts), C.byref(ctx)) == 0

    def linear(w, x, dtype_code):
        rows, cols = w.shape
        raw = w.tobytes()
        handle = C.c_void_p()
        assert lib.safetyraise_kernel_create_weight(ctx, raw, C.c_uint64(len(raw)), C.c_uint64(rows),
                                                    C.c_uint64(cols), C.c_uint32(dtype_code), C.byref(handle)) == 0
        out = np.zeros((x.shape[0], rows), dtype=np.float32)
        xin = np.ascontiguousarray(x, dtype=np.float32)
        assert lib.safetyraise_kernel_linear(ctx, handle, xin.ctypes.data_as(C.POINTER(C.c_float)),
                                             C.c_uint64(x.shape[0]), C.c_uint64(cols),
                                             out.ctypes.data_as(C.POINTER(C.c_float)), C.c_uint64(x.shape[0]),
                                             C.c_uint64(rows)) == 0
        lib.safetyraise_kernel_destroy_weight(ctx, handle)
        return out

    cases = []
    w = np.array([[1, 0, -1], [2, 3, 4]], dtype=np.float32)
    x = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    cases.append({"name": "round_trip", "weight_dtype": "F32", "weight": w.tolist(), "input": x.tolist(),
                  "output": linear(w, x, 1).tolist()})
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, size=(7, 33)).astype(np.float32)
    x = rng.normal(0, 1, size=(5, 33)).astype(np.float32)
    cases.append({"name": "seeded_f32", "weight_dtype": "F32", "weight": w.tolist(), "input": x.tolist(),
                  "output": linear(w, x, 1).tolist()})
    w16 = w.astype(np.float16)
    cases.append({"name": "seeded_f16", "weight_dtype": "F16", "weight": w16.astype(np.float32).tolist(),
                  "input": x.tolist(), "output": linear(w16, x, 2).tolist()})
    lib.safetyraise_kernel_destroy_context(ctx)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "linear_golden.json")
    with open(out, "w") as f:
        json.dump({"source": "native/cpu/safetyraise_cpu.c (safetyraise_kernel_linear)", "cases": cases}, f)
    print("wrote", out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_linear_golden.py <checkout of the reference project>")
    main(sys.argv[1])
