"""Elementwise evaluation of a lambda on the host: the oracle of the map-only operator.

Test infrastructure only. The reference has no evaluator; what it does with a map lambda is to print
it as a C++ expression into a translation unit (internal/cg/cxx/expr.go:14-101, operator spellings
internal/cg/cxx/naming.go:126-198) and let the C++ compiler give it its meaning. This module does the
same on the host: the caller's expression text -- not the kernel library's canonical form of it, so
that the library's parser is not part of its own check -- is pasted into a loop over the elements,
compiled with g++ (-ffp-contract=off: IEEE per operation, no FMA contraction) and run on numpy arrays.
Operands p0.. carry their array's element type (float32, int32, uint32, or uint16 holding bf16 bit
patterns), captures c0.. are float. bf16 is a storage type with explicit conversions only
(design/syntax-design.md:601-607); a conversion to bf16 rounds to nearest even, as the device does.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CACHE = os.path.join(_HERE, "_lambda")

_PRELUDE = r"""
#include <cmath>
#include <cstdint>
#include <cstring>
struct bf16v {
  uint16_t bits;
  bf16v() : bits(0) {}
  explicit bf16v(float f) {
    uint32_t u; std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) bits = (uint16_t)((u >> 16) | 0x0040u);
    else bits = (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
  }
  explicit operator float() const { uint32_t u = ((uint32_t)bits) << 16; float f; std::memcpy(&f, &u, 4); return f; }
  explicit operator int32_t() const { return (int32_t)(float)(*this); }
  explicit operator uint32_t() const { return (uint32_t)(float)(*this); }
};
typedef bf16v __nv_bfloat16;
template <class T> static inline float f32(T x) { return static_cast<float>(x); }
template <class T> static inline bf16v bf16(T x) { return static_cast<bf16v>(x); }
template <class T> static inline int32_t i32(T x) { return static_cast<int32_t>(x); }
template <class T> static inline uint32_t u32(T x) { return static_cast<uint32_t>(x); }
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline uint32_t umin(uint32_t a, uint32_t b) { return a < b ? a : b; }
static inline uint32_t umax(uint32_t a, uint32_t b) { return a > b ? a : b; }
"""

_CXX = {np.dtype(np.float32): "float", np.dtype(np.int32): "int32_t", np.dtype(np.uint32): "uint32_t",
        np.dtype(np.uint16): "bf16v"}


def _build(expr: str, in_types, out_type) -> C.CDLL:
    src = _PRELUDE + 'extern "C" void eval(const void* const* ins, void* out, uint64_t n, const float* c) {\n'
    for i, t in enumerate(in_types):
        src += f"  const {t}* in{i} = static_cast<const {t}*>(ins[{i}]);\n"
    src += f"  {out_type}* o = static_cast<{out_type}*>(out);\n"
    src += "".join(f"  const float c{i} = c[{i}]; (void)c{i};\n" for i in range(8))
    src += "  for (uint64_t i = 0; i < n; ++i) {\n"
    for i, t in enumerate(in_types):
        src += f"    const {t} p{i} = in{i}[i];\n"
    src += f"    o[i] = ({expr});\n  }}\n}}\n"
    key = hashlib.sha256(src.encode()).hexdigest()[:24]
    so = os.path.join(_CACHE, key + ".so")
    if not os.path.exists(so):
        os.makedirs(_CACHE, exist_ok=True)
        with tempfile.TemporaryDirectory() as d:
            cpp = os.path.join(d, "lambda.cpp")
            with open(cpp, "w") as f:
                f.write(src)
            tmp = os.path.join(d, "lambda.so")
            r = subprocess.run(["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
                                "-o", tmp, cpp], capture_output=True, text=True)
            if r.returncode != 0:
                raise ValueError(f"the host compiler refuses the lambda {expr!r}:\n{r.stderr[-1500:]}")
            os.replace(tmp, so)
    return C.CDLL(so)


def evaluate(expr: str, ins, captures=(), out_dtype=np.float32) -> np.ndarray:
    """out[i] = expr(ins[0][i], ins[1][i], ...) for identically shaped arrays; bf16 as uint16 bit patterns."""
    ins = [np.ascontiguousarray(a) for a in ins]
    shape = ins[0].shape
    for a in ins:
        if a.shape != shape:
            raise ValueError("operands of a map share one shape")
    out = np.empty(shape, dtype=out_dtype)
    lib = _build(expr, [_CXX[a.dtype] for a in ins], _CXX[np.dtype(out_dtype)])
    ptrs = (C.c_void_p * len(ins))(*[a.ctypes.data for a in ins])
    caps = (C.c_float * 8)(*(list(captures) + [0.0] * (8 - len(captures))))
    lib.eval(ptrs, C.c_void_p(out.ctypes.data), C.c_uint64(out.size), caps)
    return out
