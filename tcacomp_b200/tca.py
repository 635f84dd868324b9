"""Kernels written in the reference's .tca text language, parsed at run time and launched by name.

One-to-one with include/tcab_host.h (libtcab_host.so): `Module(text)` is tcab_module_parse, `launch` is
tcab_module_launch. The reference compiles the same text ahead of time into a <Name>Launch function
(internal/syntax/build/build.go:27-36, internal/cg/cxx/launch.go:23-156); tensors and scalar parameters are
bound here by the names the kernel's signature gives them, the output by the name of the returned `let`.
Parsing needs no GPU; launching has no CPU path.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional

from . import _lib

HOST_LIB_PATH = os.path.join(_lib.HERE, "libtcab_host.so")

# Every symbol include/tcab_host.h declares: (name, restype, argtypes).
SYMBOLS = [
    ("tcab_module_parse", C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    ("tcab_module_free", None, [C.c_void_p]),
    ("tcab_module_kernel_count", C.c_uint32, [C.c_void_p]),
    ("tcab_module_kernel_name", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_kernel_output", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_kernel_class", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_kernel_describe", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_launch", C.c_int,
     [C.c_void_p, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(_lib.Tensor), C.c_uint32, C.POINTER(C.c_char_p),
      C.POINTER(C.c_float), C.c_uint32, C.c_void_p]),
    ("tcab_host_last_error", C.c_char_p, []),
]

_host = None


def load() -> C.CDLL:
    """Load libtcab_host.so (which links libtcab.so) and bind every declared symbol."""
    global _host
    if _host is not None:
        return _host
    _lib.load()
    if not os.path.exists(HOST_LIB_PATH):
        raise ImportError(f"{HOST_LIB_PATH} is missing: build it with `python -m tcacomp_b200.build`")
    lib = C.CDLL(HOST_LIB_PATH)
    for name, restype, argtypes in SYMBOLS:
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _host = lib
    return lib


def _check(status: int) -> None:
    if status != _lib.OK:
        raise _lib.TcabError(status, load().tcab_host_last_error().decode("utf-8", "replace"))


class Module:
    """A parsed .tca module. `kernels` maps each launcher name to {"output": ..., "class": ...}."""

    def __init__(self, text: str):
        self._h = C.c_void_p()
        _check(load().tcab_module_parse(text.encode("utf-8"), C.byref(self._h)))
        lib = load()
        self.kernels: Dict[str, Dict[str, Optional[str]]] = {}
        for i in range(lib.tcab_module_kernel_count(self._h)):
            cls = lib.tcab_module_kernel_class(self._h, i)
            self.kernels[lib.tcab_module_kernel_name(self._h, i).decode()] = {
                "output": lib.tcab_module_kernel_output(self._h, i).decode(),
                "class": cls.decode() if cls is not None else None,
            }

    def __del__(self):
        if getattr(self, "_h", None) is not None and self._h.value and _host is not None:
            _host.tcab_module_free(self._h)
            self._h = C.c_void_p()

    def describe(self, kernel: str) -> Dict[str, str]:
        """What `kernel` lowers to: class, tensor names and, for the chain classes, the canonical lambda texts,
        init, capture names and the reduced axis (tcab_module_kernel_describe)."""
        i = list(self.kernels).index(kernel)
        text = load().tcab_module_kernel_describe(self._h, i)
        if text is None:
            raise _lib.TcabError(_lib.ERR_UNSUPPORTED, load().tcab_host_last_error().decode("utf-8", "replace"))
        return dict(line.split("=", 1) for line in text.decode().splitlines() if "=" in line)

    def names(self) -> List[str]:
        return list(self.kernels)

    def launch(self, kernel: str, tensors: dict, scalars: Optional[dict] = None, stream=None) -> None:
        """Launch `kernel` asynchronously. `tensors`: name -> torch CUDA tensor, the output included (under
        the name of the returned `let`); `scalars`: name -> float."""
        import torch

        from .ops import _on_device, _stream, _view
        scalars = scalars or {}
        if not tensors:
            raise ValueError("launch: no tensors bound")
        tnames = (C.c_char_p * len(tensors))(*[n.encode() for n in tensors])
        tviews = (_lib.Tensor * len(tensors))(*[_view(t, n) for n, t in tensors.items()])
        snames = (C.c_char_p * max(len(scalars), 1))(*[n.encode() for n in scalars])
        svals = (C.c_float * max(len(scalars), 1))(*[float(v) for v in scalars.values()])
        ref = next(iter(tensors.values()))
        assert isinstance(ref, torch.Tensor)
        with _on_device(ref):
            _check(load().tcab_module_launch(self._h, kernel.encode(), tnames, tviews, len(tensors), snames, svals,
                                             len(scalars), _stream(stream, ref)))
