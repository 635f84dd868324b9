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
    ("tcab_module_parse_files", C.c_int,
     [C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), C.c_uint32, C.c_char_p, C.POINTER(C.c_void_p)]),
    ("tcab_module_free", None, [C.c_void_p]),
    ("tcab_module_kernel_count", C.c_uint32, [C.c_void_p]),
    ("tcab_module_kernel_name", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_kernel_output", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_kernel_class", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_kernel_describe", C.c_char_p, [C.c_void_p, C.c_uint32]),
    ("tcab_module_kernel_signature", C.c_char_p, [C.c_void_p, C.c_uint32]),
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

    def __init__(self, text: Optional[str] = None, files: Optional[Dict[str, str]] = None, root: Optional[str] = None):
        """Module(text) parses one text; Module(files={path: text, ...}, root=path) a module spread over several
        files whose @include paths are resolved among `files` (tcab_module_parse_files)."""
        self._h = C.c_void_p()
        if files is not None:
            if root is None:
                raise ValueError("a module of several files needs the path of its root file")
            paths = (C.c_char_p * len(files))(*[p.encode() for p in files])
            texts = (C.c_char_p * len(files))(*[t.encode("utf-8") for t in files.values()])
            _check(load().tcab_module_parse_files(paths, texts, len(files), root.encode(), C.byref(self._h)))
        else:
            if text is None:
                raise ValueError("Module needs a text or a set of files")
            _check(load().tcab_module_parse(text.encode("utf-8"), C.byref(self._h)))
        lib = load()
        self.kernels: Dict[str, Dict[str, Optional[str]]] = {}
        for i in range(lib.tcab_module_kernel_count(self._h)):
            cls = lib.tcab_module_kernel_class(self._h, i)
            self.kernels[lib.tcab_module_kernel_name(self._h, i).decode()] = {
                "output": lib.tcab_module_kernel_output(self._h, i).decode(),
                "class": cls.decode() if cls is not None else None,
            }

    @classmethod
    def from_path(cls, path: str) -> "Module":
        """Reads `path` and every file it includes, transitively, from disk (the host owns file I/O) and parses them
        as one module. Include paths are relative to the including file, as in the reference's loader."""
        import os
        import re
        files: Dict[str, str] = {}
        todo = [os.path.normpath(path)]
        while todo:
            p = todo.pop()
            if p in files:
                continue
            with open(p) as f:
                files[p] = f.read()
            for inc in re.findall(r'@include\s+"([^"]+)"\s*;', files[p]):
                q = os.path.normpath(os.path.join(os.path.dirname(p), inc))
                if os.path.exists(q):      # a missing file is the parser's diagnostic to give, with its position
                    todo.append(q)
        return cls(files=files, root=os.path.normpath(path))

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

    def _extents(self, kernel: str, tensors: dict) -> Dict[str, int]:
        """Symbolic dim name -> extent, from the bound tensors of a kernel's signature (tcab_module_kernel_signature)."""
        sig = load().tcab_module_kernel_signature(self._h, list(self.kernels).index(kernel))
        ext: Dict[str, int] = {}
        for line in (sig.decode().splitlines() if sig else []):
            name, _, rest = line.partition("=")
            if name in tensors and "[" in rest:
                dims = rest.rstrip("]").split("[")[1].split(",")
                for d, e in zip(dims, tensors[name].shape):
                    if d and not d.isdigit():
                        ext.setdefault(d, int(e))
        return ext

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
        tensors = dict(tensors)
        # intermediates between statements: the caller owns their memory too; whatever is not bound is taken from
        # torch here, with the extents of the dims as the bound tensors fix them
        info = self.describe(kernel)
        missing = [n for n in info.get("locals", "").split(",") if n and n not in tensors]
        if missing:
            extents = self._extents(kernel, tensors)
            ref0 = next(iter(tensors.values()))
            for n in missing:
                elem, dims = info["local." + n].rstrip("]").split("[")
                shape = [int(d) if d.isdigit() else extents[d] for d in dims.split(",") if d]
                dt = {"f32": torch.float32, "bf16": torch.bfloat16, "i32": torch.int32, "u32": torch.uint32}[elem]
                tensors[n] = torch.empty(shape, device=ref0.device, dtype=dt)
        tnames = (C.c_char_p * len(tensors))(*[n.encode() for n in tensors])
        tviews = (_lib.Tensor * len(tensors))(*[_view(t, n) for n, t in tensors.items()])
        snames = (C.c_char_p * max(len(scalars), 1))(*[n.encode() for n in scalars])
        svals = (C.c_float * max(len(scalars), 1))(*[float(v) for v in scalars.values()])
        ref = next(iter(tensors.values()))
        assert isinstance(ref, torch.Tensor)
        with _on_device(ref):
            _check(load().tcab_module_launch(self._h, kernel.encode(), tnames, tviews, len(tensors), snames, svals,
                                             len(scalars), _stream(stream, ref)))
