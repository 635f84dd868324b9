"""Host-buffer execution: ctypes over the library's pipelined upload | kernel | download path
(tcab_pipeline_*, include/tcab.h), plus the single-process multi-device driver (tcab_multi_*).

The reference's launchers take device tensors and leave the copies to the caller; its runners copy whole
tensors around the launch (testing/runners/common.cuh:72-90). Here a problem in page-locked host memory is
cut into chunks of its independent axis (rows / batch / rows of a) and the three stages of successive
chunks overlap on three streams that the library owns. Everything that moves or computes is in
libtcab.so; torch only supplies the pinned host tensors and, for operands that stay on the device
(gamma / beta, b / bias), the device tensors.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from .ops import _DTYPES, _chain, _view

_ELEM = {_lib.F32: 4, _lib.BF16: 2, _lib.I32: 4, _lib.U32: 4}
_OPS = {"softmax_rows": _lib.OP_SOFTMAX_ROWS, "layernorm_rows": _lib.OP_LAYERNORM_ROWS,
        "reduce_outer": _lib.OP_REDUCE_OUTER, "chain_reduce": _lib.OP_CHAIN_REDUCE,
        "gemm_bias_act": _lib.OP_GEMM_BIAS_ACT, "map": _lib.OP_MAP}
_OUTER_BITS = {"sum": 1, "max": 2, "argmax": 4}


class PipelineSpec:
    """A filled-in tcab_pipeline_desc together with the Python objects it points to."""

    def __init__(self, op: str, device, chunk_units: int, unit_shape: Sequence[int], in_dtype: torch.dtype, *,
                 depth: int = 4, n_streamed: int = 1, outputs: Sequence[str] = ("sum", "max", "argmax"),
                 out_dtype: Optional[torch.dtype] = None, act: str = "relu", eps: float = 1e-5,
                 map_expr: Optional[str] = None, combine_expr: str = "(p0 + p1)", post_expr: Optional[str] = None,
                 init: float = 0.0, captures: Sequence[float] = (), resident: Sequence[Optional[torch.Tensor]] = ()):
        if op not in _OPS:
            raise ValueError(f"unknown operator {op!r}")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ValueError("a pipeline runs on a CUDA device (this library has no CPU path)")
        self.op = op
        self.device = torch.device("cuda", dev.index if dev.index is not None else torch.cuda.current_device())
        self.unit_shape = tuple(int(d) for d in unit_shape)
        self.in_dtype = in_dtype
        self.n_streamed = n_streamed
        self.outputs = tuple(outputs) if op == "reduce_outer" else ()
        d = _lib.PipelineDesc()
        d.op = _OPS[op]
        d.device = self.device.index
        d.chunk_units = chunk_units
        d.depth = depth
        d.in_dtype = _DTYPES[in_dtype]
        d.n_streamed = n_streamed
        d.unit_rank = len(self.unit_shape)
        if not 1 <= d.unit_rank <= _lib.MAX_RANK - 1:
            raise ValueError(f"a unit has rank 1..{_lib.MAX_RANK - 1}")
        for i, e in enumerate(self.unit_shape):
            d.unit_dims[i] = e
        d.outputs = sum(_OUTER_BITS[o] for o in self.outputs)
        d.out_dtype = _DTYPES[out_dtype if out_dtype is not None else in_dtype]
        d.act = {"none": _lib.ACT_NONE, "relu": _lib.ACT_RELU}[act]
        d.eps = eps
        self._chain = None
        if map_expr is not None:
            self._chain = _chain(map_expr, combine_expr, post_expr, init, captures)
            d.chain = C.pointer(self._chain)
        self._resident = list(resident)
        for i, t in enumerate(self._resident[:2]):
            if t is None:
                continue
            if t.device != self.device:
                raise ValueError(f"resident[{i}] is on {t.device}, the pipeline on {self.device}")
            d.resident[i] = _view(t, f"resident[{i}]")
        self.desc = d
        # what one unit produces, per output: (elements, element size)
        unit = 1
        for e in self.unit_shape:
            unit *= e
        self.unit_elems = unit
        if op == "reduce_outer":
            self.out_units = [(self.unit_shape[-1], 4)] * len(self.outputs)
        elif op == "chain_reduce":
            self.out_units = [(1, 4)]
        elif op == "gemm_bias_act":
            self.out_units = [(int(self._resident[0].shape[1]), 2)]
        else:
            self.out_units = [(unit, _ELEM[d.out_dtype if op == "map" else d.in_dtype])]


def _host_ptr(t: torch.Tensor, name: str, nbytes: int) -> int:
    if t.device.type != "cpu" or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous host tensor")
    if t.numel() * t.element_size() < nbytes:
        raise ValueError(f"{name} holds {t.numel() * t.element_size()} bytes, the run needs {nbytes}")
    return t.data_ptr()


def _host_args(spec: PipelineSpec, host_ins, host_outs, units: int):
    host_ins, host_outs = list(host_ins), list(host_outs)
    if len(host_ins) != spec.n_streamed or len(host_outs) != len(spec.out_units):
        raise ValueError(f"the run takes {spec.n_streamed} input and {len(spec.out_units)} output buffer(s)")
    in_bytes = units * spec.unit_elems * _ELEM[spec.desc.in_dtype]
    ins = (C.c_void_p * len(host_ins))(*[_host_ptr(t, f"host_ins[{i}]", in_bytes) for i, t in enumerate(host_ins)])
    outs = (C.c_void_p * len(host_outs))(*[_host_ptr(t, f"host_outs[{i}]", units * n * sz)
                                           for i, (t, (n, sz)) in enumerate(zip(host_outs, spec.out_units))])
    return ins, outs


class Pipeline:
    """One tcab_pipeline: reusable streams, staging slots and events for one operator and unit shape."""

    def __init__(self, spec: PipelineSpec):
        self.spec = spec
        self._h = C.c_void_p()
        _lib.check(_lib.load().tcab_pipeline_create(C.byref(spec.desc), C.byref(self._h)))

    def run(self, host_ins: Sequence[torch.Tensor], host_outs: Sequence[torch.Tensor], units: Optional[int] = None) -> None:
        """Queue `units` units (default: all of host_ins[0]). Returns with the work queued; pin the buffers."""
        if units is None:
            units = host_ins[0].numel() // self.spec.unit_elems
        ins, outs = _host_args(self.spec, host_ins, host_outs, units)
        _lib.check(_lib.load().tcab_pipeline_run(self._h, ins, units, outs))

    def order_after(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream(self.spec.device)
        _lib.check(_lib.load().tcab_pipeline_order_after(self._h, C.c_void_p(s.cuda_stream)))

    def join(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """The given (default: current) stream waits for every chunk queued so far."""
        s = stream if stream is not None else torch.cuda.current_stream(self.spec.device)
        _lib.check(_lib.load().tcab_pipeline_join(self._h, C.c_void_p(s.cuda_stream)))

    def sync(self) -> None:
        _lib.check(_lib.load().tcab_pipeline_sync(self._h))

    def close(self) -> None:
        if self._h:
            _lib.load().tcab_pipeline_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MultiDevice:
    """One problem in host memory cut over several devices of this process (tcab_multi): device r of n takes the
    contiguous block shard.block(units, n, r) of the independent axis through its own pipeline. specs[r] names
    device r and holds that device's copies of the resident operands. No collective is involved."""

    def __init__(self, specs: Sequence[PipelineSpec]):
        self.specs = list(specs)
        arr = (_lib.PipelineDesc * len(self.specs))(*[s.desc for s in self.specs])
        self._h = C.c_void_p()
        _lib.check(_lib.load().tcab_multi_create(arr, len(self.specs), C.byref(self._h)))

    def run(self, host_ins: Sequence[torch.Tensor], host_outs: Sequence[torch.Tensor], units: Optional[int] = None) -> None:
        spec = self.specs[0]
        if units is None:
            units = host_ins[0].numel() // spec.unit_elems
        ins, outs = _host_args(spec, host_ins, host_outs, units)
        _lib.check(_lib.load().tcab_multi_run(self._h, ins, units, outs))

    def sync(self) -> None:
        _lib.check(_lib.load().tcab_multi_sync(self._h))

    def close(self) -> None:
        if self._h:
            _lib.load().tcab_multi_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
