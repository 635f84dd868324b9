"""Operators over torch CUDA tensors; each is exactly one call through the C ABI.

Arguments mirror the reference's generated launchers (inputs, then the output,
then scalars, then the stream -- internal/cg/cxx/launch.go:23-156): the caller
owns all memory, outputs may be passed in to avoid an allocation, calls are
asynchronous on the given (or current) torch stream.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.int32: _lib.I32, torch.uint32: _lib.U32}


_TWO32 = 2 ** 32


def _name(name) -> str:
    return name if isinstance(name, str) else f"ins[{name}]"


def _view(t: torch.Tensor, name) -> _lib.Tensor:
    """The C view of a tensor. `name` is used in error messages only: a string, or the operand's index."""
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{_name(name)} must be a torch.Tensor")
    shape = t.shape
    rank = len(shape)
    # the C struct holds 32-bit extents and ctypes would truncate silently: refuse here what the library
    # refuses with TCAB_ERR_TOO_LARGE (the reference indexes with u32); an element count below 2^32 bounds
    # every extent of a non-empty tensor
    if t.numel() >= _TWO32 or (rank and max(shape) >= _TWO32):
        raise ValueError(f"{_name(name)}: 2^32 or more elements ({tuple(shape)}); extents and element counts are 32-bit")
    if not t.is_cuda:
        raise ValueError(f"{_name(name)} must live on a CUDA device (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{_name(name)} must be contiguous (row-major), as the reference's tensors are")
    code = _DTYPES.get(t.dtype)
    if code is None:
        raise TypeError(f"{_name(name)}: unsupported dtype {t.dtype}")
    if rank < 1 or rank > _lib.MAX_RANK:
        raise ValueError(f"{_name(name)}: rank {rank} outside 1..{_lib.MAX_RANK}")
    v = _lib.Tensor()
    v.data = t.data_ptr()
    v.dtype = code
    v.rank = rank
    v.dims[:rank] = shape
    return v


def _stream(stream: Optional[torch.cuda.Stream], ref: torch.Tensor) -> C.c_void_p:
    if stream is not None:
        return C.c_void_p(stream.cuda_stream)
    # the raw handle of torch's current stream on the operand's device (what torch.cuda.current_stream wraps)
    return C.c_void_p(torch._C._cuda_getCurrentRawStream(ref.device.index))


class _AlreadyCurrent:
    """Stands in for torch.cuda.device when the operand's device is the current one already (the usual case)."""

    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_ALREADY_CURRENT = _AlreadyCurrent()


def _on_device(t: torch.Tensor):
    dev = t.device
    if dev.index == torch.cuda.current_device():
        return _ALREADY_CURRENT
    return torch.cuda.device(dev)


def _same_device(*named) -> None:
    """Every tensor of one call lives on the first one's device (the call runs there, on its stream)."""
    first_name, first = named[0]
    for name, t in named[1:]:
        if t is not None and t.device != first.device:
            raise ValueError(f"{name} is on {t.device} but {first_name} is on {first.device}")


def _operands_on_one_device(ins, out) -> None:
    """_same_device for a list of operands and an output, without building names unless something is wrong."""
    dev = ins[0].device
    if out.device == dev and all(t.device == dev for t in ins):
        return
    _same_device(*[(f"ins[{i}]", t) for i, t in enumerate(ins)], ("out", out))


_ENCODED: dict = {}


def _encoded(text: str) -> bytes:
    """The lambda text as bytes; a program uses a handful of lambdas, many times each."""
    b = _ENCODED.get(text)
    if b is None:
        if len(_ENCODED) > 4096:
            _ENCODED.clear()
        b = _ENCODED[text] = text.encode()
    return b


def _chain(map_expr: str, combine_expr: str, post_expr: Optional[str], init: float,
           captures: Sequence[float]) -> _lib.Chain:
    if len(captures) > _lib.MAX_CAPTURES:
        raise ValueError(f"at most {_lib.MAX_CAPTURES} captures")
    chain = _lib.Chain()
    chain.map_expr = _encoded(map_expr)
    chain.combine_expr = _encoded(combine_expr)
    chain.post_expr = _encoded(post_expr) if post_expr else None
    chain.init = init
    chain.n_captures = len(captures)
    for i, c in enumerate(captures):
        chain.captures[i] = c
    return chain


def launch_count() -> int:
    """Kernels launched by the library in this process."""
    return int(_lib.load().tcab_launch_count())


def device_status() -> int:
    """0 unless a kernel gave up on a bounded device-side wait (synchronises the device)."""
    v = C.c_int(0)
    _lib.check(_lib.load().tcab_device_status(C.byref(v)))
    return int(v.value)


def tune(family: str, p0: int = 0, p1: int = 0, p2: int = 0, p3: int = 0) -> None:
    """Override (or with zeros, restore) the launch shape of one kernel family."""
    _lib.check(_lib.load().tcab_tune(family.encode(), p0, p1, p2, p3))


def chain_prepare(map_expr: str, n_ins: int = 1, combine_expr: str = "(p0 + p1)", post_expr: Optional[str] = None,
                  captures: Sequence[float] = (), use: str = "reduce", in_dtypes: Optional[Sequence[torch.dtype]] = None,
                  out_dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None) -> None:
    """Compile and load now what the first chain_reduce / chain_contract / map (use = "reduce", "contract",
    "map") with these lambdas and operand types would compile later (nothing to do for lambdas with an
    ahead-of-time kernel). Not during a stream capture."""
    chain = _chain(map_expr, combine_expr, post_expr, 0.0, captures)
    code = {"reduce": _lib.USE_REDUCE, "contract": _lib.USE_CONTRACT, "map": _lib.USE_MAP,
            "reduce_batched": _lib.USE_REDUCE_BATCHED}[use]
    types = None
    if in_dtypes is not None:
        if len(in_dtypes) != n_ins:
            raise ValueError("in_dtypes must name one dtype per operand")
        types = (C.c_int32 * n_ins)(*[_DTYPES[d] for d in in_dtypes])
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _lib.check(_lib.load().tcab_chain_prepare(C.byref(chain), types, n_ins, code, _DTYPES[out_dtype]))


def release_stream(stream: Optional[torch.cuda.Stream] = None, device: Optional[torch.device] = None) -> None:
    """Free the scratch the library allocated for launches on `stream` (default: the current stream)."""
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    s = stream if stream is not None else torch.cuda.current_stream(dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().tcab_release_stream(C.c_void_p(s.cuda_stream)))


def release_all() -> None:
    """Free every scratch buffer the library holds, on every device and stream."""
    _lib.check(_lib.load().tcab_release_all())


def softmax_rows(x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Row softmax over the innermost axis (fp32)."""
    if out is None:
        out = torch.empty_like(x)
    xv, yv = _view(x, "x"), _view(out, "out")
    _same_device(("x", x), ("out", out))
    with _on_device(x):
        _lib.check(_lib.load().tcab_softmax_rows(C.byref(xv), C.byref(yv), _stream(stream, x)))
    return out


def layernorm_rows(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5,
                   out: Optional[torch.Tensor] = None,
                   stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Layer-norm over the innermost axis, fp32 statistics, bf16 or fp32 rows."""
    if out is None:
        out = torch.empty_like(x)
    xv, gv, bv, yv = _view(x, "x"), _view(gamma, "gamma"), _view(beta, "beta"), _view(out, "out")
    _same_device(("x", x), ("gamma", gamma), ("beta", beta), ("out", out))
    with _on_device(x):
        _lib.check(_lib.load().tcab_layernorm_rows(C.byref(xv), C.byref(gv), C.byref(bv),
                                                   C.c_float(eps), C.byref(yv), _stream(stream, x)))
    return out


def reduce_outer(t: torch.Tensor, want: Sequence[str] = ("sum", "max", "argmax"),
                 out: Optional[dict] = None, stream: Optional[torch.cuda.Stream] = None) -> dict:
    """Reduce t[b, k, c] over k in one pass; returns {"sum", "max", "argmax"} as requested."""
    if t.dim() != 3:
        raise ValueError("t must be rank 3 [b, k, c]")
    res = dict(out or {})
    for name in want:
        if name not in ("sum", "max", "argmax"):
            raise ValueError(f"unknown output {name!r}")
        if name not in res:
            res[name] = torch.empty((t.shape[0], t.shape[2]), device=t.device,
                                    dtype=torch.int32 if name == "argmax" else torch.float32)
    tv = _view(t, "t")
    views = {k: _view(v, k) for k, v in res.items()}
    _same_device(("t", t), *res.items())

    def ref(k):
        return C.byref(views[k]) if k in views else None

    with _on_device(t):
        _lib.check(_lib.load().tcab_reduce_outer(C.byref(tv), ref("sum"), ref("max"), ref("argmax"),
                                                 _stream(stream, t)))
    return res


def chain_reduce(ins: Sequence[torch.Tensor], map_expr: str, combine_expr: str = "(p0 + p1)",
                 init: float = 0.0, post_expr: Optional[str] = None, captures: Sequence[float] = (),
                 axis: int = -1, out: Optional[torch.Tensor] = None,
                 stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """map | reduce | [map] over one axis of identically shaped fp32 operands.

    The lambdas are C expressions over p0.. (operands), c0.. (captures) in the
    reference's operator and builtin vocabulary, e.g. map_expr="(p0 * p1)".
    """
    ins = list(ins)
    if not 1 <= len(ins) <= _lib.MAX_INPUTS:
        raise ValueError(f"between 1 and {_lib.MAX_INPUTS} operands are required")
    t0 = ins[0]
    ax = axis % t0.dim()
    if out is None:
        # the iteration shape: per axis the largest extent among the operands (an operand may have extent 1 along
        # the innermost axis, or along every other axis)
        full = [max(t.shape[i] for t in ins if t.dim() == t0.dim()) for i in range(t0.dim())]
        shape = [d for i, d in enumerate(full) if i != ax] or [1]
        out = torch.empty(shape, device=t0.device, dtype=torch.float32)
    chain = _chain(map_expr, combine_expr, post_expr, init, captures)
    arr = (_lib.Tensor * len(ins))(*[_view(t, i) for i, t in enumerate(ins)])
    ov = _view(out, "out")
    _operands_on_one_device(ins, out)
    with _on_device(t0):
        _lib.check(_lib.load().tcab_chain_reduce(C.byref(chain), arr, len(ins), ax, C.byref(ov),
                                                 _stream(stream, t0)))
    return out


class BoundChainReduce:
    """tcab_chain_reduce with its descriptors built once and launched many times: the counterpart of a host that keeps
    its tca::Tensor views (runtime/tca/tensor.h:16-40) and calls the generated launcher in a loop, as the reference's
    runners do (testing/runners/common.cuh). Every call is one library call on the current (or the given) stream; the
    object keeps the operands and the output alive, and the caller must not resize them while it is in use."""

    def __init__(self, ins: Sequence[torch.Tensor], map_expr: str, combine_expr: str = "(p0 + p1)", init: float = 0.0,
                 post_expr: Optional[str] = None, captures: Sequence[float] = (), axis: int = -1,
                 out: Optional[torch.Tensor] = None):
        ins = list(ins)
        if not 1 <= len(ins) <= _lib.MAX_INPUTS:
            raise ValueError(f"between 1 and {_lib.MAX_INPUTS} operands are required")
        t0 = ins[0]
        ax = axis % t0.dim()
        if out is None:
            full = [max(t.shape[i] for t in ins if t.dim() == t0.dim()) for i in range(t0.dim())]
            out = torch.empty([d for i, d in enumerate(full) if i != ax] or [1], device=t0.device, dtype=torch.float32)
        self._chain = _chain(map_expr, combine_expr, post_expr, init, captures)
        self._arr = (_lib.Tensor * len(ins))(*[_view(t, i) for i, t in enumerate(ins)])
        self._ov = _view(out, "out")
        _operands_on_one_device(ins, out)
        self._ins, self.out = ins, out
        self._dev = t0.device.index
        self._fn = _lib.load().tcab_chain_reduce
        self._args = (C.byref(self._chain), self._arr, len(ins), ax, C.byref(self._ov))

    def __call__(self, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        raw = stream.cuda_stream if stream is not None else torch._C._cuda_getCurrentRawStream(self._dev)
        if torch.cuda.current_device() == self._dev:
            rc = self._fn(*self._args, C.c_void_p(raw))
        else:
            with torch.cuda.device(self._dev):
                rc = self._fn(*self._args, C.c_void_p(raw))
        if rc:
            _lib.check(rc)
        return self.out


def map(ins: Sequence[torch.Tensor], map_expr: str, captures: Sequence[float] = (),  # noqa: A001 (the operator's name)
        out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
        stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Map-only chain with a rank-preserving store: out[...] = map_expr(ins[0][...], ins[1][...], ...).

    Operands may be f32, bf16, i32 or u32; the lambda sees each with its own type and must yield exactly the
    output's element type (out.dtype, or out_dtype, default: that of ins[0]). They share the output's shape; an
    operand may instead have extent 1 along the innermost axis (one value per row, shape [..., 1]) or along every
    other axis (one row shared by all rows, shape [1, ..., C])."""
    ins = list(ins)
    if not 1 <= len(ins) <= _lib.MAX_INPUTS:
        raise ValueError(f"between 1 and {_lib.MAX_INPUTS} operands are required")
    if out is None:
        full = [max(t.shape[i] for t in ins if t.dim() == ins[0].dim()) for i in range(ins[0].dim())]
        out = torch.empty(full, device=ins[0].device, dtype=out_dtype or ins[0].dtype)
    chain = _chain(map_expr, "(p0 + p1)", None, 0.0, captures)
    arr = (_lib.Tensor * len(ins))(*[_view(t, i) for i, t in enumerate(ins)])
    ov = _view(out, "out")
    _operands_on_one_device(ins, out)
    with _on_device(ins[0]):
        _lib.check(_lib.load().tcab_map(C.byref(chain), arr, len(ins), C.byref(ov), _stream(stream, ins[0])))
    return out


def chain_reduce_batched(problems: Sequence[Sequence[torch.Tensor]], map_expr: str, outs: Optional[Sequence[torch.Tensor]] = None,
                         combine_expr: str = "(p0 + p1)", init: float = 0.0, post_expr: Optional[str] = None,
                         captures: Sequence[float] = (), stream: Optional[torch.cuda.Stream] = None) -> list:
    """chain_reduce over the innermost axis for several independent problems of one shape in ONE launch.

    problems[b] lists the operands of problem b; outs[b] receives its result. At most `_lib.MAX_BATCH`
    problems per call. For many small reductions, whose cost is the launch and not the memory."""
    problems = [list(p) for p in problems]
    n_ins = len(problems[0])
    if not 1 <= n_ins <= _lib.MAX_INPUTS or any(len(p) != n_ins for p in problems):
        raise ValueError(f"every problem takes the same 1..{_lib.MAX_INPUTS} operands")
    if not 1 <= len(problems) <= _lib.MAX_BATCH:
        raise ValueError(f"between 1 and {_lib.MAX_BATCH} problems per call")
    t0 = problems[0][0]
    if outs is None:
        outs = [torch.empty(list(t0.shape[:-1]) or [1], device=t0.device, dtype=torch.float32) for _ in problems]
    outs = list(outs)
    chain = _chain(map_expr, combine_expr, post_expr, init, captures)
    flat = [t for p in problems for t in p]
    arr = (_lib.Tensor * len(flat))(*[_view(t, f"ins[{i // n_ins}][{i % n_ins}]") for i, t in enumerate(flat)])
    oarr = (_lib.Tensor * len(outs))(*[_view(t, f"outs[{i}]") for i, t in enumerate(outs)])
    _same_device(*[(f"operand {i}", t) for i, t in enumerate(flat)], *[(f"outs[{i}]", t) for i, t in enumerate(outs)])
    with _on_device(t0):
        _lib.check(_lib.load().tcab_chain_reduce_batched(C.byref(chain), arr, n_ins, len(problems), oarr,
                                                         _stream(stream, t0)))
    return outs


def chain_reduce_noalloc(ins: Sequence[torch.Tensor], map_expr: str, out: torch.Tensor,
                         combine_expr: str = "(p0 + p1)", init: float = 0.0, post_expr: Optional[str] = None,
                         captures: Sequence[float] = (), stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """chain_reduce over the innermost axis through the entry point that never allocates.

    For hosts that cannot let the library call cudaMalloc (device memory that is already handed
    out in full, a stream capture in progress, a loop that cannot afford cudaMalloc's device
    synchronisation). The caller passes `out`; nothing is allocated here either, on the host side
    only the small ctypes argument structs are built. At most `_lib.NOALLOC_MAX_ROWS` rows; calls on
    one device share a fixed scratch array, so do not let two of them overlap on the GPU.
    """
    ins = list(ins)
    if not 1 <= len(ins) <= _lib.MAX_INPUTS:
        raise ValueError(f"between 1 and {_lib.MAX_INPUTS} operands are required")
    chain = _chain(map_expr, combine_expr, post_expr, init, captures)
    arr = (_lib.Tensor * len(ins))(*[_view(t, i) for i, t in enumerate(ins)])
    ov = _view(out, "out")
    _operands_on_one_device(ins, out)
    with _on_device(ins[0]):
        _lib.check(_lib.load().tcab_chain_reduce_noalloc(C.byref(chain), arr, len(ins), C.byref(ov),
                                                         _stream(stream, ins[0])))
    return out


def chain_contract(lhs: torch.Tensor, rhs: torch.Tensor, map_expr: str = "(p0 * p1)", rhs_is_nk: bool = False,
                   combine_expr: str = "(p0 + p1)", init: float = 0.0, post_expr: Optional[str] = None,
                   captures: Sequence[float] = (), out: Optional[torch.Tensor] = None,
                   stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """out[m,n] = post(fold_k map(lhs[m,k], rhs[k,n]))  (rhs[n,k] with rhs_is_nk), fp32."""
    n = rhs.shape[0] if rhs_is_nk else rhs.shape[1]
    if out is None:
        out = torch.empty((lhs.shape[0], n), device=lhs.device, dtype=torch.float32)
    chain = _chain(map_expr, combine_expr, post_expr, init, captures)
    lv, rv, ov = _view(lhs, "lhs"), _view(rhs, "rhs"), _view(out, "out")
    _same_device(("lhs", lhs), ("rhs", rhs), ("out", out))
    with _on_device(lhs):
        _lib.check(_lib.load().tcab_chain_contract(C.byref(chain), C.byref(lv), C.byref(rv), int(bool(rhs_is_nk)),
                                                   C.byref(ov), _stream(stream, lhs)))
    return out


def gemm_bias_act(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  act: str = "relu", out: Optional[torch.Tensor] = None,
                  stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """c = act(a @ b + bias): a [M,K] bf16, b [K,N] bf16, bias [N] fp32, c [M,N] bf16."""
    if out is None:
        out = torch.empty((a.shape[0], b.shape[1]), device=a.device, dtype=torch.bfloat16)
    av, bv, cv = _view(a, "a"), _view(b, "b"), _view(out, "out")
    biasv = _view(bias, "bias") if bias is not None else None
    _same_device(("a", a), ("b", b), ("bias", bias), ("out", out))
    code = {"none": _lib.ACT_NONE, "relu": _lib.ACT_RELU}[act]
    with _on_device(a):
        _lib.check(_lib.load().tcab_gemm_bias_act(C.byref(av), C.byref(bv),
                                                  C.byref(biasv) if biasv is not None else None, code,
                                                  C.byref(cv), _stream(stream, a)))
    return out
