"""Host-buffer execution through the C ABI (tcab_pipeline_*, tcab_multi_*): pinned host memory in, pinned host
memory out, the upload | kernel | download stages of successive chunks overlapped by the library. Every result
must equal the direct call on device tensors bit for bit -- the chunks are cut along the independent axis, so
the kernels see whole rows / batches either way."""
import numpy as np
import pytest
import torch

import tcacomp_b200 as T
from tcacomp_b200.pipeline import MultiDevice, Pipeline, PipelineSpec

pytestmark = pytest.mark.gpu

CANARY = -12345.0


def dev_bf16(bits, dev):
    return torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)


def test_softmax_pipeline_matches_direct_call_and_streams(cuda):
    rng = np.random.default_rng(8)
    x = (4 * rng.normal(0, 1, (1000, 512))).astype(np.float32)   # 1000 rows in chunks of 96: a ragged last chunk
    hx = torch.from_numpy(x).pin_memory()
    hy = torch.full_like(hx, CANARY).pin_memory()
    pipe = Pipeline(PipelineSpec("softmax_rows", cuda, 96, (512,), torch.float32, depth=3))
    for _ in range(2):  # twice: the staging slots are reused
        pipe.run([hx], [hy])
        pipe.sync()
    direct = T.softmax_rows(hx.to(cuda)).cpu()
    assert torch.equal(hy, direct)
    # streaming: batches back to back without a join in between, different host buffers per batch, one join at the end
    batches = [torch.from_numpy((4 * rng.normal(0, 1, (1000, 512))).astype(np.float32)).pin_memory() for _ in range(3)]
    outs = [torch.full_like(b, CANARY).pin_memory() for b in batches]
    for b, o in zip(batches, outs):
        pipe.run([b], [o])
    pipe.join()                                  # the current stream waits on the device ...
    torch.cuda.current_stream(cuda).synchronize()  # ... and the host on the current stream
    for b, o in zip(batches, outs):
        assert torch.equal(o, T.softmax_rows(b.to(cuda)).cpu())
    # ordered after work on the caller's stream: the upload must not overtake a producer on that stream
    pipe.order_after()
    pipe.run([hx], [hy], units=10)
    pipe.sync()
    assert torch.equal(hy[:10], direct[:10])
    pipe.close()


def test_every_operator_class_through_the_pipeline(oracle, cuda):
    rng = np.random.default_rng(9)
    # outer-axis reduce over batch chunks: three outputs per chunk
    t = rng.uniform(-100, 100, (10, 64, 96)).astype(np.float32)
    ht = torch.from_numpy(t).pin_memory()
    ho = [torch.empty((10, 96)).pin_memory(), torch.empty((10, 96)).pin_memory(),
          torch.empty((10, 96), dtype=torch.int32).pin_memory()]
    p = Pipeline(PipelineSpec("reduce_outer", cuda, 3, (64, 96), torch.float32))
    p.run([ht], ho)
    p.sync()
    s, m, a = oracle.reduce_outer(t)
    assert np.array_equal(ho[2].numpy(), a) and np.array_equal(ho[1].numpy(), m)
    assert (np.abs(ho[0].numpy() - s) <= 1e-5 * np.abs(t).sum(1)).all()
    # a subset of the outputs
    p = Pipeline(PipelineSpec("reduce_outer", cuda, 4, (64, 96), torch.float32, outputs=("max",)))
    hm = torch.empty((10, 96)).pin_memory()
    p.run([ht], [hm])
    p.sync()
    assert np.array_equal(hm.numpy(), m)

    # layer-norm bf16 with gamma / beta resident on the device
    xb = oracle.f32_to_bf16(rng.normal(0, 1, (300, 1024)).astype(np.float32))
    g = dev_bf16(oracle.f32_to_bf16(rng.normal(1, .1, 1024).astype(np.float32)), cuda)
    b = dev_bf16(oracle.f32_to_bf16(rng.normal(0, .1, 1024).astype(np.float32)), cuda)
    hx = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    p = Pipeline(PipelineSpec("layernorm_rows", cuda, 64, (1024,), torch.bfloat16, eps=1e-5, resident=(g, b)))
    p.run([hx], [hy])
    p.sync()
    assert torch.equal(hy.view(torch.int16), T.layernorm_rows(hx.to(cuda), g, b, 1e-5).cpu().view(torch.int16))

    # map + row reduce with two streamed operands: one f32 per row
    x = rng.uniform(-1, 1, (777, 260)).astype(np.float32)
    w = rng.uniform(-1, 1, (777, 260)).astype(np.float32)
    hxs = [torch.from_numpy(x).pin_memory(), torch.from_numpy(w).pin_memory()]
    hr = torch.empty((777,)).pin_memory()
    p = Pipeline(PipelineSpec("chain_reduce", cuda, 100, (260,), torch.float32, n_streamed=2, map_expr="p0 * p1"))
    p.run(hxs, [hr])
    p.sync()
    assert torch.equal(hr, T.chain_reduce([hxs[0].to(cuda), hxs[1].to(cuda)], "p0 * p1").cpu())

    # the same with bf16 rows (fp32 arithmetic and result)
    hbs = [t.to(torch.bfloat16).pin_memory() for t in hxs]
    hr = torch.empty((777,)).pin_memory()
    p = Pipeline(PipelineSpec("chain_reduce", cuda, 100, (260,), torch.bfloat16, n_streamed=2, map_expr="f32(p0) * f32(p1)"))
    p.run(hbs, [hr])
    p.sync()
    assert torch.equal(hr, T.chain_reduce([hbs[0].to(cuda), hbs[1].to(cuda)], "f32(p0) * f32(p1)").cpu())

    # contraction: rows of a streamed, b and bias resident
    a_ = oracle.f32_to_bf16((rng.normal(0, 1, (300, 256)) / 16).astype(np.float32))
    b_ = dev_bf16(oracle.f32_to_bf16((rng.normal(0, 1, (256, 128)) / 16).astype(np.float32)), cuda)
    bias = torch.from_numpy(rng.normal(0, 0.02, 128).astype(np.float32)).to(cuda)
    ha = torch.from_numpy(a_.view(np.int16)).view(torch.bfloat16).pin_memory()
    hc = torch.empty((300, 128), dtype=torch.bfloat16).pin_memory()
    p = Pipeline(PipelineSpec("gemm_bias_act", cuda, 128, (256,), torch.bfloat16, act="relu", resident=(b_, bias)))
    p.run([ha], [hc])
    p.sync()
    assert torch.equal(hc.view(torch.int16), T.gemm_bias_act(ha.to(cuda), b_, bias, "relu").cpu().view(torch.int16))
    assert T.device_status() == 0

    # map-only, f32 in, bf16 out
    hx = torch.from_numpy(x).pin_memory()
    hb = torch.empty((777, 260), dtype=torch.bfloat16).pin_memory()
    p = Pipeline(PipelineSpec("map", cuda, 50, (260,), torch.float32, out_dtype=torch.bfloat16, map_expr="bf16(fmaxf(p0, 0.0f))"))
    p.run([hx], [hb])
    p.sync()
    assert torch.equal(hb.view(torch.int16),
                       T.map([hx.to(cuda)], "bf16(fmaxf(p0, 0.0f))", out_dtype=torch.bfloat16).cpu().view(torch.int16))


def test_pipeline_arguments_are_validated(cuda):
    with pytest.raises(T.TcabError) as e:
        Pipeline(PipelineSpec("softmax_rows", cuda, 0, (512,), torch.float32))
    assert e.value.status == T._lib.ERR_INVALID_ARG
    with pytest.raises(T.TcabError) as e:
        Pipeline(PipelineSpec("softmax_rows", cuda, 8, (512,), torch.bfloat16))
    assert e.value.status == T._lib.ERR_DTYPE
    with pytest.raises(T.TcabError) as e:
        Pipeline(PipelineSpec("layernorm_rows", cuda, 8, (512,), torch.float32))   # gamma / beta missing
    assert e.value.status == T._lib.ERR_INVALID_ARG
    p = Pipeline(PipelineSpec("softmax_rows", cuda, 8, (512,), torch.float32))
    with pytest.raises(ValueError):
        p.run([torch.empty((4, 512))], [torch.empty((2, 512))])               # output buffer too small


def test_one_problem_cut_over_the_devices_of_this_process(cuda):
    """tcab_multi: every visible device takes its block of the same host problem (one device: one block)."""
    n_dev = torch.cuda.device_count()
    rng = np.random.default_rng(10)
    x = (4 * rng.normal(0, 1, (1003, 512))).astype(np.float32)
    hx = torch.from_numpy(x).pin_memory()
    hy = torch.full_like(hx, CANARY).pin_memory()
    specs = [PipelineSpec("softmax_rows", torch.device("cuda", d), 64, (512,), torch.float32) for d in range(n_dev)]
    m = MultiDevice(specs)
    m.run([hx], [hy])
    m.sync()
    assert torch.equal(hy, T.softmax_rows(hx.to(cuda)).cpu())
    m.close()
    lo, hi = (np.uint64(0), np.uint64(0))
    import ctypes as C
    a, b = C.c_uint64(), C.c_uint64()
    from tcacomp_b200 import _lib, shard
    for world in (1, 2, 3, 8):
        for r in range(world):
            assert _lib.load().tcab_shard_block(1003, world, r, C.byref(a), C.byref(b)) == 0
            assert (a.value, b.value) == shard.block(1003, world, r)
