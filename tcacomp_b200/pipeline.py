"""Host-buffer execution of a row-sharded operator: H2D copy, kernel and D2H copy pipelined over
chunks of the independent axis on rotating streams.

The reference's launchers take device tensors and leave the copies to the caller
(testing/runners/*.cu copy whole tensors, launch, synchronise, copy back). Doing that in one piece
serialises the two PCIe directions around the kernel. Every operator class here has an independent
axis (rows / batch / M), so the same cut that shards it across GPUs also pipelines it on one GPU:
chunk i+1 uploads while chunk i computes and chunk i-1 downloads. torch supplies the streams, the
pinned-memory copies and the staging buffers; the compute is the C-ABI call passed in.
"""
from __future__ import annotations

from typing import Callable, Dict, Sequence

import torch

from .shard import blocks


class RowPipeline:
    """Reusable staging buffers and streams for one (input row shape, output row shapes) signature."""

    def __init__(self, device: torch.device, chunk_rows: int, in_row_shape: Sequence[int], in_dtype: torch.dtype,
                 out_specs: Dict[str, tuple], depth: int = 3):
        self.device = device
        self.chunk_rows = chunk_rows
        self.depth = depth
        self.streams = [torch.cuda.Stream(device=device) for _ in range(depth)]
        self.din = [torch.empty((chunk_rows, *in_row_shape), device=device, dtype=in_dtype) for _ in range(depth)]
        self.dout = [{k: torch.empty((chunk_rows, *shape), device=device, dtype=dt) for k, (shape, dt) in out_specs.items()}
                     for _ in range(depth)]

    def run(self, host_in: torch.Tensor, host_out: Dict[str, torch.Tensor],
            fn: Callable[[torch.Tensor, Dict[str, torch.Tensor]], None]) -> None:
        """fn(device_in_chunk, device_out_chunks) launches the operator on the CURRENT stream.

        host_in and host_out must be pinned for the copies to be asynchronous. Returns with the work
        enqueued: the caller's current stream waits for every chunk, so an event recorded on it after
        this call marks the end of the whole job.
        """
        rows = host_in.shape[0]
        n_chunks = (rows + self.chunk_rows - 1) // self.chunk_rows
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in self.streams:
            s.wait_event(start)
        for c, (lo, hi) in enumerate(blocks(rows, n_chunks)):
            slot = c % self.depth
            s = self.streams[slot]
            n = hi - lo
            with torch.cuda.stream(s):
                # slot reuse is ordered by the stream itself: the same slot always runs on the same stream
                din = self.din[slot][:n]
                din.copy_(host_in[lo:hi], non_blocking=True)
                dout = {k: v[:n] for k, v in self.dout[slot].items()}
                fn(din, dout)
                for k, v in dout.items():
                    host_out[k][lo:hi].copy_(v, non_blocking=True)
        for s in self.streams:
            done = torch.cuda.Event()
            done.record(s)
            cur.wait_event(done)
