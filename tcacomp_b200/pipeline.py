"""Host-buffer execution of a row-sharded operator: H2D copy, kernel and D2H copy pipelined over
chunks of the independent axis on rotating streams.

The reference's launchers take device tensors and leave the copies to the caller
(testing/runners/*.cu copy whole tensors, launch, synchronise, copy back). Doing that in one piece
serialises the two PCIe directions around the kernel. Every operator class here has an independent
axis (rows / batch / M), so the same cut that shards it across GPUs also pipelines it on one GPU:
chunk i+1 uploads while chunk i computes and chunk i-1 downloads. torch supplies the streams, events, the
pinned-memory copies and the staging buffers; the compute is the C-ABI call passed in.
"""
from __future__ import annotations

from typing import Callable, Dict, Sequence

import torch

from .shard import blocks


class RowPipeline:
    """Reusable staging buffers, streams and events for one (input row shape, output row shapes) signature.

    Three streams, one per stage: every upload is queued on the upload stream, every kernel on the compute
    stream, every download on the download stream, so neither copy direction ever waits behind a copy of the
    other direction in its own queue. `depth` staging slots rotate; events order a slot's stages (upload ->
    kernel -> download) and its reuse (the next upload into a slot waits for the kernel that read it, the next
    kernel for the download that read its outputs)."""

    def __init__(self, device: torch.device, chunk_rows: int, in_row_shape: Sequence[int], in_dtype: torch.dtype,
                 out_specs: Dict[str, tuple], depth: int = 4):
        self.device = device
        self.chunk_rows = chunk_rows
        self.depth = depth
        self.up = torch.cuda.Stream(device=device)
        self.compute = torch.cuda.Stream(device=device)
        self.down = torch.cuda.Stream(device=device)
        self.din = [torch.empty((chunk_rows, *in_row_shape), device=device, dtype=in_dtype) for _ in range(depth)]
        self.dout = [{k: torch.empty((chunk_rows, *shape), device=device, dtype=dt) for k, (shape, dt) in out_specs.items()}
                     for _ in range(depth)]
        self.uploaded = [None] * depth    # events of the slot's latest upload / kernel / download
        self.computed = [None] * depth
        self.downloaded = [None] * depth
        self.next_chunk = 0

    def run(self, host_in: torch.Tensor, host_out: Dict[str, torch.Tensor],
            fn: Callable[[torch.Tensor, Dict[str, torch.Tensor]], None], join: bool = True) -> None:
        """fn(device_in_chunk, device_out_chunks) launches the operator on the CURRENT stream.

        host_in and host_out must be pinned for the copies to be asynchronous. Returns with the work
        enqueued. With join (the default) the caller's current stream waits for every chunk, so an event
        recorded on it after this call marks the end of the whole job. A caller that streams one batch after
        another passes join=False and calls join() once at the end: the first uploads of batch i+1 then run
        under the last downloads of batch i instead of after them. What this call waits for is what was on the
        current stream when it was made.
        """
        rows = host_in.shape[0]
        n_chunks = (rows + self.chunk_rows - 1) // self.chunk_rows
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.up, self.compute, self.down):
            s.wait_event(start)
        for lo, hi in blocks(rows, n_chunks):
            slot = self.next_chunk % self.depth
            self.next_chunk += 1
            n = hi - lo
            din = self.din[slot][:n]
            dout = {k: v[:n] for k, v in self.dout[slot].items()}
            with torch.cuda.stream(self.up):
                if self.computed[slot] is not None:
                    self.up.wait_event(self.computed[slot])      # the kernel that read this slot's input
                din.copy_(host_in[lo:hi], non_blocking=True)
                self.uploaded[slot] = torch.cuda.Event()
                self.uploaded[slot].record(self.up)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(self.uploaded[slot])
                if self.downloaded[slot] is not None:
                    self.compute.wait_event(self.downloaded[slot])  # the download that read this slot's outputs
                fn(din, dout)
                self.computed[slot] = torch.cuda.Event()
                self.computed[slot].record(self.compute)
            with torch.cuda.stream(self.down):
                self.down.wait_event(self.computed[slot])
                for k, v in dout.items():
                    host_out[k][lo:hi].copy_(v, non_blocking=True)
                self.downloaded[slot] = torch.cuda.Event()
                self.downloaded[slot].record(self.down)
        if join:
            self.join()

    def join(self) -> None:
        """Makes the current stream wait for every chunk enqueued so far."""
        cur = torch.cuda.current_stream(self.device)
        done = torch.cuda.Event()
        done.record(self.down)   # downloads are queued in chunk order after their kernels and uploads
        cur.wait_event(done)
