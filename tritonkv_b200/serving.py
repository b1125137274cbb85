"""A decode step with host buffers on both sides, captured once as a CUDA graph.

The reference measures its kernels under CUDA-graph replay (benchmark.py:556-694) with
inputs already on the device.  A serving loop also has to bring the step's query in and
the result out; captured together with the two kernels those copies cost one graph launch
instead of four separate host calls.  No reference counterpart.
"""

from __future__ import annotations

import torch

from .kernels import fused_decode_attention
from .quantize import QuantizedTensor


class GraphedDecodeStep:
    """``q`` from pinned host memory -> ``fused_decode_attention`` on a resident packed
    cache -> ``out`` to pinned host memory, as ONE CUDA graph.

    ``q_host`` (B, HQ, D) and ``out_host`` (B, HQ, D) float32 are the pinned buffers the
    graph reads and writes; fill ``q_host`` (or pass ``q`` to :meth:`run`), call
    :meth:`run`, then :meth:`result` to wait for and get the step's output.  The cache
    tensors must stay where they were at capture (append in place with
    ``quantize.append_kv`` and grow ``seq_lens`` on the device to lengthen the history).

    ``zero_copy=True`` takes the device-to-host copy off the step: the last kernel stores the
    result straight into ``out_host`` (pinned host memory is addressable from the device).
    The query keeps its copy node: every CTA of the split kernel reads the query rows, which
    costs nothing from L2 but made the step 2.4x slower when each of those reads crossed
    the bus.
    """

    def __init__(self, kq: QuantizedTensor, vq: QuantizedTensor, HQ: int,
                 q_dtype: torch.dtype = torch.float16, seq_lens: torch.Tensor | None = None,
                 sm_scale: float | None = None, num_splits: int | None = None,
                 zero_copy: bool = False):
        dev = kq.packed.device
        if dev.type != "cuda":
            raise RuntimeError("GraphedDecodeStep needs a CUDA cache; this package has no CPU path")
        B, D = kq.packed.shape[0], kq.head_dim
        self.q_host = torch.zeros(B, HQ, D, dtype=q_dtype).pin_memory()
        self.out_host = torch.zeros(B, HQ, D, dtype=torch.float32).pin_memory()
        self.q_dev = torch.zeros(B, HQ, D, dtype=q_dtype, device=dev)
        self.out_dev = torch.zeros(B, HQ, D, dtype=torch.float32, device=dev)
        self._ws: dict = {}
        self._dev = dev
        self._stream = torch.cuda.Stream(device=dev)  # capture stream only

        self.zero_copy = zero_copy

        def step():
            self.q_dev.copy_(self.q_host, non_blocking=True)
            if zero_copy:
                fused_decode_attention(self.q_dev, kq, vq, sm_scale=sm_scale, num_splits=num_splits,
                                       out=self.out_host, _workspace=self._ws, seq_lens=seq_lens,
                                       _host_io=True)
                return
            fused_decode_attention(self.q_dev, kq, vq, sm_scale=sm_scale, num_splits=num_splits,
                                   out=self.out_dev, _workspace=self._ws, seq_lens=seq_lens)
            self.out_host.copy_(self.out_dev, non_blocking=True)

        with torch.cuda.device(dev):
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                step()  # allocates the workspace outside the capture
            self._stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self._stream):
                step()
            self._stream.synchronize()

    def run(self, q: torch.Tensor | None = None) -> None:
        """Launch the step on the current stream (asynchronous).  ``q``: a host tensor copied
        into ``q_host`` first."""
        if q is not None:
            self.q_host.copy_(q)
        self.graph.replay()

    def result(self) -> torch.Tensor:
        """Wait for the launched step and return ``out_host`` (valid until the next run)."""
        torch.cuda.current_stream(self._dev).synchronize()
        return self.out_host
