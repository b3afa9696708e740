"""CUDA-graph replay of a fixed-shape call.

The sampler of K-Fold calls its token transformer 200 times per prediction with tensors of the same shape
(src/kfold/model/modules/ecsi.py:468-560).  One pass is about 300 kernel launches of a few microseconds each, so issued
from Python it is bound by the host; captured once into a CUDA graph and replayed it takes half the time on a B200
(bench.py --diffusion-step prints both).  The library is capturable as it is: it allocates nothing, never synchronises, and
every temporary of the Python layer comes from torch's caching allocator, which gives a capture its own pool.
"""
from __future__ import annotations

import torch


class GraphedCall:
    """``GraphedCall(fn, *example_inputs)`` captures ``fn(*example_inputs)`` once; ``self(*inputs)`` copies the inputs into
    the captured buffers, replays the graph and returns the captured output tensor(s) (overwritten by the next call).

    ``fn`` must be free of host synchronisation and of data-dependent control flow, and every call must use the shapes,
    dtypes and devices of the example.  Tensors that never change between calls (weights, a cached pair bias, masks) can
    be closed over by ``fn`` instead of being passed as inputs, which saves their copy.

    The stacks keep what they derive from per-complex tensors (the converted token pair bias, the window biases of the atom
    transformers) in caches that already hold their result when the capture runs, so those kernels are NOT part of the
    graph: the pair tensor ``z``, the window pair tensor ``p`` and ``pair_bias`` must be closed over by ``fn``, never passed
    as inputs that later calls replace -- a replay would keep using the bias of the captured tensors.  For a new complex
    build a new GraphedCall.
    """

    def __init__(self, fn, *example_inputs: torch.Tensor, warmup: int = 2):
        if not example_inputs or not all(t.is_cuda for t in example_inputs):
            raise ValueError("GraphedCall needs CUDA tensors as example inputs")
        self._inputs = [t.clone() for t in example_inputs]
        dev = example_inputs[0].device
        with torch.cuda.device(dev), torch.no_grad():
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):          # warm-up outside the capture: weight packing, workspace allocation
                for _ in range(max(warmup, 1)):
                    fn(*self._inputs)
            torch.cuda.current_stream().wait_stream(side)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._output = fn(*self._inputs)

    def __call__(self, *inputs: torch.Tensor):
        if len(inputs) != len(self._inputs):
            raise ValueError(f"expected {len(self._inputs)} inputs, got {len(inputs)}")
        for dst, src in zip(self._inputs, inputs):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise ValueError(f"input {tuple(src.shape)} {src.dtype} does not match the captured {tuple(dst.shape)} {dst.dtype}")
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self._graph.replay()
        return self._output
