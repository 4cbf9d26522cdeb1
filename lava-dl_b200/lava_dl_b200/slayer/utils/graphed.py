"""Replay of an inference call as one CUDA graph (no counterpart in lava-dl).

A neuron's ``forward`` on a small problem is a handful of launches -- the fused
kernel, the quantisation of its decay parameters, state fills -- each of which
costs more host time than the kernel runs (CUBA forward at ``[16, 512, 1000]``:
0.05 ms of GPU work, 0.12 ms per eager call).  ``Graphed`` captures the call once
and replays it; the kernels and their results are the same ones.
"""

import torch


class Graphed:
    """``Graphed(fn, example_input)`` -> callable with the semantics of ``fn`` under
    ``torch.no_grad()`` for inputs of the example's shape, dtype and device.

    ``fn`` maps one CUDA tensor to a tensor or a tuple of tensors (a neuron, a block,
    an ``nn.Sequential`` of them).  The call owns a static input and static outputs:
    every call copies its argument in (unless it *is* the static input,
    ``self.input``) and returns the same output tensors, overwritten.  Modules that
    carry state from call to call (``persistent_state=True``) are refused: the
    graph would keep reading the state tensor of the capture.
    """

    def __init__(self, fn, example_input, warmup=3):
        if not example_input.is_cuda:
            raise RuntimeError('Graphed needs a CUDA tensor')
        if isinstance(fn, torch.nn.Module):
            for m in fn.modules():
                if getattr(m, 'persistent_state', False):
                    raise RuntimeError('Graphed cannot replay a module with persistent_state=True')
        self.fn = fn
        self.input = example_input.detach().clone()
        side = torch.cuda.Stream(device=self.input.device)
        side.wait_stream(torch.cuda.current_stream(self.input.device))
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(max(1, warmup)):   # lazy shape binding, kernel attributes, allocator warm-up
                fn(self.input)
        torch.cuda.current_stream(self.input.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.output = fn(self.input)

    def __call__(self, input):
        if input.shape != self.input.shape or input.dtype != self.input.dtype or input.device != self.input.device:
            raise RuntimeError(f'Graphed was captured for {tuple(self.input.shape)} {self.input.dtype} on '
                               f'{self.input.device}, got {tuple(input.shape)} {input.dtype} on {input.device}')
        if input.data_ptr() != self.input.data_ptr():
            self.input.copy_(input)
        self.graph.replay()
        return self.output
