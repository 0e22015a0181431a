"""Instance-owned CUDA-graph execution with explicit input refresh.

Mirror of the reference's ``src/robotics_kernels/common/graph.py`` (``CudaGraphCall``): one graph
per input signature, transactional re-capture (a failed warm-up or capture leaves the previous
graph usable), inputs copied in, the output cloned out, ``captures`` / ``replays`` counters.
The kernels of this package qualify for capture: they launch on the current stream, take their
scratch from a per-stream buffer that exists after the warm-up calls, and never synchronise.
"""

import torch


def _signature(inputs):
    return tuple((tuple(t.shape), t.dtype, t.device, tuple(t.stride())) for t in inputs)


class CudaGraphCall:
    """Capture a deterministic tensor function; randomness must arrive as an input tensor."""

    WARMUPS = 3

    def __init__(self, function, *, retained_tensors=None):
        self.function = function
        self.retained_tensors = retained_tensors
        self._constants = ()
        self.signature = None
        self.graph = None
        self.inputs = None
        self.output = None
        self.captures = 0
        self.replays = 0

    def _capture(self, inputs, device):
        """Build (inputs, graph, output, constants) for a new signature without touching `self`."""
        staged = tuple(t.clone() for t in inputs)
        side = torch.cuda.Stream(device=device)
        caller = torch.cuda.current_stream(device)
        side.wait_stream(caller)
        for t in staged:
            t.record_stream(side)  # allocated on the caller's stream, used on the side stream
        try:
            with torch.cuda.stream(side):
                for _ in range(self.WARMUPS):
                    self.function(*staged)
        finally:
            caller.wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            output = self.function(*staged)
        if not isinstance(output, torch.Tensor):
            raise ValueError("Graph callable must return one Tensor")
        constants = tuple(self.retained_tensors()) if self.retained_tensors is not None else ()
        return staged, graph, output, constants

    def __call__(self, *inputs):
        if not inputs or any(not isinstance(t, torch.Tensor) or not t.is_cuda for t in inputs):
            raise ValueError("CUDA graph inputs must be CUDA tensors")
        device = inputs[0].device
        if any(t.device != device for t in inputs):
            raise ValueError("Graph inputs must share a device")
        signature = _signature(inputs)
        with torch.cuda.device(device):
            if signature != self.signature:
                staged, graph, output, constants = self._capture(inputs, device)  # may raise: state untouched
                self.inputs, self.graph, self.output, self._constants = staged, graph, output, constants
                self.signature = signature
                self.captures += 1
            for target, source in zip(self.inputs, inputs):
                target.copy_(source)
            self.graph.replay()
            stream = torch.cuda.current_stream(device)
            for constant in self._constants:
                if isinstance(constant, torch.Tensor):
                    constant.record_stream(stream)
            self.replays += 1
            return self.output.clone()
