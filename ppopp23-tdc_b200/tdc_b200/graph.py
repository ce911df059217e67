"""One forward of a network as a CUDA graph.

The batch-1 networks are launch-bound on the host: TK-DenseNet-121 is about 420 launches of a few microseconds each,
and the interpreter needs longer to issue one than the GPU to run it.  Every kernel of the library is asynchronous on
the caller's stream and allocates nothing, so a forward can be captured once and replayed: the reference's C++
skeleton gets the same effect by having no interpreter (its `forward` chain is a few hundred bare launches,
A100-evaluation/EndToEnd/densenet121-tk/src/TenDense.cu:44-67).
"""
import torch


class GraphedForward:
    """`g = GraphedForward(model, example)`; `y = g(x)` for any x of example's shape.  The model must be in eval mode
    and on the GPU; weights may change in place between calls only if no cached copy depends on them (prepared
    tensor-core operands, folded BatchNorm and channel-last filter copies are made during the warm-up forwards and
    frozen into the graph).  The returned tensor is the graph's own output buffer: clone it to keep it past the next
    call."""

    def __init__(self, model, example, warmup=3):
        if not example.is_cuda:
            raise ValueError("example must be a CUDA tensor")
        self.x = example.detach().clone()
        cur = torch.cuda.current_stream(example.device)
        side = torch.cuda.Stream(example.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                model(self.x)
        cur.wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.y = model(self.x)

    def __call__(self, x):
        if x.shape != self.x.shape:
            raise ValueError("captured for input shape %s, got %s" % (tuple(self.x.shape), tuple(x.shape)))
        self.x.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y
