"""CUDA-graph replay of a network's forward.

A Converse network at a small batch is launch-bound: ConverseDnCNN issues about 520 kernels per forward,
and at one image the host needs longer to enqueue them than the GPU needs to run them.  `GraphedForward`
captures one forward (this package's kernels, PyTorch's few 1x1 convolutions and copies, and the
allocations between them) in a CUDA graph with static input and output buffers and replays it: one
launch per forward.  Inference only (no autograd); tensor shapes, dtypes and the non-tensor arguments
are fixed at capture time; the parameters are read at replay time, but a transfer table is rebuilt only
on a new capture, so re-capture after changing a Converse2D weight.  The reference has no counterpart
(its scripts run eager PyTorch, `main_test_converse_dncnn.py:133-136`)."""
import torch


class GraphedForward:
    def __init__(self, net, *example_args, warmup=2):
        dev = next(net.parameters()).device
        if dev.type != "cuda":
            raise RuntimeError("GraphedForward needs a network on a CUDA device")
        self.net = net
        self.static_args = [a.clone() if torch.is_tensor(a) else a for a in example_args]
        self.device = dev
        stream = torch.cuda.Stream(dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(stream), torch.no_grad():
            for _ in range(max(1, warmup)):     # builds tables, workspaces and per-device constants
                net(*self.static_args)
        torch.cuda.current_stream(dev).wait_stream(stream)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = net(*self.static_args)

    def __call__(self, *args):
        """Copy the tensor arguments into the static buffers, replay, return the static output
        (overwritten by the next call: clone it to keep it)."""
        if len(args) != len(self.static_args):
            raise RuntimeError("GraphedForward was captured with %d arguments" % len(self.static_args))
        for s, a in zip(self.static_args, args):
            if torch.is_tensor(s):
                if not torch.is_tensor(a) or a.shape != s.shape or a.dtype != s.dtype:
                    raise RuntimeError("GraphedForward: tensor arguments must keep their captured shape and dtype")
                if a.data_ptr() != s.data_ptr():
                    s.copy_(a, non_blocking=True)
            elif s != a:
                raise RuntimeError("GraphedForward: non-tensor arguments are fixed at capture time")
        self.graph.replay()
        return self.static_out
