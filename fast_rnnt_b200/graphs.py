"""A whole loss step -- forward and backward -- captured once in a CUDA graph and replayed.

The pruned pipeline at 64 utterances launches about thirty kernels of this library and as
many small torch ops in well under two milliseconds; the host needs about one millisecond
to enqueue them.  One process with idle cores hides that behind the device; eight ranks on a
sixteen-core host do not.  A captured step costs one graph launch.  The reference has no
counterpart (its CUDA kernels launch on the legacy default stream and cannot be captured).

What makes the step capturable: every kernel of the library goes to the caller's current
stream, scratch comes from torch's allocator (graph-private pool under capture), and the
checks that need the content of ``boundary`` use the host copy cached on the tensor
(``provide_boundary_rows`` or the first eager call), so nothing synchronises with the device.
"""
from typing import Callable, Dict, Iterable, Optional

import torch
from torch import Tensor

from . import _lib


class GraphedStep:
    """``fn(inputs) -> loss`` (calls ``backward()`` inside) captured over the *static* tensors in
    ``inputs``: a replay recomputes the loss and the ``.grad`` of every leaf from whatever the
    input tensors hold at that moment -- write the next batch into them (``copy_``) and call the
    object.  The shapes, and everything the host derives from ``boundary`` (sequence limits
    for the range checks, the ``s_range`` adjustment), are frozen at capture: a batch with
    other boundaries needs its own capture.

        step = GraphedStep(train_step, batch)     # warm-up runs + capture
        loss = step()                             # replay; batch["enc"].grad etc. refreshed

    ``warmup`` eager runs on a side stream come first (lazy initialisation, the boundary cache,
    autograd's buffers), as torch's capture rules ask.  ``launches`` is the number of kernels of
    this library inside the graph.  ``pool`` (``torch.cuda.graph_pool_handle()``) lets several
    captures that never run at the same time share their scratch memory."""

    def __init__(self, fn: Callable[[Dict[str, Tensor]], Tensor], inputs: Dict[str, Tensor],
                 warmup: int = 3, leaves: Optional[Iterable[str]] = None, pool=None):
        dev = next(v.device for v in inputs.values() if isinstance(v, Tensor) and v.is_cuda)
        self.inputs = inputs
        self.graph = torch.cuda.CUDAGraph()
        cur = torch.cuda.current_stream(dev)
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(cur)
        with torch.cuda.stream(s):
            for _ in range(max(1, warmup)):
                fn(inputs)
        cur.wait_stream(s)
        # the gradients of the capture must be born inside it (graph-private memory that every
        # replay refills), not accumulate into tensors of the warm-up
        names = list(leaves) if leaves is not None else [k for k, v in inputs.items()
                                                         if isinstance(v, Tensor) and v.requires_grad]
        for k in names:
            inputs[k].grad = None
        torch.cuda.synchronize(dev)
        torch.cuda.empty_cache()   # the warm-up's scratch, or it stays cached beside the graph's
        n0 = _lib.lib().frnnt_launch_count()
        with torch.cuda.graph(self.graph, pool=pool):
            self.loss = fn(inputs)
        self.launches = int(_lib.lib().frnnt_launch_count() - n0)

    def __call__(self) -> Tensor:
        self.graph.replay()
        return self.loss
