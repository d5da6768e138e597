"""fast_rnnt_b200.graphs.GraphedStep: the pipeline step the benchmark times (smoothed simple
loss, prune ranges, fused joiner + pruned loss, backward; two streams) captured in a CUDA
graph must give, bit for bit, what the same step gives when it is enqueued eagerly -- on the
batch it was captured with and on another batch written into the same tensors."""
import pytest
import torch

from tests import workloads

pytestmark = pytest.mark.gpu

GRAD_KEYS = ("am", "lm", "enc", "dec", "joiner_w", "joiner_b")


def eager(step, wl, keys):
    t = {k: wl[k].cuda() for k in keys}
    loss = step(t).clone()
    return loss, {k: t[k].grad.clone() for k in GRAD_KEYS}


@pytest.mark.parametrize("joiner,overlap", [("fused", True), ("fused", False), ("tensorcore", True)])
def test_graphed_step_equals_the_eager_step(joiner, overlap):
    import bench
    import fast_rnnt_b200 as fr
    from fast_rnnt_b200.graphs import GraphedStep

    keys = bench.TENSOR_KEYS
    # B, T, S, C, D, s_range, (S_b range), (T_b range): the vocabulary a multiple of four and
    # the joiner's input a multiple of eight, as the fused operator wants them
    workloads.PIPELINE_SIZES["graph"] = (6, 90, 33, 72, 24, 5, (17, 33), (60, 90))
    wl_a = workloads.pipeline_workload("graph", seed=3)
    wl_b = workloads.pipeline_workload("graph", seed=4)
    wl_b["boundary"] = wl_a["boundary"]   # what the host derives from it is frozen at capture
    step = bench.make_step(fr, wl_a, joiner, overlap=overlap)
    ref_a, ref_b = eager(step, wl_a, keys), eager(step, wl_b, keys)

    static = {k: wl_a[k].cuda() for k in keys}
    g = GraphedStep(step, static)
    assert g.launches > 10
    for wl, (ref_loss, ref_grads) in ((wl_a, ref_a), (wl_b, ref_b), (wl_a, ref_a)):
        with torch.no_grad():
            for k in keys:
                if k != "boundary":
                    static[k].copy_(wl[k])
        loss = g()
        torch.cuda.synchronize()
        assert torch.equal(loss, ref_loss), (loss, ref_loss)
        for k in GRAD_KEYS:
            assert torch.equal(static[k].grad, ref_grads[k]), k
