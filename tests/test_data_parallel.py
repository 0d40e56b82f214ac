"""Bucketed gradient all-reduce: two and four data-parallel ranks must end up with the gradient of the whole batch."""
import pytest
import torch
import torch.nn as nn

from hccl_b200.parallel.data_parallel import DataParallel
from hccl_b200.utils.sim import run_ranks


def _model():
    torch.manual_seed(3)
    return nn.Sequential(nn.Linear(16, 64), nn.Tanh(), nn.Linear(64, 64), nn.Tanh(), nn.Linear(64, 4))


@pytest.mark.parametrize("keep_views", [False, True], ids=["grads-copied", "grads-are-bucket-views"])
@pytest.mark.parametrize("world", [2, 4])
def test_bucketed_allreduce_matches_full_batch(world, keep_views):
    torch.manual_seed(0)
    x, y = torch.randn(8 * world, 16), torch.randn(8 * world, 4)
    ref = _model()
    ((ref(x) - y) ** 2).mean().backward()
    want = [p.grad.clone() for p in ref.parameters()]

    state = {k: v.clone() for k, v in ref.state_dict().items()}
    import threading
    lock = threading.Lock()

    def body(comm, rank):
        with lock:                                           # module construction draws from the process-wide generator
            m = _model()
        m.load_state_dict(state)
        dp = DataParallel(m, comm, bucket_mb=0.01)          # tiny buckets: several launches per step
        outs = []
        for step in range(2):                                # the second step reuses the buckets
            m.zero_grad(set_to_none=not keep_views)          # kept: autograd accumulates straight into the buckets
            xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
            ((m(xs) - ys) ** 2).mean().backward()
            dp.finish()
            outs.append([p.grad.clone() for p in m.parameters()])
        return outs, len(dp.buckets), dp.launched

    for outs, nb, launched in run_ranks(world, body):
        assert nb > 1 and launched == 2 * nb
        for grads in outs:
            for g, w in zip(grads, want):
                assert torch.allclose(g, w, atol=1e-6)
