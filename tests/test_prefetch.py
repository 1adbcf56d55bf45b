"""Prefetch helpers: synchronous fall-back on CPU, side-stream copies and deferred scalar reads on a GPU."""
import pytest
import torch

from spikingjelly_b200.utils import DeferredScalar, DevicePrefetcher


def test_cpu_fallback():
    pf = DevicePrefetcher("cpu")
    x, y = pf.take(pf.stage(torch.arange(4.0), torch.tensor([1, 2])))
    assert torch.equal(x, torch.arange(4.0)) and torch.equal(y, torch.tensor([1, 2]))
    assert DeferredScalar(torch.tensor(3.5)).get() == 3.5


@pytest.mark.gpu
def test_gpu_prefetch_and_deferred_read():
    pf = DevicePrefetcher("cuda")
    hosts = [torch.full((1 << 20,), float(i)).pin_memory() for i in range(4)]
    staged = pf.stage(hosts[0])
    pending, seen = None, []
    for i in range(4):
        (x,) = pf.take(staged)
        if i + 1 < 4:
            staged = pf.stage(hosts[i + 1])
        reader = DeferredScalar((x * 2).mean())
        if pending is not None:
            seen.append(pending.get())
        pending = reader
    seen.append(pending.get())
    assert seen == [0.0, 2.0, 4.0, 6.0]
