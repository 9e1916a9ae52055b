"""DevicePrefetcher hands out the host batches in order, copied on its side stream."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_prefetcher_order_and_reuse():
    from mesh_b200.utils.data import DevicePrefetcher
    host = [torch.full((1024, 64), float(i)).pin_memory() for i in range(7)]
    pf = DevicePrefetcher(host, "cuda", depth=2)
    seen = []
    for i in range(7):
        x = pf.next()
        y = (x * 2).sum()                      # work on the consumer's stream that reads the ring slot
        seen.append(float(y.item()) / (2 * 1024 * 64))
    assert seen == [float(i) for i in range(7)]
    assert pf.bytes_copied == 7 * 1024 * 64 * 4
    with pytest.raises(StopIteration):
        pf.next()
