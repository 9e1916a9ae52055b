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


def test_host_word_gates_a_stream_and_is_written_by_it():
    """Work queued behind ``stream_wait`` starts only after the host has published; ``stream_mark_sent`` tells the
    host that the stream got past a point, with no synchronisation and no polling kernel."""
    import threading
    import time
    from mesh_b200.runtime.plan import HostWord
    w = HostWord()
    s = torch.cuda.Stream()
    x = torch.zeros(1 << 20, device="cuda")
    # the host publishes from another thread shortly after the work has been queued (a stream wait has no timeout of
    # its own, so the publication does not depend on anything below succeeding)
    t = threading.Timer(0.2, lambda: w.publish_to_streams(3))
    t.start()
    try:
        with torch.cuda.stream(s):
            w.stream_wait(3)
            x.add_(1)
            w.stream_mark_sent(7)
        time.sleep(0.05)
        assert not w.stream_sent(7) and not s.query()          # still held back: nothing has been published yet
    finally:
        t.join()
    s.synchronize()
    assert float(x.sum()) == float(1 << 20) and w.stream_sent(7) and w.arrived(3)
