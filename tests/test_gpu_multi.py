"""Several GPUs in one process: one context per device on its own host thread (ShardedSession), the batch
split with shard_bounds and no data-path collective.  Needs at least two devices; skipped on a one-GPU box."""
import numpy as np
import pytest

import oracle
from oxionnx_b200 import _ffi, models, session as S
from oxionnx_b200.shard import ShardedSession

pytestmark = pytest.mark.gpu


def device_count():
    return int(_ffi.lib().oxb200_device_count())


needs_two = pytest.mark.skipif(device_count() < 2, reason="needs two GPUs")


@needs_two
def test_sharded_int8_network_is_bit_identical_to_one_device():
    graph, weights, feeds_fn, _ = models.build_resnet50_qlinear(batch=6, image=64)
    feeds = feeds_fn(6)
    one = S.Session.builder().with_device(0).build_from_graph(graph, weights)
    want = one.run(feeds)
    one.close()
    n = min(device_count(), 4)
    sharded = ShardedSession(lambda d: S.Session.builder().with_device(d).build_from_graph(graph, weights), range(n))
    for _ in range(2):  # twice: the second run replays the plans
        got = sharded.run(feeds)
        for name in want:
            assert np.array_equal(got[name], want[name]), name
    sharded.close()


@needs_two
def test_contexts_on_two_devices_dispatch_concurrently():
    """The per-device launch state (shared-memory opt-in, SM count, scratch symbols) is set up on each device
    separately: the same node dispatched from two threads, each bound to its own device, agrees with the oracle."""
    import threading
    from oxionnx_b200.graph import Node
    rng = np.random.default_rng(1)
    x = rng.integers(0, 256, (2, 64, 14, 14)).astype(np.float32)
    w = rng.integers(-127, 128, (64, 64, 3, 3)).astype(np.float32)
    ins = [x, np.float32([0.02]), np.float32([128]), w, np.float32([0.01]), np.float32([0]), np.float32([0.05]), np.float32([120])]
    names = [f"i{k}" for k in range(len(ins))]
    node = Node("QLinearConv", "q", names, ["y"], dict(pads=[1, 1, 1, 1]))
    want, = oracle.run_node("QLinearConv", ins, dict(pads=[1, 1, 1, 1]))
    out, err = {}, {}

    def work(dev):
        try:
            ctx = S.CudaContext(dev)
            for _ in range(3):
                out[dev] = S.try_cuda_dispatch(node, {}, dict(zip(names, ins)), ctx)[0]
            ctx.close()
        except BaseException as e:
            err[dev] = e

    threads = [threading.Thread(target=work, args=(d,)) for d in (0, 1)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not err, err
    assert np.array_equal(out[0], want) and np.array_equal(out[1], want)
