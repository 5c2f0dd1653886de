"""The synthetic benchmark graphs run through the CPU oracle (determinism, healthy value
spread), and the host-side batch sharding is exercised with two gloo ranks on CPU."""
import os
import subprocess
import sys
import textwrap

import numpy as np

import oracle
from oxionnx_b200 import models
from oxionnx_b200.shard import all_bounds, shard_bounds

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_partition_the_batch():
    for total in (0, 1, 7, 32, 1024):
        for world in (1, 2, 3, 4, 8):
            b = all_bounds(total, world)
            assert b[0][0] == 0 and b[-1][1] == total
            for (a0, a1), (b0, b1) in zip(b, b[1:]):
                assert a1 == b0 and a1 - a0 >= b1 - b0 >= 0
    assert shard_bounds(10, 4, 1) == (3, 6)


def test_graph_builders_are_deterministic_and_non_degenerate():
    oracle.set_threads(4)
    g1, w1, f1, info = models.build_resnet50_qlinear(batch=2, image=32, base=8, classes=10)
    g2, w2, f2, _ = models.build_resnet50_qlinear(batch=2, image=32, base=8, classes=10)
    assert all(np.array_equal(w1[k], w2[k]) for k in w1)
    s1 = oracle.run_graph(g1, w1, f1(2))
    s2 = oracle.run_graph(g2, w2, f2(2))
    assert np.array_equal(s1["logits"], s2["logits"])
    assert np.all(np.isfinite(s1["logits"]))
    for name in ("stem_qr", "b0_c3_q", "b3_out_q", "b15_out_q", "fc_q"):
        assert np.unique(s1[name]).size > 10, name
    # batch independence: what sharding relies on
    one = oracle.run_graph(g1, w1, {"input": f1(2)["input"][1:2]})
    assert np.array_equal(one["logits"][0], s1["logits"][1])
    oracle.set_threads(1)


def test_full_size_graph_arithmetic():
    _, w, _, info = models.build_resnet50_f32(batch=32)
    assert info["macs_per_image"] == 4089184256          # 4.089 GMAC per image
    assert sum(v.size for v in w.values()) == 25530472
    _, _, _, info1 = models.build_int8_mlp()
    assert info1["ops"] == 2 * 64 * (1024 * 4096 + 4096 * 4096 + 4096 * 1024)


def test_inswapper_shaped_graph_matches_the_reference_inventory():
    """Config 3: the builder's arithmetic equals what the reference states for the real model (349 GFLOP per
    frame, oxionnx-cuda/src/reference.rs:45-49), and every sample is modulated by its own latent row."""
    _, w, _, info = models.build_inswapper_f32(batch=1)
    assert abs(2 * info["macs_per_image"] / 1e9 - 349.0) < 1.0
    assert 480e6 < sum(v.size for v in w.values()) * 4 < 600e6
    oracle.set_threads(4)
    g, w, f, _ = models.build_inswapper_f32(batch=2, size=16, widths=(8, 16, 24, 32), blocks=2, latent=32)
    feeds = f(2)
    assert np.allclose(np.sum(feeds["latent"].astype(np.float64) ** 2, axis=1), 1.0, atol=1e-5)
    full = oracle.run_graph(g, w, feeds)
    assert full["image"].shape == (2, 3, 16, 16) and np.all(np.abs(full["image"]) <= 1.0)
    one = oracle.run_graph(g, w, {k: v[1:2] for k, v in feeds.items()})
    assert np.allclose(one["image"][0], full["image"][1], atol=1e-6)   # batch independence: what sharding relies on
    swapped = dict(feeds, latent=feeds["latent"][::-1].copy())
    assert not np.allclose(oracle.run_graph(g, w, swapped)["image"], full["image"], atol=1e-3)
    oracle.set_threads(1)


def test_slice_matches_numpy_on_the_oracle():
    x = np.arange(3 * 5 * 7, dtype=np.float32).reshape(3, 5, 7)
    cases = [((1, 2), (3, 9.3e18), (0, 2), None, x[1:3, :, 2:]), ((-2,), (-9.3e18,), (1,), (-1,), x[:, -2::-1]),
             ((0, 1, 6), (2, 4, 0), None, (1, 2, -3), x[0:2, 1:4:2, 6:0:-3]), ((4,), (2,), (2,), None, x[:, :, 4:2])]
    for starts, ends, axes, steps, want in cases:
        ins = [x, np.float32(starts), np.float32(ends)]
        if axes is not None or steps is not None:
            ins.append(np.float32(axes) if axes is not None else None)
        if steps is not None:
            ins.append(np.float32(steps))
        got, = oracle.run_node("Slice", ins)
        assert got.shape == want.shape and np.array_equal(got, want), (starts, ends, axes, steps)


def test_two_gloo_ranks_shard_and_gather_bit_exact(tmp_path):
    """world_size 2 on CPU: each rank runs its slice of the batch through the oracle (standing
    in for its GPU replica), results are gathered on the host and must equal the unsharded run."""
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import numpy as np
        import torch.distributed as dist
        import oracle
        from oxionnx_b200 import models
        from oxionnx_b200.shard import shard_bounds, gather_rows, max_over_ranks
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        g, w, f, _ = models.build_resnet50_qlinear(batch=5, image=32, base=8, classes=10)
        x = f(5)["input"]
        b0, b1 = shard_bounds(5, world, rank)
        local = oracle.run_graph(g, w, {{"input": x[b0:b1]}})["logits"]
        full = gather_rows(local, world, rank)
        slow = max_over_ranks(float(rank + 1), world)
        if rank == 0:
            want = oracle.run_graph(g, w, {{"input": x}})["logits"]
            assert np.array_equal(full, want), "sharded result differs"
            assert slow == float(world)
            print("SHARD_OK", full.shape)
        dist.barrier()
        dist.destroy_process_group()
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29517", str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "SHARD_OK (5, 10)" in r.stdout
