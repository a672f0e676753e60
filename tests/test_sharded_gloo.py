"""The multi-rank combine logic on CPU: two gloo ranks, host arrays."""

import os
import socket
import subprocess
import sys
import textwrap

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    sys.path.insert(0, os.environ["REPO_ROOT"])
    import torch.distributed as dist
    from dpnp_b200 import sharded

    dist.init_process_group(backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(0)                    # every rank builds the same global arrays
    x = rng.normal(0, 1, (10, 257)).astype("f4")      # sharded on the leading axis: 5 rows each
    lo, hi = sharded.shard_bounds(x.shape[0], world, rank)
    mine = x[lo:hi]

    # sum over the sharded axis: partial column sums combined in rank order
    tot = sharded.allreduce_sum_ordered(mine.sum(axis=0))
    expect = x[:5].sum(axis=0) + x[5:].sum(axis=0)
    assert tot.dtype == np.float32 and np.array_equal(tot, expect), "ordered sum"
    # full sum
    s = sharded.allreduce_sum_ordered(np.asarray(mine.sum()))
    assert np.array_equal(s, np.asarray(x[:5].sum() + x[5:].sum()))
    # max over everything
    m = sharded.allreduce_extreme(np.asarray(mine.max()), "max")
    assert m == x.max()
    mn = sharded.allreduce_extreme(mine.min(axis=0), "min")
    assert np.array_equal(mn, x.min(axis=0))
    # argmax with ties: first occurrence across shards
    xi = rng.integers(0, 4, (10, 50)).astype("i4")
    part = xi[lo:hi]
    li = int(part.argmax())
    v, gi = sharded.combine_arg_extreme(part.reshape(-1)[li], li + lo * 50, "max")
    assert v == xi.max() and gi == xi.argmax(), (v, gi, xi.max(), xi.argmax())
    li = int(part.argmin())
    v, gi = sharded.combine_arg_extreme(part.reshape(-1)[li], li + lo * 50, "min")
    assert v == xi.min() and gi == xi.argmin()
    # NaN is the extreme value and the first NaN wins
    xf = rng.normal(0, 1, (10, 50))
    xf[7, 3] = np.nan
    part = xf[lo:hi]
    li = int(np.argmax(part))
    v, gi = sharded.combine_arg_extreme(part.reshape(-1)[li], li + lo * 50, "max")
    assert np.isnan(v) and gi == np.argmax(xf)
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_bounds_cover_the_axis():
    from dpnp_b200 import sharded

    for n in (0, 1, 7, 8, 16384, 1000003):
        for world in (1, 2, 3, 8):
            spans = [sharded.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_rank_combine_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), REPO_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"rank {rank} ok" in out
