"""World-size-2 runs of the cross-replica host logic on CPU (gloo): the
all-reduce placement and global count of SyncBN, range sharding and the
in-place all-gather of sharded Adam."""
import os
import socket
import subprocess
import sys

import pytest

from conftest import ROOT
from tensorflow_musa_extension_b200.cross_replica import shard_range


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _run(mode, world=2):
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "tests", "gloo_worker.py"), mode],
            env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, "rank %d failed:\n%s" % (rank, out)
        assert "rank %d ok" % rank in out


@pytest.mark.parametrize("mode", ["syncbn", "syncbn_ragged", "syncbn_large_mean", "adam_even", "adam_padded"])
def test_two_ranks(mode):
    _run(mode)


def test_shard_ranges_tile_the_vector():
    for n in (0, 1, 7, 8, 1001, 25_557_032):
        for world in (1, 2, 4, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b and c <= d
            per = -(-n // world) if n else 0
            assert all(hi - lo <= per for lo, hi in spans)
