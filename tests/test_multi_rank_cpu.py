"""World-size-2 and -3 gloo runs on CPU of the multi-GPU plumbing: rendezvous, barrier, max-over-ranks of the timed
value, contiguous batch shards that cover the batch exactly.  (The data path itself has no collective.)"""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,batch", [(2, 256), (3, 256), (2, 7)])
def test_replica_plumbing_over_gloo(world, batch):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist_worker.py"), str(batch)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["world"] == world
    assert out["slowest_ms"] == 10.0 + 5.0 * (world - 1)
    assert out["covered"] == batch


def test_shard_batch_is_contiguous_and_exact(pkg):
    from cuda_inference_b200.chain import shard_batch
    for total in (256, 7, 1, 33):
        for world in (1, 2, 4, 8):
            nxt = 0
            for rank in range(world):
                first, count = shard_batch(total, world, rank)
                assert first == nxt and count >= 0
                nxt += count
            assert nxt == total
    assert shard_batch(256, 8, 3) == (96, 32)
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)


def test_chain_definition(pkg):
    from cuda_inference_b200 import workloads as wl
    ops, slots = wl.resnet50_chain(256)
    convs = [o for o in ops if o.kind == "conv"]
    assert len(convs) == 53 and sum(o.kind == "add" for o in ops) == 16 and sum(o.kind == "maxpool" for o in ops) == 1
    assert wl.chain_flops(ops) == 2_092_613_763_072
    assert slots[len(slots) - 1] == (2048, 7, 7)
    stem = convs[0].shape
    assert (stem.in_channels, stem.out_channels, stem.kernel, stem.stride, stem.pad, stem.out_h) == (3, 64, 7, 2, 3, 112)
    # stride 2 sits on the 3x3 of the first block of stages 2-4; projections are 1x1
    s2 = [o.shape for o in convs if o.shape.stride == 2 and o.shape.kernel == 3]
    assert len(s2) == 3
    assert all(o.shape.kernel == 1 for o in convs if not o.relu)
    # every tensor a layer reads was produced before it
    produced = {0}
    for o in ops:
        assert o.src in produced and (o.kind != "add" or o.other in produced)
        produced.add(o.dst)
