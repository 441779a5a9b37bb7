"""Child process of tests/test_multi_rank_cpu.py: one gloo rank exercising the replica plumbing (no GPU)."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from cuda_inference_b200.chain import shard_batch  # noqa: E402
from cuda_inference_b200.dist import Ranks  # noqa: E402

r = Ranks("gloo")
first, count = shard_batch(int(sys.argv[1]), r.world, r.rank)
r.barrier()
fake_ms = 10.0 + 5.0 * r.rank            # the slowest rank decides
slowest = r.max(fake_ms)
covered = r.sum(count)
firsts = r.sum(first)
if r.rank == 0:
    print(json.dumps({"world": r.world, "slowest_ms": slowest, "covered": covered, "first_sum": firsts}))
r.close()
