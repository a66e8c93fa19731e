"""Multi-process host logic of the image-sharded path, on CPU with gloo (world size 2 and 3)."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import torch.distributed as dist
    from ogle_b200 import sharding
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    n_images = int(sys.argv[1])
    lo, hi = sharding.shard_range(n_images, rank, world)
    local = [{"image": i, "rank": rank, "boxes": [i, i + 1]} for i in range(lo, hi)]
    merged = sharding.gather_detections(local, lo)
    slowest = sharding.max_over_ranks(10.0 + rank)
    assert slowest == 10.0 + world - 1
    if rank == 0:
        assert [m["image"] for m in merged] == list(range(n_images))
        owners = [m["rank"] for m in merged]
        assert owners == sorted(owners) and set(owners) <= set(range(world))
        print("OK", n_images, world)
    else:
        assert merged is None
    dist.barrier()
    dist.destroy_process_group()
""") % ROOT


def test_shard_range_covers_every_image_once():
    from ogle_b200.sharding import shard_range
    for n in (0, 1, 7, 32, 256, 257):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("world,n_images", [(2, 9), (3, 8)])
def test_gather_over_gloo(tmp_path, world, n_images):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = 29500 + (os.getpid() % 500) + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), str(n_images)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    assert f"OK {n_images} {world}" in out.stdout
