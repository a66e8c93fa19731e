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


SHARED_WORKER = textwrap.dedent("""
    import os, sys, time
    sys.path.insert(0, %r)
    import numpy as np
    import torch.distributed as dist
    from ogle_b200 import sharding
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    scenario, n_images, steps = sys.argv[1], int(sys.argv[2]), 5
    tag = "test_%%s_%%s" %% (os.environ["MASTER_PORT"], scenario)
    # no GPU here: the regions are not registered with CUDA and a stand-in plays the detector
    sb = sharding.ShardedBatch(tag, n_images, (4, 5, 3), rank, world, mode=1, num_classes=3, top_k=2, pin=False,
                               barrier=dist.barrier, with_frames=True)
    lo, hi = sb.local_range()
    # the 8-bit frame region: same slots and ranges, a quarter of the bytes
    assert sb.frame_slot(0).shape == (n_images, 4, 5, 3) and sb.frame_slot(0).dtype == np.uint8
    assert sb.local_frame_ptr(1) - sb.frames.ptr == sb.frame_slot_bytes + lo * 60
    assert sb.local_input_ptr(1) - sb.inputs.ptr == sb.input_slot_bytes + lo * 240

    def fake_detector(step):
        x = sb.input_slot(step)[lo:hi]                 # this rank's images, read in place
        out = sb.result_block(step, rank)              # this rank's detections, written in place
        out["score"][...] = x.reshape(hi - lo, -1).sum(axis=1, keepdims=True)
        out["anchor"][...] = np.arange(lo, hi, dtype=np.int32)[:, None]
        out["count"][...] = step

    try:
        for step in range(steps):
            if rank == 0:
                sb.input_slot(step)[...] = np.arange(n_images, dtype=np.float32)[:, None, None, None] + 100 * step
                sb.publish(step)
            if scenario == "silent" and rank == 1 and step == 2:
                time.sleep(3600)                       # never reports; the owner's gather must give up
            if scenario == "raises" and rank == 1 and step == 2:
                sb.fail()
                raise SystemExit(0)
            sb.wait_input(step, timeout=20)
            fake_detector(step)
            sb.report(step)
            if rank == 0:
                got = sb.gather(step, timeout=2.0 if scenario != "ok" else 20.0, merged=True)
                assert got["anchor"][:, 0].tolist() == list(range(n_images)), got["anchor"][:, 0]
                want = (np.arange(n_images) + 100 * step) * 60.0
                assert np.array_equal(got["score"][:, 0], want.astype(np.float32))
                assert (got["count"] == step).all() and got["score"].shape == (n_images, 4)
                sb.release(step)
        if rank == 0:
            print("OK all steps")
    except sharding.ShardTimeout as e:
        print("TIMEOUT ranks", e.ranks, flush=True)
        sb.close()                                     # the owner removes the regions' names
        os._exit(0)
    except sharding.ShardFailed as e:
        print("FAILED ranks", e.ranks, flush=True)
        sb.close()
        os._exit(0)
    if scenario == "ok":
        dist.barrier()
        sb.close()
        dist.destroy_process_group()
""") % ROOT


def _run_shared(tmp_path, scenario, world, n_images, timeout=120):
    script = tmp_path / "shared_worker.py"
    script.write_text(SHARED_WORKER)
    port = 29000 + (os.getpid() % 400) + 7 * world + len(scenario)
    procs = []
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world))
    for rank in range(world):
        procs.append(subprocess.Popen([sys.executable, str(script), scenario, str(n_images)], env=dict(env, RANK=str(rank)),
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    out0, err0 = procs[0].communicate(timeout=timeout)          # the owner decides the outcome
    for p in procs[1:]:
        try:
            p.wait(timeout=10)
        except subprocess.TimeoutExpired:
            p.kill()                                            # the rank that was made to hang (exact child, by handle)
            p.wait()
    assert procs[0].returncode == 0, err0[-2000:]
    return out0


@pytest.mark.parametrize("world,n_images", [(2, 9), (3, 8)])
def test_shared_scatter_and_gather_in_place(tmp_path, world, n_images):
    """One batch written once by rank 0, every rank reads its images and writes its detections in place, rank 0
    reads all of them in image order; five steps over the two alternating slots."""
    assert "OK all steps" in _run_shared(tmp_path, "ok", world, n_images)


def test_owner_detects_a_rank_that_stops_answering(tmp_path):
    """Failure made on the host: rank 1 stops reporting at step 2 (it sleeps); the owner's gather gives up after its
    time limit and names the rank."""
    assert "TIMEOUT ranks [1]" in _run_shared(tmp_path, "silent", 2, 6)


def test_owner_learns_of_a_rank_that_reports_failure(tmp_path):
    """Rank 1 marks itself failed and exits between steps; the owner's gather raises at once, naming it."""
    assert "FAILED ranks [1]" in _run_shared(tmp_path, "raises", 2, 6)
