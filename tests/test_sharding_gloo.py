"""The N > 1 path on CPU: two gloo ranks shard a batch by plane, each computes only its own
planes (with the checker standing in for the GPU), and the pieces reassemble to the unsharded
result.  Also checks the max-over-ranks reduction used for every multi-GPU timing."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from fusedkernellibrary_b200 import chains, sharding  # noqa: E402


def test_plane_ranges_tile_the_batch():
    for n in (0, 1, 5, 64, 1023, 1024):
        for world in (1, 2, 3, 4, 8):
            got = []
            for r in range(world):
                first, count = sharding.plane_range(n, world, r)
                got += list(range(first, first + count))
            assert got == list(range(n))
            sizes = [sharding.plane_range(n, world, r)[1] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
            inter = sorted(sum((sharding.interleaved_planes(n, world, r) for r in range(world)), []))
            assert inter == list(range(n))
    with pytest.raises(ValueError):
        sharding.plane_range(10, 2, 2)


def _case(n=21, fw=160, fh=90, dw=32, dh=24):
    rng = np.random.default_rng(42)
    frames = [rng.integers(0, 256, (fh, fw * 3), dtype=np.uint8) for _ in range(3)]
    rects = chains.random_rects(rng, n, fw, fh, lo=4, hi=80)
    fi = [i % 3 for i in range(n)]
    return frames, rects, fi, (n, fw, fh, dw, dh)


def _run_planes(frames, rects, fi, dims, first, count, out):
    from oracle import port
    n, fw, fh, dw, dh = dims
    plan = chains.crop_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], frame_index=fi[first:first + count],
                                    rects=rects[first:first + count], src_width=fw, src_height=fh, src_pitch=fw * 3,
                                    dst=out.ctypes.data + first * dw * dh * 12, dst_width=dw, dst_height=dh,
                                    post_ops=chains.normalize_ops(), planar=True)
    if count:
        port.run(plan)


def _worker(rank, world, port_no, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    frames, rects, fi, dims = _case()
    n, fw, fh, dw, dh = dims
    first, count = sharding.plane_range(n, world, rank)
    out = np.zeros((n, 3, dh, dw), np.float32)
    _run_planes(frames, rects, fi, dims, first, count, out)
    # consolidated output requested: gather the contiguous slabs on every rank
    t = torch.from_numpy(out)
    dist.all_reduce(t)           # untouched planes are zero, so a sum assembles the tensor
    slowest = sharding.max_over_ranks(1.0 + rank)
    if rank == 0:
        np.save(os.path.join(tmp, "gathered.npy"), t.numpy())
        np.save(os.path.join(tmp, "slowest.npy"), np.array([slowest]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reassemble_the_unsharded_result(tmp_path, oracle_port):
    world = 2
    port_no = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port_no, str(tmp_path)), nprocs=world, join=True)
    frames, rects, fi, dims = _case()
    n, fw, fh, dw, dh = dims
    whole = np.zeros((n, 3, dh, dw), np.float32)
    _run_planes(frames, rects, fi, dims, 0, n, whole)
    gathered = np.load(tmp_path / "gathered.npy")
    assert np.array_equal(gathered.view(np.uint32), whole.view(np.uint32))
    assert np.load(tmp_path / "slowest.npy")[0] == 2.0
