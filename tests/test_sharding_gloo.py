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


def test_planes_of_an_unavailable_device_go_to_the_others():
    """The dispatcher's failure rule, on the host alone: a device that does not answer gets nothing and the
    batch is re-assigned over the rest, still in contiguous ranges in device order."""
    from fusedkernellibrary_b200 import abi
    assert abi.assign_planes(10, 4, [1, 0, 1, 1]) == [(0, 4), (4, 0), (4, 3), (7, 3)]
    assert abi.assign_planes(1024, 8, [1] * 8) == [(128 * r, 128) for r in range(8)]
    for n in (0, 1, 7, 1023):
        for avail in ([0, 1, 1], [1, 1, 0], [0, 0, 1], [1, 0, 0, 1, 0, 1, 1, 0]):
            got = abi.assign_planes(n, len(avail), avail)
            covered = []
            for (first, count), a in zip(got, avail):
                assert count == 0 or a
                covered += list(range(first, first + count))
            assert covered == list(range(n))
            sizes = [c for (f, c), a in zip(got, avail) if a]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(abi.FkbError) as e:
        abi.assign_planes(10, 3, [0, 0, 0])
    assert e.value.status == abi.ERR_NO_DEVICE


def test_multi_gpu_session_without_a_device_is_an_error_not_a_fallback():
    import ctypes as C
    from fusedkernellibrary_b200 import abi
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    frames, rects, fi, dims = _case()
    n, fw, fh, dw, dh = dims
    out = np.zeros((n, 3, dh, dw), np.float32)
    plan = chains.crop_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], frame_index=fi, rects=rects, src_width=fw,
                                    src_height=fh, src_pitch=fw * 3, dst=out.ctypes.data, dst_width=dw, dst_height=dh,
                                    post_ops=chains.normalize_ops(), planar=True)
    with pytest.raises(abi.FkbError) as e:
        abi.MultiGpuSession(plan, [0, 1])
    assert e.value.status == abi.ERR_NO_DEVICE
    assert not out.any()


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


def _worker(rank, world, port_no, tmp, available=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    frames, rects, fi, dims = _case()
    n, fw, fh, dw, dh = dims
    first, count = sharding.plane_range(n, world, rank, available)
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


def test_three_ranks_with_one_unavailable_still_cover_the_batch(tmp_path, oracle_port):
    """Rank 1 stands for a GPU that did not answer: it joins the process group but computes nothing; the planes it
    would have had are computed by ranks 0 and 2, and the gathered tensor equals the unsharded result."""
    world = 3
    port_no = 31500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port_no, str(tmp_path), [1, 0, 1]), nprocs=world, join=True)
    frames, rects, fi, dims = _case()
    n, fw, fh, dw, dh = dims
    whole = np.zeros((n, 3, dh, dw), np.float32)
    _run_planes(frames, rects, fi, dims, 0, n, whole)
    gathered = np.load(tmp_path / "gathered.npy")
    assert np.array_equal(gathered.view(np.uint32), whole.view(np.uint32))
