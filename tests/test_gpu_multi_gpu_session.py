"""fkb_multi_gpu_session_*: one batch over the GPUs of a box, sharded by plane, host buffers in.

On one GPU: the session with a single device equals the checker; a requested device that does not exist, or
that a test declared unavailable (host-side failure injection: no GPU is made to fail), is left out and its
planes go to the devices that answer.  On two or more GPUs: both devices take part, and with the gather flag
every device ends up with the whole output tensor in its own memory (NCCL moves the slabs; no kernel reads a
peer's memory).
"""
import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from tests import cases as tc

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _case(n=37):
    return tc.crop_resize_case("mgpu", 401, 3, 480, 272, n, 64, 48, True, chains.normalize_ops())


def _host_plan(case):
    arrays = {**case.sources, **case.outputs}
    return case.build(lambda name: arrays[name].ctypes.data)


def test_one_device_and_devices_that_do_not_answer(fkb_lib, oracle_port):
    case = _case()
    want = tc.run_on_host(case, oracle_port)["out"].copy()
    n_dev = torch.cuda.device_count()
    # a device ordinal beyond those present is left out; everything runs on device 0
    case.outputs["out"][...] = 0
    sess = abi.MultiGpuSession(_host_plan(case), [0, n_dev + 3])
    sess.run()
    a, b = sess.shard(0), sess.shard(1)
    assert (a.available, a.first_plane, a.n_planes) == (1, 0, 37)
    assert (b.available, b.n_planes) == (0, 0)
    assert a.last_step_ms > 0
    assert np.array_equal(tc.bits(case.outputs["out"]), tc.bits(want))
    sess.run()     # a second step over the same buffers
    assert np.array_equal(tc.bits(case.outputs["out"]), tc.bits(want))
    sess.destroy()
    # host-side failure injection: the only device is declared unavailable -> an error, never a fallback
    fkb_lib.fkb_debug_set_device_unavailable(0, 1)
    try:
        with pytest.raises(abi.FkbError) as e:
            abi.MultiGpuSession(_host_plan(case), [0])
        assert e.value.status == abi.ERR_NO_DEVICE
    finally:
        fkb_lib.fkb_debug_set_device_unavailable(0, 0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_devices_shard_by_plane_and_gather_the_consolidated_tensor(fkb_lib, oracle_port):
    case = _case(n=41)       # 21 + 20 planes: slabs of unequal size
    want = tc.run_on_host(case, oracle_port)["out"].copy()
    case.outputs["out"][...] = 0
    sess = abi.MultiGpuSession(_host_plan(case), [0, 1], abi.MULTI_GPU_DOWNLOAD | abi.MULTI_GPU_GATHER)
    sess.run()
    s0, s1 = sess.shard(0), sess.shard(1)
    assert (s0.first_plane, s0.n_planes, s1.first_plane, s1.n_planes) == (0, 21, 21, 20)
    assert np.array_equal(tc.bits(case.outputs["out"]), tc.bits(want)), "outputs copied back to the host"
    # the consolidated tensor as each device holds it: plain copies out of the library's buffers
    from cuda.bindings import runtime as cudart
    for sh in (s0, s1):
        assert sh.consolidated_bytes == want.nbytes
        got = np.empty_like(want)
        with torch.cuda.device(sh.device):
            torch.cuda.synchronize()
            (err,) = cudart.cudaMemcpy(got.ctypes.data, sh.consolidated_output, want.nbytes, cudart.cudaMemcpyKind.cudaMemcpyDeviceToHost)
            assert int(err) == 0
        assert np.array_equal(tc.bits(got), tc.bits(want)), f"consolidated tensor on device {sh.device}"
    # one device declared unavailable: the other takes the whole batch
    sess.destroy()
    fkb_lib.fkb_debug_set_device_unavailable(1, 1)
    try:
        case.outputs["out"][...] = 0
        sess = abi.MultiGpuSession(_host_plan(case), [0, 1])
        sess.run()
        assert (sess.shard(0).n_planes, sess.shard(1).available, sess.shard(1).n_planes) == (41, 0, 0)
        assert np.array_equal(tc.bits(case.outputs["out"]), tc.bits(want))
        sess.destroy()
    finally:
        fkb_lib.fkb_debug_set_device_unavailable(1, 0)
