"""The asynchronous, allocation-free call (fkb_execute_async) and the time-bounded device waits.

The reference's call is one asynchronous launch with no allocation (core/execution_model/executors.h:284-285);
fkb_execute_async is held to the same: after the first call on a device the library's allocation counters must
not move, the call must return while earlier work on the stream is still running, and its results must equal
the ordinary plan's bit for bit.

The waits: a staged kernel waits on an mbarrier for its bulk copies with a wall-clock limit.  The test makes a
wait run out WITHOUT a fault or a hang: a test-only plan option lets every block expect 16 bytes more than its
copies deliver, so the copies all complete, the barrier phase never does, the block records the time-out in the
plan's status word and returns.  fkb_plan_check then reports FKB_ERR_DEVICE_WAIT once, and the next ordinary
launch on the same device is correct.
"""
import time

import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from tests import cases as tc

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from tests.test_gpu_parity import DeviceArrays  # noqa: E402


def _want(case, oracle_port):
    return {k: v.copy() for k, v in tc.run_on_host(case, oracle_port).items()}


def _assert_outputs(case, dev, want, what):
    for k, v in case.outputs.items():
        assert np.array_equal(tc.bits(dev.download(k, v)), tc.bits(want[k])), f"{what}: {case.name}/{k}"


@pytest.mark.parametrize("kind", ["u8_staged", "nv12_staged"])
def test_a_wait_that_runs_out_is_reported_once_and_the_device_stays_usable(fkb_lib, oracle_port, kind):
    if kind == "u8_staged":
        case = tc.crop_resize_case("wait_u8", 201, 1, 256, 64, 1, 32, 32, True, chains.normalize_ops(), rects=[(16, 8, 96, 40)])
    else:
        case = tc.nv12_case("wait_nv12", 202, 1, 128, 64, 32, 32)
    want = _want(case, oracle_port)
    dev = DeviceArrays(case)
    plan = abi.DevicePlan(case.build(dev.ptr))
    plan.set_option(abi.PLAN_WAIT_LIMIT_US, 2000)
    plan.set_option(abi.PLAN_TEST_EXPECT_EXTRA_BYTES, 16)
    t0 = time.perf_counter()
    plan.launch()
    with pytest.raises(abi.FkbError) as e:
        plan.check()
    elapsed = time.perf_counter() - t0
    assert e.value.status == abi.ERR_DEVICE_WAIT
    # every block gives up after 2 ms and waits 2 ms more for stragglers: a few blocks, well under a second
    assert elapsed < 1.0, f"the kernel took {elapsed:.3f} s to give up"
    # reported once: the word was cleared, a second check of the same (finished) launch is clean
    assert plan.check() == 0
    # the same plan without the surplus, on the same device: complete and bit-exact
    plan.set_option(abi.PLAN_TEST_EXPECT_EXTRA_BYTES, 0)
    for k in case.outputs:
        dev.t[k].fill_(0xCD)
    plan.launch()
    assert plan.check() == 0
    _assert_outputs(case, dev, want, "after a timed-out launch")
    plan.destroy()


def test_wait_limit_option_is_validated(fkb_lib):
    case = tc.crop_resize_case("opt", 203, 1, 256, 64, 1, 32, 32, True, chains.normalize_ops(), rects=[(16, 8, 96, 40)])
    dev = DeviceArrays(case)
    plan = abi.DevicePlan(case.build(dev.ptr))
    for option, value in ((abi.PLAN_WAIT_LIMIT_US, 0), (abi.PLAN_WAIT_LIMIT_US, 5_000_000), (abi.PLAN_TEST_EXPECT_EXTRA_BYTES, 8), (99, 1)):
        with pytest.raises(abi.FkbError) as e:
            plan.set_option(option, value)
        assert e.value.status == abi.ERR_INVALID_ARGUMENT
    plan.destroy()


def test_async_call_allocates_nothing_after_the_first_and_returns_before_the_stream_is_done(fkb_lib, oracle_port):
    big = tc.crop_resize_case("async_big", 211, 3, 480, 272, 300, 64, 48, True, chains.normalize_ops())
    small = tc.elementwise_case("async_small", 212, 64, 33, chains.cast_mul_sub_div_ops())     # travels in the kernel arguments
    nv = tc.nv12_case("async_nv12", 213, 2, 96, 54, 40, 22)
    prepared = []
    for case in (big, small, nv):
        prepared.append((case, DeviceArrays(case, fill=0xCD), _want(case, oracle_port)))
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    # first call on the device: the arena is allocated here and never again
    abi.execute_async(prepared[0][0].build(prepared[0][1].ptr), sh)
    assert abi.async_check(sh) == 0
    before = abi.debug_counters()
    free_before, _ = torch.cuda.mem_get_info()
    descs = [(c, d, w, c.build(d.ptr)) for c, d, w in prepared]
    for rep in range(3):
        for case, dev, want, desc in descs:
            abi.execute_async(desc, sh)
    # the call returns while the stream is still busy with earlier work
    with torch.cuda.stream(stream):
        torch.cuda._sleep(int(2e8))            # about 0.1 s of spinning on the device
    t0 = time.perf_counter()
    abi.execute_async(descs[0][3], sh)
    host_s = time.perf_counter() - t0
    assert not stream.query(), "the stream finished before the call returned: nothing was shown"
    assert host_s < 0.05, f"fkb_execute_async took {host_s * 1e3:.1f} ms with a busy stream: it must not synchronise"
    assert abi.async_check(sh) == 0
    after = abi.debug_counters()
    free_after, _ = torch.cuda.mem_get_info()
    assert (after.device_allocations, after.device_frees, after.host_pinned_allocations) == \
           (before.device_allocations, before.device_frees, before.host_pinned_allocations)
    assert free_after == free_before
    # the three descriptions were lowered once each (the first one before the counters were read) and reused after
    assert after.plans_lowered - before.plans_lowered == 2
    assert after.plans_reused - before.plans_reused == 3 * 3 + 1 - 2
    for case, dev, want, _ in descs:
        _assert_outputs(case, dev, want, "fkb_execute_async")


def test_async_ring_wraps_around_without_corrupting_tables_in_flight(fkb_lib, oracle_port):
    """More distinct descriptions than the arena holds: tables are evicted and their ranges reused only after
    the launches that read them have finished."""
    rng = np.random.default_rng(214)
    fw, fh, dw, dh = 480, 272, 32, 32
    frame = rng.integers(0, 256, (fh, fw * 3), dtype=np.uint8)
    d_frame = torch.from_numpy(frame).cuda()
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    n_desc, n_planes = 40, 2500                 # 40 tables of about 0.4 MB against an arena of 8 MB
    outs, wants, rects_all = [], [], []
    check_planes = [0, 1, n_planes // 2, n_planes - 1]
    for i in range(n_desc):
        rects = chains.random_rects(rng, n_planes, fw, fh, lo=4, hi=100)
        rects_all.append(rects)
        outs.append(torch.full((n_planes, 3, dh, dw), -1.0, dtype=torch.float32, device="cuda"))
    for i in range(n_desc):
        desc = chains.crop_resize_batch(frame_ptrs=[d_frame.data_ptr()], frame_index=[0] * n_planes, rects=rects_all[i],
                                        src_width=fw, src_height=fh, src_pitch=fw * 3, dst=outs[i].data_ptr(), dst_width=dw,
                                        dst_height=dh, post_ops=chains.normalize_ops(), planar=True)
        assert abi.validate(desc).device_bytes > abi.ASYNC_ARENA_BYTES // 32
        abi.execute_async(desc, sh)            # no synchronisation in between: launches pile up behind each other
    assert abi.async_check(sh) == 0
    for i in range(n_desc):
        got = outs[i][check_planes].cpu().numpy()
        want = np.zeros((len(check_planes), 3, dh, dw), np.float32)
        plan = chains.crop_resize_batch(frame_ptrs=[frame.ctypes.data], frame_index=[0] * len(check_planes),
                                        rects=rects_all[i][check_planes], src_width=fw, src_height=fh, src_pitch=fw * 3,
                                        dst=want.ctypes.data, dst_width=dw, dst_height=dh, post_ops=chains.normalize_ops(),
                                        planar=True)
        oracle_port.run(plan)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"description {i}"


def test_async_rejects_what_plan_create_rejects(fkb_lib):
    plan = abi.HostPlan()
    plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, abi.RESIZE_NONE, [abi.op(abi.OP_MUL, 2.0)])   # Mul on uchar3
    src = torch.zeros(8 * 8 * 3, dtype=torch.uint8, device="cuda")
    dst = torch.zeros(8 * 8 * 3, dtype=torch.float32, device="cuda")
    plan.add_plane(src=src.data_ptr(), src_width=8, src_height=8, src_pitch=24, dst=dst.data_ptr(), dst_width=8, dst_height=8,
                   dst_pitch=96)
    with pytest.raises(abi.FkbError) as e:
        abi.execute_async(plan)
    assert e.value.status == abi.ERR_INVALID_ARGUMENT
