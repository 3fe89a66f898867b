"""fkb_execute_static: the one-shot run for hosts that may not allocate device memory.

Some programs that embed this library cannot call cudaMalloc while they are running: a plug-in
in a server whose framework took all of the GPU's memory for its own pool when it started, or a
frame loop with a latency bound that cannot absorb the device-wide stall of cudaMalloc/cudaFree.
For them the library keeps the plan's descriptor table in a fixed array inside the library image
(FKB_STATIC_TABLE_BYTES per GPU) instead of a freshly allocated block.

The array is shared by every call on a device and keeps what the previous call wrote, so the
GPU test runs two different plans back to back through the C ABI and compares each, bit for bit,
with the ordinary entry point (fkb_plan_create + fkb_plan_launch) on the same device buffers
(both run the same kernels, so this compares two entry points of this library; the kernels
themselves are compared with the reference in the parity tests).  It also checks the property
the entry point exists for: after a first call, the library's allocation counters and the
device's free memory do not move, on the default stream and on a stream of the caller's.
This file sorts last so that a stop-at-first-failure run has already run everything else.
"""
import numpy as np
import pytest

from fusedkernellibrary_b200 import abi
from tests import cases as tc


def test_plans_beyond_the_fixed_table_are_refused(fkb_lib):
    """Capacity is checked on the host, before any device is touched: 112 B per plane and 16 B per
    thread block put a 5000-plane batch over the 512 KiB table."""
    src = np.zeros((8, 8 * 3), np.uint8)
    out = np.zeros((5000, 8, 8, 3), np.float32)
    plan = abi.HostPlan()
    seq = plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, abi.RESIZE_NONE, [abi.op(abi.OP_CAST_F32)])
    for i in range(5000):
        plan.add_plane(src=src.ctypes.data, src_width=8, src_height=8, src_pitch=24, dst=out.ctypes.data + i * 768,
                       dst_width=8, dst_height=8, dst_pitch=96, sequence=seq)
    assert abi.validate(plan).device_bytes > abi.STATIC_TABLE_BYTES
    with pytest.raises(abi.FkbError) as e:
        abi.execute_static(plan)
    assert e.value.status == abi.ERR_TOO_LARGE
    assert "fixed table" in str(e.value)


@pytest.mark.gpu
def test_static_table_run_equals_allocating_run_twice_in_a_row(fkb_lib):
    torch = pytest.importorskip("torch")
    from tests.test_gpu_parity import DeviceArrays

    # a batched crop -> resize -> normalise -> planar plan and (smaller table, other kernel body)
    # an NV12 -> RGB -> resize plan: each call finds the previous call's table in the array
    first = tc.crop_resize_case("static_a", 91, 3, 480, 270, 41, 64, 48, True, tc.chains.normalize_ops())
    second = tc.nv12_case("static_b", 92, 3, 96, 54, 40, 22)
    prepared = []
    for case in (first, second):
        dev = DeviceArrays(case)
        plan_desc = case.build(dev.ptr)
        assert abi.validate(plan_desc).device_bytes <= abi.STATIC_TABLE_BYTES
        ordinary = abi.DevicePlan(plan_desc)
        ordinary.launch()
        torch.cuda.synchronize()
        ordinary.destroy()
        want = {k: dev.download(k, v).copy() for k, v in case.outputs.items()}
        prepared.append((case, dev, plan_desc, want))

    def clear(dev, case):
        for k in case.outputs:
            dev.t[k].fill_(0xCD)
        torch.cuda.synchronize()

    for case, dev, _, _ in prepared:
        clear(dev, case)
    # a first call loads the module's array on this device; from then on nothing may be allocated
    abi.execute_static(prepared[0][2])
    clear(prepared[0][1], prepared[0][0])
    own_stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    counters_before = abi.debug_counters()
    free_before, _ = torch.cuda.mem_get_info()
    # calls in a row: A, B, then A again over B's leftovers, the last one on a stream of the caller's
    order = [prepared[0], prepared[1], prepared[0]]
    for n, (case, dev, plan_desc, want) in enumerate(order):
        if n == 2:
            clear(dev, case)
        abi.execute_static(plan_desc, own_stream.cuda_stream if n == 2 else None)   # returns after its stream has been synchronised
        for k, v in case.outputs.items():
            got = dev.download(k, v)
            assert np.array_equal(tc.bits(got), tc.bits(want[k])), f"call {n} ({case.name}/{k}) differs from fkb_plan_launch"
    counters_after = abi.debug_counters()
    free_after, _ = torch.cuda.mem_get_info()
    assert (counters_after.device_allocations, counters_after.device_frees, counters_after.host_pinned_allocations) == \
           (counters_before.device_allocations, counters_before.device_frees, counters_before.host_pinned_allocations)
    assert free_after == free_before, "device memory was allocated or freed during fkb_execute_static"
