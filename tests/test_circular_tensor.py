"""fkb_circular_tensor_*: the reference's CircularTensor::update (core/data/circular_tensor.h:111-161) as one plan.

CPU part: the tensor is created over host buffers, every update's plan (fkb_circular_tensor_plan_update) is run by the
plain-C checker, and the visible tensor is compared after every update with a restatement of the reference's index
arithmetic (oracle/circular_model.py) fed with the chain's result computed alone.  The sliding-window mode, which the
reference does not have, must show the same visible tensor without a single copy plane.
GPU part: the same through fkb_circular_tensor_update on device memory the library allocates, with the allocation
counters still after the first updates; and, update by update, the visible tensor AND the hidden ring against the
reference's own divergent kernel running the two operation sequences that CircularTensor::update builds
(oracle/ref/fklref_circular.cpp; the reference lacks only the host launcher for that kernel).
"""
import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op
from oracle import circular_model as cm
from oracle import reference_gpu as refgpu
from tests import cases as tc

W, H = 40, 28   # plane size
FW, FH = 96, 54  # frames the new images are cropped from

FORMATS = {
    "float3": (abi.DST_F32X3_PACKED, np.float32, (H, W, 3)),
    "uchar3": (abi.DST_U8X3_PACKED, np.uint8, (H, W, 3)),
    "planar": (abi.DST_F32_PLANAR3, np.float32, (3, H, W)),
}


def _chain_plan(fmt_name, frame_ptr, rect, dst_ptr=0):
    """crop -> PRESERVE_AR resize -> normalise (or -> saturate for the uchar3 tensor) of one new image."""
    dst_fmt = FORMATS[fmt_name][0]
    ops = chains.normalize_ops() if fmt_name != "uchar3" else [op(abi.OP_MUL, 1.1), op(abi.OP_SATURATE_CAST_U8)]
    plan = abi.HostPlan()
    seq = plan.add_sequence(abi.SRC_U8X3, dst_fmt, abi.RESIZE_PRESERVE_AR, ops, background=(3.0, 2.0, 1.0))
    px = {"float3": 12, "uchar3": 3, "planar": 4}[fmt_name]
    plan.add_plane(src=frame_ptr, src_width=FW, src_height=FH, src_pitch=FW * 3, crop=rect, dst=dst_ptr, dst_width=W, dst_height=H,
                   dst_pitch=W * px, dst_channel_stride=W * H * 4 if fmt_name == "planar" else 0, sequence=seq)
    return plan


def _frames(seed, n):
    rng = np.random.default_rng(seed)
    frames = [rng.integers(0, 256, (FH, FW * 3), dtype=np.uint8) for _ in range(n)]
    rects = chains.random_rects(rng, n, FW, FH, lo=8, hi=50)
    return frames, [tuple(int(v) for v in r) for r in rects]


def _alone(oracle_port, fmt_name, frame, rect):
    _, dtype, shape = FORMATS[fmt_name]
    out = np.zeros(shape, dtype)
    oracle_port.run(_chain_plan(fmt_name, frame.ctypes.data, rect, out.ctypes.data))
    return out


@pytest.mark.parametrize("fmt_name", ["float3", "uchar3", "planar"])
@pytest.mark.parametrize("order", [abi.CIRCULAR_NEWEST_FIRST, abi.CIRCULAR_OLDEST_FIRST])
@pytest.mark.parametrize("batch", [1, 2, 5])
def test_update_plans_reproduce_the_reference_scheme(fkb_lib, oracle_port, fmt_name, order, batch):
    dst_fmt, dtype, shape = FORMATS[fmt_name]
    frames, rects = _frames(500 + batch, 2 * batch + 3)
    for sliding in (False, True):
        plane_bytes, tensor_bytes, ring_bytes = abi.CircularTensor.sizes(W, H, batch, dst_fmt, sliding)
        assert plane_bytes == int(np.prod(shape)) * np.dtype(dtype).itemsize
        assert (tensor_bytes, ring_bytes) == ((2 * batch * plane_bytes, 0) if sliding else (batch * plane_bytes, batch * plane_bytes))
        tensor = np.zeros(tensor_bytes, np.uint8)
        ring = np.zeros(max(ring_bytes, 1), np.uint8)
        ct = abi.CircularTensor(W, H, batch, dst_fmt, order, sliding, tensor.ctypes.data, ring.ctypes.data)
        model = cm.CircularTensorModel(batch, order, shape, dtype)
        for k, (frame, rect) in enumerate(zip(frames, rects)):
            assert ct.next_index == (0 if sliding else k % batch)
            plan = ct.plan_update(_chain_plan(fmt_name, frame.ctypes.data, rect))
            assert plan.n_planes == (2 if sliding else batch + 1)
            oracle_port.run(plan)
            want = model.update(_alone(oracle_port, fmt_name, frame, rect))
            off = ct.data - tensor.ctypes.data
            assert 0 <= off <= tensor_bytes - batch * plane_bytes and off % plane_bytes == 0
            got = tensor[off:off + batch * plane_bytes].view(dtype).reshape(want.shape)
            assert np.array_equal(tc.bits(got), tc.bits(want)), f"update {k} (sliding={sliding})"
        ct.destroy()


def test_the_model_orders_results_as_documented():
    """Newest first: plane z holds the result of z updates ago; oldest first: plane BATCH-1-z does."""
    for order in (cm.NEWEST_FIRST, cm.OLDEST_FIRST):
        m = cm.CircularTensorModel(4, order, (1,), np.int32)
        for k in range(1, 11):
            v = m.update(np.array([k], np.int32)).reshape(-1)
            ages = [max(k - z, 0) for z in range(4)]
            assert list(v) == (ages if order == cm.NEWEST_FIRST else ages[::-1])


def test_updates_with_another_receiver_or_bad_descriptions_are_refused(fkb_lib):
    buf = np.zeros(1 << 20, np.uint8)
    ct = abi.CircularTensor(W, H, 3, abi.DST_F32X3_PACKED, tensor=buf.ctypes.data, ring=buf.ctypes.data + (1 << 19))
    with pytest.raises(abi.FkbError) as e:
        ct.plan_update(_chain_plan("planar", buf.ctypes.data, (0, 0, 8, 8)))
    assert e.value.status == abi.ERR_INVALID_ARGUMENT and "receiver" in str(e.value)
    assert ct.next_index == 0
    ct.destroy()
    for bad in (dict(batch=0), dict(width=0), dict(order=7), dict(dst_format=99)):
        args = dict(width=W, height=H, batch=3, dst_format=abi.DST_F32X3_PACKED, order=0)
        args.update(bad)
        with pytest.raises(abi.FkbError):
            abi.CircularTensor(args["width"], args["height"], args["batch"], args["dst_format"], args["order"], False, buf.ctypes.data,
                               buf.ctypes.data)


@pytest.mark.gpu
@pytest.mark.parametrize("sliding", [False, True])
@pytest.mark.parametrize("fmt_name,order", [("planar", abi.CIRCULAR_NEWEST_FIRST), ("float3", abi.CIRCULAR_OLDEST_FIRST),
                                            ("uchar3", abi.CIRCULAR_NEWEST_FIRST)])
def test_updates_on_the_gpu(fkb_lib, oracle_port, fmt_name, order, sliding):
    torch = pytest.importorskip("torch")
    dst_fmt, dtype, shape = FORMATS[fmt_name]
    batch = 6
    frames, rects = _frames(600, 2 * batch + 2)
    d_frames = [torch.from_numpy(f).cuda() for f in frames]
    stream = torch.cuda.Stream()
    ct = abi.CircularTensor(W, H, batch, dst_fmt, order, sliding)
    model = cm.CircularTensorModel(batch, order, shape, dtype)
    counters = None
    for k, (frame, rect) in enumerate(zip(frames, rects)):
        if k == 2:
            torch.cuda.synchronize()
            counters = abi.debug_counters()
        ct.update(_chain_plan(fmt_name, d_frames[k].data_ptr(), rect), stream.cuda_stream)
        assert abi.async_check(stream.cuda_stream) == 0
        want = model.update(_alone(oracle_port, fmt_name, frame, rect))
        got = np.empty(want.shape, dtype)
        tc.cuda_copy_to_host(got, ct.data)
        assert np.array_equal(tc.bits(got), tc.bits(want)), f"update {k}"
    after = abi.debug_counters()
    assert (after.device_allocations, after.device_frees, after.host_pinned_allocations) == \
           (counters.device_allocations, counters.device_frees, counters.host_pinned_allocations), "an update allocated memory"
    ct.destroy()


@pytest.mark.gpu
@pytest.mark.skipif(not refgpu.available("nofma"), reason="reference CUDA build not present")
@pytest.mark.parametrize("planar", [True, False])
@pytest.mark.parametrize("order", [abi.CIRCULAR_NEWEST_FIRST, abi.CIRCULAR_OLDEST_FIRST])
def test_updates_equal_the_reference_divergent_kernel(fkb_lib, planar, order):
    torch = pytest.importorskip("torch")
    batch, dw, dh = 6, 70, 45           # the reference unit is built for BATCH = 6
    rng = np.random.default_rng(700)
    frames = [torch.from_numpy(rng.integers(0, 256, (540, 960 * 3), dtype=np.uint8)).cuda() for _ in range(3)]
    rects = chains.random_rects(rng, 15, 960, 540, lo=10, hi=400)
    dst_fmt = abi.DST_F32_PLANAR3 if planar else abi.DST_F32X3_PACKED
    shape = (batch, 3, dh, dw) if planar else (batch, dh, dw, 3)
    ours_v, ours_h, ref_v, ref_h = (torch.zeros(shape, dtype=torch.float32, device="cuda") for _ in range(4))
    ct = abi.CircularTensor(dw, dh, batch, dst_fmt, order, False, ours_v.data_ptr(), ours_h.data_ptr())
    stream = torch.cuda.Stream()
    refgpu.set_stream(stream.cuda_stream, "nofma")
    bg = (0.5, 0.25, 0.125)
    for k in range(15):
        rect = tuple(int(v) for v in rects[k])
        plan = abi.HostPlan()
        seq = plan.add_sequence(abi.SRC_U8X3, dst_fmt, abi.RESIZE_PRESERVE_AR, chains.normalize_ops(), background=bg)
        plan.add_plane(src=frames[k % 3].data_ptr(), src_width=960, src_height=540, src_pitch=2880, crop=rect, dst=0, dst_width=dw,
                       dst_height=dh, dst_pitch=0, sequence=seq)
        first = ct.next_index
        assert first == k % batch
        ct.update(plan, stream.cuda_stream)
        refgpu.circular_update6(frames[k % 3].data_ptr(), 960, 540, 2880, rect, dw, dh, bg, 255.0, chains.IMAGENET_MEAN, chains.IMAGENET_STD,
                                ref_v.data_ptr(), ref_h.data_ptr(), first, order, planar, flavour="nofma")
        assert abi.async_check(stream.cuda_stream) == 0
        assert torch.equal(ours_v.view(torch.int32), ref_v.view(torch.int32)), f"update {k}: visible tensor differs"
        assert torch.equal(ours_h.view(torch.int32), ref_h.view(torch.int32)), f"update {k}: hidden ring differs"
    assert ours_v.abs().sum().item() > 0
    ct.destroy()
