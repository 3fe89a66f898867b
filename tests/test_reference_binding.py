"""include/fkb200_executor.h - the binding a maintainer of the reference adds next to executors.h - compiled
against the reference's REAL operation types (oracle/ref/fklref_binding.cpp, built where the reference tree is
present into oracle/_ref/libfklref_binding.so).

CPU part: the plan the binding fills from `PerThreadRead<_2D,uchar3>::build(...).then(Crop<>::build(...))
.then(Resize<...>::build(...))...` equals, field by field, the plan the Python harness builds for the same chain,
and the resize factors and region of interest that the reference's Resize::build stored in its operation
(resize.h:105-166) equal what the library derives (fkb_derive_resize), bit for bit.

GPU part: fk::executeOperations<fkb200::TransformDPP>(stream, sender, receiver) produces, through libfkb200's
kernels, the output of the reference's own CPU backend (oracle/_ref, device branch) bit for bit.
"""
import ctypes as C

import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op
from oracle import binding_check as bc
from oracle import reference as ref

pytestmark = pytest.mark.skipif(not bc.available(), reason="oracle/_ref/libfklref_binding.so not built (reference tree absent)")

PLANE_FIELDS = [f for f, _ in abi.Plane._fields_]


def _assert_same_plan(expected: abi.HostPlan, fkb_lib):
    planes, seqs = bc.last_plan()
    assert len(planes) == expected.n_planes
    for i, (a, b) in enumerate(zip(planes, expected.planes)):
        for f in PLANE_FIELDS:
            assert getattr(a, f) == getattr(b, f), f"plane {i}.{f}: binding {getattr(a, f)} != harness {getattr(b, f)}"
    d = expected.desc()
    assert len(seqs) == d.n_sequences
    for s, (q, ops) in enumerate(seqs):
        e = d.sequences[s]
        assert (q.src_format, q.dst_format, q.resize_mode, q.n_ops, q.n_pre_ops) == \
               (e.src_format, e.dst_format, e.resize_mode, e.n_ops, e.n_pre_ops)
        assert list(q.background) == list(e.background)
        assert (q.border_mode, list(q.border_value), q.deinterlace) == (e.border_mode, list(e.border_value), e.deinterlace)
        if q.resize_mode in (abi.GEOMETRY_WARP_AFFINE, abi.GEOMETRY_WARP_PERSPECTIVE):
            assert list(q.transform) == list(e.transform)
        for k, o in enumerate(ops):
            assert o.opcode == e.ops[k].opcode
            if o.opcode in (abi.OP_MUL, abi.OP_SUB, abi.OP_DIV, abi.OP_ADD):
                assert list(o.p) == list(e.ops[k].p)
    # what the reference's Resize::build computed on the host == what the library derives
    for i, p in enumerate(expected.planes):
        rr = bc.last_reference_resize(i)
        mode = d.sequences[p.sequence].resize_mode
        if mode in (abi.RESIZE_NONE, abi.GEOMETRY_WARP_AFFINE, abi.GEOMETRY_WARP_PERSPECTIVE):
            assert rr is None
            continue
        ours = abi.ResizeParams()
        assert fkb_lib.fkb_derive_resize(p.crop_width, p.crop_height, p.dst_width, p.dst_height, mode, C.byref(ours)) == 0
        bits = lambda f: np.float32(f).view(np.uint32)
        assert (bits(rr.fx), bits(rr.fy), rr.x1, rr.y1, rr.x2, rr.y2) == (bits(ours.fx), bits(ours.fy), ours.x1, ours.y1, ours.x2, ours.y2), i


def test_readme_chain_lowers_to_the_harness_plan(fkb_lib):
    frame, out = 0x10000000, 0x20000000       # never dereferenced when lowering
    bc.readme5(bc.DESCRIBE, frame, 3840, 2160, 11520, chains.README_RECTS, (0, 0, 0), 1.4, 0.5, 255.0, out)
    want = chains.crop_resize_batch(frame_ptrs=[frame], frame_index=[0] * 5, rects=chains.README_RECTS, src_width=3840,
                                    src_height=2160, src_pitch=11520, dst=out, dst_width=60, dst_height=60,
                                    post_ops=chains.readme_ops(), planar=False)
    _assert_same_plan(want, fkb_lib)


def test_batched_planar_chain_lowers_to_the_harness_plan(fkb_lib):
    rng = np.random.default_rng(301)
    rects = chains.random_rects(rng, 16, 3840, 2160, lo=16, hi=512)
    rects[3] = (0, 0, 2, 1000)            # a target that rounds to zero columns (infinite factor in the reference)
    frames = [0x10000000 + 0x2000000 * (i % 8) for i in range(8)]
    fi = [i % 8 for i in range(16)]
    out = 0x70000000
    bc.norm_planar16(bc.DESCRIBE, [frames[i] for i in fi], 3840, 2160, 11520, rects, 224, 224, (0, 0, 0), 255.0,
                     chains.IMAGENET_MEAN, chains.IMAGENET_STD, out)
    want = chains.crop_resize_batch(frame_ptrs=frames, frame_index=fi, rects=rects, src_width=3840, src_height=2160,
                                    src_pitch=11520, dst=out, dst_width=224, dst_height=224, post_ops=chains.normalize_ops(),
                                    planar=True)
    _assert_same_plan(want, fkb_lib)


def test_nv12_chain_and_single_image_chains_lower_to_the_harness_plans(fkb_lib):
    f0, f1, out = 0x10000000, 0x18000000, 0x20000000
    bc.nv12_2(bc.DESCRIBE, [f0, f1], 3840, 2160, 3840, 1280, 720, 255.0, out)
    _assert_same_plan(chains.nv12_resize_batch(frame_ptrs=[f0, f1], width=3840, height=2160, pitch=3840, dst=out, dst_width=1280,
                                               dst_height=720), fkb_lib)
    bc.cast_mul_sub_div(bc.DESCRIBE, f0, 1920, 1080, 5760, 1.4, 0.5, 255.0, out, 23040)
    _assert_same_plan(chains.elementwise(chains.cast_mul_sub_div_ops(), src=f0, dst=out, width=1920, height=1080), fkb_lib)
    bc.cast_resize_add_cast_uint3(bc.DESCRIBE, f0, 128, 128, 384, 32, 32, (3.0, 1.0, 32.0), out, 384)
    want = abi.HostPlan()
    s = want.add_sequence(abi.SRC_U8X3, abi.DST_U32X3_PACKED, abi.RESIZE_IGNORE_AR,
                          [op(abi.OP_CAST_F32), op(abi.OP_ADD, (3.0, 1.0, 32.0)), op(abi.OP_CAST_U32)], n_pre_ops=1)
    want.add_plane(src=f0, src_width=128, src_height=128, src_pitch=384, dst=out, dst_width=32, dst_height=32, dst_pitch=384, sequence=s)
    _assert_same_plan(want, fkb_lib)
    bc.bgr_cast_mul_saturate(bc.DESCRIBE, f0, 64, 32, 192, 1.4, out, 192)
    _assert_same_plan(chains.elementwise([op(abi.OP_SWAP_RB), op(abi.OP_CAST_F32), op(abi.OP_MUL, 1.4), op(abi.OP_SATURATE_CAST_U8)],
                                         src=f0, dst=out, width=64, height=32, dst_format=abi.DST_U8X3_PACKED), fkb_lib)


def test_nv21_left_tsplit_and_partly_filled_batches_lower_to_the_harness_plans(fkb_lib):
    f0, f1, out = 0x10000000, 0x18000000, 0x20000000
    bc.nv21_bt601_2(bc.DESCRIBE, [f0, f1], 1920, 1080, 1920, 640, 360, 255.0, out)
    _assert_same_plan(chains.nv12_resize_batch(frame_ptrs=[f0, f1], width=1920, height=1080, pitch=1920, dst=out, dst_width=640,
                                               dst_height=360, src_format=abi.SRC_NV21, conversion=abi.OP_YUV_TO_RGB_BT601_FULL), fkb_lib)
    # PRESERVE_AR_LEFT into a channel-major tensor [3][4][dh][dw] (TensorTSplit)
    rng = np.random.default_rng(303)
    rects = chains.random_rects(rng, 4, 960, 540, lo=16, hi=300)
    dw, dh = 64, 48
    bc.left_tsplit4(bc.DESCRIBE, [f0, f1, f0, f1], 960, 540, 2880, rects, dw, dh, (1.0, 2.0, 3.0), 255.0, chains.IMAGENET_MEAN,
                    chains.IMAGENET_STD, out)
    want = abi.HostPlan()
    seq = want.add_sequence(abi.SRC_U8X3, abi.DST_F32_PLANAR3, abi.RESIZE_PRESERVE_AR_LEFT, chains.normalize_ops(), background=(1.0, 2.0, 3.0))
    for i in range(4):
        want.add_plane(src=[f0, f1][i % 2], src_width=960, src_height=540, src_pitch=2880, crop=tuple(int(v) for v in rects[i]),
                       dst=out + i * dw * dh * 4, dst_width=dw, dst_height=dh, dst_pitch=dw * 4, dst_channel_stride=4 * dw * dh * 4, sequence=seq)
    _assert_same_plan(want, fkb_lib)
    # BatchRead<4, CONDITIONAL_WITH_DEFAULT>: planes 2 and 3 read the default value
    bc.batch4_default_cast_mul(bc.DESCRIBE, [f0, f1, f0, f1], 64, 32, 192, 2, (7, 200, 33), (1.5, 0.25, 2.0), out)
    planes, seqs = bc.last_plan()
    assert [p.flags for p in planes] == [0, 0, abi.PLANE_DEFAULT_VALUE, abi.PLANE_DEFAULT_VALUE]
    assert [p.sequence for p in planes] == [0, 0, 1, 1] and list(seqs[1][0].background) == [7.0, 200.0, 33.0]
    assert [(p.dst_width, p.dst_height, p.dst - out) for p in planes] == [(64, 32, i * 64 * 32 * 12) for i in range(4)]


def test_circular_tensor_update_sequences_lower_to_the_library_plan(fkb_lib):
    """The two operation sequences of CircularTensor::update (core/data/circular_tensor.h:121-134), lowered by the
    Executor<DivergentBatchTransformDPP> of the binding, give the planes fkb_circular_tensor_plan_update gives."""
    frame, visible, hidden = 0x10000000, 0x20000000, 0x30000000
    dw, dh, bg = 70, 45, (0.5, 0.25, 0.125)
    for order in (abi.CIRCULAR_NEWEST_FIRST, abi.CIRCULAR_OLDEST_FIRST):
        ct = abi.CircularTensor(dw, dh, 6, abi.DST_F32_PLANAR3, order, False, visible, hidden)
        for first in range(8):
            rect = (3 + first, 5, 200 + 7 * first, 100)
            chain = abi.HostPlan()
            seq = chain.add_sequence(abi.SRC_U8X3, abi.DST_F32_PLANAR3, abi.RESIZE_PRESERVE_AR, chains.normalize_ops(), background=bg)
            chain.add_plane(src=frame, src_width=960, src_height=540, src_pitch=2880, crop=rect, dst=0, dst_width=dw, dst_height=dh,
                            dst_pitch=0, sequence=seq)
            assert ct.next_index == first % 6
            want = ct.plan_update(chain)
            bc.circular_describe6(order, frame, 960, 540, 2880, rect, dw, dh, bg, 255.0, chains.IMAGENET_MEAN, chains.IMAGENET_STD,
                                  visible, hidden, first % 6)
            planes, seqs = bc.last_plan()
            assert len(planes) == 7 and len(seqs) == 2
            key = lambda p, q: (p.src, p.src_width, p.src_height, p.src_pitch, p.crop_x, p.crop_y, p.crop_width, p.crop_height, p.dst,
                                p.dst_width, p.dst_height, p.dst_pitch, p.dst_channel_stride, q.src_format, q.dst_format, q.resize_mode,
                                q.n_ops, tuple(q.background))
            d = want.desc()
            ours = sorted(key(p, d.sequences[p.sequence]) for p in want.planes)
            theirs = sorted(key(p, seqs[p.sequence][0]) for p in planes)
            assert ours == theirs, (order, first)
        ct.destroy()


def test_yuv_layouts_lower_to_the_harness_plans(fkb_lib):
    frame, out = 0x10000000, 0x20000000
    for fmt in (abi.SRC_P010, abi.SRC_P210, abi.SRC_Y210, abi.SRC_UYVY):
        bc.yuv_layout(bc.DESCRIBE, fmt, frame, 64, 36, 256, 28, 20, (1.0, 0.5, 2.0), out)
        want = abi.HostPlan()
        seq = want.add_sequence(fmt, abi.DST_F32X3_PACKED, abi.RESIZE_IGNORE_AR, [op(abi.OP_YUV_TO_RGB_BT601_FULL), op(abi.OP_MUL, (1.0, 0.5, 2.0))],
                                n_pre_ops=1)
        want.add_plane(src=frame, src_width=64, src_height=36, src_pitch=256, dst=out, dst_width=28, dst_height=20, dst_pitch=28 * 12, sequence=seq)
        _assert_same_plan(want, fkb_lib)


READBACK_RECT = (-7, -5, 60, 37)
AFFINE = (0.8, 0.25, -3.0, -0.2, 0.7, 2.5, 0.0, 0.0, 1.0)
PERSPECTIVE = (0.9, 0.1, -2.0, 0.05, 0.8, 1.0, 0.002, 0.001, 1.0)


def _readback_plan(src, out, w, h, dw, dh, mode, ops, crop=None, **extras):
    want = abi.HostPlan()
    seq = want.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, mode, ops, **extras)
    want.add_plane(src=src, src_width=w, src_height=h, src_pitch=w * 3, crop=crop, dst=out, dst_width=dw, dst_height=dh,
                   dst_pitch=dw * 12, sequence=seq)
    return want


def test_border_reader_warping_and_deinterlace_lower_to_the_harness_plans(fkb_lib):
    src, out = 0x10000000, 0x20000000
    mul = [op(abi.OP_MUL, (1.0, 0.5, 2.0))]
    for b in range(1, 6):
        bc.border_crop_resize(bc.DESCRIBE, src, 40, 24, 120, b, (9, 99, 199), READBACK_RECT, 36, 28, out)
        _assert_same_plan(_readback_plan(src, out, 40, 24, 36, 28, abi.RESIZE_IGNORE_AR, [], crop=READBACK_RECT, border_mode=b,
                                         border_value=(9.0, 99.0, 199.0) if b == 1 else (0.0, 0.0, 0.0)), fkb_lib)
    bc.warp(bc.DESCRIBE, src, 40, 24, 120, False, AFFINE, 48, 32, (1.0, 0.5, 2.0), out)
    _assert_same_plan(_readback_plan(src, out, 40, 24, 48, 32, abi.GEOMETRY_WARP_AFFINE, mul, transform=AFFINE), fkb_lib)
    bc.warp(bc.DESCRIBE, src, 40, 24, 120, True, PERSPECTIVE, 48, 32, (1.0, 0.5, 2.0), out)
    _assert_same_plan(_readback_plan(src, out, 40, 24, 48, 32, abi.GEOMETRY_WARP_PERSPECTIVE, mul, transform=PERSPECTIVE), fkb_lib)
    for k in (1, 2, 3):
        bc.deinterlace(bc.DESCRIBE, src, 40, 24, 120, k, (1.0, 0.5, 2.0), out)
        _assert_same_plan(_readback_plan(src, out, 40, 24, 40, 24, abi.RESIZE_NONE, mul, deinterlace=k), fkb_lib)


@pytest.mark.gpu
@pytest.mark.parametrize("order", [abi.CIRCULAR_NEWEST_FIRST, abi.CIRCULAR_OLDEST_FIRST])
def test_the_reference_circular_tensor_class_updates_through_the_binding(fkb_lib, order):
    """fk::CircularTensor::update, compiled from the reference's header, against fkb_circular_tensor_update and - where the
    reference CUDA build is present - against the reference's own divergent kernel."""
    torch = pytest.importorskip("torch")
    from oracle import reference_gpu as refgpu
    from tests import cases as tc
    dw, dh, batch, bg = 70, 45, 6, (0.5, 0.25, 0.125)
    rng = np.random.default_rng(305)
    frames = [torch.from_numpy(rng.integers(0, 256, (540, 960 * 3), dtype=np.uint8)).cuda() for _ in range(3)]
    rects = chains.random_rects(rng, 14, 960, 540, lo=10, hi=400)
    stream = torch.cuda.Stream()
    theirs = bc.ReferenceCircularTensor(order, dw, dh)
    ours = abi.CircularTensor(dw, dh, batch, abi.DST_F32_PLANAR3, order)
    use_kernel = refgpu.available("nofma")
    ref_v, ref_h = (torch.zeros((batch, 3, dh, dw), dtype=torch.float32, device="cuda") for _ in range(2))
    if use_kernel:
        refgpu.set_stream(stream.cuda_stream, "nofma")
    a, b = np.empty((batch, 3, dh, dw), np.float32), np.empty((batch, 3, dh, dw), np.float32)
    for k in range(14):
        rect = tuple(int(v) for v in rects[k])
        chain = abi.HostPlan()
        seq = chain.add_sequence(abi.SRC_U8X3, abi.DST_F32_PLANAR3, abi.RESIZE_PRESERVE_AR, chains.normalize_ops(), background=bg)
        chain.add_plane(src=frames[k % 3].data_ptr(), src_width=960, src_height=540, src_pitch=2880, crop=rect, dst=0, dst_width=dw,
                        dst_height=dh, dst_pitch=0, sequence=seq)
        ours.update(chain, stream.cuda_stream)
        theirs.update(frames[k % 3].data_ptr(), 960, 540, 2880, rect, bg, 255.0, chains.IMAGENET_MEAN, chains.IMAGENET_STD, stream.cuda_stream)
        if use_kernel:
            refgpu.circular_update6(frames[k % 3].data_ptr(), 960, 540, 2880, rect, dw, dh, bg, 255.0, chains.IMAGENET_MEAN, chains.IMAGENET_STD,
                                    ref_v.data_ptr(), ref_h.data_ptr(), k % batch, order, True, flavour="nofma")
        assert abi.async_check(stream.cuda_stream) == 0
        tc.cuda_copy_to_host(a, ours.data)
        tc.cuda_copy_to_host(b, theirs.data)
        # planes that no update has reached yet hold whatever the reference's allocation held: compare the ones written
        written = min(k + 1, batch)
        sel = slice(0, written) if order == abi.CIRCULAR_NEWEST_FIRST else slice(batch - written, batch)
        assert np.array_equal(tc.bits(a[sel]), tc.bits(b[sel])), f"update {k}"
        if use_kernel:
            assert np.array_equal(tc.bits(b[sel]), tc.bits(ref_v.cpu().numpy()[sel])), f"update {k}: differs from the reference kernel"
    theirs.destroy()
    ours.destroy()


@pytest.mark.gpu
@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built")
def test_yuv_layouts_through_the_binding_equal_the_reference_cpu_backend(fkb_lib):
    torch = pytest.importorskip("torch")
    from tests import cases as tc
    rng = np.random.default_rng(306)
    stream = torch.cuda.Stream()
    for fmt in (abi.SRC_P010, abi.SRC_P210, abi.SRC_Y210, abi.SRC_UYVY):
        img = tc.yuv_layout_image(rng, fmt, 96, 54, pitch_pad=8)
        d_img = torch.from_numpy(img.view(np.uint8).reshape(-1).copy()).cuda()
        d_out = torch.zeros((30, 50, 3), dtype=torch.float32, device="cuda")
        bc.yuv_layout(bc.EXECUTE, fmt, d_img.data_ptr(), 96, 54, img.strides[0], 50, 30, (1.0, 0.5, 2.0), d_out.data_ptr(), stream.cuda_stream)
        assert abi.async_check(stream.cuda_stream) == 0
        want = ref.yuv_format_chain(img, fmt, 1, 96, 54, 50, 30, (1.0, 0.5, 2.0))
        assert np.array_equal(tc.bits(d_out.cpu().numpy()), tc.bits(want)), fmt


@pytest.mark.gpu
@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built")
def test_read_back_operations_through_the_binding_equal_the_reference_cpu_backend(fkb_lib):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(304)
    same = lambda a, b: np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    img = rng.integers(0, 256, (54, 96, 3), dtype=np.uint8)
    d_img = torch.from_numpy(img).cuda()
    rect = (-20, -11, 140, 80)
    for b in range(1, 6):
        d_out = torch.zeros((45, 70, 3), dtype=torch.float32, device="cuda")
        bc.border_crop_resize(bc.EXECUTE, d_img.data_ptr(), 96, 54, 288, b, (9, 99, 199), rect, 70, 45, d_out.data_ptr(), sh)
        assert abi.async_check(sh) == 0
        assert same(d_out.cpu().numpy(), ref.border_crop_resize(img, b, (9, 99, 199), rect, 70, 45)), b
    for persp, m in ((False, AFFINE), (True, PERSPECTIVE)):
        d_out = torch.zeros((64, 100, 3), dtype=torch.float32, device="cuda")
        bc.warp(bc.EXECUTE, d_img.data_ptr(), 96, 54, 288, persp, m, 100, 64, (1.0, 0.5, 2.0), d_out.data_ptr(), sh)
        assert abi.async_check(sh) == 0
        assert same(d_out.cpu().numpy(), ref.warp(img, persp, m, 100, 64, (1.0, 0.5, 2.0))), persp
    for k in (1, 2, 3):
        d_out = torch.zeros((54, 96, 3), dtype=torch.float32, device="cuda")
        bc.deinterlace(bc.EXECUTE, d_img.data_ptr(), 96, 54, 288, k, (1.0, 0.5, 2.0), d_out.data_ptr(), sh)
        assert abi.async_check(sh) == 0
        assert same(d_out.cpu().numpy(), ref.deinterlace(img, k, (1.0, 0.5, 2.0))), k


@pytest.mark.gpu
@pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built")
def test_reference_chains_through_the_binding_equal_the_reference_cpu_backend(fkb_lib):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(302)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    same = lambda a, b: np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream

    # README chain on a 4K frame
    fw, fh = 3840, 2160
    frame = rng.integers(0, 256, (fh, fw, 3), dtype=np.uint8)
    d_frame = dev(frame)
    d_out = torch.zeros((5, 60, 60, 3), dtype=torch.float32, device="cuda")
    bc.readme5(bc.EXECUTE, d_frame.data_ptr(), fw, fh, fw * 3, chains.README_RECTS, (0, 0, 0), 1.4, 0.5, 255.0, d_out.data_ptr(), sh)
    assert abi.async_check(sh) == 0
    assert same(d_out.cpu().numpy(), ref.crop_resize_readme([frame], [0] * 5, chains.README_RECTS, 60, 60, (0, 0, 0), 1.4, 0.5, 255.0))

    # batched crop -> resize -> normalise -> planar, 16 planes over 8 frames
    frames = [rng.integers(0, 256, (540, 960, 3), dtype=np.uint8) for _ in range(8)]
    rects = chains.random_rects(rng, 16, 960, 540, lo=16, hi=512)
    rects[3] = (0, 0, 1, 500)
    fi = [i % 8 for i in range(16)]
    d_frames = [dev(f) for f in frames]
    d_out = torch.zeros((16, 3, 224, 224), dtype=torch.float32, device="cuda")
    bc.norm_planar16(bc.EXECUTE, [d_frames[i].data_ptr() for i in fi], 960, 540, 960 * 3, rects, 224, 224, (0, 0, 0), 255.0,
                     chains.IMAGENET_MEAN, chains.IMAGENET_STD, d_out.data_ptr(), sh)
    assert abi.async_check(sh) == 0
    assert same(d_out.cpu().numpy(), ref.crop_resize_norm_planar(frames, fi, rects, 224, 224, (0, 0, 0), 255.0, chains.IMAGENET_MEAN,
                                                                 chains.IMAGENET_STD))

    # NV12 -> RGB -> resize
    w, h, dw, dh = 1920, 1080, 640, 360
    nv = [rng.integers(0, 256, (h + h // 2, w), dtype=np.uint8) for _ in range(2)]
    d_nv = [dev(f) for f in nv]
    d_out = torch.zeros((2, dh, dw, 3), dtype=torch.float32, device="cuda")
    bc.nv12_2(bc.EXECUTE, [t.data_ptr() for t in d_nv], w, h, w, dw, dh, 255.0, d_out.data_ptr(), sh)
    assert abi.async_check(sh) == 0
    assert same(d_out.cpu().numpy(), ref.nv12_resize(nv, w, h, dw, dh, 255.0))

    # one image, operations handed over one by one; and the uint3 ending of the reference's run-time test
    img = rng.integers(0, 256, (270, 480, 3), dtype=np.uint8)
    d_img = dev(img)
    d_out = torch.zeros((270, 480, 3), dtype=torch.float32, device="cuda")
    bc.cast_mul_sub_div(bc.EXECUTE, d_img.data_ptr(), 480, 270, 1440, 1.4, 0.5, 255.0, d_out.data_ptr(), 5760, sh)
    assert abi.async_check(sh) == 0
    assert same(d_out.cpu().numpy(), ref.cast_mul_sub_div(img, 1.4, 0.5, 255.0))
    zero = torch.zeros((128, 128, 3), dtype=torch.uint8, device="cuda")
    d_u = torch.zeros((32, 32, 3), dtype=torch.int32, device="cuda")
    bc.cast_resize_add_cast_uint3(bc.EXECUTE, zero.data_ptr(), 128, 128, 384, 32, 32, (3.0, 1.0, 32.0), d_u.data_ptr(), 384, sh)
    assert abi.async_check(sh) == 0
    got = d_u.cpu().numpy()
    assert (got[..., 0] == 3).all() and (got[..., 1] == 1).all() and (got[..., 2] == 32).all()
    d_u8 = torch.zeros((270, 480, 3), dtype=torch.uint8, device="cuda")
    bc.bgr_cast_mul_saturate(bc.EXECUTE, d_img.data_ptr(), 480, 270, 1440, 1.4, d_u8.data_ptr(), 1440, sh)
    assert abi.async_check(sh) == 0
    assert np.array_equal(d_u8.cpu().numpy(), ref.bgr_cast_mul_saturate(img, 1.4))

    # NV21 + bt601; PRESERVE_AR_LEFT into a channel-major tensor; a partly filled batch
    d_out = torch.zeros((2, dh, dw, 3), dtype=torch.float32, device="cuda")
    bc.nv21_bt601_2(bc.EXECUTE, [t.data_ptr() for t in d_nv], w, h, w, dw, dh, 255.0, d_out.data_ptr(), sh)
    assert abi.async_check(sh) == 0
    assert same(d_out.cpu().numpy(), ref.nv_resize_ex(nv, w, h, dw, dh, 255.0, 1, 1))
    rects4 = chains.random_rects(rng, 4, 960, 540, lo=16, hi=300)
    d_out = torch.zeros((3, 4, 48, 64), dtype=torch.float32, device="cuda")
    bc.left_tsplit4(bc.EXECUTE, [d_frames[i].data_ptr() for i in range(4)], 960, 540, 2880, rects4, 64, 48, (1.0, 2.0, 3.0), 255.0,
                    chains.IMAGENET_MEAN, chains.IMAGENET_STD, d_out.data_ptr(), sh)
    assert abi.async_check(sh) == 0
    want = ref.crop_resize_norm_planar_mode(frames, [0, 1, 2, 3], rects4, 64, 48, 4, (1.0, 2.0, 3.0), 255.0, chains.IMAGENET_MEAN,
                                            chains.IMAGENET_STD)              # (4, 3, dh, dw)
    assert same(d_out.cpu().numpy(), np.ascontiguousarray(want.transpose(1, 0, 2, 3)))
    imgs = [rng.integers(0, 256, (32, 64, 3), dtype=np.uint8) for _ in range(4)]
    d_imgs = [dev(a) for a in imgs]
    d_out = torch.zeros((4, 32, 64, 3), dtype=torch.float32, device="cuda")
    bc.batch4_default_cast_mul(bc.EXECUTE, [t.data_ptr() for t in d_imgs], 64, 32, 192, 2, (7, 200, 33), (1.5, 0.25, 2.0), d_out.data_ptr(), sh)
    assert abi.async_check(sh) == 0
    assert same(d_out.cpu().numpy(), ref.batch4_default_cast_mul(imgs, 2, (7, 200, 33), (1.5, 0.25, 2.0)))
