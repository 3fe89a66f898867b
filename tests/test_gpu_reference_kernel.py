"""Three-way agreement on the GPU box: this package's kernels (through the C ABI), the reference's
own CUDA kernel (launchTransformDPP_Kernel, executor_details/executor_kernels.h:25-29, compiled for
sm_100a from the reference's headers by oracle/Makefile) and the reference's CPU backend
(oracle/_ref, device branch of interpolation.h:65-67).

Bit for bit against the reference kernel built with -fmad=false (products and sums rounded
separately, as on the host).  The reference's default CUDA build lets nvcc contract a*b+c, so its
own GPU and CPU backends differ in the last bits; that flavour is compared within the stated
tolerance of the path: max-abs 1e-5 on float outputs scaled to [0,1].
"""
import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op
from oracle import reference as ref
from oracle import reference_gpu as refgpu

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (ref.available() and refgpu.available("nofma") and refgpu.available("default")),
                                 reason="oracle/_ref (reference CPU and CUDA builds) not present")]

torch = pytest.importorskip("torch")


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run_plan(plan):
    dplan = abi.DevicePlan(plan)
    dplan.launch()
    assert dplan.check() == 0
    dplan.destroy()


def _same(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    if a.dtype == np.float32:
        a, b = a.view(np.uint32), b.view(np.uint32)
    return np.array_equal(a, b)


def _three_way(ours, gpu_nofma, gpu_default, cpu, scale=1.0):
    """ours == reference CUDA (-fmad=false) == reference CPU bit for bit; the default CUDA build within 1e-5 * scale."""
    assert _same(gpu_nofma, cpu), "reference CUDA kernel (-fmad=false) differs from the reference CPU backend"
    assert _same(ours, cpu), "this package's kernel differs from the reference CPU backend"
    assert _same(ours, gpu_nofma)
    err = np.abs(gpu_default.astype(np.float64) - cpu.astype(np.float64)).max()
    assert err <= 1e-5 * scale, f"reference CUDA kernel (default flags) is {err} away from its CPU backend"


def test_config1_vertical_fusion(fkb_lib):
    rng = np.random.default_rng(101)
    w, h = 1920, 1080
    src = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
    d_src = _dev(src)
    outs = {}
    for name in ("ours", "nofma", "default"):
        d_out = torch.zeros((h, w, 3), dtype=torch.float32, device="cuda")
        if name == "ours":
            _run_plan(chains.elementwise(chains.cast_mul_sub_div_ops(), src=d_src.data_ptr(), dst=d_out.data_ptr(), width=w,
                                         height=h))
        else:
            refgpu.set_stream(0, name)
            refgpu.cast_mul_sub_div(d_src.data_ptr(), w, h, w * 3, 1.4, 0.5, 255.0, d_out.data_ptr(), w * 12, flavour=name)
        torch.cuda.synchronize()
        outs[name] = d_out.cpu().numpy()
    cpu = ref.cast_mul_sub_div(src, 1.4, 0.5, 255.0)
    _three_way(outs["ours"], outs["nofma"], outs["default"], cpu, scale=1.4)


@pytest.mark.parametrize("n_planes", [5, 35])
def test_config2_readme_chain_on_a_4k_frame(fkb_lib, n_planes):
    rng = np.random.default_rng(102)
    fw, fh = 3840, 2160
    frame = rng.integers(0, 256, (fh, fw, 3), dtype=np.uint8)
    rects = np.tile(chains.README_RECTS, (n_planes // 5, 1))
    fi = [0] * n_planes
    d_frame = _dev(frame)
    outs = {}
    for name in ("ours", "nofma", "default"):
        d_out = torch.zeros((n_planes, 60, 60, 3), dtype=torch.float32, device="cuda")
        if name == "ours":
            _run_plan(chains.crop_resize_batch(frame_ptrs=[d_frame.data_ptr()], frame_index=fi, rects=rects, src_width=fw,
                                               src_height=fh, src_pitch=fw * 3, dst=d_out.data_ptr(), dst_width=60,
                                               dst_height=60, post_ops=chains.readme_ops(), planar=False))
        else:
            refgpu.set_stream(0, name)
            refgpu.crop_resize_readme([d_frame.data_ptr()], fi, fw, fh, fw * 3, rects, 60, 60, (0, 0, 0), 1.4, 0.5, 255.0,
                                      d_out.data_ptr(), flavour=name)
        torch.cuda.synchronize()
        outs[name] = d_out.cpu().numpy()
    cpu = ref.crop_resize_readme([frame], fi, rects, 60, 60, (0, 0, 0), 1.4, 0.5, 255.0)
    _three_way(outs["ours"], outs["nofma"], outs["default"], cpu, scale=1.4)


def test_config3_crop_resize_normalise_planar_64_planes(fkb_lib):
    rng = np.random.default_rng(103)
    fw, fh, n, dw, dh = 3840, 2160, 64, 224, 224
    frames = [rng.integers(0, 256, (fh, fw, 3), dtype=np.uint8) for _ in range(2)]
    rects = chains.random_rects(rng, n, fw, fh, lo=16, hi=512)
    rects[0] = (0, 0, 2, 1000)      # a region that rounds to zero columns: background only
    fi = [i % 2 for i in range(n)]
    d_frames = [_dev(f) for f in frames]
    ptrs = [t.data_ptr() for t in d_frames]
    outs = {}
    for name in ("ours", "nofma", "default"):
        d_out = torch.zeros((n, 3, dh, dw), dtype=torch.float32, device="cuda")
        if name == "ours":
            _run_plan(chains.crop_resize_batch(frame_ptrs=ptrs, frame_index=fi, rects=rects, src_width=fw, src_height=fh,
                                               src_pitch=fw * 3, dst=d_out.data_ptr(), dst_width=dw, dst_height=dh,
                                               post_ops=chains.normalize_ops(), planar=True))
        else:
            refgpu.set_stream(0, name)
            refgpu.crop_resize_norm_planar(ptrs, fi, fw, fh, fw * 3, rects, dw, dh, (0, 0, 0), 255.0, chains.IMAGENET_MEAN,
                                           chains.IMAGENET_STD, d_out.data_ptr(), flavour=name)
        torch.cuda.synchronize()
        outs[name] = d_out.cpu().numpy()
    cpu = ref.crop_resize_norm_planar(frames, fi, rects, dw, dh, (0, 0, 0), 255.0, chains.IMAGENET_MEAN, chains.IMAGENET_STD)
    _three_way(outs["ours"], outs["nofma"], outs["default"], cpu, scale=1.0 / 0.224)


@pytest.mark.parametrize("w,h,dw,dh", [(3840, 2160, 1280, 720), (1920, 1080, 800, 450)])
def test_config4_nv12_two_frames(fkb_lib, w, h, dw, dh):
    rng = np.random.default_rng(104)
    frames = [rng.integers(0, 256, (h + h // 2, w), dtype=np.uint8) for _ in range(2)]
    d_frames = [_dev(f) for f in frames]
    ptrs = [t.data_ptr() for t in d_frames]
    outs = {}
    for name in ("ours", "nofma", "default"):
        d_out = torch.zeros((2, dh, dw, 3), dtype=torch.float32, device="cuda")
        if name == "ours":
            _run_plan(chains.nv12_resize_batch(frame_ptrs=ptrs, width=w, height=h, pitch=w, dst=d_out.data_ptr(),
                                               dst_width=dw, dst_height=dh))
        else:
            refgpu.set_stream(0, name)
            refgpu.nv12_resize(ptrs, w, h, w, dw, dh, 255.0, d_out.data_ptr(), flavour=name)
        torch.cuda.synchronize()
        outs[name] = d_out.cpu().numpy()
    cpu = ref.nv12_resize(frames, w, h, dw, dh, 255.0)
    _three_way(outs["ours"], outs["nofma"], outs["default"], cpu, scale=2.0)


def test_config5_long_chain_and_divergent_groups(fkb_lib):
    rng = np.random.default_rng(105)
    # part A: 16 alternating Add / Mul on a float3 image
    w, h = 640, 360
    src = rng.random((h, w, 3), dtype=np.float32)
    d_src = _dev(src)
    outs = {}
    for name in ("ours", "nofma", "default"):
        d_out = torch.zeros((h, w, 3), dtype=torch.float32, device="cuda")
        if name == "ours":
            _run_plan(chains.elementwise(chains.addmul_ops(16), src=d_src.data_ptr(), dst=d_out.data_ptr(), width=w, height=h,
                                         src_format=abi.SRC_F32X3))
        else:
            refgpu.set_stream(0, name)
            assert refgpu.addmul_chain(d_src.data_ptr(), w, h, w * 12, 16, 0.001, 1.0001, d_out.data_ptr(), w * 12, flavour=name)
        torch.cuda.synchronize()
        outs[name] = d_out.cpu().numpy()
    _three_way(outs["ours"], outs["nofma"], outs["default"], ref.addmul_chain(src, 16, 0.001, 1.0001), scale=2.0)

    # part B: the four chains, 16 images each; ours in ONE launch, the reference in four (it has no host
    # launcher for launchDivergentBatchTransformDPP_Kernel, executors.h:129-145)
    w, h, pg = 480, 270, 16
    imgs = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for _ in range(4 * pg)]
    d_imgs = [_dev(a) for a in imgs]
    p = [t.data_ptr() for t in d_imgs]

    def outputs():
        return [torch.zeros((pg, h, w, 3), dtype=torch.float32, device="cuda"),
                torch.zeros((pg, h, w, 3), dtype=torch.float32, device="cuda"),
                torch.zeros((pg, h, w, 3), dtype=torch.uint8, device="cuda"),
                torch.zeros((pg, h // 2, w // 2, 3), dtype=torch.float32, device="cuda")]

    got = {}
    for name in ("ours", "nofma"):
        o = outputs()
        if name == "ours":
            plan = chains.divergent_four_groups(src_ptrs=p, width=w, height=h, dst_ptrs=[t.data_ptr() for t in o],
                                                resize_to=(w // 2, h // 2), per_group=pg)
            assert abi.validate(plan).n_launches == 1
            _run_plan(plan)
        else:
            refgpu.set_stream(0, name)
            refgpu.cast_mul_sub_batch16(p[0:16], w, h, w * 3, 1.4, 0.5, o[0].data_ptr(), flavour=name)
            refgpu.cast_add_div_batch16(p[16:32], w, h, w * 3, 0.5, 255.0, o[1].data_ptr(), flavour=name)
            refgpu.bgr_cast_mul_saturate_batch16(p[32:48], w, h, w * 3, 1.4, o[2].data_ptr(), flavour=name)
            refgpu.cast_resize_batch16(p[48:64], w, h, w * 3, w // 2, h // 2, o[3].data_ptr(), flavour=name)
        torch.cuda.synchronize()
        got[name] = [t.cpu().numpy() for t in o]
    cpu = [np.stack([ref.cast_mul_sub(a, 1.4, 0.5) for a in imgs[0:16]]),
           np.stack([ref.cast_add_div(a, 0.5, 255.0) for a in imgs[16:32]]),
           np.stack([ref.bgr_cast_mul_saturate(a, 1.4) for a in imgs[32:48]]),
           np.stack([ref.cast_resize(a, w // 2, h // 2) for a in imgs[48:64]])]
    for g in range(4):
        assert _same(got["nofma"][g], cpu[g]), f"group {g}: reference CUDA vs reference CPU"
        assert _same(got["ours"][g], cpu[g]), f"group {g}: this package vs reference CPU"
    # the same four chains as ONE launch of the reference's divergent kernel (it ships without a host launcher)
    o = outputs()
    refgpu.divergent_four_groups64(p, w, h, w * 3, 1.4, 0.5, 0.5, 255.0, w // 2, h // 2, *[t.data_ptr() for t in o], flavour="nofma")
    torch.cuda.synchronize()
    for g in range(4):
        assert _same(o[g].cpu().numpy(), cpu[g]), f"group {g}: the reference's divergent kernel vs reference CPU"
