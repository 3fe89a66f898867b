"""The configurations at their full sizes on the GPU, through the C ABI.

The CPU checkers are too slow to redo a whole configuration in a test, so each case compares a seeded
sample of planes (or rows) bit for bit - with the plain-C checker and, where oracle/_ref is present,
with the reference's own CPU backend directly - compares EVERY plane with the reference's own CUDA
kernel (built with -fmad=false; itself compared with the reference's CPU backend in
test_gpu_reference_kernel.py), and checks the rest through properties that do not depend on the size:
every output element outside a plane's region of interest holds the one value the default takes
after the continuation, linearity of the element-wise chains in their input, and a
second launch that reproduces the first exactly.
"""
import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from oracle import reference as ref
from oracle import reference_gpu as refgpu
from tests import cases as tc

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _bits(t):
    return t.view(torch.int32)


def test_c3_full_size_sampled_planes_and_background(fkb_lib, oracle_port):
    rng = np.random.default_rng(1003)
    fw, fh, n, dw, dh, nf = 3840, 2160, 1024, 224, 224, 8
    frames = [rng.integers(0, 256, (fh, fw * 3), dtype=np.uint8) for _ in range(nf)]
    rects = chains.random_rects(rng, n, fw, fh, lo=16, hi=512)
    fi = [i % nf for i in range(n)]
    d_frames = [torch.from_numpy(f).cuda() for f in frames]
    d_out = torch.full((n, 3, dh, dw), float("nan"), dtype=torch.float32, device="cuda")

    def plan_for(ptrs, dst, sel):
        return chains.crop_resize_batch(frame_ptrs=ptrs, frame_index=[fi[i] for i in sel], rects=rects[sel], src_width=fw,
                                        src_height=fh, src_pitch=fw * 3, dst=dst, dst_width=dw, dst_height=dh,
                                        post_ops=chains.normalize_ops(), planar=True)

    every = list(range(n))
    plan = abi.DevicePlan(plan_for([t.data_ptr() for t in d_frames], d_out.data_ptr(), every))
    info = plan.info()
    assert info.n_launches == 1 and info.n_planes == n
    plan.launch()
    assert plan.check() == 0
    first = d_out.clone()
    d_out.fill_(float("nan"))
    plan.launch()
    assert plan.check() == 0
    assert torch.equal(_bits(first), _bits(d_out)), "a second launch of the same plan differs"

    # sampled planes, bit for bit (smallest, largest, widest, tallest crops plus a random draw)
    area = rects[:, 2].astype(np.int64) * rects[:, 3]
    sel = sorted(set([int(area.argmin()), int(area.argmax()), int(rects[:, 2].argmax()), int(rects[:, 3].argmax())] +
                     [int(i) for i in rng.choice(n, 60, replace=False)]))
    want = np.zeros((len(sel), 3, dh, dw), np.float32)
    oracle_port.run(plan_for([f.ctypes.data for f in frames], want.ctypes.data, sel))
    got = d_out[torch.tensor(sel, device="cuda")].cpu().numpy()
    bad = np.flatnonzero(tc.bits(got).reshape(-1) != tc.bits(want).reshape(-1))
    assert bad.size == 0, f"{bad.size} differing words in the sampled planes, first at {bad[:5]}"
    if ref.available():   # the same planes through the reference's own CPU backend
        frames3 = [f.reshape(fh, fw, 3) for f in frames]
        want_ref = ref.crop_resize_norm_planar(frames3, [fi[i] for i in sel], rects[sel], dw, dh, (0, 0, 0), 255.0,
                                               chains.IMAGENET_MEAN, chains.IMAGENET_STD)
        assert np.array_equal(tc.bits(got), tc.bits(want_ref)), "sampled planes differ from the reference CPU backend"
    if refgpu.available("nofma"):   # every plane through the reference's own CUDA kernel
        d_ref = torch.full((n, 3, dh, dw), float("nan"), dtype=torch.float32, device="cuda")
        refgpu.set_stream(0, "nofma")
        refgpu.crop_resize_norm_planar([t.data_ptr() for t in d_frames], fi, fw, fh, fw * 3, rects, dw, dh, (0, 0, 0), 255.0,
                                       chains.IMAGENET_MEAN, chains.IMAGENET_STD, d_ref.data_ptr(), flavour="nofma")
        torch.cuda.synchronize()
        assert torch.equal(_bits(d_ref), _bits(d_out)), "a plane differs from the reference's CUDA kernel"

    # every plane: outside its region of interest, the default value after Div, Sub, Div
    host = d_out.cpu().numpy()
    assert np.isfinite(host).all(), "an output element was never written"
    bg = ((np.float32(0) / np.float32(255) - np.array(chains.IMAGENET_MEAN, np.float32)) /
          np.array(chains.IMAGENET_STD, np.float32)).astype(np.float32)
    for i in range(n):
        rp = plan.resize_params(i)
        mask = np.ones((dh, dw), bool)
        mask[rp.y1:rp.y2 + 1, rp.x1:rp.x2 + 1] = False
        for c in range(3):
            assert (host[i, c][mask] == bg[c]).all(), f"plane {i} channel {c}: background differs"
    plan.destroy()


def test_c4_full_size_two_frames(fkb_lib, oracle_port):
    case = tc.nv12_case("c4_full", 1004, 2, 3840, 2160, 1280, 720)
    expected = {k: v.copy() for k, v in tc.run_on_host(case, oracle_port).items()}
    from tests.test_gpu_parity import run_cuda
    got, info = run_cuda(case, fkb_lib)
    assert info.n_launches == 1
    assert np.array_equal(tc.bits(got["out"]), tc.bits(expected["out"]))
    if ref.available():
        want_ref = ref.nv12_resize([case.sources["frame0"], case.sources["frame1"]], 3840, 2160, 1280, 720, 255.0)
        assert np.array_equal(tc.bits(got["out"]), tc.bits(want_ref)), "differs from the reference CPU backend"


@pytest.mark.skipif(not refgpu.available("nofma"), reason="reference CUDA build not present")
def test_c4_full_size_all_32_frames_against_the_reference_kernel(fkb_lib):
    rng = np.random.default_rng(1007)
    n, w, h, dw, dh = 32, 3840, 2160, 1280, 720
    d_frames = [torch.from_numpy(rng.integers(0, 256, (h + h // 2, w), dtype=np.uint8)).cuda() for _ in range(n)]
    ptrs = [t.data_ptr() for t in d_frames]
    d_out = torch.full((n, dh, dw, 3), float("nan"), dtype=torch.float32, device="cuda")
    d_ref = torch.full((n, dh, dw, 3), float("nan"), dtype=torch.float32, device="cuda")
    plan = abi.DevicePlan(chains.nv12_resize_batch(frame_ptrs=ptrs, width=w, height=h, pitch=w, dst=d_out.data_ptr(), dst_width=dw,
                                                   dst_height=dh))
    plan.launch()
    assert plan.check() == 0
    plan.destroy()
    refgpu.set_stream(0, "nofma")
    refgpu.nv12_resize(ptrs, w, h, w, dw, dh, 255.0, d_ref.data_ptr(), flavour="nofma")
    torch.cuda.synchronize()
    assert torch.equal(_bits(d_ref), _bits(d_out))


def test_c1_and_c5a_full_size(fkb_lib, oracle_port):
    from tests.test_gpu_parity import run_cuda
    c1 = tc.elementwise_case("c1_full", 1001, 1920, 1080, chains.cast_mul_sub_div_ops())
    c5a = tc.elementwise_case("c5a_full", 1005, 3840, 2160, chains.addmul_ops(64), src_fmt=abi.SRC_F32X3)
    # a long chain on an image whose last work item is ragged: the blocks prefetch later work items, the last one in part
    ragged = tc.elementwise_case("c5a_ragged", 1007, 3001, 1999, chains.addmul_ops(16), src_fmt=abi.SRC_F32X3)
    for case in (c1, c5a, ragged):
        expected = {k: v.copy() for k, v in tc.run_on_host(case, oracle_port).items()}
        got, _ = run_cuda(case, fkb_lib)
        assert np.array_equal(tc.bits(got["out"]), tc.bits(expected["out"])), case.name


def test_c5b_full_resolution_two_images_per_group(fkb_lib, oracle_port):
    from tests.test_gpu_parity import run_cuda
    case = tc.divergent_case("c5b_full", 1006, 1920, 1080, 960, 540, 2)
    expected = {k: v.copy() for k, v in tc.run_on_host(case, oracle_port).items()}
    got, info = run_cuda(case, fkb_lib)
    assert info.n_launches == 1 and info.n_sequences == 4
    for k in expected:
        assert np.array_equal(tc.bits(got[k]), tc.bits(expected[k])), k
    if ref.available():   # one image of each group through the reference's own CPU backend
        img = lambda g: case.sources[f"img{g * 2}"].reshape(1080, 1920, 3)
        assert np.array_equal(tc.bits(got["g0"][0]), tc.bits(ref.cast_mul_sub(img(0), 1.4, 0.5)))
        assert np.array_equal(tc.bits(got["g1"][0]), tc.bits(ref.cast_add_div(img(1), 0.5, 255.0)))
        assert np.array_equal(got["g2"][0], ref.bgr_cast_mul_saturate(img(2), 1.4))
        assert np.array_equal(tc.bits(got["g3"][0]), tc.bits(ref.cast_resize(img(3), 960, 540)))


def test_c2_scaled_readme_rects_over_many_planes(fkb_lib, oracle_port):
    """The README rects cycled over 1000 planes and 8 frames: every plane must equal the plane of the
    same rect and frame computed alone (horizontal fusion changes nothing per plane)."""
    rng = np.random.default_rng(1002)
    fw, fh, nf, n = 3840, 2160, 8, 1000
    frames = [rng.integers(0, 256, (fh, fw * 3), dtype=np.uint8) for _ in range(nf)]
    rects = np.tile(chains.README_RECTS, (n // 5, 1))
    fi = [(i // 5) % nf for i in range(n)]
    d_frames = [torch.from_numpy(f).cuda() for f in frames]
    d_out = torch.zeros((n, 60, 60, 3), dtype=torch.float32, device="cuda")
    plan = abi.DevicePlan(chains.crop_resize_batch(frame_ptrs=[t.data_ptr() for t in d_frames], frame_index=fi, rects=rects,
                                                   src_width=fw, src_height=fh, src_pitch=fw * 3, dst=d_out.data_ptr(),
                                                   dst_width=60, dst_height=60, post_ops=chains.readme_ops(), planar=False))
    plan.launch()
    assert plan.check() == 0
    got = d_out.cpu().numpy()
    plan.destroy()
    want = np.zeros((40, 60, 60, 3), np.float32)   # the first 40 planes cover all 8 frames x 5 rects
    oracle_port.run(chains.crop_resize_batch(frame_ptrs=[f.ctypes.data for f in frames], frame_index=fi[:40], rects=rects[:40],
                                             src_width=fw, src_height=fh, src_pitch=fw * 3, dst=want.ctypes.data, dst_width=60,
                                             dst_height=60, post_ops=chains.readme_ops(), planar=False))
    assert np.array_equal(tc.bits(got[:40]), tc.bits(want))
    if ref.available():
        want_ref = ref.crop_resize_readme([f.reshape(fh, fw, 3) for f in frames], fi[:40], rects[:40], 60, 60, (0, 0, 0), 1.4, 0.5, 255.0)
        assert np.array_equal(tc.bits(got[:40]), tc.bits(want_ref)), "differs from the reference CPU backend"
    for i in range(40, n):
        assert np.array_equal(tc.bits(got[i]), tc.bits(got[i % 40])), f"plane {i} differs from its twin {i % 40}"


def test_one_shot_call_launches_right_after_its_table_is_uploaded(fkb_lib):
    """fkb_execute makes a plan, launches it on the caller's stream at once and destroys it: the kernel must find the
    whole descriptor table (over a megabyte here: 8000 planes, with their tensor maps at its end) on the device even
    though the caller's stream does not wait for the stream the upload used."""
    rng = np.random.default_rng(1011)
    fw, fh, nf, n = 3840, 2160, 8, 8000
    d_frames = [torch.from_numpy(rng.integers(0, 256, (fh, fw * 3), dtype=np.uint8)).cuda() for _ in range(nf)]
    rects = np.tile(chains.README_RECTS, (n // 5, 1))
    fi = [(i // 5) % nf for i in range(n)]
    d_out = torch.zeros((n, 60, 60, 3), dtype=torch.float32, device="cuda")
    desc = chains.crop_resize_batch(frame_ptrs=[t.data_ptr() for t in d_frames], frame_index=fi, rects=rects, src_width=fw,
                                    src_height=fh, src_pitch=fw * 3, dst=d_out.data_ptr(), dst_width=60, dst_height=60,
                                    post_ops=chains.readme_ops(), planar=False)
    plan = abi.DevicePlan(desc)
    torch.cuda.synchronize()
    plan.launch()
    assert plan.check() == 0
    want = d_out.clone()
    plan.destroy()
    stream = torch.cuda.Stream()   # non-blocking: not ordered behind the default stream
    for _ in range(3):
        d_out.zero_()
        torch.cuda.synchronize()
        abi.execute(desc, stream.cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(_bits(d_out), _bits(want))
