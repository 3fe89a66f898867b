"""CUDA path vs the checker, through the C ABI, on the same seeded inputs.

Bit-exact for every output (integer, index and float work alike): the kernels round every
operation separately, as the reference's per-thread function does.  The stated tolerance of
the path (max-abs 1e-5 on float outputs scaled to [0,1]) is therefore met with margin 0.
"""
import ctypes as C

import numpy as np
import pytest

from fusedkernellibrary_b200 import abi
from tests import cases as tc

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


class DeviceArrays:
    """Device copies of a case's host arrays, as torch byte tensors (memory plumbing only)."""

    def __init__(self, case, fill=0):
        self.t = {}
        for name, a in case.sources.items():
            self.t[name] = torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda()
        for name, a in case.outputs.items():
            self.t[name] = torch.full((a.nbytes,), fill, dtype=torch.uint8, device="cuda")

    def ptr(self, name):
        return self.t[name].data_ptr()

    def download(self, name, like):
        return self.t[name].cpu().numpy().view(like.dtype).reshape(like.shape)


def run_cuda(case, fkb_lib, fill=0):
    dev = DeviceArrays(case, fill)
    plan = case.build(dev.ptr)
    dplan = abi.DevicePlan(plan)
    dplan.launch()
    torch.cuda.synchronize()
    info = dplan.info()
    out = {k: dev.download(k, v) for k, v in case.outputs.items()}
    dplan.destroy()
    return out, info


@pytest.mark.parametrize("case", tc.small_cases(), ids=lambda c: c.name)
def test_small_case_bit_exact(case, fkb_lib, oracle_port):
    expected = {k: v.copy() for k, v in tc.run_on_host(case, oracle_port).items()}
    got, info = run_cuda(case, fkb_lib)
    assert info.n_launches == 1
    for k in expected:
        e, g = tc.bits(expected[k]), tc.bits(got[k])
        bad = np.flatnonzero(e.reshape(-1) != g.reshape(-1))
        assert bad.size == 0, f"{case.name}/{k}: {bad.size} differing words, first at {bad[:5]}"


def test_padding_is_left_alone(fkb_lib, oracle_port):
    """Bytes between the end of a row and the pitch must not be written."""
    case = tc.elementwise_case("pad", 99, 100, 21, tc.chains.cast_mul_sub_div_ops(), src_pitch=304, dst_pitch=1216)
    got, _ = run_cuda(case, fkb_lib, fill=0xAB)
    out = got["out"]
    assert (out[:, 1200:] == 0xAB).all()


def test_resize_params_match_checker(fkb_lib, oracle_port):
    case = tc.crop_resize_case("params", 77, 2, 640, 360, 64, 224, 224, True, tc.chains.normalize_ops(), lo=8, hi=300)
    dev = DeviceArrays(case)
    dplan = abi.DevicePlan(case.build(dev.ptr))
    for i, r in enumerate(case.meta["rects"]):
        a = dplan.resize_params(i)
        b = oracle_port.derive_resize(int(r[2]), int(r[3]), 224, 224, abi.RESIZE_PRESERVE_AR)
        assert (np.float32(a.fx).view(np.uint32), np.float32(a.fy).view(np.uint32), a.x1, a.y1, a.x2, a.y2) == \
               (np.float32(b.fx).view(np.uint32), np.float32(b.fy).view(np.uint32), b.x1, b.y1, b.x2, b.y2)
    dplan.destroy()


def test_execute_one_shot_and_host_session(fkb_lib, oracle_port):
    case = tc.crop_resize_case("host", 78, 2, 320, 200, 11, 64, 48, True, tc.chains.normalize_ops())
    expected = {k: v.copy() for k, v in tc.run_on_host(case, oracle_port).items()}
    # one-shot on device pointers
    dev = DeviceArrays(case)
    abi.execute(case.build(dev.ptr))
    assert np.array_equal(tc.bits(dev.download("out", case.outputs["out"])), tc.bits(expected["out"]))
    # host-buffer session: same plan description, host pointers
    arrays = {**case.sources, **case.outputs}
    case.outputs["out"][...] = 0
    sess = abi.HostSession(case.build(lambda n: arrays[n].ctypes.data))
    sess.run()
    h2d, d2h = sess.traffic()
    assert h2d == sum(a.nbytes for a in case.sources.values())
    assert d2h == case.outputs["out"].nbytes
    assert np.array_equal(tc.bits(case.outputs["out"]), tc.bits(expected["out"]))
    case.outputs["out"][...] = 0
    sess.run()
    assert np.array_equal(tc.bits(case.outputs["out"]), tc.bits(expected["out"]))
    sess.destroy()


def test_host_session_groups_and_copy_patterns(fkb_lib, oracle_port):
    """Planes dealt to three source images in runs of uneven length, and outputs with padded rows:
    the session's per-image groups must bring every byte back (runs, strided and row-exact copies)."""
    rng = np.random.default_rng(79)
    fw, fh, n, dw, dh = 160, 96, 23, 32, 24
    frames = [rng.integers(0, 256, (fh, fw * 3), dtype=np.uint8) for _ in range(3)]
    rects = tc.chains.random_rects(rng, n, fw, fh, lo=4, hi=90)
    fi = [(i // 4) % 3 if i < 20 else 2 - (i % 3) for i in range(n)]
    for planar, pad in ((True, 0), (False, 0), (False, 16)):
        pitch = dw * (4 if planar else 12) + pad
        out = np.zeros((n, 3 * dh, pitch) if planar else (n, dh, pitch), np.uint8)
        want = np.zeros_like(out)

        def plan_for(ptrs, dst):
            plan = abi.HostPlan()
            seq = plan.add_sequence(abi.SRC_U8X3, abi.DST_F32_PLANAR3 if planar else abi.DST_F32X3_PACKED, abi.RESIZE_PRESERVE_AR,
                                    tc.chains.normalize_ops())
            for i in range(n):
                plan.add_plane(src=ptrs[fi[i]], src_width=fw, src_height=fh, src_pitch=fw * 3, crop=tuple(int(v) for v in rects[i]),
                               dst=dst + i * out[0].nbytes, dst_width=dw, dst_height=dh, dst_pitch=pitch,
                               dst_channel_stride=dh * pitch if planar else 0, sequence=seq)
            return plan

        oracle_port.run(plan_for([f.ctypes.data for f in frames], want.ctypes.data))
        sess = abi.HostSession(plan_for([f.ctypes.data for f in frames], out.ctypes.data))
        sess.run()
        h2d, d2h = sess.traffic()
        assert h2d == sum(f.nbytes for f in frames)
        assert d2h == n * 3 * dh * dw * 4
        sess.destroy()
        assert np.array_equal(out, want), f"planar={planar} pad={pad}"
