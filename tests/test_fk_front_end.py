"""The reference's operation vocabulary (include/fkb200_fk.hpp) over the C ABI.

tests/cpp/fk_shim_chains.cpp spells the chains the way the reference's own example does
(tests/examples/readme_test_code.h of the reference): build(...).then(...), executeOperations, stream.sync().
Without a GPU the program's host-only mode checks the error behaviour (std::runtime_error where the reference
fails to compile or throws, and no fallback without a device); on a GPU its outputs are compared bit for bit
with the checker running the same chains.
"""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op
from tests import cases as tc

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "cpp" / "fk_shim_chains.cpp"
CUDA = Path("/usr/local/cuda")


@pytest.fixture(scope="module")
def shim_program(fkb_lib, tmp_path_factory):
    if not (CUDA / "include" / "cuda_runtime.h").exists():
        pytest.skip("CUDA toolkit headers not found")
    exe = tmp_path_factory.mktemp("fk_shim") / "fk_shim_chains"
    libdir = ROOT / "fusedkernellibrary_b200" / "lib"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", f"-I{ROOT / 'include'}", f"-I{CUDA / 'include'}", str(SRC), "-o", str(exe),
           f"-L{libdir}", "-lfkb200", f"-L{CUDA / 'lib64'}", "-lcudart", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{CUDA / 'lib64'}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_front_end_error_behaviour(shim_program):
    r = subprocess.run([str(shim_program), "--host-only"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok arithmetic on uchar3" in r.stdout and "ok receiver type" in r.stdout and "ok border above crop" in r.stdout


@pytest.mark.gpu
def test_front_end_chains_match_the_checker(shim_program, oracle_port, tmp_path):
    rng = np.random.default_rng(2024)
    f0, f1 = (rng.integers(0, 256, (216, 384 * 3), dtype=np.uint8) for _ in range(2))
    nv = [rng.integers(0, 256, (54 + 27, 96), dtype=np.uint8) for _ in range(2)]
    f0.tofile(tmp_path / "frame0.bin"); f1.tofile(tmp_path / "frame1.bin")
    nv[0].tofile(tmp_path / "nv12_0.bin"); nv[1].tofile(tmp_path / "nv12_1.bin")
    r = subprocess.run([str(shim_program), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr

    def got(name, dtype, shape):
        return np.fromfile(tmp_path / name, dtype=dtype).reshape(shape)

    # README chain
    want = np.zeros((5, 60, 60, 3), np.float32)
    oracle_port.run(chains.crop_resize_batch(frame_ptrs=[f0.ctypes.data], frame_index=[0] * 5, rects=chains.README_RECTS, src_width=384,
                                             src_height=216, src_pitch=1152, dst=want.ctypes.data, dst_width=60, dst_height=60,
                                             post_ops=chains.readme_ops(), planar=False))
    assert np.array_equal(tc.bits(got("out_readme.bin", np.float32, want.shape)), tc.bits(want))
    # batched crop -> resize -> normalise -> planar over two frames
    rects = np.array([(5, 7, 200, 100), (100, 50, 64, 160), (0, 0, 384, 216), (383, 215, 1, 1)], np.int32)
    want = np.zeros((4, 3, 48, 64), np.float32)
    oracle_port.run(chains.crop_resize_batch(frame_ptrs=[f0.ctypes.data, f1.ctypes.data], frame_index=[0, 1, 0, 1], rects=rects,
                                             src_width=384, src_height=216, src_pitch=1152, dst=want.ctypes.data, dst_width=64,
                                             dst_height=48, post_ops=chains.normalize_ops(), planar=True))
    assert np.array_equal(tc.bits(got("out_planar.bin", np.float32, want.shape)), tc.bits(want))
    # NV12 -> RGB -> resize -> /255
    want = np.zeros((2, 22, 40, 3), np.float32)
    oracle_port.run(chains.nv12_resize_batch(frame_ptrs=[a.ctypes.data for a in nv], width=96, height=54, pitch=96,
                                             dst=want.ctypes.data, dst_width=40, dst_height=22))
    assert np.array_equal(tc.bits(got("out_nv12.bin", np.float32, want.shape)), tc.bits(want))
    # two chains in one launch
    w0 = np.zeros((216, 384, 3), np.float32)
    oracle_port.run(chains.elementwise([op(abi.OP_CAST_F32), op(abi.OP_MUL, 1.4), op(abi.OP_SUB, 0.5)], src=f0.ctypes.data,
                                       dst=w0.ctypes.data, width=384, height=216))
    w1 = np.zeros((216, 384, 3), np.uint8)
    oracle_port.run(chains.elementwise([op(abi.OP_SWAP_RB), op(abi.OP_CAST_F32), op(abi.OP_MUL, 1.4), op(abi.OP_SATURATE_CAST_U8)],
                                       src=f1.ctypes.data, dst=w1.ctypes.data, width=384, height=216, dst_format=abi.DST_U8X3_PACKED))
    assert np.array_equal(tc.bits(got("out_div0.bin", np.float32, w0.shape)), tc.bits(w0))
    assert np.array_equal(got("out_div1.bin", np.uint8, w1.shape), w1)
    # widened vocabulary: padded crop under REFLECT_101 + PRESERVE_AR_LEFT, perspective warp, INTER_LINEAR deinterlace, NV21 + bt601
    def one(out, dst_w, dst_h, mode, ops, crop=None, **extras):
        plan = abi.HostPlan()
        seq = plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, mode, ops, **extras)
        plan.add_plane(src=f0.ctypes.data, src_width=384, src_height=216, src_pitch=1152, crop=crop, dst=out.ctypes.data, dst_width=dst_w,
                       dst_height=dst_h, dst_pitch=dst_w * 12, sequence=seq)
        oracle_port.run(plan)
        return out

    mul = [op(abi.OP_MUL, (1.0, 0.5, 2.0))]
    want = one(np.zeros((45, 70, 3), np.float32), 70, 45, abi.RESIZE_PRESERVE_AR_LEFT, [], crop=(-20, -11, 430, 240), border_mode=abi.BORDER_REFLECT_101,
               background=(1.0, 2.0, 3.0))
    assert np.array_equal(tc.bits(got("out_border.bin", np.float32, want.shape)), tc.bits(want))
    want = one(np.zeros((64, 100, 3), np.float32), 100, 64, abi.GEOMETRY_WARP_PERSPECTIVE, mul,
               transform=(0.9, 0.1, -2.0, 0.05, 0.8, 1.0, 0.002, 0.001, 1.0))
    assert np.array_equal(tc.bits(got("out_warp.bin", np.float32, want.shape)), tc.bits(want))
    want = one(np.zeros((216, 384, 3), np.float32), 384, 216, abi.RESIZE_NONE, mul, deinterlace=abi.DEINTERLACE_LINEAR_ODD)
    assert np.array_equal(tc.bits(got("out_deint.bin", np.float32, want.shape)), tc.bits(want))
    want = np.zeros((2, 22, 40, 3), np.float32)
    oracle_port.run(chains.nv12_resize_batch(frame_ptrs=[a.ctypes.data for a in nv], width=96, height=54, pitch=96, dst=want.ctypes.data,
                                             dst_width=40, dst_height=22, src_format=abi.SRC_NV21, conversion=abi.OP_YUV_TO_RGB_BT601_FULL))
    assert np.array_equal(tc.bits(got("out_nv21.bin", np.float32, want.shape)), tc.bits(want))
    # the circular tensor after four updates, newest first: planes = crops 3, 2, 1 of the planar batch above
    window = got("out_window.bin", np.float32, (3, 3, 48, 64))
    planar = got("out_planar.bin", np.float32, (4, 3, 48, 64))
    for z, k in enumerate((3, 2, 1)):
        assert np.array_equal(tc.bits(window[z]), tc.bits(planar[k])), (z, k)
