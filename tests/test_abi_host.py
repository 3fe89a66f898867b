"""Host-side checks of the C-ABI library that need no GPU: it loads, exports every symbol the
header declares, derives the same host parameters as the checker and the golden table, rejects
malformed plans with a status code, and refuses to run without a device (no fallback)."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op
from tests import cases as tc

ROOT = Path(__file__).resolve().parent.parent
GOLD = Path(__file__).resolve().parent / "golden"


def test_every_declared_symbol_is_exported(fkb_lib):
    header = (ROOT / "include" / "fkb200.h").read_text()
    declared = sorted(set(re.findall(r"FKB_API\s+[\w\s\*]+?\b(fkb_\w+)\s*\(", header)))
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(fkb_lib, name), f"{name} declared in fkb200.h but not exported"
    assert sorted(abi.EXPORTS) == declared
    assert fkb_lib.fkb_version() >= 100


def test_struct_sizes_match_header():
    # sizes implied by the C declarations on LP64
    assert C.sizeof(abi.Op) == 16
    assert C.sizeof(abi.Sequence) == 96
    assert C.sizeof(abi.Plane) == 72
    assert C.sizeof(abi.PlanDesc) == 32
    assert C.sizeof(abi.ResizeParams) == 32
    assert C.sizeof(abi.PlanInfo) == 64


def test_derive_resize_matches_golden_table(fkb_lib):
    g = np.load(GOLD / "resize_params.npz")
    rp = abi.ResizeParams()
    for (sw, sh, dw, dh), res in zip(g["query"], g["result"]):
        for ar, mode in ((0, abi.RESIZE_IGNORE_AR), (1, abi.RESIZE_PRESERVE_AR)):
            assert fkb_lib.fkb_derive_resize(int(sw), int(sh), int(dw), int(dh), mode, C.byref(rp)) == abi.OK
            got = [int(np.float32(rp.fx).view(np.uint32)), int(np.float32(rp.fy).view(np.uint32))]
            assert got == list(res[ar][:2])
            if ar:
                assert [rp.x1, rp.y1, rp.x2, rp.y2] == list(res[ar][2:])


def test_derive_resize_matches_checker_on_many_pairs(fkb_lib, oracle_port):
    rng = np.random.default_rng(123)
    rp = abi.ResizeParams()
    q = rng.integers(1, 4000, (100000, 4))
    for sw, sh, dw, dh in q:
        fkb_lib.fkb_derive_resize(int(sw), int(sh), int(dw), int(dh), abi.RESIZE_PRESERVE_AR, C.byref(rp))
        o = oracle_port.derive_resize(int(sw), int(sh), int(dw), int(dh), abi.RESIZE_PRESERVE_AR)
        assert (rp.fx, rp.fy, rp.x1, rp.y1, rp.x2, rp.y2, rp.target_width, rp.target_height) == \
               (o.fx, o.fy, o.x1, o.y1, o.x2, o.y2, o.target_width, o.target_height)


def test_reference_block_size(fkb_lib, oracle_port):
    """Block shapes the reference picks for the benchmark grids (executors.h:230-242)."""
    want = {(1920, 1080): (32, 8), (224, 224): (32, 8), (1280, 720): (32, 8), (3840, 2160): (32, 8),
            (60, 60): (32, 6), (960, 540): (32, 6)}
    bx, by = C.c_uint32(), C.c_uint32()
    for (w, h), blk in want.items():
        assert fkb_lib.fkb_reference_block_size(w, h, C.byref(bx), C.byref(by)) == abi.OK
        assert (bx.value, by.value) == blk
        assert oracle_port.block_size(w, h) == blk
    rng = np.random.default_rng(7)
    for w, h in rng.integers(1, 5000, (5000, 2)):
        fkb_lib.fkb_reference_block_size(int(w), int(h), C.byref(bx), C.byref(by))
        assert (bx.value, by.value) == oracle_port.block_size(int(w), int(h))


def _plan(**over):
    src = np.zeros((16, 16, 3), np.uint8)
    out = np.zeros((8, 8, 3), np.float32)
    kw = dict(src=src.ctypes.data, src_width=16, src_height=16, src_pitch=48, dst=out.ctypes.data, dst_width=8,
              dst_height=8, dst_pitch=96, crop=(0, 0, 16, 16))
    seq = dict(src_format=abi.SRC_U8X3, dst_format=abi.DST_F32X3_PACKED, resize_mode=abi.RESIZE_IGNORE_AR,
               ops=[op(abi.OP_MUL, 2.0)], n_pre_ops=0)
    for k, v in over.items():
        (seq if k in seq else kw)[k] = v
    plan = abi.HostPlan()
    plan.add_sequence(seq["src_format"], seq["dst_format"], seq["resize_mode"], seq["ops"], n_pre_ops=seq["n_pre_ops"])
    plan.add_plane(**kw)
    plan._keep = (src, out)
    return plan


BAD_PLANS = {
    "null source": dict(src=None),
    "null destination": dict(dst=None),
    "pitch shorter than a row": dict(src_pitch=47),
    "rect outside image": dict(crop=(10, 10, 8, 8)),
    "negative rect origin": dict(crop=(-1, 0, 8, 8)),
    "empty rect": dict(crop=(0, 0, 0, 8)),
    "zero-sized output": dict(dst_width=0),
    "misaligned float output": dict(dst_pitch=98),
    "arithmetic on uchar without cast": dict(resize_mode=abi.RESIZE_NONE, dst_width=16, dst_height=16, dst_pitch=192),
    "float chain into uchar receiver": dict(dst_format=abi.DST_U8X3_PACKED, dst_pitch=24),
    "unknown opcode": dict(ops=[op(99)]),
    "yuv conversion on rgb source": dict(ops=[op(abi.OP_YUV_TO_RGB_BT709_FULL)], n_pre_ops=1),
    "size change without resize": dict(resize_mode=abi.RESIZE_NONE, ops=[op(abi.OP_CAST_F32)]),
}


@pytest.mark.parametrize("why", sorted(BAD_PLANS))
def test_malformed_plans_are_rejected(fkb_lib, why):
    plan = _plan(**BAD_PLANS[why])
    handle = C.c_void_p()
    d = plan.desc()
    rc = fkb_lib.fkb_plan_create(C.byref(d), C.byref(handle))
    assert rc == abi.ERR_INVALID_ARGUMENT, why
    assert not handle.value
    assert fkb_lib.fkb_last_error()


def test_empty_batch_is_rejected(fkb_lib):
    plan = abi.HostPlan()
    plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, abi.RESIZE_NONE, [op(abi.OP_CAST_F32)])
    handle = C.c_void_p()
    d = plan.desc()
    assert fkb_lib.fkb_plan_create(C.byref(d), C.byref(handle)) == abi.ERR_INVALID_ARGUMENT
    assert fkb_lib.fkb_plan_create(None, C.byref(handle)) == abi.ERR_INVALID_ARGUMENT


def test_no_device_means_error_not_fallback(fkb_lib):
    """Without a GPU a valid plan must fail with FKB_ERR_NO_DEVICE; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    plan = _plan()
    handle = C.c_void_p()
    d = plan.desc()
    assert fkb_lib.fkb_plan_create(C.byref(d), C.byref(handle)) == abi.ERR_NO_DEVICE
    assert b"no CPU fallback" in fkb_lib.fkb_last_error()
    with pytest.raises(abi.FkbError):
        abi.execute(plan)
    with pytest.raises(abi.FkbError):
        abi.execute_host(plan)


def test_missing_library_is_an_error(tmp_path):
    with pytest.raises(FileNotFoundError):
        abi.load_library(tmp_path / "libfkb200.so")


def _c3_like_plan(src_format=abi.SRC_U8X3):
    keep = np.zeros((64, 64 * 12), np.uint8)
    out = np.zeros((2, 3, 224, 224), np.float32)
    plan = chains.crop_resize_batch(frame_ptrs=[keep.ctypes.data], frame_index=[0, 0], rects=[(0, 0, 16, 16), (3, 5, 60, 40)],
                                    src_width=64, src_height=64, src_pitch=64 * 3, dst=out.ctypes.data, dst_width=224,
                                    dst_height=224, post_ops=chains.normalize_ops(), planar=True)
    plan._keep = (keep, out)
    return plan


def test_divisions_by_plan_constants_are_lowered_only_when_proven(fkb_lib):
    """Config 3's two divisions (255, then std) qualify for the reciprocal form; the same divisions on a
    float source of unknown range, by a denormal, or after a multiplication by a negative number
    (possible -0) must stay IEEE divisions."""
    info = abi.validate(_c3_like_plan())
    assert (info.n_constant_divisions, info.n_ieee_divisions) == (2, 0)
    assert info.compiled_chain == 1

    src = np.zeros((8, 8, 3), np.float32)
    out = np.zeros((8, 8, 3), np.float32)
    unknown = chains.elementwise([op(abi.OP_DIV, 255.0)], src=src.ctypes.data, dst=out.ctypes.data, width=8, height=8,
                                 src_format=abi.SRC_F32X3)
    info = abi.validate(unknown)
    assert (info.n_constant_divisions, info.n_ieee_divisions) == (0, 1)

    u8 = np.zeros((8, 8, 3), np.uint8)
    for ops, want in (([op(abi.OP_CAST_F32), op(abi.OP_DIV, 255.0)], (1, 0)),
                      ([op(abi.OP_CAST_F32), op(abi.OP_DIV, 1e-39)], (0, 1)),
                      ([op(abi.OP_CAST_F32), op(abi.OP_DIV, 3e7)], (0, 1)),
                      ([op(abi.OP_CAST_F32), op(abi.OP_MUL, -2.0), op(abi.OP_DIV, 255.0)], (0, 1)),
                      ([op(abi.OP_CAST_F32), op(abi.OP_DIV, -255.0), op(abi.OP_DIV, 3.0)], (1, 1)),
                      ([op(abi.OP_CAST_F32), op(abi.OP_SUB, 1.0), op(abi.OP_DIV, (0.229, 0.224, 0.225))], (1, 0))):
        plan = chains.elementwise(ops, src=u8.ctypes.data, dst=out.ctypes.data, width=8, height=8)
        info = abi.validate(plan)
        assert (info.n_constant_divisions, info.n_ieee_divisions) == want, ops


def test_repeated_operations_are_stored_once(fkb_lib):
    """A long continuation that repeats a pair of operations is lowered to a counted loop: the plan's
    device table holds the pair once (plus a header), not every repetition."""
    def table_bytes(ops):
        plan = chains.elementwise(ops, src=1 << 20, dst=1 << 24, width=64, height=8, src_format=abi.SRC_F32X3)
        return abi.validate(plan).device_bytes
    long_chain = table_bytes(chains.addmul_ops(256))
    short_chain = table_bytes(chains.addmul_ops(2))
    assert long_chain - short_chain == 16          # one header slot
    irregular = [op(abi.OP_ADD, 0.001 * (i + 1)) for i in range(256)]   # nothing repeats: every op is stored
    assert table_bytes(irregular) - short_chain == 254 * 16


def test_staged_plans_have_two_table_entries_per_block(fkb_lib):
    """uchar3 resize plans on 16-byte aligned frames run the shared-memory staged body: 32 bytes of
    work-item table per thread block (the second entry starts the block's bulk copies); frames with
    an unaligned pitch fall back to 16."""
    def info(pitch):
        rects = np.array([(0, 0, 100, 80), (20, 10, 60, 90)], np.int32)
        plan = chains.crop_resize_batch(frame_ptrs=[1 << 28], frame_index=[0, 0], rects=rects, src_width=200, src_height=120,
                                        src_pitch=pitch, dst=1 << 30, dst_width=64, dst_height=64,
                                        post_ops=chains.normalize_ops(), planar=True)
        return abi.validate(plan)
    fixed = 2 * 112 + 128 + 5 * 16 + 16             # planes, sequence, operations (two divisions take two slots), status
    staged, direct = info(608), info(600)
    assert staged.device_bytes == fixed + 32 * staged.grid_x
    assert direct.device_bytes == fixed + 16 * direct.grid_x


def test_wide_regions_are_cut_into_column_tiles_for_the_staged_body(fkb_lib):
    """A region of 960 columns is more than the 512 a block of the staged body covers (two columns per
    thread): the plane is lowered to two column tiles, each with a plane descriptor of its own, and the
    plan still reports one plane."""
    plan = abi.HostPlan()
    seq = plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, abi.RESIZE_IGNORE_AR, [abi.op(abi.OP_CAST_F32)], n_pre_ops=1)
    plan.add_plane(src=1 << 28, src_width=1920, src_height=1080, src_pitch=5760, dst=1 << 30, dst_width=960,
                   dst_height=540, dst_pitch=960 * 12, sequence=seq)
    info = abi.validate(plan)
    assert info.n_planes == 1
    fixed = 2 * 112 + 128 + 16 + 16                  # two tiles, sequence, empty operation table, status
    assert info.device_bytes == fixed + 32 * info.grid_x


def test_plans_of_several_classes_stage_their_uchar3_resize_planes(fkb_lib):
    """The four-chain divergent plan: 48 element-wise planes keep their items, the 16 planes of the
    Cast -> Resize group become two staged column tiles each, and every block has two table entries
    (the second one is empty for blocks that copy nothing)."""
    w, h = 1920, 1080
    plan = chains.divergent_four_groups(src_ptrs=[(1 << 28) + i * w * h * 3 for i in range(64)], width=w, height=h,
                                        dst_ptrs=[(1 << 32) + g * (1 << 30) for g in range(4)], per_group=16)
    info = abi.validate(plan)
    assert info.n_planes == 64 and info.n_sequences == 4 and info.n_launches == 1
    fixed = (48 + 2 * 16) * 112 + 4 * 128 + 8 * 16 + 16   # planes, sequences, operations, status
    assert info.device_bytes == fixed + 32 * info.grid_x


def test_empty_regions_of_interest_lower_to_store_only_work(fkb_lib):
    """Crops far off the destination's aspect ratio give PRESERVE_AR a target of zero columns or rows;
    lowering them must neither divide by zero nor use the infinite source step."""
    for case in (c for c in tc.small_cases() if "empty_regions" in c.name):
        arrays = {**case.sources, **case.outputs}
        info = abi.validate(case.build(lambda n: arrays[n].ctypes.data))
        assert info.grid_x >= 1 and info.n_planes >= 2
    rp = abi.ResizeParams()
    assert fkb_lib.fkb_derive_resize(2, 130, 32, 32, abi.RESIZE_PRESERVE_AR, rp) == 0
    assert rp.target_width == 0 and rp.x2 == rp.x1 - 1 and np.isinf(rp.fx)
