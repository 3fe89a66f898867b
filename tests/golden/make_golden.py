"""Generates the golden vectors under tests/golden/ from the reference's own headers.

Run where the reference tree is present, after `make -C oracle ref`:

    python tests/golden/make_golden.py

Every fixture stores the seeded inputs and the output of oracle/_ref/libfklref_device_branch.so
(the reference's unmodified source with its device branch selected on the host, see
oracle/ref/device_branch_prelude.h).  For chains that contain Resize the output of the literal
CPU build is stored next to it under `literal_*`, to document where the two differ (that build reads rows
outside the image, interpolation.h:70, so its values vary from run to run and no test compares them).
The fixtures are what travels: tests never read the reference tree.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from fusedkernellibrary_b200 import chains  # noqa: E402
from oracle import reference as ref  # noqa: E402

OUT = Path(__file__).resolve().parent

# a crop that reaches beyond a 40x24 image on every side; an affine and a perspective matrix (rows of three)
READBACK_RECT = (-7, -5, 60, 37)
READBACK_AFFINE = (0.8, 0.25, -3.0, -0.2, 0.7, 2.5, 0.0, 0.0, 1.0)
READBACK_PERSPECTIVE = (0.9, 0.1, -2.0, 0.05, 0.8, 1.0, 0.002, 0.001, 1.0)


def u8(rng, *shape):
    return rng.integers(0, 256, shape, dtype=np.uint8)


def main():
    rng = np.random.default_rng(20240607)

    # --- element-wise chains on a 53x37 uchar3 image (configs 1, 5B groups 1-3) -----------
    img = u8(rng, 37, 53, 3)
    np.savez_compressed(
        OUT / "elementwise_u8.npz", src=img,
        cast_mul_sub_div=ref.cast_mul_sub_div(img, 1.4, 0.5, 255.0),
        cast_mul_sub=ref.cast_mul_sub(img, 1.4, 0.5),
        cast_add_div=ref.cast_add_div(img, 0.5, 255.0),
        bgr_cast_mul_saturate=ref.bgr_cast_mul_saturate(img, 1.4),
        cast_resize_30x20=ref.cast_resize(img, 30, 20),
        literal_cast_resize_30x20=ref.cast_resize(img, 30, 20, flavour="literal"),
    )

    # --- long Add/Mul chains on a 31x20 float3 image (config 5A) ---------------------------
    imgf = rng.random((20, 31, 3), dtype=np.float32)
    np.savez_compressed(OUT / "addmul_chain.npz", src=imgf,
                        **{f"n{n}": ref.addmul_chain(imgf, n, 0.001, 1.0001) for n in (1, 2, 3, 16, 64, 256)})

    # --- README chain (config 2) on a 384x216 frame -----------------------------------------
    frame = u8(rng, 216, 384, 3)
    rects = chains.README_RECTS
    np.savez_compressed(
        OUT / "readme_crop_resize.npz", frame=frame, rects=rects,
        out=ref.crop_resize_readme([frame], [0] * 5, rects, 60, 60, (0, 0, 0), 1.4, 0.5, 255.0),
        out_ignore_ar=ref.crop_resize_readme([frame], [0] * 5, rects, 60, 60, (0, 0, 0), 1.4, 0.5, 255.0,
                                             preserve_ar=False),
        literal_out=ref.crop_resize_readme([frame], [0] * 5, rects, 60, 60, (0, 0, 0), 1.4, 0.5, 255.0,
                                           flavour="literal"),
    )

    # --- batched crop -> resize -> normalise -> planar (config 3), 3 frames, 37 crops -------
    frames = [u8(rng, 135, 240, 3) for _ in range(3)]
    n = 37
    rects3 = chains.random_rects(rng, n, 240, 135, lo=4, hi=120)
    fi = [i % 3 for i in range(n)]
    np.savez_compressed(
        OUT / "batched_crop_resize_norm.npz", frames=np.stack(frames), rects=rects3, frame_index=np.array(fi),
        out=ref.crop_resize_norm_planar(frames, fi, rects3, 48, 32, (0, 0, 0), 255.0, chains.IMAGENET_MEAN,
                                        chains.IMAGENET_STD),
    )

    # --- NV12 -> RGB -> resize (config 4), 3 frames of 96x54 --------------------------------
    nv = [u8(rng, 81, 96) for _ in range(3)]
    np.savez_compressed(OUT / "nv12_resize.npz", frames=np.stack(nv),
                        out_32x18=ref.nv12_resize(nv, 96, 54, 32, 18, 255.0),
                        out_40x22=ref.nv12_resize(nv, 96, 54, 40, 22, 255.0))

    # --- host-derived resize parameters (Resize::build) --------------------------------------
    q = np.zeros((4000, 4), np.int32)
    q[:, :] = rng.integers(1, 700, (4000, 4))
    q[:100, 2:] = 224
    q[100:200, 2:] = 60
    res = np.zeros((4000, 2, 6), np.int64)
    for i, (sw, sh, dw, dh) in enumerate(q):
        for ar in (0, 1):
            (fx, fy), roi = ref.resize_params(int(sw), int(sh), int(dw), int(dh), ar)
            res[i, ar] = (np.float32(fx).view(np.uint32), np.float32(fy).view(np.uint32), *roi)
    np.savez_compressed(OUT / "resize_params.npz", query=q, result=res)

    # --- Cast<float3,int3> / Cast<float3,uint3> closing a chain (own seed: added after the fixtures above) ---
    rng2 = np.random.default_rng(20240608)
    img2 = u8(rng2, 37, 53, 3)
    np.savez_compressed(OUT / "int_casts.npz", src=img2,
                        cast_mul_sub_cast_int3=ref.cast_mul_sub_cast_int3(img2, (1.37, 0.5, 2.25), (100.5, 3.25, 7.0)),
                        cast_resize_mul_cast_uint3_30x20=ref.cast_resize_mul_cast_uint3(img2, 30, 20, (3.7, 1.0, 0.01)))
    # --- the other aspect-ratio modes, NV21 and the bt601 / bt2020 matrices, a partly filled batch (own seed) ---
    rng3 = np.random.default_rng(20240609)
    frames3 = [u8(rng3, 120, 200, 3) for _ in range(2)]
    rects4 = chains.random_rects(rng3, 12, 200, 120, lo=3, hi=110)
    fi4 = [i % 2 for i in range(12)]
    np.savez_compressed(
        OUT / "ar_modes.npz", frames=np.stack(frames3), rects=rects4, frame_index=np.array(fi4),
        rn_even=ref.crop_resize_norm_planar_mode(frames3, fi4, rects4, 44, 30, 3, (3.0, 5.0, 7.0), 255.0, chains.IMAGENET_MEAN,
                                                 chains.IMAGENET_STD),
        left=ref.crop_resize_norm_planar_mode(frames3, fi4, rects4, 44, 30, 4, (3.0, 5.0, 7.0), 255.0, chains.IMAGENET_MEAN,
                                              chains.IMAGENET_STD))
    nv3 = [u8(rng3, 81, 96) for _ in range(2)]
    np.savez_compressed(OUT / "nv_layouts.npz", frames=np.stack(nv3),
                        nv12_bt601=ref.nv_resize_ex(nv3, 96, 54, 40, 22, 255.0, 0, 1),
                        nv12_bt2020=ref.nv_resize_ex(nv3, 96, 54, 40, 22, 255.0, 0, 2),
                        nv21_bt709=ref.nv_resize_ex(nv3, 96, 54, 40, 22, 255.0, 1, 0),
                        nv21_bt601=ref.nv_resize_ex(nv3, 96, 54, 32, 18, 255.0, 1, 1))
    imgs4 = [u8(rng3, 20, 36, 3) for _ in range(4)]
    np.savez_compressed(OUT / "default_planes.npz", srcs=np.stack(imgs4),
                        used2=ref.batch4_default_cast_mul(imgs4, 2, (7, 200, 33), (1.5, 0.25, 2.0)),
                        used0=ref.batch4_default_cast_mul(imgs4, 0, (7, 200, 33), (1.5, 0.25, 2.0)))
    # --- BorderReader, Warping, Deinterlace (own seed) ---------------------------------------------------------
    rng4 = np.random.default_rng(20240610)
    img4 = u8(rng4, 24, 40, 3)
    fix = {"src": img4, "rect": np.array(READBACK_RECT), "affine": np.array(READBACK_AFFINE, np.float32),
           "perspective": np.array(READBACK_PERSPECTIVE, np.float32)}
    for b in range(1, 6):
        fix[f"border{b}_crop"] = ref.border_crop(img4, b, (9, 99, 199), READBACK_RECT)
        fix[f"border{b}_crop_resize"] = ref.border_crop_resize(img4, b, (9, 99, 199), READBACK_RECT, 36, 28)
    fix["warp_affine"] = ref.warp(img4, False, READBACK_AFFINE, 48, 32, (1.0, 0.5, 2.0))
    fix["warp_perspective"] = ref.warp(img4, True, READBACK_PERSPECTIVE, 48, 32, (1.0, 0.5, 2.0))
    for k in (1, 2, 3):
        fix[f"deinterlace{k}"] = ref.deinterlace(img4, k, (1.0, 0.5, 2.0))
    np.savez_compressed(OUT / "readback_ops.npz", **fix)
    # --- YUV layouts beyond NV12 / NV21: P010, P210, Y210, UYVY (own seed) -------------------------------------
    from fusedkernellibrary_b200 import abi
    from tests import cases as tc
    rng5 = np.random.default_rng(20240611)
    fix = {}
    for fmt in (abi.SRC_P010, abi.SRC_P210, abi.SRC_Y210, abi.SRC_UYVY):
        img = tc.yuv_layout_image(rng5, fmt, 38, 22, pitch_pad=16)
        fix[f"src{fmt}"] = img
        for prim in (0, 1, 2):
            fix[f"fmt{fmt}_prim{prim}"] = ref.yuv_format_chain(img, fmt, prim, 38, 22, 38, 22, (1.0, 0.5, 2.0))
        fix[f"fmt{fmt}_resize"] = ref.yuv_format_chain(img, fmt, fmt % 3, 38, 22, 27, 15, (1.0, 0.5, 2.0))
    np.savez_compressed(OUT / "yuv_layouts.npz", **fix)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
