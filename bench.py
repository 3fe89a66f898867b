#!/usr/bin/env python
"""Benchmark of the fused-execution hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input: one plan launch
(one kernel).  The default workload is the batched crop -> resize -> normalise -> planar
configuration (1024 crops from 8 4K frames per GPU); with N > 1 every rank owns its own
frames, crops and output tensor (planes shard with no collective), so scaling is weak.

One JSON line is printed by rank 0.  `value` is output Mpix/s with inputs resident in HBM;
`e2e` is the same metric through the host-buffer C-ABI call (pinned host -> device copies,
launch, device -> pinned host copy back, every step); `roofline` relates the kernel's
algorithmic bytes to the measured HBM copy bandwidth; `cpu_baseline` is the reference's own
CPU code for the same chain, compiled from its headers, timed on this box's host cores;
`reference_gpu` is the reference's own CUDA kernel, compiled from its headers for sm_100a, on
the same device buffers; `sustained` repeats the launch for over a second with clocks and power
sampled; `other_workloads` times the other configurations the same way; with N > 1 `strong`
splits ONE batch over the ranks, with and without gathering the consolidated tensor by NCCL.

`--impl reference` times the reference's CPU implementation instead (all host threads, rank 0 only).
`--kernel-only` runs the timed region alone (what the profiler captures use).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from fusedkernellibrary_b200 import abi, chains  # noqa: E402

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's kernel, from the ncu
# capture summarised under profiles/ (None = not captured).
TRAFFIC_BYTES_PER_LAUNCH = {"c3": 776.2e6, "c4": 470.6e6}


# --------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------
class Workload:
    """Host arrays + a plan builder.  `build(ptr)` lowers the chain given a name -> address map."""

    name = ""
    description = ""
    sets = 1  # independent buffer sets rotated between steps (working sets smaller than L2)

    def __init__(self, seed: int):
        self.seed = seed
        self.sources: list[dict] = []   # one dict of numpy arrays per buffer set
        self.outputs: list[dict] = []

    def build(self, ptr, s: int) -> abi.HostPlan:
        raise NotImplementedError

    def reference_run(self, threads: int, s: int = 0, planes=None) -> float | None:
        """Runs the reference's CPU code on buffer set s; returns output pixels computed, or None."""
        return None

    def reference_gpu(self, ptr, s: int = 0) -> bool:
        """Enqueues the reference's own CUDA kernel(s) for buffer set s (device pointers from `ptr`) on the
        stream given to oracle.reference_gpu.set_stream; False when the chain is not built for it."""
        return False

    out_pixels = 0
    algorithmic_bytes = None   # None: what fkb_plan_get_info reports (source bytes inside the crops + output bytes)
    algorithmic_note = "source bytes inside the crop rects + output bytes"


def _u8(rng, *shape):
    return rng.integers(0, 256, shape, dtype=np.uint8)


def _parallel(fn, chunks, threads):
    if threads <= 1 or len(chunks) <= 1:
        for c in chunks:
            fn(c)
        return
    it = iter(chunks)
    lock = threading.Lock()

    def worker():
        while True:
            with lock:
                c = next(it, None)
            if c is None:
                return
            fn(c)

    ts = [threading.Thread(target=worker) for _ in range(min(threads, len(chunks)))]
    [t.start() for t in ts]
    [t.join() for t in ts]


class CropResizeNorm(Workload):
    """Config 3: PerThreadRead[B] -> Crop[B] -> Resize<INTER_LINEAR,PRESERVE_AR>(224x224, bg 0)
    -> Div(255) -> Sub(mean) -> Div(std) -> TensorSplit (B x 3 x 224 x 224 float)."""
    name = "c3"

    def __init__(self, seed, n_frames=8, fw=3840, fh=2160, n_planes=1024, dw=224, dh=224, lo=16, hi=512):
        super().__init__(seed)
        rng = np.random.default_rng(seed)
        self.fw, self.fh, self.dw, self.dh, self.n = fw, fh, dw, dh, n_planes
        self.rects = chains.random_rects(rng, n_planes, fw, fh, lo=lo, hi=hi)
        self.frame_index = [i % n_frames for i in range(n_planes)]
        self.sources = [{f"frame{i}": _u8(rng, fh, fw * 3) for i in range(n_frames)}]
        self.outputs = [{"out": ((n_planes, 3, dh, dw), np.float32)}]
        self.n_frames = n_frames
        self.out_pixels = n_planes * dw * dh
        self.description = (f"C3 batched crop-resize-norm: {n_frames} frames {fw}x{fh} uchar3, {n_planes} crops "
                            f"w,h~U[{lo},{hi}] -> PRESERVE_AR {dw}x{dh} -> /255 -mean /std -> planar f32")

    def build(self, ptr, s=0, first=0, count=None):
        count = self.n - first if count is None else count
        sl = slice(first, first + count)
        return chains.crop_resize_batch(
            frame_ptrs=[ptr(f"frame{i}") for i in range(self.n_frames)], frame_index=self.frame_index[sl],
            rects=self.rects[sl], src_width=self.fw, src_height=self.fh, src_pitch=self.fw * 3,
            dst=ptr("out") + first * self.dw * self.dh * 12, dst_width=self.dw, dst_height=self.dh,
            post_ops=chains.normalize_ops(), planar=True)

    def reference_run(self, threads, s=0, planes=None, out=None):
        from oracle import reference as ref
        n = self.n if planes is None else planes
        if out is None:
            if getattr(self, "_ref_out", None) is None:
                self._ref_out = np.zeros((self.n, 3, self.dh, self.dw), np.float32)
            out = self._ref_out[:n]
        frames = [self.sources[s][f"frame{i}"].reshape(self.fh, self.fw, 3) for i in range(self.n_frames)]
        step = 16
        chunks = [(a, min(a + step, n)) for a in range(0, n, step)]

        def run(c):
            a, b = c
            ref.crop_resize_norm_planar(frames, self.frame_index[a:b], self.rects[a:b], self.dw, self.dh, (0, 0, 0),
                                        255.0, chains.IMAGENET_MEAN, chains.IMAGENET_STD, out=out[a:b])

        _parallel(run, chunks, threads)
        return n * self.dw * self.dh

    def reference_gpu(self, ptr, s=0):
        from oracle import reference_gpu as rg
        rg.crop_resize_norm_planar([ptr(f"frame{i}") for i in range(self.n_frames)], self.frame_index, self.fw, self.fh,
                                   self.fw * 3, self.rects, self.dw, self.dh, (0, 0, 0), 255.0, chains.IMAGENET_MEAN,
                                   chains.IMAGENET_STD, ptr("out"))
        return True


class ReadmeCropResize(Workload):
    """Config 2: the README chain, 5 crops of one 4K frame -> 60x60x5 packed float3.
    `repeat` > 1 cycles the five rects over more planes and 8 frames (the scaled variant)."""
    name = "c2"

    def __init__(self, seed, repeat=1):
        super().__init__(seed)
        rng = np.random.default_rng(seed)
        self.fw, self.fh = 3840, 2160
        self.n = 5 * repeat
        self.n_frames = 1 if repeat == 1 else 8
        self.rects = np.tile(chains.README_RECTS, (repeat, 1))
        self.frame_index = [(i // 5) % self.n_frames for i in range(self.n)]
        self.sets = 1
        self.sources = [{f"frame{i}": _u8(rng, self.fh, self.fw * 3) for i in range(self.n_frames)}]
        self.outputs = [{"out": ((self.n, 60, 60, 3), np.float32)}]
        self.out_pixels = self.n * 3600
        self.name = "c2" if repeat == 1 else "c2s"
        self.description = (f"C2 README crop-resize: {self.n_frames} frame(s) 3840x2160 uchar3, {self.n} crops "
                            "(README rects) -> PRESERVE_AR 60x60 -> *1.4 -0.5 /255 -> RGB2BGR -> packed float3")

    def build(self, ptr, s=0):
        return chains.crop_resize_batch(
            frame_ptrs=[ptr(f"frame{i}") for i in range(self.n_frames)], frame_index=self.frame_index, rects=self.rects,
            src_width=self.fw, src_height=self.fh, src_pitch=self.fw * 3, dst=ptr("out"), dst_width=60, dst_height=60,
            post_ops=chains.readme_ops(), planar=False)

    def reference_run(self, threads, s=0, planes=None):
        from oracle import reference as ref
        frames = [self.sources[s][f"frame{i}"].reshape(self.fh, self.fw, 3) for i in range(self.n_frames)]
        n = self.n
        out = np.empty((n, 60, 60, 3), np.float32)
        chunks = [(a, min(a + 80, n)) for a in range(0, n, 80)]

        def run(c):
            a, b = c
            out[a:b] = ref.crop_resize_readme(frames, self.frame_index[a:b], self.rects[a:b], 60, 60, (0, 0, 0), 1.4,
                                              0.5, 255.0)

        _parallel(run, chunks, threads)
        return n * 3600

    def reference_gpu(self, ptr, s=0):
        from oracle import reference_gpu as rg
        rg.crop_resize_readme([ptr(f"frame{i}") for i in range(self.n_frames)], self.frame_index, self.fw, self.fh,
                              self.fw * 3, self.rects, 60, 60, (0, 0, 0), 1.4, 0.5, 255.0, ptr("out"))
        return True


class VerticalFusion(Workload):
    """Config 1: PerThreadRead<uchar3> -> Cast -> Mul(1.4) -> Sub(0.5) -> Div(255) -> PerThreadWrite<float3>."""
    name = "c1"

    def __init__(self, seed, w=1920, h=1080, sets=12):
        super().__init__(seed)
        rng = np.random.default_rng(seed)
        self.w, self.h, self.sets = w, h, sets
        self.sources = [{"src": _u8(rng, h, w * 3)} for _ in range(sets)]
        self.outputs = [{"out": ((h, w, 3), np.float32)} for _ in range(sets)]
        self.out_pixels = w * h
        self.description = f"C1 vertical fusion: {w}x{h} uchar3 -> Cast, *1.4, -0.5, /255 -> float3 ({sets} buffer sets)"

    def build(self, ptr, s=0):
        return chains.elementwise(chains.cast_mul_sub_div_ops(), src=ptr("src"), dst=ptr("out"), width=self.w,
                                  height=self.h)

    def reference_run(self, threads, s=0, planes=None):
        from oracle import reference as ref
        ref.cast_mul_sub_div(self.sources[s]["src"].reshape(self.h, self.w, 3), 1.4, 0.5, 255.0)
        return self.out_pixels

    def reference_gpu(self, ptr, s=0):
        from oracle import reference_gpu as rg
        rg.cast_mul_sub_div(ptr("src"), self.w, self.h, self.w * 3, 1.4, 0.5, 255.0, ptr("out"), self.w * 12)
        return True


class VerticalFusionBatch(Workload):
    """Config 1's chain on a batch of images in one launch (BatchRead of the same sequence): the
    single 31 MB image of config 1 is too small to show what the element-wise body sustains."""
    name = "c1b"

    def __init__(self, seed, n=16, w=1920, h=1080, sets=2):
        super().__init__(seed)
        rng = np.random.default_rng(seed)
        self.w, self.h, self.n, self.sets = w, h, n, sets
        self.sources = [{f"src{i}": _u8(rng, h, w * 3) for i in range(n)} for _ in range(sets)]
        self.outputs = [{"out": ((n, h, w, 3), np.float32)} for _ in range(sets)]
        self.out_pixels = n * w * h
        self.description = (f"C1 chain on a batch: {n} x {w}x{h} uchar3 -> Cast, *1.4, -0.5, /255 -> float3, one launch "
                            f"({sets} buffer sets)")

    def build(self, ptr, s=0):
        plan = abi.HostPlan()
        seq = plan.add_sequence(abi.SRC_U8X3, abi.DST_F32X3_PACKED, abi.RESIZE_NONE, chains.cast_mul_sub_div_ops())
        for i in range(self.n):
            plan.add_plane(src=ptr(f"src{i}"), src_width=self.w, src_height=self.h, src_pitch=self.w * 3,
                           dst=ptr("out") + i * self.w * self.h * 12, dst_width=self.w, dst_height=self.h,
                           dst_pitch=self.w * 12, sequence=seq)
        return plan

    def reference_run(self, threads, s=0, planes=None):
        from oracle import reference as ref
        for i in range(self.n):
            ref.cast_mul_sub_div(self.sources[s][f"src{i}"].reshape(self.h, self.w, 3), 1.4, 0.5, 255.0)
        return self.out_pixels

    def reference_gpu(self, ptr, s=0):
        from oracle import reference_gpu as rg
        if self.n % 16:
            return False
        for a in range(0, self.n, 16):
            rg.cast_mul_sub_div_batch16([ptr(f"src{i}") for i in range(a, a + 16)], self.w, self.h, self.w * 3, 1.4, 0.5,
                                        255.0, ptr("out") + a * self.w * self.h * 12)
        return True


class LongChain(Workload):
    """Config 5A: N alternating Add(0.001)/Mul(1.0001) on a 3840x2160 float3 image."""
    name = "c5a"

    def __init__(self, seed, n_ops=16, w=3840, h=2160, sets=2):
        super().__init__(seed)
        rng = np.random.default_rng(seed)
        self.w, self.h, self.sets, self.n_ops = w, h, sets, n_ops
        self.sources = [{"src": rng.random((h, w * 3), dtype=np.float32)} for _ in range(sets)]
        self.outputs = [{"out": ((h, w, 3), np.float32)} for _ in range(sets)]
        self.out_pixels = w * h
        self.name = f"c5a{n_ops}"
        self.description = f"C5A long chain: {w}x{h} float3, {n_ops} alternating Add(0.001)/Mul(1.0001) ({sets} buffer sets)"

    def build(self, ptr, s=0):
        return chains.elementwise(chains.addmul_ops(self.n_ops), src=ptr("src"), dst=ptr("out"), width=self.w,
                                  height=self.h, src_format=abi.SRC_F32X3)

    def reference_run(self, threads, s=0, planes=None):
        from oracle import reference as ref
        ref.addmul_chain(self.sources[s]["src"].reshape(self.h, self.w, 3), self.n_ops, 0.001, 1.0001)
        return self.out_pixels

    def reference_gpu(self, ptr, s=0):
        from oracle import reference_gpu as rg
        return rg.addmul_chain(ptr("src"), self.w, self.h, self.w * 12, self.n_ops, 0.001, 1.0001, ptr("out"), self.w * 12)


class Nv12Resize(Workload):
    """Config 4: ReadYUV<NV12>[32] -> ConvertYUVToRGB<bt709,Full,float3> -> Resize 1280x720 -> Div(255)
    -> TensorWrite<float3>."""
    name = "c4"

    def __init__(self, seed, n=32, w=3840, h=2160, dw=1280, dh=720):
        super().__init__(seed)
        rng = np.random.default_rng(seed)
        self.n, self.w, self.h, self.dw, self.dh = n, w, h, dw, dh
        self.sources = [{f"frame{i}": _u8(rng, h + h // 2, w) for i in range(n)}]
        self.outputs = [{"out": ((n, dh, dw, 3), np.float32)}]
        self.out_pixels = n * dw * dh
        # tap samples + output per output pixel: 4 luma bytes, 4.5 chroma bytes, 12 output bytes; the whole
        # frames (what the plan reports) would be (w*h*1.5*n + output) = 752 MB at the full size
        self.algorithmic_bytes = int(self.out_pixels * 20.5)
        self.algorithmic_note = "tap samples + output: (4 Y + 4.5 UV + 12) B per output pixel"
        self.description = f"C4 NV12 BVF: {n} NV12 frames {w}x{h} -> BT.709 full RGB -> resize {dw}x{dh} -> /255 -> packed float3"

    def build(self, ptr, s=0):
        return chains.nv12_resize_batch(frame_ptrs=[ptr(f"frame{i}") for i in range(self.n)], width=self.w,
                                        height=self.h, pitch=self.w, dst=ptr("out"), dst_width=self.dw,
                                        dst_height=self.dh)

    def reference_run(self, threads, s=0, planes=None):
        from oracle import reference as ref
        n = self.n if planes is None else planes
        out = np.empty((n, self.dh, self.dw, 3), np.float32)
        chunks = [(a, min(a + 2, n)) for a in range(0, n, 2)]

        def run(c):
            a, b = c
            ref.nv12_resize([self.sources[s][f"frame{i}"] for i in range(a, b)], self.w, self.h, self.dw, self.dh,
                            255.0, out=out[a:b])

        _parallel(run, chunks, threads)
        return n * self.dw * self.dh

    def reference_gpu(self, ptr, s=0):
        from oracle import reference_gpu as rg
        rg.nv12_resize([ptr(f"frame{i}") for i in range(self.n)], self.w, self.h, self.w, self.dw, self.dh, 255.0, ptr("out"))
        return True


class Divergent(Workload):
    """Config 5B: one launch, four different chains on four groups of 16 images 1920x1080 uchar3."""
    name = "c5b"

    def __init__(self, seed, per_group=16, w=1920, h=1080):
        super().__init__(seed)
        rng = np.random.default_rng(seed)
        self.w, self.h, self.pg = w, h, per_group
        self.sources = [{f"img{i}": _u8(rng, h, w * 3) for i in range(4 * per_group)}]
        self.outputs = [{"g0": ((per_group, h, w, 3), np.float32), "g1": ((per_group, h, w, 3), np.float32),
                         "g2": ((per_group, h, w, 3), np.uint8), "g3": ((per_group, h // 2, w // 2, 3), np.float32)}]
        self.out_pixels = per_group * (3 * w * h + (w // 2) * (h // 2))
        self.description = (f"C5B divergent horizontal fusion: 4 chains x {per_group} images {w}x{h} uchar3 in one launch "
                            "(Cast-Mul-Sub | Cast-Add-Div | BGR-Cast-Mul-Saturate u8 | Cast-Resize 960x540)")

    def build(self, ptr, s=0):
        return chains.divergent_four_groups(src_ptrs=[ptr(f"img{i}") for i in range(4 * self.pg)], width=self.w,
                                            height=self.h, dst_ptrs=[ptr(f"g{g}") for g in range(4)],
                                            resize_to=(self.w // 2, self.h // 2), per_group=self.pg)

    def reference_gpu(self, ptr, s=0):
        """Four launches: the reference has no host launcher for its divergent kernel (executors.h:129-145)."""
        from oracle import reference_gpu as rg
        if self.pg != 16:
            return False
        p = [ptr(f"img{i}") for i in range(64)]
        w, h = self.w, self.h
        rg.cast_mul_sub_batch16(p[0:16], w, h, w * 3, 1.4, 0.5, ptr("g0"))
        rg.cast_add_div_batch16(p[16:32], w, h, w * 3, 0.5, 255.0, ptr("g1"))
        rg.bgr_cast_mul_saturate_batch16(p[32:48], w, h, w * 3, 1.4, ptr("g2"))
        rg.cast_resize_batch16(p[48:64], w, h, w * 3, w // 2, h // 2, ptr("g3"))
        return True

    def reference_gpu_one_launch(self, ptr, s=0):
        """The reference's divergent kernel (executor_kernels.h:20-23) launched directly with the four sequences."""
        from oracle import reference_gpu as rg
        if self.pg != 16:
            return False
        w, h = self.w, self.h
        rg.divergent_four_groups64([ptr(f"img{i}") for i in range(64)], w, h, w * 3, 1.4, 0.5, 0.5, 255.0, w // 2, h // 2,
                                   ptr("g0"), ptr("g1"), ptr("g2"), ptr("g3"))
        return True


def make_workload(name: str, seed: int) -> Workload:
    if name == "c3":
        return CropResizeNorm(seed)
    if name == "c3small":
        return CropResizeNorm(seed, n_frames=8, n_planes=256)
    if name == "c2":
        return ReadmeCropResize(seed)
    if name == "c2s":
        return ReadmeCropResize(seed, repeat=8192 // 5)
    if name == "c1":
        return VerticalFusion(seed)
    if name == "c1b":
        return VerticalFusionBatch(seed)
    if name.startswith("c5a"):
        return LongChain(seed, n_ops=int(name[3:] or 16))
    if name == "c4":
        return Nv12Resize(seed)
    if name == "c4small":
        return Nv12Resize(seed, n=8)
    if name == "c5b":
        return Divergent(seed)
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
METRIC_NAMES = {"c3": "crop-resize-norm", "c3small": "crop-resize-norm, 256 crops", "c2": "README crop-resize",
                "c2s": "README crop-resize, 8190 crops", "c1": "vertical fusion", "c1b": "vertical fusion, 16 images",
                "c4": "NV12 resize", "c4small": "NV12 resize, 8 frames", "c5b": "divergent horizontal fusion"}

# bytes that one launch really moves where that differs from the canonical algorithmic figure: the staged NV12
# kernel copies only the luma and chroma rows with a non-zero tap weight (profiles/nv12_staged_c4.md)
MOVED_BYTES_PER_OUTPUT_PIXEL = {"c4": 6.0 + 12.0, "c4small": 6.0 + 12.0}


def metric_of(wl) -> str:
    return f"output Mpix/s ({METRIC_NAMES.get(wl.name, 'long chain, ' + wl.name[3:] + ' ops' if wl.name.startswith('c5a') else wl.name)})"


def working_set_bytes(wl) -> int:
    n = 0
    for srcs, outs in zip(wl.sources, wl.outputs):
        n += sum(a.nbytes for a in srcs.values())
        n += sum(int(np.prod(shape)) * np.dtype(dt).itemsize for shape, dt in outs.values())
    return n


def base_config(wl, world: int) -> dict:
    """The `config` object of the JSON line: the same keys and values in both arms."""
    ws = working_set_bytes(wl)
    return {"workload": wl.description, "name": wl.name, "output_pixels_per_gpu_per_step": wl.out_pixels,
            "working_set_bytes_per_gpu": ws,
            "l2": ("inputs and outputs larger than L2" if ws > 2 * L2_BYTES
                   else "working set below 2x L2: buffer sets rotate, numbers are L2-assisted"),
            "sharding": "independent planes per rank, no collective",
            "seeds": "numpy default_rng(1000 + 17 * rank)"}


def measured_peak_gbs() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi sampled every `interval_ms` while a timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, interval_ms: int = 200):
        self.gpu = gpu_index
        self.interval_ms = interval_ms
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", str(self.interval_ms), "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self, settle: float = 0.25) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(settle)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": float(np.median(pw)) if pw else None, "power_w_max": max(pw) if pw else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------
# reference arm (CPU)
# --------------------------------------------------------------------------------------
def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    from oracle import reference as ref
    wl = make_workload(args.workload, 1000)
    threads = os.cpu_count() or 1
    if not ref.available() or wl.reference_run(1, 0, planes=1) is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built for this workload"}))
        return
    for _ in range(args.warmup):
        wl.reference_run(threads)
    t0 = time.perf_counter()
    px = 0
    for _ in range(args.steps):
        px += wl.reference_run(threads)
    dt = time.perf_counter() - t0
    val = px / dt / 1e6
    line = {
        "impl": "reference", "metric": metric_of(wl), "value": val, "unit": "Mpix/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": base_config(wl, args.gpus),
        "note": "reference CPU backend (TransformDPP<ParArch::CPU>) compiled from its own headers with the device "
                "branch of interpolation.h selected; plane chunks of 16 on all host threads",
        "cpu_baseline": {"value": val, "unit": "Mpix/s", "cores": threads, "kind": "reference",
                         "sample": f"the whole workload ({wl.out_pixels} output px) per step"},
        "e2e": {"value": val, "unit": "Mpix/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# our arm (GPU)
# --------------------------------------------------------------------------------------
class DeviceWorkload:
    """A workload's buffers resident on the current device, one plan per buffer set."""

    def __init__(self, wl, torch):
        self.wl = wl
        self.sets, self.plans = [], []
        for s in range(wl.sets):
            d = {k: torch.from_numpy(v).cuda() for k, v in wl.sources[s].items()}
            for k, (shape, dt) in wl.outputs[s].items():
                d[k] = torch.zeros(shape, dtype=torch.float32 if dt == np.float32 else torch.uint8, device="cuda")
            self.sets.append(d)
            self.plans.append(abi.DevicePlan(wl.build(lambda n, d=d: d[n].data_ptr(), s)))
        self.info = self.plans[0].info()

    def launch(self, i, sh):
        self.plans[i % self.wl.sets].launch(sh)

    def reference_gpu(self, i):
        d = self.sets[i % self.wl.sets]
        return self.wl.reference_gpu(lambda n: d[n].data_ptr(), i % self.wl.sets)

    def check(self, sh):
        for p in self.plans:
            p.check(sh)   # raises when a block gave up a bounded wait: the number would be invalid

    def destroy(self):
        for p in self.plans:
            p.destroy()
        self.sets = []


def time_launches(torch, stream, fn, steps, warmup):
    """CUDA events on `stream` around each of `steps` calls of fn(i) after `warmup` untimed ones; ms per call."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record(stream)
    for i in range(steps):
        fn(i)
        ev[i + 1].record(stream)
    torch.cuda.synchronize()
    return [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)], ev[0].elapsed_time(ev[-1])


def reference_gpu_record(torch, stream, dw: DeviceWorkload, steps, warmup):
    """The reference's own kernel (its headers compiled for sm_100a with nvcc's defaults) on the same device
    buffers, same event protocol."""
    from oracle import reference_gpu as rg
    if not rg.available():
        return {"unavailable": "oracle/_ref/libfklref_gpu.so was not built (reference tree absent at build time)"}
    rg.set_stream(stream.cuda_stream)
    if not dw.reference_gpu(0):
        return {"unavailable": "this chain is not instantiated in the reference wrapper (nvcc cannot compile a "
                               "256-operation chain: operate() recursion, data_parallel_patterns.h:86)"}
    n0 = rg.launches()
    per, total = time_launches(torch, stream, dw.reference_gpu, steps, warmup)
    launches = (rg.launches() - n0) / (steps + warmup)
    ms = total / steps
    rec = {"ms_per_step": ms, "value": dw.wl.out_pixels / (ms * 1e-3) / 1e6, "unit": "Mpix/s",
           "launches_per_step": launches,
           "what": "launchTransformDPP_Kernel from the reference's headers, nvcc -O3 sm_100a, default flags; batches in "
                   "chunks of at most 128 planes per launch (its per-plane parameters are kernel arguments)"}
    if hasattr(dw.wl, "reference_gpu_one_launch"):
        d = dw.sets[0]
        one = lambda i: dw.wl.reference_gpu_one_launch(lambda n: d[n].data_ptr(), 0)
        if one(0):
            _, total = time_launches(torch, stream, one, steps, warmup)
            rec["one_divergent_launch_ms"] = total / steps
            rec["one_divergent_launch_what"] = ("launchDivergentBatchTransformDPP_Kernel launched directly with the four sequences "
                                                "(the reference ships the kernel without a host launcher)")
    return rec


def call_overhead(torch, stream, dw: DeviceWorkload, calls: int = 200):
    """Host time of one call, launches queued back to back on a stream and synchronised once at the end:
    this package's asynchronous call on a repeated description (fkb_execute_async), its one-shot call that
    allocates and synchronises (fkb_execute), and the reference's executeOperations on its CUDA backend.
    All three through ctypes from Python, so each carries the same few microseconds of binding overhead."""
    from oracle import reference_gpu as rg
    sh = stream.cuda_stream
    d = dw.sets[0]
    desc = dw.wl.build(lambda n: d[n].data_ptr(), 0)
    out = {}
    abi.execute_async(desc, sh)
    abi.async_check(sh)
    t0 = time.perf_counter()
    for _ in range(calls):
        abi.execute_async(desc, sh)
    out["fkb_execute_async"] = (time.perf_counter() - t0) / calls * 1e6
    abi.async_check(sh)
    t0 = time.perf_counter()
    for _ in range(20):
        abi.execute(desc, sh)
    out["fkb_execute (allocates, synchronises)"] = (time.perf_counter() - t0) / 20 * 1e6
    if rg.available():
        rg.set_stream(sh)
        dw.reference_gpu(0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            dw.reference_gpu(0)
        out["reference executeOperations (CUDA backend)"] = (time.perf_counter() - t0) / calls * 1e6
        torch.cuda.synchronize()
    return out


def side_workload(torch, stream, name, steps, warmup, peak):
    """One more configuration, timed the same way (a few ms): kernel time, roofline fraction, reference kernel."""
    wl = make_workload(name, 1000)
    dw = DeviceWorkload(wl, torch)
    sh = stream.cuda_stream
    per, total = time_launches(torch, stream, lambda i: dw.launch(i, sh), steps, warmup)
    dw.check(sh)
    ms = float(np.mean(per))
    alg = wl.algorithmic_bytes or dw.info.algorithmic_bytes
    rec = {"name": wl.name, "workload": wl.description, "kernel_ms": ms, "value": wl.out_pixels / (ms * 1e-3) / 1e6,
           "unit": "Mpix/s", "algorithmic_bytes": alg, "achieved_gbs": alg / (ms * 1e-3) / 1e9,
           "frac": alg / (ms * 1e-3) / 1e9 / peak, "grid": dw.info.grid_x, "block": dw.info.block_x}
    if wl.name in MOVED_BYTES_PER_OUTPUT_PIXEL:
        moved = MOVED_BYTES_PER_OUTPUT_PIXEL[wl.name] * wl.out_pixels
        rec["moved_bytes"] = moved
        rec["frac_of_moved_bytes"] = moved / (ms * 1e-3) / 1e9 / peak
    rec["reference_gpu"] = reference_gpu_record(torch, stream, dw, steps, warmup)
    if wl.name in ("c2", "c1", "c2s"):
        rec["host_us_per_call"] = call_overhead(torch, stream, dw)
    dw.destroy()
    del dw, wl
    torch.cuda.empty_cache()
    return rec


def circular_tensor_record(torch, stream, updates: int = 128):
    """fkb_circular_tensor_update: a window of the newest 16 normalised 3x224x224 crops of 4K frames, one update per new
    crop.  Time per update with the updates queued back to back (device_us: the host prepares each update's plan, so this
    is the larger of host and kernel time) and the kernel of one update alone (kernel_us), in the reference's scheme (15
    planes copied per update) and as a sliding window."""
    rng = np.random.default_rng(1000)
    fw, fh, w, h, batch = 3840, 2160, 224, 224, 16
    frames = [torch.from_numpy(_u8(rng, fh, fw * 3)).cuda() for _ in range(4)]
    rects = chains.random_rects(rng, 64, fw, fh, lo=16, hi=512)
    plans = []
    for k in range(64):
        p = abi.HostPlan()
        seq = p.add_sequence(abi.SRC_U8X3, abi.DST_F32_PLANAR3, abi.RESIZE_PRESERVE_AR, chains.normalize_ops())
        p.add_plane(src=frames[k % 4].data_ptr(), src_width=fw, src_height=fh, src_pitch=fw * 3, crop=tuple(int(v) for v in rects[k]),
                    dst=0, dst_width=w, dst_height=h, dst_pitch=w * 4, dst_channel_stride=w * h * 4, sequence=seq)
        plans.append(p)
    sh = stream.cuda_stream
    rec = {"name": "circular", "workload": f"circular tensor of the newest {batch} 3x{h}x{w} float planes, one 4K crop per update",
           "unit": "us/update"}
    for key, sliding in (("reference_scheme", False), ("sliding_window", True)):
        ct = abi.CircularTensor(w, h, batch, abi.DST_F32_PLANAR3, abi.CIRCULAR_NEWEST_FIRST, sliding)
        for k in range(32):
            ct.update(plans[k], sh)
        abi.async_check(sh)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        t0 = time.perf_counter()
        for k in range(updates):
            ct.update(plans[k % 64], sh)
        host = (time.perf_counter() - t0) / updates * 1e6
        e1.record(stream)
        abi.async_check(sh)
        one = abi.DevicePlan(ct.plan_update(plans[0], advance=False))   # one update's plan alone: the kernel's own time
        per, _ = time_launches(torch, stream, lambda i: one.launch(sh), 20, 3)
        one.check(sh)
        one.destroy()
        rec[key] = {"kernel_us": float(np.mean(per)) * 1e3, "device_us": e0.elapsed_time(e1) / updates * 1e3, "host_us_per_call": host,
                    "planes_per_update": 2 if sliding else batch + 1,
                    "bytes_stored_per_update": ct.plane_bytes * (2 if sliding else batch + 1)}
        ct.destroy()
    return rec


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback")
    abi.load_library()
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    wl = make_workload(args.workload, 1000 + 17 * rank)
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    dw = DeviceWorkload(wl, torch)
    info = dw.info
    warmup = max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.cuda.stream(stream):
        for i in range(warmup):
            dw.launch(i, sh)
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        # --- timed region: exactly K steps, one kernel each, per-launch events inside ----
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        barrier()
        ev[0].record(stream)
        for i in range(args.steps):
            dw.launch(i, sh)
            ev[i + 1].record(stream)
        barrier()
        total_ms = ev[0].elapsed_time(ev[-1])
        per_launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
        clocks = sampler.stop() if rank == 0 else None
        dw.check(sh)

        # --- sustained: launches back to back for at least a second, clocks and power sampled inside -------
        sustained = None
        if not args.no_sustained:
            n = max(args.steps, int(1.2e3 / max(float(np.mean(per_launch_ms)), 1e-3)) + 1)
            barrier()
            s2 = ClockSampler(local_rank, interval_ms=100)
            if rank == 0:
                s2.start()
                time.sleep(0.15)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for i in range(n):
                dw.launch(i, sh)
            b.record(stream)
            torch.cuda.synchronize()
            c2 = s2.stop(settle=0.0) if rank == 0 else None
            sus_ms = max_over_ranks(a.elapsed_time(b)) / n
            dw.check(sh)
            if rank == 0:
                sustained = {"launches": n, "seconds": sus_ms * n * 1e-3, "ms_per_launch": sus_ms,
                             "value": wl.out_pixels * world / (sus_ms * 1e-3) / 1e6, "unit": "Mpix/s",
                             "sm_mhz_median": c2["sm_mhz"], "power_w_median": c2["power_w"], "power_w_max": c2["power_w_max"],
                             "clock_samples": c2["samples"], "reasons": c2["reasons"],
                             "ms_x_mhz": sus_ms * c2["sm_mhz"] if c2["sm_mhz"] else None}

    max_ms = max_over_ranks(total_ms)
    value = wl.out_pixels * world * args.steps / (max_ms * 1e-3) / 1e6
    kernel_ms = float(np.mean(per_launch_ms))
    peak, peak_kind = measured_peak_gbs()

    # --- end to end through the host-buffer C-ABI call (pinned host buffers) ---------------
    e2e = None
    if not args.no_e2e:
        host = {k: torch.from_numpy(v).pin_memory() for k, v in wl.sources[0].items()}
        for k, (shape, dt) in wl.outputs[0].items():
            host[k] = torch.zeros(shape, dtype=torch.float32 if dt == np.float32 else torch.uint8).pin_memory()
        sess = abi.HostSession(wl.build(lambda n: host[n].data_ptr(), 0))
        h2d, d2h = sess.traffic()
        e_steps = max(20, args.steps)
        with torch.cuda.stream(stream):
            for _ in range(2):
                sess.run(sh)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(e_steps):
                sess.run(sh)   # returns after the stream has been synchronised
            e1.record(stream)
            torch.cuda.synchronize()
        e_dt = max_over_ranks(e0.elapsed_time(e1) * 1e-3)
        e2e = {"value": wl.out_pixels * world * e_steps / e_dt / 1e6, "unit": "Mpix/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e_steps,
               "ms_per_step": e_dt / e_steps * 1e3,
               "api": "fkb_host_session_run (pinned host buffers; H2D + kernel + D2H + sync per step)"}
        sess.destroy()
        # the ceiling of that call on this box: the same bytes as plain pinned copies, both directions at
        # once on two streams, by the same ranks at the same time, no kernel
        d_in = torch.empty(h2d, dtype=torch.uint8, device="cuda")
        d_out = torch.empty(d2h, dtype=torch.uint8, device="cuda")
        h_in = torch.empty(h2d, dtype=torch.uint8).pin_memory()
        h_out = torch.empty(d2h, dtype=torch.uint8).pin_memory()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

        def copies():
            with torch.cuda.stream(s_in):
                d_in.copy_(h_in, non_blocking=True)
            with torch.cuda.stream(s_out):
                h_out.copy_(d_out, non_blocking=True)
            s_in.synchronize(); s_out.synchronize()

        copies()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            copies()
        c_dt = max_over_ranks(time.perf_counter() - t0)
        e2e["copy_ceiling"] = {"ms_per_step": c_dt / e_steps * 1e3,
                               "value": wl.out_pixels * world * e_steps / c_dt / 1e6, "unit": "Mpix/s",
                               "gbs_all_ranks": (h2d + d2h) * world * e_steps / c_dt / 1e9,
                               "what": "cudaMemcpyAsync of the same h2d and d2h bytes from and to pinned memory on two "
                                       "streams, every rank at once, no kernel"}
        del d_in, d_out, h_in, h_out, host

    # --- strong scaling of ONE fixed batch split over the ranks, and the consolidated output -------------
    strong = None
    if world > 1 and isinstance(wl, CropResizeNorm) and not args.no_strong:
        strong = strong_scaling(torch, dist, stream, rank, world, args.steps, warmup, max_over_ranks, barrier)

    # --- the reference's own kernel on this GPU, the other configurations, the CPU baseline ----------------
    ref_gpu = others = cpu = None
    if rank == 0 and world == 1:
        with torch.cuda.stream(stream):
            if not args.no_reference_gpu:
                ref_gpu = reference_gpu_record(torch, stream, dw, args.steps, warmup)
            if not args.no_others and args.workload == "c3":
                dw.destroy()
                others = [side_workload(torch, stream, n, 20, 3, peak) for n in ("c2s", "c2", "c4", "c5b", "c1b", "c1", "c5a16")]
                others.append(circular_tensor_record(torch, stream))
        if not args.no_cpu:
            cpu = cpu_baseline(wl)

    if rank == 0:
        alg_bytes = wl.algorithmic_bytes or info.algorithmic_bytes
        achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(wl.name), "peak_kind": f"of {peak_kind}",
                    "algorithmic_bytes_per_launch": alg_bytes, "algorithmic_bytes_are": wl.algorithmic_note,
                    "kernel_ms": kernel_ms, "frac_of_nominal_8TBs": achieved / 8000.0}
        if wl.name in MOVED_BYTES_PER_OUTPUT_PIXEL:
            moved = MOVED_BYTES_PER_OUTPUT_PIXEL[wl.name] * wl.out_pixels
            roofline["moved_bytes_per_launch"] = moved
            roofline["frac_of_moved_bytes"] = moved / (kernel_ms * 1e-3) / 1e9 / peak
        line = {
            "metric": metric_of(wl), "value": value, "unit": "Mpix/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": max_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": base_config(wl, world),
            "launch": {"planes_per_gpu": info.n_planes, "grid": info.grid_x, "block": info.block_x},
            "roofline": roofline,
            "sustained": sustained,
            "cpu_baseline": cpu,
            "reference_gpu": ref_gpu,
            "e2e": e2e,
            "strong": strong,
            "other_workloads": others,
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line))
    dw.destroy()
    if world > 1:
        dist.destroy_process_group()


def strong_scaling(torch, dist, stream, rank, world, steps, warmup, max_over_ranks, barrier):
    """The fixed 1024-crop batch (the same on every rank: seed 1000) split by contiguous plane ranges: each
    rank computes its planes straight into its slab of a whole-batch tensor; with `gather` the slabs are
    then exchanged by one NCCL all-gather so that every GPU holds the consolidated tensor."""
    from fusedkernellibrary_b200 import sharding
    wl = CropResizeNorm(1000)
    first, count = sharding.plane_range(wl.n, world, rank)
    d = {k: torch.from_numpy(v).cuda() for k, v in wl.sources[0].items()}
    out = torch.zeros((wl.n, 3, wl.dh, wl.dw), dtype=torch.float32, device="cuda")
    d["out"] = out
    plan = abi.DevicePlan(wl.build(lambda n: d[n].data_ptr(), 0, first=first, count=count))
    sh = stream.cuda_stream
    equal = wl.n % world == 0
    slab = out[first:first + count]
    rec = {}
    with torch.cuda.stream(stream):
        for gather in (False, True):
            if gather and not equal:
                break

            def step():
                plan.launch(sh)
                if gather:
                    dist.all_gather_into_tensor(out, slab)

            for _ in range(warmup):
                step()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(steps):
                step()
            b.record(stream)
            barrier()
            ms = max_over_ranks(a.elapsed_time(b)) / steps
            plan.check(sh)
            rec["gather" if gather else "compute"] = {"ms_per_step": ms, "value": wl.out_pixels / (ms * 1e-3) / 1e6, "unit": "Mpix/s"}
    plan.destroy()
    rec["what"] = (f"one batch of {wl.n} crops split over {world} GPUs by contiguous plane ranges ({count} planes on this "
                   "rank), device-timed first launch to last completion, max over ranks; gather = the same plus one "
                   "ncclAllGather of the slabs into a consolidated tensor on every GPU")
    rec["scaling"] = "strong"
    return rec


def cpu_baseline(wl: Workload):
    from oracle import reference as ref
    if ref.available() and wl.reference_run(1, 0, planes=1) is not None:
        sample_planes = None
        if isinstance(wl, CropResizeNorm):
            sample_planes = min(wl.n, 1024)
        elif isinstance(wl, Nv12Resize):
            sample_planes = 4
        t0 = time.perf_counter()
        px = wl.reference_run(1, 0, planes=sample_planes)
        dt = time.perf_counter() - t0
        reps = 1
        while dt < 3.0 and reps < 50:   # small workloads: repeat up to a few seconds
            px += wl.reference_run(1, 0, planes=sample_planes)
            dt = time.perf_counter() - t0
            reps += 1
        return {"value": px / dt / 1e6, "unit": "Mpix/s", "cores": 1, "kind": "reference",
                "host_cores_available": os.cpu_count(),
                "sample": f"{px} output px of the same workload in {dt:.1f} s on one thread (the reference CPU "
                          "backend is single-threaded)"}
    # no compiled reference for this workload: time the plain-C restatement instead
    from oracle import port
    arrays = {**wl.sources[0]}
    for k, (shape, dt_) in wl.outputs[0].items():
        arrays[k] = np.zeros(shape, dt_)
    plan = wl.build(lambda n: arrays[n].ctypes.data, 0)
    t0 = time.perf_counter()
    port.run(plan)
    dt = time.perf_counter() - t0
    return {"value": wl.out_pixels / dt / 1e6, "unit": "Mpix/s", "cores": 1, "kind": "port",
            "host_cores_available": os.cpu_count(), "sample": f"the whole workload once ({dt:.1f} s, one thread)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true")
    ap.add_argument("--no-others", action="store_true")
    ap.add_argument("--no-strong", action="store_true")
    ap.add_argument("--kernel-only", action="store_true", help="the timed region alone (for profiler runs)")
    args = ap.parse_args()
    if args.kernel_only:
        args.no_e2e = args.no_cpu = args.no_sustained = args.no_reference_gpu = args.no_others = args.no_strong = True
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with: python -m torch.distributed.run --nnodes=1 --nproc-per-node N bench.py --gpus N ...")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
