"""The reference's own run-time checks for this path, on the CUDA path through the C ABI."""
import numpy as np
import pytest

from fusedkernellibrary_b200 import abi
from tests.known_answers import KNOWN_ANSWER_CASES, check_known_answer

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("case", KNOWN_ANSWER_CASES, ids=lambda c: c.name)
def test_known_answer_on_gpu(case, fkb_lib):
    arrays = case.make_arrays()
    dev = {k: torch.from_numpy(v.view(np.uint8).reshape(-1).copy()).cuda() for k, v in arrays.items()}
    abi.execute(case.build(lambda n: dev[n].data_ptr()))
    arrays["out"] = dev["out"].cpu().numpy().view(arrays["out"].dtype).reshape(arrays["out"].shape)
    check_known_answer(case, arrays)


def test_batched_crop_resize_grid_matches_reference_active_threads(fkb_lib):
    """Two crops resized to 100x100 run as 100 x 100 x 2 output elements
    (tests/algorithm/test_crop.h:30-45)."""
    from fusedkernellibrary_b200 import chains
    frame = torch.zeros(200 * 300 * 3, dtype=torch.uint8, device="cuda")
    out = torch.zeros(2 * 100 * 100 * 3, dtype=torch.float32, device="cuda")
    plan = chains.crop_resize_batch(frame_ptrs=[frame.data_ptr()], frame_index=[0, 0],
                                    rects=[(0, 0, 50, 40), (10, 10, 120, 80)], src_width=300, src_height=200,
                                    src_pitch=900, dst=out.data_ptr(), dst_width=100, dst_height=100, post_ops=[],
                                    planar=False, mode=abi.RESIZE_IGNORE_AR)
    d = abi.DevicePlan(plan)
    info = d.info()
    assert (info.n_planes, info.output_pixels) == (2, 100 * 100 * 2)
    d.destroy()
