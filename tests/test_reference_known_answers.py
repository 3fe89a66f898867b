"""The run-time checks the reference's own tests hold for this path, restated on the checker
(CPU) - the GPU versions are in test_gpu_reference_known_answers.py."""
import numpy as np

from fusedkernellibrary_b200 import abi, chains
from fusedkernellibrary_b200.abi import op
from tests.known_answers import KNOWN_ANSWER_CASES, check_known_answer


def test_known_answers_on_checker(oracle_port):
    for case in KNOWN_ANSWER_CASES:
        arrays = case.make_arrays()
        plan = case.build(lambda n: arrays[n].ctypes.data)
        oracle_port.run(plan)
        check_known_answer(case, arrays)
