"""What the engine does with the word that kernels set when a bounded wait ran out
(the CPU part; tests/test_gpu_generate.py sets the word on the device)."""
import pytest

from mstar_b200 import ops


def test_zero_is_silent_and_every_code_names_its_kernel():
    ops.raise_on_wait_code(0)
    for code in range(1, 15):
        with pytest.raises(ops.KernelError, match=f"code {code}"):
            ops.raise_on_wait_code(code)
    with pytest.raises(ops.KernelError, match="decode attention"):
        ops.raise_on_wait_code(4)
    with pytest.raises(ops.KernelError, match="unknown kernel"):
        ops.raise_on_wait_code(77)
