"""Which product carries the norms around it (``kernels.ops.norm_ride_parts``): decided from the
number of rows, the dtype and the weight's layout alone, so it can be checked without a GPU (the
kernel libraries are compiled and loaded, none of their kernels runs)."""

import pytest
import torch

from distengine_b200.kernels import ops


def _w(n, k, dtype=torch.bfloat16):
    return torch.zeros(n, k, dtype=dtype)


def test_rows_up_to_16_ride_on_the_weight_streaming_kernel():
    # blocks of 8 weight rows while there are few rows, of 16 beyond
    assert ops.norm_ride_parts(1, _w(2048, 2048), torch.bfloat16) == 256
    assert ops.norm_ride_parts(16, _w(2048, 5632), torch.bfloat16) == 256
    assert ops.norm_ride_parts(8, _w(8192, 2048), torch.bfloat16) == 512
    assert ops.norm_ride_parts(8, _w(331, 120), torch.bfloat16) == 42


def test_rows_17_to_32_ride_on_the_swapped_operand_kernel():
    assert ops.norm_ride_parts(17, _w(2048, 2048), torch.bfloat16) == 16
    assert ops.norm_ride_parts(32, _w(331, 120), torch.bfloat16) == 3


@pytest.mark.parametrize("rows", [0, 33, 64, 1024, 4096])
def test_other_row_counts_keep_the_norm_kernel(rows):
    assert ops.norm_ride_parts(rows, _w(2048, 2048), torch.bfloat16) == 0


def test_float32_and_unaligned_weights_keep_the_norm_kernel():
    assert ops.norm_ride_parts(8, _w(2048, 2048, torch.float32), torch.float32) == 0
    assert ops.norm_ride_parts(8, _w(2048, 2044), torch.bfloat16) == 0          # k not a multiple of 8
    assert ops.norm_ride_parts(8, _w(2048, 4096)[:, :2048], torch.bfloat16) == 0  # rows not contiguous


def test_the_switch_turns_it_off(monkeypatch):
    monkeypatch.setattr(ops, "NORM_RIDE", False)
    assert ops.norm_ride_parts(8, _w(2048, 2048), torch.bfloat16) == 0
