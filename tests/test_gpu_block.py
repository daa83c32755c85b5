"""Fused inverted-residual block (espdl_b200_fused_block) against the oracle's node-by-node chain: expand 1x1 ->
depthwise 3x3 -> project 1x1 (-> Add), bit for bit, over the block shapes of MobileNetV2 and ragged ones."""
import numpy as np
import pytest

import cases
import gpu_util
from espdl_b200 import abi

pytestmark = pytest.mark.gpu

# (h, w, cin, chid, cout, stride, expand)
SHAPES = [
    (14, 14, 32, 192, 32, 1, True),     # one full tile, residual
    (28, 28, 32, 192, 32, 1, True),     # four tiles
    (28, 28, 32, 192, 64, 2, True),     # stride 2
    (112, 112, 16, 96, 24, 2, True),    # Cin below one MMA K step, Cout padded to 32, ragged chunk (96 = 64 + 32)
    (14, 14, 64, 384, 96, 1, True),
    (14, 14, 96, 576, 160, 2, True),    # 14 -> 7
    (7, 7, 160, 960, 320, 1, True),     # 9x9 patch in one MMA block, Cout in two pieces
    (7, 7, 160, 960, 160, 1, True),
    (112, 112, 32, 32, 16, 1, False),   # depthwise -> pointwise pair (no expand)
    (20, 19, 32, 80, 40, 1, True),      # ragged tiles and channel counts
    (21, 18, 48, 144, 24, 2, True),
    (5, 9, 16, 64, 16, 1, True),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(str(v) for v in s))
def test_block_matches_node_chain(shape):
    h, w, cin, chid, cout, stride, expand = shape
    case = cases.block_case(seed=3, n=2, h=h, w=w, cin=cin, chid=chid, cout=cout, stride=stride, expand=expand)
    got = gpu_util.run_block_gpu(case)
    want = gpu_util.run_block_oracle(case)
    assert want.std() > 2, "degenerate case: the block output barely varies"
    np.testing.assert_array_equal(got, want)


def test_block_many_images_persistent_loop():
    case = cases.block_case(seed=4, n=40, h=28, w=28, cin=32, chid=192, cout=32)  # 160 tiles > 148 CTAs
    np.testing.assert_array_equal(gpu_util.run_block_gpu(case), gpu_util.run_block_oracle(case))


def test_block_clamps_fold_relu6():
    case = cases.block_case(seed=5, n=2, h=14, w=14, clip1=48, clipdw=24)
    np.testing.assert_array_equal(gpu_util.run_block_gpu(case), gpu_util.run_block_oracle(case))


@pytest.mark.parametrize("round_mode", [abi.ROUND_HALF_UP, abi.ROUND_HALF_EVEN])
def test_block_general_requantisation(round_mode):
    """Per-tensor exponents, half-even rounding and shifts outside 1..24 take the general epilogues."""
    case = cases.block_case(seed=6, n=1, h=14, w=14, per_channel=False, round_mode=round_mode, clip1=60)
    np.testing.assert_array_equal(gpu_util.run_block_gpu(case), gpu_util.run_block_oracle(case))
    case = cases.block_case(seed=7, n=1, h=10, w=10, cin=16, chid=32, cout=16, round_mode=round_mode, e=(-5, -14, -5, -5))
    np.testing.assert_array_equal(gpu_util.run_block_gpu(case), gpu_util.run_block_oracle(case))


def test_block_rejects_what_it_cannot_run():
    case = cases.block_case(seed=8, n=1, h=8, w=8, cin=24, chid=144, cout=24)  # Cin not a multiple of 16
    gpu_util.run_block_gpu(case, expect=abi.ERR_UNSUPPORTED)


# depthwise -> pointwise pairs (no expand conv): (h, w, hidden, cout, stride)
PAIRS = [
    (112, 112, 96, 24, 2),      # the network's largest pair: stride 2, 24 output channels (rows of 24 bytes)
    (56, 56, 144, 24, 1),       # residual, channel block 48 (64-byte operand rows, 16 of them padding)
    (56, 56, 144, 32, 2),
    (28, 28, 192, 32, 1),       # residual
    (28, 28, 192, 64, 2),
    (14, 14, 384, 64, 1),
    (14, 14, 384, 96, 1),
    (14, 14, 576, 96, 1),
    (14, 14, 576, 160, 2),      # 14 -> 7
    (7, 7, 960, 160, 1),        # several images per tile
    (112, 112, 32, 16, 1),      # 32-byte operand rows
    (33, 45, 64, 40, 1),        # ragged tiles, output channels that are no multiple of 16
    (15, 17, 16, 8, 2),
    (9, 9, 128, 250, 1),        # a wide pointwise conv
]


@pytest.mark.parametrize("shape", PAIRS, ids=lambda s: "x".join(str(v) for v in s))
def test_depthwise_pointwise_pair_matches_node_chain(shape):
    """The fused depthwise -> pointwise kernel (the depthwise result goes from registers into the tensor cores' operand in
    shared memory) against the oracle's two nodes (+ Add where the block has a residual), bit for bit."""
    h, w, chid, cout, stride = shape
    case = cases.block_case(seed=11, n=3, h=h, w=w, cin=chid, chid=chid, cout=cout, stride=stride, expand=False)
    got = gpu_util.run_block_gpu(case)
    want = gpu_util.run_block_oracle(case)
    assert want.std() > 2
    np.testing.assert_array_equal(got, want)


def test_depthwise_pointwise_pair_many_tiles_and_general_requantisation():
    case = cases.block_case(seed=12, n=70, h=28, w=28, cin=192, chid=192, cout=32, expand=False)   # more tiles than CTAs
    np.testing.assert_array_equal(gpu_util.run_block_gpu(case), gpu_util.run_block_oracle(case))
    # per-tensor exponents, and depthwise shifts outside 1..24 (the plain-loop form of the depthwise warps)
    case = cases.block_case(seed=13, n=2, h=14, w=14, cin=96, chid=96, cout=24, expand=False, per_channel=False)
    np.testing.assert_array_equal(gpu_util.run_block_gpu(case), gpu_util.run_block_oracle(case))
    case = cases.block_case(seed=14, n=2, h=10, w=10, cin=32, chid=32, cout=16, expand=False, e=(-5, -5, -14, -5))
    np.testing.assert_array_equal(gpu_util.run_block_gpu(case), gpu_util.run_block_oracle(case))
