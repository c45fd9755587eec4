"""The resident-weight 3^3 kernel where it marches along z: a block owns many output planes, its piece of the plane list spans one to three
runs, the three-plane accumulator window wraps around the slot ring, the last plane of a volume commits on its own.  Full-size layers of
the benchmark's network (the shapes the benchmark times) against the oracle on identical MX operands, random operands within 1e-3 relative
L2 and exact operands bit for bit; then small ragged grids cut into few blocks with umx_conv_r_block_cap, which reach the same code paths
(several runs a piece, wrapped windows, both column-tile widths, one and two blocks a multiprocessor) in seconds."""
import numpy as np
import pytest

import gpu_util as G
import orc
import synth
from test_oracle import exact_operands

pytestmark = pytest.mark.gpu
TOL = 1e-3

FULL = [
    # N, Ci, Co, D: the level-0 and level-1 3^3 convs of the benchmark's network at their full sizes
    (1, 32, 32, 128),        # enc0.c2, dec0.c2: one input block, two blocks a multiprocessor
    (1, 64, 32, 128),        # dec0.c1: two input blocks
    (1, 64, 64, 64),         # enc1.c2, dec1.c2: 64-channel column tile, one block a multiprocessor
    (1, 128, 64, 64),        # dec1.c1: four input blocks
    (2, 32, 32, 128),        # a batch: pieces that cross from one sample into the next
    (2, 64, 64, 64),
]


def run(kind, mx, w, b, N, Ci, D, H, W, Co, bits, want_kernel=1):
    got = G.run_pm32(kind, mx, w, b, N, Ci, D, H, W, Co, bits)
    assert G.L().umx_conv_last_kernel() == want_kernel, "the launch did not take the resident-weight kernel"
    return got


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("N,Ci,Co,D", FULL)
def test_full_size_layers_random_operands(dev, N, Ci, Co, D, bits):
    S = D ** 3
    x = synth.rng(301).standard_normal(N * Ci * S).astype(np.float32)
    w, b = synth.kaiming(302, Co, Ci, 27), synth.bias(303, Co, 0.1)
    mx, want = orc.conv_case("conv3", x, w, b, N, Ci, D, D, D, Co, bits)
    del x
    got = run("conv3", mx, w, b, N, Ci, D, D, D, Co, bits)
    assert np.isfinite(got).all()
    e = orc.rel_l2(got, want)
    print("3^3 %d -> %d on %d^3 x %d, MX-fp%d: rel-L2 %.3g, max abs %.3g" % (Ci, Co, D, N, bits, e, np.abs(got - want).max()))
    assert e < TOL


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("N,Ci,Co,D", [(1, 32, 32, 128), (1, 128, 64, 64), (1, 64, 32, 128)])
def test_full_size_layers_exact_operands(dev, N, Ci, Co, D, bits):
    S = D ** 3
    x = exact_operands(311, (N, Ci, D, D, D), 1).reshape(-1)
    w = exact_operands(312, (Co, Ci, 27), 1)
    b = (synth.rng(313).integers(-8, 8, Co) * 0.5).astype(np.float32)
    mx, want = orc.conv_case("conv3", x, w, b, N, Ci, D, D, D, Co, bits)
    del x
    got = run("conv3", mx, w, b, N, Ci, D, D, D, Co, bits)
    assert np.array_equal(got, want), "%d of %d differ" % (np.count_nonzero(got != want), want.size)


SMALL = [
    # N, Ci, Co, D, H, W, cap: `cap` blocks per column tile
    (1, 32, 32, 13, 19, 16, 3),     # 4 tiles x 13 planes over 3 blocks: 17-plane pieces, two or three runs each
    (1, 32, 32, 9, 19, 48, 5),      # 12 tiles
    (2, 64, 32, 7, 19, 16, 3),      # batch: pieces cross samples; two input blocks
    (1, 64, 64, 11, 16, 16, 2),     # 64-channel column tile (one block a multiprocessor)
    (1, 128, 64, 5, 35, 16, 1),     # one block takes every plane of six tiles: a run per tile, four input blocks
    (1, 96, 128, 12, 19, 16, 2),    # three input blocks, four column tiles of 32 channels
    (2, 32, 96, 6, 16, 32, 2),      # three column tiles of 32 channels
    (1, 32, 32, 1, 64, 32, 1),      # single planes: sixteen runs of one plane, each first and last at once
    (1, 32, 32, 1, 16, 16, 0),      # fewer planes than blocks: one plane a block
    (1, 32, 32, 2, 33, 16, 1),
]


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("N,Ci,Co,D,H,W,cap", SMALL)
def test_small_grids_in_few_blocks(dev, N, Ci, Co, D, H, W, cap, bits):
    L = G.L()
    S = D * H * W
    x = synth.rng(321).standard_normal(N * Ci * S).astype(np.float32)
    w, b = synth.kaiming(322, Co, Ci, 27), synth.bias(323, Co, 0.1)
    mx, want = orc.conv_case("conv3", x, w, b, N, Ci, D, H, W, Co, bits)
    xe = exact_operands(324, (N, Ci, D, H, W), 1).reshape(-1)
    we = exact_operands(325, (Co, Ci, 27), 1)
    mxe, wante = orc.conv_case("conv3", xe, we, None, N, Ci, D, H, W, Co, bits)
    L.umx_conv_r_block_cap(cap)
    try:
        got = run("conv3", mx, w, b, N, Ci, D, H, W, Co, bits)
        gote = run("conv3", mxe, we, None, N, Ci, D, H, W, Co, bits)
        # the InstanceNorm path through the same launch geometry
        c = G.Conv("conv3", w, b, Co, Ci, bits)
        raw, _ = c.fwd(mx, N, D, H, W, G.OUT_H16B)
        y, coef = c.fwd_norm(mx, N, D, H, W, epilogue_stats=True)
        assert L.umx_conv_last_kernel() == 1
        L.umx_conv_r_block_cap(0)
        y_free, coef_free = c.fwd_norm(mx, N, D, H, W, epilogue_stats=True)      # the same layer cut into as many blocks as the device holds
        same_kernel = L.umx_conv_last_kernel() == 1          # (a few of these grids then go to the general kernel: another summation order)
        c.free()
    finally:
        L.umx_conv_r_block_cap(0)
    e = orc.rel_l2(got, want)
    assert np.isfinite(got).all() and e < TOL, "relative L2 %.3g" % e
    assert np.array_equal(gote, wante), "%d of %d differ" % (np.count_nonzero(gote != wante), wante.size)
    assert np.array_equal(raw.view(np.uint16), y.view(np.uint16))
    assert np.array_equal(raw.view(np.float16), orc.pm_to_blocked(got, N, Co, S).astype(np.float16))
    # the epilogue's InstanceNorm sums: the oracle's fp64 statistics bit for bit, whatever the partition of the planes over blocks
    assert np.array_equal(coef, orc.in_coef(orc.in_sums(y.astype(np.float32), N, Co, S), N, Co, S))
    if same_kernel:
        assert np.array_equal(y_free.view(np.uint16), y.view(np.uint16)) and np.array_equal(coef, coef_free)
