"""The row kernel's grid rule, as pure arithmetic (no device): how many CTAs an n-row matrix is launched with."""
import pytest

import demonic_b200 as dmc

SMS, CPS, WARPS = 148, 2, 8          # B200: 148 SMs, 2 resident CTAs of the default configuration, 8 warps each


def grid(n, r=2, reserve=0, rule=1, warps=WARPS):
    return dmc.load().dmc_cuda_row_kernel_grid(n, warps, r, SMS, CPS, reserve, rule)


def groups_per_warp(n, r, ctas, warps=WARPS):
    """(min, max) row groups a warp owns when `ctas` CTAs take contiguous, equal blocks of the groups."""
    groups = -(-n // r)
    lo, hi = 10 ** 9, 0
    for b in range(ctas):
        g0, g1 = groups * b // ctas, groups * (b + 1) // ctas
        for w in range(warps):
            own = len(range(g0 + w, g1, warps))
            lo, hi = min(lo, own), max(hi, own)
    return lo, hi


def test_one_group_per_warp_while_that_fits():
    assert grid(4096) == 256                       # 2048 groups of two rows, 8 per CTA
    assert grid(2048, r=1) == 256
    assert grid(1) == 1
    assert grid(16 * SMS * CPS) == SMS * CPS       # exactly every slot
    for rule in (0, 1, 2):
        assert grid(4096, rule=rule) == 256


@pytest.mark.parametrize("n,want,per_warp", [
    (14336, 224, (4, 4)),                          # 3 % of the warps would own a 4th group: equal shares instead
    (6144, 192, (2, 2)),                           # the fused q/k/v projection of the decode step
    (11264, 235, (2, 3)),                          # gate/up: 5632 groups over 235 x 8 warps, three each but for a few
    (11008, 230, (2, 3)),
])
def test_few_warps_with_an_extra_group_get_equal_shares_instead(n, want, per_warp):
    ctas = grid(n)
    assert ctas == want and ctas <= SMS * CPS
    assert groups_per_warp(n, 2, ctas) == per_warp
    assert grid(n, rule=0) == SMS * CPS            # the knob's other positions
    assert grid(n, rule=2) == want


@pytest.mark.parametrize("n", [8192, 32000, 65536])
def test_many_warps_with_an_extra_group_keep_every_slot(n):
    assert grid(n) == SMS * CPS
    lo, hi = groups_per_warp(n, 2, SMS * CPS)
    assert hi - lo <= 1
    forced = grid(n, rule=2)
    assert forced <= SMS * CPS
    assert groups_per_warp(n, 2, forced)[1] == -(-(-(-n // 2)) // (SMS * CPS * WARPS))   # nobody owns more than `rounds`


def test_the_sharded_path_keeps_room_for_its_arrival_check():
    for n in (8192, 16384, 32768):                 # a rank's rows of the 65536-row matrix at 8, 4, 2 GPUs
        assert grid(n, reserve=4) <= SMS * CPS - 4
    assert grid(8192, reserve=4) == 292 and grid(16384, reserve=4) == 292
    assert grid(32768, reserve=4) == 256           # 8 groups per warp exactly
    assert grid(4096, reserve=4) == 256            # fits anyway


def test_refuses_nonsense():
    lib = dmc.load()
    assert lib.dmc_cuda_row_kernel_grid(0, 8, 2, 148, 2, 0, 1) == 0
    assert lib.dmc_cuda_row_kernel_grid(4096, 0, 2, 148, 2, 0, 1) == 0
    assert lib.dmc_cuda_row_kernel_grid(4096, 8, 2, 148, 2, -1, 1) == 0
