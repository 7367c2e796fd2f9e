"""CPU: the row-chunk planner of the host-buffer MLP call (b200fc_mlp_host_plan, a pure host function of the C ABI).
The plan decides which rows every launch and copy of b200fc_mlp_run_host covers, so its invariants are checked here:
both lists cover the M rows exactly once, in whole tiles of 256 rows except for the last entry, short chunks at the
head of gate/up and at the tail of down for large batches."""
import pytest

from mm_amx_b200 import capi

SHAPES = [(4096, 8192, 28672), (2048, 4096, 11008), (512, 4096, 11008), (513, 4096, 11008), (1000, 4096, 11008),
          (2300, 256, 512), (100000, 4096, 14336), (700, 256, 512), (16, 4096, 11008), (1, 8, 8)]


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_plan_covers_the_rows_once(M, K, N):
    gu, dn = capi.mlp_host_plan(M, K, N)
    for lst in (gu, dn):
        assert sum(lst) == M and all(r > 0 for r in lst)
        assert all(r % 256 == 0 for r in lst[:-1])
    # every down chunk finds its rows' gate/up launches issued before it: prefix sums of gate/up reach each boundary
    assert len(gu) <= (M + 255) // 256 and len(dn) <= (M + 255) // 256


def test_large_batches_start_and_end_with_short_chunks():
    gu, dn = capi.mlp_host_plan(4096, 8192, 28672)
    assert gu[0] <= 512 and dn[-1] <= 512 and max(gu) >= 1024 and max(dn) >= 1024
    # no down chunk of the Llama-70B shape leaves a nearly empty last round: 7 row tiles x 32 column tiles = 224 tiles
    # on 74 CTA pairs would be 3.03 rounds
    assert 7 * 256 not in dn
    gu, dn = capi.mlp_host_plan(100000, 4096, 14336)
    assert gu[0] <= 1024 and dn[-1] <= 1024 and len(gu) < 64 and len(dn) < 64


def test_bad_arguments_are_refused():
    with pytest.raises(capi.B200FCError):
        capi.mlp_host_plan(0, 4096, 11008)
    with pytest.raises(capi.B200FCError):
        capi.mlp_host_plan(100000, 4096, 14336, capacity=4)
