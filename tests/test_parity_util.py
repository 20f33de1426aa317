"""The local error bound of the GPU parity tests catches what the whole-tensor bound misses (CPU only)."""
import numpy as np

from parity_util import FRO_TOL, LOCAL_TOL, block_rel_fro, check_close, rel_fro


def test_one_wrong_row_passes_frobenius_but_fails_the_block_bound():
    rng = np.random.default_rng(0)
    ref = rng.standard_normal((4096, 512))
    got = ref * (1 + 1e-3 * rng.standard_normal(ref.shape))      # rounding-sized noise everywhere
    assert rel_fro(got, ref) < 2e-3 and block_rel_fro(got, ref)[0] < LOCAL_TOL
    got[1234, :] = 0.0                                           # one lost row
    assert rel_fro(got, ref) <= FRO_TOL                          # the contract bound does not see it
    w, at = block_rel_fro(got, ref)
    assert w > 10 * LOCAL_TOL and at[0] == 1234 // 128
    try:
        check_close("t", got, ref)
    except AssertionError as e:
        assert "block" in str(e)
    else:
        raise AssertionError("a lost row must fail the local bound")


def test_zero_blocks_and_ragged_edges():
    ref = np.zeros((130, 200)); ref[:, :64] = 1.0
    got = ref.copy()
    assert block_rel_fro(got, ref)[0] == 0.0
    got[129, 199] = 0.5                                          # garbage in an all-zero corner block
    assert block_rel_fro(got, ref)[0] > LOCAL_TOL
    v = np.arange(10.0)
    assert block_rel_fro(v, v)[0] == 0.0                         # 1-D input
