"""Parity of the CUDA Gated DeltaNet recurrence with the CPU checker (bit for bit: same operation order)."""
import numpy as np
import pytest

from tests.helpers import assert_close, bit_equal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nk,nv", [(2, 2), (2, 4)])
def test_recurrence_matches_cpu(checker, nk, nv):
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    dk = dv = 128
    c = g.Context(0, n_lin=2, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, max_rows=256)
    d = gwo.DeltaNet(checker, nk, nv, dk, dv)
    rows_a = synth.deltanet_rows(1, 150, nk, nv, dk, dv)
    rows_b = synth.deltanet_rows(2, 40, nk, nv, dk, dv)
    # DeltaNet-only contexts have no attention layers: sequences carry the state only
    sa, sb = c.new_seq(512, 2), c.new_seq(512, 2)
    st_a, st_b = d.new_state(), d.new_state()
    # pass 1: a 100-row chunk of a and the 40 rows of b, both from position 0
    c.pass_begin([(sa, 0, 100), (sb, 0, 40)])
    got = c.dn_rec(1, np.concatenate([rows_a[:100], rows_b]))
    c.pass_end()
    want_a, want_b = d.rec(st_a, rows_a[:100], True), d.rec(st_b, rows_b, True)
    assert_close(got[:100], want_a, "dn chunk a")
    assert bit_equal(got[:100], want_a) and bit_equal(got[100:], want_b)
    # pass 2: a continues with 49 rows, then a single decode row
    c.pass_begin([(sa, 100, 49)])
    got2 = c.dn_rec(1, rows_a[100:149])
    c.pass_end()
    c.pass_begin([(sa, 149, 1)])
    got3 = c.dn_rec(1, rows_a[149:150])
    c.pass_end()
    want2 = d.rec(st_a, rows_a[100:149], False)
    want3 = d.rec(st_a, rows_a[149:150], False)
    assert bit_equal(got2, want2) and bit_equal(got3, want3)
    assert bit_equal(sa.read_state(1)[d.conv_floats:], st_a[d.conv_floats:])
    assert not sa.read_state(0).any()  # the other layer's state is untouched
    c.close()
