"""The fused producer (QK-norm + RoPE + K/V store on the device) against the CPU checker.

The reference compiles this step with -Ofast (vectorised libm, free contraction), so the comparison is to rounding:
q within a few 1e-7 x position of the CPU rows, stored f16 K within one f16 unit in the last place, and the attention that follows
within the acceptance bar."""
import numpy as np
import pytest

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kvt,hd,gated,rd", [(2, 128, False, 128), (3, 128, False, 128), (2, 256, True, 64)])
def test_producer_then_attention(checker, port, kvt, hd, gated, rd):
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, n = 8, 2, 300
    qh = hd * (2 if gated else 1)
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=gated, max_rows=512)
    s = c.new_seq(n, kvt)
    q_raw = synth.normal(1, (n, n_heads, qh))
    k_raw = synth.normal(2, (n, n_kv, hd)) * np.float32(3.0)
    v_raw = synth.normal(3, (n, n_kv, hd))
    qw = (synth.normal(4, (hd,)) * np.float32(0.2) + np.float32(1.0)).astype(np.float32)
    kw = (synth.normal(5, (hd,)) * np.float32(0.2) + np.float32(1.0)).astype(np.float32)
    q_dev, k_dev, v_dev = c.to_device(q_raw), c.to_device(k_raw), c.to_device(v_raw)
    qw_dev, kw_dev = c.to_device(qw), c.to_device(kw)
    out_dev = c.malloc(n * n_heads * hd * 4)
    c.pass_begin([(s, 0, n)])
    c.qk_norm_rope_store_dev(0, q_dev, k_dev, v_dev, qw_dev, kw_dev, rd, 1e6)
    c.attn_decode_dev(0, q_dev, out_dev)
    q_gpu = np.empty_like(q_raw)
    out_gpu = np.empty((n, n_heads, hd), np.float32)
    c.d2h(q_gpu, q_dev)
    c.d2h(out_gpu, out_dev)
    c.sync()
    c.pass_end()
    pos = np.arange(n)
    q_cpu = checker.qk_norm_rope(q_raw, qw, hd, pos, 1e6, rd)
    k_cpu = checker.qk_norm_rope(k_raw, kw, hd, pos, 1e6, rd)
    # the rotation angle is pos * freq with freq from expf: a last-bit difference between the two expf grows with the position
    tol = 4e-7 * (pos[:, None, None] + 8) * float(np.abs(q_cpu).max())
    assert (np.abs(q_gpu - q_cpu)[:, :, :hd] <= tol).all(), float(np.abs(q_gpu - q_cpu).max())
    if gated:
        assert np.array_equal(q_gpu[:, :, hd:], q_raw[:, :, hd:])  # the gate half is untouched
    kl, vl = port.new_cache(kvt, 512, n_kv, hd)
    port.kv_store(kvt, kl, vl, 0, k_cpu, v_raw, n_kv, hd)
    gk, gv = s.read_kv(0, 0), s.read_kv(0, 1)
    if kvt == 2:
        kf_c, vf_c = port.block_f32(kvt, kl, vl, n_kv, hd, 1, 0, 16)
        kf_g, vf_g = port.block_f32(kvt, gk, gv, n_kv, hd, 1, 0, 16)
        assert np.array_equal(vf_c, vf_g)  # V is stored as given
        # one f16 unit in the last place, plus the fp32 difference of the rotation itself (grows with the position)
        assert (np.abs(kf_c - kf_g) <= np.abs(kf_c) * 2.0 ** -10 + 2e-3).all()
    # the attention on the device's cache and q equals the CPU attention on the CPU's cache and q within the bar
    want = checker.attention(kvt, kl, vl, n_kv, n_heads, hd, q_cpu, pos + 1, gated=gated)
    assert_close(out_gpu, want, f"producer + attention kvt={kvt}")
    c.close()
