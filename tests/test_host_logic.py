"""Host-side logic that needs no GPU, pinned to the NumPy oracle."""
import numpy as np
import torch

from oracle import np_oracle as O


def test_quant_weight_int8_equals_oracle_ternarize():
    """model.quant_weight_int8 (absmean ternarisation, gpu/convert_checkpoint.py:23-27) against
    np_oracle.ternarize: same ternary values, scale = bf16(1 / s); also the clamp at 1e-5."""
    from bitnet_b200.model import quant_weight_int8

    rng = np.random.default_rng(11)
    for shape, scale in [((384, 640), 1.0), ((640, 256), 0.02), ((128, 128), 50.0)]:
        w = (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)
        q_want, s_want = O.ternarize(w)
        q, s = quant_weight_int8(torch.from_numpy(w.copy()))
        assert np.array_equal(q.numpy(), q_want)
        assert s.dtype == torch.bfloat16 and s.shape == (1,)
        assert float(s.float()) == float(O.to_bf16(np.array([s_want], dtype=np.float32))[0])
        frac0 = float((q_want == 0).mean())
        assert 0.28 < frac0 < 0.35                      # P(|z| < 0.5 E|z|) for a normal z is 31 %
    w0 = np.zeros((16, 128), dtype=np.float32)          # mean |w| below the clamp
    q, s = quant_weight_int8(torch.from_numpy(w0))
    q_want, s_want = O.ternarize(w0)
    assert not q.any() and np.array_equal(q.numpy(), q_want)
    assert float(s.float()) == float(O.to_bf16(np.array([s_want], dtype=np.float32))[0]) == float(O.to_bf16(np.array([1e-5], dtype=np.float32))[0])


def test_plain_build_after_trace_build_is_stale(tmp_path, monkeypatch):
    """The library on disk may be the measurement build (phase time stamps compiled in): a plain
    build request must then rebuild instead of returning it as up to date."""
    from bitnet_b200 import build as b

    flavour = tmp_path / "flavour"
    monkeypatch.setattr(b, "FLAVOUR", str(flavour))
    flavour.write_text("plain")
    fresh = b.is_stale()            # whatever the time stamps say with a plain library on disk
    flavour.write_text("trace")
    assert b.is_stale()
    flavour.unlink()
    assert b.is_stale() == fresh    # no record: taken as plain
