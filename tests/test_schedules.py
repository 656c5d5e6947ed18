import pytest

from sample_efficient_gpt_b200.optim import get_cosine_lr, get_seesaw_lr, get_wsd_lr, muon_momentum_warmup

# golden values produced by the reference's schedule functions (training/optimizer.py:115-187)


def test_wsd_stable():
    f = lambda t, nw=True: get_wsd_lr(t, 0.011, 0.00011, 500, 2500, 0, 0, nw, "stable")
    for t, want in [(0, 0.0), (499, 0.0), (500, 0.0), (1750, 0.0055), (2999, 0.0109956), (3000, 0.011), (50000, 0.011)]:
        assert f(t) == pytest.approx(want, rel=1e-6, abs=1e-12)
    assert f(0, False) == 0.011


def test_wsd_decay():
    f = lambda t: get_wsd_lr(t, 0.0115, 0.002875, 0, 1000, 100000, 100000, False, "decay")
    for t, want in [(100000, 0.0115), (125000, 0.0071875), (150000, 0.005401204), (199999, 0.002875043)]:
        assert f(t) == pytest.approx(want, rel=1e-6)


def test_cosine_and_seesaw():
    for t, want in [(0, 0.0), (50, 0.005), (100, 0.01), (550, 0.00505), (999, 0.00010003), (1000, 0.0001), (5000, 0.0001)]:
        assert get_cosine_lr(t, 1e-2, 1e-4, 100, 1000) == pytest.approx(want, rel=1e-4, abs=1e-12)
    for t, want in [(50, 0.005), (500, 0.01), (1000, 0.00707107), (1500, 0.00707107), (2000, 0.005), (3000, 0.005)]:
        assert get_seesaw_lr(t, 1e-2, 100, [1000, 2000]) == pytest.approx(want, rel=1e-6)


def test_momentum_warmup():
    assert muon_momentum_warmup(0, 0.95) == pytest.approx(0.85 + 1 / 300 * 0.1)
    assert muon_momentum_warmup(150, 0.95) == pytest.approx(0.90)
    assert muon_momentum_warmup(300, 0.95) == 0.95
