import numpy as np

from beantensor_b200 import synth


def test_counter_based_and_split_independent():
    a = synth.normal((64, 32), 0.125, 7, 3)
    b = synth.normal((2048,), 0.125, 7, 3).reshape(64, 32)
    assert np.array_equal(a, b)
    assert not np.array_equal(a, synth.normal((64, 32), 0.125, 8, 3))
    assert not np.array_equal(a, synth.normal((64, 32), 0.125, 7, 4))


def test_distributions():
    x = synth.normal((512, 512), 1 / 64, 1)
    assert abs(x.std() * 64 - 1) < 0.01 and abs(x.mean()) < 1e-3
    u = synth.uniform((512, 512), 0.005, 0.02, 2, 1)
    assert u.min() >= 0.005 and u.max() < 0.02
    w = synth.int4((256, 256), 2)
    assert w.min() == -8 and w.max() == 7
    counts = np.bincount(w.ravel().astype(np.int64) + 8, minlength=16)
    assert counts.min() > 0.8 * counts.mean()


def test_pack_layout():
    w = np.array([[-8, 7, 1, -1]], dtype=np.int8)
    p = synth.pack_int4(w)
    assert p.tolist() == [[0x78, 0xF1]]  # even k in bits 0-3, odd k in bits 4-7


def test_bf16_rne():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e38, 1e-40], dtype=np.float32)
    import torch
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(synth.to_bf16_bits(x), want)
