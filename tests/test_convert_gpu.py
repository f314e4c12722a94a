"""Format producers beside the matmul path: dtype conversion and the int4 group quantiser. Bit-exact
against the CPU oracle."""
import numpy as np
import pytest

from beantensor_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def values(n, seed):
    # wide dynamic range plus the awkward points: zeros, subnormals of the narrow types, overflow, ties
    x = synth.normal((n,), 1.0, seed, 0) * np.exp(synth.uniform((n,), -30, 12, seed, 1))
    special = np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 6e-8, 2.98e-8, 1.0009765625, 1.00048828125, 1.00146484375,
                        -1.00048828125, 3.3e38, 1e-45, 1.00390625, 1.01171875])
    return np.concatenate([x, special]).astype(np.float32)


@pytest.mark.parametrize("dst", [_lib.F16, _lib.BF16])
def test_narrowing_is_bit_exact_rne(btm, oracle, dst):
    import torch
    x = values(100003, 5)
    td = {_lib.F16: torch.float16, _lib.BF16: torch.bfloat16}[dst]
    out = torch.empty(x.shape, dtype=td, device="cuda")
    btm.convert_gpu(torch.from_numpy(x).cuda(), out)
    got = out.cpu().view(torch.uint16).numpy()
    want = oracle.narrow(x.astype(np.float64), dst)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("src", [_lib.F16, _lib.BF16])
def test_widening_is_exact(btm, oracle, src):
    import torch
    bits = np.arange(0, 65536, dtype=np.uint16)  # every bit pattern
    ts = {_lib.F16: torch.float16, _lib.BF16: torch.bfloat16}[src]
    out = torch.empty(bits.shape, dtype=torch.float32, device="cuda")
    btm.convert_gpu(torch.from_numpy(bits).view(ts).cuda(), out)
    got = out.cpu().numpy()
    want = oracle.widen(bits, src).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_convert_rejects_other_dtypes(btm):
    import torch
    from beantensor_b200.errors import NotImplementedOp
    with pytest.raises(NotImplementedOp):
        btm.convert_gpu(torch.zeros(4, dtype=torch.int32, device="cuda"), torch.zeros(4, dtype=torch.float32, device="cuda"))


@pytest.mark.parametrize("case", [(64, 256, 128), (33, 512, 64), (11008, 4096, 128), (5, 64, 32)])
def test_quantiser_is_bit_exact_and_round_trips(btm, oracle, case):
    import torch
    N, K, group = case
    w = synth.normal((N, K), 0.02, 9 + N, 0).astype(np.float16)
    w[0, :group] = 0  # an all-zero group: scale falls back to 1
    if N > 2:
        w[2, 5] = 1.5  # an outlier that sets its group's scale
    packed = torch.empty((N, K // 2), dtype=torch.uint8, device="cuda")
    scales = torch.empty((N, K // group), dtype=torch.float16, device="cuda")
    btm.quantize_int4_gpu(torch.from_numpy(w).cuda(), packed, scales, group)
    want_p, want_s = oracle.int4_quantize(w.view(np.uint16), group)
    assert np.array_equal(scales.cpu().view(torch.uint16).numpy(), want_s)
    assert np.array_equal(packed.cpu().numpy(), want_p)
    # quantise -> dequantise stays within half a quantisation step of the input (the outlier's own group
    # included), and the produced format is what the matmul consumes
    deq = torch.empty((N, K), dtype=torch.float16, device="cuda")
    btm.dequant_int4_gpu(packed, scales, deq, group)
    step = np.repeat(scales.cpu().numpy().astype(np.float32), group, axis=1)
    err = np.abs(deq.cpu().numpy().astype(np.float32) - w.astype(np.float32))
    assert np.all(err <= 0.5 * step * 1.01 + 1e-6)
    act = synth.normal((2, K), 1.0, 3, 2).astype(np.float16)
    out = torch.empty((2, N), dtype=torch.float16, device="cuda")
    btm.matmul_int4_gpu(torch.from_numpy(act).cuda(), packed, scales, out, group)
    ref = oracle.int4_matmul(act.view(np.uint16), want_p, want_s, group)
    assert oracle.rel_frobenius(out.cpu().view(torch.uint16).numpy(), oracle.F16, ref) <= 2e-3
