"""The group quantiser and the QuantLinear module: CPU checks of the quantisation maths, a GPU check of the module."""
import numpy as np
import pytest
import torch

from int4matmul_kernels_b200 import packing, quantize
from oracle import reference_oracle as oracle


@pytest.mark.parametrize("bits,g", [(4, 128), (3, 64), (2, 64), (4, -1)])
def test_quantiser_error_is_within_half_a_step(bits, g):
    gen = torch.Generator().manual_seed(bits * 10 + 1)
    w = torch.randn((256, 128), generator=gen) * 0.05
    qz = quantize.quantize_groupwise(w, bits, g)
    assert qz["q"].max() <= (1 << bits) - 1 and qz["zeros"].eq(qz["zeros"].round()).all()
    w16 = quantize.dequantize(qz["q"], qz["scales"], qz["zeros"], g).float()
    gs = 256 if g < 0 else g
    step = qz["scales"].float().repeat_interleave(gs, dim=0)
    assert ((w16 - w).abs() <= 0.5 * step * 1.02 + 1e-3 * w.abs().max()).all()
    # the same tensors through the numpy oracle give the same fp16 weights bit for bit
    w_or = oracle.dequant_w16(bits, qz["q"].numpy(), qz["scales"].numpy(), qz["zeros"].numpy(), g)
    assert np.array_equal(w_or.view(np.uint16), quantize.dequantize(qz["q"], qz["scales"], qz["zeros"], g).numpy().view(np.uint16))


def test_sparse_quantiser_keeps_the_16_largest_of_every_32():
    w = torch.randn((128, 64), generator=torch.Generator().manual_seed(3))
    qz = quantize.quantize_groupwise(w, 4, 64, sparse=True)
    keep = qz["keep"].view(64, 4, 32)
    assert (keep.sum(dim=2) == 16).all()
    mag = w.abs().t().reshape(64, 4, 32)
    kept_min = torch.where(keep.bool(), mag, torch.full_like(mag, 1e9)).amin(dim=2)
    drop_max = torch.where(keep.bool(), torch.zeros_like(mag), mag).amax(dim=2)
    assert (kept_min >= drop_max).all()


def test_all_zero_group_quantises_to_exact_zeros():
    w = torch.randn((256, 128), generator=torch.Generator().manual_seed(5)) * 0.05
    w[64:128, :] = 0.0                      # a whole group of every column
    w[:, 7] = 0.0                           # a zero-padded column
    qz = quantize.quantize_groupwise(w, 4, 64)
    assert torch.isfinite(qz["scales"].float()).all() and (qz["scales"] > 0).all()
    w16 = quantize.dequantize(qz["q"], qz["scales"], qz["zeros"], 64)
    assert torch.isfinite(w16.float()).all()
    assert (w16[64:128, :] == 0).all() and (w16[:, 7] == 0).all()


def test_quantiser_rejects_bad_shapes():
    with pytest.raises(ValueError):
        quantize.quantize_groupwise(torch.zeros((100, 64)), 4, 64)
    with pytest.raises(ValueError):
        quantize.quantize_groupwise(torch.zeros((128, 64)), 3, 64, sparse=True)
    with pytest.raises(ValueError):
        quantize.quantize_groupwise(torch.zeros((128, 64)), 5, 64)


@pytest.mark.gpu
@pytest.mark.parametrize("bits,sparse", [(4, False), (4, True), (3, False), (2, False)])
def test_quant_linear_module(bits, sparse):
    from helpers import assert_parity
    gen = torch.Generator().manual_seed(17)
    w = torch.randn((512, 256), generator=gen) * 0.03
    lin = quantize.QuantLinear.from_float(w, bits, 64, sparse=sparse)
    for shape in ((1, 512), (2, 37, 512)):
        x = torch.randn(shape, generator=gen).to(torch.float16).cuda()
        y = lin(x)
        assert y.shape == shape[:-1] + (256,)
        qz = quantize.quantize_groupwise(w, bits, 64, sparse)
        w16 = quantize.dequantize(qz["q"], qz["scales"], qz["zeros"], 64, qz["keep"]).numpy()
        xs = x.reshape(1, -1, 512).cpu().numpy()
        want = oracle.matmul_ref(xs, w16)
        assert_parity(y.reshape(1, -1, 256).cpu().numpy(), want, oracle.matmul_abs_bound(xs, w16), "QuantLinear")
    # and the quantised layer stays close to the float layer: rounding to 2^bits levels over ~5 sigma of a group gives a
    # mean |error| of about 0.8 * sqrt(512) * 5 * 0.03 / ((2^bits - 1) * sqrt(12)) = 0.05 / 0.11 / 0.26 for 4 / 3 / 2 bits
    xf = torch.randn((8, 512), generator=gen)
    err = (lin(xf.to(torch.float16).cuda()).float().cpu() - xf @ (w if not sparse else w * qz["keep"].t().float())).abs().mean()
    assert err < {4: 0.08, 3: 0.16, 2: 0.4}[bits]
