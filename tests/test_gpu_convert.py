"""Device-side dense <-> CSR conversion against the oracle's restatement of the reference's host
dense2csr / csr2dense (src/host/csr_utils.cpp:70-145): indices and values bit for bit."""
import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import ops

pytestmark = pytest.mark.gpu


def _random_dense(H, W, keep, seed):
    rng = np.random.default_rng(seed)
    d = rng.uniform(-1, 1, (H, W)).astype(np.float32)
    d[rng.random((H, W)) > keep] = 0.0
    return d


@pytest.mark.parametrize("H,W,keep,tol", [(1, 1, 1.0, 0.0), (7, 5, 0.5, 0.0), (64, 33, 0.3, 0.0), (300, 1000, 0.02, 0.0),
                                           (129, 4097, 0.1, 0.25), (2050, 3000, 0.004, 0.0), (50, 70, 0.0, 0.0)])
def test_dense2csr_and_back(cuda_lib, H, W, keep, tol):
    d = _random_dense(H, W, keep, H * 31 + W)
    rp, ci, va, mx = ops.dense2csr(torch.from_numpy(d).cuda(), tol)
    orp, oci, ova, omx = oracle.dense2csr(d, tol)
    assert np.array_equal(rp.cpu().numpy(), orp) and mx == omx
    assert np.array_equal(ci.cpu().numpy(), oci) and np.array_equal(va.cpu().numpy(), ova)
    back = ops.csr2dense(rp, ci, va, (H, W)).cpu().numpy()
    assert np.array_equal(back, oracle.csr2dense(H, W, orp, oci, ova))
    if tol == 0.0:
        assert np.array_equal(back, d)  # the round trip the reference's stale test intends


def test_strided_input_and_large_rows(cuda_lib):
    d = _random_dense(40, 200, 0.4, 9)
    wide = torch.zeros(40, 256, device="cuda")
    wide[:, 8:208] = torch.from_numpy(d).cuda()
    rp, ci, va, mx = ops.dense2csr(wide[:, 8:208])
    orp, oci, ova, omx = oracle.dense2csr(d)
    assert np.array_equal(rp.cpu().numpy(), orp) and np.array_equal(ci.cpu().numpy(), oci) and mx == omx
    # more rows than one scan block, and a product through the converted matrix
    d = _random_dense(5000, 600, 0.01, 10)
    rp, ci, va, mx = ops.dense2csr(torch.from_numpy(d).cuda())
    orp, oci, ova, _ = oracle.dense2csr(d)
    assert np.array_equal(rp.cpu().numpy(), orp) and np.array_equal(ci.cpu().numpy(), oci)
    B = np.random.default_rng(1).standard_normal((600, 32), dtype=np.float32)
    out = ops.spmm(rp, ci, va, torch.from_numpy(B).cuda(), max_row_nnz=mx, sync=True)
    assert np.array_equal(out.cpu().numpy(), oracle.spmm(orp, oci, ova, B))  # row kernel: bit-exact


def test_csr2dense_repeated_column_keeps_last_value(cuda_lib):
    rp = torch.tensor([0, 3, 3], dtype=torch.int32, device="cuda")
    ci = torch.tensor([2, 0, 2], dtype=torch.int32, device="cuda")
    va = torch.tensor([1.0, 5.0, 7.0], device="cuda")
    out = ops.csr2dense(rp, ci, va, (2, 4)).cpu().numpy()
    assert out.tolist() == [[5.0, 0.0, 7.0, 0.0], [0.0, 0.0, 0.0, 0.0]]


def test_e2m1_device_codec_equals_host_codec(cuda_lib):
    """Scale, codes and decoded values of the device codec equal the host codec's bit for bit: random values,
    exact ties at every midpoint, saturation, signed zeros, NaN, an odd element count."""
    rng = np.random.default_rng(12)
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    special = np.concatenate([mids, -mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(9)),
                              [0.0, -0.0, 6.0, -6.0, 5.999, np.nan, 1e-30, -1e-30]]).astype(np.float32)
    # the largest magnitude is 6, so scale is exactly 1 and the special values sit exactly on the ties
    v = np.concatenate([special, rng.uniform(-6.0, 6.0, 100_001).astype(np.float32)])
    assert v.shape[0] % 2 == 1
    h_packed, h_scale = ops.e2m1_quantize(v)
    d_packed, d_scale = ops.e2m1_quantize(torch.from_numpy(v).cuda())
    assert d_packed.is_cuda and d_scale == h_scale == 1.0
    assert torch.equal(d_packed.cpu(), h_packed)
    h_dec = ops.e2m1_dequantize(h_packed, v.shape[0], h_scale)
    d_dec = ops.e2m1_dequantize(d_packed, v.shape[0], d_scale)
    assert d_dec.is_cuda and np.array_equal(d_dec.cpu().numpy().view(np.uint32), h_dec.numpy().view(np.uint32))
    # a scale that is not a power of two, all-zero input, empty input
    w = rng.standard_normal(4097).astype(np.float32) * 3.3
    hp, hs = ops.e2m1_quantize(w)
    dp, ds = ops.e2m1_quantize(torch.from_numpy(w).cuda())
    assert ds == hs and torch.equal(dp.cpu(), hp)
    zp, zs = ops.e2m1_quantize(torch.zeros(10, device="cuda"))
    assert zs == 1.0 and int(zp.sum()) == 0
    ep, es = ops.e2m1_quantize(torch.zeros(0, device="cuda"))
    assert ep.numel() == 0 and es == 1.0
