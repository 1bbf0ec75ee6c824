"""torch.library registration, in-place semantics, the gradient for B and the CsrMatrix holder."""
import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import generators as G, torch_library as TL


def _t(p):
    return [torch.from_numpy(x) for x in (p.row_ptr, p.col_idx, p.values, p.B)]


def test_transpose_csr_matches_dense_transpose():
    p = G.random_csr(37, 23, 4, 0.2, seed=3)
    rp, ci, va, _ = _t(p)
    trp, tci, tva = TL.transpose_csr(rp, ci, va, p.Kd)
    A = oracle.csr2dense(p.M, p.Kd, p.row_ptr, p.col_idx, p.values)
    At = oracle.csr2dense(p.Kd, p.M, trp.numpy(), tci.numpy(), tva.numpy())
    assert np.array_equal(At, A.T)
    assert trp.dtype == torch.int32 and tci.dtype == torch.int32 and int(trp[-1]) == p.nnz
    # ascending rows inside each column
    for k in range(p.Kd):
        seg = tci[trp[k]:trp[k + 1]].numpy()
        assert (np.diff(seg) > 0).all()


def test_fake_implementation_traces_without_a_gpu():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        out = torch.ops.csrspmm_b200.spmm(torch.empty(14, dtype=torch.int32, device="cuda"),
                                          torch.empty(30, dtype=torch.int32, device="cuda"),
                                          torch.empty(30, device="cuda"), torch.empty(9, 4, device="cuda"), 1.0, "auto")
        assert out.shape == (13, 4) and out.dtype == torch.float32


@pytest.mark.gpu
def test_registered_ops_and_inplace_semantics(cuda_lib):
    p = G.random_csr(200, 150, 64, 0.05, seed=4)
    rp, ci, va, B = (x.cuda() for x in _t(p))
    want = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, None, 1.5, 0.0)
    got = torch.ops.csrspmm_b200.spmm(rp, ci, va, B, 1.5, "auto")
    assert np.allclose(got.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    C0 = np.random.default_rng(1).standard_normal((p.M, p.Nd), dtype=np.float32)
    C = torch.from_numpy(C0).cuda()
    torch.ops.csrspmm_b200.spmm_(rp, ci, va, B, C, 2.0, -0.5, "merge")  # the reference's full alpha/beta form
    want2 = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, C0, 2.0, -0.5)
    assert np.allclose(C.cpu().numpy(), want2, rtol=1e-5, atol=2e-6)
    torch.library.opcheck(torch.ops.csrspmm_b200.spmm, (rp, ci, va, B, 1.0, "row"),
                          test_utils=("test_schema", "test_faketensor"))


@pytest.mark.gpu
def test_gradient_for_b_and_csr_matrix(cuda_lib):
    p = G.make("cfg3_powerlaw", scale=256, Nd=32)
    rp, ci, va, B = (x.cuda() for x in _t(p))
    A_dense = torch.from_numpy(oracle.csr2dense(p.M, p.Kd, p.row_ptr, p.col_idx, p.values)).cuda().double()
    W = torch.randn(p.M, p.Nd, device="cuda", generator=torch.Generator("cuda").manual_seed(0))

    Bg = B.clone().requires_grad_(True)
    out = torch.ops.csrspmm_b200.spmm(rp, ci, va, Bg, 0.75, "auto")
    (out * W).sum().backward()
    want_dB = 0.75 * (A_dense.T @ W.double())
    assert torch.allclose(Bg.grad.double(), want_dB, rtol=1e-4, atol=1e-4)

    A = TL.CsrMatrix(rp, ci, va, (p.M, p.Kd), validate=True)
    assert A.max_row_nnz == int(np.diff(p.row_ptr).max()) and A.nnz == p.nnz
    Bg2 = B.clone().requires_grad_(True)
    out2 = A.matmul(Bg2, 0.75)
    # the holder knows the longest row, so AUTO may pick another kernel: same product, other summation order
    assert torch.allclose(out2, out.detach(), rtol=1e-4, atol=1e-5)
    (out2 * W).sum().backward()
    assert torch.allclose(Bg2.grad.double(), want_dB, rtol=1e-4, atol=1e-4)
    assert A.t().t() is A and A.t().shape == (p.Kd, p.M)
    # out= / beta form through the holder
    C = torch.ones(p.M, p.Nd, device="cuda")
    A.matmul(B, 1.0, out=C, beta=2.0)
    assert torch.allclose(C, out.detach() / 0.75 + 2.0, rtol=1e-4, atol=1e-4)
    with pytest.raises(RuntimeError, match="no gradient for the stored values"):
        vg = va.clone().requires_grad_(True)
        torch.ops.csrspmm_b200.spmm(rp, ci, vg, B.clone().requires_grad_(True), 1.0, "auto").sum().backward()
