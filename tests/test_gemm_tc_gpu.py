"""tcgen05/TMEM GEMM (rg_b200_mat_mul with force_kernel = 3 and the automatic route) against the oracle.
fp16/bf16 operands, fp32 accumulation: max-abs 2e-2 / relative 1e-2 against fp64 on the rounded inputs; exact on
small-integer data.  Large cases use a torch fp32 matmul of the same rounded inputs as the reference."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200 import capi

import _ops as ops

pytestmark = pytest.mark.gpu
HALF = [torch.float16, torch.bfloat16]


def _ok():
    return capi.load().rg_b200_error_state() == 0


def test_smallest_tile_exact():
    # one 128x128 tile, one k-block, integer data: exact in fp32 accumulation
    rng = np.random.default_rng(0)
    a = rng.integers(-3, 4, (128, 64)).astype(np.float32)
    b = rng.integers(-3, 4, (128, 64)).astype(np.float32)
    y = ops.mat_mul(ops.dev(a).half(), ops.dev(b).half(), trans_b=True, force=3)
    assert _ok(), "a bounded wait expired inside the tensor-core kernel"
    np.testing.assert_array_equal(y.float().cpu().numpy(), a @ b.T)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 1024), (100, 300, 72), (129, 257, 4096), (512, 128, 256), (64, 64, 64)])
def test_against_numpy_oracle(dtype, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
    b = torch.from_numpy((0.05 * rng.standard_normal((n, k))).astype(np.float32)).to(dtype)
    y = ops.mat_mul(a.cuda(), b.cuda(), trans_b=True, force=3)
    assert _ok()
    want = onp.mat_mul(a.float().numpy(), b.float().numpy(), trans_b=True)
    np.testing.assert_allclose(y.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("m,n,k", [(512, 256, 64), (1024, 768, 512), (600, 300, 200), (513, 1000, 4096), (2050, 256, 1032)])
def test_pairs_of_ctas(dtype, m, n, k):
    """512 rows and 256 columns or more: two CTAs share a 256 x 256 tile (tcgen05 ... cta_group::2), ragged edges included;
    with a residual, alpha and beta; the second call must give the same bits."""
    rng = np.random.default_rng(m * 7 + n + k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype)
    b = torch.from_numpy((0.05 * rng.standard_normal((n, k))).astype(np.float32)).to(dtype)
    c = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(dtype)
    y = ops.mat_mul(a.cuda(), b.cuda(), trans_b=True, force=3)
    assert _ok()
    want = onp.mat_mul(a.float().numpy(), b.float().numpy(), trans_b=True)
    np.testing.assert_allclose(y.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)
    y2 = ops.mat_mul(a.cuda(), b.cuda(), c.cuda(), trans_b=True, alpha=0.5, beta=2.0, force=3)
    assert _ok()
    want2 = onp.mat_mul(a.float().numpy(), b.float().numpy(), c.float().numpy(), trans_b=True, alpha=0.5, beta=2.0)
    np.testing.assert_allclose(y2.float().cpu().numpy(), want2, atol=4e-2, rtol=1e-2)
    assert torch.equal(y, ops.mat_mul(a.cuda(), b.cuda(), trans_b=True, force=3))


@pytest.mark.parametrize("dtype", HALF)
def test_pairs_of_ctas_bias_vector_and_batch(dtype):
    """The pair kernel behind the batched call with a broadcast bias row (element-wise loads of C)."""
    rng = np.random.default_rng(11)
    a = torch.from_numpy(rng.standard_normal((2, 520, 128)).astype(np.float32)).to(dtype)
    b = torch.from_numpy((0.1 * rng.standard_normal((2, 264, 128))).astype(np.float32)).to(dtype)
    c = torch.from_numpy(rng.standard_normal((264,)).astype(np.float32)).to(dtype)
    y = ops.mat_mul(a.cuda(), b.cuda(), c.cuda(), trans_b=True, alpha=0.5, beta=2.0, force=3)
    assert _ok()
    want = onp.mat_mul(a.float().numpy(), b.float().numpy(), c.float().numpy(), trans_b=True, alpha=0.5, beta=2.0)
    np.testing.assert_allclose(y.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", HALF)
def test_alpha_beta_bias_and_batch(dtype):
    rng = np.random.default_rng(7)
    a = torch.from_numpy(rng.standard_normal((3, 130, 128)).astype(np.float32)).to(dtype)
    b = torch.from_numpy((0.1 * rng.standard_normal((3, 200, 128))).astype(np.float32)).to(dtype)
    c = torch.from_numpy(rng.standard_normal((200,)).astype(np.float32)).to(dtype)
    y = ops.mat_mul(a.cuda(), b.cuda(), c.cuda(), trans_b=True, alpha=0.5, beta=2.0, force=3)
    assert _ok()
    want = onp.mat_mul(a.float().numpy(), b.float().numpy(), c.float().numpy(), trans_b=True, alpha=0.5, beta=2.0)
    np.testing.assert_allclose(y.float().cpu().numpy(), want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (32, 11008, 4096), (64, 4096, 11008), (5, 1000, 512)])
def test_skinny_swapped_operands(dtype, m, n, k):
    rng = np.random.default_rng(m * n)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype).cuda()
    b = torch.from_numpy((0.02 * rng.standard_normal((n, k))).astype(np.float32)).to(dtype).cuda()
    y = ops.mat_mul(a, b, trans_b=True, force=3)
    assert _ok()
    want = a.float() @ b.float().T
    torch.testing.assert_close(y.float(), want, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("m,n,k,residual", [(16, 22016, 4096, False), (32, 32000, 4096, True), (8, 20000, 4104, False)])
def test_skinny_stream_k(dtype, m, n, k, residual):
    """Skinny products with at least 64 k-blocks per SM run in stream-K mode: every CTA owns one contiguous run of
    (tile, k-block) units and tiles that span CTAs are summed by the last to arrive.  The last case has a ragged last
    row tile and a partial last k-block."""
    rng = np.random.default_rng(m + n + k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dtype).cuda()
    b = torch.from_numpy((0.02 * rng.standard_normal((n, k))).astype(np.float32)).to(dtype).cuda()
    want = a.float() @ b.float().T
    if residual:
        c = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(dtype).cuda()
        y = ops.mat_mul(a, b, c=c, trans_b=True, force=3)
        want = want + c.float()
    else:
        y = ops.mat_mul(a, b, trans_b=True, force=3)
    assert _ok()
    torch.testing.assert_close(y.float(), want, atol=2e-2, rtol=1e-2)
    y2 = ops.mat_mul(a, b, c=c, trans_b=True, force=3) if residual else ops.mat_mul(a, b, trans_b=True, force=3)
    assert torch.equal(y, y2)          # fixed summation order: a second call gives the same bits


@pytest.mark.parametrize("dtype", HALF)
def test_prefill_sized_and_auto_route(dtype):
    torch.backends.cuda.matmul.allow_tf32 = False
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(2048, 4096, device="cuda", generator=g).to(dtype)
    b = (0.02 * torch.randn(4096 + 256, 4096, device="cuda", generator=g)).to(dtype)
    y = ops.mat_mul(a, b, trans_b=True)            # automatic route must pick the tensor-core kernel
    assert _ok()
    want = a.float() @ b.float().T
    torch.testing.assert_close(y.float(), want, atol=2e-2, rtol=1e-2)
    # linearity, a size-independent property: (2A) B^T = 2 (A B^T), exact except where the 16-bit result is subnormal
    y2 = ops.mat_mul((a * 2).to(dtype), b, trans_b=True)
    torch.testing.assert_close(y2.float(), 2 * y.float(), atol=1e-6, rtol=2e-3)
