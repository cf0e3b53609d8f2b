"""The tcgen05 matrix product alone against a float32 product of the same bfloat16 inputs:
every epilogue, token counts on both sides of every tile size, widths that are no multiple of
the tile, with and without split-K."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16)


def rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max()) / max(float(b.abs().max()), 1e-30)


SHAPES = [(1, 128, 64), (8, 384, 200), (16, 100, 72), (17, 3072, 2048), (64, 2048, 2048), (100, 640, 520),
          (128, 256, 8192), (300, 1000, 264), (1, 128256, 256), (8, 2048, 8192), (600, 512, 1024)]


@pytest.mark.parametrize("T,N,K", SHAPES)
@pytest.mark.parametrize("split", [True, False])
def test_tc_gemm_epilogues(T, N, K, split):
    from rllm_b200.kernels import ops, sm100
    x, w = rnd(T, K, seed=1), rnd(2 * N, K, seed=2, scale=K ** -0.5)
    xd, wd = x.to(DEV), w.to(DEV)
    w1 = wd[:N].contiguous()
    ref = x.float() @ w[:N].float().t()
    up = x.float() @ w[N:].float().t()
    assert rel(sm100.gemm(xd, w1, ops.EPI_STORE, split=split), ref) <= 6e-3
    out32 = sm100.gemm(xd, w1, ops.EPI_STORE_F32, split=split)
    assert out32.dtype == torch.float32 and rel(out32, ref) <= 2e-5
    res = torch.randn(T, N, generator=torch.Generator().manual_seed(3))
    got = sm100.gemm(xd, w1, ops.EPI_ACCUM_F32, out=res.to(DEV).clone(), split=split)
    assert rel(got, res + ref) <= 2e-5
    want = ref / (1 + torch.exp(-ref)) * up
    assert rel(sm100.gemm(xd, wd, ops.EPI_SWIGLU, split=split), want) <= 6e-3
    sm100.check_error(DEV)
    # the same call again gives the same bits (split-K sums in split order, counters reset)
    again = sm100.gemm(xd, w1, ops.EPI_STORE_F32, split=split)
    assert torch.equal(again, out32)


def test_tc_gemm_takes_a_strided_view_and_refuses_misfits():
    from rllm_b200.kernels import ops, sm100
    big = rnd(40, 3 * 128, seed=5).to(DEV)
    x = big[:, 128:256]                                   # row stride 384, offset 256 bytes
    w = rnd(96, 128, seed=6).to(DEV)
    assert rel(sm100.gemm(x, w, ops.EPI_STORE_F32), x.float().cpu() @ w.float().cpu().t()) <= 2e-5
    assert not sm100.gemm_supported(rnd(4, 100).to(DEV), rnd(8, 100).to(DEV))      # K % 8
    assert not sm100.gemm_supported(big[:, 1:129], w)                               # misaligned
    with pytest.raises(ops.KernelError):
        sm100.gemm(rnd(4, 100).to(DEV), rnd(8, 100).to(DEV), ops.EPI_STORE)


def test_plan_splits_small_batches_only():
    from rllm_b200.kernels import ops, sm100
    assert sm100.plan(ops.EPI_STORE, 8, 3072, 2048) == (16, 13) or sm100.plan(ops.EPI_STORE, 8, 3072, 2048)[1] > 1
    assert sm100.plan(ops.EPI_STORE, 2048, 3072, 2048) == (256, 1)
    assert sm100.plan(ops.EPI_SWIGLU, 2048, 8192, 2048) == (128, 1)
