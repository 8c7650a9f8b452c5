"""Tensor-core operand conventions: one CTA multiplies small tiles through the
same UMMA descriptors the attention kernels use (K-major and MN-major row
tiles, K-major and MN-major square tiles, an A operand in tensor memory), checked against a CPU GEMM."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D", [32, 64, 128])
def test_mma_operand_layouts(D):
    import _evoattn
    g = torch.Generator().manual_seed(7 + D)
    x = torch.randn((128, 128), generator=g).to(torch.bfloat16)
    y = torch.randn((128, D), generator=g).to(torch.bfloat16)
    z = torch.randn((128, D), generator=g).to(torch.bfloat16)
    dev = "cuda"
    xd, yd, zd = x.to(dev), y.to(dev), z.to(dev)
    o0 = torch.full((128, 128), float("nan"), device=dev)
    o1 = torch.full((128, D), float("nan"), device=dev)
    o2 = torch.full((128, D), float("nan"), device=dev)
    o3 = torch.full((128, D), float("nan"), device=dev)
    _evoattn.selftest_mma(D, xd, yd, zd, o0, o1, o2, o3, torch.cuda.current_stream().cuda_stream)
    _evoattn.device_status()
    xf, yf, zf = x.double(), y.double(), z.double()
    refs = {"y z^T": (yf @ zf.T, o0), "x y": (xf @ yf, o1), "x^T y": (xf.T @ yf, o2),
            "x y (A in tensor memory)": (xf @ yf, o3)}
    for name, (ref, got) in refs.items():
        err = (ref - got.double().cpu()).abs().max().item()
        # bf16 products are exact in fp32; only the accumulation order differs
        assert err < 1e-3, f"D={D} {name}: max abs err {err}"


@pytest.mark.parametrize("D", [32, 64, 128])
def test_extra_contraction_block(D):
    """y z^T + a b^T with a, b as [128][8] extra tiles (un-swizzled 16-byte rows, second half of the
    contraction block read from a zero tile): the form in which the backward kernels add the mask,
    -LSE and -delta terms inside the tensor core.  Includes the large finite padding value."""
    import _evoattn
    g = torch.Generator().manual_seed(70 + D)
    bf = torch.bfloat16
    y = torch.randn((128, D), generator=g).to(bf)
    z = torch.randn((128, D), generator=g).to(bf)
    a = (torch.randn((128, 8), generator=g) * 10).to(bf)
    b = (torch.randn((128, 8), generator=g) * 10).to(bf)
    a[5, :] = 0
    a[5, 2] = -1e30                     # a padded row: very negative, finite
    b[:, 2] = 1
    dev = "cuda"
    out = torch.full((128, 128), float("nan"), device=dev)
    _evoattn.selftest_mma_extra(D, y.to(dev), z.to(dev), a.to(dev), b.to(dev), out,
                                torch.cuda.current_stream().cuda_stream)
    _evoattn.device_status()
    ref = y.double() @ z.double().T + a.double() @ b.double().T
    got = out.double().cpu()
    keep = torch.ones(128, dtype=torch.bool)
    keep[5] = False
    err = (ref[keep] - got[keep]).abs().max().item()
    assert err < 2e-2, f"D={D}: max abs err {err}"          # fp32 accumulation of terms up to ~1e3
    assert (got[5] < -1e29).all() and torch.isfinite(got[5]).all()
