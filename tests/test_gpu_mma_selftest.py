"""Tensor-core operand conventions: one CTA multiplies small tiles through the
same UMMA descriptors the attention kernels use (K-major and MN-major row
tiles, K-major and MN-major square tiles, an A operand in tensor memory), checked against a CPU GEMM."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D", [32, 64])
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
