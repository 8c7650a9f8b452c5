"""Host-side behaviour of the operator surface (no GPU): the reference's
names, shape assertions and head-dim rules."""
import pytest
import torch


def _inputs(B=1, S=2, N=16, H=2, D=32):
    q = torch.zeros((B, S, N, H, D))
    return q, q.clone(), q.clone(), torch.zeros((B, S, 1, 1, N)), torch.zeros((B, 1, H, N, N))


def test_surface_names():
    import tk_evo_attention_layer as L
    assert hasattr(L, "TKEvoAttention") and issubclass(L.TKEvoAttention, torch.autograd.Function)
    assert L.TK_SUPPORTED_DIMS == (16, 32, 64, 96, 128)
    assert L._next_supported_dim(8) == 16 and L._next_supported_dim(16) == 16 and L._next_supported_dim(32) == 32
    assert L._next_supported_dim(24) == 32
    assert L._next_supported_dim(33) == 64 and L._next_supported_dim(64) == 64
    assert L._next_supported_dim(65) == 96 and L._next_supported_dim(96) == 96
    assert L._next_supported_dim(100) == 128 and L._next_supported_dim(128) == 128
    with pytest.raises(ValueError):
        L._next_supported_dim(129)
    with pytest.raises(ValueError):
        L._next_supported_dim(256)


def test_shape_errors_are_assertions():
    from tk_evo_attention_layer import TKEvoAttention
    q, k, v, m, b = _inputs()
    with pytest.raises(AssertionError):
        TKEvoAttention.apply(q, k[:, :1], v, m, b)
    with pytest.raises(AssertionError):
        TKEvoAttention.apply(q, k, v, m.reshape(1, 2, 16), b)
    with pytest.raises(AssertionError):
        TKEvoAttention.apply(q, k, v, m, b.squeeze(1))


def test_no_cpu_fallback():
    from tk_evo_attention_layer import TKEvoAttention
    q, k, v, m, b = _inputs()
    with pytest.raises(RuntimeError, match="no CPU path"):
        TKEvoAttention.apply(q, k, v, m, b)


def test_unsupported_head_dim():
    from tk_evo_attention_layer import TKEvoAttention
    q, k, v, m, b = _inputs(D=136)
    with pytest.raises(ValueError):
        TKEvoAttention.apply(q, k, v, m, b)


def test_strided_path_only_for_dense_views():
    """Views the kernels read in place must be permutations of a contiguous tensor.  q, k, v chunked out
    of one fused projection share strides but have holes: they are copied, so that O is contiguous."""
    import tk_evo_attention_layer as L
    bf = torch.bfloat16
    B, S, N, H, D = 1, 4, 16, 2, 32
    base = torch.zeros((B, N, S, H, D), dtype=bf)                 # "ending node" storage order
    q = base.permute(0, 2, 1, 3, 4)
    assert L._shared_view_strides(q, q, q) == tuple(q.stride())
    qkv = torch.zeros((B, S, N, H, 3 * D), dtype=bf)
    q, k, v = qkv.chunk(3, dim=-1)
    assert q.stride() == k.stride() == v.stride() and not q.is_contiguous()
    assert L._shared_view_strides(q, k, v) is None                # holes: copied, not read in place
    t = torch.zeros((B, S, N, H, D), dtype=bf)
    assert L._shared_view_strides(t, t, t) is None                # contiguous: the plain path
    e = torch.zeros((B, 1, N, H, D), dtype=bf).expand(B, S, N, H, D)
    assert L._shared_view_strides(e, e, e) is None                # overlapping (stride 0)


def test_bias_cast_is_cached_per_version():
    """The bf16 copy of an fp32 pair bias is made once per version of the tensor: a second call with the
    same tensor returns the same copy, an in-place write invalidates it."""
    import tk_evo_attention_layer as L
    B, H, N = 1, 2, 16
    pb = torch.randn((B, 1, H, N, N))
    a = L._bias_bf16(pb, B, H, N)
    b = L._bias_bf16(pb, B, H, N)
    assert a is b and a.dtype == torch.bfloat16 and a.shape == (B, H, N, N)
    pb.add_(1.0)                                              # bumps the version counter
    c = L._bias_bf16(pb, B, H, N)
    assert c is not a and torch.equal(c, pb.reshape(B, H, N, N).to(torch.bfloat16))
    h = torch.randn((B, 1, H, N, N)).to(torch.bfloat16)
    assert L._bias_bf16(h, B, H, N).data_ptr() == h.data_ptr()   # bf16 input: no copy at all


def test_views_with_holes_are_read_in_place():
    """q, k, v sliced out of one fused projection are not dense, so outputs cannot mirror them, but the
    kernels can read them where they lie: _inplace_view_strides accepts them, and rejects views whose
    steps are not multiples of 8 elements, whose strides differ, or that overlap themselves."""
    import tk_evo_attention_layer as L
    bf = torch.bfloat16
    B, S, N, H, D = 2, 3, 16, 2, 32
    qkv = torch.zeros((B, S, N, 3, H, D), dtype=bf)
    q, k, v = qkv.unbind(dim=3)
    assert L._shared_view_strides(q, k, v) is None
    assert L._inplace_view_strides(q, k, v) == (S * N * 3 * H * D, N * 3 * H * D, 3 * H * D, D, 1)
    wide = torch.zeros((B, S, N, H, 3 * D), dtype=bf)
    q2, k2, v2 = wide.chunk(3, dim=-1)
    assert L._inplace_view_strides(q2, k2, v2) == (S * N * H * 3 * D, N * H * 3 * D, H * 3 * D, 3 * D, 1)
    assert L._inplace_view_strides(q, k2, v) is None                          # different strides
    assert L._inplace_view_strides(q.float(), k.float(), v.float()) is None   # not bf16
    odd = torch.zeros((B, S, N, H, D + 4), dtype=bf)[..., :D]                 # steps of 36 elements
    assert L._inplace_view_strides(odd, odd, odd) is None
    ov = torch.zeros((N + 4, H, D), dtype=bf).as_strided((1, 1, N, H, D), (0, 0, D, D, 1))   # rows overlap heads
    assert L._inplace_view_strides(ov, ov, ov) is None
