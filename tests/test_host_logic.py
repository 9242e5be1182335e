"""CPU: the host-side mirror — layout attributes derived from tensor views, and the checks the
reference's runners make before launching."""
import pytest
import torch


def test_gemm_attrs_row_and_col_major(pkg):
    a = torch.zeros(6, 10, dtype=torch.bfloat16)
    b = torch.zeros(4, 10, dtype=torch.bfloat16).t()       # [10, 4] with K contiguous → column-major
    o = torch.zeros(6, 4, dtype=torch.bfloat16)
    at = pkg.gemm_attrs_for(a, b, o, beta=0.5)
    assert (at["lhs_order"], at["lhs_num_rows"], at["lhs_num_cols"], at["lhs_leading_dim_stride"]) == (0, 6, 10, 10)
    assert (at["rhs_order"], at["rhs_num_rows"], at["rhs_num_cols"], at["rhs_leading_dim_stride"]) == (1, 10, 4, 10)
    assert at["output_order"] == 0 and at["batch_size"] == 1 and at["beta"] == 0.5
    assert at["lhs_layout_dtype"] == pkg.IXK_BF16


def test_gemm_attrs_padded_and_batched(pkg):
    a = torch.zeros(3, 6, 16, dtype=torch.float16)[:, :, :10]   # pitch 16
    b = torch.zeros(3, 10, 8, dtype=torch.float16)
    o = torch.zeros(3, 6, 8, dtype=torch.float32)
    at = pkg.gemm_attrs_for(a, b, o)
    assert at["lhs_leading_dim_stride"] == 16 and at["lhs_batch_stride"] == 96
    assert at["batch_size"] == 3 and at["output_layout_dtype"] == pkg.IXK_F32


def test_gemm_attrs_rejects_doubly_strided(pkg):
    a = torch.zeros(6, 20, dtype=torch.bfloat16)[:, ::2]
    with pytest.raises(pkg.IxkError):
        pkg.gemm_attrs_for(a, torch.zeros(10, 4, dtype=torch.bfloat16), torch.zeros(6, 4, dtype=torch.bfloat16))


def test_unknown_epilogue_name(pkg):
    x = torch.zeros(8, 8, dtype=torch.bfloat16)
    with pytest.raises(pkg.IxkError, match="Unknown Epilogue"):
        pkg.run_gemm_custom_call(x, x, None, x, None, None, pkg.gemm_attrs_for(x, x, x), "SILU")


def test_fmha_desc_from_bsnh_views(pkg):
    B, S, N, H = 2, 12, 3, 64
    q = torch.zeros(B, S, N, H, dtype=torch.bfloat16).permute(0, 2, 1, 3)   # [B,N,S,H] view of [B,S,N,H]
    o = torch.zeros(B, N, S, H, dtype=torch.bfloat16)
    bias = torch.zeros(B, 1, S, S, dtype=torch.bfloat16)
    d = pkg._fmha_desc(q, q, q, bias, o, 0.125, True, 0.0)
    assert list(d.q_strides) == [S * N * H, H, N * H]
    assert list(d.o_strides) == [N * S * H, S * H, H]
    assert list(d.bias_strides) == [S * S, 0, S]          # head-broadcast → stride 0
    assert (d.num_batches, d.num_heads, d.num_queries, d.num_keys, d.head_size, d.causal) == (B, N, S, S, H, 1)


def test_fmha_rejects_dropout_and_strided_head(pkg):
    q = torch.zeros(1, 1, 4, 64, dtype=torch.bfloat16)
    with pytest.raises(pkg.IxkError):
        pkg._fmha_desc(q[..., ::2], q, q, None, q, 1.0, False, 0.0)
    with pytest.raises(pkg.IxkError, match="no CPU path"):
        pkg.fmha_forward_kernel(None, q, q, q, None, torch.zeros(1), 0.5, q, None, 1.0)


def test_quantize_fp8_matches_oracle(pkg, orc):
    import numpy as np
    torch.manual_seed(0)
    x = torch.randn(64, 48)
    for tdt, odt in ((torch.float8_e4m3fn, orc.F8E4M3), (torch.float8_e5m2, orc.F8E5M2)):
        q, s = pkg.quantize_fp8(x, tdt)
        codes, s2 = orc.quantize_fp8(x.numpy(), odt)
        assert s == pytest.approx(s2)
        assert np.array_equal(q.view(torch.uint8).numpy(), codes)
