"""Sizes the kernels do not take are refused by name, before anything is compiled or launched (no GPU
needed): head sizes outside 16..256 in steps of 16, more than 16 query heads per kv head, inner sizes the
specialised products are not built for, and the tensor-core attention's narrower range."""

import pytest

from dryft_b200.ops import kernels as K


@pytest.mark.parametrize("head_dim,group", [(40, 2), (0, 1), (272, 1), (64, 17), (64, 0)])
def test_attention_sizes_outside_the_range_are_refused(head_dim, group):
    with pytest.raises(K.KernelError) as e:
        K.attention_rows_lib(head_dim, group, 64)
    assert str(head_dim) in str(e.value) or str(group) in str(e.value)
    assert not K.attention_decode_supported(head_dim, group)


def test_tensor_core_prompt_attention_says_what_it_takes():
    assert K.attention_prefill_tc_supported(128, 4, 64) and K.attention_prefill_tc_supported(64, 1, 64)
    assert not K.attention_prefill_tc_supported(96, 2, 64)      # other head sizes run the mma.sync kernel
    assert not K.attention_prefill_tc_supported(128, 4, 32)     # written for 64-token pages
    with pytest.raises(K.KernelError) as e:
        K.attention_prefill_tc_lib(96, 2, 64)
    assert "64 and 128" in str(e.value)


@pytest.mark.parametrize("k", [0, 100, 2568])
def test_specialised_decode_product_refuses_other_inner_sizes(k):
    with pytest.raises(K.KernelError) as e:
        K.gemm_decode_lib(k)
    assert "256" in str(e.value)


def test_streaming_product_row_and_width_limits():
    assert K.gemm_stream_supported(64, 2560) and K.gemm_stream_supported(1, 64)
    assert not K.gemm_stream_supported(65, 2560) and not K.gemm_stream_supported(8, 100)
