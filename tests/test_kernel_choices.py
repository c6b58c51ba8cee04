"""The kernel plan (no GPU needed): which kernel every operation takes at which sizes, and how many key splits
the decode attention uses.  The parts do what these functions answer, so pinning the answers pins the path."""

import itertools

import torch

from tesseract_b200 import plan

SMS = 148      # the choices below are those of a B200; the engine asks the device
BF, F32 = torch.bfloat16, torch.float32


def resident_ctas(head_dim):
    return (2 if head_dim <= 128 else 1) * SMS


def test_split_counts_keep_every_cta_resident():
    for seqs, heads, context, head_dim in itertools.product((1, 2, 3, 8, 16, 64, 200), (1, 2, 8), (1, 17, 500, 2184, 32768, 131072),
                                                            (16, 64, 128, 256)):
        splits = plan.attention_splits(seqs, heads, context, head_dim, sms=SMS)
        assert 1 <= splits <= plan.MAX_ATTENTION_SPLITS
        if splits > 1:
            assert splits * seqs * heads <= resident_ctas(head_dim), (seqs, heads, context, head_dim, splits)
        tiles = -(-context // 16)
        assert splits <= max(1, tiles), "never more splits than tiles of keys"


def test_split_counts_follow_the_measurements():
    # batch 8 of the 1B sizes: four splits as one cluster; batch 64: none; one long sequence: as many as fit
    assert plan.attention_splits(8, 8, 2184, 64, sms=SMS) == 4
    assert plan.attention_splits(64, 8, 2184, 64, sms=SMS) == 1
    assert plan.attention_splits(1, 8, 131072, 64, sms=SMS) == 32
    # wide heads: two CTAs per SM as well, so batch 8 still takes four
    assert plan.attention_splits(8, 8, 2184, 128, sms=SMS) == 4
    # short contexts are not worth a merge
    assert plan.attention_splits(8, 8, 40, 64, sms=SMS) == 1


def test_products_of_the_1b_sizes():
    hidden, inter, qkv, vocab = 2048, 8192, 3072, 128256
    for rows, kernel in ((1, "decode_linear"), (8, "decode_linear"), (16, "decode_linear")):
        assert plan.product(BF, rows, qkv, hidden, norm="add_norm") == plan.ProductPlan(kernel, True, "bf16")
        assert plan.product(BF, rows, hidden, hidden) == plan.ProductPlan(kernel, False, "bf16")
        assert plan.product(BF, rows, 2 * inter, hidden, epilogue="swiglu", norm="add_norm") == \
            plan.ProductPlan(kernel, True, "swiglu")
        assert plan.product(BF, rows, hidden, inter) == plan.ProductPlan(kernel, False, "bf16")
        assert plan.product(BF, rows, vocab, hidden, epilogue="f32", norm="add_norm") == \
            plan.ProductPlan(kernel, True, "f32")
    for rows in (1, 8, 16):
        # a product in front of an addition and a norm of its own width does that norm's work; the product behind
        # takes the prepared rows
        assert plan.product(BF, rows, hidden, hidden, follow=True) == \
            plan.ProductPlan("decode_linear", False, "bf16", prepares_norm=True)
        assert plan.product(BF, rows, hidden, inter, follow=True).prepares_norm
        assert plan.product(BF, rows, 2 * inter, hidden, epilogue="swiglu", norm="prepared") == \
            plan.ProductPlan("decode_linear", True, "swiglu", takes_prepared=True)
        assert plan.product(BF, rows, vocab, hidden, epilogue="f32", norm="prepared") == \
            plan.ProductPlan("decode_linear", True, "f32", takes_prepared=True)
    assert not plan.product(F32, 8, hidden, hidden, follow=True).prepares_norm
    for rows in (17, 64, 128):
        # 17 to 128 rows stream their weights through the tensor-memory kernel, with the same division of a norm's
        # work; a norm that no product prepared runs as a kernel of its own in front
        assert plan.product(BF, rows, qkv, hidden, norm="add_norm") == plan.ProductPlan("skinny_tcgen05", False, "bf16")
        assert plan.product(BF, rows, qkv, hidden, norm="prepared") == \
            plan.ProductPlan("skinny_tcgen05", True, "bf16", takes_prepared=True)
        assert plan.product(BF, rows, hidden, hidden, follow=True) == \
            plan.ProductPlan("skinny_tcgen05", False, "bf16", prepares_norm=True)
        assert plan.product(BF, rows, hidden, inter, follow=True).prepares_norm
        assert plan.product(BF, rows, 2 * inter, hidden, epilogue="swiglu", norm="prepared") == \
            plan.ProductPlan("skinny_tcgen05", True, "swiglu", takes_prepared=True)
        assert plan.product(BF, rows, 2 * inter, hidden, epilogue="swiglu") == plan.ProductPlan("skinny_tcgen05", False, "swiglu")
        assert plan.product(BF, rows, vocab, hidden, epilogue="f32", norm="prepared") == \
            plan.ProductPlan("skinny_tcgen05", True, "f32", takes_prepared=True)
    for rows in (129, 2048):
        assert not plan.product(BF, rows, hidden, hidden, follow=True).prepares_norm
        assert plan.product(BF, rows, qkv, hidden, norm="add_norm") == plan.ProductPlan("library", False, "bf16")
        assert plan.product(BF, rows, 2 * inter, hidden, epilogue="swiglu") == plan.ProductPlan("gemm_tcgen05", False, "swiglu")
        assert plan.product(BF, rows, vocab, hidden, epilogue="f32") == plan.ProductPlan("library", False, "f32")
    assert plan.DECODE_LINEAR_MAX_ROWS == 16 and plan.SKINNY_MAX_ROWS == 128
    assert plan.FUSED_GATE_UP_MIN_ROWS == plan.DECODE_LINEAR_MAX_ROWS + 1


def test_products_of_sizes_a_kernel_does_not_take_fall_to_the_next():
    # rows that are not contiguous, and widths the weight-streaming kernel refuses (N % 16, K % 32), go on
    assert plan.product(BF, 4, 3072, 2048, contiguous_rows=False).kernel == "library"
    assert plan.product(BF, 4, 331, 72).kernel == "library"
    # a norm that does not fit in front (the rows of a 8,192-wide product beside its ring) runs on its own
    wide = plan.product(BF, 16, 64, 8192, norm="add_norm")
    assert wide.kernel == "decode_linear" and not wide.norm_folded
    # SwiGLU on a product the tcgen05 GEMM refuses: the library product and the activation kernel
    odd = plan.product(BF, 40, 2 * 200, 76, epilogue="swiglu")          # K is no multiple of eight
    assert odd.kernel == "library" and odd.activation_apart and odd.epilogue == "bf16"
    # the 32-bit path has one product kernel
    assert plan.product(F32, 5, 3072, 2048, epilogue="swiglu", norm="add_norm") == \
        plan.ProductPlan("gemm_f32", False, "f32", activation_apart=True)


def test_attention_plans():
    sizes = dict(num_heads=32, num_kv_heads=8, head_dim=64, page_size=16, sms=SMS)
    decode = plan.attention(BF, new_tokens=[1] * 8, max_context=2184, **sizes)
    assert decode.fused_decode and decode.splits == 4 and decode.merge == "cluster"
    lonely = plan.attention(BF, new_tokens=[1], max_context=131072, **sizes)
    assert lonely.fused_decode and lonely.splits == 32 and lonely.merge == "scratch"
    portion = plan.attention(BF, new_tokens=[2048], max_context=2048, **sizes)
    assert portion.prompt == "tcgen05" and not portion.split and not portion.fused_decode and portion.key_splits == 1
    # a 512-token portion is 128 tiles: late in a long prompt every tile is shared by two CTAs, early it is not
    assert plan.attention(BF, new_tokens=[512], max_context=2048, **sizes).key_splits == 1
    assert plan.attention(BF, new_tokens=[512], max_context=16384, **sizes).key_splits == 2
    assert plan.attention(BF, new_tokens=[512, 512, 512], max_context=16384, **sizes).key_splits == 1
    assert plan.attention(BF, new_tokens=[64], max_context=32768, **sizes).key_splits == 8
    # (the rule counts keys, not blocks: at head size 128, whose blocks are 64 keys, sharing starts at 4,096 too)
    wide = dict(sizes, head_dim=128)
    assert plan.attention(BF, new_tokens=[512], max_context=2048, **wide).key_splits == 1
    assert plan.attention(BF, new_tokens=[512], max_context=3072, **wide).key_splits == 1
    assert plan.attention(BF, new_tokens=[512], max_context=4096, **wide).key_splits == 2
    mixed = plan.attention(BF, new_tokens=[512, 1, 1, 3], max_context=4096, **sizes)
    assert mixed.prompt == "tcgen05" and mixed.split and mixed.splits >= 1
    narrow = dict(sizes, head_dim=48, num_heads=6, num_kv_heads=3)
    assert plan.attention(BF, new_tokens=[40, 1], max_context=100, **narrow).prompt == "mma_tiles"
    assert plan.attention(BF, new_tokens=[40], max_context=100, prompt_kernel="mma", **sizes).prompt == "mma_tiles"
    # a position encoding the kernels cannot apply themselves: no fused decode kernel
    assert not plan.attention(BF, new_tokens=[1, 1], max_context=100, rotary_in_kernel=False, **sizes).fused_decode
    # more than 16 query heads per kv head do not fold into the decode kernel's 16 rows
    grouped = plan.attention(BF, new_tokens=[1], max_context=100, num_heads=32, num_kv_heads=1, head_dim=64,
                             page_size=16, sms=SMS)
    assert grouped.prompt is not None and not grouped.split and not grouped.fused_decode
    assert plan.attention(F32, new_tokens=[1, 7], max_context=100, **sizes).rows
