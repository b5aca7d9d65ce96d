"""Host-side logic of the merged forward pass that needs no GPU: the timer's table, the jagged container's optional
fields, the synthetic architecture and the wrapping of its blocks."""
import numpy as np
import pytest
import torch


def test_timer_table_matches_numpy_percentiles():
    from come_b200.timer import Timer
    ms = [3.0, 1.0, 2.0, 10.0, 4.0]
    e = Timer.summarise("Accelerated Model", ms)
    assert e.count == 5 and e.P50 == 3.0
    assert e.P90 == pytest.approx(np.percentile(ms, 90)) and e.P99 == pytest.approx(np.percentile(ms, 99))
    text = Timer.format_table([Timer.summarise("Reference Model", [20.0, 22.0]), e])
    lines = text.strip().split("\n")
    assert lines[0].split() == ["Name", "Count", "Median", "(ms)", "P90", "(ms)", "P99", "(ms)"]
    assert lines[2].startswith("Reference Model") and lines[2].split()[-3:] == ["21.00", "21.80", "21.98"]
    assert lines[3].startswith("Accelerated Model") and "3.00" in lines[3]


def test_timer_inactive_records_nothing():
    from come_b200.timer import Timer
    Timer.reset()
    Timer.activate(False)
    with Timer.range("x"):
        pass
    assert Timer.results() == [] and not Timer.is_active()


def test_jagged_tokens_optional_fields_propagate():
    from come_b200.token_merger import JaggedTokens
    dev_max = torch.tensor([7], dtype=torch.int32)
    x = JaggedTokens(torch.zeros(1, 10, 4), torch.ones(10), torch.tensor([0, 3, 10]), max_seqlen=9, max_seqlen_dev=dev_max)
    y = x.apply(lambda t: t + 1)
    assert y.max_seqlen == 9 and y.max_seqlen_dev is dev_max and float(y.tokens.sum()) == 40.0
    z = JaggedTokens(torch.zeros(1, 10, 4), torch.ones(10), torch.tensor([0, 3, 10]))
    assert z.max_seqlen is None and z.max_seqlen_dev is None
    grown = x.add_suffix(torch.zeros(2, 1, 4))
    assert grown.max_seqlen is None  # lengths changed: the bound no longer holds


def test_fused_aggregator_wraps_every_block():
    from come_b200.block import JaggedBlock, JaggedBlock_w_Bias
    from come_b200.fused import FusedAggregator, fused_accelerate
    from come_b200.vggt_arch import AggregatorCore
    core = AggregatorCore(embed_dim=64, depth=4, num_heads=2, mlp_ratio=2.0, aa_block_size=2, retain_layers=frozenset({1, 3}))
    assert core.aa_block_num == 2 and not core.training
    model = fused_accelerate(core)
    assert len(model.frame_blocks) == 4 and all(isinstance(b, JaggedBlock_w_Bias) for b in model.global_blocks)
    assert all(isinstance(b, JaggedBlock) for b in model.plain_frame_blocks)
    assert model.frame_blocks[0].block is core.frame_blocks[0]
    assert core.frame_blocks[0].attn.qkv.weight.dtype == torch.bfloat16  # the attention modules run in bf16
    assert core.frame_blocks[0].mlp.fc1.weight.dtype == torch.float32    # the rest keeps the model's dtype
    plain = FusedAggregator(core, use_attn_bias_correction=False)
    assert all(type(b) is JaggedBlock for b in plain.frame_blocks)
    with pytest.raises(ValueError):
        AggregatorCore(embed_dim=64, depth=3, num_heads=2, aa_block_size=2)
    with pytest.raises(ValueError):
        FusedAggregator(core, attn_dtype="fp32")
    core.train()
    with pytest.raises(AssertionError):
        FusedAggregator(core)
