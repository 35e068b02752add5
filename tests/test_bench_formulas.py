"""The byte and flop counts that bench.py holds its timings against, checked against the figures of the
Qwen3-8B shape worked out by hand (36 layers, hidden 4,096, 32 query heads over 8 kv heads of 128, feed-forward
12,288, vocabulary 151,936, separate output table)."""
import bench


def test_bytes_of_a_decode_step_and_flops_of_a_prefill():
    cfg = bench.QWEN3_8B
    per_layer = (6144 * 4096 + 4096 * 4096 + 2 * 12288 * 4096 + 4096 * 12288) * 2          # q/k/v, output, gate+up, down
    assert per_layer == 385_875_968
    assert bench.weight_bytes_per_decode_step(cfg, 36) == 36 * per_layer + 151936 * 4096 * 2    # 15.14 GB: the embedding is not read
    assert round(bench.weight_bytes_per_decode_step(cfg, 36) / 1e9, 2) == 15.14
    assert bench.kv_bytes_per_token(cfg, 36) == 147_456                                       # 36 layers x K and V x 8 x 128 x 2 bytes
    flops = bench.prefill_flops(cfg, 36, 2048)
    products = 2 * 2048 * 36 * (per_layer // 2) + 2 * 151936 * 4096                           # one logits row
    attention = 36 * 4 * 32 * 128 * 2048 * 2049 // 2                                          # causal Q K^T and P V
    assert flops == products + attention and 29.5e12 < flops < 30.0e12
    # fewer layers, another shape: the 4B shape ties the output table to the embedding, which is still read once
    assert bench.weight_bytes_per_decode_step(bench.QWEN3_4B, 36) == 2 * (36 * (6144 * 2560 + 2560 * 4096 + 3 * 9728 * 2560) + 151936 * 2560)


def test_more_than_one_gpu_is_refused_and_the_reference_arm_is_unavailable(capsys, monkeypatch):
    import json
    import sys
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "2"])
    assert bench.main() == 2 and "one GPU" in capsys.readouterr().out
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference"])
    assert bench.main() == 0
    line = json.loads(capsys.readouterr().out)
    assert line["impl"] == "reference" and "unavailable" in line
