"""Configuration parsing, the architecture registry and the model description (CPU)."""
import json

import pytest

import plain_qwen3 as plain
from tiny_inference_engine_b200.config import (Architecture, ModelSpec, PartSpec, RunEntry, load_config,
                                               parse_qwen3_config, qwen3_spec, register_architecture,
                                               resolve_architecture)
from tiny_inference_engine_b200.errors import InvalidArgument, LoadError, UnsupportedError


def test_defaults_of_absent_keys():
    c = parse_qwen3_config(plain.TINY_C)          # no num_key_value_heads, head_dim, rope_theta, tie_word_embeddings
    assert c.num_key_value_heads == c.num_attention_heads == 3
    assert c.head_dim == 144 // 3 and c.rope_theta == 10000.0 and c.tie_word_embeddings is False
    assert c.q_dim == 144 and c.kv_dim == 144


def test_every_size_comes_from_the_file():
    c = parse_qwen3_config(plain.TINY_B)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (503, 96, 200, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (8, 1, 32)
    assert c.q_dim == 256 != c.hidden_size
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and c.max_position_embeddings == 1024


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "max_position_embeddings", "rms_norm_eps"])
def test_required_keys(key):
    cfg = dict(plain.TINY_A)
    del cfg[key]
    with pytest.raises(LoadError, match=f"config.json has no '{key}'"):
        parse_qwen3_config(cfg)


@pytest.mark.parametrize("patch,err,text", [
    ({"model_type": "llama"}, UnsupportedError, "llama"),
    ({"use_sliding_window": True}, UnsupportedError, "use_sliding_window"),
    ({"rope_scaling": {"type": "yarn"}}, UnsupportedError, "rope_scaling"),
    ({"attention_bias": True}, UnsupportedError, "attention_bias"),
    ({"num_key_value_heads": 3}, LoadError, "multiple"),
    ({"head_dim": 15}, LoadError, "even"),
    ({"vocab_size": 0}, LoadError, "vocab_size"),
    ({"hidden_size": -4}, LoadError, "hidden_size"),
    ({"rms_norm_eps": 0.0}, LoadError, "rms_norm_eps"),
    ({"rope_theta": -1.0}, LoadError, "rope_theta"),
    ({"num_hidden_layers": 2.5}, LoadError, "num_hidden_layers"),
])
def test_rejections(patch, err, text):
    with pytest.raises(err, match=text):
        parse_qwen3_config({**plain.TINY_A, **patch})


def test_null_rope_scaling_and_false_flags_are_fine():
    parse_qwen3_config({**plain.TINY_A, "rope_scaling": None, "use_sliding_window": False, "attention_bias": False,
                        "sliding_window": 4096, "max_window_layers": 2, "torch_dtype": "bfloat16"})


def test_registry_by_architecture_then_model_type():
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert resolve_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(UnsupportedError, match="LlamaForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "qwen3"})
    with pytest.raises(UnsupportedError, match="gpt2"):
        resolve_architecture({"model_type": "gpt2"})
    with pytest.raises(LoadError, match="model_type"):
        resolve_architecture({})


def test_load_config_from_a_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(plain.TINY_A))
    arch, cfg, spec = load_config(tmp_path)
    assert arch.name == "Qwen3ForCausalLM" and cfg.hidden_size == 64 and len(spec.layers) == 2
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(LoadError, match="invalid JSON"):
        load_config(tmp_path)
    with pytest.raises(LoadError, match="cannot open"):
        load_config(tmp_path / "nowhere")


def test_spec_carries_the_constants_layer_by_layer():
    spec = qwen3_spec(parse_qwen3_config(plain.TINY_B))
    assert [e.layer for e in spec.run_order] == [0, 1, 2] and all(e.cache_of is None for e in spec.run_order)
    l1 = spec.layers[1]
    assert l1.mixer.kind == "gqa_attention" and l1.ffn.kind == "swiglu" and l1.block.kind == "prenorm"
    assert l1.mixer["num_kv_heads"] == 1 and l1.mixer["head_dim"] == 32 and l1.mixer["window"] == 0
    assert l1.mixer["position"].kind == "rope" and l1.mixer["position"]["theta"] == 1e6
    assert l1.mixer["q_norm"]["eps"] == 1e-5 and l1.mixer_norm["name"] == "model.layers.1.input_layernorm.weight"
    assert spec.head["tied"] is False and spec.final_norm["size"] == 96


def test_run_order_is_checked():
    spec = qwen3_spec(parse_qwen3_config(plain.TINY_A))

    def with_order(order):
        return ModelSpec(**{**spec.__dict__, "run_order": tuple(order)})

    with_order([RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_of=1)]).validate()   # twice, and a shared cache
    with pytest.raises(InvalidArgument, match="names layer 5"):
        with_order([RunEntry(5)]).validate()
    with pytest.raises(InvalidArgument, match="not earlier"):
        with_order([RunEntry(0, cache_of=0)]).validate()
    with pytest.raises(InvalidArgument, match="none of its own"):
        with_order([RunEntry(0), RunEntry(1, cache_of=0), RunEntry(0, cache_of=1)]).validate()


def test_another_architecture_can_be_registered():
    def spec_of(cfg):
        base = qwen3_spec(parse_qwen3_config(cfg))
        return ModelSpec(**{**base.__dict__, "architecture": "ToyForCausalLM"})

    register_architecture(Architecture("ToyForCausalLM", parse_config=lambda j: j, build_spec=spec_of,
                                       model_types=("toy",)), replace=True)
    arch = resolve_architecture({"architectures": ["ToyForCausalLM"]})
    assert arch.build_spec(arch.parse_config(plain.TINY_A)).architecture == "ToyForCausalLM"
    with pytest.raises(ValueError, match="already registered"):
        register_architecture(Architecture("ToyForCausalLM", parse_config=dict, build_spec=spec_of))


def test_decode_attention_splits_respect_the_kernel_limits():
    """However long the context, however many sequences and whatever the page size: splits are whole 64-key
    tiles, their page ids fit the kernel's shared-memory table and there are at most MAX_SPLITS of them."""
    from tiny_inference_engine_b200.parts import attention as att
    for page in (8, 16, 32, 64, 128, 256):
        boxes = 64 // min(page, 64)
        for sequences in (1, 3, 8, 64, 256):
            for kv_heads in (1, 8):
                for longest in (1, 63, 64, 65, 1000, 4096, 8128, 8129, 40960, 131072):
                    split_keys, max_splits = att.decode_splits(longest, sequences, kv_heads, page)
                    assert split_keys % 64 == 0 and split_keys >= 64
                    fits = (split_keys // 64 + 1) * boxes <= att.TMA_DECODE_TABLE_ENTRIES
                    assert fits or max_splits == att.MAX_SPLITS    # only a context beyond every configuration gets there
                    assert 1 <= max_splits <= att.MAX_SPLITS and max_splits * split_keys >= longest
                    if longest <= 40960:
                        assert (split_keys // 64 + 1) * boxes <= att.TMA_DECODE_TABLE_ENTRIES
    # with the sequences' own lengths: a few long ones among short ones are cut up, and all CTAs fit at once
    lens = [3000, 2900] + [200] * 28
    sk, ms = att.decode_splits(3000, 30, 8, 16, lens)
    assert sk < 3000 and sk % 64 == 0 and ms == -(-3000 // sk) and sum(-(-c // sk) for c in lens) * 8 <= 2 * att.NUM_SMS
    assert att.decode_splits(3000, 30, 8, 16) == (3008, 1)
    assert att.decode_splits(4096, 8, 8, 16, [4096] * 8) == att.decode_splits(4096, 8, 8, 16)


def test_matrix_product_plans_are_ones_the_kernel_takes():
    """Whatever the sizes: a tile width the kernel has, splits that leave every split k-blocks to do, k whole where
    the caller asks for it, and no more partial sums than the capacity the parts size their scratch for."""
    from tiny_inference_engine_b200.ops import gemm_select as gs
    for N, K in ((6144, 4096), (4096, 12288), (2560, 9728), (151936, 4096), (72, 200), (130, 75), (300, 64), (1000, 520)):
        k_blocks = -(-K // 64)
        for M in (1, 7, 8, 64, 128, 129, 200, 256, 384, 512, 513, 1000, 2048, 8192):
            for split_many in (True, False):
                transposed, bn, splits = gs.plan(M, N, K, split_many)
                assert bn in (16, 32, 64, 128, 256) and 1 <= splits <= max(1, k_blocks)
                assert transposed == (1 if M <= 128 else 0)
                if M > 128:
                    assert splits <= 4 or N <= 128
                    assert splits == 1 or (split_many and k_blocks // splits >= 8)
                if splits > 1:
                    assert splits * M * N <= gs.partial_capacity(max(M, 512), N, K, split_many)
    # the shapes the cost estimate was fitted on: the measured best, or close to it
    assert gs.plan(512, 2560, 9728)[1:] == (256, 3) and gs.plan(384, 4096, 12288)[1:] == (256, 3)
    assert gs.plan(2048, 24576, 4096)[2] == 1


def test_pair_kernel_tile_widths_follow_the_waves():
    """The width of the pair kernel's tiles: the full 256 where narrower tiles save no wave (2,048 tokens of Qwen3-8B's
    products), narrower where the tiles of a short portion leave most pairs of SMs idle or a wave nearly empty."""
    from tiny_inference_engine_b200.ops import gemm_select as gs
    for N, K in ((6144, 4096), (4096, 4096), (4096, 12288)):
        assert gs.pair_width(2048, N, K, 74) == 256
    assert gs.pair_width(2048, 24576, 4096, 74) in (224, 256)
    assert gs.pair_width(512, 6144, 4096, 74) == 192          # 64 tiles in one wave instead of 48 wider ones
    assert gs.pair_width(512, 24576, 4096, 74) == 224         # 220 tiles: three waves, as 192 of full width, each shorter
    for M in (512, 700, 1024, 2048, 4096):
        for N in (256, 2560, 4096, 9728, 151936):
            assert gs.pair_width(M, N, 4096, 74) in gs.PAIR_WIDTHS
