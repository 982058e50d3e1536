import json

import pytest

from slipstream_b200.config.engine_config import CacheConfig, EngineConfig, SchedulerConfig
from slipstream_b200.config.model_config import ConfigError, Qwen2Config
from slipstream_b200.config.sampling_params import SamplingParams
from slipstream_b200.registry import architectures, load_config, resolve_architecture

BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 64, "num_attention_heads": 4,
        "num_hidden_layers": 2, "vocab_size": 256, "intermediate_size": 176}


def test_defaults_follow_the_reference_reader():
    c = Qwen2Config.from_dict(BASE)
    assert c.head_dim == 16 and c.num_key_value_heads == 4
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.attention_bias is True and c.mlp_bias is False and c.tie_word_embeddings is False
    assert c.max_position_embeddings == 4096 and c.torch_dtype == "bfloat16"


def test_every_key_is_read():
    d = dict(BASE, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=1e6, tie_word_embeddings=True,
             attention_bias=False, mlp_bias=True, max_position_embeddings=77, torch_dtype="float32",
             eos_token_id=[5, 6], bos_token_id=1)
    c = Qwen2Config.from_dict(d)
    assert (c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta) == (2, 32, 1e-5, 1e6)
    assert c.tie_word_embeddings and not c.attention_bias and c.mlp_bias
    assert c.max_position_embeddings == 77 and c.torch_dtype == "float32" and c.eos_token_id == 5 and c.bos_token_id == 1
    assert Qwen2Config.from_dict(c.to_dict()) == c


def test_rope_theta_inside_rope_scaling_and_generation_config_ids():
    c = Qwen2Config.from_dict(dict(BASE, rope_scaling={"rope_type": "default", "rope_theta": 5e5}), {"eos_token_id": 9})
    assert c.rope_theta == 5e5 and c.eos_token_id == 9


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": "256"}, "vocab_size"),
    ({"num_key_value_heads": 3}, "divisible"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "llama3"}}, "rope type"), ({"use_sliding_window": True}, "sliding"),
    ({"tie_word_embeddings": 1}, "tie_word_embeddings"), ({"num_attention_heads": 5}, "divisible"),
    ({"head_dim": 7}, "even"), ({"rms_norm_eps": True}, "rms_norm_eps"),
    ({"torch_dtype": "float16"}, "float16"), ({"torch_dtype": "half"}, "not supported"), ({"dtype": "fp8"}, "fp8"),
    ({"eos_token_id": True}, "boolean"), ({"rope_scaling": 3}, "object"), ({"num_hidden_layers": 2.5}, "integer"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(dict(BASE, **patch))


def test_whole_numbers_written_as_floats_and_unknown_keys_survive():
    c = Qwen2Config.from_dict(dict(BASE, max_position_embeddings=512.0, dtype="bf16", something_else=[1, 2]))
    assert c.max_position_embeddings == 512 and c.torch_dtype == "bfloat16"
    assert c.to_dict()["something_else"] == [1, 2]


def test_registry(tmp_path):
    assert "Qwen2ForCausalLM" in architectures()
    assert resolve_architecture({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="unsupported architecture"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="unsupported model_type"):
        resolve_architecture({"model_type": "mamba"})
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Qwen2ForCausalLM" and cfg.hidden_size == 64
    model = arch.build(cfg)
    assert len(model.blocks) == 2 and len(model.group_layouts) == 1 and model.group_layouts[0].num_entries == 2
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nothing")


def test_sampling_params_validation():
    assert SamplingParams(temperature=0.0).is_greedy and SamplingParams(top_k=1).is_greedy
    assert not SamplingParams(temperature=0.7).is_greedy
    for bad in ({"max_tokens": 0}, {"temperature": -1}, {"top_k": 0}, {"top_p": 0.0}, {"min_p": 1.5},
                {"repetition_penalty": 0.0}, {"n": 2}):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_engine_config_validation():
    assert CacheConfig(block_size=4).block_size == 4
    for bad in (lambda: CacheConfig(block_size=0), lambda: CacheConfig(gpu_memory_utilization=0.0),
                lambda: SchedulerConfig(policy="horizon"), lambda: SchedulerConfig(max_num_seqs=0),
                lambda: SchedulerConfig(prefill_chunk_size=0), lambda: EngineConfig.for_model("x", dtype="float16")):
        with pytest.raises(ValueError):
            bad()
    # a configuration written for the reference constructs (slipstream/core/config.py:60-134); what asks for a
    # part that is not built is refused by name
    from slipstream_b200 import ParallelConfig
    config = EngineConfig.for_model("x", cache=CacheConfig(swap_space_bytes=1 << 30, enable_paging=True, num_cpu_blocks=None),
                                    scheduler=SchedulerConfig(max_wait_ms=1e4, safety_factor=0.9, starvation_guard_ms=100.0),
                                    parallel=ParallelConfig(tensor_parallel_size=1))
    assert config.parallel.tensor_parallel_size == 1 and config.scheduler.policy == "fcfs"
    for bad, word in ((lambda: CacheConfig(enable_prefix_caching=True), "prefix caching"),
                      (lambda: CacheConfig(enable_paging=False), "unpaged"),
                      (lambda: ParallelConfig(tensor_parallel_size=2), "one GPU"),
                      (lambda: SchedulerConfig(safety_factor=0.0), "safety_factor")):
        with pytest.raises(ValueError, match=word):
            bad()
