"""Makes tests/golden/tiny_qwen2_reference.npz: logits of the REFERENCE's own model code
(slipstream.models.loader.load_model + QwenForCausalLM with its NaiveKVCache, float32, CPU)
on a tiny random Qwen2.5 folder written by this package's random-weights mode.

Run once where the reference checkout is readable:

    python tests/golden/make_golden.py /path/to/reference

The folder's tensors are stored in the .npz too, so the comparison in
tests/test_plain_reference.py needs neither the reference nor the random generator.
"""
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
sys.dont_write_bytecode = True


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from slipstream.memory.contiguous_cache import NaiveKVCache  # the reference's modules
    from slipstream.models.loader import load_model

    from slipstream_b200.config.model_config import Qwen2Config
    from slipstream_b200.weights.random_init import write_random_model

    out = {}
    cases = {
        "tied": Qwen2Config(vocab_size=96, hidden_size=48, num_hidden_layers=2, max_position_embeddings=64,
                            torch_dtype="float32", intermediate_size=80, num_attention_heads=3,
                            num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0,
                            tie_word_embeddings=True),
        "untied": Qwen2Config(vocab_size=80, hidden_size=32, num_hidden_layers=3, max_position_embeddings=64,
                              torch_dtype="float32", intermediate_size=56, num_attention_heads=2,
                              num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, rope_theta=1000000.0,
                              tie_word_embeddings=False),
    }
    for name, config in cases.items():
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(config, folder, seed=7)
            tokens = torch.randint(0, config.vocab_size, (1, 23), generator=torch.Generator().manual_seed(3))
            model = load_model(folder, dtype=torch.float32).eval()
            cache = NaiveKVCache(config.num_hidden_layers, config.num_key_value_heads, config.head_dim, 1, 64,
                                 torch.float32, torch.device("cpu"))
            with torch.inference_mode():
                logits = model(tokens, torch.arange(23).unsqueeze(0), cache)[0]
            from safetensors import safe_open
            with safe_open(str(Path(folder) / "model.safetensors"), framework="pt") as handle:
                for key in handle.keys():
                    out[f"{name}/w/{key}"] = handle.get_tensor(key).numpy()
            out[f"{name}/config"] = np.frombuffer((Path(folder) / "config.json").read_bytes(), dtype=np.uint8)
            out[f"{name}/tokens"] = tokens[0].numpy()
            out[f"{name}/logits"] = logits.numpy()
    np.savez_compressed(Path(__file__).parent / "tiny_qwen2_reference.npz", **out)
    print("wrote", Path(__file__).parent / "tiny_qwen2_reference.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
