import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = dict(architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=160,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5,
              rope_theta=10000.0, rope_scaling=None, max_position_embeddings=128, tie_word_embeddings=True,
              bos_token_id=1, eos_token_id=2)
TINY_B = dict(architectures=["LlamaForCausalLM"], vocab_size=384, hidden_size=192, intermediate_size=512,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6,
              rope_theta=500000.0,
              rope_scaling={"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 64},
              max_position_embeddings=512, tie_word_embeddings=False, bos_token_id=5, eos_token_id=[7, 9])
# sizes that are no power of two or multiple of 8: odd vocabulary, width, group of 5, head_dim 48
TINY_C = dict(architectures=["LlamaForCausalLM"], vocab_size=331, hidden_size=120, intermediate_size=200,
              num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=1, head_dim=48, rms_norm_eps=3e-6,
              rope_theta=25000.0,
              rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 2.0,
                            "original_max_position_embeddings": 32},
              max_position_embeddings=384, tie_word_embeddings=False, eos_token_id=0)

# sizes the tensor-core kernels refuse (width not a multiple of 8, head_dim not a multiple of 16):
# the bfloat16 path must fall to the CUDA-core kernels and still be right
TINY_D = dict(architectures=["LlamaForCausalLM"], vocab_size=257, hidden_size=100, intermediate_size=150,
              num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5, head_dim=20, rms_norm_eps=1e-5,
              rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=True, eos_token_id=[1, 2, 3])

# head_dim 64 (the smaller head size of the tensor-memory prompt attention), 3 query heads per KV head,
# widths that are multiples of 16 but no powers of two, a width that differs from heads x head_dim
TINY_E = dict(architectures=["LlamaForCausalLM"], vocab_size=389, hidden_size=208, intermediate_size=464,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=64, rms_norm_eps=2e-6,
              rope_theta=100000.0,
              rope_scaling={"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 128},
              max_position_embeddings=640, tie_word_embeddings=False, eos_token_id=3)

TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 5), "D": (TINY_D, 8), "E": (TINY_E, 11)}


@pytest.fixture
def pin():
    """pin(prompt_kernel="mma", ...) pins kernel choices (csrc/ops_tc.py: knobs) until the test ends,
    however it ends."""
    import contextlib
    from oracle_engine_b200.csrc import ops_tc
    with contextlib.ExitStack() as stack:
        yield lambda **kw: stack.enter_context(ops_tc.knobs(**kw))


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (config.json + model.safetensors) of the tiny configurations,
    written once per session into a temporary folder."""
    from oracle_engine_b200 import LlamaConfig, write_model_folder
    out = {}
    for name, (raw, seed) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_model_folder(d, LlamaConfig.from_dict(raw), seed=seed)
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    import plain_llama
    return {k: plain_llama.PlainLlama(v) for k, v in model_dirs.items()}
