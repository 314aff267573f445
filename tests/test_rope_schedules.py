"""RoPE frequency schedules of the fast decoder against the Hugging Face reference implementation."""
import pytest
import torch


@pytest.mark.parametrize("scaling", [
    {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
     "original_max_position_embeddings": 64},
    {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64},
    {"type": "linear", "factor": 2.0},
])
def test_fast_decoder_rope_schedules_match_transformers(scaling):
    """Every RoPE schedule of the fast decoder gives the cos/sin tables of the Hugging Face implementation."""
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    from pmetal_b200.models.config import ModelArgs
    from pmetal_b200.models.decoder import DecoderLM
    kind = scaling.get("rope_type", scaling.get("type"))
    hf = dict(model_type="llama", vocab_size=64, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=256,
              rope_theta=10000.0, rope_scaling=dict(scaling))
    m = DecoderLM(ModelArgs.from_dict(hf))
    pos = torch.arange(0, 200, 7, dtype=torch.int32)
    cos, sin = m.rope(pos)
    cfg = LlamaConfig(**{k: v for k, v in hf.items() if k != "model_type"})
    try:
        inv, att = ROPE_INIT_FUNCTIONS[kind](cfg, "cpu", seq_len=256)
    except Exception as e:                                   # the installed transformers rejects this config form
        pytest.skip(f"transformers: {e}")
    ang = pos.float()[:, None] * inv[None, :]
    torch.testing.assert_close(cos, ang.cos() * att, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(sin, ang.sin() * att, atol=1e-5, rtol=1e-5)


def test_dynamic_ntk_matches_transformers_at_the_configured_length():
    """The static NTK stretch for a context of L tokens equals the Hugging Face dynamic schedule evaluated at seq_len = L."""
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    from pmetal_b200.models.rope import rope_inv_freq
    cfg = LlamaConfig(hidden_size=64, num_attention_heads=4, head_dim=16, max_position_embeddings=256, rope_theta=10000.0,
                      rope_scaling={"rope_type": "dynamic", "factor": 2.0})
    try:
        want, att = ROPE_INIT_FUNCTIONS["dynamic"](cfg, "cpu", seq_len=512)
    except Exception as e:
        pytest.skip(f"transformers: {e}")
    got, att2 = rope_inv_freq(16, 10000.0, {"rope_type": "dynamic", "factor": 2.0,
                                            "original_max_position_embeddings": 256}, 512)
    torch.testing.assert_close(got, want, atol=1e-7, rtol=1e-5)
    assert att == att2 == 1.0
