"""Portable architecture implementations against the Hugging Face implementations of the same families: tiny random
models, identical weights (the checkpoint keys load as they are), logits compared; plus cache-consistency checks."""
import pytest
import torch

tf = pytest.importorskip("transformers")

from pmetal_b200.models.architectures.generic import GenericDecoderLM, arch_config_from_hf

BASE = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=256)

CASES = {
    "llama": ("LlamaForCausalLM", "LlamaConfig", dict(BASE)),
    "llama3_scaled": ("LlamaForCausalLM", "LlamaConfig", dict(BASE, rope_parameters=dict(
        rope_type="llama3", rope_theta=10000.0, factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
        original_max_position_embeddings=32))),
    "mistral": ("MistralForCausalLM", "MistralConfig", dict(BASE, sliding_window=8)),
    "mixtral": ("MixtralForCausalLM", "MixtralConfig", dict(BASE, num_local_experts=4, num_experts_per_tok=2)),
    "qwen2": ("Qwen2ForCausalLM", "Qwen2Config", dict(BASE)),
    "gemma": ("GemmaForCausalLM", "GemmaConfig", dict(BASE, head_dim=16)),
    "gemma2": ("Gemma2ForCausalLM", "Gemma2Config", dict(BASE, head_dim=16, sliding_window=8, query_pre_attn_scalar=24)),
    "gemma3": ("Gemma3ForCausalLM", "Gemma3TextConfig", dict(BASE, head_dim=16, sliding_window=8)),
    "phi3": ("Phi3ForCausalLM", "Phi3Config", dict(BASE, pad_token_id=0)),
    "phi": ("PhiForCausalLM", "PhiConfig", dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                                  num_attention_heads=4)),
    "cohere": ("CohereForCausalLM", "CohereConfig", dict(BASE, use_qk_norm=True)),
    "cohere2": ("Cohere2ForCausalLM", "Cohere2Config", dict(BASE, sliding_window=8)),
    "granite": ("GraniteForCausalLM", "GraniteConfig", dict(BASE, embedding_multiplier=3.0, residual_multiplier=0.5,
                                                            attention_multiplier=0.2, logits_scaling=2.0)),
    "granitemoe": ("GraniteMoeForCausalLM", "GraniteMoeConfig", dict(BASE, num_local_experts=4, num_experts_per_tok=2,
                                                                      attention_multiplier=0.2)),
    "olmo2": ("Olmo2ForCausalLM", "Olmo2Config", dict(BASE)),
    "gpt_oss": ("GptOssForCausalLM", "GptOssConfig", dict(BASE, head_dim=16, num_local_experts=4, num_experts_per_tok=2,
                                                          sliding_window=8)),
    "llama4": ("Llama4ForCausalLM", "Llama4TextConfig", dict(BASE, head_dim=16, intermediate_size_mlp=96,
                                                             num_local_experts=4, num_experts_per_tok=1,
                                                             attention_chunk_size=8, interleave_moe_layer_step=2,
                                                             floor_scale=4, attn_scale=0.1)),
    "qwen3_next": ("Qwen3NextForCausalLM", "Qwen3NextConfig", dict(
        BASE, head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
        shared_expert_intermediate_size=48, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
        linear_value_head_dim=8)),
    "deepseek_v2": ("DeepseekV2ForCausalLM", "DeepseekV2Config", dict(
        BASE, num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
        first_k_dense_replace=1, q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16)),
    "deepseek_v3": ("DeepseekV3ForCausalLM", "DeepseekV3Config", dict(
        BASE, num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, n_group=2,
        topk_group=1, first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
        v_head_dim=16)),
}


def _pair(name):
    cls, cfg_cls, kw = CASES[name]
    torch.manual_seed(0)
    cfg = getattr(tf, cfg_cls)(**kw, attn_implementation="eager")
    hf = getattr(tf, cls)(cfg).eval()
    with torch.no_grad():                       # move every parameter off its initial value (norm weights, biases, sinks)
        for p in hf.parameters():
            if p.dim() < 2:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.copy_(torch.randn_like(b) * 0.1)
    ours = GenericDecoderLM(arch_config_from_hf(cfg.to_dict())).eval()
    missing, unexpected = ours.load_state_dict(hf.state_dict(), strict=False)
    missing = [m for m in missing if "inv_freq" not in m]
    unexpected = [u for u in unexpected if "inv_freq" not in u and not (ours.c.tie_embeddings and u == "lm_head.weight")]
    assert not missing and not unexpected, (missing, unexpected)
    return hf, ours


@pytest.mark.parametrize("name", sorted(CASES))
def test_matches_hugging_face(name):
    hf, ours = _pair(name)
    ids = torch.randint(0, 128, (2, 24), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits.float()
        got = ours(ids).float()
    assert got.shape == ref.shape
    assert torch.allclose(got, ref, atol=2e-4, rtol=2e-3), float((got - ref).abs().max())


@pytest.mark.parametrize("name", ["llama", "gemma3", "cohere2", "gpt_oss", "llama4", "deepseek_v3", "qwen3_next"])
def test_cached_decode_equals_full_forward(name):
    _, ours = _pair(name)
    ids = torch.randint(0, 128, (1, 20), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        full = ours(ids)
        cache = ours.new_cache()
        a = ours(ids[:, :13], cache)
        steps = [ours(ids[:, t:t + 1], cache) for t in range(13, 20)]
    inc = torch.cat([a] + steps, 1)
    assert torch.allclose(inc, full, atol=2e-4, rtol=2e-3), float((inc - full).abs().max())
    assert len(ours.generate(ids[0, :5].tolist(), max_new_tokens=4)) == 4


# ---------------------------------------------------------------------------------------------- encoders
def _load(ours, hf, allow_unexpected=()):
    missing, unexpected = ours.load_state_dict(hf.state_dict(), strict=False)
    unexpected = [u for u in unexpected if not any(a in u for a in allow_unexpected)]
    assert not missing and not unexpected, (missing, unexpected)


def test_bert_matches_hugging_face_and_pools():
    from pmetal_b200.models.architectures.encoders import BertModel
    torch.manual_seed(0)
    cfg = tf.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                        max_position_embeddings=64, attn_implementation="eager")
    hf = tf.BertModel(cfg).eval()
    ours = BertModel(cfg.to_dict()).eval()
    _load(ours, hf, ("position_ids",))
    ids = torch.randint(0, 100, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[1, 8:] = 0
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask)
        got = ours(ids, mask)
    assert torch.allclose(got[0], ref.last_hidden_state[0], atol=1e-5)
    assert torch.allclose(got[1, :8], ref.last_hidden_state[1, :8], atol=1e-5)
    assert torch.allclose(ours.pool(got, mask, "pooler", normalize=False), ref.pooler_output, atol=1e-5)
    mean = ours.pool(got, mask, "mean")
    assert torch.allclose(mean.norm(dim=-1), torch.ones(2), atol=1e-5)
    assert torch.allclose(ours.pool(got, mask, "last", False)[1], got[1, 7])


def test_t5_matches_hugging_face():
    from pmetal_b200.models.architectures.encoders import T5Model
    torch.manual_seed(0)
    for proj, tie in (("gated-gelu", False), ("relu", True)):
        cfg = tf.T5Config(vocab_size=100, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4, feed_forward_proj=proj,
                          tie_word_embeddings=tie, decoder_start_token_id=0)
        hf = tf.T5ForConditionalGeneration(cfg).eval()
        ours = T5Model(dict(cfg.to_dict(), tie_word_embeddings=tie)).eval()
        _load(ours, hf, ("lm_head",) if tie else ())
        src, tgt = torch.randint(0, 100, (2, 11)), torch.randint(0, 100, (2, 7))
        with torch.no_grad():
            ref = hf(input_ids=src, decoder_input_ids=tgt).logits
            got = ours(src, tgt)
        assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), float((got - ref).abs().max())


def test_clip_matches_hugging_face():
    from pmetal_b200.models.architectures.encoders import ClipModel
    torch.manual_seed(0)
    cfg = tf.CLIPConfig(text_config=dict(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                         num_attention_heads=4, max_position_embeddings=16, eos_token_id=2),
                        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                           num_attention_heads=4, image_size=32, patch_size=8), projection_dim=24)
    hf = tf.CLIPModel(cfg).eval()
    ours = ClipModel(cfg.to_dict()).eval()
    _load(ours, hf, ("position_ids",))
    ids = torch.randint(3, 99, (3, 9))
    ids[:, -1] = 99                                  # the end-of-text token has the highest id
    px = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        ref = hf(input_ids=ids, pixel_values=px)
        per_image, per_text = ours(ids, px)
    assert torch.allclose(per_image, ref.logits_per_image, atol=1e-4)
    assert torch.allclose(per_text, ref.logits_per_text, atol=1e-4)


def test_whisper_matches_hugging_face():
    from pmetal_b200.models.architectures.encoders import WhisperModel
    torch.manual_seed(0)
    cfg = tf.WhisperConfig(vocab_size=100, d_model=32, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                           decoder_attention_heads=4, encoder_ffn_dim=64, decoder_ffn_dim=64, num_mel_bins=16,
                           max_source_positions=50, max_target_positions=32, pad_token_id=0, bos_token_id=1,
                           eos_token_id=2, decoder_start_token_id=1, suppress_tokens=None, begin_suppress_tokens=None)
    hf = tf.WhisperForConditionalGeneration(cfg).eval()
    ours = WhisperModel(cfg.to_dict()).eval()
    _load(ours, hf, ("proj_out",))
    mel, tgt = torch.randn(2, 16, 100), torch.randint(0, 100, (2, 6))
    with torch.no_grad():
        ref = hf(input_features=mel, decoder_input_ids=tgt).logits
        got = ours(mel, tgt)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-3), float((got - ref).abs().max())
    assert len(ours.transcribe(mel[:1], [1], max_new_tokens=3)) == 4


def test_nemotron_h_matches_hugging_face_and_cache():
    from pmetal_b200.models.architectures.hybrid import NemotronHLM
    torch.manual_seed(0)
    cfg = tf.NemotronHConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=6,
                             layers_block_type=["mamba", "moe", "attention", "moe", "mamba", "moe"],
                             n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1, moe_intermediate_size=32,
                             moe_shared_expert_intermediate_size=48, num_attention_heads=4, num_key_value_heads=2, head_dim=16, mamba_num_heads=8,
                             mamba_head_dim=8, ssm_state_size=16, n_groups=2, chunk_size=8, attn_implementation="eager")
    hf = tf.NemotronHForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() < 2:
                p.add_(torch.randn_like(p) * 0.05)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.copy_(torch.randn_like(b) * 0.1)
    ours = NemotronHLM(cfg.to_dict()).eval()
    missing, unexpected = ours.load_hf_state_dict(hf.state_dict(), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    ids = torch.randint(0, 128, (2, 19))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits
        got = ours(ids)
        cache = ours.new_cache()
        inc = torch.cat([ours(ids[:, :11], cache)] + [ours(ids[:, t:t + 1], cache) for t in range(11, 19)], 1)
    assert torch.allclose(got, ref, atol=3e-4, rtol=2e-3), float((got - ref).abs().max())
    assert torch.allclose(inc, got, atol=3e-4, rtol=2e-3), float((inc - got).abs().max())
    # the plain squared-ReLU block type (no counterpart in the installed Hugging Face version)
    mlp_only = NemotronHLM(dict(cfg.to_dict(), layers_block_type=["mamba", "mlp"])).eval()
    assert mlp_only(ids).shape == (2, 19, 128)


def test_registry_resolves_families_and_loads_from_disk(tmp_path):
    import json
    from pmetal_b200.models.architectures import build_model, family_of, load_pretrained
    from pmetal_b200.utils.safetensors_io import save_file
    assert family_of({"model_type": "qwen3"}) == "fast" and family_of({"model_type": "gemma2"}) == "generic"
    assert family_of({"model_type": "nemotron_h"}) == "nemotron_h" and family_of({"model_type": "roberta"}) == "bert"
    assert family_of({"architectures": ["Phi3ForCausalLM"]}) == "generic" and family_of({"model_type": "nope"}) is None
    assert family_of({"model_type": "gemma3", "text_config": {"model_type": "gemma3_text"}}) == "generic"
    with pytest.raises(ValueError):
        build_model({"model_type": "nope"})
    # a Mixtral checkpoint with one tensor per expert (the layout of the published files) loads into the stacked form
    cfg = tf.MixtralConfig(**dict(BASE, num_local_experts=4, num_experts_per_tok=2))
    hf = tf.MixtralForCausalLM(cfg).eval()
    sd = {}
    for k, v in hf.state_dict().items():
        if k.endswith("mlp.experts.gate_up_proj"):
            pre = k[: -len("mlp.experts.gate_up_proj")]
            for e in range(4):
                sd[f"{pre}block_sparse_moe.experts.{e}.w1.weight"] = v[e, :96].clone()
                sd[f"{pre}block_sparse_moe.experts.{e}.w3.weight"] = v[e, 96:].clone()
        elif k.endswith("mlp.experts.down_proj"):
            pre = k[: -len("mlp.experts.down_proj")]
            for e in range(4):
                sd[f"{pre}block_sparse_moe.experts.{e}.w2.weight"] = v[e].clone()
        elif k.endswith("mlp.gate.weight"):
            sd[k.replace("mlp.gate.", "block_sparse_moe.gate.")] = v.clone()
        else:
            sd[k] = v.clone()
    d = tmp_path / "mixtral"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg.to_dict()))
    save_file(sd, str(d / "model.safetensors"))
    ours = load_pretrained(str(d)).eval()
    ids = torch.randint(0, 128, (1, 9))
    with torch.no_grad():
        assert torch.allclose(ours(ids), hf(input_ids=ids).logits, atol=2e-4, rtol=2e-3)


def test_vision_towers_match_hugging_face_and_wrapper_splices_features():
    from pmetal_b200.models.architectures.vision import PixtralVision, Qwen2VLVision, build_vision_language
    torch.manual_seed(0)
    pc = tf.PixtralVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                image_size=32, patch_size=8, head_dim=8, attn_implementation="eager")
    hf = tf.PixtralVisionModel(pc).eval()
    ours = PixtralVision(pc.to_dict()).eval()
    _load(ours, hf)
    imgs = [torch.randn(3, 32, 32), torch.randn(3, 16, 24)]
    with torch.no_grad():
        ref = hf(pixel_values=torch.stack([imgs[0]]), image_sizes=[(32, 32)]).last_hidden_state[0]
        got = ours(imgs[:1])
        both = ours(imgs)
    assert torch.allclose(got, ref, atol=2e-5), float((got - ref).abs().max())
    assert torch.allclose(both[:16], got, atol=2e-5) and both.shape == (16 + 6, 32)    # images do not see each other

    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
    from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel
    vc = Qwen2VLVisionConfig(depth=2, embed_dim=32, hidden_size=48, mlp_ratio=2, num_heads=4, patch_size=4,
                             spatial_merge_size=2, temporal_patch_size=2)
    vc._attn_implementation = "eager"
    hv = Qwen2VisionTransformerPretrainedModel(vc).eval()
    ov = Qwen2VLVision(vc.to_dict()).eval()
    _load(ov, hv)
    grid = [(1, 4, 6), (1, 2, 2)]
    patches = torch.randn(4 * 6 + 2 * 2, 3 * 2 * 4 * 4)
    with torch.no_grad():
        ref = hv(patches, grid_thw=torch.tensor(grid))
        ref = ref.pooler_output if hasattr(ref, "pooler_output") else ref
        got = ov(patches, grid)
    assert got.shape == (7, 48) and torch.allclose(got, ref, atol=2e-5), float((got - ref).abs().max())

    vlm = build_vision_language({"model_type": "pixtral", "image_token_index": 5, "vision_config": pc.to_dict(),
                                 "text_config": dict(BASE, model_type="mistral")}).eval()
    ids = torch.randint(6, 128, (1, 30))
    ids[0, 3:19] = 5                                           # sixteen placeholders for a 4 x 4 patch image
    with torch.no_grad():
        feats = vlm.vision_tower([torch.randn(3, 32, 32)])
        out = vlm(ids, feats)
        out2 = vlm(ids, feats * 2)
    assert out.shape == (1, 30, 128) and not torch.allclose(out[0, 20:], out2[0, 20:])
    assert torch.allclose(out[0, :3], out2[0, :3])             # causal: tokens before the image are unaffected
    with pytest.raises(ValueError):
        vlm(ids, feats[:5])


def test_dflash_block_drafting_equals_greedy_decoding():
    from pmetal_b200.models.dflash import DFlashConfig, DFlashDecoder, DFlashDraftModel
    torch.manual_seed(0)
    target = GenericDecoderLM.from_hf_config(dict(BASE, model_type="qwen3", head_dim=16)).init_weights(0.05, 1).eval()
    dc = DFlashConfig.from_dict(dict(hidden_size=64, num_hidden_layers=2, intermediate_size=96, num_attention_heads=4,
                                     num_key_value_heads=2, head_dim=16, vocab_size=128, block_size=6,
                                     dflash_config=dict(target_layer_ids=[1, 3], mask_token_id=127)))
    draft = DFlashDraftModel(dc).eval()
    assert draft.fc.weight.shape == (64, 128)
    prompt = torch.randint(0, 120, (11,)).tolist()
    greedy = target.generate(prompt, max_new_tokens=24)
    dec = DFlashDecoder(target, draft)
    out = dec.generate(prompt, max_new_tokens=24)
    dec.close()
    assert out == greedy                                       # whatever the untrained draft proposes
    assert dec.stats.total_drafted > 0 and all(1 <= a <= 6 for a in dec.stats.acceptance_lengths)
    # a draft that cannot be wrong: block size 1 degenerates to one verified token per step
    dec1 = DFlashDecoder(target, draft)
    assert dec1.generate(prompt, 10, block_size=1) == greedy[:10] and dec1.stats.total_accepted == 0
    dec1.close()


def test_flux_transformer_and_autoencoder():
    from pmetal_b200.models.architectures import build_model
    from pmetal_b200.models.architectures.diffusion import (AutoencoderKL, FluxTransformer, flow_match_sample, flow_sigmas,
                                                            pack_latents, rope_nd, timestep_embedding, unpack_latents)
    torch.manual_seed(0)
    cfg = dict(model_type="flux", num_attention_heads=2, attention_head_dim=16, axes_dims_rope=(4, 6, 6), in_channels=16,
               joint_attention_dim=24, pooled_projection_dim=12, num_layers=2, num_single_layers=2, guidance_embeds=True)
    m = build_model(cfg).eval()
    assert isinstance(m, FluxTransformer)
    names = set(m.state_dict())
    for key in ("x_embedder.weight", "time_text_embed.guidance_embedder.linear_1.weight",
                "transformer_blocks.0.attn.add_k_proj.weight", "transformer_blocks.1.ff.net.0.proj.weight",
                "transformer_blocks.0.norm1_context.linear.bias", "single_transformer_blocks.1.proj_out.weight",
                "single_transformer_blocks.0.attn.norm_q.weight", "norm_out.linear.weight", "proj_out.bias"):
        assert key in names, key
    z = torch.randn(1, 4, 8, 12)
    p, ids = pack_latents(z)
    assert p.shape == (1, 24, 16) and torch.equal(unpack_latents(p, 8, 12), z) and ids[7].tolist() == [0, 1, 1]
    text, pooled = torch.randn(1, 5, 24), torch.randn(1, 12)
    t = torch.tensor([0.7])
    with torch.no_grad():
        v = m(p, text, pooled, t, ids, torch.zeros(5, 3), torch.tensor([3.5]))
        # permuting the image tokens together with their position ids permutes the output the same way
        perm = torch.randperm(24)
        v2 = m(p[:, perm], text, pooled, t, ids[perm], torch.zeros(5, 3), torch.tensor([3.5]))
    assert v.shape == (1, 24, 16) and torch.allclose(v[:, perm], v2, atol=1e-5)
    # zero gates (adaptive-norm projections at zero) make every block the identity on the residual stream
    with torch.no_grad():
        for n, prm in m.named_parameters():
            if "norm1" in n or ".norm.linear" in n:
                prm.zero_()
        x0 = m.x_embedder(p)
        emb = m.time_text_embed(t * 1000, torch.tensor([3500.0]), pooled)
        cos, sin = rope_nd(torch.cat((torch.zeros(5, 3), ids)), m.axes_dim)
        x1, _ = m.transformer_blocks[0](x0, m.context_embedder(text), emb, cos, sin)
    assert torch.allclose(x0, x1)
    e = timestep_embedding(torch.tensor([0.0, 500.0]), 8)
    assert torch.allclose(e[0], torch.tensor([1.0, 1, 1, 1, 0, 0, 0, 0])) and abs(float(e[1, 4]) - float(torch.sin(torch.tensor(500.0)))) < 1e-4
    s = flow_sigmas(4, 3.0)
    assert s[0] == 1 and s[-1] == 0 and (s[:-1] > s[1:]).all() and s[2] > 0.5      # the shift spends more steps at high noise
    out = flow_match_sample(m, torch.randn(1, 4, 8, 12), text, pooled, steps=2, guidance=3.5)
    assert out.shape == (1, 4, 8, 12) and torch.isfinite(out).all()

    vae = AutoencoderKL(dict(block_out_channels=(8, 16), layers_per_block=1, latent_channels=4, norm_num_groups=4)).eval()
    for key in ("encoder.down_blocks.0.downsamplers.0.conv.weight", "decoder.up_blocks.0.upsamplers.0.conv.weight",
                "decoder.mid_block.attentions.0.to_q.weight", "encoder.conv_out.weight", "decoder.up_blocks.1.resnets.0.conv_shortcut.weight"):
        assert key in vae.state_dict(), key
    img = torch.randn(2, 3, 16, 16)
    with torch.no_grad():
        lat = vae.encode(img)
        rec = vae.decode(lat)
    assert lat.shape == (2, 4, 8, 8) and rec.shape == img.shape
    assert vae.encoder.conv_out.out_channels == 8                                 # mean and log-variance


def test_dflash_tree_verification():
    from pmetal_b200.models.dflash import (DFlashConfig, DFlashDecoder, DFlashDraftModel, build_tree, follow_verified_tree)
    # hand-checked tree: depth-1 candidates a (p .6), b (.3); depth-2 candidates c (.9), d (.1)
    lg = torch.log(torch.tensor([[0.6, 0.3, 0.05, 0.05], [0.02, 0.04, 0.9, 0.04]]))
    t = build_tree(lg, 4)
    # pop order: a (.6); then its child c under a (.54) beats sibling b (.3); then b; then c under b (.27) beats d under a (.024)
    assert t.tokens == [0, 2, 1, 2] and t.depths == [1, 2, 1, 2] and t.parents == [-1, 0, 1, 0, 3]
    assert t.children[0] == {0: 1, 1: 3} and t.children[1] == {2: 2} and t.children[3] == {2: 4}
    vis = t.visibility()
    assert vis[2].tolist() == [True, True, True, False, False] and vis[4].tolist() == [True, False, False, True, True]
    assert follow_verified_tree(t, [1, 9, 9, 2, 7]) == [0, 3, 4] and follow_verified_tree(t, [3, 0, 0, 0, 0]) == [0]
    assert build_tree(lg, 0).tokens == []
    torch.manual_seed(0)
    target = GenericDecoderLM.from_hf_config(dict(BASE, model_type="qwen3", head_dim=16)).init_weights(0.05, 1).eval()
    dc = DFlashConfig.from_dict(dict(hidden_size=64, num_hidden_layers=2, intermediate_size=96, num_attention_heads=4,
                                     num_key_value_heads=2, head_dim=16, vocab_size=128, block_size=5,
                                     dflash_config=dict(target_layer_ids=[1, 3], mask_token_id=127)))
    draft = DFlashDraftModel(dc).eval()
    prompt = torch.randint(0, 120, (9,)).tolist()
    greedy = target.generate(prompt, max_new_tokens=20)
    dec = DFlashDecoder(target, draft)
    out = dec.generate_tree(prompt, 20, tree_budget=8)
    dec.close()
    assert out == greedy
    assert all(1 <= a <= 5 for a in dec.stats.acceptance_lengths) and dec.stats.total_drafted > 0


# ---------------------------------------------------------------------------------------------- Gemma 4
GEMMA4 = {
    "dense": dict(),
    "k_eq_v": dict(attention_k_eq_v=True, num_global_key_value_heads=1),
    "shared_kv_wide": dict(num_kv_shared_layers=2, use_double_wide_mlp=True),
    "experts": dict(enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32,
                    hidden_size_per_layer_input=0),
}


def _gemma4_pair(name):
    from pmetal_b200.models.architectures.gemma4 import Gemma4LM
    kw = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=6, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=8, max_position_embeddings=256,
              vocab_size_per_layer_input=128, hidden_size_per_layer_input=8, final_logit_softcapping=30.0,
              layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2)
    kw.update(GEMMA4[name])
    torch.manual_seed(0)
    cfg = tf.Gemma4TextConfig(**kw, attn_implementation="eager")
    hf = tf.Gemma4ForCausalLM(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() < 2:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("layer_scalar"):
                b.copy_(1.0 + 0.2 * torch.randn_like(b))
    ours = Gemma4LM.from_hf_config(cfg.to_dict()).eval()
    missing, unexpected = ours.load_hf_state_dict(hf.state_dict(), strict=False)
    assert not [m for m in missing if "inv_" not in m] and not [u for u in unexpected if "inv_freq" not in u], (missing, unexpected)
    return hf, ours


@pytest.mark.parametrize("name", sorted(GEMMA4))
def test_gemma4_matches_hugging_face_and_cache(name):
    from pmetal_b200.models.architectures import build_model, family_of
    hf, ours = _gemma4_pair(name)
    ids = torch.randint(0, 128, (2, 24), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids, use_cache=True).logits.float()
        got = ours(ids).float()
        assert torch.allclose(got, ref, atol=2e-4, rtol=2e-3), float((got - ref).abs().max())
        cache = ours.new_cache()
        inc = torch.cat([ours(ids[:1, :13], cache)] + [ours(ids[:1, t:t + 1], cache) for t in range(13, 24)], 1)
    assert torch.allclose(inc, got[:1], atol=2e-4, rtol=2e-3), float((inc - got[:1]).abs().max())
    assert len(ours.generate(ids[0, :5].tolist(), max_new_tokens=3)) == 3
    d = hf.config.to_dict()
    assert family_of(d) == "gemma4" and family_of({"model_type": "gemma4", "text_config": d}) == "gemma4"
    assert type(build_model({"model_type": "gemma4", "text_config": d})).__name__ == "Gemma4LM"


# ---------------------------------------------------------------------------------------------- mllama
def test_mllama_matches_hugging_face_and_decodes_with_cached_image_keys():
    from pmetal_b200.models.architectures import build_model
    torch.manual_seed(0)
    vis = dict(hidden_size=32, attention_heads=4, intermediate_size=64, num_hidden_layers=4, num_global_layers=2,
               intermediate_layers_indices=[1, 3], image_size=28, patch_size=14, max_num_tiles=4, vision_output_dim=96,
               supported_aspect_ratios=[[1, 1], [1, 2], [2, 1], [2, 2]], num_channels=3)
    txt = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=5, num_attention_heads=4,
               num_key_value_heads=2, cross_attention_layers=[1, 3], max_position_embeddings=256, pad_token_id=0,
               rope_parameters=dict(rope_type="llama3", rope_theta=10000.0, factor=8.0, low_freq_factor=1.0,
                                    high_freq_factor=4.0, original_max_position_embeddings=32))
    cfg = tf.MllamaConfig(vision_config=vis, text_config=txt, attn_implementation="eager")
    hf = tf.MllamaForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() < 2:
                p.add_(torch.randn_like(p) * 0.3)          # opens the tanh gates, moves the norm weights
    ours = build_model(cfg.to_dict()).eval()
    assert type(ours).__name__ == "MllamaForConditionalGeneration"
    _load(ours, hf, allow_unexpected=("inv_freq",))

    g = torch.Generator().manual_seed(1)
    B, T = 2, 12
    ids = torch.randint(0, 128, (B, T), generator=g)
    pix = torch.randn(B, 1, 4, 3, 28, 28, generator=g)
    ar_ids = torch.tensor([[4], [2]])
    ar_mask = torch.tensor([[[1, 1, 1, 1]], [[1, 1, 0, 0]]])
    cam = torch.zeros(B, T, 1, 4)
    cam[0, 3:, 0, :] = 1                                         # tokens after the image token see its tiles
    cam[1, 5:, 0, :2] = 1
    with torch.no_grad():
        ref = hf(input_ids=ids, pixel_values=pix, aspect_ratio_ids=ar_ids, aspect_ratio_mask=ar_mask,
                 cross_attention_mask=cam).logits.float()
        vref = hf.model.vision_model(pix, ar_ids, ar_mask).last_hidden_state
        vgot = ours.model.vision_model(pix, ar_ids, ar_mask)
        assert torch.allclose(vgot, vref, atol=2e-4, rtol=2e-3), float((vgot - vref).abs().max())
        got = ours(ids, pix, ar_ids, ar_mask, cam).float()
        assert torch.allclose(got, ref, atol=3e-4, rtol=2e-3), float((got - ref).abs().max())
        # incremental: image keys computed once with the prompt, then reused from the cache
        cache = ours.new_cache()
        a = ours(ids[:, :8], pix, ar_ids, ar_mask, cam[:, :8], cache)
        rest = [ours(ids[:, t:t + 1], cross_attention_mask=cam[:, :t + 1], cache=cache) for t in range(8, T)]
        inc = torch.cat([a] + rest, 1)
        assert torch.allclose(inc, got, atol=3e-4, rtol=2e-3), float((inc - got).abs().max())
        # text-only use skips the cross-attention layers, as the checkpoint's own code does
        t_ref = hf(input_ids=ids).logits
        assert torch.allclose(ours(ids), t_ref, atol=3e-4, rtol=2e-3)
    out = ours.generate(ids[0, :6].tolist(), 3, pixel_values=pix[:1], aspect_ratio_ids=ar_ids[:1],
                        aspect_ratio_mask=ar_mask[:1], cross_attention_mask=cam[:1, :6])
    assert len(out) == 3


def test_quantised_kv_cache_tracks_the_exact_cache():
    from pmetal_b200.models.architectures.generic import QuantKVCache
    _, ours = _pair("llama")
    ids = torch.randint(0, 128, (1, 24), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        full = ours(ids)
        errs = {}
        for name, kw in (("q8", dict(kv_bits=8, kv_group=16)), ("q4", dict(kv_bits=4, kv_group=16)),
                         ("tq4", dict(kv_bits=4, turbo=True)), ("tq2_qjl", dict(kv_bits=2, turbo=True, qjl=True))):
            cache = ours.new_cache(**kw)
            assert isinstance(cache, QuantKVCache)
            out = torch.cat([ours(ids[:, :16], cache)] + [ours(ids[:, t:t + 1], cache) for t in range(16, 24)], 1)
            errs[name] = float((out - full).abs().max() / full.abs().max())
            assert cache.length() == 24 and cache.nbytes() > 0
            if name == "q8":
                exact = sum(2 * 24 * 2 * 16 * 4 for _ in range(4))        # layers x (k,v) x tokens x kv heads x head dim x fp32
                assert cache.nbytes() < 0.45 * exact
    assert errs["q8"] < 0.02 and errs["q4"] < 0.2 and errs["tq4"] < 0.3 and errs["q8"] < errs["q4"], errs
    assert len(ours.generate(ids[0, :6].tolist(), 4, kv_bits=8)) == 4
