"""Inference settings, reasoning-channel stream formatter, vocabulary compaction and image preprocessing."""
import json

import numpy as np
import pytest
import torch

from pmetal_b200.data import inference_config as IC
from pmetal_b200.data.image_processing import (CLIP_MEAN, CLIP_STD, ImageProcessor, ImageProcessorConfig,
                                               MllamaTiledProcessor, SiglipImageProcessor, fit_to_canvas, optimal_canvas,
                                               supported_aspect_ratios)
from pmetal_b200.data.stream_format import StreamFormatter
from pmetal_b200.data.vocab_compact import VocabCompactor


class _Tok:
    """Word-level toy tokenizer with a few special tokens."""
    words = ["<pad>", "<think>", "</think>", "<|im_end|>", "</s>", "hello", "world", "let", "me", "see", "é"]
    eos_token_id = 4

    def token_to_id(self, t):
        return self.words.index(t) if t in self.words else None

    def encode_with_special_tokens(self, text):
        return [self.words.index(w) for w in text.split() if w in self.words]

    def decode(self, ids):
        return " ".join(self.words[i] for i in ids)


def test_sampling_resolution_order_and_stop_tokens(tmp_path):
    assert IC.load_sampling_defaults(None, "llama3") == IC.SamplingDefaults()
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"temperature": 0.3, "top_k": 50, "top_p": 0.9, "eos_token_id": [3, 4], "repetition_penalty": 1.05}))
    d = IC.load_sampling_defaults(str(tmp_path), "llama3")               # no family preset: the model's own values
    assert (d.temperature, d.top_k, d.top_p, d.repetition_penalty, d.presence_penalty) == (0.3, 50, 0.9, 1.05, 0.0)
    q = IC.load_sampling_defaults(str(tmp_path), "chatml", "auto", thinking=False)
    assert (q.temperature, q.top_p, q.presence_penalty) == (0.7, 0.8, 1.5)
    assert IC.load_sampling_defaults(str(tmp_path), "chatml", "auto", thinking=True).temperature == 1.0
    assert IC.load_sampling_defaults(str(tmp_path), "chatml", "coding").temperature == 0.6
    assert IC.load_sampling_defaults(str(tmp_path), "chatml", "reasoning").top_k == 40
    assert IC.available_modes("chatml") and not IC.available_modes("gemma")
    with pytest.raises(ValueError):
        IC.parse_mode("fast")
    assert IC.collect_all_stop_tokens(str(tmp_path), _Tok(), "<|im_end|>") == [3, 4]
    assert IC.collect_all_stop_tokens(None, _Tok(), None) == [3, 4]      # tokenizer eos + well-known tokens in the vocab

    class Bare(_Tok):
        words = ["a", "b"]
        eos_token_id = None
    assert IC.collect_all_stop_tokens(None, Bare(), None) == [2]


def test_stream_formatter_labels_or_hides_the_reasoning_channel():
    tok = _Tok()
    ids = [1, 7, 8, 9, 2, 5, 6]                                            # <think> let me see </think> hello world
    shown = StreamFormatter(tok, show_thinking=True)
    text = "".join(shown.push(i) for i in ids)
    assert text == "[thinking]\nlet me see\n\n[answer]\n hello world" and "<think>" not in text
    hidden = StreamFormatter(tok, show_thinking=False)
    assert "".join(hidden.push(i) for i in ids) == "hello world"
    plain = StreamFormatter(tok, show_thinking=False)                      # no reasoning channel at all
    assert "".join(plain.push(i) for i in [5, 6]) == "hello world"


def test_vocab_compactor_round_trip_and_gradient_scatter():
    samples = [[5, 9, 9, 2], [7, 5, -100, 300]]
    vc = VocabCompactor.from_dataset(samples, full_vocab=16)
    assert vc.compact_vocab == 4 and vc.compact_to_full.tolist() == [2, 5, 7, 9]
    ids = torch.tensor([5, 9, 2, 7, -100, 11])
    c = vc.to_compact(ids)
    assert c.tolist() == [1, 3, 0, 2, -100, 0]
    assert vc.to_full(c[:4]).tolist() == [5, 9, 2, 7]
    full = torch.arange(16 * 3, dtype=torch.float32).view(16, 3)
    small = vc.extract_rows(full)
    assert torch.equal(small, full[[2, 5, 7, 9]])
    g = torch.zeros(16, 3)
    vc.scatter_gradients(g, torch.ones(4, 3))
    assert g.sum() == 12 and g[5].tolist() == [1, 1, 1] and g[0].sum() == 0
    vc.update_full(full, small * 0)
    assert full[[2, 5, 7, 9]].abs().sum() == 0 and full[3].sum() > 0


def test_fixed_size_processors(tmp_path):
    from PIL import Image
    img = np.zeros((4, 4, 3), dtype=np.uint8)
    img[..., 0], img[..., 1], img[..., 2] = 128, 64, 192
    p = ImageProcessor(ImageProcessorConfig(size=(4, 4)))
    out = p.process_image(img)
    assert out.shape == (1, 3, 4, 4)
    for ch, v in enumerate((128, 64, 192)):
        assert torch.allclose(out[0, ch], torch.full((4, 4), (v / 255 - CLIP_MEAN[ch]) / CLIP_STD[ch]), atol=1e-6)
    path = tmp_path / "x.png"
    Image.fromarray(np.random.default_rng(0).integers(0, 255, (30, 50, 3), dtype=np.uint8)).save(path)
    big = ImageProcessor(ImageProcessorConfig(size=(20, 10))).preprocess(str(path))
    assert big.shape == (1, 3, 10, 20)
    s = SiglipImageProcessor((8, 8)).process_batch([img, img])
    assert s.shape == (2, 3, 8, 8) and torch.allclose(s[0, 0], torch.full((8, 8), (128 / 255 - 0.5) / 0.5), atol=1e-6)


def test_mllama_tiling_matches_hugging_face():
    tf = pytest.importorskip("transformers")
    from transformers.models.mllama import image_processing_mllama as hfm
    assert supported_aspect_ratios(4) == [tuple(x) for x in hfm.get_all_supported_aspect_ratios(4)]
    for h, w in [(100, 100), (300, 900), (900, 300), (224, 225), (1000, 1000), (50, 2000), (448, 448), (449, 300)]:
        ch, cw = hfm.get_optimal_tiled_canvas(h, w, 4, 224)
        ar = optimal_canvas(h, w, 4, 224)
        assert (ar[0] * 224, ar[1] * 224) == (int(ch), int(cw)), (h, w)
        assert fit_to_canvas(h, w, int(ch), int(cw), 224) == tuple(int(v) for v in
                                                                    hfm.get_image_size_fit_to_canvas(h, w, int(ch), int(cw), 224))
    rng = np.random.default_rng(1)
    imgs = [rng.integers(0, 255, (120, 300, 3), dtype=np.uint8), rng.integers(0, 255, (260, 90, 3), dtype=np.uint8),
            rng.integers(0, 255, (64, 64, 3), dtype=np.uint8)]
    ours = MllamaTiledProcessor(tile_size=64, max_image_tiles=4)([[imgs[0], imgs[1]], [imgs[2]]])
    hf = hfm.MllamaImageProcessor(size={"height": 64, "width": 64}, max_image_tiles=4, image_mean=list(CLIP_MEAN),
                                  image_std=list(CLIP_STD))
    ref = hf(images=[[imgs[0], imgs[1]], [imgs[2]]], return_tensors="pt")
    assert ours["pixel_values"].shape == ref["pixel_values"].shape == (2, 2, 4, 3, 64, 64)
    assert torch.equal(ours["aspect_ratio_ids"], ref["aspect_ratio_ids"])
    assert torch.equal(ours["aspect_ratio_mask"], ref["aspect_ratio_mask"])
    assert ours["num_tiles"] == ref["num_tiles"]
    diff = (ours["pixel_values"] - ref["pixel_values"]).abs()
    assert float(diff.max()) < 2.5 / 255 / min(CLIP_STD) and float(diff.mean()) < 2e-3      # resampling rounding only
