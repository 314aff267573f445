"""Image preprocessing for vision-language models.

* :class:`ImageProcessor`: resize to a fixed size (bilinear with antialiasing), NCHW float32, rescale by 1/255, per-channel
  normalisation; CLIP statistics by default, :class:`SiglipImageProcessor` uses mean = std = 0.5
  (crates/pmetal-data/src/image_processing.rs:12-245).
* :class:`MllamaTiledProcessor`: the tiled front end of Llama 3.2 Vision. An image is fitted to the tile arrangement
  ("aspect ratio", at most ``max_image_tiles`` tiles) that needs the least upscaling (or, when none fits, the least
  downscaling; ties go to the smaller canvas), resized without distortion, zero-padded to the canvas and cut into
  ``tile x tile`` tiles. Outputs are what ``models/architectures/mllama.py`` consumes: ``pixel_values``
  [B, images, max_tiles, 3, tile, tile], ``aspect_ratio_ids`` [B, images] (1-based index into the list of arrangements,
  0 = no image) and ``aspect_ratio_mask`` [B, images, max_tiles].

Images come in as file paths (decoded with Pillow), ``uint8`` arrays / tensors of shape [H, W, 3] or [3, H, W], or PIL
images; all arithmetic is done with torch, on whatever device the input tensor lives."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple, Union

import numpy as np
import torch
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def to_chw_uint8(image) -> torch.Tensor:
    """Path / PIL image / array / tensor -> uint8 tensor [3, H, W] (RGB)."""
    if isinstance(image, (str, bytes)) or hasattr(image, "__fspath__"):
        from PIL import Image
        with Image.open(image) as im:
            image = np.asarray(im.convert("RGB"))
    elif hasattr(image, "convert") and hasattr(image, "size") and not torch.is_tensor(image):
        image = np.asarray(image.convert("RGB"))
    t = torch.as_tensor(np.ascontiguousarray(image) if isinstance(image, np.ndarray) else image)
    if t.dim() == 2:
        t = t[None].expand(3, -1, -1)
    elif t.shape[-1] in (1, 3, 4) and t.shape[0] not in (1, 3):
        t = t.permute(2, 0, 1)
    if t.shape[0] == 1:
        t = t.expand(3, -1, -1)
    t = t[:3]
    if t.dtype != torch.uint8:
        t = (t.float() * (255.0 if t.is_floating_point() and float(t.max()) <= 1.0 else 1.0)).round().clamp(0, 255).to(torch.uint8)
    return t.contiguous()


def resize_uint8(img: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """Antialiased bilinear resize of a uint8 [3, H, W] image, rounded back to uint8."""
    if img.shape[-2:] == (height, width):
        return img
    y = F.interpolate(img[None].float(), size=(height, width), mode="bilinear", antialias=True, align_corners=False)
    return y[0].round().clamp(0, 255).to(torch.uint8)


@dataclass
class ImageProcessorConfig:
    size: Tuple[int, int] = (560, 560)                 # (width, height)
    mean: Tuple[float, float, float] = CLIP_MEAN
    std: Tuple[float, float, float] = CLIP_STD
    rescale_factor: float = 1.0 / 255.0


class ImageProcessor:
    def __init__(self, config: ImageProcessorConfig = None):
        self.config = config or ImageProcessorConfig()

    def normalize(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        mean = torch.tensor(c.mean, device=x.device).view(3, 1, 1)
        std = torch.tensor(c.std, device=x.device).view(3, 1, 1)
        return (x.float() * c.rescale_factor - mean) / std

    def process_image(self, image) -> torch.Tensor:
        """[1, 3, H, W] float32."""
        w, h = self.config.size
        return self.normalize(resize_uint8(to_chw_uint8(image), h, w))[None]

    preprocess = process_image

    def process_batch(self, images: Sequence) -> torch.Tensor:
        return torch.cat([self.process_image(i) for i in images], 0)


class SiglipImageProcessor(ImageProcessor):
    def __init__(self, size: Tuple[int, int] = (384, 384)):
        super().__init__(ImageProcessorConfig(size=size, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5)))


# ------------------------------------------------------------------------------------------------ mllama tiling
def supported_aspect_ratios(max_tiles: int) -> List[Tuple[int, int]]:
    """All (tiles high, tiles wide) with at most ``max_tiles`` tiles, ordered by height then width."""
    return [(h, w) for h in range(1, max_tiles + 1) for w in range(1, max_tiles + 1) if h * w <= max_tiles]


def optimal_canvas(height: int, width: int, max_tiles: int, tile: int) -> Tuple[int, int]:
    """(tiles high, tiles wide): least upscaling if any arrangement holds the image, else least downscaling; among equal
    scales the smallest area."""
    best = None
    cands = []
    for th, tw in supported_aspect_ratios(max_tiles):
        s = min(th * tile / height, tw * tile / width)
        cands.append((s, th * tw, (th, tw)))
    ups = [c for c in cands if c[0] >= 1]
    target = min(c[0] for c in ups) if ups else max(c[0] for c in cands)
    for s, area, ar in cands:
        if s == target and (best is None or area < best[0]):
            best = (area, ar)
    return best[1]


def fit_to_canvas(height: int, width: int, canvas_h: int, canvas_w: int, tile: int) -> Tuple[int, int]:
    """Size of the image inside the canvas: never below one tile per side before scaling, aspect ratio kept."""
    tw = min(max(width, tile), canvas_w)
    th = min(max(height, tile), canvas_h)
    sh, sw = th / height, tw / width
    if sw < sh:
        return min(math.floor(height * sw) or 1, th), tw
    return th, min(math.floor(width * sh) or 1, tw)


@dataclass
class MllamaTiledProcessor:
    tile_size: int = 560
    max_image_tiles: int = 4
    mean: Tuple[float, float, float] = CLIP_MEAN
    std: Tuple[float, float, float] = CLIP_STD
    rescale_factor: float = 1.0 / 255.0
    _norm: ImageProcessor = field(init=False, repr=False, default=None)

    def __post_init__(self):
        self._norm = ImageProcessor(ImageProcessorConfig((self.tile_size, self.tile_size), self.mean, self.std,
                                                         self.rescale_factor))

    def tiles_of(self, image) -> Tuple[torch.Tensor, Tuple[int, int]]:
        """([tiles, 3, tile, tile] float32 in row-major tile order, (tiles high, tiles wide))."""
        img = to_chw_uint8(image)
        H, W = img.shape[-2:]
        t = self.tile_size
        th, tw = optimal_canvas(H, W, self.max_image_tiles, t)
        nh, nw = fit_to_canvas(H, W, th * t, tw * t, t)
        img = resize_uint8(img, nh, nw)
        img = F.pad(img, (0, tw * t - nw, 0, th * t - nh))
        tiles = img.view(3, th, t, tw, t).permute(1, 3, 0, 2, 4).reshape(th * tw, 3, t, t)
        return self._norm.normalize(tiles), (th, tw)

    def __call__(self, images: Sequence[Union[Sequence, object]]) -> dict:
        """``images``: one list of images per sample (a bare image counts as a list of one)."""
        batch = [list(s) if isinstance(s, (list, tuple)) else [s] for s in images]
        B, M, T, t = len(batch), max(max(len(s) for s in batch), 1), self.max_image_tiles, self.tile_size
        ratios = supported_aspect_ratios(T)
        pixel = torch.zeros(B, M, T, 3, t, t)
        ids = torch.zeros(B, M, dtype=torch.int64)
        mask = torch.zeros(B, M, T, dtype=torch.int64)
        mask[:, :, 0] = 1                                # padding images keep their first tile visible
        num_tiles = []
        for b, sample in enumerate(batch):
            num_tiles.append([])
            for m, im in enumerate(sample):
                tiles, ar = self.tiles_of(im)
                n = tiles.shape[0]
                pixel[b, m, :n] = tiles
                ids[b, m] = ratios.index(ar) + 1
                mask[b, m, :n] = 1
                num_tiles[-1].append(n)
        return {"pixel_values": pixel, "aspect_ratio_ids": ids, "aspect_ratio_mask": mask, "num_tiles": num_tiles}
