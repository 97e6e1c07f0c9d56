"""Image-folder dataset with the ImageNet training pipeline of the reference's vision entry points:
random-resized crop, horizontal flip, colour jitter, the fixed AutoAugment ImageNet policy, normalisation to
[-1, 1] (reference: runtime/megatron/data/vit_dataset.py:22-57 builds the same chain from torchvision transforms and
runtime/megatron/data/autoaugment.py; the policy is Table 9 of "AutoAugment: Learning Augmentation Policies from
Data", arXiv:1805.09501).

Differences by design:
  * every random decision of sample i in epoch e comes from a generator seeded by (seed, e, i), so a run that is
    resumed, or split over a different number of data-parallel ranks, sees the same pictures;
  * samples come out channels-last (H, W, 3), the layout the convolution kernels of this framework use, and
    `image_batch` stacks a global batch into the {"images", "labels"} dictionary the Wide-ResNet trainer takes;
  * only Pillow is needed (torchvision is not imported).

Directory layout: `root/<class name>/<image file>`, classes numbered in sorted order (as torchvision's ImageFolder).
"""
from __future__ import annotations

import math
import os
import random
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

EXTENSIONS = (".jpg", ".jpeg", ".png", ".ppm", ".bmp", ".pgm", ".tif", ".tiff", ".webp")

# (operation, probability, magnitude 0..10) pairs of the 25 ImageNet sub-policies
IMAGENET_POLICY: Tuple[Tuple[Tuple[str, float, int], Tuple[str, float, int]], ...] = (
    (("posterize", 0.4, 8), ("rotate", 0.6, 9)), (("solarize", 0.6, 5), ("autocontrast", 0.6, 5)),
    (("equalize", 0.8, 8), ("equalize", 0.6, 3)), (("posterize", 0.6, 7), ("posterize", 0.6, 6)),
    (("equalize", 0.4, 7), ("solarize", 0.2, 4)), (("equalize", 0.4, 4), ("rotate", 0.8, 8)),
    (("solarize", 0.6, 3), ("equalize", 0.6, 7)), (("posterize", 0.8, 5), ("equalize", 1.0, 2)),
    (("rotate", 0.2, 3), ("solarize", 0.6, 8)), (("equalize", 0.6, 8), ("posterize", 0.4, 6)),
    (("rotate", 0.8, 8), ("color", 0.4, 0)), (("rotate", 0.4, 9), ("equalize", 0.6, 2)),
    (("equalize", 0.0, 7), ("equalize", 0.8, 8)), (("invert", 0.6, 4), ("equalize", 1.0, 8)),
    (("color", 0.6, 4), ("contrast", 1.0, 8)), (("rotate", 0.8, 8), ("color", 1.0, 2)),
    (("color", 0.8, 8), ("solarize", 0.8, 7)), (("sharpness", 0.4, 7), ("invert", 0.6, 8)),
    (("shear_x", 0.6, 5), ("equalize", 1.0, 9)), (("color", 0.4, 0), ("equalize", 0.6, 3)),
    (("equalize", 0.4, 7), ("solarize", 0.2, 4)), (("solarize", 0.6, 5), ("autocontrast", 0.6, 5)),
    (("invert", 0.6, 4), ("equalize", 1.0, 8)), (("color", 0.6, 4), ("contrast", 1.0, 8)),
    (("equalize", 0.8, 8), ("equalize", 0.6, 3)),
)


def _level(lo: float, hi: float, magnitude: int) -> float:
    return lo + (hi - lo) * magnitude / 10.0


def apply_operation(img, name: str, magnitude: int, rng: random.Random):
    """One AutoAugment operation at strength `magnitude` (0..10) on a PIL RGB image; signed operations pick their
    direction at random."""
    from PIL import Image, ImageEnhance, ImageOps
    sign = -1.0 if rng.random() < 0.5 else 1.0
    grey = (128, 128, 128)
    if name == "shear_x":
        return img.transform(img.size, Image.AFFINE, (1, sign * _level(0, 0.3, magnitude), 0, 0, 1, 0), Image.BICUBIC,
                             fillcolor=grey)
    if name == "shear_y":
        return img.transform(img.size, Image.AFFINE, (1, 0, 0, sign * _level(0, 0.3, magnitude), 1, 0), Image.BICUBIC,
                             fillcolor=grey)
    if name == "translate_x":
        return img.transform(img.size, Image.AFFINE, (1, 0, sign * _level(0, 0.45, magnitude) * img.size[0], 0, 1, 0),
                             fillcolor=grey)
    if name == "translate_y":
        return img.transform(img.size, Image.AFFINE, (1, 0, 0, 0, 1, sign * _level(0, 0.45, magnitude) * img.size[1]),
                             fillcolor=grey)
    if name == "rotate":
        return img.rotate(sign * _level(0, 30, magnitude), resample=Image.BICUBIC, fillcolor=grey)
    if name == "color":
        return ImageEnhance.Color(img).enhance(1.0 + sign * _level(0, 0.9, magnitude))
    if name == "contrast":
        return ImageEnhance.Contrast(img).enhance(1.0 + sign * _level(0, 0.9, magnitude))
    if name == "brightness":
        return ImageEnhance.Brightness(img).enhance(1.0 + sign * _level(0, 0.9, magnitude))
    if name == "sharpness":
        return ImageEnhance.Sharpness(img).enhance(1.0 + sign * _level(0, 0.9, magnitude))
    if name == "posterize":
        return ImageOps.posterize(img, int(round(_level(8, 4, magnitude))))
    if name == "solarize":
        return ImageOps.solarize(img, int(round(_level(256, 0, magnitude))))
    if name == "autocontrast":
        return ImageOps.autocontrast(img)
    if name == "equalize":
        return ImageOps.equalize(img)
    if name == "invert":
        return ImageOps.invert(img)
    raise ValueError(f"unknown augmentation {name!r}")


def autoaugment_imagenet(img, rng: random.Random):
    """One of the 25 sub-policies, chosen uniformly; each of its two operations fires with its own probability."""
    for name, prob, magnitude in IMAGENET_POLICY[rng.randrange(len(IMAGENET_POLICY))]:
        if rng.random() < prob:
            img = apply_operation(img, name, magnitude, rng)
    return img


def random_resized_crop(img, size: int, rng: random.Random, scale=(0.08, 1.0), ratio=(3.0 / 4.0, 4.0 / 3.0)):
    """A crop of random area (fraction of the picture in `scale`) and aspect ratio (log-uniform in `ratio`), resized
    to size x size; after ten failed draws the central crop of the nearest admissible ratio."""
    from PIL import Image
    w, h = img.size
    area = w * h
    for _ in range(10):
        target = area * rng.uniform(*scale)
        aspect = math.exp(rng.uniform(math.log(ratio[0]), math.log(ratio[1])))
        cw, ch = int(round(math.sqrt(target * aspect))), int(round(math.sqrt(target / aspect)))
        if 0 < cw <= w and 0 < ch <= h:
            x0, y0 = rng.randint(0, w - cw), rng.randint(0, h - ch)
            return img.resize((size, size), Image.BILINEAR, box=(x0, y0, x0 + cw, y0 + ch))
    aspect = min(max(w / h, ratio[0]), ratio[1])
    cw, ch = (w, int(round(w / aspect))) if w / h < aspect else (int(round(h * aspect)), h)
    cw, ch = min(cw, w), min(ch, h)
    x0, y0 = (w - cw) // 2, (h - ch) // 2
    return img.resize((size, size), Image.BILINEAR, box=(x0, y0, x0 + cw, y0 + ch))


def color_jitter(img, rng: random.Random, brightness=0.4, contrast=0.4, saturation=0.4, hue=0.1):
    """Brightness, contrast, saturation and hue changes in a random order, each by a random factor."""
    from PIL import Image, ImageEnhance
    steps = ["b", "c", "s", "h"]
    rng.shuffle(steps)
    for s in steps:
        if s == "b":
            img = ImageEnhance.Brightness(img).enhance(rng.uniform(1 - brightness, 1 + brightness))
        elif s == "c":
            img = ImageEnhance.Contrast(img).enhance(rng.uniform(1 - contrast, 1 + contrast))
        elif s == "s":
            img = ImageEnhance.Color(img).enhance(rng.uniform(1 - saturation, 1 + saturation))
        else:
            shift = int(round(rng.uniform(-hue, hue) * 255))
            hsv = np.array(img.convert("HSV"))
            hsv[..., 0] = (hsv[..., 0].astype(np.int16) + shift) % 256
            img = Image.fromarray(hsv, "HSV").convert("RGB")
    return img


def center_crop_resized(img, size: int):
    """Shorter side to `size`, then the central size x size window (the evaluation transform)."""
    from PIL import Image
    w, h = img.size
    s = size / min(w, h)
    img = img.resize((max(size, int(round(w * s))), max(size, int(round(h * s)))), Image.BILINEAR)
    w, h = img.size
    x0, y0 = (w - size) // 2, (h - size) // 2
    return img.crop((x0, y0, x0 + size, y0 + size))


def to_normalised_tensor(img, dtype=torch.bfloat16) -> torch.Tensor:
    """PIL RGB -> [H, W, 3] in [-1, 1] (mean 0.5, std 0.5 per channel)."""
    a = torch.from_numpy(np.asarray(img, dtype=np.uint8).copy())
    return ((a.to(torch.float32) / 255.0 - 0.5) / 0.5).to(dtype)


class ImageFolder:
    """`root/<class>/<file>` -> (channels-last tensor, class index).  `train=True` applies the augmentation chain with
    the generator of (seed, epoch, index); `train=False` the resize + centre crop."""

    def __init__(self, root: str, size: int = 224, train: bool = True, seed: int = 1234, jitter: bool = True,
                 autoaugment: bool = True, dtype=torch.bfloat16, loader: Optional[Callable] = None):
        self.root, self.size, self.train, self.seed = root, size, train, seed
        self.jitter, self.autoaugment, self.dtype = jitter, autoaugment, dtype
        self.classes: List[str] = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        if not self.classes:
            raise FileNotFoundError(f"no class directories under {root}")
        self.samples: List[Tuple[str, int]] = []
        for ci, c in enumerate(self.classes):
            for dirpath, _, files in sorted(os.walk(os.path.join(root, c))):
                for f in sorted(files):
                    if f.lower().endswith(EXTENSIONS):
                        self.samples.append((os.path.join(dirpath, f), ci))
        if not self.samples:
            raise FileNotFoundError(f"no image files under {root}")
        self._load = loader or self._pil_load
        self.epoch = 0

    @staticmethod
    def _pil_load(path: str):
        from PIL import Image
        with open(path, "rb") as f:
            return Image.open(f).convert("RGB")

    def __len__(self) -> int:
        return len(self.samples)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __getitem__(self, i: int):
        return self.sample(i, self.epoch)

    def sample(self, i: int, epoch: int):
        """Sample i as epoch `epoch` shows it (no state of the dataset is read, so threads may call this side by
        side for different epochs)."""
        path, label = self.samples[i]
        img = self._load(path)
        if self.train:
            rng = random.Random((self.seed * 1000003 + epoch) * 1000003 + i)
            img = random_resized_crop(img, self.size, rng)
            if rng.random() < 0.5:
                from PIL import ImageOps
                img = ImageOps.mirror(img)
            if self.jitter:
                img = color_jitter(img, rng)
            if self.autoaugment:
                img = autoaugment_imagenet(img, rng)
        else:
            img = center_crop_resized(img, self.size)
        return to_normalised_tensor(img, self.dtype), label


def image_batch(data: ImageFolder, indices: Sequence[int], pin: bool = False,
                epoch: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """{"images": [n, H, W, 3], "labels": [n]} for the Wide-ResNet trainer; `epoch` (default: the dataset's current
    one) selects the augmentation stream."""
    e = data.epoch if epoch is None else epoch
    items = [data.sample(int(i), e) for i in indices]
    out = {"images": torch.stack([x for x, _ in items]), "labels": torch.tensor([y for _, y in items], dtype=torch.int64)}
    return {k: v.pin_memory() for k, v in out.items()} if pin else out


def epoch_order(n: int, epoch: int, seed: int) -> np.ndarray:
    """The shuffled sample order of one epoch (a function of the seed and the epoch only)."""
    return np.random.RandomState((seed + 7919 * epoch) % (2 ** 31)).permutation(n)


def batch_indices(n: int, global_batch: int, iteration: int, seed: int) -> Tuple[np.ndarray, int]:
    """(indices of the global batch of training iteration `iteration` (0-based), its epoch): epochs are shuffled
    independently, the incomplete tail of an epoch is dropped, so iteration k always names the same pictures."""
    per_epoch = n // global_batch
    if per_epoch == 0:
        raise ValueError(f"{n} images do not fill one global batch of {global_batch}")
    epoch, k = divmod(iteration, per_epoch)
    return epoch_order(n, epoch, seed)[k * global_batch:(k + 1) * global_batch], epoch
