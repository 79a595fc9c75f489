"""Image datasets and the two-crop augmentation pipeline of the self-supervised entry points.

Counterparts of the reference's ``dataset/`` package: ``TwoCropsTransform`` / ``GaussianBlur`` /
``Solarize`` (`dataset/loader.py:13-42`), ``ImageNet100`` (an ``ImageFolder`` restricted to a class list,
`dataset/datasets.py:33-51`), ``ImageList`` and the small transfer sets built on it (`:17-31,53-103`).
The class list of ImageNet-100 is passed in (or read from a text file, one WordNet id per line) rather
than shipped.  BYOL's augmentation recipe follows `benchmarks/byol/main.py:65-92`.
"""
from __future__ import annotations

import os
import random
from typing import Callable, List, Optional, Sequence, Tuple

import torch


class TwoCropsTransform:
    """Two differently augmented views of one image."""

    def __init__(self, base_transform1: Callable, base_transform2: Callable):
        self.t1, self.t2 = base_transform1, base_transform2

    def __call__(self, x):
        return [self.t1(x), self.t2(x)]


class GaussianBlur:
    def __init__(self, sigma: Sequence[float] = (0.1, 2.0)):
        self.sigma = sigma

    def __call__(self, img):
        from PIL import ImageFilter
        return img.filter(ImageFilter.GaussianBlur(radius=random.uniform(self.sigma[0], self.sigma[1])))


class Solarize:
    def __call__(self, img):
        from PIL import ImageOps
        return ImageOps.solarize(img)


class ImageList(torch.utils.data.Dataset):
    """``samples`` = list of ``(path, label)``."""

    def __init__(self, samples: List[Tuple[str, int]], transform: Optional[Callable] = None):
        self.samples, self.transform = samples, transform

    def __getitem__(self, idx: int):
        from PIL import Image
        path, label = self.samples[idx]
        with open(path, "rb") as f:
            img = Image.open(f).convert("RGB")
        return (self.transform(img) if self.transform is not None else img), label

    def __len__(self) -> int:
        return len(self.samples)


def imagenet_subset(root: str, split: str, transform: Callable, classes: Optional[Sequence[str]] = None,
                    class_file: Optional[str] = None):
    """``ImageFolder(root/split)`` restricted to ``classes`` (ImageNet-100 when given its 100 ids)."""
    from torchvision.datasets import ImageFolder
    ds = ImageFolder(os.path.join(root, split), transform=transform)
    if classes is None and class_file is not None:
        with open(class_file) as f:
            classes = [l.strip() for l in f if l.strip()]
    if classes is None:
        return ds
    idx = {c: i for i, c in enumerate(classes)}
    ds.samples = [(p, idx[ds.classes[l]]) for p, l in ds.samples if ds.classes[l] in idx]
    ds.targets = [s[1] for s in ds.samples]
    ds.classes, ds.class_to_idx = list(classes), idx
    return ds


def annotation_list(root: str, annotation_file: str, image_dir: str = "images", transform: Optional[Callable] = None,
                    suffix: str = ".jpg", label_offset: int = -1) -> ImageList:
    """Transfer sets described by ``<name> <label> ...`` lines (Pets, Food-101, DTD, SUN397 style)."""
    samples = []
    with open(os.path.join(root, annotation_file)) as f:
        for line in f:
            parts = line.split()
            if len(parts) >= 2:
                name = parts[0] if parts[0].endswith(suffix) else parts[0] + suffix
                samples.append((os.path.join(root, image_dir, name), int(parts[1]) + label_offset))
    return ImageList(samples, transform)


def byol_augmentations(size: int = 224):
    import torchvision.transforms as T
    normalize = T.Normalize(mean=[0.485, 0.456, 0.406], std=[0.229, 0.224, 0.225])
    common = [T.RandomResizedCrop(size, scale=(0.08, 1.0)),
              T.RandomApply([T.ColorJitter(0.4, 0.4, 0.2, 0.1)], p=0.8), T.RandomGrayscale(p=0.2)]
    a1 = T.Compose(common + [T.RandomApply([GaussianBlur([0.1, 2.0])], p=1.0), T.RandomHorizontalFlip(), T.ToTensor(),
                             normalize])
    a2 = T.Compose(common + [T.RandomApply([GaussianBlur([0.1, 2.0])], p=0.1), T.RandomApply([Solarize()], p=0.2),
                             T.RandomHorizontalFlip(), T.ToTensor(), normalize])
    return a1, a2


def two_crop_imagefolder(root: str, name: str = "imagenet", class_file: Optional[str] = None, size: int = 224):
    a1, a2 = byol_augmentations(size)
    return imagenet_subset(root, "train", TwoCropsTransform(a1, a2), class_file=class_file)
