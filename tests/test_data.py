"""Datasets, two-crop augmentation and the loader that lives in a child process."""
import os

import pytest
import torch

from tspipe_b200.dataloader import SuperFastDataLoader
from tspipe_b200.datasets import GaussianBlur, ImageList, Solarize, TwoCropsTransform, annotation_list, imagenet_subset


def _make_images(root, classes=("n01", "n02", "n03"), per=2):
    from PIL import Image
    for c in classes:
        d = os.path.join(root, "train", c)
        os.makedirs(d)
        for i in range(per):
            Image.new("RGB", (20, 16), (i * 40, 10, 200)).save(os.path.join(d, f"{i}.jpg"))


def test_two_crops_and_pil_augmentations(tmp_path):
    from PIL import Image
    img = Image.new("RGB", (32, 32), (120, 30, 200))
    t = TwoCropsTransform(lambda x: "a", lambda x: "b")
    assert t(img) == ["a", "b"]
    assert GaussianBlur([0.1, 2.0])(img).size == (32, 32)
    assert Solarize()(img).getpixel((0, 0)) == (120, 30, 55)


def test_imagenet_subset_and_annotation_list(tmp_path):
    import torchvision.transforms as T
    _make_images(str(tmp_path))
    ds = imagenet_subset(str(tmp_path), "train", T.ToTensor(), classes=["n03", "n01"])
    assert len(ds) == 4 and sorted(set(ds.targets)) == [0, 1]
    x, y = ds[0]
    assert x.shape == (3, 16, 20) and y in (0, 1)
    os.makedirs(tmp_path / "images")
    from PIL import Image
    Image.new("RGB", (8, 8)).save(tmp_path / "images" / "cat_1.jpg")
    (tmp_path / "train.txt").write_text("cat_1 3 1 1\n")
    lst = annotation_list(str(tmp_path), "train.txt", transform=T.ToTensor())
    assert isinstance(lst, ImageList) and len(lst) == 1 and lst[0][1] == 2


def test_loader_in_child_process():
    ds = torch.utils.data.TensorDataset(torch.arange(12.).view(12, 1))
    loader = SuperFastDataLoader(ds, batch_size=5, epochs=1)
    assert len(loader) == 3
    seen = torch.cat([b[0] for b in loader])
    torch.testing.assert_close(seen.view(-1), torch.arange(12.))
