"""Image-folder pipeline: class numbering, deterministic augmentation, every AutoAugment operation, batches for the
Wide-ResNet trainer, and a training run fed from a folder of pictures."""
import os
import random

import numpy as np
import pytest
import torch

from superscaler_b200.data import images as I


def _make_folder(root, classes=("ant", "bee", "cat"), per_class=5, size=(40, 32)):
    from PIL import Image
    rs = np.random.RandomState(0)
    for c in classes:
        os.makedirs(os.path.join(root, "train", c))
        for k in range(per_class):
            a = rs.randint(0, 256, size=(size[1], size[0], 3), dtype=np.uint8)
            Image.fromarray(a, "RGB").save(os.path.join(root, "train", c, f"{k}.png"))
    return os.path.join(root, "train")


def test_classes_are_numbered_in_sorted_order_and_samples_are_repeatable(tmp_path):
    root = _make_folder(str(tmp_path))
    d = I.ImageFolder(root, size=24, train=True, seed=3)
    assert d.classes == ["ant", "bee", "cat"] and len(d) == 15
    assert [y for _, y in d.samples] == [0] * 5 + [1] * 5 + [2] * 5
    x0, y0 = d[7]
    x1, y1 = d[7]
    assert x0.shape == (24, 24, 3) and x0.dtype == torch.bfloat16 and y0 == y1 == 1
    assert torch.equal(x0, x1)                                   # same (seed, epoch, index): same picture
    assert float(x0.float().abs().max()) <= 1.0
    d.set_epoch(1)
    assert not torch.equal(d[7][0], x0)                          # another epoch: another crop / augmentation
    other = I.ImageFolder(root, size=24, train=True, seed=4)
    assert not torch.equal(other[7][0], x0)


def test_evaluation_transform_is_resize_and_centre_crop(tmp_path):
    root = _make_folder(str(tmp_path), size=(64, 48))
    d = I.ImageFolder(root, size=32, train=False)
    x, _ = d[0]
    from PIL import Image
    img = Image.open(d.samples[0][0]).convert("RGB")
    ref = I.to_normalised_tensor(I.center_crop_resized(img, 32))
    assert torch.equal(x, ref) and x.shape == (32, 32, 3)


def test_every_policy_operation_runs_and_keeps_the_size():
    from PIL import Image
    rs = np.random.RandomState(1)
    img = Image.fromarray(rs.randint(0, 256, size=(30, 30, 3), dtype=np.uint8), "RGB")
    names = {n for pair in I.IMAGENET_POLICY for n, _, _ in pair} | {"shear_y", "translate_x", "translate_y", "brightness"}
    for n in sorted(names):
        for m in (0, 5, 10):
            out = I.apply_operation(img, n, m, random.Random(m))
            assert out.size == img.size and out.mode == "RGB", n
    assert len(I.IMAGENET_POLICY) == 25
    # invert and solarize at full strength agree (threshold 0 flips every pixel)
    a = np.asarray(I.apply_operation(img, "invert", 0, random.Random(0)))
    b = np.asarray(I.apply_operation(img, "solarize", 10, random.Random(0)))
    assert np.array_equal(a, b)
    # magnitude 0 of the enhancement family leaves the picture as it is
    assert np.array_equal(np.asarray(I.apply_operation(img, "contrast", 0, random.Random(0))), np.asarray(img))


def test_batches_cover_an_epoch_once_and_iterations_are_addressable(tmp_path):
    root = _make_folder(str(tmp_path), per_class=6)
    d = I.ImageFolder(root, size=16, seed=5)
    seen = []
    for it in range(4):                                          # 18 pictures, batches of 4: four per epoch
        idx, epoch = I.batch_indices(len(d), 4, it, seed=5)
        assert epoch == 0
        seen += list(idx)
    assert len(set(seen)) == 16
    idx4, epoch4 = I.batch_indices(len(d), 4, 4, seed=5)
    assert epoch4 == 1
    again, _ = I.batch_indices(len(d), 4, 4, seed=5)
    assert np.array_equal(idx4, again)
    b = I.image_batch(d, idx4)
    assert b["images"].shape == (4, 16, 16, 3) and b["labels"].dtype == torch.int64
    with pytest.raises(ValueError):
        I.batch_indices(3, 4, 0, seed=1)


def test_wide_resnet_trains_from_an_image_folder(tmp_path):
    from helpers import tiny_resnet_plan
    from superscaler_b200.runtime.pretrain import make_image_batch_fn
    from superscaler_b200.runtime.trainer import Trainer
    root = _make_folder(str(tmp_path), per_class=6, size=(48, 48))
    plan = tiny_resnet_plan()
    t = Trainer(plan, device="cpu", lr=1e-2, lr_warmup_steps=0, model_overrides=dict(image_size=64, num_classes=8))
    fn = make_image_batch_fn(t, str(tmp_path), seed=11)
    losses = [t.loss_value(t.train_step(fn(i % 2))) for i in range(6)]
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]


def test_a_val_folder_becomes_the_held_out_batches(tmp_path):
    import shutil
    from helpers import tiny_resnet_plan
    from superscaler_b200.runtime.pretrain import make_image_batch_fn
    from superscaler_b200.runtime.trainer import Trainer
    root = _make_folder(str(tmp_path), per_class=6, size=(48, 48))
    t = Trainer(tiny_resnet_plan(), device="cpu", model_overrides=dict(image_size=64, num_classes=8))
    assert make_image_batch_fn(t, str(tmp_path), seed=11).valid is None
    shutil.copytree(root, os.path.join(str(tmp_path), "val"))
    fn = make_image_batch_fn(t, str(tmp_path), seed=11)
    a, b = fn.valid(0), fn.valid(0)
    gbs = t.plan["global_batch_size"]
    assert a["images"].shape == (gbs, 64, 64, 3) and torch.equal(a["images"], b["images"])
    assert a["labels"].tolist() == ([0] * 6 + [1] * 6 + [2] * 6 + [0] * 6 + [1] * 6 + [2] * 6)[:gbs]    # file order, wrapped
    ev = t.evaluate([t.to_device(a)])
    assert all(np.isfinite(v) for v in ev.values()) and 0.0 <= ev["accuracy"] <= 1.0


def test_wide_resnet_scores_pictures_without_labels(tmp_path):
    """Inference through the public API: `Trainer.embed` on images alone returns one score per class, and the class of
    a picture the model was trained on comes out on top."""
    from helpers import tiny_resnet_plan
    from superscaler_b200.data import synthetic as syn
    from superscaler_b200.runtime.trainer import Trainer
    t = Trainer(tiny_resnet_plan(), device="cpu", lr=1e-2, lr_warmup_steps=0, model_overrides=dict(image_size=64, num_classes=8))
    b = syn.resnet_batch(t.plan["global_batch_size"], 64, 8, seed=3, dtype=torch.float32)
    for _ in range(12):
        t.train_step(b)
    scores = t.embed({"images": b["images"]})
    assert scores.shape == (t.plan["global_batch_size"], 8)
    assert (scores.float().argmax(-1) == b["labels"]).float().mean() >= 0.75
