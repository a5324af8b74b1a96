"""Image-folder loaders on synthetic JPEG trees and the augmentation pipeline."""
import json
import os

import numpy as np
import pytest
import torch


def _write_jpeg(path, color, side=80):
    from PIL import Image

    arr = np.zeros((side, side + 16, 3), dtype=np.uint8)
    arr[..., :] = color
    Image.fromarray(arr).save(path, quality=95)


def test_tiny_imagenet_and_imagenet100_trees(tmp_path):
    pytest.importorskip("PIL")
    from tnn_b200.data.image_folder import create_image_folder_loaders

    # TinyImageNet layout: wnids.txt, train/<wnid>/images/*.JPEG, val/val_annotations.txt + val/images
    root = tmp_path / "tiny"
    wnids = ["n01", "n02", "n03"]
    colors = {"n01": (250, 10, 10), "n02": (10, 250, 10), "n03": (10, 10, 250)}
    (root / "val" / "images").mkdir(parents=True)
    (root / "wnids.txt").write_text("\n".join(wnids) + "\n")
    ann = []
    for w in wnids:
        d = root / "train" / w / "images"
        d.mkdir(parents=True)
        for i in range(4):
            _write_jpeg(str(d / f"{w}_{i}.JPEG"), colors[w], side=64)
        _write_jpeg(str(root / "val" / "images" / f"val_{w}.JPEG"), colors[w], side=64)
        ann.append(f"val_{w}.JPEG\t{w}\t0\t0\t10\t10")
    (root / "val" / "val_annotations.txt").write_text("\n".join(ann) + "\n")
    tr, va = create_image_folder_loaders("tiny_imagenet", str(root), 3, 0, None)  # partial batches are dropped
    assert len(tr) == 12 and len(va) == 3
    x, y = next(iter(va))
    assert x.shape == (3, 64, 64, 3) and x.dtype == torch.float32 and sorted(y.tolist()) == [0, 1, 2]
    for img, lab in zip(x, y):           # NHWC floats in [0,1]; the dominant channel identifies the class
        assert int(img.mean((0, 1)).argmax()) == int(lab)
    # ImageNet-100 layout: Labels.json + <split>/<wnid>/*.JPEG, 224x224 after resize / crop, mean/std normalised
    root = tmp_path / "in100"
    (root).mkdir()
    (root / "Labels.json").write_text(json.dumps({w: f"class {w}" for w in wnids}))
    for split in ("train.X1", "val.X"):
        for w in wnids:
            d = root / split / w
            d.mkdir(parents=True)
            for i in range(2):
                _write_jpeg(str(d / f"{i}.JPEG"), colors[w], side=260)
    tr, va = create_image_folder_loaders("imagenet100", str(root), 2, 0, None)
    assert len(tr) == 6 and len(va) == 6
    x, y = next(iter(tr))
    assert x.shape == (2, 224, 224, 3)
    xv, yv = next(iter(va))
    assert xv.shape == (2, 224, 224, 3) and abs(float(xv.mean())) < 3.0   # normalised, not raw 0..255


def test_augmentation_ops_and_builder():
    from tnn_b200.data.augmentation import AugmentationBuilder

    x = torch.arange(2 * 8 * 8 * 3, dtype=torch.float32).reshape(2, 8, 8, 3) / 400.0
    flip = AugmentationBuilder(seed=1).horizontal_flip(1.0).build()
    assert torch.equal(flip(x), x.flip(2))
    vflip = AugmentationBuilder(seed=1).vertical_flip(1.0).build()
    assert torch.equal(vflip(x), x.flip(1))
    norm = AugmentationBuilder().normalize([0.5, 0.5, 0.5], [0.25, 0.25, 0.25]).build()
    assert torch.allclose(norm(x), (x - 0.5) / 0.25)
    crop = AugmentationBuilder(seed=3).random_crop(1.0, 2).build()
    assert crop(x).shape == x.shape
    rrc = AugmentationBuilder(seed=3).random_resized_crop(1.0).build()
    assert rrc(x).shape == x.shape
    cut = AugmentationBuilder(seed=5).cutout(1.0, 4).build()
    out = cut(x + 1.0)
    assert (out == 0).any() and out.shape == x.shape
    full = (AugmentationBuilder(seed=7).horizontal_flip(0.5).rotation(0.5, 10.0).brightness(0.5, 0.2).contrast(0.5, 0.2)
            .saturation(0.5, 0.2).gaussian_noise(0.5, 0.01).random_crop(1.0, 2).normalize([0.4] * 3, [0.2] * 3).build())
    a, b = full(x.clone()), (AugmentationBuilder(seed=7).horizontal_flip(0.5).rotation(0.5, 10.0).brightness(0.5, 0.2).contrast(0.5, 0.2)
                             .saturation(0.5, 0.2).gaussian_noise(0.5, 0.01).random_crop(1.0, 2).normalize([0.4] * 3, [0.2] * 3).build())(x.clone())
    assert a.shape == x.shape and torch.equal(a, b)                      # same seed, same stream of decisions
    rc = AugmentationBuilder().resize_center_crop(16, 8).build()
    assert rc(x).shape == (2, 8, 8, 3)


def test_wifi_regression_loader(tmp_path):
    """Wi-Fi fingerprint CSV rules: no-signal cells, default target columns, population-std normalisation."""
    from tnn_b200.data.regression import WiFiLoader

    rows = ["ap0,ap1,ap2,x,y", "-60,100,-70,1.0,10.0", "-50,0,bad,3.0,30.0", "-40,-80,-90,5.0,50.0", "-30,-85,-95,7.0,oops"]
    p = tmp_path / "train.csv"
    p.write_text("\n".join(rows) + "\n")
    ld = WiFiLoader(batch_size=3, is_regression=True, shuffle=False)
    assert ld.load_data(str(p))
    assert (ld.num_features, ld.num_outputs, len(ld)) == (3, 2, 4)
    assert ld.data_shape() == (3, 1, 1)
    assert ld.features[0].tolist() == [-60.0, -100.0, -70.0]  # 100 means "not heard"
    assert ld.features[1].tolist() == [-50.0, -100.0, -100.0]  # 0 and unparsable cells too
    assert ld.targets[3].tolist() == [7.0, 0.0]  # unparsable target -> 0
    assert ld.coordinate_ranges()[0] == (1.0, 7.0)
    raw_f, raw_t = ld.features.copy(), ld.targets.copy()
    ld.normalize_data()
    assert ld.is_normalized()
    assert np.allclose(ld.feature_means, raw_f.mean(0)) and np.allclose(ld.feature_stds, raw_f.std(0))
    assert np.allclose(ld.features.mean(0), 0, atol=1e-6) and np.allclose(ld.features.std(0), 1, atol=1e-5)
    assert np.allclose(ld.denormalize_targets(ld.targets), raw_t, atol=1e-4)
    batches = list(ld)
    assert [tuple(b[0].shape) for b in batches] == [(3, 3, 1, 1), (1, 3, 1, 1)]
    assert batches[0][1].shape == (3, 2) and batches[0][1].dtype == torch.float32
    # validation data scaled with the training statistics
    val = WiFiLoader(batch_size=2, shuffle=False)
    assert val.load_data(str(p))
    val.apply_normalization(ld.feature_means, ld.feature_stds, ld.target_means, ld.target_stds)
    assert np.allclose(val.features, ld.features, atol=1e-6)
    # classification mode: the last column is the class id; a constant column gets std 1
    q = tmp_path / "cls.csv"
    q.write_text("a,b,label\n-10,-20,2\n-10,-30,0\n")
    c = WiFiLoader(batch_size=2, is_regression=False, shuffle=False)
    assert c.load_data(str(q))
    c.normalize_data()
    assert c.feature_stds[0] == 1.0 and c.target_means is None
    x, y = c.next_batch()
    assert y.dtype == torch.int64 and y.tolist() == [2, 0]
    assert not WiFiLoader().load_data(str(tmp_path / "missing.csv"))


def test_prepare_text_corpus_and_token_loader(tmp_path):
    """Text files -> train.bin / val.bin / vocab.bin (byte-level tokenizer), read back by the token loader and the tokenizer."""
    from tnn_b200.data.loaders import create_loaders
    from tnn_b200.data.prepare_text import prepare
    from tnn_b200.data.tokenizer import Tokenizer

    src = tmp_path / "a.txt"
    src.write_text("\n\n".join(f"document number {i} says hello world, " * 12 for i in range(40)))
    out = str(tmp_path / "owt")
    info = prepare([str(src)], out, tokenizer="bytes", val_fraction=0.1, paragraph_docs=True)
    assert info["vocab"] == 257 and info["eot"] == 256 and info["tokens"]["val"] > 0
    train = np.fromfile(os.path.join(out, "train.bin"), dtype=np.uint16)
    assert len(train) == info["tokens"]["train"] and int((train == 256).sum()) == 36 and train[-1] == 256
    tok = Tokenizer(os.path.join(out, "vocab.bin"))
    assert len(tok) == 257 and tok.decode(train[:15].tolist()).startswith("document number")
    tr, va = create_loaders("open_webtext", out, 2, seed=1, model_name="gpt2_small", steps_per_epoch=3, seq_len=32) \
        if "seq_len" in create_loaders.__code__.co_varnames else (None, None)
    if tr is not None:
        d, l = next(iter(tr))
        assert d.shape == (2, 32) and torch.equal(d[:, 1:], l[:, :-1])
