"""Image / audio transforms and samplers of the dataset package."""
import numpy as np
import pytest
import torch
from PIL import Image

from mindformers_b200.dataset.sampler import build_sampler
from mindformers_b200.dataset.transforms import (BCHW2BHWC, BatchCenterCrop, BatchNormalize, BatchPILize, BatchResize,
                                                 BatchToTensor, Compose, RandomHorizontalFlip, RandomResizedCrop,
                                                 amplitude_to_db, build_transforms, hertz_to_mel, mel_filter_bank,
                                                 mel_to_hertz, optimal_fft_length, power_to_db, spectrogram,
                                                 window_function)


def test_mel_scales_invert_and_match_their_definitions():
    f = np.array([0.0, 100.0, 440.0, 1000.0, 4000.0, 7999.0])
    for scale in ("htk", "kaldi", "slaney"):
        np.testing.assert_allclose(mel_to_hertz(hertz_to_mel(f, scale), scale), f, rtol=1e-9, atol=1e-9)
    assert abs(hertz_to_mel(1000.0, "htk") - 2595 * np.log10(1 + 1000 / 700)) < 1e-9
    assert abs(hertz_to_mel(1000.0, "slaney") - 15.0) < 1e-12 and abs(hertz_to_mel(200.0, "slaney") - 3.0) < 1e-12
    with pytest.raises(ValueError):
        hertz_to_mel(1.0, "bark")


def test_filter_bank_window_and_spectrogram_against_an_independent_implementation():
    hf = pytest.importorskip("transformers.audio_utils")
    for norm, scale in ((None, "htk"), ("slaney", "slaney"), (None, "kaldi")):
        mine = mel_filter_bank(201, 40, 20.0, 7600.0, 16000, norm=norm, mel_scale=scale)
        ref = hf.mel_filter_bank(201, 40, 20.0, 7600.0, 16000, norm=norm, mel_scale=scale)
        np.testing.assert_allclose(mine, ref, rtol=1e-6, atol=1e-9)
    for name in ("hann", "hamming", "povey", "boxcar"):
        np.testing.assert_allclose(window_function(400, name), hf.window_function(400, name), atol=1e-12)
    np.testing.assert_allclose(window_function(400, "hann", periodic=False), torch.hann_window(400, periodic=False).double().numpy(),
                               atol=1e-6)
    padded = window_function(300, "hann", frame_length=512)
    assert padded.shape == (512,) and padded[:106].sum() == 0 and padded[106 + 300:].sum() == 0
    assert optimal_fft_length(400) == 512 and optimal_fft_length(512) == 512
    rng = np.random.default_rng(0)
    wave = rng.standard_normal(4000)
    win = window_function(400, "hann")
    bank = mel_filter_bank(257, 64, 0.0, 8000.0, 16000, norm="slaney", mel_scale="slaney")
    for kw in (dict(power=1.0), dict(power=2.0, mel_filters=bank, log_mel="log10"),
               dict(power=2.0, mel_filters=bank, log_mel="dB", db_range=80.0), dict(power=2.0, preemphasis=0.97, center=False)):
        mine = spectrogram(wave, win, 400, 160, fft_length=512, **kw)
        ref = hf.spectrogram(wave, win, 400, 160, fft_length=512, **kw)
        assert mine.shape == ref.shape
        np.testing.assert_allclose(mine, ref, rtol=2e-4, atol=2e-4)
    complex_spec = spectrogram(wave, win, 400, 160, power=None)
    assert np.iscomplexobj(complex_spec) and complex_spec.shape[0] == 201
    # a pure tone peaks in the bin of its frequency
    tone = np.sin(2 * np.pi * 1000.0 * np.arange(16000) / 16000.0)
    assert int(spectrogram(tone, win, 400, 160, power=2.0).mean(1).argmax()) == round(1000.0 / (16000 / 400))
    np.testing.assert_allclose(power_to_db(np.array([1.0, 10.0, 100.0])), [0.0, 10.0, 20.0], atol=1e-9)
    np.testing.assert_allclose(amplitude_to_db(np.array([1.0, 10.0])), [0.0, 20.0], atol=1e-9)
    assert power_to_db(np.array([1e-12, 1.0]), db_range=30.0).min() == -30.0


def test_vision_transforms_chain_from_configuration():
    rng = np.random.default_rng(1)
    imgs = [rng.integers(0, 256, (60, 80, 3), dtype=np.uint8), rng.integers(0, 256, (90, 50, 3), dtype=np.uint8)]
    chain = Compose(build_transforms([{"type": "BatchResize", "image_resolution": 32, "interpolation": "bilinear"},
                                      {"type": "BatchCenterCrop", "image_resolution": 32}, {"type": "BatchToTensor"},
                                      {"type": "BatchNormalize", "mean": [0.5, 0.5, 0.5], "std": [0.25, 0.25, 0.25]}]))
    out = chain(imgs)
    assert len(out) == 2 and all(o.shape == (3, 32, 32) and o.dtype == np.float32 for o in out)
    assert -2.0 - 1e-6 <= min(o.min() for o in out) and max(o.max() for o in out) <= 2.0 + 1e-6
    resized = BatchResize(32, "bilinear")(imgs)
    assert resized[0].size == (43, 32) and resized[1].size == (32, 58)            # shorter side, aspect kept
    assert BatchResize((20, 30))(imgs[0]).size == (30, 20)
    # centre crop of an array equals the slice
    crop = np.asarray(BatchCenterCrop(40)(imgs[0]))
    np.testing.assert_array_equal(crop, imgs[0][10:50, 20:60])
    t = BatchToTensor()(imgs[0])
    np.testing.assert_allclose(t, imgs[0].transpose(2, 0, 1) / 255.0, atol=1e-7)
    np.testing.assert_array_equal(BCHW2BHWC()(np.stack([t, t])).shape, (2, 60, 80, 3))
    back = BatchPILize()(t)
    np.testing.assert_array_equal(np.asarray(back), imgs[0])
    flipped = RandomHorizontalFlip(prob=1.0)(imgs[0])
    np.testing.assert_array_equal(np.asarray(flipped), imgs[0][:, ::-1])
    a, b = RandomResizedCrop(24, seed=3)(imgs[0]), RandomResizedCrop(24, seed=3)(imgs[0])
    assert a.size == (24, 24) and np.array_equal(np.asarray(a), np.asarray(b))
    assert isinstance(build_transforms(class_name="BatchToTensor"), BatchToTensor) and build_transforms() is None


def test_samplers_from_configuration():
    seq = build_sampler({"type": "SequentialSampler", "start_index": 2, "num_samples": 3, "dataset_size": 10})
    assert list(seq) == [2, 3, 4] and len(seq) == 3
    shards = [list(build_sampler({"type": "DistributedSampler", "num_shards": 3, "shard_id": r, "shuffle": True,
                                  "dataset_size": 10, "seed": 5})) for r in range(3)]
    assert all(len(s) == 4 for s in shards) and set(sum(shards, [])) == set(range(10))
    again = list(build_sampler({"type": "DistributedSampler", "num_shards": 3, "shard_id": 1, "shuffle": True,
                                "dataset_size": 10, "seed": 5}))
    assert again == shards[1]
    rnd = build_sampler({"type": "RandomSampler", "dataset_size": 8, "seed": 1})
    assert sorted(rnd) == list(range(8))
    sub = build_sampler({"type": "SubsetRandomSampler", "indices": [3, 5, 7, 9], "num_samples": 2, "seed": 0})
    picked = list(sub)
    assert len(picked) == 2 and set(picked) <= {3, 5, 7, 9}
    assert list(build_sampler({"type": "SubsetSampler", "indices": [4, 1, 2]})) == [4, 1, 2]
    w = list(build_sampler({"type": "WeightedRandomSampler", "weights": [0.0, 1.0, 0.0], "num_samples": 5, "seed": 2}))
    assert w == [1] * 5
    pk = list(build_sampler({"type": "PKSampler", "num_val": 2, "labels": [0, 1, 0, 1, 0, 2]}))
    assert pk == [0, 2, 1, 3, 5]
    assert build_sampler() is None
    with pytest.raises(ValueError):
        build_sampler({"type": "DistributedSampler", "num_shards": 2, "shard_id": 2, "dataset_size": 4})


def test_image_layout_helpers_and_array_transforms(tmp_path):
    import base64
    import io
    from mindformers_b200.tools.image_tools import load_image
    from mindformers_b200.utils.image_transforms import (center_crop, get_resize_output_image_size, normalize, pad, rescale,
                                                         resize, to_channel_dimension_format, to_pil_image)
    from mindformers_b200.utils.image_utils import (ChannelDimension, divide_to_patches, get_image_size,
                                                    infer_channel_dimension_format, select_best_resolution)
    rng = np.random.default_rng(2)
    hwc = rng.integers(0, 256, (40, 60, 3), dtype=np.uint8)
    chw = hwc.transpose(2, 0, 1)
    assert infer_channel_dimension_format(hwc) == ChannelDimension.LAST and infer_channel_dimension_format(chw) == ChannelDimension.FIRST
    assert get_image_size(hwc) == (40, 60) == get_image_size(chw)
    np.testing.assert_array_equal(to_channel_dimension_format(hwc, "channels_first"), chw)
    # any-resolution: a 40 x 60 image fits a 2 x 3 canvas of 20-pixel tiles best
    assert select_best_resolution((40, 60), [(20, 20), (40, 40), (40, 60), (60, 40)]) == (40, 60)
    assert select_best_resolution((500, 1000), [(336, 672), (672, 336), (336, 336)]) == (336, 672)
    assert select_best_resolution((100, 300), [(336, 672), (672, 336), (336, 336)]) == (336, 336)      # nothing to gain: least waste
    tiles = divide_to_patches(chw, 20)
    assert len(tiles) == 6 and all(t.shape == (3, 20, 20) for t in tiles)
    np.testing.assert_array_equal(tiles[4], chw[:, 20:40, 20:40])
    np.testing.assert_allclose(rescale(hwc, 1 / 255.0), hwc / 255.0, atol=1e-6)
    n = normalize(hwc / 255.0, [0.5, 0.4, 0.3], [0.2, 0.2, 0.2])
    np.testing.assert_allclose(n[..., 1], (hwc[..., 1] / 255.0 - 0.4) / 0.2, atol=1e-6)
    np.testing.assert_array_equal(center_crop(hwc, (20, 30)), hwc[10:30, 15:45])
    big = center_crop(hwc, (50, 70))
    assert big.shape == (50, 70, 3) and big[:5].sum() == 0 and np.array_equal(big[5:45, 5:65], hwc)
    assert pad(chw, ((1, 2), (3, 4))).shape == (3, 43, 67) and pad(hwc, 2, mode="reflect").shape == (44, 64, 3)
    assert get_resize_output_image_size(hwc, 20, default_to_square=False) == (20, 30)
    assert get_resize_output_image_size(hwc, 20) == (20, 20) and get_resize_output_image_size(hwc, (7, 9)) == (7, 9)
    assert get_resize_output_image_size(hwc, 30, default_to_square=False, max_size=40) == (26, 40)
    small = resize(hwc, (20, 30))
    assert small.shape == (20, 30, 3) and small.dtype == np.uint8
    fl = resize(chw.astype(np.float32) / 255.0, (20, 30))
    assert fl.shape == (3, 20, 30) and 0.0 <= fl.min() and fl.max() <= 1.0
    pil = to_pil_image(chw)
    np.testing.assert_array_equal(np.asarray(pil), hwc)
    path = tmp_path / "a.png"
    pil.save(path)
    buf = io.BytesIO()
    pil.save(buf, format="PNG")
    for src in (str(path), buf.getvalue(), base64.b64encode(buf.getvalue()).decode(),
                "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode(), pil):
        np.testing.assert_array_equal(np.asarray(load_image(src)), hwc)
    with pytest.raises(ValueError):
        load_image("not an image")
