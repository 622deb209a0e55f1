"""Colour jitter, mixup and poison kernels against the CPU oracle, bit for bit, through the C ABI
and through a loader pipeline; and against the outputs of the reference's own closures."""
import os

import numpy as np
import pytest
import torch as ch

from parity import IMAGENET_MEAN, IMAGENET_STD, image_executor, oracle_batch
from oracle import oracle as O

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'pixel_cases.npz'))


@pytest.fixture(scope='module')
def ctx():
    from ffcv_b200 import libffcv as L
    c = L.Context(0, 1, 1)
    yield c
    c.close()


def _stream():
    return ch.cuda.current_stream(ch.device('cuda:0')).cuda_stream


@pytest.mark.parametrize('shape', [(5, 33, 35), (6, 32, 40), (3, 224, 224), (2, 1, 1), (1, 7, 4)])
@pytest.mark.parametrize('kind', [0, 1, 2])
def test_colour_jitter_kernels_bit_exact(ctx, shape, kind):
    n, h, w = shape
    rng = np.random.default_rng(100 * kind + n + h)
    imgs = rng.integers(0, 256, (n, h, w, 3), dtype=np.uint8)
    if n > 2:
        imgs[1] = 255
        imgs[2] = (rng.integers(0, 2, (h, w, 3)) * 255).astype(np.uint8)
    apply = rng.random(n) < 0.7
    apply[0] = True
    ratio = rng.uniform(0.0, 2.5, n)
    ratio[-1] = 1.0
    dev = ch.from_numpy(imgs).cuda()
    ctx.color_jitter(_stream(), dev.data_ptr(), n, h, w, kind, apply, ratio)
    got = dev.cpu().numpy()
    want = O.color_jitter(imgs, kind, apply, ratio)
    assert np.array_equal(got, want)
    assert np.array_equal(got[~apply], imgs[~apply])  # images not selected are untouched


def test_colour_jitter_matches_reference_closures(ctx):
    kinds = {'brightness': 0, 'contrast': 1, 'saturation': 2}
    imgs = GOLD['images']
    n, h, w, _ = imgs.shape
    for k in range(int(GOLD['jitter_count'])):
        dev = ch.from_numpy(imgs).cuda()
        ctx.color_jitter(_stream(), dev.data_ptr(), n, h, w, kinds[str(GOLD[f'jitter_{k}_kind'])],
                         GOLD[f'jitter_{k}_apply'], GOLD[f'jitter_{k}_ratio'])
        assert np.array_equal(dev.cpu().numpy(), GOLD[f'jitter_{k}_out'])


@pytest.mark.parametrize('shape', [(4, 33, 35, 3), (7, 32, 32, 3), (1, 8, 8, 3), (3, 224, 224, 3)])
def test_mixup_kernel_bit_exact(ctx, shape):
    rng = np.random.default_rng(shape[1])
    imgs = rng.integers(0, 256, shape, dtype=np.uint8)
    lam = rng.beta(0.5, 0.5, shape[0])
    lam[0] = 1.0
    src = ch.from_numpy(imgs).cuda()
    dst = ch.zeros_like(src)
    ctx.mixup(_stream(), src.data_ptr(), dst.data_ptr(), shape[0], imgs[0].size, lam)
    assert np.array_equal(dst.cpu().numpy(), O.mixup(imgs, lam))
    with pytest.raises(RuntimeError):
        ctx.mixup(_stream(), src.data_ptr(), src.data_ptr(), shape[0], imgs[0].size, lam)  # in place is refused
    with pytest.raises(RuntimeError):
        ctx.mixup(_stream(), src.data_ptr(), dst.data_ptr(), shape[0], imgs[0].size, lam + 1.5)


def test_poison_kernel_bit_exact_and_reference_closure(ctx):
    imgs = GOLD['images']
    n = imgs.shape[0]
    apply = np.isin(GOLD['poison_batch_indices'], GOLD['poison_indices'])
    alpha3 = np.repeat(GOLD['poison_alpha'][:, :, None], 3, 2)
    oma = ch.from_numpy(np.ascontiguousarray(1 - alpha3)).cuda()
    mask = ch.from_numpy(np.ascontiguousarray(GOLD['poison_mask'].astype('float') * alpha3)).cuda()
    for k in range(int(GOLD['poison_count'])):
        lo, hi = GOLD[f'poison_{k}_clamp']
        dev = ch.from_numpy(imgs).cuda()
        ctx.poison(_stream(), dev.data_ptr(), n, imgs[0].size, apply, oma.data_ptr(), mask.data_ptr(), lo, hi)
        got = dev.cpu().numpy()
        assert np.array_equal(got, GOLD[f'poison_{k}_out'])
        assert np.array_equal(got, O.poison(imgs, apply, GOLD['poison_mask'], GOLD['poison_alpha'], (lo, hi)))


def test_loader_pipeline_with_jitter_mixup_and_poison(tmp_path):
    """decoder + flip fused into one launch, then brightness / contrast / saturation / poison /
    mixup as kernels of their own, then normalisation; the label pipeline mixes the labels with
    the same lambdas.  Every stage is recomputed by the oracle from the recorded draws."""
    from ffcv_b200 import Loader, OrderOption
    from ffcv_b200.fields.decoders import IntDecoder, RandomResizedCropRGBImageDecoder
    from ffcv_b200.pipeline.sampling import batch_seed, sample_jitter
    from ffcv_b200.synthetic import write_dataset_isolated as write_dataset
    from ffcv_b200.transforms import (ImageMixup, LabelMixup, MixupToOneHot, NormalizeImage, Poison, RandomBrightness,
                                      RandomContrast, RandomHorizontalFlip, RandomSaturation, ToDevice, ToTensor,
                                      ToTorchImage)
    path = write_dataset(1, str(tmp_path / 'c1.beton'), 96, num_workers=4)
    res = 64
    rng = np.random.default_rng(3)
    pmask = rng.integers(0, 256, (res, res, 3)).astype(np.uint8)
    palpha = rng.uniform(0, 1, (res, res))
    poisoned = np.arange(0, 96, 5)
    jit = [RandomBrightness(0.4, 0.8), RandomContrast(0.4, 0.8), RandomSaturation(0.4, 0.8)]
    dev = ch.device('cuda:0')
    pipes = {'image': [RandomResizedCropRGBImageDecoder((res, res)), RandomHorizontalFlip(), *jit,
                       Poison(pmask, palpha, poisoned), ImageMixup(0.5, False), ToTensor(), ToDevice(dev),
                       ToTorchImage(), NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16)],
             'label': [IntDecoder(), LabelMixup(0.5, False), ToTensor(), ToDevice(dev), MixupToOneHot(1000)]}
    loader = Loader(path, batch_size=32, order=OrderOption.RANDOM, seed=7, num_workers=4, pipelines=pipes,
                    drop_last=False)
    exe = image_executor(loader)
    assert len(exe.plan.ops) == 1 and exe.plan.table is None  # decoder + flip fused, uint8 out
    exe.param_log = []
    epoch = loader.next_epoch
    outs = [(x.clone(), y.clone()) for x, y in loader]
    ch.cuda.synchronize()
    log = {b: (ix, prm) for (e, b, ix, prm) in exe.param_log if e == epoch}
    labels = loader.reader.metadata['f1']
    table = O.normalize_table(IMAGENET_MEAN, IMAGENET_STD, np.float16)
    from ffcv_b200.transforms.mixup import _lambdas
    for b, (x, y) in enumerate(outs):
        ixs, params = log[b]
        n = len(ixs)
        img = oracle_batch(loader, exe, ixs, params)
        for k, op in enumerate(jit):
            apply = np.zeros(n, np.uint8)
            ratio = np.zeros(n)
            sample_jitter(batch_seed(loader.seed, epoch, b, 1000 + 2 + k), n, op.p, max(0, 1 - op.magnitude),
                          1 + op.magnitude, apply, ratio)
            img = O.color_jitter(img, op.kind, apply, ratio)
        img = O.poison(img, np.isin(ixs, poisoned), pmask, palpha)
        lam = _lambdas(0.5, False, ixs, n)
        img = O.mixup(img, lam)
        want = table[img, np.arange(3)[None, None, None, :]]
        got = x.permute(0, 2, 3, 1).contiguous().cpu().numpy()
        assert np.array_equal(got.view(np.int16), want.view(np.int16)), f'batch {b}'
        lab = labels[ixs]
        soft = np.zeros((n, 1000), np.float32)
        soft[np.arange(n), lab] = lam.astype(np.float32)
        soft[np.arange(n), np.roll(lab, 1)] = (lam.astype(np.float32) * -1 + 1)
        assert np.array_equal(y.cpu().numpy(), soft), f'labels of batch {b}'
