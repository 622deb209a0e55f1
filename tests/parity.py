"""Shared helpers of the parity tests: run a loader batch by batch and recompute every batch with
the CPU oracle from the same stored bytes and the same random-parameter table."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402

IMAGENET_MEAN = np.array([0.485, 0.456, 0.406]) * 255
IMAGENET_STD = np.array([0.229, 0.224, 0.225]) * 255
CIFAR_MEAN = np.array([125.3, 123.0, 113.9])
CIFAR_STD = np.array([63.0, 62.1, 66.7])


def image_executor(loader, field='image'):
    for p in loader.graph.pipelines:
        if p.name == field:
            return p.executor
    raise KeyError(field)


def oracle_batch(loader, executor, batch_indices, params, nthreads=4):
    """Expected output of one fused batch, as a numpy array laid out like the device buffer."""
    plan = executor.plan
    mmap = np.memmap(loader.reader.file_name, dtype=np.uint8, mode='r')  # whatever the loader's own access is
    md = executor.metadata[batch_indices]
    sizes = executor.sample_sizes[batch_indices]
    payloads = [np.array(mmap[int(p):int(p) + int(s)]) for p, s in zip(md['data_ptr'], sizes)]
    ops = []
    for i in range(len(batch_indices)):
        rec = []
        for k, (typ, arg, fill, _) in enumerate(plan.ops):
            a, b = int(params[i, 4 + 2 * k]), int(params[i, 5 + 2 * k])
            if typ == O.OP_FLIP:
                rec.append((typ, a, 0, 0, fill))
            else:
                rec.append((typ, arg, a, b, fill))
        ops.append(rec)
    kind = executor.native_plan.out_kind
    out, status = O.run_batch(payloads, md['mode'], md['height'], md['width'], params[:, :4], plan.resize,
                              plan.out_h, plan.out_w, ops, plan.table, kind, nthreads, dct_scale=plan.dct_scale)
    assert (status == 0).all(), status
    return out


def compare_epoch(loader, field_pos=0, field='image', max_batches=None, tol_lsb=0):
    """Iterates one epoch and checks every batch of `field` against the oracle.  Returns the number
    of compared elements.  tol_lsb applies to uint8 outputs; table outputs must match bit for bit
    when tol_lsb == 0."""
    import torch as ch
    exe = image_executor(loader, field)
    exe.param_log = []
    epoch = loader.next_epoch
    outs = []
    for b, batch in enumerate(loader):
        outs.append(batch[field_pos].detach().clone())
        if max_batches is not None and b + 1 >= max_batches:
            break
    ch.cuda.synchronize()
    log = {b: (ix, prm) for (e, b, ix, prm) in exe.param_log if e == epoch}
    exe.param_log = None
    total = 0
    for b, got_t in enumerate(outs):
        ixs, params = log[b]
        want = oracle_batch(loader, exe, ixs, params)
        plan = exe.plan
        got = got_t
        if plan.torch_image and (plan.channels_last or plan.table is None):
            got = got.permute(0, 2, 3, 1)  # back to the NHWC buffer layout
        got = got.contiguous().cpu().numpy()
        assert got.shape == want.shape, (got.shape, want.shape)
        if got.dtype == np.uint8:
            diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
            assert diff.max() <= tol_lsb, f'batch {b}: max diff {diff.max()} at {np.argwhere(diff > tol_lsb)[:5]}'
        else:
            a = got.view(np.int16 if got.dtype == np.float16 else np.int32)
            w = want.view(np.int16 if want.dtype == np.float16 else np.int32)
            bad = a != w
            assert not bad.any(), f'batch {b}: {int(bad.sum())} mismatching elements, first {np.argwhere(bad)[:5]}'
        total += got.size
    return total
