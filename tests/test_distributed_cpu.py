"""World-size-2 run on CPU (gloo): the sample orders shard the indices across ranks without any
data-path collective.  Mirrors the reference's own multi-process order test
(tests/test_traversal_orders.py:32-93): coverage of the dataset, bounded duplication from the
sampler's padding, and a different order every epoch."""
import os
import sys

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, path, port, out_dir):
    sys.path.insert(0, ROOT)
    from types import SimpleNamespace
    from ffcv_b200.memory_managers import OSCacheManager
    from ffcv_b200.reader import Reader
    from ffcv_b200.traversal_order import QuasiRandom, Random, Sequential
    dist.init_process_group('gloo', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world)
    r = Reader(path)
    fake = SimpleNamespace(indices=np.arange(r.num_samples), seed=3, distributed=True, batch_size=4,
                           memory_manager=OSCacheManager(r))
    res = {}
    for name, cls in (('seq', Sequential), ('rand', Random), ('quasi', QuasiRandom)):
        order = cls(fake)
        res[name + '0'] = np.asarray(order.sample_order(0)).astype(np.int64)
        res[name + '1'] = np.asarray(order.sample_order(1)).astype(np.int64)
    np.savez(os.path.join(out_dir, f'rank{rank}.npz'), **res)
    dist.destroy_process_group()


def test_orders_shard_across_two_ranks(tmp_path):
    sys.path.insert(0, ROOT)
    from ffcv_b200.synthetic import write_dataset
    path = write_dataset(0, str(tmp_path / 'c0.beton'), 203, num_workers=1)
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, path, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (np.load(str(tmp_path / f'rank{r}.npz')) for r in (0, 1))
    for name in ('seq', 'rand', 'quasi'):
        for epoch in ('0', '1'):
            a, b = r0[name + epoch], r1[name + epoch]
            both = np.concatenate([a, b])
            assert set(both.tolist()) == set(range(203)), name
            counts = np.bincount(both, minlength=203)
            # every rank holds the same number of samples (the index list is padded with its own
            # head, as DistributedSampler pads): len(loader) agrees across ranks whatever the
            # dataset size, so a training loop's collectives stay matched
            assert counts.max() <= 2 and len(a) == len(b) == 102, name
            assert counts.sum() == 204 and (counts == 2).sum() == 1, name
    for name in ('rand', 'quasi'):
        assert not np.array_equal(r0[name + '0'], r0[name + '1'])
    assert np.array_equal(r0['seq0'], r0['seq1'])
