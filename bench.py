#!/usr/bin/env python
"""Benchmark of the decode-and-augment hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 0..4]

Workload (default): configuration 2 of the benchmark contract, a synthetic ImageNet-shaped `.beton`
(write_mode='proportion', 50 % JPEG q90 4:2:0 / 50 % raw, short side 300-500, max side 500) read
through RandomResizedCropRGBImageDecoder((224, 224)) -> RandomHorizontalFlip -> NormalizeImage
(fp16) -> ToTorchImage, with its labels, batch 512 per GPU, QUASI_RANDOM order.  A "step" is one
batch.  The dataset is a bounded, seeded sample of that configuration (see --images) written
before the timed region.  `--config` selects one of the other four configurations instead; the
default run also appends a short pass over each of them (`configs`).

One JSON line on stdout (rank 0):
  value      images/s with the batch bytes already resident in HBM (kernels only, CUDA events), the
             slots on their own streams as the loader runs them; value_single_stream = the same on
             one stream (the pass the per-kernel durations come from)
  e2e        images/s through `for batch in Loader(...)`: host staging from the file, host->device
             copy, kernels, and an 8-byte device->host read per step.  Timed in the steady state:
             the batches the loader had prepared ahead while this process waited are consumed
             before the clock starts, and at least `e2e.steps_timed` >= K steps are timed, as three
             segments of which the median counts (the host's memory and PCIe are shared)
  roofline   the dominant kernel against the bound that binds it (instruction issue), with the
             HBM figure beside it; per-kernel instruction and DRAM-traffic figures come from the
             ncu captures summarised in profiles/ncu_constants.json (`profile_stale` tells whether
             the kernels' sources changed since)
  cpu_baseline  the CPU oracle port on all host threads, bounded sample (rank 0, N = 1)
With --impl reference the same workload runs on the CPU oracle port only (no GPU work).
"""
import argparse
import hashlib
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

IMAGENET_MEAN = np.array([0.485, 0.456, 0.406]) * 255
IMAGENET_STD = np.array([0.229, 0.224, 0.225]) * 255
CIFAR_MEAN = np.array([125.3, 123.0, 113.9])
CIFAR_STD = np.array([63.0, 62.1, 66.7])
CIFAR_FILL = (125, 123, 114)
SM_COUNT, ISSUE_PER_SM_CLK = 148, 4  # B200: 148 SMs, four warp schedulers each, one instruction per clock
KERNELS = ('entropy_decode', 'idct', 'upsample_colour', 'resize_augment_normalise')
# source files whose change makes the ncu figures of a kernel stale
KERNEL_SOURCES = {'entropy_decode': 'entropy.cu', 'idct': 'idct.cu', 'upsample_colour': 'idct.cu',
                  'resize_augment_normalise': 'resize.cu'}

# The five configurations of the benchmark contract: batch per GPU, output size, sample order, epoch
# length, distinct synthetic images written by default (the epoch cycles through them).
WORKLOADS = {
    0: dict(batch=512, out=32, order='RANDOM', samples=50_000, distinct=50_000, dataset_cfg=0,
            text='config 0: CIFAR-shaped raw 32x32 -> flip + translate(2) + cutout(4) + fp16 normalise, labels'),
    1: dict(batch=1024, out=160, order='RANDOM', samples=100_000, distinct=4096, dataset_cfg=1,
            text='config 1: JPEG q90 4:2:0, short side 200-256 (max side 256) -> RRC-160 + flip + fp16 normalise'),
    2: dict(batch=512, out=224, order='QUASI_RANDOM', samples=200_000, distinct=4096, dataset_cfg=2,
            text='config 2: proportion(0.5) JPEG q90 4:2:0 / raw, short side 300-500, max side 500 -> '
                 'RRC-224 + flip + fp16 normalise, channels-last'),
    3: dict(batch=1024, out=256, order='SEQUENTIAL', samples=50_000, distinct=4096, dataset_cfg=3,
            text='config 3: JPEG q90 (max side 256) -> centre crop 224/256 -> 256x256 + fp16 normalise (validation)'),
    4: dict(batch=256, out=384, order='RANDOM', samples=20_000, distinct=96, dataset_cfg=4,
            text='config 4: JPEG q95 4:4:4, short side 1024-1536 -> RRC-384 (scale 0.25-1) + flip + cutout(64) + '
                 'fp16 normalise'),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=10)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--config', type=int, default=2, choices=sorted(WORKLOADS), help='configuration of the headline line')
    ap.add_argument('--images', type=int, default=0, help='distinct images in the synthetic dataset (0: per configuration)')
    ap.add_argument('--workers', type=int, default=0, help='host staging threads per rank (0: cores / ranks)')
    ap.add_argument('--batches-ahead', type=int, default=3)
    ap.add_argument('--restart-interval', type=int, default=0,
                    help='write the JPEG samples with a restart marker every N MCUs (0: as the reference writes them)')
    ap.add_argument('--no-cpu-baseline', action='store_true', help='skip the CPU oracle leg (profiling runs)')
    ap.add_argument('--no-configs', action='store_true', help='skip the short pass over the other configurations')
    ap.add_argument('--no-modes', action='store_true', help='skip the other staging modes (e2e_staged, e2e_gather, ...)')
    ap.add_argument('--decode-index', type=float, default=0.0,
                    help='GiB of GPU memory for the decode index (Loader(decode_index_gb=...)); 0 = off, the default')
    ap.add_argument('--dct-downscale', action='store_true',
                    help='decode JPEG samples at reduced scale where the crop allows (not the reference\'s pixels)')
    ap.add_argument('--batch', type=int, default=0, help='profiling runs: batch size instead of the configuration\'s')
    ap.add_argument('--kernels-only', action='store_true',
                    help='profiling runs: stage the slots once, then only re-run the kernels on one stream')
    return ap.parse_args()


def rank_info():
    return (int(os.environ.get('RANK', 0)), int(os.environ.get('LOCAL_RANK', 0)),
            int(os.environ.get('WORLD_SIZE', 1)))


# ---------------------------------------------------------------------------------------- datasets

def dataset_path(cfg, images, restart_interval=0):
    base = '/dev/shm' if os.path.isdir('/dev/shm') and os.access('/dev/shm', os.W_OK) else tempfile.gettempdir()
    tag = f'_rst{restart_interval}' if restart_interval else ''
    dcfg = WORKLOADS[cfg]['dataset_cfg']
    samples = WORKLOADS[cfg]['samples']
    return os.path.join(base, f'ffcv_b200_bench_c{dcfg}_{images}_of_{samples}{tag}.beton')


def ensure_dataset(cfg, images, restart_interval=0):
    """Written once (rank 0) before any timing; other ranks wait for the barrier that follows."""
    from ffcv_b200.synthetic import replicate_samples, write_dataset_isolated as write_dataset  # forks workers
    path = dataset_path(cfg, images, restart_interval)
    if not os.path.exists(path):
        tmp = path + f'.tmp{os.getpid()}'
        write_dataset(WORKLOADS[cfg]['dataset_cfg'], tmp, images, num_workers=len(os.sched_getaffinity(0)),
                      restart_interval=restart_interval)
        # the configuration's epoch length over the bounded set of distinct images
        replicate_samples(tmp, WORKLOADS[cfg]['samples'])
        os.replace(tmp, path)
    return path


def distinct_images(cfg, args, world):
    n = args.images if args.images and cfg == args.config else WORKLOADS[cfg]['distinct']
    if cfg != 0:
        n *= min(world, 4)
    return min(n, WORKLOADS[cfg]['samples'])


def build_pipelines(cfg, device, dct_downscale=False):
    import torch as ch
    from ffcv_b200.fields.decoders import (CenterCropRGBImageDecoder, IntDecoder, RandomResizedCropRGBImageDecoder,
                                           SimpleRGBImageDecoder)
    from ffcv_b200.transforms import (Convert, Cutout, NormalizeImage, RandomHorizontalFlip, RandomTranslate, Squeeze,
                                      ToDevice, ToTensor, ToTorchImage)
    norm = NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16)
    if cfg == 0:
        image = [SimpleRGBImageDecoder(), RandomHorizontalFlip(0.5), RandomTranslate(padding=2, fill=CIFAR_FILL),
                 Cutout(4, CIFAR_FILL), ToTensor(), ToDevice(device), ToTorchImage(), Convert(ch.float16),
                 NormalizeImage(CIFAR_MEAN, CIFAR_STD, np.float16)]
    elif cfg == 1:
        image = [RandomResizedCropRGBImageDecoder((160, 160), scale=(0.08, 1), ratio=(3 / 4, 4 / 3)),
                 RandomHorizontalFlip(), ToTensor(), ToDevice(device), ToTorchImage(), norm]
    elif cfg == 2:
        image = [RandomResizedCropRGBImageDecoder((224, 224), dct_downscale=dct_downscale), RandomHorizontalFlip(),
                 ToTensor(), ToDevice(device),
                 ToTorchImage(), norm]
    elif cfg == 3:
        image = [CenterCropRGBImageDecoder((256, 256), ratio=224 / 256), ToTensor(), ToDevice(device), ToTorchImage(),
                 norm]
    else:
        image = [RandomResizedCropRGBImageDecoder((384, 384), scale=(0.25, 1), dct_downscale=dct_downscale),
                 RandomHorizontalFlip(), Cutout(64),
                 norm, ToTorchImage()]
    return {'image': image, 'label': [IntDecoder(), ToTensor(), ToDevice(device), Squeeze()]}


def config_dict(cfg, world, images, workers, restart_interval=0):
    w = WORKLOADS[cfg]
    out = {'workload': w['text'], 'config_id': cfg, 'batch_per_gpu': w['batch'], 'global_batch': w['batch'] * world,
           'dataset_samples': w['samples'], 'distinct_images': images, 'order': w['order'], 'labels': True,
           'sharding': 'index sharding, no collective' if world > 1 else 'single GPU',
           'host_threads_per_rank': workers,
           'l2': 'inputs larger than L2: consecutive steps read different batches (one per slot of the ring)'}
    if restart_interval:
        out['jpeg_restart_interval'] = restart_interval  # not the reference's file format default
    return out


# ------------------------------------------------------------------------------ measured peaks, ncu

def read_peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        try:
            return float(json.load(open(p))['hbm_gbs']), 'measured'
        except Exception:
            pass
    return 6650.0, 'fallback'


def source_hashes():
    out = {}
    for f in sorted(set(KERNEL_SOURCES.values())):
        with open(os.path.join(ROOT, 'ffcv_b200', 'csrc', f), 'rb') as fp:
            out[f] = hashlib.sha256(fp.read()).hexdigest()[:16]
    return out


def ncu_constants(cfg):
    """Per-kernel warp instructions and DRAM bytes per unit of work, from the committed summary of
    the ncu captures.  Returns (constants or None, stale flags per kernel)."""
    p = os.path.join(ROOT, 'profiles', 'ncu_constants.json')
    if not os.path.exists(p):
        return None, {}
    try:
        doc = json.load(open(p))
    except Exception:
        return None, {}
    entry = doc.get('configs', {}).get(f'c{cfg}')
    if entry is None:
        return None, {}
    now = source_hashes()
    stale = {k: now.get(KERNEL_SOURCES[k]) != entry.get('source_sha256_16', {}).get(KERNEL_SOURCES[k]) for k in KERNELS}
    return entry, stale


def numa_placement(device_index):
    """(memory node of the GPU, node of the first CPU this process may run on, MB of shared-memory
    pages per node); -1 / [] where the system does not say."""
    import glob
    import torch
    gpu_node, cpu_node, per_node = -1, -1, []
    try:
        nodes = sorted(int(os.path.basename(p)[4:]) for p in glob.glob('/sys/devices/system/node/node[0-9]*'))
        for n in nodes:
            mb = -1.0
            with open(f'/sys/devices/system/node/node{n}/meminfo') as fp:
                for line in fp:
                    if ' Shmem:' in line:
                        mb = int(line.split()[-2]) / 1024.0
            per_node.append(mb)
        first_cpu = min(os.sched_getaffinity(0))
        for n in nodes:
            with open(f'/sys/devices/system/node/node{n}/cpulist') as fp:
                for part in fp.read().strip().split(','):
                    lo, _, hi = part.partition('-')
                    if part and int(lo) <= first_cpu <= int(hi or lo):
                        cpu_node = n
        props = torch.cuda.get_device_properties(device_index)
        bdf = f'{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0'
        with open(f'/sys/bus/pci/devices/{bdf}/numa_node') as fp:
            gpu_node = int(fp.read().strip())
    except Exception:  # noqa: BLE001 - a diagnostic must not take the measurement down
        pass
    return gpu_node, cpu_node, per_node


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
              'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                                          '-lms', '100', '-i', str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(',')]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), f[5:9]):
                if v.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': float(np.median(sm)) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': sorted(reasons), 'samples': len(sm)}


# ------------------------------------------------------------------------------------ CPU oracle leg

def oracle_batches(cfg, path, seed, n_batches, rank=0, world=1):
    """Batches (stored bytes + sampled parameters) of the configuration for the CPU oracle: the
    parameter tables come from the same samplers, seeded the same way, as the loader's."""
    import torch as ch
    from ffcv_b200.memory_managers import OSCacheManager
    from ffcv_b200.pipeline.fusion import host_plan, sample_plan_params
    from ffcv_b200.reader import Reader
    r = Reader(path)
    mm = OSCacheManager(r)
    mmap = mm.open()
    md = r.metadata['f0']
    sizes = mm.sizes_of(md['data_ptr'])
    plan = host_plan(build_pipelines(cfg, ch.device('cuda', 0))['image'], r.handlers['image'], md)
    batch = WORKLOADS[cfg]['batch']
    order = np.arange(r.num_samples)[rank::world]
    out = []
    for b in range(n_batches):
        ix = order[(np.arange(batch) + b * batch) % len(order)]
        m = md[ix]
        params = sample_plan_params(plan, m, seed, 0, b)
        payloads = [np.asarray(mmap[int(p):int(p) + int(s)]) for p, s in zip(m['data_ptr'], sizes[ix])]
        out.append((plan, payloads, m['mode'], np.ascontiguousarray(m['height']), np.ascontiguousarray(m['width']), params))
    return out


def run_oracle(batches, threads):
    """Runs the CPU oracle over the given batches; returns seconds per batch (list)."""
    from ffcv_b200 import libffcv as L
    from oracle import oracle as O
    times = []
    for plan, payloads, modes, h, w, params in batches:
        ops = []
        for i in range(len(payloads)):
            rec = []
            for k, (typ, arg, fill, _) in enumerate(plan.ops):
                a, b = int(params[i, 4 + 2 * k]), int(params[i, 5 + 2 * k])
                rec.append((typ, a, 0, 0, fill) if typ == L.OP_FLIP else (typ, arg, a, b, fill))
            ops.append(rec)
        t0 = time.perf_counter()
        _, status = O.run_batch(payloads, modes, h, w, params[:, :4], plan.resize, plan.out_h, plan.out_w, ops,
                                plan.table, plan.out_kind, threads, dct_scale=plan.dct_scale)
        times.append(time.perf_counter() - t0)
        assert (status == 0).all()
    return times


def main_reference(args):
    """The reference arm: the path on the host cores only (CPU oracle port, all threads)."""
    rank, _, world = rank_info()
    if rank != 0:
        return
    cfg = args.config
    images = distinct_images(cfg, args, world)
    path = ensure_dataset(cfg, images, args.restart_interval)
    threads = len(os.sched_getaffinity(0))
    batch = WORKLOADS[cfg]['batch']
    n = args.steps + args.warmup
    # a step of config 4 is 256 images of ~2.5 Mpx (about 10 s of CPU work): the run is bounded by
    # repeating a few prepared batches and, for that configuration, by timing fewer steps
    steps = args.steps if cfg != 4 else min(args.steps, 6)
    warm = args.warmup if cfg != 4 else min(args.warmup, 1)
    batches = oracle_batches(cfg, path, 0, min(n, 8 if cfg != 4 else 2))
    seq = [batches[i % len(batches)] for i in range(steps + warm)]
    run_oracle(seq[:warm], threads)
    times = run_oracle(seq[warm:], threads)
    total = sum(times)
    value = batch * steps / total
    line = {'impl': 'reference', 'metric': 'RRC-224 decode+augment images/s', 'value': value, 'unit': 'images/s',
            'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * total / steps,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'u8', 'data': 'synthetic',
            'config': config_dict(cfg, world, images, threads, args.restart_interval),
            'cpu_baseline': {'value': value, 'unit': 'images/s', 'cores': threads, 'kind': 'port',
                             'sample': f'{steps} batches of {batch} images of the workload',
                             'note': 'scalar C restatement of the path on all host threads; an FFCV install with '
                                     'SIMD libjpeg-turbo and OpenCV is expected to be 1.5-2x faster'},
            'e2e': {'value': value, 'unit': 'images/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
            'gpu_launches': 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------ our arm

class Bench:
    def __init__(self, args):
        import torch as ch
        import torch.distributed as dist
        self.ch, self.dist, self.args = ch, dist, args
        self.rank, self.local, self.world = rank_info()
        if not ch.cuda.is_available():
            raise SystemExit('bench.py needs a CUDA device: ffcv_b200 has no CPU fallback')
        ch.cuda.set_device(self.local)
        self.device = ch.device('cuda', self.local)
        if self.world > 1:
            os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
            # stdout carries the one JSON line: while the communicator comes up (NCCL prints its version
            # banner there) file descriptor 1 points at stderr
            sys.stdout.flush()
            saved = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group('nccl', device_id=self.device)
                dist.barrier(device_ids=[self.local])
                ch.cuda.synchronize()
            finally:
                sys.stdout.flush()
                os.dup2(saved, 1)
                os.close(saved)
        self.decode_index = args.decode_index
        self.cores = len(os.sched_getaffinity(0))
        self.workers = args.workers or max(2, self.cores // max(1, self.world))

    def barrier(self):
        if self.world > 1:
            self.dist.barrier(device_ids=[self.local])

    def max_over_ranks(self, values):
        t = self.ch.tensor(list(values), dtype=self.ch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    def gather_ranks(self, values):
        """[world, len(values)] array of every rank's values (rank order)."""
        t = self.ch.tensor(list(values), dtype=self.ch.float64, device=self.device)
        if self.world == 1:
            return t.cpu().numpy()[None]
        out = [self.ch.zeros_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return np.stack([o.cpu().numpy() for o in out])

    def make_loader(self, cfg, path, pin=None, share=None, **kw):
        from ffcv_b200 import Loader, OrderOption
        w = WORKLOADS[cfg]
        return Loader(path, batch_size=w['batch'], order=getattr(OrderOption, w['order']), distributed=self.world > 1,
                      seed=0, num_workers=self.workers,
                      pipelines=build_pipelines(cfg, self.device, self.args.dct_downscale),
                      batches_ahead=self.args.batches_ahead, drop_last=True, pin_file=pin, cpu_stage_share=share,
                      decode_index_gb=self.decode_index, **kw)

    @staticmethod
    def describe(ld):
        if getattr(ld.memory_manager, 'direct', False):
            return 'file read with pread straight into the pinned staging buffers (no page cache), one DMA copy per batch'
        if not ld.memory_manager.pinned:
            return 'file memory-mapped, staged into pinned buffers by CPU threads, one DMA copy per batch'
        if ld.stage_split == 0:
            return 'file in pinned host RAM, payloads gathered by the GPU over PCIe'
        return ('file in pinned host RAM: the GPU gathers most payload bytes over PCIe, up to 4 CPU threads and the '
                'copy engine carry the rest (share %s)' % ('balanced per batch' if ld.stage_split < 0
                                                           else '%.2f' % (ld.stage_split / 1000)))

    def run_e2e(self, loader, steps, warmup, sampler=None):
        """Returns (ms of the timed region, steps timed, mean h2d bytes, launches per batch, digest,
        mean stage times, mean gather ms)."""
        ch = self.ch
        exe = loader.graph.pipelines[0].executor
        batch = loader.batch_size

        def endless():
            while True:
                for b in loader:
                    yield b
        it = endless()
        digest = 0.0

        def consume():
            x, y = next(it)[:2]
            # the 8-byte device->host read of the step: a checksum over pixels and labels
            return float((x[:, 0, ::32, ::32].float().sum() + y.sum()).item())
        for _ in range(warmup):
            digest += consume()
        ch.cuda.synchronize()
        self.barrier()
        # While this process waited at the barrier its loader filled the queue of prepared batches.
        # They are consumed before the clock starts, so that the timed region begins in the steady
        # state of producer and consumer and bills only batches produced inside it.
        # (The clock sampler starts first: spawning it takes long enough for the queue to fill again.)
        if sampler is not None:
            sampler.start()
        t0 = time.perf_counter()
        ahead = loader.batches_ahead + 2
        for _ in range(ahead):
            digest += consume()
        ch.cuda.synchronize()
        est = max(1e-5, (time.perf_counter() - t0) / ahead)
        # at least a second's worth of steps, and several times the queue's depth
        timed = max(steps, 6 * ahead, min(600, int(math.ceil(1.0 / est)))) if steps < 100 else steps
        if self.world > 1:  # every rank times the same number of steps
            timed = int(self.max_over_ranks([timed])[0])
        # The timed steps are taken as three consecutive segments and the median segment is the
        # result: the host side of this path (DRAM and PCIe) is shared with whatever else runs on
        # the machine, and a neighbour's burst would otherwise decide the figure.
        timed = (timed + 2) // 3 * 3
        marks = [ch.cuda.Event(enable_timing=True) for _ in range(4)]
        h2d, stage, gather = [], [], []
        marks[0].record()
        for k in range(timed):
            digest += consume()
            h2d.append(exe.h2d_bytes)
            if k % 8 == 0:
                stage.append(exe.ctx.stage_times(k % (loader.batches_ahead + 2)))
            if (k + 1) % (timed // 3) == 0:
                marks[(k + 1) // (timed // 3)].record()
        ch.cuda.synchronize()
        self.barrier()
        segments = [marks[i].elapsed_time(marks[i + 1]) for i in range(3)]
        for s in range(loader.batches_ahead + 2):
            g = exe.ctx.gather_time(s)
            if g is not None:
                gather.append(g)
        loader._live_iterator.retire()
        # the worker queued batches the loop above never consumed: their copies and kernels must
        # be through before anybody restages their slots outside the loader's own fences
        ch.cuda.synchronize()
        return dict(ms=float(np.median(segments)) * 3, segments=[v / (timed // 3) for v in segments], steps=timed,
                    h2d=int(np.mean(h2d)), launches=exe.launches, digest=digest,
                    stage_ms=np.mean(np.array(stage), axis=0) if stage else np.zeros(4),
                    gather_ms=float(np.mean(gather)) if gather else None, batch=batch)

    def e2e_entry(self, res, loader=None, source=None):
        ms = self.max_over_ranks([res['ms']])[0]
        entry = {'value': res['batch'] * self.world * res['steps'] / (ms * 1e-3), 'unit': 'images/s',
                 'ms_per_step': ms / res['steps'], 'steps_timed': res['steps'],
                 'segments_ms_per_step': res['segments'],  # rank 0's three segments; the median one counts
                 'h2d_bytes_per_step': res['h2d'], 'd2h_bytes_per_step': 8}
        if source is not None:
            entry['source'] = source
        return entry

    def link_peak(self, concurrent):
        """Pinned 256 MB host->device copy, best of 10; `concurrent`: every rank copies at once."""
        ch = self.ch
        hbuf = ch.empty(256 << 20, dtype=ch.uint8).pin_memory()
        dbuf = ch.empty(256 << 20, dtype=ch.uint8, device=self.device)
        best = 1e9
        for k in range(11):
            if concurrent:
                self.barrier()
            a, b = ch.cuda.Event(enable_timing=True), ch.cuda.Event(enable_timing=True)
            a.record()
            dbuf.copy_(hbuf, non_blocking=True)
            if concurrent:  # a second copy keeps the link busy while slower ranks finish their first
                dbuf.copy_(hbuf, non_blocking=True)
            b.record()
            b.synchronize()
            if k:
                best = min(best, a.elapsed_time(b) / (2 if concurrent else 1))
        del hbuf, dbuf
        return (256 << 20) / (best * 1e-3) / 1e9

    # -------------------------------------------------------------------------------------------
    def measure(self, cfg, steps, warmup, full, sampler=None):
        """One configuration: end to end through the Loader, then the kernels with the bytes in HBM."""
        ch, args = self.ch, self.args
        w = WORKLOADS[cfg]
        batch = w['batch']
        images = distinct_images(cfg, args, self.world)
        if self.rank == 0:
            ensure_dataset(cfg, images, args.restart_interval)
        self.barrier()
        path = dataset_path(cfg, images, args.restart_interval)
        out = {'config': config_dict(cfg, self.world, images, self.workers, args.restart_interval)}
        if self.decode_index > 0:
            out['config']['decode_index_gb'] = self.decode_index  # opt-in: states recorded by a stream's first decode
        if args.dct_downscale:
            out['config']['dct_downscale'] = 'JPEG samples decoded at 1/2 .. 1/8 where the crop allows (opt-in: not the reference\'s pixels)'

        others = {}
        if full and not args.no_modes and not args.kernels_only:
            auto = self.make_loader(cfg, path)
            auto_mode = (auto.pin_file, auto.stage_split)
            del auto
            for name, pin, share, kw in [('e2e_staged', False, None, {}), ('e2e_gather', True, 0.0, {}),
                                         ('e2e_split', True, None, {}), ('e2e_direct', False, None, {'os_cache': False})]:
                probe = self.make_loader(cfg, path, pin, share, **kw)
                if not kw and ((probe.pin_file, probe.stage_split) == auto_mode or
                               (name == 'e2e_split' and probe.stage_split == 0)):
                    del probe
                    continue
                if kw:  # the file is read afresh: drop what the page cache holds of it
                    fd = os.open(path, os.O_RDONLY)
                    os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_DONTNEED)
                    os.close(fd)
                res = self.run_e2e(probe, steps, warmup)
                others[name] = self.e2e_entry(res, source=self.describe(probe))
                del probe
        t_setup = time.perf_counter()
        loader = self.make_loader(cfg, path)
        setup_s = time.perf_counter() - t_setup  # includes page-locking the file where it lies
        exe = loader.graph.pipelines[0].executor
        ctx = exe.ctx
        slots = loader.batches_ahead + 2
        stream = ch.cuda.current_stream(self.device)
        if not args.kernels_only:
            res = self.run_e2e(loader, steps, warmup, sampler)
            out['e2e'] = self.e2e_entry(res, source=self.describe(loader))
            out['e2e']['loader_setup_s'] = setup_s
            out['e2e']['file_bytes'] = os.path.getsize(path)
            out['e2e_raw'] = res
            out.update(others)
            out['launches_per_batch'] = res['launches']

        # ---- inputs resident in HBM
        outs = loader.slot_buffers()[(0, 'fused')]
        order = loader.traversal_order.sample_order(10_000)
        infos, crop_bytes = [], []
        for s in range(slots):
            ix = np.asarray(order[(np.arange(batch) + s * batch) % len(order)])
            exe(ix, s, stream.cuda_stream, outs[s], 10_000, s)
            infos.append(ctx.batch_info(s))
            p = exe.last_params
            crop_bytes.append(int((p[:, 2].astype(np.int64) * p[:, 3] * 3).sum()))
        ch.cuda.synchronize()
        out['launches_per_batch'] = out.get('launches_per_batch', ctx.launches(0))
        # (1) per-kernel durations: one stream, kernels back to back, library events around each
        ctx.set_profiling(True)
        for k in range(warmup):
            ctx.rerun(k % slots, stream.cuda_stream, outs[k % slots].data_ptr())
        ch.cuda.synchronize()
        self.barrier()
        kernel_ms = []
        s0, s1 = ch.cuda.Event(enable_timing=True), ch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for k in range(steps):
            s = k % slots
            if k >= slots:
                kernel_ms.append(ctx.batch_times(s))  # waits only for a run queued `slots` steps ago
            ctx.rerun(s, stream.cuda_stream, outs[s].data_ptr())
        s1.record(stream)
        ch.cuda.synchronize()
        self.barrier()
        for s in range(min(slots, steps)):
            kernel_ms.append(ctx.batch_times(s))
        serial_ms = s0.elapsed_time(s1)
        ctx.set_profiling(False)
        out['infos'] = infos
        if self.decode_index > 0:
            out['decode_index_stats'] = ctx.decode_index_stats()
        if args.kernels_only:
            value_ms = serial_ms
        else:
            # (2) throughput the way the loader drives the device: every slot on its own stream, so the
            # kernels of consecutive batches overlap (the entropy kernel is latency-bound at this batch
            # size and leaves issue slots to the others)
            slot_streams = loader.slot_streams()
            for k in range(warmup):
                ctx.rerun(k % slots, slot_streams[k % slots].cuda_stream, outs[k % slots].data_ptr())
            ch.cuda.synchronize()
            self.barrier()
            v0, v1 = ch.cuda.Event(enable_timing=True), ch.cuda.Event(enable_timing=True)
            v0.record(stream)
            for st_ in slot_streams:
                st_.wait_event(v0)
            for k in range(steps):
                ctx.rerun(k % slots, slot_streams[k % slots].cuda_stream, outs[k % slots].data_ptr())
            for st_ in slot_streams:
                stream.wait_stream(st_)
            v1.record(stream)
            ch.cuda.synchronize()
            self.barrier()
            value_ms = v0.elapsed_time(v1)
        value_ms, serial_ms = self.max_over_ranks([value_ms, serial_ms])
        out['value'] = batch * self.world * steps / (value_ms * 1e-3)
        out['ms_per_step'] = value_ms / steps
        out['value_single_stream'] = {'value': batch * self.world * steps / (serial_ms * 1e-3), 'unit': 'images/s',
                                      'ms_per_step': serial_ms / steps}
        km = np.mean(np.array(kernel_ms), axis=0)  # [h2d (unused here), entropy, idct, colour, resize]
        mean = {k: float(np.mean([i[k] for i in infos])) for k in infos[0]}
        out_bytes = batch * w['out'] * w['out'] * 3 * 2
        crop_mean = float(np.mean(crop_bytes))
        raw_frac = 1.0 - mean['n_jpeg'] / batch
        algo = {
            'entropy_decode': mean['scan_bytes'] + 128 * mean['blocks'],
            'idct': 128 * mean['blocks'] + mean['plane_bytes'],
            # only the crop box of the JPEG samples is converted: Y + 2 quarter-size chroma planes read
            # (1.5 B/pixel; 3 for 4:4:4), RGB written (3 B/pixel); crop_mean is the mean crop size in RGB bytes
            'upsample_colour': crop_mean * (1.0 - raw_frac) * (2.0 if cfg == 4 else 1.5),
            'resize_augment_normalise': crop_mean + out_bytes,
        }
        total_kernel_ms = float(km[1:].sum())
        kernels = {n: {'ms': float(km[i + 1]), 'share': float(km[i + 1] / total_kernel_ms) if total_kernel_ms else 0.0,
                       'algorithmic_bytes': algo[n], 'gbs': algo[n] / (km[i + 1] * 1e-3) / 1e9 if km[i + 1] > 0 else 0.0}
                   for i, n in enumerate(KERNELS)}
        out['kernels'] = kernels
        out['kernel_ms_per_step'] = total_kernel_ms
        # payload read once + output written once
        out['path_bytes'] = mean['jpeg_bytes'] + crop_mean * raw_frac + out_bytes
        # units the ncu figures are scaled by
        out['units'] = {'entropy_decode': mean['scan_bytes'], 'idct': mean['blocks'],
                        'upsample_colour': mean['n_jpeg'],
                        'resize_augment_normalise': float(batch * w['out'] * w['out'])}
        if loader._live_iterator is not None:
            loader._live_iterator.retire()
        del loader
        return out

    def roofline(self, m, cfg, clocks):
        """The dominant kernel against instruction issue (its binding roofline) and HBM."""
        kernels = m['kernels']
        consts, stale = ncu_constants(cfg)
        peak, peak_kind = read_peaks()
        sm_hz = (clocks['sm_mhz'] if clocks and clocks.get('sm_mhz') else 1965.0) * 1e6
        issue_peak = SM_COUNT * ISSUE_PER_SM_CLK * sm_hz
        for n in KERNELS:
            k = kernels[n]
            k['hbm_frac'] = k['gbs'] / peak
            if consts and n in consts.get('kernels', {}):
                c = consts['kernels'][n]
                inst = c['warp_inst_per_unit'] * m['units'][n]
                k['ncu_dram_bytes'] = c['dram_bytes_per_unit'] * m['units'][n]
                floor_ms = inst / issue_peak * 1e3
                k['issue'] = {'warp_instructions': inst, 'floor_ms': floor_ms, 'frac': floor_ms / k['ms'] if k['ms'] > 0 else 0.0}
                k['profile_stale'] = bool(stale.get(n, True))
        dom = max(KERNELS, key=lambda n: kernels[n]['ms'])
        d = kernels[dom]
        line = {'kernel': dom, 'ms_per_launch': d['ms'], 'peak_kind': peak_kind,
                'hbm': {'bound': 'hbm', 'achieved': d['gbs'], 'peak': peak, 'unit': 'GB/s', 'frac': d['hbm_frac'],
                        'algorithmic_bytes': d['algorithmic_bytes']},
                'traffic': d.get('ncu_dram_bytes'),
                'traffic_source': 'ncu capture summarised in profiles/ncu_constants.json, scaled by the work per launch',
                'kernels': kernels,
                'path': {'algorithmic_bytes_per_step': m['path_bytes'], 'kernel_ms_per_step': m['kernel_ms_per_step'],
                         'gbs': m['path_bytes'] / (m['kernel_ms_per_step'] * 1e-3) / 1e9}}
        if 'issue' in d:
            # integer/byte work: the kernel is bound by instruction issue, not by HBM
            line.update({'bound': 'issue', 'achieved': d['issue']['warp_instructions'] / (d['ms'] * 1e-3), 'peak': issue_peak,
                         'unit': 'warp instructions/s', 'frac': d['issue']['frac'],
                         'peak_source': '148 SMs x 4 schedulers x the SM clock sampled during the run',
                         'profile_stale': d['profile_stale']})
        else:
            line.update({'bound': 'hbm', 'achieved': d['gbs'], 'peak': peak, 'unit': 'GB/s', 'frac': d['hbm_frac'],
                         'profile_stale': True, 'note': 'no ncu summary for this configuration: HBM figure only'})
        return line

    # -------------------------------------------------------------------------------------------
    def main(self):
        args, ch = self.args, self.ch
        cfg = args.config
        sampler = ClockSampler(self.local) if self.rank == 0 else None
        steps = args.steps if cfg != 4 else min(args.steps, 12)
        m = self.measure(cfg, steps, args.warmup, full=True, sampler=sampler)
        clocks = sampler.stop() if sampler is not None else None
        batch = WORKLOADS[cfg]['batch']

        # host->device link: the binding roofline of the end-to-end rate
        link = {}
        if not args.kernels_only:
            conc = self.link_peak(concurrent=True) if self.world > 1 else None
            if conc is not None:
                per_rank = self.gather_ranks([conc])[:, 0]
                link['concurrent_gbs_per_rank'] = [float(v) for v in per_rank]
                link['concurrent_gbs_min'] = float(per_rank.min())
                link['concurrent_gbs_sum'] = float(per_rank.sum())
            raw = m['e2e_raw']
            stats = self.gather_ranks(list(raw['stage_ms']) + [raw['gather_ms'] if raw['gather_ms'] is not None else -1.0,
                                                               raw['ms'] / raw['steps']])
            link['per_rank'] = [{'stage_ms': {'parse': float(r[0]), 'layout': float(r[1]), 'copy': float(r[2]),
                                              'total': float(r[3])},
                                 'gather_kernel_ms': float(r[4]) if r[4] >= 0 else None, 'ms_per_step': float(r[5])}
                                for r in stats]
            # where the bytes lie and who reads them: the host's memory nodes, how much of the
            # memory file system's pages (the benchmark's file) each holds, and for every rank the
            # node of its GPU and the node its threads run on
            gpu_node, cpu_node, per_node = numa_placement(self.local)
            placement = self.gather_ranks([gpu_node, cpu_node])
            link['numa'] = {'shmem_mb_per_node': per_node,
                            'gpu_node_per_rank': [int(r[0]) for r in placement],
                            'cpu_node_per_rank': [int(r[1]) for r in placement]}

        # measured here, before the side passes below: whatever happens in those, the headline
        # line has all it needs
        solo = self.link_peak(concurrent=False) if self.world == 1 and not args.kernels_only else None

        configs = {}
        if self.world == 1 and not args.no_configs and not args.kernels_only and cfg == 2:
            for c in sorted(WORKLOADS):
                if c == cfg:
                    continue
                st = min(args.steps, 8 if c == 4 else 20)
                print(f'[bench] side pass: config {c}' + (' with the decode index' if self.decode_index else ''),
                      file=sys.stderr, flush=True)
                try:
                    r = self.measure(c, st, min(args.warmup, 3 if c == 4 else 5), full=False)
                    rl = self.roofline(r, c, clocks)
                    configs[f'c{c}'] = {'workload': WORKLOADS[c]['text'], 'batch': WORKLOADS[c]['batch'], 'steps': st,
                                        'value': r['value'], 'ms_per_step': r['ms_per_step'], 'e2e': r['e2e']['value'],
                                        'e2e_ms_per_step': r['e2e']['ms_per_step'],
                                        'h2d_bytes_per_step': r['e2e']['h2d_bytes_per_step'],
                                        'dominant_kernel': rl['kernel'], 'dominant_kernel_ms': rl['ms_per_launch'],
                                        'roofline': {k: rl.get(k) for k in ('bound', 'frac', 'profile_stale')},
                                        'kernel_ms': {n: r['kernels'][n]['ms'] for n in KERNELS}}
                except Exception as exc:  # noqa: BLE001 - a side measurement must not take the headline down
                    configs[f'c{c}'] = {'error': f'{type(exc).__name__}: {exc}'}
        # the same measurement with the decode index on (opt-in feature, reported beside the headline)
        indexed = {}
        if self.world == 1 and not args.no_configs and not args.kernels_only and self.decode_index == 0:
            self.decode_index = 1.0
            for c in sorted(WORKLOADS):
                if c == 0:
                    continue  # no JPEG samples
                st = min(args.steps, 8 if c == 4 else 20)
                print(f'[bench] side pass: config {c}' + (' with the decode index' if self.decode_index else ''),
                      file=sys.stderr, flush=True)
                try:
                    r = self.measure(c, st, min(args.warmup, 3 if c == 4 else 5), full=False)
                    indexed[f'c{c}'] = {'value': r['value'], 'ms_per_step': r['ms_per_step'], 'e2e': r['e2e']['value'],
                                        'e2e_ms_per_step': r['e2e']['ms_per_step'],
                                        'kernel_ms': {n: r['kernels'][n]['ms'] for n in KERNELS},
                                        'index': r.get('decode_index_stats')}
                except Exception as exc:  # noqa: BLE001
                    indexed[f'c{c}'] = {'error': f'{type(exc).__name__}: {exc}'}
            self.decode_index = 0.0
        if self.rank != 0:
            if self.world > 1:
                self.dist.destroy_process_group()
            return
        roofline = self.roofline(m, cfg, clocks)

        if not args.kernels_only:
            e2e = m['e2e']
            bytes_s = e2e['h2d_bytes_per_step'] / (m['e2e_raw']['ms'] / m['e2e_raw']['steps'] * 1e-3) / 1e9
            peak_link = solo if solo is not None else link.get('concurrent_gbs_min')
            e2e['h2d_roofline'] = {'bound': 'host->device link', 'achieved': bytes_s, 'peak': peak_link, 'unit': 'GB/s',
                                   'frac': bytes_s / peak_link if peak_link else None,
                                   'note': 'per GPU, rank 0; peak = pinned 256 MB cudaMemcpy measured in this run' +
                                           (', all ranks copying at once (slowest rank)' if solo is None else '')}
            e2e['h2d_roofline'].update(link)

        cpu = None
        if self.world == 1 and not args.no_cpu_baseline and not args.kernels_only:
            path = dataset_path(cfg, distinct_images(cfg, args, self.world), args.restart_interval)
            batches = oracle_batches(cfg, path, 0, 6 if cfg != 4 else 1)
            if cfg != 4:
                run_oracle(batches[:1], self.cores)
            t, done, t0 = [], 0, time.perf_counter()
            while time.perf_counter() - t0 < 12.0 and done < 60:
                t += run_oracle([batches[done % len(batches)]], self.cores)
                done += 1
            cpu = {'value': batch * done / sum(t), 'unit': 'images/s', 'cores': self.cores, 'kind': 'port',
                   'sample': f'{done} batches of {batch} images of the workload, all host threads',
                   'note': 'scalar C restatement of the path; an FFCV install with SIMD libjpeg-turbo and OpenCV is '
                           'expected to be 1.5-2x faster'}

        line = {'metric': 'RRC-224 decode+augment images/s', 'value': m['value'], 'unit': 'images/s', 'n_gpus': self.world,
                'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': m['ms_per_step'], 'higher_is_better': True,
                'scaling': 'weak', 'vs_baseline': None, 'dtype': 'u8', 'data': 'synthetic', 'config': m['config']}
        if steps != args.steps:
            line['steps_timed'] = steps
        if not args.kernels_only:
            line['e2e'] = m['e2e']
            for k in ('e2e_staged', 'e2e_gather', 'e2e_split', 'e2e_direct'):
                if k in m:
                    line[k] = m[k]
            line['gpu_launches'] = int(m['launches_per_batch'] * steps)
            line['digest'] = m['e2e_raw']['digest']
        else:
            line['gpu_launches'] = int(m['launches_per_batch'] * steps)
            line['batch_info'] = m['infos']
        line.update({'value_single_stream': m['value_single_stream'], 'roofline': roofline, 'cpu_baseline': cpu,
                     'clocks': clocks})
        if configs:
            line['configs'] = configs
        if indexed:
            line['decode_index'] = {'note': 'Loader(decode_index_gb=1): every JPEG stream decoded once before leaves the decoder states '
                                            'of its subsequences in GPU memory; later decodes take one pass from them (same pixels). '
                                            'Opt-in; the headline figures above are measured without it.', **indexed}
        print(json.dumps(line, default=float))
        if self.world > 1:
            self.dist.destroy_process_group()


if __name__ == '__main__':
    a = parse_args()
    if a.batch:
        WORKLOADS[a.config] = dict(WORKLOADS[a.config], batch=a.batch)
    if a.impl == 'reference':
        main_reference(a)
    else:
        Bench(a).main()
