#!/usr/bin/env python
"""Benchmark of the decode-and-augment hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: configuration 2 of the benchmark contract, a synthetic ImageNet-shaped `.beton`
(write_mode='proportion', 50 % JPEG q90 4:2:0 / 50 % raw, short side 300-500, max side 500) read
through RandomResizedCropRGBImageDecoder((224, 224)) -> RandomHorizontalFlip -> NormalizeImage
(fp16) -> ToTorchImage, batch 512 per GPU.  A "step" is one batch.  The dataset is a bounded,
seeded sample of that configuration (see --images) written before the timed region.

One JSON line on stdout (rank 0):
  value      images/s with the batch bytes already resident in HBM (kernels only, CUDA events), the
             slots on their own streams as the loader runs them; value_single_stream = the same on
             one stream (the pass the per-kernel durations come from)
  e2e        images/s through `for batch in Loader(...)`: host staging from the memory-mapped file,
             host->device copy, kernels, and an 8-byte device->host read per step
  roofline   the dominant kernel's algorithmic bytes / its measured duration vs the measured HBM peak
  cpu_baseline  the CPU oracle port on all host threads, bounded sample (rank 0, N = 1)
With --impl reference the same workload runs on the CPU oracle port only (no GPU work).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 512
OUT = 224
CFG = 2
EPOCH_SAMPLES = 200_000
IMAGENET_MEAN = np.array([0.485, 0.456, 0.406]) * 255
IMAGENET_STD = np.array([0.229, 0.224, 0.225]) * 255
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per unit of work, from the ncu capture
# summarised in profiles/config2_batch512_all_kernels.txt (same workload, 512-sample launches):
# per JPEG sample for the three decode kernels, per sample for the fused resize kernel.
# Warp instructions executed (smsp__inst_executed.sum) per unit of work, same captures: the decode
# and resize kernels are bound by instruction issue, not by HBM.
NCU_WARP_INST_PER_UNIT = {
    'entropy_decode': (133.35e6 / 240 + 111.50e6 / 200) / 2,
    'idct': (33.66e6 / 240 + 28.67e6 / 200) / 2,
    'upsample_colour': (87.30e6 / 240 + 74.58e6 / 200) / 2,
    'resize_augment_normalise': 321.94e6 / 512,
}
SM_COUNT, ISSUE_PER_SM_CLK = 148, 4  # B200: 148 SMs, four warp schedulers each, one instruction per clock
NCU_DRAM_BYTES_PER_UNIT = {
    'entropy_decode': ((19.13e6 + 148.67e6) / 240 + (10.12e6 + 108.26e6) / 200) / 2,
    'idct': ((69.30e6 + 11.66e6) / 240 + (59.13e6 + 5.72e6) / 200) / 2,
    'upsample_colour': ((42.54e6 + 15.69e6) / 240 + (36.06e6 + 8.52e6) / 200) / 2,
    'resize_augment_normalise': (128.75e6 + 108.14e6) / 512,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=10)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--images', type=int, default=4096, help='distinct images in the synthetic dataset')
    ap.add_argument('--workers', type=int, default=0, help='host staging threads per rank (0: cores / ranks)')
    ap.add_argument('--batches-ahead', type=int, default=3)
    ap.add_argument('--restart-interval', type=int, default=0,
                    help='write the JPEG samples with a restart marker every N MCUs (0: as the reference writes them)')
    ap.add_argument('--no-cpu-baseline', action='store_true', help='skip the CPU oracle leg (profiling runs)')
    return ap.parse_args()


def rank_info():
    return (int(os.environ.get('RANK', 0)), int(os.environ.get('LOCAL_RANK', 0)),
            int(os.environ.get('WORLD_SIZE', 1)))


def dataset_path(images, restart_interval=0):
    base = '/dev/shm' if os.path.isdir('/dev/shm') and os.access('/dev/shm', os.W_OK) else tempfile.gettempdir()
    tag = f'_rst{restart_interval}' if restart_interval else ''
    return os.path.join(base, f'ffcv_b200_bench_c{CFG}_{images}_of_{EPOCH_SAMPLES}{tag}.beton')


def ensure_dataset(images, restart_interval=0):
    """Written once (rank 0) before any timing; other ranks wait for the barrier that follows."""
    from ffcv_b200.synthetic import replicate_samples, write_dataset_isolated as write_dataset  # forks workers
    path = dataset_path(images, restart_interval)
    if not os.path.exists(path):
        tmp = path + f'.tmp{os.getpid()}'
        write_dataset(CFG, tmp, images, num_workers=len(os.sched_getaffinity(0)), restart_interval=restart_interval)
        # the configuration's epoch length (200,000 samples) over the bounded set of distinct images
        replicate_samples(tmp, EPOCH_SAMPLES)
        os.replace(tmp, path)
    return path


def read_peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        try:
            return float(json.load(open(p))['hbm_gbs']), 'measured'
        except Exception:
            pass
    return 6650.0, 'fallback'


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


def build_pipelines(device):
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToDevice, ToTensor, ToTorchImage
    return {'image': [RandomResizedCropRGBImageDecoder((OUT, OUT)), RandomHorizontalFlip(), ToTensor(),
                      ToDevice(device), ToTorchImage(), NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16)],
            'label': None}


def oracle_batches(path, seed, n_batches, rank=0, world=1):
    """The same batches (bytes + sampled parameters) the loader would see, for the CPU oracle."""
    from ffcv_b200.memory_managers import OSCacheManager
    from ffcv_b200.pipeline.sampling import batch_seed, sample_flips, sample_random_crops
    from ffcv_b200.reader import Reader
    r = Reader(path)
    mm = OSCacheManager(r)
    mmap = mm.open()
    md = r.metadata['f0']
    sizes = mm.sizes_of(md['data_ptr'])
    order = np.arange(r.num_samples)[rank::world]
    out = []
    for b in range(n_batches):
        ix = order[(np.arange(BATCH) + b * BATCH) % len(order)]
        m = md[ix]
        h, w = np.ascontiguousarray(m['height']), np.ascontiguousarray(m['width'])
        crops = np.zeros((BATCH, 4), np.int32)
        sample_random_crops(batch_seed(seed, 0, b, 0), h, w, np.array([0.08, 1.0]), np.array([0.75, 4 / 3]), crops)
        flips = np.zeros((BATCH, 2), np.int32)
        sample_flips(batch_seed(seed, 0, b, 1), BATCH, 0.5, flips)
        payloads = [np.asarray(mmap[int(p):int(p) + int(s)]) for p, s in zip(m['data_ptr'], sizes[ix])]
        out.append((payloads, m['mode'], h, w, crops, flips))
    return out


def run_oracle(batches, threads):
    """Runs the CPU oracle over the given batches; returns seconds per batch (list)."""
    from oracle import oracle as O
    table = O.normalize_table(IMAGENET_MEAN, IMAGENET_STD, np.float16)
    times = []
    for payloads, modes, h, w, crops, flips in batches:
        ops = [[(O.OP_FLIP, int(f[0]), 0, 0, (0, 0, 0))] for f in flips]
        t0 = time.perf_counter()
        _, status = O.run_batch(payloads, modes, h, w, crops, 1, OUT, OUT, ops, table, O.OUT_F16_NHWC, threads)
        times.append(time.perf_counter() - t0)
        assert (status == 0).all()
    return times


def config_dict(world, images, workers, restart_interval=0):
    cfg = {'workload': 'config 2: proportion(0.5) JPEG q90 4:2:0 / raw, short side 300-500, max side 500 -> '
                        'RRC-224 + flip + fp16 normalise, channels-last',
            'batch_per_gpu': BATCH, 'global_batch': BATCH * world, 'dataset_samples': EPOCH_SAMPLES,
            'distinct_images': images,
            'order': 'QUASI_RANDOM', 'sharding': 'index sharding, no collective' if world > 1 else 'single GPU',
            'host_threads_per_rank': workers,
            'l2': 'inputs larger than L2: consecutive steps read different batches (5 slots x ~100 MB)'}
    if restart_interval:
        cfg['jpeg_restart_interval'] = restart_interval  # not the reference's file format default
    return cfg


def main_reference(args):
    """The reference arm: the path on the host cores only (CPU oracle port, all threads)."""
    rank, _, world = rank_info()
    if rank != 0:
        return
    path = ensure_dataset(args.images * min(world, 4), args.restart_interval)
    threads = len(os.sched_getaffinity(0))
    n = args.steps + args.warmup
    batches = oracle_batches(path, 0, min(n, 8))
    seq = [batches[i % len(batches)] for i in range(n)]
    run_oracle(seq[:args.warmup], threads)
    times = run_oracle(seq[args.warmup:], threads)
    total = sum(times)
    value = BATCH * args.steps / total
    line = {'impl': 'reference', 'metric': 'RRC-224 decode+augment images/s', 'value': value, 'unit': 'images/s',
            'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * total / args.steps,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'u8', 'data': 'synthetic',
            'config': config_dict(world, args.images * min(world, 4), threads, args.restart_interval),
            'cpu_baseline': {'value': value, 'unit': 'images/s', 'cores': threads, 'kind': 'port',
                             'sample': f'{args.steps} batches of {BATCH} images of the workload'},
            'e2e': {'value': value, 'unit': 'images/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
            'gpu_launches': 0}
    print(json.dumps(line))


def main_ours(args):
    import torch as ch
    import torch.distributed as dist
    rank, local, world = rank_info()
    if not ch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: ffcv_b200 has no CPU fallback')
    ch.cuda.set_device(local)
    device = ch.device('cuda', local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        # stdout carries the one JSON line: while the communicator comes up (NCCL prints its version
        # banner there) file descriptor 1 points at stderr
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group('nccl', device_id=device)
            dist.barrier(device_ids=[local])
            ch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])

    images = args.images * min(world, 4)
    if rank == 0:
        ensure_dataset(images, args.restart_interval)
    barrier()
    path = dataset_path(images, args.restart_interval)
    cores = len(os.sched_getaffinity(0))
    workers = args.workers or max(2, cores // max(1, world))

    from ffcv_b200 import Loader, OrderOption

    def make_loader(pin, share=None):
        return Loader(path, batch_size=BATCH, order=OrderOption.QUASI_RANDOM, distributed=world > 1, seed=0,
                      num_workers=workers, pipelines=build_pipelines(device), batches_ahead=args.batches_ahead,
                      drop_last=True, pin_file=pin, cpu_stage_share=share)

    def describe(ld):
        if not ld.memory_manager.pinned:
            return 'file memory-mapped, staged into pinned buffers by CPU threads, one DMA copy per batch'
        if ld.stage_split == 0:
            return 'file in pinned host RAM, payloads gathered by the GPU over PCIe'
        return ('file in pinned host RAM: the GPU gathers most payload bytes over PCIe, up to 4 CPU threads and the '
                'copy engine carry the rest (share %s)' % ('balanced per batch' if ld.stage_split < 0
                                                           else '%.2f' % (ld.stage_split / 1000)))

    def run_e2e(loader, sampler=None):
        exe = loader.graph.pipelines[0].executor

        def endless():
            while True:
                for b in loader:
                    yield b
        it = endless()
        digest = 0.0
        for _ in range(args.warmup):
            digest += float(next(it)[0][:, 0, ::32, ::32].float().sum().item())
        ch.cuda.synchronize()
        barrier()
        if sampler is not None:
            sampler.start()
        e0, e1 = ch.cuda.Event(enable_timing=True), ch.cuda.Event(enable_timing=True)
        h2d = []
        e0.record()
        for _ in range(args.steps):
            x = next(it)[0]
            digest += float(x[:, 0, ::32, ::32].float().sum().item())  # 8-byte device->host read per step
            h2d.append(exe.h2d_bytes)
        e1.record()
        ch.cuda.synchronize()
        barrier()
        loader._live_iterator.retire()
        return e0.elapsed_time(e1), int(np.mean(h2d)), exe.launches, digest

    # ------------------------------------------------------------------ end to end (public API)
    # `e2e` is the mode Loader picks by itself on this host (pin_file=None, cpu_stage_share=None);
    # the other ways the bytes can reach the GPU are timed beside it.
    auto = make_loader(None)
    auto_mode = (auto.pin_file, auto.stage_split)
    del auto
    others = {}
    for name, pin, share in [('e2e_staged', False, None), ('e2e_gather', True, 0.0), ('e2e_split', True, None)]:
        probe = make_loader(pin, share)
        if (probe.pin_file, probe.stage_split) == auto_mode or (name == 'e2e_split' and probe.stage_split == 0):
            del probe
            continue
        ms, h2d, _, _ = run_e2e(probe)
        if world > 1:
            t = ch.tensor([ms], dtype=ch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        others[name] = {'value': BATCH * world * args.steps / (ms * 1e-3), 'unit': 'images/s',
                        'ms_per_step': ms / args.steps, 'h2d_bytes_per_step': h2d, 'source': describe(probe)}
        del probe
    sampler = ClockSampler(local)
    loader = make_loader(None)
    exe = loader.graph.pipelines[0].executor
    ctx = exe.ctx
    e2e_ms, h2d_mean, launches_per_batch, digest = run_e2e(loader, sampler if rank == 0 else None)

    # ------------------------------------------------------------------ inputs resident in HBM
    slots = loader.batches_ahead + 2
    stream = ch.cuda.current_stream(device)
    outs = loader.slot_buffers()[(0, 'fused')]
    order = loader.traversal_order.sample_order(10_000)
    infos, crop_bytes = [], []
    for s in range(slots):
        ix = np.asarray(order[(np.arange(BATCH) + s * BATCH) % len(order)])
        exe(ix, s, stream.cuda_stream, outs[s], 10_000, s)
        infos.append(ctx.batch_info(s))
        p = exe.last_params
        crop_bytes.append(int((p[:, 2].astype(np.int64) * p[:, 3] * 3).sum()))
    ch.cuda.synchronize()
    # (1) per-kernel durations: one stream, kernels back to back, library events around each
    ctx.set_profiling(True)
    for k in range(args.warmup):
        ctx.rerun(k % slots, stream.cuda_stream, outs[k % slots].data_ptr())
    ch.cuda.synchronize()
    barrier()
    kernel_ms = []
    s0, s1 = ch.cuda.Event(enable_timing=True), ch.cuda.Event(enable_timing=True)
    s0.record(stream)
    for k in range(args.steps):
        s = k % slots
        if k >= slots:
            kernel_ms.append(ctx.batch_times(s))  # waits only for a run queued `slots` steps ago
        ctx.rerun(s, stream.cuda_stream, outs[s].data_ptr())
    s1.record(stream)
    ch.cuda.synchronize()
    barrier()
    for s in range(min(slots, args.steps)):
        kernel_ms.append(ctx.batch_times(s))
    serial_ms = s0.elapsed_time(s1)
    ctx.set_profiling(False)
    # (2) throughput the way the loader drives the device: every slot on its own stream, so the
    # kernels of consecutive batches overlap (the entropy kernel is latency-bound at this batch
    # size and leaves issue slots to the others)
    slot_streams = loader.slot_streams()
    for k in range(args.warmup):
        ctx.rerun(k % slots, slot_streams[k % slots].cuda_stream, outs[k % slots].data_ptr())
    ch.cuda.synchronize()
    barrier()
    v0, v1 = ch.cuda.Event(enable_timing=True), ch.cuda.Event(enable_timing=True)
    v0.record(stream)
    for st_ in slot_streams:
        st_.wait_event(v0)
    for k in range(args.steps):
        ctx.rerun(k % slots, slot_streams[k % slots].cuda_stream, outs[k % slots].data_ptr())
    for st_ in slot_streams:
        stream.wait_stream(st_)
    v1.record(stream)
    ch.cuda.synchronize()
    barrier()
    value_ms = v0.elapsed_time(v1)
    clocks = sampler.stop() if rank == 0 else None

    times = ch.tensor([e2e_ms, value_ms, serial_ms], dtype=ch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    e2e_ms, value_ms, serial_ms = (float(v) for v in times.cpu())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ------------------------------------------------------------------ roofline of the dominant kernel
    km = np.mean(np.array(kernel_ms), axis=0)  # [h2d (unused here), entropy, idct, colour, resize]
    mean = {k: float(np.mean([i[k] for i in infos])) for k in infos[0]}
    out_bytes = BATCH * OUT * OUT * 3 * 2
    crop_mean = float(np.mean(crop_bytes))
    raw_frac = 1.0 - mean['n_jpeg'] / BATCH
    algo = {
        'entropy_decode': mean['scan_bytes'] + 128 * mean['blocks'],
        'idct': 128 * mean['blocks'] + mean['plane_bytes'],
        # only the crop box of the JPEG samples is converted: Y + 2 quarter-size chroma planes read
        # (1.5 B/pixel), RGB written (3 B/pixel); crop_mean is the mean crop size in RGB bytes
        'upsample_colour': crop_mean * (1.0 - raw_frac) * 1.5,
        'resize_augment_normalise': crop_mean + out_bytes,
    }
    names = list(algo)
    total_kernel_ms = float(km[1:].sum())
    kernels = {n: {'ms': float(km[i + 1]), 'share': float(km[i + 1] / total_kernel_ms),
                   'algorithmic_bytes': algo[n], 'gbs': algo[n] / (km[i + 1] * 1e-3) / 1e9}
               for i, n in enumerate(names)}
    dom = max(names, key=lambda n: kernels[n]['ms'])
    peak, peak_kind = read_peaks()
    path_bytes = mean['jpeg_bytes'] + crop_mean * raw_frac + out_bytes  # payload read once + output written once
    units = {'entropy_decode': mean['n_jpeg'], 'idct': mean['n_jpeg'], 'upsample_colour': mean['n_jpeg'],
             'resize_augment_normalise': float(BATCH)}
    for n in names:
        kernels[n]['ncu_dram_bytes'] = NCU_DRAM_BYTES_PER_UNIT[n] * units[n]
    # second roofline of every kernel: the time its instructions would need if every warp scheduler
    # of the GPU issued one of them per clock (clock: the median SM clock sampled during the run)
    sm_hz = (clocks['sm_mhz'] if clocks and clocks.get('sm_mhz') else 1965.0) * 1e6
    for n in names:
        inst = NCU_WARP_INST_PER_UNIT[n] * units[n]
        floor_ms = inst / (SM_COUNT * ISSUE_PER_SM_CLK * sm_hz) * 1e3
        kernels[n]['issue'] = {'warp_instructions': inst, 'floor_ms': floor_ms, 'frac': floor_ms / kernels[n]['ms']}
    roofline = {'bound': 'hbm', 'kernel': dom, 'achieved': kernels[dom]['gbs'], 'peak': peak, 'unit': 'GB/s',
                'frac': kernels[dom]['gbs'] / peak, 'traffic': kernels[dom]['ncu_dram_bytes'], 'peak_kind': peak_kind,
                'traffic_source': 'ncu capture of the same workload, scaled by the JPEG samples per launch',
                'ms_per_launch': kernels[dom]['ms'], 'kernels': kernels,
                'issue': {'bound': 'integer issue (the binding one for this kernel)', 'unit': 'warp instructions/s',
                          'achieved': kernels[dom]['issue']['warp_instructions'] / (kernels[dom]['ms'] * 1e-3),
                          'peak': SM_COUNT * ISSUE_PER_SM_CLK * sm_hz, 'frac': kernels[dom]['issue']['frac'],
                          'source': 'smsp__inst_executed.sum of the ncu capture, scaled by the JPEG samples per launch'},
                'path': {'algorithmic_bytes_per_step': path_bytes, 'kernel_ms_per_step': total_kernel_ms,
                         'gbs': path_bytes / (total_kernel_ms * 1e-3) / 1e9}}

    # host->device link: the binding roofline of the end-to-end rate (pinned copy, 256 MB, best of 5)
    hbuf = ch.empty(256 << 20, dtype=ch.uint8).pin_memory()
    dbuf = ch.empty(256 << 20, dtype=ch.uint8, device=device)
    best = 1e9
    for _ in range(6):
        a, b = ch.cuda.Event(enable_timing=True), ch.cuda.Event(enable_timing=True)
        a.record()
        dbuf.copy_(hbuf, non_blocking=True)
        b.record()
        b.synchronize()
        best = min(best, a.elapsed_time(b))
    h2d_peak = (256 << 20) / (best * 1e-3) / 1e9
    del hbuf, dbuf

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = cores
        batches = oracle_batches(path, 0, 6)
        run_oracle(batches[:1], threads)
        t, done, t0 = [], 0, time.perf_counter()
        while time.perf_counter() - t0 < 12.0 and done < 60:
            t += run_oracle([batches[done % len(batches)]], threads)
            done += 1
        cpu = {'value': BATCH * done / sum(t), 'unit': 'images/s', 'cores': threads, 'kind': 'port',
               'sample': f'{done} batches of {BATCH} images of the workload, all host threads'}

    line = {'metric': 'RRC-224 decode+augment images/s', 'value': BATCH * world * args.steps / (value_ms * 1e-3),
            'unit': 'images/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': value_ms / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
            'dtype': 'u8', 'data': 'synthetic', 'config': config_dict(world, images, workers, args.restart_interval),
            'e2e': {'value': BATCH * world * args.steps / (e2e_ms * 1e-3), 'unit': 'images/s',
                    'ms_per_step': e2e_ms / args.steps, 'h2d_bytes_per_step': h2d_mean,
                    'd2h_bytes_per_step': 8,
                    'h2d_roofline': {'bound': 'host->device link', 'achieved': h2d_mean / (e2e_ms / args.steps * 1e-3) / 1e9,
                                     'peak': h2d_peak, 'unit': 'GB/s', 'frac': h2d_mean / (e2e_ms / args.steps * 1e-3) / 1e9 / h2d_peak,
                                     'note': 'per GPU, rank 0; peak = pinned 256 MB cudaMemcpy measured in this run'},
                    'source': describe(loader)},
            **others,
            'value_single_stream': {'value': BATCH * world * args.steps / (serial_ms * 1e-3), 'unit': 'images/s',
                                    'ms_per_step': serial_ms / args.steps},
            'gpu_launches': int(launches_per_batch * args.steps), 'roofline': roofline, 'cpu_baseline': cpu,
            'clocks': clocks, 'digest': digest}
    print(json.dumps(line, default=float))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    a = parse_args()
    if a.impl == 'reference':
        main_reference(a)
    else:
        main_ours(a)
