"""Lowering of an image pipeline to one GPU launch per batch.

The reference runs ``decoder -> flip -> translate -> cutout`` as numba loops on host arrays, copies
the uint8 batch to the GPU in ``ToDevice`` and normalises it there
(``ffcv/loader/epoch_iterator.py:145-149``).  Here the longest prefix of a pipeline made of
operations that implement :meth:`Operation.fuse` becomes a :class:`FusedImagePlan`: the compressed
(or raw) sample bytes go to the GPU and one call of the native library produces the final tensor.
Operations after the fused prefix run one by one through their ``generate_code`` closures.
"""
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch as ch

from .. import libffcv as L
from .sampling import batch_seed


class FusedImagePlan:
    def __init__(self):
        self.decoder = None       # the RGB image decoder opening the pipeline
        self.crop_sampler = None  # operation that draws the crop boxes when it is not the decoder
        self.out_h = self.out_w = None
        self.resize = False
        self.dct_scale = 0        # scale of the JPEG decode (ffcvb_plan.dct_scale): 0 full, -1 by crop box
        self.ops = []             # (native type, arg, fill, operation) in pipeline order
        self.device = None        # set by ToDevice; defaults to the current CUDA device
        self.table = None         # 256 x 3 lookup table of the output type (numpy), or None
        self.torch_image = False  # result presented as (B, C, H, W)
        self.channels_last = True
        self.sealed = False       # no spatial operation may follow (values are no longer uint8)
        self.fused_ops = []

    # ---- called by Operation.fuse implementations
    def set_decoder(self, op, out_h, out_w, resize):
        if self.decoder is not None:
            return False
        self.decoder, self.out_h, self.out_w, self.resize = op, int(out_h), int(out_w), bool(resize)
        return True

    def set_post_crop(self, op, size):
        """A random-resized-crop transform right behind a pass-through decoder is the crop-and-resize
        of the decoder itself."""
        if self.decoder is None or self.resize or self.ops or self.sealed or self.torch_image:
            return False
        self.crop_sampler = op
        self.out_h = self.out_w = int(size)
        self.resize = True
        return True

    def add_spatial(self, native_type, arg, fill, op):
        if self.decoder is None or self.sealed or self.torch_image or len(self.ops) >= L.MAX_OPS:
            return False
        self.ops.append((native_type, int(arg), tuple(int(v) for v in fill), op))
        return True

    def set_table(self, table):
        """table: float16/float32 array [256, 3]; replaces an earlier one (a Convert followed by
        NormalizeImage indexes the normalisation table with the uint8 value)."""
        if self.decoder is None:
            return False
        if self.sealed and self.table is not None and not getattr(self, '_table_is_identity', False):
            return False
        self.table = np.ascontiguousarray(table)
        self.sealed = True
        return True

    def set_identity_table(self, dtype):
        ok = self.set_table(np.repeat(np.arange(256, dtype=dtype)[:, None], 3, axis=1))
        self._table_is_identity = ok
        return ok

    def set_torch_image(self, channels_last):
        if self.decoder is None or self.torch_image:
            return False
        self.torch_image, self.channels_last = True, bool(channels_last)
        return True

    # ---- derived
    @property
    def out_kind(self):
        if self.table is None:
            return L.OUT_U8_NHWC
        planar = self.torch_image and not self.channels_last
        if self.table.dtype == np.float16:
            return L.OUT_F16_NCHW if planar else L.OUT_F16_NHWC
        return L.OUT_F32_NCHW if planar else L.OUT_F32_NHWC

    @property
    def torch_dtype(self):
        if self.table is None:
            return ch.uint8
        return ch.float16 if self.table.dtype == np.float16 else ch.float32

    @property
    def buffer_shape(self):
        if self.torch_image and not self.channels_last and self.table is not None:
            return (3, self.out_h, self.out_w)
        return (self.out_h, self.out_w, 3)

    def needs_repack(self):
        # uint8 output asked for as contiguous NCHW: the kernel writes NHWC, torch repacks
        return self.torch_image and not self.channels_last and self.table is None


def host_plan(ops, field, metadata):
    """The :class:`FusedImagePlan` of the longest fusable prefix of ``ops`` (decoder first), built
    on the host alone: no native context, no GPU.  ``metadata`` is the field's metadata column."""
    plan = FusedImagePlan()
    for op in ops:
        op.accept_field(field)
        op.accept_globals(metadata, None)
        if not op.fuse(plan):
            break
        plan.fused_ops.append(op)
    return plan


def sample_plan_params(plan, md, base_seed, epoch, batch_ix):
    """Parameter table of one batch, ``[n, 4 + 2 * len(plan.ops)]`` int32: the crop box of every
    sample followed by the two values each augmentation draws.  ``md``: the batch's metadata rows.
    Every operation seeds its own stream from (seed, epoch, batch, position in the pipeline)."""
    heights = np.ascontiguousarray(md['height'])
    widths = np.ascontiguousarray(md['width'])
    n = len(md)
    params = np.zeros((n, 4 + 2 * len(plan.ops)), dtype=np.int32)
    crops = np.zeros((n, 4), dtype=np.int32)
    (plan.crop_sampler or plan.decoder).sample_crops(batch_seed(base_seed, epoch, batch_ix, 0), heights, widths, crops)
    params[:, :4] = crops
    for k, (_, _, _, op) in enumerate(plan.ops):
        col = np.zeros((n, 2), dtype=np.int32)
        op.sample_params(batch_seed(base_seed, epoch, batch_ix, k + 1), n, plan.out_h, plan.out_w, col)
        params[:, 4 + 2 * k:6 + 2 * k] = col
    return params


class FusedImageExecutor:
    """Per-batch driver of a :class:`FusedImagePlan` on one native context."""

    def __init__(self, plan: FusedImagePlan, ctx, metadata, sample_sizes, file_base_fn, base_seed):
        self.plan = plan
        self.ctx = ctx
        self.metadata = metadata
        self.sample_sizes = sample_sizes
        self.file_base_fn = file_base_fn
        self.base_seed = int(base_seed) & 0xFFFFFFFF
        self.device = plan.device if plan.device is not None else ch.device('cuda', ch.cuda.current_device())
        self.table_dev = None
        if plan.table is not None:
            raw = plan.table.view(np.int16 if plan.table.dtype == np.float16 else np.int32)
            self.table_dev = ch.from_numpy(raw.copy()).to(self.device)
        ops = [(t, a, f) for (t, a, f, _) in plan.ops]
        self.native_plan = L.make_plan(plan.out_h, plan.out_w, plan.resize, L.OUT_U8_NHWC if plan.needs_repack()
                                       else plan.out_kind, ops,
                                       self.table_dev.data_ptr() if self.table_dev is not None else 0,
                                       dct_scale=plan.dct_scale)
        self.n_params = 4 + 2 * len(ops)
        self.last_params = None
        self._prepared = None     # ((epoch, batch, n), arrays) drawn ahead for the next batch
        self.param_log = None     # set to a list to record (epoch, batch, indices, parameter table) per batch
        self.h2d_bytes = 0
        self.launches = 0
        self.riders = []          # other fields' values for the next batch (see Graph.attach_riders)
        self._helper = None       # one thread that draws the next batch's parameters (see __call__)

    def allocate(self, batch_size, slots):
        p = self.plan
        return [ch.empty((batch_size,) + p.buffer_shape, dtype=p.torch_dtype, device=self.device) for _ in range(slots)]

    def sample_params(self, batch_indices, epoch, batch_ix):
        md = self.metadata[batch_indices]
        params = sample_plan_params(self.plan, md, self.base_seed, epoch, batch_ix)
        return md, np.ascontiguousarray(md['height']), np.ascontiguousarray(md['width']), params

    def prepare(self, batch_indices, epoch, batch_ix):
        """Everything ffcvb_stage_batch needs for one batch, as contiguous arrays."""
        md, heights, widths, params = self.sample_params(batch_indices, epoch, batch_ix)
        return (np.ascontiguousarray(md['data_ptr'], dtype=np.uint64),
                np.ascontiguousarray(self.sample_sizes[batch_indices], dtype=np.uint64),
                np.ascontiguousarray(md['mode'], dtype=np.uint8), heights, widths, params)

    def __call__(self, batch_indices, slot, stream_ptr, out, epoch, batch_ix, lookahead=None):
        key = (epoch, batch_ix, len(batch_indices))
        if self._prepared is not None and self._prepared[0] == key:
            args = self._prepared[1]
        else:
            args = self.prepare(batch_indices, epoch, batch_ix)
        self._prepared = None
        params = args[5]
        self.last_params = params
        if self.param_log is not None:
            self.param_log.append((epoch, batch_ix, np.array(batch_indices), params.copy()))
        n = len(batch_indices)
        if self.riders:
            self.ctx.set_riders(slot, self.riders, n)
            self.riders = []
        # The next batch's parameters are drawn by a helper thread while this thread is inside the
        # native calls (which release the interpreter lock): the loader thread's time per batch is
        # what bounds the rate of the low-resolution configurations.
        ahead = None
        if lookahead is not None:
            if self._helper is None:
                self._helper = ThreadPoolExecutor(max_workers=1, thread_name_prefix='ffcv_b200_params')
            ahead = self._helper.submit(self.prepare, lookahead, epoch, batch_ix + 1)
        try:
            # with asynchronous staging this returns while the staging threads still copy the payloads
            self.ctx.stage(slot, self.file_base_fn(), *args[:5], self.native_plan, params)
            dst = out[:n]
            self.ctx.submit(slot, stream_ptr, dst.data_ptr())
        finally:
            if ahead is not None:
                self._prepared = ((epoch, batch_ix + 1, len(lookahead)), ahead.result())
        self.h2d_bytes = self.ctx.staged_bytes(slot)
        self.launches = self.ctx.launches(slot)
        p = self.plan
        if p.torch_image:
            if p.needs_repack():
                return dst.permute(0, 3, 1, 2).contiguous()
            if p.channels_last:
                return dst.permute(0, 3, 1, 2)
        return dst
