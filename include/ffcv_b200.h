/*
 * ffcv_b200 — C ABI of the B200 (sm_100a) decode-and-augment library, libffcv_b200.so.
 *
 * It replaces the native half of FFCV's image path: libffcv/libffcv.cpp (`imdecode` ->
 * tjDecompress2, `resize` -> cv::resize INTER_AREA, `my_memcpy`) together with the per-batch work
 * of the numba closures in ffcv/fields/rgb_image.py and ffcv/transforms/{flip,translate,cutout,
 * normalize}.py.  Plain pointers and sizes only; no torch or CUDA types appear in a signature
 * (a CUDA stream travels as `void *`, i.e. a cudaStream_t / CUstream handle, NULL = default).
 *
 * Error convention: every function that can fail returns 0 on success and a negative FFCVB_E_*
 * code otherwise; nothing throws and no kernel traps.  ffcvb_last_error() gives the message of
 * the last failure on a context.  Per-sample decode problems (corrupt or unsupported JPEG) do not
 * fail the batch: they are reported through ffcvb_batch_status().
 *
 * Threading: one context per consumer thread.  Calls on one context must not overlap.  Batch
 * work is asynchronous with respect to the given stream; a slot's host and device buffers may be
 * reused once work queued on that stream for the slot's previous batch has completed (the caller
 * fences this with events exactly as ffcv/loader/epoch_iterator.py:96-108,127-129 does).
 */
#ifndef FFCV_B200_H
#define FFCV_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    FFCVB_OK = 0,
    FFCVB_E_CUDA = -1,     /* a CUDA runtime call failed */
    FFCVB_E_ARG = -2,      /* invalid argument */
    FFCVB_E_NOMEM = -3,    /* host or device allocation failed */
    FFCVB_E_DECODE = -4,   /* JPEG stream could not be decoded (single-image entry points) */
    FFCVB_E_NODEVICE = -5, /* no usable CUDA device */
    FFCVB_E_LIMIT = -6     /* a fixed capacity was exceeded */
};

/* Sample storage modes, ffcv/fields/rgb_image.py:21-23. */
enum { FFCVB_MODE_JPG = 0, FFCVB_MODE_RAW = 1 };

/* Layout and type of the batch output. */
enum {
    FFCVB_OUT_U8_NHWC = 0,  /* uint8  [n, h, w, 3] */
    FFCVB_OUT_F16_NHWC = 1, /* fp16   [n, h, w, 3], values from the lookup table */
    FFCVB_OUT_F16_NCHW = 2, /* fp16   [n, 3, h, w] */
    FFCVB_OUT_F32_NHWC = 3, /* fp32   [n, h, w, 3] */
    FFCVB_OUT_F32_NCHW = 4  /* fp32   [n, 3, h, w] */
};

/* Augmentations applied after the decoder, in pipeline order. */
enum {
    FFCVB_OP_FLIP = 1,      /* ffcv/transforms/flip.py:31-39       param: (flip?, unused) */
    FFCVB_OP_TRANSLATE = 2, /* ffcv/transforms/translate.py:35-44  arg = padding, param: (y, x) */
    FFCVB_OP_CUTOUT = 3     /* ffcv/transforms/cutout.py:36-46     arg = size,    param: (y, x) */
};

#define FFCVB_MAX_OPS 8

typedef struct {
    int32_t type;    /* FFCVB_OP_* */
    int32_t arg;     /* padding (translate) or square size (cutout) */
    uint8_t fill[4]; /* RGB fill colour, 4th byte unused */
} ffcvb_op;

/* What one batch call computes.  The per-sample random draws are NOT made here: the caller
 * samples them (ffcv/fields/rgb_image.py:48-81, flip.py:32, translate.py:40-41, cutout.py:39-42)
 * and passes them as `params`, one row of 4 + 2 * n_ops int32 per sample:
 *   [crop_row, crop_col, crop_h, crop_w,  op0_a, op0_b,  op1_a, op1_b, ...]
 * The crop box is ignored when resize == 0. */
typedef struct {
    int32_t out_h, out_w; /* spatial size of every output image */
    int32_t resize;       /* 0: images pass through at their stored size (SimpleRGBImageDecoder,
                             rgb_image.py:84-139; every image must be out_h x out_w);
                             1: crop box + INTER_AREA resize (rgb_image.py:142-217) */
    int32_t out_kind;     /* FFCVB_OUT_* */
    int32_t n_ops;
    ffcvb_op ops[FFCVB_MAX_OPS];
    int32_t dct_scale;    /* decode JPEG samples at reduced scale, the scale_num / scale_denom of
                             libffcv/libffcv.cpp:59,89-90 (which every call of the reference sets to
                             1 / 1): 0 = full scale (default); 1, 2, 3 = every JPEG sample at 1/2,
                             1/4, 1/8 (samples whose chroma layout does not allow it are flagged);
                             -1 (needs resize == 1) = per sample the smallest scale at which its
                             crop box still has at least out_h x out_w pixels, then the box is
                             mapped to the scaled image (rows [i >> s, ceil((i + h) / 2^s)), same for
                             columns) and resized from there.  Scaled decodes equal libjpeg-turbo's
                             bit for bit, but a crop resized from a scaled decode is not the crop
                             resized from the full decode: not the reference's pixels, hence opt-in. */
    const void *lut_dev; /* DEVICE pointer to the 256 x 3 normalisation table of the output type
                            (ffcv/transforms/normalize.py:42-49); unused for FFCVB_OUT_U8_NHWC */
} ffcvb_plan;

typedef struct ffcvb_ctx ffcvb_ctx;

/* Creates a context bound to CUDA device `device` with `n_slots` independent batch slots (the
 * ring of ffcv/loader/epoch_iterator.py:62-68) and `n_threads` host staging threads (<= 0: one
 * per available core, capped at 32).  Replaces the per-thread TurboJPEG handles of
 * libffcv/libffcv.cpp:21-31,63-76. */
int ffcvb_create(int device, int n_slots, int n_threads, ffcvb_ctx **out);
void ffcvb_destroy(ffcvb_ctx *ctx);
const char *ffcvb_last_error(const ffcvb_ctx *ctx);

/* Stage one batch: gathers the payload bytes of `n` samples (sample i occupies
 * file_base[ptrs[i] .. ptrs[i] + sizes[i]), the byte range `memory_read` returns in
 * ffcv/memory_managers/os_cache.py:55-60) into the slot's pinned buffer with the staging threads,
 * parses JPEG headers, and lays out the device work.  modes/heights/widths are the per-sample
 * metadata columns of ffcv/fields/rgb_image.py:301-308.  Raw samples stage only their crop box.
 * When `file_base` lies in page-locked, device-mapped host memory (cudaHostAlloc, or
 * ffcvb_host_register below) nothing is copied here: ffcvb_submit_batch lets the GPU fetch the
 * payloads itself over PCIe (see ffcvb_set_staging_split for sharing that work with the staging
 * threads); 16-byte words around a payload may be read, never beyond the page that holds a byte
 * of it.  Host-only; does not touch the GPU except to grow buffers. */
int ffcvb_stage_batch(ffcvb_ctx *ctx, int slot, const uint8_t *file_base, const uint64_t *ptrs,
                      const uint64_t *sizes, const uint8_t *modes, const uint16_t *heights,
                      const uint16_t *widths, int n, const ffcvb_plan *plan, const int32_t *params);

/* ffcvb_stage_batch for a file that is not mapped (datasets larger than RAM; the role of
 * ffcv/memory_managers/process_cache/page_reader.py:9-40, whose reader threads load 8 MiB pages
 * into a page ring the decoders then copy from).  Here the staging threads `pread` every sample
 * straight into its place in the slot's pinned buffer -- the only host buffer the bytes ever
 * touch -- and parse the JPEG headers there.  `fd`: the file opened for reading; `fd_direct`: the
 * same file opened with O_DIRECT, or -1.  With O_DIRECT a sample travels as the 4 KiB blocks that
 * contain it (read into a 4 KiB aligned place, so at most 8 KiB more per sample cross the link) and
 * never enters the page cache; when the file system refuses O_DIRECT, reads go through `fd` and the
 * pages they brought in are handed back right away (posix_fadvise DONTNEED).  Raw samples are read
 * as the whole rows their crop box touches.  The call returns when everything has been read:
 * ffcvb_stage_times()[0] is then read + parse time.  Everything else as ffcvb_stage_batch. */
int ffcvb_stage_batch_fd(ffcvb_ctx *ctx, int slot, int fd, int fd_direct, const uint64_t *ptrs,
                         const uint64_t *sizes, const uint8_t *modes, const uint16_t *heights,
                         const uint16_t *widths, int n, const ffcvb_plan *plan, const int32_t *params);

/* Riders: values of the samples' other fields that travel inside the image batch's staged bytes, so
 * that a whole batch (pixels, labels, small arrays) is one host->device transfer.  Replaces the
 * separate per-batch copy that IntDecoder / FloatDecoder / NDArrayDecoder followed by ToTensor and
 * ToDevice cause in the reference (ffcv/fields/basics.py:28-34, ffcv/fields/ndarray.py:37-43,
 * ffcv/transforms/ops.py:50-57).  Call before ffcvb_stage_batch of the same slot with the same
 * `n`; the next ffcvb_stage_batch consumes the riders (they are not kept for later batches).
 * A rider is `n` items of `item_bytes` each: either `host` (contiguous values, copied by this call)
 * or `ptrs` (n offsets from ffcvb_stage_batch's `file_base`, read when the batch is staged).
 * ffcvb_submit_batch then copies the n * item_bytes bytes, device to device on its stream, into
 * `dst_dev`, a DEVICE buffer of the caller. */
#define FFCVB_MAX_RIDERS 8
typedef struct {
    const void *host;     /* n * item_bytes contiguous bytes, or NULL */
    const uint64_t *ptrs; /* n file offsets, or NULL (exactly one of host / ptrs) */
    uint64_t item_bytes;
    void *dst_dev;
} ffcvb_rider;
int ffcvb_set_batch_riders(ffcvb_ctx *ctx, int slot, const ffcvb_rider *riders, int n_riders, int n);

/* Header cache (no counterpart in the reference).  When enabled the context remembers, per sample
 * (told apart by its offset in the file, so the context must then serve ONE file whose bytes do not
 * change), what the marker segments of its JPEG stream said; staging the sample again is then a
 * table look-up instead of a parse.  About 50 bytes of host memory per JPEG sample seen, at most
 * 8 M samples.  Off by default (the single-image entry points pass every stream at offset 0). */
int ffcvb_set_header_cache(ffcvb_ctx *ctx, int enabled);

/* Decode index (no counterpart in the reference).  A loader decodes the same JPEG streams epoch
 * after epoch, and what makes the decode of a stream without restart markers expensive on a GPU
 * -- finding the decoder's state at the start of every subsequence -- is the same every time.
 * With an index of `bytes` bytes of device memory (0 switches it off and frees it) the first decode
 * of a stream records those states (12 bytes per subsequence of 0.5-1.3 kbit: about 7 % of the
 * stream's size) and later decodes of the same stream start every subsequence from its recorded
 * state: one pass instead of the guess-and-repair rounds, same pixels.  Streams are told apart by
 * their offset in the file, so a context with an index must serve one file; entries of streams
 * recorded while the pool was full are simply never made.  ffcvb_decode_index_stats: out[0]
 * images decoded from their entry, out[1] entries recorded, out[2] entries in the table, out[3]
 * bytes of the pool in use. */
int ffcvb_set_decode_index(ffcvb_ctx *ctx, uint64_t bytes);
int ffcvb_decode_index_stats(ffcvb_ctx *ctx, uint64_t *out);

/* With asynchronous staging enabled, ffcvb_stage_batch returns as soon as the batch is laid out
 * and leaves the payload copy running on the staging threads.  ffcvb_submit_batch of that slot
 * does not wait for it either: it queues a stream callback that holds `stream` until the copy is
 * complete (at most 120 s; a copy that misses that limit makes every later submit fail with
 * FFCVB_E_CUDA), then the host->device copy and the kernels, so the calling thread is free to
 * stage the next batch while this one's bytes are still being copied; one copy runs at a time.
 * The caller must keep `file_base` mapped until the batch has completed on the stream, and must
 * not stage a slot again before its previous batch has completed.  Off by default. */
int ffcvb_set_async_staging(ffcvb_ctx *ctx, int enabled);

/* Split staging, for a `file_base` in page-locked memory (see ffcvb_stage_batch): the staging
 * threads copy about `cpu_share_permille` / 1000 of every batch's payload bytes into the pinned
 * staging buffer, which the copy engine moves, while the GPU gathers the rest over the link at
 * the same time.  0 (the default) leaves everything to the gather; 1000 stages everything on the
 * CPU; -1 starts at 300 and then adjusts the share from batch to batch so that the threads' copy
 * and the GPU's gather of a batch take equally long (each slot's previous batch is the
 * measurement).  At most four threads copy at a time in this mode: more of them slow the gather
 * down.  Ignored for a pageable `file_base`.  No counterpart in the reference. */
int ffcvb_set_staging_split(ffcvb_ctx *ctx, int cpu_share_permille);

/* Page-locks `bytes` at `ptr` in place (cudaHostRegister) so that ffcvb_stage_batch treats a
 * `file_base` inside that range as a pinned source.  Meant for a shared, writable mapping of a
 * dataset file on a memory file system: the page cache itself becomes the pinned copy and every
 * process of the node shares it.  Returns FFCVB_E_CUDA when the driver refuses (read-only
 * mappings and files on disk are refused) and leaves no CUDA error behind.  No counterpart in
 * the reference. */
int ffcvb_host_register(void *ptr, uint64_t bytes);
/* Releases the page lock.  Waits for the device first (cudaDeviceSynchronize): batches submitted
 * earlier may still be gathering payloads from the range. */
int ffcvb_host_unregister(void *ptr);

/* The share (per mille) the next batch will be staged with. */
int ffcvb_staging_split(const ffcvb_ctx *ctx);

/* Queue the staged batch on `stream`: one host->device copy of the staged bytes, then the decode
 * (entropy decode, dequantise + IDCT, chroma upsample + colour conversion) and the fused
 * crop/resize/augment/normalise kernels, writing `n` images into `out_dev` (DEVICE pointer,
 * layout plan.out_kind).  Replaces the prange loop of rgb_image.py:185-210 and the transform
 * closures after it.  Returns after queueing. */
int ffcvb_submit_batch(ffcvb_ctx *ctx, int slot, void *stream, void *out_dev);

/* Re-runs the kernels of a batch whose staged bytes an earlier ffcvb_submit_batch on this slot
 * already copied to the GPU: same work, no host->device copy.  For measuring the rate with inputs
 * resident in HBM; no counterpart in the reference. */
int ffcvb_rerun_batch(ffcvb_ctx *ctx, int slot, void *stream, void *out_dev);

/* With profiling enabled every batch run also records CUDA events between its stages on the
 * batch's stream; ffcvb_batch_times waits for the slot's last run and returns the elapsed
 * milliseconds of ms[0] host->device copy, ms[1] entropy decode (with its memsets), ms[2]
 * dequantise + IDCT, ms[3] upsample + colour conversion, ms[4] fused resize/augment/normalise.
 * No counterpart in the reference. */
int ffcvb_set_profiling(ffcvb_ctx *ctx, int enabled);
int ffcvb_batch_times(ffcvb_ctx *ctx, int slot, float *ms);

/* Bytes the last staged batch of `slot` moves host->device, and how many of this library's
 * kernels ffcvb_submit_batch launches for it. */
int64_t ffcvb_staged_bytes(const ffcvb_ctx *ctx, int slot);
/* Host milliseconds the last ffcvb_stage_batch on `slot` spent in: ms[0] JPEG header parsing,
 * ms[1] table deduplication and layout, ms[2] payload copy into pinned memory, ms[3] total. */
int ffcvb_stage_times(const ffcvb_ctx *ctx, int slot, double *ms);
/* Sizes of the slot's staged batch, for bandwidth accounting: info[0] samples, [1] JPEG samples,
 * [2] 8x8 blocks, [3] entropy-coded bytes, [4] component-plane bytes, [5] decoded RGB bytes,
 * [6] staged raw-pixel bytes, [7] staged JPEG bytes. */
int ffcvb_batch_info(const ffcvb_ctx *ctx, int slot, int64_t *info);
int ffcvb_batch_launches(const ffcvb_ctx *ctx, int slot);
/* Milliseconds the GPU's payload gather of the slot's last submitted batch took (waits for it);
 * -1 when that batch was not gathered by the GPU.  No counterpart in the reference. */
int ffcvb_gather_time(ffcvb_ctx *ctx, int slot, float *ms);

/* After the stream has completed the slot's batch: copies the per-sample status words
 * (0 = ok, otherwise FFCVB_E_DECODE) into status[0..n).  Returns the number of failed samples.
 * The reference drops imdecode's return code (rgb_image.py:131,196); this keeps it. */
int ffcvb_batch_status(ffcvb_ctx *ctx, int slot, void *stream, int32_t *status, int n);

/* Augment + normalise a batch that already sits on the device as uint8 [n, h, w, 3]
 * (`src_dev`), e.g. the output of an earlier call; params as above (host pointer, crop box
 * honoured when plan.resize == 1).  Used when a pipeline cannot be fused into one call. */
int ffcvb_transform_device(ffcvb_ctx *ctx, void *stream, const uint8_t *src_dev, int n, int h,
                           int w, const ffcvb_plan *plan, const int32_t *params, void *out_dev);

/* ---- colour and blending transforms on uint8 device batches -------------------------------
 * Replacements of the numba closures of ffcv/transforms/color_jitter.py, mixup.py and
 * poisoning.py.  `images_dev` / `src_dev` / `dst_dev` are DEVICE pointers to [n, h, w, 3] (or
 * [n, count]) uint8 batches; the small per-image arrays are HOST pointers and are copied by the
 * call.  All calls queue their work on `stream` and return. */
#define FFCVB_JITTER_BRIGHTNESS 0
#define FFCVB_JITTER_CONTRAST 1
#define FFCVB_JITTER_SATURATION 2

/* RandomBrightness / RandomContrast / RandomSaturation (color_jitter.py:41-50, :83-94,
 * :121-136), in place: image i is changed when apply[i] != 0, with blend factor ratio[i].  The
 * float64 arithmetic, including which multiply-adds are fused, is that of the reference's
 * compiled code. */
int ffcvb_color_jitter(ffcvb_ctx *ctx, void *stream, uint8_t *images_dev, int n, int h, int w, int kind,
                       const uint8_t *apply, const double *ratio);

/* ImageMixup (mixup.py:41-50): dst[i] = lam[i] * src[i] + (1 - lam[i]) * src[i - 1] over `count`
 * values per image, image -1 being image n - 1; 0 <= lam[i] <= 1; dst must not be src. */
int ffcvb_mixup(ffcvb_ctx *ctx, void *stream, const uint8_t *src_dev, uint8_t *dst_dev, int n, int64_t count,
                const double *lam);

/* Poison (poisoning.py:45-60), in place on the images with apply[i] != 0:
 * clamp(image * one_minus_alpha + mask) evaluated through a float32 scratch value as the
 * reference does.  one_minus_alpha_dev and mask_dev are DEVICE arrays of `count` doubles (the
 * opacity repeated over the channels; the mask already multiplied by the opacity). */
int ffcvb_poison(ffcvb_ctx *ctx, void *stream, uint8_t *images_dev, int n, int64_t count, const uint8_t *apply,
                 const double *one_minus_alpha_dev, const double *mask_dev, double clamp_lo, double clamp_hi);

/* ---- decode without allocating -----------------------------------------------------------
 * No counterpart in the reference.  For callers that must not allocate GPU memory while they
 * run: a process that handed all device memory to its own pool at start-up, a plugin living
 * inside another framework's allocator, a latency-critical loop that cannot afford the
 * device-wide synchronisation a cudaMalloc / cudaFree may cause.  Decodes ONE baseline JPEG
 * (same streams and same pixels as `imdecode`) into packed RGB, height * width * 3 bytes.
 *   jpeg_host : the stream in host memory (only its headers are read, on the host)
 *   jpeg_dev  : the same `jpeg_size` bytes already in DEVICE memory (the caller copied them)
 *   rgb_dev   : DEVICE output buffer of the caller
 * The work is queued on `stream` and the call returns; a corrupt entropy segment is not reported.
 * All scratch (unstuffed bit stream, coefficients, component planes, tables) lives in a fixed
 * array inside the library image, about 4.7 MB that every GPU loading the library holds until
 * exit, which bounds one call to FFCVB_STATIC_MAX_STREAM_BYTES of JPEG data and
 * FFCVB_STATIC_MAX_PADDED_PIXELS luma samples after padding both sides up to whole MCUs (multiples
 * of 8 or 16); larger inputs are refused with FFCVB_E_LIMIT and a message on stderr.  The call
 * itself makes no cudaMalloc, cudaFree or other allocating call.  The first call on a device
 * looks up the array's device address (cudaGetSymbolAddress); make that first call outside any
 * stream capture.  All calls share the one array, which keeps what the previous call left
 * (the parts that must start at zero are cleared on the stream each time): two calls whose GPU
 * work can overlap -- different streams, or different threads without ordering -- race on it. */
#define FFCVB_STATIC_MAX_STREAM_BYTES (1u << 20)
#define FFCVB_STATIC_MAX_PADDED_PIXELS (640u * 640u)
int ffcvb_imdecode_static(const uint8_t *jpeg_host, uint64_t jpeg_size, const uint8_t *jpeg_dev,
                          uint32_t height, uint32_t width, uint8_t *rgb_dev, void *stream);

/* ---- single-image entry points with the reference's exact signatures --------------------
 * Drop-in for the symbols ffcv/libffcv.py:22-55 binds with ctypes.  HOST pointers in and out;
 * each call copies to the GPU, runs the kernels and copies back, synchronously, on a process-wide
 * context for the current device.  They exist for parity with the reference ABI; the batch calls
 * above are the fast path. */

/* libffcv/libffcv.cpp:33-42. */
void resize(int64_t cresizer, int64_t source_p, int64_t sx, int64_t sy, int64_t start_row,
            int64_t end_row, int64_t start_col, int64_t end_col, int64_t dest_p, int64_t tx,
            int64_t ty);
/* libffcv/libffcv.cpp:53-112.  Returns 0, or -1 as tjDecompress2 does. */
int imdecode(unsigned char *input_buffer, uint64_t input_size, uint32_t source_height,
             uint32_t source_width, unsigned char *output_buffer, uint32_t crop_height,
             uint32_t crop_width, uint32_t offset_x, uint32_t offset_y, uint32_t scale_num,
             uint32_t scale_denom, bool enable_crop, bool hflip);
/* libffcv/libffcv.cpp:44-46. */
void my_memcpy(void *source, void *dst, uint64_t size);
/* libffcv/libffcv.cpp:48-51: seek to `offset` in the C stream `fp` (a FILE * passed as an
 * integer) and read `size` bytes into `destination`.  The reference's Python never binds it. */
void my_fread(int64_t fp, int64_t offset, void *destination, int64_t size);

#ifdef __cplusplus
}
#endif
#endif
