/*
 * CPU oracle for one batch of FFCV's decode-and-augment path.  TEST INFRASTRUCTURE ONLY: the
 * checker for the CUDA path and the timed CPU baseline; the product never calls it.
 *
 * Per sample it chains, in the reference's order and with the reference's arithmetic:
 *   decode        ffcv/fields/rgb_image.py:185-210 (jpg -> imdecode, raw -> view)
 *   crop + resize ffcv/fields/rgb_image.py:205-208 -> libffcv/libffcv.cpp:33-42
 *   flip          ffcv/transforms/flip.py:31-39        dst = img[:, ::-1]
 *   translate     ffcv/transforms/translate.py:35-44   pad with fill, take window (y, x)
 *   cutout        ffcv/transforms/cutout.py:36-46      square at (y, x) <- fill
 *   normalise     ffcv/transforms/normalize.py:89-109  out = table[value, channel]
 * The random draws (crop box, flip bit, offsets) are inputs: the caller samples them.
 * Samples are spread over `nthreads` POSIX threads the way the reference spreads them over numba
 * prange workers.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int oracle_jpeg_scalable(const uint8_t *data, size_t n);
int oracle_jpeg_decode_scaled(const uint8_t *data, size_t n, uint8_t *out, int out_h, int out_w, int denom);
int oracle_jpeg_decode(const uint8_t *data, size_t n, uint8_t *out, int height, int width,
                       int idct, int upsample);
void oracle_resize_area(const uint8_t *src, int src_cols, int r0, int r1, int c0, int c1,
                        uint8_t *dst, int dst_rows, int dst_cols);

enum { OP_FLIP = 1, OP_TRANSLATE = 2, OP_CUTOUT = 3 };
enum { OUT_U8_NHWC = 0, OUT_F16_NHWC = 1, OUT_F16_NCHW = 2, OUT_F32_NHWC = 3, OUT_F32_NCHW = 4 };

/* ops: nops records of 8 int32: type, p0, p1, p2, fill r, g, b, unused
 *   flip: p0 = 1 to flip; translate: p0 = padding, p1 = y, p2 = x; cutout: p0 = size, p1 = y, p2 = x */
void oracle_augment(uint8_t *img, int h, int w, const int32_t *ops, int nops, uint8_t *scratch) {
    for (int k = 0; k < nops; k++) {
        const int32_t *op = ops + 8 * k;
        if (op[0] == OP_FLIP) {
            if (!op[1]) continue;
            for (int y = 0; y < h; y++)
                for (int x = 0; x < w / 2; x++)
                    for (int c = 0; c < 3; c++) {
                        uint8_t *a = img + ((size_t)y * w + x) * 3 + c;
                        uint8_t *b = img + ((size_t)y * w + (w - 1 - x)) * 3 + c;
                        uint8_t t = *a;
                        *a = *b;
                        *b = t;
                    }
        } else if (op[0] == OP_TRANSLATE) {
            int p = op[1], ty = op[2], tx = op[3], ph = h + 2 * p, pw = w + 2 * p;
            for (int y = 0; y < ph; y++)
                for (int x = 0; x < pw; x++)
                    for (int c = 0; c < 3; c++) {
                        int inside = y >= p && y < p + h && x >= p && x < p + w;
                        scratch[((size_t)y * pw + x) * 3 + c] =
                            inside ? img[((size_t)(y - p) * w + (x - p)) * 3 + c] : (uint8_t)op[4 + c];
                    }
            for (int y = 0; y < h; y++)
                memcpy(img + (size_t)y * w * 3, scratch + ((size_t)(y + ty) * pw + tx) * 3, (size_t)w * 3);
        } else if (op[0] == OP_CUTOUT) {
            int s = op[1], cy = op[2], cx = op[3];
            for (int y = cy; y < cy + s && y < h; y++)
                for (int x = cx; x < cx + s && x < w; x++)
                    for (int c = 0; c < 3; c++) img[((size_t)y * w + x) * 3 + c] = (uint8_t)op[4 + c];
        }
    }
}

/* lut: 256 x 3 entries of the output type (16-bit patterns for fp16, as the reference carries
 * them as int16). */
void oracle_normalize(const uint8_t *img, int h, int w, const void *lut, int out_kind, void *out) {
    size_t n = (size_t)h * w;
    if (out_kind == OUT_U8_NHWC) {
        memcpy(out, img, n * 3);
        return;
    }
    int f32 = out_kind == OUT_F32_NHWC || out_kind == OUT_F32_NCHW;
    int planar = out_kind == OUT_F16_NCHW || out_kind == OUT_F32_NCHW;
    for (size_t p = 0; p < n; p++)
        for (int c = 0; c < 3; c++) {
            size_t o = planar ? (size_t)c * n + p : p * 3 + c;
            int v = img[p * 3 + c];
            if (f32)
                ((uint32_t *)out)[o] = ((const uint32_t *)lut)[v * 3 + c];
            else
                ((uint16_t *)out)[o] = ((const uint16_t *)lut)[v * 3 + c];
        }
}

typedef struct {
    int n;
    const uint8_t *const *payloads;
    const uint64_t *sizes;
    const int32_t *desc; /* [n][8]: mode (0 jpg, 1 raw), h, w, crop i, crop j, crop h, crop w,
                            flags: bit 0 resize?; bits 8-15 scale of the JPEG decode: 0 full, 1..3 =
                            1/2, 1/4, 1/8, 255 = per sample, the smallest scale at which the crop
                            box keeps at least oh x ow pixels */
    int oh, ow;
    const int32_t *ops; /* [n][nops][8] */
    int nops;
    const void *lut;
    int out_kind;
    uint8_t *out;
    size_t out_stride;
    int *status;
    int next;
    pthread_mutex_t lock;
} Job;

static void run_sample(Job *j, int i) {
    const int32_t *d = j->desc + 8 * i;
    int mode = d[0], h = d[1], w = d[2];
    uint8_t *decoded = NULL;
    const uint8_t *pix;
    j->status[i] = 0;
    int oh = j->oh, ow = j->ow;
    int ci = d[3], cj = d[4], chh = d[5], cww = d[6];
    const int resize = d[7] & 1, scale_mode = (d[7] >> 8) & 255;
    if (mode == 0) {
        int shift = 0;
        if (scale_mode >= 1 && scale_mode <= 3) {
            shift = scale_mode;
        } else if (scale_mode == 255 && resize && oracle_jpeg_scalable(j->payloads[i], (size_t)j->sizes[i])) {
            while (shift < 3 && (chh >> (shift + 1)) >= oh && (cww >> (shift + 1)) >= ow) shift++;
        }
        int rc;
        if (shift == 0) {
            decoded = (uint8_t *)malloc((size_t)h * w * 3);
            rc = oracle_jpeg_decode(j->payloads[i], (size_t)j->sizes[i], decoded, h, w, 0, 0);
        } else {
            /* decode at 1 / 2^shift; the crop box becomes the box of the scaled image that covers it */
            const int sh = (h + (1 << shift) - 1) >> shift, sw = (w + (1 << shift) - 1) >> shift;
            decoded = (uint8_t *)malloc((size_t)sh * sw * 3);
            rc = oracle_jpeg_decode_scaled(j->payloads[i], (size_t)j->sizes[i], decoded, sh, sw, 1 << shift);
            int r1 = (ci + chh + (1 << shift) - 1) >> shift, c1 = (cj + cww + (1 << shift) - 1) >> shift;
            if (r1 > sh) r1 = sh;
            if (c1 > sw) c1 = sw;
            ci >>= shift;
            cj >>= shift;
            chh = r1 - ci;
            cww = c1 - cj;
            h = sh;
            w = sw;
        }
        if (rc) {
            j->status[i] = rc;
            free(decoded);
            return;
        }
        pix = decoded;
    } else {
        pix = j->payloads[i];
    }
    uint8_t *img = (uint8_t *)malloc((size_t)oh * ow * 3);
    if (resize)
        oracle_resize_area(pix, w, ci, ci + chh, cj, cj + cww, img, oh, ow);
    else
        memcpy(img, pix, (size_t)oh * ow * 3);
    int pad = 0;
    for (int k = 0; k < j->nops; k++) {
        const int32_t *op = j->ops + ((size_t)i * j->nops + k) * 8;
        if (op[0] == OP_TRANSLATE && op[1] > pad) pad = op[1];
    }
    uint8_t *scratch = pad ? (uint8_t *)malloc((size_t)(oh + 2 * pad) * (ow + 2 * pad) * 3) : NULL;
    oracle_augment(img, oh, ow, j->ops + (size_t)i * j->nops * 8, j->nops, scratch);
    oracle_normalize(img, oh, ow, j->lut, j->out_kind, j->out + (size_t)i * j->out_stride);
    free(scratch);
    free(img);
    free(decoded);
}

static void *worker(void *arg) {
    Job *j = (Job *)arg;
    for (;;) {
        pthread_mutex_lock(&j->lock);
        int i = j->next++;
        pthread_mutex_unlock(&j->lock);
        if (i >= j->n) break;
        run_sample(j, i);
    }
    return NULL;
}

int oracle_run_batch(int n, const uint8_t *const *payloads, const uint64_t *sizes,
                     const int32_t *desc, int oh, int ow, const int32_t *ops, int nops,
                     const void *lut, int out_kind, void *out, int nthreads, int *status) {
    size_t esz = out_kind == OUT_U8_NHWC ? 1 : (out_kind <= OUT_F16_NCHW ? 2 : 4);
    Job j = {n, payloads, sizes, desc, oh, ow, ops, nops, lut, out_kind, (uint8_t *)out,
             (size_t)oh * ow * 3 * esz, status, 0, PTHREAD_MUTEX_INITIALIZER};
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 512) nthreads = 512;
    pthread_t th[512];
    for (int t = 1; t < nthreads; t++) pthread_create(&th[t], NULL, worker, &j);
    worker(&j);
    for (int t = 1; t < nthreads; t++) pthread_join(th[t], NULL);
    int bad = 0;
    for (int i = 0; i < n; i++) bad |= status[i] != 0;
    return bad ? -1 : 0;
}
