/*
 * CPU oracle for the crop + resize step of FFCV's image path.  TEST INFRASTRUCTURE ONLY: the
 * checker the CUDA path is compared with (and the timed CPU baseline); the product never calls it.
 *
 * What it restates: libffcv/libffcv.cpp:33-42,
 *     cv::resize(src.colRange(c0, c1).rowRange(r0, r1), dst, dst.size(), 0, 0, cv::INTER_AREA)
 * on packed 8-bit 3-channel images.  OpenCV (pip pin opencv-python 4.5.4.58 in the reference's
 * ffcv-conda.yml) is not vendored in the reference tree; this file is written from OpenCV's
 * documented behaviour of INTER_AREA and from observation of the cv2 binary in this image, which
 * pins it in tests/test_oracle_resize.py.  INTER_AREA is three algorithms:
 *   same size           : copy;
 *   both scales integer : box sum, (s+2)>>2 for 2x2, else round-half-even(float(s) * float(1/area));
 *   both scales >= 1    : separable fractional box coverage, accumulated in float32 in source
 *                         order (x then y), rounded half-even and saturated;
 *   any scale < 1       : two-tap interpolation on BOTH axes with area-derived positions,
 *                         11-bit fixed-point weights, horizontal pass in int32 and the vertical
 *                         pass ((b0*(S0>>4))>>16 + (b1*(S1>>4))>>16 + 2) >> 2.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline uint8_t sat_round_u8(float v) {
    long r = lrintf(v); /* round half to even in the default rounding mode */
    return (uint8_t)(r < 0 ? 0 : (r > 255 ? 255 : r));
}

typedef struct {
    int src, dst;
    float w;
} AreaTap;

/* Coverage of each destination cell [d*scale, (d+1)*scale) by source cells. */
static int area_taps(int ssize, int dsize, double scale, AreaTap *tab) {
    int k = 0;
    for (int d = 0; d < dsize; d++) {
        double f1 = d * scale, f2 = f1 + scale;
        double cell = scale < ssize - f1 ? scale : ssize - f1;
        int s1 = (int)ceil(f1), s2 = (int)floor(f2);
        if (s2 > ssize - 1) s2 = ssize - 1;
        if (s1 > s2) s1 = s2;
        if (s1 - f1 > 1e-3) {
            tab[k].dst = d;
            tab[k].src = s1 - 1;
            tab[k++].w = (float)((s1 - f1) / cell);
        }
        for (int s = s1; s < s2; s++) {
            tab[k].dst = d;
            tab[k].src = s;
            tab[k++].w = (float)(1.0 / cell);
        }
        if (f2 - s2 > 1e-3) {
            double a = f2 - s2;
            if (a > 1.0) a = 1.0;
            if (a > cell) a = cell;
            tab[k].dst = d;
            tab[k].src = s2;
            tab[k++].w = (float)(a / cell);
        }
    }
    return k;
}

static void resize_area_general(const uint8_t *src, int sstride, int sh, int sw, uint8_t *dst,
                                int dh, int dw) {
    double scx = 1.0 / ((double)dw / sw), scy = 1.0 / ((double)dh / sh);
    AreaTap *xt = (AreaTap *)malloc(sizeof(AreaTap) * (size_t)(sw + 2 * dw + 2));
    AreaTap *yt = (AreaTap *)malloc(sizeof(AreaTap) * (size_t)(sh + 2 * dh + 2));
    int nx = area_taps(sw, dw, scx, xt), ny = area_taps(sh, dh, scy, yt);
    float *row = (float *)malloc(sizeof(float) * 3 * (size_t)dw);
    float *sum = (float *)malloc(sizeof(float) * 3 * (size_t)dw);
    int prev = -1;
    for (int k = 0; k < ny; k++) {
        const uint8_t *S = src + (size_t)yt[k].src * sstride;
        float beta = yt[k].w;
        for (int i = 0; i < 3 * dw; i++) row[i] = 0.f;
        for (int t = 0; t < nx; t++) {
            float a = xt[t].w;
            const uint8_t *p = S + 3 * xt[t].src;
            float *r = row + 3 * xt[t].dst;
            r[0] += p[0] * a;
            r[1] += p[1] * a;
            r[2] += p[2] * a;
        }
        if (yt[k].dst != prev) {
            if (prev >= 0)
                for (int i = 0; i < 3 * dw; i++) dst[(size_t)prev * dw * 3 + i] = sat_round_u8(sum[i]);
            for (int i = 0; i < 3 * dw; i++) sum[i] = beta * row[i];
            prev = yt[k].dst;
        } else {
            for (int i = 0; i < 3 * dw; i++) sum[i] += beta * row[i];
        }
    }
    if (prev >= 0)
        for (int i = 0; i < 3 * dw; i++) dst[(size_t)prev * dw * 3 + i] = sat_round_u8(sum[i]);
    free(xt);
    free(yt);
    free(row);
    free(sum);
}

static void resize_area_integer(const uint8_t *src, int sstride, int fy, int fx, uint8_t *dst,
                                int dh, int dw) {
    float inv = 1.f / (float)(fx * fy);
    for (int y = 0; y < dh; y++)
        for (int x = 0; x < dw; x++)
            for (int c = 0; c < 3; c++) {
                int s = 0;
                for (int j = 0; j < fy; j++)
                    for (int i = 0; i < fx; i++)
                        s += src[(size_t)(y * fy + j) * sstride + (x * fx + i) * 3 + c];
                dst[((size_t)y * dw + x) * 3 + c] =
                    (fx == 2 && fy == 2) ? (uint8_t)((s + 2) >> 2) : sat_round_u8((float)s * inv);
            }
}

/* Position and weight of the two taps for one axis when some axis upscales. */
static void linear_area_taps(int ssize, int dsize, int *ofs, int16_t *w, int clamp_last) {
    double inv = (double)dsize / ssize, scale = 1.0 / inv;
    for (int d = 0; d < dsize; d++) {
        int s = (int)floor(d * scale);
        float f = (float)((d + 1) - (s + 1) * inv);
        f = f <= 0 ? 0.f : f - floorf(f);
        if (clamp_last && s >= ssize - 1) {
            f = 0.f;
            s = ssize - 1;
        }
        ofs[d] = s;
        long w0 = lrintf((1.f - f) * 2048.f), w1 = lrintf(f * 2048.f);
        w[2 * d] = (int16_t)(w0 > 32767 ? 32767 : w0);
        w[2 * d + 1] = (int16_t)(w1 > 32767 ? 32767 : w1);
    }
}

static void resize_linear_area(const uint8_t *src, int sstride, int sh, int sw, uint8_t *dst,
                               int dh, int dw) {
    int *xo = (int *)malloc(sizeof(int) * (size_t)dw), *yo = (int *)malloc(sizeof(int) * (size_t)dh);
    int16_t *xw = (int16_t *)malloc(sizeof(int16_t) * 2 * (size_t)dw);
    int16_t *yw = (int16_t *)malloc(sizeof(int16_t) * 2 * (size_t)dh);
    linear_area_taps(sw, dw, xo, xw, 1);
    linear_area_taps(sh, dh, yo, yw, 0);
    for (int y = 0; y < dh; y++) {
        int r0 = yo[y], r1 = yo[y] + 1;
        if (r0 > sh - 1) r0 = sh - 1;
        if (r1 > sh - 1) r1 = sh - 1;
        const uint8_t *S0 = src + (size_t)r0 * sstride, *S1 = src + (size_t)r1 * sstride;
        int b0 = yw[2 * y], b1 = yw[2 * y + 1];
        for (int x = 0; x < dw; x++) {
            int s = xo[x], s1 = s + 1 < sw ? s + 1 : s;
            int a0 = xw[2 * x], a1 = xw[2 * x + 1];
            if (s + 1 >= sw) {
                a0 = 2048;
                a1 = 0;
            }
            for (int c = 0; c < 3; c++) {
                int h0 = S0[3 * s + c] * a0 + S0[3 * s1 + c] * a1;
                int h1 = S1[3 * s + c] * a0 + S1[3 * s1 + c] * a1;
                int v = (((b0 * (h0 >> 4)) >> 16) + ((b1 * (h1 >> 4)) >> 16) + 2) >> 2;
                dst[((size_t)y * dw + x) * 3 + c] = (uint8_t)(v < 0 ? 0 : (v > 255 ? 255 : v));
            }
        }
    }
    free(xo);
    free(yo);
    free(xw);
    free(yw);
}

/* INTER_AREA resize of the region rows [r0, r1), columns [c0, c1) of a packed RGB image with
 * `src_cols` columns into a packed dst_rows x dst_cols x 3 image. */
void oracle_resize_area(const uint8_t *src, int src_cols, int r0, int r1, int c0, int c1,
                        uint8_t *dst, int dst_rows, int dst_cols) {
    int sh = r1 - r0, sw = c1 - c0, sstride = src_cols * 3;
    const uint8_t *roi = src + (size_t)r0 * sstride + (size_t)c0 * 3;
    if (sh <= 0 || sw <= 0 || dst_rows <= 0 || dst_cols <= 0) return;
    if (sh == dst_rows && sw == dst_cols) {
        for (int y = 0; y < sh; y++) memcpy(dst + (size_t)y * sw * 3, roi + (size_t)y * sstride, (size_t)sw * 3);
        return;
    }
    /* OpenCV derives the factors as 1 / (dst / src) in double and calls them integer when they
     * are within DBL_EPSILON of one */
    double scx = 1.0 / ((double)dst_cols / sw), scy = 1.0 / ((double)dst_rows / sh);
    if (scx >= 1 && scy >= 1) {
        long ix = lrint(scx), iy = lrint(scy);
        if (fabs(scx - ix) < DBL_EPSILON && fabs(scy - iy) < DBL_EPSILON)
            resize_area_integer(roi, sstride, (int)iy, (int)ix, dst, dst_rows, dst_cols);
        else
            resize_area_general(roi, sstride, sh, sw, dst, dst_rows, dst_cols);
        return;
    }
    resize_linear_area(roi, sstride, sh, sw, dst, dst_rows, dst_cols);
}

/* Same signature as libffcv/libffcv.cpp:33-35 `resize`: pointers travel as 64-bit integers. */
void resize(int64_t cresizer, int64_t source_p, int64_t sx, int64_t sy, int64_t start_row,
            int64_t end_row, int64_t start_col, int64_t end_col, int64_t dest_p, int64_t tx,
            int64_t ty) {
    (void)cresizer;
    (void)sx;
    oracle_resize_area((const uint8_t *)(intptr_t)source_p, (int)sy, (int)start_row, (int)end_row,
                       (int)start_col, (int)end_col, (uint8_t *)(intptr_t)dest_p, (int)tx, (int)ty);
}
