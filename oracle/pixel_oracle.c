/* CPU restatement of the reference's per-pixel colour and blending transforms.
 *
 * TEST INFRASTRUCTURE ONLY: the product library never links or calls this file.
 *
 * Follows ffcv/transforms/color_jitter.py (RandomBrightness :41-50, RandomContrast :83-94,
 * RandomSaturation :121-136), ffcv/transforms/mixup.py (ImageMixup :41-50) and
 * ffcv/transforms/poisoning.py (Poison :45-60).  The reference compiles these closures with numba
 * under fastmath (ffcv/pipeline/compiler.py:30), which lets LLVM contract a multiply and the add
 * that consumes it into one fused multiply-add; the contractions it makes on x86-64 were
 * identified by running the reference's own closures (exhaustively over all (r, g, b) for the
 * grey value) and are written here as explicit fma() calls.  This file is compiled with
 * -ffp-contract=off so nothing else is fused.
 *
 *   grey(r, g, b)          = fma(0.114, b, fma(0.587, g, 0.2989 * r))          then cast to uint8
 *   blend(a, s scalar, t)  = fma(t, a, (1 - t) * s)                             (contrast, brightness)
 *   blend(a, grey image, t)= t * a + (1 - t) * grey, no fusion                  (saturation)
 *   mixup                  = fma(1 - t, b, t * a)
 *   result                 = (uint8) min(max(value, 0), 255)                    (truncation)
 *
 * With these the brightness, contrast, saturation and poison outputs of the reference's closures
 * (compiled single-threaded, the only mode whose random draws can be reproduced) are matched bit
 * for bit.  Mixup is matched except for isolated pixels that differ by one: the reference's
 * compiled loop treats the first image (whose partner is found by wrapping around) with
 * unfused arithmetic and the others fused, and its multi-threaded compilation differs from its
 * single-threaded one in the same way, so the last bit of a mixup is not defined by the
 * reference itself.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

static inline uint8_t clip_u8(double v) {
    if (v < 0.0) v = 0.0;
    if (v > 255.0) v = 255.0;
    return (uint8_t)v;
}

static inline uint8_t grey_u8(uint8_t r, uint8_t g, uint8_t b) {
    return (uint8_t)fma(0.114, (double)b, fma(0.587, (double)g, 0.2989 * (double)r));
}

/* images: [n, h, w, 3] uint8, in place.  apply[i] != 0 selects image i, ratio[i] is its factor. */
void oracle_brightness(uint8_t *images, int n, int h, int w, const uint8_t *apply, const double *ratio) {
    const size_t count = (size_t)h * w * 3;
    for (int i = 0; i < n; i++) {
        if (!apply[i]) continue;
        uint8_t *p = images + (size_t)i * count;
        const double t = ratio[i], c = (1.0 - t) * 0.0;
        for (size_t k = 0; k < count; k++) p[k] = clip_u8(fma(t, (double)p[k], c));
    }
}

void oracle_contrast(uint8_t *images, int n, int h, int w, const uint8_t *apply, const double *ratio) {
    const size_t pixels = (size_t)h * w;
    for (int i = 0; i < n; i++) {
        if (!apply[i]) continue;
        uint8_t *p = images + (size_t)i * pixels * 3;
        double sum = 0.0; /* integers below 2^53: exact in any order */
        for (size_t k = 0; k < pixels; k++) sum += (double)grey_u8(p[3 * k], p[3 * k + 1], p[3 * k + 2]);
        const double mean = sum / (double)pixels;
        const double t = ratio[i], c = (1.0 - t) * mean;
        for (size_t k = 0; k < pixels * 3; k++) p[k] = clip_u8(fma(t, (double)p[k], c));
    }
}

void oracle_saturation(uint8_t *images, int n, int h, int w, const uint8_t *apply, const double *ratio) {
    const size_t pixels = (size_t)h * w;
    for (int i = 0; i < n; i++) {
        if (!apply[i]) continue;
        uint8_t *p = images + (size_t)i * pixels * 3;
        const double t = ratio[i], u = 1.0 - t;
        for (size_t k = 0; k < pixels; k++) {
            const double l = (double)grey_u8(p[3 * k], p[3 * k + 1], p[3 * k + 2]);
            for (int c = 0; c < 3; c++) p[3 * k + c] = clip_u8(t * (double)p[3 * k + c] + u * l);
        }
    }
}

/* dst[i] = lam[i] * src[i] + (1 - lam[i]) * src[i - 1], image -1 being the last one
 * (mixup.py:47-48); `count` values per image; the assignment into the uint8 array truncates. */
void oracle_mixup(const uint8_t *src, uint8_t *dst, int n, size_t count, const double *lam) {
    for (int i = 0; i < n; i++) {
        const uint8_t *a = src + (size_t)i * count;
        const uint8_t *b = src + (size_t)(i == 0 ? n - 1 : i - 1) * count;
        uint8_t *o = dst + (size_t)i * count;
        const double l = lam[i], u = 1.0 - l;
        for (size_t k = 0; k < count; k++) o[k] = (uint8_t)fma(u, (double)b[k], l * (double)a[k]);
    }
}

/* Poison (poisoning.py:45-60): in a float32 scratch image, temp = image; temp *= 1 - alpha;
 * temp += mask (both double arrays, each statement rounding its double result back to float32);
 * clip; store as uint8.  one_minus_alpha and mask hold `count` doubles (already repeated over the
 * channels, the mask already multiplied by alpha as generate_code does). */
void oracle_poison(uint8_t *images, int n, size_t count, const uint8_t *apply, const double *one_minus_alpha,
                   const double *mask, double lo, double hi) {
    for (int i = 0; i < n; i++) {
        if (!apply[i]) continue;
        uint8_t *p = images + (size_t)i * count;
        for (size_t k = 0; k < count; k++) {
            float t = (float)p[k];
            t = (float)((double)t * one_minus_alpha[k]);
            t = (float)((double)t + mask[k]);
            if (t < (float)lo) t = (float)lo;
            if (t > (float)hi) t = (float)hi;
            p[k] = (uint8_t)t;
        }
    }
}
