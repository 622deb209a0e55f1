/*
 * CPU oracle for the JPEG decode step of FFCV's image path.  TEST INFRASTRUCTURE ONLY: this file
 * is the checker the CUDA path is compared with (and the timed CPU baseline); nothing in the
 * product path may call it.
 *
 * What it restates: the decode that libffcv/libffcv.cpp:104-106 asks of TurboJPEG,
 *     tjDecompress2(handle, buf, size, out, w, 0, h, TJPF_RGB, TJFLAG_FASTDCT | TJFLAG_NOREALLOC)
 * i.e. baseline sequential Huffman JPEG -> dequantise -> fast integer IDCT (the AAN factorisation
 * with 8-bit constants and truncating shifts, selected by TJFLAG_FASTDCT) -> "fancy" triangle
 * chroma upsampling (TJFLAG_FASTUPSAMPLE is NOT passed) -> fixed-point YCbCr->RGB, written as
 * tightly packed h*w*3 bytes.  The arithmetic lives in libjpeg-turbo (conda pin 2.1.0 in the
 * reference's ffcv-conda.yml), which is not vendored in the reference tree; this file is written
 * from the JPEG standard (ITU-T T.81), the published AAN and Loeffler-Ligtenberg-Moschytz IDCT
 * factorisations, and from behaviour observed through the libjpeg-turbo binaries bundled with
 * Pillow and OpenCV.  Pinned (tests/test_oracle_golden.py, tests/test_oracle_live.py) bit for bit
 * on (a) Pillow's libjpeg-turbo driven through the libjpeg API with the fast integer IDCT and fancy
 * upsampling -- the reference's configuration itself; (b) Pillow's "draft" decoder configuration
 * (fast IDCT + replicated chroma); (c) cv2.imdecode (accurate IDCT + fancy upsampling).  The
 * accurate IDCT and the replicated upsampler exist here only for (b) and (c).
 *
 * Supported streams: 8-bit baseline/extended-sequential Huffman (SOF0/SOF1), one interleaved scan,
 * 1 or 3 components, luma sampling 1x1, 2x1 or 2x2 with 1x1 chroma, optional restart intervals.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_OK 0
#define ORACLE_ERR_FORMAT -1
#define ORACLE_ERR_UNSUPPORTED -2
#define ORACLE_ERR_DIMS -3
#define ORACLE_ERR_DATA -4

#define IDCT_FAST 0
#define IDCT_ACCURATE 1
#define UPSAMPLE_FANCY 0
#define UPSAMPLE_REPLICATE 1

static const uint8_t ZIGZAG[64] = {
    0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
    41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
    30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

typedef struct {
    /* canonical Huffman code, T.81 Annex C / F.2.2.3 */
    uint8_t bits[17];
    uint8_t vals[256];
    int32_t maxcode[18]; /* largest code of each length, -1 if none */
    int32_t valptr[17];
    int32_t mincode[17];
    /* 9-bit look-ahead: (length << 8) | symbol, 0 if the code is longer */
    uint16_t look[512];
    int present;
} HuffTable;

typedef struct {
    int id, hs, vs, tq, td, ta;
    int blocks_w, blocks_h; /* padded to whole MCUs */
    int plane_w, plane_h;   /* in samples, padded */
    int real_w, real_h;     /* ceil(image * hs / hmax) */
    uint8_t *plane;
} Component;

typedef struct {
    int width, height, ncomp, hmax, vmax;
    int mcus_x, mcus_y, restart_interval;
    uint16_t quant[4][64]; /* natural (row-major) order */
    int quant_present[4];
    HuffTable dc[4], ac[4];
    Component comp[3];
    const uint8_t *scan;
    size_t scan_len;
} Jpeg;

static void build_huffman(HuffTable *t) {
    int code = 0, k = 0;
    for (int len = 1; len <= 16; len++) {
        t->valptr[len] = k;
        t->mincode[len] = code;
        code += t->bits[len];
        k += t->bits[len];
        t->maxcode[len] = t->bits[len] ? code - 1 : -1;
        code <<= 1;
    }
    t->maxcode[17] = 0x7fffffff;
    memset(t->look, 0, sizeof(t->look));
    code = 0;
    k = 0;
    for (int len = 1; len <= 9; len++) {
        for (int i = 0; i < t->bits[len]; i++, k++, code++) {
            int first = code << (9 - len);
            for (int f = 0; f < (1 << (9 - len)); f++)
                t->look[first + f] = (uint16_t)((len << 8) | t->vals[k]);
        }
        code <<= 1;
    }
    t->present = 1;
}

static int parse_headers(const uint8_t *d, size_t n, Jpeg *j) {
    memset(j, 0, sizeof(*j));
    if (n < 4 || d[0] != 0xFF || d[1] != 0xD8) return ORACLE_ERR_FORMAT;
    size_t p = 2;
    int have_sof = 0;
    while (p + 4 <= n) {
        if (d[p] != 0xFF) return ORACLE_ERR_FORMAT;
        while (p < n && d[p] == 0xFF) p++; /* fill bytes */
        if (p >= n) return ORACLE_ERR_FORMAT;
        int m = d[p++];
        if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01) continue;
        if (m == 0xD9) return ORACLE_ERR_FORMAT;
        if (p + 2 > n) return ORACLE_ERR_FORMAT;
        size_t len = ((size_t)d[p] << 8) | d[p + 1];
        if (len < 2 || p + len > n) return ORACLE_ERR_FORMAT;
        const uint8_t *s = d + p + 2;
        size_t sl = len - 2;
        if (m == 0xDB) { /* DQT */
            size_t q = 0;
            while (q < sl) {
                int pq = s[q] >> 4, tq = s[q] & 15;
                q++;
                if (tq > 3) return ORACLE_ERR_FORMAT;
                if (q + (pq ? 128 : 64) > sl) return ORACLE_ERR_FORMAT;
                for (int i = 0; i < 64; i++) {
                    int v = pq ? ((s[q] << 8) | s[q + 1]) : s[q];
                    q += pq ? 2 : 1;
                    j->quant[tq][ZIGZAG[i]] = (uint16_t)v;
                }
                j->quant_present[tq] = 1;
            }
        } else if (m == 0xC4) { /* DHT */
            size_t q = 0;
            while (q < sl) {
                int tc = s[q] >> 4, th = s[q] & 15;
                q++;
                if (tc > 1 || th > 3 || q + 16 > sl) return ORACLE_ERR_FORMAT;
                HuffTable *t = tc ? &j->ac[th] : &j->dc[th];
                int total = 0;
                t->bits[0] = 0;
                for (int i = 1; i <= 16; i++) {
                    t->bits[i] = s[q++];
                    total += t->bits[i];
                }
                if (total > 256 || q + total > sl) return ORACLE_ERR_FORMAT;
                memcpy(t->vals, s + q, total);
                q += total;
                build_huffman(t);
            }
        } else if (m == 0xC0 || m == 0xC1) { /* SOF0 / SOF1 */
            if (sl < 6 || s[0] != 8) return ORACLE_ERR_UNSUPPORTED;
            j->height = (s[1] << 8) | s[2];
            j->width = (s[3] << 8) | s[4];
            j->ncomp = s[5];
            if (j->ncomp != 1 && j->ncomp != 3) return ORACLE_ERR_UNSUPPORTED;
            if (sl < (size_t)(6 + 3 * j->ncomp)) return ORACLE_ERR_FORMAT;
            if (j->width == 0 || j->height == 0) return ORACLE_ERR_UNSUPPORTED;
            for (int c = 0; c < j->ncomp; c++) {
                j->comp[c].id = s[6 + 3 * c];
                j->comp[c].hs = s[7 + 3 * c] >> 4;
                j->comp[c].vs = s[7 + 3 * c] & 15;
                j->comp[c].tq = s[8 + 3 * c];
                if (j->comp[c].tq > 3) return ORACLE_ERR_FORMAT;
            }
            have_sof = 1;
        } else if (m >= 0xC2 && m <= 0xCF && m != 0xC8 && m != 0xCC) {
            return ORACLE_ERR_UNSUPPORTED; /* progressive, lossless, arithmetic */
        } else if (m == 0xDD) {            /* DRI */
            if (sl < 2) return ORACLE_ERR_FORMAT;
            j->restart_interval = (s[0] << 8) | s[1];
        } else if (m == 0xDA) { /* SOS */
            if (!have_sof) return ORACLE_ERR_FORMAT;
            if (sl < 1 || s[0] != j->ncomp || sl < (size_t)(4 + 2 * j->ncomp))
                return ORACLE_ERR_UNSUPPORTED; /* non-interleaved multi-scan */
            for (int c = 0; c < j->ncomp; c++) {
                if (s[1 + 2 * c] != j->comp[c].id) return ORACLE_ERR_UNSUPPORTED;
                j->comp[c].td = s[2 + 2 * c] >> 4;
                j->comp[c].ta = s[2 + 2 * c] & 15;
                if (j->comp[c].td > 3 || j->comp[c].ta > 3) return ORACLE_ERR_FORMAT;
                if (!j->dc[j->comp[c].td].present || !j->ac[j->comp[c].ta].present)
                    return ORACLE_ERR_FORMAT;
                if (!j->quant_present[j->comp[c].tq]) return ORACLE_ERR_FORMAT;
            }
            j->scan = d + p + len;
            j->scan_len = n - (p + len);
            break;
        }
        p += len;
    }
    if (!j->scan) return ORACLE_ERR_FORMAT;
    if (j->ncomp == 1) {
        j->comp[0].hs = j->comp[0].vs = 1; /* a single-component scan is never interleaved */
    } else {
        if (j->comp[1].hs != 1 || j->comp[1].vs != 1 || j->comp[2].hs != 1 || j->comp[2].vs != 1)
            return ORACLE_ERR_UNSUPPORTED;
        int hs = j->comp[0].hs, vs = j->comp[0].vs;
        if (!((hs == 1 && vs == 1) || (hs == 2 && vs == 1) || (hs == 2 && vs == 2)))
            return ORACLE_ERR_UNSUPPORTED;
    }
    j->hmax = j->comp[0].hs;
    j->vmax = j->comp[0].vs;
    j->mcus_x = (j->width + 8 * j->hmax - 1) / (8 * j->hmax);
    j->mcus_y = (j->height + 8 * j->vmax - 1) / (8 * j->vmax);
    for (int c = 0; c < j->ncomp; c++) {
        Component *k = &j->comp[c];
        k->blocks_w = j->mcus_x * k->hs;
        k->blocks_h = j->mcus_y * k->vs;
        k->plane_w = k->blocks_w * 8;
        k->plane_h = k->blocks_h * 8;
        k->real_w = (j->width * k->hs + j->hmax - 1) / j->hmax;
        k->real_h = (j->height * k->vs + j->vmax - 1) / j->vmax;
    }
    return ORACLE_OK;
}

/* ---------------------------------------------------------------- entropy decode (T.81 F.2) */

typedef struct {
    const uint8_t *p, *end;
    uint64_t acc; /* bits are left-aligned */
    int nbits;
    int hit_marker;
} BitReader;

static inline void refill(BitReader *b) {
    while (b->nbits <= 56) {
        uint64_t byte = 0;
        if (!b->hit_marker && b->p < b->end) {
            byte = *b->p;
            if (byte == 0xFF) {
                if (b->p + 1 < b->end && b->p[1] == 0x00) {
                    b->p += 2;
                } else {
                    b->hit_marker = 1; /* feed zeros past a marker */
                    byte = 0;
                }
            } else {
                b->p++;
            }
        }
        b->acc |= byte << (56 - b->nbits);
        b->nbits += 8;
    }
}

static inline int peek(BitReader *b, int n) { return (int)(b->acc >> (64 - n)); }
static inline void skip(BitReader *b, int n) {
    b->acc <<= n;
    b->nbits -= n;
}

static inline int decode_symbol(BitReader *b, const HuffTable *t) {
    if (b->nbits < 16) refill(b);
    int look = t->look[peek(b, 9)];
    if (look) {
        skip(b, look >> 8);
        return look & 255;
    }
    int code = peek(b, 16);
    for (int len = 10; len <= 16; len++) {
        int c = code >> (16 - len);
        if (t->maxcode[len] >= 0 && c <= t->maxcode[len] && c >= t->mincode[len]) {
            skip(b, len);
            return t->vals[t->valptr[len] + c - t->mincode[len]];
        }
    }
    skip(b, 16);
    return 0; /* invalid code: treated as symbol 0 */
}

static inline int receive_extend(BitReader *b, int s) {
    if (s == 0) return 0;
    if (b->nbits < s) refill(b);
    int v = peek(b, s);
    skip(b, s);
    return v < (1 << (s - 1)) ? v - (1 << s) + 1 : v;
}

/* Decodes the whole scan into quantised coefficients, natural order inside each 64-entry block,
 * blocks in scan order (MCU by MCU; inside an MCU component by component, rows then columns).
 * DC values are already un-differenced. */
static int decode_scan(const Jpeg *j, int16_t *coef, size_t nblocks) {
    BitReader b = {j->scan, j->scan + j->scan_len, 0, 0, 0};
    int pred[3] = {0, 0, 0};
    size_t blk = 0;
    int restarts_left = j->restart_interval;
    memset(coef, 0, nblocks * 64 * sizeof(int16_t));
    for (int m = 0; m < j->mcus_x * j->mcus_y; m++) {
        if (j->restart_interval && restarts_left == 0) {
            /* byte-align, expect RSTn */
            b.acc = 0;
            b.nbits = 0;
            if (b.hit_marker) {
                b.hit_marker = 0;
            }
            while (b.p + 1 < b.end && !(b.p[0] == 0xFF && b.p[1] >= 0xD0 && b.p[1] <= 0xD7)) b.p++;
            if (b.p + 1 >= b.end) return ORACLE_ERR_DATA;
            b.p += 2;
            pred[0] = pred[1] = pred[2] = 0;
            restarts_left = j->restart_interval;
        }
        for (int c = 0; c < j->ncomp; c++) {
            const Component *k = &j->comp[c];
            const HuffTable *dc = &j->dc[k->td], *ac = &j->ac[k->ta];
            for (int u = 0; u < k->hs * k->vs; u++) {
                int16_t *blkc = coef + blk * 64;
                int s = decode_symbol(&b, dc);
                if (s > 15) return ORACLE_ERR_DATA;
                pred[c] += receive_extend(&b, s);
                blkc[0] = (int16_t)pred[c];
                for (int z = 1; z < 64;) {
                    int rs = decode_symbol(&b, ac);
                    int r = rs >> 4;
                    s = rs & 15;
                    if (s == 0) {
                        if (r != 15) break;
                        z += 16;
                        continue;
                    }
                    z += r;
                    int v = receive_extend(&b, s);
                    if (z > 63) break;
                    blkc[ZIGZAG[z]] = (int16_t)v;
                    z++;
                }
                blk++;
            }
        }
        if (j->restart_interval) restarts_left--;
    }
    return ORACLE_OK;
}

/* ------------------------------------------------------------------------------------ IDCT */

/* The 8 one-dimensional AAN scale factors s[0] = 1, s[k] = sqrt(2) cos(k pi / 16), scaled by
 * 2^14 and rounded, as the fast-integer method folds them into the dequantisation table. */
static void aan_scale14(int32_t s[64]) {
    static const double f[8] = {1.0,         1.387039845, 1.306562965, 1.175875602,
                                1.0,         0.785694958, 0.541196100, 0.275899379};
    for (int r = 0; r < 8; r++)
        for (int c = 0; c < 8; c++) s[r * 8 + c] = (int32_t)(f[r] * f[c] * 16384.0 + 0.5);
}

static inline int16_t w16(int32_t v) { return (int16_t)(uint16_t)v; } /* 16-bit lane wrap */
static inline int16_t mul8(int16_t v, int32_t c) { return w16(((int32_t)v * c) >> 8); }

/* Fast integer inverse DCT (AAN), computed in wrapping 16-bit lanes as the x86 SIMD build of
 * libjpeg-turbo does; the multiplier table carries 2 fractional bits, the 1-D passes truncate
 * products to 8 fractional bits, the final shift by 5 truncates, and the result saturates to
 * [-128, 127] before the +128 level shift. */
static void idct_fast_1d(const int16_t in[8], int16_t out[8]) {
    int16_t t0 = in[0], t1 = in[2], t2 = in[4], t3 = in[6];
    int16_t t10 = w16(t0 + t2), t11 = w16(t0 - t2);
    int16_t t13 = w16(t1 + t3);
    int16_t t12 = w16(mul8(w16(t1 - t3), 362) - t13);
    t0 = w16(t10 + t13);
    t3 = w16(t10 - t13);
    t1 = w16(t11 + t12);
    t2 = w16(t11 - t12);
    int16_t t4 = in[1], t5 = in[3], t6 = in[5], t7 = in[7];
    int16_t z13 = w16(t6 + t5), z10 = w16(t6 - t5), z11 = w16(t4 + t7), z12 = w16(t4 - t7);
    t7 = w16(z11 + z13);
    t11 = mul8(w16(z11 - z13), 362);
    int16_t z5 = mul8(w16(z10 + z12), 473);
    t10 = w16(mul8(z12, 277) - z5);
    t12 = w16(mul8(z10, -669) + z5);
    t6 = w16(t12 - t7);
    t5 = w16(t11 - t6);
    t4 = w16(t10 + t5);
    out[0] = w16(t0 + t7);
    out[7] = w16(t0 - t7);
    out[1] = w16(t1 + t6);
    out[6] = w16(t1 - t6);
    out[2] = w16(t2 + t5);
    out[5] = w16(t2 - t5);
    out[4] = w16(t3 + t4);
    out[3] = w16(t3 - t4);
}

static void idct_fast_block(const int16_t *coef, const int16_t *mult, uint8_t *out, int stride) {
    int16_t ws[64], col[8], res[8];
    for (int c = 0; c < 8; c++) {
        for (int r = 0; r < 8; r++) col[r] = w16((int32_t)coef[r * 8 + c] * mult[r * 8 + c]);
        idct_fast_1d(col, res);
        for (int r = 0; r < 8; r++) ws[r * 8 + c] = res[r];
    }
    for (int r = 0; r < 8; r++) {
        idct_fast_1d(ws + r * 8, res);
        for (int c = 0; c < 8; c++) {
            int v = res[c] >> 5;
            v = v < -128 ? -128 : (v > 127 ? 127 : v);
            out[r * stride + c] = (uint8_t)(v + 128);
        }
    }
}

/* Accurate integer inverse DCT (Loeffler-Ligtenberg-Moschytz, 13-bit constants, 2 extra bits
 * kept between the passes).  Not on the reference's path; used to pin the upsampler against
 * decoders that use it. */
#define C_0_298631336 2446
#define C_0_390180644 3196
#define C_0_541196100 4433
#define C_0_765366865 6270
#define C_0_899976223 7373
#define C_1_175875602 9633
#define C_1_501321110 12299
#define C_1_847759065 15137
#define C_1_961570560 16069
#define C_2_053119869 16819
#define C_2_562915447 20995
#define C_3_072711026 25172

static void idct_accurate_1d(const int32_t in[8], int32_t out[8], int shift, int dc_bias) {
    int32_t z2 = in[2], z3 = in[6];
    int32_t z1 = (z2 + z3) * C_0_541196100;
    int32_t t2 = z1 + z3 * (-C_1_847759065);
    int32_t t3 = z1 + z2 * C_0_765366865;
    int32_t t0 = (in[0] + in[4]) * 8192 + dc_bias;
    int32_t t1 = (in[0] - in[4]) * 8192 + dc_bias;
    int32_t t10 = t0 + t3, t13 = t0 - t3, t11 = t1 + t2, t12 = t1 - t2;
    int32_t a0 = in[7], a1 = in[5], a2 = in[3], a3 = in[1];
    z1 = a0 + a3;
    z2 = a1 + a2;
    z3 = a0 + a2;
    int32_t z4 = a1 + a3;
    int32_t z5 = (z3 + z4) * C_1_175875602;
    a0 *= C_0_298631336;
    a1 *= C_2_053119869;
    a2 *= C_3_072711026;
    a3 *= C_1_501321110;
    z1 *= -C_0_899976223;
    z2 *= -C_2_562915447;
    z3 = z3 * (-C_1_961570560) + z5;
    z4 = z4 * (-C_0_390180644) + z5;
    a0 += z1 + z3;
    a1 += z2 + z4;
    a2 += z2 + z3;
    a3 += z1 + z4;
    out[0] = (t10 + a3) >> shift;
    out[7] = (t10 - a3) >> shift;
    out[1] = (t11 + a2) >> shift;
    out[6] = (t11 - a2) >> shift;
    out[2] = (t12 + a1) >> shift;
    out[5] = (t12 - a1) >> shift;
    out[3] = (t13 + a0) >> shift;
    out[4] = (t13 - a0) >> shift;
}

static void idct_accurate_block(const int16_t *coef, const uint16_t *quant, uint8_t *out,
                                int stride) {
    int32_t ws[64], col[8], res[8];
    for (int c = 0; c < 8; c++) {
        for (int r = 0; r < 8; r++) col[r] = (int32_t)coef[r * 8 + c] * quant[r * 8 + c];
        idct_accurate_1d(col, res, 11, 1 << 10);
        for (int r = 0; r < 8; r++) ws[r * 8 + c] = res[r];
    }
    for (int r = 0; r < 8; r++) {
        idct_accurate_1d(ws + r * 8, res, 18, 1 << 17);
        for (int c = 0; c < 8; c++) {
            int v = res[c] + 128;
            out[r * stride + c] = (uint8_t)(v < 0 ? 0 : (v > 255 ? 255 : v));
        }
    }
}

/* ------------------------------------------------------------ reduced-size inverse transforms
 * Decoding at 1/2, 1/4 or 1/8 scale (libjpeg's scale_num / scale_denom, the arguments
 * libffcv/libffcv.cpp:59,89-90 passes to TurboJPEG) inverts every block straight to 4x4, 2x2 or
 * 1x1 samples.  Mathematically an output sample is the mean of the r x r samples (r = 2, 4, 8)
 * of the full inverse transform that it replaces.  Per dimension, with the 8-point transform in
 * the scaling the integer transforms use, x[n] = a0 + sqrt(2) sum_k a_k cos((2n+1) k pi / 16), the
 * sum of r neighbours is
 *     S[m] = r a0 + sum_k a_k C_r(k, m),   C_r(k, m) = sqrt(2) sum_{j<r} cos((2 (r m + j) + 1) k pi / 16)
 * (C vanishes for k = 4 when r = 2 and for every even k when r >= 4).  libjpeg-turbo evaluates
 * exactly this with 13-bit constants round(|C| 2^13), 32-bit sums, dequantisation by the plain
 * quantiser step, two extra fraction bits after the column pass, and one rounding shift per pass
 * that also divides by r; the result is pinned against its binary in the tests. */
#include <math.h>

static void reduced_constants(int r, int32_t c[8][4]) {
    const double pi = 3.14159265358979323846;
    for (int k = 0; k < 8; k++)
        for (int m = 0; m < 8 / r; m++) {
            double v = 0;
            for (int j = 0; j < r; j++) v += cos((2 * (r * m + j) + 1) * k * pi / 16.0);
            v *= sqrt(2.0);
            double a = fabs(v);
            int32_t q = a < 1e-9 ? 0 : (int32_t)(a * 8192.0 + 0.5);
            c[k][m] = v < 0 ? -q : q;
        }
}

/* in[8] (in[k] for the k the size uses) -> out[8 / r], rounding shift `shift`. */
static void reduced_1d(const int32_t in[8], int32_t *out, int r, int log2r, const int32_t c[8][4], int shift) {
    for (int m = 0; m < 8 / r; m++) {
        int32_t acc = in[0] * (1 << (13 + log2r));
        for (int k = 1; k < 8; k++) acc += in[k] * c[k][m];
        out[m] = (acc + (1 << (shift - 1))) >> shift;
    }
}

/* coef: 64 quantised coefficients, natural order; writes (8 / r)^2 samples. */
static void idct_reduced_block(const int16_t *coef, const uint16_t *quant, uint8_t *out, int stride, int r) {
    const int log2r = r == 2 ? 1 : (r == 4 ? 2 : 3), n = 8 / r;
    int32_t c[8][4];
    reduced_constants(r, c);
    int32_t ws[8][4]; /* [column of the block][row of the result] */
    for (int col = 0; col < 8; col++) {
        int32_t in[8], res[4];
        for (int k = 0; k < 8; k++) in[k] = (int32_t)coef[k * 8 + col] * quant[k * 8 + col];
        reduced_1d(in, res, r, log2r, c, 13 - 2 + log2r);
        for (int m = 0; m < n; m++) ws[col][m] = res[m];
    }
    for (int row = 0; row < n; row++) {
        int32_t in[8], res[4];
        for (int k = 0; k < 8; k++) in[k] = ws[k][row];
        reduced_1d(in, res, r, log2r, c, 13 + 2 + 3 + log2r);
        for (int m = 0; m < n; m++) {
            int v = res[m] + 128;
            out[row * stride + m] = (uint8_t)(v < 0 ? 0 : (v > 255 ? 255 : v));
        }
    }
}

static void fast_multipliers(const uint16_t *quant, int16_t *mult) {
    int32_t s[64];
    aan_scale14(s);
    for (int i = 0; i < 64; i++)
        mult[i] = (int16_t)(((int32_t)quant[i] * s[i] + (1 << 11)) >> 12);
}

/* ------------------------------------------------------------- upsampling + colour conversion */

static inline int clamp8(int v) { return v < 0 ? 0 : (v > 255 ? 255 : v); }

/* Chroma sample at full resolution, column x / row y of the output image. */
static inline int chroma_at(const Component *k, int hs_ratio, int vs_ratio, int x, int y,
                            int mode) {
    const uint8_t *p = k->plane;
    int W = k->plane_w;
    if (hs_ratio == 1 && vs_ratio == 1) return p[y * W + x];
    int cx = x >> 1, cy = vs_ratio == 2 ? (y >> 1) : y;
    if (mode == UPSAMPLE_REPLICATE) return p[cy * W + cx];
    if (hs_ratio == 2 && vs_ratio == 1) {
        /* h2v1 triangle filter: 3/4 nearer + 1/4 further, biases 1 and 2 alternate */
        if (k->real_w < 3) return p[cy * W + cx]; /* too narrow for the filter: replicate */
        int cur = p[cy * W + cx];
        if ((x & 1) == 0) {
            if (cx == 0) return cur;
            return (3 * cur + p[cy * W + cx - 1] + 1) >> 2;
        }
        if (cx == k->real_w - 1) return cur;
        return (3 * cur + p[cy * W + cx + 1] + 2) >> 2;
    }
    /* h2v2 triangle filter: vertical 3:1 sums first, then horizontal 3:1 with biases 8 and 7 */
    if (k->real_w < 3) return p[cy * W + cx];
    int ny = (y & 1) ? cy + 1 : cy - 1; /* the further row; image edges replicate */
    if (ny < 0) ny = 0;
    if (ny > k->real_h - 1) ny = k->real_h - 1;
    int cur = 3 * p[cy * W + cx] + p[ny * W + cx];
    if ((x & 1) == 0) {
        if (cx == 0) return (cur * 4 + 8) >> 4;
        int last = 3 * p[cy * W + cx - 1] + p[ny * W + cx - 1];
        return (cur * 3 + last + 8) >> 4;
    }
    if (cx == k->real_w - 1) return (cur * 4 + 7) >> 4;
    int next = 3 * p[cy * W + cx + 1] + p[ny * W + cx + 1];
    return (cur * 3 + next + 7) >> 4;
}

/* 16.16 fixed-point ITU-R BT.601 full-range conversion (JFIF). */
static inline void ycc_to_rgb(int y, int cb, int cr, uint8_t *rgb) {
    cb -= 128;
    cr -= 128;
    int r = y + ((91881 * cr + 32768) >> 16);
    int g = y + ((-22554 * cb - 46802 * cr + 32768) >> 16);
    int b = y + ((116130 * cb + 32768) >> 16);
    rgb[0] = (uint8_t)clamp8(r);
    rgb[1] = (uint8_t)clamp8(g);
    rgb[2] = (uint8_t)clamp8(b);
}

/* ------------------------------------------------------------------------------ entry points */

static size_t total_blocks(const Jpeg *j) {
    size_t per_mcu = 0;
    for (int c = 0; c < j->ncomp; c++) per_mcu += (size_t)j->comp[c].hs * j->comp[c].vs;
    return per_mcu * j->mcus_x * j->mcus_y;
}

/* info[0..7] = width, height, ncomp, luma hs, luma vs, restart interval, scan offset, scan len */
int oracle_jpeg_info(const uint8_t *data, size_t n, int64_t *info) {
    Jpeg j;
    int rc = parse_headers(data, n, &j);
    if (rc) return rc;
    info[0] = j.width;
    info[1] = j.height;
    info[2] = j.ncomp;
    info[3] = j.hmax;
    info[4] = j.vmax;
    info[5] = j.restart_interval;
    info[6] = (int64_t)(j.scan - data);
    info[7] = (int64_t)j.scan_len;
    return ORACLE_OK;
}

/* Number of 8x8 blocks the scan holds (scan order). */
int64_t oracle_jpeg_num_blocks(const uint8_t *data, size_t n) {
    Jpeg j;
    if (parse_headers(data, n, &j)) return -1;
    return (int64_t)total_blocks(&j);
}

/* Quantised coefficients in scan order, natural order within a block, DC un-differenced. */
int oracle_jpeg_coefficients(const uint8_t *data, size_t n, int16_t *coef) {
    Jpeg j;
    int rc = parse_headers(data, n, &j);
    if (rc) return rc;
    return decode_scan(&j, coef, total_blocks(&j));
}

/* Full decode to packed RGB (height*width*3).  width/height must equal the stream's. */
int oracle_jpeg_decode(const uint8_t *data, size_t n, uint8_t *out, int height, int width,
                       int idct, int upsample) {
    Jpeg j;
    int rc = parse_headers(data, n, &j);
    if (rc) return rc;
    if (j.width != width || j.height != height) return ORACLE_ERR_DIMS;
    size_t nblocks = total_blocks(&j);
    int16_t *coef = (int16_t *)malloc(nblocks * 64 * sizeof(int16_t));
    if (!coef) return ORACLE_ERR_DATA;
    rc = decode_scan(&j, coef, nblocks);
    if (rc) {
        free(coef);
        return rc;
    }
    int16_t mult[3][64];
    for (int c = 0; c < j.ncomp; c++) {
        Component *k = &j.comp[c];
        k->plane = (uint8_t *)malloc((size_t)k->plane_w * k->plane_h);
        fast_multipliers(j.quant[k->tq], mult[c]);
    }
    size_t blk = 0;
    for (int my = 0; my < j.mcus_y; my++)
        for (int mx = 0; mx < j.mcus_x; mx++)
            for (int c = 0; c < j.ncomp; c++) {
                Component *k = &j.comp[c];
                for (int v = 0; v < k->vs; v++)
                    for (int h = 0; h < k->hs; h++, blk++) {
                        uint8_t *dst = k->plane + (size_t)((my * k->vs + v) * 8) * k->plane_w +
                                       (mx * k->hs + h) * 8;
                        if (idct == IDCT_FAST)
                            idct_fast_block(coef + blk * 64, mult[c], dst, k->plane_w);
                        else
                            idct_accurate_block(coef + blk * 64, j.quant[k->tq], dst, k->plane_w);
                    }
            }
    const Component *Y = &j.comp[0];
    for (int y = 0; y < height; y++)
        for (int x = 0; x < width; x++) {
            uint8_t *px = out + ((size_t)y * width + x) * 3;
            int lum = Y->plane[(size_t)y * Y->plane_w + x];
            if (j.ncomp == 1) {
                px[0] = px[1] = px[2] = (uint8_t)lum;
            } else {
                int cb = chroma_at(&j.comp[1], j.hmax, j.vmax, x, y, upsample);
                int cr = chroma_at(&j.comp[2], j.hmax, j.vmax, x, y, upsample);
                ycc_to_rgb(lum, cb, cr, px);
            }
        }
    for (int c = 0; c < j.ncomp; c++) free(j.comp[c].plane);
    free(coef);
    return ORACLE_OK;
}

/* Which scale a stream can be decoded at: three components, no chroma subsampling or 2x2. */
int oracle_jpeg_scalable(const uint8_t *data, size_t n) {
    Jpeg j;
    if (parse_headers(data, n, &j)) return 0;
    return j.ncomp == 3 && ((j.hmax == 1 && j.vmax == 1) || (j.hmax == 2 && j.vmax == 2));
}

/* Decode at 1 / denom (denom = 2, 4, 8) to packed RGB of ceil(height / denom) x ceil(width / denom)
 * pixels, the way libjpeg-turbo does with scale_num / scale_denom = 1 / denom, the fast integer
 * transform selected and fancy upsampling on: the luma blocks are inverted at 8 / denom samples a
 * side; with 2x2 chroma subsampling the chroma blocks are inverted at twice that (at most 8: the
 * full-size fast transform), which brings them to the luma resolution, so that no upsampling
 * step is left.  out_h / out_w must be those dimensions. */
int oracle_jpeg_decode_scaled(const uint8_t *data, size_t n, uint8_t *out, int out_h, int out_w, int denom) {
    Jpeg j;
    int rc = parse_headers(data, n, &j);
    if (rc) return rc;
    if (denom != 2 && denom != 4 && denom != 8) return ORACLE_ERR_UNSUPPORTED;
    if (j.ncomp != 3 || !((j.hmax == 1 && j.vmax == 1) || (j.hmax == 2 && j.vmax == 2))) return ORACLE_ERR_UNSUPPORTED;
    if (out_w != (j.width + denom - 1) / denom || out_h != (j.height + denom - 1) / denom) return ORACLE_ERR_DIMS;
    size_t nblocks = total_blocks(&j);
    int16_t *coef = (int16_t *)malloc(nblocks * 64 * sizeof(int16_t));
    if (!coef) return ORACLE_ERR_DATA;
    rc = decode_scan(&j, coef, nblocks);
    if (rc) {
        free(coef);
        return rc;
    }
    int16_t mult[3][64];
    int bs[3]; /* samples a side a block of each component is inverted to */
    for (int c = 0; c < 3; c++) {
        Component *k = &j.comp[c];
        bs[c] = 8 / denom * (j.hmax / k->hs);
        if (bs[c] > 8) bs[c] = 8;
        k->plane_w = k->blocks_w * bs[c];
        k->plane_h = k->blocks_h * bs[c];
        k->plane = (uint8_t *)malloc((size_t)k->plane_w * k->plane_h);
        fast_multipliers(j.quant[k->tq], mult[c]);
    }
    size_t blk = 0;
    for (int my = 0; my < j.mcus_y; my++)
        for (int mx = 0; mx < j.mcus_x; mx++)
            for (int c = 0; c < 3; c++) {
                Component *k = &j.comp[c];
                for (int v = 0; v < k->vs; v++)
                    for (int h = 0; h < k->hs; h++, blk++) {
                        uint8_t *dst = k->plane + (size_t)((my * k->vs + v) * bs[c]) * k->plane_w +
                                       (mx * k->hs + h) * bs[c];
                        if (bs[c] == 8)
                            idct_fast_block(coef + blk * 64, mult[c], dst, k->plane_w);
                        else
                            idct_reduced_block(coef + blk * 64, j.quant[k->tq], dst, k->plane_w, 8 / bs[c]);
                    }
            }
    for (int y = 0; y < out_h; y++)
        for (int x = 0; x < out_w; x++)
            ycc_to_rgb(j.comp[0].plane[(size_t)y * j.comp[0].plane_w + x], j.comp[1].plane[(size_t)y * j.comp[1].plane_w + x],
                       j.comp[2].plane[(size_t)y * j.comp[2].plane_w + x], out + ((size_t)y * out_w + x) * 3);
    for (int c = 0; c < 3; c++) free(j.comp[c].plane);
    free(coef);
    return ORACLE_OK;
}

/* Same signature as libffcv/libffcv.cpp:53-61 `imdecode`.  The crop and flip arguments must be
 * the identity, as in every call the reference makes (fields/rgb_image.py:131-132,196-197); the
 * scale may be 1/1 (what the reference passes) or 1/2, 1/4, 1/8: crop_height / crop_width stay
 * the stream's dimensions and the output has TJSCALED(dim, scale) = ceil(dim * num / denom) pixels
 * a side, as in the reference's tjDecompress2 call (libffcv.cpp:104-106). */
int imdecode(unsigned char *input_buffer, uint64_t input_size, uint32_t source_height,
             uint32_t source_width, unsigned char *output_buffer, uint32_t crop_height,
             uint32_t crop_width, uint32_t offset_x, uint32_t offset_y, uint32_t scale_num,
             uint32_t scale_denom, _Bool enable_crop, _Bool hflip) {
    (void)source_height;
    (void)source_width;
    (void)offset_x;
    (void)offset_y;
    if (enable_crop || hflip || scale_num == 0 || scale_denom % scale_num != 0) return -1;
    const uint32_t denom = scale_denom / scale_num;
    int rc;
    if (denom == 1)
        rc = oracle_jpeg_decode(input_buffer, (size_t)input_size, output_buffer, (int)crop_height,
                                (int)crop_width, IDCT_FAST, UPSAMPLE_FANCY);
    else
        rc = oracle_jpeg_decode_scaled(input_buffer, (size_t)input_size, output_buffer,
                                       (int)((crop_height + denom - 1) / denom), (int)((crop_width + denom - 1) / denom),
                                       (int)denom);
    return rc ? -1 : 0;
}

void my_memcpy(void *source, void *dst, uint64_t size) { memcpy(dst, source, size); }
