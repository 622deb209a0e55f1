#include "jpeg_header.h"

#include <math.h>
#include <string.h>

namespace ffcvb {

static const uint8_t kZigzag[64] = {
    0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
    41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
    30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

int parse_jpeg_header(const uint8_t *d, size_t n, JpegHeader *h) {
    memset(h, 0, sizeof(*h));
    if (n < 4 || d[0] != 0xFF || d[1] != 0xD8) return kErrFormat;
    size_t p = 2;
    bool have_sof = false, have_sos = false;
    int comp_id[3] = {0, 0, 0};
    while (p + 4 <= n) {
        if (d[p] != 0xFF) return kErrFormat;
        while (p < n && d[p] == 0xFF) p++;
        if (p >= n) return kErrFormat;
        int m = d[p++];
        if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01) continue;
        if (m == 0xD9) return kErrFormat;
        if (p + 2 > n) return kErrFormat;
        size_t len = ((size_t)d[p] << 8) | d[p + 1];
        if (len < 2 || p + len > n) return kErrFormat;
        const uint8_t *s = d + p + 2;
        size_t sl = len - 2;
        if (m == 0xDB) {
            size_t q = 0;
            while (q < sl) {
                int pq = s[q] >> 4, tq = s[q] & 15;
                q++;
                if (tq > 3 || q + (pq ? 128 : 64) > sl) return kErrFormat;
                for (int i = 0; i < 64; i++) {
                    int v = pq ? ((s[q] << 8) | s[q + 1]) : s[q];
                    q += pq ? 2 : 1;
                    h->quant[tq][kZigzag[i]] = (uint16_t)v;
                }
                h->quant_present[tq] = true;
            }
        } else if (m == 0xC4) {
            size_t q = 0;
            while (q < sl) {
                int tc = s[q] >> 4, th = s[q] & 15;
                q++;
                if (tc > 1 || th > 3 || q + 16 > sl) return kErrFormat;
                RawHuff *t = tc ? &h->ac[th] : &h->dc[th];
                int total = 0;
                t->bits[0] = 0;
                for (int i = 1; i <= 16; i++) {
                    t->bits[i] = s[q++];
                    total += t->bits[i];
                }
                if (total > 256 || q + total > sl) return kErrFormat;
                memset(t->vals, 0, sizeof(t->vals));
                memcpy(t->vals, s + q, total);
                q += total;
                t->present = true;
            }
        } else if (m == 0xC0 || m == 0xC1) {
            if (sl < 6 || s[0] != 8) return kErrUnsupported;
            h->height = (s[1] << 8) | s[2];
            h->width = (s[3] << 8) | s[4];
            h->ncomp = s[5];
            if (h->ncomp != 1 && h->ncomp != 3) return kErrUnsupported;
            if (sl < (size_t)(6 + 3 * h->ncomp)) return kErrFormat;
            if (h->width == 0 || h->height == 0) return kErrUnsupported;
            for (int c = 0; c < h->ncomp; c++) {
                comp_id[c] = s[6 + 3 * c];
                h->hs[c] = s[7 + 3 * c] >> 4;
                h->vs[c] = s[7 + 3 * c] & 15;
                h->tq[c] = s[8 + 3 * c];
                if (h->tq[c] > 3) return kErrFormat;
            }
            have_sof = true;
        } else if (m >= 0xC2 && m <= 0xCF && m != 0xC8 && m != 0xCC) {
            return kErrUnsupported;
        } else if (m == 0xDD) {
            if (sl < 2) return kErrFormat;
            h->restart_interval = (s[0] << 8) | s[1];
        } else if (m == 0xDA) {
            if (!have_sof) return kErrFormat;
            if (sl < 1 || s[0] != h->ncomp || sl < (size_t)(4 + 2 * h->ncomp)) return kErrUnsupported;
            for (int c = 0; c < h->ncomp; c++) {
                if (s[1 + 2 * c] != comp_id[c]) return kErrUnsupported;
                h->td[c] = s[2 + 2 * c] >> 4;
                h->ta[c] = s[2 + 2 * c] & 15;
                if (h->td[c] > 3 || h->ta[c] > 3) return kErrFormat;
                if (!h->dc[h->td[c]].present || !h->ac[h->ta[c]].present) return kErrFormat;
                if (!h->quant_present[h->tq[c]]) return kErrFormat;
            }
            h->scan_off = p + len;
            h->scan_len = n - (p + len);
            have_sos = true;
            break;
        }
        p += len;
    }
    if (!have_sos) return kErrFormat;
    if (h->ncomp == 1) {
        h->hs[0] = h->vs[0] = 1;
    } else {
        if (h->hs[1] != 1 || h->vs[1] != 1 || h->hs[2] != 1 || h->vs[2] != 1) return kErrUnsupported;
        int a = h->hs[0], b = h->vs[0];
        if (!((a == 1 && b == 1) || (a == 2 && b == 1) || (a == 2 && b == 2))) return kErrUnsupported;
    }
    return 0;
}

void build_huff_table(const RawHuff &raw, HuffTable *t) {
    memset(t, 0, sizeof(*t));
    memcpy(t->vals, raw.vals, 256);
    int code = 0, k = 0;
    for (int len = 1; len <= 16; len++) {
        t->valoff[len] = k - code;
        code += raw.bits[len];
        k += raw.bits[len];
        t->maxcode[len] = raw.bits[len] ? code - 1 : -1;
        code <<= 1;
    }
    t->maxcode[17] = 0x7fffffff;
    code = 0;
    k = 0;
    int n_sub = 0;
    int sub_of_prefix[512];
    for (int i = 0; i < 512; i++) sub_of_prefix[i] = -1;
    for (int len = 1; len <= 16; len++) {
        for (int i = 0; i < raw.bits[len]; i++, k++, code++) {
            if (code >= (1 << len)) continue; // over-subscribed table: ignore the excess codes
            const uint16_t entry = huff_entry(len, raw.vals[k]);
            if (len <= 9) {
                const int first = code << (9 - len);
                for (int f = 0; f < (1 << (9 - len)); f++) t->look[first + f] = entry;
            } else {
                const int prefix = code >> (len - 9);
                if (sub_of_prefix[prefix] < 0) {
                    if (n_sub < kHuffSubTables) {
                        sub_of_prefix[prefix] = n_sub;
                        t->look[prefix] = (uint16_t)(0x8000 | n_sub);
                        n_sub++;
                    } else {
                        sub_of_prefix[prefix] = kHuffSubTables; // no room: this prefix walks the code lengths
                        t->look[prefix] = 0xFFFF;
                    }
                }
                const int sub = sub_of_prefix[prefix];
                if (sub < kHuffSubTables) {
                    const int rest = (code << (16 - len)) & 127; // bits 10..16, left-aligned
                    for (int f = 0; f < (1 << (16 - len)); f++) t->sub[sub][rest + f] = entry;
                }
            }
        }
        code <<= 1;
    }
    // A bit pattern that is no code acts as a 16-bit end of block (the decoder must make progress
    // on garbage too): written into the tables, so the look-up needs no special case.
    const uint16_t invalid = (uint16_t)(16 | (63 << 9));
    for (int i = 0; i < 512; i++)
        if (t->look[i] == 0) t->look[i] = invalid;
    for (int k = 0; k < n_sub; k++)
        for (int i = 0; i < 128; i++)
            if (t->sub[k][i] == 0) t->sub[k][i] = invalid;
}

void build_mult_table(const uint16_t quant[64], MultTable *out) {
    // AAN scale factors s0 = 1, sk = sqrt(2) cos(k pi / 16), outer product scaled by 2^14.
    double f[8];
    f[0] = 1.0;
    for (int k = 1; k < 8; k++) f[k] = sqrt(2.0) * cos(k * M_PI / 16.0);
    for (int r = 0; r < 8; r++)
        for (int c = 0; c < 8; c++) {
            int32_t s = (int32_t)(f[r] * f[c] * 16384.0 + 0.5);
            out->m[r * 8 + c] = (int16_t)(((int32_t)quant[r * 8 + c] * s + (1 << 11)) >> 12);
            out->q[r * 8 + c] = quant[r * 8 + c];
        }
}

} // namespace ffcvb
