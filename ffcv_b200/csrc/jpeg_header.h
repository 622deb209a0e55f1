// Host-side parser for the marker segments of a baseline JPEG stream (ITU-T T.81 Annex B).
// Only headers are read here; the entropy-coded segment is decoded on the GPU.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "types.h"

namespace ffcvb {

struct RawHuff {
    uint8_t bits[17];
    uint8_t vals[256];
    bool present;
};

struct JpegHeader {
    int width, height, ncomp;
    int hs[3], vs[3], tq[3], td[3], ta[3];
    int restart_interval;
    uint16_t quant[4][64]; // natural (row-major) order
    bool quant_present[4];
    RawHuff dc[4], ac[4];
    size_t scan_off, scan_len;
};

// Returns 0 or a negative kErr* code.  Accepts what the GPU decoder supports: 8-bit SOF0/SOF1,
// a single interleaved scan, 1 or 3 components, luma 1x1 / 2x1 / 2x2 with 1x1 chroma.
int parse_jpeg_header(const uint8_t *d, size_t n, JpegHeader *h);

void build_huff_table(const RawHuff &raw, HuffTable *out);
void build_mult_table(const uint16_t quant[64], MultTable *out);

} // namespace ffcvb
