// Structures shared by the host staging code and the CUDA kernels.  A staged batch is one
// contiguous blob, identical in pinned host memory and in HBM:
//   [BatchHeader][ImageDesc x n][HuffTable x n_huff][MultTable x n_mult][params int32][payloads]
// so one host->device copy moves everything a batch needs.
#pragma once
#include <stdint.h>

namespace ffcvb {

constexpr int kMaxComponents = 3;
constexpr int kPayloadAlign = 16;

// Per-sample work descriptor.
struct ImageDesc {
    uint64_t payload_off;  // byte offset of the staged payload inside the blob (16-byte aligned)
    uint32_t payload_size; // staged bytes
    uint16_t mode;         // 0 jpg, 1 raw (ffcv/fields/rgb_image.py:21-23)
    int16_t host_status;   // 0, or a negative code when the host parser rejected the stream
    uint16_t height, width;
    uint16_t row0, rows;   // raw: first image row present in the staged payload, number of rows
    uint16_t col0, cols;   // raw: first image column present, number of columns
    union {
        uint32_t raw_pitch; // raw: bytes between staged rows (>= cols * 3)
        uint32_t rgb_pitch; // JPEG: bytes between rows of the decoded RGB image (>= dec_width * 3; a multiple
                            // of 16 in the batch scratch so that the colour kernels store whole words)
    };
    // ---- JPEG only ----
    uint32_t scan_off;     // entropy-coded segment, relative to payload_off
    uint32_t scan_len;
    uint8_t ncomp, hs, vs, bpm; // luma sampling factors; blocks per MCU
    uint16_t mcus_x, mcus_y;
    uint16_t restart_interval;
    uint8_t dc_tab[kMaxComponents], ac_tab[kMaxComponents]; // indices into the batch's HuffTable array
    uint8_t q_tab[kMaxComponents];                          // indices into the batch's MultTable array
    uint8_t raw_skew;      // raw, gathered row by row: row r of the staged payload starts
                           // (src_addr + r * width * 3) & 15 bytes into its raw_pitch-wide slot
    // Decoding at reduced scale (1 / 2^scale_shift, JPEG only): every block of a component is
    // inverted straight to bs x bs samples (8 at full scale), and the decoded image has
    // dec_height x dec_width = ceil(height / 2^s) x ceil(width / 2^s) pixels.  With 2x2 chroma
    // subsampling the chroma blocks use twice the luma's bs (at most 8), so all planes of a scaled
    // image have the same resolution.  dec_* equal height / width for unscaled and raw samples.
    uint8_t scale_shift, bs_luma, bs_chroma;
    uint16_t dec_height, dec_width;
    // Speculative entropy decode: length in bits of this image's subsequences (multiple of 128), and
    // its place in the decode index (index_cap == 0: none), see DecodeIndexHeader.
    uint32_t subseq_bits;
    uint32_t index_cap;    // subsequences the index entry has room for
    uint64_t index_off;    // byte offset of the entry in the context's index pool
    // The crop box decides how much of the image is needed: the entropy decoder stops after
    // `mcu_rows` rows of MCUs and the inverse transform runs only on the MCUs of the box below
    // (the crop box grown by the reach of the chroma filter).  Whole image when there is no crop.
    uint16_t mcu_rows;                           // MCU rows to entropy-decode (<= mcus_y)
    uint16_t idct_row0, idct_col0, idct_col1;    // MCU box to transform: rows [idct_row0, mcu_rows), cols [idct_col0, idct_col1)
    uint32_t nblocks;      // 8x8 blocks to decode: bpm * mcus_x * mcu_rows
    uint32_t block_base;   // first block of this image in the batch coefficient buffer
    uint64_t clean_off;    // byte offset of the unstuffed scan in the bitstream scratch (4-aligned)
    uint64_t rst_off;      // streams with restart markers: byte offset, in the same scratch, of a table of
                           // ceil(MCUs / restart_interval) + 1 uint32 interval starts (4-aligned)
    uint64_t plane_off[kMaxComponents]; // byte offsets of the Y/Cb/Cr planes in the plane scratch
    uint64_t rgb_off;      // byte offset of the decoded h*w*3 image in the RGB scratch
    uint64_t src_addr;     // device-visible address of the payload in pinned host memory (0: staged copy)
};

// Canonical Huffman code (ITU-T T.81 Annex C) prepared for table-driven decoding.
constexpr int kHuffSubTables = 8; // the standard tables need 5; others fall back to the code-length walk
struct HuffTable {
    // Table entries describe what a code does to the decoder rather than what it is (see
    // huff_entry): bits 0-4 the bits the symbol consumes (code + magnitude bits), bits 5-8 the
    // number of magnitude bits, bits 9-14 the zig-zag positions an AC symbol advances (run + 1;
    // 16 for a run of zeros; 63 for an end of block, which always reaches the block's end).
    // First level, indexed by the next 9 bits: such an entry for codes of up to 9 bits;
    // 0x8000 | k when the code is longer and continues in sub[k]; 0xFFFF when it is longer
    // and no sub-table was left (walk maxcode/valoff instead).  A prefix that is no code holds
    // the entry of a 16-bit end of block.
    uint16_t look[512];
    // Second level, indexed by bits 10..16 of the code: an entry as above.
    uint16_t sub[kHuffSubTables][128];
    int32_t maxcode[18]; // largest code of each length, -1 if none
    int32_t valoff[17];  // index of the first symbol of each length minus its first code
    uint8_t vals[256];
};

// Entry of a code of `len` bits for symbol `sym` (run << 4 | magnitude bits).  A symbol without
// magnitude bits is a run of 16 zeros when its run field is 15 and ends the block otherwise.
#if defined(__CUDACC__)
__host__ __device__
#endif
inline uint16_t huff_entry(int len, int sym) {
    const int s = sym & 15, r = sym >> 4;
    const int dz = s != 0 ? r + 1 : (r == 15 ? 16 : 63);
    return (uint16_t)((len + s) | (s << 5) | (dz << 9));
}

// Dequantisation multipliers of the fast integer IDCT: quantiser step x AAN scale, 2 fraction bits;
// and the plain quantiser steps, which the reduced-size transforms of a scaled decode use.
struct MultTable {
    int16_t m[64];
    uint16_t q[64];
};

// Decode index: what a finished speculative decode of a stream knows and the next decode of the
// same stream can start from -- the exact decoder state at the start of every subsequence and the
// number of blocks completed before it.  With it every subsequence is decoded once, straight into
// its final place: no guessing, no repair rounds.  An entry lives in device memory:
//   [DecodeIndexHeader][uint64 state x (cap + 1)][uint32 blocks_before x (cap + 1)]
// and is valid when `magic` is set (written last) and scan_len / subseq_bits / clean_len match.
struct DecodeIndexHeader {
    uint32_t magic, scan_len, subseq_bits, valid_subs; // entries 0 .. valid_subs are final
    uint32_t clean_len, reserved[3];
};
constexpr uint32_t kDecodeIndexMagic = 0x58444946u;
inline
#if defined(__CUDACC__)
__host__ __device__
#endif
size_t decode_index_bytes(uint32_t cap) {
    return (sizeof(DecodeIndexHeader) + (size_t)(cap + 1) * 12 + 15) / 16 * 16;
}

struct BatchHeader {
    uint32_t n, n_huff, n_mult, n_params; // n_params = int32 per sample
    uint64_t desc_off, huff_off, mult_off, params_off, payload_off, total_bytes;
};

// Augmentation list + output description handed to the fused kernel by value.
struct OpList {
    int32_t n_ops;
    int32_t type[8];
    int32_t arg[8];
    uint8_t fill[8][4];
};

enum : int { kErrFormat = -1, kErrUnsupported = -2, kErrDims = -3, kErrData = -4 };

} // namespace ffcvb
