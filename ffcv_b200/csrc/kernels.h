// Launch wrappers of the CUDA kernels (sm_100a).  All pointers are device pointers unless noted.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "types.h"

namespace ffcvb {

// Pulls every sample's payload from pinned host memory (descs[i].src_addr, read by the SMs over
// PCIe) into its place in the device blob.  Source and destination share their alignment mod 16.
// `ctas`: CTAs of 256 threads that fetch (< 1: kGatherCtas); `in_flight`: 16-byte loads a thread
// of a JPEG payload's copy has outstanding (4 or 8).
constexpr int kGatherCtas = 16;
void launch_gather_payloads(const ImageDesc *descs, int n, uint8_t *blob, int ctas, int in_flight, cudaStream_t stream);

// Longest subsequence whose chunk the entropy decoder stages in shared memory.
constexpr int kMaxStagedBits = 1280;
// Longer subsequences leave check-points every kCheckPointBits bits (16 bytes each) so that a
// repair pass can stop where it rejoins the previous pass: entropy_checkpoint_bytes() of scratch.
constexpr int kCheckPointBits = 4096;
inline size_t entropy_checkpoint_bytes(int n_images, int entropy_threads, int subseq_bits) {
    if (subseq_bits <= kMaxStagedBits) return 0;
    return (size_t)n_images * entropy_threads * (subseq_bits / kCheckPointBits + 1) * 16;
}

// Entropy decode of every JPEG sample listed in `list` (indices into descs): unstuffs the scan
// into `clean`, Huffman-decodes it into quantised coefficients (zig-zag order inside a block,
// blocks in scan order, DC un-differenced) in `coef`, and records a per-sample status.
// `subseq_bits` is the length of the subsequences decoded speculatively in parallel (multiple
// of 32), `entropy_threads` (128, 256, 512 or 1024) the CTA size: one CTA decodes one image,
// `entropy_threads` subsequences at a time.  Samples with restart markers are listed in `seq_list`
// instead and take the restart-interval kernel (one thread per interval, no speculation; needs
// descs[i].rst_off).  `coef` needs no initialisation: the kernels clear
// every block they decode into.  `checkpoints`: entropy_checkpoint_bytes(n_list, ...) bytes of device
// scratch when the subsequences are longer than kMaxStagedBits (may be nullptr: then every repair
// pass walks its whole subsequence).
// `subseq_bits` is the longest subsequence of the batch (an image's own length is
// descs[i].subseq_bits <= subseq_bits).  `index_pool` / `index_stats`: the decode index (see
// DecodeIndexHeader; descs[i].index_off / index_cap place an image's entry) and two counters
// (images decoded from their index entry, entries written); both may be nullptr.
void launch_entropy_decode(const ImageDesc *descs, const int32_t *list, int n_list,
                           const int32_t *seq_list, int n_seq, const uint8_t *blob,
                           const HuffTable *huff, uint8_t *clean, int16_t *coef, int32_t *status,
                           int subseq_bits, int entropy_threads, void *checkpoints, uint8_t *index_pool,
                           unsigned long long *index_stats, cudaStream_t stream);

// Dequantise + fast integer IDCT of `total_blocks` blocks into the 8-bit component planes.
void launch_idct(const ImageDesc *descs, const int32_t *list, int n_list, uint32_t total_blocks,
                 const MultTable *mult, const int16_t *coef, uint8_t *planes, cudaStream_t stream);

// Chroma upsampling (triangle filter) + YCbCr->RGB into h*w*3 images in `rgb` (rows rgb_pitch
// apart).  4:2:0 images (n_quad of them) go through the quad kernel and 4:4:4 images (n_444)
// through a 2-D kernel, both converting only the crop box given by `crop_params` (row, col, h, w
// per sample; nullptr = whole image); the other n_other images go through the generic kernel.
// max_w / max_h bound the boxes in the list.  quad_tiles (device; may be nullptr): one entry
// (sample, tile x | tile y << 16) per tile of 64 x 8 chroma samples the quad kernel has to
// convert, so that it launches exactly those CTAs instead of a grid over the largest box.
void launch_color(const ImageDesc *descs, const int32_t *list, int n_list, int n_quad, int n_444, int n_other,
                  int max_w, int max_h, const uint2 *quad_tiles, int n_quad_tiles, const uint8_t *planes,
                  uint8_t *rgb, const int32_t *crop_params, int n_params, cudaStream_t stream);

// Source of the fused kernel.
struct ResizeSource {
    const ImageDesc *descs; // per-sample descriptors, or nullptr for a uniform device batch
    const uint8_t *blob;    // raw payloads live here (descs != nullptr)
    const uint8_t *rgb;     // decoded JPEG samples live here (descs != nullptr)
    const uint8_t *uniform; // [n, h, w, 3] uint8 (descs == nullptr)
    int uniform_h, uniform_w;
};

// Fused crop + INTER_AREA resize + flip/translate/cutout + lookup-table normalise.
void launch_resize_augment(const ResizeSource &src, int n, const int32_t *params, int n_params,
                           const OpList &ops, int resize, int out_h, int out_w, int out_kind,
                           const void *lut, void *out, const int32_t *status, cudaStream_t stream);

// Colour jitter kinds (ffcv/transforms/color_jitter.py).
enum { kJitterBrightness = 0, kJitterContrast = 1, kJitterSaturation = 2 };

// Brightness / contrast / saturation of the images of a uint8 [n, h, w, 3] batch whose apply[i]
// is non-zero, in place, with factor ratio[i].  grey_sum: n scratch counters (contrast only).
void launch_color_jitter(uint8_t *images, int n, int h, int w, int kind, const uint8_t *apply,
                         const double *ratio, unsigned long long *grey_sum, cudaStream_t stream);

// dst[i] = lam[i] * src[i] + (1 - lam[i]) * src[i - 1] over `count` uint8 values per image.
void launch_mixup(const uint8_t *src, uint8_t *dst, int n, long long count, const double *lam,
                  cudaStream_t stream);

// images[i] = clamp(images[i] * one_minus_alpha + mask) for the images with apply[i] != 0.
void launch_poison(uint8_t *images, int n, long long count, const uint8_t *apply, const double *one_minus_alpha,
                   const double *mask, float lo, float hi, cudaStream_t stream);

} // namespace ffcvb
