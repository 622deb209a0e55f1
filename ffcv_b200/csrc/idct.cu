// Dequantisation + fast integer inverse DCT + chroma upsampling + colour conversion (sm_100a).
//
// The arithmetic is the variant TurboJPEG selects for the reference's call
// (libffcv/libffcv.cpp:104-106, TJFLAG_FASTDCT without TJFLAG_FASTUPSAMPLE): the AAN fast integer
// IDCT evaluated in wrapping 16-bit lanes with 8-bit constants and truncating shifts, the 3:1
// triangle ("fancy") chroma upsampler, and the 16.16 fixed-point YCbCr->RGB transform.  These are
// integer butterflies in registers; they are not a dense contraction and must not be reordered,
// so no tensor cores.
#include <stdlib.h>

#include "kernels.h"

namespace ffcvb {

// The entropy decoder leaves a block's coefficients in zig-zag order (the order it decodes them
// in); position in that order of the coefficient of row r, column c: kZigzagOf[r * 8 + c].  Used
// with compile-time indices only (fully unrolled loops), so the permutation costs nothing.
__device__ __forceinline__ constexpr int zigzag_of(int n) {
    constexpr int t[64] = {0, 1, 5, 6, 14, 15, 27, 28, 2, 4, 7, 13, 16, 26, 29, 42, 3, 8, 12, 17, 25, 30, 41, 43, 9, 11, 18, 24, 31, 40, 44, 53, 10, 19, 23, 32, 39, 45, 52, 54, 20, 22, 33, 38, 46, 51, 55, 60, 21, 34, 37, 47, 50, 56, 59, 61, 35, 36, 48, 49, 57, 58, 62, 63};
    return t[n];
}

// Loads a block (64 int16 in zig-zag order, 16-byte aligned) into 32 registers of two.
__device__ __forceinline__ void load_block(const int16_t *__restrict__ coef, int (&w)[32]) {
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const int4 v = reinterpret_cast<const int4 *>(coef)[r];
        w[4 * r] = v.x;
        w[4 * r + 1] = v.y;
        w[4 * r + 2] = v.z;
        w[4 * r + 3] = v.w;
    }
}
// Coefficient of natural position n (row-major) out of the registers load_block filled.
__device__ __forceinline__ int coef_at(const int (&w)[32], int n) {
    const int z = zigzag_of(n);
    return (z & 1) ? (w[z >> 1] >> 16) : (int)(short)(w[z >> 1] & 0xffff);
}

__device__ __forceinline__ int w16(int v) { return (int)(short)v; }
__device__ __forceinline__ int mul8(int v, int c) { return w16((v * c) >> 8); }

// One 8-point pass.  Inputs and outputs are sign-extended 16-bit lane values.
__device__ __forceinline__ void idct8(int &v0, int &v1, int &v2, int &v3, int &v4, int &v5, int &v6,
                                      int &v7) {
    int t10 = w16(v0 + v4), t11 = w16(v0 - v4);
    int t13 = w16(v2 + v6);
    int t12 = w16(mul8(w16(v2 - v6), 362) - t13);
    int t0 = w16(t10 + t13), t3 = w16(t10 - t13), t1 = w16(t11 + t12), t2 = w16(t11 - t12);
    int z13 = w16(v5 + v3), z10 = w16(v5 - v3), z11 = w16(v1 + v7), z12 = w16(v1 - v7);
    int t7 = w16(z11 + z13);
    int t11b = mul8(w16(z11 - z13), 362);
    int z5 = mul8(w16(z10 + z12), 473);
    int t10b = w16(mul8(z12, 277) - z5);
    int t12b = w16(mul8(z10, -669) + z5);
    int t6 = w16(t12b - t7);
    int t5 = w16(t11b - t6);
    int t4 = w16(t10b + t5);
    v0 = w16(t0 + t7);
    v7 = w16(t0 - t7);
    v1 = w16(t1 + t6);
    v6 = w16(t1 - t6);
    v2 = w16(t2 + t5);
    v5 = w16(t2 - t5);
    v4 = w16(t3 + t4);
    v3 = w16(t3 - t4);
}

// Reduced-size inverse transforms for decoding at 1/2, 1/4, 1/8 scale (the scale_num / scale_denom
// arguments of libffcv/libffcv.cpp:59,89-90): a block goes straight to N x N samples, N = 8 / R, each
// the mean of the R x R samples of the full transform it replaces.  Per dimension, in the scaling
// of the integer transforms, the sum of R neighbouring outputs is
//     S[m] = R a0 + sum_k a_k C(k, m),   C(k, m) = sqrt(2) sum_{j<R} cos((2 (R m + j) + 1) k pi / 16),
// evaluated as libjpeg-turbo does: constants round(|C| 2^13), 32-bit sums, plain quantiser steps,
// two extra fraction bits after the column pass, one rounding shift per pass that also divides by R.
template <int R>
__device__ __forceinline__ int reduced_constant(int k, int m) {
    // C(k, m) * 2^13 for R = 2 (k = 4 contributes nothing) and R = 4 (only odd k contribute)
    constexpr int c2[8][4] = {{0, 0, 0, 0},          {20995, 8697, -8697, -20995}, {15137, -15137, -15137, 15137},
                              {7373, -17799, 17799, -7373}, {0, 0, 0, 0},          {-4926, 11893, -11893, 4926},
                              {-6270, 6270, 6270, -6270},   {-4176, -1730, 1730, 4176}};
    constexpr int c4[8][2] = {{0, 0}, {29692, -29692}, {0, 0}, {-10426, 10426}, {0, 0}, {6967, -6967}, {0, 0}, {-5906, 5906}};
    return R == 2 ? c2[k][m & 3] : c4[k][m & 1];
}

template <int R>
__device__ __forceinline__ void reduced_block(const int16_t *__restrict__ coef, const uint16_t *__restrict__ q,
                                              uint8_t *__restrict__ dst, int pitch) {
    constexpr int N = 8 / R, L = R == 2 ? 1 : 2;
    int a[8][8], cw[32];
    load_block(coef, cw);
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const int4 qw = reinterpret_cast<const int4 *>(q)[r];
        const int qq[4] = {qw.x, qw.y, qw.z, qw.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            a[r][2 * k] = coef_at(cw, r * 8 + 2 * k) * (qq[k] & 0xffff);
            a[r][2 * k + 1] = coef_at(cw, r * 8 + 2 * k + 1) * (int)((uint32_t)qq[k] >> 16);
        }
    }
    int ws[8][N]; // [column of the block][row of the result]
#pragma unroll
    for (int col = 0; col < 8; col++)
#pragma unroll
        for (int m = 0; m < N; m++) {
            int acc = a[0][col] * (1 << (13 + L));
#pragma unroll
            for (int k = 1; k < 8; k++) acc += a[k][col] * reduced_constant<R>(k, m);
            ws[col][m] = (acc + (1 << (11 + L - 1))) >> (11 + L);
        }
#pragma unroll
    for (int row = 0; row < N; row++) {
        uint32_t packed = 0;
#pragma unroll
        for (int m = 0; m < N; m++) {
            int acc = ws[0][row] * (1 << (13 + L));
#pragma unroll
            for (int k = 1; k < 8; k++) acc += ws[k][row] * reduced_constant<R>(k, m);
            const int v = min(255, max(0, ((acc + (1 << (18 + L - 1))) >> (18 + L)) + 128));
            packed |= (uint32_t)v << (8 * m);
        }
        if (N == 4)
            *reinterpret_cast<uint32_t *>(dst + (size_t)row * pitch) = packed;
        else
            *reinterpret_cast<uint16_t *>(dst + (size_t)row * pitch) = (uint16_t)packed;
    }
}

__device__ __forceinline__ int find_image(const ImageDesc *descs, const int32_t *list, int n_list,
                                          uint32_t blk) {
    // largest k with descs[list[k]].block_base <= blk (block_base ascends along the list)
    int lo = 0, hi = n_list - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (descs[list[mid]].block_base <= blk)
            lo = mid;
        else
            hi = mid - 1;
    }
    return list[lo];
}

__global__ void __launch_bounds__(128)
idct_kernel(const ImageDesc *__restrict__ descs, const int32_t *__restrict__ list, int n_list,
            uint32_t total_blocks, const MultTable *__restrict__ mult,
            const int16_t *__restrict__ coef, uint8_t *__restrict__ planes) {
    const uint32_t gb = blockIdx.x * blockDim.x + threadIdx.x;
    if (gb >= total_blocks) return;
    const ImageDesc &d = descs[find_image(descs, list, n_list, gb)];
    if (d.host_status != 0) return;
    const uint32_t b = gb - d.block_base;
    if (b >= d.nblocks) return;
    const int luma = d.hs * d.vs;
    const uint32_t mcu = b / d.bpm;
    const int slot = (int)(b - mcu * d.bpm);
    const int my = mcu / d.mcus_x, mx = mcu - my * d.mcus_x;
    if (my < d.idct_row0 || mx < d.idct_col0 || mx >= d.idct_col1) return; // outside the crop's reach
    int comp, bx, by, plane_w, bs;
    if (d.ncomp == 1 || slot < luma) {
        comp = 0;
        const int v = slot / d.hs, h = slot - v * d.hs;
        bx = mx * d.hs + h;
        by = my * d.vs + v;
        bs = d.bs_luma;
        plane_w = d.mcus_x * d.hs * bs;
    } else {
        comp = slot - luma + 1;
        bx = mx;
        by = my;
        bs = d.bs_chroma;
        plane_w = d.mcus_x * bs;
    }
    if (bs != 8) { // scaled decode: this block becomes bs x bs samples
        const MultTable &mt = mult[d.q_tab[comp]];
        const int16_t *cb = coef + (size_t)gb * 64;
        uint8_t *dst = planes + d.plane_off[comp] + (size_t)(by * bs) * plane_w + bx * bs;
        if (bs == 4) {
            reduced_block<2>(cb, mt.q, dst, plane_w);
        } else if (bs == 2) {
            reduced_block<4>(cb, mt.q, dst, plane_w);
        } else {
            const int a0 = (int)cb[0] * (int)mt.q[0];
            dst[0] = (uint8_t)min(255, max(0, ((a0 + 4) >> 3) + 128));
        }
        return;
    }
    const int16_t *q = mult[d.q_tab[comp]].m;
    int v[8][8], cw[32];
    load_block(coef + (size_t)gb * 64, cw);
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const int4 qw = reinterpret_cast<const int4 *>(q)[r];
        const int qq[4] = {qw.x, qw.y, qw.z, qw.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            v[r][2 * k] = w16(coef_at(cw, r * 8 + 2 * k) * (int)(short)(qq[k] & 0xffff));
            v[r][2 * k + 1] = w16(coef_at(cw, r * 8 + 2 * k + 1) * (qq[k] >> 16));
        }
    }
#pragma unroll
    for (int c = 0; c < 8; c++)
        idct8(v[0][c], v[1][c], v[2][c], v[3][c], v[4][c], v[5][c], v[6][c], v[7][c]);
    uint8_t *dst = planes + d.plane_off[comp] + (size_t)(by * 8) * plane_w + bx * 8;
#pragma unroll
    for (int r = 0; r < 8; r++) {
        idct8(v[r][0], v[r][1], v[r][2], v[r][3], v[r][4], v[r][5], v[r][6], v[r][7]);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            int s = v[r][c] >> 5;
            s = min(127, max(-128, s)) + 128;
            if (c < 4)
                lo |= (uint32_t)s << (8 * c);
            else
                hi |= (uint32_t)s << (8 * (c - 4));
        }
        *reinterpret_cast<uint2 *>(dst + (size_t)r * plane_w) = make_uint2(lo, hi);
    }
}

// ------------------------------------------------------------------------------------------

__device__ __forceinline__ int chroma_sample(const uint8_t *__restrict__ p, int W, int real_w,
                                             int real_h, int hs, int vs, int x, int y) {
    if (hs == 1) return p[(size_t)y * W + x];
    const int cx = x >> 1, cy = vs == 2 ? (y >> 1) : y;
    const uint8_t *row = p + (size_t)cy * W;
    if (real_w < 3) return row[cx];
    if (vs == 1) {
        const int cur = row[cx];
        if ((x & 1) == 0) return cx == 0 ? cur : (3 * cur + row[cx - 1] + 1) >> 2;
        return cx == real_w - 1 ? cur : (3 * cur + row[cx + 1] + 2) >> 2;
    }
    int ny = (y & 1) ? cy + 1 : cy - 1;
    ny = max(0, min(real_h - 1, ny));
    const uint8_t *far = p + (size_t)ny * W;
    const int cur = 3 * row[cx] + far[cx];
    if ((x & 1) == 0) {
        if (cx == 0) return (cur * 4 + 8) >> 4;
        return (cur * 3 + 3 * row[cx - 1] + far[cx - 1] + 8) >> 4;
    }
    if (cx == real_w - 1) return (cur * 4 + 7) >> 4;
    return (cur * 3 + 3 * row[cx + 1] + far[cx + 1] + 7) >> 4;
}

void launch_idct(const ImageDesc *descs, const int32_t *list, int n_list, uint32_t total_blocks,
                 const MultTable *mult, const int16_t *coef, uint8_t *planes, cudaStream_t stream) {
    if (total_blocks == 0) return;
    idct_kernel<<<(total_blocks + 127) / 128, 128, 0, stream>>>(descs, list, n_list, total_blocks, mult,
                                                               coef, planes);
}

// 16.16 fixed-point YCbCr -> RGB of libjpeg (jdcolor.c's tables written out), one pixel.
__device__ __forceinline__ uint32_t ycc_to_rgb(int lum, int cb, int cr) {
    cb -= 128;
    cr -= 128;
    const int r = lum + ((91881 * cr + 32768) >> 16);
    const int g = lum + ((-22554 * cb - 46802 * cr + 32768) >> 16);
    const int b = lum + ((116130 * cb + 32768) >> 16);
    return (uint32_t)min(255, max(0, r)) | (uint32_t)min(255, max(0, g)) << 8 | (uint32_t)min(255, max(0, b)) << 16;
}

// Stores four RGB pixels (12 bytes, the fourth byte of each word of `px` unused) at `o`: three
// words when the address allows and all four pixels exist, else the first `count` pixels by bytes.
__device__ __forceinline__ void store_rgb4(uint8_t *o, const uint32_t *px, int count, bool words) {
    if (words && count == 4) {
        uint32_t *w = reinterpret_cast<uint32_t *>(o);
        w[0] = px[0] | px[1] << 24;
        w[1] = px[1] >> 8 | px[2] << 16;
        w[2] = px[2] >> 16 | px[3] << 8;
    } else {
        for (int k = 0; k < count; k++) {
            o[3 * k] = (uint8_t)px[k];
            o[3 * k + 1] = (uint8_t)(px[k] >> 8);
            o[3 * k + 2] = (uint8_t)(px[k] >> 16);
        }
    }
}

// The box of pixels to convert: the crop box when the batch has one (valid), else the image.
__device__ __forceinline__ void convert_box(const int32_t *params, int n_params, int img, int W, int H, int &x0,
                                            int &y0, int &x1, int &y1) {
    x0 = 0, y0 = 0, x1 = W, y1 = H;
    if (params) {
        const int32_t *p = params + (size_t)img * n_params;
        if (p[2] > 0 && p[3] > 0 && p[0] >= 0 && p[1] >= 0 && p[0] + p[2] <= H && p[1] + p[3] <= W) {
            y0 = p[0];
            x0 = p[1];
            y1 = p[0] + p[2];
            x1 = p[1] + p[3];
        }
    }
}

// 4:2:0 images: one thread per pair of chroma samples = 4 x 2 output pixels.  The triangle filter
// of the eight pixels reads a 3 x 4 chroma neighbourhood (image edges replicate, which is what the
// filter's edge formulas amount to): its vertical blends are computed once per column, the luma
// samples arrive as one word per row and the pixels leave as three words per row (the rows of the
// RGB scratch start on 16-byte boundaries and a thread's first pixel is a multiple of four).
// Only the chroma cells the crop box touches are converted.
__global__ void __launch_bounds__(256)
color_quad_kernel(const ImageDesc *__restrict__ descs, const int32_t *__restrict__ list,
                  const uint2 *__restrict__ tiles, const uint8_t *__restrict__ planes, uint8_t *__restrict__ rgb,
                  const int32_t *__restrict__ params, int n_params) {
    // which sample and which tile of 64 x 8 chroma samples of its box: from the batch's tile table
    // (one CTA per tile that exists), or, without a table, from a grid that covers the largest box
    int img, tile_x, tile_y;
    if (tiles) {
        const uint2 t = tiles[blockIdx.x];
        img = (int)t.x;
        tile_x = (int)(t.y & 0xffff);
        tile_y = (int)(t.y >> 16);
    } else {
        img = list[blockIdx.z];
        tile_x = blockIdx.x;
        tile_y = blockIdx.y;
    }
    const ImageDesc &d = descs[img];
    if (d.host_status != 0 || d.ncomp != 3 || d.hs != 2 || d.vs != 2 || d.scale_shift != 0) return;
    const int W = d.width, H = d.height;
    const int real_w = (W + 1) >> 1, real_h = (H + 1) >> 1;
    if (real_w < 3) return; // too narrow for the filter: the per-pixel kernel replicates
    int x0, y0, x1, y1;
    convert_box(params, n_params, img, W, H, x0, y0, x1, y1);
    const int cx = ((x0 >> 1) & ~1) + 2 * (tile_x * 32 + threadIdx.x); // even: pixel 2 * cx is a multiple of 4
    const int cy = (y0 >> 1) + tile_y * 8 + threadIdx.y;
    if (cx > ((x1 - 1) >> 1) || cy > ((y1 - 1) >> 1)) return;
    const int yw = d.mcus_x * 16, cw = d.mcus_x * 8;
    const int xl = max(cx - 1, 0), xr = min(cx + 2, real_w - 1);
    const bool second = cx + 1 <= real_w - 1; // the pair's second column exists
    const int yu = max(cy - 1, 0), yd = min(cy + 1, real_h - 1);
    // chroma of the 4 x 2 pixels: [Cb, Cr][row][pixel]
    int cval[2][2][4];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        const uint8_t *P = planes + d.plane_off[1 + k];
        const uint8_t *ru = P + (size_t)yu * cw, *rc = P + (size_t)cy * cw, *rd = P + (size_t)yd * cw;
        int up[4], dn[4]; // columns cx - 1 .. cx + 2 blended towards the row above / below
        {
            const int c = rc[xl];
            up[0] = 3 * c + ru[xl];
            dn[0] = 3 * c + rd[xl];
        }
        {
            const uint32_t u = *reinterpret_cast<const uint16_t *>(ru + cx), c = *reinterpret_cast<const uint16_t *>(rc + cx),
                           w = *reinterpret_cast<const uint16_t *>(rd + cx);
            up[1] = 3 * (int)(c & 255) + (int)(u & 255);
            dn[1] = 3 * (int)(c & 255) + (int)(w & 255);
            up[2] = second ? 3 * (int)(c >> 8) + (int)(u >> 8) : up[1];
            dn[2] = second ? 3 * (int)(c >> 8) + (int)(w >> 8) : dn[1];
        }
        {
            const int c = rc[xr];
            up[3] = second ? 3 * c + ru[xr] : up[1];
            dn[3] = second ? 3 * c + rd[xr] : dn[1];
        }
#pragma unroll
        for (int j = 0; j < 2; j++) { // the pair's columns
            cval[k][0][2 * j] = (3 * up[1 + j] + up[j] + 8) >> 4;
            cval[k][0][2 * j + 1] = (3 * up[1 + j] + up[2 + j] + 7) >> 4;
            cval[k][1][2 * j] = (3 * dn[1 + j] + dn[j] + 8) >> 4;
            cval[k][1][2 * j + 1] = (3 * dn[1 + j] + dn[2 + j] + 7) >> 4;
        }
    }
    const uint8_t *Y = planes + d.plane_off[0];
    uint8_t *out = rgb + d.rgb_off;
    const int x = 2 * cx, count = min(4, W - x);
    const bool words = ((reinterpret_cast<uintptr_t>(out) | d.rgb_pitch) & 3) == 0;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int y = 2 * cy + r;
        if (y >= H) continue;
        const uint32_t lum = *reinterpret_cast<const uint32_t *>(Y + (size_t)y * yw + x);
        uint32_t px[4];
#pragma unroll
        for (int q = 0; q < 4; q++) px[q] = ycc_to_rgb((lum >> (8 * q)) & 255, cval[0][r][q], cval[1][r][q]);
        store_rgb4(out + (size_t)y * d.rgb_pitch + (size_t)x * 3, px, count, words);
    }
}

// 4:4:4 images, and images decoded at reduced scale (whose chroma blocks were inverted to the luma
// resolution): no upsampling, one thread per four pixels of a row of the crop box (one word of each
// plane in, three words out), every thread walking a column strip so that the grid stays small
// for very large images.
__global__ void __launch_bounds__(256)
color_444_kernel(const ImageDesc *__restrict__ descs, const int32_t *__restrict__ list,
                 const uint8_t *__restrict__ planes, uint8_t *__restrict__ rgb,
                 const int32_t *__restrict__ params, int n_params) {
    const int img = list[blockIdx.z];
    const ImageDesc &d = descs[img];
    if (d.host_status != 0 || d.ncomp != 3 || !(d.scale_shift != 0 || (d.hs == 1 && d.vs == 1))) return;
    const int W = d.dec_width, H = d.dec_height;
    int x0, y0, x1, y1;
    convert_box(params, n_params, img, W, H, x0, y0, x1, y1);
    const int pw = d.mcus_x * d.hs * d.bs_luma; // = the chroma planes' pitch: all planes have one resolution here
    const uint8_t *Y = planes + d.plane_off[0], *Cb = planes + d.plane_off[1], *Cr = planes + d.plane_off[2];
    uint8_t *out = rgb + d.rgb_off;
    const int x = (x0 & ~3) + 4 * (blockIdx.x * 32 + threadIdx.x);
    if (x >= x1) return;
    const int count = min(4, W - x);
    // a plane's pitch is a multiple of 8 only at full scale; reduced planes may be narrower
    const bool words_in = ((pw | (int)(d.plane_off[0] | d.plane_off[1] | d.plane_off[2])) & 3) == 0;
    const bool words_out = ((reinterpret_cast<uintptr_t>(out) | d.rgb_pitch) & 3) == 0;
    for (int y = y0 + blockIdx.y * 8 + threadIdx.y; y < y1; y += gridDim.y * 8) {
        const size_t s = (size_t)y * pw + x;
        uint32_t lum = 0, cb = 0, cr = 0;
        if (words_in) {
            lum = *reinterpret_cast<const uint32_t *>(Y + s);
            cb = *reinterpret_cast<const uint32_t *>(Cb + s);
            cr = *reinterpret_cast<const uint32_t *>(Cr + s);
        } else {
            for (int q = 0; q < count; q++) {
                lum |= (uint32_t)Y[s + q] << (8 * q);
                cb |= (uint32_t)Cb[s + q] << (8 * q);
                cr |= (uint32_t)Cr[s + q] << (8 * q);
            }
        }
        uint32_t px[4];
#pragma unroll
        for (int q = 0; q < 4; q++)
            px[q] = ycc_to_rgb((lum >> (8 * q)) & 255, (cb >> (8 * q)) & 255, (cr >> (8 * q)) & 255);
        store_rgb4(out + (size_t)y * d.rgb_pitch + (size_t)x * 3, px, count, words_out);
    }
}

// Per-pixel kernel for everything the kernels above leave out (4:2:2, greyscale, 4:2:0 images
// narrower than the triangle filter).
__global__ void __launch_bounds__(256)
color_other_kernel(const ImageDesc *__restrict__ descs, const int32_t *__restrict__ list,
                   const uint8_t *__restrict__ planes, uint8_t *__restrict__ rgb) {
    const ImageDesc &d = descs[list[blockIdx.y]];
    if (d.host_status != 0) return;
    const int W = d.width, H = d.height;
    const int real_w = (W + d.hs - 1) / d.hs, real_h = (H + d.vs - 1) / d.vs;
    if (d.scale_shift != 0) return;                                      // equal-resolution kernel's
    if (d.ncomp == 3 && d.hs == 2 && d.vs == 2 && real_w >= 3) return; // quad kernel's
    if (d.ncomp == 3 && d.hs == 1 && d.vs == 1) return;                  // 4:4:4 kernel's
    const int npix = W * H;
    const int yw = d.mcus_x * d.hs * 8, cw = d.mcus_x * 8;
    const uint8_t *Y = planes + d.plane_off[0];
    const uint8_t *Cb = planes + d.plane_off[1];
    const uint8_t *Cr = planes + d.plane_off[2];
    uint8_t *out = rgb + d.rgb_off;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < npix; i += gridDim.x * blockDim.x) {
        const int y = i / W, x = i - y * W;
        const int lum = Y[(size_t)y * yw + x];
        int r = lum, g = lum, b = lum;
        if (d.ncomp == 3) {
            const int cb = chroma_sample(Cb, cw, real_w, real_h, d.hs, d.vs, x, y) - 128;
            const int cr = chroma_sample(Cr, cw, real_w, real_h, d.hs, d.vs, x, y) - 128;
            r = lum + ((91881 * cr + 32768) >> 16);
            g = lum + ((-22554 * cb - 46802 * cr + 32768) >> 16);
            b = lum + ((116130 * cb + 32768) >> 16);
        }
        uint8_t *o = out + (size_t)y * d.rgb_pitch + (size_t)x * 3;
        o[0] = (uint8_t)min(255, max(0, r));
        o[1] = (uint8_t)min(255, max(0, g));
        o[2] = (uint8_t)min(255, max(0, b));
    }
}

void launch_color(const ImageDesc *descs, const int32_t *list, int n_list, int n_quad, int n_444, int n_other,
                  int max_w, int max_h, const uint2 *quad_tiles, int n_quad_tiles, const uint8_t *planes, uint8_t *rgb, const int32_t *crop_params,
                  int n_params, cudaStream_t stream) {
    if (n_list == 0) return;
    if (n_444 > 0) {
        int gy = (max_h + 7) / 8;
        if (gy > 64) gy = 64;
        dim3 grid(((max_w + 3) / 4 + 1 + 31) / 32, gy, n_list); // + 1: a box starts up to 3 pixels into its first group
        color_444_kernel<<<grid, dim3(32, 8), 0, stream>>>(descs, list, planes, rgb, crop_params, n_params);
    }
    if (n_quad > 0 && quad_tiles != nullptr) {
        if (n_quad_tiles > 0)
            color_quad_kernel<<<n_quad_tiles, dim3(32, 8), 0, stream>>>(descs, list, quad_tiles, planes, rgb, crop_params,
                                                                        n_params);
    } else if (n_quad > 0) {
        dim3 grid((((max_w + 1) / 2 + 1) / 2 + 1 + 31) / 32, ((max_h + 1) / 2 + 7) / 8, n_list); // pairs of chroma columns
        color_quad_kernel<<<grid, dim3(32, 8), 0, stream>>>(descs, list, nullptr, planes, rgb, crop_params, n_params);
    }
    if (n_other > 0) {
        int bx = (max_w * max_h + 256 * 4 - 1) / (256 * 4);
        bx = bx < 1 ? 1 : (bx > 1024 ? 1024 : bx);
        color_other_kernel<<<dim3(bx, n_list), 256, 0, stream>>>(descs, list, planes, rgb);
    }
}

} // namespace ffcvb
