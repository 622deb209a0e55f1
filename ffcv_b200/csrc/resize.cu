// Fused crop + INTER_AREA resize + flip / translate / cutout + lookup-table normalise (sm_100a).
//
// Replaces, in one pass over the output, the chain the reference runs as separate CPU loops:
//   cv::resize(roi, dst, INTER_AREA)      libffcv/libffcv.cpp:33-42 (from rgb_image.py:205-208)
//   RandomHorizontalFlip                  ffcv/transforms/flip.py:31-39
//   RandomTranslate                       ffcv/transforms/translate.py:35-44
//   Cutout                                ffcv/transforms/cutout.py:36-46
//   NormalizeImage (256x3 table gather)   ffcv/transforms/normalize.py:58-109
// Every output pixel is traced backwards through the augmentations to either a fill colour or a
// pixel of the resized crop, whose value is computed with OpenCV's INTER_AREA arithmetic:
//   equal size -> copy; integer factors -> box sum ((s+2)>>2 for 2x2, else
//   round-half-even(float(s) * float(1/area))); both factors >= 1 -> separable fractional
//   coverage accumulated in fp32 in source order (no FMA contraction); any factor < 1 -> 2-tap
//   interpolation on both axes with 11-bit fixed-point weights.
// Byte work bound by instruction issue: a few CTAs per sample, each producing every k-th band of
// output rows; tap positions and weights are computed once per CTA into shared memory and serve all
// its bands; the source rows a band reads are staged in shared memory by asynchronous 16-byte
// copies when they fit (taps straight from global memory otherwise); every band's normalised tile
// is assembled in shared memory and leaves with coalesced 16-byte stores.  In the fractional
// shrinking and the enlarging regime a thread owns an output column for a run of rows, so that
// what a source row contributes (its horizontal sums, its interpolated values) is shared by the
// output rows that touch it.
#include <float.h>

#include <type_traits>

#include "kernels.h"

namespace ffcvb {

enum { kOpFlip = 1, kOpTranslate = 2, kOpCutout = 3 };
enum { kOutU8 = 0, kOutF16Nhwc = 1, kOutF16Nchw = 2, kOutF32Nhwc = 3, kOutF32Nchw = 4 };
enum { kCopy = 0, kInteger = 1, kArea = 2, kLinear = 3 };
constexpr int kMaxWindowRows = 96; // source rows of a band that can be staged in shared memory

struct AreaTaps {
    int first, n;
    float wl, wm, wr;
    bool has_l, has_r;
};

// a / b correctly rounded, given the correctly rounded 1 / b: the product with the reciprocal is
// within 1.5 ulp, a first remainder step makes it faithful, a second one correctly rounded
// (Markstein); three double-precision divisions per tap would otherwise dominate the CTA's set-up.
__device__ __forceinline__ double quotient(double a, double b, double inv_b) {
    double q = a * inv_b;
    q = fma(fma(-b, q, a), inv_b, q);
    return fma(fma(-b, q, a), inv_b, q);
}

// Source cells covering destination cell d of an axis shrunk by `scale` (>= 1).
__device__ __forceinline__ AreaTaps area_taps(int d, int ssize, double scale) {
    AreaTaps t;
    const double f1 = d * scale, f2 = f1 + scale;
    const double cell = fmin(scale, ssize - f1);
    int s1 = (int)ceil(f1), s2 = (int)floor(f2);
    s2 = min(s2, ssize - 1);
    s1 = min(s1, s2);
    t.has_l = (s1 - f1) > 1e-3;
    t.has_r = (f2 - s2) > 1e-3;
    const double inv_cell = 1.0 / cell;
    t.wl = (float)quotient(s1 - f1, cell, inv_cell);
    t.wm = (float)inv_cell;
    t.wr = (float)quotient(fmin(fmin(f2 - s2, 1.0), cell), cell, inv_cell);
    t.first = t.has_l ? s1 - 1 : s1;
    t.n = (t.has_l ? 1 : 0) + (s2 - s1) + (t.has_r ? 1 : 0);
    return t;
}

// Two-tap position and 11-bit weights of destination index d when some axis is enlarged.
__device__ __forceinline__ void linear_taps(int d, int ssize, double inv, double scale, bool clamp_last,
                                            int &s, int &w0, int &w1) {
    s = (int)floor(d * scale);
    float f = (float)((d + 1) - (s + 1) * inv);
    f = f <= 0.f ? 0.f : f - floorf(f);
    if (clamp_last && s >= ssize - 1) {
        f = 0.f;
        s = ssize - 1;
    }
    w0 = min(32767, __float2int_rn(__fmul_rn(__fsub_rn(1.f, f), 2048.f)));
    w1 = min(32767, __float2int_rn(__fmul_rn(f, 2048.f)));
}

__device__ __forceinline__ int sat_round(float v) { return min(255, max(0, __float2int_rn(v))); }

// uint8 -> float without the conversion pipe: 2^23 + v is representable; the 2^23 is taken off again
// inside the multiplication, fma(2^23 + v, w, -2^23 * w)
__device__ __forceinline__ float u8biased(uint32_t v) { return __uint_as_float(0x4B000000u | v); }

// 16 bytes from global to shared memory without passing through registers (L2 only: each source
// byte is staged once); copies_wait() returns when this thread's copies have landed.
__device__ __forceinline__ void copy16_async(uint32_t dst_shared, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_shared), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_wait() {
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Per-axis tap tables in shared memory, computed once per CTA (double-precision position
// arithmetic as OpenCV does it, then only fp32 / integer work per pixel).
struct TapTables {
    int *first;  // first source index (area) / source index (linear)
    int *count;  // area: taps | has_l << 16 | has_r << 17; linear: w0 << 16 | w1
    float *wl, *wm, *wr;
};

__device__ __forceinline__ void fill_taps(const TapTables &t, int k, int d, int regime, int ssize, double inv,
                                          double scale, bool clamp_last) {
    if (regime == kArea) {
        const AreaTaps a = area_taps(d, ssize, scale);
        t.first[k] = a.first;
        t.count[k] = a.n | (a.has_l ? 1 << 16 : 0) | (a.has_r ? 1 << 17 : 0);
        t.wl[k] = a.wl;
        t.wm[k] = a.wm;
        t.wr[k] = a.wr;
    } else if (regime == kLinear) {
        int s, w0, w1;
        linear_taps(d, ssize, inv, scale, clamp_last, s, w0, w1);
        if (clamp_last && s + 1 >= ssize) {
            w0 = 2048;
            w1 = 0;
        }
        t.first[k] = s;
        t.count[k] = (w0 << 16) | w1;
    }
}

// Scaling regime of a crop of ch x cw pixels resized to out_h x out_w, as OpenCV decides it.
struct Scaling {
    int regime, isx, isy;
    double inv_x, inv_y, sc_x, sc_y;
};
__device__ __forceinline__ Scaling scaling_of(int ch, int cw, int out_h, int out_w) {
    Scaling s{kCopy, 1, 1, 1, 1, 1, 1};
    if (ch != out_h || cw != out_w) {
        s.inv_x = (double)out_w / cw;
        s.inv_y = (double)out_h / ch;
        s.sc_x = 1.0 / s.inv_x;
        s.sc_y = 1.0 / s.inv_y;
        if (s.sc_x >= 1 && s.sc_y >= 1) {
            s.isx = __double2int_rn(s.sc_x);
            s.isy = __double2int_rn(s.sc_y);
            s.regime = (fabs(s.sc_x - s.isx) < DBL_EPSILON && fabs(s.sc_y - s.isy) < DBL_EPSILON) ? kInteger : kArea;
        } else {
            s.regime = kLinear;
        }
    }
    return s;
}

template <typename OutT>
__global__ void __launch_bounds__(256)
resize_augment_kernel(const __grid_constant__ ResizeSource src, const int32_t *__restrict__ params, int n_params,
                      const __grid_constant__ OpList ops,
                      int resize, int out_h, int out_w, int band_rows, int groups, int planar, int win_bytes,
                      const OutT *__restrict__ lut, OutT *__restrict__ out,
                      const int32_t *__restrict__ status) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    constexpr bool kU8 = sizeof(OutT) == 1;
    // shared layout: [out tile][lut][x taps (5 arrays of out_w)][y taps (5 arrays of out_h)]
    //                [start of each window row][window of source rows (win_bytes)]
    int band0 = 0, rows = 0; // the band of output rows being produced (see the loop below)
    const int tile_elems = band_rows * out_w * 3;
    OutT *s_out = reinterpret_cast<OutT *>(s_raw);
    size_t off = ((size_t)tile_elems * sizeof(OutT) + 15) & ~(size_t)15;
    OutT *s_lut = reinterpret_cast<OutT *>(s_raw + off);
    off += (768 * sizeof(OutT) + 15) & ~(size_t)15;
    // y taps are indexed by the row of the resized crop (a translation can move a band anywhere)
    int *ibase = reinterpret_cast<int *>(s_raw + off);
    TapTables tx{ibase, ibase + out_w, reinterpret_cast<float *>(ibase + 2 * out_w),
                 reinterpret_cast<float *>(ibase + 3 * out_w), reinterpret_cast<float *>(ibase + 4 * out_w)};
    int *jbase = ibase + 5 * out_w;
    TapTables ty{jbase, jbase + out_h, reinterpret_cast<float *>(jbase + 2 * out_h),
                 reinterpret_cast<float *>(jbase + 3 * out_h), reinterpret_cast<float *>(jbase + 4 * out_h)};
    int *s_rowoff = jbase + 5 * out_h;
    unsigned char *s_win =
        s_raw + ((off + sizeof(int) * (5 * ((size_t)out_w + out_h) + kMaxWindowRows) + 15) & ~(size_t)15);

    const int i = blockIdx.y;
    if (!kU8)
        for (int k = threadIdx.x; k < 768; k += blockDim.x) s_lut[(k % 3) * 256 + k / 3] = lut[k]; // per channel

    // ---- where the sample's pixels are
    const uint8_t *base;
    int stride, row0 = 0, col0 = 0, img_h, img_w;
    // rows of a gathered crop box start at their source alignment inside their slot (raw_skew)
    uint32_t skew_base = 0, skew_pitch = 0;
    bool skew = false;
    bool ok = true;
    if (src.descs) {
        const ImageDesc &d = src.descs[i];
        img_h = d.dec_height; // the decoded size: smaller than the stored one after a scaled decode
        img_w = d.dec_width;
        stride = (int)d.rgb_pitch;
        if (d.mode == 1) {
            base = src.blob + d.payload_off;
            row0 = d.row0;
            col0 = d.col0;
            stride = (int)d.raw_pitch;
            ok = d.host_status == 0;
            if (d.raw_skew) {
                skew = true;
                skew_base = (uint32_t)(d.src_addr & 15);
                skew_pitch = (uint32_t)d.width * 3;
            }
        } else {
            base = src.rgb + d.rgb_off;
            ok = d.host_status == 0 && (status == nullptr || status[i] == 0);
        }
    } else {
        img_h = src.uniform_h;
        img_w = src.uniform_w;
        stride = img_w * 3;
        base = src.uniform + (size_t)i * img_h * stride;
    }
    const int32_t *prm = params + (size_t)i * n_params;
    int ci = 0, cj = 0, ch = out_h, cw = out_w;
    if (resize) {
        ci = prm[0];
        cj = prm[1];
        ch = prm[2];
        cw = prm[3];
        ok = ok && ch > 0 && cw > 0 && ci >= 0 && cj >= 0 && ci + ch <= img_h && cj + cw <= img_w;
    } else {
        ok = ok && img_h == out_h && img_w == out_w;
    }
    // With flips only (or no augmentation) nothing is ever filled and the column an output column
    // comes from does not depend on the row: the trace is done once per column.
    bool flips_only = true;
    for (int k = 0; k < ops.n_ops; k++) flips_only = flips_only && ops.type[k] == kOpFlip;
    bool rows_in_place = true; // no translation: output row y comes from row y of the resized crop
    for (int k = 0; k < ops.n_ops; k++) rows_in_place = rows_in_place && ops.type[k] != kOpTranslate;

    // The scale factors (four double-precision divisions) are worked out by one thread.
    __shared__ Scaling s_scaling;
    if (threadIdx.x == 0 && ok) s_scaling = scaling_of(ch, cw, out_h, out_w);
    __syncthreads();
    int regime = kCopy, isx = 1, isy = 1;
    const int nbands = (out_h + band_rows - 1) / band_rows;
    if (ok) {
        const Scaling &sc = s_scaling;
        regime = sc.regime;
        isx = sc.isx;
        isy = sc.isy;
        if (regime == kArea || regime == kLinear) {
            // x taps of every column; y taps of the rows this CTA produces (of all rows when a
            // translation can move a band anywhere)
            const int my_bands = rows_in_place ? (nbands - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : nbands;
            const int band_step = rows_in_place ? (int)gridDim.x : 1, band_first = rows_in_place ? (int)blockIdx.x : 0;
            for (int e = threadIdx.x; e < out_w + my_bands * band_rows; e += blockDim.x) {
                if (e < out_w) {
                    fill_taps(tx, e, e, regime, cw, sc.inv_x, sc.sc_x, true);
                } else {
                    const int k = e - out_w, b = k / band_rows;
                    const int y = (band_first + b * band_step) * band_rows + (k - b * band_rows);
                    if (y < out_h) fill_taps(ty, y, y, regime, ch, sc.inv_y, sc.sc_y, false);
                }
            }
        }
    }
    __syncthreads();

    const int roff = ci - row0, coff = (cj - col0) * 3;
    auto row_ptr = [&](int y) -> const uint8_t * { // first pixel of row y of the crop
        const int rr = roff + y;
        const uint8_t *p = base + (ptrdiff_t)rr * stride + coff;
        if (skew) p += (skew_base + (uint32_t)rr * skew_pitch) & 15u;
        return p;
    };
    int npix = 0;
    const uint32_t inv_w = (uint32_t)((0x100000000ull + out_w - 1) / out_w); // pix / out_w for pix < 2^16
    // Traces an output pixel back through the augmentations: either a fill colour, or the position
    // (y, x) of a pixel of the resized crop.
    auto trace = [&](int oy, int ox, int &y, int &x, int *val) -> bool {
        y = oy;
        x = ox;
        bool filled = false;
        for (int k = ops.n_ops - 1; k >= 0 && !filled; k--) {
            const int a = prm[4 + 2 * k], b = prm[5 + 2 * k];
            const int type = ops.type[k], arg = ops.arg[k];
            if (type == kOpCutout) {
                filled = y >= a && y < a + arg && x >= b && x < b + arg;
            } else if (type == kOpTranslate) {
                y += a - arg;
                x += b - arg;
                filled = y < 0 || y >= out_h || x < 0 || x >= out_w;
            } else if (type == kOpFlip) {
                if (a) x = out_w - 1 - x;
            }
            if (filled) {
                val[0] = ops.fill[k][0];
                val[1] = ops.fill[k][1];
                val[2] = ops.fill[k][2];
            }
        }
        return filled;
    };
    // normalise (table gather, one 256-entry table per channel) into the shared tile, in final
    // memory order: element = pix * pix_step + c * chan_step
    int pix_step = 3, chan_step = 1;
    auto emit = [&](int pix, const int *val) {
        OutT *o = s_out + pix * pix_step;
#pragma unroll
        for (int c = 0; c < 3; c++) {
            if constexpr (kU8)
                o[c * chan_step] = (OutT)val[c];
            else
                o[c * chan_step] = s_lut[c * 256 + val[c]];
        }
    };
    bool mirrored = false;
    if (flips_only)
        for (int k = 0; k < ops.n_ops; k++) mirrored ^= prm[4 + 2 * k] != 0;
    // A CTA produces every gridDim.x-th band of its image: what was set up above (descriptor, tap
    // tables, lookup table) serves all of them.
    for (int band = blockIdx.x; band < nbands; band += gridDim.x) {
    band0 = band * band_rows;
    rows = min(band_rows, out_h - band0);
    npix = rows * out_w;
    pix_step = planar ? 1 : 3;
    chan_step = planar ? npix : 1;
    // The source rows this band reads are staged in shared memory first, when they fit: whole
    // 16-byte words, many in flight per thread, instead of byte loads that each wait for a first
    // touch of their sector in L2 or HBM (asynchronous copies, no registers in between).  The
    // window keeps every row at its 16-byte phase.
    bool staged = false;
    int win_lo = 0;
    if (win_bytes > 0 && rows_in_place && ok && (regime == kArea || regime == kLinear)) {
        const int yb = band0 + rows - 1;
        int hi;
        if (regime == kArea) {
            win_lo = ty.first[band0];
            hi = ty.first[yb] + (ty.count[yb] & 0xffff) - 1;
        } else {
            win_lo = min(ty.first[band0], ch - 1);
            hi = min(ty.first[yb] + 1, ch - 1);
        }
        const int nrows = hi - win_lo + 1, pitch = ((cw * 3 + 15) & ~15) + 16;
        if (nrows <= kMaxWindowRows && nrows * pitch <= win_bytes) {
            staged = true;
            const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            for (int row = warp; row < nrows; row += blockDim.x >> 5) {
                const uint8_t *p = row_ptr(win_lo + row);
                const uint32_t phase = (uint32_t)(reinterpret_cast<uintptr_t>(p) & 15);
                const uint4 *g = reinterpret_cast<const uint4 *>(p - phase);
                const uint32_t d = (uint32_t)__cvta_generic_to_shared(s_win + row * pitch);
                const int chunks = (int)(phase + cw * 3 + 15) >> 4;
                for (int k = lane; k < chunks; k += 32) copy16_async(d + 16u * k, g + k);
                if (lane == 0) s_rowoff[row] = row * pitch + (int)phase;
            }
            copies_wait();
            __syncthreads();
        }
    }
    if (regime == kArea && ok) {
        // Shrinking by fractional factors is separable: OpenCV first sums every source row
        // horizontally with the x weights, then combines those row sums with the y weights.  A
        // thread therefore owns one output column for a run of consecutive output rows: the x taps
        // and weights of its column live in registers for the whole run, and the horizontal sum of
        // a source row that two neighbouring output rows share (the row their boundary cuts) is
        // computed once.  Same operations in the same order as the per-pixel form, so the same bits.
        const int run = (rows + groups - 1) / groups;
        auto area_columns = [&](auto from_window) {
        for (int t = threadIdx.x; t < groups * out_w; t += blockDim.x) {
            const int g = (int)__umulhi((uint32_t)t, inv_w), ox = t - g * out_w;
            const int r_end = min(rows, (g + 1) * run);
            int cx = -1, xoff = 0, xmid = 0, xlast = 0; // column whose taps are loaded
            bool two = false;
            float w_first = 0.f, w_mid = 0.f, w_last = 0.f, c_first = 0.f, c_mid = 0.f, c_last = 0.f;
            int pj = -1;                       // source row whose horizontal sums are held
            float p0 = 0.f, p1 = 0.f, p2 = 0.f;
            const int x_plain = mirrored ? out_w - 1 - ox : ox;
            // horizontal sums of one source row: first tap, the whole cells between, last tap.
            // fma(2^23 + v, w, -2^23 * w) is the correctly rounded v * w, exactly what the
            // multiplication of the converted value gives (2^23 * w is exact).
            auto across = [&](int row) {
                const uint8_t *p;
                if constexpr (decltype(from_window)::value)
                    p = s_win + s_rowoff[row - win_lo] + xoff;
                else
                    p = row_ptr(row) + xoff;
                p0 = __fmaf_rn(u8biased(p[0]), w_first, c_first);
                p1 = __fmaf_rn(u8biased(p[1]), w_first, c_first);
                p2 = __fmaf_rn(u8biased(p[2]), w_first, c_first);
                const uint8_t *q = p + 3;
                for (int k = 0; k < xmid; k++, q += 3) {
                    p0 = __fadd_rn(p0, __fmaf_rn(u8biased(q[0]), w_mid, c_mid));
                    p1 = __fadd_rn(p1, __fmaf_rn(u8biased(q[1]), w_mid, c_mid));
                    p2 = __fadd_rn(p2, __fmaf_rn(u8biased(q[2]), w_mid, c_mid));
                }
                if (two) {
                    p0 = __fadd_rn(p0, __fmaf_rn(u8biased(p[xlast]), w_last, c_last));
                    p1 = __fadd_rn(p1, __fmaf_rn(u8biased(p[xlast + 1]), w_last, c_last));
                    p2 = __fadd_rn(p2, __fmaf_rn(u8biased(p[xlast + 2]), w_last, c_last));
                }
            };
            for (int r = g * run; r < r_end; r++) {
                int y = band0 + r, x = x_plain, val[3] = {0, 0, 0};
                if (flips_only || !trace(band0 + r, ox, y, x, val)) {
                    if (x != cx) {
                        cx = x;
                        pj = -1;
                        const int xc = tx.count[x], xn = xc & 0xffff;
                        const bool xl = xc & (1 << 16), xr = xc & (1 << 17);
                        xoff = tx.first[x] * 3;
                        w_mid = tx.wm[x];
                        w_last = xr ? tx.wr[x] : w_mid;
                        w_first = xl ? tx.wl[x] : (xn == 1 ? w_last : w_mid);
                        two = xn >= 2;
                        xmid = max(xn - 2, 0);
                        xlast = (xn - 1) * 3;
                        c_first = -8388608.0f * w_first;
                        c_mid = -8388608.0f * w_mid;
                        c_last = -8388608.0f * w_last;
                    }
                    const int yf = ty.first[y], yc = ty.count[y], yn = yc & 0xffff;
                    const float ywm = ty.wm[y];
                    const float y_last = (yc & (1 << 17)) ? ty.wr[y] : ywm;
                    const float y_first = (yc & (1 << 16)) ? ty.wl[y] : (yn == 1 ? y_last : ywm);
                    // only the first source row can be the one the previous output row ended with
                    if (yf != pj) across(yf);
                    float a0 = __fmul_rn(y_first, p0), a1 = __fmul_rn(y_first, p1), a2 = __fmul_rn(y_first, p2);
                    for (int j = 1; j < yn; j++) {
                        across(yf + j);
                        const float beta = j == yn - 1 ? y_last : ywm;
                        a0 = __fadd_rn(a0, __fmul_rn(beta, p0));
                        a1 = __fadd_rn(a1, __fmul_rn(beta, p1));
                        a2 = __fadd_rn(a2, __fmul_rn(beta, p2));
                    }
                    pj = yf + yn - 1;
                    val[0] = sat_round(a0);
                    val[1] = sat_round(a1);
                    val[2] = sat_round(a2);
                }
                emit(r * out_w + ox, val);
            }
        }
        };
        if (staged)
            area_columns(std::true_type{});
        else
            area_columns(std::false_type{});
    } else if (regime == kLinear && ok) {
        // Enlarging (OpenCV's fixed-point bilinear) with the same ownership: the two taps of the
        // column stay in registers, and of the two source rows an output row blends, the next
        // output row nearly always shares one or both, whose horizontally interpolated values
        // are kept instead of being fetched and interpolated again.
        const int run = (rows + groups - 1) / groups;
        auto linear_columns = [&](auto from_window) {
        for (int t = threadIdx.x; t < groups * out_w; t += blockDim.x) {
            const int g = (int)__umulhi((uint32_t)t, inv_w), ox = t - g * out_w;
            const int r_end = min(rows, (g + 1) * run);
            int cx = -1, o0 = 0, o1 = 0, xa0 = 0, xa1 = 0;
            int ra = -1, rb = -1; // source rows whose interpolated values ha / hb hold
            int ha[3] = {0, 0, 0}, hb[3] = {0, 0, 0};
            const int x_plain = mirrored ? out_w - 1 - ox : ox;
            for (int r = g * run; r < r_end; r++) {
                int y = band0 + r, x = x_plain, val[3] = {0, 0, 0};
                if (flips_only || !trace(band0 + r, ox, y, x, val)) {
                    if (x != cx) {
                        cx = x;
                        ra = rb = -1;
                        const int sx = tx.first[x], xw = tx.count[x];
                        xa0 = xw >> 16;
                        xa1 = xw & 0xffff;
                        o0 = 3 * sx;
                        o1 = 3 * min(sx + 1, cw - 1);
                    }
                    const int sy = ty.first[y], yw = ty.count[y], b0 = yw >> 16, b1 = yw & 0xffff;
                    const int ry0 = min(sy, ch - 1), ry1 = min(sy + 1, ch - 1);
                    auto across = [&](int row, int *h) {
                        const uint8_t *S;
                        if constexpr (decltype(from_window)::value)
                            S = s_win + s_rowoff[row - win_lo];
                        else
                            S = row_ptr(row);
#pragma unroll
                        for (int c = 0; c < 3; c++) h[c] = (S[o0 + c] * xa0 + S[o1 + c] * xa1) >> 4;
                    };
                    // rows only move forward: the upper row is the former upper or lower one
                    // (selects, no branch), or both rows are new
                    if (ry0 == rb) {
#pragma unroll
                        for (int c = 0; c < 3; c++) ha[c] = hb[c];
                    } else if (ry0 != ra) {
                        across(ry0, ha);
                    }
                    if (ry1 == ry0) {
#pragma unroll
                        for (int c = 0; c < 3; c++) hb[c] = ha[c];
                    } else if (ry1 != rb) {
                        across(ry1, hb);
                    }
                    ra = ry0;
                    rb = ry1;
#pragma unroll
                    for (int c = 0; c < 3; c++) {
                        // non-negative terms: only the upper bound can be exceeded (by rounding of the weights)
                        const int v = (((b0 * ha[c]) >> 16) + ((b1 * hb[c]) >> 16) + 2) >> 2;
                        val[c] = min(255, v);
                    }
                }
                emit(r * out_w + ox, val);
            }
        }
        };
        if (staged)
            linear_columns(std::true_type{});
        else
            linear_columns(std::false_type{});
    } else {
        for (int pix = threadIdx.x; pix < npix; pix += blockDim.x) {
            const int r = (int)__umulhi((uint32_t)pix, inv_w), ox = pix - r * out_w;
            int y, x, val[3] = {0, 0, 0};
            if (!trace(band0 + r, ox, y, x, val) && ok) {
                if (regime == kCopy) {
                    const uint8_t *p = row_ptr(y) + x * 3;
                    val[0] = p[0];
                    val[1] = p[1];
                    val[2] = p[2];
                } else if (regime == kInteger) {
                    int s0 = 0, s1 = 0, s2 = 0;
                    for (int j = 0; j < isy; j++) {
                        const uint8_t *p = row_ptr(y * isy + j) + (x * isx) * 3;
                        for (int k = 0; k < isx; k++, p += 3) {
                            s0 += p[0];
                            s1 += p[1];
                            s2 += p[2];
                        }
                    }
                    if (isx == 2 && isy == 2) {
                        val[0] = (s0 + 2) >> 2;
                        val[1] = (s1 + 2) >> 2;
                        val[2] = (s2 + 2) >> 2;
                    } else {
                        const float inv = __fdiv_rn(1.f, (float)(isx * isy));
                        val[0] = sat_round(__fmul_rn((float)s0, inv));
                        val[1] = sat_round(__fmul_rn((float)s1, inv));
                        val[2] = sat_round(__fmul_rn((float)s2, inv));
                    }
                }
            }
            emit(pix, val);
        }
    }
    __syncthreads();

    // ---- coalesced copy-out: one contiguous run (NHWC) or one per channel (NCHW), 16-byte vectors
    const size_t plane = (size_t)out_h * out_w;
    const int runs = planar ? 3 : 1;
    const int run_elems = planar ? npix : npix * 3;
    for (int c = 0; c < runs; c++) {
        OutT *dst = planar ? out + ((size_t)i * 3 + c) * plane + (size_t)band0 * out_w
                           : out + ((size_t)i * plane + (size_t)band0 * out_w) * 3;
        const OutT *srcp = s_out + (size_t)c * run_elems;
        constexpr int kVec = 16 / sizeof(OutT);
        const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(srcp)) & 15) == 0;
        const int nvec = aligned ? run_elems / kVec : 0;
        for (int k = threadIdx.x; k < nvec; k += blockDim.x)
            reinterpret_cast<uint4 *>(dst)[k] = reinterpret_cast<const uint4 *>(srcp)[k];
        for (int k = nvec * kVec + threadIdx.x; k < run_elems; k += blockDim.x) dst[k] = srcp[k];
    }
    __syncthreads(); // the tile is rewritten by the next band
    }
}

template <typename OutT>
static void launch_typed(const ResizeSource &src, int n, const int32_t *params, int n_params, const OpList &ops,
                         int resize, int out_h, int out_w, int planar, const void *lut, void *out,
                         const int32_t *status, cudaStream_t stream) {
    int band = (2048 + out_w - 1) / out_w;
    if (band < 1) band = 1;
    if (band > out_h) band = out_h;
    auto smem_for = [&](int b) {
        size_t tile = (((size_t)b * out_w * 3 * sizeof(OutT)) + 15) & ~(size_t)15;
        size_t lutb = (768 * sizeof(OutT) + 15) & ~(size_t)15;
        return ((tile + lutb + sizeof(int) * (5 * ((size_t)out_w + out_h) + kMaxWindowRows)) + 15) & ~(size_t)15;
    };
    while (band > 1 && smem_for(band) > 200 * 1024) band /= 2;
    // window of source rows: what is left of a quarter of the SM's shared memory (four resident
    // CTAs of 256 threads is what the registers allow), at most 32 KiB
    const size_t quarter = (227 * 1024) / 4 - 1024;
    size_t win = smem_for(band) + 4096 <= quarter ? quarter - smem_for(band) : 0;
    if (win > 32 * 1024) win = 32 * 1024;
    win &= ~(size_t)15;
    const size_t smem = smem_for(band) + win;
    auto kern = resize_augment_kernel<OutT>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // CTAs per image: enough of them for about eight waves of the GPU (148 SMs x 4 resident CTAs;
    // fewer waves measured slower, more cost the set-up its amortisation), at most one per band
    const int nbands = (out_h + band - 1) / band;
    int per_image = (8 * 148 * 4 + n - 1) / n;
    if (per_image > nbands) per_image = nbands;
    if (per_image < 1) per_image = 1;
    dim3 grid(per_image, n);
    // column path of the area regime: the band's rows are dealt to `groups` runs per column so that
    // the (column, run) items fill the CTA's 256 threads evenly, with runs of at least 3 rows
    int groups = 1;
    double best = 0;
    for (int g = 1; g <= 4 && (band + g - 1) / g >= 3; g++) {
        const int items = g * out_w;
        const double use = (double)items / (((items + 255) / 256) * 256);
        if (use > best + 1e-9) {
            best = use;
            groups = g;
        }
    }
    kern<<<grid, 256, smem, stream>>>(src, params, n_params, ops, resize, out_h, out_w, band, groups, planar,
                                      (int)win, (const OutT *)lut, (OutT *)out, status);
}

void launch_resize_augment(const ResizeSource &src, int n, const int32_t *params, int n_params,
                           const OpList &ops, int resize, int out_h, int out_w, int out_kind,
                           const void *lut, void *out, const int32_t *status, cudaStream_t stream) {
    if (n <= 0) return;
    const int planar = out_kind == kOutF16Nchw || out_kind == kOutF32Nchw;
    if (out_kind == kOutU8)
        launch_typed<uint8_t>(src, n, params, n_params, ops, resize, out_h, out_w, 0, nullptr, out, status, stream);
    else if (out_kind == kOutF16Nhwc || out_kind == kOutF16Nchw)
        launch_typed<uint16_t>(src, n, params, n_params, ops, resize, out_h, out_w, planar, lut, out, status, stream);
    else
        launch_typed<uint32_t>(src, n, params, n_params, ops, resize, out_h, out_w, planar, lut, out, status, stream);
}

} // namespace ffcvb
