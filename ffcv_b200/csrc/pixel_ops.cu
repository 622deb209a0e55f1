// Per-pixel colour and blending transforms on uint8 device batches (sm_100a): brightness,
// contrast, saturation (ffcv/transforms/color_jitter.py), image mixup (ffcv/transforms/mixup.py)
// and poisoning (ffcv/transforms/poisoning.py).
//
// The reference evaluates these in float64 under numba's fastmath, which fuses some multiply-add
// pairs; which ones decides the last bit of a truncated result.  Every operation below is written
// with explicit rounding intrinsics (__dmul_rn, __dadd_rn, __fma_rn) so that nvcc fuses nothing
// by itself and the arithmetic is, operation for operation, the one the reference's compiled code
// performs:
//   grey      = (uint8) fma(0.114, b, fma(0.587, g, 0.2989 * r))
//   brightness, contrast:  fma(t, v, (1 - t) * s)     (s = 0, or the mean of the grey image)
//   saturation:            t * v + (1 - t) * grey      (not fused)
//   mixup:                 fma(1 - t, partner, t * v)
// HBM-bound byte work: each kernel reads and writes every byte of the selected images once.
#include "kernels.h"

namespace ffcvb {

namespace {

__device__ __forceinline__ uint32_t clip_u8(double v) {
    v = fmax(v, 0.0);
    v = fmin(v, 255.0);
    return __double2uint_rz(v);
}

__device__ __forceinline__ uint32_t grey_u8(uint32_t r, uint32_t g, uint32_t b) {
    return __double2uint_rz(__fma_rn(0.114, (double)b, __fma_rn(0.587, (double)g, __dmul_rn(0.2989, (double)r))));
}

__device__ __forceinline__ uint32_t byte_of(const uint32_t (&w)[3], int k) { return (w[k >> 2] >> (8 * (k & 3))) & 255u; }

// One thread per group of four pixels (12 bytes = three aligned words when `pixels` is a multiple
// of four, which the launcher checks; otherwise one thread per pixel with byte accesses).
template <int KIND, bool VEC>
__global__ void __launch_bounds__(256)
jitter_kernel(uint8_t *__restrict__ images, int pixels, const uint8_t *__restrict__ apply,
              const double *__restrict__ ratio, const unsigned long long *__restrict__ grey_sum) {
    const int img = blockIdx.y;
    if (!apply[img]) return;
    const double t = ratio[img], u = __dsub_rn(1.0, t);
    double c = 0.0;
    if (KIND == kJitterBrightness) c = __dmul_rn(u, 0.0);
    if (KIND == kJitterContrast) c = __dmul_rn(u, __ddiv_rn((double)grey_sum[img], (double)pixels));
    uint8_t *base = images + (size_t)img * pixels * 3;
    const int per = VEC ? 4 : 1;
    for (int p0 = (blockIdx.x * blockDim.x + threadIdx.x) * per; p0 < pixels; p0 += gridDim.x * blockDim.x * per) {
        uint32_t w[3];
        if (VEC) {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(base + (size_t)p0 * 3);
            w[0] = src[0];
            w[1] = src[1];
            w[2] = src[2];
        } else {
            const uint8_t *src = base + (size_t)p0 * 3;
            w[0] = src[0] | (src[1] << 8) | (src[2] << 16);
            w[1] = w[2] = 0;
        }
        uint32_t o[3] = {0, 0, 0};
#pragma unroll
        for (int q = 0; q < per; q++) {
            const uint32_t r = byte_of(w, 3 * q), g = byte_of(w, 3 * q + 1), b = byte_of(w, 3 * q + 2);
            const uint32_t v[3] = {r, g, b};
            double l = 0.0;
            if (KIND == kJitterSaturation) l = __dmul_rn(u, (double)grey_u8(r, g, b));
#pragma unroll
            for (int ch = 0; ch < 3; ch++) {
                double x;
                if (KIND == kJitterSaturation)
                    x = __dadd_rn(__dmul_rn(t, (double)v[ch]), l);
                else
                    x = __fma_rn(t, (double)v[ch], c);
                const int k = 3 * q + ch;
                o[k >> 2] |= clip_u8(x) << (8 * (k & 3));
            }
        }
        if (VEC) {
            uint32_t *dst = reinterpret_cast<uint32_t *>(base + (size_t)p0 * 3);
            dst[0] = o[0];
            dst[1] = o[1];
            dst[2] = o[2];
        } else {
            uint8_t *dst = base + (size_t)p0 * 3;
            dst[0] = (uint8_t)o[0];
            dst[1] = (uint8_t)(o[0] >> 8);
            dst[2] = (uint8_t)(o[0] >> 16);
        }
    }
}

// Sum of the (truncated) grey values of every selected image, for the contrast mean.  Integer
// sums, so the order of the additions does not matter.
__global__ void __launch_bounds__(256)
grey_sum_kernel(const uint8_t *__restrict__ images, int pixels, const uint8_t *__restrict__ apply,
                unsigned long long *__restrict__ grey_sum) {
    const int img = blockIdx.y;
    if (!apply[img]) return;
    const uint8_t *base = images + (size_t)img * pixels * 3;
    unsigned int acc = 0; // at most 2^31 / 255 pixels per thread
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < pixels; p += gridDim.x * blockDim.x)
        acc += grey_u8(base[(size_t)p * 3], base[(size_t)p * 3 + 1], base[(size_t)p * 3 + 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    __shared__ unsigned int s_part[8];
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long total = 0;
        for (int k = 0; k < (int)(blockDim.x >> 5); k++) total += s_part[k];
        atomicAdd(&grey_sum[img], total);
    }
}

// dst[i] = lam[i] * src[i] + (1 - lam[i]) * src[i - 1] (image -1 = the last), truncated.
template <bool VEC>
__global__ void __launch_bounds__(256)
mixup_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int n, long long count,
             const double *__restrict__ lam) {
    const int img = blockIdx.y;
    const double l = lam[img], u = __dsub_rn(1.0, l);
    const uint8_t *a = src + (size_t)img * count;
    const uint8_t *b = src + (size_t)(img == 0 ? n - 1 : img - 1) * count;
    uint8_t *o = dst + (size_t)img * count;
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (VEC) {
        const uint32_t *a4 = reinterpret_cast<const uint32_t *>(a), *b4 = reinterpret_cast<const uint32_t *>(b);
        uint32_t *o4 = reinterpret_cast<uint32_t *>(o);
        for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < count / 4; k += stride) {
            const uint32_t x = a4[k], y = b4[k];
            uint32_t r = 0;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const double va = (double)((x >> (8 * q)) & 255u), vb = (double)((y >> (8 * q)) & 255u);
                r |= (__double2uint_rz(__fma_rn(u, vb, __dmul_rn(l, va))) & 255u) << (8 * q);
            }
            o4[k] = r;
        }
    } else {
        for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < count; k += stride)
            o[k] = (uint8_t)__double2uint_rz(__fma_rn(u, (double)b[k], __dmul_rn(l, (double)a[k])));
    }
}

// Poison: float32 scratch value per element, two statements that each round a float64 result to
// float32, clamp, truncate (ffcv/transforms/poisoning.py:52-58).
__global__ void __launch_bounds__(256)
poison_kernel(uint8_t *__restrict__ images, long long count, const uint8_t *__restrict__ apply,
              const double *__restrict__ one_minus_alpha, const double *__restrict__ mask, float lo, float hi) {
    const int img = blockIdx.y;
    if (!apply[img]) return;
    uint8_t *p = images + (size_t)img * count;
    for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < count;
         k += (long long)gridDim.x * blockDim.x) {
        float t = (float)p[k];
        t = __double2float_rn(__dmul_rn((double)t, one_minus_alpha[k]));
        t = __double2float_rn(__dadd_rn((double)t, mask[k]));
        t = fmaxf(t, lo);
        t = fminf(t, hi);
        p[k] = (uint8_t)__float2uint_rz(t);
    }
}

int blocks_for(long long items, int per_block) {
    long long b = (items + per_block - 1) / per_block;
    if (b < 1) b = 1;
    if (b > 148 * 8) b = 148 * 8; // grid-stride beyond eight CTAs per SM
    return (int)b;
}

} // namespace

void launch_color_jitter(uint8_t *images, int n, int h, int w, int kind, const uint8_t *apply,
                         const double *ratio, unsigned long long *grey_sum, cudaStream_t stream) {
    const int pixels = h * w;
    const bool vec = pixels % 4 == 0 && (reinterpret_cast<uintptr_t>(images) & 3) == 0;
    const dim3 grid(blocks_for(pixels / (vec ? 4 : 1), 256), n);
    if (kind == kJitterContrast) {
        cudaMemsetAsync(grey_sum, 0, sizeof(unsigned long long) * (size_t)n, stream);
        grey_sum_kernel<<<dim3(blocks_for(pixels, 256 * 8), n), 256, 0, stream>>>(images, pixels, apply, grey_sum);
    }
#define FFCVB_JITTER(K)                                                                            \
    if (vec)                                                                                       \
        jitter_kernel<K, true><<<grid, 256, 0, stream>>>(images, pixels, apply, ratio, grey_sum);  \
    else                                                                                           \
        jitter_kernel<K, false><<<grid, 256, 0, stream>>>(images, pixels, apply, ratio, grey_sum);
    if (kind == kJitterBrightness) {
        FFCVB_JITTER(kJitterBrightness)
    } else if (kind == kJitterContrast) {
        FFCVB_JITTER(kJitterContrast)
    } else {
        FFCVB_JITTER(kJitterSaturation)
    }
#undef FFCVB_JITTER
}

void launch_mixup(const uint8_t *src, uint8_t *dst, int n, long long count, const double *lam,
                  cudaStream_t stream) {
    const bool vec = count % 4 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 3) == 0;
    const dim3 grid(blocks_for(count / (vec ? 4 : 1), 256), n);
    if (vec)
        mixup_kernel<true><<<grid, 256, 0, stream>>>(src, dst, n, count, lam);
    else
        mixup_kernel<false><<<grid, 256, 0, stream>>>(src, dst, n, count, lam);
}

void launch_poison(uint8_t *images, int n, long long count, const uint8_t *apply, const double *one_minus_alpha,
                   const double *mask, float lo, float hi, cudaStream_t stream) {
    poison_kernel<<<dim3(blocks_for(count, 256), n), 256, 0, stream>>>(images, count, apply, one_minus_alpha, mask,
                                                                      lo, hi);
}

} // namespace ffcvb
