// Payload gather from pinned host memory over PCIe (sm_100a): the SMs read the sample bytes of a
// batch straight out of the page-locked dataset file, so no host core touches them.
#include "kernels.h"

namespace ffcvb {

// 16 CTAs of 256 threads with eight 16-byte loads in flight each (512 KB outstanding) move 43-44
// GB/s inside the loader's pipeline (four in flight: 43.0, eight: 44.0; a single pinned DMA copy:
// 55); more CTAs are slower (32: 38.9 GB/s, 8: 42.3): more outstanding system-memory reads only
// congest the memory system for the decode kernels running beside it.
template <int kInFlight>
__global__ void __launch_bounds__(256)
gather_payloads_kernel(const ImageDesc *__restrict__ descs, int n, uint8_t *__restrict__ blob) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int i = blockIdx.x; i < n; i += gridDim.x) {
        const ImageDesc &d = descs[i];
        if (d.src_addr == 0 || d.payload_size == 0) continue;
        const uint8_t *src = reinterpret_cast<const uint8_t *>(d.src_addr);
        uint8_t *dst = blob + d.payload_off;
        if (d.mode == 1 && d.raw_skew) {
            // Raw sample, crop box only.  A row is fetched as the aligned 16-byte words of host
            // memory that contain it and stored as such into its 16-byte aligned slot, so the
            // pixels keep their source alignment inside the slot and no byte is shuffled.  (A
            // word that holds one byte of the row lies in the same page as that byte: the reads
            // stay inside the pinned allocation.)  Two rows per warp and pass, all loads of a
            // pass issued before its stores: up to 8 x 512 bytes in flight per warp.
            const uint32_t run = (uint32_t)d.cols * 3, pitch = (uint32_t)d.width * 3;
            for (int r0 = 2 * warp; r0 < d.rows; r0 += 2 * nwarps) {
                const uint4 *s16[2];
                uint4 *d16[2];
                uint32_t nchunk[2];
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int r = r0 + q;
                    const uint8_t *s = src + (size_t)r * pitch;
                    const uint32_t a = (uint32_t)(reinterpret_cast<uintptr_t>(s) & 15);
                    s16[q] = reinterpret_cast<const uint4 *>(s - a);
                    d16[q] = reinterpret_cast<uint4 *>(dst + (size_t)r * d.raw_pitch);
                    nchunk[q] = r < d.rows ? (a + run + 15) >> 4 : 0;
                }
                const uint32_t most = nchunk[0] > nchunk[1] ? nchunk[0] : nchunk[1];
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < most; c0 += 128) {
                    uint4 v[2][4];
#pragma unroll
                    for (int q = 0; q < 2; q++)
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const uint32_t c = c0 + u * 32 + lane;
                            if (c < nchunk[q]) v[q][u] = s16[q][c];
                        }
#pragma unroll
                    for (int q = 0; q < 2; q++)
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const uint32_t c = c0 + u * 32 + lane;
                            if (c < nchunk[q]) d16[q][c] = v[q][u];
                        }
                }
            }
            continue;
        }
        const uint32_t size = d.payload_size;
        uint32_t head = (uint32_t)((16 - (d.src_addr & 15)) & 15);
        if (head > size) head = size;
        if ((reinterpret_cast<uintptr_t>(dst) & 15) != (d.src_addr & 15)) head = size; // never: bytes only
        for (uint32_t k = threadIdx.x; k < head; k += blockDim.x) dst[k] = src[k];
        const uint32_t nvec = (size - head) >> 4;
        const uint4 *s16 = reinterpret_cast<const uint4 *>(src + head);
        uint4 *d16 = reinterpret_cast<uint4 *>(dst + head);
        uint32_t k = threadIdx.x;
        for (; k + (kInFlight - 1) * blockDim.x < nvec; k += kInFlight * blockDim.x) {
            uint4 v[kInFlight]; // all loads of a pass are issued before its stores
#pragma unroll
            for (int u = 0; u < kInFlight; u++) v[u] = s16[k + u * blockDim.x];
#pragma unroll
            for (int u = 0; u < kInFlight; u++) d16[k + u * blockDim.x] = v[u];
        }
        for (; k < nvec; k += blockDim.x) d16[k] = s16[k];
        for (uint32_t t = head + (nvec << 4) + threadIdx.x; t < size; t += blockDim.x) dst[t] = src[t];
    }
}

void launch_gather_payloads(const ImageDesc *descs, int n, uint8_t *blob, int ctas, int in_flight, cudaStream_t stream) {
    if (n <= 0) return;
    if (ctas < 1) ctas = kGatherCtas;
    const int grid = n < ctas ? n : ctas;
    if (in_flight >= 8)
        gather_payloads_kernel<8><<<grid, 256, 0, stream>>>(descs, n, blob);
    else
        gather_payloads_kernel<4><<<grid, 256, 0, stream>>>(descs, n, blob);
}

} // namespace ffcvb
