// ffcvb_imdecode_static: JPEG -> RGB decode of one image that allocates nothing.
//
// Who needs it: code that already owns all of its GPU memory and is not allowed to ask the driver
// for more while it runs -- a serving process whose memory pool was carved up at start-up, a
// plugin running inside another framework's allocator, or a latency-critical loop where a
// cudaMalloc (which can synchronise the whole device) is unacceptable.  The regular entry points grow pinned and device buffers on demand; this one
// uses a fixed scratch area that is part of the library image instead, so every GPU that loads
// the library carries kScratchBytes of it until the process exits.
//
// The decode itself is the same chain of kernels as everywhere else (entropy decode, dequantise +
// IDCT, upsample + colour conversion); only the scratch comes from the static array.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/ffcv_b200.h"
#include "jpeg_header.h"
#include "kernels.h"
#include "types.h"

using namespace ffcvb;

namespace {

// Limits of one call (stated in include/ffcv_b200.h).
constexpr size_t kMaxStreamBytes = FFCVB_STATIC_MAX_STREAM_BYTES;    // compressed size
constexpr size_t kMaxPaddedSamples = FFCVB_STATIC_MAX_PADDED_PIXELS; // per component, padded to MCUs

// Scratch layout inside the static array (all offsets multiples of 256).
constexpr size_t kMetaBytes = 48 * 1024;                             // descriptor, tables, list, status
constexpr size_t kCleanBytes = kMaxStreamBytes + 512;                // unstuffed bit stream
constexpr size_t kCoefBytes = 3 * kMaxPaddedSamples * sizeof(int16_t); // 64 coefficients per 64 samples
constexpr size_t kPlaneBytes = 3 * kMaxPaddedSamples + 1024;         // each plane rounded up to 256
constexpr size_t kCleanOff = kMetaBytes;
constexpr size_t kCoefOff = kCleanOff + kCleanBytes;
constexpr size_t kPlaneOff = kCoefOff + kCoefBytes;
constexpr size_t kScratchBytes = kPlaneOff + kPlaneBytes;

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can
// use; the device address is looked up once per device and cached here.
constexpr int kMaxDevices = 64;
unsigned char *g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;

struct Meta {
    ImageDesc desc;
    int32_t list[4];
    int32_t status[4];
    HuffTable huff[6];
    alignas(16) MultTable mult[3]; // read with 16-byte loads
};
static_assert(sizeof(Meta) <= kMetaBytes, "metadata must fit its scratch region");

int reject(int code, const char *why) {
    fprintf(stderr, "ffcvb_imdecode_static: %s\n", why);
    return code;
}

} // namespace

extern "C" int ffcvb_imdecode_static(const uint8_t *jpeg_host, uint64_t jpeg_size, const uint8_t *jpeg_dev,
                                     uint32_t height, uint32_t width, uint8_t *rgb_dev, void *stream) {
    if (!jpeg_host || !jpeg_dev || !rgb_dev || jpeg_size < 4) return reject(FFCVB_E_ARG, "null or empty argument");
    if (jpeg_size > kMaxStreamBytes) return reject(FFCVB_E_LIMIT, "JPEG stream larger than FFCVB_STATIC_MAX_STREAM_BYTES");
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return reject(FFCVB_E_NODEVICE, "no current CUDA device");

    // ---- set-up, once per device (the first call on a device; make it before any stream capture)
    unsigned char *scratch;
    {
        std::lock_guard<std::mutex> g(g_setup_mutex);
        if (!g_scratch_addr[dev]) {
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p) return reject(FFCVB_E_CUDA, cudaGetErrorString(e));
            g_scratch_addr[dev] = static_cast<unsigned char *>(p);
        }
        scratch = g_scratch_addr[dev];
    }

    // ---- headers on the host, limits
    JpegHeader h;
    int rc = parse_jpeg_header(jpeg_host, (size_t)jpeg_size, &h);
    if (rc != 0) return reject(FFCVB_E_DECODE, "not a baseline JPEG stream this library decodes");
    if ((uint32_t)h.width != width || (uint32_t)h.height != height)
        return reject(FFCVB_E_DECODE, "stream dimensions differ from the given height and width");
    if (height > 65535 || width > 65535) return reject(FFCVB_E_LIMIT, "image larger than FFCVB_STATIC_MAX_PADDED_PIXELS");
    Meta m;
    memset(&m, 0, sizeof(m));
    ImageDesc &d = m.desc;
    d.payload_size = (uint32_t)jpeg_size;
    d.height = d.dec_height = (uint16_t)height;
    d.width = d.dec_width = (uint16_t)width;
    d.bs_luma = d.bs_chroma = 8; // full scale
    d.rgb_pitch = (uint32_t)width * 3; // the caller's buffer is packed
    d.scan_off = (uint32_t)h.scan_off;
    d.scan_len = (uint32_t)h.scan_len;
    d.ncomp = (uint8_t)h.ncomp;
    d.hs = (uint8_t)h.hs[0];
    d.vs = (uint8_t)h.vs[0];
    d.bpm = (uint8_t)(h.ncomp == 1 ? 1 : h.hs[0] * h.vs[0] + 2);
    d.mcus_x = (uint16_t)((h.width + 8 * h.hs[0] - 1) / (8 * h.hs[0]));
    d.mcus_y = (uint16_t)((h.height + 8 * h.vs[0] - 1) / (8 * h.vs[0]));
    d.restart_interval = (uint16_t)h.restart_interval;
    d.mcu_rows = d.mcus_y;
    d.idct_row0 = d.idct_col0 = 0;
    d.idct_col1 = d.mcus_x;
    d.nblocks = (uint32_t)d.bpm * d.mcus_x * d.mcus_y;
    if (d.restart_interval) { // table of restart-interval starts behind the clean stream
        d.rst_off = ((size_t)d.scan_len + 96 + 15) & ~(size_t)15;
        const size_t mcus = (size_t)d.mcus_x * d.mcus_y;
        if (d.rst_off + 4 * ((mcus + d.restart_interval - 1) / d.restart_interval + 2) > kCleanBytes)
            return reject(FFCVB_E_LIMIT, "stream with restart markers too large for the static scratch");
    }
    const size_t luma_samples = (size_t)d.mcus_x * d.hs * 8 * d.mcus_y * d.vs * 8;
    if (luma_samples > kMaxPaddedSamples)
        return reject(FFCVB_E_LIMIT, "image larger than FFCVB_STATIC_MAX_PADDED_PIXELS");
    size_t plane = 0;
    for (int c = 0; c < h.ncomp; c++) {
        build_huff_table(h.dc[h.td[c]], &m.huff[2 * c]);
        build_huff_table(h.ac[h.ta[c]], &m.huff[2 * c + 1]);
        build_mult_table(h.quant[h.tq[c]], &m.mult[c]);
        d.dc_tab[c] = (uint8_t)(2 * c);
        d.ac_tab[c] = (uint8_t)(2 * c + 1);
        d.q_tab[c] = (uint8_t)c;
        d.plane_off[c] = plane;
        plane += ((size_t)d.mcus_x * (c == 0 ? d.hs : 1) * 8 * d.mcus_y * (c == 0 ? d.vs : 1) * 8 + 255) & ~(size_t)255;
    }

    // ---- queue the work; everything the kernels need beyond input and output lives in `scratch`
    cudaStream_t st = (cudaStream_t)stream;
    Meta *meta_dev = reinterpret_cast<Meta *>(scratch);
    // `m` lives on this thread's stack (pageable memory): for such a source the runtime stages the
    // bytes before cudaMemcpyAsync returns, so `m` may go out of scope when this call does
    if (cudaMemcpyAsync(meta_dev, &m, sizeof(m), cudaMemcpyHostToDevice, st) != cudaSuccess)
        return reject(FFCVB_E_CUDA, "copy of the descriptor failed");
    const ImageDesc *desc_dev = &meta_dev->desc;
    const int32_t *list_dev = meta_dev->list; // {0}: the only image
    const bool sequential = d.restart_interval != 0;
    const size_t max_scan = d.scan_len;
    size_t subseq = ((max_scan * 8 / 512 + 1) + 127) / 128 * 128;
    subseq = subseq < 512 ? 512 : (subseq > 1280 ? 1280 : subseq);
    launch_entropy_decode(desc_dev, list_dev, sequential ? 0 : 1, list_dev, sequential ? 1 : 0, jpeg_dev, meta_dev->huff,
                          scratch + kCleanOff, reinterpret_cast<int16_t *>(scratch + kCoefOff), meta_dev->status,
                          (int)subseq, 512, nullptr, nullptr, nullptr, st);
    launch_idct(desc_dev, list_dev, 1, d.nblocks, meta_dev->mult, reinterpret_cast<const int16_t *>(scratch + kCoefOff),
                scratch + kPlaneOff, st);
    const bool quad = d.ncomp == 3 && d.hs == 2 && d.vs == 2 && (width + 1) / 2 >= 3;
    const bool full = d.ncomp == 3 && d.hs == 1 && d.vs == 1;
    launch_color(desc_dev, list_dev, 1, quad ? 1 : 0, full ? 1 : 0, (quad || full) ? 0 : 1, (int)width, (int)height,
                 nullptr, 0, scratch + kPlaneOff, rgb_dev, nullptr, 0, st);
    if (cudaGetLastError() != cudaSuccess) return reject(FFCVB_E_CUDA, "kernel launch failed");
    return FFCVB_OK;
}
