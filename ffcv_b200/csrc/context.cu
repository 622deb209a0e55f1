// Host side of libffcv_b200.so: contexts, batch slots, the staging thread pool and the C ABI
// declared in include/ffcv_b200.h.
#include <cuda_runtime.h>
#include <emmintrin.h>
#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <array>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <string>
#include <memory>
#include <thread>
#include <unordered_map>
#include <chrono>
#include <vector>

#include "../../include/ffcv_b200.h"
#include "jpeg_header.h"
#include "kernels.h"
#include "types.h"

using namespace ffcvb;

namespace {

// ------------------------------------------------------------------ staging thread pool
// Worker threads with two job lanes.  The synchronous lane (parallel_for) serves the header
// parse of the batch being staged; the asynchronous lane carries the payload copy of the batch
// staged before it, which keeps running while the caller goes on.  Workers drain the synchronous
// lane first, so a parse never queues behind a copy.  Items are handed out under the mutex,
// `grain` at a time.
class Pool {
  public:
    enum Lane { kSync = 0, kAsync = 1 };
    explicit Pool(int n) {
        for (int i = 0; i < n; i++) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(m_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto &t : workers_) t.join();
    }
    // Runs fn(i) for i in [0, n) on the pool and the calling thread; returns when all are done.
    void parallel_for(int n, int grain, std::function<void(int)> fn) {
        post(kSync, n, grain, std::move(fn), nullptr);
        wait(kSync);
    }
    // Hands fn(i), i in [0, n), to the workers and returns.  `done` runs once after the last item
    // (under the pool's mutex: it must be short and must not call the pool).  The lane must be idle.
    // At most `max_threads` threads work on the job at a time (0 = no limit).
    void post(Lane lane, int n, int grain, std::function<void(int)> fn, std::function<void()> done,
              int max_threads = 0) {
        wait(lane);
        if (n <= 0) {
            if (done) done();
            return;
        }
        {
            std::lock_guard<std::mutex> g(m_);
            Job &j = jobs_[lane];
            j.fn = std::move(fn);
            j.done = std::move(done);
            j.n = n;
            j.next = 0;
            j.grain = grain < 1 ? 1 : grain;
            j.inflight = 0;
            j.limit = max_threads > 0 ? max_threads : 1 << 30;
            j.active = true;
        }
        if (workers_.empty())
            wait(lane); // nobody else would run it
        else
            cv_.notify_all();
    }
    // Lends the calling thread to the lane's job, then waits until the job is complete.
    void wait(Lane lane) {
        std::unique_lock<std::mutex> g(m_);
        Job &j = jobs_[lane];
        while (j.active) {
            if (j.next < j.n)
                run_some(j, g);
            else
                done_cv_.wait(g, [&] { return !j.active; });
        }
    }
    void wait_all() {
        wait(kSync);
        wait(kAsync);
    }
    int size() const { return (int)workers_.size() + 1; }

  private:
    struct Job {
        std::function<void(int)> fn;
        std::function<void()> done;
        int n = 0, next = 0, grain = 1, inflight = 0, limit = 1 << 30;
        bool active = false;
    };
    // Called with the mutex held and items left; returns with it held.
    void run_some(Job &j, std::unique_lock<std::mutex> &g) {
        const int lo = j.next;
        const int hi = lo + j.grain < j.n ? lo + j.grain : j.n;
        j.next = hi;
        j.inflight++;
        g.unlock();
        for (int i = lo; i < hi; i++) j.fn(i);
        g.lock();
        j.inflight--;
        if (j.next >= j.n && j.inflight == 0) {
            if (j.done) j.done();
            j.done = nullptr;
            j.active = false;
            done_cv_.notify_all();
        }
    }
    Job *pending() {
        for (Job &j : jobs_)
            if (j.active && j.next < j.n && j.inflight < j.limit) return &j;
        return nullptr;
    }
    void loop() {
        std::unique_lock<std::mutex> g(m_);
        for (;;) {
            cv_.wait(g, [&] { return stop_ || pending() != nullptr; });
            if (stop_) return;
            while (Job *j = pending()) run_some(*j, g);
        }
    }
    std::vector<std::thread> workers_;
    std::mutex m_;
    std::condition_variable cv_, done_cv_;
    bool stop_ = false;
    Job jobs_[2];
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Multiplicative hash over a table's bytes, eight at a time: lets the (serial) table
// deduplication of a batch compare 8 bytes per table instead of the tables themselves; the hashes
// are computed by the parallel header parse.
uint64_t hash_bytes(const void *p, size_t n) {
    const uint8_t *b = static_cast<const uint8_t *>(p);
    uint64_t h = 0x9E3779B97F4A7C15ull ^ n;
    size_t i = 0;
    for (; i + 8 <= n; i += 8) {
        uint64_t w;
        memcpy(&w, b + i, 8);
        h = (h ^ w) * 0xFF51AFD7ED558CCDull;
        h ^= h >> 29;
    }
    uint64_t w = 0;
    if (i < n) memcpy(&w, b + i, n - i);
    h = (h ^ w) * 0xC4CEB9FE1A85EC53ull;
    return h ^ (h >> 32);
}

// Copy into the pinned staging buffer with non-temporal stores: the destination is read next by
// the DMA engine, not by the CPU, so it should not displace the cache or cost a read-for-ownership.
// dst is 16-byte aligned (payload offsets are).
void stream_copy(uint8_t *dst, const uint8_t *src, size_t n) {
    if ((reinterpret_cast<uintptr_t>(dst) & 15) != 0 || n < 4096) {
        memcpy(dst, src, n);
        return;
    }
    size_t k = 0;
    for (; k + 64 <= n; k += 64) {
        __m128i a = _mm_loadu_si128(reinterpret_cast<const __m128i *>(src + k));
        __m128i b = _mm_loadu_si128(reinterpret_cast<const __m128i *>(src + k + 16));
        __m128i c = _mm_loadu_si128(reinterpret_cast<const __m128i *>(src + k + 32));
        __m128i d = _mm_loadu_si128(reinterpret_cast<const __m128i *>(src + k + 48));
        _mm_stream_si128(reinterpret_cast<__m128i *>(dst + k), a);
        _mm_stream_si128(reinterpret_cast<__m128i *>(dst + k + 16), b);
        _mm_stream_si128(reinterpret_cast<__m128i *>(dst + k + 32), c);
        _mm_stream_si128(reinterpret_cast<__m128i *>(dst + k + 48), d);
    }
    if (k < n) memcpy(dst + k, src + k, n - k);
}

struct DevBuf {
    void *p = nullptr;
    size_t cap = 0;
};

struct Slot {
    uint8_t *host = nullptr; // pinned
    size_t host_cap = 0;
    DevBuf blob, clean, coef, planes, rgb, status, ckpt;
    BatchHeader hdr{};
    ffcvb_plan plan{};
    int n = 0, n_jpeg = 0, n_par = 0, n_seq = 0, max_pixels = 0, subseq_bits = 512, entropy_threads = 512;
    int n_quad = 0, n_444 = 0, n_other = 0, max_w = 0, max_h = 0;
    uint64_t jpeg_list_off = 0, par_list_off = 0, seq_list_off = 0, quad_tiles_off = 0;
    int n_quad_tiles = 0;
    uint32_t total_blocks = 0;
    size_t clean_bytes = 0, plane_bytes = 0, rgb_bytes = 0, scan_bytes = 0, raw_bytes = 0, jpeg_bytes = 0;
    bool staged = false;
    bool direct = false; // payloads are gathered by the GPU from pinned host memory
    size_t staged_end = 0; // blob bytes [0, staged_end) come from the pinned staging buffer
    bool copy_done = true; // the staging threads have finished this slot's payload copy (guarded by ctx->copy_m)
    std::vector<ImageDesc> descs;
    std::vector<uint64_t> src_ptrs;
    // values of the sample's other fields that travel in the head of this batch's blob
    struct Rider {
        std::vector<uint8_t> inline_bytes; // n * item_bytes, or empty when gathered from the file
        std::vector<uint64_t> ptrs;        // file offsets of the n items (gathered riders)
        uint64_t item_bytes = 0;
        void *dst_dev = nullptr;
        uint64_t off = 0, bytes = 0;       // place in the blob (set by ffcvb_stage_batch)
    };
    std::vector<Rider> pending_riders, riders; // set for the next staging / staged with the current batch
    double stage_ms[4] = {0, 0, 0, 0}; // header parse, layout, payload copy, total
    std::vector<JpegHeader> headers;
    std::vector<uint64_t> table_hash; // per sample: hashes of its (DC, AC, quantisation) tables x 3 components
    std::vector<uint16_t> table_id;   // per sample: the same nine tables as indices into the context's stores
    std::vector<uint8_t> from_cache;  // per sample: its header came from the context's header cache
    cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    // payload gather runs on its own high-priority stream so that its few CTAs are placed ahead of
    // the large grids other slots have queued, and the PCIe transfer overlaps their compute
    cudaStream_t gather_stream = nullptr;
    cudaEvent_t ev_begin = nullptr, ev_gather_start = nullptr, ev_gathered = nullptr;
    // recorded behind the last work queued on the slot: staging the slot again waits for it, so a
    // caller that forgets to fence the ring gets a stall instead of a batch whose descriptors are
    // overwritten under its kernels
    cudaEvent_t ev_done = nullptr;
    bool in_flight = false;
    bool gather_timed = false; // ev_gather_start .. ev_gathered bracket the last gather of this slot
    bool timed = false; // events of the last run are valid
};

struct AuxBuf {
    DevBuf dev;
    uint8_t *host = nullptr;
    size_t host_cap = 0;
    cudaEvent_t ev = nullptr;
    bool used = false;
};

} // namespace

struct WaitArg {
    ffcvb_ctx *ctx;
    int slot;
};

struct ffcvb_ctx {
    int device = 0;
    std::vector<Slot> slots;
    std::vector<WaitArg> wait_args; // one per slot, for the stream callback that waits for its copy
    std::mutex copy_m;
    std::condition_variable copy_cv;
    std::atomic<bool> copy_timeout{false};
    std::atomic<bool> direct_broken{false}; // an O_DIRECT read was refused: buffered reads from now on
    Pool *pool = nullptr;
    std::string err;
    AuxBuf aux[16];
    int aux_next = 0;
    bool profile = false;
    bool async_staging = false;
    int cpu_share_permille = 0; // pinned source: share of the payload bytes the staging threads copy
    bool adaptive_split = false; // ... adjusted from batch to batch so that both sides take equally long
    double share = 0.0;          // the adjusted share, 0..1
    int split_copy_threads = 4; // ... and how many of them copy at a time (more only crowd the gather out)
    // Tuning overrides, read from the environment once when the context is created (0 = none):
    // FFCV_B200_COPY_THREADS, FFCV_B200_SUBSEQ_BITS, FFCV_B200_ENTROPY_THREADS, FFCV_B200_GATHER_CTAS,
    // FFCV_B200_GATHER_IN_FLIGHT.
    int tune_copy_threads = 0, tune_subseq_bits = 0, tune_entropy_threads = 0, gather_ctas = 0, gather_in_flight = 8;
    DevBuf one_src, one_dst; // single-image entry points
    // Decode index (ffcvb_set_decode_index): a pool of device memory that keeps, per JPEG stream seen,
    // the decoder states a finished decode left behind; entries are handed out in order and never
    // moved.  Keyed by the sample's offset in the file: the context then serves one file.
    struct IndexEntry {
        uint64_t off;
        uint32_t cap;
        uint32_t subseq_bits;
        uint64_t created_seq;
    };
    // Header cache: what the marker segments of a JPEG sample said, kept per sample (key: its
    // offset in the file) so that from the second epoch on staging a sample is a table look-up
    // instead of a parse; the few distinct Huffman and quantisation tables of a file live in a
    // store of their own and the cache holds indices into it.
    struct CachedHeader {
        uint64_t size;
        uint32_t scan_off, scan_len;
        uint16_t restart_interval, width, height;
        uint8_t ncomp, hs, vs;
        uint16_t table[9]; // per component: DC, AC (huff_store), quantisation (quant_store)
    };
    bool cache_headers = false; // ffcvb_set_header_cache: sample offsets identify samples (one file per context)
    std::unordered_map<uint64_t, CachedHeader> header_cache;
    std::vector<std::unique_ptr<RawHuff>> huff_store;
    std::vector<std::unique_ptr<std::array<uint16_t, 64>>> quant_store;
    std::vector<uint64_t> huff_store_hash, quant_store_hash;
    DevBuf index_pool, index_stats;
    size_t index_used = 0;
    std::unordered_map<uint64_t, IndexEntry> index_map;
    uint64_t stage_seq = 0;
};

namespace {

int fail(ffcvb_ctx *c, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (c) c->err = buf;
    return code;
}

#define CU(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess)                                                                     \
            return fail(ctx, e_ == cudaErrorMemoryAllocation ? FFCVB_E_NOMEM : FFCVB_E_CUDA,       \
                        "%s: %s", #call, cudaGetErrorString(e_));                                  \
    } while (0)

int grow_dev(ffcvb_ctx *ctx, DevBuf &b, size_t need) {
    if (need <= b.cap) return 0;
    size_t cap = align_up(need + need / 4, 1 << 20);
    if (b.p) {
        CU(cudaDeviceSynchronize());
        CU(cudaFree(b.p));
        b.p = nullptr;
        b.cap = 0;
    }
    CU(cudaMalloc(&b.p, cap));
    b.cap = cap;
    return 0;
}

int grow_host(ffcvb_ctx *ctx, uint8_t *&p, size_t &cap_io, size_t need) {
    if (need <= cap_io) return 0;
    size_t cap = align_up(need + need / 4, 1 << 20);
    if (p) {
        CU(cudaDeviceSynchronize());
        CU(cudaFreeHost(p));
        p = nullptr;
        cap_io = 0;
    }
    CU(cudaHostAlloc((void **)&p, cap, cudaHostAllocDefault));
    cap_io = cap;
    return 0;
}

bool valid_plan(const ffcvb_plan *p) {
    if (!p || p->out_h <= 0 || p->out_w <= 0 || p->n_ops < 0 || p->n_ops > FFCVB_MAX_OPS) return false;
    if (p->out_kind < FFCVB_OUT_U8_NHWC || p->out_kind > FFCVB_OUT_F32_NCHW) return false;
    if (p->out_kind != FFCVB_OUT_U8_NHWC && !p->lut_dev) return false;
    for (int k = 0; k < p->n_ops; k++) {
        int t = p->ops[k].type;
        if (t != FFCVB_OP_FLIP && t != FFCVB_OP_TRANSLATE && t != FFCVB_OP_CUTOUT) return false;
        if (t != FFCVB_OP_FLIP && p->ops[k].arg < 0) return false;
    }
    if (p->dct_scale < -1 || p->dct_scale > 3 || (p->dct_scale < 0 && !p->resize)) return false;
    return true;
}

OpList make_oplist(const ffcvb_plan &p) {
    OpList o{};
    o.n_ops = p.n_ops;
    for (int k = 0; k < p.n_ops; k++) {
        o.type[k] = p.ops[k].type;
        o.arg[k] = p.ops[k].arg;
        memcpy(o.fill[k], p.ops[k].fill, 4);
    }
    return o;
}

// CTA size and subsequence length of the speculative entropy decoder for a batch whose largest
// scan has `max_scan_bytes`.  One pass of the CTA's threads should cover the largest image (the
// decoder needs about 7 kbit to re-synchronise, so shorter subsequences only add repair rounds),
// with subsequences of at most 1280 bits (a chunk of 512 of them must fit shared memory twice per
// SM) and no more threads than that takes: small images decode faster with 128 or 256 threads per
// CTA because more CTAs are resident (config 1: 0.98 ms with 512 threads, 0.79-0.84 with 256).
// Multiples of 128 bits keep chunk starts 16-byte aligned.
void pick_entropy_config(size_t max_scan_bytes, int *threads, int *subseq_bits) {
    const size_t bits = max_scan_bytes * 8 + 1;
    int nt = 512;
    if (bits <= 128 * 1280) nt = 128;
    else if (bits <= 256 * 1280) nt = 256;
    size_t s = align_up(bits / nt + 1, 128);
    if (s < 512) s = 512;
    // Larger images: one chunk of long subsequences read from global memory (a chunk of 1280-bit
    // subsequences per 655 kbit would serialise dozens of chunks per image); 65535 blocks per
    // subsequence is the kernel's limit, a block has at least 6 bits
    if (s > 256 * 1024) s = 256 * 1024;
    *threads = nt;
    *subseq_bits = (int)s;
}

} // namespace

extern "C" {

int ffcvb_create(int device, int n_slots, int n_threads, ffcvb_ctx **out) {
    if (!out || n_slots < 1 || n_slots > 64) return FFCVB_E_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0 || device < 0 || device >= count)
        return FFCVB_E_NODEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return FFCVB_E_CUDA;
    if (n_threads <= 0) {
        long cores = sysconf(_SC_NPROCESSORS_ONLN);
        n_threads = (int)(cores < 1 ? 1 : (cores > 32 ? 32 : cores));
    }
    ffcvb_ctx *c = new ffcvb_ctx();
    c->device = device;
    c->slots.resize(n_slots);
    for (int i = 0; i < n_slots; i++) c->wait_args.push_back(WaitArg{c, i});
    c->pool = new Pool(n_threads - 1);
    auto env_int = [](const char *name, int lo, int hi) {
        const char *e = getenv(name);
        const int v = e ? atoi(e) : 0;
        return v >= lo && v <= hi ? v : 0;
    };
    c->tune_copy_threads = env_int("FFCV_B200_COPY_THREADS", 1, 256);
    c->tune_subseq_bits = (env_int("FFCV_B200_SUBSEQ_BITS", 128, 256 * 1024) + 127) / 128 * 128;
    c->tune_entropy_threads = env_int("FFCV_B200_ENTROPY_THREADS", 128, 1024);
    if (c->tune_entropy_threads != 128 && c->tune_entropy_threads != 256 && c->tune_entropy_threads != 512 &&
        c->tune_entropy_threads != 1024)
        c->tune_entropy_threads = 0; // only the CTA sizes the kernel is built for
    c->gather_ctas = env_int("FFCV_B200_GATHER_CTAS", 1, 1024);
    if (env_int("FFCV_B200_GATHER_IN_FLIGHT", 4, 4)) c->gather_in_flight = 4;
    *out = c;
    return FFCVB_OK;
}

void ffcvb_destroy(ffcvb_ctx *ctx) {
    if (!ctx) return;
    ctx->pool->wait_all();
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    for (auto &s : ctx->slots) {
        if (s.host) cudaFreeHost(s.host);
        for (DevBuf *b : {&s.blob, &s.clean, &s.coef, &s.planes, &s.rgb, &s.status, &s.ckpt})
            if (b->p) cudaFree(b->p);
        for (auto &e : s.ev)
            if (e) cudaEventDestroy(e);
        if (s.gather_stream) cudaStreamDestroy(s.gather_stream);
        if (s.ev_begin) cudaEventDestroy(s.ev_begin);
        if (s.ev_done) cudaEventDestroy(s.ev_done);
        if (s.ev_gathered) cudaEventDestroy(s.ev_gathered);
        if (s.ev_gather_start) cudaEventDestroy(s.ev_gather_start);
    }
    for (auto &a : ctx->aux) {
        if (a.dev.p) cudaFree(a.dev.p);
        if (a.host) cudaFreeHost(a.host);
        if (a.ev) cudaEventDestroy(a.ev);
    }
    if (ctx->index_pool.p) cudaFree(ctx->index_pool.p);
    if (ctx->index_stats.p) cudaFree(ctx->index_stats.p);
    if (ctx->one_src.p) cudaFree(ctx->one_src.p);
    if (ctx->one_dst.p) cudaFree(ctx->one_dst.p);
    delete ctx->pool;
    delete ctx;
}

const char *ffcvb_last_error(const ffcvb_ctx *ctx) { return ctx ? ctx->err.c_str() : "null context"; }

} // extern "C"

namespace {

// Where a batch's stored bytes come from: a mapping of the file (`base`), or file descriptors the
// staging threads read from straight into the slot's pinned buffer (`fd` buffered, `fd_direct`
// opened with O_DIRECT or -1).
struct Source {
    const uint8_t *base = nullptr;
    int fd = -1, fd_direct = -1;
    bool from_fd() const { return base == nullptr; }
};

// Reads [lo, lo + len) of the file into dst.  With O_DIRECT (offset, length and address are
// multiples of 4096 then) the bytes never enter the page cache; a file system that refuses it at
// read time is served through the buffered descriptor, whose pages are handed back afterwards so
// that resident memory stays bounded by the slot ring.  Returns the bytes read (short at EOF).
size_t read_range(const Source &src, std::atomic<bool> &direct_broken, uint8_t *dst, uint64_t lo, size_t len) {
    size_t done = 0;
    bool use_direct = src.fd_direct >= 0 && !direct_broken.load(std::memory_order_relaxed);
    while (done < len) {
        const ssize_t got = pread(use_direct ? src.fd_direct : src.fd, dst + done, len - done, (off_t)(lo + done));
        if (got < 0) {
            if (errno == EINTR) continue;
            if (use_direct && errno == EINVAL) { // O_DIRECT not supported here after all
                direct_broken.store(true, std::memory_order_relaxed);
                use_direct = false;
                continue;
            }
            break;
        }
        if (got == 0) break; // end of file
        done += (size_t)got;
        if (use_direct && (done & 4095)) break; // a short direct read only happens at the end of the file
    }
    if (!use_direct && done) posix_fadvise(src.fd, (off_t)lo, (off_t)done, POSIX_FADV_DONTNEED);
    return done;
}

int stage_impl(ffcvb_ctx *ctx, int slot, const Source &source, const uint64_t *ptrs,
               const uint64_t *sizes, const uint8_t *modes, const uint16_t *heights,
               const uint16_t *widths, int n, const ffcvb_plan *plan, const int32_t *params) {
    const uint8_t *file_base = source.base;
    const bool from_fd = source.from_fd();
    if (!ctx) return FFCVB_E_ARG;
    if (slot < 0 || slot >= (int)ctx->slots.size() || n <= 0 || (!file_base && source.fd < 0) || !ptrs || !sizes ||
        !modes || !heights || !widths || !params)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_stage_batch: bad argument");
    if (!valid_plan(plan)) return fail(ctx, FFCVB_E_ARG, "ffcvb_stage_batch: invalid plan");
    CU(cudaSetDevice(ctx->device));
    Slot &s = ctx->slots[slot];
    if (s.in_flight) { // normally complete long ago (the caller fences the ring): returns at once
        CU(cudaEventSynchronize(s.ev_done));
        s.in_flight = false;
    }
    s.staged = false;
    s.plan = *plan;
    s.n = n;
    const int n_params = 4 + 2 * plan->n_ops;
    const auto t0 = std::chrono::steady_clock::now();
    // A source that lives in pinned (page-locked, device-mapped) host memory is not copied by the
    // CPU: the GPU gathers the payloads itself.
    uint64_t src_dev_base = 0;
    if (!from_fd) {
        cudaPointerAttributes attr;
        memset(&attr, 0, sizeof(attr));
        if (cudaPointerGetAttributes(&attr, file_base) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
            attr.devicePointer != nullptr)
            src_dev_base = (uint64_t)(uintptr_t)attr.devicePointer;
        else
            cudaGetLastError(); // pageable memory: not an error
    }
    const bool direct = src_dev_base != 0;
    s.direct = direct;
    {   // a copy of this very slot that was never submitted may still be running
        bool done;
        {
            std::lock_guard<std::mutex> g(ctx->copy_m);
            done = s.copy_done;
        }
        if (!done) ctx->pool->wait(Pool::kAsync);
    }
    std::vector<ImageDesc> &descs = s.descs;
    descs.assign(n, ImageDesc{});
    s.src_ptrs.assign(ptrs, ptrs + n);
    s.headers.resize(n);
    s.table_hash.assign((size_t)n * 9, 0);
    s.table_id.assign((size_t)n * 9, 0);
    s.from_cache.assign((size_t)n, 0);

    // ---- reading from file descriptors: every sample's bytes get their place in the pinned buffer
    // before anything is parsed (a JPEG header can only be parsed once it has been read), so the
    // parts of the blob whose size depends on the headers (tables, index lists) follow the payloads.
    // With O_DIRECT a sample is read as the 4 KiB file blocks that contain it, into a 4 KiB aligned
    // place: its first byte sits at the same offset inside a block as in the file.
    struct Span {
        uint64_t lo = 0;   // file offset the read starts at
        size_t len = 0;    // bytes to read
        size_t dst = 0;    // offset in the pinned buffer the read goes to
        size_t skip = 0;   // the sample's first byte is dst + skip
        uint64_t want = 0; // bytes of the sample needed from lo + skip on
    };
    std::vector<Span> spans;
    const int n_params_early = 4 + 2 * plan->n_ops;
    size_t fd_payload_begin = 0, fd_payload_end = 0;
    if (from_fd) {
        const size_t A = source.fd_direct >= 0 && !ctx->direct_broken.load() ? 4096 : kPayloadAlign;
        size_t off = align_up(sizeof(BatchHeader), 16);
        off = align_up(off + sizeof(ImageDesc) * (size_t)n, 16);
        off = align_up(off + sizeof(int32_t) * (size_t)n * n_params_early, 16);
        for (const auto &r : s.pending_riders) off = align_up(off, 64) + r.item_bytes * (uint64_t)n;
        fd_payload_begin = off = align_up(off, A);
        spans.resize(n);
        for (int i = 0; i < n; i++) {
            uint64_t start = ptrs[i], want = sizes[i];
            if (modes[i] != FFCVB_MODE_JPG) {
                int r0 = 0, rows = heights[i];
                const int32_t *p = params + (size_t)i * n_params_early;
                if (plan->resize && p[0] >= 0 && p[2] > 0 && p[0] + p[2] <= (int)heights[i] && p[1] >= 0 && p[3] > 0 &&
                    p[1] + p[3] <= (int)widths[i]) {
                    r0 = p[0];
                    rows = p[2];
                }
                const uint64_t pitch = (uint64_t)widths[i] * 3;
                if (sizes[i] < pitch * heights[i]) rows = 0; // short payload: flagged below, nothing read
                start += (uint64_t)r0 * pitch;
                want = (uint64_t)rows * pitch;
            }
            Span &sp = spans[i];
            sp.want = want;
            sp.lo = start / A * A;
            sp.skip = (size_t)(start - sp.lo);
            sp.len = want ? align_up(sp.skip + want, A) : 0;
            sp.dst = off = align_up(off, A);
            off += sp.len;
        }
        fd_payload_end = off;
        // room behind the payloads for what is laid out after the parse: at most 255 tables of each kind
        size_t tail = 255 * (sizeof(HuffTable) + sizeof(MultTable)) + 3 * (sizeof(int32_t) * (size_t)n + 16) + 256;
        for (int i = 0; i < n; i++) // and the colour kernel's tile table: at most the tiles of whole images
            tail += sizeof(uint2) * (size_t)((((heights[i] + 1) / 2 + 7) / 8) * ((((widths[i] + 1) / 2 + 1) / 2 + 1 + 31) / 32));
        int grc;
        if ((grc = grow_host(ctx, s.host, s.host_cap, fd_payload_end + tail))) return grc;
    }

    // ---- per-sample: parse headers, decide what to stage
    ctx->pool->parallel_for(n, from_fd ? 1 : 8, [&](int i) {
        ImageDesc &d = descs[i];
        memset(&d, 0, sizeof(d));
        d.mode = modes[i];
        d.height = heights[i];
        d.width = widths[i];
        bool short_read = false;
        if (from_fd && spans[i].len) {
            const Span &sp = spans[i];
            const size_t got = read_range(source, ctx->direct_broken, s.host + sp.dst, sp.lo, sp.len);
            short_read = got < sp.skip + sp.want;
        }
        const uint8_t *src = from_fd ? s.host + spans[i].dst + spans[i].skip : file_base + ptrs[i];
        if (modes[i] == FFCVB_MODE_JPG) {
            JpegHeader &h = s.headers[i];
            int rc;
            const auto hit = (short_read || !ctx->cache_headers) ? ctx->header_cache.end() : ctx->header_cache.find(ptrs[i]);
            if (hit != ctx->header_cache.end() && hit->second.size == sizes[i]) {
                // seen before: only the fields the layout needs are restored (the tables are in the store)
                const ffcvb_ctx::CachedHeader &ch = hit->second;
                h.width = ch.width;
                h.height = ch.height;
                h.ncomp = ch.ncomp;
                h.hs[0] = ch.hs;
                h.vs[0] = ch.vs;
                h.scan_off = ch.scan_off;
                h.scan_len = ch.scan_len;
                h.restart_interval = ch.restart_interval;
                for (int k = 0; k < 9; k++) s.table_id[(size_t)i * 9 + k] = ch.table[k];
                s.from_cache[i] = 1;
                rc = 0;
            } else {
                rc = short_read ? kErrData : parse_jpeg_header(src, (size_t)sizes[i], &h);
            }
            if (rc == 0 && (h.width != d.width || h.height != d.height)) rc = kErrDims;
            d.host_status = (int16_t)rc;
            d.payload_size = (uint32_t)sizes[i];
            if (rc == 0) {
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
                // With a crop box only part of the image is needed.  The colour kernels of 4:2:0
                // and 4:4:4 images convert the box alone and reach at most one chroma sample
                // (two pixels, three with an odd edge) beyond it; other layouts convert the whole image.
                const bool boxed = h.ncomp == 3 && ((h.hs[0] == 2 && h.vs[0] == 2 && (h.width + 1) / 2 >= 3) ||
                                                    (h.hs[0] == 1 && h.vs[0] == 1));
                if (plan->resize && boxed) {
                    const int32_t *p = params + (size_t)i * n_params;
                    if (p[0] >= 0 && p[2] > 0 && p[0] + p[2] <= (int)d.height && p[1] >= 0 && p[3] > 0 &&
                        p[1] + p[3] <= (int)d.width) {
                        const int mh = 8 * d.vs, mw = 8 * d.hs;
                        const int y0 = p[0] - 3 < 0 ? 0 : p[0] - 3, x0 = p[1] - 3 < 0 ? 0 : p[1] - 3;
                        const int y1 = p[0] + p[2] + 3 > (int)d.height ? (int)d.height : p[0] + p[2] + 3;
                        const int x1 = p[1] + p[3] + 3 > (int)d.width ? (int)d.width : p[1] + p[3] + 3;
                        d.idct_row0 = (uint16_t)(y0 / mh);
                        d.mcu_rows = (uint16_t)((y1 - 1) / mh + 1);
                        d.idct_col0 = (uint16_t)(x0 / mw);
                        d.idct_col1 = (uint16_t)((x1 - 1) / mw + 1);
                    }
                }
                d.nblocks = (uint32_t)d.bpm * d.mcus_x * d.mcu_rows;
                for (int c = 0; c < h.ncomp && !s.from_cache[i]; c++) {
                    uint64_t *th = &s.table_hash[(size_t)i * 9 + 3 * c];
                    // (bits[17] and vals[256] lie next to each other in RawHuff)
                    static_assert(offsetof(RawHuff, vals) == 17, "RawHuff: vals must follow bits");
                    th[0] = hash_bytes(h.dc[h.td[c]].bits, 17 + 256);
                    th[1] = hash_bytes(h.ac[h.ta[c]].bits, 17 + 256);
                    th[2] = hash_bytes(h.quant[h.tq[c]], 128);
                }
                // scale of the decode (plan->dct_scale): only layouts whose planes end up at one resolution
                const bool scalable = h.ncomp == 3 && ((h.hs[0] == 1 && h.vs[0] == 1) || (h.hs[0] == 2 && h.vs[0] == 2));
                int shift = 0;
                if (plan->dct_scale > 0) {
                    shift = plan->dct_scale;
                    if (!scalable) d.host_status = (int16_t)kErrUnsupported;
                } else if (plan->dct_scale < 0 && scalable) {
                    const int32_t *p = params + (size_t)i * n_params;
                    if (p[0] >= 0 && p[2] > 0 && p[0] + p[2] <= (int)d.height && p[1] >= 0 && p[3] > 0 &&
                        p[1] + p[3] <= (int)d.width)
                        while (shift < 3 && (p[2] >> (shift + 1)) >= plan->out_h && (p[3] >> (shift + 1)) >= plan->out_w) shift++;
                }
                d.scale_shift = (uint8_t)shift;
                d.bs_luma = (uint8_t)(8 >> shift);
                d.bs_chroma = (uint8_t)((8 >> shift) * h.hs[0] > 8 ? 8 : (8 >> shift) * h.hs[0]);
            }
            d.dec_height = (uint16_t)((d.height + (1 << d.scale_shift) - 1) >> d.scale_shift);
            d.dec_width = (uint16_t)((d.width + (1 << d.scale_shift) - 1) >> d.scale_shift);
            if (d.bs_luma == 0) d.bs_luma = d.bs_chroma = 8; // rejected stream: fields stay consistent
        } else {
            d.dec_height = d.height;
            d.dec_width = d.width;
            int r0 = 0, rows = d.height, c0 = 0, cols = d.width;
            if (plan->resize) {
                const int32_t *p = params + (size_t)i * n_params;
                if (p[0] >= 0 && p[2] > 0 && p[0] + p[2] <= (int)d.height && p[1] >= 0 && p[3] > 0 &&
                    p[1] + p[3] <= (int)d.width) {
                    r0 = p[0];
                    rows = p[2];
                    c0 = p[1];
                    cols = p[3];
                }
            }
            const uint64_t need = (uint64_t)d.height * d.width * 3;
            if (sizes[i] < need || short_read) {
                d.host_status = (int16_t)kErrData;
                rows = 0;
            }
            if (from_fd) { // whole rows were read: the crop's columns are picked on the GPU
                c0 = 0;
                cols = d.width;
            }
            d.row0 = (uint16_t)r0;
            d.rows = (uint16_t)rows;
            d.col0 = (uint16_t)c0;
            d.cols = (uint16_t)cols;
            d.raw_pitch = (uint32_t)cols * 3;
            d.payload_size = (uint32_t)((size_t)rows * d.raw_pitch);
            if (direct && rows > 0) d.src_addr = src_dev_base + ptrs[i] + ((uint64_t)r0 * d.width + c0) * 3;
        }
        if (direct && modes[i] == FFCVB_MODE_JPG) d.src_addr = src_dev_base + ptrs[i];
    });

    const auto t1 = std::chrono::steady_clock::now();
    // Split staging: with a pinned source the staging threads (and the copy engine) can carry part
    // of the bytes while the GPU gathers the rest, so that neither path alone has to fill the link.
    // Samples are dealt to the CPU side greedily so that its share of the running byte count holds.
    if (direct && ctx->adaptive_split) {
        // The slot's previous batch tells how long its two halves took: the staging threads' copy
        // (host clock) and the GPU's gather (events).  Move the share towards equal times; the
        // step is small because the measurement is several batches old.
        float tg = 0;
        if (s.gather_timed && cudaEventElapsedTime(&tg, s.ev_gather_start, s.ev_gathered) == cudaSuccess) {
            const double tc = s.staged_end > s.hdr.payload_off ? s.stage_ms[2] : 0.0;
            if (tg + tc > 0) ctx->share += 0.04 * ((double)tg - tc) / ((double)tg + tc);
            if (ctx->share < 0) ctx->share = 0;
            if (ctx->share > 0.5) ctx->share = 0.5;
        } else {
            cudaGetLastError(); // not run yet, or still running: keep the share
        }
        s.gather_timed = false;
        ctx->cpu_share_permille = (int)(ctx->share * 1000 + 0.5);
    }
    if (direct && ctx->cpu_share_permille > 0) {
        uint64_t total = 0, cpu = 0;
        for (int i = 0; i < n; i++) {
            total += descs[i].payload_size;
            if (cpu * 1000 < total * (uint64_t)ctx->cpu_share_permille) {
                cpu += descs[i].payload_size;
                descs[i].src_addr = 0;
            }
        }
    }
    // ---- serial: headers parsed just now enter the cache, their tables the store
    for (int i = 0; i < n; i++) {
        const ImageDesc &d = descs[i];
        if (d.mode != FFCVB_MODE_JPG || d.host_status != 0 || s.from_cache[i]) continue;
        const JpegHeader &h = s.headers[i];
        uint16_t *ids = &s.table_id[(size_t)i * 9];
        bool room = true;
        for (int c = 0; c < h.ncomp; c++) {
            const uint64_t *th = &s.table_hash[(size_t)i * 9 + 3 * c];
            const RawHuff *tabs[2] = {&h.dc[h.td[c]], &h.ac[h.ta[c]]};
            for (int k = 0; k < 2; k++) {
                int found = -1;
                for (int u = (int)ctx->huff_store.size() - 1; u >= 0 && found < 0; u--)
                    if (ctx->huff_store_hash[u] == th[k] && memcmp(ctx->huff_store[u]->bits, tabs[k]->bits, 17) == 0) found = u;
                if (found < 0 && ctx->huff_store.size() < 60000) {
                    found = (int)ctx->huff_store.size();
                    ctx->huff_store.emplace_back(new RawHuff(*tabs[k]));
                    ctx->huff_store_hash.push_back(th[k]);
                }
                room = room && found >= 0;
                ids[3 * c + k] = (uint16_t)(found < 0 ? 0 : found);
            }
            int qfound = -1;
            for (int u = (int)ctx->quant_store.size() - 1; u >= 0 && qfound < 0; u--)
                if (ctx->quant_store_hash[u] == th[2] && (*ctx->quant_store[u])[0] == h.quant[h.tq[c]][0]) qfound = u;
            if (qfound < 0 && ctx->quant_store.size() < 60000) {
                qfound = (int)ctx->quant_store.size();
                ctx->quant_store.emplace_back(new std::array<uint16_t, 64>());
                memcpy(ctx->quant_store.back()->data(), h.quant[h.tq[c]], 128);
                ctx->quant_store_hash.push_back(th[2]);
            }
            room = room && qfound >= 0;
            ids[3 * c + 2] = (uint16_t)(qfound < 0 ? 0 : qfound);
        }
        if (!room) return fail(ctx, FFCVB_E_LIMIT, "more than 60000 distinct Huffman or quantisation tables in a file");
        if (ctx->cache_headers && ctx->header_cache.size() < (size_t)1 << 23) { // ~0.5 GB of host memory at most
            ffcvb_ctx::CachedHeader ch{};
            ch.size = sizes[i];
            ch.scan_off = (uint32_t)h.scan_off;
            ch.scan_len = (uint32_t)h.scan_len;
            ch.restart_interval = (uint16_t)h.restart_interval;
            ch.width = (uint16_t)h.width;
            ch.height = (uint16_t)h.height;
            ch.ncomp = (uint8_t)h.ncomp;
            ch.hs = (uint8_t)h.hs[0];
            ch.vs = (uint8_t)h.vs[0];
            memcpy(ch.table, ids, sizeof(ch.table));
            ctx->header_cache[ptrs[i]] = ch;
        }
    }
    // ---- serial: the batch's own table lists (indices into the store -> indices into the blob)
    std::vector<const RawHuff *> huff_src;
    std::vector<const uint16_t *> mult_src;
    std::vector<int> huff_of_store(ctx->huff_store.size(), -1), mult_of_store(ctx->quant_store.size(), -1);
    std::vector<int32_t> jpeg_list, par_list, seq_list;
    std::vector<uint2> quad_tiles; // (sample, tile x | tile y << 16) of the 4:2:0 colour kernel's CTAs
    size_t clean_bytes = 0, plane_bytes = 0, rgb_bytes = 0, scan_bytes_par = 0;  // scan_bytes_par: largest scan
    uint32_t total_blocks = 0;
    int max_pixels = 0, max_w = 0, max_h = 0, n_quad = 0, n_444 = 0, n_other = 0;
    for (int i = 0; i < n; i++) {
        ImageDesc &d = descs[i];
        if (d.mode != FFCVB_MODE_JPG) continue;
        jpeg_list.push_back(i);
        if (d.host_status != 0) {
            par_list.push_back(i); // the kernel only records the status
            d.block_base = total_blocks;
            continue;
        }
        const JpegHeader &h = s.headers[i];
        const uint16_t *ids = &s.table_id[(size_t)i * 9];
        for (int c = 0; c < h.ncomp; c++) {
            uint8_t *dst[2] = {&d.dc_tab[c], &d.ac_tab[c]};
            for (int k = 0; k < 2; k++) {
                int &slot_of = huff_of_store[ids[3 * c + k]];
                if (slot_of < 0) {
                    slot_of = (int)huff_src.size();
                    huff_src.push_back(ctx->huff_store[ids[3 * c + k]].get());
                }
                *dst[k] = (uint8_t)slot_of;
            }
            int &qslot = mult_of_store[ids[3 * c + 2]];
            if (qslot < 0) {
                qslot = (int)mult_src.size();
                mult_src.push_back(ctx->quant_store[ids[3 * c + 2]]->data());
            }
            d.q_tab[c] = (uint8_t)qslot;
        }
        if (huff_src.size() > 255 || mult_src.size() > 255)
            return fail(ctx, FFCVB_E_LIMIT, "more than 255 distinct Huffman or quantisation tables in a batch");
        d.block_base = total_blocks;
        total_blocks += d.nblocks;
        d.clean_off = clean_bytes;
        clean_bytes += align_up((size_t)d.scan_len + 96, 16);
        if (d.restart_interval) { // table of interval starts behind the clean stream
            d.rst_off = clean_bytes;
            const size_t mcus = (size_t)d.mcus_x * d.mcus_y;
            clean_bytes += align_up(4 * ((mcus + d.restart_interval - 1) / d.restart_interval + 2), 16);
        }
        for (int c = 0; c < h.ncomp; c++) {
            d.plane_off[c] = plane_bytes;
            const size_t pw = (size_t)d.mcus_x * (c == 0 ? d.hs * d.bs_luma : d.bs_chroma);
            const size_t ph = (size_t)d.mcus_y * (c == 0 ? d.vs * d.bs_luma : d.bs_chroma);
            plane_bytes += align_up(pw * ph, 16);
        }
        d.rgb_off = rgb_bytes;
        d.rgb_pitch = (uint32_t)align_up((size_t)d.dec_width * 3, 16);
        rgb_bytes += (size_t)d.dec_height * d.rgb_pitch;
        if ((int)d.dec_height * d.dec_width > max_pixels) max_pixels = (int)d.dec_height * d.dec_width;
        int bw = d.dec_width, bh = d.dec_height;
        {   // extent the colour kernels' grids must cover: the crop box (plus the odd edge of a
            // chroma cell) where the kernel converts only that, else the whole image
            const bool boxed = d.ncomp == 3 && ((d.hs == 2 && d.vs == 2 && (d.width + 1) / 2 >= 3) || (d.hs == 1 && d.vs == 1));
            if (plan->resize && boxed) {
                const int32_t *p = params + (size_t)i * n_params;
                if (p[0] >= 0 && p[2] > 0 && p[0] + p[2] <= (int)d.height && p[1] >= 0 && p[3] > 0 &&
                    p[1] + p[3] <= (int)d.width) {
                    const int sw = (p[3] >> d.scale_shift) + 2, sh = (p[2] >> d.scale_shift) + 2; // the box at the decode's scale
                    bw = sw < bw ? sw : bw;
                    bh = sh < bh ? sh : bh;
                }
            }
            if (bw > max_w) max_w = bw;
            if (bh > max_h) max_h = bh;
        }
        if (d.scale_shift != 0)
            n_444++; // decoded at reduced scale: all planes at one resolution, no upsampling
        else if (d.ncomp == 3 && d.hs == 2 && d.vs == 2 && (d.width + 1) / 2 >= 3) {
            n_quad++;
            // the tiles of 64 x 8 chroma samples (one CTA each) that cover this image's box
            const uint32_t tiles_x = (uint32_t)((((bw + 1) / 2 + 1) / 2 + 1 + 31) / 32), tiles_y = (uint32_t)(((bh + 1) / 2 + 7) / 8);
            for (uint32_t ty = 0; ty < tiles_y; ty++)
                for (uint32_t tx = 0; tx < tiles_x; tx++) quad_tiles.push_back(make_uint2((uint32_t)i, tx | ty << 16));
        } else if (d.ncomp == 3 && d.hs == 1 && d.vs == 1)
            n_444++;
        else
            n_other++;
        if (d.restart_interval) {
            seq_list.push_back(i);
        } else {
            par_list.push_back(i);
            if (d.scan_len > scan_bytes_par) scan_bytes_par = d.scan_len;
        }
    }

    // ---- entropy decode configuration: CTA size and longest subsequence by the batch's largest
    // scan; with a decode index every image gets a subsequence length of its own and its entry
    pick_entropy_config(scan_bytes_par, &s.entropy_threads, &s.subseq_bits);
    if (ctx->tune_subseq_bits) s.subseq_bits = ctx->tune_subseq_bits;
    if (ctx->tune_entropy_threads) s.entropy_threads = ctx->tune_entropy_threads;
    ctx->stage_seq++;
    for (int i : par_list) {
        ImageDesc &d = descs[i];
        d.subseq_bits = (uint32_t)s.subseq_bits;
        d.index_cap = 0;
        d.index_off = 0;
        if (!ctx->index_pool.p || d.host_status != 0) continue;
        // a function of the stream alone (the CTA size its own length would get), so that the
        // recorded states stay usable whatever batch the sample lands in next time
        int own_threads, own_bits;
        pick_entropy_config(d.scan_len, &own_threads, &own_bits);
        const size_t own = (size_t)own_bits;
        d.subseq_bits = (uint32_t)own;
        const uint64_t key = ptrs[i];
        auto it = ctx->index_map.find(key);
        if (it != ctx->index_map.end() && it->second.subseq_bits != d.subseq_bits) {
            // the batch's CTA size changed the subsequence length: the old entry is of no use
            // (its memory stays with the pool); a new one is recorded
            ctx->index_map.erase(it);
            it = ctx->index_map.end();
        }
        if (it == ctx->index_map.end()) {
            const uint32_t cap = (uint32_t)(((size_t)d.scan_len * 8 + own - 1) / own + 2);
            const size_t bytes = decode_index_bytes(cap);
            if (ctx->index_used + bytes > ctx->index_pool.cap) continue; // pool full: this stream stays unindexed
            ffcvb_ctx::IndexEntry e{ctx->index_used, cap, d.subseq_bits, ctx->stage_seq};
            ctx->index_used += bytes;
            it = ctx->index_map.emplace(key, e).first;
        } else if (ctx->stage_seq - it->second.created_seq < ctx->slots.size()) {
            // recorded by a batch that may still be running on another slot's stream: hands off
            continue;
        }
        d.index_off = it->second.off;
        d.index_cap = it->second.cap;
    }

    BatchHeader &hd = s.hdr;
    memset(&hd, 0, sizeof(hd));
    hd.n = (uint32_t)n;
    hd.n_huff = (uint32_t)huff_src.size();
    hd.n_mult = (uint32_t)mult_src.size();
    hd.n_params = (uint32_t)n_params;
    size_t off = align_up(sizeof(BatchHeader), 16);
    hd.desc_off = off;
    off = align_up(off + sizeof(ImageDesc) * (size_t)n, 16);
    auto place_tables = [&] {
        hd.huff_off = off;
        off = align_up(off + sizeof(HuffTable) * huff_src.size(), 16);
        hd.mult_off = off;
        off = align_up(off + sizeof(MultTable) * mult_src.size(), 16);
    };
    auto place_lists = [&] {
        s.jpeg_list_off = off;
        off = align_up(off + sizeof(int32_t) * jpeg_list.size(), 16);
        s.par_list_off = off;
        off = align_up(off + sizeof(int32_t) * par_list.size(), 16);
        s.seq_list_off = off;
        off = align_up(off + sizeof(int32_t) * seq_list.size(), 16);
        s.quad_tiles_off = off;
        off = align_up(off + sizeof(uint2) * quad_tiles.size(), 16);
    };
    if (!from_fd) place_tables();
    hd.params_off = off;
    off = align_up(off + sizeof(int32_t) * (size_t)n * n_params, 16);
    s.riders.swap(s.pending_riders);
    s.pending_riders.clear();
    for (auto &r : s.riders) {
        r.bytes = r.item_bytes * (uint64_t)n;
        if ((!r.inline_bytes.empty() && r.inline_bytes.size() != r.bytes) ||
            (r.inline_bytes.empty() && r.ptrs.size() != (size_t)n)) {
            s.riders.clear();
            return fail(ctx, FFCVB_E_ARG, "ffcvb_stage_batch: a rider was set for a different number of samples");
        }
        r.off = off = align_up(off, 64);
        off += r.bytes;
    }
    off = align_up(off, 16);
    if (from_fd) {
        // the payloads were read into their places before the parse; tables and lists follow them
        if (off > fd_payload_begin) return fail(ctx, FFCVB_E_ARG, "ffcvb_stage_batch: the riders changed while the batch was staged");
        hd.payload_off = fd_payload_begin;
        for (int i = 0; i < n; i++) descs[i].payload_off = spans[i].dst + spans[i].skip;
        off = align_up(fd_payload_end, 16);
        place_tables();
        place_lists();
        s.staged_end = off;
    } else {
        place_lists();
        hd.payload_off = off;
        // payloads the staging threads copy come first: they travel with the head of the blob
        for (int i = 0; i < n; i++) {
            if (descs[i].src_addr != 0) continue;
            descs[i].payload_off = off;
            off = align_up(off + descs[i].payload_size, kPayloadAlign);
        }
        s.staged_end = off;
        for (int i = 0; i < n; i++) {
            ImageDesc &d = descs[i];
            if (d.src_addr == 0) continue;
            // Gathered payloads keep their source alignment mod 16 so that both sides move in whole
            // 16-byte words.  A crop box is fetched row by row: every row gets a 16-byte aligned slot
            // wide enough for the aligned words that contain it, and its pixels start inside the slot
            // at the row's own source alignment (ImageDesc::raw_skew tells the reader).
            const bool rowwise = d.mode == FFCVB_MODE_RAW && d.cols != d.width;
            if (rowwise) {
                d.raw_pitch = (uint32_t)align_up((size_t)d.cols * 3 + 15, 16);
                d.payload_size = (uint32_t)((size_t)d.rows * d.raw_pitch);
                d.raw_skew = 1;
                d.payload_off = off;
            } else {
                d.payload_off = off + (d.src_addr & 15);
            }
            off = align_up(d.payload_off + d.payload_size, kPayloadAlign);
        }
    }
    hd.total_bytes = off;

    int rc;
    // The staging buffer is sized for the whole batch although a pinned source uses only part of
    // it: the part varies from batch to batch, and regrowing page-locked memory stalls the device.
    if (from_fd && off + 64 > s.host_cap) // the payloads already sit in the buffer: it cannot be regrown now
        return fail(ctx, FFCVB_E_ARG, "ffcvb_stage_batch_fd: tables and lists do not fit behind the payloads");
    if ((rc = grow_host(ctx, s.host, s.host_cap, off + 64))) return rc;
    if ((rc = grow_dev(ctx, s.blob, off + 64))) return rc;
    if ((rc = grow_dev(ctx, s.clean, clean_bytes + 64))) return rc;
    if ((rc = grow_dev(ctx, s.coef, (size_t)total_blocks * 128 + 64))) return rc;
    if ((rc = grow_dev(ctx, s.planes, plane_bytes + 64))) return rc;
    if ((rc = grow_dev(ctx, s.rgb, rgb_bytes + 64))) return rc;
    if ((rc = grow_dev(ctx, s.status, sizeof(int32_t) * (size_t)n + 64))) return rc;

    memcpy(s.host, &hd, sizeof(hd));
    memcpy(s.host + hd.desc_off, descs.data(), sizeof(ImageDesc) * (size_t)n);
    for (size_t k = 0; k < huff_src.size(); k++)
        build_huff_table(*huff_src[k], reinterpret_cast<HuffTable *>(s.host + hd.huff_off) + k);
    for (size_t k = 0; k < mult_src.size(); k++)
        build_mult_table(mult_src[k], reinterpret_cast<MultTable *>(s.host + hd.mult_off) + k);
    memcpy(s.host + hd.params_off, params, sizeof(int32_t) * (size_t)n * n_params);
    for (int i = 0; i < n; i++) {
        // a sample decoded at reduced scale: its crop box, for the kernels, is the box of the scaled
        // image that covers it
        const int sh = descs[i].scale_shift;
        if (sh == 0 || !plan->resize) continue;
        int32_t *p = reinterpret_cast<int32_t *>(s.host + hd.params_off) + (size_t)i * n_params;
        const int r0 = p[0] >> sh, c0 = p[1] >> sh;
        int r1 = (p[0] + p[2] + (1 << sh) - 1) >> sh, c1 = (p[1] + p[3] + (1 << sh) - 1) >> sh;
        if (r1 > (int)descs[i].dec_height) r1 = descs[i].dec_height;
        if (c1 > (int)descs[i].dec_width) c1 = descs[i].dec_width;
        p[0] = r0;
        p[1] = c0;
        p[2] = r1 - r0;
        p[3] = c1 - c0;
    }
    for (const auto &r : s.riders) {
        if (!r.inline_bytes.empty()) {
            memcpy(s.host + r.off, r.inline_bytes.data(), r.bytes);
        } else {
            for (int i = 0; i < n; i++) {
                uint8_t *dst = s.host + r.off + (size_t)i * r.item_bytes;
                if (!from_fd) {
                    memcpy(dst, file_base + r.ptrs[i], r.item_bytes);
                } else { // small items: buffered reads
                    size_t done = 0;
                    while (done < r.item_bytes) {
                        const ssize_t got = pread(source.fd, dst + done, r.item_bytes - done, (off_t)(r.ptrs[i] + done));
                        if (got < 0 && errno == EINTR) continue;
                        if (got <= 0) {
                            memset(dst + done, 0, r.item_bytes - done);
                            break;
                        }
                        done += (size_t)got;
                    }
                }
            }
        }
    }
    if (!jpeg_list.empty()) memcpy(s.host + s.jpeg_list_off, jpeg_list.data(), 4 * jpeg_list.size());
    if (!par_list.empty()) memcpy(s.host + s.par_list_off, par_list.data(), 4 * par_list.size());
    if (!seq_list.empty()) memcpy(s.host + s.seq_list_off, seq_list.data(), 4 * seq_list.size());
    if (!quad_tiles.empty()) memcpy(s.host + s.quad_tiles_off, quad_tiles.data(), sizeof(uint2) * quad_tiles.size());
    s.n_quad_tiles = (int)quad_tiles.size();

    const auto t2 = std::chrono::steady_clock::now();
    // ---- parallel: gather the payload bytes into pinned memory
    uint8_t *host = s.host;
    if (!from_fd && s.staged_end > hd.payload_off) {
        Slot *sp = &s; // the job may outlive this call: it only touches slot-owned data and the source
        ctx->pool->wait(Pool::kAsync); // one copy at a time: the batch staged before this one
        int copy_threads = direct ? ctx->split_copy_threads : 0;
        if (ctx->tune_copy_threads) copy_threads = ctx->tune_copy_threads;
        {
            std::lock_guard<std::mutex> g(ctx->copy_m);
            s.copy_done = false;
        }
        ctx->pool->post(
            Pool::kAsync, n, 1,
            [sp, host, file_base](int i) {
                const ImageDesc &d = sp->descs[i];
                if (d.payload_size == 0 || d.src_addr != 0) return;
                const uint8_t *src = file_base + sp->src_ptrs[i];
                uint8_t *dst = host + d.payload_off;
                if (d.mode == FFCVB_MODE_RAW && d.cols != d.width) {
                    // only the crop box travels: one run per row.  Plain copies: streaming stores on
                    // ~1 KB rows leave partial write-combining lines and measured almost twice slower
                    const size_t pitch = (size_t)d.width * 3, run = (size_t)d.cols * 3;
                    src += (size_t)d.row0 * pitch + (size_t)d.col0 * 3;
                    for (int r = 0; r < d.rows; r++) memcpy(dst + r * (size_t)d.raw_pitch, src + r * pitch, run);
                } else {
                    if (d.mode == FFCVB_MODE_RAW) src += (size_t)d.row0 * d.width * 3;
                    stream_copy(dst, src, d.payload_size);
                }
                _mm_sfence(); // streaming stores are weakly ordered: publish them before the copy is reported done
            },
            [ctx, sp, t2] {
                std::lock_guard<std::mutex> g(ctx->copy_m);
                sp->stage_ms[2] = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t2).count();
                sp->copy_done = true;
                ctx->copy_cv.notify_all();
            },
            copy_threads);
        if (!ctx->async_staging) ctx->pool->wait(Pool::kAsync);
    }
    const auto t3 = std::chrono::steady_clock::now();
    auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
    s.stage_ms[0] = ms(t0, t1);
    s.stage_ms[1] = ms(t1, t2);
    if (from_fd || s.staged_end <= hd.payload_off) s.stage_ms[2] = 0; // else: written when the copy completes
    s.stage_ms[3] = ms(t0, t3);
    s.n_jpeg = (int)jpeg_list.size();
    s.n_par = (int)par_list.size();
    s.n_seq = (int)seq_list.size();
    s.total_blocks = total_blocks;
    s.max_pixels = max_pixels;
    s.max_w = max_w;
    s.max_h = max_h;
    s.n_quad = n_quad;
    s.n_444 = n_444;
    s.n_other = n_other;
    s.clean_bytes = clean_bytes;
    s.plane_bytes = plane_bytes;
    s.rgb_bytes = rgb_bytes;
    {
        const size_t need = entropy_checkpoint_bytes((int)par_list.size(), s.entropy_threads, s.subseq_bits);
        if (need && (rc = grow_dev(ctx, s.ckpt, need))) return rc;
    }
    s.scan_bytes = s.raw_bytes = s.jpeg_bytes = 0;
    for (int i = 0; i < n; i++) {
        if (descs[i].mode == FFCVB_MODE_JPG) {
            s.jpeg_bytes += descs[i].payload_size;
            if (descs[i].host_status == 0) s.scan_bytes += descs[i].scan_len;
        } else {
            s.raw_bytes += descs[i].payload_size;
        }
    }
    s.staged = true;
    return FFCVB_OK;
}

} // namespace

extern "C" {

int ffcvb_stage_batch(ffcvb_ctx *ctx, int slot, const uint8_t *file_base, const uint64_t *ptrs,
                      const uint64_t *sizes, const uint8_t *modes, const uint16_t *heights,
                      const uint16_t *widths, int n, const ffcvb_plan *plan, const int32_t *params) {
    if (ctx && !file_base) return fail(ctx, FFCVB_E_ARG, "ffcvb_stage_batch: bad argument");
    Source src;
    src.base = file_base;
    return stage_impl(ctx, slot, src, ptrs, sizes, modes, heights, widths, n, plan, params);
}

int ffcvb_stage_batch_fd(ffcvb_ctx *ctx, int slot, int fd, int fd_direct, const uint64_t *ptrs,
                         const uint64_t *sizes, const uint8_t *modes, const uint16_t *heights,
                         const uint16_t *widths, int n, const ffcvb_plan *plan, const int32_t *params) {
    if (ctx && fd < 0) return fail(ctx, FFCVB_E_ARG, "ffcvb_stage_batch_fd: bad file descriptor");
    Source src;
    src.fd = fd;
    src.fd_direct = fd_direct;
    return stage_impl(ctx, slot, src, ptrs, sizes, modes, heights, widths, n, plan, params);
}

// Stream callback: holds the stream until the staging threads have finished the slot's payload
// copy, so that a batch can be queued while its bytes are still being staged.  Makes no CUDA call.
// The wait is bounded; running out of time is recorded and reported by the next call.
static void CUDART_CB wait_for_copy(void *arg) {
    WaitArg *w = static_cast<WaitArg *>(arg);
    ffcvb_ctx *c = w->ctx;
    std::unique_lock<std::mutex> g(c->copy_m);
    if (!c->copy_cv.wait_for(g, std::chrono::seconds(120), [&] { return c->slots[w->slot].copy_done; }))
        c->copy_timeout.store(true);
}

static int hold_for_copy(ffcvb_ctx *ctx, Slot &s, cudaStream_t st) {
    bool done;
    {
        std::lock_guard<std::mutex> g(ctx->copy_m);
        done = s.copy_done;
    }
    if (!done) CU(cudaLaunchHostFunc(st, wait_for_copy, &ctx->wait_args[&s - ctx->slots.data()]));
    return FFCVB_OK;
}

static int run_batch(ffcvb_ctx *ctx, Slot &s, cudaStream_t st, void *out_dev, bool copy) {
    if (ctx->copy_timeout.load())
        return fail(ctx, FFCVB_E_CUDA, "a payload copy did not finish within its time limit: the batch that waited for it is invalid");
    const BatchHeader &hd = s.hdr;
    uint8_t *blob = (uint8_t *)s.blob.p;
    const bool prof = ctx->profile;
    s.timed = false;
    if (prof) {
        for (auto &e : s.ev)
            if (!e) CU(cudaEventCreate(&e));
        CU(cudaEventRecord(s.ev[0], st));
    }
    int hrc;
    if (copy && !s.direct) {
        if ((hrc = hold_for_copy(ctx, s, st))) return hrc;
        CU(cudaMemcpyAsync(blob, s.host, hd.total_bytes, cudaMemcpyHostToDevice, st));
    } else if (copy) {
        if (!s.gather_stream) {
            int lo = 0, hi = 0;
            CU(cudaDeviceGetStreamPriorityRange(&lo, &hi));
            CU(cudaStreamCreateWithPriority(&s.gather_stream, cudaStreamNonBlocking, hi));
            CU(cudaEventCreateWithFlags(&s.ev_begin, cudaEventDisableTiming));
            CU(cudaEventCreate(&s.ev_gather_start));
            CU(cudaEventCreate(&s.ev_gathered));
        }
        CU(cudaEventRecord(s.ev_begin, st)); // everything the caller ordered before this batch
        CU(cudaStreamWaitEvent(s.gather_stream, s.ev_begin, 0));

        CU(cudaMemcpyAsync(blob, s.host, hd.payload_off, cudaMemcpyHostToDevice, s.gather_stream));
        CU(cudaEventRecord(s.ev_gather_start, s.gather_stream)); // after the head's copy: that one queues behind other batches' transfers
        s.gather_timed = true;
        launch_gather_payloads(reinterpret_cast<const ImageDesc *>(blob + hd.desc_off), s.n, blob, ctx->gather_ctas, ctx->gather_in_flight, s.gather_stream);
        CU(cudaEventRecord(s.ev_gathered, s.gather_stream));
        if (s.staged_end > hd.payload_off) { // the CPU-staged share rides the copy engine meanwhile
            if ((hrc = hold_for_copy(ctx, s, st))) return hrc;
            CU(cudaMemcpyAsync(blob + hd.payload_off, s.host + hd.payload_off, s.staged_end - hd.payload_off,
                               cudaMemcpyHostToDevice, st));
        }
        CU(cudaStreamWaitEvent(st, s.ev_gathered, 0));
    }
    if (copy)
        for (const auto &r : s.riders)
            if (r.bytes) CU(cudaMemcpyAsync(r.dst_dev, blob + r.off, r.bytes, cudaMemcpyDeviceToDevice, st));
    if (prof) CU(cudaEventRecord(s.ev[1], st));
    const ImageDesc *descs = reinterpret_cast<const ImageDesc *>(blob + hd.desc_off);
    const HuffTable *huff = reinterpret_cast<const HuffTable *>(blob + hd.huff_off);
    const MultTable *mult = reinterpret_cast<const MultTable *>(blob + hd.mult_off);
    const int32_t *params = reinterpret_cast<const int32_t *>(blob + hd.params_off);
    int32_t *status = (int32_t *)s.status.p;
    CU(cudaMemsetAsync(status, 0, sizeof(int32_t) * (size_t)s.n, st));
    if (s.n_jpeg > 0) {
        const int32_t *jl = reinterpret_cast<const int32_t *>(blob + s.jpeg_list_off);
        const int32_t *pl = reinterpret_cast<const int32_t *>(blob + s.par_list_off);
        const int32_t *sl = reinterpret_cast<const int32_t *>(blob + s.seq_list_off);
        launch_entropy_decode(descs, pl, s.n_par, sl, s.n_seq, blob, huff, (uint8_t *)s.clean.p,
                              (int16_t *)s.coef.p, status, s.subseq_bits, s.entropy_threads,
                              s.subseq_bits > kMaxStagedBits ? s.ckpt.p : nullptr, (uint8_t *)ctx->index_pool.p,
                              (unsigned long long *)ctx->index_stats.p, st);
        if (prof) CU(cudaEventRecord(s.ev[2], st));
        launch_idct(descs, jl, s.n_jpeg, s.total_blocks, mult, (const int16_t *)s.coef.p,
                    (uint8_t *)s.planes.p, st);
        if (prof) CU(cudaEventRecord(s.ev[3], st));
        launch_color(descs, jl, s.n_jpeg, s.n_quad, s.n_444, s.n_other, s.max_w, s.max_h,
                     reinterpret_cast<const uint2 *>(blob + s.quad_tiles_off), s.n_quad_tiles, (const uint8_t *)s.planes.p,
                     (uint8_t *)s.rgb.p, s.plan.resize ? params : nullptr, (int)hd.n_params, st);
        if (prof) CU(cudaEventRecord(s.ev[4], st));
    } else if (prof) {
        for (int k = 2; k <= 4; k++) CU(cudaEventRecord(s.ev[k], st));
    }
    ResizeSource src{};
    src.descs = descs;
    src.blob = blob;
    src.rgb = (const uint8_t *)s.rgb.p;
    launch_resize_augment(src, s.n, params, (int)hd.n_params, make_oplist(s.plan), s.plan.resize,
                          s.plan.out_h, s.plan.out_w, s.plan.out_kind, s.plan.lut_dev, out_dev, status, st);
    CU(cudaGetLastError());
    if (prof) {
        CU(cudaEventRecord(s.ev[5], st));
        s.timed = true;
    }
    if (!s.ev_done) CU(cudaEventCreateWithFlags(&s.ev_done, cudaEventDisableTiming));
    CU(cudaEventRecord(s.ev_done, st));
    s.in_flight = true;
    return FFCVB_OK;
}

int ffcvb_set_batch_riders(ffcvb_ctx *ctx, int slot, const ffcvb_rider *riders, int n_riders, int n) {
    if (!ctx) return FFCVB_E_ARG;
    if (slot < 0 || slot >= (int)ctx->slots.size() || n_riders < 0 || n_riders > FFCVB_MAX_RIDERS || n <= 0 ||
        (n_riders > 0 && !riders))
        return fail(ctx, FFCVB_E_ARG, "ffcvb_set_batch_riders: bad argument");
    Slot &s = ctx->slots[slot];
    s.pending_riders.clear();
    for (int k = 0; k < n_riders; k++) {
        const ffcvb_rider &in = riders[k];
        if (!in.dst_dev || in.item_bytes == 0 || in.item_bytes > (1u << 24) || (!in.host == !in.ptrs)) {
            s.pending_riders.clear();
            return fail(ctx, FFCVB_E_ARG, "ffcvb_set_batch_riders: rider %d needs a destination, an item size and "
                                          "exactly one of host / ptrs", k);
        }
        Slot::Rider r;
        r.item_bytes = in.item_bytes;
        r.dst_dev = in.dst_dev;
        if (in.host) {
            const uint8_t *b = static_cast<const uint8_t *>(in.host);
            r.inline_bytes.assign(b, b + (size_t)n * in.item_bytes);
        } else {
            r.ptrs.assign(in.ptrs, in.ptrs + n);
        }
        s.pending_riders.push_back(std::move(r));
    }
    return FFCVB_OK;
}

int ffcvb_set_header_cache(ffcvb_ctx *ctx, int enabled) {
    if (!ctx) return FFCVB_E_ARG;
    ctx->pool->wait_all();
    ctx->cache_headers = enabled != 0;
    ctx->header_cache.clear();
    return FFCVB_OK;
}

int ffcvb_set_decode_index(ffcvb_ctx *ctx, uint64_t bytes) {
    if (!ctx) return FFCVB_E_ARG;
    ctx->pool->wait_all();
    CU(cudaSetDevice(ctx->device));
    CU(cudaDeviceSynchronize());
    if (ctx->index_pool.p) {
        CU(cudaFree(ctx->index_pool.p));
        ctx->index_pool = DevBuf{};
    }
    ctx->index_map.clear();
    ctx->index_used = 0;
    if (bytes == 0) return FFCVB_OK;
    bytes = align_up((size_t)bytes, 1 << 20);
    CU(cudaMalloc(&ctx->index_pool.p, (size_t)bytes));
    ctx->index_pool.cap = (size_t)bytes;
    CU(cudaMemset(ctx->index_pool.p, 0, (size_t)bytes)); // no entry is valid yet
    if (!ctx->index_stats.p) {
        CU(cudaMalloc(&ctx->index_stats.p, 64));
        ctx->index_stats.cap = 64;
    }
    CU(cudaMemset(ctx->index_stats.p, 0, 64));
    return FFCVB_OK;
}

int ffcvb_decode_index_stats(ffcvb_ctx *ctx, uint64_t *out) {
    if (!ctx || !out) return FFCVB_E_ARG;
    out[0] = out[1] = 0;
    out[2] = ctx->index_map.size();
    out[3] = ctx->index_used;
    if (!ctx->index_stats.p) return FFCVB_OK;
    CU(cudaSetDevice(ctx->device));
    CU(cudaMemcpy(out, ctx->index_stats.p, 16, cudaMemcpyDeviceToHost));
    return FFCVB_OK;
}

int ffcvb_set_async_staging(ffcvb_ctx *ctx, int enabled) {
    if (!ctx) return FFCVB_E_ARG;
    ctx->pool->wait_all();
    ctx->async_staging = enabled != 0;
    return FFCVB_OK;
}

int ffcvb_set_staging_split(ffcvb_ctx *ctx, int cpu_share_permille) {
    if (!ctx) return FFCVB_E_ARG;
    if (cpu_share_permille < -1 || cpu_share_permille > 1000)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_set_staging_split: share must be 0..1000, or -1");
    ctx->adaptive_split = cpu_share_permille < 0;
    ctx->share = ctx->adaptive_split ? 0.3 : cpu_share_permille / 1000.0;
    ctx->cpu_share_permille = (int)(ctx->share * 1000 + 0.5);
    return FFCVB_OK;
}

int ffcvb_staging_split(const ffcvb_ctx *ctx) { return ctx ? ctx->cpu_share_permille : -1; }

int ffcvb_set_profiling(ffcvb_ctx *ctx, int enabled) {
    if (!ctx) return FFCVB_E_ARG;
    ctx->profile = enabled != 0;
    return FFCVB_OK;
}

int ffcvb_batch_times(ffcvb_ctx *ctx, int slot, float *ms) {
    if (!ctx) return FFCVB_E_ARG;
    if (slot < 0 || slot >= (int)ctx->slots.size() || !ms)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_batch_times: bad argument");
    Slot &s = ctx->slots[slot];
    if (!s.timed) return fail(ctx, FFCVB_E_ARG, "ffcvb_batch_times: slot %d was not run with profiling on", slot);
    CU(cudaSetDevice(ctx->device));
    CU(cudaEventSynchronize(s.ev[5]));
    for (int k = 0; k < 5; k++) CU(cudaEventElapsedTime(&ms[k], s.ev[k], s.ev[k + 1]));
    return FFCVB_OK;
}

int ffcvb_submit_batch(ffcvb_ctx *ctx, int slot, void *stream, void *out_dev) {
    if (!ctx) return FFCVB_E_ARG;
    if (slot < 0 || slot >= (int)ctx->slots.size() || !out_dev)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_submit_batch: bad argument");
    Slot &s = ctx->slots[slot];
    if (!s.staged) return fail(ctx, FFCVB_E_ARG, "ffcvb_submit_batch: slot %d has no staged batch", slot);
    CU(cudaSetDevice(ctx->device));
    return run_batch(ctx, s, (cudaStream_t)stream, out_dev, true);
}

/* Re-runs the kernels of a batch whose bytes a previous ffcvb_submit_batch already put in HBM
 * (no host->device copy).  For measuring the device-resident rate. */
int ffcvb_rerun_batch(ffcvb_ctx *ctx, int slot, void *stream, void *out_dev) {
    if (!ctx) return FFCVB_E_ARG;
    if (slot < 0 || slot >= (int)ctx->slots.size() || !out_dev)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_rerun_batch: bad argument");
    Slot &s = ctx->slots[slot];
    if (!s.staged) return fail(ctx, FFCVB_E_ARG, "ffcvb_rerun_batch: slot %d has no staged batch", slot);
    CU(cudaSetDevice(ctx->device));
    return run_batch(ctx, s, (cudaStream_t)stream, out_dev, false);
}

int64_t ffcvb_staged_bytes(const ffcvb_ctx *ctx, int slot) {
    if (!ctx || slot < 0 || slot >= (int)ctx->slots.size() || !ctx->slots[slot].staged) return -1;
    return (int64_t)ctx->slots[slot].hdr.total_bytes;
}

int ffcvb_stage_times(const ffcvb_ctx *ctx, int slot, double *ms) {
    // (no `staged` check: the figures of the slot's last completed staging stay readable while
    // another thread stages the slot again)
    if (!ctx || !ms || slot < 0 || slot >= (int)ctx->slots.size()) return FFCVB_E_ARG;
    for (int k = 0; k < 4; k++) ms[k] = ctx->slots[slot].stage_ms[k];
    return FFCVB_OK;
}

int ffcvb_gather_time(ffcvb_ctx *ctx, int slot, float *ms) {
    if (!ctx) return FFCVB_E_ARG;
    if (!ms || slot < 0 || slot >= (int)ctx->slots.size()) return fail(ctx, FFCVB_E_ARG, "ffcvb_gather_time: bad argument");
    Slot &s = ctx->slots[slot];
    *ms = -1.0f;
    if (!s.gather_timed) return FFCVB_OK; // this slot's last batch was not gathered by the GPU
    CU(cudaSetDevice(ctx->device));
    CU(cudaEventSynchronize(s.ev_gathered));
    CU(cudaEventElapsedTime(ms, s.ev_gather_start, s.ev_gathered));
    return FFCVB_OK;
}

int ffcvb_batch_info(const ffcvb_ctx *ctx, int slot, int64_t *info) {
    if (!ctx || !info || slot < 0 || slot >= (int)ctx->slots.size() || !ctx->slots[slot].staged) return FFCVB_E_ARG;
    const Slot &s = ctx->slots[slot];
    info[0] = s.n;
    info[1] = s.n_jpeg;
    info[2] = s.total_blocks;
    info[3] = (int64_t)s.scan_bytes;
    info[4] = (int64_t)s.plane_bytes;
    info[5] = (int64_t)s.rgb_bytes;
    info[6] = (int64_t)s.raw_bytes;
    info[7] = (int64_t)s.jpeg_bytes;
    return FFCVB_OK;
}

int ffcvb_batch_launches(const ffcvb_ctx *ctx, int slot) {
    if (!ctx || slot < 0 || slot >= (int)ctx->slots.size() || !ctx->slots[slot].staged) return -1;
    const Slot &s = ctx->slots[slot];
    int k = 1 + (s.direct ? 1 : 0); // fused resize/augment/normalise (+ payload gather)
    if (s.n_jpeg > 0) k += 1 + (s.n_quad > 0) + (s.n_444 > 0) + (s.n_other > 0) + (s.n_par > 0) + (s.n_seq > 0);
    return k;
}

int ffcvb_batch_status(ffcvb_ctx *ctx, int slot, void *stream, int32_t *status, int n) {
    if (!ctx) return FFCVB_E_ARG;
    if (slot < 0 || slot >= (int)ctx->slots.size() || !status || n < 0)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_batch_status: bad argument");
    Slot &s = ctx->slots[slot];
    if (!s.staged || n > s.n) return fail(ctx, FFCVB_E_ARG, "ffcvb_batch_status: nothing staged");
    CU(cudaSetDevice(ctx->device));
    CU(cudaMemcpyAsync(status, s.status.p, sizeof(int32_t) * (size_t)n, cudaMemcpyDeviceToHost,
                       (cudaStream_t)stream));
    CU(cudaStreamSynchronize((cudaStream_t)stream));
    int bad = 0;
    for (int i = 0; i < n; i++) {
        if (status[i] != 0) {
            status[i] = FFCVB_E_DECODE;
            bad++;
        }
    }
    return bad;
}

// Small per-call parameter arrays travel through a ring of sixteen pinned/device buffer pairs: copies
// `bytes` from `host` into the next pair (plus `extra` bytes of uninitialised device scratch behind
// them) on `st`.  The caller records a->ev on `st` once its kernels are queued.
static int stage_aux(ffcvb_ctx *ctx, cudaStream_t st, const void *host, size_t bytes, size_t extra, AuxBuf **out) {
    AuxBuf &a = ctx->aux[ctx->aux_next];
    ctx->aux_next = (ctx->aux_next + 1) % 16;
    if (!a.ev) CU(cudaEventCreateWithFlags(&a.ev, cudaEventDisableTiming));
    if (a.used) CU(cudaEventSynchronize(a.ev));
    int rc;
    if ((rc = grow_dev(ctx, a.dev, bytes + extra))) return rc;
    if ((rc = grow_host(ctx, a.host, a.host_cap, bytes))) return rc;
    memcpy(a.host, host, bytes);
    CU(cudaMemcpyAsync(a.dev.p, a.host, bytes, cudaMemcpyHostToDevice, st));
    *out = &a;
    return FFCVB_OK;
}

int ffcvb_transform_device(ffcvb_ctx *ctx, void *stream, const uint8_t *src_dev, int n, int h, int w,
                           const ffcvb_plan *plan, const int32_t *params, void *out_dev) {
    if (!ctx) return FFCVB_E_ARG;
    if (!src_dev || n <= 0 || h <= 0 || w <= 0 || !params || !out_dev || !valid_plan(plan))
        return fail(ctx, FFCVB_E_ARG, "ffcvb_transform_device: bad argument");
    CU(cudaSetDevice(ctx->device));
    cudaStream_t st = (cudaStream_t)stream;
    const int n_params = 4 + 2 * plan->n_ops;
    const size_t bytes = sizeof(int32_t) * (size_t)n * n_params;
    AuxBuf *ap;
    int rc;
    if ((rc = stage_aux(ctx, st, params, bytes, 0, &ap))) return rc;
    AuxBuf &a = *ap;
    ResizeSource src{};
    src.uniform = src_dev;
    src.uniform_h = h;
    src.uniform_w = w;
    launch_resize_augment(src, n, (const int32_t *)a.dev.p, n_params, make_oplist(*plan), plan->resize,
                          plan->out_h, plan->out_w, plan->out_kind, plan->lut_dev, out_dev, nullptr, st);
    CU(cudaGetLastError());
    CU(cudaEventRecord(a.ev, st));
    a.used = true;
    return FFCVB_OK;
}

int ffcvb_color_jitter(ffcvb_ctx *ctx, void *stream, uint8_t *images_dev, int n, int h, int w, int kind,
                       const uint8_t *apply, const double *ratio) {
    if (!ctx) return FFCVB_E_ARG;
    if (!images_dev || n <= 0 || h <= 0 || w <= 0 || kind < 0 || kind > 2 || !apply || !ratio ||
        (int64_t)h * w > (int64_t)1 << 30)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_color_jitter: bad argument");
    CU(cudaSetDevice(ctx->device));
    cudaStream_t st = (cudaStream_t)stream;
    // [ratio: n doubles][apply: n bytes, padded][grey sums: n counters (device only)]
    const size_t apply_off = sizeof(double) * (size_t)n, sums_off = align_up(apply_off + n, 8);
    std::vector<uint8_t> pack(sums_off, 0);
    memcpy(pack.data(), ratio, sizeof(double) * (size_t)n);
    memcpy(pack.data() + apply_off, apply, (size_t)n);
    AuxBuf *a;
    int rc;
    if ((rc = stage_aux(ctx, st, pack.data(), sums_off, sizeof(unsigned long long) * (size_t)n, &a))) return rc;
    uint8_t *dev = (uint8_t *)a->dev.p;
    launch_color_jitter(images_dev, n, h, w, kind, dev + apply_off, (const double *)dev,
                        (unsigned long long *)(dev + sums_off), st);
    CU(cudaGetLastError());
    CU(cudaEventRecord(a->ev, st));
    a->used = true;
    return FFCVB_OK;
}

int ffcvb_mixup(ffcvb_ctx *ctx, void *stream, const uint8_t *src_dev, uint8_t *dst_dev, int n, int64_t count,
                const double *lam) {
    if (!ctx) return FFCVB_E_ARG;
    if (!src_dev || !dst_dev || src_dev == dst_dev || n <= 0 || count <= 0 || !lam)
        return fail(ctx, FFCVB_E_ARG, "ffcvb_mixup: bad argument");
    for (int i = 0; i < n; i++)
        if (!(lam[i] >= 0.0 && lam[i] <= 1.0)) return fail(ctx, FFCVB_E_ARG, "ffcvb_mixup: lam[%d] outside [0, 1]", i);
    CU(cudaSetDevice(ctx->device));
    cudaStream_t st = (cudaStream_t)stream;
    AuxBuf *a;
    int rc;
    if ((rc = stage_aux(ctx, st, lam, sizeof(double) * (size_t)n, 0, &a))) return rc;
    launch_mixup(src_dev, dst_dev, n, (long long)count, (const double *)a->dev.p, st);
    CU(cudaGetLastError());
    CU(cudaEventRecord(a->ev, st));
    a->used = true;
    return FFCVB_OK;
}

int ffcvb_poison(ffcvb_ctx *ctx, void *stream, uint8_t *images_dev, int n, int64_t count, const uint8_t *apply,
                 const double *one_minus_alpha_dev, const double *mask_dev, double clamp_lo, double clamp_hi) {
    if (!ctx) return FFCVB_E_ARG;
    if (!images_dev || n <= 0 || count <= 0 || !apply || !one_minus_alpha_dev || !mask_dev || !(clamp_lo <= clamp_hi))
        return fail(ctx, FFCVB_E_ARG, "ffcvb_poison: bad argument");
    CU(cudaSetDevice(ctx->device));
    cudaStream_t st = (cudaStream_t)stream;
    AuxBuf *a;
    int rc;
    if ((rc = stage_aux(ctx, st, apply, (size_t)n, 0, &a))) return rc;
    launch_poison(images_dev, n, (long long)count, (const uint8_t *)a->dev.p, one_minus_alpha_dev, mask_dev,
                  (float)clamp_lo, (float)clamp_hi, st);
    CU(cudaGetLastError());
    CU(cudaEventRecord(a->ev, st));
    a->used = true;
    return FFCVB_OK;
}

int ffcvb_host_register(void *ptr, uint64_t bytes) {
    if (!ptr || bytes == 0) return FFCVB_E_ARG;
    if (cudaHostRegister(ptr, (size_t)bytes, cudaHostRegisterDefault) != cudaSuccess) {
        cudaGetLastError(); // refused (a read-only mapping, a file on disk): not an error of the process
        return FFCVB_E_CUDA;
    }
    return FFCVB_OK;
}

int ffcvb_host_unregister(void *ptr) {
    if (!ptr) return FFCVB_E_ARG;
    // gather kernels and copies that still read the range must be through before it is released
    cudaDeviceSynchronize();
    if (cudaHostUnregister(ptr) != cudaSuccess) {
        cudaGetLastError();
        return FFCVB_E_CUDA;
    }
    return FFCVB_OK;
}

// ------------------------------------------------------------ reference-signature entry points

static ffcvb_ctx *g_ctx = nullptr;
static std::mutex g_mutex;

static ffcvb_ctx *global_ctx() {
    if (!g_ctx) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
        if (ffcvb_create(dev, 1, 1, &g_ctx) != FFCVB_OK) return nullptr;
    }
    return g_ctx;
}

int imdecode(unsigned char *input_buffer, uint64_t input_size, uint32_t source_height,
             uint32_t source_width, unsigned char *output_buffer, uint32_t crop_height,
             uint32_t crop_width, uint32_t offset_x, uint32_t offset_y, uint32_t scale_num,
             uint32_t scale_denom, bool enable_crop, bool hflip) {
    (void)source_height;
    (void)source_width;
    (void)offset_x;
    (void)offset_y;
    // Every call the reference makes passes the identity transform and scale 1/1
    // (rgb_image.py:131-132,196-197).  Scales 1/2, 1/4 and 1/8 are decoded too: as in the reference's
    // call, the output then has TJSCALED(crop, scale) = ceil(crop * num / denom) pixels a side.
    if (enable_crop || hflip || !input_buffer || !output_buffer || scale_num == 0 || scale_denom % scale_num != 0) return -1;
    const uint32_t denom = scale_denom / scale_num;
    if (denom != 1 && denom != 2 && denom != 4 && denom != 8) return -1;
    const int shift = denom == 1 ? 0 : (denom == 2 ? 1 : (denom == 4 ? 2 : 3));
    std::lock_guard<std::mutex> g(g_mutex);
    ffcvb_ctx *ctx = global_ctx();
    if (!ctx) return -1;
    if (crop_height == 0 || crop_width == 0 || crop_height > 65535 || crop_width > 65535) return -1;
    ffcvb_plan plan{};
    plan.out_h = (int32_t)((crop_height + denom - 1) / denom);
    plan.out_w = (int32_t)((crop_width + denom - 1) / denom);
    plan.resize = 0;
    plan.dct_scale = shift;
    plan.out_kind = FFCVB_OUT_U8_NHWC;
    const uint64_t ptr = 0, size = input_size;
    const uint8_t mode = FFCVB_MODE_JPG;
    const uint16_t hh = (uint16_t)crop_height, ww = (uint16_t)crop_width;
    const int32_t params[4] = {0, 0, (int32_t)crop_height, (int32_t)crop_width};
    if (ffcvb_stage_batch(ctx, 0, input_buffer, &ptr, &size, &mode, &hh, &ww, 1, &plan, params)) return -1;
    const size_t out_bytes = (size_t)plan.out_h * plan.out_w * 3;
    if (grow_dev(ctx, ctx->one_dst, out_bytes)) return -1;
    if (ffcvb_submit_batch(ctx, 0, nullptr, ctx->one_dst.p)) return -1;
    int32_t status = 0;
    if (ffcvb_batch_status(ctx, 0, nullptr, &status, 1) != 0) return -1;
    if (cudaMemcpy(output_buffer, ctx->one_dst.p, out_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return 0;
}

void resize(int64_t cresizer, int64_t source_p, int64_t sx, int64_t sy, int64_t start_row,
            int64_t end_row, int64_t start_col, int64_t end_col, int64_t dest_p, int64_t tx, int64_t ty) {
    (void)cresizer;
    std::lock_guard<std::mutex> g(g_mutex);
    ffcvb_ctx *ctx = global_ctx();
    if (!ctx || !source_p || !dest_p || sx <= 0 || sy <= 0 || tx <= 0 || ty <= 0) return;
    if (start_row < 0 || start_col < 0 || end_row > sx || end_col > sy || end_row <= start_row ||
        end_col <= start_col)
        return;
    // Only the rows of the region travel to the GPU.
    const int rows = (int)(end_row - start_row);
    const size_t src_bytes = (size_t)rows * sy * 3, dst_bytes = (size_t)tx * ty * 3;
    if (grow_dev(ctx, ctx->one_src, src_bytes) || grow_dev(ctx, ctx->one_dst, dst_bytes)) return;
    const uint8_t *src = (const uint8_t *)(intptr_t)source_p + (size_t)start_row * sy * 3;
    if (cudaMemcpy(ctx->one_src.p, src, src_bytes, cudaMemcpyHostToDevice) != cudaSuccess) return;
    ffcvb_plan plan{};
    plan.out_h = (int32_t)tx;
    plan.out_w = (int32_t)ty;
    plan.resize = 1;
    plan.out_kind = FFCVB_OUT_U8_NHWC;
    const int32_t params[4] = {0, (int32_t)start_col, rows, (int32_t)(end_col - start_col)};
    if (ffcvb_transform_device(ctx, nullptr, (const uint8_t *)ctx->one_src.p, 1, rows, (int)sy, &plan, params,
                               ctx->one_dst.p))
        return;
    cudaMemcpy((void *)(intptr_t)dest_p, ctx->one_dst.p, dst_bytes, cudaMemcpyDeviceToHost);
}

void my_memcpy(void *source, void *dst, uint64_t size) { memcpy(dst, source, size); }

void my_fread(int64_t fp, int64_t offset, void *destination, int64_t size) {
    FILE *f = reinterpret_cast<FILE *>(static_cast<intptr_t>(fp));
    if (!f || !destination || size <= 0 || offset < 0) return;
    if (fseek(f, (long)offset, SEEK_SET) != 0) return;
    size_t got = fread(destination, 1, (size_t)size, f);
    (void)got;
}

} // extern "C"
