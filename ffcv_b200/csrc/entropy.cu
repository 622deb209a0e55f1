// Batched baseline-JPEG entropy decode (ITU-T T.81 F.2) for sm_100a.
//
// One CTA per image.  The scan has no restart markers in FFCV-written files
// (ffcv/fields/rgb_image.py:26-34 passes only the quality to cv2.imencode), so parallelism inside
// an image comes from the self-synchronising property of Huffman codes: the unstuffed bit stream
// is cut into fixed-length subsequences, every thread decodes its subsequence from a guessed
// state, and the guesses are repaired by re-decoding from the left neighbour's exit state until
// no input changes (a Jacobi iteration on a chain whose first link is exact, so it converges in
// a few rounds in practice -- about 7 kbit of stream, dominated by the block's slot inside the
// MCU -- and in at most one round per subsequence in the worst case).  A prefix sum
// of completed blocks then gives every thread its output position and a last pass writes the
// coefficients.  DC differences are integrated per component by a block-wide scan.
//
// Integer / issue-bound work: tables live in shared memory, no tensor cores.
#include "kernels.h"

namespace ffcvb {


// Exclusive prefix sum over the block; `total` receives the block sum.  s_warp holds 33 ints.
__device__ __forceinline__ int block_scan_exclusive(int v, int *s_warp, int &total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < nwarps ? s_warp[lane] : 0;
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        s_warp[lane] = winc - w;
        if (lane == 31) s_warp[32] = winc;
    }
    __syncthreads();
    int r = inc - v + s_warp[warp];
    total = s_warp[32];
    __syncthreads();
    return r;
}

// 32 bits of the bit stream starting at bit p.  The unstuffed stream is stored as 32-bit words
// whose most significant bit comes first, so two word loads and one funnel shift do it.
__device__ __forceinline__ uint32_t peek32(const uint32_t *__restrict__ words, uint32_t p) {
    const uint32_t i = p >> 5;
    return __funnelshift_l(words[i + 1], words[i], p);
}

// A 96-bit window over the stream kept in registers: hi holds the word the current position lies
// in, lo the next one, nx the one after.  Looking at the next 32 bits is one funnel shift, and the
// stream is touched once per 32 bits consumed (a predicated load, issued a symbol or more before
// its value is needed) instead of twice per symbol, which takes the stream's load latency out of
// the chain symbol -> table look-up -> next symbol.  Lanes never diverge: advancing is a select.
struct BitWindow {
    const uint32_t *__restrict__ w;
    uint32_t wi, r, hi, lo, nx;
    __device__ __forceinline__ BitWindow(const uint32_t *__restrict__ words, uint32_t p) : w(words), wi(p >> 5), r(p & 31) {
        hi = w[wi];
        lo = w[wi + 1];
        nx = w[wi + 2];
    }
    __device__ __forceinline__ uint32_t peek() const { return __funnelshift_l(lo, hi, r); }
    // consume n < 32 bits
    __device__ __forceinline__ void skip(uint32_t n) {
        r += n;
        const bool adv = r >= 32;
        hi = adv ? lo : hi;
        lo = adv ? nx : lo;
        wi += adv ? 1u : 0u;
        r &= 31;
        if (adv) nx = w[wi + 2];
    }
};

// Entry (see HuffTable) of the Huffman code at the top of w: at most two dependent table reads.
// An invalid code consumes 16 bits and acts as an end of block, so that speculative decoding
// always makes progress.
__device__ __forceinline__ uint32_t huff_lookup(const HuffTable &t, uint32_t w) {
    uint32_t e = t.look[w >> 23];
    if (e & 0x8000u) {
        if (e != 0xFFFFu) {
            e = t.sub[e & 0x7fffu][(w >> 16) & 127];
        } else {
            // more long-code prefixes than sub-tables (never with the tables encoders emit)
            const int code = w >> 16;
            e = 16u | (63u << 9); // no code at all: a 16-bit end of block
#pragma unroll 1
            for (int l = 10; l <= 16; l++) {
                const int c = code >> (16 - l);
                if (c <= t.maxcode[l]) {
                    e = huff_entry(l, t.vals[(t.valoff[l] + c) & 255]);
                    break;
                }
            }
        }
    }
    return e;
}

__device__ __forceinline__ int extend(uint32_t bits, int s) {
    // bits: the s-bit magnitude field (s >= 1)
    return bits < (1u << (s - 1)) ? (int)bits - (1 << s) + 1 : (int)bits;
}

struct Cursor {
    uint32_t p; // bit position in the unstuffed stream
    int c;      // block slot inside the MCU
    int z;      // next zigzag index, 0 = DC expected
};

__device__ __forceinline__ uint64_t pack(const Cursor &s) {
    return ((uint64_t)s.p << 32) | ((uint32_t)s.c << 8) | (uint32_t)s.z;
}
__device__ __forceinline__ Cursor unpack(uint64_t v) {
    Cursor s;
    s.p = (uint32_t)(v >> 32);
    s.c = (int)((v >> 8) & 0xffffff);
    s.z = (int)(v & 0xff);
    return s;
}

// Decodes symbols from `cur` until its position reaches `end`.  Returns the number of blocks
// completed.  With WRITE, coefficients go to cf (image base) starting at block `blk`.
// `words` holds the stream from bit `bit_base` on (the chunk's copy in shared memory).
// The 32 lanes of a warp walk unrelated parts of the stream, so the step is written as straight
// line code with selects (DC / AC / end-of-block / zero-run / block end all take the same path);
// codes longer than the 9-bit first-level table cost one more table read.
template <bool WRITE>
__device__ __forceinline__ int decode_span(const uint32_t *__restrict__ words, uint32_t bit_base, Cursor &cur,
                                           uint32_t end, int bpm, int luma, int ncomp,
                                           const HuffTable *s_tab,
                                           int16_t *__restrict__ cf, uint32_t blk,
                                           uint32_t nblocks) {
    int done = 0;
    uint32_t p = cur.p;
    int c = cur.c, z = cur.z;
    int comp2 = (ncomp == 1 || c < luma) ? 0 : 2 * (c - luma + 1);
    int16_t *out = cf + (size_t)blk * 64;
    if (p >= end) return 0;
    // Coefficients are stored in the order they are decoded (zig-zag order inside a block; the
    // inverse transform undoes it when it loads the block), which lets a thread collect the four
    // coefficients of an aligned group of zig-zag positions in a register and store them with one
    // 8-byte store: a block's ~15 non-zero coefficients sit in ~5 such groups, and scattered stores
    // are what the write pass is bound by.  Only a block this thread decodes from its first symbol
    // is packed: a block shared with a neighbouring subsequence is written coefficient by
    // coefficient, so that the two threads never touch the same bytes.
    bool packing = z == 0;
    int group = -1; // group of four positions held in `held`, -1: none
    unsigned long long held = 0;
    BitWindow win(words, p - bit_base);
    while (p < end) {
        const uint32_t w = win.peek();
        const bool dc = z == 0;
        const HuffTable &t = s_tab[comp2 + (dc ? 0 : 1)];
        const uint32_t e = huff_lookup(t, w);
        const int n = e & 31, s = (e >> 5) & 15;
        const int zn = dc ? 1 : z + (int)(e >> 9); // DC: on to the first AC position
        if (WRITE) {
            // where this symbol's coefficient goes, if it has one
            const int zpos = zn - 1;
            if (s != 0 && zpos < 64 && blk < nblocks) {
                const int v = extend((w << (n - s)) >> (32 - s), s);
                if (packing) {
                    const int g = zpos >> 2;
                    if (g != group) {
                        if (group >= 0) *reinterpret_cast<unsigned long long *>(out + 4 * group) = held;
                        group = g;
                        held = 0;
                    }
                    held |= (unsigned long long)(uint16_t)v << (16 * (zpos & 3));
                } else {
                    out[zpos] = (int16_t)v;
                }
            }
        }
        p += n;
        win.skip(n);
        const bool eob = zn >= 64;
        z = eob ? 0 : zn;
        done += eob ? 1 : 0;
        if (WRITE) {
            if (eob) {
                if (group >= 0) *reinterpret_cast<unsigned long long *>(out + 4 * group) = held;
                group = -1;
                packing = true;
            }
            blk += eob ? 1 : 0;
            out += eob ? 64 : 0;
        }
        c = eob ? ((c + 1 == bpm) ? 0 : c + 1) : c;
        comp2 = (ncomp == 1 || c < luma) ? 0 : 2 * (c - luma + 1);
    }
    if (WRITE && group >= 0) {
        // the subsequence ends inside a block: the next thread continues it, so only the
        // coefficients themselves are written
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t lane = (uint32_t)(held >> (16 * k)) & 0xffffu;
            if (lane) out[4 * group + k] = (int16_t)lane;
        }
    }
    cur.p = p;
    cur.c = c;
    cur.z = z;
    return done;
}

// Counting walk for long subsequences (the variant that reads the stream from global memory).
// A re-decode of a long subsequence from a corrected entry state soon runs exactly where the
// previous decode ran: the two walks merge once position, slot and zig-zag index coincide.  Every
// walk therefore leaves its state at check-points every `ck_bits` bits; a later walk that finds
// the same state at a check-point stops there -- the exit state stands and the block count is its
// own count so far plus what the previous walk counted from that check-point to the end.  The repair pass
// of a multi-megabit image then costs the re-synchronisation distance, not the whole subsequence.
struct CheckPoint {
    unsigned long long state; // pack(position, slot, zig-zag index)
    uint32_t rest;            // blocks the walk completed from here to the end of the subsequence
    uint32_t pad;
};

template <bool COMPARE>
__device__ __forceinline__ int count_span_checked(const uint32_t *__restrict__ words, Cursor &cur, uint32_t start,
                                                  uint32_t end, int bpm, int luma, int ncomp,
                                                  const HuffTable *s_tab, CheckPoint *__restrict__ ck, uint32_t ck_bits,
                                                  bool &merged) {
    int done = 0;
    uint32_t p = cur.p;
    int c = cur.c, z = cur.z;
    int comp2 = (ncomp == 1 || c < luma) ? 0 : 2 * (c - luma + 1);
    const uint32_t k0 = (p - start) / ck_bits;
    uint32_t k = k0;
    uint32_t next_ck = start + (k + 1) * ck_bits;
    int total = -1;
    merged = false;
    BitWindow win(words, p < end ? p : 0);
    while (p < end) {
        const uint32_t w = win.peek();
        const bool dc = z == 0;
        const HuffTable &t = s_tab[comp2 + (dc ? 0 : 1)];
        const uint32_t e = huff_lookup(t, w);
        const int zn = dc ? 1 : z + (int)(e >> 9);
        p += e & 31;
        win.skip(e & 31);
        const bool eob = zn >= 64;
        z = eob ? 0 : zn;
        done += eob ? 1 : 0;
        c = eob ? ((c + 1 == bpm) ? 0 : c + 1) : c;
        comp2 = (ncomp == 1 || c < luma) ? 0 : 2 * (c - luma + 1);
        if (p >= next_ck && p < end) {
            Cursor here = {p, c, z};
            const unsigned long long st = pack(here);
            if (COMPARE && ck[k].state == st) {
                merged = true; // from here on this walk is the previous one
                total = done + (int)ck[k].rest;
                break;
            }
            ck[k].state = st;
            ck[k].rest = (uint32_t)done; // blocks so far; turned into blocks-to-the-end below
            k++;
            next_ck += ck_bits;
        }
    }
    if (!merged) {
        total = done;
        cur.p = p;
        cur.c = c;
        cur.z = z;
    }
    for (uint32_t j = k0; j < k; j++) ck[j].rest = (uint32_t)total - ck[j].rest;
    return total;
}

// kStaged: the chunk's bits are copied to shared memory first (subsequences of up to 1280 bits);
// otherwise the threads read the unstuffed stream in global memory, which allows subsequences of
// any length: a multi-megabit image is then one chunk of kEntropyThreads long subsequences that
// re-synchronise in two or three (long, fully parallel) rounds instead of dozens of chunks that
// wait for one another.
template <int kEntropyThreads, bool kStaged>
// (resident CTAs per SM: shared memory -- 27 KB of tables plus the stream -- allows 2 CTAs of 512
// threads, 3 of 256 and 4 of 128 in the staged variants, so the register budget is set for those
// counts rather than for full thread occupancy)
__global__ void __launch_bounds__(kEntropyThreads, kEntropyThreads >= 1024 ? 1 : (kEntropyThreads == 512 ? 2 : (kEntropyThreads == 256 ? 4 : 6)))
entropy_parallel_kernel(const ImageDesc *__restrict__ descs, const int32_t *__restrict__ list,
                        const uint8_t *__restrict__ blob, const HuffTable *__restrict__ huff,
                        uint8_t *__restrict__ clean, int16_t *__restrict__ coef,
                        int32_t *__restrict__ status, int subseq_bits, CheckPoint *__restrict__ ckpt, int ck_bits,
                        uint8_t *__restrict__ index_pool, unsigned long long *__restrict__ index_stats) {
    extern __shared__ __align__(16) uint32_t s_stream[]; // this chunk of the unstuffed stream
    __shared__ HuffTable s_tab[6];
    __shared__ unsigned long long s_state[kEntropyThreads + 1];
    __shared__ uint16_t s_blocks[kEntropyThreads]; // blocks completed inside each subsequence
    __shared__ uint16_t s_list[kEntropyThreads];   // compacted indices of the dirty subsequences
    __shared__ uint8_t s_dirty[kEntropyThreads + 1];
    __shared__ int s_warp[33];
    __shared__ uint32_t s_ix[2]; // decisions about the decode index, taken by one thread for the whole CTA

    const int img = list[blockIdx.x];
    const ImageDesc d = descs[img];
    const int tid = threadIdx.x;
    if (d.host_status != 0) {
        if (tid == 0) status[img] = d.host_status;
        return;
    }
    // ---- tables into shared memory
    for (int c = 0; c < d.ncomp; c++) {
        const uint32_t *sd = reinterpret_cast<const uint32_t *>(&huff[d.dc_tab[c]]);
        const uint32_t *sa = reinterpret_cast<const uint32_t *>(&huff[d.ac_tab[c]]);
        uint32_t *dd = reinterpret_cast<uint32_t *>(&s_tab[2 * c]);
        uint32_t *da = reinterpret_cast<uint32_t *>(&s_tab[2 * c + 1]);
        for (int i = tid; i < (int)(sizeof(HuffTable) / 4); i += kEntropyThreads) {
            dd[i] = sd[i];
            da[i] = sa[i];
        }
    }

    // ---- remove byte stuffing (FF 00 -> FF) into the clean stream.  When the whole scan fits the
    // shared-memory stream buffer (the usual case: the subsequence length is chosen so that the
    // largest image of the batch is one chunk) the clean stream is built there and never touches
    // global memory; otherwise it goes to the scratch buffer and is staged chunk by chunk.
    const uint8_t *scan = blob + d.payload_off + d.scan_off;
    const uint32_t stream_bytes = kStaged ? ((uint32_t)kEntropyThreads * (uint32_t)subseq_bits / 8 + 63) / 16 * 16 + 16 : 0;
    const bool resident = kStaged && d.scan_len + 80 <= stream_bytes; // 64 zero bytes follow the stream
    uint8_t *cl = resident ? reinterpret_cast<uint8_t *>(s_stream) : clean + d.clean_off;
    uint32_t clean_len = 0, flush_base = 0;
    // Every thread takes one aligned 16-byte word of the scan per pass (one load instead of sixteen);
    // the byte before it, which decides whether a leading 00 is stuffing, comes from the lane below.
    const uint32_t lead = (uint32_t)(reinterpret_cast<uintptr_t>(scan) & 15); // bytes of the first word before the scan
    const uint4 *scan16 = reinterpret_cast<const uint4 *>(scan - lead);
    for (uint32_t base = 0; base < d.scan_len + lead; base += kEntropyThreads * 16) {
        const uint32_t chunk = base + tid * 16;         // offset of this thread's word from scan - lead
        const int my = (int)chunk - (int)lead;           // scan offset of its first byte (negative in the first word)
        uint4 v = make_uint4(0, 0, 0, 0);
        if (chunk < d.scan_len + lead) v = scan16[chunk >> 4];
        const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
        uint8_t b[16];
#pragma unroll
        for (int i = 0; i < 16; i++) b[i] = (uint8_t)(wv[i >> 2] >> (8 * (i & 3)));
        int prev = __shfl_up_sync(0xffffffffu, (int)b[15], 1);
        if ((tid & 31) == 0) prev = (my > 0 && my <= (int)d.scan_len) ? scan[my - 1] : 0;
        uint32_t keep = 0;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int at = my + i;
            const bool inside = at >= 0 && at < (int)d.scan_len;
            if (inside && !(b[i] == 0 && prev == 0xFF)) keep |= 1u << i;
            prev = inside ? b[i] : 0;
        }
        int total;
        int off = block_scan_exclusive(__popc(keep), s_warp, total);
        // byte k of the stream lives at address k ^ 3: every 32-bit word holds its bits MSB first
        uint32_t o = clean_len + off;
        if (kStaged) {
            // into the stream buffer in shared memory (or, for the rare scan that does not fit it,
            // byte by byte into the scratch buffer)
#pragma unroll
            for (int i = 0; i < 16; i++)
                if (keep & (1u << i)) cl[(o++) ^ 3u] = b[i];
        } else {
            // The variant for multi-megabit scans keeps the stream in global memory: it is collected
            // in shared memory first and leaves as whole 16-byte vectors, one store per 16 bytes
            // instead of one per byte.  flush_base (a multiple of 16) is the stream
            // position of the buffer's first byte; fewer than 16 bytes stay behind per pass.
            uint8_t *buf = reinterpret_cast<uint8_t *>(s_stream);
#pragma unroll
            for (int i = 0; i < 16; i++)
                if (keep & (1u << i)) buf[((o++) - flush_base) ^ 3u] = b[i];
            __syncthreads();
            const uint32_t have = clean_len + (uint32_t)total - flush_base, nvec = have >> 4;
            uint4 *dst16 = reinterpret_cast<uint4 *>(cl + flush_base);
            const uint4 *src16 = reinterpret_cast<const uint4 *>(buf);
            for (uint32_t k = tid; k < nvec; k += kEntropyThreads) dst16[k] = src16[k];
            uint4 rest = make_uint4(0, 0, 0, 0);
            if (tid == 0) rest = src16[nvec];
            __syncthreads();
            if (tid == 0) reinterpret_cast<uint4 *>(buf)[0] = rest; // the incomplete vector moves to the front
            flush_base += nvec << 4;
            // (the next pass's block scan has barriers between this store and the first byte written)
        }
        clean_len += total;
    }
    if (!kStaged) { // what is left in the buffer: fewer than 16 bytes
        __syncthreads();
        if (tid < 16 && flush_base + tid < clean_len) cl[(flush_base + tid) ^ 3u] = reinterpret_cast<uint8_t *>(s_stream)[tid ^ 3u];
        __syncthreads();
    }
    if (tid < 64) cl[(clean_len + tid) ^ 3u] = 0;
    __syncthreads();

    const uint32_t *words = reinterpret_cast<const uint32_t *>(cl);
    const uint32_t total_bits = clean_len * 8;
    // this image's subsequence length; `subseq_bits` is the batch's longest, which sized the buffers
    const uint32_t S = d.subseq_bits ? d.subseq_bits : (uint32_t)subseq_bits;
    const int bpm = d.bpm, luma = d.hs * d.vs, ncomp = d.ncomp;
    int16_t *cf = coef + (size_t)d.block_base * 64;

    // ---- decode index: the states a finished decode of this very stream left behind
    DecodeIndexHeader *ix_hdr = nullptr;
    unsigned long long *ix_state = nullptr;
    uint32_t *ix_blocks = nullptr;
    bool indexed = false;
    if (index_pool != nullptr && d.index_cap != 0) {
        ix_hdr = reinterpret_cast<DecodeIndexHeader *>(index_pool + d.index_off);
        ix_state = reinterpret_cast<unsigned long long *>(ix_hdr + 1);
        ix_blocks = reinterpret_cast<uint32_t *>(ix_state + d.index_cap + 1);
        if (tid == 0) {
            const volatile DecodeIndexHeader *h = ix_hdr; // entries are written by other launches: no caching
            const uint32_t v = h->valid_subs;
            const bool ok = h->magic == kDecodeIndexMagic && h->scan_len == d.scan_len && h->subseq_bits == S &&
                            h->clean_len == clean_len && v <= d.index_cap && __ldcg(ix_blocks + v) >= d.nblocks;
            s_ix[0] = ok ? 1u : 0u;
            s_ix[1] = v;
        }
        __syncthreads();
        indexed = s_ix[0] != 0;
        const uint32_t valid = s_ix[1];
        if (indexed) {
            // Every subsequence starts from its recorded state and writes straight to its recorded
            // place: one pass, no guessing.  (Uniform branch: all threads read the same header.)
            {
                uint4 *z16 = reinterpret_cast<uint4 *>(cf);
                for (uint32_t k = tid; k < d.nblocks * 8; k += kEntropyThreads) z16[k] = make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
            for (uint32_t t = tid; t < valid; t += kEntropyThreads) {
                const uint32_t b0 = __ldcg(ix_blocks + t);
                if (b0 >= d.nblocks) break; // the crop needs nothing from here on
                Cursor cur = unpack(__ldcg(ix_state + t));
                uint32_t t_end = (t + 1) * S;
                if (t_end > total_bits) t_end = total_bits;
                decode_span<true>(words, 0, cur, t_end, bpm, luma, ncomp, s_tab, cf, b0, d.nblocks);
            }
            if (tid == 0) {
                status[img] = 0;
                if (index_stats) atomicAdd(index_stats, 1ull);
            }
            __syncthreads();
        }
    }

    if (!indexed) {
    Cursor zero = {0, 0, 0};
    unsigned long long carry = pack(zero);
    uint32_t blk_base = 0, zeroed_to = 0;
    // every chunk moves the carry forward by at least one subsequence; the count is bounded all the
    // same so that no input, however malformed, can keep the kernel running
    const uint32_t max_chunks = total_bits / S + 2;
    for (uint32_t chunk = 0; chunk < max_chunks; chunk++) {
        const uint32_t carry_p = (uint32_t)(carry >> 32);
        if (carry_p >= total_bits || blk_base >= d.nblocks) break;
        const uint32_t first_sub = carry_p / S;
        // subsequences of this chunk that hold data; threads beyond them stay out of the repair
        uint32_t left = (total_bits - first_sub * S + S - 1) / S;
        // When the crop needs only the upper part of the image, so does the decoder: the bits still
        // to decode are estimated from the blocks still missing (at the rate seen so far, or the
        // stream's average for the first chunk) with a quarter to spare; a short estimate only
        // costs another chunk.
        if (d.mcu_rows < d.mcus_y) {
            const uint64_t all_blocks = (uint64_t)d.bpm * d.mcus_x * d.mcus_y;
            const uint64_t missing = d.nblocks - blk_base;
            const uint64_t bits = blk_base ? missing * (carry_p + 1) / blk_base : missing * total_bits / all_blocks;
            const uint64_t want = (bits + bits / 4 + (carry_p - first_sub * S)) / S + 2;
            if (want < left) left = (uint32_t)want;
        }
        const int nsub = left < (uint32_t)kEntropyThreads ? (int)left : kEntropyThreads;
        const bool active = tid < nsub;
        const uint32_t g = first_sub + tid;
        const uint32_t sub_start = g * S;
        uint32_t sub_end = sub_start + S;
        if (sub_end > total_bits) sub_end = total_bits;
        // The chunk's bits go to shared memory: every lane of a warp reads a different part of the
        // stream for every symbol, which shared memory serves at a few cycles per warp while the
        // same pattern on global memory saturates the L1 tag stage (one sector lookup per cycle).
        const uint32_t bit_base = (kStaged && !resident) ? first_sub * S : 0; // S is a multiple of 128: 16-byte aligned in the stream
        // the staged copy starts at bit_base: a pointer moved back by that many words takes absolute bit positions
        const uint32_t *stream = (kStaged ? s_stream : words) - (bit_base >> 5);
        if (kStaged && !resident) {
            uint32_t n16 = ((uint32_t)nsub * S + 127) / 128 + 1; // one vector of overrun for the last symbol
            const uint32_t have16 = (clean_len + 64 - (bit_base >> 3)) / 16; // zero padding included
            if (n16 > have16) n16 = have16;
            const uint4 *src16 = reinterpret_cast<const uint4 *>(words + (bit_base >> 5));
            uint4 *dst16 = reinterpret_cast<uint4 *>(s_stream);
            for (uint32_t k = tid; k < n16; k += kEntropyThreads) dst16[k] = src16[k];
        }
        Cursor guess = {sub_start, 0, 0};
        s_state[tid] = tid == 0 ? carry : pack(guess);
        s_dirty[tid] = 1;
        s_blocks[tid] = 0;
        __syncthreads();
        // Repair rounds.  A subsequence is dirty when its entry state changed since it was last
        // decoded.  Dirty subsequences are compacted each round so that the work fills
        // whole warps (after the first rounds only a minority is dirty) and idle warps only meet
        // at the barriers.
        for (int iter = 0; iter <= nsub; iter++) {
            const bool dirty = active && s_dirty[tid];
            int n_dirty;
            const int pos = block_scan_exclusive(dirty ? 1 : 0, s_warp, n_dirty);
            if (n_dirty == 0) break;
            if (dirty) s_list[pos] = (uint16_t)tid;
            __syncthreads();
            int t = -1;
            unsigned long long in = 0;
            if (tid < n_dirty) {
                t = s_list[tid];
                in = s_state[t];
                s_dirty[t] = 0; // cleared before the barrier, set again (by the left neighbour) only after it
            }
            __syncthreads(); // every entry state is read before any exit state is written
            if (t >= 0) {
                Cursor cur = unpack(in);
                const uint32_t t_start = (first_sub + (uint32_t)t) * S;
                uint32_t t_end = t_start + S;
                if (t_end > total_bits) t_end = total_bits;
                bool merged = false;
                if (!kStaged && ckpt != nullptr) {
                    // long subsequences: stop where this walk rejoins the previous one
                    const uint32_t per_sub = (uint32_t)subseq_bits / (uint32_t)ck_bits + 1; // stride: the batch's longest
                    CheckPoint *ck = ckpt + ((size_t)blockIdx.x * kEntropyThreads + (size_t)t) * per_sub;
                    int total;
                    if (iter == 0)
                        total = count_span_checked<false>(stream, cur, t_start, t_end, bpm, luma, ncomp, s_tab, ck,
                                                          (uint32_t)ck_bits, merged);
                    else
                        total = count_span_checked<true>(stream, cur, t_start, t_end, bpm, luma, ncomp, s_tab, ck,
                                                         (uint32_t)ck_bits, merged);
                    s_blocks[t] = (uint16_t)total;
                } else {
                    s_blocks[t] = (uint16_t)decode_span<false>(stream, 0, cur, t_end, bpm, luma, ncomp, s_tab, nullptr, 0, 0);
                }
                if (!merged) {
                    const unsigned long long out = pack(cur);
                    if (s_state[t + 1] != out) { // only this thread writes entry t + 1 in this round
                        s_state[t + 1] = out;
                        s_dirty[t + 1] = 1;
                    }
                }
            }
            __syncthreads();
        }
        const int my_blocks = active ? s_blocks[tid] : 0;
        int chunk_blocks;
        const int first = block_scan_exclusive(my_blocks, s_warp, chunk_blocks);
        if (ix_hdr != nullptr && chunk == 0 && first_sub == 0 && (uint32_t)nsub <= d.index_cap) {
            // the entry states are final now: leave them, and the blocks before each, for the next
            // decode of this stream (unless an entry that reaches at least as far is there already)
            if (tid == 0) {
                const volatile DecodeIndexHeader *h = ix_hdr;
                const bool keep = h->magic == kDecodeIndexMagic && h->scan_len == d.scan_len && h->subseq_bits == S &&
                                  h->clean_len == clean_len && h->valid_subs >= (uint32_t)nsub;
                s_ix[0] = keep ? 1u : 0u;
                if (!keep) ix_hdr->magic = 0;
            }
            __syncthreads();
            if (s_ix[0] == 0) {
                if (active) {
                    ix_state[tid] = s_state[tid];
                    ix_blocks[tid] = (uint32_t)first;
                }
                if (tid == 0) {
                    ix_state[nsub] = s_state[nsub];
                    ix_blocks[nsub] = (uint32_t)chunk_blocks;
                }
                __threadfence();
                __syncthreads();
                if (tid == 0) {
                    ix_hdr->scan_len = d.scan_len;
                    ix_hdr->subseq_bits = S;
                    ix_hdr->clean_len = clean_len;
                    ix_hdr->valid_subs = (uint32_t)nsub;
                    __threadfence();
                    ix_hdr->magic = kDecodeIndexMagic;
                    if (index_stats) atomicAdd(index_stats + 1, 1ull);
                }
            }
        }
        // Only non-zero coefficients are stored, so the blocks this chunk writes to are cleared
        // first: the ones it completes and the one left in progress at its end.  Done here rather
        // than by a device-wide memset long before, the cleared lines are still in L2 when the
        // coefficients arrive and reach DRAM once, as whole lines.
        {
            uint32_t target = blk_base + (uint32_t)chunk_blocks + 1;
            if (target > d.nblocks) target = d.nblocks;
            if (target > zeroed_to) {
                uint4 *z16 = reinterpret_cast<uint4 *>(cf + (size_t)zeroed_to * 64);
                const uint32_t nvec = (target - zeroed_to) * 8;
                for (uint32_t k = tid; k < nvec; k += kEntropyThreads) z16[k] = make_uint4(0, 0, 0, 0);
                zeroed_to = target;
            }
            __syncthreads();
        }
        if (active) {
            Cursor cur = unpack(s_state[tid]);
            decode_span<true>(stream, 0, cur, sub_end, bpm, luma, ncomp, s_tab, cf,
                              blk_base + (uint32_t)first, d.nblocks);
        }
        carry = s_state[nsub];
        blk_base += (uint32_t)chunk_blocks;
        __syncthreads();
    }
    if (tid == 0) status[img] = blk_base >= d.nblocks ? 0 : kErrData;
    if (zeroed_to < d.nblocks) { // a stream that ended early: the blocks it never reached read as zero
        uint4 *z16 = reinterpret_cast<uint4 *>(cf + (size_t)zeroed_to * 64);
        const uint32_t nvec = (d.nblocks - zeroed_to) * 8;
        for (uint32_t k = tid; k < nvec; k += kEntropyThreads) z16[k] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    } // !indexed

    // ---- integrate the DC differences of each component over the scan
    const int nmcu = d.mcus_x * d.mcu_rows; // the MCUs that were decoded
    int carry_y = 0, carry_cb = 0, carry_cr = 0;
    for (int base = 0; base < nmcu; base += kEntropyThreads) {
        const int m = base + tid;
        int y[4] = {0, 0, 0, 0}, cb = 0, cr = 0;
        if (m < nmcu) {
            int acc = 0;
            for (int k = 0; k < luma; k++) {
                acc += cf[((size_t)m * bpm + k) * 64];
                y[k] = acc;
            }
            if (ncomp == 3) {
                cb = cf[((size_t)m * bpm + luma) * 64];
                cr = cf[((size_t)m * bpm + luma + 1) * 64];
            }
        }
        int ty, tcb, tcr;
        const int ey = block_scan_exclusive(y[luma - 1], s_warp, ty);
        const int ecb = block_scan_exclusive(cb, s_warp, tcb);
        const int ecr = block_scan_exclusive(cr, s_warp, tcr);
        if (m < nmcu) {
            for (int k = 0; k < luma; k++)
                cf[((size_t)m * bpm + k) * 64] = (int16_t)(carry_y + ey + y[k]);
            if (ncomp == 3) {
                cf[((size_t)m * bpm + luma) * 64] = (int16_t)(carry_cb + ecb + cb);
                cf[((size_t)m * bpm + luma + 1) * 64] = (int16_t)(carry_cr + ecr + cr);
            }
        }
        carry_y += ty;
        carry_cb += tcb;
        carry_cr += tcr;
    }
}

// ------------------------------------------------------------------------------------------
// Streams with restart markers (DRI != 0): every restart interval is an independent piece of the
// stream (byte aligned, DC predictors reset, T.81 F.2.1.3.1 / E.2.4), so no speculation is
// needed: the unstuffing pass also removes the RSTn markers and records where each interval
// starts, then one thread decodes one interval straight into its blocks' final positions, DC
// prediction included.  One CTA per image.

// Decodes `nblk` blocks starting at bit p (slot 0 of an MCU, predictors zero) into cf + blk * 64.
// Returns the bit position reached, or 0xFFFFFFFF when the interval's bits ran out first.
__device__ __forceinline__ uint32_t decode_interval(const uint32_t *__restrict__ words, uint32_t p, uint32_t limit,
                                                    uint32_t nblk, int bpm, int luma, int ncomp,
                                                    const HuffTable *s_tab,
                                                    int16_t *__restrict__ cf, uint32_t blk) {
    int pred[3] = {0, 0, 0};
    int c = 0, z = 0;
    int16_t *out = cf + (size_t)blk * 64;
    uint32_t done = 0;
    BitWindow win(words, p);
    while (done < nblk) {
        if (p >= limit) return 0xFFFFFFFFu;
        const uint32_t w = win.peek();
        const bool dc = z == 0;
        const int comp = (ncomp == 1 || c < luma) ? 0 : c - luma + 1;
        const HuffTable &t = s_tab[2 * comp + (dc ? 0 : 1)];
        const uint32_t e = huff_lookup(t, w);
        const int n = e & 31, s = (e >> 5) & 15;
        const int zn = dc ? 1 : z + (int)(e >> 9);
        const int zpos = zn - 1;
        const int v = s ? extend((w << (n - s)) >> (32 - s), s) : 0;
        if (dc) {
            pred[comp] += v;
            out[0] = (int16_t)pred[comp];
        } else if (s != 0 && zpos < 64) {
            out[zpos] = (int16_t)v; // zig-zag order, as everywhere
        }
        p += n;
        win.skip(n);
        if (zn >= 64) {
            z = 0;
            done++;
            out += 64;
            c = (c + 1 == bpm) ? 0 : c + 1;
        } else {
            z = zn;
        }
    }
    return p;
}

template <int kThreads>
__global__ void __launch_bounds__(kThreads)
entropy_restart_kernel(const ImageDesc *__restrict__ descs, const int32_t *__restrict__ list,
                       const uint8_t *__restrict__ blob, const HuffTable *__restrict__ huff,
                       uint8_t *__restrict__ clean, int16_t *__restrict__ coef, int32_t *__restrict__ status) {
    __shared__ HuffTable s_tab[6];
    __shared__ int s_warp[33];
    __shared__ int s_bad;

    const int img = list[blockIdx.x];
    const ImageDesc d = descs[img];
    const int tid = threadIdx.x;
    if (d.host_status != 0) {
        if (tid == 0) status[img] = d.host_status;
        return;
    }
    for (int c = 0; c < d.ncomp; c++) {
        const uint32_t *sd = reinterpret_cast<const uint32_t *>(&huff[d.dc_tab[c]]);
        const uint32_t *sa = reinterpret_cast<const uint32_t *>(&huff[d.ac_tab[c]]);
        uint32_t *dd = reinterpret_cast<uint32_t *>(&s_tab[2 * c]);
        uint32_t *da = reinterpret_cast<uint32_t *>(&s_tab[2 * c + 1]);
        for (int i = tid; i < (int)(sizeof(HuffTable) / 4); i += kThreads) {
            dd[i] = sd[i];
            da[i] = sa[i];
        }
    }
    if (tid == 0) s_bad = 0;

    // ---- remove byte stuffing and restart markers; note where every interval starts
    const uint8_t *scan = blob + d.payload_off + d.scan_off;
    uint8_t *cl = clean + d.clean_off;
    uint32_t *starts = reinterpret_cast<uint32_t *>(clean + d.rst_off); // byte offsets in the clean stream
    const int nmcu_all = d.mcus_x * d.mcus_y, ri = d.restart_interval;
    const uint32_t cap = (uint32_t)((nmcu_all + ri - 1) / ri) + 1; // entries the table holds
    if (tid == 0) starts[0] = 0;
    uint32_t clean_len = 0, n_mark = 0;
    for (uint32_t base = 0; base < d.scan_len; base += kThreads * 16) {
        const uint32_t my = base + tid * 16;
        uint8_t b[17];
        uint32_t keep = 0, marks = 0;
        int prev = (my > 0 && my <= d.scan_len) ? scan[my - 1] : 0;
#pragma unroll
        for (int i = 0; i < 17; i++) b[i] = my + i < d.scan_len ? scan[my + i] : 0;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const uint32_t at = my + i;
            const bool rst_ff = b[i] == 0xFF && (b[i + 1] & 0xF8) == 0xD0;
            const bool rst_code = prev == 0xFF && (b[i] & 0xF8) == 0xD0;
            const bool stuffing = b[i] == 0 && prev == 0xFF;
            if (at < d.scan_len && !rst_ff && !rst_code && !stuffing) keep |= 1u << i;
            if (at < d.scan_len && rst_code) marks |= 1u << i;
            prev = b[i];
        }
        int total, mtotal;
        const int off = block_scan_exclusive(__popc(keep), s_warp, total);
        const int moff = block_scan_exclusive(__popc(marks), s_warp, mtotal);
        uint32_t o = clean_len + off, m = n_mark + moff;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (keep & (1u << i)) cl[(o++) ^ 3u] = b[i];
            if (marks & (1u << i)) {
                m++;
                if (m < cap) starts[m] = o; // interval m begins with the next byte kept
            }
        }
        clean_len += total;
        n_mark += mtotal;
    }
    if (tid < 64) cl[(clean_len + tid) ^ 3u] = 0;
    __syncthreads();

    // ---- clear the image's blocks (only non-zero coefficients are stored), then one thread per
    // restart interval
    int16_t *cf = coef + (size_t)d.block_base * 64;
    {
        uint4 *z16 = reinterpret_cast<uint4 *>(cf);
        for (uint32_t k = tid; k < d.nblocks * 8; k += kThreads) z16[k] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    const uint32_t *words = reinterpret_cast<const uint32_t *>(cl);
    const int bpm = d.bpm, luma = d.hs * d.vs, ncomp = d.ncomp;
    const int nmcu = d.mcus_x * d.mcu_rows; // the crop may need only the upper rows
    const uint32_t needed = (uint32_t)((nmcu + ri - 1) / ri);
    const uint32_t found = n_mark + 1 < cap ? n_mark + 1 : cap;
    if (found < needed) {
        if (tid == 0) s_bad = 1; // fewer intervals than the frame needs
    }
    for (uint32_t k = tid; k < needed && k < found; k += kThreads) {
        const int first = (int)k * ri;
        const int count = nmcu - first < ri ? nmcu - first : ri;
        const uint32_t p0 = starts[k] * 8;
        const uint32_t limit = (k + 1 < found ? starts[k + 1] : clean_len) * 8;
        const uint32_t p = decode_interval(words, p0, limit, (uint32_t)count * bpm, bpm, luma, ncomp, s_tab, cf,
                                           (uint32_t)first * bpm);
        if (p == 0xFFFFFFFFu) s_bad = 1;
    }
    __syncthreads();
    if (tid == 0) status[img] = s_bad ? kErrData : 0;
}

void launch_entropy_decode(const ImageDesc *descs, const int32_t *list, int n_list,
                           const int32_t *seq_list, int n_seq, const uint8_t *blob,
                           const HuffTable *huff, uint8_t *clean, int16_t *coef, int32_t *status,
                           int subseq_bits, int entropy_threads, void *checkpoints, uint8_t *index_pool,
                           unsigned long long *index_stats, cudaStream_t stream) {
    if (n_list > 0) {
        const bool staged = subseq_bits <= kMaxStagedBits;
        auto launch = [&](auto kernel, int threads) {
            // (the non-staged variant uses the buffer only to collect the unstuffed stream: 16 bytes
            // per thread and pass plus the incomplete vector carried over)
            const size_t smem = staged ? ((size_t)threads * subseq_bits / 8 + 63) / 16 * 16 + 16 : (size_t)threads * 16 + 32;
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            kernel<<<n_list, threads, smem, stream>>>(descs, list, blob, huff, clean, coef, status, subseq_bits,
                                                      static_cast<CheckPoint *>(checkpoints), kCheckPointBits,
                                                      index_pool, index_stats);
        };
        switch (entropy_threads) {
        case 128:
            if (staged) launch(entropy_parallel_kernel<128, true>, 128); else launch(entropy_parallel_kernel<128, false>, 128);
            break;
        case 256:
            if (staged) launch(entropy_parallel_kernel<256, true>, 256); else launch(entropy_parallel_kernel<256, false>, 256);
            break;
        case 1024:
            if (staged) launch(entropy_parallel_kernel<1024, true>, 1024); else launch(entropy_parallel_kernel<1024, false>, 1024);
            break;
        default:
            if (staged) launch(entropy_parallel_kernel<512, true>, 512); else launch(entropy_parallel_kernel<512, false>, 512);
        }
    }
    if (n_seq > 0)
        entropy_restart_kernel<256><<<n_seq, 256, 0, stream>>>(descs, seq_list, blob, huff, clean, coef, status);
}

} // namespace ffcvb
