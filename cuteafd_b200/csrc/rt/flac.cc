// FLAC stream -> interleaved 32-bit PCM, on the host.  A complete decoder of the format's subset 1..8 channels,
// 4..32 bits per sample: constant / verbatim / fixed / LPC subframes, Rice and Rice2 residuals with escaped partitions,
// wasted bits, the three stereo decorrelations, variable block sizes.  Every frame's CRC-8 and CRC-16 are checked;
// a bad frame is an error, not silence.  No allocation beyond the caller's buffer and one block of scratch.
//
//   cafd_flac_info(data, n, &rate, &channels, &bits, &total)          -> 0 or a negative code
//   cafd_flac_decode(data, n, out, cap_frames)                        -> frames written, or a negative code
//   cafd_flac_decode_mono(data, n, out, cap_frames)                   -> the same, channels averaged into floats
//
// `out` of the first holds cap_frames * channels samples, interleaved, each a signed integer of `bits` bits in an
// int32; of the second cap_frames floats in [-1, 1).  A null `out` only counts the frames (still bounded by
// cap_frames), which is how a stream that does not declare its length is sized before it is decoded.
//
// Counterpart: the reference decodes request audio on the API side with claxon (FLAC), hound (WAV) and nanomp3
// (rust/crates/cuteafd-api, docs/multimodal-design.md:230 "input_audio {data, format: wav|mp3|flac}").
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

enum : int { kBadMagic = -1, kNoStreamInfo = -2, kTruncated = -3, kBadHeader = -4, kBadCrc = -5, kBadSubframe = -6,
             kBadResidual = -7, kTooLong = -8, kUnsupported = -9 };

struct Bits {
    const uint8_t* p; size_t n; size_t pos = 0;       // pos in bits
    bool fail = false;
    Bits(const uint8_t* d, size_t len) : p(d), n(len) {}
    size_t byte() const { return pos >> 3; }
    bool aligned() const { return (pos & 7) == 0; }
    uint32_t bit() {
        if ((pos >> 3) >= n) { fail = true; return 0; }
        uint32_t b = (p[pos >> 3] >> (7 - (pos & 7))) & 1u; ++pos; return b;
    }
    uint64_t u(int k) {                                // k <= 57
        uint64_t v = 0;
        while (k > 0) {
            if ((pos >> 3) >= n) { fail = true; return 0; }
            int have = 8 - static_cast<int>(pos & 7), take = k < have ? k : have;
            uint32_t chunk = (p[pos >> 3] >> (have - take)) & ((1u << take) - 1u);
            v = (v << take) | chunk; pos += take; k -= take;
        }
        return v;
    }
    int64_t s(int k) {                                 // two's complement, k bits
        if (k == 0) return 0;
        uint64_t v = u(k);
        return (v >> (k - 1)) & 1 ? static_cast<int64_t>(v) - (int64_t{1} << k) : static_cast<int64_t>(v);
    }
    uint32_t unary() {                                 // zeros before the next one
        uint32_t z = 0;
        for (;;) {
            if ((pos >> 3) >= n) { fail = true; return 0; }
            uint32_t rest = p[pos >> 3] & (0xffu >> (pos & 7));
            if (rest == 0) { z += 8 - (pos & 7); pos = (pos | 7) + 1; continue; }
            int lead = __builtin_clz(rest) - 24 - static_cast<int>(pos & 7);
            z += lead; pos += lead + 1; return z;
        }
    }
    void align() { pos = (pos + 7) & ~size_t{7}; }
};

uint8_t crc8(const uint8_t* d, size_t n) {
    uint8_t c = 0;
    for (size_t i = 0; i < n; ++i) { c ^= d[i]; for (int b = 0; b < 8; ++b) c = (c & 0x80) ? (c << 1) ^ 0x07 : (c << 1); }
    return c;
}
uint16_t crc16(const uint8_t* d, size_t n) {
    static uint16_t table[256]; static bool ready = false;
    if (!ready) {
        for (int i = 0; i < 256; ++i) { uint16_t c = i << 8; for (int b = 0; b < 8; ++b) c = (c & 0x8000) ? (c << 1) ^ 0x8005 : (c << 1); table[i] = c; }
        ready = true;
    }
    uint16_t c = 0;
    for (size_t i = 0; i < n; ++i) c = (c << 8) ^ table[(c >> 8) ^ d[i]];
    return c;
}

struct Info { uint32_t rate = 0; int channels = 0, bits = 0; uint64_t total = 0; size_t first_frame = 0; };

int read_info(const uint8_t* d, size_t n, Info* out) {
    if (n < 4 || std::memcmp(d, "fLaC", 4) != 0) return kBadMagic;
    size_t at = 4; bool seen = false;
    for (;;) {
        if (at + 4 > n) return kTruncated;
        bool last = d[at] & 0x80; int type = d[at] & 0x7f;
        size_t len = (size_t{d[at + 1]} << 16) | (size_t{d[at + 2]} << 8) | d[at + 3];
        at += 4;
        if (at + len > n) return kTruncated;
        if (type == 0) {
            if (len < 34) return kBadHeader;
            Bits b(d + at, len);
            b.u(16); b.u(16); b.u(24); b.u(24);
            out->rate = static_cast<uint32_t>(b.u(20));
            out->channels = static_cast<int>(b.u(3)) + 1;
            out->bits = static_cast<int>(b.u(5)) + 1;
            out->total = b.u(36);
            seen = true;
        }
        at += len;
        if (last) break;
    }
    if (!seen) return kNoStreamInfo;
    if (out->rate == 0 || out->bits < 4) return kBadHeader;
    out->first_frame = at;
    return 0;
}

int residual(Bits& b, int order, int block, int64_t* dst) {          // dst[order..block) receive the residual
    int method = static_cast<int>(b.u(2));
    if (method > 1) return kBadResidual;
    int pbits = method ? 5 : 4, esc = method ? 31 : 15;
    int porder = static_cast<int>(b.u(4)), parts = 1 << porder;
    if ((block >> porder) << porder != block && porder > 0) return kBadResidual;
    if (porder > 0 && (block >> porder) < order) return kBadResidual;
    int i = order;
    for (int p = 0; p < parts; ++p) {
        int count = (porder == 0 ? block : block >> porder) - (p == 0 ? order : 0);
        if (count < 0) return kBadResidual;
        int k = static_cast<int>(b.u(pbits));
        if (k == esc) {
            int raw = static_cast<int>(b.u(5));
            for (int j = 0; j < count; ++j) dst[i++] = b.s(raw);
        } else {
            for (int j = 0; j < count; ++j) {
                uint64_t q = b.unary();
                uint64_t v = (q << k) | (k ? b.u(k) : 0);
                dst[i++] = static_cast<int64_t>(v >> 1) ^ -static_cast<int64_t>(v & 1);
            }
        }
        if (b.fail) return kTruncated;
    }
    return i == block ? 0 : kBadResidual;
}

int subframe(Bits& b, int bps, int block, int64_t* s) {
    if (b.bit()) return kBadSubframe;
    int type = static_cast<int>(b.u(6));
    int wasted = 0;
    if (b.bit()) { wasted = static_cast<int>(b.unary()) + 1; }
    if (wasted >= bps) return kBadSubframe;
    bps -= wasted;
    if (type == 0) {
        int64_t v = b.s(bps);
        for (int i = 0; i < block; ++i) s[i] = v;
    } else if (type == 1) {
        for (int i = 0; i < block; ++i) s[i] = b.s(bps);
    } else if (type >= 8 && type <= 12) {
        int order = type - 8;
        if (order > block) return kBadSubframe;
        for (int i = 0; i < order; ++i) s[i] = b.s(bps);
        if (int rc = residual(b, order, block, s)) return rc;
        for (int i = order; i < block; ++i) {
            int64_t pred = 0;
            switch (order) {
                case 1: pred = s[i - 1]; break;
                case 2: pred = 2 * s[i - 1] - s[i - 2]; break;
                case 3: pred = 3 * s[i - 1] - 3 * s[i - 2] + s[i - 3]; break;
                case 4: pred = 4 * s[i - 1] - 6 * s[i - 2] + 4 * s[i - 3] - s[i - 4]; break;
                default: break;
            }
            s[i] += pred;
        }
    } else if (type >= 32) {
        int order = type - 31;
        if (order > block) return kBadSubframe;
        for (int i = 0; i < order; ++i) s[i] = b.s(bps);
        int prec = static_cast<int>(b.u(4)) + 1;
        if (prec == 16) return kBadSubframe;
        int shift = static_cast<int>(b.s(5));
        if (shift < 0) return kBadSubframe;
        int64_t coef[32];
        for (int j = 0; j < order; ++j) coef[j] = b.s(prec);
        if (int rc = residual(b, order, block, s)) return rc;
        for (int i = order; i < block; ++i) {
            int64_t acc = 0;
            for (int j = 0; j < order; ++j) acc += coef[j] * s[i - 1 - j];
            s[i] += acc >> shift;
        }
    } else {
        return kBadSubframe;
    }
    if (wasted) for (int i = 0; i < block; ++i) s[i] = static_cast<int64_t>(static_cast<uint64_t>(s[i]) << wasted);
    return b.fail ? kTruncated : 0;
}

template <class Sink>
long long decode_stream(const uint8_t* data, uint64_t n, uint64_t cap_frames, Sink&& sink) {
    Info in;
    if (int rc = read_info(data, n, &in)) return rc;
    static const int kBlock[16] = {0, 192, 576, 1152, 2304, 4608, 0, 0, 256, 512, 1024, 2048, 4096, 8192, 16384, 32768};
    static const int kBits[8] = {0, 8, 12, 0, 16, 20, 24, 32};
    std::vector<int64_t> chan;
    uint64_t done = 0;
    size_t at = in.first_frame;
    while (at + 2 <= n) {
        if (!(data[at] == 0xff && (data[at + 1] & 0xfe) == 0xf8)) {
            // trailing bytes that are not a frame (an ID3v1 tag, padding) end the stream
            if (done > 0) break;
            return kBadHeader;
        }
        Bits b(data + at, n - at);
        b.u(14);
        if (b.bit()) return kBadHeader;
        b.bit();                                                   // blocking strategy: only numbers the frames
        int bs_code = static_cast<int>(b.u(4)), sr_code = static_cast<int>(b.u(4));
        int ch_code = static_cast<int>(b.u(4)), ss_code = static_cast<int>(b.u(3));
        if (b.bit()) return kBadHeader;
        // frame / sample number: UTF-8 style, up to 7 bytes
        uint32_t lead = static_cast<uint32_t>(b.u(8));
        int extra = 0;
        if (lead & 0x80) { while (extra < 7 && (lead & (0x80u >> extra))) ++extra; if (extra < 2) return kBadHeader; --extra; }
        for (int i = 0; i < extra; ++i) if ((b.u(8) & 0xc0) != 0x80) return kBadHeader;
        int block = kBlock[bs_code];
        if (bs_code == 0) return kBadHeader;
        if (bs_code == 6) block = static_cast<int>(b.u(8)) + 1;
        if (bs_code == 7) block = static_cast<int>(b.u(16)) + 1;
        if (sr_code == 12) b.u(8); else if (sr_code == 13 || sr_code == 14) b.u(16); else if (sr_code == 15) return kBadHeader;
        if (b.fail) return kTruncated;
        size_t hdr = b.byte();
        if (static_cast<uint8_t>(b.u(8)) != crc8(data + at, hdr)) return kBadCrc;
        int bps = ss_code == 0 ? in.bits : kBits[ss_code];
        if (bps == 0 || bps != in.bits) return kUnsupported;       // a stream keeps one sample size
        int channels = ch_code < 8 ? ch_code + 1 : 2;
        if (ch_code > 10 || channels != in.channels) return kBadHeader;
        if (done + static_cast<uint64_t>(block) > cap_frames) return kTooLong;
        chan.resize(static_cast<size_t>(channels) * block);
        for (int c = 0; c < channels; ++c) {
            bool side = (ch_code == 8 && c == 1) || (ch_code == 9 && c == 0) || (ch_code == 10 && c == 1);
            if (int rc = subframe(b, bps + (side ? 1 : 0), block, chan.data() + static_cast<size_t>(c) * block)) return rc;
        }
        b.align();
        size_t body = b.byte();
        uint16_t want = static_cast<uint16_t>(b.u(16));
        if (b.fail) return kTruncated;
        if (want != crc16(data + at, body)) return kBadCrc;
        int64_t* a = chan.data(); int64_t* c1 = channels > 1 ? chan.data() + block : nullptr;
        if (ch_code == 8) { for (int i = 0; i < block; ++i) c1[i] = a[i] - c1[i]; }
        else if (ch_code == 9) { for (int i = 0; i < block; ++i) a[i] = a[i] + c1[i]; }
        else if (ch_code == 10) {
            for (int i = 0; i < block; ++i) {
                int64_t side = c1[i], mid = (a[i] << 1) | (side & 1);
                a[i] = (mid + side) >> 1; c1[i] = (mid - side) >> 1;
            }
        }
        sink(chan.data(), channels, block, done, in.bits);
        done += block;
        at += b.byte();
    }
    if (in.total && done > in.total) done = in.total;              // the last block may be padded by a streaming encoder
    return static_cast<long long>(done);
}

}  // namespace

extern "C" {

int cafd_flac_info(const uint8_t* data, uint64_t n, uint32_t* rate, int* channels, int* bits, uint64_t* total) {
    Info in;
    if (int rc = read_info(data, n, &in)) return rc;
    *rate = in.rate; *channels = in.channels; *bits = in.bits; *total = in.total;
    return 0;
}

long long cafd_flac_decode(const uint8_t* data, uint64_t n, int32_t* out, uint64_t cap_frames) {
    return decode_stream(data, n, cap_frames, [out](const int64_t* chan, int channels, int block, uint64_t done, int) {
        if (!out) return;
        int32_t* o = out + done * channels;
        for (int i = 0; i < block; ++i)
            for (int c = 0; c < channels; ++c) o[static_cast<size_t>(i) * channels + c] = static_cast<int32_t>(chan[static_cast<size_t>(c) * block + i]);
    });
}

long long cafd_flac_decode_mono(const uint8_t* data, uint64_t n, float* out, uint64_t cap_frames) {
    return decode_stream(data, n, cap_frames, [out](const int64_t* chan, int channels, int block, uint64_t done, int bits) {
        if (!out) return;
        const double scale = 1.0 / (static_cast<double>(int64_t{1} << (bits - 1)) * channels);
        for (int i = 0; i < block; ++i) {
            int64_t acc = 0;
            for (int c = 0; c < channels; ++c) acc += chan[static_cast<size_t>(c) * block + i];
            out[done + i] = static_cast<float>(acc * scale);
        }
    });
}

}  // extern "C"
