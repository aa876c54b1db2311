// Weight ingest from safetensors checkpoints for the CUDA backend: parser, checkpoint
// directory, and file tensor -> device Tensor with the loader's dtype conversions.
// Same surface as vAi's loader — SafetensorsParser / SafetensorRef
// (vai/engine/safetensors-parser.h:18-56), Checkpoint (vai/engine/weights.h:30-64),
// Tensor(ref, dtype) / concat / slice (vai/engine/tensor.cpp:248-330) — rebuilt for this
// backend: the file is memory-mapped, and a tensor goes to the GPU in 8 MiB parts through
// two pinned staging buffers, each part converted (or just copied) into one buffer while
// the previous part's host-to-device copy is in flight.  BF16 is a tensor dtype here, so
// the usual BF16 checkpoint -> BF16 weights path converts nothing.
#ifndef VAI_B200_HOST_SAFETENSORS_H
#define VAI_B200_HOST_SAFETENSORS_H

#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <bit>
#include <initializer_list>
#include <string_view>
#include <unordered_map>

#include "linear.h"

namespace vai {

// ---- 16-bit conversions (rules of vai/engine/tensor.cpp:22-85) ---------------------
inline float halfToFloat(uint16_t h)
{
    const uint32_t sign = uint32_t(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
    if (exp == 0x1Fu) return std::bit_cast<float>(sign | 0x7F800000u | (mant << 13));
    if (exp == 0) {                                    // zero or subnormal: mant * 2^-24, exact in fp32
        const float v = float(mant) * 5.9604644775390625e-8f;
        return std::bit_cast<float>(std::bit_cast<uint32_t>(v) | sign);
    }
    return std::bit_cast<float>(sign | ((exp + 112u) << 23) | (mant << 13));
}
// fp32 -> fp16 with the loader's rules (the bit rule of vai/engine/tensor.cpp:46-69, which a
// reader of vAi checkpoints has to reproduce exactly): round to nearest even, anything below
// the smallest normal half (2^-14) flushes to a signed zero, overflow saturates to infinity,
// NaN becomes the quiet NaN 0x7E00.  Done on the magnitude bits: adding 0xFFF plus the
// keep-bit rounds at bit 13, and the shifted result minus the bias difference (112 << 10) is
// the half's exponent and mantissa, carry included.
inline uint16_t floatToHalf(float f)
{
    const uint32_t bits = std::bit_cast<uint32_t>(f);
    const uint16_t sgn = uint16_t((bits >> 16) & 0x8000u);
    const uint32_t mag = bits & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return uint16_t(sgn | 0x7E00u);
    if (mag == 0x7F800000u) return uint16_t(sgn | 0x7C00u);
    if (mag < 0x38800000u) return sgn;                                   // |f| < 2^-14
    const uint32_t rounded = mag + 0xFFFu + ((mag >> 13) & 1u);
    const uint32_t half = (rounded >> 13) - (112u << 10);
    return uint16_t(sgn | (half < 0x7C00u ? half : 0x7C00u));
}
inline float bfloatToFloat(uint16_t b) { return std::bit_cast<float>(uint32_t(b) << 16); }
// fp32 -> bf16, round to nearest even on the upper 16 bits; a NaN keeps its upper payload and
// gets the quiet bit (vai/engine/tensor.cpp:73-85).
inline uint16_t floatToBfloat(float f)
{
    const uint32_t bits = std::bit_cast<uint32_t>(f);
    const bool nan = (bits & 0x7FFFFFFFu) > 0x7F800000u;
    if (nan) return uint16_t((bits >> 16) | 0x0040u);
    const uint32_t keep = (bits >> 16) & 1u;
    return uint16_t((bits + 0x7FFFu + keep) >> 16);
}

class SafetensorsParser;

struct SafetensorRef {
    const SafetensorsParser* parser;
    std::string key;
    std::vector<uint32_t> getShape() const;
    std::string getDataType() const;
    size_t byteSize() const;
    const void* data() const;                                            // zero-copy: inside the mapping
    void readInto(void* dst) const;
    void readInto(void* dst, size_t byteOffset, size_t byteCount) const;
};

class SafetensorsParser
{
    struct Meta {
        std::string dtype;
        std::vector<uint32_t> shape;
        size_t begin = 0, end = 0;
    };
    std::unordered_map<std::string, Meta> tensors_;
    std::vector<std::string> order_;
    const uint8_t* map_ = nullptr;
    size_t fileSize_ = 0, startOfData_ = 0;

    // ---- a JSON reader for the header: objects, arrays, strings, numbers, literals ----
    struct Cursor {
        const char* p;
        const char* end;
        void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
        char peek() { ws(); if (p >= end) throw std::runtime_error("JSON parse error: unexpected end"); return *p; }
        void expect(char c) { if (peek() != c) throw std::runtime_error(std::string("JSON parse error: expected ") + c); ++p; }
        std::string string()
        {
            expect('"');
            std::string out;
            while (p < end && *p != '"') {
                if (*p == '\\') {
                    if (++p >= end) break;
                    switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u':                                  // keep the escape verbatim: names stay comparable
                        out += "\\u";
                        break;
                    default: out += *p;
                    }
                    ++p;
                } else {
                    out += *p++;
                }
            }
            if (p >= end) throw std::runtime_error("JSON parse error: unterminated string");
            ++p;
            return out;
        }
        uint64_t number()
        {
            ws();
            const char* s = p;
            uint64_t v = 0;
            while (p < end && *p >= '0' && *p <= '9') {
                const uint64_t digit = uint64_t(*p++ - '0');
                if (v > (UINT64_MAX - digit) / 10u) throw std::runtime_error("JSON parse error: integer out of range");
                v = v * 10u + digit;
            }
            if (p == s) throw std::runtime_error("JSON parse error: expected a non-negative integer");
            return v;
        }
        void skipValue()
        {
            const char c = peek();
            if (c == '"') { string(); return; }
            if (c == '{' || c == '[') {
                const char close = c == '{' ? '}' : ']';
                ++p;
                if (peek() == close) { ++p; return; }
                for (;;) {
                    if (c == '{') { string(); expect(':'); }
                    skipValue();
                    if (peek() == ',') { ++p; continue; }
                    expect(close);
                    return;
                }
            }
            while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;      // number / true / false / null
        }
    };

    void parseHeader(const char* text, size_t len)
    {
        Cursor c{text, text + len};
        if (c.peek() != '{') throw std::runtime_error("Invalid Safetensors: root is not object");
        ++c.p;
        if (c.peek() == '}') return;
        for (;;) {
            const std::string key = c.string();
            c.expect(':');
            if (key == "__metadata__") {
                c.skipValue();
            } else {
                if (c.peek() != '{') throw std::runtime_error("Invalid tensor entry: " + key);
                ++c.p;
                Meta m;
                bool haveOffsets = false;
                if (c.peek() != '}')
                    for (;;) {
                        const std::string field = c.string();
                        c.expect(':');
                        if (field == "dtype") {
                            m.dtype = c.string();
                        } else if (field == "shape" || field == "data_offsets") {
                            std::vector<uint64_t> v;
                            c.expect('[');
                            if (c.peek() != ']')
                                for (;;) {
                                    v.push_back(c.number());
                                    if (c.peek() == ',') { ++c.p; continue; }
                                    break;
                                }
                            c.expect(']');
                            if (field == "shape") {
                                for (uint64_t d : v) {
                                    if (d > UINT32_MAX) throw std::runtime_error("Invalid tensor entry (axis too long): " + key);
                                    m.shape.push_back((uint32_t)d);
                                }
                            } else {
                                if (v.size() != 2) throw std::runtime_error("Invalid tensor entry: " + key);
                                m.begin = v[0]; m.end = v[1];
                                haveOffsets = true;
                            }
                        } else {
                            c.skipValue();
                        }
                        if (c.peek() == ',') { ++c.p; continue; }
                        break;
                    }
                c.expect('}');
                // compared against the size of the data section, so that no sum can wrap
                if (!haveOffsets || m.begin > m.end || m.end > fileSize_ - startOfData_)
                    throw std::runtime_error("Tensor data runs past the end of the file: " + key);
                if (tensors_.emplace(key, std::move(m)).second) order_.push_back(key);
            }
            if (c.peek() == ',') { ++c.p; continue; }
            c.expect('}');
            break;
        }
    }

    const Meta& meta(std::string_view key) const
    {
        auto it = tensors_.find(std::string(key));
        if (it == tensors_.end()) throw std::out_of_range("Tensor key not found: " + std::string(key));
        return it->second;
    }

public:
    explicit SafetensorsParser(const char* path)
    {
        const int fd = ::open(path, O_RDONLY);
        if (fd < 0) throw std::runtime_error("Could not open Safetensors file: " + std::string(path));
        struct stat st {};
        if (::fstat(fd, &st) != 0 || st.st_size < 8) {
            ::close(fd);
            throw std::runtime_error("Failed to read header length.");
        }
        fileSize_ = (size_t)st.st_size;
        void* m = ::mmap(nullptr, fileSize_, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (m == MAP_FAILED) throw std::runtime_error("Could not map Safetensors file: " + std::string(path));
        map_ = static_cast<const uint8_t*>(m);
        uint64_t headerLength = 0;
        std::memcpy(&headerLength, map_, 8);
        if (headerLength > fileSize_ - 8) {
            ::munmap(m, fileSize_);
            map_ = nullptr;
            throw std::runtime_error("Failed to read header string.");
        }
        startOfData_ = 8 + (size_t)headerLength;
        try {
            parseHeader(reinterpret_cast<const char*>(map_ + 8), (size_t)headerLength);
        } catch (...) {
            ::munmap(m, fileSize_);
            map_ = nullptr;
            throw;
        }
    }
    ~SafetensorsParser()
    {
        if (map_) ::munmap(const_cast<uint8_t*>(map_), fileSize_);
    }
    SafetensorsParser(const SafetensorsParser&) = delete;
    SafetensorsParser& operator=(const SafetensorsParser&) = delete;

    std::vector<std::string> getTensorNames() const { return order_; }
    SafetensorRef operator[](std::string_view key) const { return {this, std::string(key)}; }
    std::vector<uint32_t> getShape(std::string_view key) const { return meta(key).shape; }
    std::string getDataType(std::string_view key) const { return meta(key).dtype; }

    size_t byteSize(std::string_view key) const
    {
        const Meta& m = meta(key);
        const size_t bytes = m.end - m.begin;
        size_t esz = 0;
        if (m.dtype == "F32") esz = 4;
        else if (m.dtype == "F16" || m.dtype == "BF16") esz = 2;
        else throw std::runtime_error("Unsupported dtype: " + m.dtype);
        // element count with the product checked: it can never exceed the bytes the file holds
        size_t n = 1;
        for (uint32_t s : m.shape) {
            if (s != 0 && n > fileSize_ / s) throw std::runtime_error("Data size mismatch for " + m.dtype + " tensor.");
            n *= s;
        }
        if (n > fileSize_ / esz || bytes != n * esz) throw std::runtime_error("Data size mismatch for " + m.dtype + " tensor.");
        return bytes;
    }
    const void* data(std::string_view key) const { return map_ + startOfData_ + meta(key).begin; }
    void readInto(std::string_view key, void* dst) const { readInto(key, dst, 0, byteSize(key)); }
    void readInto(std::string_view key, void* dst, size_t byteOffset, size_t byteCount) const
    {
        const Meta& m = meta(key);
        const size_t total = m.end - m.begin;
        if (byteOffset > total || byteCount > total - byteOffset) throw std::runtime_error("Tensor read runs past the end of the tensor.");
        std::memcpy(dst, map_ + startOfData_ + m.begin + byteOffset, byteCount);
    }
};

inline std::vector<uint32_t> SafetensorRef::getShape() const { return parser->getShape(key); }
inline std::string SafetensorRef::getDataType() const { return parser->getDataType(key); }
inline size_t SafetensorRef::byteSize() const { return parser->byteSize(key); }
inline const void* SafetensorRef::data() const { return parser->data(key); }
inline void SafetensorRef::readInto(void* dst) const { parser->readInto(key, dst); }
inline void SafetensorRef::readInto(void* dst, size_t o, size_t n) const { parser->readInto(key, dst, o, n); }

// Every *.safetensors under a directory, addressed by tensor name.
class Checkpoint
{
    std::vector<std::unique_ptr<SafetensorsParser>> shards_;
    std::unordered_map<std::string, const SafetensorsParser*> owner_;

public:
    explicit Checkpoint(const std::string& dir)
    {
        std::vector<std::string> files;
        if (DIR* d = ::opendir(dir.c_str())) {
            while (dirent* e = ::readdir(d)) {
                const std::string name = e->d_name;
                if (name.size() > 12 && name.compare(name.size() - 12, 12, ".safetensors") == 0) files.push_back(dir + "/" + name);
            }
            ::closedir(d);
        }
        std::sort(files.begin(), files.end());
        for (const std::string& f : files) {
            auto& shard = shards_.emplace_back(std::make_unique<SafetensorsParser>(f.c_str()));
            for (const std::string& key : shard->getTensorNames()) owner_.emplace(key, shard.get());
        }
        if (owner_.empty()) throw std::runtime_error("no *.safetensors under " + dir);
    }
    bool contains(std::string_view key) const { return owner_.count(std::string(key)) != 0; }
    SafetensorRef operator[](std::string_view key) const
    {
        auto it = owner_.find(std::string(key));
        if (it == owner_.end()) throw std::runtime_error("checkpoint has no tensor " + std::string(key));
        return (*it->second)[key];
    }
};

namespace detail {

inline Dtype dtypeOfFile(const std::string& stored)
{
    if (stored == "F32") return Dtype::Fp32;
    if (stored == "F16") return Dtype::Fp16;
    if (stored == "BF16") return Dtype::Bf16;
    throw std::runtime_error("Unsupported dtype: " + stored);
}

// count elements of the file's dtype -> dst's dtype; 16-bit to the other 16-bit kind
// goes through fp32 (exact) and rounds once.
inline void convertStored(const void* src, Dtype from, void* dst, Dtype to, size_t count)
{
    if (from == to) { std::memcpy(dst, src, count * bytesPerElement(to)); return; }
    auto sU = static_cast<const uint16_t*>(src);
    auto sF = static_cast<const float*>(src);
    auto dU = static_cast<uint16_t*>(dst);
    auto dF = static_cast<float*>(dst);
    auto widen = [&](size_t i) { return from == Dtype::Fp32 ? sF[i] : (from == Dtype::Fp16 ? halfToFloat(sU[i]) : bfloatToFloat(sU[i])); };
    if (to == Dtype::Fp32) for (size_t i = 0; i < count; ++i) dF[i] = widen(i);
    else if (to == Dtype::Fp16) for (size_t i = 0; i < count; ++i) dU[i] = floatToHalf(widen(i));
    else for (size_t i = 0; i < count; ++i) dU[i] = floatToBfloat(widen(i));
}

// Two pinned staging buffers with an event each; owned by the calling thread and reused
// across loads (so their pages are pinned once).
struct Staging {
    static constexpr size_t kPartBytes = size_t(8) << 20;
    void* buf[2] = {nullptr, nullptr};
    vaicu_event* done[2] = {nullptr, nullptr};
    bool used[2] = {false, false};
    vaicu_stream_t stream = nullptr;
    void init()
    {
        if (buf[0]) return;
        initVAIEngine();
        check(vaicu_stream_create(deviceHandle(), &stream), "vaicu_stream_create");
        for (int i = 0; i < 2; ++i) {
            check(vaicu_host_alloc_pinned(kPartBytes, &buf[i]), "vaicu_host_alloc_pinned");
            check(vaicu_event_create(&done[i]), "vaicu_event_create");
        }
    }
    ~Staging()
    {
        for (int i = 0; i < 2; ++i) {
            if (done[i]) vaicu_event_destroy(done[i]);
            if (buf[i]) vaicu_host_free_pinned(buf[i]);
        }
        if (stream) vaicu_stream_destroy(stream);
    }
};
inline Staging& staging()
{
    thread_local Staging s;
    s.init();
    return s;
}

// srcBytes of file data at `src` -> device memory at `dst` as dtype `to`, in parts.
inline void uploadConverted(const void* src, size_t srcBytes, Dtype from, char* dst, Dtype to)
{
    if (srcBytes == 0) return;
    Staging& s = staging();
    const size_t srcElem = bytesPerElement(from), dstElem = bytesPerElement(to);
    // parts are sized by the larger element so that a converted part fits its buffer
    const size_t perPart = Staging::kPartBytes / std::max(srcElem, dstElem);
    const size_t count = srcBytes / srcElem;
    int which = 0;
    for (size_t pos = 0; pos < count; pos += perPart, which ^= 1) {
        const size_t n = std::min(perPart, count - pos);
        if (s.used[which]) check(vaicu_event_synchronize(s.done[which]), "vaicu_event_synchronize");
        convertStored(static_cast<const char*>(src) + pos * srcElem, from, s.buf[which], to, n);
        check(vaicu_memcpy_h2d(dst + pos * dstElem, s.buf[which], n * dstElem, s.stream), "vaicu_memcpy_h2d");
        check(vaicu_event_record(s.done[which], s.stream), "vaicu_event_record");
        s.used[which] = true;
    }
    check(vaicu_stream_sync(s.stream), "vaicu_stream_sync");
}

}   // namespace detail

// Tensor(ref, dtype): the whole file tensor on the device as `dtype` (None keeps the file's).
inline Tensor loadTensor(const SafetensorRef& ref, Dtype target = Dtype::None)
{
    const Dtype from = detail::dtypeOfFile(ref.getDataType());
    Tensor out(ref.getShape(), target == Dtype::None ? from : target);
    if (out.numBytes()) out.allocate();
    detail::uploadConverted(ref.data(), ref.byteSize(), from, static_cast<char*>(out.devicePtr()), out.dtype());
    return out;
}

// File tensors stacked along the leading axis (gate_proj over up_proj -> the [2H, K]
// weight of a gate|value Linear); each part lands at its own offset of one device range.
inline Tensor concat(std::initializer_list<SafetensorRef> refs, Dtype target)
{
    if (refs.size() == 0 || target == Dtype::None) throw std::invalid_argument("concat needs tensors and a target dtype");
    const std::string stored = refs.begin()->getDataType();
    std::vector<uint32_t> shape = refs.begin()->getShape();
    if (shape.empty()) throw std::invalid_argument("concat: scalars cannot be stacked");
    shape[0] = 0;
    for (const SafetensorRef& r : refs) {
        const std::vector<uint32_t> part = r.getShape();
        if (r.getDataType() != stored || part.size() != shape.size() || !std::equal(part.begin() + 1, part.end(), shape.begin() + 1))
            throw std::invalid_argument("concat: tensors differ in dtype or trailing shape");
        shape[0] += part[0];
    }
    const Dtype from = detail::dtypeOfFile(stored);
    Tensor out(shape, target);
    if (out.numBytes()) out.allocate();
    char* dst = static_cast<char*>(out.devicePtr());
    for (const SafetensorRef& r : refs) {
        const size_t bytes = r.byteSize();
        detail::uploadConverted(r.data(), bytes, from, dst, target);
        dst += bytes / bytesPerElement(from) * bytesPerElement(target);
    }
    return out;
}

// Rows [begin, end) of the leading axis; only those bytes of the file are touched — the
// slab of one rank of a column-split Linear.
inline Tensor slice(const SafetensorRef& ref, uint32_t begin, uint32_t end, Dtype target)
{
    std::vector<uint32_t> shape = ref.getShape();
    if (shape.empty() || begin > end || end > shape[0] || target == Dtype::None) throw std::invalid_argument("slice: bad row range");
    const size_t rowBytes = shape[0] ? ref.byteSize() / shape[0] : 0;
    const Dtype from = detail::dtypeOfFile(ref.getDataType());
    shape[0] = end - begin;
    Tensor out(shape, target);
    if (out.numBytes()) out.allocate();
    detail::uploadConverted(static_cast<const char*>(ref.data()) + (size_t)begin * rowBytes, (size_t)(end - begin) * rowBytes, from,
                            static_cast<char*>(out.devicePtr()), target);
    return out;
}

}   // namespace vai

#endif   // VAI_B200_HOST_SAFETENSORS_H
