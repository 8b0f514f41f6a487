// The reference's SafeTensors class (interface: engine/src/safetensors.h:17-38) on POSIX: open + mmap in place of the
// CreateFileW / CreateFileMappingW / MapViewOfFile sequence of engine/src/safetensors.cpp:19-28, which is the only part of
// that file that does not build outside Windows. Test infrastructure: it exists so that the reference's own engine can be
// built on Linux as the checker. Same observable behaviour: the same exceptions for a missing file, a short header, a
// tensor that runs past the end of the file and a missing name; tensors are views into the read-only mapping; paths may
// use '\\' as separator (the engine joins them that way).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

#include "json.h"
#include "safetensors.h"

namespace {
std::string native_path(std::string p) {
    for (char& c : p)
        if (c == '\\') c = '/';
    return p;
}
DType dtype_of(const std::string& s) {
    if (s == "BF16") return DType::BF16;
    if (s == "F16") return DType::F16;
    if (s == "F32") return DType::F32;
    if (s == "I64") return DType::I64;
    return DType::Other;
}
struct Mapping { size_t bytes; };   // what mapping_ points to: the length munmap needs
}  // namespace

SafeTensors::SafeTensors(const std::string& path) : path_(path) {
    const int fd = open(native_path(path).c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("cannot open " + path);
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); throw std::runtime_error("cannot map " + path); }
    const size_t total = (size_t)sb.st_size;
    void* view = mmap(nullptr, total, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);   // the mapping keeps the file alive
    if (view == MAP_FAILED) throw std::runtime_error("cannot view " + path);
    base_ = (const uint8_t*)view;
    mapping_ = new Mapping{total};

    uint64_t header_len = 0;
    memcpy(&header_len, base_, sizeof header_len);
    if (header_len > total - 8) throw std::runtime_error("bad safetensors header: " + path);
    const Json header = Json::parse(std::string((const char*)base_ + 8, (size_t)header_len));
    const uint8_t* payload = base_ + 8 + header_len;
    const uint64_t payload_bytes = total - 8 - header_len;
    for (const auto& entry : header.o) {
        if (entry.first == "__metadata__") continue;
        const Json& desc = entry.second;
        StTensor t;
        t.dtype = dtype_of(desc["dtype"].str());
        for (const auto& dim : desc["shape"].a) t.shape.push_back(dim.i64());
        const uint64_t lo = (uint64_t)desc["data_offsets"][0].i64(), hi = (uint64_t)desc["data_offsets"][1].i64();
        if (hi > payload_bytes) throw std::runtime_error("truncated safetensors (still downloading?): " + path);
        t.data = payload + lo;
        t.bytes = (size_t)(hi - lo);
        tensors_[entry.first] = t;
    }
}

SafeTensors::~SafeTensors() {
    Mapping* m = (Mapping*)mapping_;
    if (base_ && m) munmap((void*)base_, m->bytes);
    delete m;
}

const StTensor& SafeTensors::get(const std::string& name) const {
    const auto hit = tensors_.find(name);
    if (hit == tensors_.end()) throw std::runtime_error("missing tensor " + name + " in " + path_);
    return hit->second;
}

// one stored element as float (engine/src/safetensors.h:41; the text encoder gathers its embedding rows with it)
float st_elem_f32(const StTensor& t, int64_t i) {
    if (t.dtype == DType::F32) return ((const float*)t.data)[i];
    if (t.dtype == DType::BF16) {
        const uint32_t bits = (uint32_t)((const uint16_t*)t.data)[i] << 16;
        float f;
        memcpy(&f, &bits, 4);
        return f;
    }
    if (t.dtype == DType::F16) {
        const uint16_t h = ((const uint16_t*)t.data)[i];
        const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
        int e = (h >> 10) & 31;
        uint32_t m = h & 1023u, bits;
        if (e == 31) bits = sign | 0x7f800000u | (m << 13);                 // inf / nan
        else if (e == 0 && m == 0) bits = sign;                             // zero
        else {
            if (e == 0) {                                                   // subnormal: normalise
                e = 1;
                while (!(m & 1024u)) { m <<= 1; e--; }
                m &= 1023u;
            }
            bits = sign | ((uint32_t)(e + 112) << 23) | (m << 13);
        }
        float f;
        memcpy(&f, &bits, 4);
        return f;
    }
    throw std::runtime_error("unsupported dtype");
}
