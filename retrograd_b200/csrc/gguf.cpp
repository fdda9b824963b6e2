#include "gguf.hpp"
#include "blocks.hpp"

#include <cstring>
#include <stdexcept>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace rb200 {

namespace {

enum ValueType : uint32_t {
    V_U8 = 0, V_I8 = 1, V_U16 = 2, V_I16 = 3, V_U32 = 4, V_I32 = 5, V_F32 = 6, V_BOOL = 7,
    V_STRING = 8, V_ARRAY = 9, V_U64 = 10, V_I64 = 11, V_F64 = 12,
};

struct Reader {
    const uint8_t * cur;
    const uint8_t * end;
    void need(uint64_t n) const {
        if ((uint64_t)(end - cur) < n) throw std::runtime_error("GGUF file is truncated");
    }
    template <class T> T take() {
        need(sizeof(T));
        T v;
        std::memcpy(&v, cur, sizeof(T));
        cur += sizeof(T);
        return v;
    }
    std::string take_string() {
        const uint64_t n = take<uint64_t>();
        need(n);
        std::string s(reinterpret_cast<const char *>(cur), n);
        cur += n;
        return s;
    }
    void skip(uint64_t n) {
        need(n);
        cur += n;
    }
};

uint64_t value_width(uint32_t t) {
    switch (t) {
        case V_U8: case V_I8: case V_BOOL: return 1;
        case V_U16: case V_I16: return 2;
        case V_U32: case V_I32: case V_F32: return 4;
        case V_U64: case V_I64: case V_F64: return 8;
        default: throw std::runtime_error("GGUF metadata holds an unknown value type");
    }
}

} // namespace

GgufFile::GgufFile(const std::string & path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("failed to load model GGUF: " + path);
    struct stat st {};
    if (fstat(fd_, &st) != 0 || st.st_size < 24) {
        ::close(fd_);
        fd_ = -1;
        throw std::runtime_error("failed to load model GGUF: " + path);
    }
    size_ = (uint64_t)st.st_size;
    void * map = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (map == MAP_FAILED) {
        ::close(fd_);
        fd_ = -1;
        throw std::runtime_error("failed to map model GGUF: " + path);
    }
    base_ = static_cast<const uint8_t *>(map);

    Reader r{base_, base_ + size_};
    if (r.take<uint32_t>() != 0x46554747u) throw std::runtime_error("not a GGUF file: " + path);
    const uint32_t version = r.take<uint32_t>();
    if (version != 3 && version != 2) throw std::runtime_error("unsupported GGUF version");
    const uint64_t n_tensors = r.take<uint64_t>();
    const uint64_t n_kv = r.take<uint64_t>();
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = r.take_string();
        const uint32_t type = r.take<uint32_t>();
        switch (type) {
            case V_STRING: str_[key] = r.take_string(); break;
            case V_U32: u32_[key] = r.take<uint32_t>(); break;
            case V_I32: u32_[key] = (uint32_t)r.take<int32_t>(); break;
            case V_F32: f32_[key] = r.take<float>(); break;
            case V_BOOL: u32_[key] = r.take<uint8_t>() ? 1 : 0; break;
            case V_U64: u32_[key] = (uint32_t)r.take<uint64_t>(); break;
            case V_ARRAY: {
                const uint32_t et = r.take<uint32_t>();
                const uint64_t n = r.take<uint64_t>();
                if (et == V_STRING) {
                    std::vector<std::string> & out = str_arrays_[key];
                    out.reserve(n);
                    for (uint64_t j = 0; j < n; ++j) out.push_back(r.take_string());
                } else if (et == V_I32 || et == V_U32) {
                    std::vector<int32_t> & out = i32_arrays_[key];
                    out.resize(n);
                    r.need(n * 4);
                    std::memcpy(out.data(), r.cur, n * 4);
                    r.cur += n * 4;
                } else {
                    r.skip(value_width(et) * n);
                }
                break;
            }
            default: r.skip(value_width(type)); break;
        }
    }
    const uint32_t alignment = u32("general.alignment", 32);
    std::vector<uint64_t> offsets;
    tensors_.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensor t;
        t.name = r.take_string();
        const uint32_t nd = r.take<uint32_t>();
        if (nd == 0 || nd > 4) throw std::runtime_error("tensor " + t.name + " has an unsupported rank");
        for (uint32_t d = 0; d < nd; ++d) t.ne.push_back(r.take<uint64_t>());
        t.type = r.take<uint32_t>();
        offsets.push_back(r.take<uint64_t>());
        BlockGeom g{};
        if (!block_geom(t.type, g)) {
            throw std::runtime_error("tensor " + t.name + " uses a storage type this backend does not read (ggml type " +
                                     std::to_string(t.type) + ")");
        }
        if (t.ne[0] % g.elems != 0) throw std::runtime_error("tensor " + t.name + " has a partial block");
        t.n_bytes = t.ne[0] / g.elems * g.bytes * t.rows();
        index_[t.name] = tensors_.size();
        tensors_.push_back(std::move(t));
    }
    uint64_t data_start = (uint64_t)(r.cur - base_);
    data_start = (data_start + alignment - 1) / alignment * alignment;
    for (size_t i = 0; i < tensors_.size(); ++i) {
        GgufTensor & t = tensors_[i];
        if (data_start + offsets[i] + t.n_bytes > size_) throw std::runtime_error("tensor " + t.name + " lies outside the file");
        t.data = base_ + data_start + offsets[i];
    }
}

GgufFile::~GgufFile() {
    if (base_) munmap(const_cast<uint8_t *>(base_), size_);
    if (fd_ >= 0) ::close(fd_);
}

} // namespace rb200
