// Minimal GGUF v3 reader: metadata as typed values, tensors as views into a read-only mapping.
// Container layout as the reference's fixture writers produce it
// (scripts/gen-tiny-fixture.py:343-374): header, key/values, tensor infos, padding to
// general.alignment, then tensor data at aligned offsets.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace rb200 {

struct GgufTensor {
    std::string name;
    std::vector<uint64_t> ne;   // fastest dimension first
    uint32_t type = 0;
    const uint8_t * data = nullptr;
    uint64_t n_bytes = 0;
    uint64_t rows() const {
        uint64_t r = 1;
        for (size_t i = 1; i < ne.size(); ++i) r *= ne[i];
        return r;
    }
};

class GgufFile {
public:
    explicit GgufFile(const std::string & path);
    ~GgufFile();
    GgufFile(const GgufFile &) = delete;
    GgufFile & operator=(const GgufFile &) = delete;

    bool has_u32(const std::string & k) const { return u32_.count(k) != 0; }
    uint32_t u32(const std::string & k, uint32_t fallback) const {
        auto it = u32_.find(k);
        return it == u32_.end() ? fallback : it->second;
    }
    float f32(const std::string & k, float fallback) const {
        auto it = f32_.find(k);
        return it == f32_.end() ? fallback : it->second;
    }
    std::string str(const std::string & k, const std::string & fallback = "") const {
        auto it = str_.find(k);
        return it == str_.end() ? fallback : it->second;
    }
    const std::vector<std::string> * str_array(const std::string & k) const {
        auto it = str_arrays_.find(k);
        return it == str_arrays_.end() ? nullptr : &it->second;
    }
    const std::vector<int32_t> * i32_array(const std::string & k) const {
        auto it = i32_arrays_.find(k);
        return it == i32_arrays_.end() ? nullptr : &it->second;
    }
    const GgufTensor * find(const std::string & name) const {
        auto it = index_.find(name);
        return it == index_.end() ? nullptr : &tensors_[it->second];
    }
    const std::vector<GgufTensor> & tensors() const { return tensors_; }
    uint64_t file_size() const { return size_; }

private:
    int fd_ = -1;
    const uint8_t * base_ = nullptr;
    uint64_t size_ = 0;
    std::map<std::string, uint32_t> u32_;
    std::map<std::string, float> f32_;
    std::map<std::string, std::string> str_;
    std::map<std::string, std::vector<std::string>> str_arrays_;
    std::map<std::string, std::vector<int32_t>> i32_arrays_;
    std::vector<GgufTensor> tensors_;
    std::map<std::string, size_t> index_;
};

} // namespace rb200
