// Checkpoints: the safetensors container read by tensor name, and the comparison of what a
// checkpoint holds with what a model declares.
//
// Container layout (as the reference's converter reads it, tools/convert_to_gguf.py:282-343):
// an 8-byte little-endian header length, a JSON header {name: {dtype, shape, data_offsets:
// [begin, end]}} with offsets relative to the end of the header, then the raw little-endian
// bytes.  A sharded checkpoint has model.safetensors.index.json whose weight_map names the
// shard of each tensor.  Files are mapped, tensors are views of the mapping.
//
// The reference binds its tensors by exact name, type and shape and fails on the first
// problem (src/kipp.c:859-1007, 1108-1118); here every problem is collected and reported in
// ONE error: every missing tensor, every unexpected one, every wrong shape and every
// unsupported element type.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <set>
#include <tuple>

#include "json.hpp"
#include "runtime.hpp"

namespace kipp {

// One checkpoint tensor a part needs.
struct TensorSpec {
    std::string name;
    std::vector<int64_t> shape;
    std::string init = "normal";       // random-weights mode: "normal" N(0, sigma), "near_one" 1 + U(-a, a), "int"
    bool optional = false;             // may be absent (a tied output head)
    std::string alias_of;              // the tensor that stands in when this one is absent
    bool ignore_if_present = false;    // present in the checkpoint but not used (a tied head stored anyway)

    Json to_json() const {
        Json j = Json::object();
        j.set("name", name);
        Json s = Json::array();
        for (auto d : shape) s.push((long long)d);
        j.set("shape", std::move(s));
        j.set("init", init);
        j.set("optional", optional);
        j.set("alias_of", alias_of.empty() ? Json(nullptr) : Json(alias_of));
        j.set("ignore_if_present", ignore_if_present);
        return j;
    }
    static TensorSpec from_json(const Json& j) {
        TensorSpec t;
        t.name = j.get("name").as_string();
        for (auto& d : j.get("shape").items()) t.shape.push_back(d.as_int());
        t.init = j.get_string("init", "normal");
        t.optional = j.get_bool("optional", false);
        t.alias_of = j.get_string("alias_of", "");
        t.ignore_if_present = j.get_bool("ignore_if_present", false);
        return t;
    }
};

struct StoredTensor {
    std::string name;
    int dtype = -1;                    // DType, or -1 for an element type the engine does not take
    std::string dtype_text;            // as the file names it
    std::vector<int64_t> shape;
    const uint8_t* data = nullptr;
    size_t bytes = 0;
    int64_t count() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};

inline std::string shape_text(const std::vector<int64_t>& shape) {
    std::string s = "[";
    for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

class MappedFile {
public:
    explicit MappedFile(const std::string& path) : path_(path) {
        int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) fail(KIPP_E_IO, path + ": cannot be opened");
        struct stat st;
        if (fstat(fd, &st) != 0) { ::close(fd); fail(KIPP_E_IO, path + ": cannot be read"); }
        size_ = (size_t)st.st_size;
        if (size_ > 0) {
            void* p = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
            if (p == MAP_FAILED) { ::close(fd); fail(KIPP_E_IO, path + ": cannot be mapped"); }
            data_ = static_cast<const uint8_t*>(p);
        }
        ::close(fd);
    }
    MappedFile(const MappedFile&) = delete;
    MappedFile& operator=(const MappedFile&) = delete;
    ~MappedFile() { if (data_) munmap(const_cast<uint8_t*>(data_), size_); }
    const uint8_t* data() const { return data_; }
    size_t size() const { return size_; }
    const std::string& path() const { return path_; }

private:
    std::string path_;
    const uint8_t* data_ = nullptr;
    size_t size_ = 0;
};

inline bool file_exists(const std::string& path) {
    struct stat st;
    return stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

inline std::string read_text_file(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) fail(KIPP_E_IO, path + ": cannot be opened");
    std::string out;
    char buf[65536];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out.append(buf, n);
    fclose(f);
    return out;
}

class Checkpoint {
public:
    // Maps model.safetensors, or the shards that model.safetensors.index.json names.
    explicit Checkpoint(const std::string& folder) : folder_(folder) {
        const std::string index_path = folder + "/model.safetensors.index.json";
        if (file_exists(index_path)) {
            Json index;
            try {
                index = Json::parse(read_text_file(index_path));
            } catch (const JsonError& e) {
                fail(KIPP_E_WEIGHTS, index_path + ": " + e.what());
            }
            const Json* map = index.find("weight_map");
            if (!map || !map->is_object()) fail(KIPP_E_WEIGHTS, index_path + ": no weight_map");
            std::map<std::string, std::map<std::string, StoredTensor>> shards;
            for (auto& kv : map->members()) {
                if (!kv.second.is_string()) fail(KIPP_E_WEIGHTS, index_path + ": weight_map values must be file names");
                const std::string& shard = kv.second.as_string();
                if (!shards.count(shard)) {
                    const std::string path = folder + "/" + shard;
                    if (!file_exists(path))
                        fail(KIPP_E_WEIGHTS, index_path + " names shard '" + shard + "', which is absent");
                    for (auto& t : read_file(path)) shards[shard][t.name] = t;
                }
                auto it = shards[shard].find(kv.first);
                if (it == shards[shard].end())
                    fail(KIPP_E_WEIGHTS, shard + ": index lists tensor '" + kv.first + "' but the file lacks it");
                add(it->second);
            }
            return;
        }
        const std::string single = folder + "/model.safetensors";
        if (!file_exists(single))
            fail(KIPP_E_WEIGHTS, folder + ": neither model.safetensors nor model.safetensors.index.json found");
        for (auto& t : read_file(single)) add(t);
    }

    const std::vector<StoredTensor>& tensors() const { return tensors_; }
    const StoredTensor* find(const std::string& name) const {
        auto it = by_name_.find(name);
        return it == by_name_.end() ? nullptr : &tensors_[it->second];
    }
    const std::string& folder() const { return folder_; }

    // What differs between the checkpoint and what a model declares.
    struct Report {
        std::vector<std::string> missing, unexpected;
        std::vector<std::tuple<std::string, std::vector<int64_t>, std::vector<int64_t>>> wrong_shape;   // name, is, expected
        std::vector<std::pair<std::string, std::string>> wrong_dtype;                                   // name, stored type
        bool clean() const { return missing.empty() && unexpected.empty() && wrong_shape.empty() && wrong_dtype.empty(); }
        Json to_json() const {
            Json j = Json::object();
            Json m = Json::array(), u = Json::array(), ws = Json::array(), wd = Json::array();
            for (auto& n : missing) m.push(n);
            for (auto& n : unexpected) u.push(n);
            for (auto& t : wrong_shape) {
                Json e = Json::array(), got = Json::array(), want = Json::array();
                for (auto d : std::get<1>(t)) got.push((long long)d);
                for (auto d : std::get<2>(t)) want.push((long long)d);
                e.push(std::get<0>(t));
                e.push(std::move(got));
                e.push(std::move(want));
                ws.push(std::move(e));
            }
            for (auto& t : wrong_dtype) {
                Json e = Json::array();
                e.push(t.first);
                e.push(t.second);
                wd.push(std::move(e));
            }
            j.set("missing", std::move(m));
            j.set("unexpected", std::move(u));
            j.set("wrong_shape", std::move(ws));
            j.set("wrong_dtype", std::move(wd));
            return j;
        }
    };

    Report compare(const std::vector<TensorSpec>& specs) const {
        Report r;
        std::set<std::string> declared;
        for (auto& s : specs) declared.insert(s.name);
        for (auto& s : specs) {
            const StoredTensor* t = find(s.name);
            if (!t) {
                if (s.optional && (s.alias_of.empty() || find(s.alias_of))) continue;
                r.missing.push_back(s.name);
                continue;
            }
            if (t->shape != s.shape) r.wrong_shape.emplace_back(s.name, t->shape, s.shape);
            if (t->dtype < 0) r.wrong_dtype.emplace_back(s.name, t->dtype_text);
        }
        for (auto& t : tensors_)
            if (!declared.count(t.name)) r.unexpected.push_back(t.name);
        std::sort(r.unexpected.begin(), r.unexpected.end());
        return r;
    }

    std::string describe(const Report& r) const {
        std::string msg = "checkpoint " + folder_ + " does not match the model:";
        auto join = [](const std::vector<std::string>& v) {
            std::string s;
            for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + v[i];
            return s;
        };
        if (!r.missing.empty())
            msg += "\n  missing tensors (" + std::to_string(r.missing.size()) + "): " + join(r.missing);
        if (!r.unexpected.empty())
            msg += "\n  unexpected tensors (" + std::to_string(r.unexpected.size()) + "): " + join(r.unexpected);
        for (auto& t : r.wrong_shape)
            msg += "\n  wrong shape: " + std::get<0>(t) + " is " + shape_text(std::get<1>(t)) + ", expected " +
                   shape_text(std::get<2>(t));
        for (auto& t : r.wrong_dtype) msg += "\n  unsupported dtype: " + t.first + " is " + t.second;
        return msg;
    }

    // Compares with what a model declares; throws KIPP_E_WEIGHTS listing every difference.
    void check(const std::vector<TensorSpec>& specs) const {
        const Report r = compare(specs);
        if (!r.clean()) fail(KIPP_E_WEIGHTS, describe(r));
    }

private:
    std::string folder_;
    std::vector<std::unique_ptr<MappedFile>> files_;
    std::vector<StoredTensor> tensors_;
    std::map<std::string, size_t> by_name_;

    void add(const StoredTensor& t) {
        if (by_name_.count(t.name)) fail(KIPP_E_WEIGHTS, folder_ + ": tensor '" + t.name + "' is stored twice");
        by_name_[t.name] = tensors_.size();
        tensors_.push_back(t);
    }

    static int dtype_of(const std::string& text, size_t& element) {
        static const struct { const char* name; int dtype; size_t size; } table[] = {
            {"BF16", BF16, 2}, {"F16", F16, 2}, {"F32", F32, 4}, {"I64", I64, 8}, {"I32", I32, 4},
            {"I16", I16, 2},   {"I8", I8, 1},   {"U8", U8, 1},   {"F64", -1, 8},  {"BOOL", -1, 1},
            {"U16", -1, 2},    {"U32", -1, 4},  {"U64", -1, 8},  {"F8_E4M3", -1, 1}, {"F8_E5M2", -1, 1}};
        for (auto& e : table)
            if (text == e.name) { element = e.size; return e.dtype; }
        element = 0;
        return -2;
    }

    std::vector<StoredTensor> read_file(const std::string& path) {
        files_.push_back(std::make_unique<MappedFile>(path));
        const MappedFile& f = *files_.back();
        if (f.size() < 8) fail(KIPP_E_WEIGHTS, path + ": truncated safetensors header");
        uint64_t hlen = 0;
        for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | f.data()[i];
        if (hlen > 100ull * 1024 * 1024 || 8 + hlen > f.size())
            fail(KIPP_E_WEIGHTS, path + ": unreasonable safetensors header length " + std::to_string(hlen));
        Json header;
        try {
            header = Json::parse(reinterpret_cast<const char*>(f.data()) + 8, (size_t)hlen);
        } catch (const JsonError& e) {
            fail(KIPP_E_WEIGHTS, path + ": header is not JSON (" + e.what() + ")");
        }
        if (!header.is_object()) fail(KIPP_E_WEIGHTS, path + ": header is not a JSON object");
        const size_t data_start = 8 + (size_t)hlen;
        const size_t data_size = f.size() - data_start;
        std::vector<StoredTensor> out;
        for (auto& kv : header.members()) {
            if (kv.first == "__metadata__") continue;
            StoredTensor t;
            t.name = kv.first;
            long long begin = 0, end = 0;
            size_t element = 0;
            try {
                t.dtype_text = kv.second.get("dtype").as_string();
                for (auto& d : kv.second.get("shape").items()) {
                    if (d.as_int() < 0) throw JsonError("negative size");
                    t.shape.push_back(d.as_int());
                }
                const Json& off = kv.second.get("data_offsets");
                if (off.size() != 2) throw JsonError("data_offsets");
                begin = off.at(0).as_int();
                end = off.at(1).as_int();
            } catch (const JsonError&) {
                fail(KIPP_E_WEIGHTS, path + ": bad header entry for '" + t.name + "'");
            }
            t.dtype = dtype_of(t.dtype_text, element);
            if (t.dtype == -2) { t.dtype = -1; element = 0; }
            const long long expect = element ? (long long)(t.count() * (int64_t)element) : end - begin;
            if (begin < 0 || end < begin || (size_t)end > data_size || end - begin != expect)
                fail(KIPP_E_WEIGHTS, format("%s: tensor '%s' has byte range [%lld, %lld) that does not fit %s %s in a "
                                            "data section of %zu bytes",
                                            path.c_str(), t.name.c_str(), begin, end, t.dtype_text.c_str(),
                                            shape_text(t.shape).c_str(), data_size));
            t.data = f.data() + data_start + begin;
            t.bytes = (size_t)(end - begin);
            out.push_back(std::move(t));
        }
        return out;
    }
};

}  // namespace kipp
