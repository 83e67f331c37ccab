// What everything of the host core stands on: the error type, element types, checked CUDA
// calls, device memory that is freed with its owner, the kernel libraries (found and loaded
// at first use) and the named activation workspace.
#pragma once
#include <cuda_runtime_api.h>
#include <dlfcn.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "kipp_b200.h"

namespace kipp {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
};

inline std::string format(const char* fmt, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return buf;
}

[[noreturn]] inline void fail(int code, const std::string& what) { throw Error(code, what); }

enum DType : int { F32 = 0, BF16 = 1, F16 = 2, I32 = 3, I64 = 4, I16 = 5, I8 = 6, U8 = 7 };

inline size_t dtype_size(int d) {
    switch (d) {
        case F32: case I32: return 4;
        case BF16: case F16: case I16: return 2;
        case I64: return 8;
        case I8: case U8: return 1;
    }
    fail(KIPP_E_ARGUMENT, format("unknown element type %d", d));
}
inline const char* dtype_name(int d) {
    static const char* names[] = {"float32", "bfloat16", "float16", "int32", "int64", "int16", "int8", "uint8"};
    return d >= 0 && d <= 7 ? names[d] : "?";
}
inline bool is_float_dtype(int d) { return d == F32 || d == BF16 || d == F16; }
// The type a checkpoint tensor is kept in: 16-bit floats as bfloat16, 32-bit floats stay,
// integer tables become int32.
inline int storage_dtype(int d) { return d == F32 ? F32 : is_float_dtype(d) ? BF16 : I32; }

inline void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail(KIPP_E_CUDA, format("%s: %s", what, cudaGetErrorString(e)));
    }
}

// Device memory owned by an object.
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes, const char* what = "device buffer") { reset(bytes, what); }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), bytes_(o.bytes_) { o.p_ = nullptr; o.bytes_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) { release(); p_ = o.p_; bytes_ = o.bytes_; o.p_ = nullptr; o.bytes_ = 0; }
        return *this;
    }
    ~DeviceBuffer() { release(); }
    void reset(size_t bytes, const char* what = "device buffer") {
        release();
        if (bytes == 0) bytes = 16;
        cudaError_t e = cudaMalloc(&p_, bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            p_ = nullptr;
            fail(KIPP_E_MEMORY, format("%s: %zu device bytes could not be allocated (%s)", what, bytes,
                                       cudaGetErrorString(e)));
        }
        bytes_ = bytes;
    }
    void release() {
        if (p_) cudaFree(p_);
        p_ = nullptr;
        bytes_ = 0;
    }
    void* get() const { return p_; }
    template <typename T> T* as() const { return static_cast<T*>(p_); }
    size_t bytes() const { return bytes_; }

private:
    void* p_ = nullptr;
    size_t bytes_ = 0;
};

class PinnedBuffer {
public:
    PinnedBuffer() = default;
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    ~PinnedBuffer() { if (p_) cudaFreeHost(p_); }
    void ensure(size_t bytes) {
        if (bytes <= bytes_) return;
        if (p_) cudaFreeHost(p_);
        p_ = nullptr;
        bytes_ = 0;
        cuda_check(cudaMallocHost(&p_, bytes), "pinned host buffer");
        bytes_ = bytes;
    }
    template <typename T> T* as() const { return static_cast<T*>(p_); }
    size_t bytes() const { return bytes_; }

private:
    void* p_ = nullptr;
    size_t bytes_ = 0;
};

// ---------------------------------------------------------------------------------------------
// The kernel libraries.  Every kernel file is a shared library of its own (lib<name>.so) with
// `extern "C" int kipp_<kernel>(..., void* stream)` launchers; a library is loaded the first
// time one of its kernels is asked for, so a model loads (and a fresh checkout builds) only
// what it uses.  There is no fallback: a missing library is an error.
class KernelLibraries {
public:
    static KernelLibraries& get() {
        static KernelLibraries libs;
        return libs;
    }
    void set_resolver(kipp_library_resolver r) {
        std::lock_guard<std::mutex> lock(mutex_);
        resolver_ = r;
    }
    void* symbol(const char* library, const char* name) {
        std::lock_guard<std::mutex> lock(mutex_);
        std::string key = std::string(library) + ":" + name;
        auto it = symbols_.find(key);
        if (it != symbols_.end()) return it->second;
        void* handle = open(library);
        void* sym = dlsym(handle, name);
        if (!sym) fail(KIPP_E_BUILD, format("kernel library lib%s.so has no symbol %s", library, name));
        symbols_[key] = sym;
        return sym;
    }

private:
    std::mutex mutex_;
    kipp_library_resolver resolver_ = nullptr;
    std::map<std::string, void*> handles_;
    std::map<std::string, void*> symbols_;

    static std::string own_directory() {
        Dl_info info;
        if (dladdr(reinterpret_cast<void*>(&own_directory), &info) && info.dli_fname) {
            std::string path = info.dli_fname;
            size_t slash = path.rfind('/');
            return slash == std::string::npos ? "." : path.substr(0, slash);
        }
        return ".";
    }
    void* open(const char* library) {
        auto it = handles_.find(library);
        if (it != handles_.end()) return it->second;
        std::string path;
        if (resolver_) {
            const char* p = resolver_(library);
            if (p) path = p;
        }
        if (path.empty()) path = own_directory() + "/lib" + library + ".so";
        void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!h)
            fail(KIPP_E_BUILD, format("kernel library %s could not be loaded (%s); build the kernels first "
                                      "(python -c 'import __graft_entry__ as g; g.build()'); there is no fallback",
                                      path.c_str(), dlerror()));
        handles_[library] = h;
        return h;
    }
};

template <typename Fn> Fn kernel_symbol(const char* library, const char* name) {
    return reinterpret_cast<Fn>(KernelLibraries::get().symbol(library, name));
}

// Turns a launcher's return code into an error.
inline void kernel_check(int code, const char* what) {
    if (code == 0) return;
    if (code == -1) fail(KIPP_E_KERNEL, format("%s: the kernel refuses these sizes", what));
    if (code == -2) fail(KIPP_E_KERNEL, format("%s: unsupported dtype combination", what));
    if (code == -3) fail(KIPP_E_KERNEL, format("%s: a pointer or stride is not aligned as the kernel needs", what));
    if (code == -4) fail(KIPP_E_KERNEL, format("%s: these sizes need more scratch than the library holds", what));
    fail(KIPP_E_CUDA, format("%s: CUDA error %d (%s)", what, code, cudaGetErrorString((cudaError_t)code)));
}

// ---------------------------------------------------------------------------------------------
// Named activation buffers that grow to the largest size asked for and are then reused by every
// step (one workspace per engine, as the reference's Metal bridge keeps one per model,
// src/metal/kipp_metal.m:151-158).  `generation` changes whenever a buffer moved: graphs captured
// before that are stale.
class Workspace {
public:
    void* buffer(const std::string& key, size_t bytes) {
        auto& slot = buffers_[key];
        if (slot.bytes() < bytes || slot.get() == nullptr) {
            if (capturing) fail(KIPP_E_STATE, "workspace buffer '" + key + "' would be allocated inside a graph capture");
            size_t want = bytes < 256 ? 256 : bytes;
            slot.reset(want, ("workspace buffer " + key).c_str());
            ++generation;
        }
        return slot.get();
    }
    template <typename T> T* get(const std::string& key, size_t count) {
        return static_cast<T*>(buffer(key, count * sizeof(T)));
    }
    size_t bytes() const {
        size_t n = 0;
        for (auto& kv : buffers_) n += kv.second.bytes();
        return n;
    }
    long long generation = 0;
    bool capturing = false;

private:
    std::map<std::string, DeviceBuffer> buffers_;
};

}  // namespace kipp
