// Host side of the B200 quantization path: caching device-memory pool.
//
// Keeps the public interface of the reference's MemoryAllocator
// (include/sovereigngrad/allocator.hpp:10-69, src/allocator.cpp:34-247): singleton, best-fit reuse
// of freed blocks, splitting, coalescing of neighbours on free, active/cached/total/peak
// statistics, std::runtime_error on device out-of-memory.  The inside is redesigned for a
// 180 GB device and for the kernels' needs:
//   * every block starts on a 512-byte boundary (TMA wants 16, the C ABI's workspace 256);
//   * raw device segments are multiples of 2 MiB; requests >= 64 MiB get their own segment;
//   * blocks are indexed by address and, when free, by size: allocate and free are O(log n)
//     instead of a linear scan plus a sort per free;
//   * blocks remember the CUDA device ordinal they came from (one process may see 8 GPUs);
//   * on cudaMalloc failure the pool returns its completely free segments to the driver and
//     retries once before throwing.
#pragma once

#include <cstddef>
#include <map>
#include <mutex>
#include <string>

namespace sovereigngrad {

enum class Device { CPU, CUDA };

inline std::string device_to_string(Device d) { return (d == Device::CPU) ? "CPU" : "CUDA"; }

struct Block {
    void* ptr = nullptr;
    size_t size = 0;
    bool in_use = false;
    Device device = Device::CPU;
    bool is_raw_allocation = false;   // first block of a raw segment
    void* raw_parent = nullptr;       // base of the raw segment this block lies in
    int ordinal = 0;                  // CUDA device ordinal (0 for CPU)
};

// Raw memory source of the CUDA pool.  The default calls cudaMalloc/cudaFree; tests install a
// host-memory stand-in to exercise the pool without a GPU.
struct RawBackend {
    void* (*alloc)(size_t bytes, int* ordinal_out) = nullptr;   // nullptr on failure
    void (*release)(void* ptr, int ordinal) = nullptr;
    const char* (*last_error)() = nullptr;
};

class MemoryAllocator {
public:
    static MemoryAllocator& instance() {
        static MemoryAllocator inst;
        return inst;
    }

    void* allocate(size_t bytes, Device device);
    void free(void* ptr, Device device);
    void release_all();

    size_t active_allocations(Device device) const;
    size_t cached_allocations(Device device) const;
    size_t total_memory_allocated(Device device) const;
    size_t peak_memory_allocated(Device device) const;
    void reset_peak_memory_stats();
    std::string get_memory_summary(Device device) const;

    // Bytes a request is rounded to, and the raw segment size used for it.
    static size_t round_block(size_t bytes);
    static size_t segment_size(size_t bytes, Device device);

    void set_cuda_backend(const RawBackend& backend);   // test hook; call with an empty pool
    void reset_cuda_backend();

    ~MemoryAllocator();

private:
    MemoryAllocator();
    MemoryAllocator(const MemoryAllocator&) = delete;
    MemoryAllocator& operator=(const MemoryAllocator&) = delete;

    struct Pool {
        std::map<char*, Block> blocks;                    // by address
        std::multimap<size_t, char*> free_by_size;        // free blocks only
        size_t active_bytes = 0, active_count = 0, total_bytes = 0, peak_bytes = 0;
    };
    Pool& pool(Device d) { return d == Device::CPU ? cpu_ : cuda_; }
    const Pool& pool(Device d) const { return d == Device::CPU ? cpu_ : cuda_; }

    void* raw_alloc(size_t bytes, Device device, int* ordinal);
    void raw_free(void* ptr, Device device, int ordinal);
    void erase_free_index(Pool& p, char* ptr, size_t size);
    size_t release_free_segments(Pool& p, Device device);

    Pool cpu_, cuda_;
    RawBackend cuda_backend_;
    mutable std::mutex mutex_;
};

}  // namespace sovereigngrad
