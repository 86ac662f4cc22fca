#include "sovereigngrad/allocator.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <iomanip>
#include <new>
#include <sstream>
#include <stdexcept>
#include <vector>

namespace sovereigngrad {
namespace {

constexpr size_t kAlign = 512;
constexpr size_t kCudaSegment = 2u << 20;     // 2 MiB
constexpr size_t kCpuSegment = 4096;
constexpr size_t kOwnSegment = 64u << 20;     // requests this large get a segment of their own
constexpr size_t kMinSplit = 1024;            // as the reference: keep a remainder only if >= 1 KiB

thread_local std::string g_cuda_error;

void* cuda_alloc(size_t bytes, int* ordinal) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    void* p = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        g_cuda_error = cudaGetErrorString(e);
        cudaGetLastError();
        return nullptr;
    }
    *ordinal = dev;
    return p;
}

void cuda_release(void* p, int ordinal) {
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) return;
    if (cur != ordinal) cudaSetDevice(ordinal);
    cudaFree(p);
    if (cur != ordinal) cudaSetDevice(cur);
}

const char* cuda_last_error() { return g_cuda_error.c_str(); }

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

MemoryAllocator::MemoryAllocator() { reset_cuda_backend(); }
MemoryAllocator::~MemoryAllocator() { release_all(); }

void MemoryAllocator::set_cuda_backend(const RawBackend& backend) {
    std::lock_guard<std::mutex> lock(mutex_);
    cuda_backend_ = backend;
}

void MemoryAllocator::reset_cuda_backend() {
    std::lock_guard<std::mutex> lock(mutex_);
    cuda_backend_.alloc = cuda_alloc;
    cuda_backend_.release = cuda_release;
    cuda_backend_.last_error = cuda_last_error;
}

size_t MemoryAllocator::round_block(size_t bytes) { return round_up(bytes, kAlign); }

size_t MemoryAllocator::segment_size(size_t bytes, Device device) {
    const size_t b = round_block(bytes);
    if (device == Device::CPU) return std::max(b, kCpuSegment);
    return round_up(std::max(b, size_t(1)), kCudaSegment);
}

void* MemoryAllocator::raw_alloc(size_t bytes, Device device, int* ordinal) {
    *ordinal = 0;
    if (device == Device::CPU) {
        void* p = std::aligned_alloc(kAlign, round_up(bytes, kAlign));
        if (!p) throw std::bad_alloc();
        return p;
    }
    return cuda_backend_.alloc(bytes, ordinal);
}

void MemoryAllocator::raw_free(void* ptr, Device device, int ordinal) {
    if (device == Device::CPU) std::free(ptr);
    else cuda_backend_.release(ptr, ordinal);
}

void MemoryAllocator::erase_free_index(Pool& p, char* ptr, size_t size) {
    auto range = p.free_by_size.equal_range(size);
    for (auto it = range.first; it != range.second; ++it) {
        if (it->second == ptr) {
            p.free_by_size.erase(it);
            return;
        }
    }
}

// Returns segments that are one single free block to the driver.  Caller holds the mutex.
size_t MemoryAllocator::release_free_segments(Pool& p, Device device) {
    size_t released = 0;
    for (auto it = p.blocks.begin(); it != p.blocks.end();) {
        Block& b = it->second;
        bool whole = !b.in_use && b.is_raw_allocation;
        if (whole) {
            auto next = std::next(it);
            whole = (next == p.blocks.end()) || next->second.raw_parent != b.raw_parent;
        }
        if (whole) {
            erase_free_index(p, it->first, b.size);
            raw_free(b.ptr, device, b.ordinal);
            p.total_bytes -= b.size;
            released += b.size;
            it = p.blocks.erase(it);
        } else {
            ++it;
        }
    }
    return released;
}

void* MemoryAllocator::allocate(size_t bytes, Device device) {
    if (bytes == 0) return nullptr;   // src/allocator.cpp:35
    const size_t need = round_block(bytes);
    std::lock_guard<std::mutex> lock(mutex_);
    Pool& p = pool(device);

    int want_ordinal = 0;
    if (device == Device::CUDA && cuda_backend_.alloc == cuda_alloc) cudaGetDevice(&want_ordinal);

    // best fit among the free blocks of this device ordinal
    char* found = nullptr;
    for (auto it = p.free_by_size.lower_bound(need); it != p.free_by_size.end(); ++it) {
        if (p.blocks[it->second].ordinal == want_ordinal || device == Device::CPU) {
            found = it->second;
            p.free_by_size.erase(it);
            break;
        }
    }
    if (!found) {
        const size_t seg = (need >= kOwnSegment) ? segment_size(need, device) : segment_size(std::max(need, size_t(1)), device);
        int ordinal = 0;
        void* raw = raw_alloc(seg, device, &ordinal);
        if (!raw && device == Device::CUDA) {
            release_free_segments(p, device);
            raw = raw_alloc(seg, device, &ordinal);
        }
        if (!raw) {
            std::ostringstream ss;   // same flavour as src/allocator.cpp:92-98
            ss << "CUDA Allocator Out of Memory: requested " << seg << " bytes, active allocations: " << p.active_count
               << ", total managed: " << p.total_bytes << " bytes. Error: "
               << (cuda_backend_.last_error ? cuda_backend_.last_error() : "unknown");
            throw std::runtime_error(ss.str());
        }
        Block b;
        b.ptr = raw;
        b.size = seg;
        b.device = device;
        b.is_raw_allocation = true;
        b.raw_parent = raw;
        b.ordinal = ordinal;
        found = static_cast<char*>(raw);
        p.blocks[found] = b;
        p.total_bytes += seg;
    }

    Block& blk = p.blocks[found];
    if (blk.size - need >= kMinSplit) {
        Block rest;
        rest.ptr = found + need;
        rest.size = blk.size - need;
        rest.device = device;
        rest.raw_parent = blk.raw_parent;
        rest.ordinal = blk.ordinal;
        blk.size = need;
        p.blocks[found + need] = rest;
        p.free_by_size.emplace(rest.size, found + need);
    }
    blk.in_use = true;
    p.active_bytes += blk.size;
    p.active_count += 1;
    p.peak_bytes = std::max(p.peak_bytes, p.active_bytes);
    return found;
}

void MemoryAllocator::free(void* ptr, Device device) {
    if (!ptr) return;
    std::lock_guard<std::mutex> lock(mutex_);
    Pool& p = pool(device);
    auto it = p.blocks.find(static_cast<char*>(ptr));
    if (it == p.blocks.end() || !it->second.in_use) return;   // unknown pointer: ignored, as the reference does
    Block& b = it->second;
    b.in_use = false;
    p.active_bytes -= b.size;
    p.active_count -= 1;
    // merge with the next block, then with the previous one, inside the same raw segment
    auto next = std::next(it);
    if (next != p.blocks.end() && !next->second.in_use && next->second.raw_parent == b.raw_parent &&
        it->first + b.size == next->first) {
        erase_free_index(p, next->first, next->second.size);
        b.size += next->second.size;
        p.blocks.erase(next);
    }
    if (it != p.blocks.begin()) {
        auto prev = std::prev(it);
        if (!prev->second.in_use && prev->second.raw_parent == b.raw_parent && prev->first + prev->second.size == it->first) {
            erase_free_index(p, prev->first, prev->second.size);
            prev->second.size += b.size;
            p.blocks.erase(it);
            it = prev;
        }
    }
    p.free_by_size.emplace(it->second.size, it->first);
}

void MemoryAllocator::release_all() {
    std::lock_guard<std::mutex> lock(mutex_);
    for (Device d : {Device::CPU, Device::CUDA}) {
        Pool& p = pool(d);
        for (auto& kv : p.blocks)
            if (kv.second.is_raw_allocation) raw_free(kv.second.ptr, d, kv.second.ordinal);
        p = Pool();
    }
}

size_t MemoryAllocator::active_allocations(Device device) const {
    std::lock_guard<std::mutex> lock(mutex_);
    return pool(device).active_count;
}

size_t MemoryAllocator::cached_allocations(Device device) const {
    std::lock_guard<std::mutex> lock(mutex_);
    return pool(device).free_by_size.size();
}

size_t MemoryAllocator::total_memory_allocated(Device device) const {
    std::lock_guard<std::mutex> lock(mutex_);
    return pool(device).total_bytes;
}

size_t MemoryAllocator::peak_memory_allocated(Device device) const {
    std::lock_guard<std::mutex> lock(mutex_);
    return pool(device).peak_bytes;
}

void MemoryAllocator::reset_peak_memory_stats() {
    std::lock_guard<std::mutex> lock(mutex_);
    cpu_.peak_bytes = cpu_.active_bytes;
    cuda_.peak_bytes = cuda_.active_bytes;
}

std::string MemoryAllocator::get_memory_summary(Device device) const {
    std::lock_guard<std::mutex> lock(mutex_);
    const Pool& p = pool(device);
    std::ostringstream ss;   // same line format as src/allocator.cpp:240-245
    ss << "[" << device_to_string(device) << " Memory Summary] "
       << "Active: " << p.active_bytes / 1024.0f << " KB (" << p.active_count << " blocks), "
       << "Cached: " << (p.total_bytes - p.active_bytes) / 1024.0f << " KB (" << p.free_by_size.size() << " blocks), "
       << "Peak: " << p.peak_bytes / 1024.0f << " KB";
    return ss.str();
}

}  // namespace sovereigngrad
