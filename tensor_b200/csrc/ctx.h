// Device context shared by every translation unit of the library: one CUDA device, one stream and one
// caching allocator per ott_ctx (include/otter_b200.h). Host code only.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/otter_b200.h"

// Stream-ordered, size-keyed cache of device blocks. Every block is used on the owning context's single
// stream only, so a block freed at stream position p can be handed out again at any later position
// without an event: the stream orders the old user's kernels before the new user's.
class DeviceCachingAllocator {
public:
    explicit DeviceCachingAllocator(int device) : device_(device) {}
    ~DeviceCachingAllocator() { release_cached(); }

    static size_t round_size(size_t bytes) {
        if (bytes == 0) bytes = 1;
        if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);       // 512 B granules up to 1 MiB
        return (bytes + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);  // 2 MiB granules above
    }

    // Failure injection for tests of the error paths (host side only): the n-th allocate call from now on fails with
    // cudaErrorMemoryAllocation without touching the device; n <= 0 switches it off.
    void fail_after(long n) {
        std::lock_guard<std::mutex> g(mu_);
        fail_countdown_ = n;
    }

    // Guard bands for tests (the memory checker this pool does not offer): every block obtained from the driver from now on is
    // `bytes` (a multiple of 512) larger on both sides, the bands hold kGuardByte, and check_guards reads every band of every
    // block, in use or cached, back and counts the blocks a kernel has written outside of. 0 switches it off for new blocks.
    static constexpr int kGuardByte = 0xC5;
    void set_guard(size_t bytes) {
        std::lock_guard<std::mutex> g(mu_);
        guard_ = (bytes + 511) & ~size_t(511);
    }
    cudaError_t check_guards(long* bad_blocks, size_t* first_bad_size) {
        std::lock_guard<std::mutex> g(mu_);
        *bad_blocks = 0;
        std::vector<unsigned char> host;
        for (const auto& kv : guards_) {
            const size_t gb = kv.second, sz = sizes_.at(kv.first);
            host.resize(2 * gb);
            char* user = static_cast<char*>(kv.first);
            cudaError_t e = cudaMemcpy(host.data(), user - gb, gb, cudaMemcpyDeviceToHost);
            if (e == cudaSuccess) e = cudaMemcpy(host.data() + gb, user + sz, gb, cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) return e;
            bool ok = true;
            for (size_t i = 0; i < 2 * gb && ok; ++i) ok = host[i] == kGuardByte;
            if (!ok && (*bad_blocks)++ == 0 && first_bad_size) *first_bad_size = sz;
        }
        return cudaSuccess;
    }

    cudaError_t allocate(size_t bytes, void** out) {
        const size_t sz = round_size(bytes);
        std::lock_guard<std::mutex> g(mu_);
        if (fail_countdown_ > 0 && --fail_countdown_ == 0) return cudaErrorMemoryAllocation;
        auto it = available_.find(sz);
        if (it != available_.end() && !it->second.empty()) {
            *out = it->second.back();
            it->second.pop_back();
            bytes_cached_ -= sz;
            bytes_in_use_ += sz;
            ++n_cache_hits_;
            if (logging_) log_.insert(*out);
            return cudaSuccess;
        }
        void* p = nullptr;
        const size_t gb = guard_;
        cudaError_t e = cudaMalloc(&p, sz + 2 * gb);
        if (e != cudaSuccess) {
            // give cached blocks back to the driver and retry once
            (void)cudaGetLastError();
            release_cached_locked();
            e = cudaMalloc(&p, sz + 2 * gb);
            if (e != cudaSuccess) return e;
        }
        if (gb != 0) {
            e = cudaMemset(p, kGuardByte, gb);
            if (e == cudaSuccess) e = cudaMemset(static_cast<char*>(p) + gb + sz, kGuardByte, gb);
            if (e != cudaSuccess) {
                cudaFree(p);
                return e;
            }
            p = static_cast<char*>(p) + gb;
            guards_[p] = gb;
        }
        ++n_device_mallocs_;
        sizes_[p] = sz;
        bytes_in_use_ += sz;
        *out = p;
        if (logging_) log_.insert(p);
        return cudaSuccess;
    }

    // For work that is frozen into a CUDA graph: the graph keeps addressing the blocks that were handed out while it was
    // captured, so those blocks must not go to anybody else (nor back to the driver) while the graph lives. begin_log starts
    // recording every block handed out; take_logged ends it and takes the recorded blocks that are free again out of the
    // cache (blocks still in use stay with their owner); give_back returns them to the cache.
    void begin_log() {
        std::lock_guard<std::mutex> g(mu_);
        logging_ = true;
        log_.clear();
    }
    std::vector<void*> take_logged() {
        std::lock_guard<std::mutex> g(mu_);
        logging_ = false;
        std::vector<void*> taken;
        for (auto& kv : available_) {
            auto& v = kv.second;
            for (size_t i = 0; i < v.size();) {
                if (log_.count(v[i])) {
                    taken.push_back(v[i]);
                    bytes_cached_ -= kv.first;
                    bytes_in_use_ += kv.first;
                    v[i] = v.back();
                    v.pop_back();
                } else {
                    ++i;
                }
            }
        }
        log_.clear();
        return taken;
    }
    void give_back(const std::vector<void*>& blocks) {
        for (void* p : blocks) free(p);
    }

    bool free(void* p) {
        if (!p) return true;
        std::lock_guard<std::mutex> g(mu_);
        auto it = sizes_.find(p);
        if (it == sizes_.end()) return false;
        available_[it->second].push_back(p);
        bytes_in_use_ -= it->second;
        bytes_cached_ += it->second;
        return true;
    }

    void release_cached() {
        std::lock_guard<std::mutex> g(mu_);
        release_cached_locked();
    }

    void stats(uint64_t* mallocs, uint64_t* hits, uint64_t* in_use, uint64_t* cached) {
        std::lock_guard<std::mutex> g(mu_);
        if (mallocs) *mallocs = n_device_mallocs_;
        if (hits) *hits = n_cache_hits_;
        if (in_use) *in_use = bytes_in_use_;
        if (cached) *cached = bytes_cached_;
    }

private:
    void release_cached_locked() {
        for (auto& kv : available_) {
            for (void* p : kv.second) {
                auto gi = guards_.find(p);
                cudaFree(gi == guards_.end() ? p : static_cast<void*>(static_cast<char*>(p) - gi->second));
                if (gi != guards_.end()) guards_.erase(gi);
                sizes_.erase(p);
            }
            kv.second.clear();
        }
        bytes_cached_ = 0;
    }

    int device_;
    std::mutex mu_;
    std::map<size_t, std::vector<void*>> available_;
    std::unordered_map<void*, size_t> sizes_;
    std::unordered_map<void*, size_t> guards_;  // blocks with guard bands: user pointer -> band size
    size_t guard_ = 0;
    bool logging_ = false;
    long fail_countdown_ = 0;
    std::unordered_set<void*> log_;
    uint64_t n_device_mallocs_ = 0, n_cache_hits_ = 0, bytes_in_use_ = 0, bytes_cached_ = 0;
};

struct ott_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t aux_stream[2] = {nullptr, nullptr};  // host->device and device->host copies that overlap the compute stream
    DeviceCachingAllocator* alloc = nullptr;
    std::string last_error;
    uint64_t launches = 0;
    uint64_t capture_launches0 = UINT64_MAX;  // value of `launches` when the open graph capture began; UINT64_MAX: none open
    int dw_tensor_cores = 1;  // depthwise 3x3 layers with int8 input on the tensor cores: 0 never, 1 narrow layers, 2 always (ott_set_depthwise_tensor_cores)
    unsigned long long wait_limit_ns = 2000000000ull;  // limit of every bounded wait inside the kernels (ott_set_wait_limit_ms)
    uint32_t* status_dev = nullptr;   // default status word the kernels report into
    uint32_t* status_host = nullptr;  // pinned mirror
    // pinned staging buffers of the *_host entry points
    void* stage_in = nullptr;
    size_t stage_in_bytes = 0;
    void* stage_out = nullptr;
    size_t stage_out_bytes = 0;

    int fail(int code, const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        last_error = buf;
        return code;
    }
};

struct ott_event {
    cudaEvent_t ev = nullptr;
};

#define OTT_CUDA_CHECK(ctx, expr)                                                                         \
    do {                                                                                                  \
        cudaError_t _e = (expr);                                                                          \
        if (_e != cudaSuccess)                                                                            \
            return (ctx)->fail(OTT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

// RAII device block from the context's caching allocator.
struct DeviceBlock {
    ott_ctx* ctx = nullptr;
    void* p = nullptr;
    DeviceBlock() = default;
    DeviceBlock(const DeviceBlock&) = delete;
    DeviceBlock& operator=(const DeviceBlock&) = delete;
    ~DeviceBlock() { reset(); }
    cudaError_t alloc(ott_ctx* c, size_t bytes) {
        reset();
        ctx = c;
        return c->alloc->allocate(bytes, &p);
    }
    void reset() {
        if (p && ctx) ctx->alloc->free(p);
        p = nullptr;
    }
};
